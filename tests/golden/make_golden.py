"""Generate tests/golden/reference_vectors.npz from the upstream package.

Run in a container that has the upstream checkout:

    python tests/golden/make_golden.py /path/to/upstream/src

It imports ``white_matter.ops`` (the portable PyTorch backend) and the
caller-side ``prepare_feedback_metadata``, evaluates them on small seeded
inputs on the CPU, and stores inputs, outputs and gradients.  The test-suite
replays the file; it never imports the upstream package.

Array names are ``<case>/<field>``; ``cases.json`` beside the archive holds the
scalar parameters of every case.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def main(upstream_src: str) -> None:
    sys.path.insert(0, upstream_src)
    from white_matter.blocks._execution.metadata import prepare_feedback_metadata
    from white_matter.ops import (
        cyclic_attention,
        prepare_cyclic_attention_metadata,
        prepare_strict_causal_metadata,
        strict_causal_attention,
    )

    arrays: dict[str, np.ndarray] = {}
    cases: dict[str, dict] = {}

    def put(case: str, **tensors) -> None:
        for name, t in tensors.items():
            if t is None:
                continue
            t = t.detach()
            if t.dtype == torch.bfloat16:
                t = t.float()
            arrays[f"{case}/{name}"] = t.cpu().numpy()

    # ------------------------------------------------------------------ cyclic
    def cyclic_case(name, B, HQ, HKV, Q, K, D, stride, offset, strict_past, docs, seed, store_inputs=True):
        torch.manual_seed(seed)
        q = torch.randn(B, HQ, Q, D)
        k = torch.randn(B, HKV, K, D)
        v = torch.randn(B, HKV, K, D)
        probe = torch.randn(B, HQ, Q, D)
        metadata = None
        if docs == "sorted":
            seg = torch.stack([torch.arange(K) // (19 + 12 * b) for b in range(B)])
            metadata = prepare_cyclic_attention_metadata(
                seg[:, offset::stride][:, :Q], torch.cat((seg.new_full((B, 1), -1), seg[:, :-1]), 1)
            )
        elif docs == "feedback":
            # token documents without a dummy slot, as the no-dummy cyclic schedule builds them
            lengths = [[29, 41, K], [57, 13, K]]
            ids = torch.zeros(B, K, dtype=torch.long)
            for b in range(B):
                at = 0
                for d, n in enumerate(lengths[b % 2]):
                    ids[b, at : at + n] = d
                    at += n
                    if at >= K:
                        break
            groups = [torch.arange(r, K, stride) for r in range(stride)]
            metadata = prepare_feedback_metadata(ids, groups, K, use_dummy_token=False)[offset]
            metadata = type(metadata)(*(t[:, :Q] if i in (0, 2) else t for i, t in enumerate(metadata)))
        for dtype, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
            if dtype == torch.bfloat16 and not store_inputs:
                continue  # large cases keep only the fp32 results
            qq, kk, vv = (t.to(dtype).requires_grad_() for t in (q, k, v))
            out = cyclic_attention(
                qq, kk, vv, query_stride=stride, query_offset=offset, strict_past=strict_past, metadata=metadata
            )
            grads = torch.autograd.grad(out, (qq, kk, vv), probe.to(dtype))
            put(name, **{f"out_{tag}": out, f"dq_{tag}": grads[0], f"dk_{tag}": grads[1], f"dv_{tag}": grads[2]})
        if store_inputs:
            put(name, q=q, k=k, v=v, probe=probe)
        if metadata is not None:
            put(name, q_seg=metadata[0], k_seg=metadata[1], q_start=metadata[2], k_end=metadata[3])
        cases[name] = dict(
            kind="cyclic", B=B, HQ=HQ, HKV=HKV, Q=Q, K=K, D=D, stride=stride, offset=offset,
            strict_past=strict_past, docs=docs, seed=seed, inputs_stored=store_inputs,
        )

    # the CPU-runnable fp32 configuration (B=2, H=4, 256 keys, stride 4): inputs are regenerated from the seed, only results are stored
    cyclic_case("c1", 2, 4, 4, 64, 256, 64, 4, 0, True, None, 0, store_inputs=False)
    cyclic_case("cyc_gqa", 2, 4, 2, 33, 132, 64, 4, 1, False, None, 23)
    cyclic_case("cyc_gqa_docs", 2, 4, 2, 33, 132, 64, 4, 1, False, "sorted", 23)
    cyclic_case("cyc_strict_docs", 2, 2, 2, 34, 137, 32, 4, 2, True, "feedback", 5)
    cyclic_case("cyc_strict_docs_r0", 2, 2, 1, 35, 137, 64, 4, 0, True, "feedback", 6)
    cyclic_case("cyc_d128", 1, 6, 2, 17, 71, 128, 4, 3, False, None, 7)
    cyclic_case("cyc_d96", 1, 3, 1, 19, 83, 96, 4, 0, False, "sorted", 8)
    cyclic_case("cyc_d8", 2, 4, 2, 5, 11, 8, 2, 1, False, None, 42)
    cyclic_case("cyc_stride1", 1, 2, 2, 130, 130, 64, 1, 0, True, None, 9, store_inputs=False)

    # ------------------------------------------------------------------ strict
    def strict_case(name, B, H, HKV, T, N, D, seed, *, query_start=0, kv_lengths=None, dummy=False, docs=None,
                    key_mask=None, nan_tail=False, grads=True, store_inputs=True):
        torch.manual_seed(seed)
        q = torch.randn(B, H, T, D)
        k = torch.randn(B, HKV, N, D)
        v = torch.randn(B, HKV, N, D)
        probe = torch.randn(B, T, H, D)
        if nan_tail:
            for b, n in enumerate(kv_lengths.tolist()):
                k[b, :, n + int(dummy):] = float("nan")
                v[b, :, n + int(dummy):] = float("nan")
        metadata = None
        if docs is not None:
            metadata = prepare_strict_causal_metadata(
                docs, T, query_start=query_start, kv_lengths=kv_lengths, use_dummy_token=dummy
            )
            put(name, docs=docs, query_indices=metadata.query_indices, key_indices=metadata.key_indices,
                cu_queries=metadata.cu_queries, cu_keys=metadata.cu_keys)
        for dtype, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
            if dtype == torch.bfloat16 and not store_inputs:
                continue
            qq, kk, vv = (t.to(dtype).requires_grad_(grads) for t in (q, k, v))
            out = strict_causal_attention(
                qq, kk, vv, query_start=query_start, kv_lengths=kv_lengths, use_dummy_token=dummy,
                metadata=metadata, key_mask=key_mask, backend="reference",
            )
            put(name, **{f"out_{tag}": out})
            if grads:
                g = torch.autograd.grad(out, (qq, kk, vv), probe.to(dtype))
                put(name, **{f"dq_{tag}": g[0], f"dk_{tag}": g[1], f"dv_{tag}": g[2]})
        if store_inputs:
            put(name, q=q, k=k, v=v, probe=probe)
        put(name,
            query_start_t=query_start if isinstance(query_start, torch.Tensor) else None,
            kv_lengths=kv_lengths, key_mask=key_mask)
        cases[name] = dict(
            kind="strict", B=B, H=H, HKV=HKV, T=T, N=N, D=D, seed=seed, dummy=dummy, grads=grads,
            inputs_stored=store_inputs, nan_tail=nan_tail,
            query_start=None if isinstance(query_start, torch.Tensor) else query_start,
            packed=docs is not None, key_extent=None if metadata is None else metadata.key_extent,
            max_queries=None if metadata is None else metadata.max_queries,
            max_keys=None if metadata is None else metadata.max_keys,
        )

    for dummy in (False, True):
        tag = "dummy" if dummy else "plain"
        docs = torch.arange(8)[None].expand(2, -1).clone() // 3
        docs[1] = torch.arange(8) // 2
        strict_case(f"strict_packed_{tag}", 2, 4, 2, 5, 8 + int(dummy), 64, 29, query_start=3, dummy=dummy, docs=docs)
        strict_case(f"strict_dense_{tag}", 2, 4, 2, 7, 11 + int(dummy), 64, 30, query_start=4, dummy=dummy)
        strict_case(f"strict_decode_{tag}", 3, 4, 2, 1, 9 + int(dummy), 64, 31,
                    query_start=torch.tensor([0, 3, 7], dtype=torch.int32),
                    kv_lengths=torch.tensor([0, 3, 7], dtype=torch.int32), dummy=dummy, nan_tail=True, grads=False)
        pads = torch.tensor([[0, 0, -2, -2, 0, 0, -2, 0], [0, -2, 1, -2, 1, 0, 0, -2]])
        strict_case(f"strict_pads_{tag}", 2, 4, 2, 4, 8 + int(dummy), 64, 32, query_start=4, dummy=dummy, docs=pads)
        strict_case(f"strict_trunc_{tag}", 2, 4, 2, 4, 8 + int(dummy), 64, 33,
                    query_start=torch.tensor([0, 3]), kv_lengths=torch.tensor([1, 4]), dummy=dummy)
        ragged = torch.tensor([[0, 0, 1, -1, -1, -1, -1], [0, 0, 0, 0, 1, 1, -1]])
        strict_case(f"strict_ragged_{tag}", 2, 4, 2, 4, 7 + int(dummy), 8, 34,
                    query_start=torch.tensor([0, 3]), dummy=dummy, docs=ragged)
        mask = torch.rand(3, 21 + int(dummy), generator=torch.Generator().manual_seed(3)) > 0.35
        strict_case(f"strict_keymask_{tag}", 3, 4, 2, 1, 21 + int(dummy), 64, 35,
                    query_start=torch.tensor([5, 20, 13]), dummy=dummy, key_mask=mask, grads=False)
        long_docs = (torch.arange(160) // 67)[None].clone()
        strict_case(f"strict_jacobi_{tag}", 1, 2, 2, 160, 160 + int(dummy), 64, 36, dummy=dummy, docs=long_docs,
                    store_inputs=False)

    # ------------------------------------------------------------------ schedule known answers
    gen = torch.Generator().manual_seed(11)
    for n in range(8):
        B, extent = 3, 40 + 7 * n
        T = 9 + n
        docs = torch.randint(0, 4, (B, extent), generator=gen).sort(dim=1).values
        pad = torch.rand(B, extent, generator=gen) < (0.0 if n % 2 == 0 else 0.25)
        docs = torch.where(pad, torch.full_like(docs, -1 - (n % 2)), docs)
        start = torch.randint(0, extent - T + 1, (B,), generator=gen)
        lengths = None if n % 3 else torch.randint(0, extent + 1, (B,), generator=gen)
        dummy = bool(n % 2) if n < 6 else bool((n + 1) % 2)
        m = prepare_strict_causal_metadata(docs, T, query_start=start, kv_lengths=lengths, use_dummy_token=dummy)
        name = f"schedule_{n}"
        put(name, docs=docs, start=start, lengths=lengths, query_indices=m.query_indices, key_indices=m.key_indices,
            cu_queries=m.cu_queries, cu_keys=m.cu_keys)
        cases[name] = dict(kind="schedule", T=T, dummy=dummy, max_queries=m.max_queries, max_keys=m.max_keys,
                           key_extent=m.key_extent)
    for n, (stride, T, dummy) in enumerate(((1, 17, True), (2, 33, True), (4, 33, False), (8, 64, False))):
        docs = torch.randint(0, 3, (2, T), generator=gen).sort(dim=1).values
        if n == 1:
            docs[0, -4:] = -1
        groups = [torch.arange(r, T, stride) for r in range(stride)]
        ms = prepare_feedback_metadata(docs, groups, T + int(dummy) - (1 if dummy else 0), use_dummy_token=dummy)
        name = f"feedback_{n}"
        put(name, docs=docs)
        for r, m in enumerate(ms):
            put(name, **{f"q_seg_{r}": m[0], f"k_seg_{r}": m[1], f"q_start_{r}": m[2], f"k_end_{r}": m[3]})
        cases[name] = dict(kind="feedback", stride=stride, T=T, dummy=dummy, key_length=T + int(dummy) - (1 if dummy else 0))

    np.savez_compressed(HERE / "reference_vectors.npz", **arrays)
    (HERE / "cases.json").write_text(json.dumps(cases, indent=1, sort_keys=True))
    total = sum(a.nbytes for a in arrays.values())
    print(f"{len(cases)} cases, {len(arrays)} arrays, {total / 1e6:.2f} MB raw")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
