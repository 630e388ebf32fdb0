"""Generate tests/golden/decode_vectors.npz from the upstream package.

    python tests/golden/make_decode_golden.py /path/to/upstream/src

Plays three decode steps over a small static KV pool in the upstream wire format -- keys and values
(B, k*HKV, slots, D), read through the per-channel views the upstream reader layers take
(models/white_matter/modeling_white_matter.py:244-247) -- with ragged committed lengths, grouped query heads, with and
without the dummy slot and with packed documents (modules/documents.py:61-64).  Every read is evaluated by the upstream
operator's portable backend on the CPU; for the document cases the upstream FlashAttention route (pack_kv_cache,
layers/backends.py:25-34, then a plain length-bounded read) is evaluated as well and has to agree.  Inputs and results
are stored; the tests replay the file and never import the upstream package.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def main(upstream_src: str) -> None:
    sys.path.insert(0, upstream_src)
    from white_matter.layers.backends import pack_kv_cache
    from white_matter.modules.documents import feedback_document_mask
    from white_matter.ops import strict_causal_attention

    arrays: dict[str, np.ndarray] = {}
    B, CH, HKV, HQ, CAP, D, STEPS = 3, 2, 2, 4, 12, 64, 3
    for dummy in (False, True):
        for documents in (False, True):
            case = f"dummy{int(dummy)}_docs{int(documents)}"
            torch.manual_seed(17 + 2 * int(dummy) + int(documents))
            lead = int(dummy)
            lengths = torch.tensor([2, 5, 0])
            keys = torch.randn(B, CH * HKV, CAP + lead, D)
            values = torch.randn(B, CH * HKV, CAP + lead, D)
            past_docs = torch.tensor([[0, 0, 9, 9, 9, 9, 9, 9], [0, 0, 1, 1, 1, 9, 9, 9], [9, 9, 9, 9, 9, 9, 9, 9]])
            arrays[f"{case}/keys0"] = keys.numpy().copy()
            arrays[f"{case}/values0"] = values.numpy().copy()
            arrays[f"{case}/lengths0"] = lengths.numpy().copy()
            arrays[f"{case}/past_docs0"] = past_docs.numpy().copy()
            for step in range(STEPS):
                q = torch.randn(B, HQ, 1, D)
                new_k = torch.randn(B, CH * HKV, 1, D)
                new_v = torch.randn(B, CH * HKV, 1, D)
                current = torch.tensor([[0], [1 if step < 2 else 2], [0]])
                arrays[f"{case}/q{step}"] = q.numpy()
                arrays[f"{case}/new_k{step}"] = new_k.numpy()
                arrays[f"{case}/new_v{step}"] = new_v.numpy()
                arrays[f"{case}/current{step}"] = current.numpy()
                keep = None
                if documents:
                    keep = torch.zeros(B, CAP + lead, dtype=torch.bool)
                    for b in range(B):
                        n = int(lengths[b])
                        row = feedback_document_mask(past_docs[b : b + 1, :n], current[b : b + 1], use_dummy_token=dummy)
                        keep[b, : n + lead] = row[0]
                state_k = keys.unflatten(1, (CH, HKV))
                state_v = values.unflatten(1, (CH, HKV))
                for channel in range(CH):
                    out = strict_causal_attention(
                        q, state_k[:, channel], state_v[:, channel], query_start=lengths, kv_lengths=lengths,
                        use_dummy_token=dummy, key_mask=keep, backend="reference",
                    )
                    arrays[f"{case}/out{step}_c{channel}"] = out.numpy()
                    if documents:
                        # the upstream GPU route: visible slots first, then a read bounded by their count
                        pk, pv, plen = pack_kv_cache(state_k, state_v, keep)
                        packed = strict_causal_attention(
                            q, pk[:, channel], pv[:, channel], query_start=plen.long(), kv_lengths=plen.long(),
                            use_dummy_token=False, backend="reference",
                        )
                        assert torch.allclose(packed, out, atol=1e-5), (case, step, channel)
                # commit the step's rows behind each sequence's tokens
                for b in range(B):
                    slot = int(lengths[b]) + lead
                    keys[b, :, slot] = new_k[b, :, 0]
                    values[b, :, slot] = new_v[b, :, 0]
                    past_docs[b, int(lengths[b])] = current[b, 0]
                lengths = lengths + 1
            arrays[f"{case}/keys_final"] = keys.numpy().copy()
            arrays[f"{case}/lengths_final"] = lengths.numpy().copy()
    np.savez_compressed(HERE / "decode_vectors.npz", **arrays)
    print(f"wrote {len(arrays)} arrays")


if __name__ == "__main__":
    main(sys.argv[1])
