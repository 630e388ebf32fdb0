"""The decode step around the pool read: upstream vectors (tests/golden/make_decode_golden.py) replayed against the CPU
oracle and, on the GPU, against the static pool with device-side commits and CUDA-graph replay."""

from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import BF16_TOL, F32_TOL, assert_parity
from oracle import attention_oracle as oracle

VECTORS = np.load(Path(__file__).resolve().parent / "golden" / "decode_vectors.npz")
CASES = sorted({name.split("/")[0] for name in VECTORS.files})
B, CH, HKV, HQ, CAP, D, STEPS = 3, 2, 2, 4, 12, 64, 3


def get(case, name):
    return torch.from_numpy(VECTORS[f"{case}/{name}"])


def keep_mask(past_docs, lengths, current, dummy, slots):
    lead = int(dummy)
    keep = torch.zeros(B, slots, dtype=torch.bool)
    for b in range(B):
        n = int(lengths[b])
        keep[b, :lead] = True
        keep[b, lead : lead + n] = (past_docs[b, :n] == current[b, 0]) & (current[b, 0] >= 0)
    return keep


@pytest.mark.parametrize("case", CASES)
def test_oracle_replays_the_upstream_decode_steps(case):
    dummy, documents = case.startswith("dummy1"), case.endswith("docs1")
    lead = int(dummy)
    keys, values = get(case, "keys0").clone(), get(case, "values0").clone()
    lengths, past = get(case, "lengths0").clone(), get(case, "past_docs0").clone()
    for step in range(STEPS):
        q, current = get(case, f"q{step}"), get(case, f"current{step}")
        keep = keep_mask(past, lengths, current, dummy, CAP + lead) if documents else None
        for channel in range(CH):
            heads = slice(channel * HKV, (channel + 1) * HKV)
            out = oracle.strict_causal_oracle(
                q, keys[:, heads], values[:, heads], query_start=lengths, kv_lengths=lengths, use_dummy_token=dummy, key_mask=keep
            )
            assert_parity(out.float(), get(case, f"out{step}_c{channel}"), what=f"step {step} channel {channel}", max_abs_tol=2e-5, rel_l2_tol=5e-5)
        for b in range(B):
            keys[b, :, int(lengths[b]) + lead] = get(case, f"new_k{step}")[b, :, 0]
            values[b, :, int(lengths[b]) + lead] = get(case, f"new_v{step}")[b, :, 0]
            past[b, int(lengths[b])] = current[b, 0]
        lengths = lengths + 1
    assert torch.equal(keys, get(case, "keys_final"))


gpu = [pytest.mark.gpu, pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", CASES)
@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")
def test_pool_reads_and_commits_match_upstream(case, dtype):
    from white_matter_b200.decode_step import KVPoolCache, document_key_mask

    dummy, documents = case.startswith("dummy1"), case.endswith("docs1")
    lead = int(dummy)
    cache = KVPoolCache(B, CH, HKV, CAP, D, use_dummy_token=dummy, dtype=dtype)
    cache.keys.copy_(get(case, "keys0"))
    cache.values.copy_(get(case, "values0"))
    # what lies behind the committed tokens is unused capacity: poison it
    lengths0 = get(case, "lengths0")
    for b in range(B):
        cache.keys[b, :, int(lengths0[b]) + lead :] = float("nan")
        cache.values[b, :, int(lengths0[b]) + lead :] = float("nan")
    cache.lengths.copy_(lengths0)
    past = get(case, "past_docs0").clone().cuda()
    tol = F32_TOL if dtype == torch.float32 else BF16_TOL
    for step in range(STEPS):
        q = get(case, f"q{step}").to("cuda", dtype)
        current = get(case, f"current{step}").cuda()
        keep = None
        if documents:
            seen = past.shape[1]
            visible = torch.arange(seen, device="cuda")[None, :] < cache.lengths[:, None]
            keep = document_key_mask(torch.where(visible, past, -7), current, use_dummy_token=dummy, slots=CAP + lead)
        for channel in range(CH):
            out = cache.read(q, channel, key_mask=keep)
            assert out.shape == (B, 1, HQ, D) and torch.isfinite(out).all()
            exp = get(case, f"out{step}_c{channel}")
            if dtype == torch.bfloat16:  # the same arithmetic on the rounded inputs
                heads = slice(channel * HKV, (channel + 1) * HKV)
                kk = torch.nan_to_num(cache.keys[:, heads].float().cpu()).double()
                vv = torch.nan_to_num(cache.values[:, heads].float().cpu()).double()
                exp = oracle.strict_causal_oracle(
                    q.float().cpu().double(), kk, vv, query_start=cache.lengths.cpu().long(), kv_lengths=cache.lengths.cpu().long(),
                    use_dummy_token=dummy, key_mask=None if keep is None else keep.cpu(),
                )
            assert_parity(out.float(), exp, what=f"step {step} channel {channel}", **tol)
        before = cache.lengths.clone()
        cache.append(get(case, f"new_k{step}").to("cuda", dtype), get(case, f"new_v{step}").to("cuda", dtype))
        assert torch.equal(cache.lengths, before + 1)
        past[torch.arange(B, device="cuda"), before.long()] = current[:, 0]
    if dtype == torch.float32:
        final = get(case, "keys_final")
        for b in range(B):
            n = int(cache.lengths[b]) + lead
            assert torch.equal(cache.keys[b, :, :n].cpu(), final[b, :, :n])


@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")
def test_a_captured_step_replays_while_the_lengths_grow_on_the_device():
    from white_matter_b200.decode_step import DecodeStepGraph, KVPoolCache

    torch.manual_seed(8)
    batch, channels, kv_heads, heads, capacity, dim, layers = 4, 2, 2, 4, 40, 64, 4
    cache = KVPoolCache(batch, channels, kv_heads, capacity, dim, use_dummy_token=True)
    cache.set_dummy(torch.randn(channels * kv_heads, dim, device="cuda").bfloat16(), torch.randn(channels * kv_heads, dim, device="cuda").bfloat16())
    prefix = 9
    cache.append(torch.randn(batch, channels * kv_heads, prefix, dim, device="cuda").bfloat16(), torch.randn(batch, channels * kv_heads, prefix, dim, device="cuda").bfloat16(), advance=False)
    cache.lengths.copy_(torch.tensor([0, 3, 9, 5], dtype=torch.int32))
    queries = torch.randn(layers, batch, heads, 1, dim, device="cuda", dtype=torch.bfloat16)
    new_k = torch.randn(batch, channels * kv_heads, 1, dim, device="cuda", dtype=torch.bfloat16)
    new_v = torch.randn_like(new_k)

    def step():
        # every layer reads the channel it is tied to; the token's own rows are committed after the sweep
        outs = [cache.read(queries[layer], layer % channels) for layer in range(layers)]
        cache.append(new_k, new_v)
        return torch.stack(outs)

    graph = DecodeStepGraph(step, cache)
    eager = KVPoolCache(batch, channels, kv_heads, capacity, dim, use_dummy_token=True)
    eager.keys.copy_(cache.keys)
    eager.values.copy_(cache.values)
    eager.lengths.copy_(cache.lengths)
    for turn in range(5):
        queries.normal_()
        new_k.normal_()
        new_v.normal_()
        replayed = graph().clone()
        expected = torch.stack([eager.read(queries[layer], layer % channels) for layer in range(layers)])
        eager.append(new_k, new_v)
        assert torch.equal(replayed, expected), f"turn {turn}"
        assert torch.equal(cache.lengths, eager.lengths)
        ref = oracle.strict_per_query_oracle(
            queries[1].cpu(), eager.keys[:, kv_heads:].cpu(), eager.values[:, kv_heads:].cpu(), (eager.lengths - 1).cpu(), True
        )
        assert_parity(replayed[1].float(), ref, what=f"turn {turn} layer 1", **BF16_TOL)
    assert torch.equal(cache.keys, eager.keys)
