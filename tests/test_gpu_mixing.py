"""KV source mixing on the GPU against the CPU oracle (through the C ABI)."""

import pytest
import torch

from helpers import assert_parity
from oracle import attention_oracle as oracle
from white_matter_b200 import cyclic_attention, mix_kv_sources

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(25, 2, 3, 37, 64), (3, 1, 1, 5, 8), (64, 2, 2, 16, 64), (1, 2, 2, 9, 16)])
def test_forward_and_gradients(shape, dtype):
    torch.manual_seed(3)
    src = torch.randn(shape).to(dtype)
    logits = torch.randn(shape[0])
    probe = torch.randn(shape[1:]).to(dtype)
    s = src.cuda().requires_grad_()
    w = logits.cuda().requires_grad_()
    out = mix_kv_sources(s, w)
    ds, dw = torch.autograd.grad(out, (s, w), probe.cuda())
    so, wo = src.double().requires_grad_(), logits.double().requires_grad_()
    exp = oracle.mix_sources_oracle(so, wo)
    eds, edw = torch.autograd.grad(exp, (so, wo), probe.double())
    # fp32: 1e-4; bf16: one rounding of the result (max-abs 2e-2, relative L2 1e-2)
    tol = dict(max_abs_tol=1e-4, rel_l2_tol=1e-4) if dtype == torch.float32 else dict(max_abs_tol=2e-2, rel_l2_tol=1e-2)
    assert_parity(out.float(), exp, what="out", **tol)
    assert_parity(ds.float(), eds, what="dsources", **tol)
    scale = max(1.0, edw.abs().max().item())
    assert_parity(dw.float() / scale, edw / scale, what="dlogits", max_abs_tol=2e-3 if dtype == torch.float32 else 3e-2,
                  rel_l2_tol=1e-3 if dtype == torch.float32 else 3e-2)


def test_single_source_is_identity_and_weights_sum_to_one():
    src = torch.randn(1, 4, 8, 16, device="cuda", dtype=torch.bfloat16)
    assert torch.equal(mix_kv_sources(src, torch.zeros(1, device="cuda")), src[0])
    ones = torch.ones(25, 3, 128, device="cuda", dtype=torch.bfloat16)
    out = mix_kv_sources(ones, torch.randn(25, device="cuda"))
    assert_parity(out.float(), torch.ones(3, 128), what="convexity", max_abs_tol=8e-3, rel_l2_tol=8e-3)


def test_mixed_sources_feed_attention_with_gradients_to_logits():
    """K and V are mixtures of source stacks; gradients flow through attention into sources and logits."""
    torch.manual_seed(9)
    S, B, H, T, D = 5, 1, 2, 64, 64
    ksrc, vsrc = torch.randn(S, B, H, T, D), torch.randn(S, B, H, T, D)
    lk, lv = torch.randn(S), torch.randn(S)
    q = torch.randn(B, H, T // 4, D)
    probe = torch.randn(B, H, T // 4, D)
    dev = [t.cuda().requires_grad_() for t in (q, ksrc, vsrc, lk, lv)]
    out = cyclic_attention(dev[0], mix_kv_sources(dev[1], dev[3]), mix_kv_sources(dev[2], dev[4]), query_stride=4)
    grads = torch.autograd.grad(out, dev, probe.cuda())
    ref = [t.double().requires_grad_() for t in (q, ksrc, vsrc, lk, lv)]
    exp = oracle.cyclic_attention_oracle(
        ref[0], oracle.mix_sources_oracle(ref[1], ref[3]), oracle.mix_sources_oracle(ref[2], ref[4]), query_stride=4
    )
    exp_grads = torch.autograd.grad(exp, ref, probe.double())
    assert_parity(out, exp, what="out", max_abs_tol=1e-4, rel_l2_tol=1e-4)
    for g, e, name in zip(grads, exp_grads, ("dq", "dksrc", "dvsrc", "dlogits_k", "dlogits_v")):
        assert_parity(g, e, what=name, max_abs_tol=2e-4, rel_l2_tol=2e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sources,heads,kv_heads,dummy,masked", [(25, 4, 4, False, False), (3, 4, 2, True, False), (2, 8, 2, False, True), (1, 3, 1, True, True)])
def test_decode_with_the_mixture_formed_in_the_load_path(sources, heads, kv_heads, dummy, masked, dtype):
    """mixed_pool_decode against the oracle's mixture followed by the oracle's strict attention; slots beyond the
    committed lengths hold NaN in every source and must not be read."""
    from white_matter_b200 import mixed_pool_decode, strict_causal_attention

    torch.manual_seed(21)
    batch, slots, dim = 3, 300, 64
    lead = int(dummy)
    lengths = torch.tensor([299 - lead, 17, 0])
    ksrc = torch.randn(sources, batch, kv_heads, slots, dim).to(dtype)
    vsrc = torch.randn(sources, batch, kv_heads, slots, dim).to(dtype)
    for b in range(batch):
        ksrc[:, b, :, lead + int(lengths[b]):] = float("nan")
        vsrc[:, b, :, lead + int(lengths[b]):] = float("nan")
    lk, lv = torch.randn(sources), torch.randn(sources)
    q = torch.randn(batch, heads, 1, dim).to(dtype)
    mask = None
    if masked:
        mask = torch.rand(batch, slots) < 0.7
        mask[:, 0] = True
    got = mixed_pool_decode(
        q.cuda(), ksrc.cuda(), vsrc.cuda(), lk.cuda(), lv.cuda(), query_start=lengths.cuda(), kv_lengths=lengths.cuda(),
        use_dummy_token=dummy, key_mask=None if mask is None else mask.cuda(),
    )
    clean_k, clean_v = torch.nan_to_num(ksrc.double()), torch.nan_to_num(vsrc.double())
    want = oracle.strict_causal_oracle(
        q.double(), oracle.mix_sources_oracle(clean_k, lk.double()), oracle.mix_sources_oracle(clean_v, lv.double()),
        query_start=lengths, kv_lengths=lengths, use_dummy_token=dummy, key_mask=mask,
    )
    tol = dict(max_abs_tol=1e-4, rel_l2_tol=1e-4) if dtype == torch.float32 else dict(max_abs_tol=2e-2, rel_l2_tol=1e-2)
    assert_parity(got.float(), want, what="mixed decode", **tol)
    # and against the two-step form of this library
    two_step = strict_causal_attention(
        q.cuda(), mix_kv_sources(torch.nan_to_num(ksrc).cuda(), lk.cuda()), mix_kv_sources(torch.nan_to_num(vsrc).cuda(), lv.cuda()),
        query_start=lengths.cuda(), kv_lengths=lengths.cuda(), use_dummy_token=dummy, key_mask=None if mask is None else mask.cuda(),
    )
    assert_parity(got.float(), two_step.float(), what="fused vs materialised", **tol)
