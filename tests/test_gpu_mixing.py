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
