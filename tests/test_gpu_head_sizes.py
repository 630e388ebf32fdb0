"""Head sizes 128 and 96 on the tensor-core kernels: the forward, and the key-stationary backward."""

import pytest
import torch

from helpers import BF16_TOL, assert_parity, geometric_documents
from oracle import attention_oracle as oracle
from white_matter_b200 import (
    _native,
    cyclic_attention,
    prepare_feedback_metadata,
    prepare_strict_causal_metadata,
    strict_causal_attention,
)

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")]


@pytest.mark.parametrize("D", [128, 96])
@pytest.mark.parametrize("documents", [False, True])
@pytest.mark.parametrize("stride,residue,length", [(8, 3, 1100), (4, 0, 520), (1, 0, 300)])
def test_cyclic_forward(stride, residue, length, documents, D):
    torch.manual_seed(5)
    B, H, HKV = 2, 4, 2
    queries = len(range(residue, length, stride))
    q = torch.randn(B, H, queries, D).bfloat16()
    k, v = (torch.randn(B, HKV, length, D).bfloat16() for _ in range(2))
    metadata = None
    if documents:
        docs = geometric_documents(B, length, 200, seed=3)
        metadata = prepare_feedback_metadata(docs, [torch.arange(r, length, stride) for r in range(stride)], length, use_dummy_token=False)[residue]
    args = dict(query_stride=stride, query_offset=residue, strict_past=True)
    with torch.no_grad():
        dev_md = None if metadata is None else tuple(t.cuda() for t in metadata)
        out = cyclic_attention(q.cuda(), k.cuda(), v.cuda(), metadata=dev_md, backend="sm100_tcgen05", **args)
        simt = cyclic_attention(q.cuda(), k.cuda(), v.cuda(), metadata=dev_md, backend="sm100_simt", **args)
    assert _native.device_status(True) == 0
    exp = oracle.cyclic_attention_oracle(q.double(), k.double(), v.double(), metadata=metadata, **args)
    assert_parity(out.float(), exp, what=f"tcgen05 forward, head {D}", **BF16_TOL)
    assert_parity(out.float(), simt.float(), what="tcgen05 vs simt", **BF16_TOL)


@pytest.mark.parametrize("D", [128, 96])
@pytest.mark.parametrize("masked", [False, True])
@pytest.mark.parametrize("length", [128, 70])
def test_cached_prefix_prefill_with_nan_capacity(length, masked, D):
    torch.manual_seed(6)
    B, H, HKV, N = 3, 4, 4, 900
    lengths = torch.tensor([880, 400, 129])
    starts = (lengths - length).clamp_min(0)
    q = torch.randn(B, H, length, D).bfloat16()
    k, v = (torch.randn(B, HKV, N, D).bfloat16() for _ in range(2))
    key_mask = None
    if masked:
        key_mask = torch.rand(B, N) > 0.3
    kn, vn = k.clone(), v.clone()
    for b in range(B):
        kn[b, :, int(lengths[b]):] = float("nan")
        vn[b, :, int(lengths[b]):] = float("nan")
        if masked:
            kn[b][:, ~key_mask[b]] = float("nan")
            vn[b][:, ~key_mask[b]] = float("nan")
    with torch.no_grad():
        out = strict_causal_attention(
            q.cuda(), kn.cuda(), vn.cuda(), query_start=starts.cuda(), kv_lengths=lengths.cuda(),
            key_mask=None if key_mask is None else key_mask.cuda(), backend="sm100_tcgen05",
        )
    assert torch.isfinite(out).all()
    exp = oracle.strict_causal_oracle(q.double(), k.double(), v.double(), query_start=starts, kv_lengths=lengths, key_mask=key_mask)
    assert_parity(out.float(), exp, what=f"prefill, head {D}", **BF16_TOL)


@pytest.mark.parametrize("D", [128, 96])
def test_jacobi_with_documents_and_gradients(D):
    """Forward and gradients through the default backend."""
    torch.manual_seed(7)
    B, H, T = 2, 2, 384
    docs = geometric_documents(B, T, 120, seed=4)
    q, probe = (torch.randn(B, H, T, D).bfloat16() for _ in range(2))
    k, v = (torch.randn(B, H, T, D).bfloat16() for _ in range(2))
    schedule = prepare_strict_causal_metadata(docs.cuda(), T)
    qq, kk, vv = (t.cuda().requires_grad_() for t in (q, k, v))
    out = strict_causal_attention(qq, kk, vv, metadata=schedule)
    grads = torch.autograd.grad(out, (qq, kk, vv), probe.transpose(1, 2).cuda())
    qo, ko, vo = (t.double().requires_grad_() for t in (q, k, v))
    exp = oracle.strict_causal_oracle(qo, ko, vo, metadata=prepare_strict_causal_metadata(docs, T))
    exp_grads = torch.autograd.grad(exp, (qo, ko, vo), probe.transpose(1, 2).double())
    assert_parity(out.float(), exp, what="out", **BF16_TOL)
    for g, e, name in zip(grads, exp_grads, ("dq", "dk", "dv")):
        assert_parity(g.float(), e, what=name, **BF16_TOL)


@pytest.mark.parametrize("D", [128, 96])
@pytest.mark.parametrize("documents", [False, True])
@pytest.mark.parametrize("stride,residue,length,heads,kv_heads", [(8, 3, 1100, 4, 4), (4, 0, 520, 4, 2), (1, 0, 300, 2, 1), (8, 7, 2048, 2, 2)])
def test_cyclic_gradients_on_the_tensor_cores(stride, residue, length, heads, kv_heads, documents, D):
    torch.manual_seed(8)
    B = 2
    queries = len(range(residue, length, stride))
    q, probe = (torch.randn(B, heads, queries, D).bfloat16() for _ in range(2))
    k, v = (torch.randn(B, kv_heads, length, D).bfloat16() for _ in range(2))
    metadata = None
    if documents:
        docs = geometric_documents(B, length, 200, seed=9)
        metadata = prepare_feedback_metadata(docs, [torch.arange(r, length, stride) for r in range(stride)], length, use_dummy_token=False)[residue]
    args = dict(query_stride=stride, query_offset=residue, strict_past=True)
    dev_md = None if metadata is None else tuple(t.cuda() for t in metadata)
    results = {}
    for backend in ("sm100_tcgen05", "sm100_simt"):
        qq, kk, vv = (t.cuda().requires_grad_() for t in (q, k, v))
        out = cyclic_attention(qq, kk, vv, metadata=dev_md, backend=backend, **args)
        results[backend] = torch.autograd.grad(out, (qq, kk, vv), probe.cuda())
    assert _native.device_status(True) == 0
    qo, ko, vo = (t.double().requires_grad_() for t in (q, k, v))
    exp = oracle.cyclic_attention_oracle(qo, ko, vo, metadata=metadata, **args)
    exp_grads = torch.autograd.grad(exp, (qo, ko, vo), probe.double())
    for g, s, e, name in zip(results["sm100_tcgen05"], results["sm100_simt"], exp_grads, ("dq", "dk", "dv")):
        assert_parity(g.float(), e, what=f"{name}, head {D}", **BF16_TOL)
        assert_parity(g.float(), s.float(), what=f"{name} against the SIMT family", **BF16_TOL)


@pytest.mark.parametrize("masked", [False, True])
@pytest.mark.parametrize("D", [128, 96])
def test_dense_strict_gradients_with_nan_capacity(D, masked):
    """Several query tiles per key tile, grouped heads, and NaN in the slots no query may read."""
    torch.manual_seed(10)
    B, H, HKV, Q, N = 2, 4, 2, 300, 700
    lengths = torch.tensor([650, 301])
    starts = lengths - Q
    q, probe = (torch.randn(B, H, Q, D).bfloat16() for _ in range(2))
    k, v = (torch.randn(B, HKV, N, D).bfloat16() for _ in range(2))
    key_mask = (torch.rand(B, N) > 0.3) if masked else None
    kn, vn = k.clone(), v.clone()
    for b in range(B):
        kn[b, :, int(lengths[b]):] = float("nan")
        vn[b, :, int(lengths[b]):] = float("nan")
        if masked:
            kn[b][:, ~key_mask[b]] = float("nan")
            vn[b][:, ~key_mask[b]] = float("nan")
    qq, kk, vv = (t.cuda().requires_grad_() for t in (q, kn, vn))
    out = strict_causal_attention(qq, kk, vv, query_start=starts.cuda(), kv_lengths=lengths.cuda(), backend="sm100_tcgen05",
                                  key_mask=None if key_mask is None else key_mask.cuda())
    grads = torch.autograd.grad(out, (qq, kk, vv), probe.transpose(1, 2).cuda())
    assert _native.device_status(True) == 0
    qo, ko, vo = (t.double().requires_grad_() for t in (q, k, v))
    exp = oracle.strict_causal_oracle(qo, ko, vo, query_start=starts, kv_lengths=lengths, key_mask=key_mask)
    exp_grads = torch.autograd.grad(exp, (qo, ko, vo), probe.transpose(1, 2).double())
    for g, e, name in zip(grads, exp_grads, ("dq", "dk", "dv")):
        assert torch.isfinite(g).all(), name
        assert_parity(g.float(), e, what=f"{name}, head {D}", **BF16_TOL)
