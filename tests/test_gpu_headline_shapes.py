"""Value checks of the tensor-core kernels at the benchmark's own shapes.

The training shape (B=16, H=16, 2048 keys, 256 queries per residue, stride 8, D=64, packed documents of mean
length 1024) and the Jacobi prefill shape (B=8, H=16, T=2048, documents of mean 512) run at full size on the
GPU; the CPU oracle evaluates a slice of (batch row, head) pairs in fp64 on the same bf16 inputs -- attention never
mixes batch rows or heads, so a slice of the full-size result is compared with the oracle of the sliced inputs.
Forward, dQ, dK and dV are all gated by the parity contract.
"""

import ctypes

import pytest
import torch

from helpers import BF16_TOL, assert_parity, geometric_documents
from oracle import attention_oracle as oracle
from white_matter_b200 import (
    _native,
    cyclic_attention,
    operators,
    prepare_feedback_metadata,
    prepare_strict_causal_metadata,
    strict_causal_attention,
)

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")]

B, H, T, D, S = 16, 16, 2048, 64, 8


def rows_with_most_documents(docs: torch.Tensor, count: int) -> list[int]:
    changes = (docs[:, 1:] != docs[:, :-1]).sum(1)
    order = torch.argsort(changes, descending=True).tolist()
    picked = order[: count - 1] + [order[-1]]  # the busiest rows and the quietest one
    return sorted(set(picked))


def backward_scratch_bytes(q, k, v):
    """What the library asks for when it differentiates this problem: the short-query pipeline needs the row
    statistics only, the key-stationary one an fp32 dQ accumulator as well."""
    a, keep = operators._cyclic_args(q, k, v, None, S, 0, _native.WM_KERNEL_AUTO)
    a.dout, a.dq, a.dk, a.dv = q.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.dout_strides = a.dq_strides = _native.strides3(q)
    a.dk_strides = a.dv_strides = _native.strides3(k)
    return _native.load_library().wm_attn_bwd_workspace_bytes(ctypes.byref(a))


def compare_slice(out, grads, q, k, v, probe, rows, heads, what, **oracle_args):
    """Oracle in fp64 on the CPU for the chosen (batch rows, heads); metadata rows are sliced alike."""
    metadata = oracle_args.pop("metadata", None)
    idx_b = torch.tensor(rows)
    idx_h = torch.tensor(heads)
    pick = lambda t: t.detach().cpu()[idx_b][:, idx_h]
    qo, ko, vo = (pick(t).double().requires_grad_() for t in (q, k, v))
    md = None if metadata is None else tuple(t.cpu()[idx_b] for t in metadata)
    exp = oracle.cyclic_attention_oracle(qo, ko, vo, metadata=md, **oracle_args)
    exp_grads = torch.autograd.grad(exp, (qo, ko, vo), pick(probe).double())
    assert_parity(pick(out).float(), exp, what=f"{what} out", **BF16_TOL)
    for g, e, name in zip(grads, exp_grads, ("dq", "dk", "dv")):
        assert_parity(pick(g).float(), e, what=f"{what} {name}", **BF16_TOL)


@pytest.mark.parametrize("documents", [True, False])
@pytest.mark.parametrize("residue", [0, 3, 7])
def test_training_shape_forward_and_gradients(residue, documents):
    torch.manual_seed(residue)
    docs = geometric_documents(B, T, 1024, seed=7)
    groups = [torch.arange(r, T, S) for r in range(S)]
    metadata = None
    if documents:
        metadata = tuple(t.cuda() for t in prepare_feedback_metadata(docs, groups, T, use_dummy_token=False)[residue])
    q = torch.randn(B, H, T // S, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, H, T, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, H, T, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    probe = torch.randn(B, H, T // S, D, device="cuda", dtype=torch.bfloat16)
    # the resident-query backward pipeline is the one that serves this shape: no dQ accumulator in its scratch
    rows_total = B * H * (T // S)
    assert backward_scratch_bytes(q, k, v) == ((rows_total + 63) // 64) * 64 * 4
    _native.device_status(True)
    out = cyclic_attention(q, k, v, query_stride=S, query_offset=residue, strict_past=True, metadata=metadata, backend="sm100")
    grads = torch.autograd.grad(out, (q, k, v), probe)
    assert _native.device_status(True) == 0
    rows = rows_with_most_documents(docs, 4)
    heads = [0, 5, 10, 15]
    compare_slice(
        out, grads, q, k, v, probe, rows, heads, f"residue {residue}", query_stride=S, query_offset=residue,
        strict_past=True, metadata=metadata,
    )
    if documents:
        starts = torch.ones_like(docs, dtype=torch.bool)
        starts[:, 1:] = docs[:, 1:] != docs[:, :-1]
        first_rows = starts[:, residue::S].cuda()
        assert out.transpose(1, 2)[first_rows].abs().max().item() == 0
        assert grads[0].transpose(1, 2)[first_rows].abs().max().item() == 0


@pytest.mark.parametrize("documents", [True, False])
def test_training_shape_with_a_leading_dummy(documents):
    """256 queries against 2049 key slots: slot 0 is the shared dummy every query sees (17 key tiles)."""
    torch.manual_seed(11)
    residue = 5
    docs = geometric_documents(B, T, 1024, seed=9)
    groups = [torch.arange(r, T, S) for r in range(S)]
    metadata = None
    if documents:
        metadata = tuple(t.cuda() for t in prepare_feedback_metadata(docs, groups, T + 1, use_dummy_token=True)[residue])
    q = torch.randn(B, H, T // S, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, H, T + 1, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, H, T + 1, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    probe = torch.randn(B, H, T // S, D, device="cuda", dtype=torch.bfloat16)
    _native.device_status(True)
    out = cyclic_attention(q, k, v, query_stride=S, query_offset=residue, strict_past=False, metadata=metadata, backend="sm100")
    grads = torch.autograd.grad(out, (q, k, v), probe)
    assert _native.device_status(True) == 0
    compare_slice(
        out, grads, q, k, v, probe, rows_with_most_documents(docs, 3), [1, 14], "dummy", query_stride=S,
        query_offset=residue, strict_past=False, metadata=metadata,
    )


def test_jacobi_prefill_shape_forward_and_gradients():
    """B=8, H=16, T=2048, documents of mean length 512, through strict_causal_attention(metadata=...)."""
    batch = 8
    docs = geometric_documents(batch, T, 512, seed=7)
    schedule = prepare_strict_causal_metadata(docs.cuda(), T)
    rows, heads = rows_with_most_documents(docs, 2), [3, 12]
    cpu_schedule = prepare_strict_causal_metadata(docs[torch.tensor(rows)], T)
    for it in range(2):
        torch.manual_seed(100 + it)
        q = (torch.randn(batch, H, T, D) / 8).bfloat16().cuda().requires_grad_()
        k = torch.randn(batch, H, T, D).bfloat16().cuda().requires_grad_()
        v = torch.randn(batch, H, T, D).bfloat16().cuda().requires_grad_()
        probe = torch.randn(batch, T, H, D).bfloat16().cuda()
        _native.device_status(True)
        out = strict_causal_attention(q, k, v, metadata=schedule, backend="sm100")
        grads = torch.autograd.grad(out, (q, k, v), probe)
        assert _native.device_status(True) == 0
        idx_b, idx_h = torch.tensor(rows), torch.tensor(heads)
        pick = lambda t: t.detach().cpu()[idx_b][:, idx_h]
        qo, ko, vo = (pick(t).double().requires_grad_() for t in (q, k, v))
        exp = oracle.strict_causal_oracle(qo, ko, vo, metadata=cpu_schedule)
        exp_grads = torch.autograd.grad(exp, (qo, ko, vo), probe.cpu()[idx_b][:, :, idx_h].double())
        assert_parity(out.detach().cpu()[idx_b][:, :, idx_h].float(), exp, what=f"iteration {it} out", **BF16_TOL)
        for g, e, name in zip(grads, exp_grads, ("dq", "dk", "dv")):
            assert_parity(pick(g).float(), e, what=f"iteration {it} {name}", **BF16_TOL)
        starts = torch.ones_like(docs, dtype=torch.bool)
        starts[:, 1:] = docs[:, 1:] != docs[:, :-1]
        assert out[starts.cuda()].abs().max().item() == 0  # each document's first token
