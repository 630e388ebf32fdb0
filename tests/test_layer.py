"""Query preparation of the attention layer: the oracle against the upstream vectors (CPU), the kernels against the
oracle and the vectors (GPU, through the C ABI)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import BF16_TOL, F32_TOL, assert_parity
from oracle.layer_oracle import prepare_queries_oracle

VECTORS = np.load(Path(__file__).resolve().parent / "golden" / "layer_vectors.npz")
CASES = sorted({name.rsplit("/", 1)[0] for name in VECTORS.files})


def load(case):
    return {name: torch.from_numpy(VECTORS[f"{case}/{name}"]) for name in ("projected", "weight", "cos", "sin", "out", "probe", "dx", "dw")}


@pytest.mark.parametrize("case", CASES)
def test_oracle_matches_upstream_vectors(case):
    v = load(case)
    x = v["projected"].double().requires_grad_()
    w = v["weight"].double().requires_grad_()
    out = prepare_queries_oracle(x, w, v["cos"], v["sin"])
    dx, dw = torch.autograd.grad(out, (x, w), v["probe"].double())
    if case.endswith("f32"):
        tol = dict(max_abs_tol=2e-5, rel_l2_tol=5e-6)  # fp32 round-off of the stored upstream results
    else:
        tol = dict(max_abs_tol=6e-2, rel_l2_tol=1e-2)  # upstream rounds to bf16 after every one of its five operations
    assert_parity(out, v["out"].double(), what="out", **tol)
    assert_parity(dx, v["dx"].double(), what="dx", **tol)
    assert_parity(dw, v["dw"].double(), what="dw", **tol)


def test_rotation_is_the_upstream_permutation():
    # modules/rotary.py:30-34: rotate_half(x) = cat(-x2, x1); with cos = 0 and sin = 1 the result is that rotation
    x = torch.arange(2 * 3 * 1 * 64, dtype=torch.float64).reshape(2, 3, 1, 64) + 1
    ones = torch.ones(64, dtype=torch.float64)
    out = prepare_queries_oracle(x, ones, torch.zeros(1, 3, 64), torch.ones(1, 3, 64), eps=0.0)
    normed = (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True))).transpose(1, 2)
    assert torch.allclose(out, torch.cat((-normed[..., 32:], normed[..., :32]), -1))


@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")
@pytest.mark.parametrize("case", CASES)
def test_kernels_match_oracle_and_upstream(case):
    from white_matter_b200 import prepare_queries

    v = load(case)
    dtype = torch.float32 if case.endswith("f32") else torch.bfloat16
    x = v["projected"].to("cuda", dtype).requires_grad_()
    w = v["weight"].to("cuda", dtype).requires_grad_()
    cos, sin, probe = (v[n].to("cuda", dtype) for n in ("cos", "sin", "probe"))
    out = prepare_queries(x, w, cos, sin, eps=1e-6, out_dtype=dtype)
    assert out.shape == (x.shape[0], x.shape[2], x.shape[1], x.shape[3]) and out.is_contiguous() and out.dtype == dtype
    dx, dw = torch.autograd.grad(out, (x, w), probe)
    # the reference arithmetic on the same (rounded) inputs
    xo, wo = x.detach().double().cpu().requires_grad_(), w.detach().double().cpu().requires_grad_()
    exp = prepare_queries_oracle(xo, wo, cos.cpu(), sin.cpu())
    edx, edw = torch.autograd.grad(exp, (xo, wo), probe.double().cpu())
    tol = F32_TOL if dtype == torch.float32 else BF16_TOL
    assert_parity(out.double().cpu(), exp, what="out", **tol)
    assert_parity(dx.double().cpu(), edx, what="dx", **tol)
    assert_parity(dw.double().cpu(), edw, what="dw", **tol)
    # and the stored upstream results (bf16: upstream's own intermediate roundings included)
    loose = F32_TOL if dtype == torch.float32 else dict(max_abs_tol=6e-2, rel_l2_tol=1e-2)
    assert_parity(out.double().cpu(), v["out"].double(), what="out vs upstream", **loose)
    assert_parity(dx.double().cpu(), v["dx"].double(), what="dx vs upstream", **loose)


@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")
def test_layer_function_matches_the_two_steps_and_feeds_o_proj_without_a_copy():
    from white_matter_b200 import cyclic_attention, cyclic_attention_layer, prepare_queries

    torch.manual_seed(2)
    b, t, h, d, stride = 2, 64, 4, 64, 4
    projected = torch.randn(b, t // stride, h * d, device="cuda", dtype=torch.bfloat16)
    weight = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
    angles = torch.rand(1, t // stride, d, device="cuda") * 6
    cos, sin = angles.cos().bfloat16(), angles.sin().bfloat16()
    k = torch.randn(b, h, t, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn_like(k)
    got = cyclic_attention_layer(projected, weight, cos, sin, k, v, query_stride=stride, query_offset=1, strict_past=True)
    q = prepare_queries(projected, weight, cos, sin)
    ref = cyclic_attention(q, k, v, query_stride=stride, query_offset=1, strict_past=True)
    assert got.shape == (b, t // stride, h * d)
    assert torch.equal(got, ref.transpose(1, 2).reshape(b, t // stride, h * d))
    assert got._is_view() and got.is_contiguous()  # the (B,T,H*D) matrix is a view of the operator's (B,T,H,D) storage


@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")
def test_fp32_projection_to_bf16_queries_and_strided_input():
    from white_matter_b200 import prepare_queries

    torch.manual_seed(4)
    wide = torch.randn(2, 33, 5, 128 + 64, device="cuda")  # the query heads are a slice of a wider projection
    x = wide[..., :128].requires_grad_()
    w = torch.rand(128, device="cuda") + 0.5
    angles = torch.rand(2, 33, 128, device="cuda") * 6
    out = prepare_queries(x, w, angles.cos(), angles.sin(), out_dtype=torch.bfloat16)
    assert out.dtype == torch.bfloat16
    exp = prepare_queries_oracle(x.detach().cpu(), w.cpu(), angles.cos().cpu(), angles.sin().cpu())
    assert_parity(out.double().cpu(), exp, what="out", **BF16_TOL)
    (dx,) = torch.autograd.grad(out, (x,), torch.ones_like(out))
    assert dx.shape == x.shape


def test_contract_errors():
    from white_matter_b200 import prepare_queries

    x = torch.randn(1, 4, 2, 64)
    with pytest.raises(ValueError, match="requires CUDA"):
        prepare_queries(x, torch.ones(64), torch.ones(1, 4, 64), torch.ones(1, 4, 64))
