"""KV-pool projection path: the oracle against the upstream vectors (CPU); the kernels against the oracle and the
vectors (GPU, through the C ABI)."""

from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import BF16_TOL, F32_TOL, assert_parity
from oracle.pool_oracle import mix_pool_oracle, project_pool_oracle

VECTORS = np.load(Path(__file__).resolve().parent / "golden" / "pool_vectors.npz")
CASES = sorted({name.split("/", 1)[0] for name in VECTORS.files})
HKV, D = 2, 64  # of the stored cases


def get(case, name):
    key = f"{case}/{name}"
    return torch.from_numpy(VECTORS[key]) if key in VECTORS.files else None


def state(case):
    prefix = f"{case}/state/"
    return {name[len(prefix):]: torch.from_numpy(VECTORS[name]) for name in VECTORS.files if name.startswith(prefix)}


def oracle_params(st):
    return {
        "pre_mix_k": st["pre_mix_k_weight"], "pre_mix_v": st["pre_mix_v_weight"],
        "router_k_weight": st["mixer.k_router.linear.weight"], "router_k_bias": st["mixer.k_router.linear.bias"],
        "router_v_weight": st["mixer.v_router.linear.weight"], "router_v_bias": st["mixer.v_router.linear.bias"],
        "gain_k": st["post_mix.k_gain"], "gain_v": st["post_mix.v_gain"],
        "proj_k": st["k_proj_weight"], "proj_v": st["v_proj_weight"], "k_norm": st["k_norm_weight"],
    }


def oracle_for(case, stacked, cos, sin, dummy):
    return project_pool_oracle(
        stacked, oracle_params(state(case)), cos, sin, kv_heads=HKV, head_dim=D,
        route_stride=int(get(case, "route_stride")), dynamic=bool(get(case, "dynamic")), dummy=dummy,
    )


@pytest.mark.parametrize("case", CASES)
def test_oracle_matches_upstream_vectors(case):
    stacked, cos, sin, dummy = (get(case, n) for n in ("stacked", "cos", "sin", "dummy"))
    keys, values = oracle_for(case, stacked, cos, sin, dummy)
    tol = dict(max_abs_tol=5e-5, rel_l2_tol=1e-5)  # fp32 round-off of the stored upstream results
    assert_parity(keys, get(case, "keys").double(), what="keys", **tol)
    assert_parity(values, get(case, "values").double(), what="values", **tol)
    # the decode row: the last token alone, with the last row of the position tables
    token_keys, token_values = oracle_for(case, stacked[:, -1:], cos[:, -1:], sin[:, -1:], None)
    assert_parity(token_keys.transpose(0, 1), get(case, "token_keys").double(), what="token keys", **tol)
    assert_parity(token_values.transpose(0, 1), get(case, "token_values").double(), what="token values", **tol)


def test_static_router_ignores_the_router_weight():
    case = "static"
    st = oracle_params(state(case))
    stacked, cos, sin = (get(case, n) for n in ("stacked", "cos", "sin"))
    base = project_pool_oracle(stacked, st, cos, sin, kv_heads=HKV, head_dim=D, dynamic=False)
    st["router_k_weight"] = torch.randn_like(st["router_k_weight"])
    again = project_pool_oracle(stacked, st, cos, sin, kv_heads=HKV, head_dim=D, dynamic=False)
    assert torch.equal(base[0], again[0])


# ------------------------------------------------------------------------------------------------------- GPU
gpu = [pytest.mark.gpu, pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")]


def build_pool(case, dtype, **kw):
    from white_matter_b200 import KVPool

    st = state(case)
    layers, hidden = st["pre_mix_k_weight"].shape
    channels = st["post_mix.k_gain"].shape[0]
    pool = KVPool(
        hidden, HKV, D, layers, channels, router_layer_stride=int(get(case, "route_stride")),
        router_dynamic=bool(get(case, "dynamic")), device="cuda", dtype=dtype, **kw,
    )
    pool.load_state_dict(st)
    return pool


@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")
@pytest.mark.parametrize("chunk_rows", [1024, 4])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", CASES)
def test_kernels_match_oracle_and_upstream(case, dtype, chunk_rows):
    pool = build_pool(case, dtype, chunk_rows=chunk_rows)
    stacked, cos, sin, dummy = (get(case, n) for n in ("stacked", "cos", "sin", "dummy"))
    x = stacked.cuda().to(dtype)
    dummy_dev = None if dummy is None else dummy.cuda()
    keys, values = pool.project_sequence(x, (cos.cuda(), sin.cuda()), dummy_token=dummy_dev)
    assert keys.dtype == dtype and keys.shape == tuple(get(case, "keys").shape)
    # the oracle sees the inputs as the kernel does (rounded to the compute dtype)
    dummy_seen = None if dummy is None else dummy.to(dtype)
    want_k, want_v = oracle_for(case, x.cpu(), cos, sin, dummy_seen)
    tol = F32_TOL if dtype == torch.float32 else BF16_TOL
    assert_parity(keys.cpu().double(), want_k, what="keys vs oracle", **tol)
    assert_parity(values.cpu().double(), want_v, what="values vs oracle", **tol)
    assert_parity(keys.cpu().double(), get(case, "keys").double(), what="keys vs upstream", **tol)
    assert_parity(values.cpu().double(), get(case, "values").double(), what="values vs upstream", **tol)
    layers = x.shape[2]
    token_keys, token_values = pool.project_token([x[:, -1:, l] for l in range(layers)], (cos[:, -1:].cuda(), sin[:, -1:].cuda()))
    assert token_keys.shape == tuple(get(case, "token_keys").shape)
    assert_parity(token_keys.cpu().double(), get(case, "token_keys").double(), what="token keys vs upstream", **tol)
    assert_parity(token_values.cpu().double(), get(case, "token_values").double(), what="token values vs upstream", **tol)


@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")
def test_rows_are_published_into_the_decode_cache_in_place():
    """project_into writes slots of a pool in the decode wire format; untouched slots keep their contents (NaN)."""
    from white_matter_b200 import KVPoolCache

    case, dtype = "dynamic", torch.bfloat16
    pool = build_pool(case, dtype)
    stacked, cos, sin = (get(case, n) for n in ("stacked", "cos", "sin"))
    batch, tokens = stacked.shape[:2]
    channels = pool.num_kv_channels
    cache = KVPoolCache(batch, channels, HKV, 16, D, use_dummy_token=True, dtype=dtype, device="cuda")
    cache.keys.fill_(float("nan"))
    cache.values.fill_(float("nan"))
    pool.project_into(stacked.cuda().to(dtype), (cos.cuda(), sin.cuda()), cache.keys, cache.values, token_offset=3)
    want_k, want_v = oracle_for(case, stacked.to(dtype), cos, sin, None)
    got_k = cache.keys[:, :, 3 : 3 + tokens].view(batch, channels, HKV, tokens, D)
    got_v = cache.values[:, :, 3 : 3 + tokens].view(batch, channels, HKV, tokens, D)
    assert_parity(got_k.cpu().double(), want_k, what="published keys", **BF16_TOL)
    assert_parity(got_v.cpu().double(), want_v, what="published values", **BF16_TOL)
    untouched = torch.ones(cache.keys.shape[2], dtype=torch.bool)
    untouched[3 : 3 + tokens] = False
    assert cache.keys[:, :, untouched.cuda()].isnan().all() and cache.values[:, :, untouched.cuda()].isnan().all()


@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")
@pytest.mark.parametrize("dynamic,stride", [(True, 1), (True, 4), (False, 1)])
def test_model_sized_pool_matches_the_oracle(dynamic, stride):
    """25 sources of width 1024 into 8 channels of 16 heads (the full model's pool), random parameters, 2 x 96 rows."""
    from white_matter_b200 import KVPool

    torch.manual_seed(5)
    layers, hidden, channels, heads, dim, batch, tokens = 25, 1024, 8, 16, 64, 2, 96
    pool = KVPool(hidden, heads, dim, layers, channels, router_layer_stride=stride, router_dynamic=dynamic, device="cuda", chunk_rows=64)
    n = pool.num_sources
    st = {
        "pre_mix_k_weight": 1 + 0.3 * torch.randn(layers, hidden), "pre_mix_v_weight": 1 + 0.3 * torch.randn(layers, hidden),
        "k_proj_weight": 0.02 * torch.randn(channels, heads * dim, hidden), "v_proj_weight": 0.02 * torch.randn(channels, heads * dim, hidden),
        "k_norm_weight": 1 + 0.2 * torch.randn(channels, dim),
        "mixer.k_router.linear.weight": 0.004 * torch.randn(channels * layers, n * hidden),
        "mixer.v_router.linear.weight": 0.004 * torch.randn(channels * layers, n * hidden),
        "mixer.k_router.linear.bias": 0.5 * torch.randn(channels * layers), "mixer.v_router.linear.bias": 0.5 * torch.randn(channels * layers),
        "post_mix.k_gain": 1 + 0.2 * torch.randn(channels, hidden), "post_mix.v_gain": 1 + 0.2 * torch.randn(channels, hidden),
    }
    pool.load_state_dict(st)
    stacked = (torch.randn(batch, tokens, layers, hidden) * (0.5 + torch.rand(1, 1, layers, 1))).bfloat16()
    angle = torch.rand(1, tokens, dim // 2) * 6.283
    cos, sin = torch.cat((angle.cos(), angle.cos()), -1), torch.cat((angle.sin(), angle.sin()), -1)
    keys, values = pool.project_sequence(stacked.cuda(), (cos.cuda(), sin.cuda()))
    want_k, want_v = project_pool_oracle(
        stacked, oracle_params(st), cos, sin, kv_heads=heads, head_dim=dim, route_stride=stride, dynamic=dynamic
    )
    assert_parity(keys.cpu().double(), want_k, what="keys", **BF16_TOL)
    assert_parity(values.cpu().double(), want_v, what="values", **BF16_TOL)


@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", ["dynamic", "strided_dummy", "static"])
def test_mix_entry_point_applies_the_post_mix_gain_when_given(case, dtype):
    """wm_pool_mix called directly with gain tables (the host module folds them into the projections instead)."""
    from white_matter_b200 import _native

    pool = build_pool(case, dtype)
    st = state(case)
    x = get(case, "stacked").cuda().to(dtype)
    batch, tokens, layers, hidden = x.shape
    rows, k = batch * tokens, pool.num_kv_channels
    mixed = torch.empty(2, k, rows, hidden, device="cuda", dtype=dtype)
    a = _native.PoolMixArgs()
    a.stacked, a.stacked_strides = x.data_ptr(), _native._Strides(x.stride(0), x.stride(1), x.stride(2))
    a.pre_mix_k, a.pre_mix_v = pool.pre_mix_k_weight.data_ptr(), pool.pre_mix_v_weight.data_ptr()
    a.bias_k, a.bias_v = pool.k_router_bias.data_ptr(), pool.v_router_bias.data_ptr()
    keep = []
    if pool.router_dynamic:
        flat = x[:, :, pool.source_start :: pool.router_layer_stride].reshape(rows, pool.num_sources, hidden).transpose(0, 1)
        both = torch.bmm(flat, pool._route)  # K side and V side in every row
        keep = [both[..., : k * layers].contiguous(), both[..., k * layers :].contiguous()]
        a.partial_k, a.partial_v = keep[0].data_ptr(), keep[1].data_ptr()  # separate tensors: the default row stride
        a.route_start, a.route_stride, a.n_routed = pool.source_start, pool.router_layer_stride, pool.num_sources
    a.gain_k, a.gain_v = pool.k_gain.data_ptr(), pool.v_gain.data_ptr()
    a.mixed_k, a.mixed_v = mixed[0].data_ptr(), mixed[1].data_ptr()
    a.dtype = _native.dtype_code(dtype)
    a.batch, a.tokens, a.sources, a.channels, a.hidden = batch, tokens, layers, k, hidden
    a.source_eps, a.mix_eps = pool.rms_norm_eps, pool.mix_norm_eps
    _native.call("wm_pool_mix", a, x.device)
    want = mix_pool_oracle(x.cpu(), oracle_params(st), route_stride=pool.router_layer_stride, dynamic=pool.router_dynamic)
    tol = F32_TOL if dtype == torch.float32 else BF16_TOL
    assert_parity(mixed.cpu().double(), want, what="gained mixtures", **tol)


@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")
def test_argument_errors():
    pool = build_pool("dynamic", torch.bfloat16)
    stacked, cos, sin = (get("dynamic", n) for n in ("stacked", "cos", "sin"))
    with pytest.raises(ValueError, match="expected"):
        pool.project_sequence(stacked.cuda().bfloat16()[:, :, :-1], (cos.cuda(), sin.cuda()))
    with pytest.raises(ValueError, match="built for"):
        pool.project_sequence(stacked.cuda(), (cos.cuda(), sin.cuda()))
    with pytest.raises(ValueError, match="position embeddings"):
        pool.project_sequence(stacked.cuda().bfloat16(), (cos.cuda()[:, :-1], sin.cuda()[:, :-1]))
    with pytest.raises(ValueError, match="CUDA"):
        pool.project_sequence(stacked.bfloat16(), (cos, sin))
