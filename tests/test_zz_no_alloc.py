"""The allocation-free pool read (`wm_strict_decode_no_alloc`) against the regular entry point.

Collected last on purpose: a run that stops at the first failure has then
already exercised every other test.  The entry point exists for callers that
were handed device buffers but have no allocator to lend to the library, so
its split partials live in an array inside the library image.
"""

import ctypes

import pytest
import torch

from white_matter_b200 import _native, operators, strict_causal_attention

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")]


def _problem(seed, batch=5, heads=8, kv_heads=4, slots=700, dim=64):
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(batch, heads, 1, dim, generator=gen).bfloat16().cuda()
    k = torch.randn(batch, kv_heads, slots, dim, generator=gen).bfloat16().cuda()
    v = torch.randn(batch, kv_heads, slots, dim, generator=gen).bfloat16().cuda()
    lengths = torch.randint(0, slots + 1, (batch,), generator=gen).to(torch.int32).cuda()
    for b in range(batch):
        k[b, :, int(lengths[b]):] = float("nan")  # unused capacity must never be read
        v[b, :, int(lengths[b]):] = float("nan")
    return q, k, v, lengths


def test_two_calls_in_a_row_match_the_allocating_entry_point():
    out = torch.full((5, 1, 8, 64), float("nan"), dtype=torch.bfloat16, device="cuda")
    for seed in (11, 12):  # the second call finds the first call's partials in the shared array
        q, k, v, lengths = _problem(seed)
        expected = strict_causal_attention(q, k, v, query_start=lengths, kv_lengths=lengths)
        before = torch.cuda.memory_stats()["allocation.all.current"]
        got = operators.strict_decode_no_alloc(q, k, v, out, lengths, 0, lengths, None, False, 64**-0.5)
        assert torch.cuda.memory_stats()["allocation.all.current"] == before  # nothing was taken from the allocator
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        # same kernels, same split layout: the two entry points agree bit for bit (tolerance of the suite: 2e-2)
        assert torch.equal(got, expected)


def test_rejects_problems_beyond_the_built_in_scratch():
    lib = _native.load_library()
    q = torch.zeros(64, 64, 1, 64, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(64, 64, 8192, 64, dtype=torch.bfloat16, device="meta")
    a = _native.AttnArgs()
    a.q = a.k = a.v = a.out = q.data_ptr()  # never dereferenced: the call is refused before any launch
    a.q_strides = _native.strides3(q)
    a.k_strides = a.v_strides = _native.strides3(k)
    a.out_strides = _native.strides3(q)
    a.dtype = _native.WM_BF16
    a.batch, a.q_heads, a.q_len, a.head_dim = q.shape
    a.kv_heads, a.k_len = 64, 8192
    a.scale, a.mask = 0.125, _native.WM_MASK_STRICT
    assert lib.wm_strict_decode_workspace_bytes(ctypes.byref(a)) > 16 << 20
    status = lib.wm_strict_decode_no_alloc(ctypes.byref(a), None)
    assert status == -4 and b"built-in array" in lib.wm_last_error()
