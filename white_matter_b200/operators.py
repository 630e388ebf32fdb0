"""Registered operators in front of the C ABI (``torch.library`` custom ops).

The schemas mirror the operator layer the upstream kernels sit behind
(src/white_matter/ops/cyclic_attention/_tilelang/registration.py:164-302 and
src/white_matter/ops/flash_attention.py:15-24): the same five roles --
``cyclic_attn_fwd``, ``cyclic_attn_bwd``, ``cyclic_attn_doc_fwd``,
``cyclic_attn_doc_bwd`` and the cached single-query read -- plus the strict
prefill pair, the packed-schedule pair and source mixing, all in the
``wm_b200`` namespace.  Each op allocates its outputs, fills a plain argument
record and calls one entry point of libwm_b200.so on the current stream; there
is no host synchronisation and no fallback implementation.

PyTorch is used for device memory, streams and autograd bookkeeping only.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _native
from ._native import AttnArgs, MixArgs

Tensor = torch.Tensor

_KERNELS = {"auto": _native.WM_KERNEL_AUTO, "simt": _native.WM_KERNEL_SIMT, "tcgen05": _native.WM_KERNEL_TCGEN05}


def kernel_code(name: str) -> int:
    return _KERNELS[name]


# --------------------------------------------------------------------------- helpers


def _unit_inner(x: Tensor, dtype: torch.dtype) -> Tensor:
    """A view with unit stride in head_dim and the operator dtype (copy only if needed)."""
    if x.dtype != dtype:
        x = x.to(dtype)
    if x.stride(-1) != 1:
        x = x.contiguous()
    return x


def _int32(x: Tensor) -> Tensor:
    if x.dtype != torch.int32:
        x = x.to(torch.int32)
    return x if x.is_contiguous() else x.contiguous()


def _base_args(q: Tensor, k: Tensor, v: Tensor, scale: float, mask: int, kernel: int) -> AttnArgs:
    a = AttnArgs()
    a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.q_strides, a.k_strides, a.v_strides = _native.strides3(q), _native.strides3(k), _native.strides3(v)
    a.dtype = _native.dtype_code(q.dtype)
    a.batch, a.q_heads, a.q_len, a.head_dim = q.shape
    a.kv_heads, a.k_len = k.shape[1], k.shape[2]
    a.scale = scale
    a.mask = mask
    a.kernel = kernel
    return a


def _set_out(a: AttnArgs, out_bhtd: Tensor, lse: Optional[Tensor]) -> None:
    a.out = out_bhtd.data_ptr()
    a.out_strides = _native.strides3(out_bhtd)
    a.lse = lse.data_ptr() if lse is not None else None


def _set_grads(a: AttnArgs, dout: Tensor, dq: Tensor, dk: Tensor, dv: Tensor) -> None:
    a.dout, a.dq, a.dk, a.dv = dout.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.dout_strides = _native.strides3(dout)
    a.dq_strides, a.dk_strides, a.dv_strides = _native.strides3(dq), _native.strides3(dk), _native.strides3(dv)


def _attach_workspace(a, nbytes: int, device: torch.device) -> Optional[Tensor]:
    if nbytes == 0:
        return None
    buf = torch.empty(nbytes, dtype=torch.uint8, device=device)
    a.workspace = buf.data_ptr()
    a.workspace_bytes = nbytes
    return buf


def _bwd_workspace(a: AttnArgs, device: torch.device) -> Optional[Tensor]:
    nbytes = _native.load_library().wm_attn_bwd_workspace_bytes(ctypes.byref(a))
    return _attach_workspace(a, nbytes, device)


def _new_output(q: Tensor) -> tuple[Tensor, Tensor]:
    """(B,T,H,D) storage viewed as (B,H,T,D), and the (B,H,T) fp32 log-sum-exp."""
    batch, heads, length, dim = q.shape
    out = torch.empty((batch, length, heads, dim), dtype=q.dtype, device=q.device).transpose(1, 2)
    lse = torch.empty((batch, heads, length), dtype=torch.float32, device=q.device)
    return out, lse


def _fake_output(q: Tensor) -> tuple[Tensor, Tensor]:
    batch, heads, length, dim = q.shape
    out = torch.empty((batch, length, heads, dim), dtype=q.dtype, device=q.device).transpose(1, 2)
    return out, torch.empty((batch, heads, length), dtype=torch.float32, device=q.device)


def _fake_grads(q: Tensor, k: Tensor, v: Tensor) -> tuple[Tensor, Tensor, Tensor]:
    return (
        torch.empty(q.shape, dtype=q.dtype, device=q.device),
        torch.empty(k.shape, dtype=q.dtype, device=q.device),
        torch.empty(v.shape, dtype=q.dtype, device=q.device),
    )


def _new_grads(q: Tensor, k: Tensor, v: Tensor) -> tuple[Tensor, Tensor, Tensor]:
    return _fake_grads(q, k, v)


# --------------------------------------------------------------------------- cyclic


def _cyclic_args(Q, K, V, docs, K_stride, residue, kernel, softmax_scale=0.0):
    if not -1 <= residue < K_stride:
        raise ValueError(f"cyclic residue must be in [-1, {K_stride}), got {residue}")
    q = _unit_inner(Q, Q.dtype)
    k = _unit_inner(K, Q.dtype)
    v = _unit_inner(V, Q.dtype)
    scale = float(softmax_scale) if softmax_scale > 0.0 else Q.shape[-1] ** -0.5
    a = _base_args(q, k, v, scale, _native.WM_MASK_CYCLIC, kernel)
    a.query_stride, a.query_offset = K_stride, residue
    keep = [q, k, v]
    if docs is not None:
        tables = [_int32(t) for t in docs]
        a.q_seg, a.k_seg, a.q_key_start, a.k_query_end = (t.data_ptr() for t in tables)
        keep += tables
    return a, keep


def _cyclic_fwd(Q, K, V, docs, K_stride, residue, kernel, softmax_scale=0.0):
    a, keep = _cyclic_args(Q, K, V, docs, K_stride, residue, kernel, softmax_scale)
    out, lse = _new_output(Q)
    _set_out(a, out, lse)
    _native.call("wm_cyclic_attn_fwd" if docs is None else "wm_cyclic_attn_doc_fwd", a, Q.device)
    return out, lse


def _cyclic_bwd(Q, K, V, docs, Out, Lse, dOut, K_stride, residue, kernel, softmax_scale=0.0):
    a, keep = _cyclic_args(Q, K, V, docs, K_stride, residue, kernel, softmax_scale)
    out = _unit_inner(Out, Q.dtype)
    dout = _unit_inner(dOut, Q.dtype)
    lse = Lse.contiguous()
    _set_out(a, out, lse)
    dq, dk, dv = _new_grads(Q, K, V)
    _set_grads(a, dout, dq, dk, dv)
    ws = _bwd_workspace(a, Q.device)
    _native.call("wm_cyclic_attn_bwd" if docs is None else "wm_cyclic_attn_doc_bwd", a, Q.device)
    del ws, keep
    return dq, dk, dv


@torch.library.custom_op("wm_b200::cyclic_attn_fwd", mutates_args=())
def cyclic_attn_fwd(
    Q: Tensor, K: Tensor, V: Tensor, K_stride: int, residue: int, block_M: int, softmax_scale: float = 0.0
) -> tuple[Tensor, Tensor]:
    """Out (B,HQ,Q,D) view of (B,Q,HQ,D) storage and Lse (B,HQ,Q); block_M selects the kernel family.

    ``softmax_scale`` (not in the upstream schema, which always scales by head_dim**-0.5) is the multiplier of the
    scores; 0 stands for head_dim**-0.5."""
    return _cyclic_fwd(Q, K, V, None, K_stride, residue, block_M, softmax_scale)


@cyclic_attn_fwd.register_fake
def _(Q, K, V, K_stride, residue, block_M, softmax_scale=0.0):
    return _fake_output(Q)


@torch.library.custom_op("wm_b200::cyclic_attn_bwd", mutates_args=())
def cyclic_attn_bwd(
    Q: Tensor,
    K: Tensor,
    V: Tensor,
    Out: Tensor,
    Lse: Tensor,
    dOut: Tensor,
    K_stride: int,
    residue: int,
    block_M: int,
    softmax_scale: float = 0.0,
) -> tuple[Tensor, Tensor, Tensor]:
    return _cyclic_bwd(Q, K, V, None, Out, Lse, dOut, K_stride, residue, block_M, softmax_scale)


@cyclic_attn_bwd.register_fake
def _(Q, K, V, Out, Lse, dOut, K_stride, residue, block_M, softmax_scale=0.0):
    return _fake_grads(Q, K, V)


@torch.library.custom_op("wm_b200::cyclic_attn_doc_fwd", mutates_args=())
def cyclic_attn_doc_fwd(
    Q: Tensor,
    K: Tensor,
    V: Tensor,
    QSeg: Tensor,
    KSeg: Tensor,
    QStart: Tensor,
    KQEnd: Tensor,
    K_stride: int,
    residue: int,
    block_M: int,
    softmax_scale: float = 0.0,
) -> tuple[Tensor, Tensor]:
    return _cyclic_fwd(Q, K, V, (QSeg, KSeg, QStart, KQEnd), K_stride, residue, block_M, softmax_scale)


@cyclic_attn_doc_fwd.register_fake
def _(Q, K, V, QSeg, KSeg, QStart, KQEnd, K_stride, residue, block_M, softmax_scale=0.0):
    return _fake_output(Q)


@torch.library.custom_op("wm_b200::cyclic_attn_doc_bwd", mutates_args=())
def cyclic_attn_doc_bwd(
    Q: Tensor,
    K: Tensor,
    V: Tensor,
    QSeg: Tensor,
    KSeg: Tensor,
    QStart: Tensor,
    KQEnd: Tensor,
    Out: Tensor,
    Lse: Tensor,
    dOut: Tensor,
    K_stride: int,
    residue: int,
    block_M: int,
    softmax_scale: float = 0.0,
) -> tuple[Tensor, Tensor, Tensor]:
    return _cyclic_bwd(Q, K, V, (QSeg, KSeg, QStart, KQEnd), Out, Lse, dOut, K_stride, residue, block_M, softmax_scale)


@cyclic_attn_doc_bwd.register_fake
def _(Q, K, V, QSeg, KSeg, QStart, KQEnd, Out, Lse, dOut, K_stride, residue, block_M, softmax_scale=0.0):
    return _fake_grads(Q, K, V)


def _cyclic_setup(ctx, inputs, output):
    *tensors, ctx.K_stride, ctx.residue, ctx.block_M, ctx.softmax_scale = inputs
    ctx.save_for_backward(*tensors, *output)
    ctx.set_materialize_grads(False)  # no zero fill for the unused gradient of Lse on every backward call


def _cyclic_backward(ctx, dOut, dLse):
    tensors = ctx.saved_tensors
    if dOut is None:
        dOut = torch.zeros_like(tensors[-2])
    op = cyclic_attn_doc_bwd if len(tensors) == 9 else cyclic_attn_bwd
    grads = op(*tensors, dOut, ctx.K_stride, ctx.residue, ctx.block_M, ctx.softmax_scale)
    return (*grads, *((None,) * (len(tensors) - 1)))


cyclic_attn_fwd.register_autograd(_cyclic_backward, setup_context=_cyclic_setup)
cyclic_attn_doc_fwd.register_autograd(_cyclic_backward, setup_context=_cyclic_setup)


# --------------------------------------------------------------------------- strict, dense bounds


def _strict_args(Q, K, V, query_start, query_start_value, kv_lengths, key_mask, use_dummy, scale, kernel):
    q = _unit_inner(Q, Q.dtype)
    k = _unit_inner(K, Q.dtype)
    v = _unit_inner(V, Q.dtype)
    a = _base_args(q, k, v, scale, _native.WM_MASK_STRICT, kernel)
    keep = [q, k, v]
    if query_start is not None:
        qs = query_start.contiguous()
        a.query_start = qs.data_ptr()
        a.query_start_is64 = int(qs.dtype == torch.int64)
        keep.append(qs)
    a.query_start_value = query_start_value
    if kv_lengths is not None:
        kl = kv_lengths.contiguous()
        a.kv_lengths = kl.data_ptr()
        a.kv_lengths_is64 = int(kl.dtype == torch.int64)
        keep.append(kl)
    if key_mask is not None:
        km = key_mask.contiguous().view(torch.uint8)
        a.key_mask = km.data_ptr()
        keep.append(km)
    a.use_dummy = int(use_dummy)
    return a, keep


@torch.library.custom_op("wm_b200::strict_attn_fwd", mutates_args=())
def strict_attn_fwd(
    Q: Tensor,
    K: Tensor,
    V: Tensor,
    query_start: Optional[Tensor],
    query_start_value: int,
    kv_lengths: Optional[Tensor],
    key_mask: Optional[Tensor],
    use_dummy: bool,
    scale: float,
    kernel: int,
) -> tuple[Tensor, Tensor]:
    """Out (B,H,T,D) view of (B,T,H,D) storage and Lse (B,H,T)."""
    a, keep = _strict_args(Q, K, V, query_start, query_start_value, kv_lengths, key_mask, use_dummy, scale, kernel)
    out, lse = _new_output(Q)
    _set_out(a, out, lse)
    _native.call("wm_strict_attn_fwd", a, Q.device)
    return out, lse


@strict_attn_fwd.register_fake
def _(Q, K, V, query_start, query_start_value, kv_lengths, key_mask, use_dummy, scale, kernel):
    return _fake_output(Q)


@torch.library.custom_op("wm_b200::strict_attn_bwd", mutates_args=())
def strict_attn_bwd(
    Q: Tensor,
    K: Tensor,
    V: Tensor,
    Out: Tensor,
    Lse: Tensor,
    dOut: Tensor,
    query_start: Optional[Tensor],
    query_start_value: int,
    kv_lengths: Optional[Tensor],
    key_mask: Optional[Tensor],
    use_dummy: bool,
    scale: float,
    kernel: int,
) -> tuple[Tensor, Tensor, Tensor]:
    a, keep = _strict_args(Q, K, V, query_start, query_start_value, kv_lengths, key_mask, use_dummy, scale, kernel)
    _set_out(a, _unit_inner(Out, Q.dtype), Lse.contiguous())
    dq, dk, dv = _new_grads(Q, K, V)
    dout = _unit_inner(dOut, Q.dtype)
    _set_grads(a, dout, dq, dk, dv)
    ws = _bwd_workspace(a, Q.device)
    _native.call("wm_strict_attn_bwd", a, Q.device)
    del ws, keep
    return dq, dk, dv


@strict_attn_bwd.register_fake
def _(Q, K, V, Out, Lse, dOut, query_start, query_start_value, kv_lengths, key_mask, use_dummy, scale, kernel):
    return _fake_grads(Q, K, V)


def _strict_setup(ctx, inputs, output):
    Q, K, V, query_start, ctx.query_start_value, kv_lengths, key_mask, ctx.use_dummy, ctx.scale, ctx.kernel = inputs
    ctx.save_for_backward(Q, K, V, *output)
    ctx.bounds = (query_start, kv_lengths, key_mask)
    ctx.set_materialize_grads(False)


def _strict_backward(ctx, dOut, dLse):
    Q, K, V, Out, Lse = ctx.saved_tensors
    if dOut is None:
        dOut = torch.zeros_like(Out)
    query_start, kv_lengths, key_mask = ctx.bounds
    grads = strict_attn_bwd(
        Q, K, V, Out, Lse, dOut, query_start, ctx.query_start_value, kv_lengths, key_mask, ctx.use_dummy, ctx.scale,
        ctx.kernel,
    )
    return (*grads, None, None, None, None, None, None, None)


strict_attn_fwd.register_autograd(_strict_backward, setup_context=_strict_setup)


def _strict_doc_args(Q, K, V, tables, query_start, query_start_value, kv_lengths, use_dummy, scale, kernel):
    a, keep = _strict_args(Q, K, V, query_start, query_start_value, kv_lengths, None, use_dummy, scale, kernel)
    tables = [_int32(t) for t in tables]
    a.q_seg, a.k_seg, a.q_key_start, a.k_query_end = (t.data_ptr() for t in tables)
    return a, keep + tables


@torch.library.custom_op("wm_b200::strict_doc_fwd", mutates_args=())
def strict_doc_fwd(
    Q: Tensor,
    K: Tensor,
    V: Tensor,
    QSeg: Tensor,
    KSeg: Tensor,
    QStart: Tensor,
    KQEnd: Tensor,
    query_start: Optional[Tensor],
    query_start_value: int,
    kv_lengths: Optional[Tensor],
    use_dummy: bool,
    scale: float,
    kernel: int,
) -> tuple[Tensor, Tensor]:
    """Strict-past attention with dense per-row bounds and packed documents (cached-prefix Jacobi): Out (B,H,T,D)
    view of (B,T,H,D) storage and Lse.  The tables are those of the cyclic document operators, over the query rows
    and the key slots of this call."""
    a, keep = _strict_doc_args(Q, K, V, (QSeg, KSeg, QStart, KQEnd), query_start, query_start_value, kv_lengths, use_dummy, scale, kernel)
    out, lse = _new_output(Q)
    _set_out(a, out, lse)
    _native.call("wm_strict_attn_fwd", a, Q.device)
    del keep
    return out, lse


@strict_doc_fwd.register_fake
def _(Q, K, V, QSeg, KSeg, QStart, KQEnd, query_start, query_start_value, kv_lengths, use_dummy, scale, kernel):
    return _fake_output(Q)


@torch.library.custom_op("wm_b200::strict_doc_bwd", mutates_args=())
def strict_doc_bwd(
    Q: Tensor,
    K: Tensor,
    V: Tensor,
    QSeg: Tensor,
    KSeg: Tensor,
    QStart: Tensor,
    KQEnd: Tensor,
    query_start: Optional[Tensor],
    query_start_value: int,
    kv_lengths: Optional[Tensor],
    Out: Tensor,
    Lse: Tensor,
    dOut: Tensor,
    use_dummy: bool,
    scale: float,
    kernel: int,
) -> tuple[Tensor, Tensor, Tensor]:
    a, keep = _strict_doc_args(Q, K, V, (QSeg, KSeg, QStart, KQEnd), query_start, query_start_value, kv_lengths, use_dummy, scale, kernel)
    out = _unit_inner(Out, Q.dtype)
    dout = _unit_inner(dOut, Q.dtype)
    lse = Lse.contiguous()
    _set_out(a, out, lse)
    dq, dk, dv = _new_grads(Q, K, V)
    _set_grads(a, dout, dq, dk, dv)
    ws = _bwd_workspace(a, Q.device)
    _native.call("wm_strict_attn_bwd", a, Q.device)
    del ws, keep
    return dq, dk, dv


@strict_doc_bwd.register_fake
def _(Q, K, V, QSeg, KSeg, QStart, KQEnd, query_start, query_start_value, kv_lengths, Out, Lse, dOut, use_dummy, scale, kernel):
    return _fake_grads(Q, K, V)


def _strict_doc_setup(ctx, inputs, output):
    *tensors, ctx.query_start_value, kv_lengths, ctx.use_dummy, ctx.scale, ctx.kernel = inputs
    ctx.has_start = tensors[7] is not None
    ctx.has_limit = kv_lengths is not None
    saved = tensors[:7] + ([tensors[7]] if ctx.has_start else []) + ([kv_lengths] if ctx.has_limit else [])
    ctx.save_for_backward(*saved, *output)
    ctx.set_materialize_grads(False)


def _strict_doc_backward(ctx, dOut, dLse):
    saved = list(ctx.saved_tensors)
    out, lse = saved[-2:]
    tensors = saved[:7]
    at = 7
    start = saved[at] if ctx.has_start else None
    at += int(ctx.has_start)
    limit = saved[at] if ctx.has_limit else None
    if dOut is None:
        dOut = torch.zeros_like(out)
    grads = strict_doc_bwd(*tensors, start, ctx.query_start_value, limit, out, lse, dOut, ctx.use_dummy, ctx.scale, ctx.kernel)
    return (*grads, *((None,) * 10))


strict_doc_fwd.register_autograd(_strict_doc_backward, setup_context=_strict_doc_setup)


@torch.library.custom_op("wm_b200::strict_decode", mutates_args=())
def strict_decode(
    Q: Tensor,
    K: Tensor,
    V: Tensor,
    query_start: Optional[Tensor],
    query_start_value: int,
    kv_lengths: Optional[Tensor],
    key_mask: Optional[Tensor],
    use_dummy: bool,
    scale: float,
) -> Tensor:
    """Single-query read of the KV pool: (B,1,H,D).  Bounds stay on the device."""
    a, keep = _strict_args(Q, K, V, query_start, query_start_value, kv_lengths, key_mask, use_dummy, scale, 0)
    out, _ = _new_output(Q)
    _set_out(a, out, None)
    nbytes = _native.load_library().wm_strict_decode_workspace_bytes(ctypes.byref(a))
    ws = _attach_workspace(a, nbytes, Q.device)
    _native.call("wm_strict_decode", a, Q.device)
    del ws, keep
    return out.transpose(1, 2)


@strict_decode.register_fake
def _(Q, K, V, query_start, query_start_value, kv_lengths, key_mask, use_dummy, scale):
    batch, heads, length, dim = Q.shape
    return torch.empty((batch, length, heads, dim), dtype=Q.dtype, device=Q.device)


def decode_supported(Q: Tensor, K: Tensor, V: Tensor) -> bool:
    """Whether the split-KV read kernel takes these layouts (16-byte rows).

    While a compiler traces the caller there are no addresses to look at: the strides decide alone, and a view that
    does turn out to start off a 16-byte boundary is refused by the library when the call runs."""
    esize = Q.element_size()
    vec = 16 // esize
    if Q.shape[-1] % vec or Q.shape[-1] > 32 * vec:
        return False
    tracing = torch.compiler.is_compiling()
    for t in (Q, K, V):
        misaligned = False if tracing else t.data_ptr() % 16 != 0
        if t.stride(-1) != 1 or misaligned or any((s * esize) % 16 for s in t.stride()[:3]):
            return False
    return True


# --------------------------------------------------------------------------- strict, packed schedule


def _packed_args(Q, K, V, groups, query_indices, key_indices, query_tiles, key_tiles, scale, kernel):
    q = _unit_inner(Q, Q.dtype)
    k = _unit_inner(K, Q.dtype)
    v = _unit_inner(V, Q.dtype)
    a = _base_args(q, k, v, scale, _native.WM_MASK_PACKED, kernel)
    a.n_groups = groups.shape[0]
    a.groups = groups.data_ptr()
    a.query_indices = query_indices.data_ptr()
    a.key_indices = key_indices.data_ptr()
    a.n_query_tiles = query_tiles.shape[0]
    a.query_tiles = query_tiles.data_ptr()
    a.n_key_tiles = key_tiles.shape[0]
    a.key_tiles = key_tiles.data_ptr()
    return a, [q, k, v]


@torch.library.custom_op("wm_b200::strict_packed_fwd", mutates_args=())
def strict_packed_fwd(
    Q: Tensor,
    K: Tensor,
    V: Tensor,
    groups: Tensor,
    query_indices: Tensor,
    key_indices: Tensor,
    query_tiles: Tensor,
    key_tiles: Tensor,
    scale: float,
    kernel: int,
) -> tuple[Tensor, Tensor]:
    a, keep = _packed_args(Q, K, V, groups, query_indices, key_indices, query_tiles, key_tiles, scale, kernel)
    out, lse = _new_output(Q)
    _set_out(a, out, lse)
    _native.call("wm_strict_packed_fwd", a, Q.device)
    return out, lse


@strict_packed_fwd.register_fake
def _(Q, K, V, groups, query_indices, key_indices, query_tiles, key_tiles, scale, kernel):
    return _fake_output(Q)


@torch.library.custom_op("wm_b200::strict_packed_bwd", mutates_args=())
def strict_packed_bwd(
    Q: Tensor,
    K: Tensor,
    V: Tensor,
    Out: Tensor,
    Lse: Tensor,
    dOut: Tensor,
    groups: Tensor,
    query_indices: Tensor,
    key_indices: Tensor,
    query_tiles: Tensor,
    key_tiles: Tensor,
    scale: float,
    kernel: int,
) -> tuple[Tensor, Tensor, Tensor]:
    a, keep = _packed_args(Q, K, V, groups, query_indices, key_indices, query_tiles, key_tiles, scale, kernel)
    _set_out(a, _unit_inner(Out, Q.dtype), Lse.contiguous())
    dq, dk, dv = _new_grads(Q, K, V)
    dout = _unit_inner(dOut, Q.dtype)
    _set_grads(a, dout, dq, dk, dv)
    ws = _bwd_workspace(a, Q.device)
    _native.call("wm_strict_packed_bwd", a, Q.device)
    del ws, keep
    return dq, dk, dv


@strict_packed_bwd.register_fake
def _(Q, K, V, Out, Lse, dOut, groups, query_indices, key_indices, query_tiles, key_tiles, scale, kernel):
    return _fake_grads(Q, K, V)


def _packed_setup(ctx, inputs, output):
    Q, K, V, *tables, ctx.scale, ctx.kernel = inputs
    ctx.save_for_backward(Q, K, V, *output)
    ctx.tables = tables
    ctx.set_materialize_grads(False)


def _packed_backward(ctx, dOut, dLse):
    Q, K, V, Out, Lse = ctx.saved_tensors
    if dOut is None:
        dOut = torch.zeros_like(Out)
    grads = strict_packed_bwd(Q, K, V, Out, Lse, dOut, *ctx.tables, ctx.scale, ctx.kernel)
    return (*grads, None, None, None, None, None, None, None)


strict_packed_fwd.register_autograd(_packed_backward, setup_context=_packed_setup)


def packed_tile_rows(Q: Tensor, K: Tensor, kernel: int) -> tuple[int, int, int]:
    """Tile heights (fwd queries, bwd queries, bwd keys) the library will use for this problem."""
    a = AttnArgs()
    a.dtype = _native.dtype_code(Q.dtype)
    a.batch, a.q_heads, a.q_len, a.head_dim = Q.shape
    a.kv_heads, a.k_len = K.shape[1], K.shape[2]
    a.mask = _native.WM_MASK_PACKED
    a.kernel = kernel
    a.q, a.k, a.v = Q.data_ptr(), K.data_ptr(), K.data_ptr()
    a.q_strides, a.k_strides, a.v_strides = _native.strides3(Q), _native.strides3(K), _native.strides3(K)
    lib = _native.load_library()
    return (
        lib.wm_attn_tile_rows(ctypes.byref(a), 0, 0),
        lib.wm_attn_tile_rows(ctypes.byref(a), 1, 0),
        lib.wm_attn_tile_rows(ctypes.byref(a), 1, 1),
    )


# --------------------------------------------------------------------------- source mixing


def _mix_args(sources: Tensor, logits: Tensor) -> MixArgs:
    a = MixArgs()
    a.sources = sources.data_ptr()
    a.source_stride = sources.stride(0)
    a.logits = logits.data_ptr()
    a.n = sources[0].numel()
    a.n_sources = sources.shape[0]
    a.dtype = _native.dtype_code(sources.dtype)
    return a


def _dense_sources(sources: Tensor) -> Tensor:
    """Sources whose per-source block is contiguous (any stride between sources)."""
    if sources.shape[0] and not sources[0].is_contiguous():
        sources = sources.contiguous()
    return sources


@torch.library.custom_op("wm_b200::mix_sources", mutates_args=())
def mix_sources(sources: Tensor, logits: Tensor) -> Tensor:
    """sum_s softmax(logits)[s] * sources[s]; sources (S, ...), logits (S,) fp32."""
    sources = _dense_sources(sources)
    logits = logits.to(torch.float32).contiguous()
    out = torch.empty(sources.shape[1:], dtype=sources.dtype, device=sources.device)
    a = _mix_args(sources, logits)
    a.out = out.data_ptr()
    _native.call("wm_mix_sources_fwd", a, sources.device)
    return out


@mix_sources.register_fake
def _(sources, logits):
    return torch.empty(sources.shape[1:], dtype=sources.dtype, device=sources.device)


@torch.library.custom_op("wm_b200::mix_sources_bwd", mutates_args=())
def mix_sources_bwd(sources: Tensor, logits: Tensor, dout: Tensor, need_sources: bool) -> tuple[Tensor, Tensor]:
    sources = _dense_sources(sources)
    logits32 = logits.to(torch.float32).contiguous()
    dout = dout.contiguous()
    a = _mix_args(sources, logits32)
    a.dout = dout.data_ptr()
    if need_sources:
        dsources = torch.empty(sources.shape, dtype=sources.dtype, device=sources.device)
        a.dsources = dsources.data_ptr()
        a.source_stride = sources.stride(0)
        if dsources.stride(0) != sources.stride(0):
            sources = sources.contiguous()
            a.sources = sources.data_ptr()
            a.source_stride = sources.stride(0)
    else:
        dsources = torch.empty((0,), dtype=sources.dtype, device=sources.device)
    dlogits = torch.empty((sources.shape[0],), dtype=torch.float32, device=sources.device)
    a.dlogits = dlogits.data_ptr()
    nbytes = _native.load_library().wm_mix_workspace_bytes(ctypes.byref(a))
    ws = _attach_workspace(a, nbytes, sources.device)
    _native.call("wm_mix_sources_bwd", a, sources.device)
    del ws
    return dsources, dlogits


@mix_sources_bwd.register_fake
def _(sources, logits, dout, need_sources):
    ds = torch.empty(sources.shape if need_sources else (0,), dtype=sources.dtype, device=sources.device)
    return ds, torch.empty((sources.shape[0],), dtype=torch.float32, device=sources.device)


def _mix_setup(ctx, inputs, output):
    sources, logits = inputs
    ctx.save_for_backward(sources, logits)
    ctx.logits_dtype = logits.dtype


def _mix_backward(ctx, dout):
    sources, logits = ctx.saved_tensors
    need_sources = ctx.needs_input_grad[0]
    dsources, dlogits = mix_sources_bwd(sources, logits, dout, need_sources)
    return (dsources if need_sources else None), dlogits.to(ctx.logits_dtype)


mix_sources.register_autograd(_mix_backward, setup_context=_mix_setup)


# ---------------------------------------------------------------------------
# query preparation of the attention layer: rms_norm * gain, rotary embedding, (B,T,H,D) -> (B,H,T,D)


def _qprep_args(x: Tensor, weight: Tensor, cos: Tensor, sin: Tensor, eps: float, q_dtype: torch.dtype) -> "_native.QueryPrepArgs":
    a = _native.QueryPrepArgs()
    a.x = x.data_ptr()
    a.weight = weight.data_ptr()
    a.cos = cos.data_ptr()
    a.sin = sin.data_ptr()
    a.x_strides = (ctypes.c_int64 * 3)(x.stride(0), x.stride(1), x.stride(2))
    a.cs_strides = (ctypes.c_int64 * 2)(cos.stride(0) if cos.shape[0] > 1 else 0, cos.stride(1))
    a.dtype = _native.dtype_code(x.dtype)
    a.q_dtype = _native.dtype_code(q_dtype)
    a.batch, a.tokens, a.heads, a.head_dim = x.shape
    a.eps = float(eps)
    return a


def _qprep_inputs(x: Tensor, weight: Tensor, cos: Tensor, sin: Tensor):
    if x.stride(-1) != 1 or any(st % 2 for st in x.stride()[:3]):
        x = x.contiguous()
    weight = weight.to(x.dtype).contiguous()
    cos = cos.to(x.dtype)
    sin = sin.to(x.dtype)
    if cos.stride(-1) != 1 or cos.stride(1) % 2 or cos.stride(0) % 2:
        cos = cos.contiguous()
    if sin.stride() != cos.stride():
        sin = sin.contiguous()
        cos = cos.contiguous()
    return x, weight, cos, sin


@torch.library.custom_op("wm_b200::query_prepare", mutates_args=())
def query_prepare(x: Tensor, weight: Tensor, cos: Tensor, sin: Tensor, eps: float, to_bf16: bool) -> Tensor:
    """x (B,T,H,D), weight (D,), cos/sin (B|1,T,D) -> q (B,H,T,D) = rope(rms_norm(x) * weight)."""
    x, weight, cos, sin = _qprep_inputs(x, weight, cos, sin)
    q_dtype = torch.bfloat16 if to_bf16 else x.dtype
    b, t, h, d = x.shape
    q = torch.empty((b, h, t, d), dtype=q_dtype, device=x.device)
    a = _qprep_args(x, weight, cos, sin, eps, q_dtype)
    a.q = q.data_ptr()
    _native.call("wm_query_prepare_fwd", a, x.device)
    return q


@query_prepare.register_fake
def _(x, weight, cos, sin, eps, to_bf16):
    b, t, h, d = x.shape
    return torch.empty((b, h, t, d), dtype=torch.bfloat16 if to_bf16 else x.dtype, device=x.device)


@torch.library.custom_op("wm_b200::query_prepare_bwd", mutates_args=())
def query_prepare_bwd(x: Tensor, weight: Tensor, cos: Tensor, sin: Tensor, dq: Tensor, eps: float) -> tuple[Tensor, Tensor]:
    x, weight, cos, sin = _qprep_inputs(x, weight, cos, sin)
    dq = dq.contiguous()
    dx = torch.empty_like(x)
    if dx.stride() != x.stride():
        x = x.contiguous()
        dx = torch.empty_like(x)
    dweight = torch.empty_like(weight)
    a = _qprep_args(x, weight, cos, sin, eps, dq.dtype)
    a.dq = dq.data_ptr()
    a.dx = dx.data_ptr()
    a.dweight = dweight.data_ptr()
    nbytes = _native.load_library().wm_query_prepare_workspace_bytes(ctypes.byref(a))
    ws = _attach_workspace(a, nbytes, x.device)
    _native.call("wm_query_prepare_bwd", a, x.device)
    del ws
    return dx, dweight


@query_prepare_bwd.register_fake
def _(x, weight, cos, sin, dq, eps):
    return torch.empty_like(x), torch.empty_like(weight, dtype=x.dtype)


def _qprep_setup(ctx, inputs, output):
    x, weight, cos, sin, eps, _ = inputs
    ctx.save_for_backward(x, weight, cos, sin)
    ctx.eps = eps
    ctx.weight_dtype = weight.dtype


def _qprep_backward(ctx, dq):
    x, weight, cos, sin = ctx.saved_tensors
    dx, dweight = query_prepare_bwd(x, weight, cos, sin, dq, ctx.eps)
    return dx, dweight.to(ctx.weight_dtype), None, None, None, None


query_prepare.register_autograd(_qprep_backward, setup_context=_qprep_setup)


def strict_decode_mixed(
    Q: Tensor,
    K_sources: Tensor,
    V_sources: Tensor,
    k_logits: Tensor,
    v_logits: Tensor,
    query_start: Optional[Tensor],
    query_start_value: int,
    kv_lengths: Optional[Tensor],
    key_mask: Optional[Tensor],
    use_dummy: bool,
    scale: float,
) -> Tensor:
    """Single-query read of K/V given as (S,B,HKV,N,D) stacks, mixed in the load path: (B,1,H,D)."""
    a, keep = _strict_args(Q, K_sources[0], V_sources[0], query_start, query_start_value, kv_lengths, key_mask, use_dummy, scale, 0)
    out, _ = _new_output(Q)
    _set_out(a, out, None)
    mix = _native.SourceMix()
    kl, vl = k_logits.float().contiguous(), v_logits.float().contiguous()
    mix.k_logits, mix.v_logits = kl.data_ptr(), vl.data_ptr()
    mix.k_source_stride, mix.v_source_stride = K_sources.stride(0), V_sources.stride(0)
    mix.n_sources = K_sources.shape[0]
    nbytes = _native.load_library().wm_strict_decode_workspace_bytes(ctypes.byref(a))
    ws = _attach_workspace(a, nbytes, Q.device)
    lib = _native.load_library()
    with torch.cuda.device(Q.device):
        status = lib.wm_strict_decode_mixed(ctypes.byref(a), ctypes.byref(mix), _native.current_stream(Q.device))
    if status != 0:
        raise RuntimeError(f"wm_strict_decode_mixed failed ({status}): {lib.wm_last_error().decode(errors='replace')}")
    del ws, keep, kl, vl
    return out.transpose(1, 2)


def strict_decode_no_alloc(
    Q: Tensor,
    K: Tensor,
    V: Tensor,
    out: Tensor,
    query_start: Optional[Tensor],
    query_start_value: int,
    kv_lengths: Optional[Tensor],
    key_mask: Optional[Tensor],
    use_dummy: bool,
    scale: float,
) -> Tensor:
    """Pool read into a caller-owned ``out`` (B,1,H,D) without any allocation on the way.

    For hosts that hold pre-assigned device buffers and no allocator (a serving
    process that split the whole device into its KV pool, a thin binding from
    another language): inputs and ``out`` are passed in, the split partials go
    to the 16 MiB array inside the library (``wm_strict_decode_no_alloc``).
    Larger problems raise.  Calls share that array, so keep them on one stream.
    """
    a, keep = _strict_args(Q, K, V, query_start, query_start_value, kv_lengths, key_mask, use_dummy, scale, 0)
    if out.shape != (Q.shape[0], 1, Q.shape[1], Q.shape[3]) or out.dtype != Q.dtype or out.stride(-1) != 1:
        raise ValueError("out must be (B,1,H,D) in the query dtype with unit stride in D")
    _set_out(a, out.transpose(1, 2), None)
    _native.call("wm_strict_decode_no_alloc", a, Q.device)
    del keep
    return out
