"""ctypes binding of libwm_b200.so (the C ABI declared in include/wm_b200.h).

The library is looked up beside this file.  There is no fallback: when it is
missing, every operator of the package raises.
"""

from __future__ import annotations

import ctypes
import threading
from pathlib import Path

import torch

LIBRARY_PATH = Path(__file__).resolve().parent / "libwm_b200.so"

WM_F32, WM_BF16 = 0, 1
WM_MASK_CYCLIC, WM_MASK_STRICT, WM_MASK_PACKED = 0, 1, 2
WM_KERNEL_AUTO, WM_KERNEL_SIMT, WM_KERNEL_TCGEN05 = 0, 1, 2

_Strides = ctypes.c_int64 * 3


class AttnArgs(ctypes.Structure):
    """Mirror of ``wm_attn_args``; field order and types follow include/wm_b200.h."""

    _fields_ = [
        ("q", ctypes.c_void_p),
        ("k", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("out", ctypes.c_void_p),
        ("lse", ctypes.c_void_p),
        ("dout", ctypes.c_void_p),
        ("dq", ctypes.c_void_p),
        ("dk", ctypes.c_void_p),
        ("dv", ctypes.c_void_p),
        ("q_strides", _Strides),
        ("k_strides", _Strides),
        ("v_strides", _Strides),
        ("out_strides", _Strides),
        ("dout_strides", _Strides),
        ("dq_strides", _Strides),
        ("dk_strides", _Strides),
        ("dv_strides", _Strides),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("dtype", ctypes.c_int32),
        ("batch", ctypes.c_int32),
        ("q_heads", ctypes.c_int32),
        ("kv_heads", ctypes.c_int32),
        ("q_len", ctypes.c_int32),
        ("k_len", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("scale", ctypes.c_float),
        ("mask", ctypes.c_int32),
        ("kernel", ctypes.c_int32),
        ("query_stride", ctypes.c_int32),
        ("query_offset", ctypes.c_int32),
        ("q_seg", ctypes.c_void_p),
        ("k_seg", ctypes.c_void_p),
        ("q_key_start", ctypes.c_void_p),
        ("k_query_end", ctypes.c_void_p),
        ("query_start", ctypes.c_void_p),
        ("kv_lengths", ctypes.c_void_p),
        ("query_start_is64", ctypes.c_int32),
        ("kv_lengths_is64", ctypes.c_int32),
        ("query_start_value", ctypes.c_int64),
        ("key_mask", ctypes.c_void_p),
        ("use_dummy", ctypes.c_int32),
        ("n_groups", ctypes.c_int32),
        ("groups", ctypes.c_void_p),
        ("query_indices", ctypes.c_void_p),
        ("key_indices", ctypes.c_void_p),
        ("n_query_tiles", ctypes.c_int32),
        ("query_tiles", ctypes.c_void_p),
        ("n_key_tiles", ctypes.c_int32),
        ("key_tiles", ctypes.c_void_p),
    ]


class MixArgs(ctypes.Structure):
    """Mirror of ``wm_mix_args``."""

    _fields_ = [
        ("sources", ctypes.c_void_p),
        ("source_stride", ctypes.c_int64),
        ("logits", ctypes.c_void_p),
        ("out", ctypes.c_void_p),
        ("dout", ctypes.c_void_p),
        ("dsources", ctypes.c_void_p),
        ("dlogits", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("n", ctypes.c_int64),
        ("n_sources", ctypes.c_int32),
        ("dtype", ctypes.c_int32),
    ]


class SourceMix(ctypes.Structure):
    """Mirror of ``wm_source_mix``."""

    _fields_ = [
        ("k_logits", ctypes.c_void_p),
        ("v_logits", ctypes.c_void_p),
        ("k_source_stride", ctypes.c_int64),
        ("v_source_stride", ctypes.c_int64),
        ("n_sources", ctypes.c_int32),
    ]


class QueryPrepArgs(ctypes.Structure):
    """Mirror of ``wm_qprep_args``."""

    _fields_ = [
        ("x", ctypes.c_void_p),
        ("weight", ctypes.c_void_p),
        ("cos", ctypes.c_void_p),
        ("sin", ctypes.c_void_p),
        ("q", ctypes.c_void_p),
        ("dq", ctypes.c_void_p),
        ("dx", ctypes.c_void_p),
        ("dweight", ctypes.c_void_p),
        ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_size_t),
        ("x_strides", ctypes.c_int64 * 3),
        ("cs_strides", ctypes.c_int64 * 2),
        ("dtype", ctypes.c_int32),
        ("q_dtype", ctypes.c_int32),
        ("batch", ctypes.c_int32),
        ("tokens", ctypes.c_int32),
        ("heads", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("eps", ctypes.c_float),
    ]


class PoolAppendArgs(ctypes.Structure):
    """Mirror of ``wm_pool_append_args``."""

    _fields_ = [
        ("pool", ctypes.c_void_p),
        ("src", ctypes.c_void_p),
        ("lengths", ctypes.c_void_p),
        ("pool_strides", _Strides),
        ("src_strides", _Strides),
        ("dtype", ctypes.c_int32),
        ("batch", ctypes.c_int32),
        ("heads", ctypes.c_int32),
        ("capacity", ctypes.c_int32),
        ("n_new", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("lead", ctypes.c_int32),
    ]


class PoolMixArgs(ctypes.Structure):
    """Mirror of ``wm_pool_mix_args``."""

    _fields_ = [
        ("stacked", ctypes.c_void_p),
        ("stacked_strides", _Strides),
        ("pre_mix_k", ctypes.c_void_p),
        ("pre_mix_v", ctypes.c_void_p),
        ("bias_k", ctypes.c_void_p),
        ("bias_v", ctypes.c_void_p),
        ("partial_k", ctypes.c_void_p),
        ("partial_v", ctypes.c_void_p),
        ("gain_k", ctypes.c_void_p),
        ("gain_v", ctypes.c_void_p),
        ("mixed_k", ctypes.c_void_p),
        ("mixed_v", ctypes.c_void_p),
        ("dtype", ctypes.c_int32),
        ("batch", ctypes.c_int32),
        ("tokens", ctypes.c_int32),
        ("sources", ctypes.c_int32),
        ("channels", ctypes.c_int32),
        ("hidden", ctypes.c_int32),
        ("route_start", ctypes.c_int32),
        ("route_stride", ctypes.c_int32),
        ("n_routed", ctypes.c_int32),
        ("source_eps", ctypes.c_float),
        ("mix_eps", ctypes.c_float),
        ("partial_row_stride", ctypes.c_int64),
    ]


class PoolFinishArgs(ctypes.Structure):
    """Mirror of ``wm_pool_finish_args``."""

    _fields_ = [
        ("k_proj", ctypes.c_void_p),
        ("v_proj", ctypes.c_void_p),
        ("k_norm_weight", ctypes.c_void_p),
        ("cos", ctypes.c_void_p),
        ("sin", ctypes.c_void_p),
        ("k_out", ctypes.c_void_p),
        ("v_out", ctypes.c_void_p),
        ("cs_strides", ctypes.c_int64 * 2),
        ("out_strides", _Strides),
        ("in_dtype", ctypes.c_int32),
        ("out_dtype", ctypes.c_int32),
        ("batch", ctypes.c_int32),
        ("tokens", ctypes.c_int32),
        ("channels", ctypes.c_int32),
        ("kv_heads", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("token_offset", ctypes.c_int32),
        ("rope_offset", ctypes.c_int32),
        ("eps", ctypes.c_float),
        ("slot_stride", ctypes.c_int32),
    ]


ATTN_ENTRY_POINTS = (
    "wm_cyclic_attn_fwd",
    "wm_cyclic_attn_bwd",
    "wm_cyclic_attn_doc_fwd",
    "wm_cyclic_attn_doc_bwd",
    "wm_strict_attn_fwd",
    "wm_strict_attn_bwd",
    "wm_strict_packed_fwd",
    "wm_strict_packed_bwd",
    "wm_strict_decode",
    "wm_strict_decode_no_alloc",
)
MIX_ENTRY_POINTS = ("wm_mix_sources_fwd", "wm_mix_sources_bwd")
QUERY_PREP_ENTRY_POINTS = ("wm_query_prepare_fwd", "wm_query_prepare_bwd")
QUERY_ENTRY_POINTS = (
    "wm_abi_version",
    "wm_last_error",
    "wm_kernel_launch_count",
    "wm_device_status",
    "wm_attn_tile_rows",
    "wm_attn_fwd_workspace_bytes",
    "wm_attn_bwd_workspace_bytes",
    "wm_strict_decode_workspace_bytes",
    "wm_mix_workspace_bytes",
    "wm_query_prepare_workspace_bytes",
)

_lock = threading.Lock()
_library = None


def load_library() -> ctypes.CDLL:
    """dlopen the kernel library once; raises when it has not been built."""
    global _library
    if _library is not None:
        return _library
    with _lock:
        if _library is not None:
            return _library
        if not LIBRARY_PATH.exists():
            raise RuntimeError(
                f"{LIBRARY_PATH} is missing: build it with `python -m white_matter_b200.build` "
                "(the sm_100a kernels have no fallback)"
            )
        lib = ctypes.CDLL(str(LIBRARY_PATH))
        for name in ATTN_ENTRY_POINTS:
            fn = getattr(lib, name)
            fn.argtypes = [ctypes.POINTER(AttnArgs), ctypes.c_void_p]
            fn.restype = ctypes.c_int
        for name in MIX_ENTRY_POINTS:
            fn = getattr(lib, name)
            fn.argtypes = [ctypes.POINTER(MixArgs), ctypes.c_void_p]
            fn.restype = ctypes.c_int
        for name in QUERY_PREP_ENTRY_POINTS:
            fn = getattr(lib, name)
            fn.argtypes = [ctypes.POINTER(QueryPrepArgs), ctypes.c_void_p]
            fn.restype = ctypes.c_int
        lib.wm_pool_append.argtypes = [ctypes.POINTER(PoolAppendArgs), ctypes.c_void_p]
        lib.wm_pool_append.restype = ctypes.c_int
        lib.wm_strict_decode_mixed.argtypes = [ctypes.POINTER(AttnArgs), ctypes.POINTER(SourceMix), ctypes.c_void_p]
        lib.wm_strict_decode_mixed.restype = ctypes.c_int
        lib.wm_pool_mix.argtypes = [ctypes.POINTER(PoolMixArgs), ctypes.c_void_p]
        lib.wm_pool_mix.restype = ctypes.c_int
        lib.wm_pool_finish.argtypes = [ctypes.POINTER(PoolFinishArgs), ctypes.c_void_p]
        lib.wm_pool_finish.restype = ctypes.c_int
        lib.wm_query_prepare_workspace_bytes.argtypes = [ctypes.POINTER(QueryPrepArgs)]
        lib.wm_query_prepare_workspace_bytes.restype = ctypes.c_size_t
        lib.wm_abi_version.argtypes = []
        lib.wm_abi_version.restype = ctypes.c_int
        lib.wm_last_error.argtypes = []
        lib.wm_last_error.restype = ctypes.c_char_p
        lib.wm_kernel_launch_count.argtypes = []
        lib.wm_kernel_launch_count.restype = ctypes.c_ulonglong
        lib.wm_device_status.argtypes = [ctypes.c_int]
        lib.wm_device_status.restype = ctypes.c_int
        lib.wm_attn_tile_rows.argtypes = [ctypes.POINTER(AttnArgs), ctypes.c_int, ctypes.c_int]
        lib.wm_attn_tile_rows.restype = ctypes.c_int
        for name in ("wm_attn_fwd_workspace_bytes", "wm_attn_bwd_workspace_bytes", "wm_strict_decode_workspace_bytes"):
            fn = getattr(lib, name)
            fn.argtypes = [ctypes.POINTER(AttnArgs)]
            fn.restype = ctypes.c_size_t
        lib.wm_mix_workspace_bytes.argtypes = [ctypes.POINTER(MixArgs)]
        lib.wm_mix_workspace_bytes.restype = ctypes.c_size_t
        if lib.wm_abi_version() != 1:
            raise RuntimeError("libwm_b200.so has an unexpected ABI version; rebuild it")
        _library = lib
    return _library


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return WM_F32
    if dtype == torch.bfloat16:
        return WM_BF16
    raise ValueError(f"sm100 kernels support float32 and bfloat16, got {dtype}")


def strides3(t: torch.Tensor) -> _Strides:
    """(batch, head, token) element strides of a (B,H,T,D) view."""
    return _Strides(t.stride(0), t.stride(1), t.stride(2))


def current_stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def call(name: str, args, device: torch.device) -> None:
    """Invoke an entry point on the current stream of ``device``; raise on failure."""
    lib = load_library()
    if device.index is None or device.index == torch.cuda.current_device():
        status = getattr(lib, name)(ctypes.byref(args), current_stream(device))
    else:  # the library launches on the current device: make the tensors' device current for the call
        with torch.cuda.device(device):
            status = getattr(lib, name)(ctypes.byref(args), current_stream(device))
    if status != 0:
        message = lib.wm_last_error().decode(errors="replace")
        raise RuntimeError(f"{name} failed ({status}): {message}")


def device_status(reset: bool = True) -> int:
    """Status word of the pipelined kernels (0 = every bounded wait completed); synchronises the device."""
    return load_library().wm_device_status(int(reset))
