"""``strict_causal_attention``: Jacobi prefill, cached-prefix prefill and decode.

Signature, argument checks and error texts follow upstream
src/white_matter/ops/strict_causal_attention.py:158-220.  The three modes map
onto three entry points of the kernel library: a packed-schedule kernel when
``metadata`` is given, a split-KV read for a single query without gradients,
and the dense-bound kernel otherwise.  ``query_start`` / ``kv_lengths`` stay
on the device, so the decode call can be captured in a CUDA graph and replayed
with changing lengths.
"""

from __future__ import annotations

from typing import Literal

import torch

from . import operators
from .metadata import StrictCausalMetadata

_BACKENDS = {"sm100": "auto", "sm100_simt": "simt", "sm100_tcgen05": "tcgen05"}


def strict_causal_attention(
    query: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    *,
    query_start: int | torch.Tensor = 0,
    kv_lengths: torch.Tensor | None = None,
    use_dummy_token: bool = False,
    metadata: StrictCausalMetadata | None = None,
    key_mask: torch.Tensor | None = None,
    softmax_scale: float | None = None,
    backend: Literal["sm100", "sm100_simt", "sm100_tcgen05"] = "sm100",
    num_splits: int = 0,
    static_cache: bool = False,
) -> torch.Tensor:
    """Attend only to earlier real tokens, plus an optional leading dummy.

    Q/K/V are (B,H,T,D); the result is (B,T,H,D).  ``query_start`` and
    ``kv_lengths`` count real tokens and exclude the dummy slot: the query at
    real position p sees real slots s < min(p, kv_lengths) and, with
    ``use_dummy_token``, slot 0.  K/V may hold current tokens or unused cache
    capacity (even NaN); neither is read.  Rows without a visible key return
    zero.  ``metadata`` comes from ``prepare_strict_causal_metadata`` and is
    meant to be built once and reused; ``key_mask`` is boolean (B,N) and
    mutually exclusive with it.  ``num_splits`` and ``static_cache`` are
    accepted for call compatibility; the split count is chosen by the kernel
    and offsets never depend on the cache capacity being static.
    """
    if backend not in _BACKENDS:
        raise ValueError(f"unsupported strict causal backend: {backend!r}")
    if type(use_dummy_token) is not bool:
        raise ValueError("use_dummy_token must be boolean")
    if any(t.ndim != 4 for t in (query, key, value)) or key.shape != value.shape:
        raise ValueError("Q/K/V require (B,H,T,D) tensors with matching K/V")
    batch, heads, length, dim = query.shape
    if key.shape[0] != batch or key.shape[-1] != dim or heads % key.shape[1]:
        raise ValueError("Q/K/V require matching batch/head_dim and divisible heads")
    if any(t.device != query.device for t in (key, value)):
        raise ValueError("Q/K/V must share a device")
    lead = int(use_dummy_token)
    if key.shape[-2] - lead < 0:
        raise ValueError("dummy-enabled K/V must contain the leading dummy slot")
    if kv_lengths is not None and (kv_lengths.shape != (batch,) or kv_lengths.dtype not in (torch.int32, torch.int64)):
        raise ValueError("kv_lengths must be integer (B,)")
    if isinstance(query_start, torch.Tensor) and (
        query_start.shape != (batch,) or query_start.dtype not in (torch.int32, torch.int64)
    ):
        raise ValueError("query_start must be an integer or integer (B,) tensor")
    if metadata is not None and key_mask is not None:
        raise ValueError("metadata and key_mask are mutually exclusive")
    if key_mask is not None and (key_mask.shape != (batch, key.shape[-2]) or key_mask.dtype != torch.bool):
        raise ValueError("key_mask must be boolean (B,N)")
    if not query.is_cuda:
        raise ValueError("sm100 strict causal attention requires CUDA tensors")
    if query.dtype not in (torch.bfloat16, torch.float32) or dim > 128:
        raise RuntimeError("sm100 strict causal attention does not support these inputs (BF16/FP32, head_dim <= 128)")
    scale = dim**-0.5 if softmax_scale is None else float(softmax_scale)
    # Empty slices keep zero gradients without touching cache storage.
    if not length or not key.shape[-2]:
        zero = (query[..., :0, :].sum() + key[..., :0, :].sum() + value[..., :0, :].sum()).to(query.dtype)
        return query.new_zeros(batch, length, heads, dim) + zero
    kernel = operators.kernel_code(_BACKENDS[backend])
    key = key if key.dtype == query.dtype else key.to(query.dtype)
    value = value if value.dtype == query.dtype else value.to(query.dtype)
    if metadata is not None:
        metadata = metadata.with_key_extent(key.shape[-2])
        if metadata.query_indices.numel() == 0:
            zero = (query[..., :0, :].sum() + key[..., :0, :].sum() + value[..., :0, :].sum()).to(query.dtype)
            return query.new_zeros(batch, length, heads, dim) + zero
        # A schedule built from rows of document ids is strict-past attention with dense per-row bounds plus document
        # tables; that form runs on the tensor-core kernels without gathering.
        if (
            metadata.dense_documents is not None
            and metadata.dense_documents[1] == use_dummy_token
            and metadata.dense_documents[0].shape[0] == batch
            and metadata.max_queries_per_row == length
            and _BACKENDS[backend] != "simt"
        ):
            slots = min(key.shape[-2], metadata.dense_documents[0].shape[1] + int(use_dummy_token))
            tables = metadata.document_tables(query.device, slots)
            start_t, limit_t = metadata.dense_bounds(query.device)
            out = operators.strict_doc_fwd(
                query, key[..., :slots, :], value[..., :slots, :], *tables, start_t, 0, limit_t, use_dummy_token, scale, kernel
            )[0]
            out = out.transpose(1, 2)
            padded = metadata.padded_queries(query.device)
            if padded is not None and use_dummy_token:
                # the shared dummy key is open to every query row; padding rows are not part of the schedule
                out = out.masked_fill(padded[:, :, None, None], 0)
            return out
        fwd_q, bwd_q, bwd_k = operators.packed_tile_rows(query, key, kernel)
        if fwd_q != bwd_q:
            raise RuntimeError("forward and backward kernels disagree on the query tile height")
        tables = metadata.device_tables(query.device, fwd_q, bwd_k)
        out = operators.strict_packed_fwd(query, key, value, *tables, scale, kernel)[0]
        return out.transpose(1, 2)
    start_tensor = query_start if isinstance(query_start, torch.Tensor) else None
    start_value = 0 if start_tensor is not None else int(query_start)
    if start_tensor is not None and start_tensor.device != query.device:
        start_tensor = start_tensor.to(query.device)
    if kv_lengths is not None and kv_lengths.device != query.device:
        kv_lengths = kv_lengths.to(query.device)
    needs_grad = torch.is_grad_enabled() and any(t.requires_grad for t in (query, key, value))
    if length == 1 and not needs_grad and operators.decode_supported(query, key, value):
        return operators.strict_decode(
            query, key, value, start_tensor, start_value, kv_lengths, key_mask, use_dummy_token, scale
        )
    out = operators.strict_attn_fwd(
        query, key, value, start_tensor, start_value, kv_lengths, key_mask, use_dummy_token, scale, kernel
    )[0]
    return out.transpose(1, 2)
