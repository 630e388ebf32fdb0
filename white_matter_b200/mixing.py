"""KV source mixing: the soft-max weighted mixture of stacked K (or V) sources, materialised
(``mix_kv_sources``) or formed inside the K/V load path of the decode read (``mixed_pool_decode``).

The mixture over the L+1 depth sources forms each layer's shared KV channel.
Upstream mixes with ``einsum("btld,btkl->btkd")`` over routed weights
(src/white_matter/modules/routing.py:116-122) or a static soft-max
(src/white_matter/blocks/feedback_transformer.py:35-36); this operator is the
static soft-max form applied to stacked, already projected sources
``(S, B, H, T, D)``.  It streams every source once at HBM speed.
"""

from __future__ import annotations

import torch

from . import operators


def mix_kv_sources(sources: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
    """``einsum('s,s...->...', softmax(logits), sources)`` on the GPU.

    ``sources`` is (S, ...) in bf16 or fp32 with 1 <= S <= 64, ``logits`` is
    (S,).  Accumulation is fp32.  Differentiable in both arguments.
    """
    if sources.ndim < 2 or logits.ndim != 1 or logits.shape[0] != sources.shape[0]:
        raise ValueError("sources must be (S, ...) and logits (S,)")
    if not 1 <= sources.shape[0] <= 64:
        raise ValueError("between 1 and 64 sources are supported")
    if not sources.is_cuda or logits.device != sources.device:
        raise ValueError("sm100 source mixing requires CUDA tensors on one device")
    if sources.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("sm100 source mixing supports BF16 and FP32 sources")
    return operators.mix_sources(sources, logits)


def mixed_pool_decode(
    query: torch.Tensor,
    key_sources: torch.Tensor,
    value_sources: torch.Tensor,
    key_logits: torch.Tensor,
    value_logits: torch.Tensor,
    *,
    query_start: int | torch.Tensor = 0,
    kv_lengths: torch.Tensor | None = None,
    use_dummy_token: bool = False,
    key_mask: torch.Tensor | None = None,
    softmax_scale: float | None = None,
) -> torch.Tensor:
    """``strict_causal_attention`` for one query token over K/V that are soft-max mixtures of stacked sources,
    without materialising the mixtures.

    ``query`` is (B,H,1,D); ``key_sources`` / ``value_sources`` are (S,B,HKV,N,D) with 1 <= S <= 64 and the
    logits (S,).  Equal to ``strict_causal_attention(query, mix_kv_sources(key_sources, key_logits),
    mix_kv_sources(value_sources, value_logits), ...)`` up to the rounding of the materialised mixture; every
    visible source row is read once, nothing is written but the (B,1,H,D) result.  Inference only.
    """
    if query.ndim != 4 or query.shape[2] != 1:
        raise ValueError("query must be (B,H,1,D)")
    if key_sources.ndim != 5 or key_sources.shape != value_sources.shape:
        raise ValueError("key and value sources must be matching (S,B,HKV,N,D) stacks")
    sources, batch, kv_heads, slots, dim = key_sources.shape
    if not 1 <= sources <= 64:
        raise ValueError("between 1 and 64 sources are supported")
    if key_logits.shape != (sources,) or value_logits.shape != (sources,):
        raise ValueError("logits must be (S,)")
    if query.shape[0] != batch or query.shape[3] != dim or query.shape[1] % kv_heads:
        raise ValueError("Q/K/V require matching batch/head_dim and divisible heads")
    if not query.is_cuda or any(t.device != query.device for t in (key_sources, value_sources, key_logits, value_logits)):
        raise ValueError("sm100 mixed decode requires CUDA tensors on one device")
    if query.dtype not in (torch.bfloat16, torch.float32) or key_sources.dtype != query.dtype or value_sources.dtype != query.dtype:
        raise ValueError("query and sources must share BF16 or FP32")
    if key_sources.stride(-1) != 1 or value_sources.stride(-1) != 1:
        raise ValueError("sources must have unit stride in head_dim")
    if type(use_dummy_token) is not bool:
        raise ValueError("use_dummy_token must be boolean")
    if kv_lengths is not None and (kv_lengths.shape != (batch,) or kv_lengths.dtype not in (torch.int32, torch.int64)):
        raise ValueError("kv_lengths must be integer (B,)")
    if key_mask is not None and (key_mask.shape != (batch, slots) or key_mask.dtype != torch.bool):
        raise ValueError("key_mask must be boolean (B,N)")
    start_tensor = query_start if isinstance(query_start, torch.Tensor) else None
    start_value = 0 if start_tensor is not None else int(query_start)
    scale = dim**-0.5 if softmax_scale is None else float(softmax_scale)
    if not operators.decode_supported(query, key_sources[0], value_sources[0]):
        raise RuntimeError("mixed decode needs head_dim rows of a multiple of 16 bytes, 16-byte aligned")
    return operators.strict_decode_mixed(
        query, key_sources, value_sources, key_logits, value_logits, start_tensor, start_value, kv_lengths, key_mask,
        use_dummy_token, scale,
    )
