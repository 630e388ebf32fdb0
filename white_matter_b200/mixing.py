"""KV source mixing: the soft-max weighted mixture of stacked K (or V) sources.

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
