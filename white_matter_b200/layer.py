"""The step either side of the attention operators inside the attention layer.

Upstream (``layers/white_matter.py:105-111,171-199``) views the query projection as
``(B,T,H,D)``, applies ``q_norm`` (RMS normalisation over the head with a learned
gain), transposes to ``(B,H,T,D)``, applies the rotary embedding
(``q * cos + rotate_half(q) * sin``, ``modules/rotary.py:30-45``), casts to bf16 for
the GPU kernels, calls the operator, casts back, transposes and reshapes for
``o_proj``.  Here the part in front is one kernel (``prepare_queries``) and the part
behind is free: the operators already store their result as ``(B,T,H,D)``, so the
``(B,T,H*D)`` matrix ``o_proj`` wants is a view.
"""

from __future__ import annotations

import torch

from . import operators
from .cyclic import cyclic_attention
from .metadata import CyclicAttentionMetadata


def prepare_queries(
    projected: torch.Tensor,
    weight: torch.Tensor,
    cos: torch.Tensor,
    sin: torch.Tensor,
    *,
    eps: float = 1e-6,
    head_dim: int | None = None,
    out_dtype: torch.dtype | None = torch.bfloat16,
) -> torch.Tensor:
    """``rope(rms_norm(q) * weight)`` in the layout the attention operators read.

    ``projected`` is the output of ``q_proj``: ``(B,T,H*D)`` (give ``head_dim``) or
    ``(B,T,H,D)``, bf16 or fp32 on CUDA; ``weight`` is ``q_norm.weight`` ``(D,)``; ``cos``
    and ``sin`` are ``(B,T,D)`` or ``(1,T,D)``.  Returns ``(B,H,T,D)`` in ``out_dtype``
    (bf16 by default, ``None`` keeps the input dtype).  Differentiable with respect to
    ``projected`` and ``weight``.
    """
    if projected.dim() == 3:
        if head_dim is None:
            head_dim = weight.shape[0]
        if projected.shape[-1] % head_dim:
            raise ValueError("the projection width must be a multiple of head_dim")
        projected = projected.view(*projected.shape[:2], -1, head_dim)
    if projected.dim() != 4:
        raise ValueError("projected must be (B,T,H*D) or (B,T,H,D)")
    if not projected.is_cuda:
        raise ValueError("prepare_queries requires CUDA tensors: the sm_100a kernels have no CPU path")
    b, t, _, d = projected.shape
    if weight.shape != (d,):
        raise ValueError("weight must be (head_dim,)")
    if d not in (64, 128):
        raise ValueError("prepare_queries supports head_dim 64 and 128")
    for name, table in (("cos", cos), ("sin", sin)):
        if table.dim() != 3 or table.shape[0] not in (1, b) or table.shape[1:] != (t, d):
            raise ValueError(f"{name} must be (B,T,D) or (1,T,D)")
    if projected.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("prepare_queries supports bfloat16 and float32")
    if out_dtype is None:
        out_dtype = projected.dtype
    if out_dtype not in (torch.bfloat16, projected.dtype):
        raise ValueError("out_dtype must be bfloat16, the input dtype or None")
    return operators.query_prepare(projected, weight, cos, sin, float(eps), out_dtype == torch.bfloat16)


def cyclic_attention_layer(
    projected: torch.Tensor,
    weight: torch.Tensor,
    cos: torch.Tensor,
    sin: torch.Tensor,
    key: torch.Tensor,
    value: torch.Tensor,
    *,
    query_stride: int,
    query_offset: int = 0,
    strict_past: bool = False,
    metadata: CyclicAttentionMetadata | tuple | None = None,
    eps: float = 1e-6,
) -> torch.Tensor:
    """The cyclic branch of the upstream attention layer between ``q_proj`` and ``o_proj``.

    Returns ``(B,T,H*D)`` in the dtype of ``projected``, a view of the operator's
    ``(B,T,H,D)`` result when that dtype is bf16 (no transpose copy, no reshape copy).
    """
    queries = prepare_queries(projected, weight, cos, sin, eps=eps, out_dtype=torch.bfloat16)
    out = cyclic_attention(
        queries, key.to(torch.bfloat16), value.to(torch.bfloat16), query_stride=query_stride, query_offset=query_offset,
        strict_past=strict_past, metadata=metadata,
    )
    b, h, t, d = out.shape
    return out.transpose(1, 2).reshape(b, t, h * d).to(projected.dtype)
