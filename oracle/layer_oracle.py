"""CPU oracle for the step in front of the attention operators inside the attention layer.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module; only the tests do.

Restates src/white_matter/layers/white_matter.py:105-111 of the upstream project:

    query_states = q_proj(hidden).view(B, T, H, D)                       # :107
    query_states = q_norm(query_states).transpose(1, 2)                  # :109, nn.RMSNorm(head_dim, eps)
    query_states = query_states * cos.unsqueeze(1) + rotate_half(query_states) * sin.unsqueeze(1)   # :111

with ``rotate_half`` of src/white_matter/modules/rotary.py:30-34 (``cat(-x2, x1)`` over the two halves of the head)
written out as an index permutation, and the RMS normalisation written out as ``x * rsqrt(mean(x^2) + eps) * weight``.
Everything is evaluated in ``compute_dtype`` (float64 by default).

Parity pin: tests/golden/make_layer_golden.py runs the upstream layer's own q_norm / rotate_half / RotaryEmbedding on
seeded inputs (fp32 and bf16, with gradients) and stores the results in tests/golden/layer_vectors.npz;
tests/test_layer.py replays them against this module.
"""

from __future__ import annotations

import torch


def prepare_queries_oracle(projected, weight, cos, sin, eps=1e-6, compute_dtype=torch.float64):
    """projected (B,T,H,D), weight (D,), cos/sin (B|1,T,D) -> (B,H,T,D) in compute_dtype."""
    x = projected.to(compute_dtype)
    w = weight.to(compute_dtype)
    c = cos.to(compute_dtype)[:, None]  # broadcast over heads
    s = sin.to(compute_dtype)[:, None]
    normed = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w
    y = normed.transpose(1, 2)  # (B,H,T,D)
    half = y.shape[-1] // 2
    index = torch.cat((torch.arange(half, 2 * half), torch.arange(0, half)))
    sign = torch.cat((-torch.ones(half, dtype=compute_dtype), torch.ones(half, dtype=compute_dtype)))
    rotated = y[..., index] * sign  # element d: -y[d + D/2] in the first half, y[d - D/2] in the second
    return y * c + rotated * s
