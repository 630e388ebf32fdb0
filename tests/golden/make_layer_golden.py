"""Generate tests/golden/layer_vectors.npz from the upstream package.

    python tests/golden/make_layer_golden.py /path/to/upstream/src

Evaluates the query preparation of the upstream attention layer (its own ``q_norm`` module, ``rotate_half`` and
``RotaryEmbedding``; layers/white_matter.py:105-111) on small seeded inputs on the CPU, in fp32 and in bf16, with
gradients for the projection and the gain, and stores inputs and results.  The tests replay the file and never
import the upstream package.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def main(upstream_src: str) -> None:
    sys.path.insert(0, upstream_src)
    from white_matter.layers.white_matter import WhiteMatterAttention
    from white_matter.modules.rotary import RotaryEmbedding, rotate_half

    arrays: dict[str, np.ndarray] = {}

    def put(case, **tensors):
        for name, t in tensors.items():
            t = t.detach()
            arrays[f"{case}/{name}"] = (t.float() if t.dtype == torch.bfloat16 else t).cpu().numpy()

    for case, (batch, tokens, heads, dim, shared_positions) in {
        "d64": (2, 9, 3, 64, False),
        "d64_shared": (2, 17, 4, 64, True),
        "d128": (1, 5, 2, 128, False),
    }.items():
        for dtype, tag in ((torch.float32, "f32"), (torch.bfloat16, "bf16")):
            torch.manual_seed(11)
            layer = WhiteMatterAttention(hidden_size=heads * dim, num_attention_heads=heads, head_dim=dim, rms_norm_eps=1e-6)
            with torch.no_grad():
                layer.q_norm.weight.copy_(1.0 + 0.3 * torch.randn(dim))
            layer = layer.to(dtype)
            projected = (2.0 * torch.randn(batch, tokens, heads, dim)).to(dtype).requires_grad_()
            positions = torch.arange(tokens)[None, :].expand(1 if shared_positions else batch, -1).clone()
            if not shared_positions:
                positions = positions + torch.arange(batch)[:, None] * 1000
            cos, sin = RotaryEmbedding(dim)(projected, positions)
            # layers/white_matter.py:109-111
            query_states = layer.q_norm(projected).transpose(1, 2)
            query_states = query_states * cos.unsqueeze(1) + rotate_half(query_states) * sin.unsqueeze(1)
            probe = torch.randn(query_states.shape).to(dtype)
            dx, dw = torch.autograd.grad(query_states, (projected, layer.q_norm.weight), probe)
            put(f"{case}/{tag}", projected=projected, weight=layer.q_norm.weight, cos=cos, sin=sin, out=query_states,
                probe=probe, dx=dx, dw=dw)
    np.savez_compressed(HERE / "layer_vectors.npz", **arrays)
    print(f"wrote {len(arrays)} arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
