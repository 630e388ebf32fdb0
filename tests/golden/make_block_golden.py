"""Generate tests/golden/block_vectors.npz from the upstream package.

    python tests/golden/make_block_golden.py /path/to/upstream/src

Builds the upstream feedback region without Transformers (blocks.WhiteMatterBlock of FeedbackDecoderLayer with
WhiteMatterAttention and GatedMLP over a KVPool, as examples/feedback_block.py does), randomises every parameter and
runs its cyclic prefill (blocks/_execution/cyclic.py: forward_cyclic / run_pass) in FP32 on the CPU without
gradients: 4 layers of width 128 (2 heads of 64), 5 pool sources into 2 channels of 2 KV heads, 40 tokens in 4
residue groups, 2 passes, with and without the dummy token and with and without packed documents.  The four cases
share one set of parameters (stored once).  Inputs, parameters, the hidden result and the final pool are stored; the tests replay the file and never import the
upstream package.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
HIDDEN, LAYERS, HEADS, HEAD_DIM, KV_HEADS, CHANNELS, MLP, THETA = 128, 4, 2, 64, 2, 2, 128, 10_000.0
B, T, GROUPS, PASSES = 2, 40, 4, 2


def main(upstream_src: str) -> None:
    sys.path.insert(0, upstream_src)
    from white_matter.blocks import FeedbackDecoderLayer, WhiteMatterBlock
    from white_matter.layers import WhiteMatterAttention
    from white_matter.modules import GatedMLP, KVPool, RotaryEmbedding

    arrays: dict[str, np.ndarray] = {}
    index = 0
    shared: dict[str, torch.Tensor] = {}
    for dummy in (False, True):
        for documents in (False, True):
            case = f"dummy{int(dummy)}_docs{int(documents)}"
            torch.manual_seed(90 + index)
            index += 1
            layers = [
                FeedbackDecoderLayer(HIDDEN, WhiteMatterAttention(HIDDEN, HEADS, HEAD_DIM), GatedMLP(HIDDEN, MLP))
                for _ in range(LAYERS)
            ]
            pool = KVPool(HIDDEN, KV_HEADS, HEAD_DIM, LAYERS + 1, CHANNELS, router_layer_stride=2)
            block = WhiteMatterBlock(layers, pool, RotaryEmbedding(HEAD_DIM, THETA), num_passes=PASSES, use_dummy_token=dummy).eval()
            with torch.no_grad():
                for name, parameter in block.named_parameters():
                    if name in shared:
                        parameter.copy_(shared[name])
                        continue
                    if parameter.ndim >= 2 and "router" not in name and "gain" not in name and "pre_mix" not in name:
                        parameter.copy_(torch.randn_like(parameter) * parameter.shape[-1] ** -0.5)
                    elif "router" in name and name.endswith("weight"):
                        parameter.copy_(torch.randn_like(parameter) * 0.02)
                    elif "router" in name:
                        parameter.copy_(torch.randn_like(parameter) * 0.5)
                    else:  # norm gains, pre/post-mix gains, the dummy token
                        parameter.copy_(1 + 0.2 * torch.randn_like(parameter))
                    shared[name] = parameter.detach().clone()
            x = torch.randn(B, T, HIDDEN)
            docs = None
            if documents:
                docs = torch.zeros(B, T, dtype=torch.long)
                docs[0, 13:] = 1
                docs[0, 31:] = 2
                docs[1, 22:] = 1
            with torch.no_grad():
                hidden, (keys, values) = block(
                    x, num_passes=PASSES, cyclic_groups=GROUPS, document_ids=docs, output_final_state=True
                )
            lead = int(dummy)
            assert hidden.shape == (B, T, HIDDEN) and keys.shape == (B, CHANNELS, KV_HEADS, T + lead, HEAD_DIM)
            arrays[f"{case}/x"] = x.numpy()
            arrays[f"{case}/hidden"] = hidden.numpy()
            arrays[f"{case}/keys"] = keys.numpy()
            arrays[f"{case}/values"] = values.numpy()
            if docs is not None:
                arrays[f"{case}/documents"] = docs.numpy()
    for name, value in shared.items():
        arrays[f"state/{name}"] = value.numpy()
    np.savez_compressed(HERE / "block_vectors.npz", **arrays)
    print(f"wrote {len(arrays)} arrays")


if __name__ == "__main__":
    main(sys.argv[1])
