"""Generate tests/golden/pool_vectors.npz from the upstream package.

    python tests/golden/make_pool_golden.py /path/to/upstream/src

Runs the upstream ``KVPool`` (modules/kv_pool.py) with every parameter randomised -- pre-mix gains, router weights
and biases, post-mix gains, projections, key-norm gains -- on small seeded layer stacks, in FP32 on the CPU:
``project_sequence`` for a dynamic router over every source, a dynamic router over every second source with a
leading dummy token, and a static router; ``project_token`` for a single decode row.  Inputs, parameters and
results are stored; the tests replay the file and never import the upstream package.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

CASES = {
    # name: (router_layer_stride, router_dynamic, dummy token, tokens)
    "dynamic": (1, True, False, 6),
    "strided_dummy": (2, True, True, 5),
    "static": (1, False, False, 4),
    "static_dummy": (1, False, True, 3),
}
B, L, DM, CH, HKV, D = 2, 5, 128, 3, 2, 64


def main(upstream_src: str) -> None:
    sys.path.insert(0, upstream_src)
    from white_matter.modules import KVPool

    arrays: dict[str, np.ndarray] = {}
    for index, (case, (stride, dynamic, dummy, tokens)) in enumerate(CASES.items()):
        torch.manual_seed(40 + index)
        pool = KVPool(DM, HKV, D, L, CH, router_layer_stride=stride, router_dynamic=dynamic).eval()
        with torch.no_grad():
            for parameter in pool.parameters():
                parameter.copy_(torch.randn_like(parameter) * (0.05 if parameter.ndim == 3 else 0.5))
            for router in (pool.mixer.k_router, pool.mixer.v_router):
                router.linear.weight.mul_(0.1)
            pool.k_norm_weight.add_(1.0)
        stacked = torch.randn(B, tokens, L, DM) * (1.0 + torch.rand(1, 1, L, 1))
        dummy_token = torch.randn(1, 1, DM) if dummy else None
        total = tokens + int(dummy)
        angle = torch.rand(B, total, D // 2) * 6.283
        cos = torch.cat((angle.cos(), angle.cos()), -1)
        sin = torch.cat((angle.sin(), angle.sin()), -1)
        with torch.no_grad():
            keys, values = pool.project_sequence(stacked, (cos, sin), dummy_token=dummy_token)
            token_keys, token_values = pool.project_token(
                [stacked[:, -1:, l] for l in range(L)], (cos[:, -1:], sin[:, -1:])
            )
        assert keys.shape == (B, CH, HKV, total, D) and token_keys.shape == (CH, B, HKV, 1, D)
        state = pool.state_dict()
        arrays.update(
            {
                f"{case}/stacked": stacked.numpy(),
                f"{case}/cos": cos.numpy(),
                f"{case}/sin": sin.numpy(),
                f"{case}/keys": keys.numpy(),
                f"{case}/values": values.numpy(),
                f"{case}/token_keys": token_keys.numpy(),
                f"{case}/token_values": token_values.numpy(),
                f"{case}/route_stride": np.array(stride),
                f"{case}/dynamic": np.array(dynamic),
            }
        )
        if dummy:
            arrays[f"{case}/dummy"] = dummy_token.numpy()
        for name, value in state.items():
            arrays[f"{case}/state/{name}"] = value.numpy()
    np.savez_compressed(HERE / "pool_vectors.npz", **arrays)
    print(f"wrote {len(arrays)} arrays for {len(CASES)} cases")


if __name__ == "__main__":
    main(sys.argv[1])
