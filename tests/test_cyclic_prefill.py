"""Cyclic prefill of a feedback block (the pass driver around the operators) against vectors of the upstream block."""

from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import assert_parity

VECTORS = np.load(Path(__file__).resolve().parent / "golden" / "block_vectors.npz")
CASES = sorted({name.split("/", 1)[0] for name in VECTORS.files if not name.startswith("state/")})
STATE = {name[len("state/"):]: torch.from_numpy(VECTORS[name]) for name in VECTORS.files if name.startswith("state/")}
HIDDEN, LAYERS, HEADS, HEAD_DIM, KV_HEADS, CHANNELS, MLP, THETA, GROUPS, PASSES = 128, 4, 2, 64, 2, 2, 128, 10_000.0, 4, 2


def get(case, name):
    key = f"{case}/{name}"
    return torch.from_numpy(VECTORS[key]) if key in VECTORS.files else None


def test_the_stored_cases_cover_dummy_and_documents():
    assert CASES == ["dummy0_docs0", "dummy0_docs1", "dummy1_docs0", "dummy1_docs1"]
    assert get("dummy1_docs1", "keys").shape == (2, CHANNELS, KV_HEADS, 41, HEAD_DIM)
    assert "dummy_token" in STATE and "kv_pool.mixer.k_router.linear.weight" in STATE


@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", CASES)
def test_prefill_matches_the_upstream_block(case, dtype):
    from white_matter_b200 import FeedbackBlock, _native

    dummy = case.startswith("dummy1")
    block = FeedbackBlock(
        HIDDEN, LAYERS, HEADS, HEAD_DIM, MLP, KV_HEADS, CHANNELS, rope_theta=THETA, use_dummy_token=dummy,
        router_layer_stride=2, num_passes=PASSES, device="cuda", dtype=dtype,
    )
    block.load_state_dict(STATE)
    x = get(case, "x").cuda().to(dtype)
    docs = get(case, "documents")
    hidden, (keys, values) = block(
        x, cyclic_groups=GROUPS, document_ids=None if docs is None else docs.cuda(), output_final_state=True
    )
    assert _native.device_status(True) == 0
    if dtype == torch.float32:
        # fp32 kernels (SIMT attention, FP32-pipe pool mixing) against the fp32 upstream run: round-off only
        tol = dict(max_abs_tol=2e-3, rel_l2_tol=5e-4)
    else:
        # bf16 through 2 passes x 4 layers of residual updates, against fp32: a few bf16 roundings deep
        tol = dict(max_abs_tol=6e-2, rel_l2_tol=3e-2)
    assert_parity(hidden.float(), get(case, "hidden"), what="hidden", **tol)
    assert_parity(keys.float(), get(case, "keys"), what="pool keys", **tol)
    assert_parity(values.float(), get(case, "values"), what="pool values", **tol)


@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")
def test_argument_errors():
    from white_matter_b200 import FeedbackBlock

    block = FeedbackBlock(HIDDEN, LAYERS, HEADS, HEAD_DIM, MLP, KV_HEADS, CHANNELS, device="cuda")
    x = torch.randn(1, 12, HIDDEN, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="more tokens than residue groups"):
        block(x[:, :4], cyclic_groups=4)
    with pytest.raises(ValueError, match="positive integer"):
        block(x, cyclic_groups=0)
    with pytest.raises(ValueError, match="built for"):
        block(x.float(), cyclic_groups=4)
