"""Argument checks of the public operators (no GPU needed: every check precedes the launch)."""

import pytest
import torch

from white_matter_b200 import cyclic_attention, mix_kv_sources, strict_causal_attention


def test_cyclic_argument_errors():
    q = torch.randn(1, 2, 3, 8)
    with pytest.raises(ValueError, match="unknown cyclic attention backend"):
        cyclic_attention(q, q, q, backend="tilelang")
    with pytest.raises(ValueError, match="query_stride must be a positive integer"):
        cyclic_attention(q, q, q, query_stride=0)
    with pytest.raises(ValueError, match="query_offset"):
        cyclic_attention(q, q, q, query_offset=-1)
    with pytest.raises(ValueError, match="query slots must be within the key sequence"):
        cyclic_attention(q, q, q, query_stride=2)
    with pytest.raises(ValueError, match="Q/K/V must share dtype and device"):
        cyclic_attention(q, q.double(), q.double())
    with pytest.raises(ValueError, match="document metadata requires four tensors"):
        cyclic_attention(q, q, q, metadata=(torch.zeros(1, 3),))
    with pytest.raises(ValueError, match="CUDA BF16"):
        cyclic_attention(q, q, q)  # CPU tensors: there is no fallback


def test_strict_argument_errors():
    q = torch.randn(1, 2, 3, 8)
    with pytest.raises(ValueError, match="unsupported strict causal backend"):
        strict_causal_attention(q, q, q, backend="torch_flash")
    with pytest.raises(ValueError, match="use_dummy_token must be boolean"):
        strict_causal_attention(q, q, q, use_dummy_token=1)
    with pytest.raises(ValueError, match=r"kv_lengths must be integer \(B,\)"):
        strict_causal_attention(q, q, q, kv_lengths=torch.zeros(2, dtype=torch.long))
    with pytest.raises(ValueError, match="metadata and key_mask are mutually exclusive"):
        strict_causal_attention(q, q, q, metadata=object(), key_mask=torch.ones(1, 3, dtype=torch.bool))
    with pytest.raises(ValueError, match=r"key_mask must be boolean \(B,N\)"):
        strict_causal_attention(q, q, q, key_mask=torch.ones(1, 3))
    with pytest.raises(ValueError, match="requires CUDA"):
        strict_causal_attention(q, q, q)


def test_mixing_argument_errors():
    with pytest.raises(ValueError, match="sources must be"):
        mix_kv_sources(torch.randn(3), torch.randn(3))
    with pytest.raises(ValueError, match="requires CUDA"):
        mix_kv_sources(torch.randn(3, 4), torch.randn(3))
