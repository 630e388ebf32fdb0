"""The CPU oracle against the vectors produced by the upstream portable backend."""

from types import SimpleNamespace

import pytest
import torch

from helpers import Golden, max_abs
from oracle import attention_oracle as oracle

G = Golden()


def _meta_from_golden(case):
    c = G.cases[case]
    return SimpleNamespace(
        query_indices=G.get(case, "query_indices"),
        key_indices=G.get(case, "key_indices"),
        cu_queries=G.get(case, "cu_queries"),
        cu_keys=G.get(case, "cu_keys"),
        key_extent=c["key_extent"],
    )


@pytest.mark.parametrize("case", G.names("cyclic"))
def test_cyclic_oracle_matches_reference_outputs_and_gradients(case):
    c = G.cases[case]
    q, k, v, probe, metadata = G.cyclic_inputs(case)
    q, k, v = (t.double().requires_grad_() for t in (q, k, v))
    out = oracle.cyclic_attention_oracle(
        q, k, v, query_stride=c["stride"], query_offset=c["offset"], strict_past=c["strict_past"], metadata=metadata
    )
    grads = torch.autograd.grad(out, (q, k, v), probe.double())
    # the stored results are fp32 evaluations; fp64 agrees to fp32 round-off
    assert max_abs(out, G.get(case, "out_f32")) < 2e-5
    for g, name in zip(grads, ("dq_f32", "dk_f32", "dv_f32")):
        assert max_abs(g, G.get(case, name)) < 5e-5, name


def test_config1_first_token_is_zero_and_sees_only_earlier_keys():
    q, k, v, probe, _ = G.cyclic_inputs("c1")
    out = oracle.cyclic_attention_oracle(q, k, v, query_stride=4, query_offset=0, strict_past=True)
    assert out[:, :, 0].abs().max() == 0
    keep = oracle.cyclic_keep_mask(64, 256, 4, 0, None, strict_past=True)
    assert int(keep.sum()) == 8064  # sum_i 4*i pairs per (batch, head)


@pytest.mark.parametrize("case", G.names("strict"))
def test_strict_oracle_matches_reference(case):
    c = G.cases[case]
    d = G.strict_inputs(case)
    q, k, v = (d[n].double().requires_grad_(c["grads"]) for n in ("q", "k", "v"))
    metadata = _meta_from_golden(case) if c["packed"] else None
    out = oracle.strict_causal_oracle(
        q, k, v, query_start=d["query_start"], kv_lengths=d["kv_lengths"], use_dummy_token=d["dummy"],
        metadata=metadata, key_mask=d["key_mask"],
    )
    assert torch.isfinite(out).all()
    assert max_abs(out, G.get(case, "out_f32")) < 2e-5
    if c["grads"]:
        grads = torch.autograd.grad(out, (q, k, v), d["probe"].double())
        for g, name in zip(grads, ("dq_f32", "dk_f32", "dv_f32")):
            assert max_abs(g, G.get(case, name)) < 5e-5, name


@pytest.mark.parametrize("case", [n for n in G.names("strict") if G.cases[n]["T"] <= 8])
def test_per_query_oracle_agrees_with_reference(case):
    c = G.cases[case]
    d = G.strict_inputs(case)
    if d["key_mask"] is not None:
        pytest.skip("the per-query restatement has no key_mask")
    start = d["query_start"]
    starts = start if isinstance(start, torch.Tensor) else torch.full((c["B"],), start)
    out = oracle.strict_per_query_oracle(d["q"], d["k"], d["v"], starts, d["dummy"], d["docs"], d["kv_lengths"])
    assert max_abs(out, G.get(case, "out_f32")) < 2e-5


def test_current_and_future_keys_have_zero_gradient():
    torch.manual_seed(0)
    q = torch.randn(1, 2, 1, 8, requires_grad=True)
    k = torch.randn(1, 1, 7, 8, requires_grad=True)
    v = torch.randn_like(k, requires_grad=True)
    oracle.strict_causal_oracle(q, k, v, query_start=3).sum().backward()
    assert k.grad[..., 3:, :].count_nonzero() == v.grad[..., 3:, :].count_nonzero() == 0


def test_mixing_oracle_is_a_convex_combination():
    torch.manual_seed(1)
    src = torch.randn(5, 3, 4)
    logits = torch.randn(5)
    out = oracle.mix_sources_oracle(src, logits)
    w = torch.softmax(logits.double(), 0)
    assert torch.allclose(out, sum(w[s] * src[s].double() for s in range(5)))
    assert torch.allclose(oracle.mix_sources_oracle(src[:1], logits[:1]), src[0].double())
