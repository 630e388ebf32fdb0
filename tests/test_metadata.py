"""Host-side schedule building against the upstream results and known answers."""

import pytest
import torch

from helpers import Golden
from white_matter_b200 import (
    prepare_cyclic_attention_metadata,
    prepare_feedback_metadata,
    prepare_strict_causal_metadata,
)

G = Golden()


@pytest.mark.parametrize("case", G.names("schedule"))
def test_strict_schedule_equals_upstream(case):
    c = G.cases[case]
    m = prepare_strict_causal_metadata(
        G.get(case, "docs"), c["T"], query_start=G.get(case, "start"), kv_lengths=G.maybe(case, "lengths"),
        use_dummy_token=c["dummy"],
    )
    assert torch.equal(m.query_indices, G.get(case, "query_indices"))
    assert torch.equal(m.key_indices, G.get(case, "key_indices"))
    assert torch.equal(m.cu_queries, G.get(case, "cu_queries")) and m.cu_queries.dtype == torch.int32
    assert torch.equal(m.cu_keys, G.get(case, "cu_keys")) and m.cu_keys.dtype == torch.int32
    assert (m.max_queries, m.max_keys, m.key_extent) == (c["max_queries"], c["max_keys"], c["key_extent"])


@pytest.mark.parametrize("case", [n for n in G.names("strict") if G.cases[n]["packed"]])
def test_strict_schedule_of_attention_cases(case):
    c = G.cases[case]
    d = G.strict_inputs(case)
    m = prepare_strict_causal_metadata(
        d["docs"], c["T"], query_start=d["query_start"], kv_lengths=d["kv_lengths"], use_dummy_token=c["dummy"]
    )
    for name in ("query_indices", "key_indices", "cu_queries", "cu_keys"):
        assert torch.equal(getattr(m, name), G.get(case, name)), name


def test_packed_jacobi_known_group_offsets():
    # upstream tests/unit/test_jacobi_flash_packing.py:15-16
    documents = torch.tensor([[0, 0, 1, 1, 1, 2], [0, 1, 1, 2, 3, 3]])
    schedule = prepare_strict_causal_metadata(documents, 6, use_dummy_token=True)
    assert schedule.cu_queries.tolist() == [0, 2, 5, 6, 7, 9, 10, 12]


def test_empty_schedule():
    # upstream tests/unit/test_strict_causal_attention.py:177-180
    m = prepare_strict_causal_metadata(torch.empty(2, 0, dtype=torch.long), 0)
    assert m.query_indices.numel() == m.key_indices.numel() == 0
    assert m.cu_queries.tolist() == m.cu_keys.tolist() == [0]


def test_schedule_rejects_unlabelled_query_positions():
    with pytest.raises(ValueError, match="label every query position"):
        prepare_strict_causal_metadata(torch.zeros(1, 4, dtype=torch.long), 3, query_start=2)


def test_with_key_extent_readdresses_slots():
    docs = torch.tensor([[0, 0, 1, 1]])
    m = prepare_strict_causal_metadata(docs, 4, use_dummy_token=True)
    wide = m.with_key_extent(9)
    assert wide.key_extent == 9 and torch.equal(wide.key_indices % 9, m.key_indices % 5)
    assert m.with_key_extent(5) is m


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_cyclic_metadata_known_answer(dtype):
    # upstream tests/unit/test_ops.py:77-86
    top = torch.iinfo(torch.int32).max
    metadata = prepare_cyclic_attention_metadata(
        torch.tensor([[0, top]], dtype=dtype), torch.tensor([[-1, 0, top]], dtype=dtype)
    )
    expected = ([[0, top]], [[-1, 0, top]], [[1, 2]], [[2, 1, 2]])
    for actual, values in zip(metadata, expected, strict=True):
        assert torch.equal(actual, torch.tensor(values, dtype=torch.int32))


@pytest.mark.parametrize("which", ["query", "key"])
def test_cyclic_metadata_rejects_ids_beyond_int32(which):
    q = torch.tensor([[0]], dtype=torch.int64)
    k = torch.tensor([[-1, 0]], dtype=torch.int64)
    (q if which == "query" else k)[:, -1] = torch.iinfo(torch.int32).max + 1
    with pytest.raises(ValueError, match="segment IDs must fit int32"):
        prepare_cyclic_attention_metadata(q, k)


def test_cyclic_metadata_requires_dummy():
    with pytest.raises(ValueError, match="dummy"):
        prepare_cyclic_attention_metadata(torch.zeros(1, 3, dtype=torch.long), torch.zeros(1, 3, dtype=torch.long))


@pytest.mark.parametrize("case", [n for n in G.names("cyclic") if G.cases[n]["docs"] == "sorted"])
def test_cyclic_metadata_equals_upstream(case):
    c = G.cases[case]
    seg = torch.stack([torch.arange(c["K"]) // (19 + 12 * b) for b in range(c["B"])])
    m = prepare_cyclic_attention_metadata(
        seg[:, c["offset"] :: c["stride"]][:, : c["Q"]], torch.cat((seg.new_full((c["B"], 1), -1), seg[:, :-1]), 1)
    )
    for got, name in zip(m, ("q_seg", "k_seg", "q_start", "k_end")):
        assert torch.equal(got, G.get(case, name)), name


@pytest.mark.parametrize("case", G.names("feedback"))
def test_feedback_metadata_equals_upstream(case):
    c = G.cases[case]
    docs = G.get(case, "docs")
    groups = [torch.arange(r, c["T"], c["stride"]) for r in range(c["stride"])]
    ms = prepare_feedback_metadata(docs, groups, c["key_length"], use_dummy_token=c["dummy"])
    assert len(ms) == c["stride"]
    for r, m in enumerate(ms):
        for got, name in zip(m, ("q_seg", "k_seg", "q_start", "k_end")):
            assert torch.equal(got, G.get(case, f"{name}_{r}")), (r, name)
