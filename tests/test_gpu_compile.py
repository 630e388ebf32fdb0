"""The operators under torch.compile(fullgraph=True), CUDA-graph replay and torch.library.opcheck.

Upstream keeps its operators traceable as one graph and its decode step replayable with lengths that change on the
device (tests/unit/test_strict_causal_attention.py:277-331, tests/gpu/test_cyclic_strict_past.py:77-89).  The graphs
are compiled with the "aot_eager" backend: what is under test is that the Python wrappers trace without a graph break,
that the fake implementations describe the real outputs, and that autograd is registered -- not a code generator.
"""

import pytest
import torch

from helpers import BF16_TOL, assert_parity, geometric_documents
from oracle import attention_oracle as oracle
from white_matter_b200 import cyclic_attention, operators, prepare_feedback_metadata, strict_causal_attention

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")]


@pytest.mark.parametrize("documents", [False, True])
def test_cyclic_attention_traces_as_one_graph_for_every_residue(documents):
    torch._dynamo.reset()
    torch.manual_seed(3)
    B, H, T, D, S = 2, 4, 264, 64, 8
    k = torch.randn(B, H, T, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, H, T, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    docs = geometric_documents(B, T, 90, seed=2)
    groups = [torch.arange(r, T, S) for r in range(S)]
    metas = prepare_feedback_metadata(docs, groups, T, use_dummy_token=False) if documents else [None] * S

    def run(q, k, v, residue, metadata):
        return cyclic_attention(q, k, v, query_stride=S, query_offset=residue, strict_past=True, metadata=metadata, backend="sm100")

    compiled = torch.compile(run, fullgraph=True, backend="aot_eager")
    for residue in range(S):
        md = None if metas[residue] is None else tuple(t.cuda() for t in metas[residue])
        q = torch.randn(B, H, T // S, D, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        probe = torch.randn_like(q)
        out = compiled(q, k, v, residue, md)
        grads = torch.autograd.grad(out, (q, k, v), probe)
        # the residue is a plain kernel argument: a second call with the same residue and fresh data compiles nothing
        with torch.compiler.set_stance("fail_on_recompile"):
            again = compiled(q, k, v, residue, md)
        assert torch.equal(out, again)
        qo, ko, vo = (t.detach().cpu().double().requires_grad_() for t in (q, k, v))
        exp = oracle.cyclic_attention_oracle(qo, ko, vo, query_stride=S, query_offset=residue, strict_past=True, metadata=metas[residue])
        exp_grads = torch.autograd.grad(exp, (qo, ko, vo), probe.cpu().double())
        assert_parity(out.float(), exp, what=f"out r={residue}", **BF16_TOL)
        for g, e, name in zip(grads, exp_grads, ("dq", "dk", "dv")):
            assert_parity(g.float(), e, what=f"{name} r={residue}", **BF16_TOL)


@pytest.mark.parametrize("dummy", [False, True])
@pytest.mark.parametrize("strided", [False, True])
@torch.no_grad()
def test_compiled_decode_replays_with_lengths_that_change_on_the_device(dummy, strided):
    torch._dynamo.reset()
    torch.manual_seed(4)
    q = torch.randn(3, 4, 1, 64, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(3, 4 if strided else 2, 33 + int(dummy), 64, device="cuda", dtype=torch.bfloat16)
    v = torch.randn_like(k)
    if strided:
        k, v = k[:, :2], v[:, :2]
    lengths = torch.tensor([0, 7, 16], device="cuda", dtype=torch.int32)

    def run(q, k, v, lengths):
        return strict_causal_attention(q, k, v, query_start=lengths, use_dummy_token=dummy, static_cache=True)

    compiled = torch.compile(run, fullgraph=True, backend="aot_eager")
    compiled(q, k, v, lengths)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        compiled(q, k, v, lengths)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = compiled(q, k, v, lengths)
    for values in ([0, 7, 16], [3, 12, 32]):
        lengths.copy_(torch.tensor(values, device="cuda", dtype=torch.int32))
        for row, n in enumerate(values):
            k[row, :, : n + int(dummy)].normal_()
            v[row, :, : n + int(dummy)].normal_()
            k[row, :, n + int(dummy):] = float("nan")
            v[row, :, n + int(dummy):] = float("nan")
        with torch.compiler.set_stance("fail_on_recompile"):
            actual = compiled(q, k, v, lengths)
        graph.replay()
        exp = oracle.strict_per_query_oracle(q.cpu(), k.cpu(), v.cpu(), lengths.cpu(), dummy)
        assert_parity(actual.float(), exp, what="compiled", **BF16_TOL)
        assert_parity(captured.float(), exp, what="replayed", **BF16_TOL)


def _opcheck(op, args, **kwargs):
    torch.library.opcheck(op, args, kwargs, test_utils=("test_schema", "test_faketensor", "test_autograd_registration", "test_aot_dispatch_dynamic"))


def test_opcheck_of_the_registered_operators():
    torch.manual_seed(6)
    dev, bf = "cuda", torch.bfloat16
    q = torch.randn(2, 4, 33, 64, device=dev, dtype=bf, requires_grad=True)
    k = torch.randn(2, 2, 132, 64, device=dev, dtype=bf, requires_grad=True)
    v = torch.randn(2, 2, 132, 64, device=dev, dtype=bf, requires_grad=True)
    _opcheck(operators.cyclic_attn_fwd, (q, k, v, 4, 1, 0))
    out, lse = operators.cyclic_attn_fwd(q, k, v, 4, 1, 0)
    # the backward operator is not differentiable itself: every tensor goes in detached
    _opcheck(operators.cyclic_attn_bwd, (q.detach(), k.detach(), v.detach(), out.detach(), lse.detach(), torch.randn_like(out).detach(), 4, 1, 0))
    seg = torch.stack((torch.arange(132) // 19, torch.arange(132) // 31))
    from white_matter_b200 import prepare_cyclic_attention_metadata

    md = tuple(t.to(dev) for t in prepare_cyclic_attention_metadata(seg[:, 1::4], torch.cat((seg.new_full((2, 1), -1), seg[:, :-1]), 1)))
    _opcheck(operators.cyclic_attn_doc_fwd, (q, k, v, *md, 4, 1, 0))
    lengths = torch.tensor([5, 100], device=dev, dtype=torch.int32)
    _opcheck(operators.strict_attn_fwd, (q, k, v, lengths, 0, lengths, None, False, 0.125, 0))
    # strict family with document tables: 33 queries at per-row positions over 132 key slots
    from white_matter_b200 import prepare_strict_causal_metadata

    starts = torch.tensor([10, 90], device=dev, dtype=torch.int32)
    schedule = prepare_strict_causal_metadata(seg.to(dev), 33, query_start=starts, kv_lengths=lengths + 20)
    tables = schedule.document_tables(torch.device(dev), 132)
    start_t, limit_t = schedule.dense_bounds(torch.device(dev))
    _opcheck(operators.strict_doc_fwd, (q, k, v, *tables, start_t, 0, limit_t, False, 0.125, 0))
    sout, slse = operators.strict_doc_fwd(q, k, v, *tables, start_t, 0, limit_t, False, 0.125, 0)
    _opcheck(operators.strict_doc_bwd, (q.detach(), k.detach(), v.detach(), *tables, start_t, 0, limit_t, sout.detach(),
                                        slse.detach(), torch.randn_like(sout).detach(), False, 0.125, 0))
    q1 = torch.randn(2, 4, 1, 64, device=dev, dtype=bf)
    _opcheck(operators.strict_decode, (q1, k.detach(), v.detach(), lengths, 0, lengths, None, False, 0.125))
    src = torch.randn(5, 2, 2, 16, 64, device=dev, dtype=bf, requires_grad=True)
    logits = torch.randn(5, device=dev, requires_grad=True)
    _opcheck(operators.mix_sources, (src, logits))
    x = torch.randn(2, 16, 4, 64, device=dev, dtype=bf, requires_grad=True)
    w = torch.ones(64, device=dev, dtype=bf, requires_grad=True)
    ang = torch.rand(1, 16, 64, device=dev)
    _opcheck(operators.query_prepare, (x, w, ang.cos().to(bf), ang.sin().to(bf), 1e-6, True))
