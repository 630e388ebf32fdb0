"""strict_causal_attention on the GPU: Jacobi prefill, cached-prefix prefill and decode (through the C ABI)."""

import pytest
import torch

from helpers import BF16_TOL, F32_TOL, Golden, assert_parity, geometric_documents
from oracle import attention_oracle as oracle
from white_matter_b200 import _native, prepare_strict_causal_metadata, strict_causal_attention

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")]
G = Golden()
BACKENDS = ["sm100_simt", "sm100"]


def run_case(case, dtype, backend):
    c = G.cases[case]
    d = G.strict_inputs(case)
    dev = "cuda"
    q, k, v = (d[n].to(dev, dtype).requires_grad_(c["grads"]) for n in ("q", "k", "v"))
    start = d["query_start"].to(dev) if isinstance(d["query_start"], torch.Tensor) else d["query_start"]
    lengths = None if d["kv_lengths"] is None else d["kv_lengths"].to(dev)
    mask = None if d["key_mask"] is None else d["key_mask"].to(dev)
    metadata = None
    if c["packed"]:
        metadata = prepare_strict_causal_metadata(
            d["docs"].to(dev), c["T"], query_start=start, kv_lengths=lengths, use_dummy_token=c["dummy"]
        )
    out = strict_causal_attention(
        q, k, v, query_start=start, kv_lengths=lengths, use_dummy_token=c["dummy"], metadata=metadata, key_mask=mask,
        backend=backend,
    )
    assert out.shape == (c["B"], c["T"], c["H"], c["D"])
    grads = None
    if c["grads"]:
        grads = torch.autograd.grad(out, (q, k, v), d["probe"].to(dev, dtype))
    return out, grads, d


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("case", G.names("strict"))
def test_fp32_matches_reference_vectors(case, backend):
    out, grads, _ = run_case(case, torch.float32, backend)
    assert_parity(out, G.get(case, "out_f32"), what="out", **F32_TOL)
    if grads is not None:
        for g, name in zip(grads, ("dq_f32", "dk_f32", "dv_f32")):
            assert_parity(g, G.get(case, name), what=name, **F32_TOL)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("case", G.names("strict"))
def test_bf16_matches_reference(case, backend):
    c = G.cases[case]
    out, grads, d = run_case(case, torch.bfloat16, backend)
    qo, ko, vo = (d[n].bfloat16().double().requires_grad_(c["grads"]) for n in ("q", "k", "v"))
    metadata = None
    if c["packed"]:
        metadata = prepare_strict_causal_metadata(
            d["docs"], c["T"], query_start=d["query_start"], kv_lengths=d["kv_lengths"], use_dummy_token=c["dummy"]
        )
    exp = oracle.strict_causal_oracle(
        qo, ko, vo, query_start=d["query_start"], kv_lengths=d["kv_lengths"], use_dummy_token=c["dummy"],
        metadata=metadata, key_mask=d["key_mask"],
    )
    assert_parity(out.float(), exp, what="out", **BF16_TOL)
    if grads is not None:
        exp_grads = torch.autograd.grad(exp, (qo, ko, vo), d["probe"].bfloat16().double())
        for g, e, name in zip(grads, exp_grads, ("dq", "dk", "dv")):
            assert_parity(g.float(), e, what=name, **BF16_TOL)


TENSOR_CORE_CASES = [n for n in G.names("strict") if G.cases[n]["D"] == 64 and G.cases[n]["T"] > 1]


@pytest.mark.parametrize("case", TENSOR_CORE_CASES)
def test_bf16_reference_cases_on_the_tensor_core_kernels(case):
    """Every stored strict case with several queries and heads of 64 -- dense, truncated, packed, padded, Jacobi, with
    and without the dummy slot -- runs the tcgen05 kernels when they are forced (a problem they cannot take is an
    error then), forward and gradients."""
    test_bf16_matches_reference(case, "sm100_tcgen05")
    assert _native.device_status(True) == 0


@pytest.mark.parametrize("dummy", [False, True])
def test_unused_capacity_may_hold_nan(dummy):
    # upstream tests/unit/test_strict_causal_attention.py:80-94
    torch.manual_seed(2)
    q = torch.randn(3, 4, 1, 64, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(3, 2, 9 + int(dummy), 64, device="cuda", dtype=torch.bfloat16)
    v = torch.randn_like(k)
    lengths = torch.tensor([0, 3, 7], device="cuda", dtype=torch.int32)
    for b, n in enumerate(lengths.tolist()):
        k[b, :, n + int(dummy):] = float("nan")
        v[b, :, n + int(dummy):] = float("nan")
    out = strict_causal_attention(q, k, v, query_start=lengths, kv_lengths=lengths, use_dummy_token=dummy)
    exp = oracle.strict_per_query_oracle(q.cpu(), k.cpu(), v.cpu(), lengths.cpu(), dummy)
    assert torch.isfinite(out).all()
    assert_parity(out.float(), exp, what="decode", **BF16_TOL)
    if not dummy:
        assert out[0].abs().max().item() == 0  # a row without keys is exactly zero


def test_future_keys_get_exactly_zero_gradient():
    q = torch.randn(1, 2, 1, 64, device="cuda", requires_grad=True)
    k = torch.randn(1, 1, 7, 64, device="cuda", requires_grad=True)
    v = torch.randn_like(k, requires_grad=True)
    strict_causal_attention(q, k, v, query_start=3).sum().backward()
    assert k.grad[..., 3:, :].count_nonzero() == v.grad[..., 3:, :].count_nonzero() == 0
    assert k.grad[..., :3, :].count_nonzero() > 0


@pytest.mark.parametrize("dummy", [False, True])
def test_decode_in_cuda_graph_with_device_lengths(dummy):
    # upstream tests/unit/test_strict_causal_attention.py:277-331: lengths change between replays
    torch.manual_seed(4)
    q = torch.randn(3, 4, 1, 64, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(3, 4, 33 + int(dummy), 64, device="cuda", dtype=torch.bfloat16)[:, :2]  # strided head view
    v = torch.randn(3, 4, 33 + int(dummy), 64, device="cuda", dtype=torch.bfloat16)[:, :2]
    lengths = torch.tensor([0, 7, 16], device="cuda", dtype=torch.int32)

    def step():
        return strict_causal_attention(q, k, v, query_start=lengths, use_dummy_token=dummy, static_cache=True)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = step()
    for values in ([0, 7, 16], [3, 12, 32]):
        lengths.copy_(torch.tensor(values, device="cuda", dtype=torch.int32))
        for row, n in enumerate(values):
            k[row, :, : n + int(dummy)].normal_()
            v[row, :, : n + int(dummy)].normal_()
            k[row, :, n + int(dummy):] = float("nan")
            v[row, :, n + int(dummy):] = float("nan")
        graph.replay()
        eager = step()
        exp = oracle.strict_per_query_oracle(q.cpu(), k.cpu(), v.cpu(), lengths.cpu(), dummy)
        assert_parity(captured.float(), exp, what="replayed", **BF16_TOL)
        assert torch.equal(captured, eager)


@pytest.mark.parametrize("backend", BACKENDS)
def test_jacobi_prefill_reuses_one_schedule(backend):
    """Packed documents (geometric lengths), one schedule reused over iterations with fresh Q/K/V."""
    B, H, T, D = 2, 4, 512, 64
    docs = geometric_documents(B, T, 128, seed=7)
    schedule = prepare_strict_causal_metadata(docs.cuda(), T)
    cpu_schedule = prepare_strict_causal_metadata(docs, T)
    for it in range(2):
        torch.manual_seed(100 + it)
        q = (torch.randn(B, H, T, D) / 8).bfloat16()
        k = torch.randn(B, H, T, D).bfloat16()
        v = torch.randn(B, H, T, D).bfloat16()
        out = strict_causal_attention(q.cuda(), k.cuda(), v.cuda(), metadata=schedule, backend=backend)
        exp = oracle.strict_causal_oracle(q, k, v, metadata=cpu_schedule)
        assert_parity(out.float(), exp, what=f"iteration {it}", **BF16_TOL)
        starts = torch.ones_like(docs, dtype=torch.bool)
        starts[:, 1:] = docs[:, 1:] != docs[:, :-1]
        assert out[starts.cuda()].abs().max().item() == 0  # each document's first token


def test_pool_read_at_full_size_matches_a_device_side_evaluation():
    """B=64,H=16,D=64 pool of 8192 slots, lengths uniform in [1,8192]; decode and 128-token cached-prefix prefill.

    Too large for the CPU oracle: the expected values are evaluated per batch
    row with plain fp32 tensor arithmetic on the device.
    """
    torch.manual_seed(0)
    B, H, N, D = 64, 16, 8192, 64
    lengths = torch.randint(1, N + 1, (B,), device="cuda")
    k = torch.randn(B, H, N, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(B, H, N, D, device="cuda", dtype=torch.bfloat16)
    for b in range(B):
        k[b, :, int(lengths[b]):] = float("nan")
        v[b, :, int(lengths[b]):] = float("nan")
    q1 = torch.randn(B, H, 1, D, device="cuda", dtype=torch.bfloat16)
    out = strict_causal_attention(q1, k, v, query_start=lengths, kv_lengths=lengths)
    q128 = torch.randn(B, H, 128, D, device="cuda", dtype=torch.bfloat16)
    starts = (lengths - 128).clamp_min(0)
    pre = strict_causal_attention(q128, k, v, query_start=starts, kv_lengths=lengths)
    for b in range(0, B, 7):
        n = int(lengths[b])
        kk, vv = k[b, :, :n].float(), v[b, :, :n].float()
        exp = torch.softmax(q1[b].float() @ kk.transpose(-1, -2) / 8, -1) @ vv
        assert_parity(out[b].transpose(0, 1).float(), exp, what=f"decode row {b}", **BF16_TOL)
        pos = int(starts[b]) + torch.arange(128, device="cuda")
        keep = torch.arange(n, device="cuda")[None, :] < pos[:, None]
        s = (q128[b].float() @ kk.transpose(-1, -2) / 8).masked_fill(~keep, float("-inf"))
        p = torch.softmax(s, -1).nan_to_num(0.0)
        assert_parity(pre[b].transpose(0, 1).float(), p @ vv, what=f"prefill row {b}", **BF16_TOL)


@pytest.mark.parametrize("backend", ["sm100_simt", "sm100"])
@pytest.mark.parametrize("pads", [False, True])
def test_softmax_scale_is_honoured_on_every_route(pads, backend):
    """A plain Jacobi schedule goes to the cyclic document kernels, a schedule with padding to the gathered ones:
    both have to use the caller's multiplier, forward and backward."""
    torch.manual_seed(31)
    B, H, T, D = 2, 2, 160, 64
    docs = geometric_documents(B, T, 40, seed=5)
    if pads:
        docs[:, 50:55] = -1
    q, k, v, probe = (torch.randn(B, H, T, D).bfloat16() for _ in range(4))
    schedule = prepare_strict_causal_metadata(docs.cuda(), T)
    qq, kk, vv = (t.cuda().requires_grad_() for t in (q, k, v))
    out = strict_causal_attention(qq, kk, vv, metadata=schedule, softmax_scale=0.3, backend=backend)
    grads = torch.autograd.grad(out, (qq, kk, vv), probe.transpose(1, 2).cuda())
    qo, ko, vo = (t.double().requires_grad_() for t in (q, k, v))
    exp = oracle.strict_causal_oracle(qo, ko, vo, metadata=prepare_strict_causal_metadata(docs, T), softmax_scale=0.3)
    exp_grads = torch.autograd.grad(exp, (qo, ko, vo), probe.transpose(1, 2).double())
    assert_parity(out.float(), exp, what="out", **BF16_TOL)
    for g, e, name in zip(grads, exp_grads, ("dq", "dk", "dv")):
        assert_parity(g.float(), e, what=name, **BF16_TOL)
    default = strict_causal_attention(qq, kk, vv, metadata=schedule, backend=backend)
    assert (default.float() - out.float()).abs().max().item() > 1e-2  # the multiplier does change the result


@pytest.mark.parametrize("backend", ["sm100_simt", "sm100_tcgen05"])
@pytest.mark.parametrize("masked", [False, True])
@pytest.mark.parametrize("length", [128, 200])
def test_gradients_with_nan_in_unused_capacity(length, masked, backend):
    """Cached-prefix prefill with gradients: slots at or beyond kv_lengths hold NaN; the gradients must be finite,
    match the oracle, and be exactly zero for the slots nobody sees."""
    torch.manual_seed(41)
    B, H, N, D = 2, 2, 333, 64
    lengths = torch.tensor([150, 290])
    starts = (lengths - length).clamp_min(0)
    q, probe = (torch.randn(B, H, length, D).bfloat16() for _ in range(2))
    k, v = (torch.randn(B, H, N, D).bfloat16() for _ in range(2))
    key_mask = None
    if masked:
        key_mask = torch.rand(B, N) > 0.2
    kn, vn = k.clone(), v.clone()
    for b in range(B):
        kn[b, :, int(lengths[b]):] = float("nan")
        vn[b, :, int(lengths[b]):] = float("nan")
    qq, kk, vv = (t.cuda().requires_grad_() for t in (q, kn, vn))
    out = strict_causal_attention(
        qq, kk, vv, query_start=starts.cuda(), kv_lengths=lengths.cuda(), key_mask=None if key_mask is None else key_mask.cuda(),
        backend=backend,
    )
    grads = torch.autograd.grad(out, (qq, kk, vv), probe.transpose(1, 2).cuda())
    qo, ko, vo = (t.double().requires_grad_() for t in (q, k, v))
    exp = oracle.strict_causal_oracle(qo, ko, vo, query_start=starts, kv_lengths=lengths, key_mask=key_mask)
    exp_grads = torch.autograd.grad(exp, (qo, ko, vo), probe.transpose(1, 2).double())
    assert_parity(out.float(), exp, what="out", **BF16_TOL)
    for g, e, name in zip(grads, exp_grads, ("dq", "dk", "dv")):
        assert torch.isfinite(g).all(), name
        assert_parity(g.float(), e, what=name, **BF16_TOL)
    for b in range(B):
        assert grads[1][b, :, int(lengths[b]):].abs().max().item() == 0
        assert grads[2][b, :, int(lengths[b]):].abs().max().item() == 0


@pytest.mark.parametrize("dummy", [False, True])
@pytest.mark.parametrize("heads,kv_heads", [(4, 4), (4, 2)])
@pytest.mark.parametrize("length", [128, 200, 37])
def test_key_mask_prefill_on_the_tcgen05_forward(length, heads, kv_heads, dummy):
    """Document-masked cached-prefix prefill: the key mask is applied per tile inside the tensor-core forward.  Slots
    the mask removes and slots beyond the committed lengths hold NaN in K and V; nothing of it may reach the result."""
    torch.manual_seed(77)
    B, N, D = 3, 700, 64
    lead = int(dummy)
    lengths = torch.tensor([650, 300, 129])
    starts = (lengths - length).clamp_min(0)
    q = torch.randn(B, heads, length, D).bfloat16()
    k, v = (torch.randn(B, kv_heads, N + lead, D).bfloat16() for _ in range(2))
    key_mask = torch.rand(B, N + lead) > 0.3
    key_mask[:, 0] = True
    key_mask[0, 128:256] = False  # a whole tile removed
    key_mask[1, :128] = True      # a whole tile kept
    kn, vn = k.clone(), v.clone()
    for b in range(B):
        kn[b, :, lead + int(lengths[b]):] = float("nan")
        vn[b, :, lead + int(lengths[b]):] = float("nan")
        kn[b][:, ~key_mask[b]] = float("nan")
        vn[b][:, ~key_mask[b]] = float("nan")
    args = dict(query_start=starts.cuda(), kv_lengths=lengths.cuda(), use_dummy_token=dummy, key_mask=key_mask.cuda())
    with torch.no_grad():
        out = strict_causal_attention(q.cuda(), kn.cuda(), vn.cuda(), backend="sm100_tcgen05", **args)
        simt = strict_causal_attention(q.cuda(), kn.cuda(), vn.cuda(), backend="sm100_simt", **args)
    exp = oracle.strict_causal_oracle(
        q.double(), k.double(), v.double(), query_start=starts, kv_lengths=lengths, use_dummy_token=dummy, key_mask=key_mask
    )
    assert torch.isfinite(out).all()
    assert_parity(out.float(), exp, what="tcgen05 forward with key_mask", **BF16_TOL)
    assert_parity(out.float(), simt.float(), what="tcgen05 vs simt", **BF16_TOL)
    # gradients: the key-stationary tensor-core backward clears the rows the mask removes in shared memory as well
    qq, kk, vv = (t.cuda().requires_grad_() for t in (q, kn, vn))
    out2 = strict_causal_attention(qq, kk, vv, backend="sm100_tcgen05", **args)
    probe = torch.randn_like(out2)
    grads = torch.autograd.grad(out2, (qq, kk, vv), probe)
    assert _native.device_status(True) == 0
    for b in range(B):
        assert all(torch.isfinite(g).all() for g in grads)
        assert grads[1][b][:, ~key_mask[b].cuda()].abs().max().item() == 0
        assert grads[2][b][:, ~key_mask[b].cuda()].abs().max().item() == 0
    qo, ko, vo = (t.double().requires_grad_() for t in (q, k, v))
    exp2 = oracle.strict_causal_oracle(qo, ko, vo, query_start=starts, kv_lengths=lengths, use_dummy_token=dummy, key_mask=key_mask)
    exp_grads = torch.autograd.grad(exp2, (qo, ko, vo), probe.cpu().double())
    for g, e, name in zip(grads, exp_grads, ("dq", "dk", "dv")):
        assert_parity(g.float(), e, what=name, **BF16_TOL)


@pytest.mark.parametrize("dummy", [False, True])
@pytest.mark.parametrize("backend", ["sm100_tcgen05", "sm100_simt"])
def test_padded_jacobi_schedule_on_the_tensor_core_kernels(backend, dummy):
    """Rows with padding (negative ids) at the end, in the middle of a document and at the start: padding is neither a
    query nor a key and does not end a run of equal ids.  Forward and gradients against the oracle's packed path."""
    torch.manual_seed(63)
    B, H, T, D = 3, 2, 300, 64
    lead = int(dummy)
    docs = torch.zeros(B, T, dtype=torch.long)
    docs[0, 120:] = 1
    docs[0, 250:] = -1                 # padded tail
    docs[1, 40:200] = 2
    docs[1, 90:110] = -1               # padding inside document 2: the run goes on behind it
    docs[1, 200:] = 0                  # id 0 again: a new run
    docs[2, :17] = -1                  # padded head
    docs[2, 17:] = 5
    q, probe = (torch.randn(B, H, T, D).bfloat16() for _ in range(2))
    k, v = (torch.randn(B, H, T + lead, D).bfloat16() for _ in range(2))
    schedule = prepare_strict_causal_metadata(docs.cuda(), T, use_dummy_token=dummy)
    assert schedule.dense_documents is not None  # whole rows: eligible for the stride-1 cyclic form
    qq, kk, vv = (t.cuda().requires_grad_() for t in (q, k, v))
    out = strict_causal_attention(qq, kk, vv, metadata=schedule, use_dummy_token=dummy, backend=backend)
    grads = torch.autograd.grad(out, (qq, kk, vv), probe.transpose(1, 2).cuda())
    qo, ko, vo = (t.double().requires_grad_() for t in (q, k, v))
    exp = oracle.strict_causal_oracle(qo, ko, vo, metadata=prepare_strict_causal_metadata(docs, T, use_dummy_token=dummy), use_dummy_token=dummy)
    exp_grads = torch.autograd.grad(exp, (qo, ko, vo), probe.transpose(1, 2).double())
    assert_parity(out.float(), exp, what="out", **BF16_TOL)
    assert out[0, 250:].abs().max().item() == 0 and out[1, 90:110].abs().max().item() == 0 and out[2, :17].abs().max().item() == 0
    for g, e, name in zip(grads, exp_grads, ("dq", "dk", "dv")):
        assert_parity(g.float(), e, what=name, **BF16_TOL)


@pytest.mark.parametrize("dummy", [False, True])
@pytest.mark.parametrize("backend", ["sm100_tcgen05", "sm100_simt"])
def test_cached_prefix_jacobi_with_documents_on_the_tensor_core_kernels(backend, dummy):
    """Jacobi over the last 150 tokens of rows whose earlier tokens are committed history: per-row first query
    position, per-row key limits, packed documents and padding, forward and gradients against the oracle's packed
    path (the tensor-core route takes the schedule as dense bounds plus document tables)."""
    torch.manual_seed(64)
    B, H, T, Q, D = 3, 2, 400, 150, 64
    lead = int(dummy)
    docs = torch.zeros(B, T, dtype=torch.long)
    docs[0, 130:] = 1
    docs[0, 300:] = 2
    docs[1, 60:390] = 4
    docs[1, 200:215] = -1              # padding inside the document, among the queries
    docs[1, 390:] = -1
    docs[2, :250] = 7
    docs[2, 250:] = 8                  # the queries of row 2 begin exactly at a document start
    starts = torch.tensor([250, 180, 250])
    limits = torch.tensor([400, 260, 333])  # row 1 and 2: keys stop before the last queries
    q, probe = (torch.randn(B, H, Q, D).bfloat16() for _ in range(2))
    k, v = (torch.randn(B, H, T + lead, D).bfloat16() for _ in range(2))
    schedule = prepare_strict_causal_metadata(docs.cuda(), Q, query_start=starts.cuda(), kv_lengths=limits.cuda(), use_dummy_token=dummy)
    assert schedule.dense_documents is not None
    qq, kk, vv = (t.cuda().requires_grad_() for t in (q, k, v))
    out = strict_causal_attention(qq, kk, vv, metadata=schedule, use_dummy_token=dummy, backend=backend)
    grads = torch.autograd.grad(out, (qq, kk, vv), probe.transpose(1, 2).cuda())
    qo, ko, vo = (t.double().requires_grad_() for t in (q, k, v))
    host_schedule = prepare_strict_causal_metadata(docs, Q, query_start=starts, kv_lengths=limits, use_dummy_token=dummy)
    exp = oracle.strict_causal_oracle(qo, ko, vo, metadata=host_schedule, use_dummy_token=dummy)
    exp_grads = torch.autograd.grad(exp, (qo, ko, vo), probe.transpose(1, 2).double())
    assert_parity(out.float(), exp, what="out", **BF16_TOL)
    assert out[1, 20:35].abs().max().item() == 0  # the padded queries of row 1
    for g, e, name in zip(grads, exp_grads, ("dq", "dk", "dv")):
        assert_parity(g.float(), e, what=name, **BF16_TOL)
