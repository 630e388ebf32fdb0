"""cyclic_attention on the GPU against the golden vectors and the CPU oracle (calls go through the C ABI)."""

import pytest
import torch

from helpers import BF16_TOL, F32_TOL, Golden, assert_parity, geometric_documents
from oracle import attention_oracle as oracle
from white_matter_b200 import cyclic_attention, prepare_cyclic_attention_metadata, prepare_feedback_metadata

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not torch.cuda.is_available(), reason="requires CUDA")]
G = Golden()
BACKENDS = ["sm100_simt", "sm100"]


def run(q, k, v, probe, metadata, c, dtype, backend):
    dev = "cuda"
    qq, kk, vv = (t.to(dev, dtype).requires_grad_() for t in (q, k, v))
    md = None if metadata is None else tuple(t.to(dev) for t in metadata)
    out = cyclic_attention(
        qq, kk, vv, query_stride=c["stride"], query_offset=c["offset"], strict_past=c["strict_past"], metadata=md,
        backend=backend,
    )
    assert out.transpose(1, 2).is_contiguous()  # (B,Q,H,D) storage, ready for the output projection
    grads = torch.autograd.grad(out, (qq, kk, vv), probe.to(dev, dtype))
    return out, grads


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("case", G.names("cyclic"))
def test_fp32_matches_reference_vectors(case, backend):
    c = G.cases[case]
    q, k, v, probe, metadata = G.cyclic_inputs(case)
    out, grads = run(q, k, v, probe, metadata, c, torch.float32, backend)
    assert_parity(out, G.get(case, "out_f32"), what="out", **F32_TOL)
    for g, name in zip(grads, ("dq_f32", "dk_f32", "dv_f32")):
        assert_parity(g, G.get(case, name), what=name, **F32_TOL)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("case", G.names("cyclic"))
def test_bf16_matches_reference(case, backend):
    c = G.cases[case]
    q, k, v, probe, metadata = G.cyclic_inputs(case)
    q, k, v, probe = (t.bfloat16() for t in (q, k, v, probe))
    out, grads = run(q, k, v, probe, metadata, c, torch.bfloat16, backend)
    # reference arithmetic on the same bf16 inputs
    qo, ko, vo = (t.double().requires_grad_() for t in (q, k, v))
    exp = oracle.cyclic_attention_oracle(
        qo, ko, vo, query_stride=c["stride"], query_offset=c["offset"], strict_past=c["strict_past"], metadata=metadata
    )
    exp_grads = torch.autograd.grad(exp, (qo, ko, vo), probe.double())
    assert_parity(out.float(), exp, what="out", **BF16_TOL)
    for g, e, name in zip(grads, exp_grads, ("dq", "dk", "dv")):
        assert_parity(g.float(), e, what=name, **BF16_TOL)
    if G.has(case, "out_bf16"):
        # the upstream backend evaluated in bf16 on the CPU (its own rounding included)
        assert_parity(out.float(), G.get(case, "out_bf16"), what="out vs upstream bf16", max_abs_tol=3e-2, rel_l2_tol=2e-2)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("head_dim", [64, 96, 128])
@pytest.mark.parametrize("gqa", [1, 2, 3])
@pytest.mark.parametrize("documents", [False, True])
def test_ragged_tiles_groups_and_documents(documents, gqa, head_dim, backend):
    torch.manual_seed(23)
    q = torch.randn(2, 2 * gqa, 33, head_dim).bfloat16()
    k = torch.randn(2, 2, 132, head_dim).bfloat16()
    v = torch.randn(2, 2, 132, head_dim).bfloat16()
    probe = torch.randn(2, 2 * gqa, 33, head_dim).bfloat16()
    metadata = None
    if documents:
        seg = torch.stack((torch.arange(132) // 19, torch.arange(132) // 31))
        metadata = prepare_cyclic_attention_metadata(seg[:, 1::4], torch.cat((seg.new_full((2, 1), -1), seg[:, :-1]), 1))
    c = dict(stride=4, offset=1, strict_past=False)
    out, grads = run(q, k, v, probe, metadata, c, torch.bfloat16, backend)
    qo, ko, vo = (t.double().requires_grad_() for t in (q, k, v))
    exp = oracle.cyclic_attention_oracle(qo, ko, vo, query_stride=4, query_offset=1, metadata=metadata)
    exp_grads = torch.autograd.grad(exp, (qo, ko, vo), probe.double())
    assert_parity(out.float(), exp, what="out", **BF16_TOL)
    for g, e, name in zip(grads, exp_grads, ("dq", "dk", "dv")):
        assert_parity(g.float(), e, what=name, **BF16_TOL)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("stride", [1, 4])
@pytest.mark.parametrize("packed", [False, True])
def test_strict_past_all_residues(packed, stride, backend):
    torch.manual_seed(5)
    T, B, H, D = 137, 2, 2, 64
    k = torch.randn(B, H, T, D).bfloat16()
    v = torch.randn(B, H, T, D).bfloat16()
    docs = geometric_documents(B, T, 40, seed=3)
    groups = [torch.arange(r, T, stride) for r in range(stride)]
    metas = prepare_feedback_metadata(docs, groups, T, use_dummy_token=False) if packed else [None] * stride
    for r in range(stride):
        n = groups[r].numel()
        q = torch.randn(B, H, n, D).bfloat16()
        probe = torch.randn(B, H, n, D).bfloat16()
        c = dict(stride=stride, offset=r, strict_past=True)
        out, grads = run(q, k, v, probe, metas[r], c, torch.bfloat16, backend)
        qo, ko, vo = (t.double().requires_grad_() for t in (q, k, v))
        exp = oracle.cyclic_attention_oracle(qo, ko, vo, query_stride=stride, query_offset=r, strict_past=True, metadata=metas[r])
        exp_grads = torch.autograd.grad(exp, (qo, ko, vo), probe.double())
        assert_parity(out.float(), exp, what=f"out r={r}", **BF16_TOL)
        for g, e, name in zip(grads, exp_grads, ("dq", "dk", "dv")):
            assert_parity(g.float(), e, what=f"{name} r={r}", **BF16_TOL)
        if r == 0:
            assert out[:, :, 0].abs().max().item() == 0  # the first token of the row sees nothing


@pytest.mark.parametrize("mean", [6, 48, 300])
@pytest.mark.parametrize("dummy", [False, True])
def test_document_masks_by_runs_and_by_rows(dummy, mean):
    # the tcgen05 kernels build a key tile's document masks from its runs of equal (document, query bound) when the
    # tile has at most 8 of them and row by row otherwise: documents of mean length 6 put ~20 runs in every 128-key
    # tile, mean 48 mixes both ways, mean 300 stays with the runs
    torch.manual_seed(17)
    T, B, H, D, stride = 640, 2, 2, 64, 2
    lead = int(dummy)
    k = torch.randn(B, H, T + lead, D).bfloat16()
    v = torch.randn(B, H, T + lead, D).bfloat16()
    docs = geometric_documents(B, T, mean, seed=mean)
    groups = [torch.arange(r, T, stride) for r in range(stride)]
    metas = prepare_feedback_metadata(docs, groups, T + lead, use_dummy_token=dummy)
    for r in range(stride):
        n = groups[r].numel()
        q = torch.randn(B, H, n, D).bfloat16()
        probe = torch.randn(B, H, n, D).bfloat16()
        c = dict(stride=stride, offset=r, strict_past=not dummy)
        out, grads = run(q, k, v, probe, metas[r], c, torch.bfloat16, "sm100_tcgen05")
        qo, ko, vo = (t.double().requires_grad_() for t in (q, k, v))
        exp = oracle.cyclic_attention_oracle(qo, ko, vo, query_stride=stride, query_offset=r, strict_past=not dummy, metadata=metas[r])
        exp_grads = torch.autograd.grad(exp, (qo, ko, vo), probe.double())
        assert_parity(out.float(), exp, what=f"out r={r}", **BF16_TOL)
        for g, e, name in zip(grads, exp_grads, ("dq", "dk", "dv")):
            assert_parity(g.float(), e, what=f"{name} r={r}", **BF16_TOL)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("documents", [False, True])
def test_equal_scores_average_exactly_to_zero(documents, backend):
    # upstream tests/gpu/test_cyclic_attention.py:61-76: rescaling by anything but one biases earlier tiles
    q = torch.full((1, 2, 1, 128), 13.0, device="cuda", dtype=torch.bfloat16)
    k = torch.full((1, 1, 4096, 128), 29.0, device="cuda", dtype=torch.bfloat16)
    v = torch.ones_like(k)
    v[:, :, 2048:].neg_()
    metadata = None
    if documents:
        kseg = torch.zeros((1, 4096), device="cuda", dtype=torch.long)
        kseg[:, 0] = -1
        metadata = prepare_cyclic_attention_metadata(torch.zeros((1, 1), device="cuda", dtype=torch.long), kseg)
    out = cyclic_attention(q, k, v, query_stride=4096, query_offset=4095, metadata=metadata, backend=backend)
    assert out.abs().max().item() == 0


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("documents", [False, True])
def test_invisible_keys_get_exactly_zero_gradient(documents, backend):
    # upstream tests/gpu/test_cyclic_attention.py:134-157
    torch.manual_seed(127)
    q = torch.randn(1, 4, 1, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(1, 2, 513, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn_like(k, requires_grad=True)
    metadata = None
    if documents:
        kseg = torch.zeros((1, 513), device="cuda", dtype=torch.int32)
        kseg[:, 0] = -1
        metadata = prepare_cyclic_attention_metadata(torch.zeros((1, 1), device="cuda", dtype=torch.int32), kseg)
    out = cyclic_attention(q, k, v, query_stride=4, query_offset=0, metadata=metadata, backend=backend)
    grads = torch.autograd.grad(out, (q, k, v), torch.randn_like(out))
    for g in grads[1:]:
        assert g[:, :, 1:].abs().max().item() == 0
    # the single visible key takes all the weight: dV there is the upstream gradient, dK is exactly zero
    assert grads[2][:, :, :1].abs().max().item() > 0


@pytest.mark.parametrize("backend", BACKENDS)
def test_strided_cache_views_are_bitwise_equal_to_contiguous(backend):
    # upstream tests/gpu/test_cyclic_attention.py:79-96: batch slice, channel selection, unused capacity
    torch.manual_seed(29)
    q = torch.randn(2, 4, 33, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    storage = [torch.randn(4, 3, 2, 145, 128, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    k, v = [t[1:3, 1, :, :132].detach().requires_grad_() for t in storage]
    assert not k.is_contiguous()
    kc, vc = [t.detach().contiguous().requires_grad_() for t in (k, v)]
    opts = dict(query_stride=4, query_offset=1, backend=backend)
    a = cyclic_attention(q, k, v, **opts)
    b = cyclic_attention(q, kc, vc, **opts)
    probe = torch.randn_like(a)
    ga = torch.autograd.grad(a, (q, k, v), probe)
    gb = torch.autograd.grad(b, (q, kc, vc), probe)
    assert torch.equal(a, b)
    for x, y in zip(ga, gb):
        assert torch.equal(x, y)


@pytest.mark.parametrize("backend", BACKENDS)
def test_deterministic(backend):
    torch.manual_seed(1)
    q = torch.randn(2, 4, 65, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(2, 4, 260, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn_like(k, requires_grad=True)
    probe = torch.randn_like(q)
    runs = []
    for _ in range(2):
        out = cyclic_attention(q, k, v, query_stride=4, backend=backend)
        runs.append((out, *torch.autograd.grad(out, (q, k, v), probe)))
    for x, y in zip(*runs):
        assert torch.equal(x, y)


@pytest.mark.parametrize("backend", ["sm100"])
def test_training_shape_properties_at_full_size(backend):
    """B=16,H=16,K=2048,D=64, stride 8 with packed documents: too large for the CPU oracle.

    Checked through properties that do not depend on the size: the SIMT and the
    selected kernel agree, every document's first token is exactly zero, and
    the result is linear in V.
    """
    torch.manual_seed(0)
    B, H, T, D, S = 16, 16, 2048, 64, 8
    docs = geometric_documents(B, T, 1024, seed=7).cuda()
    groups = [torch.arange(r, T, S, device="cuda") for r in range(S)]
    metas = prepare_feedback_metadata(docs, groups, T, use_dummy_token=False)
    k = torch.randn(B, H, T, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(B, H, T, D, device="cuda", dtype=torch.bfloat16)
    r = 3
    q = torch.randn(B, H, T // S, D, device="cuda", dtype=torch.bfloat16)
    opts = dict(query_stride=S, query_offset=r, strict_past=True, metadata=metas[r])
    out = cyclic_attention(q, k, v, backend=backend, **opts)
    ref = cyclic_attention(q, k, v, backend="sm100_simt", **opts)
    assert_parity(out.float(), ref.float(), what="kernel families", **BF16_TOL)
    starts = torch.ones_like(docs, dtype=torch.bool)
    starts[:, 1:] = docs[:, 1:] != docs[:, :-1]
    first_rows = starts[:, r::S]
    assert out.transpose(1, 2)[first_rows].abs().max().item() == 0
    out2 = cyclic_attention(q, k, 2 * v, backend=backend, **opts)
    assert_parity(out2.float(), 2 * out.float(), what="linearity in V", max_abs_tol=4e-2, rel_l2_tol=1e-2)


@pytest.mark.parametrize("backend", BACKENDS)
@pytest.mark.parametrize("boost", [6.0, 40.0, 400.0])
def test_scores_that_outgrow_the_running_reference(boost, backend):
    """Later key tiles whose scores exceed everything seen before by a little, a lot, and by far more than fp32
    exponentials can hold: the soft-max reference has to follow (deferred rescale, and the re-exponentiation of a
    tile that outgrew its reference by more than 2^64)."""
    torch.manual_seed(5)
    T, S = 1024, 2
    q = torch.randn(1, 2, T // S, 64)
    k = torch.randn(1, 2, T, 64)
    v = torch.randn(1, 2, T, 64)
    # a few keys in the 4th, 6th and 7th key tile point along the mean query direction with a growing norm
    direction = q[0, 0].mean(0) / q[0, 0].mean(0).norm()
    q = q + 2.0 * direction
    for slot, gain in ((400, boost), (700, 2 * boost), (801, 4 * boost)):
        k[:, :, slot] = gain * direction
    q, k, v = (t.bfloat16() for t in (q, k, v))
    probe = torch.randn(1, 2, T // S, 64).bfloat16()
    c = dict(stride=S, offset=0, strict_past=False)
    out, grads = run(q, k, v, probe, None, c, torch.bfloat16, backend)
    qo, ko, vo = (t.double().requires_grad_() for t in (q, k, v))
    exp = oracle.cyclic_attention_oracle(qo, ko, vo, query_stride=S, query_offset=0)
    exp_grads = torch.autograd.grad(exp, (qo, ko, vo), probe.double())
    assert_parity(out.float(), exp, what="out", **BF16_TOL)
    # The gradients multiply bf16-rounded P and dS by keys whose norm is up to 4*boost, which amplifies the
    # rounding of any bf16 tensor-core backward: the usual bound is asked for the moderate case only, the extreme
    # ones must stay finite and keep the direction of the exact gradient.
    for g, e, name in zip(grads, exp_grads, ("dq", "dk", "dv")):
        if boost <= 6.0:
            assert_parity(g.float(), e, what=name, **BF16_TOL)
        else:
            assert torch.isfinite(g).all(), name
            cos = torch.nn.functional.cosine_similarity(g.double().flatten().cpu(), e.flatten(), dim=0).item()
            assert cos > 0.995, f"{name}: cosine {cos}"


@pytest.mark.parametrize("level", [-60.0, -90.0, -150.0, 120.0])
def test_scores_far_from_zero_everywhere(level):
    """All scores of a row near a large negative (or positive) level: the weights formed against the provisional
    zero reference of a row's first tile would be tiny, subnormal or zero (or overflow); the result must not care."""
    torch.manual_seed(11)
    T, S, D = 512, 2, 64
    u = torch.nn.functional.normalize(torch.randn(D), dim=0)
    c = (abs(level) * D ** 0.5) ** 0.5
    q = 0.3 * torch.randn(1, 2, T // S, D) + c * u
    k = 0.3 * torch.randn(1, 2, T, D) + (c if level > 0 else -c) * u
    v = torch.randn(1, 2, T, D)
    q, k, v = (t.bfloat16() for t in (q, k, v))
    from white_matter_b200 import _native

    with torch.no_grad():
        out = cyclic_attention(q.cuda(), k.cuda(), v.cuda(), query_stride=S, query_offset=0, backend="sm100_tcgen05")
    assert _native.device_status(True) == 0
    exp = oracle.cyclic_attention_oracle(q.double(), k.double(), v.double(), query_stride=S, query_offset=0)
    assert_parity(out.float(), exp, what=f"out at level {level}", **BF16_TOL)


def test_many_launches_leave_the_status_word_clean():
    """The pipelined kernels synchronise their roles through parity barriers with bounded waits: a protocol slip
    shows as a wait that gives up (status word != 0), typically once in hundreds of launches.  Several hundred
    forward and backward launches over the shapes that exercise the different walks must leave the word clean."""
    from white_matter_b200 import _native

    _native.device_status(True)
    torch.manual_seed(3)
    shapes = [  # batch, heads, keys, stride, documents
        (16, 16, 2048, 8, True), (16, 16, 2048, 8, False), (4, 8, 1024, 4, True), (2, 4, 260, 4, False), (2, 4, 4096, 1, False),
    ]
    for batch, heads, keys, stride, documents in shapes:
        q = torch.randn(batch, heads, keys // stride, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        k = torch.randn(batch, heads, keys, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        v = torch.randn_like(k, requires_grad=True)
        probe = torch.randn_like(q)
        metas = [None] * stride
        if documents:
            docs = geometric_documents(batch, keys, keys // 2, seed=11)
            groups = [torch.arange(r, keys, stride) for r in range(stride)]
            metas = [tuple(t.cuda() for t in m) for m in prepare_feedback_metadata(docs, groups, keys, use_dummy_token=False)]
        for launch in range(60):
            r = launch % stride
            out = cyclic_attention(q, k, v, query_stride=stride, query_offset=r, strict_past=True, metadata=metas[r], backend="sm100")
            torch.autograd.grad(out, (q, k, v), probe)
        status = _native.device_status(True)
        assert status == 0, f"shape {(batch, heads, keys, stride, documents)}: wait {status & 255} gave up in block {status >> 8}"


def test_first_cuda_action_of_a_thread_may_be_the_backward_call():
    # In a fresh process the autograd worker thread has made no CUDA call of its own when the backward operator
    # reaches the library: the tensor-map encoder (a driver entry point) then finds no context bound to the thread
    # and the library has to bind the primary one itself.
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    code = (
        "import torch\n"
        "from white_matter_b200 import cyclic_attention\n"
        "q = torch.randn(1, 2, 64, 64, device='cuda', dtype=torch.bfloat16, requires_grad=True)\n"
        "k = torch.randn(1, 2, 256, 64, device='cuda', dtype=torch.bfloat16, requires_grad=True)\n"
        "v = torch.randn(1, 2, 256, 64, device='cuda', dtype=torch.bfloat16, requires_grad=True)\n"
        "out = cyclic_attention(q, k, v, query_stride=4, query_offset=1, backend='sm100_tcgen05')\n"
        "g = torch.autograd.grad(out, (q, k, v), torch.ones_like(out))\n"
        "torch.cuda.synchronize()\n"
        "assert all(torch.isfinite(t.float()).all() for t in g)\n"
        "print('ok')\n"
    )
    done = subprocess.run([sys.executable, "-c", code], cwd=root, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0 and "ok" in done.stdout, done.stderr[-2000:]


@pytest.mark.expects_wait_timeout
def test_a_wait_that_runs_out_is_reported_and_the_next_launch_is_clean():
    """Every mbarrier wait of the pipelined kernels is bounded.  A one-block kernel of the library waits, with the
    limit shortened to a millisecond, on a barrier that nothing arrives on: the wait has to give up, leave its code
    in the status word and return normally (no trap, no fault), and the launches after it must be unaffected."""
    import ctypes

    from white_matter_b200 import _native

    lib = _native.load_library()
    lib.wm_debug_expire_wait.argtypes = [ctypes.c_longlong, ctypes.c_void_p]
    lib.wm_debug_expire_wait.restype = ctypes.c_int
    assert _native.device_status(True) == 0
    assert lib.wm_debug_expire_wait(2_000_000, torch.cuda.current_stream().cuda_stream) == 0
    status = _native.device_status(True)  # synchronises, reads and clears
    assert status & 255 == 250 and status >> 8 == 0
    assert _native.device_status(False) == 0
    # limits outside (0, the production limit] are refused before any launch
    assert lib.wm_debug_expire_wait(0, None) != 0
    torch.manual_seed(9)
    q = torch.randn(2, 4, 65, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(2, 4, 260, 64, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn_like(k, requires_grad=True)
    out = cyclic_attention(q, k, v, query_stride=4, backend="sm100_tcgen05")
    grads = torch.autograd.grad(out, (q, k, v), torch.randn_like(out))
    assert _native.device_status(True) == 0
    exp = oracle.cyclic_attention_oracle(q.detach().cpu().double(), k.detach().cpu().double(), v.detach().cpu().double(), query_stride=4)
    assert_parity(out.float(), exp, what="out after an expired wait", **BF16_TOL)
    assert all(torch.isfinite(g).all() for g in grads)
