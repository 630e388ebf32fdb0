"""Benchmark of the WhiteMatter attention hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload (N=1 and per rank for N>1, weak scaling): the training configuration
of cyclic attention -- bf16, B=16, H=16, key length 2048 (256 queries per
residue), head_dim 64, query_stride 8, packed documents with geometric lengths
of mean 1024, no dummy token (strict past).  One step is one sweep over the 8
residues, forward and backward, 16 operator calls.  Inputs are synthetic
(seeded N(0,1)); K+V alone are 134 MB per sweep, larger than the 126 MB L2.

The headline ``value`` is TFLOP/s on the visible (query,key) pairs only,
14*head_dim FLOP per pair (4 forward, 10 backward), with inputs resident in
HBM, the 16 operator calls of a step stream-ordered one after another (in the
model the residue groups depend on one another: K/V are refreshed after each
group), replayed from a CUDA graph.  ``multi_stream`` is a labelled extra: the
same calls spread over 8 streams, which a caller whose calls are independent
may do.  ``eager`` is the same step without the graph (host-bound).
``--scaling strong`` splits the B=16 rows over the ranks instead of giving
every rank its own 16.  ``e2e`` is the same metric through the public functions with every step's
inputs copied in from pinned host buffers and every step's results copied back
inside the timed region; the copies run on their own streams beside the kernels
of the neighbouring steps (``e2e.serialized`` is the same work on one stream).  The same line also reports the
pool-read (decode) bandwidth, the cached-prefix prefill over the same pool,
the Jacobi prefill and the source-mixing bandwidth, each with its roofline
fraction, and the CPU oracle timed on a bounded sample.
"""

from __future__ import annotations

import argparse
import ctypes
import datetime
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

B, H, T, D, STRIDE = 16, 16, 2048, 64, 8
DOC_MEAN = 1024
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernels on exactly these
# workloads, from the ncu captures summarised under profiles/ (one capture each; the bench cannot run ncu itself).
NCU_TRAFFIC_BYTES = {
    "attn_bwd_resident_kernel": 255.0e6,
    "attn_fwd_tc_kernel": 178.2e6,
    "decode_split_kernel": 1083.7e6,
    # captured on 4 of the 16 batch rows (1 053.8 MB for 1 050.6 MB of visible source rows) and scaled by the visible
    # rows of the full launch, which is how this kernel's traffic grows
    "decode_split_kernel_mixed": 8205.5e6 * 1053.8 / 1050.6,
    "mix_fwd_kernel": 1730.0e6,
    "query_prepare_fwd_bf16_kernel": 225.1e6,
    "pool_mix_mma_kernel": 1335.9e6,
    "pool_finish_kernel": 1014.4e6,
}


def load_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return json.loads(path.read_text()), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def geometric_documents(batch, length, mean, seed):
    """(batch, length) document ids with geometric lengths (support >= 1) truncated to fill each row exactly."""
    gen = torch.Generator().manual_seed(seed)
    dist_p = 1.0 / mean
    rows = []
    for _ in range(batch):
        ids, at, doc = torch.empty(length, dtype=torch.long), 0, 0
        while at < length:
            u = torch.rand((), generator=gen).item()
            n = max(1, int(torch.ceil(torch.log(torch.tensor(max(1.0 - u, 1e-12))) / torch.log(torch.tensor(1.0 - dist_p))).item()))
            n = min(n, length - at)
            ids[at : at + n] = doc
            at += n
            doc += 1
        rows.append(ids)
    return torch.stack(rows)


def visible_pairs_per_head(docs, residue, stride):
    """Visible (query,key) pairs of one residue, summed over the batch rows (strict past, same document)."""
    total = 0
    for row in docs.tolist():
        start = 0
        for t in range(len(row)):
            if t and row[t] != row[t - 1]:
                start = t
            if t % stride == residue:
                total += t - start
    return total


class ClockSampler:
    """nvidia-smi queried every 25 ms in a child process.  Samples carry nvidia-smi's own timestamp; ``stop`` keeps
    those between ``mark_load`` (the same work starts running, untimed) and the end of the timed region, and says
    how many of them fell inside the timed region itself (a default run times 20 steps, about 40 ms)."""

    QUERY = (
        "timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
        "clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.load_from = self.timed_from = self.timed_to = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "25", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
        except OSError:
            self.proc = None

    def mark_load(self):
        self.load_from = datetime.datetime.now()

    def mark_timed(self, begin):
        if begin:
            self.timed_from = datetime.datetime.now()
        else:
            self.timed_to = datetime.datetime.now()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            text, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            text, _ = self.proc.communicate()
        clocks, top, reasons, timed = [], None, set(), 0
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in text.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                stamp = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f")
                clock, top_now = float(parts[1]), float(parts[2])
            except ValueError:
                continue
            if self.load_from is not None and not (self.load_from <= stamp <= (self.timed_to or stamp)):
                continue
            clocks.append(clock)
            top = top_now
            timed += int(self.timed_from is not None and self.timed_from <= stamp <= (self.timed_to or stamp))
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": top,
            "reasons": sorted(reasons),
            "samples": len(clocks),
            "samples_in_timed_region": timed,
            "window": "the same steps run untimed for 0.4 s before the warm-up; samples from there to the end of the timed region",
        }


# --------------------------------------------------------------------------- workload


class TrainingSweep:
    """Device-resident inputs of one 8-residue sweep and the calls of one step."""

    def __init__(self, device, seed, backend="sm100", rows=slice(0, B)):
        from white_matter_b200 import cyclic_attention, prepare_feedback_metadata

        self.attention = cyclic_attention
        self.backend = backend
        self.device = device
        self.docs = geometric_documents(B, T, DOC_MEAN, seed=7 + seed)[rows]
        self.batch = self.docs.shape[0]
        groups = [torch.arange(r, T, STRIDE) for r in range(STRIDE)]
        metas = prepare_feedback_metadata(self.docs, groups, T, use_dummy_token=False)
        self.metas = [tuple(t.to(device) for t in m) for m in metas]
        gen = torch.Generator().manual_seed(seed)
        shape_q, shape_k = (self.batch, H, T // STRIDE, D), (self.batch, H, T, D)
        # pinned host copies feed the end-to-end arm; the device copies feed the kernel arm
        self.host = {
            "q": [torch.randn(shape_q, generator=gen).bfloat16().pin_memory() for _ in range(STRIDE)],
            "g": [torch.randn(shape_q, generator=gen).bfloat16().pin_memory() for _ in range(STRIDE)],
            "k": torch.randn(shape_k, generator=gen).bfloat16().pin_memory(),
            "v": torch.randn(shape_k, generator=gen).bfloat16().pin_memory(),
        }
        self.q = [t.to(device).requires_grad_() for t in self.host["q"]]
        self.g = [t.to(device) for t in self.host["g"]]
        self.k = self.host["k"].to(device).requires_grad_()
        self.v = self.host["v"].to(device).requires_grad_()
        self.pairs = sum(visible_pairs_per_head(self.docs, r, STRIDE) for r in range(STRIDE)) * H
        self.flops_fwd = 4 * D * self.pairs
        self.flops = 14 * D * self.pairs

    def forward(self, r, q=None, k=None, v=None):
        return self.attention(
            self.q[r] if q is None else q, self.k if k is None else k, self.v if v is None else v,
            query_stride=STRIDE, query_offset=r, strict_past=True, metadata=self.metas[r], backend=self.backend,
        )

    def step(self, streams=None):
        """All 8 residues forward and backward; returns nothing, gradients are discarded.

        The residue calls do not depend on one another.  With `streams` they are issued round-robin on those
        streams (forked from and joined to the current one), so that the blocks of one call fill the SMs the last,
        partial wave of another leaves idle: 256 blocks of one backward call are 1.7 waves on 148 SMs."""
        if not streams:
            for r in range(STRIDE):
                out = self.forward(r)
                torch.autograd.grad(out, (self.q[r], self.k, self.v), self.g[r])
            return
        main = torch.cuda.current_stream()
        for stream in streams:
            stream.wait_stream(main)
        for r in range(STRIDE):
            with torch.cuda.stream(streams[r % len(streams)]):
                out = self.forward(r)
                torch.autograd.grad(out, (self.q[r], self.k, self.v), self.g[r])
        for stream in streams:
            main.wait_stream(stream)

    def _capture(self, streams):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.step(streams)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.step(streams)
        return graph

    def capture(self, n_streams=1):
        """Capture one step in a CUDA graph (the 16 operator calls are launch-bound when issued eagerly).

        Returns the number of kernels of this library inside the graph."""
        from white_matter_b200 import _native

        lib = _native.load_library()
        before = lib.wm_kernel_launch_count()
        self.graph_one_stream = self._capture(None)
        per_step = (lib.wm_kernel_launch_count() - before) // 2  # the dry run and the captured one
        self.graph = self.graph_one_stream
        if n_streams > 1:
            self.streams = [torch.cuda.Stream() for _ in range(n_streams)]
            self.graph = self._capture(self.streams)
        return per_step

    def replay(self):
        self.graph.replay()

    def one_stream_ms(self, reps=10):
        """Device time (ms) of one step with the 24 launches one after another (the per-kernel figures)."""
        self.graph_one_stream.replay()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(reps):
            self.graph_one_stream.replay()
        end.record()
        torch.cuda.synchronize()
        return begin.elapsed_time(end) / reps

    def forward_only_ms(self, reps=10):
        """Device time (ms) of the 8 forward launches of one step, from a CUDA graph replayed `reps` times."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for r in range(STRIDE):
                self.forward(r)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph), torch.no_grad():
            for r in range(STRIDE):
                self.forward(r)
        graph.replay()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(reps):
            graph.replay()
        end.record()
        torch.cuda.synchronize()
        return begin.elapsed_time(end) / reps

    def step_e2e(self, staging):
        """One step from pinned host buffers to pinned host results."""
        k = staging["k"].copy_(self.host["k"], non_blocking=True).detach().requires_grad_()
        v = staging["v"].copy_(self.host["v"], non_blocking=True).detach().requires_grad_()
        dk_sum = dv_sum = None
        for r in range(STRIDE):
            q = staging["q"][r].copy_(self.host["q"][r], non_blocking=True).detach().requires_grad_()
            g = staging["g"][r].copy_(self.host["g"][r], non_blocking=True)
            out = self.forward(r, q, k, v)
            dq, dk, dv = torch.autograd.grad(out, (q, k, v), g)
            staging["out_host"][r].copy_(out.detach().transpose(1, 2), non_blocking=True)
            staging["dq_host"][r].copy_(dq, non_blocking=True)
            dk_sum = dk if dk_sum is None else dk_sum.add_(dk)
            dv_sum = dv if dv_sum is None else dv_sum.add_(dv)
        staging["dk_host"].copy_(dk_sum, non_blocking=True)
        staging["dv_host"].copy_(dv_sum, non_blocking=True)

    def e2e_pipelined_ms(self, steps, warmup=2):
        """Device time (ms) of `steps` end-to-end steps with the copies on their own streams.

        Every step still copies all of its inputs from pinned host memory and all of its results back, inside the
        timed region; the host-to-device copy of step i+1 and the device-to-host copy of step i-1 run beside the
        kernels of step i (two sets of device staging buffers).  PCIe is full duplex, so the steady state is bound
        by the larger of the two copy directions instead of their sum plus the compute.
        """
        main = torch.cuda.current_stream()
        h2d, d2h = torch.cuda.Stream(), torch.cuda.Stream()
        slots = [self.staging() for _ in range(2)]
        for slot in slots:
            slot["consumed"] = torch.cuda.Event()
            slot["loaded"] = torch.cuda.Event()
            slot["computed"] = torch.cuda.Event()
            slot["consumed"].record(main)
        host = slots[0]  # one set of pinned result buffers: the device-to-host stream is sequential

        def run(n):
            for i in range(n):
                slot = slots[i % 2]
                with torch.cuda.stream(h2d):
                    h2d.wait_event(slot["consumed"])  # the kernels that read this slot two steps ago are done
                    slot["k"].copy_(self.host["k"], non_blocking=True)
                    slot["v"].copy_(self.host["v"], non_blocking=True)
                    for r in range(STRIDE):
                        slot["q"][r].copy_(self.host["q"][r], non_blocking=True)
                        slot["g"][r].copy_(self.host["g"][r], non_blocking=True)
                    slot["loaded"].record(h2d)
                main.wait_event(slot["loaded"])
                k = slot["k"].detach().requires_grad_()
                v = slot["v"].detach().requires_grad_()
                results, dk_sum, dv_sum = [], None, None
                for r in range(STRIDE):
                    q = slot["q"][r].detach().requires_grad_()
                    out = self.forward(r, q, k, v)
                    dq, dk, dv = torch.autograd.grad(out, (q, k, v), slot["g"][r])
                    results.append((out.detach(), dq))
                    dk_sum = dk if dk_sum is None else dk_sum.add_(dk)
                    dv_sum = dv if dv_sum is None else dv_sum.add_(dv)
                slot["consumed"].record(main)
                slot["computed"].record(main)
                with torch.cuda.stream(d2h):
                    d2h.wait_event(slot["computed"])
                    for r, (out, dq) in enumerate(results):
                        host["out_host"][r].copy_(out.transpose(1, 2), non_blocking=True)
                        host["dq_host"][r].copy_(dq, non_blocking=True)
                        out.record_stream(d2h)
                        dq.record_stream(d2h)
                    host["dk_host"].copy_(dk_sum, non_blocking=True)
                    host["dv_host"].copy_(dv_sum, non_blocking=True)
                    dk_sum.record_stream(d2h)
                    dv_sum.record_stream(d2h)
            main.wait_stream(d2h)
            main.wait_stream(h2d)

        run(warmup)
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record(main)
        run(steps)
        end.record(main)
        torch.cuda.synchronize()
        return begin.elapsed_time(end)

    def staging_bytes(self):
        q_bytes = self.batch * H * (T // STRIDE) * D * 2
        k_bytes = self.batch * H * T * D * 2
        return 2 * STRIDE * q_bytes + 2 * k_bytes, 2 * STRIDE * q_bytes + 2 * k_bytes

    def call_bytes(self):
        """Algorithmic HBM bytes of one residue call: forward reads Q, K, V and writes O and the row statistics;
        backward reads Q, K, V, O, dO and the statistics and writes dQ, dK, dV."""
        q_bytes = self.batch * H * (T // STRIDE) * D * 2
        k_bytes = self.batch * H * T * D * 2
        stat = self.batch * H * (T // STRIDE) * 4
        return 2 * q_bytes + 2 * k_bytes + stat, 4 * q_bytes + 4 * k_bytes + 2 * stat

    def staging(self):
        dev = self.device
        shape_q, shape_k = (self.batch, H, T // STRIDE, D), (self.batch, H, T, D)
        mk = lambda s: torch.empty(s, dtype=torch.bfloat16, device=dev)
        pin = lambda s: torch.empty(s, dtype=torch.bfloat16).pin_memory()
        s = {
            "q": [mk(shape_q) for _ in range(STRIDE)], "g": [mk(shape_q) for _ in range(STRIDE)],
            "k": mk(shape_k), "v": mk(shape_k),
            "out_host": [pin((self.batch, T // STRIDE, H, D)) for _ in range(STRIDE)],
            "dq_host": [pin(shape_q) for _ in range(STRIDE)],
            "dk_host": pin(shape_k), "dv_host": pin(shape_k),
        }
        s["h2d"], s["d2h"] = self.staging_bytes()
        return s


def time_steps(fn, steps, warmup, sync):
    """Device time of exactly ``steps`` calls of fn (ms), events on the current stream, barriers both sides."""
    for _ in range(warmup):
        fn()
    sync()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(steps):
        fn()
    end.record()
    sync()
    return begin.elapsed_time(end)


# --------------------------------------------------------------------------- secondary workloads


def bench_decode(device, peaks, iters=20):
    """Pool read: B=64, H=16, D=64, 8192 slots, lengths uniform in [1,8192]; GB/s over the visible K/V bytes."""
    from white_matter_b200 import strict_causal_attention

    gen = torch.Generator().manual_seed(0)
    batch, heads, slots, dim = 64, 16, 8192, 64
    lengths = torch.randint(1, slots + 1, (batch,), generator=gen).to(device)
    k = torch.randn(batch, heads, slots, dim, device=device, dtype=torch.bfloat16)
    v = torch.randn(batch, heads, slots, dim, device=device, dtype=torch.bfloat16)
    q = torch.randn(batch, heads, 1, dim, device=device, dtype=torch.bfloat16)
    call = lambda: strict_causal_attention(q, k, v, query_start=lengths, kv_lengths=lengths)
    ms = time_steps(call, iters, 3, torch.cuda.synchronize) / iters
    nbytes = int(lengths.sum().item()) * 2 * heads * dim * 2
    gbs = nbytes / (ms * 1e-3) / 1e9
    result = {
        "workload": "strict decode B=64 H=16 D=64 lengths~U[1,8192] bf16 (pool 2.15 GB > L2)",
        "ms": ms, "bytes": nbytes, "value": gbs, "unit": "GB/s",
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES["decode_split_kernel"]},
    }
    # cached-prefix prefill over the same pool: 128 new tokens per sequence, query_start = kv_length - 128 (>= 0)
    q128 = torch.randn(batch, heads, 128, dim, device=device, dtype=torch.bfloat16)
    starts = (lengths - 128).clamp_min(0)
    call = lambda: strict_causal_attention(q128, k, v, query_start=starts, kv_lengths=lengths)
    ms128 = time_steps(call, iters, 3, torch.cuda.synchronize) / iters
    pos = starts.cpu()[:, None] + torch.arange(128)[None, :]
    pairs = int(torch.minimum(pos, lengths.cpu()[:, None]).sum().item()) * heads
    gbs128 = nbytes / (ms128 * 1e-3) / 1e9
    prefill = {
        "workload": "strict cached-prefix prefill: 128 new tokens per sequence over the same pool",
        "ms": ms128, "bytes": nbytes, "value": gbs128, "unit": "GB/s", "tflops": 4 * dim * pairs / (ms128 * 1e-3) / 1e12,
        "roofline": {"bound": "hbm", "achieved": gbs128, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs128 / peaks["hbm_gbs"], "traffic": None},
    }
    # the same prefill with a document key mask (70 % of the slots kept): tensor-core forward against the SIMT family
    key_mask = torch.rand(batch, slots, device=device) < 0.7
    with torch.no_grad():
        masked = {}
        for name, backend in (("tcgen05", "sm100"), ("simt", "sm100_simt")):
            call = lambda: strict_causal_attention(q128, k, v, query_start=starts, kv_lengths=lengths, key_mask=key_mask, backend=backend)
            masked[name] = time_steps(call, max(3, iters // 4), 2, torch.cuda.synchronize) / max(3, iters // 4)
    prefill["with_key_mask"] = {
        "ms": masked["tcgen05"], "value": nbytes / (masked["tcgen05"] * 1e-3) / 1e9, "unit": "GB/s",
        "simt_ms": masked["simt"], "note": "K/V bytes as above (masked rows are loaded with their tile)",
    }
    return result, prefill


def bench_jacobi(device, peaks, iters=10):
    """Jacobi prefill: B=8, H=16, T=2048, D=64 bf16, packed documents (geometric, mean 512), schedule built once."""
    from white_matter_b200 import prepare_strict_causal_metadata, strict_causal_attention

    batch, heads, length, dim = 8, 16, 2048, 64
    docs = geometric_documents(batch, length, 512, seed=7)
    metadata = prepare_strict_causal_metadata(docs.to(device), length)
    gen = torch.Generator().manual_seed(100)
    mk = lambda scale: (torch.randn(batch, heads, length, dim, generator=gen) * scale).to(device, torch.bfloat16)
    q, k, v = mk(dim ** -0.5), mk(1.0), mk(1.0)
    call = lambda: strict_causal_attention(q, k, v, metadata=metadata)
    ms = time_steps(call, iters, 3, torch.cuda.synchronize) / iters
    pairs = 0
    for row in docs.tolist():
        run = 0
        for t in range(length):
            run = run + 1 if t and row[t] == row[t - 1] else 1
            pairs += run - 1  # strictly earlier tokens of the same document
    tf = 4 * dim * pairs * heads / (ms * 1e-3) / 1e12
    result = {
        "workload": "strict Jacobi prefill forward B=8 H=16 T=2048 D=64 bf16, packed documents (geometric, mean 512)",
        "ms": ms, "value": tf, "unit": "TFLOP/s",
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": tf / peaks["bf16_tflops"], "traffic": None, "peak_kind": "bf16_tflops (kernel timed alone)"},
    }
    # gradients of the same call (the key-stationary tensor-core backward: 2048 queries per row are more than the
    # resident backward keeps)
    leaves = [t.clone().requires_grad_() for t in (q, k, v)]
    out = strict_causal_attention(*leaves, metadata=metadata)
    probe = torch.randn_like(out)
    grad_call = lambda: torch.autograd.grad(out, leaves, probe, retain_graph=True)
    bwd_ms = time_steps(grad_call, iters, 3, torch.cuda.synchronize) / iters
    del out, leaves
    result["backward"] = {"ms": bwd_ms, "value": 10 * dim * pairs * heads / (bwd_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                          "kernels": "bwd_delta_kernel, attn_bwd_tc_kernel<64> (one block per key tile), bwd_dq_convert_kernel"}
    # cached-prefix Jacobi with documents: the last 512 tokens of 4096-token rows are the queries, the rest is
    # committed history; the schedule runs as dense per-row bounds plus document tables on the tensor-core kernel,
    # and as gathered index lists on the SIMT kernels
    rows, new = 4096, 512
    docs = geometric_documents(batch, rows, 512, seed=11)
    schedule = prepare_strict_causal_metadata(docs.to(device), new, query_start=rows - new)
    qn = (torch.randn(batch, heads, new, dim, generator=gen) * dim ** -0.5).to(device, torch.bfloat16)
    kn, vn = (torch.randn(batch, heads, rows, dim, generator=gen).to(device, torch.bfloat16) for _ in range(2))
    nq = (schedule.cu_queries[1:] - schedule.cu_queries[:-1]).cpu().long()
    nk = (schedule.cu_keys[1:] - schedule.cu_keys[:-1]).cpu().long()
    visible = int((nq * (nk - nq + 1) + nq * (nq - 1) // 2).sum().item())
    with torch.no_grad():
        timed = {}
        for name, backend in (("tcgen05", "sm100"), ("simt", "sm100_simt")):
            call = lambda: strict_causal_attention(qn, kn, vn, metadata=schedule, backend=backend)
            timed[name] = time_steps(call, max(3, iters // 2), 2, torch.cuda.synchronize) / max(3, iters // 2)
    result["cached_prefix_with_documents"] = {
        "workload": "Jacobi over the last 512 of 4096 tokens per row, B=8 H=16 D=64 bf16, documents of mean 512",
        "ms": timed["tcgen05"], "value": 4 * dim * visible * heads / (timed["tcgen05"] * 1e-3) / 1e12, "unit": "TFLOP/s",
        "simt_ms": timed["simt"],
    }
    return result


def bench_mixing(device, peaks, iters=10):
    """25-source mixture at the training configuration's size: sources (25, 16, 16, 2048, 64) bf16 = 1.68 GB, read once."""
    from white_matter_b200 import mix_kv_sources

    src = torch.empty(25, B, H, T, D, device=device, dtype=torch.bfloat16)
    for i in range(25):  # filled source by source: no fp32 temporary of the whole stack
        src[i].normal_()
    logits = torch.randn(25, device=device)
    call = lambda: mix_kv_sources(src, logits)
    ms = time_steps(call, iters, 3, torch.cuda.synchronize) / iters
    nbytes = src.numel() * 2 + src[0].numel() * 2
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {
        "workload": "mix 25 sources (25,16,16,2048,64) bf16, 1678 MB read + 67 MB written",
        "ms": ms, "bytes": nbytes, "value": gbs, "unit": "GB/s",
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES["mix_fwd_kernel"]},
    }


def bench_query_prepare(device, peaks, iters=20):
    """q_norm + rotary embedding + layout change of the query projection: B=32, T=2048, H=16, D=64 bf16 (134 MB in, 134 MB out: larger than L2)."""
    from white_matter_b200 import prepare_queries

    batch, tokens, heads, dim = 32, 2048, 16, 64
    x = torch.randn(batch, tokens, heads * dim, device=device, dtype=torch.bfloat16)
    weight = torch.ones(dim, device=device, dtype=torch.bfloat16)
    angles = torch.rand(1, tokens, dim, device=device) * 6.0
    cos, sin = angles.cos().bfloat16(), angles.sin().bfloat16()
    call = lambda: prepare_queries(x, weight, cos, sin)
    # a 40 us kernel: replayed from a CUDA graph so that the operator's host cost does not enter
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            call()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(iters):
            call()
    ms = time_steps(graph.replay, 3, 1, torch.cuda.synchronize) / (3 * iters)
    nbytes = 2 * x.numel() * 2 + 2 * cos.numel() * 2
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {
        "workload": "query preparation (rms_norm * gain, rotary embedding, BTHD -> BHTD) B=32 T=2048 H=16 D=64 bf16, 268 MB > L2",
        "ms": ms, "bytes": nbytes, "value": gbs, "unit": "GB/s",
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES["query_prepare_fwd_bf16_kernel"]},
    }


def bench_pool_projection(device, peaks, iters=5):
    """KV-pool projection of the 24-layer model's prefill: layer stack (8, 2048, 25, 1024) bf16 -> keys, values
    (8, 8, 16, 2048, 64), dynamic router over every second source (the upstream default) and static router.  The
    whole path (routing GEMM, mixing kernel, projection GEMMs, key norm + rotary + publication) is timed; the mixing
    and publication kernels are also timed alone, against their algorithmic bytes."""
    from white_matter_b200 import KVPool, _native

    batch, tokens, layers, hidden, channels, heads, dim = 8, 2048, 25, 1024, 8, 16, 64
    stacked = torch.empty(batch, tokens, layers, hidden, device=device, dtype=torch.bfloat16)
    for b in range(batch):
        stacked[b].normal_()
    angle = torch.rand(1, tokens, dim // 2, device=device) * 6.283
    tables = (torch.cat((angle.cos(), angle.cos()), -1), torch.cat((angle.sin(), angle.sin()), -1))
    rows = batch * tokens
    stack_bytes, pool_bytes = stacked.numel() * 2, 2 * rows * channels * heads * dim * 2
    mixed_bytes = 2 * channels * rows * hidden * 2
    out = {"workload": "KV-pool projection (8,2048,25,1024) bf16 -> K,V (8,8,16,2048,64); 839 MB stack read, 537 MB pool (K and V) written"}
    for name, dynamic in (("dynamic_router", True), ("static_router", False)):
        pool = KVPool(hidden, heads, dim, layers, channels, router_layer_stride=2, router_dynamic=dynamic, device=device)
        pool.k_router_weight.normal_(0, 0.004)
        pool.v_router_weight.normal_(0, 0.004)
        pool.k_router_bias.normal_()
        pool.v_router_bias.normal_()
        pool.refresh()
        call = lambda: pool.project_sequence(stacked, tables)
        ms = time_steps(call, iters, 3, torch.cuda.synchronize) / iters
        gbs = (stack_bytes + pool_bytes) / (ms * 1e-3) / 1e9
        out[name] = {"ms": ms, "bytes": stack_bytes + pool_bytes, "value": gbs, "unit": "GB/s",
                     "hbm_frac": gbs / peaks["hbm_gbs"], "note": "whole path; floor = stack read + pool write"}
    # the two kernels of this library alone (static router: no partials), through the C ABI
    mixed = torch.empty(2, channels, rows, hidden, device=device, dtype=torch.bfloat16)
    a = _native.PoolMixArgs()
    a.stacked, a.stacked_strides = stacked.data_ptr(), _native._Strides(stacked.stride(0), stacked.stride(1), stacked.stride(2))
    a.pre_mix_k, a.pre_mix_v = pool.pre_mix_k_weight.data_ptr(), pool.pre_mix_v_weight.data_ptr()
    a.bias_k, a.bias_v = pool.k_router_bias.data_ptr(), pool.v_router_bias.data_ptr()
    a.mixed_k, a.mixed_v = mixed[0].data_ptr(), mixed[1].data_ptr()
    a.dtype = _native.WM_BF16
    a.batch, a.tokens, a.sources, a.channels, a.hidden = batch, tokens, layers, channels, hidden
    a.source_eps, a.mix_eps = pool.rms_norm_eps, pool.mix_norm_eps
    mix_call = lambda: _native.call("wm_pool_mix", a, device)
    mix_ms = time_steps(mix_call, iters, 3, torch.cuda.synchronize) / iters
    mix_gbs = (stack_bytes + mixed_bytes) / (mix_ms * 1e-3) / 1e9
    out["mix_kernel"] = {"ms": mix_ms, "bytes": stack_bytes + mixed_bytes, "value": mix_gbs, "unit": "GB/s",
                         "roofline": {"bound": "hbm", "achieved": mix_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                      "frac": mix_gbs / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES.get("pool_mix_mma_kernel")}}
    del mixed
    proj = torch.randn(2, channels, rows, heads * dim, device=device, dtype=torch.bfloat16)
    keys = torch.empty(batch, channels * heads, tokens, dim, device=device, dtype=torch.bfloat16)
    values = torch.empty_like(keys)
    f = _native.PoolFinishArgs()
    f.k_proj, f.v_proj = proj[0].data_ptr(), proj[1].data_ptr()
    f.k_norm_weight = pool.k_norm_weight.data_ptr()
    f.cos, f.sin = tables[0].data_ptr(), tables[1].data_ptr()
    f.k_out, f.v_out = keys.data_ptr(), values.data_ptr()
    f.cs_strides = (ctypes.c_int64 * 2)(0, tables[0].stride(1))
    f.out_strides = _native._Strides(keys.stride(0), keys.stride(1), keys.stride(2))
    f.in_dtype = f.out_dtype = _native.WM_BF16
    f.batch, f.tokens, f.channels, f.kv_heads, f.head_dim = batch, tokens, channels, heads, dim
    f.eps = pool.rms_norm_eps
    finish_call = lambda: _native.call("wm_pool_finish", f, device)
    finish_ms = time_steps(finish_call, iters, 3, torch.cuda.synchronize) / iters
    finish_gbs = 2 * pool_bytes / (finish_ms * 1e-3) / 1e9
    out["finish_kernel"] = {"ms": finish_ms, "bytes": 2 * pool_bytes, "value": finish_gbs, "unit": "GB/s",
                            "roofline": {"bound": "hbm", "achieved": finish_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                         "frac": finish_gbs / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES.get("pool_finish_kernel")}}
    return out


def bench_mixed_decode(device, peaks, iters=5, batch=16):
    """Decode over K/V that are mixtures of 25 stacked sources, both forms: the mixture formed in the K/V load path of
    the decode kernel (every visible source row read once, nothing written), and the mixture materialised by the
    streaming kernel over the whole pool followed by the plain decode read.  B=16, H=HKV=16, 8192 slots, D=64 bf16,
    lengths uniform in [1, 8192]: 25 x 2 x 268 MB of sources."""
    from white_matter_b200 import mix_kv_sources, mixed_pool_decode, strict_causal_attention

    sources, heads, slots, dim = 25, 16, 8192, 64
    gen = torch.Generator().manual_seed(0)
    lengths = torch.randint(1, slots + 1, (batch,), generator=gen).to(device)
    ksrc = torch.empty(sources, batch, heads, slots, dim, device=device, dtype=torch.bfloat16)
    vsrc = torch.empty_like(ksrc)
    for i in range(sources):
        ksrc[i].normal_()
        vsrc[i].normal_()
    lk, lv = torch.randn(sources, device=device), torch.randn(sources, device=device)
    q = torch.randn(batch, heads, 1, dim, device=device, dtype=torch.bfloat16)
    fused = lambda: mixed_pool_decode(q, ksrc, vsrc, lk, lv, query_start=lengths, kv_lengths=lengths)
    fused_ms = time_steps(fused, iters, 3, torch.cuda.synchronize) / iters
    visible = int(lengths.sum().item()) * heads * dim * 2 * 2 * sources
    fused_gbs = visible / (fused_ms * 1e-3) / 1e9

    def two_step():
        return strict_causal_attention(q, mix_kv_sources(ksrc, lk), mix_kv_sources(vsrc, lv), query_start=lengths, kv_lengths=lengths)

    two_ms = time_steps(two_step, iters, 3, torch.cuda.synchronize) / iters
    whole = 2 * (ksrc.numel() * 2 + ksrc[0].numel() * 2) + int(lengths.sum().item()) * heads * dim * 2 * 2
    err = (fused().float() - two_step().float()).abs().max().item()
    return {
        "workload": f"decode over 25-source K/V mixtures, B={batch} H=16 slots=8192 D=64 bf16, lengths U[1,8192]",
        "fused_in_load_path": {"ms": fused_ms, "bytes": visible, "value": fused_gbs, "unit": "GB/s",
                               "roofline": {"bound": "hbm", "achieved": fused_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                            "frac": fused_gbs / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES.get("decode_split_kernel_mixed")}},
        "materialised_then_decode": {"ms": two_ms, "bytes": whole, "value": whole / (two_ms * 1e-3) / 1e9, "unit": "GB/s",
                                     "note": "mixes the whole pool capacity (the streaming kernel does not know the lengths), writes both mixtures, then reads them"},
        "max_abs_difference": err,
        "note": "per decode step the fused form re-reads all sources; a server that keeps the mixture resident pays the "
                "materialisation once per token and then reads 1/25 of these bytes per step",
    }


def bench_cyclic_prefill(device, peaks, reps=3):
    """Full cyclic prefill of the 24-layer model, random-initialised (weights ~ N(0, 0.02)): d_model 1024, 16 heads of
    64, SwiGLU 3072, RoPE base 1e6, vocabulary 151936, 25 pool sources into 8 channels of 16 KV heads, no dummy token;
    token ids uniform over the vocabulary, B=8, T=2048, 8 passes of 8 residue groups, bf16.  Embedding lookup, the
    block's passes (linear layers and norms are library calls; query preparation, attention, pool mixing and
    publication are this library's kernels), final norm and the last token's logits, replayed from one CUDA graph."""
    from white_matter_b200 import FeedbackBlock

    batch, tokens, hidden, layers, heads, dim, mlp, vocab, channels, passes, groups = 8, 2048, 1024, 24, 16, 64, 3072, 151936, 8, 8, 8
    gen = torch.Generator(device=device).manual_seed(4)
    block = FeedbackBlock(hidden, layers, heads, dim, mlp, heads, channels, rope_theta=1e6, use_dummy_token=False,
                          router_layer_stride=2, num_passes=passes, device=device)
    block.kv_pool.k_router_weight.normal_(0, 0.02, generator=gen)
    block.kv_pool.v_router_weight.normal_(0, 0.02, generator=gen)
    block.kv_pool.refresh()
    embedding = (torch.randn(vocab, hidden, device=device, generator=gen) * 0.02).to(torch.bfloat16)
    final_norm = torch.ones(hidden, device=device, dtype=torch.bfloat16)
    ids = torch.randint(0, vocab, (batch, tokens), device=device, generator=gen)

    def prefill():
        x = embedding[ids]
        h, _ = block(x, cyclic_groups=groups)
        last = torch.nn.functional.rms_norm(h[:, -1], (hidden,), final_norm, 1e-6)
        return torch.nn.functional.linear(last, embedding)  # tied head, last position only

    prefill()  # warm-up outside the capture: one-time attribute and symbol look-ups
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        prefill()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        logits = prefill()
    ms = time_steps(graph.replay, reps, 1, torch.cuda.synchronize) / reps
    t0 = time.perf_counter()
    prefill()
    torch.cuda.synchronize()
    eager_ms = (time.perf_counter() - t0) * 1e3
    rows = batch * tokens
    linear = 2 * rows * (2 * hidden * heads * dim + 3 * hidden * mlp) * layers * passes
    attention = 4 * dim * (tokens * (tokens - 1) // 2) * heads * batch * layers * passes
    pool = 2 * rows * (2 * channels * hidden * heads * dim + 2 * 13 * hidden * channels * (layers + 1)) * (passes + 1)
    flops = linear + attention + pool
    return {
        "workload": "full cyclic prefill, 24 layers d_model=1024 16 heads x 64, SwiGLU 3072, 25 sources -> 8 channels, "
                    "B=8 T=2048, 8 passes x 8 groups, bf16, random-init, CUDA-graph replay",
        "ms": ms, "value": rows / (ms * 1e-3), "unit": "prefill tokens/s", "eager_ms": eager_ms,
        "tflops": flops / (ms * 1e-3) / 1e12, "flops": {"linear": linear, "attention_visible": attention, "pool": pool},
        "finite": bool(torch.isfinite(logits.float()).all().item()),
    }


def bench_head_dim_128(device, peaks, iters=10):
    """Heads of 128 on the tensor-core kernels: the training configuration's call shape (B=16 H=16 K=2048 Q=256, stride
    8, residue 7) with head_dim 128, forward and gradients, against the SIMT family that served this head size before."""
    from white_matter_b200 import cyclic_attention

    dim = 128
    gen = torch.Generator(device=device).manual_seed(8)
    q, probe = (torch.randn(B, H, T // STRIDE, dim, device=device, generator=gen).to(torch.bfloat16) for _ in range(2))
    k, v = (torch.randn(B, H, T, dim, device=device, generator=gen).to(torch.bfloat16) for _ in range(2))
    residue = STRIDE - 1
    pairs = sum(residue + STRIDE * i for i in range(T // STRIDE)) * B * H  # strict past: key slots below the query's
    opts = dict(query_stride=STRIDE, query_offset=residue, strict_past=True)
    timed = {}
    for name, backend in (("tcgen05", "sm100"), ("simt", "sm100_simt")):
        n = iters if name == "tcgen05" else 3
        with torch.no_grad():
            call = lambda: cyclic_attention(q, k, v, backend=backend, **opts)
            timed[name] = time_steps(call, n, 2, torch.cuda.synchronize) / n
        leaves = [t.clone().requires_grad_() for t in (q, k, v)]
        out = cyclic_attention(*leaves, backend=backend, **opts)
        call = lambda: torch.autograd.grad(out, leaves, probe, retain_graph=True)
        timed[name + "_bwd"] = time_steps(call, n, 2, torch.cuda.synchronize) / n
        del out, leaves
    tf = 4 * dim * pairs / (timed["tcgen05"] * 1e-3) / 1e12
    tf_bwd = 10 * dim * pairs / (timed["tcgen05_bwd"] * 1e-3) / 1e12
    return {
        "workload": "cyclic_attention B=16 H=16 K=2048 Q=256 stride 8 residue 7, head_dim 128, bf16",
        "ms": timed["tcgen05"], "value": tf, "unit": "TFLOP/s", "simt_ms": timed["simt"],
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": tf / peaks["bf16_tflops"], "traffic": None, "peak_kind": "bf16_tflops (kernel timed alone)"},
        "backward": {"ms": timed["tcgen05_bwd"], "value": tf_bwd, "unit": "TFLOP/s", "simt_ms": timed["simt_bwd"],
                     "kernels": "bwd_delta_kernel, attn_bwd_tc_kernel<128> (one block per key tile), bwd_dq_convert_kernel",
                     "frac_of_burst_peak": tf_bwd / peaks["bf16_tflops"]},
    }


def bench_incumbents(device, iters=10):
    """The library kernels the upstream GPU backends call (src/white_matter/ops/flash_attention.py:15-36,52-103), timed
    on the same GPU as comparators: FlashAttention-2 (flash_attn package) and PyTorch's flash SDPA.  Labelled extras:
    nothing of this library's path runs here."""
    out = {}
    batch, heads, slots, dim = 64, 16, 8192, 64
    gen = torch.Generator().manual_seed(0)
    lengths = torch.randint(1, slots + 1, (batch,), generator=gen).to(device)
    k = torch.randn(batch, slots, heads, dim, device=device, dtype=torch.bfloat16)
    v = torch.randn(batch, slots, heads, dim, device=device, dtype=torch.bfloat16)
    q = torch.randn(batch, 1, heads, dim, device=device, dtype=torch.bfloat16)
    nbytes = int(lengths.sum().item()) * 2 * heads * dim * 2
    try:
        from flash_attn import flash_attn_varlen_func, flash_attn_with_kvcache

        call = lambda: flash_attn_with_kvcache(q, k, v, cache_seqlens=lengths.int(), causal=True)
        ms = time_steps(call, iters, 3, torch.cuda.synchronize) / iters
        out["flash_attn_with_kvcache decode"] = {"ms": ms, "value": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s",
                                                 "workload": "B=64 H=16 D=64 lengths~U[1,8192], cache (B,N,H,D)"}
        # Jacobi prefill as the upstream flash path runs it: packed documents as varlen sequences (strict past = causal
        # attention of each token over its predecessors, without the diagonal: the upstream path shifts by one)
        b2, t2 = 8, 2048
        docs = geometric_documents(b2, t2, 512, seed=7)
        lens = []
        for row in docs.tolist():
            run = 1
            for t in range(1, t2):
                if row[t] == row[t - 1]:
                    run += 1
                else:
                    lens.append(run)
                    run = 1
            lens.append(run)
        cu = torch.tensor([0] + lens, device=device).cumsum(0).int()
        qv = torch.randn(b2 * t2, heads, dim, device=device, dtype=torch.bfloat16)
        kv = torch.randn(b2 * t2, heads, dim, device=device, dtype=torch.bfloat16)
        vv = torch.randn(b2 * t2, heads, dim, device=device, dtype=torch.bfloat16)
        call = lambda: flash_attn_varlen_func(qv, kv, vv, cu, cu, max(lens), max(lens), causal=True)
        ms = time_steps(call, iters, 3, torch.cuda.synchronize) / iters
        pairs = sum(n * (n + 1) // 2 for n in lens) * heads
        out["flash_attn_varlen_func prefill"] = {"ms": ms, "value": 4 * dim * pairs / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                                                 "workload": "B=8 T=2048 documents of mean 512 as varlen sequences, causal"}
    except Exception as exc:  # the package is optional
        out["flash_attn"] = {"unavailable": str(exc)[:200]}
    try:
        from torch.nn.attention import SDPBackend, sdpa_kernel

        b2, t2 = 8, 2048
        qd = torch.randn(b2, heads, t2, dim, device=device, dtype=torch.bfloat16)
        kd, vd = torch.randn_like(qd), torch.randn_like(qd)
        with sdpa_kernel([SDPBackend.FLASH_ATTENTION]):
            call = lambda: torch.nn.functional.scaled_dot_product_attention(qd, kd, vd, is_causal=True)
            ms = time_steps(call, iters, 3, torch.cuda.synchronize) / iters
        pairs = b2 * heads * t2 * (t2 + 1) // 2
        out["torch flash SDPA dense causal"] = {"ms": ms, "value": 4 * dim * pairs / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                                                "workload": "B=8 H=16 T=2048 D=64 dense causal (no documents)"}
    except Exception as exc:
        out["torch_sdpa"] = {"unavailable": str(exc)[:200]}
    return out


def use_all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1 to its ranks; the CPU legs are meant to use every core the process may run on."""
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    if torch.get_num_threads() < cores:
        torch.set_num_threads(cores)
    return torch.get_num_threads()


def cpu_sample(rows=B, residues=tuple(range(STRIDE)), repeats=1, dtype=torch.float32):
    """The CPU oracle on a bounded sample of the training workload: `rows` batch rows, the given residues, fwd+bwd,
    in `dtype` (fp32, or bf16 as the upstream portable backend runs bf16 tensors on the CPU).

    The default sample is one whole step (all 16 rows, all 8 residues).
    Returns (TFLOP/s over the sample's visible pairs, seconds per repeat, threads, description).
    """
    from oracle import attention_oracle as oracle
    from white_matter_b200 import prepare_feedback_metadata

    use_all_host_threads()

    docs = geometric_documents(B, T, DOC_MEAN, seed=7)[:rows]
    groups = [torch.arange(r, T, STRIDE) for r in range(STRIDE)]
    metas = prepare_feedback_metadata(docs, groups, T, use_dummy_token=False)
    gen = torch.Generator().manual_seed(0)
    q = torch.randn(rows, H, T // STRIDE, D, generator=gen).to(dtype).requires_grad_()
    k = torch.randn(rows, H, T, D, generator=gen).to(dtype).requires_grad_()
    v = torch.randn(rows, H, T, D, generator=gen).to(dtype).requires_grad_()
    g = torch.randn(rows, H, T // STRIDE, D, generator=gen).to(dtype)
    flops = 14 * D * sum(visible_pairs_per_head(docs, r, STRIDE) for r in residues) * H
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        for r in residues:
            out = oracle.cyclic_attention_oracle(
                q, k, v, query_stride=STRIDE, query_offset=r, strict_past=True, metadata=metas[r],
                compute_dtype=dtype,
            )
            torch.autograd.grad(out, (q, k, v), g)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    name = {torch.float32: "fp32", torch.bfloat16: "bf16"}.get(dtype, str(dtype))
    what = (f"{rows} of {B} batch rows, {len(residues)} of {STRIDE} residues, fwd+bwd {name}, "
            "oracle port on torch CPU, all host threads")
    return flops / best / 1e12, best, torch.get_num_threads(), what


# --------------------------------------------------------------------------- drivers


REFERENCE_BUDGET_S = 150.0  # wall clock the timed steps of the reference arm may take together


def run_reference_arm(args, rank, world):
    """The upstream algorithm on the host cores (the CPU oracle port), in whichever of fp32 and bf16 the host runs
    faster (the configuration is bf16; the upstream portable backend evaluates bf16 tensors in bf16 on the CPU).
    A step is the whole workload step -- all 16 batch rows, all 8 residues -- when the requested number of steps
    fits the time budget at that size, else a bounded sample of it (fewer batch rows, then fewer residues), which
    the line names; TFLOP/s are over the sample's own visible pairs."""
    if rank != 0:
        return
    probes = {dt: cpu_sample(dtype=dt) for dt in (torch.float32, torch.bfloat16)}
    dtype = max(probes, key=lambda dt: probes[dt][0])
    full_seconds = probes[dtype][1]
    per_step = REFERENCE_BUDGET_S / max(args.steps + max(args.warmup - 1, 0), 1)
    rows, residues = B, tuple(range(STRIDE))
    if full_seconds > per_step:
        rows = max(1, min(B, int(B * per_step / full_seconds)))
        if full_seconds * rows / B > per_step:  # one row is still too much: fewer residues of it (first, last, ...)
            keep = max(1, min(STRIDE, int(STRIDE * per_step / (full_seconds / B))))
            residues = tuple(sorted({round(i * (STRIDE - 1) / max(keep - 1, 1)) for i in range(keep)}))
    for _ in range(max(args.warmup - 1, 0)):
        cpu_sample(rows=rows, residues=residues, dtype=dtype)
    t0 = time.perf_counter()
    values = [cpu_sample(rows=rows, residues=residues, dtype=dtype) for _ in range(args.steps)]
    wall = time.perf_counter() - t0
    tflops = statistics.median(v[0] for v in values)
    line = {
        "impl": "reference", "metric": "cyclic_attention fwd+bwd TFLOP/s", "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": wall / args.steps * 1e3,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": "bf16" if dtype == torch.bfloat16 else "f32", "data": "synthetic",
        "config": workload_config(args.gpus, args.scaling),
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": values[0][2], "kind": "port", "sample": values[0][3],
                         "fp32_tflops": probes[torch.float32][0], "bf16_tflops": probes[torch.bfloat16][0],
                         "whole_step_seconds": full_seconds},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus, scaling="weak"):
    per_gpu = B if scaling == "weak" else -(-B // n_gpus)
    return {
        "workload": "cyclic_attention training sweep fwd+bwd: B=16 H=16 K=2048 Q=256/residue D=64 stride=8, "
                    "8 residues per step, packed documents (geometric, mean 1024), strict_past, bf16",
        "per_gpu_batch": per_gpu, "global_batch": B * n_gpus if scaling == "weak" else B, "heads": H, "key_len": T,
        "head_dim": D, "query_stride": STRIDE,
        "parallelism": f"replicas x{n_gpus} over batch (no collective), {scaling} scaling",
        "calls": "16 operator calls per step, stream-ordered one after another, replayed from a CUDA graph",
        "l2": "inputs larger than L2: K+V 134 MB per sweep, rotated over 2 input sets",
        "flops": "14*D per visible (query,key) pair",
    }


def eager_step_us(work, steps=5):
    """Host time (us) of one operator call when a step is issued eagerly: 16 calls, wall clock around `steps` steps
    with one synchronisation at the end (the calls are launch-bound, so the host is what is being timed)."""
    work.step(None)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        work.step(None)
    torch.cuda.synchronize()
    return (time.perf_counter() - t0) / (steps * 2 * STRIDE) * 1e6


LEGS = {
    "decode": lambda device, peaks, small: dict(zip(("decode", "prefill128"), bench_decode(device, peaks))),
    "jacobi": lambda device, peaks, small: bench_jacobi(device, peaks),
    "mixing": lambda device, peaks, small: bench_mixing(device, peaks),
    "query_prepare": lambda device, peaks, small: bench_query_prepare(device, peaks),
    "pool_projection": lambda device, peaks, small: bench_pool_projection(device, peaks),
    "mixed_decode": lambda device, peaks, small: bench_mixed_decode(device, peaks, batch=4 if small else 16),
    "cyclic_prefill": lambda device, peaks, small: bench_cyclic_prefill(device, peaks),
    "head_dim_128": lambda device, peaks, small: bench_head_dim_128(device, peaks),
}


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--backend", default="sm100", help="kernel family: sm100 | sm100_simt | sm100_tcgen05")
    parser.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                        help="weak: every rank runs its own B=16 rows; strong: the B=16 rows are split over the ranks")
    parser.add_argument("--no-graph", action="store_true", help="issue the operator calls eagerly instead of replaying a CUDA graph")
    parser.add_argument("--skip-extras", action="store_true", help="only the headline workload (used for profiling)")
    parser.add_argument("--leg", action="append", choices=sorted(LEGS), default=None,
                        help="run only the named secondary leg(s) and print their results (used for profiling)")
    parser.add_argument("--skip-leg", action="append", choices=sorted(LEGS), default=[],
                        help="leave the named secondary leg(s) out of the full run (the launch-list capture leaves out the "
                             "full-model prefill, tens of thousands of launches)")
    parser.add_argument("--small", action="store_true", help="with --leg mixed_decode: 4 batch rows instead of 16")
    args = parser.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the sm_100a kernels have no CPU path")
    args.warmup = max(args.warmup, 3)
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    import torch.distributed as dist

    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def sync():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    if args.leg:
        peaks_only, _ = load_peaks()
        results = {name: LEGS[name](device, peaks_only, args.small) for name in args.leg}
        torch.cuda.synchronize()
        print(json.dumps(results), flush=True)
        return

    from white_matter_b200 import _native
    from white_matter_b200.replicas import aggregate_throughput, shard_batch_heads

    lib = _native.load_library()
    peaks, peak_kind = load_peaks()
    rows = slice(0, B)
    if args.scaling == "strong":
        if world > B:
            raise SystemExit("strong scaling splits the 16 batch rows: at most 16 ranks")
        rows = shard_batch_heads(B, H, rank, world)[0]
    seed_of = (lambda i: rank * 2 + i) if args.scaling == "weak" else (lambda i: i)  # strong: slices of one problem
    sets = [TrainingSweep(device, seed=seed_of(i), backend=args.backend, rows=rows) for i in range(2)]
    status = {}

    def check(where):
        status[where] = int(lib.wm_device_status(1))

    # end to end (measured first, before the CUDA graphs of the device-resident arm exist): pinned host -> device -> pinned host every step
    staging = sets[0].staging()
    e2e_step = lambda: sets[0].step_e2e(staging)
    e2e_steps = max(2, min(args.steps // 2, 20))
    e2e_ms = time_steps(e2e_step, e2e_steps, 2, sync)
    e2e_max_ms, e2e_flops = aggregate_throughput(e2e_ms, float(sets[0].flops * e2e_steps), device)
    e2e_serial = e2e_flops / (e2e_max_ms * 1e-3) / 1e12
    del staging
    sync()
    # host-side effects (page migration of the pinned buffers, another tenant on the PCIe switch) make single runs
    # of this arm vary by 2x from box to box: the better of two runs is reported
    piped_ms = min(sets[0].e2e_pipelined_ms(e2e_steps, warmup=3) for _ in range(2))
    sync()
    check("e2e")
    torch.cuda.empty_cache()
    piped_max_ms, piped_flops = aggregate_throughput(piped_ms, float(sets[0].flops * e2e_steps), device)
    e2e_value = piped_flops / (piped_max_ms * 1e-3) / 1e12
    eager_us = eager_step_us(sets[0])

    turn = [0]
    per_step_launches = None
    if not args.no_graph:
        per_step_launches = [s.capture(1) for s in sets][0]

    def step():
        if args.no_graph:
            sets[turn[0] % 2].step(None)
        else:
            sets[turn[0] % 2].replay()
        turn[0] += 1

    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.3)  # nvidia-smi takes a moment to deliver its first sample
    sampler.mark_load()
    settle = time.perf_counter()
    while time.perf_counter() - settle < 0.4:  # the timed region is short: give the sampler the same load for longer
        step()
        torch.cuda.synchronize()
    for _ in range(args.warmup):
        step()
    sync()
    launches0 = lib.wm_kernel_launch_count()
    sampler.mark_timed(True)
    ms = time_steps(step, args.steps, 0, sync)
    sampler.mark_timed(False)
    launches = lib.wm_kernel_launch_count() - launches0
    if per_step_launches is not None:
        launches = per_step_launches * args.steps  # kernels inside the replayed graphs
    clocks = sampler.stop()
    check("headline")

    flops = sum(sets[i % 2].flops for i in range(args.steps))
    step_ms, total_flops = aggregate_throughput(ms, float(flops), device)
    value = total_flops / (step_ms * 1e-3) / 1e12

    # per-kernel device time: a graph with the 8 forward launches alone, replayed and timed with CUDA events; the
    # backward kernel group is the step minus the forward part
    work = sets[0]
    fwd_ms = work.forward_only_ms(reps=max(3, min(args.steps, 20))) / STRIDE
    step_device_ms = step_ms / args.steps
    if not args.no_graph:
        step_device_ms = work.one_stream_ms(reps=max(3, min(args.steps, 20)))
    bwd_ms = max(step_device_ms / STRIDE - fwd_ms, 1e-6)
    tensor_peak = peaks["bf16_tflops_sustained"]
    fwd_tf = work.flops_fwd / STRIDE / (fwd_ms * 1e-3) / 1e12
    bwd_tf = (work.flops - work.flops_fwd) / STRIDE / (bwd_ms * 1e-3) / 1e12
    fwd_bytes, bwd_bytes = work.call_bytes()
    hbm = peaks["hbm_gbs"]

    def hbm_view(nbytes, call_ms, flops_of_call):
        """Where the call stands against the HBM-limited ceiling: at the stride-8 shape a call moves 128 FLOP per
        byte, below the ridge of the machine, so bandwidth bounds it before the tensor pipe does."""
        floor_ms = nbytes / (hbm * 1e9) * 1e3
        return {"algorithmic_bytes": nbytes, "achieved_gbs": nbytes / (call_ms * 1e-3) / 1e9, "hbm_frac": floor_ms / call_ms,
                "ceiling_tflops": flops_of_call / (floor_ms * 1e-3) / 1e12}

    multi = None
    if not args.no_graph and not args.skip_extras:
        # labelled extra, not the headline: the same 16 calls spread over 8 streams, which only a caller whose residue
        # calls do not depend on one another may do
        getattr(torch.autograd.graph, "set_warn_on_accumulate_grad_stream_mismatch", lambda flag: None)(False)
        work.capture(STRIDE)
        multi_ms = time_steps(work.replay, max(3, min(args.steps, 20)), 2, sync) / max(3, min(args.steps, 20))
        multi = {"ms_per_step": multi_ms, "value": work.flops / (multi_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "streams": STRIDE,
                 "note": "not the headline: the 8 residue calls of a step on 8 streams fill each other's partial waves; in the model "
                         "the residue groups depend on one another and run one after another"}
        check("multi_stream")

    extras = {}
    if not args.skip_extras:
        torch.cuda.empty_cache()
        for name in ("decode", "jacobi", "mixing", "query_prepare", "pool_projection", "mixed_decode", "cyclic_prefill", "head_dim_128"):
            if name in args.skip_leg:
                continue
            torch.cuda.empty_cache()
            result = LEGS[name](device, peaks, False)
            if name == "decode":
                extras.update(result)  # decode and the cached-prefix prefill over the same pool
            else:
                extras[name] = result
        torch.cuda.empty_cache()
        check("extras")
        if world == 1:
            torch.cuda.empty_cache()
            extras["incumbents"] = bench_incumbents(device)
    if rank == 0:
        line = {
            "metric": "cyclic_attention fwd+bwd TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms / args.steps,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(world, args.scaling), "clocks": clocks, "gpu_launches": int(launches),
            "device_status": status, "backend": args.backend,
            "launch_mode": "eager" if args.no_graph else "cuda graph replay of one step, its 24 launches one after another",
            "multi_stream": multi,
            "eager": {"host_us_per_call": eager_us, "note": "the same step without the graph: 16 operator calls, host-bound"},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": sets[0].staging_bytes()[0],
                    "d2h_bytes_per_step": sets[0].staging_bytes()[1],
                    "mode": "copies on their own streams beside the kernels of the neighbouring steps (two staging sets)",
                    "serialized": e2e_serial, "steps": e2e_steps, "runs": "best of 2"},
            "roofline": {"bound": "tensor", "kernel": "backward kernels of one residue call (attn_bwd_resident_kernel + bwd_delta_kernel)",
                         "achieved": bwd_tf, "peak": tensor_peak, "unit": "TFLOP/s", "frac": bwd_tf / tensor_peak,
                         "traffic": NCU_TRAFFIC_BYTES["attn_bwd_resident_kernel"] if args.backend != "sm100_simt" else None,
                         "peak_kind": f"{peak_kind} bf16_tflops_sustained", "ms": bwd_ms,
                         "hbm": hbm_view(bwd_bytes, bwd_ms, (work.flops - work.flops_fwd) / STRIDE)},
            "roofline_forward": {"bound": "tensor", "kernel": "attn_fwd_tc_kernel, one residue call",
                                 "achieved": fwd_tf, "peak": tensor_peak, "unit": "TFLOP/s",
                                 "frac": fwd_tf / tensor_peak,
                                 "traffic": NCU_TRAFFIC_BYTES["attn_fwd_tc_kernel"] if args.backend != "sm100_simt" else None,
                                 "ms": fwd_ms, "hbm": hbm_view(fwd_bytes, fwd_ms, work.flops_fwd / STRIDE)},
        }
        line.update(extras)
        if world == 1 and not args.skip_extras:
            tf, secs, cores, what = cpu_sample(repeats=2)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                                    "sample": what, "seconds": secs}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
