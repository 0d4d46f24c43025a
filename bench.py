#!/usr/bin/env python
"""Benchmark of the fused GEMM-SwiGLU path:  python bench.py --gpus N --steps K --warmup W [--impl reference]

A step is one pass of the op over one batch of synthetic input (X ~ N(0,1), W ~ N(0,0.02), bf16).  The headline
workload is the Llama-3-8B-shaped FFN up-projection, X[8192,4096] x W[2*14336,4096] -> Y[8192,14336]; the same JSON
line carries, under "workloads", one sub-record for each of the other benchmark configurations (video-DiT FFN, the
three decode shapes, the full SwiGLU MLP block), each with its own timing, roofline and output check.  On N > 1 GPUs
the packed weight is column-sharded along N (rank r owns N/P gate and N/P up rows), X is replicated and no collective
is on the op's data path; the job's work is the whole problem, so scaling is "strong".  Only the MLP block has an
exchange step: the reduction after the row-parallel down projection.  At N > 1 its record is the fused all-reduce
("peer_all_reduce": the down projection's epilogue stores each row block straight into its owner GPU's memory, the
owners sum and store their rows into every GPU's result; every rank ends with the whole result, as after the
reference's row-parallel linear) and carries three more timings of the same block: NCCL's all-reduce with row chunks
overlapped with the next chunk's GEMMs ("nccl_all_reduce"), NCCL's reduce-scatter, and the fused reduce-scatter
("peer_scatter").  Without symmetric memory the record is NCCL's all-reduce and says why ("peer_unavailable").

Timing: W warm-up steps, then exactly K steps, each bracketed by its own pair of CUDA events on the launch stream
with an L2 flush (256 MiB written, then 256 MiB read, so no dirty lines remain) before it; a barrier and a device
synchronise surround the timed region; the per-rank sum of the K step times is reduced with MAX over ranks.  SM
clocks and throttle reasons are sampled with nvidia-smi (read-only) while the steps run.

Output check (outside every timed region, on every rank): sampled rows of the rank's own output against an fp32
computation of the same rows on the GPU; the worst rank's errors are printed as "parity" and a failed check makes the
process exit non-zero.

One JSON line is printed by rank 0.  `value` is device-resident throughput; `e2e` is the same metric with the step's
X coming from pinned host memory and its Y going back to pinned host memory inside the timed region; `roofline`
describes the kernel against the measured peak of this GPU pool; `cpu_baseline` times the reference's eager PyTorch
expression on the host cores on a bounded slice of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

WORKLOADS = {
    # name: (M, K, N, bound, description)
    "llama3_8b_ffn": (8192, 4096, 14336, "tensor", "Llama-3-8B-shaped FFN up-projection X[8192,4096] W[2x14336,4096]"),
    "video_dit_ffn": (32760, 5120, 13824, "tensor", "video-DiT-shaped FFN X[32760,5120] W[2x13824,5120]"),
    "decode_m16": (16, 8192, 28672, "hbm", "decode-shaped weight streaming X[16,8192] W[2x28672,8192]"),
    "decode_m64": (64, 8192, 28672, "hbm", "decode-shaped weight streaming X[64,8192] W[2x28672,8192]"),
    "decode_m128": (128, 8192, 28672, "hbm", "decode-shaped weight streaming X[128,8192] W[2x28672,8192]"),
    "cpu_ref_case": (256, 1024, 2816, "tensor", "reference CPU-sized case X[256,1024] W[2x2816,1024]"),
    # full SwiGLU MLP: fused column-parallel gate/up, row-parallel down projection, NCCL all-reduce (see run_mlp_block)
    "mlp_block": (16384, 8192, 28672, "tensor", "SwiGLU MLP block X[16384,8192], gate/up [2x28672,8192], down [8192,28672]"),
}
# the other benchmark configurations, timed after the headline workload and reported under "workloads"
# (the short HBM-bound shapes first: they are timed before the long tensor-bound loops heat the GPU into its power cap)
SUB_WORKLOADS = ("decode_m16", "decode_m64", "decode_m128", "video_dit_ffn", "mlp_block")
SETTLE_S = 0.5  # idle time before each workload: lets the power-cap controller release the previous workload's clocks
# DRAM bytes (read + write) of ONE launch of the dominant kernel as an earlier one-launch ncu capture RECORDED them;
# not measured in this run, and reported only while the schedule is still the one that was profiled.
RECORDED_TRAFFIC = {
    # workload@gpus: (bytes, {plan keys that must match}); the captures are summarised under profiles/
    "llama3_8b_ffn@1": (1088.0e6, {"variant": 4, "block_n": 256, "stages": 4, "group_m": 16, "y_tma": 1, "sk_tiles": 90}),
    "video_dit_ffn@1": (9330.3e6, {"variant": 4, "block_n": 256, "stages": 4, "group_m": 12, "y_tma": 1, "sk_tiles": 0}),
    "decode_m64@1": (946.6e6, {"variant": 2, "block_n": 208, "stages": 3, "k_splits": 1}),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
L2_FLUSH_BYTES = 256 << 20
# tolerance of the path against an fp32-accumulated gold: max|y-gold|/max|gold| and ||y-gold||_F/||gold||_F
TOL_MAX_NORM, TOL_FROB = 1e-2, 5e-3
# the MLP block's output is a sum over ranks of bf16-rounded partial products of a bf16-rounded activation
TOL_MLP_MAX_NORM, TOL_MLP_FROB = 2e-2, 1e-2
PARITY_ROWS = 256


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return json.loads(p.read_text()), "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def flops_of(M, K, N):
    return 2.0 * M * K * 2 * N


def bytes_of(M, K, N):
    return 2.0 * (M * K + 2 * N * K + M * N)


def make_inputs_cpu(M, K, N, seed=0):
    """The headline workload's inputs: CPU generator, X ~ N(0,1) then W ~ N(0,0.02), cast to bf16 (the generator the
    CPU oracle's tests use, so the CPU baseline and the GPU see the same bits)."""
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * N, K, generator=g) * 0.02).to(torch.bfloat16)
    return x, w


def make_inputs_cuda(M, K, N, dev, seed=0, with_down=False):
    """Inputs of the sub-workloads, generated on the device (same distributions; every rank draws the same global
    tensors from the same seed and keeps its shard).  Rows are drawn in blocks so no multi-GB fp32 temporary exists."""
    g = torch.Generator(device=dev)
    g.manual_seed(seed)

    def draw(rows, cols, scale):
        out = torch.empty(rows, cols, dtype=torch.bfloat16, device=dev)
        step = 8192
        for lo in range(0, rows, step):
            hi = min(rows, lo + step)
            out[lo:hi] = (torch.randn(hi - lo, cols, generator=g, device=dev) * scale).to(torch.bfloat16)
        return out

    x = draw(M, K, 1.0)
    w = draw(2 * N, K, 0.02)
    if with_down:
        return x, w, draw(K, N, 0.02)
    return x, w


def config_of(workload, n_gpus):
    """The `config` object, identical in the GPU arm and the reference arm."""
    M, K, N, _, desc = WORKLOADS[workload]
    return {"workload": workload, "shape": desc, "M": M, "K": K, "N": N,
            "parallelism": f"column-shard of W over {n_gpus} GPU(s), X replicated, no collective on the op's data path",
            "l2": "flushed before every timed step (256 MiB written, then 256 MiB read)"}


class ClockSampler:
    """Reads SM clock and throttle reasons with nvidia-smi while the timed region runs (never sets anything)."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
                power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [c for c, p in zip(sm, power) if p >= 0.5 * max(power)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(smax), "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power)}


def cpu_eager(M, K, N, x, w, target_s=12.0):
    """The reference's eager expression on the host cores, on the first rows of the same X (bounded sample)."""
    from oracle import swiglu_ref_eager

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    rows = min(M, 256)
    xs = x[:rows].contiguous()
    swiglu_ref_eager(xs, w)  # warm-up (thread pool, oneDNN primitive cache)
    t0 = time.perf_counter()
    swiglu_ref_eager(xs, w)
    dt = max(time.perf_counter() - t0, 1e-6)
    # grow the slice towards ~target_s of work in total, 3 timed repetitions
    rows2 = int(min(M, max(rows, rows * (target_s / 3.0) / dt)))
    rows2 = max(16, rows2 // 16 * 16) if M >= 16 else M
    xs = x[:rows2].contiguous()
    times = []
    reps = 3
    while len(times) < reps:
        t0 = time.perf_counter()
        swiglu_ref_eager(xs, w)
        times.append(time.perf_counter() - t0)
        if len(times) == 3:  # about target_s of CPU work in total, at most 40 repetitions
            reps = int(min(40, max(3, target_s / max(statistics.median(times), 1e-6))))
    t = statistics.median(times)
    return rows2, threads, t, len(times)


def run_reference_arm(args, rank, world):
    """--impl reference: MagiCompiler's eager SwiGLU on the host CPU (its only implementation of this path)."""
    if rank != 0:
        return
    from oracle import swiglu_ref_eager

    M, K, N, bound, desc = WORKLOADS[args.workload]
    x, w = make_inputs_cpu(M, K, N, seed=0)
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    # one step = the expression on a bounded row-slice of the workload; size it from a probe so K+W steps take ~1-2 min
    rows = min(M, 128)
    swiglu_ref_eager(x[:rows], w)
    t0 = time.perf_counter()
    swiglu_ref_eager(x[:rows], w)
    dt = max(time.perf_counter() - t0, 1e-6)
    budget_per_step = 90.0 / max(1, args.steps + args.warmup)
    rows = int(min(M, max(16, rows * budget_per_step / dt)))
    rows = rows // 16 * 16 if rows >= 16 else rows
    xs = x[:rows].contiguous()
    for _ in range(args.warmup):
        swiglu_ref_eager(xs, w)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        swiglu_ref_eager(xs, w)
    total = time.perf_counter() - t0
    per_step = total / args.steps
    if bound == "hbm":
        value, unit, metric = bytes_of(rows, K, N) / per_step / 1e9, "GB/s", "fused GEMM-SwiGLU HBM GB/s (small-M)"
    else:
        value, unit, metric = flops_of(rows, K, N) / per_step / 1e12, "TFLOP/s", "fused GEMM-SwiGLU TFLOP/s"
    sample = f"eager F.silu(F.linear(x,Wg))*F.linear(x,Wu) on the first {rows} of {M} rows, full W, {threads} threads"
    line = {
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (CPU generator seed 0, X~N(0,1), W~N(0,0.02), bf16)",
        "config": config_of(args.workload, args.gpus),
        "detail": {"rows_per_step": rows, "where": "host CPU cores; no GPU is used by this arm"},
        "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


class Bench:
    """Shared state of one rank's run: device, process group, L2 flush buffers, timing helpers."""

    def __init__(self, args, rank, world, local_rank):
        import torch.distributed as dist

        self.args, self.rank, self.world, self.local_rank, self.dist = args, rank, world, local_rank, dist
        self.dev = torch.device("cuda", local_rank)
        self.flush_w = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=self.dev)
        self.flush_r = torch.zeros(L2_FLUSH_BYTES // 4, dtype=torch.int32, device=self.dev)
        self.peaks, self.peak_kind = measured_peaks()

    def flush_l2(self):
        # write a buffer larger than L2, then read another one: the timed kernel starts from an L2 that holds
        # neither its inputs nor dirty lines whose write-back would be charged to it
        if not self.args.no_flush:
            self.flush_w.zero_()
            self.flush_r.max()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize(self.dev)

    def reduce(self, value, op="max"):
        t = torch.tensor([float(value)], dtype=torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX if op == "max" else self.dist.ReduceOp.MIN)
        return float(t.item())

    def time_steps(self, step, steps, warmup, flush=True):
        """`warmup` untimed steps, then exactly `steps` steps each inside its own CUDA-event pair on the current
        stream.  Returns (ms per step = MAX over ranks of the per-rank sum / steps, this rank's per-step list, wall s)."""
        for _ in range(warmup):
            if flush:
                self.flush_l2()
            step()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
        self.barrier()
        wall0 = time.perf_counter()
        for i in range(steps):
            if flush:
                self.flush_l2()
            starts[i].record()
            step()
            ends[i].record()
        self.barrier()
        wall = time.perf_counter() - wall0
        per_step = [s.elapsed_time(e) for s, e in zip(starts, ends)]
        return self.reduce(sum(per_step)) / steps, per_step, wall

    def timed_median(self, fn, reps=10, warm=3):
        for _ in range(warm):
            fn()
        ts = []
        for _ in range(reps):
            self.flush_l2()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            fn()
            s1.record()
            torch.cuda.synchronize(self.dev)
            ts.append(s0.elapsed_time(s1))
        return statistics.median(ts)

    def check_status(self, mb):
        status = mb.device_status(self.local_rank)
        if status["code"] != 0:
            raise SystemExit(f"kernel watchdog fired: {status}")

    def parity(self, y, gold, tol_max, tol_frob):
        """Worst rank's normalised errors of y against the fp32 gold of the same rows; `ok` only if every rank passes."""
        diff = y.float() - gold
        gmax = gold.abs().max().item()
        max_norm = diff.abs().max().item() / gmax if gmax > 0 else float("inf")
        frob = diff.norm().item() / gold.norm().item() if gmax > 0 else float("inf")
        finite = bool(torch.isfinite(y.float()).all().item())
        ok = finite and max_norm <= tol_max and frob <= tol_frob
        worst_max, worst_frob = self.reduce(max_norm), self.reduce(frob)
        all_ok = self.reduce(1.0 if ok else 0.0, op="min") > 0.5
        return {"max_norm": worst_max, "frob": worst_frob, "ok": bool(all_ok), "rows_checked_per_rank": int(y.shape[0]),
                "tolerance": {"max_norm": tol_max, "frob": tol_frob}, "ranks": self.world}


def sample_rows(M, dev, seed=1):
    """Row indices for the output check: every row when there are few, else a seeded sample that includes the last rows
    (the ragged tile)."""
    if M <= PARITY_ROWS:
        return torch.arange(M, device=dev)
    g = torch.Generator().manual_seed(seed)
    idx = torch.cat([torch.randperm(M - 8, generator=g)[:PARITY_ROWS - 8], torch.arange(M - 8, M)])
    return idx.to(dev)


def gold_rows(x, w, rows):
    """fp32 gold of the op on the given rows (TF32 off): silu(x·Wg^T) * (x·Wu^T)."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        n = w.shape[0] // 2
        xs = x[rows].float()
        out = torch.empty(xs.shape[0], n, dtype=torch.float32, device=x.device)
        for lo in range(0, n, 4096):  # column blocks keep the fp32 copy of W small
            hi = min(n, lo + 4096)
            g = xs @ w[lo:hi].float().t()
            u = xs @ w[n + lo:n + hi].float().t()
            out[:, lo:hi] = torch.nn.functional.silu(g) * u
        return out
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def op_roofline(b, bound, M, K, n_local, rank0_ms, kclk_mhz=None):
    flops_rank, bytes_rank = flops_of(M, K, n_local), bytes_of(M, K, n_local)
    if bound == "hbm":
        achieved = bytes_rank / (rank0_ms * 1e-3) / 1e9
        peak = float(b.peaks["hbm_gbs"])
        roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": None, "peak_kind": f"{b.peak_kind} copy bandwidth", "nominal_frac": achieved / 8000.0}
    else:
        achieved = flops_rank / (rank0_ms * 1e-3) / 1e12
        peak = float(b.peaks["bf16_tflops"])
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": None, "peak_kind": f"{b.peak_kind} cuBLAS bf16 burst (kernel timed alone)",
                "nominal_frac": achieved / 2250.0}
        if b.peaks.get("bf16_tflops_sustained"):
            # the same library GEMM run back to back for seconds under the power cap: the fairer yardstick when
            # --steps is large enough for the cap to bite (the timed loop keeps the GPU busy for that long too)
            roof["peak_sustained"] = float(b.peaks["bf16_tflops_sustained"])
            roof["frac_of_sustained"] = achieved / float(b.peaks["bf16_tflops_sustained"])
        if kclk_mhz and kclk_mhz > 0:
            n_sm = torch.cuda.get_device_properties(b.dev).multi_processor_count
            roof["tensor_pipe_frac_at_kernel_clock"] = achieved / (8192 * n_sm * kclk_mhz * 1e6 / 1e12)
    roof["kernel"] = "swiglu_tc_kernel"
    roof["kernel_ms"] = rank0_ms
    roof["algorithmic_bytes"] = bytes_rank
    roof["algorithmic_flops"] = flops_rank
    return roof


def time_op_workload(b, mb, name, x, w_local, steps, warmup, knobs=None):
    """Device-resident timing + output check of the fused op on one workload (this rank's column shard)."""
    M, K, N, bound, desc = WORKLOADS[name]
    knobs = knobs or {}
    n_local = w_local.shape[0] // 2
    y = torch.empty(M, n_local, dtype=torch.bfloat16, device=b.dev)
    plan = mb.plan(M, n_local, K, device=b.local_rank, **knobs)

    def step():
        mb.gemm_swiglu_out(x, w_local, out=y, **knobs)

    ms_per_step, per_step, wall = b.time_steps(step, steps, warmup)
    kclk = mb.kernel_clock(b.local_rank)  # SM clock of the last timed kernel, measured inside the kernel
    b.check_status(mb)
    rank0_ms = sum(per_step) / len(per_step)
    flops, nbytes = flops_of(M, K, N), bytes_of(M, K, N)
    unit = "GB/s" if bound == "hbm" else "TFLOP/s"
    scale = (nbytes / 1e9) if bound == "hbm" else (flops / 1e12)
    rec = {
        "shape": desc, "n_per_gpu": n_local, "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step,
        "ms_median": b.reduce(statistics.median(per_step)), "ms_min": b.reduce(min(per_step)),
        "value": scale / (ms_per_step * 1e-3), "unit": unit,
        "roofline": op_roofline(b, bound, M, K, n_local, rank0_ms, kclk["sm_mhz"]),
        "clocks": {"kernel_sm_mhz": kclk["sm_mhz"]}, "plan": plan,
        "gpu_launches": steps * (2 if plan.get("k_splits", 1) > 1 else 1),
    }
    recorded = RECORDED_TRAFFIC.get(f"{name}@{b.world}")
    if recorded and all(plan.get(k) == v for k, v in recorded[1].items()):
        rec["roofline"]["traffic"] = recorded[0]
        rec["roofline"]["traffic_kind"] = "recorded from a one-launch ncu capture of this schedule, not measured in this run"
    # ---- the same step replayed from a CUDA graph (the small-M shapes run for 20-160 us: a replay takes the host's
    # launch path out of the picture)
    if bound == "hbm":
        side = torch.cuda.Stream(b.dev)
        side.wait_stream(torch.cuda.current_stream(b.dev))
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream(b.dev).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        ts = []
        for _ in range(max(5, min(steps, 30))):
            b.flush_l2()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record()
            graph.replay()
            g1.record()
            torch.cuda.synchronize(b.dev)
            ts.append(g0.elapsed_time(g1))
        graph_ms = b.reduce(statistics.median(ts))
        rec["cuda_graph"] = {"ms_per_step": graph_ms, "value": nbytes / (graph_ms * 1e-3) / 1e9, "unit": unit,
                             "frac": bytes_of(M, K, n_local) / (graph_ms * 1e-3) / 1e9 / float(b.peaks["hbm_gbs"]),
                             "how": "one captured op call replayed, L2 flushed before each replay, median, max over ranks"}
        del graph
    # ---- output check, outside the timed region: this rank's shard on sampled rows against the fp32 gold
    y.fill_(float("nan"))
    step()
    rows = sample_rows(M, b.dev)
    rec["parity"] = b.parity(y[rows], gold_rows(x, w_local, rows), TOL_MAX_NORM, TOL_FROB)
    return rec, y, step, plan, per_step, wall, kclk


def run_mlp_block(b, mb, steps, warmup, chunks, reduce, down):
    """Config 5: gate/up column-parallel through the fused op, down projection row-parallel, one reduction over NVLink
    (NCCL), optionally chunked so the reduce of chunk i overlaps the GEMMs of chunk i+1."""
    M, K, N, _, desc = WORKLOADS["mlp_block"]
    x, w, wd = make_inputs_cuda(M, K, N, b.dev, seed=0, with_down=True)
    mlp = mb.TensorParallelSwiGLUMLP(w, wd, b.rank, b.world, chunks=chunks, reduce=reduce, borrow_result=True,
                                     down_fn=mb.gemm_nt_out if down == "own" else None).to(b.dev)
    out_box = [None]

    def step():
        out_box[0] = mlp(x)

    # inputs (1.7 GB) are far larger than L2 and every step streams them, so no flush kernels between steps
    ms_per_step, per_step, wall = b.time_steps(step, steps, warmup, flush=False)
    b.check_status(mb)
    flops = 2.0 * M * K * 2 * N + 2.0 * M * N * K
    value = flops / (ms_per_step * 1e-3) / 1e12
    per_gpu = value / b.world
    peak = float(b.peaks["bf16_tflops_sustained"])
    # ---- output check: sampled rows against the unsharded MLP in fp32 (full weights are on every GPU here)
    rows = sample_rows(M, b.dev, seed=5)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        h = gold_rows(x, w, rows)
        ref = torch.zeros(rows.numel(), K, dtype=torch.float32, device=b.dev)
        for lo in range(0, N, 4096):
            ref += h[:, lo:lo + 4096] @ wd[:, lo:lo + 4096].float().t()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    out = out_box[0]
    if reduce in ("reduce_scatter", "peer_scatter") and b.world > 1:  # this rank holds only its rows of the sum: check those
        own = mlp.owned_rows(M).to(b.dev)
        pos = torch.arange(0, own.numel(), max(1, own.numel() // PARITY_ROWS), device=b.dev)[:PARITY_ROWS]
        rows = own[pos]
        h = gold_rows(x, w, rows)
        ref = torch.zeros(rows.numel(), K, dtype=torch.float32, device=b.dev)
        for lo in range(0, N, 4096):
            ref += h[:, lo:lo + 4096] @ wd[:, lo:lo + 4096].float().t()
        got = out[pos]
    else:
        got = out.reshape(M, K)[rows]
    parity = b.parity(got, ref, TOL_MLP_MAX_NORM, TOL_MLP_FROB)
    rec = {
        "shape": desc, "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step,
        "ms_median": b.reduce(statistics.median(per_step)), "ms_min": b.reduce(min(per_step)),
        "value": value, "unit": "TFLOP/s", "chunks": chunks, "reduce": reduce,
        "down_projection": "magi_swiglu_gemm_nt_bf16 (own tile kernel)" if down == "own" else "torch.matmul (library GEMM)",
        "parallelism": (f"tp{b.world}: column-parallel gate/up, row-parallel down, " +
                        ("row blocks of the partial products stored by the down projection's epilogue into their owner's "
                         "memory over NVLink (no collective kernel), barrier, slot sum" +
                         (" stored into every GPU's result, barrier" if reduce == "peer_all_reduce" else "")
                         if reduce in ("peer_scatter", "peer_all_reduce") else f"NCCL {reduce.replace('_', '-')}") + f" of [{M},{K}] bf16") if b.world > 1 else "1 GPU: no reduction",
        "l2": "inputs (1.7 GB) larger than L2, back-to-back steps",
        "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s", "frac": per_gpu / peak,
                     "nominal_frac": per_gpu / 2250.0, "algorithmic_flops": flops / b.world, "traffic": None,
                     "peak_kind": f"{b.peak_kind} cuBLAS bf16 sustained (kernels timed inside a long step)"},
        "gpu_launches": steps * (3 if reduce in ("peer_scatter", "peer_all_reduce") and b.world > 1
                                 else chunks * (2 if down == "own" else 1)),
        "parity": parity,
    }
    del mlp, x, w, wd
    return rec


def e2e_single_gpu(b, mb, x_cpu, w, y, knobs, n_steps):
    """N = 1: every step pinned X -> device, op, Y -> pinned host, in row chunks on three side streams."""
    M, K = x_cpu.shape
    n_local = w.shape[0] // 2
    x_host = x_cpu.pin_memory()
    y_host = torch.empty(M, n_local, dtype=torch.bfloat16).pin_memory()
    chunks = 8 if M >= 4096 else 1
    rows = -(-M // chunks)
    # Large M: chunk c of every step owns rows [lo, hi) of one set of buffers and always runs on stream c % 3.
    # Small M (one chunk): three complete buffer sets, step k uses set k % 3 on stream k % 3.
    sets = 1 if chunks > 1 else 3
    streams = [torch.cuda.Stream(b.dev) for _ in range(3)]
    x_devs = [torch.empty(M, K, dtype=torch.bfloat16, device=b.dev) for _ in range(sets)]
    y_devs = [y] + [torch.empty_like(y) for _ in range(sets - 1)]
    y_hosts = [y_host] + [torch.empty_like(y_host).pin_memory() for _ in range(sets - 1)]
    step_no = [0]

    def e2e_step():
        # buffers are reused only in stream order, so steps are NOT joined in between: the next step's
        # host->device copies run while this step's results are still going device->host (full-duplex PCIe)
        k = step_no[0]
        step_no[0] += 1
        for c in range(chunks):
            lo, hi = c * rows, min(M, (c + 1) * rows)
            slot = k % sets
            with torch.cuda.stream(streams[(c if chunks > 1 else k) % len(streams)]):
                x_devs[slot][lo:hi].copy_(x_host[lo:hi], non_blocking=True)
                mb.gemm_swiglu_out(x_devs[slot][lo:hi], w, out=y_devs[slot][lo:hi], **knobs)
                y_hosts[slot][lo:hi].copy_(y_devs[slot][lo:hi], non_blocking=True)

    how = (f"every step: pinned X -> device, op, Y -> pinned host; {chunks} row chunk(s) per step on 3 side streams, "
           f"consecutive steps pipelined (no join between steps), time = whole run / steps; no L2 flush here (W is larger "
           f"than L2, at most its last 126 MB can be re-used by the next step)")
    return e2e_step, streams, x_host.numel() * 2, y_host.numel() * 2, how, (x_host, y_host)


def e2e_multi_gpu(b, mb, x_cpu, w, y, knobs):
    """N > 1: each rank uploads only ITS M/N rows of X from pinned host memory, the ranks all-gather X over NVLink
    (NCCL), run the op on their column shard and copy their shard of Y back to pinned host memory."""
    M, K = x_cpu.shape
    n_local = w.shape[0] // 2
    per = M // b.world
    x_host = x_cpu[b.rank * per:(b.rank + 1) * per].contiguous().pin_memory()
    sets = 3
    streams = [torch.cuda.Stream(b.dev) for _ in range(sets)]
    x_parts = [torch.empty(per, K, dtype=torch.bfloat16, device=b.dev) for _ in range(sets)]
    x_fulls = [torch.empty(M, K, dtype=torch.bfloat16, device=b.dev) for _ in range(sets)]
    y_devs = [y] + [torch.empty_like(y) for _ in range(sets - 1)]
    y_hosts = [torch.empty(M, n_local, dtype=torch.bfloat16).pin_memory() for _ in range(sets)]
    step_no = [0]

    def e2e_step():
        k = step_no[0] % sets
        step_no[0] += 1
        with torch.cuda.stream(streams[k]):
            x_parts[k].copy_(x_host, non_blocking=True)
            b.dist.all_gather_into_tensor(x_fulls[k], x_parts[k])
            mb.gemm_swiglu_out(x_fulls[k], w, out=y_devs[k], **knobs)
            y_hosts[k].copy_(y_devs[k], non_blocking=True)

    how = (f"every step and rank: pinned X rows [{per} of {M}] -> device, all-gather of X over NVLink (NCCL), op on the "
           f"rank's column shard, Y shard -> pinned host; 3 buffer sets on 3 side streams, consecutive steps pipelined, "
           f"time = whole run / steps, max over ranks; bytes are per rank")
    return e2e_step, streams, x_host.numel() * 2, y_hosts[0].numel() * 2, how, (x_host, y_hosts[0])


def copy_rates(b, host_in, dev_out_like, host_out):
    """Pinned-host <-> device copy rates on this rank alone (CUDA events around ten copies each way)."""
    dev_in = torch.empty(host_in.shape, dtype=host_in.dtype, device=b.dev)
    res = {}
    for name, dst, src in (("h2d", dev_in, host_in), ("d2h", host_out, dev_out_like)):
        dst.copy_(src, non_blocking=True)
        torch.cuda.synchronize(b.dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b.barrier()
        e0.record()
        for _ in range(10):
            dst.copy_(src, non_blocking=True)
        e1.record()
        torch.cuda.synchronize(b.dev)
        ms = b.reduce(e0.elapsed_time(e1) / 10)
        res[name + "_ms"] = ms
        res[name + "_gbs_per_rank"] = src.numel() * src.element_size() / (ms * 1e-3) / 1e9
    return res


def run_single_kernel(b, mb, args):
    """--only: one of the library's other kernels by itself, for launch lists and counter captures."""
    dev = b.dev
    g = torch.Generator(device=dev)
    g.manual_seed(0)

    def rnd(r, c, scale):
        return (torch.randn(r, c, generator=g, device=dev) * scale).to(torch.bfloat16)

    if args.only == "gemm_nt":       # down projection of the MLP block on one GPU: [16384, 28672] x [8192, 28672]^T
        a, w = rnd(16384, 28672, 1.0), rnd(8192, 28672, 0.02)
        out = torch.empty(16384, 8192, dtype=torch.bfloat16, device=dev)
        fn, flops, nbytes = (lambda: mb.gemm_nt_out(a, w, out=out)), 2.0 * 16384 * 28672 * 8192, None
    elif args.only == "backward_dh":  # recomputing backward of the op, Llama-3-8B FFN shape: dH from x, W and dY
        M, K, N = WORKLOADS["llama3_8b_ffn"][:3]
        x, w, dy = rnd(M, K, 1.0), rnd(2 * N, K, 0.02), rnd(M, N, 1.0)
        fn, flops, nbytes = (lambda: mb.swiglu_backward_dh(x, w, dy)), flops_of(M, K, N), None
    elif args.only == "scatter":      # the 8-GPU rank's down projection with its row blocks scattered to eight buffers
        from magicompiler_b200 import ops  # (all on this GPU here) + the slot sum that finishes the reduce-scatter
        a, w = rnd(16384, 3584, 1.0), rnd(8192, 3584, 0.02)
        recv = torch.empty(8, 2048, 8192, dtype=torch.bfloat16, device=dev)
        out = torch.empty(2048, 8192, dtype=torch.bfloat16, device=dev)
        ops.scatter_setup(0, [recv[o].data_ptr() for o in range(8)], 2048, 8192)

        def fn():
            ops.gemm_nt_scatter(a, w, 0)
            ops.sum_slots(recv, out)

        flops, nbytes = 2.0 * 16384 * 3584 * 8192, None
    else:                             # 1/8 column shard of the decode weight, M = 64: split-K tile kernel + ordered reduce
        M, K, N = 64, 8192, 3584
        x, w = rnd(M, K, 1.0), rnd(2 * N, K, 0.02)
        out = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        fn, flops, nbytes = (lambda: mb.gemm_swiglu_out(x, w, out=out)), None, bytes_of(M, K, N)
    ms, per_step, _ = b.time_steps(fn, args.steps, args.warmup)
    b.check_status(mb)
    line = {"only": args.only, "ms_per_step": ms, "ms_median": statistics.median(per_step), "steps": args.steps}
    if flops:
        line["tflops"] = flops / (ms * 1e-3) / 1e12
    if nbytes:
        line["gbs"] = nbytes / (ms * 1e-3) / 1e9
    print(json.dumps(line), flush=True)


def bind_to_gpu_numa_node(local_rank):
    """N > 1: run this rank on the CPU cores next to its GPU (read from NVML, nothing is set on the GPU), so that the
    pinned host buffers of the end-to-end leg are allocated on that NUMA node and the copies do not cross sockets.
    Returns a short description for the JSON line."""
    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
        ncpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (ncpu + 63) // 64)
        near = {i for i in range(ncpu) if (words[i // 64] >> (i % 64)) & 1}
        allowed = os.sched_getaffinity(0)
        cpus = sorted(near & allowed)
        if not cpus or len(cpus) == len(allowed):
            return f"not bound ({len(near)} cores next to the GPU, {len(allowed)} allowed)"
        os.sched_setaffinity(0, cpus)
        return f"bound to the {len(cpus)} cores next to the GPU ({cpus[0]}..{cpus[-1]})"
    except Exception as exc:  # no NVML, no such call, not permitted: stay where we are
        return f"not bound ({type(exc).__name__})"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="llama3_8b_ffn", choices=sorted(WORKLOADS))
    ap.add_argument("--variant", default="auto")
    ap.add_argument("--block-n", type=int, default=0)
    ap.add_argument("--stages", type=int, default=0)
    ap.add_argument("--group-m", type=int, default=0)
    ap.add_argument("--chunks", type=int, default=4, help="mlp_block: row chunks whose reduction overlaps the next chunk")
    ap.add_argument("--reduce", default="all_reduce", choices=["all_reduce", "reduce_scatter", "peer_scatter", "peer_all_reduce"],
                    help="mlp_block: all ranks get the whole result, or each keeps its rows of the sum")
    ap.add_argument("--down", default="own", choices=["own", "library"], help="mlp_block: kernel of the down projection")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-incumbents", action="store_true", help="skip timing eager CUDA, the library GEMM and torch.compile")
    ap.add_argument("--no-sub-workloads", action="store_true", help="headline workload only (profiling runs)")
    ap.add_argument("--train", action="store_true",
                    help="also time forward + backward of the op (both autograd forms) against the eager expression")
    ap.add_argument("--no-flush", action="store_true", help="profiling runs only: skip the L2 flush kernels")
    ap.add_argument("--no-numa-bind", action="store_true",
                    help="N > 1: leave the rank on whatever cores it was started on (default: the cores next to its GPU)")
    ap.add_argument("--no-peer-scatter", action="store_true",
                    help="N > 1: skip the MLP block variant whose down projection stores into the other GPUs' memory")
    ap.add_argument("--only", default=None, choices=["gemm_nt", "backward_dh", "decode_shard", "scatter"],
                    help="profiling runs only: time one of the other kernels of the library by itself (1 GPU) and print a "
                         "short JSON line: the down projection of the MLP block (gemm_nt), the recomputing backward "
                         "(backward_dh, Llama shape), a 1/8 decode column shard (split-K tile kernel + ordered reduce), or "
                         "the scattered down projection of an 8-GPU rank + its slot sum with all eight buffers local (scatter)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" and not args.no_flush else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N > 1")

    import torch.distributed as dist

    import magicompiler_b200 as mb

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    cpu_binding = bind_to_gpu_numa_node(local_rank) if world > 1 and not args.no_numa_bind else "not bound"
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    lib = mb.load_library()  # raises if the CUDA library is missing: there is no fallback
    if lib.magi_swiglu_supported(local_rank) != 1:
        raise SystemExit("this benchmark needs a B200 (sm_100)")
    b = Bench(args, rank, world, local_rank)
    sub_steps = max(5, min(args.steps, 20))
    sub_warmup = max(3, min(args.warmup, 5))

    if args.only:
        run_single_kernel(b, mb, args)
        return
    if args.workload == "mlp_block":  # the MLP block alone, as the line's headline
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        rec = run_mlp_block(b, mb, args.steps, args.warmup,
                            1 if args.reduce in ("peer_scatter", "peer_all_reduce") else args.chunks, args.reduce, args.down)
        clocks = sampler.stop() if rank == 0 else None
        if rank == 0:
            M, K, N, _, desc = WORKLOADS["mlp_block"]
            print(json.dumps({
                "metric": f"SwiGLU MLP block TFLOP/s (fused gate/up + down projection + {args.reduce.replace('_', '-')})",
                "value": rec["value"], "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic (CUDA generator seed 0, X~N(0,1), W~N(0,0.02), bf16)",
                "config": {"workload": "mlp_block", "shape": desc, "chunks": args.chunks, "M": M, "K": K, "N": N,
                           "parallelism": rec["parallelism"], "l2": rec["l2"]},
                "roofline": rec["roofline"], "gpu_launches": rec["gpu_launches"], "parity": rec["parity"],
                "clocks": clocks, "detail": rec}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        if not rec["parity"]["ok"]:
            raise SystemExit(3)
        return

    M, K, N, bound, desc = WORKLOADS[args.workload]
    x_cpu, w_cpu = make_inputs_cpu(M, K, N, seed=0)
    w_local_cpu = mb.shard_gate_up(w_cpu, rank, world) if world > 1 else w_cpu
    x = x_cpu.to(dev)
    w = w_local_cpu.to(dev)
    knobs = dict(variant=args.variant, block_n=args.block_n, stages=args.stages, group_m=args.group_m)

    # ---------------------------------------------------------------- device-resident timing of the headline workload
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    head, y, step, plan, step_ms, wall, kclk = time_op_workload(b, mb, args.workload, x, w, args.steps, args.warmup, knobs)
    n_local = w.shape[0] // 2
    ms_per_step = head["ms_per_step"]
    clocks = sampler.stop() if rank == 0 else None  # the samples cover the headline workload's timed region only

    # ---------------------------------------------------------------- the paths this op replaces, same GPU, same state
    incumbents, training = None, None
    if world == 1 and not args.no_incumbents:
        # timed right after the headline loop, each the same way (L2 flush, CUDA events, median of 10): the reference's
        # eager expression (two library GEMMs + silu + mul), what torch.compile (Inductor) makes of it (two library
        # GEMMs + one generated element-wise kernel; this is what the reference's compiler emits for the path) and one
        # library GEMM [M,K]x[K,2N] alone
        import torch.nn.functional as F

        flops_h, nbytes_h = flops_of(M, K, N), bytes_of(M, K, N)
        unit_h = "GB/s" if bound == "hbm" else "TFLOP/s"

        def as_metric(ms):
            return (nbytes_h / 1e9 if bound == "hbm" else flops_h / 1e12) / (ms * 1e-3)

        def eager(a, bb):
            return F.silu(F.linear(a, bb[:N])) * F.linear(a, bb[N:])

        time.sleep(SETTLE_S)
        t_ours = b.timed_median(step)  # the fused op timed exactly like the others (a burst of 10, not the long loop)
        t_gemm = b.timed_median(lambda: F.linear(x, w))
        t_eager = b.timed_median(lambda: eager(x, w))
        incumbents = {
            "fused_same_method": {"ms": t_ours, "value": as_metric(t_ours), "unit": unit_h,
                                  "what": "this op, median of 10 like the incumbents below"},
            "eager_cuda": {"ms": t_eager, "value": as_metric(t_eager), "unit": unit_h,
                           "what": "F.silu(F.linear(x,Wg))*F.linear(x,Wu): 2 library GEMMs + 2 element-wise kernels"},
            "library_gemm_only": {"ms": t_gemm, "value": as_metric(t_gemm), "unit": unit_h,
                                  "what": "F.linear(x, W[2N,K]) alone, no activation"}}
        try:
            compiled = torch.compile(eager)
            with torch.no_grad():
                t_comp = b.timed_median(lambda: compiled(x, w))
            incumbents["torch_compile"] = {
                "ms": t_comp, "value": as_metric(t_comp), "unit": unit_h,
                "what": "torch.compile (Inductor) of the eager expression: 2 library GEMMs + 1 generated kernel"}
        except Exception as exc:  # a box without a working Inductor tool chain still gives the other figures
            incumbents["torch_compile"] = {"unavailable": repr(exc)[:200]}
        if args.train:
            # forward + backward of the op alone (dY given), 3 x the forward FLOPs of useful work
            dy = torch.randn(M, N, device=dev, dtype=torch.float32).to(torch.bfloat16)
            xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)

            def fwd_bwd(fn):
                def run():
                    xr.grad = None
                    wr.grad = None
                    fn(xr, wr).backward(dy)
                return run

            t_rec = b.timed_median(fwd_bwd(mb.gemm_swiglu))
            t_keep = b.timed_median(fwd_bwd(mb.gemm_swiglu_train))
            t_eag = b.timed_median(fwd_bwd(eager))
            training = {
                "unit": "ms per forward+backward", "flops": 3 * flops_h,
                "gemm_swiglu_recompute": {"ms": t_rec, "tflops": 3 * flops_h / (t_rec * 1e-3) / 1e12},
                "gemm_swiglu_train_kept_preactivations": {"ms": t_keep, "tflops": 3 * flops_h / (t_keep * 1e-3) / 1e12},
                "eager_cuda": {"ms": t_eag, "tflops": 3 * flops_h / (t_eag * 1e-3) / 1e12}}
            del dy, xr, wr

    # ---------------------------------------------------------------- end to end from host buffers
    e2e = None
    if not args.no_e2e:
        if world == 1 or M % world != 0:
            e2e_step, streams, h2d, d2h, how, bufs = e2e_single_gpu(b, mb, x_cpu, w, y, knobs, args.steps)
        else:
            e2e_step, streams, h2d, d2h, how, bufs = e2e_multi_gpu(b, mb, x_cpu, w, y, knobs)
        cur = torch.cuda.current_stream(dev)
        n_e2e = max(3, min(args.steps, 20))
        for s in streams:
            s.wait_stream(cur)
        for _ in range(3):
            e2e_step()
        for s in streams:
            cur.wait_stream(s)
        b.barrier()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in streams:
            s.wait_stream(cur)
        for _ in range(n_e2e):
            e2e_step()
        for s in streams:
            cur.wait_stream(s)
        e1.record()
        b.barrier()
        e2e_ms = b.reduce(e0.elapsed_time(e1) / n_e2e)
        rates = copy_rates(b, bufs[0], y, bufs[1])
        e2e = (e2e_ms, h2d, d2h, how, rates)

    # ---------------------------------------------------------------- the other benchmark configurations
    subs = {}
    if not args.no_sub_workloads and args.workload == "llama3_8b_ffn":
        del x, w
        for name in SUB_WORKLOADS:
            torch.cuda.synchronize(dev)
            time.sleep(SETTLE_S)
            if name == "mlp_block":
                nccl = run_mlp_block(b, mb, sub_steps, sub_warmup, args.chunks if world > 1 else 1, args.reduce, args.down)
                subs[name] = nccl
                if world > 1:
                    short = ("ms_per_step", "ms_median", "ms_min", "value", "unit", "chunks", "reduce", "parallelism", "parity")
                    # the same block with each rank keeping only its rows of the sum (half the link bytes)
                    alt = run_mlp_block(b, mb, sub_steps, sub_warmup, 1, "reduce_scatter", args.down)
                    extra = {"reduce_scatter": {k: alt[k] for k in short}}
                    if not args.no_peer_scatter:  # ... and with the reduction fused into the down projection's epilogue
                        try:
                            alt = run_mlp_block(b, mb, sub_steps, sub_warmup, 1, "peer_scatter", "own")
                            extra["peer_scatter"] = {k: alt[k] for k in short}
                            fused = run_mlp_block(b, mb, sub_steps, sub_warmup, 1, "peer_all_reduce", "own")
                            # The block's record is the fused all-reduce (every rank ends with the whole result, the
                            # contract of the reference's row-parallel linear); NCCL's all-reduce is kept beside it.
                            extra["nccl_all_reduce"] = {k: nccl[k] for k in short}
                            subs[name] = fused
                        except (RuntimeError, ValueError, ImportError) as exc:  # e.g. no symmetric memory on this machine
                            extra["peer_unavailable"] = f"{type(exc).__name__}: {str(exc)[:200]}"
                    subs[name].update(extra)
                continue
            sM, sK, sN, _, _ = WORKLOADS[name]
            xs, ws = make_inputs_cuda(sM, sK, sN, dev, seed=0)
            if world > 1:
                ws = mb.shard_gate_up(ws, rank, world)
            subs[name] = time_op_workload(b, mb, name, xs, ws, sub_steps, sub_warmup)[0]
            del xs, ws
    ok = head["parity"]["ok"] and all(
        r["parity"]["ok"] and all(r.get(k, {}).get("parity", {}).get("ok", True)
                                  for k in ("reduce_scatter", "peer_scatter", "nccl_all_reduce")) for r in subs.values())

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        if not ok:
            raise SystemExit(3)
        return

    flops, nbytes = flops_of(M, K, N), bytes_of(M, K, N)
    if bound == "hbm":
        metric, unit, e2e_scale = "fused GEMM-SwiGLU HBM GB/s (small-M)", "GB/s", nbytes / 1e9
    else:
        metric, unit, e2e_scale = "fused GEMM-SwiGLU TFLOP/s", "TFLOP/s", flops / 1e12

    line = {
        "metric": metric, "value": head["value"], "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic (X~N(0,1), W~N(0,0.02), bf16; headline: CPU generator seed 0; sub-workloads: CUDA generator seed 0)",
        "config": config_of(args.workload, world),
        "detail": {"n_per_gpu": n_local, "plan": plan, "wall_s_timed_region": wall, "ms_median": head["ms_median"],
                   "ms_min": head["ms_min"]},
        "roofline": head["roofline"],
        # one tile kernel per step, plus the ordered-reduce kernel when the plan splits K
        "gpu_launches": head["gpu_launches"],
        "parity": head["parity"],
        "clocks": clocks,
    }
    if clocks is not None:
        # nvidia-smi samples every 50 ms and mostly sees the gaps between millisecond kernels; the kernel's own
        # cycle counter / wall timer ratio is the clock it really ran at (lower under the power cap)
        line["clocks"]["kernel_sm_mhz"] = kclk["sm_mhz"]
    if "cuda_graph" in head:
        line["cuda_graph"] = head["cuda_graph"]
    if e2e is not None:
        ms, h2d, d2h, how, rates = e2e
        line["e2e"] = {"value": e2e_scale / (ms * 1e-3), "unit": unit, "h2d_bytes_per_step": h2d,
                       "d2h_bytes_per_step": d2h, "ms_per_step": ms, "how": how, "copies_alone": rates,
                       "cpu_binding_rank0": cpu_binding}
    if subs:
        line["workloads"] = subs
    if incumbents is not None:
        line["incumbents"] = incumbents
    if training is not None:
        line["training"] = training
    if world == 1 and not args.no_cpu_baseline:
        rows, threads, t, reps = cpu_eager(M, K, N, x_cpu, w_cpu)
        v = bytes_of(rows, K, N) / t / 1e9 if bound == "hbm" else flops_of(rows, K, N) / t / 1e12
        line["cpu_baseline"] = {
            "value": v, "unit": unit, "cores": threads, "kind": "port",
            "sample": f"reference eager expression (torch CPU, bf16) on the first {rows} of {M} rows with the full W, "
                      f"median of {reps} runs of {t:.2f} s"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if not ok:
        raise SystemExit(3)


if __name__ == "__main__":
    main()
