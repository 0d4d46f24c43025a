#!/usr/bin/env python
"""Benchmark of the fused GEMM-SwiGLU path:  python bench.py --gpus N --steps K --warmup W [--impl reference]

A step is one pass of the op over one batch of synthetic input (CPU generator, seed 0, X ~ N(0,1),
W ~ N(0,0.02), bf16).  Default workload: the Llama-3-8B-shaped FFN up-projection, X[8192,4096] x
W[2*14336,4096] -> Y[8192,14336].  On N > 1 GPUs the packed weight is column-sharded along N (rank r
owns N/P gate and N/P up rows), X is replicated and no collective is on the data path; the job's work is
the whole problem, so scaling is "strong".

Timing: W warm-up steps, then exactly K steps, each bracketed by its own pair of CUDA events on the launch
stream with an L2 flush (256 MiB written, then 256 MiB read, so no dirty lines remain) before it; a barrier and a device synchronise surround the timed
region; the per-rank sum of the K step times is reduced with MAX over ranks.  SM clocks and throttle
reasons are sampled with nvidia-smi (read-only) while the steps run.

One JSON line is printed by rank 0.  `value` is device-resident throughput; `e2e` is the same metric with
the step's X copied from pinned host memory and its Y copied back inside the timed region; `roofline`
describes the kernel against the measured peak of this GPU pool; `cpu_baseline` times the reference's eager
PyTorch expression on the host cores on a bounded slice of the same workload.
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
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the ncu captures
# summarised under profiles/ (bytes; key = workload@gpus).
NCU_TRAFFIC = {
    "llama3_8b_ffn@1": 978.2e6,   # profiles/swiglu_tc_kernel_pair_llama3_8b_ffn.md
    "video_dit_ffn@1": 8377.7e6,
    "decode_m64@1": 946.7e6,     # profiles/swiglu_tc_kernel_stream_decode_m64.md
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
L2_FLUSH_BYTES = 256 << 20


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


def cpu_eager_tflops(M, K, N, x, w, target_s=12.0, max_rows=None):
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
    rows2 = int(min(max_rows or M, M, max(rows, rows * (target_s / 3.0) / dt)))
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
    return flops_of(rows2, K, N) / t / 1e12, rows2, threads, t, len(times)


def run_reference_arm(args, rank, world):
    """--impl reference: MagiCompiler's eager SwiGLU on the host CPU (its only implementation of this path)."""
    if rank != 0:
        return
    from oracle import make_inputs, swiglu_ref_eager

    M, K, N, bound, desc = WORKLOADS[args.workload]
    x, w = make_inputs(M, K, N, seed=0)
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
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seed 0, X~N(0,1), W~N(0,0.02))",
        "config": {"workload": args.workload, "shape": desc, "rows_per_step": rows},
        "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_mlp_block(args, rank, world, local_rank):
    """Config 5: gate/up column-parallel through the fused op, down projection row-parallel (library GEMM), one
    all-reduce over NVLink, optionally chunked so the reduce of chunk i overlaps the GEMMs of chunk i+1."""
    import torch.distributed as dist

    import magicompiler_b200 as mb
    from oracle import make_inputs

    dev = torch.device("cuda", local_rank)
    M, K, N, _, desc = WORKLOADS["mlp_block"]
    x_cpu, w_cpu, wd_cpu = make_inputs(M, K, N, seed=0, with_down=True)
    mlp = mb.TensorParallelSwiGLUMLP(w_cpu, wd_cpu, rank, world, chunks=args.chunks, reduce=args.reduce,
                                     down_fn=mb.gemm_nt_out if args.down == "own" else None).to(dev)
    del w_cpu, wd_cpu
    x = x_cpu.to(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(args.warmup):
        mlp(x)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        out = mlp(x)
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    status = mb.device_status(local_rank)
    if status["code"] != 0:
        raise SystemExit(f"kernel watchdog fired: {status}")
    if rank == 0:
        flops = 2.0 * M * K * 2 * N + 2.0 * M * N * K
        peaks, kind = measured_peaks()
        value = flops / (ms * 1e-3) / 1e12
        per_gpu = value / world
        print(json.dumps({
            "metric": f"SwiGLU MLP block TFLOP/s (fused gate/up + down projection + {args.reduce.replace('_', '-')})",
            "value": value,
            "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (CPU generator seed 0, X~N(0,1), W~N(0,0.02), bf16)",
            "config": {"workload": "mlp_block", "shape": desc, "chunks": args.chunks,
                       "down_projection": "magi_swiglu_gemm_nt_bf16 (own tile kernel)" if args.down == "own"
                       else "torch.matmul (library GEMM)",
                       "parallelism": f"tp{world}: column-parallel gate/up, row-parallel down, NCCL "
                                      f"{args.reduce.replace('_', '-')} of [{M},{K}] bf16", "l2": "inputs (1.7 GB) larger than L2, back-to-back steps"},
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": float(peaks["bf16_tflops_sustained"]),
                         "unit": "TFLOP/s", "frac": per_gpu / float(peaks["bf16_tflops_sustained"]), "traffic": None,
                         "peak_kind": f"{kind} cuBLAS bf16 sustained (kernels timed inside a long step)"},
            "gpu_launches": args.steps * args.chunks * (2 if args.down == "own" else 1)}), flush=True)
    if world > 1:
        dist.destroy_process_group()


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
    ap.add_argument("--chunks", type=int, default=1, help="mlp_block: row chunks whose all-reduce overlaps the next chunk")
    ap.add_argument("--reduce", default="all_reduce", choices=["all_reduce", "reduce_scatter"],
                    help="mlp_block: all ranks get the whole result, or each keeps its rows of the sum")
    ap.add_argument("--down", default="own", choices=["own", "library"], help="mlp_block: kernel of the down projection")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-incumbents", action="store_true", help="skip timing eager CUDA and the library GEMM")
    ap.add_argument("--compiled-incumbent", action="store_true",
                    help="also time torch.compile (Inductor) of the eager expression: 2 library GEMMs + 1 generated kernel")
    ap.add_argument("--train", action="store_true",
                    help="also time forward + backward of the op (both autograd forms) against the eager expression")
    ap.add_argument("--no-flush", action="store_true", help="profiling runs only: skip the L2 flush kernels")
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
    from oracle import make_inputs  # input generator only; the oracle's compute is used for cpu_baseline alone

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    lib = mb.load_library()  # raises if the CUDA library is missing: there is no fallback
    if lib.magi_swiglu_supported(local_rank) != 1:
        raise SystemExit("this benchmark needs a B200 (sm_100)")

    if args.workload == "mlp_block":
        run_mlp_block(args, rank, world, local_rank)
        return
    M, K, N, bound, desc = WORKLOADS[args.workload]
    x_cpu, w_cpu = make_inputs(M, K, N, seed=0)
    w_local_cpu = mb.shard_gate_up(w_cpu, rank, world) if world > 1 else w_cpu
    n_local = w_local_cpu.shape[0] // 2
    x = x_cpu.to(dev)
    w = w_local_cpu.to(dev)
    y = torch.empty(M, n_local, dtype=torch.bfloat16, device=dev)
    flush_w = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
    flush_r = torch.zeros(L2_FLUSH_BYTES // 4, dtype=torch.int32, device=dev)

    def flush_l2():
        # write a buffer larger than L2, then read another one: the timed kernel starts from an L2 that holds
        # neither its inputs nor dirty lines whose write-back would be charged to it
        flush_w.zero_()
        flush_r.max()
    knobs = dict(variant=args.variant, block_n=args.block_n, stages=args.stages, group_m=args.group_m)
    plan = mb.plan(M, n_local, K, device=local_rank, **knobs)

    def step():
        mb.gemm_swiglu_out(x, w, out=y, **knobs)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---------------------------------------------------------------- device-resident timing
    for _ in range(args.warmup):
        if not args.no_flush:
            flush_l2()
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    wall0 = time.perf_counter()
    for i in range(args.steps):
        if not args.no_flush:
            flush_l2()
        starts[i].record()
        step()
        ends[i].record()
    barrier()
    wall = time.perf_counter() - wall0
    step_ms = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    total_ms = torch.tensor([sum(step_ms)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
    total_ms = float(total_ms.item())
    ms_per_step = total_ms / args.steps
    kclk = mb.kernel_clock(local_rank)  # SM clock of the last timed kernel, measured inside the kernel
    status = mb.device_status(local_rank)
    if status["code"] != 0:
        raise SystemExit(f"kernel watchdog fired: {status}")

    # ---------------------------------------------------------------- the same step replayed from a CUDA graph
    # (the small-M shapes run for 20-70 us: a replay takes the host's launch path out of the picture)
    graph_ms = None
    if bound == "hbm":
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream(dev).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        ts = []
        for _ in range(max(5, min(args.steps, 30))):
            if not args.no_flush:
                flush_l2()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record()
            graph.replay()
            g1.record()
            torch.cuda.synchronize(dev)
            ts.append(g0.elapsed_time(g1))
        gm = torch.tensor([statistics.median(ts)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(gm, op=dist.ReduceOp.MAX)
        graph_ms = float(gm.item())

    # ---------------------------------------------------------------- end to end from host buffers
    e2e = None
    if not args.no_e2e:
        x_host = x_cpu.pin_memory()
        y_host = torch.empty(M, n_local, dtype=torch.bfloat16).pin_memory()
        chunks = 8 if M >= 4096 else 1
        rows = -(-M // chunks)
        streams = [torch.cuda.Stream(dev) for _ in range(min(chunks, 3))]
        # Large M: chunk c of every step owns rows [lo, hi) of one set of buffers and always runs on stream c % 3.
        # Small M (one chunk): three complete buffer sets, step k uses set k % 3 on stream k % 3.
        sets = 1 if chunks > 1 else 3
        if chunks == 1:
            streams = [torch.cuda.Stream(dev) for _ in range(3)]
        x_devs = [torch.empty_like(x) for _ in range(sets)]
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

        def fork():
            cur = torch.cuda.current_stream(dev)
            for s in streams:
                s.wait_stream(cur)

        def join():
            cur = torch.cuda.current_stream(dev)
            for s in streams:
                cur.wait_stream(s)

        n_e2e = max(3, min(args.steps, 20))
        fork()
        for _ in range(2):
            e2e_step()
        join()
        barrier()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        fork()
        for _ in range(n_e2e):
            e2e_step()
        join()
        e1.record()
        barrier()
        e2e_ms = torch.tensor([e0.elapsed_time(e1) / n_e2e], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
        e2e = (float(e2e_ms.item()), x_host.numel() * 2, y_host.numel() * 2, chunks)
    clocks = sampler.stop() if rank == 0 else None

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks, peak_kind = measured_peaks()
    flops, nbytes = flops_of(M, K, N), bytes_of(M, K, N)
    flops_rank, bytes_rank = flops_of(M, K, n_local), bytes_of(M, K, n_local)
    rank0_ms = sum(step_ms) / args.steps
    if bound == "hbm":
        metric, unit = "fused GEMM-SwiGLU HBM GB/s (small-M)", "GB/s"
        value = nbytes / (ms_per_step * 1e-3) / 1e9
        achieved = bytes_rank / (rank0_ms * 1e-3) / 1e9
        peak = float(peaks["hbm_gbs"])
        roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": None, "peak_kind": f"{peak_kind} copy bandwidth", "nominal_frac": achieved / 8000.0}
        e2e_scale = nbytes
    else:
        metric, unit = "fused GEMM-SwiGLU TFLOP/s", "TFLOP/s"
        value = flops / (ms_per_step * 1e-3) / 1e12
        achieved = flops_rank / (rank0_ms * 1e-3) / 1e12
        peak = float(peaks["bf16_tflops"])
        roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "traffic": None, "peak_kind": f"{peak_kind} cuBLAS bf16 burst (kernel timed alone)",
                "nominal_frac": achieved / 2250.0}
        if peaks.get("bf16_tflops_sustained"):
            # the same library GEMM run back to back for seconds under the power cap: the fairer yardstick when
            # --steps is large enough for the cap to bite (the timed loop keeps the GPU busy for that long too)
            roof["peak_sustained"] = float(peaks["bf16_tflops_sustained"])
            roof["frac_of_sustained"] = achieved / float(peaks["bf16_tflops_sustained"])
        e2e_scale = flops
    roof["kernel"] = "swiglu_tc_kernel"
    roof["kernel_ms"] = rank0_ms
    roof["traffic"] = NCU_TRAFFIC.get(f"{args.workload}@{world}")
    roof["algorithmic_bytes"] = bytes_rank

    line = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (CPU generator seed 0, X~N(0,1), W~N(0,0.02), bf16)",
        "config": {"workload": args.workload, "shape": desc, "M": M, "K": K, "N": N, "n_per_gpu": n_local,
                   "parallelism": f"column-shard of W over {world} GPU(s), X replicated, no collective",
                   "l2": "flushed before every timed step (256 MiB written, then 256 MiB read)" if not args.no_flush else "not flushed",
                   "plan": plan, "wall_s_timed_region": wall},
        "roofline": roof,
        # one tile kernel per step, plus the ordered-reduce kernel when the plan splits K
        "gpu_launches": args.steps * (2 if plan.get("k_splits", 1) > 1 else 1),
        "clocks": clocks,
    }
    if clocks is not None:
        # nvidia-smi samples every 50 ms and mostly sees the gaps between millisecond kernels; the kernel's own
        # cycle counter / wall timer ratio is the clock it really ran at (lower under the power cap)
        line["clocks"]["kernel_sm_mhz"] = kclk["sm_mhz"]
        if bound == "tensor" and kclk["sm_mhz"] > 0:
            n_sm = torch.cuda.get_device_properties(dev).multi_processor_count
            line["roofline"]["tensor_pipe_frac_at_kernel_clock"] = achieved / (8192 * n_sm * kclk["sm_mhz"] * 1e6 / 1e12)
    if graph_ms is not None:
        line["cuda_graph"] = {"ms_per_step": graph_ms, "value": nbytes / (graph_ms * 1e-3) / 1e9, "unit": unit,
                              "how": "one captured op call replayed, L2 flushed before each replay, median"}
    if e2e is not None:
        ms, h2d, d2h, chunks = e2e
        line["e2e"] = {"value": e2e_scale / (ms * 1e-3) / (1e9 if bound == "hbm" else 1e12), "unit": unit,
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": ms,
                       "how": f"every step: pinned X -> device, op, Y -> pinned host; {chunks} row chunk(s) per step on 3 side "
                              f"streams, consecutive steps pipelined (no join between steps), time = whole run / steps; no L2 "
                              f"flush here (W is larger than L2, at most its last 126 MB can be re-used by the next step)"}
    if world == 1 and not args.no_incumbents:
        # the paths this op replaces on the same GPU, timed the same way (L2 flush, CUDA events, median of 10):
        # the reference's eager expression (two library GEMMs + silu + mul) and one library GEMM [M,K]x[K,2N] alone
        import torch.nn.functional as F

        def timed(fn):
            for _ in range(3):
                fn()
            ts = []
            for _ in range(10):
                if not args.no_flush:
                    flush_l2()
                s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s0.record()
                fn()
                s1.record()
                torch.cuda.synchronize(dev)
                ts.append(s0.elapsed_time(s1))
            return statistics.median(ts)

        def as_metric(ms):
            return (nbytes if bound == "hbm" else flops) / (ms * 1e-3) / (1e9 if bound == "hbm" else 1e12)

        t_eager = timed(lambda: F.silu(F.linear(x, w[:N])) * F.linear(x, w[N:]))
        t_gemm = timed(lambda: F.linear(x, w))
        t_ours = timed(step)  # the fused op timed exactly like the two above (a burst of 10, not the long loop)
        line["incumbents"] = {
            "fused_same_method": {"ms": t_ours, "value": as_metric(t_ours), "unit": unit,
                                  "what": "this op, median of 10 like the incumbents below"},
            "eager_cuda": {"ms": t_eager, "value": as_metric(t_eager), "unit": unit,
                           "what": "F.silu(F.linear(x,Wg))*F.linear(x,Wu): 2 library GEMMs + 2 element-wise kernels"},
            "library_gemm_only": {"ms": t_gemm, "value": as_metric(t_gemm), "unit": unit,
                                  "what": "F.linear(x, W[2N,K]) alone, no activation"}}
        if args.compiled_incumbent:
            compiled = torch.compile(lambda a, b: F.silu(F.linear(a, b[:N])) * F.linear(a, b[N:]))
            with torch.no_grad():
                t_comp = timed(lambda: compiled(x, w))
            line["incumbents"]["torch_compile"] = {
                "ms": t_comp, "value": as_metric(t_comp), "unit": unit,
                "what": "torch.compile (Inductor) of the eager expression: 2 library GEMMs + 1 generated kernel"}
        if args.train:
            # forward + backward of the op alone (dY given), 3 x the forward FLOPs of useful work
            dy = torch.randn(M, N, device=dev, dtype=torch.float32).to(torch.bfloat16)
            xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)

            def step(fn):
                def run():
                    xr.grad = None
                    wr.grad = None
                    fn(xr, wr).backward(dy)
                return run

            t_rec = timed(step(mb.gemm_swiglu))
            t_keep = timed(step(mb.gemm_swiglu_train))
            t_eag = timed(step(lambda a, b: F.silu(F.linear(a, b[:N])) * F.linear(a, b[N:])))
            line["training"] = {
                "unit": "ms per forward+backward", "flops": 3 * flops,
                "gemm_swiglu_recompute": {"ms": t_rec, "tflops": 3 * flops / (t_rec * 1e-3) / 1e12},
                "gemm_swiglu_train_kept_preactivations": {"ms": t_keep, "tflops": 3 * flops / (t_keep * 1e-3) / 1e12},
                "eager_cuda": {"ms": t_eag, "tflops": 3 * flops / (t_eag * 1e-3) / 1e12}}
    if world == 1 and not args.no_cpu_baseline:
        v, rows, threads, t, reps = cpu_eager_tflops(M, K, N, x_cpu, w_cpu)
        if bound == "hbm":
            v = bytes_of(rows, K, N) / t / 1e9
        line["cpu_baseline"] = {
            "value": v, "unit": unit, "cores": threads, "kind": "port",
            "sample": f"reference eager expression (torch CPU, bf16) on the first {rows} of {M} rows with the full W, "
                      f"median of {reps} runs of {t:.2f} s"}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
