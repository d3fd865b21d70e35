#!/usr/bin/env python
"""Benchmark of the MXFP8 hot path on B200: quantize GB/s (headline line) and block-scaled GEMM
TFLOP/s (the "gemm" object of the same line), with roofline fractions, clocks, an end-to-end
number through host buffers and the CPU port of the reference's torch code timed beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl mx8|reference] [--workload quantize|gemm|ffn|moe]

One JSON line on stdout (rank 0).  Under torchrun every rank works on its own shard; there is no
data-path collective, only the barrier and the max-over-ranks reduction of the timing.

Workloads (synthetic, seeded; stand-ins with the shapes and value distributions the benchmark
configurations name):
  quantize  bf16 16384 x 16384 ~ N(0,1), 0.1 % of entries x1000, one all-zero 1x32 block per 1024
            rows; row-wise and transposed E4M3 + E8M0 (tcgen05 scale layout).  Each rank quantizes
            its own matrix (weak scaling).
  gemm      M = N = K = 8192, operands quantized from bf16 ~ N(0, 1/sqrt(K)), bf16 output.  With N
            GPUs the rows of A and C are split M/N per rank, B replicated (strong scaling).
  ffn       X [16384 x 8192] -> quantize -> GEMM with an MXFP8-quantizing epilogue -> GEMM; tokens split.
  moe       the MoE layer (256 experts, hidden 7168, intermediate 2048, 32768 tokens, top-8): forward as one
            launch sequence and in minibatches on three streams, and backward, over peer-mapped memory;
            experts and tokens split across the GPUs.
The quantize line carries the other three as objects ("gemm", "ffn", "moe") unless --no-gemm / --no-layers.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "gpu-experiments_b200"))

import torch  # noqa: E402

QM = QN = 16384
LAYER_STEPS = 20            # timed steps of the FFN and MoE objects, whatever --steps says
E2E_BAND_ROWS = 2048          # rows per band of the host-buffer (end-to-end) pipeline
GM = GN = GK = 8192
L2_BYTES = 126 * 1024 * 1024

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures
# summarised under profiles/; None until a capture exists for that kernel.
NCU_TRAFFIC_BYTES = {"quantize_16384x16384_both": 1045880000, "gemm_8192": 370370000}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


_fp8_roof = {}


def measure_fp8_roof(local):
    """Tensor-core roof for the MXFP8 GEMM, measured on this GPU right now: the kernel's own MMA instruction issued
    back to back from shared memory by every CTA pair (mx8_probe_mma_peak), three launches of about a millisecond
    after an idle moment, i.e. at the clock a short burst gets.  Cached per device."""
    if local in _fp8_roof:
        return _fp8_roof[local]
    import ctypes
    import mx8
    lib = mx8.load()
    st = torch.cuda.current_stream().cuda_stream
    fl = ctypes.c_double()
    k_steps = 4096
    for _ in range(2):
        mx8._lib.check(lib.mx8_probe_mma_peak(k_steps, ctypes.byref(fl), st), "mx8_probe_mma_peak")
    torch.cuda.synchronize()
    time.sleep(0.3)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        lib.mx8_probe_mma_peak(k_steps, ctypes.byref(fl), st)
    e1.record()
    torch.cuda.synchronize()
    mx8.device_status()
    _fp8_roof[local] = {"tflops": 3 * fl.value / (e0.elapsed_time(e1) * 1e-3) / 1e12,
                        "source": "measured on this GPU in this run: tcgen05.mma kind::mxf8f6f4.block_scale 256x256x32 issued back to "
                                  "back from shared memory by all CTA pairs (mx8_probe_mma_peak), 3 launches of ~1 ms"}
    time.sleep(0.3)
    return _fp8_roof[local]


def tensor_roofline(achieved, local, clocks=None, **extra):
    roof = measure_fp8_roof(local)
    r = {"bound": "tensor", "achieved": achieved, "peak": roof["tflops"], "unit": "TFLOP/s", "frac": achieved / roof["tflops"],
         "peak_source": roof["source"], "frac_of_nominal_4500": achieved / 4500.0}
    if clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz"):
        # what the same cycle count would give at the maximum SM clock (the power cap lowers the clock inside long runs)
        r["achieved_at_max_clock"] = achieved * clocks["sm_max_mhz"] / clocks["sm_mhz"]
        r["median_sm_mhz"] = clocks["sm_mhz"]
    r.update(extra)
    return r


class ClockSampler:
    """Polls SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = get_reasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self.nv:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def dist_setup(n_gpus):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    return world, rank, local


def barrier(world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(ms, world):
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return ms


def timed(fn, steps, world, sampler=None):
    """K calls of fn(i) between two CUDA events on the current stream; barrier + synchronize on
    both sides; returns the max over ranks of the elapsed milliseconds."""
    barrier(world)
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    if sampler:
        sampler.stop()
    ms = e0.elapsed_time(e1)
    barrier(world)
    return max_over_ranks(ms, world)


# ------------------------------------------------------------------------------------------
# CPU port of the reference's torch code (the oracle), timed on the host cores
# ------------------------------------------------------------------------------------------
def cpu_quantize_step(x):
    """Row-wise + transposed quantize with the oracle's float restatement of the reference's
    mxfp8_quantize_ref (the same torch ops in the same order)."""
    from oracle import mx8_oracle as O
    O.quantize_ref_float(x, "rceil")
    O.quantize_ref_float(x.t().contiguous(), "rceil")


def cpu_quantize_input(rows, cols):
    from oracle import mx8_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    return O.make_input(rows, cols, seed=1234, outliers=True, zero_blocks=True)


def cpu_gemm_operands(n):
    from oracle import mx8_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    a = O.make_input(n, n, seed=1, std=n ** -0.5)
    b = O.make_input(n, n, seed=2, std=n ** -0.5)
    return O.quantize_tiled(a) + O.quantize_tiled(b)


def cpu_gemm_step(ops):
    """dequantize + fp32 matmul + bf16 round with the oracle."""
    from oracle import mx8_oracle as O
    O.gemm_ref(*ops)


def time_cpu(fn, arg, steps, warmup):
    for _ in range(warmup):
        fn(arg)
    t0 = time.perf_counter()
    for _ in range(steps):
        fn(arg)
    return (time.perf_counter() - t0) / steps


def cpu_baseline_quantize(target_s=12.0):
    rows = 1024
    x = cpu_quantize_input(rows, QN)
    per = time_cpu(cpu_quantize_step, x, 1, 1)
    reps = max(2, min(100, int(target_s / per)))
    per = time_cpu(cpu_quantize_step, x, reps, 0)
    return {"value": rows * QN * 4.0625 / per / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{reps} passes over a {rows} x {QN} row slab of the workload, row-wise + transposed ({per * reps:.1f} s)"}


def cpu_baseline_gemm(target_s=8.0):
    n = 2048
    ops = cpu_gemm_operands(n)
    per = time_cpu(cpu_gemm_step, ops, 1, 1)
    reps = max(2, min(100, int(target_s / per)))
    per = time_cpu(cpu_gemm_step, ops, reps, 0)
    return {"value": 2.0 * n ** 3 / per / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{reps} passes of a {n}^3 sub-problem: dequantize + fp32 matmul + bf16 round ({per * reps:.1f} s)"}


def cpu_ffn_operands(T=512, H=8192, F=4096):
    from oracle import mx8_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    x = O.make_input(T, H, seed=3)
    w1 = O.quantize_tiled(O.make_input(F, H, seed=4, std=0.02))
    w2 = O.quantize_tiled(O.make_input(H, F, seed=5, std=0.02))
    return x, w1, w2


def cpu_ffn_step(ops):
    """quantize X, H = X W1^T rounded to bf16 and re-quantized, Y = H W2^T, all with the oracle."""
    from oracle import mx8_oracle as O
    x, w1, w2 = ops
    xq, xs = O.quantize_ref_float(x, "rceil")
    h = O.gemm_ref(xq, O.scale_swizzle(xs), *w1)
    hq, hs = O.quantize_ref_float(h, "rceil")
    O.gemm_ref(hq, O.scale_swizzle(hs), *w2)


def cpu_moe_operands(rows=1024, H=7168, I=2048):
    from oracle import mx8_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    x = O.make_input(rows, H, seed=6)
    q = lambda r, c, sd: O.quantize_both(O.make_input(r, c, seed=sd, std=0.02).unsqueeze(0))[:2]
    return x, torch.tensor([rows], dtype=torch.int32), q(I, H, 7), q(I, H, 8), q(H, I, 9)


def cpu_moe_step(ops):
    """One expert's routed forward (quantize, gate/up GEMMs, SwiGLU, down GEMM) with the oracle."""
    from oracle import moe_oracle as MO
    x, tpe, wg, wu, wd = ops
    MO.expert_mlp_ref(x, tpe, wg, wu, wd)


def cpu_baseline_layer(kind, target_s=6.0):
    if kind == "ffn":
        ops, fn, flops, what = cpu_ffn_operands(), cpu_ffn_step, 2.0 * 2.0 * 512 * 8192 * 4096, "512 tokens x 8192 -> 4096 -> 8192 slice of the FFN"
    else:
        ops, fn, flops, what = cpu_moe_operands(), cpu_moe_step, 6.0 * 1024 * 7168 * 2048, "one expert x 1024 routed rows of the MoE layer"
    per = time_cpu(fn, ops, 1, 0)
    reps = max(1, min(20, int(target_s / per)))
    per = time_cpu(fn, ops, reps, 0)
    return {"value": flops / per / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{reps} passes over {what} ({per * reps:.1f} s)"}


def run_reference(args, rank):
    """--impl reference: the reference's own CPU implementation of the path (its torch code,
    restated in oracle/) on all host threads; each step is a bounded sample of the workload."""
    if rank != 0:
        return
    total = max(1, args.steps + args.warmup)
    if args.workload == "quantize":
        rows = 1024
        x = cpu_quantize_input(rows, QN)
        est = time_cpu(cpu_quantize_step, x, 1, 1)
        while rows > 128 and est * total > 150.0:      # keep the whole run within a few minutes
            rows //= 2
            est /= 2
        x = x[:rows].contiguous()
        per = time_cpu(cpu_quantize_step, x, args.steps, args.warmup)
        value, unit, metric = rows * QN * 4.0625 / per / 1e9, "GB/s", "mxfp8_quantize_bandwidth"
        sample = f"{rows} x {QN} row slab of the 16384 x 16384 input per step, row-wise + transposed"
        cfg = {"workload": "quantize bf16 16384x16384 -> E4M3 + E8M0 scales, row-wise + transposed", "scale_mode": "rceil"}
    elif args.workload in ("ffn", "moe"):
        if args.workload == "ffn":
            ops, fn, flops = cpu_ffn_operands(), cpu_ffn_step, 2.0 * 2.0 * 512 * 8192 * 4096
            sample, metric = "512-token, 4096-wide slice of the FFN per step", "mxfp8_ffn_throughput"
            cfg = {"workload": "FFN X[16384x8192] -> [28672x8192] -> [8192x28672], MXFP8"}
        else:
            ops, fn, flops = cpu_moe_operands(), cpu_moe_step, 6.0 * 1024 * 7168 * 2048
            sample, metric = "one expert x 1024 routed rows per step", "mxfp8_moe_forward_throughput"
            cfg = {"workload": "MoE forward, 256 experts, hidden 7168, intermediate 2048, 32768 tokens, top-8"}
        steps = args.steps
        est = time_cpu(fn, ops, 1, 0)
        while steps > 1 and est * (steps + args.warmup) > 150.0:
            steps = max(1, steps // 2)
        per = time_cpu(fn, ops, steps, min(args.warmup, 1))
        value, unit = flops / per / 1e12, "TFLOP/s"
        sample += f" ({steps} timed steps)"
    else:
        n = 2048
        ops = cpu_gemm_operands(n)
        est = time_cpu(cpu_gemm_step, ops, 1, 1)
        if est * total > 150.0:
            n = 1024
            ops = cpu_gemm_operands(n)
        per = time_cpu(cpu_gemm_step, ops, args.steps, args.warmup)
        value, unit, metric = 2.0 * n ** 3 / per / 1e12, "TFLOP/s", "mxfp8_gemm_throughput"
        sample = f"{n}^3 sub-problem of the 8192^3 GEMM per step (dequantize + fp32 matmul + bf16 round)"
        cfg = {"workload": "MXFP8 GEMM M=N=K=8192, bf16 out"}
    line = {"impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": per * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u8", "data": "synthetic", "config": cfg,
            "cpu_baseline": {"value": value, "unit": unit, "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
def bench_quantize(args, world, rank, local, peaks, with_cpu):
    import mx8
    from oracle import mx8_oracle as O   # input generator only (make_input); nothing is computed with it
    dev = torch.device("cuda", local)
    M, N = QM, QN
    x_h = O.make_input(M, N, seed=1234 + rank, outliers=True, zero_blocks=True).pin_memory()
    x = x_h.to(dev, non_blocking=True)
    outs = list(mx8.mxfp8_quantize(x, True, True))
    algo_bytes = M * N * 2 + 2 * (M * N + M * N // 32)

    def step(_):
        mx8.mxfp8_quantize(x, outs[0], outs[1], outs[2], outs[3], True, True)

    for i in range(args.warmup):
        step(i)
    sampler = ClockSampler(local) if rank == 0 else None
    ms = timed(step, args.steps, world, sampler)
    mx8.device_status()
    per_ms = ms / args.steps
    value = world * algo_bytes / (per_ms * 1e-3) / 1e9
    achieved = algo_bytes / (per_ms * 1e-3) / 1e9

    # end to end through host buffers (mx8_quantize_host): pinned input -> device, quantize, all four
    # outputs -> pinned host, in bands of rows so that the two PCIe directions and the kernel overlap
    outs_h = [torch.empty(o.shape, dtype=torch.uint8).pin_memory() for o in outs]
    h2d = x_h.numel() * 2
    d2h = sum(o.numel() * o.element_size() for o in outs)
    ws = torch.empty(mx8.quantize_host_workspace(N, E2E_BAND_ROWS), dtype=torch.uint8, device=dev)

    def e2e_step(_):
        mx8.mxfp8_quantize_host(x_h, outs_h[0], outs_h[1], outs_h[2], outs_h[3], True, True,
                                band_rows=E2E_BAND_ROWS, workspace=ws, device=dev)

    e2e_steps = max(3, min(args.steps, 10))
    if args.quick:
        e2e_steps, e2e_ms, e2e_val = 0, None, None
    else:
        for i in range(2):
            e2e_step(i)
        e2e_ms = timed(e2e_step, e2e_steps, world) / e2e_steps
        e2e_val = world * algo_bytes / (e2e_ms * 1e-3) / 1e9

    line = {
        "metric": "mxfp8_quantize_bandwidth", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": per_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u8", "data": "synthetic",
        "config": {"workload": "quantize bf16 16384x16384 (N(0,1), 0.1% outliers x1000, zero blocks) -> E4M3 + E8M0 scales "
                               "in tcgen05 layout, row-wise + transposed, per GPU",
                   "scale_mode": "rceil", "l2": "inputs (512 MiB) and outputs (528 MiB) larger than L2",
                   "bytes_per_step_per_gpu": algo_bytes, "sharding": "one matrix per GPU, no collective"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES["quantize_16384x16384_both"],
                     "peak_source": peaks["source"], "frac_of_nominal_8000": achieved / 8000.0,
                     "kernel": "quantize_kernel<8,1,SRC_DENSE,true,true>", "algorithmic_bytes_per_launch": algo_bytes},
        "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms, "steps": e2e_steps, "api": "mx8_quantize_host, bands of %d rows" % E2E_BAND_ROWS},
        "gpu_launches": args.steps,
    }
    if sampler:
        line["clocks"] = sampler.summary()
    if with_cpu and rank == 0:
        line["cpu_baseline"] = cpu_baseline_quantize()
    return line


def gemm_shard_rows(world):
    """(total M, rows per rank): rows of A and C are split evenly across ranks, B is replicated."""
    rows = max(128, (GM // world // 128) * 128)
    return rows * world, rows


def bench_gemm(args, world, rank, local, peaks, with_cpu):
    import mx8
    from oracle import mx8_oracle as O   # input generator only
    dev = torch.device("cuda", local)
    _, M = gemm_shard_rows(world)
    N, K = GN, GK
    sets = []
    for s in range(3):                    # rotate operand sets so no iteration finds its inputs in L2
        a = O.make_input(M, K, seed=100 + 10 * s + rank, std=K ** -0.5).to(dev)
        b = O.make_input(N, K, seed=200 + 10 * s, std=K ** -0.5).to(dev)
        aq, asc, _, _ = mx8.mxfp8_quantize(a, True, False)
        bq, bsc, _, _ = mx8.mxfp8_quantize(b, True, False)
        sets.append((aq, asc, bq, bsc, torch.empty(M, N, dtype=torch.bfloat16, device=dev)))
        del a, b
    flops = 2.0 * M * N * K
    # --gemm-form: the activation arrives as bf16 and is quantized by a separate launch (a-bf16) or inside the GEMM's
    # main loop (a-bf16-fused, the optional prologue); default: operands already MXFP8
    a16 = a16_ws = None
    if args.gemm_form != "mxfp8" or (rank == 0 and not args.quick):
        a16 = O.make_input(M, K, seed=100 + rank, std=K ** -0.5).to(dev)
        a16_ws = torch.empty(mx8.load().mx8_gemm_a_bf16_workspace(M, K), dtype=torch.uint8, device=dev)

    def step(i):
        aq, asc, bq, bsc, c = sets[i % 3]
        if args.gemm_form == "mxfp8":
            mx8.kernel(aq, asc, bq, bsc, c)
        else:
            mx8.kernel_a_bf16(a16, bq, bsc, c, a16_ws, fused=args.gemm_form == "a-bf16-fused")

    for i in range(args.warmup):
        step(i)
    sampler = ClockSampler(local) if rank == 0 else None
    ms = timed(step, args.steps, world, sampler)
    mx8.device_status()
    per_ms = ms / args.steps
    achieved = flops / (per_ms * 1e-3) / 1e12
    value = world * achieved

    # the vendor library on the same operands, for context (not part of the roofline): cuBLAS through
    # torch._scaled_mm with the same E8M0 block scales, and with per-tensor scales (plain FP8)
    library = {}
    if rank == 0 and hasattr(torch, "float8_e8m0fnu") and not args.quick:
        aq, asc, bq, bsc, c = sets[0]
        def lib_rate(fn, iters=20):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return flops / (e0.elapsed_time(e1) / iters * 1e-3) / 1e12
        try:
            sa, sb = asc.reshape(-1).view(torch.float8_e8m0fnu), bsc.reshape(-1).view(torch.float8_e8m0fnu)
            library["cublas_mxfp8_tflops"] = lib_rate(lambda: torch._scaled_mm(aq, bq.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16))
            one = torch.ones((), device=dev)
            library["cublas_fp8_per_tensor_tflops"] = lib_rate(lambda: torch._scaled_mm(aq, bq.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16))
            library["mx8_same_loop_tflops"] = lib_rate(lambda: mx8.kernel(aq, asc, bq, bsc, c))
        except Exception as ex:
            library["error"] = f"{type(ex).__name__}: {ex}"[:200]
    # the three forms of the product for a bf16 activation, same loop (the evidence behind "the prologue is not used")
    forms = {}
    if rank == 0 and not args.quick and a16 is not None:
        aq, asc, bq, bsc, c = sets[0]
        def form_rate(fn, iters=10):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            time.sleep(0.3)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters):
                fn()
            e1.record()
            torch.cuda.synchronize()
            return flops / (e0.elapsed_time(e1) / iters * 1e-3) / 1e12
        forms = {"operands_already_mxfp8_tflops": form_rate(lambda: mx8.kernel(aq, asc, bq, bsc, c)),
                 "a_bf16_quantize_then_gemm_tflops": form_rate(lambda: mx8.kernel_a_bf16(a16, bq, bsc, c, a16_ws)),
                 "a_bf16_quantized_in_main_loop_tflops": form_rate(lambda: mx8.kernel_a_bf16(a16, bq, bsc, c, a16_ws, fused=True))}
        mx8.device_status()
    aq, asc, bq, bsc, c = sets[0]
    host_in = [t.cpu().pin_memory() for t in (aq, asc, bq, bsc)]
    c_h = torch.empty(c.shape, dtype=c.dtype).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = c.numel() * 2

    band = min(E2E_BAND_ROWS, M)
    host_in[0] = host_in[0].view(torch.uint8)
    host_in[2] = host_in[2].view(torch.uint8)
    ws = torch.empty(mx8.load().mx8_gemm_host_workspace(bq.shape[0], bq.shape[1], band, 0), dtype=torch.uint8, device=dev)

    def e2e_step(_):
        mx8.kernel_host(host_in[0], host_in[1], host_in[2], host_in[3], c_h, band_rows=band, workspace=ws, device=dev)

    e2e_steps = max(3, min(args.steps, 10))
    if args.quick:
        e2e_steps, e2e_ms = 0, None
    else:
        for i in range(2):
            e2e_step(i)
        e2e_ms = timed(e2e_step, e2e_steps, world) / e2e_steps
    # a sustained figure next to the burst above: 200 launches back to back (the power cap lowers the clock)
    sus_sampler = ClockSampler(local) if rank == 0 else None
    sus_steps = 1 if args.quick else 200
    sus_ms = timed(step, sus_steps, world, sus_sampler) / sus_steps
    sustained = {"tflops_per_gpu": flops / (sus_ms * 1e-3) / 1e12, "launches": sus_steps, "ms_per_launch": sus_ms}
    if sus_sampler:
        sustained["clocks"] = sus_sampler.summary()
    clocks = sampler.summary() if sampler else None
    line = {
        "metric": "mxfp8_gemm_throughput", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": per_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp8_e4m3 x ue8m0 -> f32 accumulate -> bf16", "data": "synthetic",
        "config": {"workload": f"MXFP8 GEMM M=N=K=8192 (per GPU {M}x{N}x{K}), operands quantized from bf16 N(0,1/sqrt(K)), bf16 out",
                   "l2": "three operand/output sets (256 MiB each at 1 GPU) used in rotation", "tile": "256x256x128, 2-CTA cluster, 6 stages",
                   "sharding": "rows of A and C split across GPUs, B replicated, no collective"},
        "roofline": tensor_roofline(achieved, local, clocks, traffic=NCU_TRAFFIC_BYTES["gemm_8192"], kernel="gemm_kernel<2>",
                                    algorithmic_flops_per_launch=flops, frac_of_2x_bf16_burst=achieved / (2.0 * peaks["bf16_tflops"])),
        "sustained": sustained,
        "e2e": {"value": world * flops / (e2e_ms * 1e-3) / 1e12 if e2e_ms else None, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps, "api": "mx8_gemm_host, bands of %d rows" % band},
        "gpu_launches": args.steps + sus_steps,
        "library": library,
        "bf16_activation_forms": forms,
    }
    if clocks:
        line["clocks"] = clocks
    if with_cpu and rank == 0:
        line["cpu_baseline"] = cpu_baseline_gemm()
    return line


def bench_ffn(args, world, rank, local, peaks, with_cpu=False):
    """Configuration 4: Llama-70B-shaped FFN, tokens sharded across ranks, weights replicated and
    pre-quantized; X is quantized per step and the intermediate H never exists in bf16: the first
    GEMM's epilogue emits MXFP8 directly."""
    import mx8
    dev = torch.device("cuda", local)
    T, H, F = 16384 // world, 8192, 28672
    g = torch.Generator(device=dev).manual_seed(4000 + rank)
    x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    gw = torch.Generator(device=dev).manual_seed(4100)
    w1 = (torch.randn(F, H, device=dev, generator=gw) * 0.02).to(torch.bfloat16)
    w1q, w1s, _, _ = mx8.mxfp8_quantize(w1, True, False)
    del w1
    w2 = (torch.randn(H, F, device=dev, generator=gw) * 0.02).to(torch.bfloat16)
    w2q, w2s, _, _ = mx8.mxfp8_quantize(w2, True, False)
    del w2
    xq = torch.empty(T, H, dtype=torch.float8_e4m3fn, device=dev)
    xs = torch.empty(T // 128, H // 128, 32, 16, dtype=torch.uint8, device=dev)
    hq = torch.empty(T, F, dtype=torch.float8_e4m3fn, device=dev)
    hs = torch.empty(T // 128, F // 128, 32, 16, dtype=torch.uint8, device=dev)
    y = torch.empty(T, H, dtype=torch.bfloat16, device=dev)

    def step(_):
        mx8.mxfp8_quantize(x, xq, xs, None, None, True, False)
        mx8.gemm_grouped(xq, xs, w1q, w1s, hq, hs)       # H = X W1^T, emitted as MXFP8
        mx8.kernel(hq, hs, w2q, w2s, y)                  # Y = H W2^T

    steps = LAYER_STEPS
    for i in range(3):
        step(i)
    sampler = ClockSampler(local) if rank == 0 else None
    ms = timed(step, steps, world, sampler) / steps
    mx8.device_status()
    flops = 2.0 * 2.0 * T * H * F
    achieved = flops / (ms * 1e-3) / 1e12
    return {"metric": "mxfp8_ffn_throughput", "value": world * achieved, "unit": "TFLOP/s", "ms_per_step": ms, "steps": steps,
            "scaling": "strong",
            "config": {"workload": f"FFN X[{T}x{H}] bf16 -> quantize -> [{F}x{H}] GEMM with MXFP8-quantizing epilogue -> [{H}x{F}] GEMM -> bf16, per GPU",
                       "l2": "per step about 1 GB of activations and 0.47 GB of weights per GPU at one GPU: larger than L2",
                       "sharding": "tokens split across GPUs, weights replicated, no collective"},
            "roofline": tensor_roofline(achieved, local, sampler.summary() if sampler else None, traffic=None),
            **({"clocks": sampler.summary()} if sampler else {}),
            "gpu_launches": 3 * steps, **({"cpu_baseline": cpu_baseline_layer("ffn")} if with_cpu and rank == 0 else {})}


def bench_moe(args, world, rank, local, peaks, with_cpu=False):
    """Configuration 5: DeepSeek-V3-like expert-parallel layer, 256 experts and 32768 tokens split over
    the ranks, top-8 routing, routed experts only.  A step is the reference harness's run_fwd_once."""
    import mx8
    dev = torch.device("cuda", local)
    E_total, H, I, k = args.moe_experts, 7168, 2048, 8
    tokens_total = args.moe_tokens
    T, E = tokens_total // world, E_total // world
    cap = ((T * k * max(2, world // 4)) // 256) * 256
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    logits = torch.randn(T, E_total, device=dev, generator=g)
    dist = symm_mem = None
    if world > 1:
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        x = symm_mem.empty(T, H, dtype=torch.bfloat16, device=dev)
        x.normal_(generator=g)
        x_ptrs = list(symm_mem.rendezvous(x, dist.group.WORLD.group_name).buffer_ptrs)
        cb = symm_mem.empty(T * k, H, dtype=torch.bfloat16, device=dev)
        cb_ptrs = list(symm_mem.rendezvous(cb, dist.group.WORLD.group_name).buffer_ptrs)
    else:
        x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
        cb = torch.empty(T * k, H, dtype=torch.bfloat16, device=dev)
        x_ptrs, cb_ptrs = [x.data_ptr()], [cb.data_ptr()]

    def make_w(rows, cols):
        q = torch.empty(E, rows, cols, dtype=torch.float8_e4m3fn, device=dev)
        sc = torch.empty(E * rows // 128, cols // 128, 32, 16, dtype=torch.uint8, device=dev)
        for e0 in range(0, E, 16):                       # quantize in slices to bound the bf16 temporary
            n = min(16, E - e0)
            w = (torch.randn(n, rows, cols, device=dev, generator=g) * 0.02).to(torch.bfloat16)
            mx8.mxfp8_quantize(w, q[e0:e0 + n], sc[e0 * rows // 128:(e0 + n) * rows // 128], None, None, True, False)
        return q, sc

    wg, wgs = make_w(I, H)
    wu, wus = make_w(I, H)
    wd, wds = make_w(H, I)
    vals, ids = torch.topk(logits, k, dim=1)            # the reference's router: top-k, softmax over the k values
    weights = torch.softmax(vals.float(), dim=-1)
    ids = ids.to(torch.int32)
    ids_all = torch.empty(world, T, k, dtype=torch.int32, device=dev)

    # the reference harness's knobs: communication SMs and rows of the schedule per minibatch
    comm_sms = args.moe_comm_sms
    nb_default = args.moe_minibatches
    minibatch = args.moe_minibatch if args.moe_minibatch > 0 else -(-cap // (nb_default * 256)) * 256
    tuning = {"ramp": args.moe_ramp, "combine_sms": args.moe_combine_sms, "combine_own_sms": args.moe_combine_own_sms}
    pipe = [0, 0]

    def layer(pr, pt, nt, tpe):
        return mx8.dispatch_mlp_swiglu_combine_fwd(x, x_ptrs, cb, cb_ptrs, None, wg, wgs, None, wu, wus, None, wd, wds,
                                                   pr, pt, nt, tpe, k, pipe[0], 0, pipe[1], tuning=tuning)

    def step(_):
        if world > 1:
            import torch.distributed as dist
            dist.all_gather_into_tensor(ids_all, ids)
        else:
            ids_all.copy_(ids.view(1, T, k))
        pr, pt, nt, tpe = mx8.schedule(ids_all, E, cap, rank)
        layer(pr, pt, nt, tpe)
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        return mx8.fwd_epilogue(None, cb, weights)

    # ---- parity, before anything is timed: (1) the layer in minibatches on three streams leaves the bytes of the
    # one-sequence layer, in this rank's routed outputs and in its combine buffer after every rank's pushes;
    # (2) sampled rows of this rank's expert outputs against the CPU oracle of the expert MLP (every step of the
    # chain is row-wise, so a row can be checked alone); (3) the weighted sum of the combine buffer against the
    # oracle's epilogue on sampled tokens.  Rank 0 reports the worst rank.
    parity = None
    if not args.no_parity:
        step(0)
        barrier(world)
        pr, pt, nt, tpe = mx8.schedule(ids_all, E, cap, rank)
        cb.zero_()
        barrier(world)
        single = layer(pr, pt, nt, tpe)
        barrier(world)
        cb_single = cb.clone()
        out_single = mx8.fwd_epilogue(None, cb, weights)
        cb.zero_()
        barrier(world)
        pipe[:] = [comm_sms, minibatch]
        piped = layer(pr, pt, nt, tpe)
        pipe[:] = [0, 0]
        barrier(world)
        n = int(nt)
        same = torch.equal(cb, cb_single)
        # the thirteen outputs, cut to the rows in use: (index, which axis holds the routed rows, rows per index step)
        for idx, axis, unit in ((0, 1, 1), (1, 1, 128), (3, 0, 1), (4, 0, 128), (6, 0, 1), (7, 0, 128), (9, 1, 1), (10, 1, 128), (12, 0, 1)):
            a_, b_ = single[idx].narrow(axis, 0, n // unit), piped[idx].narrow(axis, 0, n // unit)
            view = torch.int16 if a_.dtype == torch.bfloat16 else torch.uint8
            same = same and torch.equal(a_.contiguous().view(view), b_.contiguous().view(view))
        from oracle import moe_oracle as MO
        from oracle import mx8_oracle as O
        if world > 1:
            x_all = torch.empty(world, T, H, dtype=torch.bfloat16, device=dev)
            dist.all_gather_into_tensor(x_all, x)
        else:
            x_all = x.view(1, T, H)
        tpe_c, pr_c, pt_c = tpe.cpu(), pr.cpu(), pt.cpu()
        live = torch.nonzero(tpe_c > 0).squeeze(1)
        worst, checked = 0.0, 0
        for e in [int(live[0]), int(live[len(live) // 2]), int(live[-1])]:
            r0 = int(tpe_c[:e].sum())
            rows = slice(r0, r0 + 128)
            src_r, src_t = pr_c[rows].long(), pt_c[rows].long() // k
            xr = torch.zeros(128, H, dtype=torch.bfloat16)
            ok = src_r >= 0
            xr[ok] = x_all[src_r[ok].to(dev), src_t[ok].to(dev)].cpu()
            one = lambda wq, ws, r_: (wq[e:e + 1].view(torch.uint8).cpu(), ws[e * r_ // 128:(e + 1) * r_ // 128].cpu())
            ref = MO.expert_mlp_ref(xr, torch.tensor([128], dtype=torch.int32), one(wg, wgs, I), one(wu, wus, I), one(wd, wds, H))
            worst = max(worst, O.rel_frobenius(single[12][rows].cpu(), ref["y"]))
            checked += 128
        tok = torch.arange(0, T, max(1, T // 16))[:16]
        ref_out = MO.fwd_epilogue_ref(torch.zeros(len(tok), H, dtype=torch.bfloat16),
                                      cb_single.view(T, k, H)[tok.to(dev)].reshape(-1, H).cpu(), weights[tok.to(dev)].cpu())
        epi_exact = torch.equal(out_single[tok.to(dev)].cpu().view(torch.int16), ref_out.view(torch.int16))
        flags = torch.tensor([0.0 if same else 1.0, 0.0 if epi_exact else 1.0, worst, float(mx8.device_status())], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(flags, op=dist.ReduceOp.MAX)
        parity = {"pipelined_equals_single_sequence": flags[0].item() == 0.0, "epilogue_exact_on_sampled_tokens": flags[1].item() == 0.0,
                  "expert_rows_checked_per_gpu": checked, "max_rel_frobenius_vs_oracle": flags[2].item(), "tolerance": 1e-2,
                  "device_status": int(flags[3].item()),
                  "ok": flags[0].item() == 0.0 and flags[1].item() == 0.0 and flags[2].item() < 1e-2 and flags[3].item() == 0.0}
        del single, piped, cb_single, out_single

    steps = 2 if args.quick else LAYER_STEPS
    for i in range(1 if args.quick else 3):
        step(i)
    sampler_single = ClockSampler(local) if rank == 0 else None
    ms_single = timed(step, steps, world, sampler_single) / steps
    mx8.device_status()
    # the same layer with the routed experts cut into minibatches whose transfers overlap the GEMMs
    pipe[:] = [comm_sms, minibatch]
    for i in range(3):
        step(i)
    sampler = ClockSampler(local) if rank == 0 else None
    ms_pipe = timed(step, steps, world, sampler) / steps
    mx8.device_status()
    pipe[:] = [0, 0]
    # the figure reported is the form a multi-GPU job uses (minibatches, as the reference's harness asks for); at one GPU
    # there is nothing to overlap and the default arguments (one sequence) are the form to report
    use_pipe = world > 1
    ms = ms_pipe if use_pipe else ms_single
    if not use_pipe:
        sampler = sampler_single              # the clocks reported are those of the timed region that is reported
    pipeline = {"reported": "minibatches" if use_pipe else "single sequence", "comm_sms": comm_sms, "minibatch_rows": minibatch,
                "minibatches": min(E, -(-cap // minibatch)), "ramp": args.moe_ramp, "combine_sms": args.moe_combine_sms, "combine_own_sms": args.moe_combine_own_sms,
                "ms_per_step": ms_pipe, "single_sequence_ms_per_step": ms_single}

    # ---- backward of the same layer (routed experts): prologue, barrier, fused backward, barrier, epilogue
    bwd = None
    if not getattr(args, "no_bwd", False):
        def transposed(q_src_rows, q_src_cols, seed_shift):
            # weights of the backward are the transposes, quantized along their own K; regenerate the same
            # random matrices slice by slice (the generator state differs, the distribution is what matters)
            q = torch.empty(E, q_src_cols, q_src_rows, dtype=torch.float8_e4m3fn, device=dev)
            sc = torch.empty(E * q_src_cols // 128, q_src_rows // 128, 32, 16, dtype=torch.uint8, device=dev)
            for e0 in range(0, E, 16):
                n = min(16, E - e0)
                w = (torch.randn(n, q_src_cols, q_src_rows, device=dev, generator=g) * 0.02).to(torch.bfloat16)
                mx8.mxfp8_quantize(w, q[e0:e0 + n], sc[e0 * q_src_cols // 128:(e0 + n) * q_src_cols // 128], None, None, True, False)
            return q, sc
        wgT, wgTs = transposed(I, H, 1)      # [E, H, I]
        wuT, wuTs = transposed(I, H, 2)
        wdT, wdTs = transposed(H, I, 3)      # [E, I, H]
        if world > 1:
            d_cb = symm_mem.empty(T * k, H, dtype=torch.bfloat16, device=dev)
            d_cb_ptrs = list(symm_mem.rendezvous(d_cb, dist.group.WORLD.group_name).buffer_ptrs)
            d_xb = symm_mem.empty(T * k, H, dtype=torch.bfloat16, device=dev)
            d_xb_ptrs = list(symm_mem.rendezvous(d_xb, dist.group.WORLD.group_name).buffer_ptrs)
        else:
            d_cb = torch.empty(T * k, H, dtype=torch.bfloat16, device=dev)
            d_xb = torch.empty(T * k, H, dtype=torch.bfloat16, device=dev)
            d_cb_ptrs, d_xb_ptrs = [d_cb.data_ptr()], [d_xb.data_ptr()]
        d_out = (torch.randn(T, H, device=dev, generator=g) * H ** -0.5).to(torch.bfloat16)
        ids_all.copy_(ids.view(1, T, k)) if world == 1 else dist.all_gather_into_tensor(ids_all, ids)
        pr, pt, nt, tpe = mx8.schedule(ids_all, E, cap, rank)
        f = mx8.dispatch_mlp_swiglu_combine_fwd(x, x_ptrs, cb, cb_ptrs, None, wg, wgs, None, wu, wus, None, wd, wds, pr, pt, nt, tpe, k)

        def bstep(_):
            mx8.bwd_prologue(d_out, weights, d_cb)
            if world > 1:
                dist.barrier()
            mx8.dispatch_mlp_swiglu_combine_bwd(None, d_cb, d_cb_ptrs, d_xb, d_xb_ptrs, None, wgT, wgTs, None, wuT, wuTs, None, wdT, wdTs,
                                                f[0], f[1], None, f[3], f[4], None, f[6], f[7], None, f[9], f[10], x, x_ptrs,
                                                wg, wgs, wu, wus, pr, pt, nt, tpe, k, pipe[0], 0, pipe[1], tuning=tuning)
            if world > 1:
                dist.barrier()
            return mx8.bwd_epilogue_routed(None, d_xb, k)

        for i in range(2):
            bstep(i)
        bms_single = timed(bstep, steps, world) / steps
        mx8.device_status()
        pipe[:] = [comm_sms, minibatch]
        for i in range(2):
            bstep(i)
        bms_pipe = timed(bstep, steps, world) / steps
        mx8.device_status()
        pipe[:] = [0, 0]
        bms = bms_pipe if use_pipe else bms_single
        pipeline["backward_ms_per_step"] = bms_pipe
        pipeline["backward_single_sequence_ms_per_step"] = bms_single
        bwd = {"ms_per_step": bms, "value": 12.0 * (tokens_total * k) * H * I / (bms * 1e-3) / 1e12, "unit": "TFLOP/s",
               "flops": "12 * routed rows * hidden * intermediate"}
    flops_total = 6.0 * (tokens_total * k) * H * I
    value = flops_total / (ms * 1e-3) / 1e12
    per_gpu = value / world
    return {"metric": "mxfp8_moe_forward_throughput", "value": value, "unit": "TFLOP/s", "ms_per_step": ms, "steps": steps,
            "scaling": "strong",
            "config": {"workload": f"MoE forward, {E_total} experts / {world} GPUs, hidden {H}, intermediate {I}, {tokens_total} tokens, top-{k}, routed experts only",
                       "flops": "6 * routed rows * hidden * intermediate (padding rows not counted)",
                       "l2": "per step 11 GB of expert weights over all GPUs plus the routed activations: larger than L2",
                       "sharding": "experts and tokens split across GPUs; dispatch pulls and combine pushes over peer-mapped memory"},
            "roofline": tensor_roofline(per_gpu, local, sampler.summary() if sampler else None, traffic=None),
            **({"clocks": sampler.summary()} if sampler else {}),
            "parity": parity,
            "pipeline": pipeline,
            "backward": bwd,
            "gpu_launches": (10 + (14 if bwd else 0)) * steps, **({"cpu_baseline": cpu_baseline_layer("moe")} if with_cpu and rank == 0 else {})}


def summary_of(line, world):
    """the figures of every object of the line in one short object"""
    def rnd(v, nd=4):
        return round(v, nd) if isinstance(v, (int, float)) else v
    out = {"n_gpus": world}
    objs = {line.get("metric", "").replace("mxfp8_", "").split("_")[0]: line}
    for k in ("gemm", "ffn", "moe"):
        if isinstance(line.get(k), dict):
            objs[k] = line[k]
    for name, o in objs.items():
        if "error" in o:
            out[name] = {"error": o["error"][:120]}
            continue
        e = {"value": rnd(o.get("value"), 1), "unit": o.get("unit"), "ms_per_step": rnd(o.get("ms_per_step")),
             "frac_of_measured_roof": rnd(o.get("roofline", {}).get("frac"))}
        if "sustained" in o:
            e["sustained_tflops_per_gpu"] = rnd(o["sustained"]["tflops_per_gpu"], 1)
        if o.get("parity"):
            e["parity_ok"] = o["parity"]["ok"]
            e["max_rel_vs_oracle"] = rnd(o["parity"]["max_rel_frobenius_vs_oracle"], 6)
        if isinstance(o.get("backward"), dict):
            e["backward_ms_per_step"] = rnd(o["backward"]["ms_per_step"])
        if isinstance(o.get("pipeline"), dict):
            e["single_sequence_ms_per_step"] = rnd(o["pipeline"]["single_sequence_ms_per_step"])
            e["minibatches_ms_per_step"] = rnd(o["pipeline"]["ms_per_step"])
        out[name] = e
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="mx8", choices=["mx8", "reference"])
    ap.add_argument("--workload", default="quantize", choices=["quantize", "gemm", "ffn", "moe"])
    ap.add_argument("--gemm-form", default="mxfp8", choices=["mxfp8", "a-bf16", "a-bf16-fused"],
                    help="GEMM: what the timed step launches (bf16 activation quantized by its own launch, or inside the main loop)")
    ap.add_argument("--moe-comm-sms", type=int, default=28, help="MoE: multiprocessors left to the dispatch of the next minibatch")
    ap.add_argument("--moe-minibatch", type=int, default=0,
                    help="MoE: schedule rows per minibatch of the pipelined layer (0 = a quarter of the schedule capacity; "
                         "the reference harness uses 16384, which is the same at 8 GPUs)")
    ap.add_argument("--moe-minibatches", type=int, default=4, help="MoE: minibatches when --moe-minibatch is 0")
    ap.add_argument("--moe-combine-own-sms", type=int, default=0,
                    help="MoE: > 0 gives a combine that runs beside GEMMs that many multiprocessors of its own")
    ap.add_argument("--moe-ramp", type=int, default=0, help="MoE: 1 = first and last minibatch half as large; > 100 = growth in percent from both ends toward the middle")
    ap.add_argument("--moe-combine-sms", type=int, default=0, help="MoE: multiprocessors' worth of blocks for a combine beside GEMMs (0 = comm SMs / 4)")
    ap.add_argument("--moe-tokens", type=int, default=32768, help="MoE: tokens in total (smaller for profiler captures)")
    ap.add_argument("--moe-experts", type=int, default=256, help="MoE: experts in total (smaller for profiler captures)")
    ap.add_argument("--no-parity", action="store_true", help="MoE: skip the parity checks that precede the timing")
    ap.add_argument("--no-bwd", action="store_true", help="MoE: skip the backward")
    ap.add_argument("--with-bwd", action="store_true", help="MoE: keep the backward under --quick")
    ap.add_argument("--no-layers", action="store_true", help="skip the FFN and MoE objects of the quantize line")
    ap.add_argument("--no-gemm", action="store_true", help="skip the GEMM object of the quantize line")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--quick", action="store_true",
                    help="timed loop only: no end-to-end leg, no library comparison, no sustained loop, no CPU leg, no extra objects "
                         "(for profiler captures, which should see few launches)")
    args = ap.parse_args()
    if args.quick:
        args.no_cpu = args.no_gemm = args.no_layers = args.no_parity = True
        args.no_bwd = not args.with_bwd
    args.warmup = max(args.warmup, 3)
    args.steps = max(args.steps, 1)

    if args.impl == "reference":
        run_reference(args, int(os.environ.get("RANK", "0")))
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the mx8 path has no CPU fallback")
    world, rank, local = dist_setup(args.gpus)
    peaks = load_peaks()
    with_cpu = world == 1 and not args.no_cpu
    if args.workload == "quantize":
        line = bench_quantize(args, world, rank, local, peaks, with_cpu)
        if not args.no_gemm:
            g = bench_gemm(args, world, rank, local, peaks, with_cpu)
            line["gemm"] = {k: g[k] for k in ("metric", "value", "unit", "ms_per_step", "scaling", "config", "roofline", "e2e",
                                              "gpu_launches", "clocks", "cpu_baseline", "library", "sustained", "bf16_activation_forms") if k in g}
            line["gpu_launches"] += g["gpu_launches"]
        if not args.no_layers:
            for name, fn in (("ffn", bench_ffn), ("moe", bench_moe)):
                try:
                    torch.cuda.empty_cache()
                    line[name] = fn(args, world, rank, local, peaks, with_cpu)
                    line["gpu_launches"] += line[name]["gpu_launches"]
                except Exception as ex:      # a layer benchmark must not take the headline line down
                    line[name] = {"error": f"{type(ex).__name__}: {ex}"[:300]}
    elif args.workload == "gemm":
        line = bench_gemm(args, world, rank, local, peaks, with_cpu)
    else:
        line = (bench_ffn if args.workload == "ffn" else bench_moe)(args, world, rank, local, peaks, with_cpu)
        line.update({"n_gpus": world, "warmup": args.warmup, "higher_is_better": True, "vs_baseline": None, "dtype": "fp8_e4m3 x ue8m0",
                     "data": "synthetic"})
    if rank == 0:
        line["summary"] = summary_of(line, world)       # last key: the part of the line a log tail keeps
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
