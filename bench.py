#!/usr/bin/env python
"""Benchmark of the V:N:M SpMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (config.workload = "cfg1-sweep"): the N:M / V sweep at BERT-large linear-layer shapes,
(M,K) in {(1024,1024), (4096,1024), (1024,4096)}, N = 16384, V in {32,64,128}, n:m in {2:4,2:8,2:16,2:32},
36 SpMM launches.  One "step" is one pass over the 36 launches.  Inputs are seeded synthetic V:N:M
operands (venom_b200.synth), resident in HBM before the timed region starts.

metric/value: useful TFLOP/s = sum over the sweep of 2*M*N*K*(n/m) / time, whole job (all ranks).
e2e: the same metric through the host-buffer C-ABI entry point (vnm_spmm_f16_host): every launch copies
its dense operand from pinned host memory and its result back.
For --gpus N > 1 (launched under torchrun) every rank runs the same sweep on its own N-shard of a
G-times larger dense operand (weak scaling, no data-path collective); time = max over ranks.
--impl reference times the CPU check path (reference to_dense + restated host GEMM + compare).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = [(1024, 1024), (4096, 1024), (1024, 4096)]
VS = [32, 64, 128]
MS = [4, 8, 16, 32]
N_COLS = 16384
# dram__bytes_read.sum + dram__bytes_write.sum per launch (mean of the 36 launches of one step) from an ncu
# capture of this workload; the summary with the full command is kept under profiles/.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 96.5e6
METRIC = "vnm_spmm_useful_tflops"
UNIT = "TFLOP/s (useful = 2*M*N*K*n/m)"


def sweep_points():
    return [(M, K, V, m, N_COLS) for (M, K) in SHAPES for V in VS for m in MS]


def useful_flops(M, K, m, N):
    return 2.0 * M * N * K * 2.0 / m


def algorithmic_bytes(M, K, V, m, N):
    """values + metadata + column-loc + B once + C once (reference-format sizes)."""
    ksp = -(-(-(-K // m) * 2) // 16) * 16
    return 2 * M * ksp + 4 * (M // 2) * (ksp // 8) + 16 * (M // V) * (ksp // 2) + 2 * K * N + 2 * M * N


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "tflops_burst": d["bf16_tflops"], "tflops_sustained": d["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops_burst": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons (NVML, read-only) while the timed region runs; falls back
    to polling nvidia-smi when the NVML binding is unavailable."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.sm, self.mx, self.reasons = [], [], set()
        self._stop = threading.Event()
        self._t = threading.Thread(target=self._run, daemon=True)

    def _run_nvml(self):
        import pynvml as nv
        nv.nvmlInit()
        h = nv.nvmlDeviceGetHandleByIndex(self.index)
        mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
        bits = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}
        while not self._stop.is_set():
            self.sm.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
            self.mx.append(float(mx))
            try:
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
            except Exception:
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
            for name, bit in bits.items():
                if r & bit:
                    self.reasons.add(name)
            self._stop.wait(0.01)

    def _run_smi(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                f = [x.strip() for x in out.split(",")]
                if len(f) >= 6:
                    self.sm.append(float(f[0]))
                    self.mx.append(float(f[1]))
                    for i in range(4):
                        if f[2 + i].lower().startswith("active"):
                            self.reasons.add(names[i])
            except Exception:
                pass
            self._stop.wait(0.05)

    def _run(self):
        try:
            self._run_nvml()
        except Exception:
            self._run_smi()

    def __enter__(self):
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        return {"sm_mhz": float(np.median(self.sm)) if self.sm else None, "sm_max_mhz": max(self.mx) if self.mx else None,
                "reasons": sorted(self.reasons), "samples": len(self.sm)}


# ---------------------------------------------------------------------------------------------
# CPU check path (the reference's host side of --check: to_dense + dense product + compare)
# ---------------------------------------------------------------------------------------------
def cpu_check_path(points, seed=2024):
    """Times the CPU check path on `points`.  Uses the reference's own to_dense (oracle/_ref) when that
    library was built, else the C restatement; the fp32 host GEMM is the restatement in both cases
    (the reference itself runs this product on the GPU with cuBLAS).  Returns (useful_tflops, info)."""
    from oracle.oracle import Oracle, Reference
    from venom_b200.synth import random_dense_b, random_vnm_dense
    orc = Oracle()
    ref = Reference.load()
    flops = 0.0
    secs = 0.0
    for (M, K, V, m, N) in points:
        dense, cols, _ = random_vnm_dense(M, K, V, m, seed=seed)
        B = random_dense_b(K, N, seed=seed + 1)
        values, meta, _ = orc.compress(dense, cols, V, m)
        t0 = time.perf_counter()
        A = ref.to_dense(values, meta, cols, M, K, V, m) if ref is not None else orc.to_dense(values, meta, cols, M, K, V, m)
        C = orc.dense_gemm(A, B)
        bad, _, _ = orc.check(C, C, mode=0, tol=1.0)
        secs += time.perf_counter() - t0
        assert bad == 0
        flops += useful_flops(M, K, m, N)
    # kind is "port": the timed work is dominated by the restated host GEMM (the reference has none)
    return flops / secs / 1e12, {"cores": orc.num_threads(), "kind": "port", "seconds": secs,
                                 "to_dense": "compiled reference" if ref is not None else "restatement"}


CPU_SAMPLE = [(1024, 1024, 64, 8, N_COLS), (4096, 1024, 64, 8, N_COLS), (1024, 4096, 64, 8, N_COLS)]
CPU_SAMPLE_DESC = ("3 of the 36 sweep points (V=64, 2:8, all three (M,K) shapes, full N=16384): reference to_dense + restated "
                   "fp32 host GEMM (OpenMP, all cores) + elementwise compare")


def run_reference_arm(args, rank, world):
    if rank != 0:
        return
    vals = []
    for i in range(args.warmup + args.steps):
        v, info = cpu_check_path(CPU_SAMPLE, seed=100 + i)
        if i >= args.warmup:
            vals.append((v, info))
    value = float(np.mean([v for v, _ in vals]))
    info = vals[-1][1]
    secs = float(np.mean([i["seconds"] for _, i in vals]))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": secs * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16 in / f32 accumulate", "data": "synthetic",
        "config": {"workload": "cfg1-sweep", "sample": CPU_SAMPLE_DESC, "N": N_COLS},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": info["cores"], "kind": info["kind"], "sample": CPU_SAMPLE_DESC},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--kernel-only", action="store_true", help="skip the e2e, cuBLAS and CPU legs (used for ncu captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist
    from venom_b200 import capi
    from venom_b200.synth import random_vnm_dense

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path")
    capi.lib()  # fails loudly if the CUDA library is missing
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    points = sweep_points()
    # operands: one prepared sparse matrix per point, one dense B per K, one output per M
    rng = torch.Generator(device=dev)
    rng.manual_seed(1234 + rank)
    Bs = {K: (torch.rand((K, N_COLS), device=dev, generator=rng, dtype=torch.float32) * 2 - 1).half() for K in {k for _, k in SHAPES}}
    outs = {M: torch.empty((M, N_COLS), dtype=torch.float16, device=dev) for M in {mm for mm, _ in SHAPES}}
    preps = []
    for i, (M, K, V, m, N) in enumerate(points):
        dense, cols, _ = random_vnm_dense(M, K, V, m, seed=7000 + i)
        d = torch.from_numpy(dense).to(dev)
        c = torch.from_numpy(cols.view(np.int32)).to(dev)
        values, meta, bad = capi.compress(d, c, V, m)      # the GPU compressor produces the operands
        assert bad == 0
        preps.append(capi.Prepared(values, meta, c, M, K, V, m))
    torch.cuda.synchronize()

    def one_pass():
        for prep, (M, K, V, m, N) in zip(preps, points):
            prep.spmm(Bs[K], out=outs[M])

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        one_pass()
    barrier()
    # per-launch device times (CUDA events on the launching stream), one extra pass outside the timed region
    per_launch = []
    for prep, (M, K, V, m, N) in zip(preps, points):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        prep.spmm(Bs[K], out=outs[M])
        e1.record()
        e1.synchronize()
        per_launch.append(e0.elapsed_time(e1))
    barrier()
    with ClockSampler(local_rank) as clocks:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(args.steps):
            one_pass()
        stop.record()
        stop.synchronize()
        ms_total = start.elapsed_time(stop)
    barrier()
    status = max(p.device_status() for p in preps)
    if status != 0:
        raise SystemExit("device-side wait timed out (status %d): result invalid" % status)
    if world > 1:
        t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    flops_step = sum(useful_flops(M, K, m, N) for (M, K, V, m, N) in points)
    bytes_step = sum(algorithmic_bytes(M, K, V, m, N) for (M, K, V, m, N) in points)
    value = world * flops_step / (ms_step * 1e-3) / 1e12

    if args.kernel_only:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "ms_per_step": ms_step, "kernel_only": True,
                              "per_launch_ms": [round(t, 5) for t in per_launch]}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- end to end through the host-buffer C-ABI entry point (pinned host memory) ----
    hB = {K: torch.empty((K, N_COLS), dtype=torch.float16).pin_memory() for K in Bs}
    for K in Bs:
        hB[K].copy_(Bs[K].cpu())
    # every product of the pass gets its own pinned result buffer: the 36 calls are queued without waiting
    # (uploads of one product overlap the downloads of the one before) and collected at the end of the pass
    hO = [torch.empty((M, N), dtype=torch.float16).pin_memory() for (M, K, V, m, N) in points]
    h2d = sum(2 * K * N for (M, K, V, m, N) in points)
    d2h = sum(2 * M * N for (M, K, V, m, N) in points)

    def one_pass_e2e():
        for prep, out, (M, K, V, m, N) in zip(preps, hO, points):
            prep.spmm_host_async(hB[K], out)
        for prep in preps:
            prep.host_wait()

    one_pass_e2e()
    barrier()
    t0 = time.perf_counter()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(args.e2e_steps):
        one_pass_e2e()
    s1.record()
    s1.synchronize()
    e2e_ms = max(s0.elapsed_time(s1), (time.perf_counter() - t0) * 1e3) / args.e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = world * flops_step / (e2e_ms * 1e-3) / 1e12

    # ---- cuBLAS dense fp16 on the same shapes (speed-up denominator of the reference's CSV line) ----
    cublas_ms = 0.0
    if rank == 0:
        dens = {}
        for (M, K) in SHAPES:
            dens[(M, K)] = (torch.rand((M, K), device=dev, generator=rng, dtype=torch.float32) * 2 - 1).half()
        for (M, K) in SHAPES:
            for _ in range(3):
                torch.matmul(dens[(M, K)], Bs[K], out=outs[M])
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        reps = 5
        for _ in range(reps):
            for (M, K) in SHAPES:
                torch.matmul(dens[(M, K)], Bs[K], out=outs[M])
        c1.record()
        c1.synchronize()
        cublas_ms = c0.elapsed_time(c1) / reps * len(VS) * len(MS)   # the sweep runs each shape 12 times
    barrier()

    if rank == 0:
        peaks = measured_peaks()
        t_tensor = flops_step / (peaks["tflops_sustained"] * 1e12)
        t_hbm = bytes_step / (peaks["hbm_gbs"] * 1e9)
        nl = len(points)
        kernel_ms = float(sum(per_launch))
        # The sweep is HBM-bound in the ideal model for 27 of its 36 points (every m >= 8); the aggregate
        # roofline is therefore stated against HBM: algorithmic bytes per launch / mean launch duration.
        achieved = bytes_step / nl / (kernel_ms / nl * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                    "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH, "peak_source": peaks["source"], "kernel": "vnm::spmm_dense_b_kernel (83 % of the step) + vnm::spmm_kernel, mean of the 36 launches",
                    "algorithmic_bytes_per_launch": bytes_step / nl, "mean_launch_ms": kernel_ms / nl,
                    "tensor_frac_of_sustained_dense_peak": (flops_step / (kernel_ms * 1e-3) / 1e12) / peaks["tflops_sustained"],
                    "ideal_ms_per_step": {"hbm": t_hbm * 1e3, "tensor": t_tensor * 1e3}}
        cpu = None
        if not args.no_cpu_baseline:
            v, info = cpu_check_path(CPU_SAMPLE)
            cpu = {"value": v, "unit": UNIT, "cores": info["cores"], "kind": info["kind"], "sample": CPU_SAMPLE_DESC}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16 in / f32 accumulate", "data": "synthetic",
            "config": {"workload": "cfg1-sweep", "shapes_MK": SHAPES, "N": N_COLS, "V": VS, "n:m": ["2:%d" % m for m in MS],
                       "launches_per_step": nl, "l2": "inputs larger than L2: one pass cycles through 320 MB of dense operands and outputs",
                       "parallelism": "N-sharded x%d (weak)" % world},
            "clocks": clocks.summary(),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world, "ms_per_step": e2e_ms},
            "gpu_launches": nl * args.steps,
            "roofline": roofline,
            "cpu_baseline": cpu,
            "speedup_vs_cublas_dense_fp16": (cublas_ms / ms_step) if cublas_ms else None,
            "per_launch_ms": {"%dx%d_V%d_2:%d" % (M, K, V, m): round(t, 5) for (M, K, V, m, N), t in zip(points, per_launch)},
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
