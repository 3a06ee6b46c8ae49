#!/usr/bin/env python
"""Benchmark of the V:N:M SpMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extras]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 ... bench.py --gpus N ...

Headline workload (config.workload = "cfg4"): one product C = A_vnm * B with M = 49152, K = 12288, N = 32768,
V = 128, 2:8, fp16 in / fp32 accumulate / fp16 out -- the largest single-GPU configuration, tensor-bound.  One
"step" is one product.  Under --gpus N the dense operand and the result are sharded by columns over the ranks
through venom_b200.sharded.ShardedSpmm (total N fixed: strong scaling; the sparse operand is compressed on rank 0
by the GPU compressor and broadcast once); the step time is the maximum over ranks.  Inputs are seeded synthetic
operands (venom_b200.synth) resident in HBM before the timed region starts; every step reads and writes 4 GB, far
more than L2.

  value   whole-job useful TFLOP/s = 2*M*N*K*(2/m) / step time.
  e2e     the same product through the host-buffer C-ABI entry point (vnm_spmm_f16_host): each step copies this
          rank's dense operand up from pinned host memory and its result back down.
  extra   with_allgather (N > 1): the step with the whole [N, M] result replicated on every rank
          (vnm_mgpu_spmm_gathered, chunked exchange beside the product, and the plain product-then-all-gather form);
          cfg1_sweep: the 36-point N:M / V sweep at BERT-large layer shapes; compressor: dense -> V:N:M compression of
          the 49152 x 12288 matrix; bert_large: encoder tokens/s dense and 64:2:8 through the torch op.
Before anything is timed, a seeded sample of output rows of every product the benchmark launches is compared with the
CPU oracle; a mismatch ends the run with a non-zero exit code.
--impl reference times the reference's host-side check path (reference to_dense + restated fp32 host GEMM + compare)
on a bounded sample of the same workload, on rank 0 only, with every host core.
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

CFG4 = dict(M=49152, K=12288, N=32768, V=128, m=8)
SHAPES = [(1024, 1024), (4096, 1024), (1024, 4096)]
VS = [32, 64, 128]
MS = [4, 8, 16, 32]
N_COLS = 16384
METRIC = "vnm_spmm_useful_tflops"
UNIT = "TFLOP/s (useful = 2*M*N*K*n/m)"
CONFIG = {"workload": "cfg4", "M": CFG4["M"], "K": CFG4["K"], "N": CFG4["N"], "V": CFG4["V"], "n:m": "2:%d" % CFG4["m"],
          "l2": "inputs larger than L2: every step reads 0.8 GB of B and writes 3.2 GB of C (per job)"}
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the headline kernel at full size on one GPU, from the
# one-pass ncu capture summarised under profiles/ (re-capture whenever the kernel or its tile order changes).
NCU_TRAFFIC = {"bytes_per_launch": 22193078016 + 3277997824,
               "source": "profiles/spmm_dense_b_pair_kernel_cfg4_launch.md: one-pass ncu capture of a full-size launch (1 GPU, N = 32768)"}
CPU_SAMPLE_ROWS = 256
CPU_SAMPLE_DESC = ("first %d of the %d rows of the cfg4 sparse operand (2 vector blocks), full K and N: reference to_dense + restated "
                   "fp32 host GEMM (OpenMP) + elementwise compare; rate on the sample, the whole product is %dx this work"
                   % (CPU_SAMPLE_ROWS, CFG4["M"], CFG4["M"] // CPU_SAMPLE_ROWS))


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


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def bind_to_gpu_numa_node(local_rank):
    """Pins this process (and, through first-touch, its pinned host buffers) to the CPUs of the NUMA node the GPU hangs
    off, so that eight ranks do not all stage through node 0.  Best effort: returns a description or None."""
    try:
        import torch
        p = torch.cuda.get_device_properties(local_rank)
        bdf = "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
        node = int(open("/sys/bus/pci/devices/%s/numa_node" % bdf).read().strip())
        if node < 0:
            return {"pci": bdf, "numa_node": None}
        cpus = set()
        for part in open("/sys/devices/system/node/node%d/cpulist" % node).read().strip().split(","):
            a, _, b = part.partition("-")
            cpus.update(range(int(a), int(b or a) + 1))
        allowed = cpus & set(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else cpus
        if allowed:
            os.sched_setaffinity(0, allowed)
        return {"pci": bdf, "numa_node": node, "cpus": len(allowed)}
    except Exception as e:  # no sysfs entry, no permission ...: run unbound
        return {"error": str(e)[:80]}


# ---------------------------------------------------------------------------------------------
# CPU check path (the reference's host side of --check: to_dense + dense product + compare)
# ---------------------------------------------------------------------------------------------
class CpuCheckPath:
    """The reference's check path on the first CPU_SAMPLE_ROWS rows of the cfg4 operand (a prefix of the three
    reference-format arrays is itself a valid operand).  The reference's own to_dense (oracle/_ref) is used when that
    library was built, else the C restatement; the fp32 host GEMM is the restatement in both cases (the reference runs
    this product on the GPU with cuBLAS), hence kind "port"."""

    def __init__(self, seed=2024):
        from oracle.oracle import Oracle, Reference
        from venom_b200.synth import random_dense_b, random_vnm_dense
        self.orc = Oracle()
        self.cores = self.orc.set_num_threads(host_cores())   # explicit: launchers export OMP_NUM_THREADS=1
        self.ref = Reference.load()
        c = CFG4
        self.R = CPU_SAMPLE_ROWS
        dense, self.cols, _ = random_vnm_dense(self.R, c["K"], c["V"], c["m"], seed=seed)
        self.values, self.meta, bad = self.orc.compress(dense, self.cols, c["V"], c["m"])
        assert bad == 0
        self.B = random_dense_b(c["K"], c["N"], seed=seed + 1)
        self.flops = useful_flops(self.R, c["K"], c["m"], c["N"])

    def step(self):
        c = CFG4
        t0 = time.perf_counter()
        if self.ref is not None:
            A = self.ref.to_dense(self.values, self.meta, self.cols, self.R, c["K"], c["V"], c["m"])
        else:
            A = self.orc.to_dense(self.values, self.meta, self.cols, self.R, c["K"], c["V"], c["m"])
        C = self.orc.dense_gemm(A, self.B)
        bad, _, _ = self.orc.check(C, C, mode=0, tol=1.0)
        dt = time.perf_counter() - t0
        assert bad == 0
        return dt

    def info(self):
        return {"cores": self.cores, "kind": "port", "to_dense": "compiled reference" if self.ref is not None else "restatement"}


def run_reference_arm(args, rank):
    if rank != 0:
        return
    path = CpuCheckPath()
    secs = []
    for i in range(args.warmup + args.steps):
        dt = path.step()
        if i >= args.warmup:
            secs.append(dt)
    mean = float(np.mean(secs))
    value = path.flops / mean / 1e12
    info = path.info()
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": mean * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16 in / f32 accumulate", "data": "synthetic", "config": CONFIG,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": info["cores"], "kind": info["kind"], "sample": CPU_SAMPLE_DESC,
                         "to_dense": info["to_dense"]},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def check_rows_against_oracle(orc, out, values, meta, colloc, M, K, V, m, B, nrows, seed, what):
    """Compares `nrows` seeded rows of out [M, n] with the CPU oracle's fp32 product; raises SystemExit on a mismatch."""
    import torch
    rows = np.sort(np.random.default_rng(seed).choice(M, size=min(nrows, M), replace=False)).astype(np.int32)
    want = orc.spmm(values, meta, colloc, M, K, V, m, B, rows=rows)
    got = out[torch.from_numpy(rows).long().to(out.device)].cpu().numpy()
    bad, first, worst = orc.check(got, want[rows], mode=1, tol=1e-2)
    if bad:
        raise SystemExit("bench.py: %s differs from the CPU oracle in %d sampled elements (max abs err %g): no number is reported" % (what, bad, worst))


def time_events(fn, steps, torch):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / steps


def extra_cfg1_sweep(torch, capi, orc, dev, steps):
    """The N:M / V sweep at BERT-large layer shapes (36 launches per pass), every launch checked on sampled rows first."""
    from venom_b200.synth import random_vnm_dense_cuda
    points = sweep_points()
    rng = torch.Generator(device=dev)
    rng.manual_seed(1234)
    Bs = {K: (torch.rand((K, N_COLS), device=dev, generator=rng, dtype=torch.float32) * 2 - 1).half() for K in {k for _, k in SHAPES}}
    Bh = {K: b.cpu().numpy() for K, b in Bs.items()}
    outs = {M: torch.empty((M, N_COLS), dtype=torch.float16, device=dev) for M in {mm for mm, _ in SHAPES}}
    preps, forms = [], []
    for i, (M, K, V, m, N) in enumerate(points):
        d, c = random_vnm_dense_cuda(M, K, V, m, seed=7000 + i)
        values, meta, bad = capi.compress(d, c, V, m)
        assert bad == 0
        prep = capi.Prepared(values, meta, c, M, K, V, m)
        prep.spmm(Bs[K], out=outs[M])
        check_rows_against_oracle(orc, outs[M], values.cpu().numpy(), meta.cpu().numpy().view(np.uint32), c.cpu().numpy().view(np.uint32),
                                  M, K, V, m, Bh[K], 8, 100 + i, "sweep point %dx%d V=%d 2:%d" % (M, K, V, m))
        preps.append(prep)
        forms.append("dense-B" if prep.dense_b_form() else "gather")

    def one_pass():
        for prep, (M, K, V, m, N) in zip(preps, points):
            prep.spmm(Bs[K], out=outs[M])
    for _ in range(3):
        one_pass()
    torch.cuda.synchronize()
    per_launch = []
    for prep, (M, K, V, m, N) in zip(preps, points):
        per_launch.append(time_events(lambda: prep.spmm(Bs[K], out=outs[M]), 3, torch))
    ms_step = time_events(one_pass, steps, torch)
    if max(p.device_status() for p in preps) != 0:
        raise SystemExit("bench.py: a device-side wait timed out in the sweep")
    dens = {(M, K): (torch.rand((M, K), device=dev, generator=rng, dtype=torch.float32) * 2 - 1).half() for (M, K) in SHAPES}

    def cublas_pass():
        for (M, K) in SHAPES:
            torch.matmul(dens[(M, K)], Bs[K], out=outs[M])
    for _ in range(3):
        cublas_pass()
    cublas_ms = time_events(cublas_pass, 5, torch) * len(VS) * len(MS)
    flops = sum(useful_flops(M, K, m, N) for (M, K, V, m, N) in points)
    nbytes = sum(algorithmic_bytes(M, K, V, m, N) for (M, K, V, m, N) in points)
    peaks = measured_peaks()
    return {"useful_tflops": flops / (ms_step * 1e-3) / 1e12, "ms_per_pass": ms_step, "launches_per_pass": len(points),
            "speedup_vs_cublas_dense_fp16": cublas_ms / ms_step, "hbm_gbs": nbytes / (ms_step * 1e-3) / 1e9,
            "frac_of_hbm_peak": nbytes / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "per_launch_ms": {"%dx%d_V%d_2:%d(%s)" % (M, K, V, m, f): round(t, 5) for (M, K, V, m, N), t, f in zip(points, per_launch, forms)}}


def extra_compressor(torch, capi, dense, colloc, V, m, ms):
    """GPU compressor on the cfg4 matrix (timed by the caller) and, beside it, the reference's own single-threaded
    to_sparse_sr_nm on a smaller matrix of the same row length."""
    from venom_b200.synth import vnm_sizes
    M, K = dense.shape
    ksp, nv, nm, nc = vnm_sizes(M, K, V, m)
    nbytes = 2 * M * K + 4 * nc + 2 * nv + 4 * nm
    peaks = measured_peaks()
    rec = {"matrix": "%dx%d V=%d 2:%d" % (M, K, V, m), "ms": ms, "gbs": nbytes / ms / 1e6, "frac_of_hbm_peak": nbytes / ms / 1e6 / peaks["hbm_gbs"],
           "algorithmic_bytes": nbytes}
    try:
        from oracle.oracle import Reference
        ref = Reference.load()
        R = 1024
        sub = dense[:R].cpu().numpy()
        cols = colloc.cpu().numpy().view(np.uint32)[: (R // V) * (ksp // 2) * 4]
        if ref is not None:
            t0 = time.perf_counter()
            ref.compress(sub, cols, V, m)
            dt = time.perf_counter() - t0
            sub_bytes = nbytes * R / M
            rec["cpu_baseline"] = {"kind": "reference", "cores": 1, "sample": "first %d rows (%dx%d), reference to_sparse_sr_nm as shipped" % (R, R, K),
                                   "ms": dt * 1e3, "gbs": sub_bytes / dt / 1e9}
    except Exception as e:
        rec["cpu_baseline_error"] = str(e)[:120]
    return rec


def extra_bert(torch):
    from venom_b200 import e2e_bert
    import contextlib
    import io
    with contextlib.redirect_stdout(io.StringIO()):
        d, s = e2e_bert.main(["-m", "8", "-n", "2", "-v", "64", "--repeats", "5"])
    tokens = 32 * 512
    return {"model": "BERT-large encoder, 24 layers, batch 32 x seq 512, fp16, random-init weights, all 144 linears pruned to 64:2:8 by magnitude",
            "dense_tokens_per_s": tokens / d * 1e3, "vnm_tokens_per_s": tokens / s * 1e3, "dense_ms": d, "vnm_ms": s, "speedup": d / s}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the cfg1 sweep, compressor and BERT records")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--kernel-only", action="store_true", help="only the headline product (used for ncu captures)")
    ap.add_argument("--sweep-only", action="store_true", help="only the cfg1 sweep record (used for ncu launch lists); one GPU")
    ap.add_argument("--n-cols", type=int, default=CFG4["N"], help="total N of the headline product (smaller values are for ncu captures only)")
    ap.add_argument("--m-rows", type=int, default=CFG4["M"], help="M of the headline product (smaller values are for ncu captures only)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    import torch
    import torch.distributed as dist
    from oracle.oracle import Oracle   # the checker: used outside the timed regions only
    from venom_b200 import capi
    from venom_b200.sharded import ShardedSpmm, shard_bounds
    from venom_b200.synth import random_vnm_dense_cuda

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path")
    capi.lib()  # fails loudly if the CUDA library is missing
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    numa = bind_to_gpu_numa_node(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    orc = Oracle()
    orc.set_num_threads(host_cores())

    if args.sweep_only:
        print(json.dumps({"cfg1_sweep": extra_cfg1_sweep(torch, capi, orc, dev, args.steps)}), flush=True)
        return

    M, K, V, m = args.m_rows, CFG4["K"], CFG4["V"], CFG4["m"]
    N = args.n_cols
    full_size = (M == CFG4["M"] and N == CFG4["N"])
    lo, hi = shard_bounds(N, world, rank)
    ns = hi - lo

    # ---- operands: rank 0 draws and compresses the sparse operand on the GPU, every rank gets a copy ----
    values = meta = colloc = dense = None
    compress_ms = None
    if rank == 0:
        dense, colloc = random_vnm_dense_cuda(M, K, V, m, seed=4)
        values, meta, bad = capi.compress(dense, colloc, V, m)
        if bad:
            raise SystemExit("bench.py: the compressor reported %d violations on a valid operand" % bad)
        if not args.kernel_only:
            for _ in range(3):
                capi.compress(dense, colloc, V, m, count_violations=False)
            compress_ms = time_events(lambda: capi.compress(dense, colloc, V, m, count_violations=False), 10, torch)
    sh = ShardedSpmm.from_reference_arrays(values, meta, colloc, M, K, V, m)
    prep = sh.prepared
    g = torch.Generator(device=dev)
    g.manual_seed(100 + rank)
    B = (torch.rand((K, ns), device=dev, generator=g) * 2 - 1).half()
    out = torch.empty((M, ns), dtype=torch.float16, device=dev)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        if sh.ctx is not None:
            sh.ctx.spmm_shard(prep, B, out=out)
        else:
            prep.spmm(B, out=out)

    # ---- parity gate, outside every timed region: rank 0's product against the CPU oracle on sampled rows ----
    step()
    torch.cuda.synchronize()
    if rank == 0:
        hv, hm, hc = values.cpu().numpy(), meta.cpu().numpy().view(np.uint32), colloc.cpu().numpy().view(np.uint32)
        check_rows_against_oracle(orc, out, hv, hm, hc, M, K, V, m, B.cpu().numpy(), 16, 1, "the headline product")
    if prep.device_status() != 0:
        raise SystemExit("device-side wait timed out: result invalid")

    for _ in range(args.warmup):
        step()
    barrier()
    with ClockSampler(local_rank) as clocks:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(args.steps):
            step()
        stop.record()
        stop.synchronize()
        ms_total = start.elapsed_time(stop)
    barrier()
    if prep.device_status() != 0:
        raise SystemExit("device-side wait timed out: result invalid")
    if world > 1:
        t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    flops_step = useful_flops(M, K, m, N)          # the whole job
    value = flops_step / (ms_step * 1e-3) / 1e12
    form = "dense-B" if prep.dense_b_form() else "gather"
    kcfg = prep.config(ns)
    kernel_name = ("vnm::spmm_dense_b_pair_kernel (clusters of two CTAs, tcgen05 cta_group::2)" if (form == "dense-B" and kcfg["stages"] == 2) else
                   "vnm::spmm_dense_b_kernel" if form == "dense-B" else "vnm::spmm_kernel")

    if args.kernel_only:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "ms_per_step": ms_step, "kernel_only": True, "operand_form": form,
                              "M": M, "N": N}), flush=True)
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- the replicated [N, M] result: chunked exchange beside the product, and product-then-all-gather ----
    gathered = None
    if world > 1 and N % (8 * world) == 0:
        full = torch.empty((N, M), dtype=torch.float16, device=dev)
        rec = {}
        for name, chunks in (("overlapped_ms", 4), ("plain_ms", 1)):
            sh.gathered(B, N, chunks=chunks, out=full)
            barrier()
            t_ms = time_events(lambda: sh.gathered(B, N, chunks=chunks, out=full), max(3, args.steps // 4), torch)
            tt = torch.tensor([t_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            rec[name] = float(tt.item())
            barrier()
        # every rank's rows must have arrived everywhere: compare the copy on this rank with each owner's checksum
        def check_replicas(what):
            sums = full.float().sum(dim=1).reshape(world, ns).sum(dim=1).double()
            ref = sums.clone()
            dist.broadcast(ref, src=0)
            if not torch.allclose(sums, ref, rtol=0, atol=0) or not bool((sums != 0).all()):
                raise SystemExit("bench.py: the gathered result (%s) differs between ranks" % what)
        check_replicas("NCCL exchange")
        # peer-store form: one launch whose epilogue stores every tile to all ranks' buffers (registered through CUDA IPC)
        try:
            full.zero_()
            sh.gathered_p2p(B, N, full)
            barrier()
            t_ms = time_events(lambda: sh.gathered_p2p(B, N, full), max(3, args.steps // 4), torch)
            tt = torch.tensor([t_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            rec["peer_store_ms"] = float(tt.item())
            barrier()
            check_replicas("peer stores")
            sh.release_outputs()
        except capi.VenomError as exc:   # the same verdict on every rank: registration is agreed collectively
            rec["peer_store_unavailable"] = str(exc)
        bytes_in = (world - 1) * ns * M * 2
        exposed_plain = max(rec["plain_ms"] - ms_step, 1e-6)
        rec.update({"chunks": 4, "spmm_only_ms": ms_step, "bytes_received_per_rank": bytes_in,
                    "allgather_gbs_per_rank_in": bytes_in / (exposed_plain * 1e-3) / 1e9,
                    "exposed_ms": dict({"plain": rec["plain_ms"] - ms_step, "overlapped": rec["overlapped_ms"] - ms_step},
                                       **({"peer_store": rec["peer_store_ms"] - ms_step} if "peer_store_ms" in rec else {})),
                    "collective": "plain: one in-place ncclAllGather after the product; overlapped: grouped ncclSend/ncclRecv per chunk on a second "
                                  "stream; peer_store: no collective, the product's epilogue stores every tile to all ranks' buffers over NVLink "
                                  "(two 4-byte all-gathers order the ranks)"})
        gathered = rec
        del full
        torch.cuda.empty_cache()

    # ---- cuBLAS dense fp16 on the same shard (speed-up denominator of the reference's CSV line) ----
    cublas_ms = None
    if rank == 0:
        for _ in range(3):
            torch.matmul(dense, B, out=out)
        cublas_ms = time_events(lambda: torch.matmul(dense, B, out=out), 5, torch)
    barrier()

    # ---- end to end through the host-buffer C-ABI entry point (pinned host memory, per-rank shard) ----
    hB = torch.empty((K, ns), dtype=torch.float16).pin_memory()
    hB.copy_(B.cpu())
    hO = torch.empty((M, ns), dtype=torch.float16).pin_memory()
    prep.spmm_host(hB, hO)
    barrier()
    # plain copy rates of this rank's buffers, for the record (what the host side can deliver at this N)
    h2d_ms = time_events(lambda: B.copy_(hB, non_blocking=True), 3, torch)
    d2h_ms = time_events(lambda: hO.copy_(out, non_blocking=True), 2, torch)
    prep.spmm_host(hB, hO)
    barrier()
    t0 = time.perf_counter()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(args.e2e_steps):
        prep.spmm_host(hB, hO)
    s1.record()
    s1.synchronize()
    e2e_ms = max(s0.elapsed_time(s1), (time.perf_counter() - t0) * 1e3) / args.e2e_steps
    rates = torch.tensor([e2e_ms, 2.0 * K * ns / h2d_ms / 1e6, 2.0 * M * ns / d2h_ms / 1e6], device=dev, dtype=torch.float64)
    if world > 1:
        mx = rates.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        mn = rates.clone()
        dist.all_reduce(mn, op=dist.ReduceOp.MIN)
        e2e_ms = float(mx[0].item())
        h2d_rate, d2h_rate = float(mn[1].item()), float(mn[2].item())
    else:
        h2d_rate, d2h_rate = float(rates[1].item()), float(rates[2].item())
    e2e_value = flops_step / (e2e_ms * 1e-3) / 1e12
    # the e2e result is the product too: check it
    if rank == 0:
        check_rows_against_oracle(orc, hO, hv, hm, hc, M, K, V, m, hB.numpy(), 8, 2, "the end-to-end product")
    del hB, hO

    extras = {}
    if rank == 0 and not args.no_extras and full_size:
        extras["compressor"] = extra_compressor(torch, capi, dense, colloc, V, m, compress_ms)
    if world > 1:
        barrier()
    if rank == 0 and not args.no_extras and world == 1 and full_size:
        del dense, B, out
        sh = prep = None
        torch.cuda.empty_cache()
        for name, fn in (("cfg1_sweep", lambda: extra_cfg1_sweep(torch, capi, orc, dev, args.steps)), ("bert_large", lambda: extra_bert(torch))):
            try:
                extras[name] = fn()
            except SystemExit:
                raise
            except Exception as e:
                extras[name] = {"error": "%s: %s" % (type(e).__name__, str(e)[:200])}

    if rank == 0:
        peaks = measured_peaks()
        per_gpu = value / world
        roofline = {"bound": "tensor", "achieved": per_gpu, "peak": peaks["tflops_sustained"], "unit": "TFLOP/s", "frac": per_gpu / peaks["tflops_sustained"],
                    "traffic": NCU_TRAFFIC["bytes_per_launch"] if (world == 1 and full_size) else None, "traffic_source": NCU_TRAFFIC["source"], "peak_source": peaks["source"] + " (sustained dense bf16; useful FLOPs of a 2:4 MMA run at most at the dense rate)",
                    "kernel": kernel_name, "operand_form": form, "grid": kcfg["grid"],
                    "useful_flops_per_launch": flops_step / world, "launch_ms": ms_step,
                    "frac_of_burst_peak": per_gpu / peaks["tflops_burst"],
                    "algorithmic_bytes_per_launch": algorithmic_bytes(M, K, V, m, ns),
                    "hbm_frac": algorithmic_bytes(M, K, V, m, ns) / (ms_step * 1e-3) / 1e9 / peaks["hbm_gbs"]}
        cpu = None
        if not args.no_cpu_baseline:
            path = CpuCheckPath()
            path.step()
            secs = [path.step() for _ in range(3)]
            info = path.info()
            cpu = {"value": path.flops / float(np.mean(secs)) / 1e12, "unit": UNIT, "cores": info["cores"], "kind": info["kind"],
                   "sample": CPU_SAMPLE_DESC, "to_dense": info["to_dense"]}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 in / f32 accumulate", "data": "synthetic",
            "config": dict(CONFIG, **({} if full_size else {"M": M, "N": N, "note": "reduced size: not a benchmark result"})),
            "parallelism": "N-sharded x%d through ShardedSpmm / vnm_mgpu_spmm_shard (%d columns per rank, sparse operand replicated, no collective in the product)" % (world, ns),
            "clocks": clocks.summary(),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 2 * K * N, "d2h_bytes_per_step": 2 * M * N, "ms_per_step": e2e_ms,
                    "slowest_rank_h2d_gbs": h2d_rate, "slowest_rank_d2h_gbs": d2h_rate, "numa_binding_rank0": numa},
            "gpu_launches": args.steps,
            "roofline": roofline,
            "cpu_baseline": cpu,
            "speedup_vs_cublas_dense_fp16": (cublas_ms / ms_step) if cublas_ms else None,
            "cublas_dense_fp16_ms": cublas_ms,
            "parity_checked": "16 sampled rows of the headline product and 8 of the end-to-end product against the CPU oracle before timing",
            "extra": dict(extras, **({"with_allgather": gathered} if gathered else {})),
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
