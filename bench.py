#!/usr/bin/env python
"""Benchmark of the TCEC GEMM hot path.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N --steps K ...  # CPU arm (see below)

One step = one C = alpha*A*B + beta*C call through the cuMpSGEMM C ABI in
FP16TCEC mode on a seeded synthetic m = n = k = 16384 problem (A, B uniform(-1,1)
times 2^e with e uniform over the integers [-8, 8], C uniform(-1,1), alpha = 1,
beta = 0.5).  The metric is effective TFLOP/s = 2*m*n*k / t.

N = 1 : the whole problem on one GPU.
N > 1 : one process per GPU (torchrun).  C and B are split by column blocks with
        16384 columns per rank (weak scaling: n = 16384 * N), A (1 GiB) is
        broadcast from rank 0 with NCCL inside every step, then every rank runs
        its block with no further communication.

The JSON line also carries
  roofline     : the GEMM kernel's own device time (CUDA events on the launching
                 stream around the kernel, recorded by the library) against the
                 emulation roofline = measured dense 16-bit tensor peak / 3 MMAs;
  rel_err      : the accuracy half of the metric, checked after the timed region
                 on every rank: one more call on a fresh copy of C, compared on
                 sampled rows and columns with an FP64 product computed on the GPU
                 (relative Frobenius residual, the reference's criterion
                 residual < 2^-23*sqrt(K), test/main.cu:68-74; max and mean
                 relative error), next to cuBLAS FP32 SGEMM on the same inputs.
                 The worst rank is reported; the run exits non-zero above the
                 threshold;
  aux_roofline : HBM-bound helpers (split pass, exponent statistics, maximum
                 exponent, scaling) in GB/s against the measured copy bandwidth
                 (N = 1 only);
  batch_sharded: strided-batch throughput with the batch spread over the ranks
                 (complex 512 x 256^3 in FP16TCEC_SCALING, strong scaling; real
                 8 x 8192^3 per rank in AUTO, weak scaling), statistics
                 all-reduces included, one sampled batch checked against FP64;
  e2e          : the same metric with A, B, C in pinned host memory, host<->device
                 copies inside the timed region (N > 1: rank 0 uploads A once and
                 it reaches the other ranks over NVLink);
  cpu_baseline : FP32 host GEMM (the oracle's register-blocked kernel, all host
                 cores) on a bounded column slice of the same problem (rank 0,
                 N = 1 only).

`--impl reference`: the reference's own kernels target sm_80/sm_86 and depend on
three absent submodules, so there is no reference GPU arm; the CPU arm times the
FP32 host GEMM on a bounded column slice per step.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "effective TFLOP/s of FP16TCEC SGEMM at N=16384"
UNIT = "TFLOP/s"


# dram__bytes_read.sum + dram__bytes_write.sum of one GEMM-kernel launch, from a one-pass ncu
# capture of this script (--steps 1 --warmup 1, kernel filter tcec_gemm_pair); keyed by
# (mode, m, n, k).
# Algorithmic minimum for the same launch: panels 2 x 1 GiB + C read 1 GiB + C written 1 GiB.
MEASURED_DRAM_BYTES = {("FP16TCEC", 16384, 16384, 16384): 18.84e9 + 1.12e9}


def read_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"burst": float(d["bf16_tflops"]), "sustained": float(d["bf16_tflops_sustained"]),
                "source": "measured"}
    return {"burst": 1590.0, "sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None,
                "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def make_inputs_device(torch, n_rows, n_cols_b, k, seed, device):
    """Seeded uniform(-1,1) * 2^e, e in [-8, 8]; C0 uniform(-1,1).  Column-major flat storage."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)

    def scaled(count):
        u = torch.rand(count, device=device, generator=g) * 2 - 1
        e = torch.randint(-8, 9, (count,), device=device, generator=g, dtype=torch.int32)
        return torch.ldexp(u, e)

    a = scaled(n_rows * k)
    b = scaled(k * n_cols_b)
    c = torch.rand(n_rows * n_cols_b, device=device, generator=g) * 2 - 1
    return a, b, c


def oracle_with_all_cores():
    """The CPU oracle with as many OpenMP threads as this process may use.  torchrun exports
    OMP_NUM_THREADS=1 when it starts several ranks; the timed CPU arm must not inherit that."""
    cores = host_cores()
    os.environ["OMP_NUM_THREADS"] = str(cores)
    from oracle import oracle as orc

    return orc, orc.set_num_threads(cores)


def cpu_gemm_sample(n_full: int, target_seconds: float, seed: int = 1):
    """Times the oracle's FP32 host GEMM on a column slice of the n_full^3 problem.
    Returns (TFLOP/s, seconds, columns, threads)."""
    import numpy as np

    orc, threads = oracle_with_all_cores()
    m = k = n_full
    rng = orc.rng(seed)
    a = rng.uniform(-1, 1, size=m * k).astype(np.float32)
    cols_cal = 96
    b = rng.uniform(-1, 1, size=k * cols_cal).astype(np.float32)
    c = np.zeros(m * cols_cal, dtype=np.float32)
    orc.gemm_f32(0, 0, m, cols_cal, k, 1.0, a, m, b, k, 0.0, c, m)      # warm-up (threads, pages)
    t0 = time.perf_counter()
    orc.gemm_f32(0, 0, m, cols_cal, k, 1.0, a, m, b, k, 0.0, c, m)
    per_col = max((time.perf_counter() - t0) / cols_cal, 1e-7)
    cols = int(max(cols_cal, min(n_full, target_seconds / per_col)))
    cols = max(6, cols // 6 * 6)
    b = rng.uniform(-1, 1, size=k * cols).astype(np.float32)
    c = np.zeros(m * cols, dtype=np.float32)
    t0 = time.perf_counter()
    orc.gemm_f32(0, 0, m, cols, k, 1.0, a, m, b, k, 0.0, c, m)
    dt = time.perf_counter() - t0
    return 2.0 * m * cols * k / dt / 1e12, dt, cols, threads


def run_reference(args, rank, world):
    """CPU arm: FP32 host GEMM on the box's host cores, bounded sample per step."""
    if rank != 0:
        return
    import numpy as np

    orc, threads = oracle_with_all_cores()
    n_full = args.n
    m = k = n_full
    rng = orc.rng(1)
    a = rng.uniform(-1, 1, size=m * k).astype(np.float32)
    # size one step at about 3 s
    tf, dt, cols, _ = cpu_gemm_sample(n_full, 3.0)
    b = rng.uniform(-1, 1, size=k * cols).astype(np.float32)
    c = rng.uniform(-1, 1, size=m * cols).astype(np.float32)
    for _ in range(args.warmup):
        orc.gemm_f32(0, 0, m, cols, k, 1.0, a, m, b, k, 0.5, c, m)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.gemm_f32(0, 0, m, cols, k, 1.0, a, m, b, k, 0.5, c, m)
    dt = time.perf_counter() - t0
    ms = dt / args.steps * 1e3
    value = 2.0 * m * cols * k * args.steps / dt / 1e12
    sample = (f"FP32 host GEMM (oracle port of the path's arithmetic in plain FP32), m=k={n_full}, "
              f"{cols} of {n_full} columns per step, {threads} OpenMP threads "
              f"(omp_get_max_threads; {host_cores()} cores in the affinity mask)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"FP32 SGEMM m=k={n_full}, column slice n={cols}, alpha=1, beta=0.5",
                   "note": "the reference's GPU kernels (sm_80/sm_86, absent submodules) cannot "
                           "be built; this arm is the CPU restatement on host cores"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------- accuracy
SAMPLE_ROWS = 6
SAMPLE_COLS = 4


def sample_indices(m, n):
    rows = sorted({0, 1, min(127, m - 1), min(128, m - 1), min(m // 2 + 3, m - 1), m - 1})
    cols = sorted({0, min(255, n - 1), min(256, n - 1), n - 1})
    return rows, cols


def fp64_samples(torch, a, b, c0, m, n, k, beta, rows, cols, chunk=2048):
    """FP64 truth of alpha=1, op N/N on the sampled rows (returned as n x len(rows)) and
    columns (len(cols) x m) of column-major flat operands, computed on the GPU in chunks so
    that no full-size FP64 copy of an operand is made."""
    av, bv, cv = a.view(k, m), b.view(n, k), c0.view(n, m)      # av[l, i] = A(i, l) etc.
    a_rows = av[:, rows].double()                               # k x R
    t_rows = torch.empty(n, len(rows), dtype=torch.float64, device=a.device)
    for j0 in range(0, n, chunk):
        j1 = min(n, j0 + chunk)
        t_rows[j0:j1] = bv[j0:j1].double() @ a_rows
    t_rows += beta * cv[:, rows].double()
    b_cols = bv[cols].double()                                  # Ccount x k
    t_cols = torch.zeros(len(cols), m, dtype=torch.float64, device=a.device)
    for l0 in range(0, k, chunk):
        l1 = min(k, l0 + chunk)
        t_cols += b_cols[:, l0:l1] @ av[l0:l1].double()
    t_cols += beta * cv[cols].double()
    return t_rows, t_cols


def sampled_errors(torch, truth_rows, truth_cols, got_flat, m, n, rows, cols):
    gv = got_flat.view(n, m)
    t = torch.cat([truth_rows.reshape(-1), truth_cols.reshape(-1)])
    g = torch.cat([gv[:, rows].double().reshape(-1), gv[cols].double().reshape(-1)])
    diff = (t - g).abs()
    residual = (diff.pow(2).sum() / t.pow(2).sum()).sqrt().item()
    nz = t != 0
    rel = diff[nz] / t[nz].abs()
    return residual, rel.max().item(), rel.mean().item()


def accuracy_block(torch, dist, device, step_into, a, b, c0, m, n, k, beta):
    """One more call on a fresh copy of C, compared with FP64 on sampled rows and columns; the
    same for cuBLAS FP32 SGEMM.  Worst rank wins."""
    rows, cols = sample_indices(m, n)
    c_chk = c0.clone()
    step_into(c_chk)
    torch.cuda.synchronize()
    t_rows, t_cols = fp64_samples(torch, a, b, c0, m, n, k, beta, rows, cols)
    res, mx, mean = sampled_errors(torch, t_rows, t_cols, c_chk, m, n, rows, cols)
    del c_chk
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    # column-major C = A B  <=>  row-major C^T (n x m) = B^T (n x k) A^T (k x m)
    c32 = torch.addmm(c0.view(n, m), b.view(n, k), a.view(k, m), beta=beta, alpha=1.0)
    torch.backends.cuda.matmul.allow_tf32 = prev
    res32, mx32, mean32 = sampled_errors(torch, t_rows, t_cols, c32.reshape(-1), m, n, rows, cols)
    del c32
    vals = torch.tensor([res, mx, mean, res32, mx32, mean32], device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    res, mx, mean, res32, mx32, mean32 = (float(v) for v in vals.tolist())
    threshold = 2.0 ** -23 * (k ** 0.5)
    return {
        "residual": res, "threshold": threshold, "max": mx, "mean": mean,
        "fp32_simt_residual": res32, "fp32_simt_max": mx32, "fp32_simt_mean": mean32,
        "passed": bool(res < threshold),
        "samples": f"rows {rows} and columns {cols} of every rank's C block "
                   f"({len(rows) * n + len(cols) * m} entries per rank), FP64 truth computed on "
                   "the GPU; worst rank reported",
        "comparator": "cuBLAS FP32 SGEMM (torch.addmm, TF32 off) on the same inputs",
    }, (rows, t_rows)


def host_row_check(torch, a, b, c0, m, n, k, beta, row, truth_row_gpu):
    """Cross-check of the GPU's FP64 truth on one row against the host oracle's FP64 GEMM."""
    import numpy as np

    orc, _ = oracle_with_all_cores()
    ah, bh, ch = a.cpu().numpy(), b.cpu().numpy(), c0.cpu().numpy()
    truth = orc.gemm_f64(0, 0, 1, n, k, 1.0, ah[row:], m, bh, k, beta, ch[row:], m).reshape(-1)
    g = truth_row_gpu.cpu().numpy()
    return float(np.abs(truth - g).max() / np.abs(truth).max())


# ---------------------------------------------------------------------- helpers' bandwidth
def aux_rooflines(torch, handle, device, split_ms, n_main, hbm):
    """GB/s of the HBM-bound helpers: the split pass of the main problem (from the library's
    own events) and statistics / maximum exponent / scaling on 8192 x 8192 FP32 inputs."""
    out = {}

    def entry(ms, nbytes, what):
        gbs = nbytes / ms / 1e6
        return {"ms": ms, "bytes": nbytes, "gbs": gbs, "frac": (gbs / hbm) if hbm else None,
                "algorithmic_bytes": what}

    if split_ms > 0:
        out["split_dual_kernel"] = entry(
            split_ms, 16.0 * n_main * n_main,
            "2 operands x N^2 x (4 B read + 2 x 2 B hi/lo written)")
    n = 8192
    g = torch.Generator(device=device)
    g.manual_seed(5)
    sgn = torch.where(torch.rand(n * n, device=device, generator=g) < 0.5, -1.0, 1.0)
    x = torch.ldexp(sgn * (1 + torch.rand(n * n, device=device, generator=g)),
                    torch.randint(-30, 11, (n * n,), device=device, generator=g,
                                  dtype=torch.int32))
    y = torch.rand(n * n, device=device, generator=g) + 1
    nbytes = 4.0 * n * n
    sid = handle.exp_max_ext(n, n, y, n)

    def timeit(fn, iters=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    out["exp_stats_ext (both stages run: wide exponent range)"] = entry(
        timeit(lambda: handle.exp_stats_ext(n, n, x, n)), 2 * nbytes, "2 passes x m*n*4 B read")
    out["exp_max_ext"] = entry(timeit(lambda: handle.exp_max_ext(n, n, x, n)), nbytes,
                               "m*n*4 B read")
    out["scale_A + reset_scale_A (in place)"] = entry(
        timeit(lambda: (handle.scale_A(sid, 1, n, n, y, n), handle.reset_scale_A(sid, 1, n, n, y, n))),
        4 * nbytes, "2 calls x m*n*4 B read + written")
    return {"unit": "GB/s", "peak": hbm, "peak_source": "measured copy bandwidth",
            "inputs": f"{n} x {n} FP32 (268 MB, larger than L2), 20 calls each", "kernels": out}


# ---------------------------------------------------------------------- batch partition
def batch_sharded_block(torch, dist, device, sharded, rank, world):
    """Strided-batch throughput with the batch spread over the ranks, through
    ShardedGemm.gemm_strided_batch_local (its statistics all-reduces are inside the time)."""
    from cumpsgemm_b200 import api
    from cumpsgemm_b200.sharded import batch_range

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, warmup, steps):
        for _ in range(warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1) / steps], device=device, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def worst(x):
        t = torch.tensor([x], device=device, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    out = {}
    g = torch.Generator(device=device)
    g.manual_seed(4242 + rank)
    # complex 512 x 256^3, unit Frobenius norm per matrix, FP16TCEC_SCALING; strong scaling
    total, s = 512, 256
    b0, b1 = batch_range(total, world, rank)
    nb = b1 - b0

    def unit(count):
        z = torch.complex(torch.randn(count, s * s, device=device, generator=g),
                          torch.randn(count, s * s, device=device, generator=g))
        return (z / z.abs().pow(2).sum(1, keepdim=True).sqrt()).to(torch.complex64).contiguous()

    za, zb = unit(nb), unit(nb)
    zc = torch.zeros(nb * s * s, dtype=torch.complex64, device=device)
    mode = api.ComputeMode.FP16TCEC_SCALING
    ms = timed(lambda: sharded.gemm_strided_batch_local(0, 0, s, s, s, 1.0, za, s, s * s, zb, s,
                                                        s * s, 0.0, zc, s, s * s, nb, mode), 3, 20)
    i = nb // 2
    A = za[i].view(s, s).t().to(torch.complex128)
    B = zb[i].view(s, s).t().to(torch.complex128)
    got = zc.view(nb, s, s)[i].t().to(torch.complex128)
    truth = A @ B
    res = ((truth - got).abs().pow(2).sum() / truth.abs().pow(2).sum()).sqrt().item()
    out["cgemm_512x256^3_FP16TCEC_SCALING"] = {
        "scaling": "strong", "batches_per_rank": nb, "ms": ms,
        "tflops": 8.0 * total * s ** 3 / ms / 1e9,
        "sampled_batch_residual": worst(res), "threshold": 2.0 ** -23 * s ** 0.5,
        "collectives": "one 64-byte all-gather (both operands' maximum exponents) when world > 1"}
    del za, zb, zc
    # real 8 x 8192^3 per rank, N(0,1), AUTO; weak scaling
    n, nb = 8192, 8
    a = torch.randn(nb * n * n, device=device, generator=g)
    b = torch.randn(nb * n * n, device=device, generator=g)
    c = torch.zeros(nb * n * n, device=device)
    mode = api.ComputeMode.AUTO
    ms = timed(lambda: sharded.gemm_strided_batch_local(0, 0, n, n, n, 1.0, a, n, n * n, b, n,
                                                        n * n, 0.0, c, n, n * n, nb, mode), 1, 3)
    i = 5
    rows = [0, 129, n - 1]
    Ar = a[i * n * n:(i + 1) * n * n].view(n, n)[:, rows].double()            # k x R
    truth = b[i * n * n:(i + 1) * n * n].view(n, n).double() @ Ar              # n x R
    got = c[i * n * n:(i + 1) * n * n].view(n, n)[:, rows].double()
    res = ((truth - got).pow(2).sum() / truth.pow(2).sum()).sqrt().item()
    out["sgemm_8x8192^3_per_rank_AUTO"] = {
        "scaling": "weak", "batches_per_rank": nb, "ms": ms,
        "tflops": 2.0 * nb * world * n ** 3 / ms / 1e9,
        "sampled_batch_residual": worst(res), "threshold": 2.0 ** -23 * n ** 0.5,
        "collectives": "two 64-byte all-gathers (both operands' slot words after each statistics "
                       "stage) when world > 1"}
    del a, b, c
    return out


def run_ours(args, rank, local_rank, world):
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=device)

    from cumpsgemm_b200 import api
    from cumpsgemm_b200.sharded import ShardedGemm

    mode = api.ComputeMode[args.mode]
    n = args.n
    m = k = n
    n_local = n                      # weak scaling: every rank owns n columns of C
    handle = api.Handle()
    handle.use_current_torch_stream()
    sharded = ShardedGemm(handle)

    a, b, c = make_inputs_device(torch, m, n_local, k, seed=1234 + rank, device=device)
    c0 = c.clone()
    if world > 1 and rank != 0:
        a.zero_()                    # content arrives through the broadcast in every step

    def step_into(c_out):
        if world > 1:
            sharded.gemm_column_block(0, 0, m, n_local, k, 1.0, a, m, b, k, args.beta, c_out, m,
                                      mode, root=0, broadcast_A=True)
        else:
            handle.gemm(0, 0, m, n_local, k, 1.0, a, m, b, k, args.beta, c_out, m, mode)

    def step():
        step_into(c)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    handle.set_kernel_timing(True)
    handle.get_kernel_timing()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    elapsed_ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    groups, split_ms, gemm_ms = handle.get_kernel_timing()
    handle.set_kernel_timing(False)
    kstatus = handle.kernel_status()
    if dist is not None:
        t = torch.tensor([elapsed_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    flops_per_step = 2.0 * m * (n_local * world) * k
    value = flops_per_step / (ms_per_step * 1e-3) / 1e12

    # ---- roofline of the dominant kernel (the tcgen05 GEMM kernel), this rank
    peaks = read_peaks()
    long_run = elapsed_ms > 2000.0
    peak_dense = peaks["sustained"] if long_run else peaks["burst"]
    mma_per_product = 3 if mode in (api.ComputeMode.FP16TCEC, api.ComputeMode.FP16TCEC_SCALING,
                                    api.ComputeMode.AUTO) else (3 if mode == api.ComputeMode.TF32TCEC
                                                                else 1)
    tf32 = mode in (api.ComputeMode.TF32TCEC, api.ComputeMode.TF32TC)
    peak = peak_dense / (2.0 if tf32 else 1.0) / mma_per_product
    gemm_ms_avg = gemm_ms / max(groups, 1)
    split_ms_avg = split_ms / max(groups, 1)
    achieved = 2.0 * m * n_local * k / (gemm_ms_avg * 1e-3) / 1e12 if gemm_ms_avg > 0 else 0.0
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
        "frac": achieved / peak if peak else None,
        "traffic": MEASURED_DRAM_BYTES.get((mode.name, m, n_local, k)),
        "kernel": "tcec_gemm_pair_kernel (tcgen05 cta_group::2, 256x256 tile per CTA pair)",
        "kernel_ms": gemm_ms_avg, "split_pass_ms": split_ms_avg,
        "peak_source": f"{peaks['source']} dense 16-bit tensor peak "
                       f"({'sustained' if long_run else 'burst'}) {peak_dense} TFLOP/s / "
                       f"{'2 (TF32) / ' if tf32 else ''}{mma_per_product} MMAs per product",
    }

    # ---- accuracy (outside the timed region): the other half of the metric
    rel_err, row_truth = None, None
    if not args.skip_check:
        rel_err, row_truth = accuracy_block(torch, dist, device, step_into, a, b, c0, m, n_local,
                                            k, args.beta)

    # ---- end to end through host buffers (rank-local problem, max over ranks)
    e2e = None
    if args.e2e_steps > 0:
        host = api.HostGemm(handle, device)
        bh = torch.empty(b.numel(), dtype=torch.float32, pin_memory=True)
        ch = torch.empty(c.numel(), dtype=torch.float32, pin_memory=True)
        bh.copy_(b)
        ch.copy_(c)
        ah = None
        if rank == 0:
            ah = torch.empty(a.numel(), dtype=torch.float32, pin_memory=True)
            ah.copy_(a)
        # the device tensors of the resident run double as staging buffers
        host.adopt_staging(A=a, B=b, C=c)
        side = torch.cuda.Stream(device=device)
        torch.cuda.synchronize()

        def e2e_step():
            if world == 1:
                return host.gemm(0, 0, m, n_local, k, 1.0, ah, m, bh, k, args.beta, ch, m, mode)
            # rank 0 uploads A once; it reaches the other ranks over NVLink while they already
            # upload their own B and C blocks
            caller = torch.cuda.current_stream(device)
            ev = torch.cuda.Event()
            ev.record(caller)
            with torch.cuda.stream(side):
                side.wait_event(ev)
                if rank == 0:
                    a.copy_(ah, non_blocking=True)
                dist.broadcast(a, src=0)
                ready = torch.cuda.Event()
                ready.record(side)
            h2d, d2h = host.gemm(0, 0, m, n_local, k, 1.0, None, m, bh, k, args.beta, ch, m, mode,
                                 A_device=a, A_ready=ready)
            return h2d + (a.numel() * 4 if rank == 0 else 0), d2h

        h2d, d2h = e2e_step()
        barrier()
        e0.record()
        for _ in range(args.e2e_steps):
            h2d, d2h = e2e_step()
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1) / args.e2e_steps
        totals = torch.tensor([e2e_ms, float(h2d), float(d2h)], device=device, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(totals[0:1], op=dist.ReduceOp.MAX)
            dist.all_reduce(totals[1:3], op=dist.ReduceOp.SUM)
        e2e_ms, h2d, d2h = float(totals[0]), int(totals[1]), int(totals[2])
        e2e = {"value": 2.0 * m * (n_local * world) * k / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
               "steps": args.e2e_steps,
               "note": "api.HostGemm: operands in pinned host memory, copies inside the timed "
                       "region, pipelined over 16 column blocks per rank; bytes are whole-job "
                       "sums over the ranks" +
                       ("" if world == 1 else "; A is uploaded by rank 0 only and broadcast "
                                              "with NCCL while the other ranks upload B and C")}
        del bh, ch, ah

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        tf, dt, cols, threads = cpu_gemm_sample(n, 15.0)
        cpu = {"value": tf, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"FP32 host GEMM on {cols} of {n} columns of an m=k={n} problem "
                         f"({dt:.1f} s, {threads} OpenMP threads)"}
        if row_truth is not None:
            rows, t_rows = row_truth
            j = rows.index(min(128, m - 1)) if min(128, m - 1) in rows else 0
            cpu["fp64_truth_cross_check"] = {
                "row": rows[j],
                "max_abs_diff_over_max_abs": host_row_check(torch, a, b, c0, m, n_local, k,
                                                            args.beta, rows[j], t_rows[:, j]),
                "what": "the GPU-computed FP64 truth of one sampled row against the host "
                        "oracle's FP64 GEMM"}

    aux = None
    if world == 1 and not args.skip_aux:
        hbm = None
        pk = ROOT / "MEASURED_PEAKS.json"
        if pk.exists():
            hbm = float(json.loads(pk.read_text())["hbm_gbs"])
        aux = aux_rooflines(torch, handle, device, split_ms_avg, n, hbm or 6650.0)
        if hbm is None:
            aux["peak_source"] = "fallback 6650 GB/s"

    del a, b, c, c0
    torch.cuda.empty_cache()
    batch = None
    if not args.skip_batch:
        batch = batch_sharded_block(torch, dist, device, sharded, rank, world)
    kstatus = kstatus or handle.kernel_status()

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16" if not tf32 else "tf32",
            "data": "synthetic",
            "config": {
                "workload": (f"SGEMM {mode.name} NN column-major m=k={n}, n={n_local * world} "
                             f"({n_local} columns per GPU), alpha=1, beta={args.beta}, "
                             "A,B ~ U(-1,1)*2^e e in [-8,8], C ~ U(-1,1)"),
                "parallelism": ("single GPU" if world == 1 else
                                f"C/B column blocks over {world} GPUs, A broadcast from rank 0 "
                                "with NCCL inside every step"),
                "l2": (f"A, B, C are {m * k * 4 / 2**20:.0f} + {k * n_local * 4 / 2**20:.0f} + "
                       f"{m * n_local * 4 / 2**20:.0f} MiB per GPU against a 126 MB L2; "
                       "no explicit flush"),
            },
            "roofline": roofline, "rel_err": rel_err, "aux_roofline": aux, "batch_sharded": batch,
            "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": 2 * args.steps * (2 if mode == api.ComputeMode.AUTO else 1),
            "kernel_status": kstatus, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    handle.destroy()
    if rel_err is not None and not rel_err["passed"]:
        raise SystemExit(f"accuracy check failed: residual {rel_err['residual']:.3e} >= "
                         f"threshold {rel_err['threshold']:.3e}")


def run_sweep(args):
    """Documentation runs for the other benchmark configurations (one JSON line each, marked
    "sweep": true): square SGEMM sweep in both kinds, the wide-exponent SCALING / AUTO case,
    the strided-batch complex case, and the bandwidth of the statistics / scaling kernels."""
    import torch

    from cumpsgemm_b200 import api

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    h = api.Handle()
    h.use_current_torch_stream()
    g = torch.Generator(device=dev)
    g.manual_seed(99)
    hbm = None
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        hbm = float(json.loads(pk.read_text())["hbm_gbs"])

    def timeit(fn, iters):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    def emit(**kw):
        kw["sweep"] = True
        print(json.dumps(kw), flush=True)

    def uexp(count, lo, hi):
        u = torch.rand(count, device=dev, generator=g) * 2 - 1
        e = torch.randint(lo, hi + 1, (count,), device=dev, generator=g, dtype=torch.int32)
        return torch.ldexp(u, e)

    # config 1 and 2: square SGEMM
    for n in (1024, 2048, 4096, 8192, 16384):
        a, b = uexp(n * n, -8, 8), uexp(n * n, -8, 8)
        c = torch.rand(n * n, device=dev, generator=g) * 2 - 1
        for mode in ("FP16TCEC", "TF32TCEC"):
            ms = timeit(lambda: h.gemm(0, 0, n, n, n, 1.0, a, n, b, n, 0.5, c, n,
                                       api.ComputeMode[mode]), 20 if n <= 8192 else 5)
            emit(config=f"sgemm {mode} m=n=k={n} beta=0.5", ms=ms, tflops=2.0 * n ** 3 / ms / 1e9)
        del a, b, c
    # config 3: wide exponent range, 8192^3, SCALING and AUTO; statistics / scaling bandwidth
    n = 8192
    sgn = torch.where(torch.rand(n * n, device=dev, generator=g) < 0.5, -1.0, 1.0)
    a = torch.ldexp(sgn * (1 + torch.rand(n * n, device=dev, generator=g)),
                    torch.randint(-30, 11, (n * n,), device=dev, generator=g, dtype=torch.int32))
    b = a.flip(0).contiguous()
    c = torch.zeros(n * n, device=dev)
    for mode in ("FP16TCEC_SCALING", "AUTO"):
        lib_mode = api.ComputeMode[mode]
        if mode == "AUTO":
            def call():
                ia = h.exp_stats_ext(n, n, a, n)
                ib = h.exp_stats_ext(n, n, b, n)
                h.gemm_strided_batch_with_stats(0, 0, n, n, n, 1.0, a, n, 0, b, n, 0, 0.0, c, n, 0,
                                                1, lib_mode, ia, ib)
        else:
            def call():
                h.gemm(0, 0, n, n, n, 1.0, a, n, b, n, 0.0, c, n, lib_mode)
        ms = timeit(call, 10)
        emit(config=f"sgemm {mode} m=n=k={n} exponents in [-30,10] (statistics + fused scaling + GEMM)",
             ms=ms, tflops=2.0 * n ** 3 / ms / 1e9)
    nbytes = n * n * 4
    for name, fn, traffic in (
            ("exp_stats_ext (stage 1 + stage 2, wide range)", lambda: h.exp_stats_ext(n, n, a, n), 2 * nbytes),
            ("exp_max_ext", lambda: h.exp_max_ext(n, n, a, n), nbytes),
            ("scale_A then reset_scale_A (in place, read + write each)",
             lambda: (h.scale_A(sid, 1, n, n, c2, n), h.reset_scale_A(sid, 1, n, n, c2, n)), 4 * nbytes)):
        if name.startswith("scale"):
            c2 = torch.rand(n * n, device=dev, generator=g) + 1
            sid = h.exp_max_ext(n, n, c2, n)
        ms = timeit(fn, 20)
        gbs = traffic / ms / 1e6
        emit(config=f"{name} on {n}x{n} FP32", ms=ms, gbs=gbs,
             frac_of_measured_hbm=(gbs / hbm if hbm else None))
    del a, b, c
    # config 4: strided-batch complex GEMM, unit-Frobenius operands, SCALING
    batch, s = 512, 256
    za = torch.randn(batch, s * s, device=dev, generator=g, dtype=torch.float32) + \
        1j * torch.randn(batch, s * s, device=dev, generator=g, dtype=torch.float32)
    zb = torch.randn(batch, s * s, device=dev, generator=g, dtype=torch.float32) + \
        1j * torch.randn(batch, s * s, device=dev, generator=g, dtype=torch.float32)
    za = (za / za.abs().pow(2).sum(1, keepdim=True).sqrt()).to(torch.complex64).contiguous()
    zb = (zb / zb.abs().pow(2).sum(1, keepdim=True).sqrt()).to(torch.complex64).contiguous()
    zc = torch.zeros(batch * s * s, dtype=torch.complex64, device=dev)
    for mode in ("FP16TCEC", "FP16TCEC_SCALING"):
        ms = timeit(lambda: h.gemm_strided_batch(0, 0, s, s, s, 1.0, za, s, s * s, zb, s, s * s, 0.0,
                                                 zc, s, s * s, batch, api.ComputeMode[mode]), 20)
        emit(config=f"cgemm strided batch {mode} batch={batch} m=n=k={s}", ms=ms,
             tflops=8.0 * batch * s ** 3 / ms / 1e9)
    del za, zb, zc
    # the regimes the on-the-fly split kernel and split-K exist for: many small products, and
    # few tiles with a long K
    batch, s = 2048, 128
    a = torch.rand(batch * s * s, device=dev, generator=g) * 2 - 1
    b = torch.rand(batch * s * s, device=dev, generator=g) * 2 - 1
    c = torch.zeros(batch * s * s, device=dev)
    ms = timeit(lambda: h.gemm_strided_batch(0, 0, s, s, s, 1.0, a, s, s * s, b, s, s * s, 0.0, c, s,
                                             s * s, batch, api.ComputeMode.FP16TCEC), 20)
    emit(config=f"sgemm strided batch FP16TCEC batch={batch} m=n=k={s}", ms=ms,
         tflops=2.0 * batch * s ** 3 / ms / 1e9)
    m, k = 256, 65536
    a = torch.rand(m * k, device=dev, generator=g) * 2 - 1
    b = torch.rand(k * m, device=dev, generator=g) * 2 - 1
    c = torch.zeros(m * m, device=dev)
    ms = timeit(lambda: h.gemm(0, 0, m, m, k, 1.0, a, m, b, k, 0.0, c, m, api.ComputeMode.FP16TCEC), 20)
    emit(config=f"sgemm FP16TCEC m=n={m} k={k} (split-K)", ms=ms, tflops=2.0 * m * m * k / ms / 1e9)
    del a, b, c
    if args.sweep_large:
        # config 5a, one GPU's share at 8 GPUs: batch 8 of 8192^3, N(0,1), AUTO
        n, batch = 8192, 8
        a = torch.randn(batch * n * n, device=dev, generator=g)
        b = torch.randn(batch * n * n, device=dev, generator=g)
        c = torch.zeros(batch * n * n, device=dev)
        ms = timeit(lambda: h.gemm_strided_batch(0, 0, n, n, n, 1.0, a, n, n * n, b, n, n * n,
                                                 0.0, c, n, n * n, batch,
                                                 api.ComputeMode.FP16TCEC), 3)
        emit(config=f"sgemm strided batch FP16TCEC batch={batch} m=n=k={n} N(0,1)", ms=ms,
             tflops=2.0 * batch * n ** 3 / ms / 1e9)

        def auto_call():
            ia = h.exp_stats_ext(n, n, a, n, batch, n * n)
            ib = h.exp_stats_ext(n, n, b, n, batch, n * n)
            h.gemm_strided_batch_with_stats(0, 0, n, n, n, 1.0, a, n, n * n, b, n, n * n, 0.0, c, n,
                                            n * n, batch, api.ComputeMode.AUTO, ia, ib)
        ms = timeit(auto_call, 3)
        emit(config=f"sgemm strided batch AUTO batch={batch} m=n=k={n} N(0,1) (statistics + GEMM)",
             ms=ms, tflops=2.0 * batch * n ** 3 / ms / 1e9)
        del a, b, c
        # config 5b on one GPU: m=n=65536, k=8192, N(0,1)
        m, k = 65536, 8192
        a = torch.randn(m * k, device=dev, generator=g)
        b = torch.randn(k * m, device=dev, generator=g)
        c = torch.zeros(m * m, device=dev)
        ms = timeit(lambda: h.gemm(0, 0, m, m, k, 1.0, a, m, b, k, 0.0, c, m,
                                   api.ComputeMode.FP16TCEC), 2)
        # spot check of three rows against FP64 on the GPU
        A = a.view(k, m).t()
        B = b.view(m, k).t()
        worst = 0.0
        for i in (0, 40000, m - 1):
            truth = A[i].double() @ B.double()
            got = c.view(m, m)[:, i].double()
            worst = max(worst, ((truth - got).norm() / truth.norm()).item())
        emit(config=f"sgemm FP16TCEC m=n={m} k={k} N(0,1), one GPU", ms=ms,
             tflops=2.0 * m * m * k / ms / 1e9, worst_row_residual=worst)
        del a, b, c
    status = h.kernel_status()
    emit(config="kernel status after sweep", status=status)
    h.destroy()


def run_case(args):
    """One small configuration alone (for profiler captures and quick timings; one JSON line
    marked "case": true): --case sgemm | sgemm_batch | cgemm_batch with --n (m=n=k), --batch,
    --mode, --beta, --steps, --warmup."""
    import torch

    from cumpsgemm_b200 import api

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    h = api.Handle()
    h.use_current_torch_stream()
    g = torch.Generator(device=dev)
    g.manual_seed(7)
    n, batch = args.n, (args.batch if args.case != "sgemm" else 1)
    mode = api.ComputeMode[args.mode]
    cplx = args.case == "cgemm_batch"
    count = batch * n * n

    def rnd():
        x = torch.rand(count * (2 if cplx else 1), device=dev, generator=g) * 2 - 1
        return torch.view_as_complex(x.view(-1, 2)) if cplx else x
    a, b, c = rnd(), rnd(), rnd()
    if args.case == "sgemm":
        def call():
            h.gemm(0, 0, n, n, n, 1.0, a, n, b, n, args.beta, c, n, mode)
    else:
        def call():
            h.gemm_strided_batch(0, 0, n, n, n, 1.0, a, n, n * n, b, n, n * n, args.beta, c, n,
                                 n * n, batch, mode)
    for _ in range(args.warmup):
        call()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        call()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    flops = (8.0 if cplx else 2.0) * batch * n ** 3
    print(json.dumps({"case": True, "config": f"{args.case} {args.mode} batch={batch} m=n=k={n} "
                      f"beta={args.beta}", "ms": ms, "tflops": flops / ms / 1e9,
                      "steps": args.steps, "kernel_status": h.kernel_status()}), flush=True)
    h.destroy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--n", type=int, default=16384)
    ap.add_argument("--mode", default="FP16TCEC")
    ap.add_argument("--beta", type=float, default=0.5)
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--skip-check", action="store_true", help="leave the accuracy block out")
    ap.add_argument("--skip-aux", action="store_true", help="leave the helper bandwidths out")
    ap.add_argument("--skip-batch", action="store_true", help="leave the batch-sharded block out")
    ap.add_argument("--sweep-large", action="store_true",
                    help="with --sweep: also the 8 x 8192^3 batch and the 65536 x 65536 x 8192 GEMM")
    ap.add_argument("--case", default=None, choices=["sgemm", "sgemm_batch", "cgemm_batch"],
                    help="run one small configuration alone (see run_case)")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--sweep", action="store_true",
                    help="run the other benchmark configurations (documentation runs)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.sweep:
        run_sweep(args)
        return
    if args.case is not None:
        run_case(args)
        return
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
