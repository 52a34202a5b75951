#!/usr/bin/env python3
"""Benchmark of the quantized-Gram hot path behind hyacinTsvdFit.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--rows-log2 20] [--n 4096]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (BASELINE configuration 2; configuration 3 for N > 1, weak scaling): real FP64, opA = 'N', 2^20 rows per
GPU, 4096 columns, eps = 1e-10; A = (Gaussian / sqrt(M)) diag(10^(-14 i / 4095)) V^T with orthonormal V and
log-uniform column scales in [1e-3, 1e3], generated on the device from fixed seeds (synthetic; the reference
publishes no dataset).

One step = one pass of the hot path over the local matrix:
    hyacinXquantizeScaleBatch -> hyacinAllReduceVExp -> hyacinXherkBatch -> hyacinAllReduce1Drow
    -> hyacinXdequantizeInit -> hyacinXdequantize
`value` is FP64-equivalent Gram TFLOP/s = globalM N (N + 1) / time with A resident in HBM; `e2e` is the same
figure through hyacinTsvdFit with the matrix coming from pinned host memory and S, V going back to the host
every step.  The dominant kernel (tcgen05 residue Gram) is timed in situ with CUDA events on its own stream.
`--impl reference` drives the reference's own CUDA library (oracle/_ref, built from the reference sources)
through the same C ABI on the same GPUs -- the reference has no CPU implementation of this path; the CPU
baseline reported next to it is LAPACK dsyrk + dsyevd on the host cores.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

REF_LIB = os.path.join(ROOT, "oracle", "_ref", "libhyacin_ref.so")
PEAKS = os.path.join(ROOT, "MEASURED_PEAKS.json")
EPS = 1e-10
# DRAM traffic of the Gram kernel from an ncu capture of a smaller launch (16384 rows, 13 moduli, N = 4096):
# 1.92 GB read and 116 MB written.  Reads grow in proportion to rows x moduli (9016 bytes per row and modulus),
# the residue bytes written (and re-read when accumulating) depend on N and the moduli only.
GRAM_DRAM_READ_BYTES_PER_ROW_MODULUS = 9016.0
GRAM_TRAFFIC_SOURCE = "ncu dram__bytes_read.sum + dram__bytes_write.sum of a 16384-row launch (profiles/gram_pair_kernel_n4096_rows16384.txt), reads scaled by rows"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--rows-log2", type=int, default=20, help="log2 of the rows per GPU (20 = the headline workload)")
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-fit", action="store_true", help="skip the hyacinTsvdFit timings (hot path only, e.g. under a profiler)")
    ap.add_argument("--complex", action="store_true",
                    help="complex FP64 input (the Gram of BASELINE configuration 4: use --rows-log2 19 --n 2048): hot path only, "
                         "for profiles of the complex route; not the headline workload")
    return ap.parse_args()


# ---------------------------------------------------------------------------------------------------------
# plumbing: process group, NCCL communicator for the handle, clocks
# ---------------------------------------------------------------------------------------------------------
class _NcclId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_byte * 128)]


def make_nccl_comm(torch, dist, rank, world):
    """ncclComm_t for the handle (the library borrows it, as the reference does)."""
    nccl = ctypes.CDLL("libnccl.so.2")
    uid = _NcclId()
    if rank == 0:
        assert nccl.ncclGetUniqueId(ctypes.byref(uid)) == 0
    buf = torch.frombuffer(bytearray(bytes(uid)), dtype=torch.uint8).cuda()
    dist.broadcast(buf, 0)
    ctypes.memmove(ctypes.byref(uid), bytes(buf.cpu().numpy().tobytes()), 128)
    comm = ctypes.c_void_p()
    nccl.ncclCommInitRank.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, _NcclId, ctypes.c_int]
    assert nccl.ncclCommInitRank(ctypes.byref(comm), world, uid, rank) == 0
    return nccl, comm


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.file.name)
        if sm:
            # samples taken under load: the upper half of the observed clocks is idle time between steps
            out["sm_mhz"] = statistics.median(sm)
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


# ---------------------------------------------------------------------------------------------------------
# workload
# ---------------------------------------------------------------------------------------------------------
def make_complex_matrix(torch, rows, n, seed):
    """Column-major rows x n complex FP64 matrix (rank 200, singular values 1 .. 1e-13, noise 1e-15): tensor (n, rows)."""
    g = torch.Generator(device="cuda")
    g.manual_seed(20240611 + 4)
    r = min(200, n)
    W, _ = torch.linalg.qr(torch.randn(n, r, dtype=torch.complex128, device="cuda", generator=g))
    s = 10.0 ** (-13.0 * torch.arange(r, dtype=torch.float64, device="cuda") / max(r - 1, 1))
    g.manual_seed(seed)
    At = torch.empty((n, rows), dtype=torch.complex128, device="cuda")
    blk = 1 << 15
    for r0 in range(0, rows, blk):
        k = min(blk, rows - r0)
        U = torch.randn(k, r, dtype=torch.complex128, device="cuda", generator=g) / (rows ** 0.5)
        At[:, r0:r0 + k] = ((U * s) @ W.conj().T + 1e-15 * torch.randn(k, n, dtype=torch.complex128, device="cuda", generator=g)).T
    return At


def make_matrix(torch, rows, n, seed):
    """Column-major rows x n FP64 matrix on the device as a tensor of shape (n, rows)."""
    g = torch.Generator(device="cuda")
    g.manual_seed(20240611 + 2)                    # V, spectrum and column scales are shared by all ranks
    V, _ = torch.linalg.qr(torch.randn(n, n, dtype=torch.float64, device="cuda", generator=g))
    s = 10.0 ** (-14.0 * torch.arange(n, dtype=torch.float64, device="cuda") / max(n - 1, 1))
    scale = 10.0 ** (torch.rand(n, dtype=torch.float64, device="cuda", generator=g) * 6.0 - 3.0)
    B = (s[:, None] * V.T) * scale[None, :]
    g.manual_seed(seed)                            # the Gaussian row factor differs per rank
    At = torch.empty((n, rows), dtype=torch.float64, device="cuda")
    blk = 1 << 16
    for r0 in range(0, rows, blk):
        r = min(blk, rows - r0)
        Gs = torch.randn(r, n, dtype=torch.float64, device="cuda", generator=g) / (rows ** 0.5)
        At[:, r0:r0 + r] = (Gs @ B).T
    del V, B
    return At


def cpu_baseline(n, rows, sample_rows=1 << 15):
    """LAPACK Gram + eigen-decomposition on the host cores (the reference has no CPU path of its own)."""
    import numpy as np
    from scipy.linalg import blas, lapack
    rng = np.random.default_rng(0)
    A = np.asfortranarray(rng.standard_normal((sample_rows, n)))
    t0 = time.perf_counter(); G = blas.dsyrk(1.0, A, trans=1, lower=0); t_syrk = time.perf_counter() - t0
    G = G + G.T
    t0 = time.perf_counter(); w, v, info = lapack.dsyevd(G, compute_v=1); t_evd = time.perf_counter() - t0
    scaled = t_syrk * (rows / sample_rows) + t_evd
    flops = rows * n * (n + 1)
    return {"value": flops / scaled / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"LAPACK (SciPy/OpenBLAS) dsyrk on {sample_rows} of {rows} rows scaled linearly ({t_syrk:.2f} s) + dsyevd {n}x{n} ({t_evd:.2f} s); "
                      "the reference has no CPU path, so this stands for it",
            "fit_seconds_estimate": scaled}


def main():
    args = parse()
    import torch
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    if args.impl == "reference" and not os.path.exists(REF_LIB):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libhyacin_ref.so was not built (reference sources absent at build time)"}))
        return

    os.environ.setdefault("HYACIN_CREATE_TIMER", "1")
    from hyacinth_b200 import api
    comm = None
    if world > 1:
        nccl, comm = make_nccl_comm(torch, dist, rank, world)
    lib_path = REF_LIB if args.impl == "reference" else None
    h = api.Hyacin(lib_path=lib_path, stream=0, nccl_comm=comm.value if comm else None)
    mine = args.impl == "b200"

    n, rows = args.n, 1 << args.rows_log2
    global_m = rows * world
    if args.complex:
        args.no_e2e = args.no_cpu = args.no_fit = True
    atype = api.F64_COMPLEX if args.complex else api.F64
    At = make_complex_matrix(torch, rows, n, seed=777 + rank) if args.complex else make_matrix(torch, rows, n, seed=777 + rank)
    u, cp, lp, tri = h.herk_batch_init(EPS, global_m, n, atype)
    b, sg, l = h.segments(rows)
    vexp = torch.zeros((b + 1, n), dtype=torch.int32, device="cuda")
    C = torch.zeros((cp * lp, tri), dtype=torch.int64, device="cuda")
    Gbuf = torch.empty((n, n * 32), dtype=torch.uint8, device="cuda")
    flops = float(global_m) * n * (n + 1) * (4.0 if args.complex else 1.0)

    def barrier():
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
            torch.cuda.synchronize()

    def gram_step():
        h.quantize_scale_batch(b, sg, l, n, atype, At, rows, u, vexp)
        h.allreduce_vexp(n, vexp)
        h.herk_batch(b, sg, l, n, atype, At, rows, u, vexp, 0, lp, C)
        h.allreduce_1drow(cp, lp, tri, C)
        gtype, gbytes = h.dequantize_init(n, lp, C, vexp, atype)
        h.dequantize(n, lp, C, vexp, gtype, Gbuf, n)
        return gtype

    def max_over_ranks(x):
        if not dist:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---------------- value: hot path with the matrix resident in HBM ----------------
    for _ in range(max(args.warmup, 0)):
        gram_step()
    barrier()
    if mine:
        h.launch_count(reset=True)
        h.profile_enable(True)
    clocks = ClockSampler(local) if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        gtype = gram_step()
    e1.record()
    barrier()
    clock_info = clocks.stop() if clocks else None
    step_ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    launches = h.launch_count() if mine else None
    prof = h.profile_read() if mine else None
    if mine:
        h.profile_enable(False)
        status = h.status()
        if status:
            raise RuntimeError(f"a bounded wait inside the Gram kernel expired (code {status})")

    # ---------------- fit with the matrix resident: seconds per hyacinTsvdFit and its timer classes ----------------
    S = torch.zeros(n, dtype=torch.float64, device="cuda"); V = torch.zeros((n, n), dtype=torch.float64, device="cuda")
    fit_times, seg, fit_rank = [0.0], None, None
    for it in range(0 if args.no_fit else 2 + min(args.steps, 3)):
        h.sync_timer(); barrier()
        t0 = time.perf_counter()
        fit_rank = h.tsvd_fit(EPS, "N", rows, n, n, At, rows, S, V, n, global_m, atype)
        seg = h.sync_timer(); torch.cuda.synchronize()
        if it == 2:
            fit_times = []
        if it >= 2:
            fit_times.append(time.perf_counter() - t0)
    fit_seconds = max_over_ranks(statistics.median(fit_times))

    # ---------------- e2e: host matrix -> hyacinTsvdFit -> host results, every step ----------------
    e2e = None
    if not args.no_e2e and not args.no_fit:
        # pinned bytes this rank may hold: at most half of what the host has free, split over the ranks
        try:
            import psutil
            free_host = float(psutil.virtual_memory().available)
        except Exception:
            free_host = float(96 << 30)
        free_host = -max_over_ranks(-free_host)                      # the same figure on every rank
        host_budget = int(min(144 * (1 << 30), 0.5 * free_host)) // world
        host_rows = rows
        while host_rows * n * 8 > host_budget and host_rows > 1024:
            host_rows //= 2
        hostA = torch.empty((n, host_rows), dtype=torch.float64, pin_memory=True)
        hostA.copy_(At[:, :host_rows])
        hostS = torch.empty(n, dtype=torch.float64, pin_memory=True); hostV = torch.empty((n, n), dtype=torch.float64, pin_memory=True)
        dA = At                                                         # the device buffer is overwritten from the host copy
        reps = rows // host_rows

        def e2e_step():
            for r in range(reps):
                dA[:, r * host_rows:(r + 1) * host_rows].copy_(hostA, non_blocking=True)
            rk = h.tsvd_fit(EPS, "N", rows, n, n, dA, rows, S, V, n, global_m, atype)
            hostS.copy_(S, non_blocking=True)
            hostV[:max(rk, 1)].copy_(V[:max(rk, 1)], non_blocking=True)
            torch.cuda.synchronize()
            return rk

        for _ in range(min(args.warmup, 2)):
            rk = e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            rk = e2e_step()
        barrier()
        e2e_s = max_over_ranks((time.perf_counter() - t0) / args.steps)
        e2e = {"value": flops / e2e_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": rows * n * 8 * world,
               "d2h_bytes_per_step": (n * 8 + max(rk, 1) * n * 8) * world, "seconds_per_step": e2e_s,
               "host_rows_per_rank": host_rows, "note": "hyacinTsvdFit on host data: pinned H2D of A + fit + D2H of S and V[:, :rank] per step"
               + ("" if reps == 1 else f"; host RAM holds a {host_rows}-row block per rank that is sent {reps} times per step")}
        del hostA, hostV

    if rank != 0:
        h.destroy()
        if dist:
            dist.destroy_process_group()
        return

    out = {
        "metric": "hyacinTsvdFit FP64-equivalent Gram TFLOP/s (%s FP64, 2^%d rows per GPU, N=%d, eps=1e-10)" % ("complex" if args.complex else "real", args.rows_log2, n),
        "value": flops / (step_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s8",
        "data": "synthetic",
        "config": {"workload": (f"integer Gram of complex FP64 input, opA=N M=2^{args.rows_log2} per GPU N={n} eps=1e-10 (the Gram of BASELINE configuration 4; hot path only)" if args.complex else
                                f"hyacinTsvdFit real FP64 opA=N M=2^{args.rows_log2} per GPU N={n} K={n} eps=1e-10 (BASELINE configuration {2 if world == 1 else 3})"),
                   "global_rows": global_m, "quantize_bits": u, "limb_panels": lp, "gram_format": int(gtype),
                   "cache": "inputs (%.1f GiB per GPU) are far larger than the 126 MB L2; no flush needed" % (rows * n * 8 / 2**30)},
        "clocks": clock_info,
        "e2e": e2e,
        "gpu_launches": launches,
        "fit_seconds": fit_seconds, "fit_rank": fit_rank, "fit_timer_ms": seg,
        "impl": args.impl,
    }
    peaks = json.load(open(PEAKS)) if os.path.exists(PEAKS) else None
    if mine and prof and prof["gram_launches"] and not args.complex:
        plan = h.crt_plan(u, 0, rows)
        per_launch_rows = min(plan["chunk_rows"], rows)
        alg_ops = 2.0 * plan["moduli"] * per_launch_rows * n * (n + 1) / 2.0          # int8 multiply-adds of the upper triangle, x2
        avg_ms = prof["gram_ms"] / prof["gram_launches"]
        achieved = alg_ops / (avg_ms * 1e-3) / 1e12
        if peaks:
            peak, src = 2.0 * peaks["bf16_tflops_sustained"], "2 x measured sustained dense bf16 (MEASURED_PEAKS.json); no int8 figure is measured on this pool"
        else:
            peak, src = 2.0 * 1400.0, "2 x fallback sustained dense bf16 (1.4 PFLOP/s)"
        out["roofline"] = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                           "traffic": None, "kernel": "gram_pair_kernel: residue Gram (tcgen05.mma.cta_group::2 kind::i8)", "avg_launch_ms": avg_ms,
                           "launches_timed": prof["gram_launches"], "ops_per_launch": alg_ops, "peak_source": src,
                           "frac_of_nominal_int8_4500": achieved / 4500.0,
                           "quantize_avg_launch_ms": prof["quantize_ms"] / max(prof["quantize_launches"], 1),
                           "quantize_gbs": (per_launch_rows * n * (8 + plan["moduli"])) / (prof["quantize_ms"] / max(prof["quantize_launches"], 1) * 1e-3) / 1e9}
        if n == 4096:
            tiles = h.tile_info(n)
            residue_bytes = plan["moduli"] * tiles["num_tiles"] * tiles["tile_y"] * tiles["tile_x"]
            chunks = -(-rows // per_launch_rows)
            out["roofline"]["traffic"] = (GRAM_DRAM_READ_BYTES_PER_ROW_MODULUS * per_launch_rows * plan["moduli"]
                                          + residue_bytes * (2.0 - 1.0 / chunks))
            out["roofline"]["algorithmic_bytes"] = float(per_launch_rows) * n * plan["moduli"] + residue_bytes * (2.0 - 1.0 / chunks)
            out["roofline"]["traffic_source"] = GRAM_TRAFFIC_SOURCE
    if args.impl == "reference":
        out["cpu_baseline"] = {"value": out["value"], "unit": "TFLOP/s", "cores": 1, "kind": "reference",
                               "sample": "the reference's own CUDA library (cuBLAS INT8 GEMM + SIMT kernels + cuSOLVER) on the same GPU(s); it has no CPU path"}
    elif not args.no_cpu and world == 1:
        out["cpu_baseline"] = cpu_baseline(n, rows)
    print(json.dumps(out))
    h.destroy()
    if dist:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
