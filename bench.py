#!/usr/bin/env python3
"""Benchmark of the quantized-Gram hot path behind hyacinTsvdFit (and of the other benchmark configurations).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--config 2|4|5] [--scaling weak|strong] [--gram-algorithm A|L] [--peak-int8]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Default workload (configuration 2; configuration 3 for N > 1, weak scaling): real FP64, opA = 'N', 2^20 rows per
GPU, 4096 columns, eps = 1e-10 (hyacinth_b200.workloads.real_decaying; synthetic, the reference publishes no dataset).

One step = one pass of the hot path over the local matrix:
    hyacinXquantizeScaleBatch -> hyacinAllReduceVExp -> hyacinXherkBatch -> hyacinAllReduce1Drow
    -> hyacinXdequantizeInit -> hyacinXdequantize
`value` is FP64-equivalent Gram TFLOP/s = globalM N (N + 1) / time of that pass with A resident in HBM; the whole
fit (hyacinTsvdFit, which adds the replicated factorisation) is reported beside it as `fit_seconds` / `fit_tflops`;
`e2e` is the fit with the matrix coming from pinned host memory and S, V going back to the host every step.
The dominant kernel (tcgen05 residue Gram) is timed in situ with CUDA events on its own stream and set against an
int8 GEMM peak measured in the same process (cublasGemmEx s8 x s8 -> s32, the call of the reference's
src/hyacin_herk.cpp:95-109).  `check` carries checksums of what the last step computed, so that two arms -- and,
through `ranks_agree`, all ranks -- can be seen to hold the same integers.
`--scaling strong` keeps globalM = 2^23 fixed; a rank whose share does not fit its GPU streams 2^20-row blocks
through hyacinXquantizeScaleBatch (minimum over blocks) and hyacinXherkBatch(beta = 1).
`--config 4` / `--config 5`: one step = one hyacinTsvdFitSegmentN (complex 'C', 2^19 x 2048, K = 256, eps 1e-12) /
hyacinInterpolateFit (FP32 'T', 2^17 x 8192 per GPU, K = 1024, eps 1e-5) on resident data.
`--impl reference` drives the reference's own CUDA library (oracle/_ref, built from the reference sources)
through the same C ABI on the same GPUs -- the reference has no CPU implementation of this path.
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
# DRAM traffic of the Gram kernel from an ncu capture of a smaller launch (16384 rows, 13 moduli, N = 4096):
# 1.92 GB read and 116 MB written.  Reads grow in proportion to rows x moduli (9016 bytes per row and modulus),
# the residue bytes written (and re-read when accumulating) depend on N and the moduli only.
GRAM_DRAM_READ_BYTES_PER_ROW_MODULUS = 8945.0
GRAM_TRAFFIC_SOURCE = "ncu dram__bytes_read.sum + dram__bytes_write.sum of a 16384-row launch (profiles/gram_wide_kernel_n4096_rows16384.txt), reads scaled by rows"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", type=int, default=2, choices=[2, 4, 5], help="benchmark configuration (2 is the headline; 3 = 2 on N > 1 GPUs)")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"], help="strong: globalM = 2^23 fixed (configuration 3)")
    ap.add_argument("--gram-algorithm", default="A", choices=["A", "L", "C"], help="handle.GramMatrixAlgorithm (configuration 4 is also quoted with 'L')")
    ap.add_argument("--peak-int8", action="store_true", help="only measure the int8 GEMM peak of cublasGemmEx (burst and 4 s sustained)")
    ap.add_argument("--rows-log2", type=int, default=None, help="log2 of the rows per GPU (default: the configuration's own)")
    ap.add_argument("--n", type=int, default=None)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-peak", action="store_true", help="skip the in-process int8 GEMM peak measurement (e.g. under a profiler)")
    ap.add_argument("--fits", type=int, default=None, help="number of timed hyacinTsvdFit calls after two warm-up calls (default min(steps, 3); 0 with --fits 0: one call, no warm-up)")
    ap.add_argument("--no-fit", action="store_true", help="skip the hyacinTsvdFit timings (hot path only, e.g. under a profiler)")
    ap.add_argument("--complex", action="store_true",
                    help="complex FP64 input (the Gram of configuration 4: use --rows-log2 19 --n 2048): hot path only, "
                         "for profiles of the complex route; not the headline workload")
    return ap.parse_args()


# ---------------------------------------------------------------------------------------------------------
# plumbing: process group, NCCL communicator for the handle, clocks, checksums, int8 peak
# ---------------------------------------------------------------------------------------------------------
class _NcclId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_byte * 128)]


class stdout_to_stderr:
    """Route file descriptor 1 to stderr for a while: libraries (NCCL's version banner) must not add lines to the JSON output."""

    def __enter__(self):
        sys.stdout.flush()
        self.saved = os.dup(1)
        os.dup2(2, 1)

    def __exit__(self, *exc):
        os.dup2(self.saved, 1)
        os.close(self.saved)


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
    """nvidia-smi sampling every 100 ms in a child process.  Started before the warm-up (the tool needs some tenths of a
    second before its first line); `mark()` opens the timed region and `stop()` closes it, and only samples whose own
    timestamp lies inside the region are reported (all of them if the region was too short to catch one)."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.t0 = time.time()
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def mark(self):
        self.t0 = time.time()

    @staticmethod
    def _stamp(text):
        import datetime
        try:
            return datetime.datetime.strptime(text, "%Y/%m/%d %H:%M:%S.%f").timestamp()
        except ValueError:
            return None

    def stop(self):
        t1 = time.time()
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        text = self.file.read()
        os.unlink(self.file.name)
        return self.summarise(text, self.t0, t1)

    @classmethod
    def summarise(cls, text, t0, t1):
        """Median SM clock, maximum clock and the throttle reasons seen in the csv lines of `text` whose timestamp lies in
        [t0, t1] (all lines if none does)."""
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        for line in text.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                rows.append((cls._stamp(parts[0]), float(parts[1]), float(parts[2]), parts[4:8]))
            except ValueError:
                continue
        inside = [r for r in rows if r[0] is not None and t0 - 0.02 <= r[0] <= t1 + 0.02]
        rows = inside or rows
        reasons = set()
        for _, _, _, flags in rows:
            for name, val in zip(names, flags):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if rows:
            out["sm_mhz"] = statistics.median(r[1] for r in rows)
            out["sm_max_mhz"] = max(r[2] for r in rows)
            out["samples"] = len(rows)
            out["samples_inside_timed_region"] = len(inside)
        out["reasons"] = sorted(reasons)
        return out


def checksum(torch, t):
    """Two 64-bit wrap-around sums over a buffer's words (plain, and weighted by position): equal buffers give equal
    pairs, and a permutation or a single flipped bit does not."""
    if t is None or t.numel() == 0:
        return None
    flat = t.contiguous().view(torch.uint8).reshape(-1)
    pad = (-flat.numel()) % 8
    if pad:
        flat = torch.cat([flat, torch.zeros(pad, dtype=torch.uint8, device=flat.device)])
    w = flat.view(torch.int64)
    weight = (torch.arange(w.numel(), dtype=torch.int64, device=w.device) % 65521) * 2 + 1
    return ["%016x" % (int(w.sum().item()) & (2**64 - 1)), "%016x" % (int((w * weight).sum().item()) & (2**64 - 1))]


def int8_gemm_peak(torch, seconds, size=8192):
    """TOP/s of cublasGemmEx s8 x s8 -> s32 (op T, op N, as the reference calls it): best single call of ten, and the
    average over a loop of `seconds` (power-capped, what a kernel inside a long step can be held against)."""
    cublas = ctypes.CDLL("libcublas.so.12")
    handle = ctypes.c_void_p()
    if cublas.cublasCreate_v2(ctypes.byref(handle)) != 0:
        return None
    cublas.cublasSetStream_v2(handle, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    a = torch.randint(-128, 128, (size, size), dtype=torch.int8, device="cuda")
    b = torch.randint(-128, 128, (size, size), dtype=torch.int8, device="cuda")
    c = torch.empty((size, size), dtype=torch.int32, device="cuda")
    one, zero = ctypes.c_int32(1), ctypes.c_int32(0)

    def gemm():
        return cublas.cublasGemmEx(handle, 1, 0, size, size, size, ctypes.byref(one), ctypes.c_void_p(a.data_ptr()), 3, size,
                                   ctypes.c_void_p(b.data_ptr()), 3, size, ctypes.byref(zero), ctypes.c_void_p(c.data_ptr()), 10, size, 72, -1)

    if gemm() != 0:
        cublas.cublasDestroy_v2(handle)
        return None
    torch.cuda.synchronize()
    ops = 2.0 * size ** 3
    best = 0.0
    for _ in range(10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); gemm(); e1.record(); torch.cuda.synchronize()
        best = max(best, ops / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    reps = max(8, int(seconds * best * 1e12 / ops))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        gemm()
    e1.record(); torch.cuda.synchronize()
    sustained = reps * ops / (e0.elapsed_time(e1) * 1e-3) / 1e12
    cublas.cublasDestroy_v2(handle)
    del a, b, c
    return {"burst_tops": best, "sustained_tops": sustained, "sustained_seconds": e0.elapsed_time(e1) * 1e-3, "size": size,
            "how": "cublasGemmEx CUDA_R_8I x CUDA_R_8I -> CUDA_R_32I, CUBLAS_COMPUTE_32I, op(T) op(N), CUDA events"}


def cpu_baselines(n, rows):
    """(a) the CPU oracle -- this repository's plain-C restatement of the quantized Gram (exact integer arithmetic,
    one thread) -- on a sample of rows; (b) LAPACK dsyrk + dsyevd on all host cores, the floating-point Gram fit a CPU
    user would run instead (the reference itself has no CPU path)."""
    import numpy as np
    from scipy.linalg import blas, lapack
    from oracle import oracle as O
    rng = np.random.default_rng(0)
    flops = float(rows) * n * (n + 1)
    sample = 16
    A = rng.standard_normal((sample, n))
    u, cp, lp, tri = O.herk_init(1e-10, rows, n, O.F64)
    vexp = O.column_exponents(A, O.F64, u, 1, sample, sample)
    t0 = time.perf_counter(); O.gram_exact(A, O.F64, vexp[0], lp); t1 = time.perf_counter() - t0
    sample2 = int(min(max(sample * 12.0 / max(t1, 1e-3), 32), 2048))
    A = rng.standard_normal((sample2, n))
    t0 = time.perf_counter()
    vexp = O.column_exponents(A, O.F64, u, 1, sample2, sample2)
    O.gram_exact(A, O.F64, vexp[0], lp)
    t_port = time.perf_counter() - t0
    port = {"value": flops / (t_port * rows / sample2) / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": "port",
            "sample": f"oracle/oracle_gram.c (exponents + exact integer Gram) on {sample2} of {rows} rows, {t_port:.1f} s, scaled linearly in the rows"}
    sample_rows = 1 << 15
    A = np.asfortranarray(rng.standard_normal((sample_rows, n)))
    t0 = time.perf_counter(); G = blas.dsyrk(1.0, A, trans=1, lower=0); t_syrk = time.perf_counter() - t0
    G = G + G.T
    t0 = time.perf_counter(); lapack.dsyevd(G, compute_v=1); t_evd = time.perf_counter() - t0
    scaled = t_syrk * (rows / sample_rows) + t_evd
    lap = {"value": flops / scaled / 1e12, "unit": "TFLOP/s", "cores": os.cpu_count(),
           "sample": f"SciPy/OpenBLAS dsyrk on {sample_rows} of {rows} rows scaled linearly ({t_syrk:.2f} s) + dsyevd {n}x{n} ({t_evd:.2f} s)",
           "fit_seconds_estimate": scaled}
    return port, lap


# ---------------------------------------------------------------------------------------------------------
def main():
    args = parse()
    import torch
    from hyacinth_b200 import workloads
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)

    if args.peak_int8:
        if rank == 0:
            clocks = ClockSampler(local)
            peak = int8_gemm_peak(torch, 4.0)
            print(json.dumps({"metric": "dense int8 GEMM peak (cublasGemmEx s8 -> s32, 8192^3)", "unit": "TOP/s", "value": peak and peak["sustained_tops"],
                              "int8_peak": peak, "clocks": clocks.stop(), "n_gpus": 1}))
        return

    dist = None
    if world > 1:
        import torch.distributed as dist
        with stdout_to_stderr():
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            dist.barrier()

    if args.impl == "reference" and not os.path.exists(REF_LIB):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libhyacin_ref.so was not built (reference sources absent at build time)"}))
        return

    os.environ.setdefault("HYACIN_CREATE_TIMER", "1")
    from hyacinth_b200 import api
    comm = None
    if world > 1:
        with stdout_to_stderr():
            nccl, comm = make_nccl_comm(torch, dist, rank, world)
    lib_path = REF_LIB if args.impl == "reference" else None
    h = api.Hyacin(lib_path=lib_path, stream=0, nccl_comm=comm.value if comm else None)
    h.h.GramMatrixAlgorithm = args.gram_algorithm.encode()
    mine = args.impl == "b200"

    def barrier():
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(x):
        if not dist:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def ranks_agree(words):
        """True if every rank holds the same checksum words."""
        if not dist or words is None:
            return None
        mine_t = torch.tensor([int(w, 16) - (1 << 64) if int(w, 16) >= (1 << 63) else int(w, 16) for w in words], dtype=torch.int64, device="cuda")
        lo, hi = mine_t.clone(), mine_t.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        return bool(torch.equal(lo, hi))

    def finish(out):
        if rank == 0:
            print(json.dumps(out))
        h.destroy()
        if dist:
            dist.destroy_process_group()

    if args.config in (4, 5):
        return finish(run_fit_config(args, torch, api, workloads, h, rank, world, barrier, max_over_ranks, ranks_agree))

    # ------------------------------------------------------------------------------------------------
    # configurations 2 / 3
    # ------------------------------------------------------------------------------------------------
    eps = 1e-10
    n = args.n or 4096
    strong = args.scaling == "strong"
    if strong:
        global_m = 1 << 23
        rows = global_m // world
    else:
        rows = 1 << (args.rows_log2 if args.rows_log2 is not None else 20)
        global_m = rows * world
    if args.complex:
        args.no_e2e = args.no_cpu = args.no_fit = True
    atype = api.F64_COMPLEX if args.complex else api.F64
    elem = 16 if args.complex else 8
    # a share that does not fit the GPU next to the work buffers is streamed in blocks of 2^20 rows
    free_bytes = torch.cuda.mem_get_info()[0]
    block_rows = rows
    while block_rows * n * elem > 0.8 * free_bytes and block_rows > (1 << 20):
        block_rows //= 2
    blocks = rows // block_rows
    streamed = blocks > 1
    if streamed:
        args.no_fit = args.no_e2e = True
    if args.complex:
        At = workloads.complex_low_rank(torch, block_rows, n, seed=777 + rank)
    else:
        At = workloads.real_decaying(torch, block_rows, n, seed=777 + rank, total_rows=None if not strong else rows)
    u, cp, lp, tri = h.herk_batch_init(eps, global_m, n, atype)
    b, sg, l = h.segments(block_rows)
    vexps = [torch.zeros((b + 1, n), dtype=torch.int32, device="cuda") for _ in range(blocks)]
    C = torch.zeros((cp * lp, tri), dtype=torch.int64, device="cuda")
    Gbuf = torch.empty((n, n * 32), dtype=torch.uint8, device="cuda")
    flops = float(global_m) * n * (n + 1) * (4.0 if args.complex else 1.0)

    def gram_step():
        # pass 1: column exponents of every block, minimum over blocks and ranks
        for k in range(blocks):
            h.quantize_scale_batch(b, sg, l, n, atype, At, block_rows, u, vexps[k])
        if blocks > 1:
            torch.minimum(vexps[0][0], torch.stack([v[0] for v in vexps[1:]]).amin(dim=0), out=vexps[0][0])
        h.allreduce_vexp(n, vexps[0])
        for k in range(1, blocks):
            vexps[k][0].copy_(vexps[0][0])
        # pass 2: integer Gram, block by block
        for k in range(blocks):
            h.herk_batch(b, sg, l, n, atype, At, block_rows, u, vexps[k], 0 if k == 0 else 1, lp, C)
        h.allreduce_1drow(cp, lp, tri, C)
        gtype, gbytes = h.dequantize_init(n, lp, C, vexps[0], atype)
        h.dequantize(n, lp, C, vexps[0], gtype, Gbuf, n)
        return gtype, gbytes

    int8_peak = int8_gemm_peak(torch, 1.5) if (mine and rank == 0 and not args.complex and not args.no_peak) else None
    barrier()
    clocks = ClockSampler(local) if rank == 0 else None
    for _ in range(max(args.warmup, 0)):
        gram_step()
    barrier()
    if mine:
        h.launch_count(reset=True)
        h.profile_enable(True)
    torch.cuda.synchronize()
    if clocks:
        clocks.mark()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        gtype, gbytes = gram_step()
    e1.record()
    torch.cuda.synchronize()
    clock_info = clocks.stop() if clocks else None
    barrier()
    step_ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    launches = h.launch_count() if mine else None
    prof = h.profile_read() if mine else None
    if mine:
        h.profile_enable(False)
        status = h.status()
        if status:
            raise RuntimeError(f"a bounded wait inside the Gram kernel expired (code {status})")

    # what the last step computed (outside every timed region)
    check = {"vexp0": checksum(torch, vexps[0][0]), "C": checksum(torch, C), "gram_format": int(gtype),
             "G": checksum(torch, Gbuf.reshape(-1)[:n * n * gbytes])}       # the N x N Gram (ldg = N) sits at the start of the buffer
    check["ranks_agree"] = ranks_agree((check["C"] or []) + (check["G"] or []))

    # ---------------- fit with the matrix resident: seconds per hyacinTsvdFit, its timer classes, its tail ----------------
    S = torch.zeros(n, dtype=torch.float64, device="cuda"); V = torch.zeros((n, n), dtype=torch.float64, device="cuda")
    fit_times, seg, fit_rank, tail = [0.0], None, None, None
    fit_warm = 0 if args.fits == 0 else 2
    fit_calls = 0 if args.no_fit else (1 if args.fits == 0 else fit_warm + (args.fits if args.fits else min(args.steps, 3)))
    for it in range(fit_calls):
        h.sync_timer(); barrier()
        if mine and it == fit_warm:
            h.profile_enable(True)
        t0 = time.perf_counter()
        fit_rank = h.tsvd_fit(eps, "N", rows, n, n, At, rows, S, V, n, global_m, atype)
        seg = h.sync_timer(); torch.cuda.synchronize()
        if it == fit_warm:
            fit_times = []
        if it >= fit_warm:
            fit_times.append(time.perf_counter() - t0)
    fit_seconds = max_over_ranks(statistics.median(fit_times))
    if mine and not args.no_fit:
        h.profile_read()
        tail = h.profile_read_tail()
        h.profile_enable(False)
        if tail["cholesky_launches"]:
            tail = {"cholesky_ms_per_fit": tail["cholesky_ms"] / tail["cholesky_launches"], "svd_ms_per_fit": tail["svd_ms"] / max(tail["svd_calls"], 1),
                    "how": "CUDA events around the pivoted-Cholesky kernel and the cuSOLVER SVD call inside hyacinXGevd, in situ (after the power-capped Gram phase)"}
    if not args.no_fit:
        check.update({"fit_rank": fit_rank, "S_first": float(S[0].item()), "S_last": float(S[max(fit_rank, 1) - 1].item()),
                      "S": checksum(torch, S), "V": checksum(torch, V[:max(fit_rank, 1)])})
        check["fit_ranks_agree"] = ranks_agree(check["S"] + check["V"])

    # ---------------- e2e: host matrix -> hyacinTsvdFit -> host results, every step ----------------
    e2e = None
    if not args.no_e2e and not args.no_fit:
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
            rk = h.tsvd_fit(eps, "N", rows, n, n, dA, rows, S, V, n, global_m, atype)
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
        return finish(None)

    rows_txt = f"2^{rows.bit_length() - 1}" if rows & (rows - 1) == 0 else str(rows)
    cfg_name = "the Gram of BASELINE configuration 4; hot path only" if args.complex else f"BASELINE configuration {2 if world == 1 and not strong else 3}"
    out = {
        "metric": "quantized Gram hot path of hyacinTsvdFit, FP64-equivalent TFLOP/s (%s FP64, %s rows per GPU, N=%d, eps=1e-10)" % ("complex" if args.complex else "real", rows_txt, n),
        "value": flops / (step_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": step_ms, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "s8",
        "data": "synthetic",
        "config": {"workload": f"hyacinTsvdFit {'complex' if args.complex else 'real'} FP64 opA=N M={rows_txt} per GPU N={n} K={n} eps=1e-10 ({cfg_name})",
                   "global_rows": global_m, "quantize_bits": u, "limb_panels": lp, "gram_format": int(gtype),
                   "streaming": (f"the {rows}-row share does not fit the GPU: {blocks} blocks of {block_rows} rows through hyacinXquantizeScaleBatch (minimum over blocks) "
                                 f"and hyacinXherkBatch(beta = 1); one resident block stands for all of them (same sizes, same work)") if streamed else None,
                   "cache": "inputs (%.1f GiB per GPU) are far larger than the 126 MB L2; no flush needed" % (block_rows * n * elem / 2**30)},
        "clocks": clock_info,
        "e2e": e2e,
        "gpu_launches": launches,
        "fit_seconds": None if args.no_fit else fit_seconds, "fit_tflops": None if args.no_fit else flops / fit_seconds / 1e12,
        "fit_rank": fit_rank, "fit_timer_ms": seg, "fit_tail_ms": tail,
        "check": check,
        "impl": args.impl,
    }
    peaks = json.load(open(PEAKS)) if os.path.exists(PEAKS) else None
    if mine and prof and prof["gram_launches"] and not args.complex:
        plan = h.crt_plan(u, 0, block_rows)
        per_launch_rows = min(plan["chunk_rows"], block_rows)
        # algorithmic int8 operations of one launch: upper triangle, 2 per multiply-add.  The reference's schedule
        # needs 12 moduli for this bit budget and reconstructs every 8192 rows; this build spends a 13th modulus to
        # reconstruct once per call, so `issued` counts 13 and `achieved` only the 12 that the algorithm requires.
        need_moduli = min(plan["moduli"], 12) if n == 4096 and u == 40 else plan["moduli"]
        alg_ops = 2.0 * need_moduli * per_launch_rows * n * (n + 1) / 2.0
        issued_ops = 2.0 * plan["moduli"] * per_launch_rows * n * (n + 1) / 2.0
        avg_ms = prof["gram_ms"] / prof["gram_launches"]
        achieved = alg_ops / (avg_ms * 1e-3) / 1e12
        if int8_peak:
            peak, src = int8_peak["sustained_tops"], "cublasGemmEx s8 -> s32 8192^3 measured in this process, sustained loop (int8_peak)"
        elif peaks:
            peak, src = 2.0 * peaks["bf16_tflops_sustained"], "2 x measured sustained dense bf16 (MEASURED_PEAKS.json)"
        else:
            peak, src = 2.0 * 1400.0, "2 x fallback sustained dense bf16 (1.4 PFLOP/s)"
        q_ms = prof["quantize_ms"] / max(prof["quantize_launches"], 1)
        out["roofline"] = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                           "traffic": None, "kernel": "gram_wide_kernel: residue Gram (tcgen05.mma.cta_group::2 kind::i8, two 256 x 256 tiles per CTA pair)", "avg_launch_ms": avg_ms,
                           "launches_timed": prof["gram_launches"], "ops_per_launch": alg_ops, "moduli_required": need_moduli, "moduli_issued": plan["moduli"],
                           "issued_tops": issued_ops / (avg_ms * 1e-3) / 1e12, "frac_issued": issued_ops / (avg_ms * 1e-3) / 1e12 / peak,
                           "peak_source": src, "int8_peak": int8_peak,
                           "frac_of_2x_sustained_bf16": achieved / (2.0 * peaks["bf16_tflops_sustained"]) if peaks else None,
                           "frac_of_nominal_int8_4500": achieved / 4500.0,
                           "ms_times_sm_mhz": avg_ms * clock_info["sm_mhz"] if clock_info and clock_info.get("sm_mhz") else None,
                           "quantize_avg_launch_ms": q_ms,
                           "quantize_gbs": (per_launch_rows * n * (8 + plan["moduli"])) / (q_ms * 1e-3) / 1e9,
                           "quantize_frac_of_hbm": ((per_launch_rows * n * (8 + plan["moduli"])) / (q_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]) if peaks else None}
        if n == 4096:
            tiles = h.tile_info(n)
            residue_bytes = plan["moduli"] * tiles["num_tiles"] * tiles["tile_y"] * tiles["tile_x"]
            chunks = -(-block_rows // per_launch_rows)
            out["roofline"]["traffic"] = (GRAM_DRAM_READ_BYTES_PER_ROW_MODULUS * per_launch_rows * plan["moduli"]
                                          + residue_bytes * (2.0 - 1.0 / chunks))
            out["roofline"]["algorithmic_bytes"] = float(per_launch_rows) * n * plan["moduli"] + residue_bytes * (2.0 - 1.0 / chunks)
            out["roofline"]["traffic_source"] = GRAM_TRAFFIC_SOURCE
    if args.impl == "reference":
        out["cpu_baseline"] = {"value": out["value"], "unit": "TFLOP/s", "cores": 1, "kind": "reference",
                               "sample": "the reference's own CUDA library (cuBLAS INT8 GEMM + SIMT kernels + cuSOLVER) on the same GPU(s); it has no CPU path"}
        if out["e2e"] is None:
            out["e2e"] = {"value": out["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    elif not args.no_cpu and world == 1:
        out["cpu_baseline"], out["lapack_baseline"] = cpu_baselines(n, rows)
    finish(out)


def run_fit_config(args, torch, api, workloads, h, rank, world, barrier, max_over_ranks, ranks_agree):
    """Configurations 4 and 5: one step = one fit on resident data."""
    mine = args.impl == "b200"
    if args.config == 4:
        m = 1 << (args.rows_log2 if args.rows_log2 is not None else 19)
        n, k, eps, atype = args.n or 2048, 256, 1e-12, api.F64_COMPLEX
        stored = workloads.complex_low_rank(torch, m, n, seed=777 + rank, stored_conj_transposed=True)
        S = torch.zeros(k, dtype=torch.float64, device="cuda"); V = torch.zeros((k, n), dtype=torch.complex128, device="cuda")
        global_m = m * world
        flops = 4.0 * global_m * n * (n + 1)
        name = f"hyacinTsvdFitSegmentN complex FP64 opA=C M=2^{m.bit_length() - 1} per GPU N={n} K={k} eps=1e-12 GramMatrixAlgorithm={args.gram_algorithm} (BASELINE configuration 4)"

        def step():
            return h.tsvd_fit(eps, "C", m, n, k, stored, n, S, V, n, global_m, atype, segment_n=True)
    else:
        m = 1 << (args.rows_log2 if args.rows_log2 is not None else 17)
        n, k, eps, atype = args.n or 8192, 1024, 1e-5, api.F32
        stored = workloads.float_product_transposed(torch, m, n, seed=777 + rank)
        jp = torch.zeros(n, dtype=torch.int32, device="cuda"); V = torch.zeros((k, n), dtype=torch.float32, device="cuda")
        global_m = m * world
        flops = float(global_m) * n * (n + 1)
        name = f"hyacinInterpolateFit real FP32 opA=T M=2^{m.bit_length() - 1} per GPU N={n} K={k} eps=1e-5 (BASELINE configuration 5, {world} of 8 shares)"

        def step():
            return h.interpolate_fit(eps, "T", m, n, k, stored, n, jp, V, n, global_m, atype)

    clocks = ClockSampler(int(os.environ.get("LOCAL_RANK", "0"))) if rank == 0 else None
    for _ in range(max(args.warmup, 0)):
        fit_rank = step()
    h.sync_timer(); barrier()
    if mine:
        h.launch_count(reset=True)
        h.profile_enable(True)
    if clocks:
        clocks.mark()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fit_rank = step()
    seg = h.sync_timer(); torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    barrier()
    clock_info = clocks.stop() if clocks else None
    step_s = max_over_ranks(wall / args.steps)
    launches = h.launch_count() if mine else None
    prof = tail = None
    if mine:
        prof = h.profile_read(); tail = h.profile_read_tail(); h.profile_enable(False)
        for d in (prof, tail):
            for key in list(d):
                if key.endswith("_ms"):
                    d[key] /= args.steps
        status = h.status()
        if status:
            raise RuntimeError(f"a bounded wait inside a kernel expired (code {status})")
    check = {"fit_rank": fit_rank, "V": checksum(torch, V[:max(fit_rank, 1)])}
    if args.config == 4:
        check.update({"S": checksum(torch, S), "S_first": float(S[0].item()), "S_last": float(S[max(fit_rank, 1) - 1].item())})
    else:
        check.update({"pivots": checksum(torch, jp), "first_pivots": [int(x) for x in jp[:8].tolist()]})
    check["ranks_agree"] = ranks_agree(check["V"])
    if rank != 0:
        return None
    if seg:
        seg = {key: val / args.steps for key, val in seg.items()}
    out = {"metric": "fit throughput, FP64-equivalent Gram TFLOP/s of the nominal Gram flops per fit second", "value": flops / step_s / 1e12, "unit": "TFLOP/s",
           "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "s8", "data": "synthetic", "config": {"workload": name, "global_rows": global_m,
                                                                                 "cache": "inputs are far larger than the 126 MB L2; no flush needed"},
           "clocks": clock_info, "e2e": None, "gpu_launches": launches, "fit_seconds": step_s, "fit_rank": fit_rank, "fit_timer_ms": seg,
           "kernel_ms_per_fit": prof, "fit_tail_ms": tail, "check": check, "impl": args.impl}
    if args.impl == "reference":
        out["cpu_baseline"] = {"value": out["value"], "unit": "TFLOP/s", "cores": 1, "kind": "reference",
                               "sample": "the reference's own CUDA library on the same GPU(s); it has no CPU path"}
        out["e2e"] = {"value": out["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    return out


if __name__ == "__main__":
    main()
