"""ctypes mirror of ``include/hyacin.h`` (and ``include/hyacin_b200.h``) over ``libhyacin.so``.

The product is the C-ABI library; this module only exists so that Python callers (the tests, ``bench.py``) can
drive it with torch tensors as device buffers.  Names, argument order and argument meaning are those of the
reference's header (``include/hyacin.h`` in QxGbM/hyacinth).  There is no fallback: if the shared library is
missing or fails to load, importing :func:`load` raises.

Matrices are column-major device buffers.  A column-major ``M x N`` matrix with leading dimension ``lda`` is a
torch tensor of shape ``(N, lda)`` (row ``j`` of the tensor is column ``j`` of the matrix).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char, c_double, c_int32, c_int64, c_uint32, c_uint64, c_void_p, POINTER, byref

_PKG = os.path.dirname(os.path.abspath(__file__))
DEFAULT_LIB = os.path.join(_PKG, "libhyacin.so")

# hyacinPrecision_t
F64, F64_COMPLEX, F32, F32_COMPLEX, F16, F16_COMPLEX, DD, DD_COMPLEX, TF, TF_COMPLEX, QF, QF_COMPLEX = range(12)
ELEM_BYTES = [8, 16, 4, 8, 2, 4, 16, 32, 12, 24, 16, 32]

PUBLIC_SYMBOLS = [
    "hyacinCreate", "hyacinDestroy", "hyacinInterpolateFit", "hyacinTsvdFit", "hyacinTsvdFitSegmentN",
    "hyacinXherkBatchInit", "hyacinXherkBatch", "hyacinXquantizeScaleBatch", "hyacinXdequantizeInit",
    "hyacinXdequantize", "hyacinXGevd", "hyacinXGinterp", "hyacinCheckNorm", "hyacinAllReduce1Drow",
    "hyacinAllReduceVExp", "hyacinSync_TimerSegments",
]
B200_SYMBOLS = [
    "hyacinB200Status", "hyacinB200CrtPlan", "hyacinB200TileInfo", "hyacinB200QuantizeCrt",
    "hyacinB200GramResidues", "hyacinB200Reconstruct", "hyacinB200LaunchCount", "hyacinB200ProfileEnable",
    "hyacinB200ProfileRead", "hyacinB200SlicePlan", "hyacinB200HerkBatchStatic", "hyacinB200QuantizeLimbs", "hyacinB200GramLimbs",
    "hyacinB200DequantizeViaSlices", "hyacinB200ProfileReadTail", "hyacinB200PivotedCholesky", "hyacinB200SelfTestWait", "hyacinB200VectorRange",
    "hyacinB200GramItem",
]


class HyacinHandle(ctypes.Structure):
    """``hyacinHandle_t`` (include/hyacin.h:20-53 of the reference); zero-initialised by ctypes."""
    _fields_ = [
        ("GramMatrixAlgorithm", c_char), ("StrideBatchPerfPenalty", c_double),
        ("GramSegmentK", c_int32), ("TCGemmTargetK", c_int32),
        ("QuantizeBitCorrection", c_int32), ("QRCPTruncateRank", c_int32), ("JacobiSVDSweeps", c_int32),
        ("DeviceID", c_int32), ("DeviceSMs", c_int32), ("DeviceIsF64Capable", c_int32),
        ("HandleOwnedResource", c_uint32),
        ("cudaStream", c_void_p), ("cublasHandle", c_void_p), ("cusolverHandle", c_void_p), ("mempool", c_void_p),
        ("pinnedWorkspace", c_void_p), ("timer", c_void_p), ("logger", c_void_p), ("ncclComm", c_void_p),
    ]


def load(path: str | None = None) -> ctypes.CDLL:
    """Load the shared library and declare the argument types of every entry point."""
    path = path or DEFAULT_LIB
    if not os.path.exists(path):
        raise RuntimeError(f"{path} not found: build it with `python -m hyacinth_b200._build` (there is no CPU fallback)")
    lib = ctypes.CDLL(path, mode=ctypes.RTLD_LOCAL)
    H = POINTER(HyacinHandle)
    i32, i64, u64, f64, vp = c_int32, c_int64, c_uint64, c_double, c_void_p
    sig = {
        "hyacinCreate": (None, [H]),
        "hyacinDestroy": (None, [H]),
        "hyacinInterpolateFit": (i32, [H, f64, c_char, i32, i32, i32, vp, i32, vp, vp, i32, i64, i32]),
        "hyacinTsvdFit": (i32, [H, f64, c_char, i32, i32, i32, vp, i32, vp, vp, i32, i64, i32]),
        "hyacinTsvdFitSegmentN": (i32, [H, f64, c_char, i32, i32, i32, vp, i32, vp, vp, i32, i64, i32]),
        "hyacinXherkBatchInit": (None, [H, f64, u64, i32, i32, POINTER(i32), POINTER(i32), POINTER(i32), POINTER(u64)]),
        "hyacinXherkBatch": (None, [H, i32, i32, i32, i32, i32, vp, i32, i32, vp, i32, i32, vp]),
        "hyacinXquantizeScaleBatch": (None, [H, i32, i32, i32, i32, i32, vp, i32, i32, vp]),
        "hyacinXdequantizeInit": (None, [H, i32, i32, vp, vp, i32, POINTER(i32), POINTER(i32)]),
        "hyacinXdequantize": (None, [H, i32, i32, vp, vp, i32, vp, i32]),
        "hyacinXGevd": (i32, [H, f64, i32, i32, i32, vp, i32, vp, i32, vp, i32]),
        "hyacinXGinterp": (i32, [H, f64, i32, i32, i32, vp, i32, vp, i32, vp, i32]),
        "hyacinCheckNorm": (f64, [H, c_char, i32, i32, vp, i32, i32, vp, i32, i32]),
        "hyacinAllReduce1Drow": (None, [H, i32, i32, u64, vp]),
        "hyacinAllReduceVExp": (None, [H, u64, vp]),
        "hyacinSync_TimerSegments": (None, [H, POINTER(f64), i32]),
        # B200-only stage entry points (absent from the reference library)
        "hyacinB200Status": (c_uint32, [i32]),
        "hyacinB200CrtPlan": (None, [i32, i32, i64, POINTER(i32), POINTER(i32), POINTER(i32), POINTER(i32)]),
        "hyacinB200TileInfo": (None, [i32, POINTER(i32), POINTER(i32), POINTER(i32), POINTER(i32)]),
        "hyacinB200QuantizeCrt": (None, [H, i32, i32, i32, vp, i32, vp, i32, i32, vp, i64]),
        "hyacinB200GramResidues": (None, [H, i32, i32, vp, i64, i64, i32, i32, i32, i32, vp]),
        "hyacinB200Reconstruct": (None, [H, i32, i32, vp, i32, i32, vp]),
        "hyacinB200SlicePlan": (None, [i32, i32, POINTER(i32), POINTER(i32)]),
        "hyacinB200DequantizeViaSlices": (None, [H, i32, i32, vp, vp, i32, i32, POINTER(i32), vp, i32]),
        "hyacinB200HerkBatchStatic": (i32, [H, i32, i32, i32, i32, i32, vp, i32, i32, vp, i32, i32, vp]),
        "hyacinB200QuantizeLimbs": (None, [H, i32, i32, i32, vp, i32, vp, i32, vp, i64]),
        "hyacinB200GramLimbs": (None, [H, i32, i32, vp, i64, i64, i32, i32, i32, i32, i32, vp]),
        "hyacinB200LaunchCount": (i64, [i32]),
        "hyacinB200ProfileEnable": (None, [i32]),
        "hyacinB200ProfileRead": (None, [POINTER(f64), POINTER(i32), POINTER(f64), POINTER(i32)]),
        "hyacinB200ProfileReadTail": (None, [POINTER(f64), POINTER(i32), POINTER(f64), POINTER(i32)]),
        "hyacinB200VectorRange": (None, [H, i32, i32, i32, vp, vp]),
        "hyacinB200SelfTestWait": (i32, [H, c_uint32, c_uint32]),
        "hyacinB200PivotedCholesky": (i32, [H, f64, i32, i32, i32, vp, i32, vp, vp, i32]),
        "hyacinB200GramItem": (i32, [i32, i32, i32, i32, i32, i32, i32, POINTER(i32), POINTER(i32), POINTER(i32), POINTER(i32)]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name, None)
        if fn is None:
            if name in PUBLIC_SYMBOLS:
                raise RuntimeError(f"{path} does not export {name}")
            continue
        fn.restype, fn.argtypes = res, args
    return lib


def gram_items(tiles_x: int, pair_rows: int, full: bool, moduli: int, pairs: int, pair: int, lib=None):
    """Work items (modulus, tile_row, tile_col, width) of one CTA pair of the residue Gram kernel, in order."""
    lib = lib or load()
    m, ty, tx, w = c_int32(), c_int32(), c_int32(), c_int32()
    out, k = [], 0
    while lib.hyacinB200GramItem(tiles_x, pair_rows, 1 if full else 0, moduli, pairs, pair, k, byref(m), byref(ty), byref(tx), byref(w)):
        out.append((m.value, ty.value, tx.value, w.value))
        k += 1
    return out


def _dp(t) -> c_void_p:
    """Device (or host) pointer of a torch tensor / raw integer address / None."""
    if t is None:
        return c_void_p(0)
    if isinstance(t, int):
        return c_void_p(t)
    return c_void_p(t.data_ptr())


class Hyacin:
    """One handle on the current CUDA device.  Thin: every method is one C call.

    ``stream`` is a raw ``cudaStream_t`` (e.g. ``torch.cuda.current_stream().cuda_stream``); ``nccl_comm`` a raw
    ``ncclComm_t`` or None.  Set environment variables (HYACIN_*) before constructing.
    """

    def __init__(self, lib_path: str | None = None, stream: int = 0, nccl_comm: int | None = None):
        self.lib = load(lib_path)
        self.h = HyacinHandle()
        self.h.cudaStream = stream
        if nccl_comm:
            self.h.ncclComm = nccl_comm
        self.lib.hyacinCreate(byref(self.h))
        self._alive = True

    def destroy(self):
        if self._alive:
            self.lib.hyacinDestroy(byref(self.h))
            self._alive = False

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.destroy()

    # ---- stage functions -------------------------------------------------------------------------
    def herk_batch_init(self, eps: float, global_m: int, n: int, atype: int):
        u, cp, lp, st = c_int32(), c_int32(), c_int32(), c_uint64()
        self.lib.hyacinXherkBatchInit(byref(self.h), eps, global_m, n, atype, byref(u), byref(cp), byref(lp), byref(st))
        return u.value, cp.value, lp.value, st.value

    def segments(self, m: int):
        """(batches, segM, lastM) exactly as the fitting drivers derive them (src/lra.cpp:55-57)."""
        k = self.h.GramSegmentK
        it = m if k <= 0 else min(k, m)
        q, r = divmod(m, max(1, it))
        return q + (1 if r else 0), it, (r if r else it)

    def quantize_scale_batch(self, batches, seg_m, last_m, n, atype, A, lda, u, vexp):
        self.lib.hyacinXquantizeScaleBatch(byref(self.h), batches, seg_m, last_m, n, atype, _dp(A), lda, u, _dp(vexp))

    def herk_batch(self, batches, seg_m, last_m, n, atype, A, lda, u, vexp, beta, order_c, C):
        self.lib.hyacinXherkBatch(byref(self.h), batches, seg_m, last_m, n, atype, _dp(A), lda, u, _dp(vexp), beta, order_c, _dp(C))

    def herk_batch_static(self, batches, seg_m, last_m, n, atype, A, lda, u, vexp, beta, order_c, C) -> int:
        """hyacinXherkBatch with all scratch in the module's fixed array (no allocation); 0 on success."""
        return int(self.lib.hyacinB200HerkBatchStatic(byref(self.h), batches, seg_m, last_m, n, atype, _dp(A), lda, u, _dp(vexp),
                                                     beta, order_c, _dp(C)))

    def allreduce_vexp(self, n, vexp):
        self.lib.hyacinAllReduceVExp(byref(self.h), n, _dp(vexp))

    def allreduce_1drow(self, cpanels, order, count, C):
        self.lib.hyacinAllReduce1Drow(byref(self.h), cpanels, order, count, _dp(C))

    def dequantize_init(self, n, order_c, C, vexp, atype):
        g, b = c_int32(-1), c_int32(0)
        self.lib.hyacinXdequantizeInit(byref(self.h), n, order_c, _dp(C), _dp(vexp), atype, byref(g), byref(b))
        return g.value, b.value

    def dequantize(self, n, order_c, C, vexp, gtype, G, ldg):
        self.lib.hyacinXdequantize(byref(self.h), n, order_c, _dp(C), _dp(vexp), gtype, _dp(G), ldg)

    def gevd(self, eps, n, k, atype, X, ldx, S, gtype, G, ldg) -> int:
        return self.lib.hyacinXGevd(byref(self.h), eps, n, k, atype, _dp(X), ldx, _dp(S), gtype, _dp(G), ldg)

    def ginterp(self, eps, n, k, atype, X, ldx, jpiv, gtype, G, ldg) -> int:
        return self.lib.hyacinXGinterp(byref(self.h), eps, n, k, atype, _dp(X), ldx, _dp(jpiv), gtype, _dp(G), ldg)

    # ---- fits -----------------------------------------------------------------------------------
    def tsvd_fit(self, eps, op, m, n, k, A, lda, S, V, ldv, global_m, ctype, segment_n=False) -> int:
        fn = self.lib.hyacinTsvdFitSegmentN if segment_n else self.lib.hyacinTsvdFit
        return fn(byref(self.h), eps, op.encode(), m, n, k, _dp(A), lda, _dp(S), _dp(V), ldv, global_m, ctype)

    def interpolate_fit(self, eps, op, m, n, k, A, lda, jpvt, V, ldv, global_m, ctype) -> int:
        return self.lib.hyacinInterpolateFit(byref(self.h), eps, op.encode(), m, n, k, _dp(A), lda, _dp(jpvt), _dp(V), ldv, global_m, ctype)

    def check_norm(self, op, m, n, A, lda, rank, V, ldv, ctype) -> float:
        return self.lib.hyacinCheckNorm(byref(self.h), op.encode(), m, n, _dp(A), lda, rank, _dp(V), ldv, ctype)

    def sync_timer(self, want: str = "DRC"):
        """Synchronise; returns {'D': ms, 'R': ms, 'C': ms} when the handle owns a timer (HYACIN_CREATE_TIMER=1)."""
        arr = (c_double * len(want))(*[float(ord(c)) for c in want])
        self.lib.hyacinSync_TimerSegments(byref(self.h), arr, len(want))
        return {c: arr[i] for i, c in enumerate(want)} if self.h.timer else None

    # ---- B200-only stage entry points ----------------------------------------------------------------
    def status(self, clear: bool = True) -> int:
        return int(self.lib.hyacinB200Status(1 if clear else 0))

    def vector_range(self, batches, n, u, vexp, seg_u):
        self.lib.hyacinB200VectorRange(byref(self.h), batches, n, u, _dp(vexp), _dp(seg_u))

    def self_test_wait(self, poll_limit: int, code: int) -> int:
        """Make a bounded wait expire on purpose (harmlessly); the code then shows in status()."""
        return int(self.lib.hyacinB200SelfTestWait(byref(self.h), poll_limit, code))

    def launch_count(self, reset: bool = False) -> int:
        return int(self.lib.hyacinB200LaunchCount(1 if reset else 0))

    def profile_enable(self, on: bool):
        self.lib.hyacinB200ProfileEnable(1 if on else 0)

    def profile_read(self):
        gm, gn, qm, qn = c_double(), c_int32(), c_double(), c_int32()
        self.lib.hyacinB200ProfileRead(byref(gm), byref(gn), byref(qm), byref(qn))
        return {"gram_ms": gm.value, "gram_launches": gn.value, "quantize_ms": qm.value, "quantize_launches": qn.value}

    def profile_read_tail(self):
        cm, cn, sm, sn = c_double(), c_int32(), c_double(), c_int32()
        self.lib.hyacinB200ProfileReadTail(byref(cm), byref(cn), byref(sm), byref(sn))
        return {"cholesky_ms": cm.value, "cholesky_launches": cn.value, "svd_ms": sm.value, "svd_calls": sn.value}

    def pivoted_cholesky(self, eps, n, k, gtype, G, ldg, jpiv, R, ldr) -> int:
        """Pivoted Cholesky alone: rank, pivots and the factor in pivoted column order (Gram format)."""
        return int(self.lib.hyacinB200PivotedCholesky(byref(self.h), eps, n, k, gtype, _dp(G), ldg, _dp(jpiv), _dp(R), ldr))

    def crt_plan(self, u: int, cplx: int, rows: int):
        a, b, c, d = c_int32(), c_int32(), c_int32(), c_int32()
        self.lib.hyacinB200CrtPlan(u, cplx, rows, byref(a), byref(b), byref(c), byref(d))
        return {"moduli": a.value, "value_bytes": b.value, "group_rows": c.value, "chunk_rows": d.value}

    def tile_info(self, n: int):
        a, b, c, d = c_int32(), c_int32(), c_int32(), c_int32()
        self.lib.hyacinB200TileInfo(n, byref(a), byref(b), byref(c), byref(d))
        return {"tile_y": a.value, "tile_x": b.value, "tiles_y": c.value, "num_tiles": d.value}

    def quantize_crt(self, atype, rows, n, A, lda, vexp, moduli, value_bytes, W, ldk):
        self.lib.hyacinB200QuantizeCrt(byref(self.h), atype, rows, n, _dp(A), lda, _dp(vexp), moduli, value_bytes, _dp(W), ldk)

    def gram_residues(self, n, moduli, W, ldw, plane_stride, ka0, kb0, k_rows, accumulate, residues):
        self.lib.hyacinB200GramResidues(byref(self.h), n, moduli, _dp(W), ldw, plane_stride, ka0, kb0, k_rows, accumulate, _dp(residues))

    def quantize_limbs(self, atype, rows, n, A, lda, vexp, order, W, ldk):
        self.lib.hyacinB200QuantizeLimbs(byref(self.h), atype, rows, n, _dp(A), lda, _dp(vexp), order, _dp(W), ldk)

    def gram_limbs(self, n, order, W, ldw, plane_stride, ka0, kb0, k_rows, beta, order_c, C):
        self.lib.hyacinB200GramLimbs(byref(self.h), n, order, _dp(W), ldw, plane_stride, ka0, kb0, k_rows, beta, order_c, _dp(C))

    def dequantize_via_slices(self, n, order_c, C, vexp, atype, ranks, G, ldg):
        """Gram format and matrix from the slices `ranks` ranks would exchange (the fits' post-collective route)."""
        g = c_int32()
        self.lib.hyacinB200DequantizeViaSlices(byref(self.h), n, order_c, _dp(C), _dp(vexp), atype, ranks, byref(g), _dp(G), ldg)
        return g.value

    def reconstruct(self, n, moduli, residues, beta, order_c, C):
        self.lib.hyacinB200Reconstruct(byref(self.h), n, moduli, _dp(residues), beta, order_c, _dp(C))
