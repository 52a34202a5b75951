"""CPU oracle for the quantized-Gram path.  TEST INFRASTRUCTURE ONLY.

Two independent statements of the same contract:

* thin ctypes wrappers around ``liboracle.so`` (``oracle_gram.c``; fast enough for a few thousand rows), and
* pure-Python big-integer versions for small cases, including emulations of the reference's two int8
  decompositions (balanced base-256 limbs and centred CRT residues) that show both reduce to the plain
  sum of products.

Only tests, the smoke check and the benchmark's CPU leg may import this module; the product library never
does.  Parity status: the reference has no tests or golden vectors of its own, so these functions are
pinned against fixtures recorded from the reference's CUDA build (``tests/golden``).
"""
from __future__ import annotations

import ctypes
import math
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

INT_MAX = 2**31 - 1
INT_MIN = -(2**31)

# hyacinPrecision_t values
F64, F64C, F32, F32C, F16, F16C, DD, DDC, TF, TFC, QF, QFC = range(12)
_NP_OF = {F64: np.float64, F64C: np.complex128, F32: np.float32, F32C: np.complex64, F16: np.float16}


def reference_tree() -> str:
    """Directory of the reference's source tree: $HYACIN_REFERENCE_SRC, else the default of oracle/Makefile."""
    return subprocess.check_output(["make", "-s", "--no-print-directory", "-C", _HERE, "print-ref"], text=True).strip()


def build(force: bool = False) -> str:
    """Compile oracle_gram.c into liboracle.so next to it (gcc, no external dependencies)."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "oracle_gram.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["gcc", "-O2", "-std=c11", "-ffp-contract=off", "-fPIC", "-shared", src, "-o", so, "-lm"])
    return so


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build())
        _LIB.orc_dequantize_init.restype = ctypes.c_int32
    return _LIB


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def _kind(atype: int):
    """(element kind for the C code, complex flag, flush-subnormal flag) of an input precision."""
    cplx = atype & 1
    base = atype & ~1
    if base == F64:
        return 0, cplx, 0
    if base == F32:
        return 2, cplx, 1
    if base == F16:
        return 2, cplx, 0      # widened to float by the caller; half subnormals are float normals
    raise ValueError("input precision must be one of the first six")


def as_c_input(A: np.ndarray, atype: int) -> np.ndarray:
    """Column-major copy of A in the element type the C oracle reads (half widened to float)."""
    base = atype & ~1
    if base == F16:
        A = A.astype(np.complex64 if atype & 1 else np.float32)
    return np.asfortranarray(A)


def herk_init(eps: float, global_m: int, n: int, atype: int, corr: int = 7):
    """(u_corr, cPanels, lPanels, stride) -- src/hyacin_herk.cpp:45-59."""
    u, cp, lp = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
    st = ctypes.c_uint64()
    lib().orc_herk_init(ctypes.c_double(eps), ctypes.c_uint64(max(global_m, 0)), ctypes.c_int32(n),
                        ctypes.c_int32(atype), ctypes.c_int32(corr), ctypes.byref(u), ctypes.byref(cp),
                        ctypes.byref(lp), ctypes.byref(st))
    return u.value, cp.value, lp.value, st.value


def segments(m: int, seg_k: int = 8192):
    """(batches, segM, lastM) as the fitting drivers derive them -- src/lra.cpp:55-57."""
    it = m if seg_k <= 0 else min(seg_k, m)
    q, r = divmod(m, max(1, it))
    return q + (1 if r else 0), it, (r if r else it)


def column_exponents(A: np.ndarray, atype: int, u: int, batches: int, seg_m: int, last_m: int) -> np.ndarray:
    """(batches+1) x N int32 exponent table -- src/fp_exponent.cu:25-51."""
    Ac = as_c_input(A, atype)
    n = Ac.shape[1]
    kind, cplx, _ = _kind(atype)
    rows = (batches + 1) if batches > 0 and u >= 0 else 1
    vexp = np.zeros((rows, n), dtype=np.int32)
    lib().orc_column_exponents(ctypes.c_int32(kind), ctypes.c_int32(cplx), ctypes.c_int32(batches),
                               ctypes.c_int32(seg_m), ctypes.c_int32(last_m), ctypes.c_int32(n), _ptr(Ac),
                               ctypes.c_int64(Ac.shape[0]), ctypes.c_int32(u), _ptr(vexp))
    return vexp


def vector_range(vexp: np.ndarray, u: int) -> np.ndarray:
    """Bits needed per row segment -- src/fp_exponent.cu:67-73."""
    batches, n = vexp.shape[0] - 1, vexp.shape[1]
    out = np.zeros(batches, dtype=np.int32)
    v = np.ascontiguousarray(vexp)
    lib().orc_vector_range(ctypes.c_int32(batches), ctypes.c_int32(n), ctypes.c_int32(u), _ptr(v), _ptr(out))
    return out


def quantize_raw(A: np.ndarray, atype: int, vexp0: np.ndarray) -> np.ndarray:
    """Quantised integers as a uint64 array [parts][N][M][2] (little-endian halves of a signed 128-bit value)."""
    Ac = as_c_input(A, atype)
    m, n = Ac.shape
    kind, cplx, ftz = _kind(atype)
    q = np.zeros((1 + cplx, n, m, 2), dtype=np.uint64)
    v = np.ascontiguousarray(vexp0, dtype=np.int32)
    lib().orc_quantize(ctypes.c_int32(kind), ctypes.c_int32(cplx), ctypes.c_int32(ftz), ctypes.c_int32(m),
                       ctypes.c_int32(n), _ptr(Ac), ctypes.c_int64(m), _ptr(v), _ptr(q))
    return q


def quantize_ints(A: np.ndarray, atype: int, vexp0: np.ndarray):
    """Quantised values as nested Python ints: q[part][col][row] (small inputs only)."""
    raw = quantize_raw(A, atype, vexp0)
    out = []
    for part in raw:
        cols = []
        for col in part:
            vals = []
            for lo, hi in col.tolist():
                v = (hi << 64) | lo
                vals.append(v - (1 << 128) if v >> 127 else v)
            cols.append(vals)
        out.append(cols)
    return out


def gram_exact(A: np.ndarray, atype: int, vexp0: np.ndarray, order: int, C: np.ndarray | None = None) -> np.ndarray:
    """Packed integer Gram [cPanels*order, tri] (uint64) of the quantised matrix; accumulates into C if given."""
    raw = quantize_raw(A, atype, vexp0)
    parts, n, m, _ = raw.shape
    tri = n * (n + 1) // 2
    beta = 0 if C is None else 1
    if C is None:
        C = np.zeros((parts * order, tri), dtype=np.uint64)
    else:
        C = np.ascontiguousarray(C, dtype=np.uint64).copy()
    lib().orc_gram_exact(ctypes.c_int32(parts - 1), ctypes.c_int32(m), ctypes.c_int32(n), _ptr(raw),
                         ctypes.c_int32(order), ctypes.c_int32(beta), _ptr(C))
    return C


def allreduce_sum(parts: list[np.ndarray], panels: int, order: int) -> np.ndarray:
    """Exact sum of per-rank packed Grams -- the contract of src/allreduce_1drow.cu:145-169."""
    stack = np.ascontiguousarray(np.stack([np.ascontiguousarray(p, dtype=np.uint64).reshape(-1) for p in parts]))
    count = stack.shape[1] // (panels * order)
    out = np.zeros(stack.shape[1], dtype=np.uint64)
    lib().orc_allreduce_sum(ctypes.c_int32(len(parts)), ctypes.c_int32(panels), ctypes.c_int32(order),
                            ctypes.c_int64(count), _ptr(stack), _ptr(out))
    return out.reshape(panels * order, count)


def dequantize_init(C: np.ndarray, vexp0: np.ndarray, n: int, order: int, atype: int, corr: int = 7,
                    f64_capable: int = 1):
    """(Gtype, element bytes, bits) -- src/fp_i63tp_dequantize.cu:17-54."""
    eb, bits = ctypes.c_int32(), ctypes.c_int32()
    Cc = np.ascontiguousarray(C, dtype=np.uint64)
    v = np.ascontiguousarray(vexp0, dtype=np.int32)
    g = lib().orc_dequantize_init(ctypes.c_int32(n), ctypes.c_int32(order), _ptr(Cc), _ptr(v), ctypes.c_int32(atype),
                                  ctypes.c_int32(corr), ctypes.c_int32(f64_capable), ctypes.byref(eb), ctypes.byref(bits))
    return g, eb.value, bits.value


def dequantize(C: np.ndarray, vexp0: np.ndarray, n: int, order: int, gtype: int) -> np.ndarray:
    """Full N x N Gram in the chosen format, returned as raw float64/float32 words.

    Shape (N, N, w) in column-major element order [x][y][w]: w = 1 (F64/F32), 2 (complex or double-double),
    4 (complex double-double: re.hi, re.lo, im.hi, im.lo) -- src/fp_i63tp_dequantize.cu:121-129.
    """
    base, cplx = gtype & ~1, gtype & 1
    if base not in (F64, F32, DD):
        raise ValueError("oracle dequantises to F64, F32 and double-double only")
    words = (2 if base == DD else 1) * (2 if cplx else 1)
    dt = np.float32 if base == F32 else np.float64
    G = np.zeros((n, n, words), dtype=dt)
    Cc = np.ascontiguousarray(C, dtype=np.uint64)
    v = np.ascontiguousarray(vexp0, dtype=np.int32)
    lib().orc_dequantize(ctypes.c_int32(n), ctypes.c_int32(order), _ptr(Cc), _ptr(v), ctypes.c_int32(gtype), _ptr(G),
                         ctypes.c_int64(n))
    return G


# ------------------------------------------------------------------------------------------------------
# Pure-Python big-integer statements (small cases)
# ------------------------------------------------------------------------------------------------------

def pivoted_cholesky(G: np.ndarray, cap: int, eps: float):
    """Truncated pivoted Cholesky of an n x n FP64 (real or complex) Gram matrix with the reference's rounding --
    src/hyacin_potrfp.cu:214-272.  Returns (rank, one-based pivots, R) with R[k, x] = factor entry of row k and the
    column at pivot position x (zero below the diagonal), `min(cap + 1, n)` rows."""
    n = G.shape[0]
    cplx = 1 if np.iscomplexobj(G) else 0
    Gc = np.asfortranarray(G.astype(np.complex128 if cplx else np.float64))
    rows = min(cap + 1, n)
    R = np.zeros((rows, n), dtype=Gc.dtype, order="F")
    jpiv = np.zeros(n, dtype=np.int32)
    fn = lib().orc_potrfp_f64
    fn.restype = ctypes.c_int32
    rank = fn(ctypes.c_int32(n), ctypes.c_int32(cap), ctypes.c_double(eps), ctypes.c_int32(cplx), _ptr(Gc), ctypes.c_int64(n),
              _ptr(jpiv), _ptr(R), ctypes.c_int64(rows))
    return int(rank), jpiv, R


def trace_in_reference_order(d: np.ndarray, special=None) -> float:
    """Sum of the remaining diagonal entries `d` (by candidate number) in the order of the reference's reduction
    (src/hyacin_potrfp.cu:128-132, 243-261); `special` is the extra value its first thread takes before its own."""
    d = np.ascontiguousarray(d, dtype=np.float64)
    fn = lib().orc_trace_in_reference_order
    fn.restype = ctypes.c_double
    return float(fn(_ptr(d), ctypes.c_int32(d.size), ctypes.c_int32(0 if special is None else 1), ctypes.c_double(0.0 if special is None else special)))


def limbs_to_int(words, order: int) -> int:
    """Value of one packed entry given its `order` 63-bit limbs (last limb signed)."""
    v = 0
    for l in range(order):
        w = int(words[l])
        if l + 1 == order and w >> 63:
            w -= 1 << 64
        v += w << (63 * l)
    return v


def int_to_limbs(v: int, order: int):
    out = []
    for l in range(order):
        if l + 1 == order:
            out.append(v & ((1 << 64) - 1))
        else:
            out.append(v & ((1 << 63) - 1))
            v >>= 63
    return out


def py_quantize(a: float, expon: int) -> int:
    """rint_ties_even(a * 2^expon) with exact rational arithmetic -- src/quantize_limbs.cu:14-18."""
    if expon == INT_MAX or a == 0.0:
        return 0
    from fractions import Fraction
    v = Fraction(a) * (Fraction(2) ** expon)
    fl = math.floor(v)
    r = v - fl
    if r > Fraction(1, 2) or (r == Fraction(1, 2) and fl % 2 == 1):
        fl += 1
    return fl


def py_gram(q, cplx: bool):
    """Exact Gram of quantised ints q[part][col][row]; returns dict[(part, y, x)] for y <= x."""
    n = len(q[0])
    out = {}
    for x in range(n):
        for y in range(x + 1):
            re = sum(a * b for a, b in zip(q[0][y], q[0][x]))
            if cplx:
                re += sum(a * b for a, b in zip(q[1][y], q[1][x]))
                im = sum(a * b for a, b in zip(q[0][y], q[1][x])) - sum(a * b for a, b in zip(q[1][y], q[0][x]))
                out[(1, y, x)] = im
            out[(0, y, x)] = re
    return out


# The reference's real CRT moduli (include/crt_constants.hpp:7) and its limb capacities
# (src/hyacin_herk.cpp:12).
REF_CRT_MODULI = [256, 253, 251, 249, 247, 241, 239, 235, 233, 229, 227, 223, 217, 211, 199, 197, 193, 191, 181, 179,
                  173, 167, 163, 157]
REF_LIMB_BITS = [7, 14, 22, 30, 38, 46, 54, 62, 70, 78, 86, 94]


def ref_crt_gram_entry(qy, qx, order: int) -> int:
    """One Gram entry the way the reference's CRT route forms it: centred int8 residues
    (src/quantize_crt_real.cu:30-34), residue products summed mod m (src/crt_diag_real.cu:5-10), then
    reconstruction into the symmetric range (-P/2, P/2) (src/crt_reconstruct_real.cu:66-89)."""
    mods = REF_CRT_MODULI[:order]
    P = math.prod(mods)
    total = 0
    for m in mods:
        def centred(v):
            r = v % m
            return r - m if r > 127 else r
        s = sum(centred(a) * centred(b) for a, b in zip(qy, qx)) % m
        Pm = P // m
        total += ((s * pow(Pm, -1, m)) % m) * Pm
    total %= P
    return total - P if total > P // 2 else total


def ref_limb_gram_entry(qy, qx, order: int) -> int:
    """One Gram entry the way the reference's limb route forms it: balanced base-256 digits
    (src/quantize_limbs.cu:29-44) and the shifted sum of digit-plane products (src/limbs_diag.cu:20-41,
    src/limbs_cross_real.cu:20-42)."""
    def digits(v):
        out = []
        for _ in range(order):
            d = ((v + 128) % 256) - 128
            out.append(d)
            v = (v - d) // 256
        return out
    dy = [digits(v) for v in qy]
    dx = [digits(v) for v in qx]
    total = 0
    for i in range(order):
        for j in range(order):
            total += sum(a[i] * b[j] for a, b in zip(dy, dx)) << (8 * (i + j))
    return total
