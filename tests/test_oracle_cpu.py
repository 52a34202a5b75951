"""CPU tests: the oracle against exact big-integer arithmetic, the reference's two int8 decompositions, and the
C-ABI surface of the built library (symbols and struct layout only -- no compute without a GPU)."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

from hyacinth_b200 import api
from oracle import oracle as O
from tests.helpers import random_matrix

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("atype,eps", [(O.F64, 1e-10), (O.F64C, 1e-12), (O.F32, 1e-5), (O.F32C, 1e-4)])
def test_c_oracle_equals_python_bigint(atype, eps):
    rng = np.random.default_rng(atype)
    m, n = 70, 9
    A = random_matrix(rng, m, n, atype, zero_cols=(3,))
    u, cp, lp, tri = O.herk_init(eps, m, n, atype)
    b, s, l = O.segments(m, 32)
    vexp = O.column_exponents(A, atype, u, b, s, l)
    assert vexp[0, 3] == O.INT_MAX and np.array_equal(vexp[0], vexp[1:].min(axis=0))
    q = O.quantize_ints(A, atype, vexp[0])
    for j in range(n):
        for i in range(0, m, 5):
            parts = [A[i, j].real, A[i, j].imag] if atype & 1 else [A[i, j]]
            for p, val in enumerate(parts):
                assert q[p][j][i] == O.py_quantize(float(val), int(vexp[0][j]))
    C = O.gram_exact(A, atype, vexp[0], lp)
    for (p, y, x), v in O.py_gram(q, bool(atype & 1)).items():
        words = [C[p * lp + k, y + x * (x + 1) // 2] for k in range(lp)]
        assert O.limbs_to_int(words, lp) == v
        assert [int(w) for w in words] == O.int_to_limbs(v, lp)


def test_exponent_rule_and_rounding_known_answers():
    """Hand-computed values: column scale from frexp, ties-to-even rounding, zero and subnormal columns."""
    A = np.array([[1.0, 0.75, 0.0, 5e-324], [-3.0, 0.5, 0.0, 0.0]], dtype=np.float64)
    vexp = O.column_exponents(A, O.F64, 10, 1, 2, 2)
    # max|col| = 3 -> e = 2; 0.75 -> e = 0; zero and subnormal maxima -> INT_MAX
    assert vexp[0].tolist() == [8, 10, O.INT_MAX, O.INT_MAX]
    assert O.py_quantize(2.5, 0) == 2 and O.py_quantize(3.5, 0) == 4 and O.py_quantize(-2.5, 0) == -2
    q = O.quantize_ints(np.array([[2.5], [3.5], [-0.5], [1.5]]), O.F64, np.array([0], dtype=np.int32))
    assert q[0][0] == [2, 4, 0, 2]
    # herk sizing: eps = 2^-33.2.. -> u = 33, +7 guard bits, two limb panels for 2^20 rows
    assert O.herk_init(1e-10, 1 << 20, 4096, O.F64) == (40, 1, 2, 4096 * 4097 // 2)
    assert O.herk_init(1e-12 * np.sqrt(0.5), 1 << 19, 1024, O.F64C)[:3] == (47, 2, 2)
    assert O.herk_init(1e-5, 1 << 20, 8192, O.F32)[:3] == (23, 1, 2)
    assert O.herk_init(0.5, 4, 4, O.F64)[0] == 1 + 7      # eps a power of two: one more bit


def test_reference_decompositions_reduce_to_the_plain_gram():
    """The reference's CRT-residue route and its balanced-limb route both give sum(q_y q_x) exactly."""
    rng = np.random.default_rng(5)
    for u in (7, 14, 30, 40, 59):
        qy = [int(v) for v in rng.integers(-2**u, 2**u, size=300, dtype=np.int64)]
        qx = [int(v) for v in rng.integers(-2**u, 2**u, size=300, dtype=np.int64)]
        exact = sum(a * b for a, b in zip(qy, qx))
        order_crt = next(k for k in range(1, 25) if 2 * u + 1 + 9 <= [8, 15, 23, 31, 39, 47, 55, 63, 71, 79, 87, 94, 102, 110, 118,
                                                                         125, 133, 140, 148, 155, 163, 170, 177, 185][k - 1])
        assert O.ref_crt_gram_entry(qy, qx, order_crt) == exact
        order_limb = 1 + next(i for i, b in enumerate(O.REF_LIMB_BITS) if b >= u + 1)
        assert O.ref_limb_gram_entry(qy, qx, order_limb) == exact


def test_allreduce_sum_and_dequantize_roundtrip():
    rng = np.random.default_rng(11)
    m, n, atype = 64, 12, O.F64
    parts = [random_matrix(rng, m, n, atype, col_scale_decades=0.0) for _ in range(3)]
    full = np.vstack(parts)
    u, cp, lp, tri = O.herk_init(1e-10, 3 * m, n, atype)
    vexp = O.column_exponents(full, atype, u, 1, 3 * m, 3 * m)
    Cs = [O.gram_exact(p, atype, vexp[0], lp) for p in parts]
    total = O.allreduce_sum(Cs, cp, lp)
    assert np.array_equal(total, O.gram_exact(full, atype, vexp[0], lp))
    g, gbytes, bits = O.dequantize_init(total, vexp[0], n, lp, atype)
    assert g == O.DD and gbytes == 16
    G = O.dequantize(total, vexp[0], n, lp, g)
    Gf = (G[:, :, 0] + G[:, :, 1]).T
    ref = full.T @ full
    assert np.abs(Gf - ref).max() <= 1e-9 * np.abs(ref).max()
    assert np.array_equal(Gf, Gf.T)


def test_library_exports_the_whole_abi():
    lib_path = api.DEFAULT_LIB
    assert os.path.exists(lib_path), "build the library first: python -m hyacinth_b200._build"
    out = subprocess.check_output(["nm", "-D", "--defined-only", lib_path], text=True)
    exported = {line.split()[-1] for line in out.splitlines() if " T " in line}
    for name in api.PUBLIC_SYMBOLS + api.B200_SYMBOLS:
        assert name in exported, name
    lib = api.load(lib_path)             # dlopen + prototypes; no CUDA call is made
    assert lib.hyacinTsvdFit.restype is ctypes.c_int32


def test_handle_layout_matches_the_c_header(tmp_path):
    """sizeof/offsetof of hyacinHandle_t as the C compiler sees include/hyacin.h == the ctypes mirror
    (and == the reference's header when its tree is mounted)."""
    fields = [f for f, _ in api.HyacinHandle._fields_]
    prog = "#include <stdio.h>\n#include <stddef.h>\n#include <hyacin.h>\nint main(){printf(\"%zu\", sizeof(hyacinHandle_t));" + \
        "".join(f'printf(" %zu", offsetof(hyacinHandle_t, {f}));' for f in fields) + "return 0;}\n"
    src = tmp_path / "layout.c"
    src.write_text(prog)
    want = [ctypes.sizeof(api.HyacinHandle)] + [getattr(api.HyacinHandle, f).offset for f in fields]
    includes = [os.path.join(ROOT, "include")]
    ref_include = os.path.join(O.reference_tree(), "include")
    if os.path.isdir(ref_include):
        includes.append(ref_include)
    for inc in includes:
        exe = tmp_path / "layout"
        subprocess.check_call(["gcc", "-I", inc, "-I", "/usr/local/cuda/include", str(src), "-o", str(exe)])
        got = [int(v) for v in subprocess.check_output([str(exe)], text=True).split()]
        assert got == want, inc


def test_trace_summation_order_of_the_cholesky_stop_rule():
    """The stop rule of the pivoted Cholesky compares rounding noise for exactly rank-deficient matrices, so the order
    of the trace sum is part of the result.  A pure-Python statement of the reference's reduction (candidate th in
    thread th % 128 of block th // 128; its first thread takes one extra value first; shuffle tree over 32 lanes,
    four warps left to right; thread t of block 0 then walks blocks t + 1, t + 129, ...; same tree again) against the
    C oracle, on values whose sum depends on the order."""
    def tree128(x):
        g = []
        for w in range(4):
            v = list(x[32 * w:32 * w + 32])
            o = 1
            while o < 32:
                for i in range(0, 32 - o, 2 * o):
                    v[i] = v[i] + v[i + o]
                o *= 2
            g.append(v[0])
        return ((g[0] + g[1]) + g[2]) + g[3]

    def reference_sum(d, special):
        count = len(d)
        nb = max(1, -(-count // 128))
        agg = []
        for b in range(nb):
            x = [float(d[128 * b + t]) if 128 * b + t < count else 0.0 for t in range(128)]
            if b == 0 and special is not None:
                x[0] = (0.0 + special) + x[0]
            agg.append(tree128(x))
        u = []
        for t in range(128):
            acc = agg[0] if t == 0 else 0.0
            for i in range(t + 1, nb, 128):
                acc += agg[i]
            u.append(acc)
        return tree128(u)

    rng = np.random.default_rng(5)
    differs = 0
    for count, special in [(1, None), (5, 0.3), (127, None), (128, 1e-3), (129, None), (1000, -2.5e-9), (4095, 7.0), (18943, None), (0, 1.5)]:
        d = rng.standard_normal(count) * 10.0 ** rng.uniform(-12, 0, count)
        want = reference_sum(d, special)
        assert O.trace_in_reference_order(d, special) == want
        differs += want != float(np.sum(d) + (special or 0.0))
    assert differs > 0            # the order does matter for such values
