"""Pins the CPU oracle to outputs recorded from the reference's own CUDA library (tests/golden/*.npz, written by
tests/golden/make_golden.py on a B200): column exponents, packed integer Gram, Gram format and every byte of the
dequantised Gram must be reproduced exactly; the recorded rank and singular values must agree with LAPACK."""
import glob
import os

import numpy as np
import pytest

from oracle import oracle as O
from tests.helpers import CHOLESKY_CASES, cholesky_case, factor_digest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FIXTURES = sorted(p for p in glob.glob(os.path.join(GOLDEN, "*.npz")) if not os.path.basename(p).startswith("chol_"))


def test_fixtures_are_present():
    assert len(FIXTURES) >= 6


@pytest.mark.parametrize("path", FIXTURES, ids=[os.path.basename(p)[:-4] for p in FIXTURES])
def test_oracle_reproduces_reference_outputs(path):
    f = np.load(path)
    A, atype, eps = f["A"], int(f["atype"]), float(f["eps"])
    m, n = A.shape
    u, cp, lp, tri = O.herk_init(eps, m, n, atype)
    assert (u, cp, lp) == (int(f["u"]), int(f["cpanels"]), int(f["lpanels"]))
    b, s, l = O.segments(m, int(f["seg_k"]))
    assert [b, s, l] == f["segments"].tolist()
    vexp = O.column_exponents(A, atype, u, b, s, l)
    np.testing.assert_array_equal(vexp, f["vexp"])
    C = O.gram_exact(A, atype, vexp[0], lp)
    np.testing.assert_array_equal(C, f["C"])
    g, gbytes, _ = O.dequantize_init(C, vexp[0], n, lp, atype, corr=7, f64_capable=1)
    assert (g, gbytes) == (int(f["gtype"]), int(f["gbytes"]))
    G = O.dequantize(C, vexp[0], n, lp, g)
    np.testing.assert_array_equal(G.view(np.uint8).reshape(n, n * gbytes), f["G"])


@pytest.mark.parametrize("path", FIXTURES, ids=[os.path.basename(p)[:-4] for p in FIXTURES])
def test_recorded_fit_agrees_with_lapack(path):
    """The reference's rank follows the tail-energy rule on the true singular values, and its singular values
    are the true ones to the accuracy the quantisation allows."""
    f = np.load(path)
    A, eps, rank = f["A"].astype(np.complex128 if int(f["atype"]) & 1 else np.float64), float(f["eps"]), int(f["svd_rank"])
    s = np.linalg.svd(A, compute_uv=False)
    tail = np.sqrt(np.cumsum((s ** 2)[::-1])[::-1])
    want = int((tail > eps * tail[0]).sum())
    assert abs(rank - want) <= 1
    got = f["S"][:rank].astype(np.float64)
    base = int(f["atype"]) & ~1
    tol = {0: 1e-9, 2: 1e-4, 4: 2e-2}[base]
    assert np.max(np.abs(got - s[:rank])) <= tol * s[0]
    jp = f["jpiv"]
    assert sorted(jp.tolist()) == list(range(1, A.shape[1] + 1))      # a permutation, one-based


@pytest.mark.parametrize("name", sorted(CHOLESKY_CASES))
def test_oracle_cholesky_reproduces_reference_factor(name):
    """The restated pivoted Cholesky gives the recorded rank, every recorded pivot and every bit of the factor the
    reference's kernel left in its Gram matrix (src/hyacin_potrfp.cu:214-272), on matrices with ties at nearly every
    step, with more steps than chains, with a column cap, and with a counted last column."""
    path = os.path.join(GOLDEN, name + ".npz")
    assert os.path.exists(path), "fixture missing: run tests/golden/make_golden.py on a B200"
    f = np.load(path)
    G, cap, eps = cholesky_case(name)
    rank, jpiv, R = O.pivoted_cholesky(G, cap, eps)
    assert rank == int(f["rank"])
    np.testing.assert_array_equal(jpiv, f["jpiv"])
    R = np.ascontiguousarray(R[:rank])
    np.testing.assert_array_equal(np.diagonal(R).real, f["diag"])
    if f["R"].size:
        np.testing.assert_array_equal(R.view(np.uint8), np.ascontiguousarray(f["R"]).view(np.uint8))
    assert factor_digest(R) == str(f["digest"])
