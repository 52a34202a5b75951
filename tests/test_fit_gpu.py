"""GPU tests of the fits behind the public entry points: hyacinTsvdFit, hyacinTsvdFitSegmentN,
hyacinInterpolateFit, hyacinCheckNorm, and the replicated stage functions hyacinXGevd / hyacinXGinterp.

Checked against host LAPACK (numpy) on the small BASELINE configuration and, side by side, against the
reference's own CUDA library: identical rank and pivots, singular values within 1e-12 relative for FP64
(1e-5 for FP32), relative projection error <= eps.
"""
import numpy as np
import pytest

from hyacinth_b200 import api
from tests.helpers import low_rank_matrix, random_matrix, to_device_colmajor

pytestmark = pytest.mark.gpu


def _torch():
    import torch
    return torch


def _real_dtype(atype):
    torch = _torch()
    return {api.F64: torch.float64, api.F32: torch.float32, api.F16: torch.float16}[atype & ~1]


def _alloc_v(n, k, atype):
    torch = _torch()
    words = 2 if atype & 1 else 1
    return torch.zeros((k, n * words), dtype=_real_dtype(atype), device="cuda")


def _tsvd(lib, dA, op, m, n, k, lda, eps, atype, global_m=None, segment_n=False):
    torch = _torch()
    S = torch.zeros(k, dtype=_real_dtype(atype), device="cuda")
    V = _alloc_v(n, k, atype)
    rank = lib.tsvd_fit(eps, op, m, n, k, dA, lda, S, V, n, global_m or m, atype, segment_n=segment_n)
    torch.cuda.synchronize()
    return rank, S, V


def _rel_error(lib, dA, op, m, n, lda, rank, V, atype):
    tot = lib.check_norm(op, m, n, dA, lda, 0, None, 0, atype)
    res = lib.check_norm(op, m, n, dA, lda, rank, V, n, atype)
    return float(np.sqrt(res / tot)) if tot > 0 else 0.0


def test_tsvd_fit_small_configuration_against_lapack(hy):
    """512 x 128 FP64, rank-16 spectrum 10^(-12 i / 15), noise 1e-14, eps 1e-10: rank 16, sigma to 1e-12 relative."""
    rng = np.random.default_rng(20240611 + 1)
    m, n, k, eps = 512, 128, 128, 1e-10
    sigma = 10.0 ** (-12.0 * np.arange(16) / 15.0)
    A = low_rank_matrix(rng, m, n, 16, sigma, 1e-14)
    dA = to_device_colmajor(A)
    rank, S, V = _tsvd(hy, dA, "N", m, n, k, m, eps, api.F64)
    s_ref = np.linalg.svd(A, compute_uv=False)
    tail = np.sqrt(np.cumsum((s_ref ** 2)[::-1])[::-1])
    want_rank = int((tail > eps * tail[0]).sum())
    assert rank == want_rank
    got = S.cpu().numpy()
    assert np.all(got[rank:] == 0)
    # singular values relative to the largest one: the Gram route resolves sigma_i / sigma_1 down to about eps
    assert np.max(np.abs(got[:rank] - s_ref[:rank]) / s_ref[0]) < 1e-12
    assert np.max(np.abs(got[:8] - s_ref[:8]) / s_ref[:8]) < 1e-9
    Vh = V.cpu().numpy()[:rank].T          # n x rank
    assert np.abs(Vh.T @ Vh - np.eye(rank)).max() < 1e-10
    assert _rel_error(hy, dA, "N", m, n, m, rank, V, api.F64) <= eps
    assert hy.status() == 0


FIT_CASES = [
    # (atype, op, M, N, K, eps, tolS)
    (api.F64, "N", 512, 128, 128, 1e-10, 1e-12),
    (api.F64, "T", 3000, 200, 150, 1e-8, 1e-12),
    (api.F32, "N", 4000, 256, 256, 1e-4, 1e-5),
    (api.F64_COMPLEX, "C", 2000, 160, 160, 1e-9, 1e-12),
    (api.F32_COMPLEX, "N", 1500, 96, 64, 1e-3, 1e-5),
]


def _decaying_matrix(rng, m, n, atype, decades):
    r = min(m, n)
    U, _ = np.linalg.qr(rng.standard_normal((m, r)) + (1j * rng.standard_normal((m, r)) if atype & 1 else 0))
    Vm, _ = np.linalg.qr(rng.standard_normal((n, r)) + (1j * rng.standard_normal((n, r)) if atype & 1 else 0))
    s = 10.0 ** (-decades * np.arange(r) / (r - 1))
    A = (U * s) @ Vm.conj().T
    A = A * 10.0 ** rng.uniform(-2, 2, size=n)
    from tests.helpers import NP_DTYPE
    return A.astype(NP_DTYPE[atype])


@pytest.mark.parametrize("atype,op,m,n,k,eps,tol", FIT_CASES)
def test_tsvd_fit_matches_reference_library(hy, ref, atype, op, m, n, k, eps, tol):
    """Same buffers through both libraries: identical rank, singular values within tolerance, error <= eps."""
    rng = np.random.default_rng(77 + m)
    A = _decaying_matrix(rng, m, n, atype, 12.0 if (atype & ~1) == api.F64 else 6.0)
    stored = A if op == "N" else (A.T if op == "T" else A.conj().T)
    stored = np.ascontiguousarray(stored)
    dA = to_device_colmajor(stored)
    lda = stored.shape[0]
    r1, S1, V1 = _tsvd(hy, dA, op, m, n, k, lda, eps, atype)
    r2, S2, V2 = _tsvd(ref, dA, op, m, n, k, lda, eps, atype)
    assert r1 == r2, (r1, r2)
    s1, s2 = S1.cpu().numpy().astype(np.float64), S2.cpu().numpy().astype(np.float64)
    assert np.max(np.abs(s1 - s2)) <= tol * s2[0]
    e1 = _rel_error(hy, dA, op, m, n, lda, r1, V1, atype)
    e2 = _rel_error(ref, dA, op, m, n, lda, r2, V2, atype)
    assert e1 <= max(eps, 1.05 * e2)
    assert hy.status() == 0


def test_check_norm_matches_reference_and_numpy(hy, ref):
    rng = np.random.default_rng(5)
    m, n, r = 2500, 120, 30
    A = random_matrix(rng, m, n, api.F64, col_scale_decades=1.0)
    V = np.linalg.qr(rng.standard_normal((n, r)))[0] @ rng.standard_normal((r, r))      # not orthonormal on purpose
    dA, dV = to_device_colmajor(A), to_device_colmajor(V)
    Q = np.linalg.qr(V)[0]
    want = np.linalg.norm(A - A @ Q @ Q.T) ** 2
    got = hy.check_norm("N", m, n, dA, m, r, dV, n, api.F64)
    got_ref = ref.check_norm("N", m, n, dA, m, r, dV, n, api.F64)
    assert abs(got - want) <= 1e-10 * want and abs(got - got_ref) <= 1e-12 * want
    assert abs(hy.check_norm("N", m, n, dA, m, 0, None, 0, api.F64) - np.linalg.norm(A) ** 2) <= 1e-12 * np.linalg.norm(A) ** 2
    dAt = to_device_colmajor(np.ascontiguousarray(A.T))
    assert abs(hy.check_norm("T", m, n, dAt, n, r, dV, n, api.F64) - want) <= 1e-10 * want


@pytest.mark.parametrize("atype,op,m,n,k,eps", [
    (api.F32, "T", 6000, 512, 96, 1e-5),
    (api.F64, "N", 3000, 300, 300, 1e-9),
    (api.F64_COMPLEX, "N", 1200, 100, 40, 1e-8),
])
def test_interpolate_fit_pivots_identical_to_reference(hy, ref, atype, op, m, n, k, eps):
    """One-based pivots and rank are identical; the interpolation basis reproduces the matrix to eps."""
    torch = _torch()
    rng = np.random.default_rng(31 + n)
    inner = 60 if k < n else n
    A = rng.standard_normal((m, inner)) @ rng.standard_normal((inner, n)) + 1e-7 * rng.standard_normal((m, n))
    if atype & 1:
        A = A + 1j * (rng.standard_normal((m, inner)) @ rng.standard_normal((inner, n)))
    A = A * 10.0 ** rng.uniform(-2, 2, size=n)
    from tests.helpers import NP_DTYPE
    A = A.astype(NP_DTYPE[atype])
    stored = np.ascontiguousarray(A if op == "N" else A.T)
    dA = to_device_colmajor(stored)
    lda = stored.shape[0]
    out = []
    for lib in (hy, ref):
        jp = torch.zeros(n, dtype=torch.int32, device="cuda")
        V = _alloc_v(n, k, atype)
        rank = lib.interpolate_fit(eps, op, m, n, k, dA, lda, jp, V, n, m, atype)
        torch.cuda.synchronize()
        out.append((rank, jp, V))
    assert out[0][0] == out[1][0]
    rank = out[0][0]
    assert torch.equal(out[0][1], out[1][1]), "pivots differ from the reference"
    V1, V2 = out[0][2].cpu().numpy()[:rank], out[1][2].cpu().numpy()[:rank]
    assert np.max(np.abs(V1.astype(np.float64) - V2.astype(np.float64))) <= (1e-4 if (atype & ~1) == api.F32 else 1e-9) * max(1.0, np.abs(V2).max())
    if rank < k or k == n:
        err = _rel_error(hy, dA, op, m, n, lda, rank, out[0][2], atype)
        assert err <= 10 * eps
    assert hy.status() == 0


def test_segmented_fit_matches_reference(hy, ref):
    """hyacinTsvdFitSegmentN on a complex conjugate-transposed input with two column segments."""
    rng = np.random.default_rng(404)
    m, n, k, eps, atype = 4096, 1024, 128, 1e-9, api.F64_COMPLEX
    r = 100
    U = np.linalg.qr(rng.standard_normal((m, r)) + 1j * rng.standard_normal((m, r)))[0]
    W = np.linalg.qr(rng.standard_normal((n, r)) + 1j * rng.standard_normal((n, r)))[0]
    s = 10.0 ** (-13.0 * np.arange(r) / (r - 1))
    A = ((U * s) @ W.conj().T + 1e-15 * rng.standard_normal((m, n))).astype(np.complex128)
    stored = np.ascontiguousarray(A.conj().T)                 # N x M, passed with opA = 'C'
    dA = to_device_colmajor(stored)
    r1, S1, V1 = _tsvd(hy, dA, "C", m, n, k, n, eps, atype, segment_n=True)
    r2, S2, V2 = _tsvd(ref, dA, "C", m, n, k, n, eps, atype, segment_n=True)
    assert r1 == r2
    s1, s2 = S1.cpu().numpy(), S2.cpu().numpy()
    assert np.max(np.abs(s1 - s2)) <= 1e-12 * s2[0]
    assert _rel_error(hy, dA, "C", m, n, n, r1, V1, atype) <= eps
    assert hy.status() == 0


def test_stage_functions_on_a_shared_gram(hy, ref):
    """hyacinXGevd and hyacinXGinterp of both libraries on bit-identical Gram matrices."""
    torch = _torch()
    rng = np.random.default_rng(9)
    m, n, k, eps, atype = 5000, 400, 400, 1e-10, api.F64
    A = _decaying_matrix(rng, m, n, atype, 14.0)
    dA = to_device_colmajor(A)
    res = []
    for lib in (hy, ref):
        u, cp, lp, tri = lib.herk_batch_init(eps, m, n, atype)
        b, s, l = lib.segments(m)
        vexp = torch.zeros((b + 1, n), dtype=torch.int32, device="cuda")
        C = torch.zeros((cp * lp, tri), dtype=torch.int64, device="cuda")
        lib.quantize_scale_batch(b, s, l, n, atype, dA, m, u, vexp)
        lib.herk_batch(b, s, l, n, atype, dA, m, u, vexp, 0, lp, C)
        gtype, gbytes = lib.dequantize_init(n, lp, C, vexp, atype)
        G = torch.zeros((n, n * gbytes), dtype=torch.uint8, device="cuda")
        lib.dequantize(n, lp, C, vexp, gtype, G, n)
        G2 = G.clone()
        S = torch.zeros(k, dtype=torch.float64, device="cuda"); X = torch.zeros((k, n), dtype=torch.float64, device="cuda")
        r_svd = lib.gevd(eps, n, k, atype, X, n, S, gtype, G, n)
        jp = torch.zeros(n, dtype=torch.int32, device="cuda"); Xi = torch.zeros((k, n), dtype=torch.float64, device="cuda")
        r_id = lib.ginterp(eps, n, 64, atype, Xi, n, jp, gtype, G2, n)
        torch.cuda.synchronize()
        res.append((r_svd, S, r_id, jp))
    assert res[0][0] == res[1][0] and res[0][2] == res[1][2] == 64
    assert torch.equal(res[0][3], res[1][3])
    s1, s2 = res[0][1].cpu().numpy(), res[1][1].cpu().numpy()
    assert np.max(np.abs(s1 - s2)) <= 1e-12 * s2[0]


@pytest.mark.parametrize("atype,op,m,n,eps", [(api.F64, "T", 2100, 150, 1e-9), (api.F64_COMPLEX, "C", 1300, 70, 1e-9),
                                               (api.F32, "T", 5000, 300, 1e-4), (api.F16, "T", 700, 40, 1e-2),
                                               (api.F32_COMPLEX, "T", 900, 50, 1e-4)])
def test_transposed_input_gives_bitwise_the_same_fit_as_an_explicit_transpose(hy, atype, op, m, n, eps):
    """op = 'T' / 'C' is quantised straight from the stored layout; the integer Gram, and with it every bit of S
    and V, must equal what the fit produces from an explicitly transposed copy passed with op = 'N'."""
    torch = _torch()
    rng = np.random.default_rng(600 + m)
    base = atype & ~1
    A = _decaying_matrix(rng, m, n, (api.F64 | (atype & 1)), 8.0 if base == api.F64 else 3.0)      # op(A), m x n
    if base == api.F32:
        A = A.astype(np.complex64 if atype & 1 else np.float32)
    stored = A.T if op == "T" else A.conj().T
    d_op = to_device_colmajor(np.ascontiguousarray(stored), stored.shape[0] + 3, atype)
    d_n = to_device_colmajor(np.ascontiguousarray(A), None, atype)
    r1, S1, V1 = _tsvd(hy, d_op, op, m, n, n, stored.shape[0] + 3, eps, atype)
    r2, S2, V2 = _tsvd(hy, d_n, "N", m, n, n, m, eps, atype)
    assert r1 == r2 and r1 > 0
    assert torch.equal(S1, S2) and torch.equal(V1, V2)
    assert hy.status() == 0


def _synthetic_gram(rng, n, gtype, decades):
    """Hermitian positive semi-definite n x n matrix in the storage format of a Gram type (column-major)."""
    torch = _torch()
    cplx = bool(gtype & 1)
    B = rng.standard_normal((n, n)) + (1j * rng.standard_normal((n, n)) if cplx else 0)
    Q = np.linalg.qr(B)[0]
    s = 10.0 ** (-decades * np.arange(n) / max(n - 1, 1))
    G = (Q * s ** 2) @ Q.conj().T
    d = 10.0 ** rng.uniform(-1, 1, n)
    G = G * np.outer(d, d)                                  # congruence keeps it Hermitian and semi-definite
    G = 0.5 * (G + G.conj().T)
    base = gtype & ~1
    if base == api.F32:
        arr = G.astype(np.complex64 if cplx else np.float32)
        t = torch.from_numpy(np.ascontiguousarray(arr.T)).cuda()
    elif base == api.F64:
        arr = G.astype(np.complex128 if cplx else np.float64)
        t = torch.from_numpy(np.ascontiguousarray(arr.T)).cuda()
    else:                                                   # double-double: (hi, lo) pairs, lo = 0
        arr = G.astype(np.complex128 if cplx else np.float64)
        planes = [arr.real, arr.imag] if cplx else [arr]
        dd = np.zeros((n, n, 2 * len(planes)))
        for q, pl in enumerate(planes):
            dd[:, :, 2 * q] = pl.T
        t = torch.from_numpy(dd).cuda()
    return t


@pytest.mark.parametrize("gtype,n,cap", [
    (api.F32, 130, 130),            # 520-byte rows: the factor's pitch is padded to 16 bytes
    (api.F32, 512, 200),
    (api.F64, 40, 40),
    (api.F64, 1001, 600),           # odd n with 8-byte elements: padded pitch
    (api.F64, 1500, 1500),
    (api.F64_COMPLEX, 333, 333),
    (api.F32_COMPLEX, 200, 120),
    (api.DD, 1024, 700),
    (api.DD_COMPLEX, 200, 200),
    (api.DD_COMPLEX, 1024, 300),
    (api.F32, 5000, 64),            # more column runs than SMs: blocks loop over runs
])
def test_pivoted_cholesky_factor_bits_identical_to_reference(hy, ref, gtype, n, cap):
    """The same Gram matrix through both pivoted Choleskys: rank, the whole one-based pivot array and every bit of
    the factor agree (the reference leaves its factor in the upper triangle of the Gram matrix it overwrites);
    hyacinXGinterp on top of it then gives identical coefficients."""
    torch = _torch()
    rng = np.random.default_rng(1000 + n + gtype)
    G = _synthetic_gram(rng, n, gtype, {api.F32: 2.0, api.F64: 6.0, api.DD: 12.0}[gtype & ~1])
    eps = 1e-3 if (gtype & ~1) == api.F32 else 1e-9
    _compare_cholesky(hy, ref, G, gtype, n, cap, eps)


def _compare_cholesky(hy, ref, G, gtype, n, cap, eps):
    torch = _torch()
    xtype = (api.F32 if (gtype & ~1) == api.F32 else api.F64) | (gtype & 1)
    xdt = {api.F32: torch.float32, api.F64: torch.float64}[xtype & ~1]
    words = 2 if gtype & 1 else 1
    gbytes = api.ELEM_BYTES[gtype]
    # reference: hyacinXGinterp overwrites its Gram matrix; rows < rank of the upper triangle are the factor
    Gr = G.clone()
    jp_ref = torch.zeros(n, dtype=torch.int32, device="cuda")
    X_ref = torch.zeros((cap, n * words), dtype=xdt, device="cuda")        # N x cap, column-major
    rank_ref = ref.ginterp(eps, n, cap, xtype, X_ref, n, jp_ref, gtype, Gr, n)
    torch.cuda.synchronize()
    # this build: the factor through the test hook, the coefficients through hyacinXGinterp
    Gm = G.clone()
    jp = torch.zeros(n, dtype=torch.int32, device="cuda")
    R = torch.zeros((n, cap * gbytes), dtype=torch.uint8, device="cuda")   # cap x N, column-major, Gram format
    rank = hy.pivoted_cholesky(eps, n, cap, gtype, Gm, n, jp, R, cap)
    assert torch.equal(Gm.view(torch.uint8), G.view(torch.uint8)), "the Gram matrix must stay untouched"
    jp2 = torch.zeros(n, dtype=torch.int32, device="cuda")
    X = torch.zeros((cap, n * words), dtype=xdt, device="cuda")
    rank2 = hy.ginterp(eps, n, cap, xtype, X, n, jp2, gtype, Gm, n)
    torch.cuda.synchronize()
    assert rank == rank2 == rank_ref > 0, (rank, rank2, rank_ref)
    assert torch.equal(jp, jp_ref) and torch.equal(jp2, jp_ref), "pivots differ from the reference"
    assert sorted(jp.cpu().tolist()) == list(range(1, n + 1))
    mine = R.cpu().numpy().reshape(n, cap, gbytes)[:, :rank]                # [x][k][bytes]
    theirs = Gr.contiguous().view(torch.uint8).cpu().numpy().reshape(n, n, gbytes)[:, :rank]
    upper = np.arange(rank)[None, :] <= np.arange(n)[:, None]             # k <= x
    bad = np.argwhere((mine != theirs).any(axis=2) & upper)
    assert bad.size == 0, f"{len(bad)} factor entries differ from the reference, first at (x, k) = {bad[0].tolist()}"
    assert not mine[~upper].any(), "entries below the diagonal must be zero"
    if rank < n:
        assert torch.equal(X[:rank].view(torch.uint8), X_ref[:rank].view(torch.uint8)), "interpolation coefficients differ"
    assert hy.status() == 0
    return rank


@pytest.mark.parametrize("gtype,n,rho,cap", [(api.F64, 96, 0.5, 96), (api.F64, 300, 0.9, 300), (api.DD, 257, 0.5, 200),
                                              (api.F32, 200, 0.5, 64), (api.F64_COMPLEX, 130, 0.75, 130)])
def test_pivoted_cholesky_ties_are_broken_like_the_reference(hy, ref, gtype, n, rho, cap):
    """G[i, j] = rho^|i - j| has a constant diagonal, and after every step the remaining diagonal is symmetric
    about the pivots chosen so far, so equal maxima occur at nearly every step: the pivot order then depends only
    on which of them the reduction meets first."""
    torch = _torch()
    idx = np.arange(n)
    G = rho ** np.abs(idx[:, None] - idx[None, :]).astype(np.float64)
    base = gtype & ~1
    if gtype & 1:
        G = G * np.exp(0.25j * np.pi * (idx[:, None] - idx[None, :]))      # Hermitian, still Toeplitz
    if base == api.F32:
        t = torch.from_numpy(np.ascontiguousarray(G.astype(np.complex64 if gtype & 1 else np.float32).T)).cuda()
    elif base == api.F64:
        t = torch.from_numpy(np.ascontiguousarray(G.T)).cuda()
    else:
        dd = np.zeros((n, n, 2)); dd[:, :, 0] = G.T
        t = torch.from_numpy(dd).cuda()
    _compare_cholesky(hy, ref, t, gtype, n, cap, 1e-3 if base == api.F32 else 1e-7)


@pytest.mark.parametrize("cplx,n,cap,eps", [(False, 700, 700, 1e-9), (False, 513, 300, 1e-12), (True, 400, 400, 1e-9), (False, 1, 1, 1e-9),
                                            (False, 2, 2, 1e-9), (True, 129, 129, 1e-13)])
def test_pivoted_cholesky_matches_cpu_oracle(hy, cplx, n, cap, eps):
    """FP64 and complex FP64 Gram matrices: rank, pivots and every bit of the factor equal the CPU restatement of the
    reference's kernel (oracle.pivoted_cholesky, itself pinned to factors recorded from the reference library)."""
    torch = _torch()
    from oracle import oracle as O
    rng = np.random.default_rng(4000 + n)
    gtype = api.F64_COMPLEX if cplx else api.F64
    dG = _synthetic_gram(rng, n, gtype, 7.0)
    G = dG.cpu().numpy().T.copy()
    want_rank, want_jp, want_R = O.pivoted_cholesky(G, cap, eps)
    jp = torch.zeros(n, dtype=torch.int32, device="cuda")
    R = torch.zeros((n, cap), dtype=dG.dtype, device="cuda")               # cap x N, column-major
    rank = hy.pivoted_cholesky(eps, n, cap, gtype, dG, n, jp, R, cap)
    torch.cuda.synchronize()
    assert rank == want_rank, (rank, want_rank)
    np.testing.assert_array_equal(jp.cpu().numpy(), want_jp)
    rows = min(rank, cap)
    got = np.ascontiguousarray(R.cpu().numpy().T[:rows])
    np.testing.assert_array_equal(got.view(np.uint8), np.ascontiguousarray(want_R[:rows]).view(np.uint8))
    assert hy.status() == 0


@pytest.mark.parametrize("cplx,n,r", [(False, 300, 7), (True, 200, 3), (False, 1000, 130), (True, 64, 1)])
def test_pivoted_cholesky_of_a_rank_deficient_gram_matches_cpu_oracle(hy, cplx, n, r):
    """G = X X^H with r < n columns in X: after r steps the remaining diagonal is rounding noise of both signs and the
    stop comparison is taken on it.  The kernel and the CPU restatement (which sums the trace in the reference's order)
    must take the same decisions: rank, pivots and every bit of the factor equal."""
    torch = _torch()
    from oracle import oracle as O
    rng = np.random.default_rng(7000 + n)
    X = rng.standard_normal((n, r)) + (1j * rng.standard_normal((n, r)) if cplx else 0)
    G = X @ X.conj().T
    G = 0.5 * (G + G.conj().T)
    gtype = api.F64_COMPLEX if cplx else api.F64
    dG = torch.from_numpy(np.ascontiguousarray(G.T)).cuda()
    for eps in (1e-7, 1e-14):
        want_rank, want_jp, want_R = O.pivoted_cholesky(G, n, eps)
        jp = torch.zeros(n, dtype=torch.int32, device="cuda")
        R = torch.zeros((n, n), dtype=dG.dtype, device="cuda")
        rank = hy.pivoted_cholesky(eps, n, n, gtype, dG, n, jp, R, n)
        torch.cuda.synchronize()
        assert rank == want_rank, (eps, rank, want_rank)
        np.testing.assert_array_equal(jp.cpu().numpy(), want_jp)
        rows = min(rank, n)
        got = np.ascontiguousarray(R.cpu().numpy().T[:rows])
        np.testing.assert_array_equal(got.view(np.uint8), np.ascontiguousarray(want_R[:rows]).view(np.uint8))
    assert hy.status() == 0


def test_exactly_rank_deficient_inputs_give_the_reference_bits(hy, ref):
    """Inputs of exact rank one to three: once the rank is used up the remaining diagonal of the Gram matrix is rounding
    noise, and whether the Cholesky takes one more (noise) row depends on the last bits of the remaining trace, i.e. on
    the order in which the reference sums it.  Rank, S and every bit of V must still agree."""
    torch = _torch()
    gen = torch.Generator(device="cuda"); gen.manual_seed(2024)
    rng = np.random.default_rng(2024)
    checked = 0
    for case in range(240):
        cplx = case % 3 != 0
        m, n, r = int(rng.integers(50, 3000)), int(rng.integers(2, 120)), int(rng.integers(1, 4))
        dt = torch.complex128 if cplx else torch.float64
        A = torch.randn((m, r), generator=gen, device="cuda", dtype=dt) @ torch.randn((r, n), generator=gen, device="cuda", dtype=dt)
        dA = A.transpose(0, 1).contiguous()
        atype = api.F64_COMPLEX if cplx else api.F64
        eps = float(10.0 ** rng.uniform(-11, -6))
        a = _tsvd(hy, dA, "N", m, n, n, m, eps, atype)
        b = _tsvd(ref, dA, "N", m, n, n, m, eps, atype)
        assert a[0] == b[0] > 0, (case, a[0], b[0])
        rank = a[0]
        assert torch.equal(a[1][:rank], b[1][:rank]), f"case {case}: singular values differ"
        assert torch.equal(a[2][:rank].view(torch.uint8), b[2][:rank].view(torch.uint8)), f"case {case}: basis differs (m={m}, n={n}, rank {r}, complex={cplx})"
        checked += 1
    assert checked == 240 and hy.status() == 0


def test_pivoted_cholesky_counts_a_last_single_column(hy, ref):
    """With K = N the loop stops when one column is left and counts it (src/hyacin_potrfp.cu:264,269 of the
    reference): a full-rank matrix gives rank N and a complete factor."""
    rng = np.random.default_rng(3)
    n = 70
    G = _synthetic_gram(rng, n, api.F64, 2.0)
    assert _compare_cholesky(hy, ref, G, api.F64, n, n, 1e-12) == n


@pytest.mark.parametrize("atype,op", [(api.F32, "T"), (api.F32_COMPLEX, "C")])
def test_segmented_fit_in_single_precision_with_odd_leading_dimension(hy, atype, op):
    """The stage products of single-precision input ask cuBLAS for its emulated FP32 mode, as the reference does
    (src/lra.cpp:92,104).  The library refuses that mode for some leading dimensions and column offsets; the
    reference then carries on with an unwritten product, this build repeats the product in plain FP32.  Checked
    against the matrix itself: the basis reproduces it to the tolerance."""
    torch = _torch()
    rng = np.random.default_rng(537)
    m, n, k, eps = 4000, 537, 74, 3e-5
    r = 40
    A = (rng.standard_normal((m, r)) * 10.0 ** (-6.0 * np.arange(r) / r)) @ rng.standard_normal((r, n)) / np.sqrt(m)
    if atype & 1:
        A = A + 1j * ((rng.standard_normal((m, r)) * 10.0 ** (-6.0 * np.arange(r) / r)) @ rng.standard_normal((r, n)) / np.sqrt(m))
    from tests.helpers import NP_DTYPE
    A = A.astype(NP_DTYPE[atype])
    stored = np.ascontiguousarray(A.conj().T if op == "C" else A.T)           # stored N x M, lda = n
    dA = to_device_colmajor(stored)
    rank, S, V = _tsvd(hy, dA, op, m, n, k, n, eps, atype, segment_n=True)
    assert 0 < rank <= k
    s_true = np.linalg.svd(A.astype(np.complex128 if atype & 1 else np.float64), compute_uv=False)
    assert np.max(np.abs(S.cpu().numpy()[:rank].astype(np.float64) - s_true[:rank])) <= 2e-4 * s_true[0]
    assert _rel_error(hy, dA, op, m, n, n, rank, V, atype) <= 20 * eps
    assert hy.status() == 0


@pytest.mark.parametrize("op", ["N", "C"])
def test_segmented_fit_on_complex_half_input(hy, ref, op):
    """hyacinTsvdFitSegmentN with complex-half storage: the stage products go through planar real half GEMMs."""
    rng = np.random.default_rng(77)
    m, n, k, eps, atype = 3000, 1024, 128, 2e-2, api.F16_COMPLEX
    r = 40
    U = np.linalg.qr(rng.standard_normal((m, r)) + 1j * rng.standard_normal((m, r)))[0]
    W = np.linalg.qr(rng.standard_normal((n, r)) + 1j * rng.standard_normal((n, r)))[0]
    s = 30.0 * 10.0 ** (-3.0 * np.arange(r) / (r - 1))
    A = (U * s) @ W.conj().T
    stored = A if op == "N" else np.ascontiguousarray(A.conj().T)
    dA = to_device_colmajor(stored, atype=atype)
    lda = stored.shape[0]
    r1, S1, V1 = _tsvd(hy, dA, op, m, n, k, lda, eps, atype, segment_n=True)
    r2, S2, V2 = _tsvd(ref, dA, op, m, n, k, lda, eps, atype, segment_n=True)
    # the stage products ask cuBLAS for the same half-precision GEMMs on the same operand layouts as the reference
    # (src/matmul_fp16_complex.cu), so rank, S and V agree to the bit
    torch = _torch()
    assert r1 == r2 > 0
    assert torch.equal(S1[:r1].view(torch.uint8), S2[:r2].view(torch.uint8))
    assert torch.equal(V1[:r1].view(torch.uint8), V2[:r2].view(torch.uint8))
    assert _rel_error(hy, dA, op, m, n, lda, r1, V1, atype) <= 3 * eps
    assert hy.status() == 0
