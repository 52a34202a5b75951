"""Shared helpers of the test-suite: seeded inputs and column-major device buffers."""
from __future__ import annotations

import numpy as np

from hyacinth_b200 import api

NP_DTYPE = {api.F64: np.float64, api.F64_COMPLEX: np.complex128, api.F32: np.float32, api.F32_COMPLEX: np.complex64,
            api.F16: np.float16}


def random_matrix(rng, m, n, atype, col_scale_decades=3.0, zero_cols=(), spread_rows=0.0):
    """Dense Gaussian matrix with log-uniform column scales (and optionally decaying row-block magnitude)."""
    A = rng.standard_normal((m, n))
    if atype & 1:
        A = A + 1j * rng.standard_normal((m, n))
    A = A * 10.0 ** rng.uniform(-col_scale_decades, col_scale_decades, size=n)
    if spread_rows:
        A = A * (10.0 ** (-float(spread_rows) * np.arange(m) / max(m - 1, 1)))[:, None]
    for j in zero_cols:
        A[:, j] = 0
    base = atype & ~1
    if base == api.F16:
        A = np.clip(A.real, -6e4, 6e4) + (1j * np.clip(A.imag, -6e4, 6e4) if atype & 1 else 0)
        if not atype & 1:
            A = A.real
        return A   # caller converts (complex half has no numpy dtype)
    return A.astype(NP_DTYPE[atype])


def low_rank_matrix(rng, m, n, rank, sigma, noise, atype=api.F64):
    """U diag(sigma) V^T with orthonormal Gaussian factors plus Gaussian noise (BASELINE configuration 1 shape)."""
    U, _ = np.linalg.qr(rng.standard_normal((m, rank)))
    V, _ = np.linalg.qr(rng.standard_normal((n, rank)))
    A = (U * sigma) @ V.T + noise * rng.standard_normal((m, n))
    return A.astype(NP_DTYPE[atype])


def to_device_colmajor(A, lda=None, atype=None):
    """Column-major device copy of a host matrix: torch tensor of shape (N, lda) whose row j is column j."""
    import torch
    m, n = A.shape
    lda = lda or m
    if atype is not None and (atype & ~1) == api.F16:
        if atype & 1:
            host = np.zeros((n, lda, 2), dtype=np.float16)
            host[:, :m, 0] = A.real.T; host[:, :m, 1] = A.imag.T
        else:
            host = np.zeros((n, lda), dtype=np.float16); host[:, :m] = A.T
        return torch.from_numpy(host).cuda()
    host = np.zeros((n, lda), dtype=A.dtype)
    host[:, :m] = A.T
    return torch.from_numpy(host).cuda()


def half_roundtrip(A, atype):
    """The values a half-precision device buffer really holds, as float32/complex64 for the oracle."""
    if atype & 1:
        return (A.real.astype(np.float16).astype(np.float32) + 1j * A.imag.astype(np.float16).astype(np.float32)).astype(np.complex64)
    return A.astype(np.float16).astype(np.float32)


# ---- Gram matrices for the pivoted-Cholesky fixtures ----------------------------------------------------------------
# Every entry is an exact sum of dyadic numbers well inside 53 bits, so the matrix has the same bits whatever BLAS or
# summation order builds it; the fixtures therefore store only the case name, not the matrix.
CHOLESKY_CASES = {
    # name: (kind, complex, n, cap, eps)
    "chol_f64_toeplitz": ("toeplitz", False, 96, 96, 1e-7),          # constant diagonal: ties at nearly every step
    "chol_f64c_toeplitz": ("toeplitz", True, 130, 130, 1e-7),
    "chol_f64_product_420": ("product", False, 420, 420, 1e-5),      # 280 steps: chains of up to three terms
    "chol_f64_product_cap": ("product", False, 200, 50, 1e-9),       # stopped by the column cap
    "chol_f64c_product_240": ("product", True, 240, 240, 1e-5),     # 160 steps
    "chol_f64_last_column": ("product_full", False, 40, 40, 1e-14),  # full rank with K = N: the last column is counted
    # rank 3 / rank 2 with a tolerance below the rounding noise: the stop comparison is taken on the noise that is left
    "chol_f64_rank3_noise": ("lowrank3", False, 90, 90, 1e-14),
    "chol_f64c_rank2_noise": ("lowrank2", True, 70, 70, 1e-14),
    "chol_f64_rank3_noise_wide": ("lowrank3", False, 300, 300, 1e-15),
}


def cholesky_case(name):
    """(G, cap, eps) of a fixture case; G is n x n, float64 or complex128, Hermitian positive semi-definite."""
    kind, cplx, n, cap, eps = CHOLESKY_CASES[name]
    idx = np.arange(n)
    if kind == "toeplitz":
        G = 0.5 ** np.abs(idx[:, None] - idx[None, :]).astype(np.float64)
        if cplx:                                                      # phase i^(row - column): exact, Hermitian
            G = G * np.array([1, 1j, -1, -1j])[(idx[:, None] - idx[None, :]) % 4]
        return G, cap, eps
    rng = np.random.default_rng(sum(map(ord, name)))
    rows = n if kind == "product_full" else 3 if kind == "lowrank3" else 2 if kind == "lowrank2" else (2 * n) // 3
    B = rng.integers(-15, 16, size=(rows, n)).astype(np.float64)
    if cplx:
        B = B + 1j * rng.integers(-15, 16, size=(rows, n))
    shift = np.zeros(rows) if kind in ("product_full", "lowrank3", "lowrank2") else np.floor(14.0 * np.arange(rows) / rows)
    B = B * (2.0 ** -shift)[:, None]                                  # row weights 1 ... 2^-13: G spans 2^-26, exact
    return B.conj().T @ B, cap, eps


def factor_digest(R):
    """SHA-256 over the bytes of the factor's upper trapezoid, position by position: R[0..min(x, rank - 1), x]."""
    import hashlib
    h = hashlib.sha256()
    rank, n = R.shape
    for x in range(n):
        h.update(np.ascontiguousarray(R[:min(x + 1, rank), x]).tobytes())
    return h.hexdigest()
