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
