"""Seeded synthetic inputs with the shapes, spectra and scalings of the benchmark configurations.

The reference publishes no dataset; its README and the benchmark configurations describe the matrices by
construction.  Everything is generated on the current CUDA device from fixed seeds, in row blocks, so that a
32 GiB matrix never needs a second copy.  Used by ``bench.py`` and by the full-size parity tests.

A column-major ``rows x cols`` matrix with leading dimension ``ld`` is a torch tensor of shape ``(cols, ld)``.
"""
from __future__ import annotations

SEED = 20240611


def real_decaying(torch, rows, n, seed, total_rows=None):
    """Configurations 2 / 3: real FP64, op 'N'.  A = (Gaussian / sqrt(M)) diag(10^(-14 i / (n - 1))) V^T with
    orthonormal V and log-uniform column scales in [1e-3, 1e3].  V, the spectrum and the scales depend on n only;
    the Gaussian row factor on `seed` (one per rank).  Returns the tensor (n, rows)."""
    g = torch.Generator(device="cuda")
    g.manual_seed(SEED + 2)
    V, _ = torch.linalg.qr(torch.randn(n, n, dtype=torch.float64, device="cuda", generator=g))
    s = 10.0 ** (-14.0 * torch.arange(n, dtype=torch.float64, device="cuda") / max(n - 1, 1))
    scale = 10.0 ** (torch.rand(n, dtype=torch.float64, device="cuda", generator=g) * 6.0 - 3.0)
    B = (s[:, None] * V.T) * scale[None, :]
    g.manual_seed(seed)
    At = torch.empty((n, rows), dtype=torch.float64, device="cuda")
    norm = float(total_rows or rows) ** 0.5
    blk = 1 << 16
    for r0 in range(0, rows, blk):
        r = min(blk, rows - r0)
        Gs = torch.randn(r, n, dtype=torch.float64, device="cuda", generator=g) / norm
        At[:, r0:r0 + r] = (Gs @ B).T
    del V, B
    return At


def complex_low_rank(torch, rows, n, seed, stored_conj_transposed=False):
    """Configuration 4: complex FP64, rank 200, singular values 1 .. 1e-13 (geometric), noise 1e-15.
    Returns op(A) = rows x n as the tensor (n, rows) -- or, with stored_conj_transposed, the matrix as the fits take
    it with opA = 'C': stored n x rows column-major, i.e. the tensor (rows, n) holding conj(A)."""
    g = torch.Generator(device="cuda")
    g.manual_seed(SEED + 4)
    r = min(200, n)
    W, _ = torch.linalg.qr(torch.randn(n, r, dtype=torch.complex128, device="cuda", generator=g))
    s = 10.0 ** (-13.0 * torch.arange(r, dtype=torch.float64, device="cuda") / max(r - 1, 1))
    g.manual_seed(seed)
    out = torch.empty((rows, n) if stored_conj_transposed else (n, rows), dtype=torch.complex128, device="cuda")
    blk = 1 << 15
    for r0 in range(0, rows, blk):
        k = min(blk, rows - r0)
        U = torch.randn(k, r, dtype=torch.complex128, device="cuda", generator=g) / (rows ** 0.5)
        block = (U * s) @ W.conj().T + 1e-15 * torch.randn(k, n, dtype=torch.complex128, device="cuda", generator=g)
        if stored_conj_transposed:
            out[r0:r0 + k] = block.conj()
        else:
            out[:, r0:r0 + k] = block.T
    return out


def float_product_transposed(torch, rows, n, seed, inner=600):
    """Configuration 5 (one rank's share): real FP32 with opA = 'T'.  op(A) = Gaussian(rows x inner) Gaussian(inner x n)
    + 1e-7 noise, columns scaled log-uniformly in [1e-2, 1e2]; returned as stored, n x rows column-major = tensor
    (rows, n)."""
    g = torch.Generator(device="cuda")
    g.manual_seed(SEED + 5)
    Rm = torch.randn(inner, n, dtype=torch.float32, device="cuda", generator=g)
    scale = 10.0 ** (torch.rand(n, dtype=torch.float32, device="cuda", generator=g) * 4.0 - 2.0)
    g.manual_seed(seed)
    out = torch.empty((rows, n), dtype=torch.float32, device="cuda")
    blk = 1 << 14
    for r0 in range(0, rows, blk):
        k = min(blk, rows - r0)
        L = torch.randn(k, inner, dtype=torch.float32, device="cuda", generator=g)
        out[r0:r0 + k] = (L @ Rm + 1e-7 * torch.randn(k, n, dtype=torch.float32, device="cuda", generator=g)) * scale[None, :]
    return out
