"""Record golden vectors from the REFERENCE's own CUDA library (oracle/_ref/libhyacin_ref.so).

Run on a machine with a B200 and the reference library built:
    python tests/golden/make_golden.py <output directory>
and copy the .npz files it writes next to this script.  Every fixture stores the seeded input matrix and the
reference's stage outputs for it (column exponents, packed integer Gram, Gram format, raw Gram bytes) plus the
results of its fits (rank, singular values, one-based pivots).  The CPU tests check the oracle against them.

The cholesky_*.npz fixtures hold the reference's pivoted Cholesky of the Gram matrices of tests/helpers.py
(CHOLESKY_CASES, rebuilt exactly from the case name): rank, one-based pivots, the diagonal of the factor and the
SHA-256 of the factor's upper trapezoid (position-major, rows <= position), plus the whole factor for n <= 100.
"""

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

CASES = [
    # name, atype, M, N, eps, GramSegmentK, algorithm
    ("f64_real_crt", 0, 96, 24, 1e-10, 40, b"C"),
    ("f64_real_limbs", 0, 200, 17, 1e-10, 8192, b"L"),
    ("f64_complex_crt", 1, 80, 12, 1e-12, 8192, b"A"),
    ("f32_real", 2, 300, 20, 1e-5, 128, b"A"),
    ("f32_complex", 3, 64, 9, 1e-4, 8192, b"A"),
    ("f16_real", 4, 128, 16, 1e-2, 8192, b"A"),
]


def main(out_dir):
    import torch
    from hyacinth_b200 import api
    from tests.helpers import NP_DTYPE, half_roundtrip, to_device_colmajor
    os.makedirs(out_dir, exist_ok=True)
    ref = api.Hyacin(lib_path=os.path.join(ROOT, "oracle", "_ref", "libhyacin_ref.so"), stream=0)
    for name, atype, m, n, eps, seg_k, alg in CASES:
        rng = np.random.default_rng(abs(hash(name)) % (2**31) if False else sum(map(ord, name)))
        r = max(3, n // 3)
        A = rng.standard_normal((m, r)) @ (rng.standard_normal((r, n)) * (10.0 ** (-8.0 * np.arange(r) / r))[:, None])
        if atype & 1:
            A = A + 1j * (rng.standard_normal((m, r)) @ rng.standard_normal((r, n)) * 1e-2)
        A = A * 10.0 ** rng.uniform(-2, 2, size=n)
        A[:, 1] = 0
        if (atype & ~1) == api.F16:
            A = half_roundtrip(np.clip(A.real, -6e4, 6e4) + (1j * np.clip(A.imag, -6e4, 6e4) if atype & 1 else 0), atype)
            if not atype & 1:
                A = A.real.astype(np.float32)
        else:
            A = A.astype(NP_DTYPE[atype])
        dA = to_device_colmajor(A, None, atype)
        ref.h.GramSegmentK = seg_k
        ref.h.GramMatrixAlgorithm = alg
        u, cp, lp, tri = ref.herk_batch_init(eps, m, n, atype)
        b, s, l = ref.segments(m)
        vexp = torch.zeros((b + 1, n), dtype=torch.int32, device="cuda")
        C = torch.zeros((cp * lp, tri), dtype=torch.int64, device="cuda")
        ref.quantize_scale_batch(b, s, l, n, atype, dA, m, u, vexp)
        ref.herk_batch(b, s, l, n, atype, dA, m, u, vexp, 0, lp, C)
        gtype, gbytes = ref.dequantize_init(n, lp, C, vexp, atype)
        G = torch.zeros((n, n * gbytes), dtype=torch.uint8, device="cuda")
        ref.dequantize(n, lp, C, vexp, gtype, G, n)
        torch.cuda.synchronize()
        words = 2 if atype & 1 else 1
        rdt = {0: torch.float64, 2: torch.float32, 4: torch.float16}[atype & ~1]
        S = torch.zeros(n, dtype=rdt, device="cuda"); V = torch.zeros((n, n * words), dtype=rdt, device="cuda")
        rank = ref.tsvd_fit(eps, "N", m, n, n, dA, m, S, V, n, m, atype)
        jp = torch.zeros(n, dtype=torch.int32, device="cuda"); Vi = torch.zeros((n, n * words), dtype=rdt, device="cuda")
        irank = ref.interpolate_fit(eps, "N", m, n, max(1, n // 2), dA, m, jp, Vi, n, m, atype)
        torch.cuda.synchronize()
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), A=A, atype=atype, eps=eps, seg_k=seg_k, u=u, cpanels=cp, lpanels=lp,
                            segments=np.array([b, s, l]), vexp=vexp.cpu().numpy(), C=C.cpu().numpy().view(np.uint64), gtype=gtype,
                            gbytes=gbytes, G=G.cpu().numpy(), svd_rank=rank, S=S.float().cpu().numpy() if rdt == torch.float16 else S.cpu().numpy(),
                            interp_rank=irank, jpiv=jp.cpu().numpy())
        print(name, "u", u, "lp", lp, "gtype", gtype, "rank", rank, "irank", irank)
    ref.h.GramSegmentK = 8192
    ref.h.GramMatrixAlgorithm = b"A"
    from tests.helpers import CHOLESKY_CASES, cholesky_case, factor_digest
    for name in CHOLESKY_CASES:
        G, cap, eps = cholesky_case(name)
        n = G.shape[0]
        cplx = np.iscomplexobj(G)
        gtype = api.F64_COMPLEX if cplx else api.F64
        dG = torch.from_numpy(np.ascontiguousarray(G.T)).cuda()             # column-major
        jp = torch.zeros(n, dtype=torch.int32, device="cuda")
        X = torch.zeros((cap, n), dtype=dG.dtype, device="cuda")
        rank = ref.ginterp(eps, n, cap, gtype, X, n, jp, gtype, dG, n)      # overwrites dG: rows < rank of the upper triangle
        torch.cuda.synchronize()
        R = dG.cpu().numpy()[:, :rank].T.copy()                              # R[k, x]
        R[np.arange(rank)[:, None] > np.arange(n)[None, :]] = 0
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), rank=rank, jpiv=jp.cpu().numpy(), diag=np.diagonal(R).real.copy(),
                            digest=factor_digest(R), R=R if n <= 100 else np.zeros((0, 0)))
        print(name, "n", n, "cap", cap, "rank", rank)
    ref.destroy()


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__)))
