"""GPU parity tests of the quantized-Gram path, through the C ABI.

Every check is bit-exact: column exponents (int32), residue planes (modulo m), residue Grams (bytes), the
packed integer Gram (uint64 limbs) and the dequantised matrix (raw float bits).  The checker is the CPU oracle
(``oracle/``) at sizes it finishes in seconds, and the reference's own CUDA library (``oracle/_ref``, when it
was built) at larger sizes.
"""
import numpy as np
import pytest

from hyacinth_b200 import api
from oracle import oracle as O
from tests.helpers import half_roundtrip, random_matrix, to_device_colmajor

pytestmark = pytest.mark.gpu

CRT_MODULI = [256, 255, 253, 251, 247, 241, 239, 233, 229, 227, 223, 217, 211, 199, 197, 193, 191, 181, 179, 173,
              167, 163, 157, 151]


def _torch():
    import torch
    return torch


def _eps_for(atype):
    return {api.F64: 1e-10, api.F32: 1e-5, api.F16: 1e-2}[atype & ~1]


def _oracle_input(A, atype):
    return half_roundtrip(A, atype) if (atype & ~1) == api.F16 else A


def _run_exponents(h, dA, m, n, lda, atype, u, seg_k=None):
    torch = _torch()
    if seg_k is not None:
        h.h.GramSegmentK = seg_k
    b, s, l = h.segments(m)
    vexp = torch.full(((b + 1), n), 12345, dtype=torch.int32, device="cuda")
    h.quantize_scale_batch(b, s, l, n, atype, dA, lda, u, vexp)
    torch.cuda.synchronize()
    return (b, s, l), vexp


def _run_herk(h, dA, m, n, lda, atype, u, order, cpanels, segs, vexp, beta=0, C=None):
    torch = _torch()
    tri = n * (n + 1) // 2
    if C is None:
        C = torch.full((cpanels * order, tri), 0x5555555555555555, dtype=torch.int64, device="cuda")
    h.herk_batch(segs[0], segs[1], segs[2], n, atype, dA, lda, u, vexp, beta, order, C)
    torch.cuda.synchronize()
    assert h.status() == 0, "a bounded wait inside the Gram kernel expired"
    return C


CASES = [
    # (atype, M, N, lda_pad, seg_k, zero_cols)
    (api.F64, 512, 128, 0, 8192, ()),
    (api.F64, 1000, 300, 7, 256, (3, 299)),
    (api.F64, 100, 1, 0, 8192, ()),
    (api.F64, 257, 129, 1, 100, ()),
    (api.F32, 700, 260, 3, 8192, (0,)),
    (api.F16, 384, 96, 2, 128, ()),
    (api.F64_COMPLEX, 300, 140, 1, 8192, (5,)),
    (api.F32_COMPLEX, 260, 70, 0, 64, ()),
    (api.F16_COMPLEX, 200, 33, 1, 8192, ()),
]


@pytest.mark.parametrize("atype,m,n,pad,seg_k,zero_cols", CASES)
def test_exponents_and_integer_gram_match_oracle(hy, atype, m, n, pad, seg_k, zero_cols):
    """vexp table and packed integer Gram equal the CPU oracle bit for bit (ragged sizes, zero columns, lda > M)."""
    rng = np.random.default_rng(1000 + m + n + atype)
    A = random_matrix(rng, m, n, atype, zero_cols=zero_cols)
    lda = m + pad
    dA = to_device_colmajor(A, lda, atype)
    u, cp, lp, tri = hy.herk_batch_init(_eps_for(atype), m, n, atype)
    assert (u, cp, lp, tri) == O.herk_init(_eps_for(atype), m, n, atype)
    segs, vexp = _run_exponents(hy, dA, m, n, lda, atype, u, seg_k)
    Ao = _oracle_input(A, atype)
    want_vexp = O.column_exponents(Ao, atype, u, *segs)
    np.testing.assert_array_equal(vexp.cpu().numpy(), want_vexp)
    C = _run_herk(hy, dA, m, n, lda, atype, u, lp, cp, segs, vexp)
    want_C = O.gram_exact(Ao, atype, want_vexp[0], lp)
    np.testing.assert_array_equal(C.cpu().numpy().view(np.uint64), want_C)
    hy.h.GramSegmentK = 8192


def test_row_groups_reconstructed_separately_add_up_exactly(hy, ref):
    """FP32 input at eps 1e-5 over more than 2^17 rows needs 65 bits in one piece (9 moduli) but 63 bits per 65536-row
    group (8 moduli): the schedule then reconstructs every group on its own and adds them.  The packed integer Gram
    equals the CPU oracle and the reference library (which flushes every 65536 rows here) bit for bit."""
    torch = _torch()
    rng = np.random.default_rng(99)
    m, n, atype, eps = (1 << 17) + 300, 24, api.F32, 1e-5
    A = random_matrix(rng, m, n, atype)
    dA = to_device_colmajor(A, None, atype)
    u, cp, lp, tri = hy.herk_batch_init(eps, m, n, atype)
    plan = hy.crt_plan(u, 0, m)
    assert plan["group_rows"] == 65536 and plan["moduli"] == 8, plan
    segs, vexp = _run_exponents(hy, dA, m, n, m, atype, u)
    C = _run_herk(hy, dA, m, n, m, atype, u, lp, cp, segs, vexp)
    want_vexp = O.column_exponents(A, atype, u, *segs)
    np.testing.assert_array_equal(vexp.cpu().numpy(), want_vexp)
    np.testing.assert_array_equal(C.cpu().numpy().view(np.uint64), O.gram_exact(A, atype, want_vexp[0], lp))
    C_ref = torch.zeros_like(C)
    ref.herk_batch(segs[0], segs[1], segs[2], n, atype, dA, m, u, vexp, 0, lp, C_ref)
    torch.cuda.synchronize()
    assert torch.equal(C, C_ref)


@pytest.mark.parametrize("rows,eps,seg_k", [(151845, 1.38e-12, 8192), (133022, 2.7e-6, 1024), (140000, 1e-10, 65536)])
def test_more_than_130816_rows_match_the_oracle(hy, rows, eps, seg_k):
    """Row counts beyond one K chunk of the reference (130816 rows, src/hyacin_herk.cpp:117-137).  The checker here is the
    CPU oracle alone: in the first two cases the reference library itself returns a different integer Gram (its flush
    length exceeds that chunk for these bit budgets), in the third it agrees; a randomized side-by-side sweep found no
    other disagreement between the libraries."""
    rng = np.random.default_rng(rows)
    n, atype = 12, api.F64
    A = rng.standard_normal((rows, n)) * 10.0 ** rng.uniform(-2, 2, n)
    dA = to_device_colmajor(A)
    u, cp, lp, tri = hy.herk_batch_init(eps, rows, n, atype)
    segs, vexp = _run_exponents(hy, dA, rows, n, rows, atype, u, seg_k)
    want_vexp = O.column_exponents(A, atype, u, *segs)
    np.testing.assert_array_equal(vexp.cpu().numpy(), want_vexp)
    C = _run_herk(hy, dA, rows, n, rows, atype, u, lp, cp, segs, vexp)
    np.testing.assert_array_equal(C.cpu().numpy().view(np.uint64), O.gram_exact(A, atype, want_vexp[0], lp))
    hy.h.GramSegmentK = 8192


def test_beta_accumulates_and_row_blocks_add_up(hy):
    """C(beta=1) over two row blocks equals C over the stacked matrix (the hook used to stream a tall matrix)."""
    torch = _torch()
    rng = np.random.default_rng(7)
    m, n, atype = 900, 200, api.F64
    A = random_matrix(rng, m, n, atype)
    u, cp, lp, tri = hy.herk_batch_init(1e-10, m, n, atype)
    dA = to_device_colmajor(A)
    segs, vexp = _run_exponents(hy, dA, m, n, m, atype, u)
    C_all = _run_herk(hy, dA, m, n, m, atype, u, lp, cp, segs, vexp)
    m1 = 388
    d1, d2 = to_device_colmajor(A[:m1]), to_device_colmajor(A[m1:])
    C = _run_herk(hy, d1, m1, n, m1, atype, u, lp, cp, (1, m1, m1), vexp)
    C = _run_herk(hy, d2, m - m1, n, m - m1, atype, u, lp, cp, (1, m - m1, m - m1), vexp, beta=1, C=C)
    assert torch.equal(C, C_all)


def test_empty_and_negative_budget_define_zero_gram(hy):
    """No rows, or u < 0: beta = 0 zeroes C and beta = 1 leaves it alone (src/hyacin_herk.cpp:287)."""
    torch = _torch()
    n, order = 40, 2
    tri = n * (n + 1) // 2
    vexp = torch.zeros((2, n), dtype=torch.int32, device="cuda")
    dA = torch.ones((n, 64), dtype=torch.float64, device="cuda")
    C = torch.full((order, tri), 77, dtype=torch.int64, device="cuda")
    hy.herk_batch(1, 0, 0, n, api.F64, dA, 64, 40, vexp, 1, order, C)
    torch.cuda.synchronize()
    assert int((C != 77).sum()) == 0
    hy.herk_batch(1, 64, 64, n, api.F64, dA, 64, -1, vexp, 0, order, C)
    torch.cuda.synchronize()
    assert int(C.abs().sum()) == 0
    # quantize-scale with u < 0 marks every column as zero and touches only the global row
    v2 = torch.full((2, n), 5, dtype=torch.int32, device="cuda")
    hy.quantize_scale_batch(1, 64, 64, n, api.F64, dA, 64, -1, v2)
    torch.cuda.synchronize()
    assert int((v2[0] != 2**31 - 1).sum()) == 0 and int((v2[1] != 5).sum()) == 0


@pytest.mark.parametrize("atype,u", [(api.F64, 40), (api.F64, 59), (api.F64, 70), (api.F32, 23), (api.F64_COMPLEX, 47), (api.F16, 12)])
def test_quantize_stage_residues(hy, atype, u):
    """Residue planes are congruent to rint(a 2^vexp) modulo every modulus, and the padding rows are zero."""
    torch = _torch()
    rng = np.random.default_rng(50 + u)
    m, n = 203, 17
    A = random_matrix(rng, m, n, atype, zero_cols=(2,))
    dA = to_device_colmajor(A, None, atype)
    segs, vexp = _run_exponents(hy, dA, m, n, m, atype, u)
    plan = hy.crt_plan(u, atype & 1, m)
    k, nb = plan["moduli"], plan["value_bytes"]
    parts = 3 if atype & 1 else 1
    ldk = 256
    W = torch.full((k, n, parts * ldk), 99, dtype=torch.int8, device="cuda")
    hy.quantize_crt(atype, m, n, dA, m, vexp, k, nb, W, ldk)
    torch.cuda.synchronize()
    Wh = W.cpu().numpy().astype(np.int64)
    q = O.quantize_ints(_oracle_input(A, atype), atype, vexp[0].cpu().numpy())
    for p in range(parts):
        src = q[0] if p == 0 else q[1] if p == 1 else [[-v for v in col] for col in q[0]]
        for i in range(k):
            want = np.array([[v % CRT_MODULI[i] for v in col] for col in src], dtype=np.int64)
            got = Wh[i, :, p * ldk:p * ldk + m]
            assert np.all((got - want) % CRT_MODULI[i] == 0)
            assert got.min() >= -128 and got.max() <= 127
            assert np.all(Wh[i, :, p * ldk + m:(p + 1) * ldk] == 0)


@pytest.mark.parametrize("n,k_rows,moduli", [(128, 128, 1), (300, 512, 3), (700, 1024, 13), (1030, 256, 24)])
def test_gram_residue_kernel_against_integer_matmul(hy, n, k_rows, moduli):
    """tcgen05 residue Gram == plain integer matmul modulo m, for every tile, with and without accumulation."""
    torch = _torch()
    rng = np.random.default_rng(n + k_rows)
    W = torch.from_numpy(rng.integers(-128, 128, size=(moduli, n, k_rows), dtype=np.int8)).cuda()
    info = hy.tile_info(n)
    ty, tx, nt = info["tile_y"], info["tile_x"], info["num_tiles"]
    R = torch.full((moduli, nt, ty, tx), 0xEE, dtype=torch.uint8, device="cuda")
    hy.gram_residues(n, moduli, W, k_rows, k_rows * n, 0, 0, k_rows, 0, R)
    hy.gram_residues(n, moduli, W, k_rows, k_rows * n, 0, 0, k_rows, 1, R)     # accumulate the same chunk again
    torch.cuda.synchronize()
    assert hy.status() == 0
    Rh = R.cpu().numpy().astype(np.int64)
    Wd = W.to(torch.float64)
    tiles_y = info["tiles_y"]
    t = 0
    for bx in range((n + tx - 1) // tx):
        for by in range(min(tiles_y, 2 * bx + 2)):
            ys, xs = slice(by * ty, min(n, (by + 1) * ty)), slice(bx * tx, min(n, (bx + 1) * tx))
            for i in range(moduli):
                G = (Wd[i, ys] @ Wd[i, xs].T).cpu().numpy().astype(np.int64)     # exact: |sum| < 2^53
                want = (2 * G) % CRT_MODULI[i]
                got = Rh[i, t, :G.shape[0], :G.shape[1]]
                np.testing.assert_array_equal(got, want)
            t += 1
    assert t == nt


@pytest.mark.parametrize("atype", [api.F64, api.F64_COMPLEX, api.F32])
def test_dequantize_matches_oracle_bits(hy, atype):
    """Gram format choice and every bit of the dequantised matrix equal the oracle's (same operation order)."""
    torch = _torch()
    rng = np.random.default_rng(99 + atype)
    m, n = 640, 150
    A = random_matrix(rng, m, n, atype, zero_cols=(7,))
    dA = to_device_colmajor(A)
    eps = _eps_for(atype)
    u, cp, lp, tri = hy.herk_batch_init(eps, m, n, atype)
    segs, vexp = _run_exponents(hy, dA, m, n, m, atype, u)
    C = _run_herk(hy, dA, m, n, m, atype, u, lp, cp, segs, vexp)
    gtype, gbytes = hy.dequantize_init(n, lp, C, vexp, atype)
    Ch, vh = C.cpu().numpy().view(np.uint64), vexp[0].cpu().numpy()
    want_g, want_b, _ = O.dequantize_init(Ch, vh, n, lp, atype, corr=7, f64_capable=1)
    assert (gtype, gbytes) == (want_g, want_b)
    ldg = n + 3
    G = torch.zeros((n, ldg * gbytes), dtype=torch.uint8, device="cuda")
    hy.dequantize(n, lp, C, vexp, gtype, G, ldg)
    torch.cuda.synchronize()
    want = O.dequantize(Ch, vh, n, lp, gtype)
    got = G.cpu().numpy()[:, :n * gbytes].reshape(n, n, gbytes)
    np.testing.assert_array_equal(got, want.view(np.uint8).reshape(n, n, gbytes))


# ---------------------------------------------------------------------------------------------------------
# Side by side with the reference's CUDA library
# ---------------------------------------------------------------------------------------------------------

REF_CASES = [
    (api.F64, 20000, 700, 1e-10),
    (api.F64, 9000, 513, 1e-13),
    (api.F32, 30000, 520, 1e-5),
    (api.F64_COMPLEX, 6000, 300, 1e-10),
    (api.F16, 5000, 256, 1e-2),
]


@pytest.mark.parametrize("atype,m,n,eps", REF_CASES)
def test_stage_outputs_equal_reference_library(hy, ref, atype, m, n, eps):
    """Same device buffers through both libraries: vexp, packed integer Gram, Gram format and Gram bits agree."""
    torch = _torch()
    rng = np.random.default_rng(4242 + m)
    A = random_matrix(rng, m, n, atype, zero_cols=(1,), spread_rows=(10.0 if atype == api.F64 else 0.0))
    dA = to_device_colmajor(A, None, atype)
    out = []
    for lib in (hy, ref):
        u, cp, lp, tri = lib.herk_batch_init(eps, m, n, atype)
        segs, vexp = _run_exponents(lib, dA, m, n, m, atype, u)
        C = torch.zeros((cp * lp, tri), dtype=torch.int64, device="cuda")
        lib.herk_batch(segs[0], segs[1], segs[2], n, atype, dA, m, u, vexp, 0, lp, C)
        torch.cuda.synchronize()
        gtype, gbytes = lib.dequantize_init(n, lp, C, vexp, atype)
        G = torch.zeros((n, n * gbytes), dtype=torch.uint8, device="cuda")
        lib.dequantize(n, lp, C, vexp, gtype, G, n)
        torch.cuda.synchronize()
        out.append(((u, cp, lp, tri), vexp, C, (gtype, gbytes), G))
    assert hy.status() == 0
    assert out[0][0] == out[1][0]
    assert torch.equal(out[0][1], out[1][1]), "column exponents differ from the reference"
    assert torch.equal(out[0][2], out[1][2]), "packed integer Gram differs from the reference"
    assert out[0][3] == out[1][3]
    assert torch.equal(out[0][4], out[1][4]), "dequantised Gram bits differ from the reference"


# ---------------------------------------------------------------------------------------------------------
# Limb route (balanced base-256 digits, digit-pair products on the tensor cores)
# ---------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("atype,u", [(api.F64, 6), (api.F64, 40), (api.F64, 70), (api.F32_COMPLEX, 23)])
def test_limb_quantizer_digits_recompose_the_quantised_value(hy, atype, u):
    """sum_k digit_k 256^k equals rint(a 2^vexp) for every entry; digits are int8; padding rows are zero."""
    torch = _torch()
    rng = np.random.default_rng(800 + u)
    m, n = 150, 11
    A = random_matrix(rng, m, n, atype, zero_cols=(4,))
    dA = to_device_colmajor(A, None, atype)
    segs, vexp = _run_exponents(hy, dA, m, n, m, atype, u)
    order = (u + 9) // 8
    parts = 3 if atype & 1 else 1
    ldk = 256
    W = torch.full((order, n, parts * ldk), 77, dtype=torch.int8, device="cuda")
    hy.quantize_limbs(atype, m, n, dA, m, vexp, order, W, ldk)
    torch.cuda.synchronize()
    Wh = W.cpu().numpy().astype(object)
    q = O.quantize_ints(_oracle_input(A, atype), atype, vexp[0].cpu().numpy())
    for p in range(parts):
        src = q[0] if p == 0 else q[1] if p == 1 else [[-v for v in col] for col in q[0]]
        got = sum(Wh[k, :, p * ldk:p * ldk + m] * (256 ** k) for k in range(order))
        assert np.array_equal(got, np.array(src, dtype=object))
        assert np.all(W.cpu().numpy()[:, :, p * ldk + m:(p + 1) * ldk] == 0)


@pytest.mark.parametrize("atype,m,n,pad,seg_k,zero_cols", CASES)
def test_forced_limb_route_gives_the_same_integer_gram(hy, atype, m, n, pad, seg_k, zero_cols):
    """GramMatrixAlgorithm = 'L': packed integer Gram equals the oracle bit for bit, also when accumulating."""
    torch = _torch()
    rng = np.random.default_rng(1000 + m + n + atype)
    A = random_matrix(rng, m, n, atype, zero_cols=zero_cols)
    lda = m + pad
    dA = to_device_colmajor(A, lda, atype)
    u, cp, lp, tri = hy.herk_batch_init(_eps_for(atype), m, n, atype)
    segs, vexp = _run_exponents(hy, dA, m, n, lda, atype, u, seg_k)
    Ao = _oracle_input(A, atype)
    want_vexp = O.column_exponents(Ao, atype, u, *segs)
    want_C = O.gram_exact(Ao, atype, want_vexp[0], lp)
    hy.h.GramMatrixAlgorithm = b"L"
    try:
        C = _run_herk(hy, dA, m, n, lda, atype, u, lp, cp, segs, vexp)
        np.testing.assert_array_equal(C.cpu().numpy().view(np.uint64), want_C)
        C2 = _run_herk(hy, dA, m, n, lda, atype, u, lp, cp, segs, vexp, beta=1, C=C)
        np.testing.assert_array_equal(C2.cpu().numpy().view(np.uint64), O.gram_exact(Ao, atype, want_vexp[0], lp, C=want_C))
    finally:
        hy.h.GramMatrixAlgorithm = b"A"
        hy.h.GramSegmentK = 8192


@pytest.mark.parametrize("atype,m,n,eps,ref_alg", [(api.F64, 120000, 520, 1e-10, b"L"), (api.F64_COMPLEX, 40000, 300, 1e-12, b"L"),
                                                     (api.F32, 9000, 260, 1e-5, b"L"), (api.F64, 150000, 520, 1e-10, b"C")])
def test_limb_route_equals_reference_limb_route(hy, ref, atype, m, n, eps, ref_alg):
    """Both libraries forced onto their limb decompositions (several K chunks on our side): identical integer
    Gram, and identical to this build's CRT route.  Beyond 130816 rows the reference's limb route disagrees with
    the reference's own CRT route (its K-chunked accumulation, src/hyacin_herk.cpp:117-137); there the checker is
    the reference's CRT route."""
    torch = _torch()
    rng = np.random.default_rng(31337 + n)
    A = random_matrix(rng, m, n, atype, col_scale_decades=1.0)
    dA = to_device_colmajor(A, None, atype)
    out = {}
    for name, lib, alg in (("limbs", hy, b"L"), ("crt", hy, b"C"), ("ref", ref, ref_alg)):
        lib.h.GramMatrixAlgorithm = alg
        u, cp, lp, tri = lib.herk_batch_init(eps, m, n, atype)
        segs, vexp = _run_exponents(lib, dA, m, n, m, atype, u)
        C = torch.zeros((cp * lp, tri), dtype=torch.int64, device="cuda")
        lib.herk_batch(segs[0], segs[1], segs[2], n, atype, dA, m, u, vexp, 0, lp, C)
        torch.cuda.synchronize()
        lib.h.GramMatrixAlgorithm = b"A"
        out[name] = C
    assert hy.status() == 0
    assert torch.equal(out["limbs"], out["crt"])
    assert torch.equal(out["limbs"], out["ref"])


@pytest.mark.parametrize("atype,op,m,n,corr", [
    (api.F64_COMPLEX, "N", 66000, 160, 7),      # two row chunks accumulate modulo m; moduli with a square root of -1
    (api.F64_COMPLEX, "C", 1500, 520, 7),       # conjugate-transposed storage, more than one tile row and column
    (api.F32_COMPLEX, "T", 900, 130, 7),
    (api.F64_COMPLEX, "N", 1200, 96, 33),       # 73-bit values: beyond the range of that moduli set, three-part route
])
def test_complex_integer_gram_on_both_crt_routes(hy, atype, op, m, n, corr):
    """Complex input: the sqrt(-1)-moduli route (two planes, one product over all tiles) and, for bit budgets
    it cannot hold, the three-part route give the oracle's packed integer Gram bit for bit."""
    torch = _torch()
    rng = np.random.default_rng(5000 + m + n)
    A = random_matrix(rng, m, n, atype, col_scale_decades=2.0, zero_cols=(1,))
    if op == "C":
        stored = np.ascontiguousarray(A.conj().T)
    elif op == "T":
        stored = np.ascontiguousarray(A.T)
    else:
        stored = A
    eps = _eps_for(atype)
    u, cp, lp, tri = O.herk_init(eps, m, n, atype, corr)
    Ao = _oracle_input(A, atype)
    segs = O.segments(m)
    want_vexp = O.column_exponents(Ao, atype, u, *segs)
    want_C = O.gram_exact(Ao, atype, want_vexp[0], lp)
    dA = to_device_colmajor(stored, atype=atype)
    vexp = torch.from_numpy(want_vexp).cuda()
    C = torch.full((cp * lp, tri), 0x5555555555555555, dtype=torch.int64, device="cuda")
    if op == "N":
        hy.herk_batch(segs[0], segs[1], segs[2], n, atype, dA, m, u, vexp, 0, lp, C)
        torch.cuda.synchronize()
        np.testing.assert_array_equal(C.cpu().numpy().view(np.uint64), want_C)
    else:
        # transposed storage goes through the fit (the stage call takes the 'N' layout only): compare ranks and
        # singular values of the fit on the stored matrix with the fit on an explicit copy
        k = min(n, 64)
        S1 = torch.zeros(k, dtype=torch.float64 if (atype & ~1) == api.F64 else torch.float32, device="cuda")
        S2 = torch.zeros_like(S1)
        V1 = torch.zeros((k, 2 * n), dtype=S1.dtype, device="cuda"); V2 = torch.zeros_like(V1)
        r1 = hy.tsvd_fit(eps, op, m, n, k, dA, n, S1, V1, n, m, atype)
        dN = to_device_colmajor(A, atype=atype)
        r2 = hy.tsvd_fit(eps, "N", m, n, k, dN, m, S2, V2, n, m, atype)
        torch.cuda.synchronize()
        assert r1 == r2 and torch.equal(S1, S2) and torch.equal(V1, V2)
    assert hy.status() == 0


@pytest.mark.parametrize("atype,spread,zero_block", [(api.F64, 12.0, False), (api.F64, 0.0, True), (api.F32_COMPLEX, 0.0, True)])
def test_precision_ladder_over_row_segments_is_exact(hy, atype, spread, zero_block):
    """Row segments far below the column maxima (or all zero) go through cheaper runs; the integer Gram is unchanged."""
    rng = np.random.default_rng(99)
    m, n, seg_k = 120000, 96, 8192
    A = random_matrix(rng, m, n, atype, col_scale_decades=1.0, spread_rows=spread)
    if zero_block:
        A[3 * seg_k:7 * seg_k] = 0                     # four all-zero segments in the middle
        A[10 * seg_k:] *= 1e-5                         # and a tail seventeen bits below the column maxima
    dA = to_device_colmajor(A, atype=atype)
    eps = _eps_for(atype)
    u, cp, lp, tri = hy.herk_batch_init(eps, m, n, atype)
    segs, vexp = _run_exponents(hy, dA, m, n, m, atype, u, seg_k)
    assert segs[0] > 1
    Ao = _oracle_input(A, atype)
    want_vexp = O.column_exponents(Ao, atype, u, *segs)
    np.testing.assert_array_equal(vexp.cpu().numpy(), want_vexp)
    # bits per row segment, the input of the ladder (reference: src/fp_exponent.cu:67-76)
    import torch
    seg_u = torch.zeros(segs[0], dtype=torch.int32, device="cuda")
    hy.vector_range(segs[0], n, u, vexp, seg_u)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(seg_u.cpu().numpy(), O.vector_range(want_vexp, u))
    hy.launch_count(reset=True)
    C = _run_herk(hy, dA, m, n, m, atype, u, lp, cp, segs, vexp)
    used = hy.launch_count(reset=True)
    want_C = O.gram_exact(Ao, atype, want_vexp[0], lp)
    np.testing.assert_array_equal(C.cpu().numpy().view(np.uint64), want_C)
    # the plain schedule needs two chunks (quantise + Gram each) and one reconstruction per panel; the ladder adds the
    # segment scan and one reconstruction per run
    assert used >= 8, used


@pytest.mark.parametrize("atype,eps,ranks", [(api.F64, 1e-10, 1), (api.F64, 1e-10, 8), (api.F64_COMPLEX, 1e-13, 2),
                                             (api.F32, 1e-5, 64), (api.F64, 1e-16, 1000)])
def test_dequantize_from_slices_gives_the_bits_of_the_two_step_route(hy, atype, eps, ranks):
    """The fits' post-collective route (format scan and conversion straight from the exchanged slices) against
    hyacinXdequantizeInit + hyacinXdequantize on the limbs: same format, same bits, any communicator size."""
    torch = _torch()
    rng = np.random.default_rng(123 + atype + ranks)
    m, n = 900, 203
    A = random_matrix(rng, m, n, atype, zero_cols=(11,))
    dA = to_device_colmajor(A)
    # size the limbs as a job of `ranks` such row blocks would (the slices must hold the sum over all ranks)
    u, cp, lp, tri = hy.herk_batch_init(eps, m * ranks, n, atype)
    segs, vexp = _run_exponents(hy, dA, m, n, m, atype, u)
    C = _run_herk(hy, dA, m, n, m, atype, u, lp, cp, segs, vexp)
    gtype, gbytes = hy.dequantize_init(n, lp, C, vexp, atype)
    ldg = n + 1
    G1 = torch.zeros((n, ldg * gbytes), dtype=torch.uint8, device="cuda")
    hy.dequantize(n, lp, C, vexp, gtype, G1, ldg)
    G2 = torch.zeros_like(G1)
    g2 = hy.dequantize_via_slices(n, lp, C, vexp, atype, ranks, G2, ldg)
    torch.cuda.synchronize()
    assert g2 == gtype
    assert torch.equal(G1, G2)


def test_an_expired_wait_is_reported_and_leaves_the_device_usable(hy):
    """The bounded waits of the Gram and Cholesky kernels never expire in a healthy run.  The self-test kernel makes
    one expire harmlessly (a barrier that nothing completes, a short poll limit): the kernel returns, the code shows
    in the status word, clearing works, and the next real call is still bit-exact."""
    import torch
    assert hy.status() == 0
    assert hy.self_test_wait(2000, 77) == 0
    assert hy.status(clear=False) == 77
    assert hy.status(clear=True) == 77
    assert hy.status() == 0
    rng = np.random.default_rng(12)
    m, n, atype, eps = 3000, 200, api.F64, 1e-10
    A = random_matrix(rng, m, n, atype)
    dA = to_device_colmajor(A)
    u, cp, lp, tri = hy.herk_batch_init(eps, m, n, atype)
    b, s, l = hy.segments(m)
    vexp = torch.zeros((b + 1, n), dtype=torch.int32, device="cuda")
    C = torch.zeros((cp * lp, tri), dtype=torch.int64, device="cuda")
    hy.quantize_scale_batch(b, s, l, n, atype, dA, m, u, vexp)
    hy.herk_batch(b, s, l, n, atype, dA, m, u, vexp, 0, lp, C)
    torch.cuda.synchronize()
    want_vexp = O.column_exponents(A, atype, u, b, s, l)
    assert np.array_equal(C.cpu().numpy().view(np.uint64), O.gram_exact(A, atype, want_vexp[0], lp))
    assert hy.status() == 0
