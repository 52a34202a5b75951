#!/usr/bin/env python3
"""Generate crt_tables.h: the CRT moduli of the B200 Gram kernels and every constant derived from them.

Run from anywhere: ``python gen_crt_tables.py > crt_tables.h`` (the generated header is committed so that a
build needs no Python).  The moduli are chosen here, not taken from a table: every modulus must fit an int8
operand after centring (<= 256), the set must be pairwise coprime, and each prefix of the list should have
a large product so that few moduli cover a given bit budget.  Large primes are taken as they are; each small
prime enters through the largest number <= 256 whose smallest prime factor it is (2^8, 3*5*17, 7*31, 11*23,
13*19), which spends the small primes without wasting a slot on a small modulus.

A second set (namespace crt2m) serves complex input: every modulus there is odd and has a square root of -1
(all its prime factors are 1 mod 4), so a complex value re + i im maps to the two residues re -+ iota im and the
Hermitian Gram needs one integer product per entry pair instead of two.
"""
import math
from itertools import combinations

NMOD = 24
NBYTES = 12          # quantised values are at most 96 bits wide


def choose_moduli():
    def prime_factors(n):
        f, p = set(), 2
        while p * p <= n:
            while n % p == 0:
                f.add(p)
                n //= p
            p += 1
        if n > 1:
            f.add(n)
        return f

    # For every prime, the largest number <= 256 that is built from that prime and at most one other prime
    # factor which is too small to be worth a modulus of its own (p*q with q < 128), or a pure prime power.
    best = {}
    for n in range(256, 128, -1):
        f = prime_factors(n)
        small = [p for p in f if p < 128]
        big = [p for p in f if p >= 128]
        if big and small:
            continue                      # a large prime times anything exceeds 256 anyway
        key = min(f)
        if key not in best:
            best[key] = n
    # keep candidates pairwise coprime, largest first
    chosen = []
    for n in sorted(set(best.values()), reverse=True):
        if all(math.gcd(n, c) == 1 for c in chosen):
            chosen.append(n)
    assert len(chosen) >= NMOD
    mods = chosen[:NMOD]
    for a, b in combinations(mods, 2):
        assert math.gcd(a, b) == 1
    return mods


def choose_moduli_2m():
    """Odd numbers <= 256 whose prime factors are all 1 mod 4, pairwise coprime, largest first."""
    def ok(n):
        p, m = 2, n
        while p * p <= m:
            while m % p == 0:
                if p % 4 != 1:
                    return False
                m //= p
            p += 1
        return m == 1 or m % 4 == 1
    chosen = []
    for n in range(255, 4, -2):
        if ok(n) and all(math.gcd(n, c) == 1 for c in chosen):
            chosen.append(n)
    return chosen


def sqrt_minus_one(m):
    for i in range(2, m):
        if (i * i + 1) % m == 0:
            return i
    raise ValueError(m)


# ---- float reduction of the quantiser's residue sums ---------------------------------------------------------
# The quantiser forms t = bias + sum_b byte_b * weight_b (a non-negative integer below t_max) with dp4a and needs
# some r = t (mod m) in [-128, 127].  It starts the dp4a accumulator at the BITS of a float X (X = 256 w, 2^23 <= X,
# X + t_max < 2^24, where floats are the integers), so that the accumulator read as a float is X + t exactly; then
#     q_m = fmaf(X + t, inv, add)            inv = float(1 / m), add = Y - round(X * inv), Y = 1.5 * 2^23
# is Y + q with q an integer within 1/2 + slack of t / m (the fused multiply-add rounds once, to unit spacing), and
#     r   = (X + t) - bits(q_m) * m          (32-bit integer arithmetic, low byte taken)
# because bits(q_m) = bits(Y) + q and both X and bits(Y) * m are multiples of 256.  w is chosen so that X * inv is as
# close to an integer as possible, which keeps the slack far below the margin (128 - m / 2) / m; fr_constants()
# checks every t in [0, t_max) with exact integer arithmetic before a table is emitted.
FR_Y = 3 << 22


def float32_parts(x):
    """x (a Python float that is exactly a float32) as (mantissa, exponent): x = mantissa * 2^exponent."""
    import struct
    bits = struct.unpack("<I", struct.pack("<f", x))[0]
    e, mant = (bits >> 23) & 0xFF, bits & 0x7FFFFF
    assert 0 < e < 255
    return (mant | 0x800000), e - 150, bits


def fr_verify(m, X, inv_mant, inv_exp, add, t_max):
    """Exhaustive check of the float reduction for modulus m; returns the largest |r| seen."""
    import numpy as np
    assert inv_exp < 0
    den = 1 << (-inv_exp)
    t = np.arange(t_max, dtype=np.int64)
    tb = X + t
    assert X % 256 == 0 and X >= (1 << 23) and X + t_max <= (1 << 24)
    num = tb * inv_mant + add * den                      # exact value of (X + t) * inv + add, times den
    q_m = num // den
    rem = num - q_m * den
    up = (2 * rem > den) | ((2 * rem == den) & (q_m % 2 == 1))      # round to nearest, ties to even
    q_m = q_m + up
    assert q_m.min() >= (1 << 23) and q_m.max() < (1 << 24)
    r = t - (q_m - FR_Y) * m
    assert r.min() >= -128 and r.max() <= 127 and np.all((r - t) % m == 0)
    x_bits = 0x4B000000 + (X - (1 << 23))
    q_bits = 0x4B000000 + (q_m - (1 << 23))
    low = ((x_bits + t) - q_bits * m) & 0xFF                # what the kernel keeps
    assert np.all(low == (r & 0xFF))
    return int(np.abs(r).max())


def fr_constants(m, t_max):
    """(bits of X, bits of inv, bits of add) for modulus m, verified for every t < t_max."""
    import numpy as np
    import struct
    inv = float(np.float32(1.0) / np.float32(m))
    inv_mant, inv_exp, inv_bits = float32_parts(inv)
    w = np.arange((1 << 23) // 256, ((1 << 24) - t_max) // 256, dtype=np.int64)
    den = 1 << (-inv_exp)
    prod = (w * 256) * inv_mant                          # X * inv, times den
    frac = prod % den
    dist = np.minimum(frac, den - frac)
    best = int(w[int(np.argmin(dist))])
    X = best * 256
    z = (X * inv_mant + den // 2) // den                 # round(X * inv)
    add = FR_Y - z
    fr_verify(m, X, inv_mant, inv_exp, add, t_max)
    add_bits = struct.unpack("<I", struct.pack("<f", float(add)))[0]
    assert struct.unpack("<f", struct.pack("<I", add_bits))[0] == float(add)
    return 0x4B000000 + (X - (1 << 23)), inv_bits, add_bits


def words(v, n):
    return [(v >> (64 * i)) & (2**64 - 1) for i in range(n)]


def emit_set(emit, ns, prefix, mods, complex_set):
    nmod = len(mods)
    emit("namespace hyb { namespace " + ns + " {")
    emit(f"constexpr int kMaxModuli = {nmod};")
    emit(f"constexpr int kMaxBytes = {NBYTES};")
    emit("// Pairwise-coprime moduli, each <= 256 so that centred residues fit an int8 operand.")
    emit("constexpr uint16_t kModulus[kMaxModuli] = { " + ", ".join(map(str, mods)) + " };")
    caps = []
    P = 1
    for m in mods:
        P *= m
        caps.append((P - 1).bit_length() - 1 if P & (P - 1) else P.bit_length() - 2)
    emit("// kRangeBits[k-1] = largest b with 2^b < product of the first k moduli: those k moduli represent every")
    emit("// integer v with |v| <= 2^(b-1) uniquely in the symmetric range (-P/2, P/2).")
    emit("constexpr uint16_t kRangeBits[kMaxModuli] = { " + ", ".join(map(str, caps)) + " };")
    emit("// ceil(2^32 / m): exact quotient by __umulhi for any t with t * m < 2^32.")
    emit("constexpr uint32_t kMagicCeil[kMaxModuli] = { " + ", ".join(str(-(-2**32 // m) & 0xFFFFFFFF) + "u" for m in mods) + " };")
    emit("// floor(2^32 / m): quotient estimate (off by at most one) for any 32-bit t.")
    emit("constexpr uint32_t kMagicFloor[kMaxModuli] = { " + ", ".join(str(2**32 // m) + "u" for m in mods) + " };")

    def weight_table(name, comment, factor):
        emit(comment)
        rows = []
        for m in mods:
            f = factor(m)
            ws = []
            for w in range(NBYTES // 4):
                v = 0
                for b in range(4):
                    v |= ((f * pow(256, 4 * w + b, m)) % m & 0xFF) << (8 * b)
                ws.append(f"0x{v:08x}u")
            rows.append("{ " + ", ".join(ws) + " }")
        emit(f"constexpr uint32_t {name}[kMaxModuli][{NBYTES // 4}] = {{\n  " + ",\n  ".join(rows) + " };")

    weight_table("kByteWeight", "// kByteWeight[i][w]: the four weights 256^(4w+b) mod m_i, b = 0..3, packed little-endian for dp4a.", lambda m: 1)
    emit("// kPow2Bias[i][nb-1] = (128 - 2^(8 nb - 1)) mod m_i: folded into the dp4a accumulator so that a value")
    emit("// biased by 2^(8 nb - 1) (to make its bytes unsigned) reduces to (q + 128) mod m_i.")
    rows = []
    for m in mods:
        rows.append("{ " + ", ".join(str((128 - 2 ** (8 * nb - 1)) % m) for nb in range(1, NBYTES + 1)) + " }")
    emit(f"constexpr uint16_t kPow2Bias[kMaxModuli][{NBYTES}] = {{\n  " + ",\n  ".join(rows) + " };")
    # residue sums: bias (< m) + 255 * 255 per byte, 12 bytes (24 for the complex set: real and imaginary bytes)
    t_max = 1 << (21 if complex_set else 20)
    assert 256 + (2 if complex_set else 1) * NBYTES * 255 * 255 < t_max
    fr = [fr_constants(m, t_max) if m != 256 else (0, 0, 0) for m in mods]
    emit("// Float reduction of a residue sum t < 2^%d (see gen_crt_tables.py): the dp4a accumulator starts at kFrBase (the" % (21 if complex_set else 20))
    emit("// bits of a float X), q_m = fmaf(float(X + t), kFrInv, kFrAdd), and the low byte of (X + t) - bits(q_m) * m is a")
    emit("// residue of t in [-128, 127].  Float constants are given as bit patterns.  Unused for modulus 256.")
    emit("constexpr uint32_t kFrBase[kMaxModuli] = { " + ", ".join(f"0x{a:08x}u" for a, _, _ in fr) + " };")
    emit("constexpr uint32_t kFrInv[kMaxModuli] = { " + ", ".join(f"0x{b:08x}u" for _, b, _ in fr) + " };")
    emit("constexpr uint32_t kFrAdd[kMaxModuli] = { " + ", ".join(f"0x{c:08x}u" for _, _, c in fr) + " };")
    if complex_set:
        iota = {m: sqrt_minus_one(m) for m in mods}
        emit("// iota_i with iota_i^2 = -1 mod m_i; a complex value maps to p = re - iota im and q = re + iota im.")
        emit("constexpr uint16_t kImagUnit[kMaxModuli] = { " + ", ".join(str(iota[m]) for m in mods) + " };")
        weight_table("kByteWeightMinusI", "// (-iota 256^(4w+b)) mod m_i: weights of the imaginary bytes in p.", lambda m: (m - iota[m]) % m)
        weight_table("kByteWeightPlusI", "// (+iota 256^(4w+b)) mod m_i: weights of the imaginary bytes in q.", lambda m: iota[m])
        emit("// Additive constants of p and q when re and im are both biased by B = 2^(8 nb - 1):")
        emit("// kBiasP = (128 - B + iota B) mod m, kBiasQ = (128 - B - iota B) mod m.")
        for name, sign in (("kBiasP", 1), ("kBiasQ", -1)):
            rows = []
            for m in mods:
                rows.append("{ " + ", ".join(str((128 - 2 ** (8 * nb - 1) + sign * iota[m] * 2 ** (8 * nb - 1)) % m) for nb in range(1, NBYTES + 1)) + " }")
            emit(f"constexpr uint16_t {name}[kMaxModuli][{NBYTES}] = {{\n  " + ",\n  ".join(rows) + " };")
        emit("// With X = P^T Q (entry pair (y,x), (x,y)): Re = (X_yx + X_xy) / 2 and Im = (X_yx - X_xy) / (2 iota) mod m_i.")
        emit("constexpr uint16_t kInvTwo[kMaxModuli] = { " + ", ".join(str(pow(2, -1, m)) for m in mods) + " };")
        emit("constexpr uint16_t kInvTwoIota[kMaxModuli] = { " + ", ".join(str(pow(2 * iota[m], -1, m)) for m in mods) + " };")
    emit("// Garner: kInv[j][i] = m_j^-1 mod m_i for j < i (0 elsewhere).")
    rows = []
    for j, mj in enumerate(mods):
        rows.append("{ " + ", ".join(str(pow(mj, -1, mi)) if j < i else "0" for i, mi in enumerate(mods)) + " }")
    emit("constexpr uint8_t kInv[kMaxModuli][kMaxModuli] = {\n  " + ",\n  ".join(rows) + " };")
    emit("// Product of the first k moduli and its half (floor), as three little-endian 64-bit words.")
    P = 1
    prod_rows, half_rows = [], []
    for m in mods:
        P *= m
        assert P < 2**190
        prod_rows.append("{ " + ", ".join(f"0x{w:016x}ull" for w in words(P, 3)) + " }")
        half_rows.append("{ " + ", ".join(f"0x{w:016x}ull" for w in words(P // 2, 3)) + " }")
    emit("constexpr uint64_t kProduct[kMaxModuli][3] = {\n  " + ",\n  ".join(prod_rows) + " };")
    emit("constexpr uint64_t kHalfProduct[kMaxModuli][3] = {\n  " + ",\n  ".join(half_rows) + " };")
    emit("} }  // namespace hyb::" + ns)
    emit("// Brace initialisers of the same tables for __constant__ device copies.")
    emit(f"#define {prefix}_MODULUS_INIT {{ " + ", ".join(map(str, mods)) + " }")
    emit(f"#define {prefix}_MAGIC_CEIL_INIT {{ " + ", ".join(str(-(-2**32 // m) & 0xFFFFFFFF) + "u" for m in mods) + " }")
    inv_rows = []
    for j, mj in enumerate(mods):
        inv_rows.append("{ " + ", ".join(str(pow(mj, -1, mi)) if j < i else "0" for i, mi in enumerate(mods)) + " }")
    emit(f"#define {prefix}_INV_INIT {{ " + ", ".join(inv_rows) + " }")
    emit(f"#define {prefix}_PRODUCT_INIT {{ " + ", ".join(prod_rows) + " }")
    emit(f"#define {prefix}_HALF_PRODUCT_INIT {{ " + ", ".join(half_rows) + " }")
    emit("// Smallest multiple of each modulus above 255: added before subtracting a Garner digit (a byte) so that the")
    emit("// difference stays positive.")
    emit(f"#define {prefix}_LIFT_INIT {{ " + ", ".join(str((255 // m + 1) * m) for m in mods) + " }")
    if complex_set:
        emit(f"#define {prefix}_INV_TWO_INIT {{ " + ", ".join(str(pow(2, -1, m)) for m in mods) + " }")
        emit(f"#define {prefix}_INV_TWO_IOTA_INIT {{ " + ", ".join(str(pow(2 * iota[m], -1, m)) for m in mods) + " }")


def main():
    out = []
    emit = out.append
    emit("// Generated by gen_crt_tables.py -- do not edit by hand.")
    emit("#pragma once")
    emit("#include <stdint.h>")
    emit_set(emit, "crt", "HYB_CRT", choose_moduli(), False)
    mods2 = choose_moduli_2m()
    for a, b in combinations(mods2, 2):
        assert math.gcd(a, b) == 1
    emit_set(emit, "crt2m", "HYB_CRT2M", mods2, True)
    print("\n".join(out))


if __name__ == "__main__":
    main()
