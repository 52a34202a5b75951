"""The committed CRT tables: in step with their generator, and arithmetically what the kernels assume."""
import importlib.util
import io
import math
import os
import re
from contextlib import redirect_stdout
from itertools import combinations

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "hyacinth_b200", "csrc")


def _generator():
    spec = importlib.util.spec_from_file_location("gen_crt_tables", os.path.join(CSRC, "gen_crt_tables.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_committed_header_is_what_the_generator_prints():
    gen = _generator()
    buf = io.StringIO()
    with redirect_stdout(buf):
        gen.main()
    with open(os.path.join(CSRC, "crt_tables.h")) as f:
        assert f.read() == buf.getvalue()


def test_moduli_sets_are_coprime_and_fit_an_int8_operand():
    gen = _generator()
    for mods in (gen.choose_moduli(), gen.choose_moduli_2m()):
        assert all(2 <= m <= 256 for m in mods)
        assert all(math.gcd(a, b) == 1 for a, b in combinations(mods, 2))
        assert mods == sorted(mods, reverse=True)


def test_complex_moduli_have_a_square_root_of_minus_one_and_invert_two():
    gen = _generator()
    mods = gen.choose_moduli_2m()
    assert len(mods) >= 16 and all(m % 2 == 1 for m in mods)
    for m in mods:
        iota = gen.sqrt_minus_one(m)
        assert (iota * iota + 1) % m == 0
        # p = re - iota im, q = re + iota im  =>  p_y q_x = (re_y re_x + im_y im_x) + iota (re_y im_x - im_y re_x)
        for re_y, im_y, re_x, im_x in ((3, 5, 7, 11), (200, 1, 17, 250), (0, 9, 9, 0)):
            p_y, q_x = (re_y - iota * im_y) % m, (re_x + iota * im_x) % m
            q_y, p_x = (re_y + iota * im_y) % m, (re_x - iota * im_x) % m
            real, imag = re_y * re_x + im_y * im_x, re_y * im_x - im_y * re_x
            x_yx, x_xy = (p_y * q_x) % m, (p_x * q_y) % m
            assert x_yx == (real + iota * imag) % m and x_xy == (real - iota * imag) % m
            assert ((x_yx + x_xy) * pow(2, -1, m)) % m == real % m
            assert ((x_yx - x_xy) * pow(2 * iota, -1, m)) % m == imag % m


def test_range_bits_of_the_header_match_the_products():
    text = open(os.path.join(CSRC, "crt_tables.h")).read()
    for ns in ("crt", "crt2m"):
        block = text[text.index("namespace " + ns + " {"):]
        mods = [int(v) for v in re.search(r"kModulus\[kMaxModuli\] = \{([^}]*)\}", block).group(1).split(",")]
        bits = [int(v) for v in re.search(r"kRangeBits\[kMaxModuli\] = \{([^}]*)\}", block).group(1).split(",")]
        prod = 1
        for m, b in zip(mods, bits):
            prod *= m
            assert 2 ** b < prod <= 2 ** (b + 1)


def test_float_reduction_constants_of_the_header_hold_for_every_residue_sum():
    """The quantiser's float reduction (q = fmaf(X + t, 1 / m, add); residue = low byte of (X + t) - bits(q) m) must
    give a residue of t in [-128, 127] for EVERY sum t the kernel can form.  Re-checked here from the committed
    header with exact integer arithmetic, modulus by modulus."""
    import struct
    gen = _generator()
    text = open(os.path.join(CSRC, "crt_tables.h")).read()
    for ns, t_max in (("crt", 1 << 20), ("crt2m", 1 << 21)):
        block = text[text.index("namespace " + ns + " {"):]
        mods = [int(v) for v in re.search(r"kModulus\[kMaxModuli\] = \{([^}]*)\}", block).group(1).split(",")]
        arr = {name: [int(v.strip().rstrip("u"), 16) for v in re.search(name + r"\[kMaxModuli\] = \{([^}]*)\}", block).group(1).split(",")]
               for name in ("kFrBase", "kFrInv", "kFrAdd")}
        # the largest sum: additive constant below m, 255 * 255 per byte, 12 bytes (real and imaginary for the complex set)
        assert 256 + (2 if ns == "crt2m" else 1) * 12 * 255 * 255 < t_max
        for i, m in enumerate(mods):
            if m == 256:
                continue
            X = (arr["kFrBase"][i] - 0x4B000000) + (1 << 23)
            inv = struct.unpack("<f", struct.pack("<I", arr["kFrInv"][i]))[0]
            add = struct.unpack("<f", struct.pack("<I", arr["kFrAdd"][i]))[0]
            assert add == int(add)
            mant, exp, _ = gen.float32_parts(inv)
            assert gen.fr_verify(m, X, mant, exp, int(add), t_max) <= 127
