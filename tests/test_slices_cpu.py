"""World-size-2 CPU (gloo) test of the cross-rank reduction scheme: the slice layout the library derives for a
communicator size makes a plain unsigned 64-bit sum exact, whatever the signs and magnitudes of the limbs."""
import ctypes
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hyacinth_b200 import api
from oracle import oracle as O

MASK64 = (1 << 64) - 1


def slice_plan(order, ranks):
    lib = api.load()
    s, w = ctypes.c_int32(), ctypes.c_int32()
    lib.hyacinB200SlicePlan(order, ranks, ctypes.byref(s), ctypes.byref(w))
    return s.value, w.value


def to_slices(value, slices, width):
    out = []
    for _ in range(slices - 1):
        out.append(value & ((1 << width) - 1))
        value >>= width
    out.append(value & MASK64)            # signed remainder in two's complement
    return out


def from_slices(words, slices, width):
    total = 0
    for i, w in enumerate(words):
        if i + 1 == slices and w >> 63:
            w -= 1 << 64
        total += w << (i * width)
    return total


@pytest.mark.parametrize("order", [1, 2, 3])
@pytest.mark.parametrize("ranks", [2, 8, 1 << 15, 1 << 20])
def test_slice_plan_cannot_overflow(order, ranks):
    slices, width = slice_plan(order, ranks)
    assert 2 <= slices <= order + 3 and 1 <= width <= 62
    total_bits = 63 * order + 1
    assert width + (ranks - 1).bit_length() <= 64
    assert total_bits - (slices - 1) * width + (ranks - 1).bit_length() <= 64
    # extreme values survive the round trip
    for v in (0, 1, -1, (1 << (63 * order)) - 1, -(1 << (63 * order))):
        assert from_slices(to_slices(v, slices, width), slices, width) == v


def _worker(rank, world, port, order, seed, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(seed + rank)
    count = 257
    top = 63 * order - 2                               # two ranks: the sum still fits the limb format
    vals = []
    for _ in range(count):
        bits = int(rng.integers(1, top + 1))
        mag = int.from_bytes(rng.bytes(24), "little") % (1 << bits)
        vals.append(-mag if rng.integers(0, 2) else mag)
    vals[0], vals[1] = (1 << (63 * order - 2)) - 1, -(1 << (63 * order - 2))          # near the representable edge
    slices, width = slice_plan(order, world)
    wire = np.array([to_slices(v, slices, width) for v in vals], dtype=np.uint64).T.copy()        # [slices][count]
    t = torch.from_numpy(wire.view(np.int64))          # gloo sums int64 with wrap-around, i.e. unsigned sums mod 2^64
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    summed = t.numpy().view(np.uint64)
    got = [from_slices([int(summed[s, i]) for s in range(slices)], slices, width) for i in range(count)]
    limbs = np.array([O.int_to_limbs(v, order) for v in vals], dtype=np.uint64).T.copy()        # [order][count]
    q.put((rank, got, limbs))
    dist.destroy_process_group()


@pytest.mark.parametrize("order", [1, 2, 3])
def test_two_rank_sum_of_slices_equals_exact_limb_sum(order):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + order + (os.getpid() % 500)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, order, 99, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted((q.get(timeout=120) for _ in range(2)), key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
    exact = O.allreduce_sum([res[0][2], res[1][2]], 1, order)          # oracle: exact sum in limb format
    for r in res:
        want = [O.limbs_to_int([exact[l, i] for l in range(order)], order) for i in range(exact.shape[1])]
        assert r[1] == want


@pytest.mark.parametrize("full", [False, True])
def test_gram_schedule_covers_every_tile_once_and_is_balanced(full):
    """The residue Gram kernel deals items of one or two 256 x 256 tiles to its CTA pairs: over all pairs every tile
    of every modulus plane appears exactly once, items stay inside the tile grid, and no pair gets more than one tile
    above the even share (host mirror of the device schedule; 74 pairs = one B200)."""
    from hyacinth_b200 import api
    lib = api.load()
    for tiles_x in (1, 2, 3, 4, 7, 8, 16, 17, 32):
        pair_rows = tiles_x if not full else max(1, tiles_x - 1)        # a full product may have fewer tile rows
        for moduli in (1, 8, 13, 15):
            for pairs in (1, 2, 5, 74):
                seen, loads = set(), []
                for pair in range(pairs):
                    items = api.gram_items(tiles_x, pair_rows, full, moduli, pairs, pair, lib)
                    loads.append(sum(w for *_, w in items))
                    for m, ty, tx, w in items:
                        assert w in (1, 2) and 0 <= m < moduli
                        for d in range(w):
                            assert (0 <= ty < pair_rows and 0 <= tx + d < tiles_x) if full else (0 <= ty <= tx + d < tiles_x)
                            assert (m, ty, tx + d) not in seen
                            seen.add((m, ty, tx + d))
                total = moduli * (pair_rows * tiles_x if full else tiles_x * (tiles_x + 1) // 2)
                assert len(seen) == total
                assert max(loads) <= -(-total // pairs) + 1, (tiles_x, moduli, pairs, max(loads), total / pairs)
    # the headline case: 13 planes of 136 pair tiles over 74 pairs -> 24 tile-units at most (ideal 23.9)
    assert max(sum(w for *_, w in api.gram_items(16, 16, False, 13, 74, c, lib)) for c in range(74)) == 24


def test_crt_plan_groups_rows_when_that_saves_a_modulus():
    """hyacinB200CrtPlan (host logic): the moduli always cover the bits of one row group, 2 u + 1 + ceil(log2 group), and
    the group size is the cheaper of 'one more modulus for every row' and 'one more reconstruction per group'."""
    import math
    import re
    lib = api.load()
    header = open(os.path.join(os.path.dirname(os.path.abspath(api.__file__)), "csrc", "crt_tables.h")).read()
    bits = [int(v) for v in re.search(r"kRangeBits\[kMaxModuli\] = \{([^}]*)\}", header).group(1).split(",")]

    def plan(u, rows):
        m, vb, g, c = (ctypes.c_int32() for _ in range(4))
        lib.hyacinB200CrtPlan(u, 0, ctypes.c_int64(rows), ctypes.byref(m), ctypes.byref(vb), ctypes.byref(g), ctypes.byref(c))
        return m.value, g.value, c.value

    for u, rows in [(40, 1 << 20), (40, 1 << 22), (40, 1 << 23), (23, 1 << 17), (23, (1 << 17) + 300), (23, 1 << 20), (13, 1 << 20), (40, 512),
                    (30, 1 << 22), (70, 1 << 20)]:
        moduli, group, chunk = plan(u, rows)
        need = 2 * u + 1 + (math.ceil(math.log2(group)) if group > 1 else 0)
        assert bits[moduli - 1] >= need and (moduli == 1 or bits[moduli - 2] < need), (u, rows, moduli, group)
        assert group <= rows and chunk <= max(group, 128) and (group == rows or group % chunk == 0)
    assert plan(40, 1 << 20)[:2] == (13, 1 << 20)            # benchmark configuration 2: one group
    assert plan(23, 1 << 17)[:2] == (8, 1 << 16)             # configuration 5: two groups of 65536 rows instead of 9 moduli
    assert plan(40, 1 << 22)[:2] == (13, 1 << 21)            # two groups instead of 14 moduli
