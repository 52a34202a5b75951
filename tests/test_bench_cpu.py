"""Host-side pieces of bench.py that need no GPU: the checksums that let two arms (and all ranks) be compared, and
the stdout guard that keeps library banners out of the one JSON line."""
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_checksum_separates_permutations_and_single_bit_flips():
    g = torch.Generator().manual_seed(7)
    a = torch.randint(-2**40, 2**40, (3, 1001), dtype=torch.int64, generator=g)
    same = bench.checksum(torch, a.clone())
    assert same == bench.checksum(torch, a)
    flipped = a.clone(); flipped[1, 500] ^= 1 << 33
    assert bench.checksum(torch, flipped) != same
    swapped = a.clone(); swapped[0, 3], swapped[0, 4] = a[0, 4].clone(), a[0, 3].clone()
    got = bench.checksum(torch, swapped)
    assert got[0] == same[0] and got[1] != same[1]          # the plain sum cannot see a permutation, the weighted one does
    odd = torch.arange(13, dtype=torch.uint8)               # byte counts that are not a multiple of eight are padded
    assert bench.checksum(torch, odd) == bench.checksum(torch, odd.clone())
    assert bench.checksum(torch, torch.zeros(0)) is None


def test_stdout_guard_moves_library_output_to_stderr():
    code = ("import bench, os\nprint('first')\nwith bench.stdout_to_stderr():\n    os.write(1, b'banner\\n')\nprint('second')\n")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0 and r.stdout == "first\nsecond\n" and "banner" in r.stderr


def test_clock_samples_are_cut_to_the_timed_region():
    """ClockSampler.summarise keeps the nvidia-smi lines whose own timestamp lies inside the timed region and reports the
    median clock and the throttle reasons of those lines only."""
    import datetime
    import bench
    base = datetime.datetime(2026, 1, 2, 3, 4, 5).timestamp()

    def line(offset, mhz, cap):
        stamp = datetime.datetime.fromtimestamp(base + offset).strftime("%Y/%m/%d %H:%M:%S.%f")[:-3]
        return f"{stamp}, {mhz}, 1965, 700.00, Not Active, Not Active, Not Active, {'Active' if cap else 'Not Active'}"

    text = "\n".join([line(0.0, 1965, False), line(0.1, 1900, False), line(0.5, 1200, True), line(0.6, 1300, True), line(0.7, 1250, True),
                      line(1.5, 1800, False), "garbage line"])
    got = bench.ClockSampler.summarise(text, base + 0.45, base + 0.75)
    assert got["samples"] == 3 and got["samples_inside_timed_region"] == 3
    assert got["sm_mhz"] == 1250 and got["sm_max_mhz"] == 1965 and got["reasons"] == ["sw_power_cap"]
    # a region too short to catch a line falls back to all lines
    got = bench.ClockSampler.summarise(text, base + 0.31, base + 0.32)
    assert got["samples"] == 6 and got["samples_inside_timed_region"] == 0
