"""hyacinB200HerkBatchStatic -- the Gram entry point for callers that must not allocate (their application owns
all device memory through its own arena, or they sit in a latency-bound loop) -- must give exactly the integer
Gram of hyacinXherkBatch.  Two calls in a row share the module's fixed scratch array, so the second call runs on
top of the first one's leftovers; sizes beyond the array must be refused, not attempted.

Collected last on purpose: a failure here cannot hide the result of any other test under `pytest -x`."""
import numpy as np
import pytest

from hyacinth_b200 import api
from tests.helpers import random_matrix, to_device_colmajor

pytestmark = pytest.mark.gpu


def _pair(hy, torch, atype, m, n, eps, seed, beta_first=0):
    rng = np.random.default_rng(seed)
    A = random_matrix(rng, m, n, atype, zero_cols=(1,))
    dA = to_device_colmajor(A)
    u, cp, lp, tri = hy.herk_batch_init(eps, m, n, atype)
    b, s, l = hy.segments(m)
    vexp = torch.zeros((b + 1, n), dtype=torch.int32, device="cuda")
    hy.quantize_scale_batch(b, s, l, n, atype, dA, m, u, vexp)
    start = torch.randint(-5, 5, (cp * lp, tri), dtype=torch.int64, device="cuda") if beta_first else torch.zeros((cp * lp, tri), dtype=torch.int64, device="cuda")
    want, got = start.clone(), start.clone()
    hy.herk_batch(b, s, l, n, atype, dA, m, u, vexp, beta_first, lp, want)
    rc = hy.herk_batch_static(b, s, l, n, atype, dA, m, u, vexp, beta_first, lp, got)
    torch.cuda.synchronize()
    return rc, want, got


def test_static_scratch_gram_equals_pool_gram_twice_in_a_row(hy):
    import torch
    # first call: real FP64, ragged sizes, several row chunks inside the fixed array
    rc, want, got = _pair(hy, torch, api.F64, 20000, 700, 1e-10, seed=1)
    assert rc == 0 and torch.equal(want, got)
    # second call straight after, different type and shape, accumulating into a non-zero C: the array still holds
    # the planes and residues of the first call
    rc, want, got = _pair(hy, torch, api.F32_COMPLEX, 3000, 260, 1e-4, seed=2, beta_first=1)
    assert rc == 0 and torch.equal(want, got)
    assert hy.status() == 0


def test_static_scratch_refuses_what_does_not_fit(hy):
    import torch
    n = 4096                                   # residues alone (13 moduli x 272 tiles x 32 KiB) exceed 64 MiB
    dA = torch.ones((n, 256), dtype=torch.float64, device="cuda")
    vexp = torch.zeros((2, n), dtype=torch.int32, device="cuda")
    C = torch.full((2, n * (n + 1) // 2), 7, dtype=torch.int64, device="cuda")
    rc = hy.herk_batch_static(1, 256, 256, n, api.F64, dA, 256, 40, vexp, 0, 2, C)
    torch.cuda.synchronize()
    assert rc == -2
    assert int((C != 7).sum()) == 0            # refused before touching the output
