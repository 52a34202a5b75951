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


def _pool_attr(pool, attr):
    """cuMemPoolGetAttribute on the handle's pool: 5 reserved now, 7 used now, 8 used high-water mark."""
    import ctypes
    cuda = ctypes.CDLL("libcuda.so.1")
    val = ctypes.c_uint64(0)
    assert cuda.cuMemPoolGetAttribute(ctypes.c_void_p(pool), ctypes.c_int(attr), ctypes.byref(val)) == 0
    return val.value


def test_static_scratch_call_allocates_nothing(hy):
    """A zero-row call binds the module's array and returns 0; after it, a full call leaves the free device memory,
    the pool's reservation and the pool's high-water mark where they were."""
    import ctypes
    import torch
    n, m, atype, eps = 300, 5000, api.F64, 1e-9
    rng = np.random.default_rng(11)
    dA = to_device_colmajor(random_matrix(rng, m, n, atype))
    u, cp, lp, tri = hy.herk_batch_init(eps, m, n, atype)
    b, s, l = hy.segments(m)
    vexp = torch.zeros((b + 1, n), dtype=torch.int32, device="cuda")
    hy.quantize_scale_batch(b, s, l, n, atype, dA, m, u, vexp)
    C = torch.zeros((cp * lp, tri), dtype=torch.int64, device="cuda")
    assert hy.herk_batch_static(1, 0, 0, n, atype, dA, m, u, vexp, 0, lp, C) == 0          # warm-up: no rows
    assert hy.herk_batch_static(b, s, l, n, atype, dA, m, u, vexp, 0, lp, C) == 0          # loads every kernel once
    torch.cuda.synchronize()
    pool = hy.h.mempool
    cuda = ctypes.CDLL("libcuda.so.1")
    zero = ctypes.c_uint64(0)
    assert cuda.cuMemPoolSetAttribute(ctypes.c_void_p(pool), ctypes.c_int(8), ctypes.byref(zero)) == 0   # reset the high-water mark
    free0, reserved0, used0 = torch.cuda.mem_get_info()[0], _pool_attr(pool, 5), _pool_attr(pool, 7)
    assert hy.herk_batch_static(b, s, l, n, atype, dA, m, u, vexp, 0, lp, C) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free0
    assert _pool_attr(pool, 5) == reserved0 and _pool_attr(pool, 7) == used0 and _pool_attr(pool, 8) <= used0
    want = torch.zeros_like(C)
    hy.herk_batch(b, s, l, n, atype, dA, m, u, vexp, 0, lp, want)
    torch.cuda.synchronize()
    assert torch.equal(C, want) and hy.status() == 0
