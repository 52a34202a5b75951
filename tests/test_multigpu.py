"""Row-distributed path on 2 GPUs of one box: one process per GPU, NCCL communicator borrowed by the handle.

The exact integer Gram after hyacinAllReduce1Drow must equal, bit for bit, the Gram one GPU computes for the
stacked matrix (integer addition is associative, so rank order and NCCL's algorithm cannot matter), the column
exponents must agree across ranks after hyacinAllReduceVExp, and the distributed fit must return the
single-GPU rank and singular values.  Ranks leave only after their last collective has completed.
"""
import ctypes
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


class _NcclId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_byte * 128)]


def _rank_main(rank, world, port, path_out):
    import torch
    import torch.distributed as dist
    from hyacinth_b200 import api
    from tests.helpers import random_matrix, to_device_colmajor
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    nccl = ctypes.CDLL("libnccl.so.2")
    uid = _NcclId()
    if rank == 0:
        assert nccl.ncclGetUniqueId(ctypes.byref(uid)) == 0
    box = [bytes(uid)]
    dist.broadcast_object_list(box, src=0)
    ctypes.memmove(ctypes.byref(uid), box[0], 128)
    comm = ctypes.c_void_p()
    nccl.ncclCommInitRank.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, _NcclId, ctypes.c_int]
    assert nccl.ncclCommInitRank(ctypes.byref(comm), world, uid, rank) == 0

    results = {}
    for case, (atype, m_local, n, eps) in enumerate([(api.F64, 9000, 384, 1e-10), (api.F32_COMPLEX, 5000, 130, 1e-4)]):
        rng = np.random.default_rng(1234 + case)             # every rank builds the same stacked matrix
        full = random_matrix(rng, m_local * world, n, atype, col_scale_decades=2.0, zero_cols=(2,))
        full[m_local:, 5] *= 1e-3                            # the ranks disagree on a local column exponent
        local = np.ascontiguousarray(full[rank * m_local:(rank + 1) * m_local])
        dA = to_device_colmajor(local)
        h = api.Hyacin(stream=0, nccl_comm=comm.value)
        gm = m_local * world
        u, cp, lp, tri = h.herk_batch_init(eps, gm, n, atype)
        b, s, l = h.segments(m_local)
        vexp = torch.zeros((b + 1, n), dtype=torch.int32, device="cuda")
        C = torch.zeros((cp * lp, tri), dtype=torch.int64, device="cuda")
        h.quantize_scale_batch(b, s, l, n, atype, dA, m_local, u, vexp)
        h.allreduce_vexp(n, vexp)
        h.herk_batch(b, s, l, n, atype, dA, m_local, u, vexp, 0, lp, C)
        h.allreduce_1drow(cp, lp, tri, C)
        torch.cuda.synchronize()
        words = 2 if atype & 1 else 1
        rdt = torch.float64 if (atype & ~1) == api.F64 else torch.float32
        S = torch.zeros(n, dtype=rdt, device="cuda"); V = torch.zeros((n, n * words), dtype=rdt, device="cuda")
        fit_rank = h.tsvd_fit(eps, "N", m_local, n, n, dA, m_local, S, V, n, gm, atype)
        torch.cuda.synchronize()
        assert h.status() == 0
        results[case] = {"vexp0": vexp[0].cpu().numpy(), "C": C.cpu().numpy(), "rank": fit_rank, "S": S.cpu().numpy()}
        if rank == 0:
            # single-GPU answer for the stacked matrix on this rank's GPU, no communicator
            h1 = api.Hyacin(stream=0)
            dF = to_device_colmajor(full)
            b1, s1, l1 = h1.segments(gm)
            v1 = torch.zeros((b1 + 1, n), dtype=torch.int32, device="cuda")
            C1 = torch.zeros((cp * lp, tri), dtype=torch.int64, device="cuda")
            h1.quantize_scale_batch(b1, s1, l1, n, atype, dF, gm, u, v1)
            h1.herk_batch(b1, s1, l1, n, atype, dF, gm, u, v1, 0, lp, C1)
            S1 = torch.zeros(n, dtype=rdt, device="cuda"); V1 = torch.zeros((n, n * words), dtype=rdt, device="cuda")
            r1 = h1.tsvd_fit(eps, "N", gm, n, n, dF, gm, S1, V1, n, gm, atype)
            torch.cuda.synchronize()
            results[case].update({"vexp0_single": v1[0].cpu().numpy(), "C_single": C1.cpu().numpy(), "rank_single": r1, "S_single": S1.cpu().numpy()})
            h1.destroy()
        dist.barrier()                                   # nobody tears anything down while a peer is still computing
        h.destroy()
    np.save(path_out + f".rank{rank}.npy", results, allow_pickle=True)
    torch.cuda.synchronize()
    dist.barrier()
    nccl.ncclCommDestroy(comm)
    dist.destroy_process_group()


def test_two_gpu_row_split_equals_single_gpu(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = str(tmp_path / "res")
    port = 29700 + os.getpid() % 200
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=600)
        assert p.exitcode == 0
    r0 = np.load(out + ".rank0.npy", allow_pickle=True).item()
    r1 = np.load(out + ".rank1.npy", allow_pickle=True).item()
    for case in r0:
        a, b = r0[case], r1[case]
        assert np.array_equal(a["vexp0"], b["vexp0"]) and np.array_equal(a["vexp0"], a["vexp0_single"])
        assert np.array_equal(a["C"], b["C"]), "ranks hold different sums"
        assert np.array_equal(a["C"], a["C_single"]), "distributed Gram differs from the single-GPU Gram"
        assert a["rank"] == b["rank"] == a["rank_single"]
        tol = 1e-12 if a["S"].dtype == np.float64 else 1e-5
        assert np.max(np.abs(a["S"] - a["S_single"])) <= tol * a["S_single"][0]
        assert np.array_equal(a["S"], b["S"])
