"""GPU, 2 ranks, NCCL: row split (no exchange) and column split + all-gather give the
single-GPU bits.  Skipped on a box with one GPU."""
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpu_count():
    import ctypes
    try:
        n = ctypes.c_int(0)
        lib = ctypes.CDLL("libcuda.so.1")
        if lib.cuInit(0) != 0 or lib.cuDeviceGetCount(ctypes.byref(n)) != 0:
            return 0
        return n.value
    except OSError:
        return 0


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    try:
        import torch
        import torch.distributed as dist
        sys.path.insert(0, ROOT)
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        import __graft_entry__ as ge
        from oracle.binding import Oracle
        from util import packed_weights
        pkg = ge.load_package()
        par, S = pkg.parallel, pkg.sdq
        s = pkg.Sdq(rank)
        orc = Oracle()
        rng = np.random.default_rng(23)
        M, K, N = 3000, 1024, 1536
        A = rng.standard_normal((M, K)).astype(np.float32)
        wq, ws = packed_weights(rng, N, K, orc)
        rows = np.sort(rng.choice(M, 64, replace=False))
        want_rows = orc.qgemm(A[rows], wq, ws)
        dA = torch.from_numpy(A).cuda()
        sp = torch.cuda.current_stream().cuda_stream

        # column split: this rank's weight rows only, then all-gather of the column blocks
        n0, n1 = par.local_cols(N)
        w = s.weight_upload(wq[n0:n1], ws[n0:n1])
        block = torch.empty((M, n1 - n0), device="cuda", dtype=torch.float32)
        s.qgemm(w, dA.data_ptr(), M, block.data_ptr(), None, 0, sp)
        full = par.allgather_columns(block, N)
        torch.cuda.synchronize()
        ok_cols = full[torch.from_numpy(rows).cuda()].cpu().numpy().tobytes() == want_rows.tobytes()

        # the same column split with the exchange fused into the GEMM epilogue: every rank's
        # block is stored straight into every rank's [M, N] buffer over NVLink
        shared = par.SharedOutput(s, M * N * 4)
        par.qgemm_colsplit_fused(s, w, dA.data_ptr(), M, N, shared, stream=sp)
        s.sync(sp)
        dist.barrier()
        fused = shared.local.to_numpy(np.float32, (M, N))
        ok_cols = ok_cols and fused.tobytes() == full.cpu().numpy().tobytes()
        shared.close()

        # row split: full weights, this rank's rows; gathered only for the comparison
        wf = s.weight_upload(wq, ws)
        r0, r1 = par.local_rows(M)
        mine = torch.empty((r1 - r0, N), device="cuda", dtype=torch.float32)
        s.qgemm(wf, dA[r0:r1].data_ptr(), r1 - r0, mine.data_ptr(), None, 0, sp)
        allrows = par.gather_rows(mine, M)
        torch.cuda.synchronize()
        ok_rows = allrows.cpu().numpy().tobytes() == full.cpu().numpy().tobytes()
        s.sync(sp)
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, ok_cols, ok_rows))
    except Exception as e:  # pragma: no cover
        q.put((rank, "error", repr(e)))


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_two_ranks_nccl():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for r in res:
        assert r[1] is True and r[2] is True, r
