"""CPU, world_size 2, gloo: the host-side logic of the multi-GPU paths.

The partition arithmetic, the gather/assembly of column blocks and of row blocks, and
the max-over-ranks reduction run as two real ranks; the CPU oracle stands in for the
device GEMM (a checker of the plumbing, not a product path)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    try:
        sys.path.insert(0, ROOT)
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        import __graft_entry__ as ge
        from oracle.binding import Oracle
        from util import packed_weights
        pkg = ge.load_package()
        par = pkg.parallel
        orc = Oracle()
        orc.set_threads(2)
        rng = np.random.default_rng(17)                 # same inputs on every rank
        M, K, N = 300, 96, 200                          # N not a multiple of the shard width
        A = rng.standard_normal((M, K)).astype(np.float32)
        wq, ws = packed_weights(rng, N, K, orc)
        full = orc.qgemm(A, wq, ws)

        # column split + all-gather
        n0, n1 = par.local_cols(N)
        block = torch.from_numpy(orc.qgemm(A, wq[n0:n1], ws[n0:n1]))
        out = par.allgather_columns(block, N).numpy()
        ok_cols = out.tobytes() == full.tobytes()

        # row split, no exchange in the data path; gather only to compare
        r0, r1 = par.local_rows(M)
        rows = torch.from_numpy(orc.qgemm(A[r0:r1], wq, ws)) if r1 > r0 else torch.empty((0, N))
        out = par.gather_rows(rows, M).numpy()
        ok_rows = out.tobytes() == full.tobytes()

        slowest = par.max_over_ranks(1.0 + rank)
        dist.barrier()
        dist.destroy_process_group()
        q.put((rank, ok_cols, ok_rows, slowest, (n0, n1), (r0, r1)))
    except Exception as e:  # pragma: no cover
        q.put((rank, "error", repr(e)))


def test_two_ranks_gloo():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for r in res:
        assert r[1] is True and r[2] is True, r
        assert r[3] == 2.0                               # the max over ranks, on every rank
    by_rank = {r[0]: r for r in res}
    assert by_rank[0][4] == (0, 128) and by_rank[1][4] == (128, 200)
    assert by_rank[0][5] == (0, 256) and by_rank[1][5] == (256, 300)


def test_shard_arithmetic(pkg):
    sh = pkg.sharding
    for M in (0, 1, 127, 128, 192, 27280, 54560):
        for world in (1, 2, 4, 8):
            spans = [sh.row_shard(M, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == M
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all(b % 256 == 0 or b == M for b, _ in spans)
            # balanced in whole 256-row tiles: nobody carries more than ceil(tiles / world)
            tiles = [-(-(e - b) // 256) for b, e in spans]
            assert max(tiles) == -(-(-(-M // 256)) // world) and max(tiles) - min(tiles) <= 1
    assert sh.row_shard(27280, 8, 0) == (0, 3584) and sh.row_shard(27280, 8, 3) == (10752, 14080)
    assert sh.row_shard(27280, 8, 7) == (24064, 27280)
    for N in (13, 192, 3072, 14336, 18432):
        for world in (1, 2, 4, 8):
            spans = [sh.col_shard(N, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == N
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    with pytest.raises(ValueError):
        sh.row_shard(10, 2, 2)
