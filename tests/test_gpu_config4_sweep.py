"""GPU: the whole shape sweep of the DiT linears as parity cases.

Every (K, N) of the model -- q/k/v/o 3072->3072, fused QKV 3072->9216, FFN up 3072->14336,
FFN down 14336->3072, modulation 3072->18432 -- at every token count of the sweep, M in
{192, 1024, 4096, 16384, 27280, 54560}.  Inputs and outputs stay on the device; sampled rows
(the first and the last among them) are brought back and compared bit for bit with the CPU
oracle (rows of a quantized linear are independent, reference src/core/qgemm.cpp:84-96).  At
M = 54560 the linear is also run split by output columns into eight blocks through
sdq_qgemm_colsplit (the multi-GPU form, here with one destination buffer on one GPU) and the
assembled [M, N] must equal the unsplit result in every bit.
"""
import ctypes as C

import numpy as np
import pytest

from util import bits_equal, packed_weights

pytestmark = pytest.mark.gpu

SWEEP_KN = [(3072, 3072), (3072, 9216), (3072, 14336), (14336, 3072), (3072, 18432)]
SWEEP_M = [192, 1024, 4096, 16384, 27280, 54560]


def _rows_from_device(sdq, dbuf, N, rows):
    out = np.empty((len(rows), N), np.float32)
    for i, r in enumerate(rows):
        sdq._ck(sdq.lib.sdq_memcpy_d2h(out[i].ctypes.data_as(C.c_void_p), dbuf.ptr + int(r) * N * 4, N * 4, None))
    sdq.sync()
    return out


@pytest.mark.parametrize("K,N", SWEEP_KN)
def test_every_token_count(sdq, pkg, oracle, K, N):
    rng = np.random.default_rng(K * 7 + N)
    Mmax = SWEEP_M[-1]
    A = rng.standard_normal((Mmax, K), dtype=np.float32)
    wq, ws = packed_weights(rng, N, K, oracle)
    w = sdq.weight_upload(wq, ws)
    dA = sdq.to_device(A)
    dout = sdq.alloc(Mmax * N * 4)
    for M in SWEEP_M:
        sdq._ck(sdq.lib.sdq_memset(dout.ptr, 0xff, M * N * 4, None))     # NaN pattern: nothing may be left unwritten
        sdq.qgemm(w, dA.ptr, M, dout.ptr, None, pkg.sdq.SYNC)
        rows = np.sort(rng.choice(M, min(M, 40), replace=False))
        rows[0], rows[-1] = 0, M - 1
        # a tile boundary and the rows around the middle of the range as well
        rows = np.unique(np.concatenate([rows, [min(M - 1, 255), min(M - 1, 256), M // 2]]))
        got = _rows_from_device(sdq, dout, N, rows)
        assert bits_equal(got, oracle.qgemm(A[rows], wq, ws)), (K, N, M)
    # ---- M = 54560 split by columns into 8 blocks: the multi-GPU form on one destination
    M = Mmax
    dsplit = sdq.alloc(M * N * 4)
    sdq._ck(sdq.lib.sdq_memset(dsplit.ptr, 0xff, M * N * 4, None))
    blocks = []
    for r in range(8):
        n0, n1 = pkg.sharding.col_shard(N, 8, r)
        if n1 > n0:
            blocks.append((n0, sdq.weight_upload(wq[n0:n1], ws[n0:n1])))
    for n0, wb in blocks:
        sdq.qgemm_colsplit(wb, dA.ptr, M, n0, N, [dsplit.ptr])
    sdq.sync()
    step = 2048                                                           # compare in slabs: bounded host memory
    for r0 in range(0, M, step):
        r1 = min(M, r0 + step)
        a = np.empty((r1 - r0, N), np.float32)
        b = np.empty((r1 - r0, N), np.float32)
        sdq._ck(sdq.lib.sdq_memcpy_d2h(a.ctypes.data_as(C.c_void_p), dout.ptr + r0 * N * 4, a.nbytes, None))
        sdq._ck(sdq.lib.sdq_memcpy_d2h(b.ctypes.data_as(C.c_void_p), dsplit.ptr + r0 * N * 4, b.nbytes, None))
        sdq.sync()
        assert bits_equal(a, b), (K, N, r0)
    for _, wb in blocks:
        sdq.weight_release(wb)
    sdq.weight_release(w)
    for d in (dA, dout, dsplit):
        d.free()


def test_remaining_linears_of_a_branch(sdq, pkg, oracle):
    """The linears outside the blocks, at the row counts the reference calls them with
    (src/model/ovi_dit.cpp:490-499, :662-700, :298-314): text embedding 4096->3072->3072 on the
    512 padded text rows, time embedding 256->3072->3072 and time projection 3072->18432 on ONE
    row, the video head 3072->192 on every token, and the block linears at the audio branch's
    token count."""
    rng = np.random.default_rng(490)
    cases = [(512, 4096, 3072), (512, 3072, 3072), (1, 256, 3072), (1, 3072, 3072), (1, 3072, 18432),
             (27280, 3072, 192), (157, 3072, 3072), (157, 3072, 9216), (157, 3072, 14336), (157, 14336, 3072)]
    for (M, K, N) in cases:
        A = rng.standard_normal((M, K), dtype=np.float32)
        wq, ws = packed_weights(rng, N, K, oracle)
        w = sdq.weight_upload(wq, ws)
        out = sdq.qgemm_host(w, A)
        rows = np.unique(np.concatenate([[0, M - 1], rng.choice(M, min(M, 64), replace=False)]))
        assert bits_equal(out[rows], oracle.qgemm(A[rows], wq, ws)), (M, K, N)
        sdq.weight_release(w)
