"""GPU: Full-size shapes of the benchmark configurations.  The oracle checks sampled rows bit-for-bit (rows of a
quantized linear are independent), and whole outputs are checked through
properties that need no oracle: splitting rows or columns, or permuting rows,
must not change a single bit.
"""
import numpy as np
import pytest

from util import bits_equal, max_rel_err, packed_weights

pytestmark = pytest.mark.gpu


def _sampled_rows_exact(sdq, oracle, w, wq, ws, A, out, rng, n=48):
    rows = np.sort(rng.choice(A.shape[0], n, replace=False))
    rows[0], rows[-1] = 0, A.shape[0] - 1           # include the edges of the M range
    want = oracle.qgemm(A[rows], wq, ws)
    assert bits_equal(out[rows], want)


def test_config2_ffn_pair_m4096(sdq, oracle):
    """M=4096: 3072->14336, GELU-tanh, 14336->3072; activations N(0,1)*0.5."""
    rng = np.random.default_rng(2)
    M, D, F = 4096, 3072, 14336
    A = (rng.standard_normal((M, D)) * 0.5).astype(np.float32)
    w1q, w1s = packed_weights(rng, F, D, oracle)
    w2q, w2s = packed_weights(rng, D, F, oracle)
    b1 = (rng.standard_normal(F) * 0.02).astype(np.float32)
    b2 = (rng.standard_normal(D) * 0.02).astype(np.float32)
    w1, w2 = sdq.weight_upload(w1q, w1s), sdq.weight_upload(w2q, w2s)

    # each GEMM alone, exact, on sampled rows
    h_gpu = sdq.qgemm_host(w1, A)
    _sampled_rows_exact(sdq, oracle, w1, w1q, w1s, A, h_gpu, rng)
    # second GEMM fed with the CPU's intermediate so that the comparison stays bit-exact
    rows = np.sort(rng.choice(M, 32, replace=False))
    h_cpu = oracle.gelu_tanh(oracle.bias_add(oracle.qgemm(A[rows], w1q, w1s), b1))
    y_cpu = oracle.bias_add(oracle.qgemm(h_cpu, w2q, w2s), b2)
    assert bits_equal(sdq.qgemm_host(w2, h_cpu, bias=b2), y_cpu)

    # the chained pair with the fused epilogues: within 1e-3 of the CPU chain
    h = sdq.qgemm_host(w1, A[rows], bias=b1, gelu=True)
    y = sdq.qgemm_host(w2, h, bias=b2)
    assert max_rel_err(y, y_cpu) < 1e-3
    sdq.weight_release(w1)
    sdq.weight_release(w2)


@pytest.mark.parametrize("K,N", [(3072, 3072), (3072, 9216), (3072, 14336), (14336, 3072)])
def test_config3_linears_m27280(sdq, oracle, K, N):
    """The video-branch linears at 720p/121 frames: M = 22*40*31 = 27280 (213 tiles + 16 rows)."""
    rng = np.random.default_rng(K + N)
    M = 27280
    A = rng.standard_normal((M, K)).astype(np.float32)
    wq, ws = packed_weights(rng, N, K, oracle)
    w = sdq.weight_upload(wq, ws)
    out = sdq.qgemm_host(w, A)
    _sampled_rows_exact(sdq, oracle, w, wq, ws, A, out, rng)

    # row split (the multi-GPU M-split) and an unaligned split: identical bits
    cut = 13 * 128
    assert bits_equal(sdq.qgemm_host(w, A[:cut]), out[:cut])
    assert bits_equal(sdq.qgemm_host(w, A[20001:20900]), out[20001:20900])
    # column split (the multi-GPU N-split): a weight slice gives the same columns
    n0, n1 = N // 2 - 96, N // 2 + 160
    wpart = sdq.weight_upload(wq[n0:n1], ws[n0:n1])
    assert bits_equal(sdq.qgemm_host(wpart, A[:4000]), out[:4000, n0:n1])
    # row permutation equivariance
    perm = rng.permutation(2048)
    assert bits_equal(sdq.qgemm_host(w, A[perm]), out[perm])
    sdq.weight_release(w)
    sdq.weight_release(wpart)


def test_cross_attention_kv_m512_and_adaln(sdq, oracle):
    """K/V projections over 512 text tokens and the 3072->18432 modulation projection."""
    rng = np.random.default_rng(77)
    for (M, K, N) in [(512, 3072, 3072), (1024, 3072, 18432)]:
        A = rng.standard_normal((M, K)).astype(np.float32)
        wq, ws = packed_weights(rng, N, K, oracle)
        w = sdq.weight_upload(wq, ws)
        out = sdq.qgemm_host(w, A)
        _sampled_rows_exact(sdq, oracle, w, wq, ws, A, out, rng, n=24)
        sdq.weight_release(w)


def test_fused_qkv_equals_three_calls(sdq, oracle):
    """N=9216 as the row-concatenation of q, k, v: same bits as three separate linears,
    with the activations quantized once (the reference quantizes x three times)."""
    rng = np.random.default_rng(31)
    M, D = 1500, 3072
    A = rng.standard_normal((M, D)).astype(np.float32)
    parts = [packed_weights(rng, D, D, oracle) for _ in range(3)]
    wcat = sdq.weight_upload(np.concatenate([p[0] for p in parts]), np.concatenate([p[1] for p in parts]))
    fused = sdq.qgemm_host(wcat, A)
    for i, (q, s) in enumerate(parts):
        w = sdq.weight_upload(q, s)
        assert bits_equal(sdq.qgemm_host(w, A), fused[:, i * D:(i + 1) * D])
        sdq.weight_release(w)
    sdq.weight_release(wcat)


def test_ffn_pair_entry_point(sdq, pkg, oracle):
    """sdq_ffn_pair (fc1 -> GELU -> fc2): the chunked host-pointer pipeline and the device
    path give the same bits as two sdq_qgemm calls, and stay within 1e-3 of the CPU chain."""
    rng = np.random.default_rng(55)
    M, D, F = 9000, 512, 1024                       # 3 chunks of 4096 rows, the last one partial
    x = (rng.standard_normal((M, D)) * 0.5).astype(np.float32)
    w1q, w1s = packed_weights(rng, F, D, oracle)
    w2q, w2s = packed_weights(rng, D, F, oracle)
    b1 = (rng.standard_normal(F) * 0.02).astype(np.float32)
    b2 = (rng.standard_normal(D) * 0.02).astype(np.float32)
    w1, w2 = sdq.weight_upload(w1q, w1s), sdq.weight_upload(w2q, w2s)
    y_pipe = sdq.ffn_pair_host(w1, b1, w2, b2, x)
    h = sdq.qgemm_host(w1, x, bias=b1, gelu=True)
    y_two = sdq.qgemm_host(w2, h, bias=b2)
    assert bits_equal(y_pipe, y_two)
    # device pointers, hidden activations returned
    dx, db1, db2 = sdq.to_device(x), sdq.to_device(b1), sdq.to_device(b2)
    dh, dy = sdq.alloc(M * F * 4), sdq.alloc(M * D * 4)
    sdq._ck(sdq.lib.sdq_ffn_pair(w1, db1.ptr, w2, db2.ptr, dx.ptr, M, dh.ptr, dy.ptr, pkg.sdq.SYNC, None))
    assert bits_equal(dy.to_numpy(np.float32, (M, D)), y_two)
    assert bits_equal(dh.to_numpy(np.float32, (M, F)), h)
    # against the CPU chain (GELU is the only inexact step): 1e-3 of the output's max
    rows = np.sort(rng.choice(M, 256, replace=False))
    h_cpu = oracle.gelu_tanh(oracle.bias_add(oracle.qgemm(x[rows], w1q, w1s), b1))
    y_cpu = oracle.bias_add(oracle.qgemm(h_cpu, w2q, w2s), b2)
    assert max_rel_err(y_pipe[rows], y_cpu) < 1e-3
    # mismatched widths and mixed host/device pointers are rejected
    with pytest.raises(pkg.SdqError):
        sdq._ck(sdq.lib.sdq_ffn_pair(w1, None, w1, None, dx.ptr, M, None, dy.ptr, 0, None))
    with pytest.raises(pkg.SdqError):
        sdq._ck(sdq.lib.sdq_ffn_pair(w1, None, w2, None, dx.ptr, M, None, dy.ptr, pkg.sdq.A_HOST, None))
    sdq.weight_release(w1)
    sdq.weight_release(w2)


def test_column_split_fused_stores_on_one_gpu(sdq, pkg, oracle):
    """sdq_qgemm_colsplit, the multi-GPU column split with the exchange fused into the GEMM
    epilogue, exercised on one GPU: two "ranks" each own half of the weight rows and store
    their column block into both of two [M, N] buffers (here both local; on several GPUs the
    second is a peer's, mapped through CUDA IPC).  Every buffer must end up with the bits of
    the unsplit linear."""
    rng = np.random.default_rng(91)
    M, K, N = 5000, 1024, 1088                      # 1088 = 544 + 544: blocks of 17 x 32 columns
    A = rng.standard_normal((M, K)).astype(np.float32)
    wq, ws = packed_weights(rng, N, K, oracle)
    b = (rng.standard_normal(N) * 0.02).astype(np.float32)
    full = sdq.weight_upload(wq, ws)
    want = sdq.qgemm_host(full, A, bias=b)
    rows = np.sort(rng.choice(M, 40, replace=False))
    assert bits_equal(want[rows], oracle.bias_add(oracle.qgemm(A[rows], wq, ws), b))
    dA, db = sdq.to_device(A), sdq.to_device(b)
    outs = [sdq.alloc(M * N * 4), sdq.alloc(M * N * 4)]
    for o in outs:
        sdq._ck(sdq.lib.sdq_memset(o.ptr, 0xFF, M * N * 4, None))
    for r in range(2):
        n0, n1 = pkg.sharding.col_shard(N, 2, r)
        w = sdq.weight_upload(wq[n0:n1], ws[n0:n1])
        sdq.qgemm_colsplit(w, dA.ptr, M, n0, N, [o.ptr for o in outs], db.ptr + 4 * n0, pkg.sdq.SYNC)
        sdq.weight_release(w)
    for o in outs:
        assert bits_equal(o.to_numpy(np.float32, (M, N)), want)
    # a block that neither starts on a multiple of 32 nor ends the matrix is refused
    w = sdq.weight_upload(wq[:40], ws[:40])
    with pytest.raises(pkg.SdqError) as e:
        sdq.qgemm_colsplit(w, dA.ptr, M, 0, N, [outs[0].ptr])
    assert e.value.code == 1
    sdq.weight_release(w)
    sdq.weight_release(full)


def test_random_shapes_match_oracle(sdq, oracle):
    """Seeded random (M, K, N), odd sizes and alignments included: whole outputs exact."""
    rng = np.random.default_rng(2024)
    for _ in range(24):
        M = int(rng.integers(1, 700))
        K = int(rng.choice([int(rng.integers(1, 300)), 16 * int(rng.integers(1, 80)), 128 * int(rng.integers(1, 30))]))
        N = int(rng.choice([int(rng.integers(1, 300)), 4 * int(rng.integers(1, 200)), 32 * int(rng.integers(1, 40))]))
        A = (rng.standard_normal((M, K)) * float(rng.choice([1e-3, 1.0, 50.0]))).astype(np.float32)
        wq, ws = packed_weights(rng, N, K, oracle)
        bias = (rng.standard_normal(N) * 0.02).astype(np.float32) if rng.integers(2) else None
        w = sdq.weight_upload(wq, ws)
        want = oracle.qgemm(A, wq, ws)
        if bias is not None:
            want = oracle.bias_add(want, bias)
        got = sdq.qgemm_host(w, A, bias=bias)
        assert bits_equal(got, want), (M, K, N)
        sdq.weight_release(w)
