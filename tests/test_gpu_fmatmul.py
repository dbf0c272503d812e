"""GPU: the fp32 linears (sd::matmul behind blk::linear) on the tensor cores.

Three tf32 products per fp32 product remove the 2^-11 input rounding of a plain tf32 GEMM, and
K is accumulated in groups of 256 elements that are added in fp32 registers (the tensor core's
own accumulator truncates, which over one long chain costs ~7e-9 * K): measured about 2e-6 of the
largest output for every K from 36 to 14336 -- the level of an fp32 BLAS.  The reference's own
sums depend on its SIMD / BLAS order and its test gates matmul at max-abs error <= 1e-3 of the
largest output (tests/test_core.cpp:82-84).  Here: that gate against the reference's outputs
(fixtures from the compiled sd::matmul) and the left-to-right restatement, and 4e-6 against a
float64 product.
"""
import os

import numpy as np
import pytest

from util import max_rel_err

pytestmark = pytest.mark.gpu

REF_TOL = 1e-3      # the reference's own gate for matmul


def acc_tol(K):
    """Bound on max-abs error / max-abs output against float64 (independent of K)."""
    return 4e-6


@pytest.fixture(scope="module")
def caller(golden_dir):
    return np.load(os.path.join(golden_dir, "dit_caller.npz"))


def test_matches_reference_fixture(sdq, caller):
    z = caller
    w = sdq.fweight_upload(z["mm_W"])
    for simt in (False, True):
        got = sdq.fmatmul_host(w, z["mm_A"], z["mm_W"].shape[1], bias=z["mm_bias"], force_simt=simt)
        assert max_rel_err(got, z["mm_out"]) < REF_TOL
        assert max_rel_err(got, z["mm_out"]) < 1e-5
    sdq.weight_release(w)
    w = sdq.fweight_upload(z["mm2_W"])                       # K = 31: not a multiple of 4, CUDA cores
    assert max_rel_err(sdq.fmatmul_host(w, z["mm2_A"], 13), z["mm2_out"]) < 1e-5
    sdq.weight_release(w)


@pytest.mark.parametrize("M,K,N", [
    (1, 256, 3072),        # time_embedding.0 at M = 1
    (64, 3072, 3072),
    (300, 3072, 192),      # a head-sized output
    (1000, 140, 3072),     # K = 140: the audio patch embedding as im2col; ragged last k-block
    (129, 36, 130),        # N % 4 != 0: per-thread stores
    (2500, 1024, 640),     # several row tiles per SM
    (4096, 3072, 1024),
    (256, 14336, 512),     # the longest K of the model
])
def test_against_float64_and_restatement(sdq, oracle, M, K, N):
    rng = np.random.default_rng(M + K + N)
    A = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(N) * 0.02).astype(np.float32)
    w = sdq.fweight_upload(W)
    got = sdq.fmatmul_host(w, A, N, bias=b)
    want64 = (A.astype(np.float64) @ W.astype(np.float64) + b).astype(np.float32)
    assert max_rel_err(got, want64) < acc_tol(K)
    if M * K * N <= 2 ** 31:
        assert max_rel_err(got, oracle.matmul_f32(A, W, b)) < REF_TOL
    got_nb = sdq.fmatmul_host(w, A, N)
    assert max_rel_err(got_nb, (A.astype(np.float64) @ W.astype(np.float64)).astype(np.float32)) < acc_tol(K)
    sdq.weight_release(w)


def test_large_dynamic_range_and_exact_small_integers(sdq):
    """Values spanning 2^-20 .. 2^20, and small integers whose products are exact in any order."""
    rng = np.random.default_rng(3)
    M, K, N = 130, 512, 256
    A = (rng.standard_normal((M, K)) * np.exp2(rng.integers(-20, 21, (M, 1)))).astype(np.float32)
    W = (rng.standard_normal((K, N)) * np.exp2(rng.integers(-20, 21, (1, N)))).astype(np.float32)
    w = sdq.fweight_upload(W)
    got = sdq.fmatmul_host(w, A, N)
    want = A.astype(np.float64) @ W.astype(np.float64)
    # row/column scales vary by 2^40: compare element-wise against the size of the terms
    mag = np.abs(A).astype(np.float64) @ np.abs(W).astype(np.float64)
    assert np.max(np.abs(got - want) / mag) < acc_tol(K)
    sdq.weight_release(w)
    Ai = rng.integers(-64, 65, (70, 256)).astype(np.float32)
    Wi = rng.integers(-64, 65, (256, 96)).astype(np.float32)
    w = sdq.fweight_upload(Wi)
    assert np.array_equal(sdq.fmatmul_host(w, Ai, 96), (Ai.astype(np.int64) @ Wi.astype(np.int64)).astype(np.float32))
    sdq.weight_release(w)


def test_handles_are_typed(sdq, pkg, oracle):
    rng = np.random.default_rng(5)
    wf = sdq.fweight_upload(rng.standard_normal((64, 32)).astype(np.float32))
    with pytest.raises(pkg.SdqError):
        sdq.qgemm_host(wf, np.zeros((4, 64), np.float32))          # an fp32 weight is not an int8 one
    wq = sdq.weight_upload(np.zeros((32, 64), np.int8), np.ones(32, np.float32))
    with pytest.raises(pkg.SdqError):
        sdq.fmatmul_host(wq, np.zeros((4, 64), np.float32), 32)
    assert sdq.fmatmul_host(wf, np.zeros((0, 64), np.float32), 32).shape == (0, 32)   # M == 0
    sdq.weight_release(wf)
    sdq.weight_release(wq)


def test_device_pointers_on_a_stream(sdq, pkg):
    """Device-resident A / out / bias on a caller's stream, two calls back to back (the scratch
    planes are per stream and reused)."""
    rng = np.random.default_rng(9)
    M, K, N = 700, 512, 384
    W = (rng.standard_normal((K, N)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(N) * 0.02).astype(np.float32)
    w = sdq.fweight_upload(W)
    st = sdq.stream_create()
    db, dout = sdq.to_device(b), sdq.alloc(M * N * 4)
    for seed in (1, 2):
        A = np.random.default_rng(seed).standard_normal((M, K)).astype(np.float32)
        dA = sdq.to_device(A)
        sdq._ck(sdq.lib.sdq_fmatmul(w, dA.ptr, M, dout.ptr, db.ptr, 0, st))
        sdq.sync(st)
        want = (A.astype(np.float64) @ W.astype(np.float64) + b).astype(np.float32)
        assert max_rel_err(dout.to_numpy(np.float32, (M, N)), want) < acc_tol(K)
    sdq.stream_destroy(st)
    sdq.weight_release(w)
