"""GPU: sdq_qgemm_static_scratch, the entry point for callers that cannot allocate.

Some hosts of this library may not call cudaMalloc while they run: they have handed
all device memory to their own pool, or they sit in a section where the device-wide
synchronisation that cudaMalloc and cudaFree imply would stall other streams.
sdq_qgemm grows a workspace on demand, so it is not for them; the variant tested
here keeps its scratch in a fixed array inside the library image instead.  The
test checks, through the C ABI, that it returns exactly what sdq_qgemm returns --
twice in a row with different inputs, because the array is shared between calls
and keeps the previous call's contents -- and that it refuses sizes beyond its
stated maximum.  The file is named to be collected last.
"""
import numpy as np
import pytest

from util import bits_equal, packed_weights

pytestmark = pytest.mark.gpu


def _both(sdq, pkg, w, wq_ptr, ws_ptr, N, K, A, bias, flags):
    M = A.shape[0]
    dA = sdq.to_device(A)
    db = sdq.to_device(bias) if bias is not None else None
    out_a, out_b = sdq.alloc(M * N * 4), sdq.alloc(M * N * 4)
    bp = db.ptr if db else None
    sdq.qgemm(w, dA.ptr, M, out_a.ptr, bp, flags | pkg.sdq.SYNC)
    sdq.qgemm_static_scratch(wq_ptr, ws_ptr, N, K, dA.ptr, M, out_b.ptr, bp, flags | pkg.sdq.SYNC)
    return out_a.to_numpy(np.float32, (M, N)), out_b.to_numpy(np.float32, (M, N))


def test_static_scratch_matches_qgemm_twice(sdq, pkg, oracle):
    rng = np.random.default_rng(123)
    N, K = 640, 1024
    wq, ws = packed_weights(rng, N, K, oracle)
    w = sdq.weight_upload(wq, ws)
    _, _, wq_ptr, ws_ptr = sdq.weight_info(w)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float32)
    # first call: a larger M, bias + GELU; second call: smaller M, plain -- stale bytes of
    # the first call are still in the array behind the second call's rows
    A1 = rng.standard_normal((700, K)).astype(np.float32)
    a, b = _both(sdq, pkg, w, wq_ptr, ws_ptr, N, K, A1, bias, pkg.sdq.GELU_TANH)
    assert bits_equal(a, b)                      # tolerance 0: same kernels, same bits
    A2 = (rng.standard_normal((333, K)) * 3).astype(np.float32)
    a, b = _both(sdq, pkg, w, wq_ptr, ws_ptr, N, K, A2, None, 0)
    assert bits_equal(a, b)
    assert bits_equal(b, oracle.qgemm(A2, wq, ws))
    # an odd shape goes through the CUDA-core kernel on the same scratch
    wq3, ws3 = packed_weights(rng, 13, 31, oracle)
    w3 = sdq.weight_upload(wq3, ws3)
    _, _, p3, s3 = sdq.weight_info(w3)
    A3 = rng.standard_normal((17, 31)).astype(np.float32)
    a, b = _both(sdq, pkg, w3, p3, s3, 13, 31, A3, None, 0)
    assert bits_equal(a, b)
    sdq.weight_release(w)
    sdq.weight_release(w3)


def test_static_scratch_rejects_oversize_and_host_pointers(sdq, pkg, oracle):
    rng = np.random.default_rng(5)
    wq, ws = packed_weights(rng, 32, 64, oracle)
    w = sdq.weight_upload(wq, ws)
    _, _, wq_ptr, ws_ptr = sdq.weight_info(w)
    d = sdq.alloc(1024)
    with pytest.raises(pkg.SdqError) as e:     # too many rows
        sdq.qgemm_static_scratch(wq_ptr, ws_ptr, 32, 64, d.ptr, pkg.sdq.STATIC_MAX_ROWS + 1, d.ptr)
    assert e.value.code == 1 and "exceeds the fixed scratch" in e.value.msg
    with pytest.raises(pkg.SdqError) as e:     # M*K too large
        sdq.qgemm_static_scratch(wq_ptr, ws_ptr, 32, 14336, d.ptr, 4096, d.ptr)
    assert e.value.code == 1 and "exceeds the fixed scratch" in e.value.msg
    with pytest.raises(pkg.SdqError) as e:     # host pointers would need staging
        sdq.qgemm_static_scratch(wq_ptr, ws_ptr, 32, 64, d.ptr, 4, d.ptr, None, pkg.sdq.A_HOST)
    assert e.value.code == 1
    sdq.weight_release(w)


@pytest.mark.parametrize("M,K,N", [(32768, 1024, 256),      # M at its limit AND M*K at its limit: the array's last byte is used
                                   (16384, 2048, 512),      # M*K at its limit with fewer rows
                                   (32768, 16, 32)])        # M at its limit, one k-block
def test_static_scratch_at_its_limits(sdq, pkg, oracle, M, K, N):
    """Exactly at SDQ_STATIC_MAX_ROWS and SDQ_STATIC_MAX_AQ_BYTES (where an off-by-one in the
    array's size or in the offsets of its parts would show), through the 2-CTA kernel where the
    shape has enough tiles: the CPU oracle's bits on sampled rows including the last one, and
    sdq_qgemm's bits everywhere; one row or one byte more is refused."""
    assert M <= pkg.sdq.STATIC_MAX_ROWS and M * K <= pkg.sdq.STATIC_MAX_AQ_BYTES
    assert M == pkg.sdq.STATIC_MAX_ROWS or M * K == pkg.sdq.STATIC_MAX_AQ_BYTES
    rng = np.random.default_rng(M + K)
    A = rng.standard_normal((M, K), dtype=np.float32)
    wq, ws = packed_weights(rng, N, K, oracle)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float32)
    w = sdq.weight_upload(wq, ws)
    _, _, wq_ptr, ws_ptr = sdq.weight_info(w)
    for flags in (0, 0):                           # twice: the second call finds the first one's bytes in the array
        a, b = _both(sdq, pkg, w, wq_ptr, ws_ptr, N, K, A, bias, flags)
        assert bits_equal(a, b)
    rows = np.unique(np.concatenate([[0, M - 1, M - 2, M // 2], rng.choice(M, 61, replace=False)]))
    assert bits_equal(b[rows], oracle.bias_add(oracle.qgemm(A[rows], wq, ws), bias))
    dA = sdq.to_device(A[:8])
    d = sdq.alloc(1024)
    with pytest.raises(pkg.SdqError) as e:         # one row more
        sdq.qgemm_static_scratch(wq_ptr, ws_ptr, N, K, dA.ptr, M + 1, d.ptr)
    assert e.value.code == 1 and "exceeds the fixed scratch" in e.value.msg
    sdq.weight_release(w)
