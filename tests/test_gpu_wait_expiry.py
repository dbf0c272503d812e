"""GPU: the time-out path of the tensor-core kernels, made to run without anything being stuck.

Every barrier wait of the GEMM / attention kernels is bounded; when one gives up, the kernel
records a code in the library's status word, raises its abort flag and returns, and the host
reports SDQ_ERR_DEVICE_TIMEOUT at the next synchronisation.  `sdq_selftest_wait_expiry` runs that
same wait on a barrier nothing arrives on, with a limit of a few milliseconds: the wait runs
out by itself, no kernel hangs, and the host side of the path (status word read and cleared, the
error and its code, scratch accumulators re-zeroed, context usable) is what these tests check.
"""
import time

import numpy as np
import pytest

from util import bits_equal, packed_weights

pytestmark = pytest.mark.gpu


def test_wait_runs_out_and_is_reported_once(sdq, pkg):
    t0 = time.time()
    out = sdq.selftest_wait_expiry(20)
    with pytest.raises(pkg.SdqError) as e:
        sdq.sync()
    assert e.value.code == pkg.sdq.ERR_DEVICE_TIMEOUT
    assert "0x%x" % pkg.sdq.SELFTEST_WAIT_CODE in e.value.msg
    assert time.time() - t0 < 2.0                     # ~20 ms of waiting, not the kernels' 2 s
    # bit 0: the wait was satisfied (never); bit 1: the abort flag was raised for the other roles
    assert int(out.to_numpy(np.int32, (1,))[0]) == 2
    sdq.sync()                                        # reported once: the word is clear again


def test_argument_checks(sdq, pkg):
    d = sdq.alloc(4)
    for bad in (0, -5, 1001):
        assert sdq.lib.sdq_selftest_wait_expiry(bad, d.ptr, None) == 1      # SDQ_ERR_INVALID
    assert sdq.lib.sdq_selftest_wait_expiry(10, None, None) == 1
    sdq.sync()                                        # nothing was launched


def test_library_keeps_working_after_a_time_out(sdq, pkg, oracle):
    """A shape that uses the shared last wave (its scratch accumulators must be all zero between
    launches): after a reported time-out the scratch is cleared again before its next use and
    the results are the oracle's bits, on the default stream and on a stream of its own."""
    rng = np.random.default_rng(77)
    M, K, N = 3410, 14336, 3072                       # 168 pair-tiles on 74 pairs: a shared last wave
    A = rng.standard_normal((M, K), dtype=np.float32)
    wq, ws = packed_weights(rng, N, K, oracle)
    w = sdq.weight_upload(wq, ws)
    want = oracle.qgemm(A, wq, ws)
    assert bits_equal(sdq.qgemm_host(w, A), want)
    sdq.selftest_wait_expiry(5)
    with pytest.raises(pkg.SdqError):
        sdq.sync()
    n0 = sdq.launches()
    assert bits_equal(sdq.qgemm_host(w, A), want)
    assert sdq.launches() - n0 == 3                   # quantize, GEMM, the pass over the shared tiles
    st = sdq.stream_create()
    sdq.selftest_wait_expiry(5, stream=st)
    with pytest.raises(pkg.SdqError) as e:
        sdq.sync(st)
    assert e.value.code == pkg.sdq.ERR_DEVICE_TIMEOUT
    assert bits_equal(sdq.qgemm_host(w, A), want)
    sdq.stream_destroy(st)
    sdq.weight_release(w)


def test_a_synchronous_call_reports_an_earlier_time_out(sdq, pkg, oracle):
    """A time-out recorded by an earlier launch surfaces at the next call that synchronises (here
    a host-pointer GEMM), which fails instead of returning numbers from a poisoned run; the call
    after it succeeds."""
    rng = np.random.default_rng(78)
    M, K, N = 200, 256, 384
    A = rng.standard_normal((M, K), dtype=np.float32)
    wq, ws = packed_weights(rng, N, K, oracle)
    w = sdq.weight_upload(wq, ws)
    sdq.selftest_wait_expiry(5)
    with pytest.raises(pkg.SdqError) as e:
        sdq.qgemm_host(w, A)
    assert e.value.code == pkg.sdq.ERR_DEVICE_TIMEOUT
    assert bits_equal(sdq.qgemm_host(w, A), oracle.qgemm(A, wq, ws))
    sdq.weight_release(w)
