"""GPU: scale, bias and gate vectors that are only 4-byte aligned.

The fast epilogues of the tensor-core kernels read the weight scales, the bias and the gate four
floats at a time.  A caller may well pass a slice of a larger vector -- the bias of q inside a
fused q/k/v bias, one row of a modulation table at an odd offset -- whose address is a multiple
of 4 but not of 16.  Such calls must take the per-element epilogue and give the oracle's bits;
only the column-split form, which has no other kernel, refuses them (with a message that says
which pointer it is).
"""
import numpy as np
import pytest

from util import bits_equal, packed_weights

pytestmark = pytest.mark.gpu


def _offset_vec(sdq, v, floats=1):
    """Device copy of v that starts `floats` floats into a 256-byte aligned allocation."""
    buf = sdq.to_device(np.concatenate([np.zeros(floats, np.float32), v.astype(np.float32)]))
    return buf, buf.ptr + 4 * floats


@pytest.mark.parametrize("M,K,N", [(300, 512, 384), (20000, 1024, 2048)])   # 1-CTA kernel; enough tiles for the 2-CTA kernel
def test_offset_bias_scale_and_gate(sdq, pkg, oracle, M, K, N):
    rng = np.random.default_rng(M + N)
    A = rng.standard_normal((M, K), dtype=np.float32)
    wq, ws = packed_weights(rng, N, K, oracle)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float32)
    gate = rng.standard_normal(N).astype(np.float32)
    x = rng.standard_normal((M, N), dtype=np.float32)
    y = oracle.bias_add(oracle.qgemm(A, wq, ws), bias)
    dA, dout = sdq.to_device(A), sdq.alloc(M * N * 4)
    dq = sdq.to_device(wq)
    keep_s, s_ptr = _offset_vec(sdq, ws, 3)
    keep_b, b_ptr = _offset_vec(sdq, bias, 1)
    keep_g, g_ptr = _offset_vec(sdq, gate, 2)
    assert s_ptr % 16 == 12 and b_ptr % 16 == 4 and g_ptr % 16 == 8
    w = sdq.weight_wrap_device(dq.ptr, s_ptr, N, K)
    sdq.qgemm(w, dA.ptr, M, dout.ptr, b_ptr, pkg.sdq.SYNC)
    assert bits_equal(dout.to_numpy(np.float32, (M, N)), y)
    # the same through the no-allocation entry point (raw pointers)
    sdq.qgemm_static_scratch(dq.ptr, s_ptr, N, K, dA.ptr, M, dout.ptr, b_ptr, pkg.sdq.SYNC)
    assert bits_equal(dout.to_numpy(np.float32, (M, N)), y)
    # gated residual with an offset gate; aligned scales this time, so only the gate is odd
    w2 = sdq.weight_upload(wq, ws)
    dx = sdq.to_device(x)
    sdq._ck(sdq.lib.sdq_qgemm_residual(w2, dA.ptr, M, dx.ptr, g_ptr, dx.ptr, b_ptr, pkg.sdq.SYNC, None))
    assert bits_equal(dx.to_numpy(np.float32, (M, N)), oracle.residual_add(x, y, gate))
    # the column-split form has only the bulk-store epilogue: it says no, and says why
    with pytest.raises(pkg.SdqError) as e:
        sdq.qgemm_colsplit(w2, dA.ptr, M, 0, N, [dout.ptr], b_ptr)
    assert e.value.code == 1 and "bias" in e.value.msg
    with pytest.raises(pkg.SdqError) as e:
        sdq.qgemm_colsplit(w, dA.ptr, M, 0, N, [dout.ptr])
    assert e.value.code == 1 and "scales" in e.value.msg
    sdq.weight_release(w)
    sdq.weight_release(w2)
