"""GPU: the residual epilogue (x += y * gate, x += y) and the whole ffn_fwd block.

The fused multiply-add of the gated update is bit-identical to the reference's own build
(fixtures from the compiled src/model/ovi_dit.cpp: tests/golden/dit_caller.npz), on every
kernel and store path; the chained block is held to the 1e-3 bound (its GELU is not
bit-reproducible across math libraries; everything else in it is exact).
"""
import os

import numpy as np
import pytest

from util import bits_equal, max_rel_err, packed_weights

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def caller(golden_dir):
    return np.load(os.path.join(golden_dir, "dit_caller.npz"))


def test_gated_and_plain_residual_match_reference_fixture(sdq, caller):
    z = caller
    w = sdq.weight_upload(z["lin_Bq"], z["lin_bs"])
    for simt in (False, True):
        for inplace in (True, False):
            got = sdq.qgemm_residual_np(w, z["lin_A"], z["lin_x"], z["lin_gate"], z["lin_bias"],
                                        inplace=inplace, force_simt=simt)
            assert bits_equal(got, z["lin_gated"]), (simt, inplace)
            got = sdq.qgemm_residual_np(w, z["lin_A"], z["lin_x"], None, z["lin_bias"],
                                        inplace=inplace, force_simt=simt)
            assert bits_equal(got, z["lin_added"]), (simt, inplace)
    sdq.weight_release(w)


@pytest.mark.parametrize("M,K,N", [
    (300, 512, 640),        # one-CTA kernel, bulk tensor stores
    (129, 144, 257),        # odd N: per-thread stores
    (192, 14336, 3072),     # K split: the finalize pass applies the residual
    (4096, 256, 3072),      # CTA-pair kernel
    (2100, 14336, 3072),    # CTA-pair kernel at the FFN-down shape, ragged last row tile
    (5, 48, 36),
])
def test_residual_matches_oracle_on_every_path(sdq, oracle, M, K, N):
    rng = np.random.default_rng(M + K + N)
    A = rng.standard_normal((M, K)).astype(np.float32)
    wq, ws = packed_weights(rng, N, K, oracle)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float32)
    gate = rng.standard_normal(N).astype(np.float32)
    x = rng.standard_normal((M, N)).astype(np.float32)
    y = oracle.bias_add(oracle.qgemm(A, wq, ws), bias)
    w = sdq.weight_upload(wq, ws)
    assert bits_equal(sdq.qgemm_residual_np(w, A, x, gate, bias, inplace=True), oracle.residual_add(x, y, gate))
    assert bits_equal(sdq.qgemm_residual_np(w, A, x, gate, bias, inplace=False), oracle.residual_add(x, y, gate))
    assert bits_equal(sdq.qgemm_residual_np(w, A, x, None, None, inplace=True),
                      oracle.residual_add(x, oracle.qgemm(A, wq, ws)))
    sdq.weight_release(w)


def test_residual_rejects_bad_arguments(sdq, pkg, oracle):
    rng = np.random.default_rng(2)
    wq, ws = packed_weights(rng, 32, 64, oracle)
    w = sdq.weight_upload(wq, ws)
    d = sdq.alloc(4 * 32 * 4)
    with pytest.raises(pkg.SdqError) as e:
        sdq._ck(sdq.lib.sdq_qgemm_residual(w, d.ptr, 4, None, None, d.ptr, None, 0, None))
    assert e.value.code == 1
    with pytest.raises(pkg.SdqError):
        sdq._ck(sdq.lib.sdq_qgemm_residual(w, d.ptr, 4, d.ptr, None, d.ptr, None, pkg.sdq.A_HOST, None))
    assert sdq.lib.sdq_qgemm_residual(w, d.ptr, 0, d.ptr, None, d.ptr, None, 0, None) == 0   # M == 0
    sdq.weight_release(w)


def test_ffn_block_matches_reference_fixture(sdq, caller):
    z = caller
    e = z["ffn_e"]
    w1, w2 = sdq.weight_upload(z["ffn_q1"], z["ffn_s1"]), sdq.weight_upload(z["ffn_q2"], z["ffn_s2"])
    got = sdq.ffn_block_np(w1, z["ffn_b1"], w2, z["ffn_b2"], z["ffn_x"], e[3], e[4], e[5])
    assert max_rel_err(got, z["ffn_out"]) < 1e-3
    assert max_rel_err(got - z["ffn_x"], z["ffn_out"] - z["ffn_x"]) < 1e-3   # the update itself
    sdq.weight_release(w1)
    sdq.weight_release(w2)


def test_ffn_block_full_width_matches_oracle_chain(sdq, pkg, oracle):
    """DiT widths (3072 -> 14336 -> 3072) on enough rows for the CTA-pair kernel in both linears."""
    rng = np.random.default_rng(77)
    M, D, F = 2100, 3072, 14336
    x = (rng.standard_normal((M, D)) * 1.5 + 0.1).astype(np.float32)
    shift, scale, gate = [(rng.standard_normal(D) * 0.3).astype(np.float32) for _ in range(3)]
    q1, s1 = packed_weights(rng, F, D, oracle)
    q2, s2 = packed_weights(rng, D, F, oracle)
    b1 = (rng.standard_normal(F) * 0.02).astype(np.float32)
    b2 = (rng.standard_normal(D) * 0.02).astype(np.float32)
    w1, w2 = sdq.weight_upload(q1, s1), sdq.weight_upload(q2, s2)
    got = sdq.ffn_block_np(w1, b1, w2, b2, x, shift, scale, gate)
    h = oracle.layernorm_mod(x, shift, scale, 1e-6)
    u = oracle.gelu_tanh(oracle.bias_add(oracle.qgemm(h, q1, s1), b1))
    v = oracle.bias_add(oracle.qgemm(u, q2, s2), b2)
    want = oracle.residual_add(x, v, gate)
    assert max_rel_err(got, want) < 1e-3
    assert max_rel_err(got - x, want - x) < 1e-3          # the update alone (x cancels)
    # With tree sums in the layernorm a few int8 steps of h flip (about 1 % of the rows have
    # one), which two chained int8 linears carry to ~2.5e-3 of the largest update on those rows.
    fast = sdq.ffn_block_np(w1, b1, w2, b2, x, shift, scale, gate, tree_sums=True)
    assert max_rel_err(fast - x, want - x) < 5e-3
    # and the block equals its parts run one by one through the other entry points
    aq, a_s = sdq.layernorm_mod_quantize(x, shift, scale, 1e-6)
    dq, ds = sdq.to_device(aq), sdq.to_device(a_s)
    dh, db1 = sdq.alloc(M * F * 4), sdq.to_device(b1)
    sdq._ck(sdq.lib.sdq_qgemm_prequantized(w1, dq.ptr, ds.ptr, M, dh.ptr, db1.ptr, None,
                                           pkg.sdq.GELU_TANH | pkg.sdq.SYNC, None))
    parts = sdq.qgemm_residual_np(w2, dh.to_numpy(np.float32, (M, F)), x, gate, b2)
    assert bits_equal(got, parts)
    sdq.weight_release(w1)
    sdq.weight_release(w2)
