"""GPU: the row quantization kernels are bit-identical to the oracle and the golden fixtures.

Everything goes through the C ABI (sdq_quantize_activations, sdq_quantize_rows,
sdq_dequant_rows).
"""
import os

import numpy as np
import pytest

from util import bits_equal, max_rel_err, packed_weights, weights_bf16

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K", [(1, 4), (17, 31), (3, 33), (64, 256), (192, 3072), (130, 4100),
                                 (9, 14336), (5, 18432), (4, 20000), (300, 1000)])
def test_activation_quant_matches_oracle(sdq, oracle, M, K):
    rng = np.random.default_rng(M * 100003 + K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    if M > 2:
        A[1, :] = 0.0                      # zero row: scale 1, bytes 0
        A[2, :] *= 1e-30                   # tiny values
    aq, a_s = sdq.quantize_activations(A)
    aq_c, as_c = oracle.act_quant_rows(A)
    assert bits_equal(a_s, as_c)
    assert bits_equal(aq, aq_c)


def test_activation_quant_ties_and_nonfinite(sdq, oracle):
    A = np.zeros((6, 64), np.float32)
    A[0, 0] = 127.0
    A[0, 1:9] = [0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5, -126.5]   # exact .5 after scaling
    A[1, :] = 1.0
    A[1, 3] = np.nan
    A[2, :] = 2.0
    A[2, 5] = np.inf
    A[3, :] = 1e-45
    A[4, :] = -3.0
    A[4, 7] = -np.inf
    A[5, :] = np.float32(3.4e38)
    aq, a_s = sdq.quantize_activations(A)
    aq_c, as_c = oracle.act_quant_rows(A)
    assert bits_equal(a_s, as_c)
    assert bits_equal(aq, aq_c)
    assert list(aq[0, 1:9]) == [0, 2, 2, 0, -2, -2, 126, -126]      # round half to even


def test_activation_quant_large_rows_sampled(sdq, oracle):
    # the 720p token count at both DiT widths; the oracle checks a sample of rows
    rng = np.random.default_rng(5)
    for K in (3072, 14336):
        M = 27280 if K == 3072 else 4096
        A = rng.standard_normal((M, K)).astype(np.float32)
        aq, a_s = sdq.quantize_activations(A)
        rows = rng.choice(M, 512, replace=False)
        aq_c, as_c = oracle.act_quant_rows(A[rows])
        assert bits_equal(a_s[rows], as_c)
        assert bits_equal(aq[rows], aq_c)
        assert int(np.abs(aq).max()) == 127


def test_packer_rows_match_golden(sdq, pkg, golden_dir):
    z = np.load(os.path.join(golden_dir, "packer_rows.npz"))
    for tag in ("w64x256", "w33x1000", "w8x7"):
        q, s = sdq.quantize_rows(z[tag + "_bf16"], pkg.sdq.BF16, pkg.sdq.MODE_PACKER)
        assert bits_equal(q, z[tag + "_q"]), tag
        assert bits_equal(s, z[tag + "_scale"]), tag
    q, s = sdq.quantize_rows(z["ties_f32"], pkg.sdq.F32, pkg.sdq.MODE_PACKER)
    assert bits_equal(q, z["ties_q"]) and bits_equal(s, z["ties_scale"])
    q, s = sdq.quantize_rows(z["h16x512_f16"], pkg.sdq.F16, pkg.sdq.MODE_PACKER)
    assert bits_equal(q, z["h16x512_q"]) and bits_equal(s, z["h16x512_scale"])


@pytest.mark.parametrize("rows,last", [(3072, 3072), (1000, 14336), (8192, 7), (3072 * 48, 2),
                                       (257, 65), (5, 64)])
def test_packer_rows_match_oracle(sdq, pkg, oracle, rows, last):
    rng = np.random.default_rng(rows + last)
    bits = weights_bf16(rng, rows, last, oracle)
    bits[0, :] = 0
    q, s = sdq.quantize_rows(bits, pkg.sdq.BF16, pkg.sdq.MODE_PACKER)
    q_c, s_c = oracle.quant_rows_packer(oracle.bf16_to_f32(bits))
    assert bits_equal(s, s_c)
    assert bits_equal(q, q_c)


def test_rowwise_matches_golden_and_oracle(sdq, pkg, oracle, golden_dir):
    z = np.load(os.path.join(golden_dir, "qgemm_small.npz"))
    q, s = sdq.quantize_rows(z["rowwise_W"], pkg.sdq.F32, pkg.sdq.MODE_ROWWISE)
    assert bits_equal(q, z["rowwise_q"]) and bits_equal(s, z["rowwise_scale"])
    rng = np.random.default_rng(8)
    W = rng.uniform(-1, 1, (512, 3072)).astype(np.float32)
    W[:, 1] = np.float32(0.5) * np.abs(W).max(axis=1) / np.float32(127.0) * 3   # near-tie values
    q, s = sdq.quantize_rows(W, pkg.sdq.F32, pkg.sdq.MODE_ROWWISE)
    q_c, s_c = oracle.quantize_rowwise(W)
    assert bits_equal(q, q_c) and bits_equal(s, s_c)
    # the two recipes really differ (half-away vs half-even, divide vs multiply)
    t = np.zeros((1, 64), np.float32)
    t[0, 0], t[0, 1] = 127.0, 0.5
    qa, _ = sdq.quantize_rows(t, pkg.sdq.F32, pkg.sdq.MODE_ROWWISE)
    qb, _ = sdq.quantize_rows(t, pkg.sdq.F32, pkg.sdq.MODE_PACKER)
    assert qa[0, 1] == 1 and qb[0, 1] == 0


def test_rowwise_rejects_non_f32(sdq, pkg):
    with pytest.raises(pkg.SdqError) as e:
        sdq.quantize_rows(np.zeros((2, 8), np.uint16), pkg.sdq.BF16, pkg.sdq.MODE_ROWWISE)
    assert e.value.code == 1


def test_dequant_rows(sdq, oracle):
    rng = np.random.default_rng(2)
    q = rng.integers(-127, 128, (100, 77)).astype(np.int8)
    s = rng.uniform(1e-4, 1e-2, 100).astype(np.float32)
    assert bits_equal(sdq.dequant_rows(q, s), oracle.dequant_rows(q, s))
    # the reference's own gate for the weight quantizer: |w - q*s| < 1 scale unit
    W = rng.uniform(-1, 1, (37, 513)).astype(np.float32)
    qq, ss = sdq.quantize_rows(W, 0, 1)
    assert np.all(np.abs(sdq.dequant_rows(qq, ss) - W) < ss[:, None])


@pytest.mark.parametrize("M,K", [(300, 3072), (64, 14336), (1000, 512), (33, 100), (1, 4), (2049, 3072),
                                 (2500, 3072), (2400, 516), (3000, 1024)])   # many rows: one warp per row
def test_fused_layernorm_modulation_quantize_is_exact(sdq, oracle, M, K):
    """LayerNorm + modulation + activation quantization with the reference's left-to-right row
    sums (the default): h, the int8 bytes and the scales are bit-identical to the CPU chain."""
    rng = np.random.default_rng(M + K)
    x = (rng.standard_normal((M, K)) * 2 + 0.3).astype(np.float32)
    if M > 2:
        x[1, :] = 0.25                     # constant row: variance 0, h = shift
        x[2, :] *= 1e-20
    shift = (rng.standard_normal(K) * 0.5).astype(np.float32)
    scale = (rng.standard_normal(K) * 0.1).astype(np.float32)
    aq, a_s, h = sdq.layernorm_mod_quantize(x, shift, scale, 1e-6, want_h=True)
    h_c = oracle.layernorm_mod(x, shift, scale, 1e-6)
    aq_c, as_c = oracle.act_quant_rows(h_c)
    assert bits_equal(h, h_c)
    assert bits_equal(a_s, as_c)
    assert bits_equal(aq, aq_c)


def test_fused_affine_layernorm_quantize_is_exact(sdq, oracle):
    """The layernorm that has a weight and a bias (cross-attention input), SDQ_LN_AFFINE."""
    rng = np.random.default_rng(40)
    for (M, K) in [(512, 3072), (77, 260), (2600, 3072)]:
        x = (rng.standard_normal((M, K)) * 2 + 0.3).astype(np.float32)
        w = (1 + rng.standard_normal(K) * 0.2).astype(np.float32)
        b = (rng.standard_normal(K) * 0.3).astype(np.float32)
        aq, a_s, h = sdq.layernorm_mod_quantize(x, b, w, 1e-6, want_h=True, affine=True)
        h_c = oracle.layernorm_affine(x, w, b, 1e-6)
        aq_c, as_c = oracle.act_quant_rows(h_c)
        assert bits_equal(h, h_c) and bits_equal(a_s, as_c) and bits_equal(aq, aq_c)


@pytest.mark.parametrize("M,K", [(300, 3072), (64, 14336), (1000, 512)])
def test_fused_layernorm_modulation_quantize_tree_sums(sdq, pkg, oracle, M, K):
    """The one-pass variant (SDQ_LN_TREE_SUMS).  The row sums are tree sums while the CPU adds K
    fp32 values left to right (whose own rounding error grows with K), so h is compared under a
    tolerance -- 5e-5 of the row's max -- and an int8 value may differ by one step on a rounding
    boundary; the linear fed with it stays inside the 1e-3 bound."""
    rng = np.random.default_rng(M + K)
    x = (rng.standard_normal((M, K)) * 2 + 0.3).astype(np.float32)
    shift = (rng.standard_normal(K) * 0.5).astype(np.float32)
    scale = (rng.standard_normal(K) * 0.1).astype(np.float32)
    aq, a_s, h = sdq.layernorm_mod_quantize(x, shift, scale, 1e-6, want_h=True, tree_sums=True)
    h_c = oracle.layernorm_mod(x, shift, scale, 1e-6)
    aq_c, as_c = oracle.act_quant_rows(h_c)
    assert np.max(np.abs(h - h_c) / np.max(np.abs(h_c), axis=1, keepdims=True)) < 5e-5
    assert np.max(np.abs(a_s - as_c) / as_c) < 5e-5
    diff = np.abs(aq.astype(np.int32) - aq_c.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 2e-2
    # the quantization itself is exact given the kernel's own h
    aq_h, as_h = oracle.act_quant_rows(h)
    assert bits_equal(aq, aq_h) and bits_equal(a_s, as_h)
    # end to end through the linear: within 1e-3 of the CPU chain
    N = 256
    wq, ws = packed_weights(rng, N, K, oracle)
    w = sdq.weight_upload(wq, ws)
    dq, ds, dout = sdq.to_device(aq), sdq.to_device(a_s), sdq.alloc(M * N * 4)
    sdq._ck(sdq.lib.sdq_qgemm_prequantized(w, dq.ptr, ds.ptr, M, dout.ptr, None, None, pkg.sdq.SYNC, None))
    got = dout.to_numpy(np.float32, (M, N))
    assert max_rel_err(got, oracle.qgemm(h_c, wq, ws)) < 1e-3
    sdq.weight_release(w)
