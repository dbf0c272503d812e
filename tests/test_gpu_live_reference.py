"""GPU against the reference's own compiled code, run side by side on the same inputs.

oracle/_ref/libsdref.so is the reference's sd::qgemm, sd::matmul, blk::sdpa and the caller-side
helpers of its ovi_dit.cpp, compiled from its sources; where it is present (it travels with the
repository's built files) these tests compare the CUDA path with it directly, at sizes beyond the
committed fixtures.  They skip where the library is absent.
"""
import numpy as np
import pytest

from util import bits_equal, max_rel_err, packed_weights

pytestmark = pytest.mark.gpu


def test_qgemm_with_bias_pass_is_bit_identical_to_mlin(sdq, reference, oracle):
    rng = np.random.default_rng(101)
    for (M, K, N) in [(700, 3072, 1024), (2100, 1024, 3072)]:       # both sides of the M >= 2048 branch
        A = rng.standard_normal((M, K)).astype(np.float32)
        wq, ws = packed_weights(rng, N, K, oracle)
        b = (rng.standard_normal(N) * 0.02).astype(np.float32)
        w = sdq.weight_upload(wq, ws)
        assert bits_equal(sdq.qgemm_host(w, A, bias=b), reference.mlin_i8(A, wq, ws, b))
        sdq.weight_release(w)


def test_gated_residual_is_bit_identical_to_the_compiled_helpers(sdq, reference, oracle):
    rng = np.random.default_rng(102)
    M, K, N = 900, 3072, 3072
    A = rng.standard_normal((M, K)).astype(np.float32)
    wq, ws = packed_weights(rng, N, K, oracle)
    b = (rng.standard_normal(N) * 0.02).astype(np.float32)
    gate = rng.standard_normal(N).astype(np.float32)
    x = rng.standard_normal((M, N)).astype(np.float32)
    y = reference.mlin_i8(A, wq, ws, b)
    w = sdq.weight_upload(wq, ws)
    assert bits_equal(sdq.qgemm_residual_np(w, A, x, gate, b), reference.gated_add(x, y, gate))
    assert bits_equal(sdq.qgemm_residual_np(w, A, x, None, b), reference.add(x, y))
    sdq.weight_release(w)


def test_ffn_block_against_the_compiled_ffn_fwd(sdq, reference, oracle):
    """The reference's whole ffn_fwd at the DiT widths; exact here up to the GELU."""
    rng = np.random.default_rng(103)
    M, D, F = 512, 3072, 14336
    x = (rng.standard_normal((M, D)) * 1.5 + 0.1).astype(np.float32)
    e = (rng.standard_normal((6, D)) * 0.3).astype(np.float32)
    q1, s1 = packed_weights(rng, F, D, oracle)
    q2, s2 = packed_weights(rng, D, F, oracle)
    b1 = (rng.standard_normal(F) * 0.02).astype(np.float32)
    b2 = (rng.standard_normal(D) * 0.02).astype(np.float32)
    want = reference.ffn_fwd(x, e, q1, s1, b1, q2, s2, b2)
    w1, w2 = sdq.weight_upload(q1, s1), sdq.weight_upload(q2, s2)
    got = sdq.ffn_block_np(w1, b1, w2, b2, x, e[3], e[4], e[5])
    assert max_rel_err(got, want) < 1e-3
    assert max_rel_err(got - x, want - x) < 1e-3
    sdq.weight_release(w1)
    sdq.weight_release(w2)


def test_layernorm_quantize_feeds_the_same_bytes_as_the_compiled_chain(sdq, reference, oracle):
    rng = np.random.default_rng(104)
    M, K = 777, 3072
    x = (rng.standard_normal((M, K)) * 2 + 0.3).astype(np.float32)
    shift = (rng.standard_normal(K) * 0.5).astype(np.float32)
    scale = (rng.standard_normal(K) * 0.1).astype(np.float32)
    h_ref = reference.mod_rows(reference.layernorm(x, 1e-6), shift, scale)
    aq, a_s, h = sdq.layernorm_mod_quantize(x, shift, scale, 1e-6, want_h=True)
    assert bits_equal(h, h_ref)
    aq_c, as_c = oracle.act_quant_rows(h_ref)
    assert bits_equal(aq, aq_c) and bits_equal(a_s, as_c)
    w = (1 + rng.standard_normal(K) * 0.2).astype(np.float32)
    b = (rng.standard_normal(K) * 0.3).astype(np.float32)
    _, _, h2 = sdq.layernorm_mod_quantize(x, b, w, 1e-6, want_h=True, affine=True)
    assert bits_equal(h2, reference.layernorm_affine(x, w, b, 1e-6))


def test_matmul_and_attention_against_the_compiled_reference(sdq, reference):
    rng = np.random.default_rng(105)
    A = rng.standard_normal((300, 3072)).astype(np.float32)
    W = (rng.standard_normal((3072, 640)) * 0.05).astype(np.float32)
    b = (rng.standard_normal(640) * 0.02).astype(np.float32)
    w = sdq.fweight_upload(W)
    assert max_rel_err(sdq.fmatmul_host(w, A, 640, bias=b), reference.matmul(A, W, b)) < 1e-5
    sdq.weight_release(w)
    heads = 4
    q = rng.standard_normal((600, heads * 128)).astype(np.float32)
    k = rng.standard_normal((1500, heads * 128)).astype(np.float32)
    v = rng.standard_normal((1500, heads * 128)).astype(np.float32)
    assert max_rel_err(sdq.sdpa_np(q, k, v, heads), reference.sdpa(q, k, v, heads)) < 1e-4
