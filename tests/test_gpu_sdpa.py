"""GPU: exact-softmax attention (blk::sdpa) against the reference's outputs and the restatement.

The reference gates attention like its other fp32 kernels: max-abs error <= 1e-3 of the largest
output.  The tensor-core path splits every operand (times a power of two) into two fp16 numbers
and computes the scores and P*V with three fp16 products per fp32 product; measured errors are
~1e-5 at a few thousand keys and ~1e-4 at 27280 keys (the tensor core's accumulator truncates,
so the error grows with the length of the key range accumulated in it).
"""
import os

import numpy as np
import pytest

from util import bits_equal, max_rel_err

pytestmark = pytest.mark.gpu

TOL = 1e-3


def attention64(q, k, v, heads):
    Lq, C = q.shape
    hd = C // heads
    q64, k64, v64 = [x.astype(np.float64).reshape(-1, heads, hd).transpose(1, 0, 2) for x in (q, k, v)]
    s = q64 @ k64.transpose(0, 2, 1) / np.sqrt(hd)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    return (p @ v64).transpose(1, 0, 2).reshape(Lq, C).astype(np.float32)


def test_matches_reference_fixture(sdq, golden_dir):
    z = np.load(os.path.join(golden_dir, "dit_caller.npz"))
    for simt in (False, True):
        got = sdq.sdpa_np(z["at_q"], z["at_k"], z["at_v"], 3, force_simt=simt)
        assert max_rel_err(got, z["at_out"]) < TOL, simt
        assert max_rel_err(got, z["at_out"]) < (1e-5 if simt else 1e-4), simt


@pytest.mark.parametrize("Lq,Lk,heads", [
    (1, 1, 1),            # one key: the output is that key's value row
    (5, 63, 2), (128, 64, 1), (129, 65, 2), (300, 1000, 2),
    (1024, 512, 24),      # the text cross-attention of a 1024-token tile: all 24 heads
    (2048, 2048, 4),
    (700, 4100, 3),       # many key blocks per row, ragged at both ends
    (1300, 200, 32),      # 352 work items: several per CTA, an odd number of 128-key blocks
    (260, 129, 5),        # three key blocks: the two score-issuing lanes get 2 and 1
])
def test_against_float64(sdq, Lq, Lk, heads):
    rng = np.random.default_rng(Lq + Lk + heads)
    C = heads * 128
    q = rng.standard_normal((Lq, C)).astype(np.float32)
    k = rng.standard_normal((Lk, C)).astype(np.float32)
    v = rng.standard_normal((Lk, C)).astype(np.float32)
    got = sdq.sdpa_np(q, k, v, heads)
    want = attention64(q, k, v, heads)
    assert np.isfinite(got).all()
    assert max_rel_err(got, want) < TOL
    assert max_rel_err(got, want) < 1e-4


def test_peaked_and_shifted_scores(sdq):
    """Large logits (one key dominates a row), a common offset on all keys, and rows whose best
    key sits in the last, ragged key block."""
    rng = np.random.default_rng(8)
    heads, Lq, Lk = 2, 200, 333
    C = heads * 128
    q = (rng.standard_normal((Lq, C)) * 4).astype(np.float32)
    k = (rng.standard_normal((Lk, C)) * 2 + 0.5).astype(np.float32)
    v = rng.standard_normal((Lk, C)).astype(np.float32)
    k[-1] = 3.0 * q[7]                                   # row 7's best key is the very last one
    got = sdq.sdpa_np(q, k, v, heads)
    want = attention64(q, k, v, heads)
    assert np.isfinite(got).all()
    assert max_rel_err(got, want) < TOL


@pytest.mark.parametrize("sq,sk,sv", [
    (1e4, 1e-4, 1e6),       # magnitudes far outside fp16 on every operand
    (1e-6, 1e6, 1e-9),
    (3e-12, 2e-13, 1.0),    # scores ~ 0: uniform weights
    (30.0, 30.0, 1.0),      # scores ~ 1e4: the 22 bits of the split operands begin to show
    (300.0, 300.0, 1e20),   # scores ~ 1e6: one key takes each row; rows recomputed in plain fp32
])
def test_operand_magnitudes(sdq, sq, sk, sv):
    """The fp16 planes carry q, k and v times powers of two chosen from the data (per query row,
    per k, per v), so the magnitudes of the inputs do not matter; rows of very different size
    sit in one tile.  Where the scores can be so large that the dropped lo*lo terms would show,
    the rows are marked and come from the fp32 CUDA-core kernel."""
    rng = np.random.default_rng(5)
    heads, Lq, Lk = 2, 257, 391
    C = heads * 128
    q = (rng.standard_normal((Lq, C)) * sq).astype(np.float32)
    q[::3] *= 1e-3
    q[5] = 0.0                                            # a row of zeros: uniform weights
    k = (rng.standard_normal((Lk, C)) * sk).astype(np.float32)
    k[::7] *= 1e-4
    v = (rng.standard_normal((Lk, C)) * sv).astype(np.float32)
    got = sdq.sdpa_np(q, k, v, heads)
    want = attention64(q, k, v, heads)
    assert np.isfinite(got).all()
    # scores in the thousands show the 22 bits the split operands carry (fp32 dot products have
    # 24): ~1e-4 at scores ~1e3; beyond ~1e4 the rows are recomputed in plain fp32, whose own
    # distance from float64 is then the yardstick
    fp32_err = max_rel_err(sdq.sdpa_np(q, k, v, heads, force_simt=True), want)
    assert max_rel_err(got, want) < max(3e-4 if sq * sk > 100 else 1e-4, 2 * fp32_err)


def test_scores_growing_along_the_keys(sdq):
    """Key magnitudes ramp up by 40x along the key axis, so every row's running maximum moves
    many times (the accumulated output and row sum are rescaled each time), by different amounts
    in different rows of one tile."""
    rng = np.random.default_rng(33)
    heads, Lq, Lk = 2, 300, 1700
    C = heads * 128
    q = (rng.standard_normal((Lq, C)) * np.linspace(0.3, 2.0, Lq)[:, None]).astype(np.float32)
    k = (rng.standard_normal((Lk, C)) * np.linspace(0.1, 4.0, Lk)[:, None]).astype(np.float32)
    v = rng.standard_normal((Lk, C)).astype(np.float32)
    got = sdq.sdpa_np(q, k, v, heads)
    want = attention64(q, k, v, heads)
    assert np.isfinite(got).all()
    assert max_rel_err(got, want) < 1e-4
    # and the reverse order: the maximum is found at once, later blocks only add small weights
    got = sdq.sdpa_np(q, k[::-1].copy(), v[::-1].copy(), heads)
    assert max_rel_err(got, want) < 1e-4


def test_v_as_one_fp16_number(sdq):
    """SDQ_SDPA_V_FP16: two MMAs per P*V product; v rounded to 11 bits moves the outputs by a few
    1e-4 at most, inside the reference's 1e-3 bound."""
    rng = np.random.default_rng(12)
    heads, Lq, Lk = 3, 500, 1111
    q, k, v = [rng.standard_normal((n, heads * 128)).astype(np.float32) for n in (Lq, Lk, Lk)]
    q *= 3.0                                              # peaked rows: little averaging of v's rounding
    want = attention64(q, k, v, heads)
    full = sdq.sdpa_np(q, k, v, heads)
    fast = sdq.sdpa_np(q, k, v, heads, v_fp16=True)
    assert max_rel_err(full, want) < 2e-5
    assert 2e-5 < max_rel_err(fast, want) < 4e-4           # (the flag did something, and stayed in bounds)


def test_k_as_one_fp16_number(sdq):
    """SDQ_SDPA_K_FP16: two MMAs per score product (q keeps both planes, k only its leading one);
    alone and together with SDQ_SDPA_V_FP16 the outputs stay inside the reference's 1e-3 bound,
    also on rows peaked enough that one key carries most of the weight."""
    rng = np.random.default_rng(13)
    heads, Lq, Lk = 3, 500, 1111
    q, k, v = [rng.standard_normal((n, heads * 128)).astype(np.float32) for n in (Lq, Lk, Lk)]
    for qmul in (1.0, 3.0):
        want = attention64(q * qmul, k, v, heads)
        full = sdq.sdpa_np(q * qmul, k, v, heads)
        fast = sdq.sdpa_np(q * qmul, k, v, heads, k_fp16=True)
        both = sdq.sdpa_np(q * qmul, k, v, heads, k_fp16=True, v_fp16=True)
        assert max_rel_err(full, want) < 2e-5
        assert 2e-5 < max_rel_err(fast, want) < 1e-3
        assert max_rel_err(both, want) < 1e-3
    # an odd number of key blocks, fewer keys than one block, several work items per CTA
    for Lq2, Lk2 in [(130, 129), (300, 77), (1000, 1600)]:
        q2, k2, v2 = [rng.standard_normal((n, 128)).astype(np.float32) for n in (Lq2, Lk2, Lk2)]
        assert max_rel_err(sdq.sdpa_np(q2, k2, v2, 1, k_fp16=True), attention64(q2, k2, v2, 1)) < 1e-3


def test_other_head_sizes_take_the_cuda_core_kernel(sdq):
    rng = np.random.default_rng(2)
    for heads, hd, Lq, Lk in [(3, 64, 40, 77), (2, 96, 9, 130), (1, 20, 5, 3)]:
        C = heads * hd
        q, k, v = [rng.standard_normal((n, C)).astype(np.float32) for n in (Lq, Lk, Lk)]
        assert max_rel_err(sdq.sdpa_np(q, k, v, heads), attention64(q, k, v, heads)) < 1e-5


def test_arguments(sdq, pkg):
    d = sdq.alloc(1024)
    with pytest.raises(pkg.SdqError):
        sdq._ck(sdq.lib.sdq_sdpa(d.ptr, d.ptr, d.ptr, 1, 1, 100, 3, d.ptr, 0, None))     # C % heads
    with pytest.raises(pkg.SdqError):
        sdq._ck(sdq.lib.sdq_sdpa(None, d.ptr, d.ptr, 1, 1, 128, 1, d.ptr, 0, None))
    assert sdq.lib.sdq_sdpa(d.ptr, d.ptr, d.ptr, 0, 5, 128, 1, d.ptr, 0, None) == 0       # no queries
    out = sdq.sdpa_np(np.ones((2, 128), np.float32), np.zeros((0, 128), np.float32),
                      np.zeros((0, 128), np.float32), 1)
    assert np.array_equal(out, np.zeros((2, 128), np.float32))                            # no keys


def test_runs_are_bit_reproducible(sdq):
    """Every accumulation has a fixed order (one MMA-issuing lane per accumulator, one thread per
    row sum): two runs on the same inputs give the same bits."""
    rng = np.random.default_rng(21)
    heads, Lq, Lk = 4, 900, 1500
    q, k, v = [rng.standard_normal((n, heads * 128)).astype(np.float32) for n in (Lq, Lk, Lk)]
    a = sdq.sdpa_np(q, k, v, heads)
    b = sdq.sdpa_np(q, k, v, heads)
    assert bits_equal(a, b)
