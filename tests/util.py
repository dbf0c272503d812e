"""Shared helpers of the tests: seeded inputs and comparison metrics."""
import hashlib

import numpy as np


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def weights_bf16(rng, n, k, oracle, std=0.02):
    """N(0, std) weights rounded to bf16 bit patterns, the synthetic checkpoint dtype."""
    w = (rng.standard_normal((n, k)) * std).astype(np.float32)
    return oracle.f32_to_bf16(w)


def packed_weights(rng, n, k, oracle, std=0.02):
    """(int8 [n,k], f32 scale [n]) as the .sdcpp packer stores them."""
    return oracle.quant_rows_packer(oracle.bf16_to_f32(weights_bf16(rng, n, k, oracle, std)))


def bits_equal(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    return a.shape == b.shape and a.dtype == b.dtype and a.tobytes() == b.tobytes()


def max_rel_err(got, want):
    """max|got-want| / max|want| -- the normalisation the reference's tests use
    (tests/test_core.cpp:82-84)."""
    denom = float(np.max(np.abs(want))) or 1.0
    return float(np.max(np.abs(got.astype(np.float64) - want.astype(np.float64)))) / denom


def cosine(a, b):
    a, b = a.astype(np.float64).ravel(), b.astype(np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b) + 1e-300))
