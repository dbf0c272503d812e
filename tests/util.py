"""Shared helpers of the tests: seeded inputs and comparison metrics."""
import hashlib
import os

import numpy as np


def reference_tree():
    """The reference checkout: $REF, else a directory `reference` beside this repository."""
    here = os.path.dirname(os.path.abspath(__file__))
    return os.environ.get("REF") or os.path.join(os.path.dirname(os.path.dirname(here)), "reference")


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


def random_safetensors(rng, path, oracle):
    """A small random checkpoint: a mix of source dtypes, ranks and sizes on both sides of the
    packer's 65536-element threshold, rows as short as 2, an empty tensor, integer tensors."""
    from oracle import pack_oracle
    tens = []
    n = int(rng.integers(3, 9))
    for i in range(n):
        dt = ["BF16", "F16", "F32", "I8", "U8", "I32", "I64"][int(rng.integers(0, 7))]
        kind = int(rng.integers(0, 5))
        if kind == 0:
            shape = (int(rng.integers(256, 600)), int(rng.integers(256, 400)))        # quantized, 2-D
        elif kind == 1:
            shape = (int(rng.integers(64, 128)), int(rng.integers(16, 40)), int(rng.choice([2, 7, 33])))
        elif kind == 2:
            shape = (int(rng.integers(1, 300)),)                                       # small 1-D
        elif kind == 3:
            shape = (65536 // 64, 64) if rng.integers(2) else (65535,)                 # at the threshold
        else:
            shape = (0, 5) if rng.integers(2) else ()
        numel = int(np.prod(shape)) if shape else 1
        if dt == "BF16":
            raw = oracle.f32_to_bf16((rng.standard_normal(numel) * 0.02).astype(np.float32)).tobytes()
        elif dt == "F16":
            raw = (rng.standard_normal(numel) * 0.02).astype(np.float16).tobytes()
        elif dt == "F32":
            raw = (rng.standard_normal(numel) * 0.02).astype(np.float32).tobytes()
        else:
            npdt = {"I8": np.int8, "U8": np.uint8, "I32": np.int32, "I64": np.int64}[dt]
            raw = rng.integers(0, 100, numel).astype(npdt).tobytes()
        tens.append(("t%d.%s" % (i, ["weight", "bias", "w"][i % 3]), dt, shape, raw))
    order = rng.permutation(len(tens))                  # header order != data order
    pack_oracle.write_safetensors(path, tens)
    return [tens[i][0] for i in order]
