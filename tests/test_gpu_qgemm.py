"""GPU: sd::qgemm through the C ABI is bit-identical to the reference.

Small cases are compared whole against the golden fixtures (outputs of the
reference's own compiled sd::qgemm) and the oracle; full-size cases are
compared on sampled rows (rows are independent) and through size-independent
properties: row-split and column-split invariance, row permutation.
Tolerance: 0 (bit-exact) for int8 bytes, int32 accumulators and fp32 outputs;
1e-3 max-abs/max-abs for the fused GELU epilogue (stated where used).
"""
import json
import os

import numpy as np
import pytest

from util import bits_equal, cosine, max_rel_err, packed_weights, sha, weights_bf16

pytestmark = pytest.mark.gpu

GELU_TOL = 1e-3


@pytest.fixture(scope="module")
def gold(golden_dir):
    return json.load(open(os.path.join(golden_dir, "golden.json")))


def test_golden_small_cases(sdq, golden_dir):
    z = np.load(os.path.join(golden_dir, "qgemm_small.npz"))
    for tag in ("m17k31n13", "m64k256n128", "m130k96n200"):
        w = sdq.weight_upload(z[tag + "_Bq"], z[tag + "_bs"])
        out = sdq.qgemm_host(w, z[tag + "_A"])
        assert bits_equal(out, z[tag + "_out"]), tag
        out = sdq.qgemm_host(w, z[tag + "_A"], force_simt=True)
        assert bits_equal(out, z[tag + "_out"]), tag + " (simt)"
        sdq.weight_release(w)


def test_golden_digests(sdq, oracle, gold):
    """config 1 (M=192, K=N=3072), both sides of the reference's M>=2048 branch, FFN-up slice."""
    for tag, d in gold["qgemm_digests"].items():
        rng = np.random.default_rng(d["seed"])
        A = (rng.standard_normal((d["M"], d["K"])) * d["a_mul"]).astype(np.float32)
        wq, ws = oracle.quant_rows_packer(oracle.bf16_to_f32(weights_bf16(rng, d["N"], d["K"], oracle)))
        assert sha(A) == d["A_sha256"] and sha(wq) == d["Bq_sha256"]
        w = sdq.weight_upload(wq, ws)
        out = sdq.qgemm_host(w, A)
        assert sha(out) == d["out_sha256"], tag
        sdq.weight_release(w)


@pytest.mark.parametrize("M,K,N", [
    (1, 16, 1), (1, 256, 3072), (5, 48, 36), (128, 128, 256), (129, 144, 257), (192, 3072, 3072),
    (200, 512, 384), (256, 1024, 192), (300, 272, 1000), (1000, 64, 4100), (2048, 512, 256),
    (2500, 3072, 192), (4096, 256, 3072), (19072, 128, 512), (512, 4096, 3072),
    (192, 14336, 3072), (100, 8192, 200), (64, 14336, 1024),          # large K, few rows: K is split
])
def test_intermediates_match_oracle(sdq, oracle, M, K, N):
    """aq, a_scale, int32 accumulators and fp32 outputs, all exact, over every tile width."""
    rng = np.random.default_rng(M * 7 + K * 3 + N)
    A = rng.standard_normal((M, K)).astype(np.float32)
    wq, ws = packed_weights(rng, N, K, oracle)
    w = sdq.weight_upload(wq, ws)
    aq, a_s, acc, out = sdq.qgemm_debug(w, A)
    aq_c, as_c = oracle.act_quant_rows(A)
    acc_c = oracle.dot_s32(aq_c, wq)
    assert bits_equal(aq, aq_c) and bits_equal(a_s, as_c)
    assert bits_equal(acc, acc_c)
    assert bits_equal(out, oracle.rescale(acc_c, as_c, ws))
    sdq.weight_release(w)


def test_split_k_host_path_matches_oracle(sdq, oracle):
    """The few-rows / long-K shapes take the split-K plan (int32 partial sums added by bulk
    tensor reductions, then a finalize pass); bias and the host-pointer path included."""
    rng = np.random.default_rng(77)
    for (M, K, N) in [(192, 14336, 3072), (64, 14336, 512)]:
        A = rng.standard_normal((M, K)).astype(np.float32)
        wq, ws = packed_weights(rng, N, K, oracle)
        b = (rng.standard_normal(N) * 0.02).astype(np.float32)
        w = sdq.weight_upload(wq, ws)
        want = oracle.qgemm(A, wq, ws)
        assert bits_equal(sdq.qgemm_host(w, A), want)
        assert bits_equal(sdq.qgemm_host(w, A), want)          # the accumulator is cleared per call
        assert bits_equal(sdq.qgemm_host(w, A, bias=b), oracle.bias_add(want, b))
        sdq.weight_release(w)


def test_extreme_accumulators(sdq, oracle):
    """+-127 everywhere: the largest sums the path can see at the widest DiT K."""
    K, N, M = 14336, 64, 130
    A = np.full((M, K), 1.0, np.float32)
    A[1::2] *= -1
    wq = np.full((N, K), 127, np.int8)
    wq[::3] = -127
    ws = np.full((N,), 1e-3, np.float32)
    w = sdq.weight_upload(wq, ws)
    _, _, acc, out = sdq.qgemm_debug(w, A)
    assert int(np.abs(acc).max()) == 127 * 127 * K
    assert bits_equal(out, oracle.qgemm(A, wq, ws))
    sdq.weight_release(w)


def test_bias_and_gelu_epilogue(sdq, oracle):
    rng = np.random.default_rng(21)
    M, K, N = 300, 512, 640
    A = (rng.standard_normal((M, K)) * 0.5).astype(np.float32)
    wq, ws = packed_weights(rng, N, K, oracle)
    b = (rng.standard_normal(N) * 0.02).astype(np.float32)
    w = sdq.weight_upload(wq, ws)
    y = oracle.qgemm(A, wq, ws)
    yb = oracle.bias_add(y, b)
    # bias: one IEEE add after the rescale, as the reference's separate pass does -> exact
    assert bits_equal(sdq.qgemm_host(w, A, bias=b), yb)
    assert bits_equal(sdq.qgemm_host(w, A, bias=b, force_simt=True), yb)
    # GELU: tanh is not bit-reproducible across libms; tolerance 1e-3 of the output's max
    g = sdq.qgemm_host(w, A, bias=b, gelu=True)
    assert max_rel_err(g, oracle.gelu_tanh(yb)) < GELU_TOL
    assert max_rel_err(sdq.qgemm_host(w, A, gelu=True), oracle.gelu_tanh(y)) < GELU_TOL
    sdq.weight_release(w)


def test_empty_and_bad_arguments(sdq, pkg, oracle):
    rng = np.random.default_rng(1)
    wq, ws = packed_weights(rng, 32, 64, oracle)
    w = sdq.weight_upload(wq, ws)
    assert sdq.qgemm_host(w, np.zeros((0, 64), np.float32)).shape == (0, 32)   # M == 0: no-op
    with pytest.raises(pkg.SdqError) as e:
        sdq.qgemm(12345, None, 4, None)
    assert e.value.code == 1 and "handle" in e.value.msg
    with pytest.raises(pkg.SdqError):
        sdq.qgemm(w, None, 4, None)
    with pytest.raises(pkg.SdqError):
        sdq.weight_upload(np.zeros((0, 8), np.int8), np.zeros((0,), np.float32))
    sdq.weight_release(w)
    with pytest.raises(pkg.SdqError):
        sdq.weight_info(w)


def test_weight_registry_lookup(sdq, pkg, oracle):
    """The reference's caller only has the host pointer of the int8 view in hand."""
    rng = np.random.default_rng(4)
    wq, ws = packed_weights(rng, 48, 96, oracle)
    w = sdq.weight_upload(wq, ws)
    assert sdq.weight_lookup(wq.ctypes.data) == w
    N, K, qp, sp = sdq.weight_info(w)
    assert (N, K) == (48, 96) and qp % 256 == 0 and sp % 256 == 0
    sdq.weight_release(w)
    with pytest.raises(pkg.SdqError) as e:
        sdq.weight_lookup(wq.ctypes.data)
    assert e.value.code == 7


def test_reference_gate_cosine(sdq, oracle):
    """The reference's own acceptance test: cosine > 0.999 vs fp32 matmul on dequantized
    weights at (17,31,13) and (64,1024,512)  (tests/test_core.cpp:93-118)."""
    rng = np.random.default_rng(9)
    for (M, K, N) in [(17, 31, 13), (64, 1024, 512)]:
        A = rng.uniform(-1, 1, (M, K)).astype(np.float32)
        W = rng.uniform(-1, 1, (N, K)).astype(np.float32)
        wq, ws = oracle.quantize_rowwise(W)
        w = sdq.weight_upload(wq, ws)
        out = sdq.qgemm_host(w, A)
        ref = A @ (wq.astype(np.float32) * ws[:, None]).T
        assert cosine(out, ref) > 0.999
        assert np.isfinite(out).all() and out.shape == (M, N)
        sdq.weight_release(w)


def test_concurrent_host_threads_and_streams(sdq, pkg, oracle):
    """Four host threads, each with its own stream, weight and shape, calling sdq_qgemm at the
    same time: the scratch is per stream and the registry is locked, so every result is exact."""
    import threading
    rng = np.random.default_rng(12)
    jobs = []
    for (M, K, N) in [(700, 1024, 512), (300, 3072, 1024), (2500, 512, 768), (129, 2048, 384)]:
        A = rng.standard_normal((M, K)).astype(np.float32)
        wq, ws = packed_weights(rng, N, K, oracle)
        jobs.append((A, wq, ws, oracle.qgemm(A, wq, ws)))
    errors = []

    def run(job):
        try:
            A, wq, ws, want = job
            M, K = A.shape
            N = wq.shape[0]
            w = sdq.weight_upload(wq, ws)
            dA, dout = sdq.to_device(A), sdq.alloc(M * N * 4)
            st = sdq.stream_create()
            for _ in range(20):
                sdq.qgemm(w, dA.ptr, M, dout.ptr, None, 0, st)
            sdq.sync(st)
            got = dout.to_numpy(np.float32, (M, N))
            if not bits_equal(got, want):
                errors.append((M, K, N))
            sdq.stream_destroy(st)
            sdq.weight_release(w)
        except Exception as e:  # pragma: no cover
            errors.append(repr(e))
    threads = [threading.Thread(target=run, args=(j,)) for j in jobs]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors


def test_two_threads_run_the_host_pointer_ffn_pipeline(sdq, pkg, oracle):
    """sdq_ffn_pair with host x and y keeps its copy streams, events and chunk buffers with the
    caller's stream: two host threads on two streams run the chunked pipeline at the same time
    and both get the bits of the two-call form."""
    import ctypes as C
    import threading
    rng = np.random.default_rng(99)
    D, F = 512, 1024
    w1q, w1s = packed_weights(rng, F, D, oracle)
    w2q, w2s = packed_weights(rng, D, F, oracle)
    w1, w2 = sdq.weight_upload(w1q, w1s), sdq.weight_upload(w2q, w2s)
    jobs = []
    for M in (5000, 6100):                                # 3 chunks of 2048 rows each, different tails
        x = (rng.standard_normal((M, D)) * 0.5).astype(np.float32)
        h = sdq.qgemm_host(w1, x, gelu=True)
        jobs.append((x, sdq.qgemm_host(w2, h)))
    errors = []

    def run(job):
        try:
            x, want = job
            M = x.shape[0]
            y = np.empty((M, D), np.float32)
            st = sdq.stream_create()
            for _ in range(6):
                y[:] = 0
                sdq._ck(sdq.lib.sdq_ffn_pair(w1, None, w2, None, x.ctypes.data_as(C.c_void_p), M, None,
                                             y.ctypes.data_as(C.c_void_p), pkg.sdq.A_HOST | pkg.sdq.OUT_HOST, st))
                if not bits_equal(y, want):
                    errors.append(M)
            sdq.stream_destroy(st)
        except Exception as e:  # pragma: no cover
            errors.append(repr(e))
    threads = [threading.Thread(target=run, args=(j,)) for j in jobs]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    sdq.weight_release(w1)
    sdq.weight_release(w2)
    assert not errors, errors


def test_stream_destroy_returns_all_scratch(sdq, pkg, oracle):
    """Every buffer a stream's calls grew -- quantized activations, split-K sums, layernorm
    statistics, the tf32 planes of sdq_fmatmul, the fp16 planes of sdq_sdpa, the chunk buffers of the
    host-pointer FFN pipeline -- goes back to the device when the stream is destroyed."""
    import torch
    rng = np.random.default_rng(3)
    wq, ws = packed_weights(rng, 384, 512, oracle)
    w = sdq.weight_upload(wq, ws)
    fw = sdq.fweight_upload((rng.standard_normal((512, 256)) * 0.05).astype(np.float32))
    A = rng.standard_normal((1000, 512)).astype(np.float32)
    dA, dout = sdq.to_device(A), sdq.alloc(1000 * 512 * 4)
    q = sdq.to_device(rng.standard_normal((2048, 1024)).astype(np.float32))
    o = sdq.alloc(2048 * 1024 * 4)
    sh = sdq.to_device(np.zeros(512, np.float32))
    daq, dsc = sdq.alloc(1000 * 512), sdq.alloc(4000)

    def use(st):
        sdq.qgemm(w, dA.ptr, 1000, dout.ptr, None, 0, st)
        sdq._ck(sdq.lib.sdq_fmatmul(fw, dA.ptr, 1000, dout.ptr, None, 0, st))
        sdq._ck(sdq.lib.sdq_sdpa(q.ptr, q.ptr, q.ptr, 2048, 2048, 1024, 8, o.ptr, 0, st))
        sdq._ck(sdq.lib.sdq_layernorm_mod_quantize(dA.ptr, 1000, 512, sh.ptr, sh.ptr, 1e-6, daq.ptr, dsc.ptr,
                                                   None, 0, st))
        sdq.sync(st)
    st = sdq.stream_create()
    use(st)                                               # first use also pays one-time driver allocations
    sdq.stream_destroy(st)
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    st = sdq.stream_create()
    use(st)
    held = free0 - torch.cuda.mem_get_info()[0]
    assert held > (16 << 20), held                        # the scratch is really there (k / v^T planes alone: 16 MiB) ...
    sdq.stream_destroy(st)
    torch.cuda.synchronize()
    # ... and it comes back (2 MiB of slack for what the driver keeps per stream)
    assert torch.cuda.mem_get_info()[0] >= free0 - (2 << 20), (free0, torch.cuda.mem_get_info()[0])
    sdq.weight_release(w)
    sdq.weight_release(fw)
