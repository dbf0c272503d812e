"""CPU: the oracle is pinned against the reference's own outputs.

Fixtures under tests/golden/ were produced by the reference's code
(tools/quantize/pack_sdcpp.py and sd::qgemm / sd::quantize_rowwise compiled from
source) by tests/golden/make_golden.py.  Where oracle/_ref is present the same
checks also run live against the compiled reference.
"""
import json
import os

import numpy as np
import pytest

from oracle import pack_oracle
from util import bits_equal, cosine, max_rel_err, sha, weights_bf16


@pytest.fixture(scope="module")
def gold(golden_dir):
    return json.load(open(os.path.join(golden_dir, "golden.json")))


def test_packer_rows_match_reference_packer(oracle, golden_dir):
    z = np.load(os.path.join(golden_dir, "packer_rows.npz"))
    for tag in ("w64x256", "w33x1000", "w8x7"):
        x = oracle.bf16_to_f32(z[tag + "_bf16"])
        q, s = oracle.quant_rows_packer(x)
        assert bits_equal(q, z[tag + "_q"]), tag
        assert bits_equal(s, z[tag + "_scale"]), tag
    q, s = oracle.quant_rows_packer(z["ties_f32"])
    assert bits_equal(q, z["ties_q"]) and bits_equal(s, z["ties_scale"])
    q, s = oracle.quant_rows_packer(oracle.f16_to_f32(z["h16x512_f16"]))
    assert bits_equal(q, z["h16x512_q"]) and bits_equal(s, z["h16x512_scale"])
    # an all-zero row: bytes 0 and scale 0 (pack_sdcpp.py:47-51)
    assert not z["w64x256_q"][5].any() and z["w64x256_scale"][5] == 0.0


def test_f16_widening_is_exact(oracle):
    h = np.arange(0, 1 << 16, dtype=np.uint16)
    got = oracle.f16_to_f32(h)
    want = h.view(np.float16).astype(np.float32)
    ok = (got.view(np.uint32) == want.view(np.uint32)) | (np.isnan(got) & np.isnan(want))
    assert ok.all()


def test_qgemm_small_match_reference(oracle, golden_dir):
    z = np.load(os.path.join(golden_dir, "qgemm_small.npz"))
    for tag in ("m17k31n13", "m64k256n128", "m130k96n200"):
        out = oracle.qgemm(z[tag + "_A"], z[tag + "_Bq"], z[tag + "_bs"])
        assert bits_equal(out, z[tag + "_out"]), tag
    q, s = oracle.quantize_rowwise(z["rowwise_W"])
    assert bits_equal(q, z["rowwise_q"]) and bits_equal(s, z["rowwise_scale"])
    assert s[3] == 1.0  # all-zero row: scale 1 (src/core/tensor.cpp:70)


def test_qgemm_digests_match_reference(oracle, gold):
    for tag, d in gold["qgemm_digests"].items():
        rng = np.random.default_rng(d["seed"])
        A = (rng.standard_normal((d["M"], d["K"])) * d["a_mul"]).astype(np.float32)
        wq, ws = oracle.quant_rows_packer(oracle.bf16_to_f32(weights_bf16(rng, d["N"], d["K"], oracle)))
        assert sha(A) == d["A_sha256"], "input generator drifted: " + tag
        assert sha(wq) == d["Bq_sha256"] and sha(ws) == d["bs_sha256"], tag
        assert sha(oracle.qgemm(A, wq, ws)) == d["out_sha256"], tag


def test_qgemm_halves_compose(oracle):
    rng = np.random.default_rng(3)
    A = rng.standard_normal((37, 200)).astype(np.float32)
    A[4, :] = 0  # zero row: scale 1, all-zero bytes (src/core/qgemm.cpp:90-91)
    wq = rng.integers(-127, 128, (29, 200)).astype(np.int8)
    ws = rng.uniform(0.001, 0.01, 29).astype(np.float32)
    aq, a_s = oracle.act_quant_rows(A)
    assert a_s[4] == 1.0 and not aq[4].any()
    assert np.abs(aq).max() == 127
    acc = oracle.dot_s32(aq, wq)
    assert np.array_equal(acc, aq.astype(np.int64) @ wq.astype(np.int64).T)
    assert bits_equal(oracle.rescale(acc, a_s, ws), oracle.qgemm(A, wq, ws))
    # the reference's own gate: cosine > 0.999 against fp32 (tests/test_core.cpp:116)
    ref = A @ (wq.astype(np.float32) * ws[:, None]).T
    assert cosine(oracle.qgemm(A, wq, ws), ref) > 0.999


def test_act_quant_nonfinite_follows_cvtss2si(oracle):
    A = np.ones((3, 8), np.float32)
    A[0, 1] = np.nan          # ignored by the max; rounds to INT_MIN -> clamped to -127
    A[1, 2] = np.inf          # scale inf, inv 0: inf*0 = NaN -> -127, finite*0 -> 0
    A[2, :] = 1e-45           # denormal max: scale underflows to 0 -> 1
    aq, a_s = oracle.act_quant_rows(A)
    assert aq[0, 1] == -127 and aq[0, 0] == 127
    assert np.isinf(a_s[1]) and aq[1, 2] == -127 and aq[1, 0] == 0
    assert a_s[2] == 1.0 and not aq[2].any()


def test_live_reference_agrees(oracle, reference):
    rng = np.random.default_rng(99)
    for (M, K, N) in [(5, 33, 7), (64, 1024, 512), (2048, 256, 128)]:
        A = rng.standard_normal((M, K)).astype(np.float32)
        wq = rng.integers(-127, 128, (N, K)).astype(np.int8)
        ws = rng.uniform(0.001, 0.01, N).astype(np.float32)
        assert bits_equal(oracle.qgemm(A, wq, ws), reference.qgemm(A, wq, ws))
    W = rng.uniform(-1, 1, (37, 513)).astype(np.float32)
    q0, s0 = oracle.quantize_rowwise(W)
    q1, s1 = reference.quantize_rowwise(W)
    assert bits_equal(q0, q1) and bits_equal(s0, s1)
    x = rng.standard_normal(1000).astype(np.float32)
    assert bits_equal(oracle.f32_to_bf16(x), reference.to_bf16(x))


def test_layernorm_restates_reference(oracle, reference):
    """The step in front of the linears: blk::layernorm without affine parameters."""
    rng = np.random.default_rng(6)
    x = (rng.standard_normal((64, 3072)) * 3 + 0.5).astype(np.float32)
    zero = np.zeros(3072, np.float32)
    assert bits_equal(oracle.layernorm_mod(x, zero, zero, 1e-6), reference.layernorm(x, 1e-6))
    # modulation: y = ln * (1 + scale) + shift, per channel (src/model/ovi_dit.cpp:162-173)
    shift = rng.standard_normal(3072).astype(np.float32)
    scale = (rng.standard_normal(3072) * 0.1).astype(np.float32)
    # the compiled reference fuses the multiply and the add into one operation
    ln = reference.layernorm(x, 1e-6)
    assert bits_equal(oracle.layernorm_mod(x, shift, scale, 1e-6), reference.mod_rows(ln, shift, scale))


def test_caller_side_matches_reference_fixture(oracle, golden_dir):
    """mlin's bias pass, gated_add_inplace / add_inplace and a whole ffn_fwd, against outputs of
    the compiled src/model/ovi_dit.cpp (tests/golden/dit_caller.npz)."""
    z = np.load(os.path.join(golden_dir, "dit_caller.npz"))
    y = oracle.bias_add(oracle.qgemm(z["lin_A"], z["lin_Bq"], z["lin_bs"]), z["lin_bias"])
    assert bits_equal(y, z["lin_y"])
    assert bits_equal(oracle.residual_add(z["lin_x"], y, z["lin_gate"]), z["lin_gated"])
    assert bits_equal(oracle.residual_add(z["lin_x"], y), z["lin_added"])
    # and the fused form really is what the compiled code does: mul-then-add differs
    assert not bits_equal(z["lin_x"] + y * z["lin_gate"][None, :], z["lin_gated"])
    # ffn_fwd: exact up to the GELU (tanhf vs the reference build's), so a tolerance of 1e-5 here
    e = z["ffn_e"]
    h = oracle.layernorm_mod(z["ffn_x"], e[3], e[4], 1e-6)
    u = oracle.gelu_tanh(oracle.bias_add(oracle.qgemm(h, z["ffn_q1"], z["ffn_s1"]), z["ffn_b1"]))
    v = oracle.bias_add(oracle.qgemm(u, z["ffn_q2"], z["ffn_s2"]), z["ffn_b2"])
    got = oracle.residual_add(z["ffn_x"], v, e[5])
    assert max_rel_err(got, z["ffn_out"]) < 1e-5


def test_affine_layernorm_restates_reference(oracle, reference):
    """blk::layernorm with weight and bias (in front of the cross-attention projections)."""
    rng = np.random.default_rng(16)
    x = (rng.standard_normal((48, 3072)) * 2 + 0.4).astype(np.float32)
    w = (1 + rng.standard_normal(3072) * 0.2).astype(np.float32)
    b = (rng.standard_normal(3072) * 0.3).astype(np.float32)
    assert bits_equal(oracle.layernorm_affine(x, w, b, 1e-6), reference.layernorm_affine(x, w, b, 1e-6))


def test_fp32_matmul_restatement_within_reference_tolerance(oracle, golden_dir):
    """sd::matmul's result depends on its summation order (AVX2 tiles here); the restatement adds
    left to right, so the two agree to fp32 rounding, far inside the reference's 1e-3 gate."""
    z = np.load(os.path.join(golden_dir, "dit_caller.npz"))
    assert max_rel_err(oracle.matmul_f32(z["mm_A"], z["mm_W"], z["mm_bias"]), z["mm_out"]) < 1e-5
    assert max_rel_err(oracle.matmul_f32(z["mm2_A"], z["mm2_W"]), z["mm2_out"]) < 1e-5


def test_attention_restatement_within_reference_tolerance(oracle, golden_dir):
    z = np.load(os.path.join(golden_dir, "dit_caller.npz"))
    assert max_rel_err(oracle.sdpa(z["at_q"], z["at_k"], z["at_v"], 3), z["at_out"]) < 1e-5


def test_caller_side_live_reference(oracle, reference):
    rng = np.random.default_rng(31)
    x = rng.standard_normal((33, 130)).astype(np.float32)
    y = rng.standard_normal((33, 130)).astype(np.float32)
    g = rng.standard_normal(130).astype(np.float32)
    assert bits_equal(oracle.residual_add(x, y, g), reference.gated_add(x, y, g))
    assert bits_equal(oracle.residual_add(x, y), reference.add(x, y))


def test_pack_file_matches_reference_packer(oracle, gold, golden_dir, tmp_path):
    src = os.path.join(golden_dir, "tiny_model.safetensors")
    dst = str(tmp_path / "o.sdcpp")
    pack_oracle.pack(src, dst, oracle)
    assert open(dst, "rb").read() == open(os.path.join(golden_dir, "tiny_model.sdcpp"), "rb").read()
    pack_oracle.pack(src, dst, oracle, only="blocks.0.ffn,step")
    assert sha(np.fromfile(dst, np.uint8)) == gold["sdcpp_listing_only"]["sha256"]
    pack_oracle.pack(src, dst, oracle, dtype_preserve="F32:F16")
    assert sha(np.fromfile(dst, np.uint8)) == gold["sdcpp_listing_keepf32"]["sha256"]


def _listing(entries):
    dt = {"F32": 0, "I8": 2}
    lines = []
    for name in sorted(entries):
        d, shape, off, nb = entries[name]
        lines.append("%s %d %d %s %d %d" % (name, dt[d], len(shape),
                                            ",".join(map(str, shape)) if shape else "-", off, nb))
    return "\n".join(lines) + "\n"


def test_parse_matches_reference_loader(gold, golden_dir):
    buf = open(os.path.join(golden_dir, "tiny_model.sdcpp"), "rb").read()
    ents = pack_oracle.parse(buf)
    assert len(ents) == gold["sdcpp_listing"]["count"]
    assert _listing(ents) == gold["sdcpp_listing"]["listing"]


def test_parse_errors_match_reference_loader(gold, golden_dir):
    good = open(os.path.join(golden_dir, "tiny_model.sdcpp"), "rb").read()
    cases = {"truncated_half": good[: len(good) // 2], "truncated_header": good[:40],
             "short": good[:10], "bad_magic": b"XDCP" + good[4:],
             "bad_version": good[:4] + (2).to_bytes(4, "little") + good[8:]}
    for tag, data in cases.items():
        with pytest.raises(ValueError) as e:
            pack_oracle.parse(data)
        want = gold["loader_errors"][tag].replace(" <path>", "")
        assert str(e.value) == want, tag


def test_pack_restatement_matches_reference_packer_on_random_checkpoints(oracle, tmp_path):
    """Where the reference tree is mounted: random small checkpoints through the reference's
    python packer and through the restatement give identical files."""
    import subprocess
    import sys
    from util import random_safetensors
    from util import reference_tree
    ref_packer = os.path.join(reference_tree(), "tools", "quantize", "pack_sdcpp.py")
    if not os.path.exists(ref_packer):
        pytest.skip("reference tree not mounted")
    rng = np.random.default_rng(404)
    for i in range(8):
        src = str(tmp_path / ("r%d.safetensors" % i))
        names = random_safetensors(rng, src, oracle)
        extra = [[], ["--only", names[0][:2]], ["--dtype-preserve", "F16:BF16"]][i % 3]
        a, b = str(tmp_path / "ref.sdcpp"), str(tmp_path / "mine.sdcpp")
        subprocess.run([sys.executable, ref_packer, src, a] + extra, check=True, stdout=subprocess.DEVNULL)
        kw = {}
        if extra:
            kw = {"only": extra[1]} if extra[0] == "--only" else {"dtype_preserve": extra[1]}
        pack_oracle.pack(src, b, oracle, **kw)
        assert open(a, "rb").read() == open(b, "rb").read(), (i, extra)
