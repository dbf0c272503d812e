#!/usr/bin/env python3
"""Regenerates the committed golden fixtures in this directory.

Run in a checkout that has the reference tree mounted (its location is taken from
the REF environment variable) and oracle/_ref built:  python tests/golden/make_golden.py

It drives the REFERENCE's own code -- tools/quantize/pack_sdcpp.py (imported and
run as a script) and sd::qgemm / sd::quantize_rowwise compiled from source --
on seeded inputs, and stores inputs and outputs (small cases) or SHA-256 digests
(large cases).  The tests then check the oracle and the CUDA path against these
files without needing the reference tree.
"""
import hashlib
import json
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("REF") or os.path.join(os.path.dirname(ROOT), "reference")   # beside this repository
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(REF, "tools", "quantize"))

from oracle.binding import Oracle, Reference  # noqa: E402
from oracle import pack_oracle  # noqa: E402
import pack_sdcpp  # the reference packer  # noqa: E402


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def weights_bf16(rng, n, k, orc, std=0.02):
    w = (rng.standard_normal((n, k)) * std).astype(np.float32)
    return orc.f32_to_bf16(w)


def main():
    orc, ref = Oracle(), Reference()
    out = {}

    # ---- 1. quant_rows of the reference packer: bytes and scales, small cases stored whole
    rng = np.random.default_rng(20240)
    cases = {}
    for tag, (rows, last) in {"w64x256": (64, 256), "w33x1000": (33, 1000), "w8x7": (8, 7)}.items():
        bits = weights_bf16(rng, rows, last, orc)
        if tag == "w64x256":
            bits[5, :] = 0                       # an all-zero row: scale 0, bytes 0
            bits[6, :] = 0x8000                  # all negative zero
        x = pack_sdcpp.to_f32(bits.tobytes(), "BF16").reshape(rows, last)
        q, s = pack_sdcpp.quant_rows(x)
        cases[tag + "_bf16"] = bits
        cases[tag + "_q"] = q
        cases[tag + "_scale"] = s
    # ties: values that land exactly on .5 after scaling (round-half-even vs half-away)
    t = np.zeros((4, 256), np.float32)
    t[:, 0] = 127.0
    t[0, 1:9] = [0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5, -126.5]
    t[1, 1:5] = [63.5, 64.5, -63.5, -64.5]
    q, s = pack_sdcpp.quant_rows(t)
    cases["ties_f32"], cases["ties_q"], cases["ties_scale"] = t, q, s
    # f16 source
    h = (rng.standard_normal((16, 512)) * 0.02).astype(np.float16)
    x = pack_sdcpp.to_f32(h.tobytes(), "F16").reshape(16, 512)
    q, s = pack_sdcpp.quant_rows(x)
    cases["h16x512_f16"], cases["h16x512_q"], cases["h16x512_scale"] = h.view(np.uint16), q, s
    np.savez(os.path.join(HERE, "packer_rows.npz"), **cases)

    # ---- 2. a whole .sdcpp file written by the reference packer from a small safetensors
    rng = np.random.default_rng(20241)
    tens = [
        ("blocks.0.ffn.0.weight", "BF16", (384, 256), weights_bf16(rng, 384, 256, orc).tobytes()),
        ("blocks.0.ffn.0.bias", "BF16", (384,), weights_bf16(rng, 1, 384, orc).tobytes()),
        ("blocks.0.norm.weight", "F32", (256,), rng.standard_normal(256).astype(np.float32).tobytes()),
        ("patch_embedding.weight", "F16", (256, 16, 1, 2, 8),
         (rng.standard_normal((256, 16, 1, 2, 8)) * 0.02).astype(np.float16).tobytes()),
        ("blocks.0.attn.q.weight", "F32", (256, 256),
         (rng.standard_normal((256, 256)) * 0.02).astype(np.float32).tobytes()),
        ("step", "I64", (1,), np.array([7], np.int64).tobytes()),
        ("other.ids", "I32", (4, 3), np.arange(12, dtype=np.int32).tobytes()),
    ]
    st = os.path.join(HERE, "tiny_model.safetensors")
    pack_oracle.write_safetensors(st, tens)
    for tag, extra in {"": [], "_only": ["--only", "blocks.0.ffn,step"],
                       "_keepf32": ["--dtype-preserve", "F32:F16"]}.items():
        dst = os.path.join(HERE, "tiny_model%s.sdcpp" % tag)
        subprocess.run([sys.executable, os.path.join(REF, "tools/quantize/pack_sdcpp.py"), st, dst]
                       + extra, check=True, stdout=subprocess.DEVNULL)
        n, listing = ref.load_sdcpp_listing(dst)
        out["sdcpp_listing" + tag] = {"count": n, "listing": listing, "sha256": sha(
            np.fromfile(dst, np.uint8))}
        if tag:                                  # variants: digest and listing only
            os.remove(dst)

    # ---- 3. loader error behaviour of the reference on damaged files
    good = open(os.path.join(HERE, "tiny_model.sdcpp"), "rb").read()
    import tempfile
    errs = {}
    with tempfile.TemporaryDirectory() as td:
        def probe(tag, data):
            p = os.path.join(td, tag)
            open(p, "wb").write(data)
            try:
                ref.load_sdcpp_listing(p)
                errs[tag] = None
            except RuntimeError as e:
                errs[tag] = str(e).replace(p, "<path>")
        probe("truncated_half", good[: len(good) // 2])
        probe("truncated_header", good[:40])
        probe("short", good[:10])
        probe("bad_magic", b"XDCP" + good[4:])
        probe("bad_version", good[:4] + (2).to_bytes(4, "little") + good[8:])
        try:
            ref.load_sdcpp_listing(os.path.join(td, "missing.sdcpp"))
            errs["missing"] = None
        except RuntimeError as e:
            errs["missing"] = str(e).replace(td, "<dir>")
    out["loader_errors"] = errs

    # ---- 4. sd::qgemm / sd::quantize_rowwise outputs of the compiled reference
    q = {}
    small = {}
    for tag, (M, K, N, seed) in {"m17k31n13": (17, 31, 13, 11), "m64k256n128": (64, 256, 128, 12),
                                 "m130k96n200": (130, 96, 200, 13)}.items():
        rng = np.random.default_rng(seed)
        A = rng.standard_normal((M, K)).astype(np.float32)
        wq, ws = orc.quant_rows_packer(orc.bf16_to_f32(weights_bf16(rng, N, K, orc)))
        small[tag + "_A"], small[tag + "_Bq"], small[tag + "_bs"] = A, wq, ws
        small[tag + "_out"] = ref.qgemm(A, wq, ws)
    rng = np.random.default_rng(14)
    W = rng.uniform(-1, 1, (37, 513)).astype(np.float32)
    W[3, :] = 0
    small["rowwise_W"] = W
    small["rowwise_q"], small["rowwise_scale"] = ref.quantize_rowwise(W)
    np.savez(os.path.join(HERE, "qgemm_small.npz"), **small)
    # the two CPU-sized configurations: digests only (inputs are regenerated from the seed)
    for tag, (M, K, N, seed, a_mul) in {
            "config1_m192_k3072_n3072": (192, 3072, 3072, 42, 1.0),
            "branch_m2048_k512_n256": (2048, 512, 256, 43, 1.0),
            "branch_m2047_k512_n256": (2047, 512, 256, 43, 1.0),
            "ffn_up_m256_k3072_n14336": (256, 3072, 14336, 44, 0.5)}.items():
        rng = np.random.default_rng(seed)
        A = (rng.standard_normal((M, K)) * a_mul).astype(np.float32)
        wbits = weights_bf16(rng, N, K, orc)
        wq, ws = pack_sdcpp.quant_rows(pack_sdcpp.to_f32(wbits.tobytes(), "BF16").reshape(N, K))
        y = ref.qgemm(A, wq, ws)
        q[tag] = {"M": M, "K": K, "N": N, "seed": seed, "a_mul": a_mul, "A_sha256": sha(A),
                  "Bq_sha256": sha(wq), "bs_sha256": sha(ws), "out_sha256": sha(y)}
    out["qgemm_digests"] = q

    # ---- 5. the caller side of the linear, from the compiled src/model/ovi_dit.cpp: mlin (qgemm +
    # bias pass), gated_add_inplace / add_inplace on its output, and a whole ffn_fwd
    blk = {}
    rng = np.random.default_rng(15)
    M, K, N = 70, 256, 384
    A = rng.standard_normal((M, K)).astype(np.float32)
    wq, ws = orc.quant_rows_packer(orc.bf16_to_f32(weights_bf16(rng, N, K, orc)))
    bias = (rng.standard_normal(N) * 0.02).astype(np.float32)
    gate = rng.standard_normal(N).astype(np.float32)
    x = rng.standard_normal((M, N)).astype(np.float32)
    y = ref.mlin_i8(A, wq, ws, bias)
    blk.update(lin_A=A, lin_Bq=wq, lin_bs=ws, lin_bias=bias, lin_gate=gate, lin_x=x, lin_y=y,
               lin_gated=ref.gated_add(x, y, gate), lin_added=ref.add(x, y))
    M, D, F = 96, 256, 640
    x = (rng.standard_normal((M, D)) * 1.5 + 0.2).astype(np.float32)
    e = (rng.standard_normal((6, D)) * 0.3).astype(np.float32)
    q1, s1 = orc.quant_rows_packer(orc.bf16_to_f32(weights_bf16(rng, F, D, orc)))
    q2, s2 = orc.quant_rows_packer(orc.bf16_to_f32(weights_bf16(rng, D, F, orc)))
    b1 = (rng.standard_normal(F) * 0.02).astype(np.float32)
    b2 = (rng.standard_normal(D) * 0.02).astype(np.float32)
    blk.update(ffn_x=x, ffn_e=e, ffn_q1=q1, ffn_s1=s1, ffn_b1=b1, ffn_q2=q2, ffn_s2=s2, ffn_b2=b2,
               ffn_out=ref.ffn_fwd(x, e, q1, s1, b1, q2, s2, b2))
    # sd::matmul (the fp32 linears): a time-embedding-sized case with bias and a ragged one
    A = rng.standard_normal((40, 256)).astype(np.float32)
    Wf = (rng.standard_normal((256, 384)) * 0.05).astype(np.float32)
    bf = (rng.standard_normal(384) * 0.02).astype(np.float32)
    blk.update(mm_A=A, mm_W=Wf, mm_bias=bf, mm_out=ref.matmul(A, Wf, bf))
    A = rng.standard_normal((17, 31)).astype(np.float32)
    Wf = rng.standard_normal((31, 13)).astype(np.float32)
    blk.update(mm2_A=A, mm2_W=Wf, mm2_out=ref.matmul(A, Wf))
    # blk::sdpa (exact fp32 attention): 3 heads of 128, ragged token counts
    q = rng.standard_normal((70, 384)).astype(np.float32)
    k = rng.standard_normal((130, 384)).astype(np.float32)
    v = rng.standard_normal((130, 384)).astype(np.float32)
    blk.update(at_q=q, at_k=k, at_v=v, at_out=ref.sdpa(q, k, v, 3))
    np.savez(os.path.join(HERE, "dit_caller.npz"), **blk)
    out["numpy"] = np.__version__
    json.dump(out, open(os.path.join(HERE, "golden.json"), "w"), indent=1, sort_keys=True)
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    main()
