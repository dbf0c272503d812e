"""GPU: the .sdcpp packer writes the reference packer's bytes, and a pack opened with
upload serves sd::qgemm from device-resident weights."""
import json
import os

import numpy as np
import pytest

from oracle import pack_oracle
from util import bits_equal, sha, weights_bf16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gold(golden_dir):
    return json.load(open(os.path.join(golden_dir, "golden.json")))


def test_packer_file_is_byte_identical_to_reference(sdq, gold, golden_dir, tmp_path):
    src = os.path.join(golden_dir, "tiny_model.safetensors")
    dst = str(tmp_path / "gpu.sdcpp")
    sdq.pack_sdcpp(src, dst)
    assert open(dst, "rb").read() == open(os.path.join(golden_dir, "tiny_model.sdcpp"), "rb").read()
    sdq.pack_sdcpp(src, dst, only="blocks.0.ffn,step")
    assert sha(np.fromfile(dst, np.uint8)) == gold["sdcpp_listing_only"]["sha256"]
    sdq.pack_sdcpp(src, dst, dtype_preserve="F32:F16")
    assert sha(np.fromfile(dst, np.uint8)) == gold["sdcpp_listing_keepf32"]["sha256"]


def test_packer_larger_model_matches_oracle_packer(sdq, oracle, tmp_path):
    """One DiT block's linears at full width (bf16), chunked through the GPU."""
    rng = np.random.default_rng(11)
    D, F = 3072, 14336
    tens = []
    for name, (n, k) in {"blocks.0.self_attn.q.weight": (D, D), "blocks.0.ffn.0.weight": (F, D),
                         "blocks.0.ffn.2.weight": (D, F)}.items():
        tens.append((name, "BF16", (n, k), weights_bf16(rng, n, k, oracle).tobytes()))
        tens.append((name[:-6] + "bias", "BF16", (n,), weights_bf16(rng, 1, n, oracle).tobytes()))
    tens.append(("audio.conv.weight", "F32", (4096, 24, 7),
                 (rng.standard_normal((4096, 24, 7)) * 0.02).astype(np.float32).tobytes()))
    src, a, b = str(tmp_path / "m.safetensors"), str(tmp_path / "gpu.sdcpp"), str(tmp_path / "cpu.sdcpp")
    pack_oracle.write_safetensors(src, tens)
    sdq.pack_sdcpp(src, a)
    pack_oracle.pack(src, b, oracle)
    assert sha(np.fromfile(a, np.uint8)) == sha(np.fromfile(b, np.uint8))


def test_packer_errors(sdq, pkg, tmp_path):
    with pytest.raises(pkg.SdqError) as e:
        sdq.pack_sdcpp(str(tmp_path / "nope.safetensors"), str(tmp_path / "o.sdcpp"))
    assert e.value.code == 4
    bad = tmp_path / "bad.safetensors"
    bad.write_bytes((5).to_bytes(8, "little") + b"{oops")
    with pytest.raises(pkg.SdqError) as e:
        sdq.pack_sdcpp(str(bad), str(tmp_path / "o.sdcpp"))
    assert e.value.code == 5
    src = str(tmp_path / "f64.safetensors")
    pack_oracle.write_safetensors(src, [("x", "F64", (2,), b"\0" * 16)])
    with pytest.raises(pkg.SdqError) as e:
        sdq.pack_sdcpp(src, str(tmp_path / "o.sdcpp"))
    assert "unsupported dtype F64 for x" in e.value.msg


def test_open_pack_upload_and_qgemm(sdq, pkg, oracle, golden_dir):
    """load -> weights resident -> qgemm by host-pointer lookup, like the reference's
    load_quantized_pack + mlin (src/model/ovi_dit.cpp:355-415, 66-70)."""
    pack = sdq.open_pack(os.path.join(golden_dir, "tiny_model.sdcpp"), upload=True)
    ents = {e["name"]: e for e in pack.entries()}
    e = ents["blocks.0.ffn.0.weight"]
    sc = ents["blocks.0.ffn.0.weight.scale"]
    assert e["dtype"] == pkg.sdq.DT_I8 and e["dims"] == [384, 256] and e["weight"] != 0
    assert sc["data"] == e["data"] + e["nbytes"]            # scales sit right after the bytes
    assert sdq.weight_lookup(e["data"]) == e["weight"]
    wq, ws = pack.array(e), pack.array(sc)
    rng = np.random.default_rng(3)
    A = rng.standard_normal((70, 256)).astype(np.float32)
    assert bits_equal(sdq.qgemm_host(e["weight"], A), oracle.qgemm(A, wq, ws))
    # an N-d quantized tensor is uploaded as [numel/last, last]
    p = ents["patch_embedding.weight"]
    assert sdq.weight_info(p["weight"])[:2] == (8192, 8)
    # raw tensors are float32 views; the fp32 source passes through untouched
    assert ents["blocks.0.norm.weight"]["dtype"] == pkg.sdq.DT_F32 and ents["blocks.0.norm.weight"]["weight"] == 0
    h = e["weight"]
    pack.close()
    with pytest.raises(pkg.SdqError):
        sdq.weight_info(h)                                   # released with the pack


def test_packer_random_checkpoints_match_oracle_packer(sdq, oracle, tmp_path):
    """Random small checkpoints (mixed dtypes, ranks, sizes around the 65536-element threshold,
    rows of 2 / 7 / 33, empty and scalar tensors, --only and --dtype-preserve): the GPU packer's
    file equals the CPU packer restatement's byte for byte."""
    from util import random_safetensors
    rng = np.random.default_rng(505)
    for i in range(10):
        src = str(tmp_path / ("r%d.safetensors" % i))
        names = random_safetensors(rng, src, oracle)
        kw = [{}, {"only": names[0][:2]}, {"dtype_preserve": "F16:BF16"}][i % 3]
        a, b = str(tmp_path / "gpu.sdcpp"), str(tmp_path / "cpu.sdcpp")
        sdq.pack_sdcpp(src, a, **kw)
        pack_oracle.pack(src, b, oracle, **kw)
        assert open(a, "rb").read() == open(b, "rb").read(), (i, kw)
        # and the reader accepts what the packer wrote
        p = sdq.open_pack(a)
        assert len(p.entries()) >= 1 or os.path.getsize(a) == 12
        p.close()
