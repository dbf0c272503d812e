"""GPU: a whole DiT branch packed on the GPU, compared with the CPU packer.

30 blocks of the block linears (fused QKV, the two attention output projections, cross-attention
q / k / v, FFN up and down: 163.6 M weights per block, 4.9 G per branch) as bf16 N(0, 0.02),
quantized to the .sdcpp int8 layout by sdq_quantize_rows and by the oracle's packer arithmetic
(tools/quantize/pack_sdcpp.py:38-51): every int8 byte and every scale of every tensor must be
equal, and so must the SHA-256 over all of them.  The audio branch has the same block shapes
plus the two fusion projections (src/model/ovi_dit.cpp:490-536); its extra tensors are packed
and compared too.
"""
import hashlib

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

BLOCK = [("self_attn.qkv", 9216, 3072), ("self_attn.o", 3072, 3072), ("cross_attn.q", 3072, 3072),
         ("cross_attn.k", 3072, 3072), ("cross_attn.v", 3072, 3072), ("cross_attn.o", 3072, 3072),
         ("ffn.0", 14336, 3072), ("ffn.2", 3072, 14336)]
AUDIO_EXTRA = [("cross_attn.k_fusion", 3072, 3072), ("cross_attn.v_fusion", 3072, 3072)]


def test_thirty_blocks_byte_identical(sdq, pkg, oracle):
    rng = np.random.default_rng(30)
    # one N(0, 0.02) base tensor per shape; block b uses base * (1 + b / 64) with the rows rolled by
    # 7 b: different bits in every block without drawing 4.9 G normals on the host
    base = {}
    for (_, n, k) in BLOCK:
        if (n, k) not in base:
            base[(n, k)] = (rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02))
    sha_gpu, sha_cpu = hashlib.sha256(), hashlib.sha256()
    tensors = 0
    for b in range(30):
        for (name, n, k) in BLOCK + (AUDIO_EXTRA if b < 2 else []):
            w = np.roll(base[(n, k)], 7 * b + len(name), axis=0) * np.float32(1.0 + b / 64.0)
            bits = oracle.f32_to_bf16(w)
            q_g, s_g = sdq.quantize_rows(bits, pkg.sdq.BF16, pkg.sdq.MODE_PACKER)
            q_c, s_c = oracle.quant_rows_packer(oracle.bf16_to_f32(bits))
            assert q_g.tobytes() == q_c.tobytes(), (b, name)
            assert s_g.tobytes() == s_c.tobytes(), (b, name)
            sha_gpu.update(q_g.tobytes())
            sha_gpu.update(s_g.tobytes())
            sha_cpu.update(q_c.tobytes())
            sha_cpu.update(s_c.tobytes())
            tensors += 1
    assert tensors == 30 * 8 + 4
    assert sha_gpu.hexdigest() == sha_cpu.hexdigest()
