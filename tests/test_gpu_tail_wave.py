"""GPU: the shared last wave of the 2-CTA GEMM.

When the tiles of a problem do not fill a whole number of waves of CTA pairs, the k-blocks of
the last wave's tiles are shared between all pairs, the int32 partial sums meet in a scratch
accumulator (integer addition: exact in any order) and a second pass finishes those tiles.
The row shard of the 720p FFN on 8 GPUs (3410 rows, K = 14336) is the case it exists for; it
must give the oracle's bits with every epilogue, repeatedly (the scratch is left zero for the
next launch), and on shapes whose edges are ragged.
"""
import os
import subprocess
import sys

import numpy as np
import pytest

from util import bits_equal, max_rel_err, packed_weights

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_ffn_down_shard_of_8_gpus(sdq, pkg, oracle):
    rng = np.random.default_rng(3410)
    M, K, N = 3410, 14336, 3072                      # 14 x 12 = 168 pair-tiles on 74 pairs: 2 rounds + 20 tiles
    A = rng.standard_normal((M, K), dtype=np.float32)
    wq, ws = packed_weights(rng, N, K, oracle)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float32)
    gate = rng.standard_normal(N).astype(np.float32)
    x = rng.standard_normal((M, N), dtype=np.float32)
    w = sdq.weight_upload(wq, ws)
    want = oracle.qgemm(A, wq, ws)
    n0 = sdq.launches()
    for _ in range(3):                               # the scratch must come back clean every time
        assert bits_equal(sdq.qgemm_host(w, A), want)
    assert sdq.launches() - n0 == 9                  # quantize + GEMM + the pass over the shared tiles
    assert bits_equal(sdq.qgemm_host(w, A, bias=bias), oracle.bias_add(want, bias))
    # gated residual in place through the same path (x + (y + bias) * gate, one fused multiply-add)
    got = sdq.qgemm_residual_np(w, A, x, gate=gate, bias=bias, inplace=True)
    assert bits_equal(got, oracle.residual_add(x, oracle.bias_add(want, bias), gate))
    # GELU in the second pass: the bound of the fused activation
    got = sdq.qgemm_host(w, A, bias=bias, gelu=True)
    assert max_rel_err(got, oracle.gelu_tanh(oracle.bias_add(want, bias))) < 1e-3
    # the unshared kernel on the same input gives the same bits
    assert bits_equal(sdq.qgemm_host(w, A[:3328]), want[:3328])
    sdq.weight_release(w)


_FORCED = r"""
import sys
sys.path.insert(0, %(root)r); sys.path.insert(0, %(root)r + "/tests")
import numpy as np
import __graft_entry__ as ge
from oracle.binding import Oracle
from util import bits_equal, packed_weights
pkg, orc = ge.load_package(), Oracle()
s = pkg.Sdq(0)
rng = np.random.default_rng(8)
for (M, K, N) in [(19000, 512, 1000), (9500, 2064, 2308), (20000, 128, 520), (5000, 1024, 4100)]:
    A = rng.standard_normal((M, K), dtype=np.float32)
    wq, ws = packed_weights(rng, N, K, orc)
    bias = (rng.standard_normal(N) * 0.02).astype(np.float32)
    w = s.weight_upload(wq, ws)
    want = orc.bias_add(orc.qgemm(A, wq, ws), bias)
    n0 = s.launches()
    for _ in range(2):
        assert bits_equal(s.qgemm_host(w, A, bias=bias), want), (M, K, N)
    print("launches", (M, K, N), s.launches() - n0)
    s.weight_release(w)
print("ok")
"""


def test_ragged_shapes_with_the_shared_wave_forced():
    """SDQ_TC2_TAIL=2 shares the last wave whenever there is one, also where it does not pay:
    ragged M and N (tiles cut by both edges), K of one or a few k-blocks (segments of a single
    k-block), more k-blocks than pairs.  Read once per process, so this runs in a child."""
    r = subprocess.run([sys.executable, "-c", _FORCED % {"root": ROOT}], capture_output=True, text=True, timeout=900,
                       env=dict(os.environ, SDQ_TC2_TAIL="2", SDQ_TC_VARIANT="2"))
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), (r.stdout[-2000:], r.stderr[-2000:])
    # every case really took the three-launch form (quantize, GEMM, pass over the shared tiles)
    assert all(line.split()[-1] == "6" for line in r.stdout.splitlines() if line.startswith("launches")), r.stdout
