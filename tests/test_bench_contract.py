"""CPU: the benchmark's reference arm runs here and prints the contracted JSON line."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                        "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600,
                       env=dict(os.environ, SDQ_BENCH_REF_BUDGET_S="4"))
    assert r.returncode == 0, r.stderr
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "TOPS" and d["higher_is_better"] is True
    assert d["config"]["workload"] == "ffn_pair_720p" and d["value"] > 0
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["value"] == d["value"]


def test_other_ranks_of_the_reference_arm_do_nothing():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                       capture_output=True, text=True, timeout=60, env=dict(os.environ, RANK="1", WORLD_SIZE="2"))
    assert r.returncode == 0 and r.stdout.strip() == ""


def _bench():
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_roofline_denominator_and_traffic_table():
    """The int8 tensor roofline is twice the measured dense bf16 rate -- the burst figure for a timed
    region under a second, the sustained one above -- and the DRAM traffic comes from the committed
    table of ncu captures, None where no capture matches."""
    b = _bench()
    pk = {"bf16_tflops": 1688.4, "bf16_tflops_sustained": 1426.3}
    peak, kind = b.int8_peak(pk, "measured", 0.04)
    assert abs(peak - 3376.8) < 1e-9 and "burst" in kind and "measured" in kind
    peak, kind = b.int8_peak(pk, "measured", 2.0)
    assert abs(peak - 2852.6) < 1e-9 and "sustained" in kind
    peak, kind = b.int8_peak({}, "fallback", 0.1)                      # no file: the stated fallback figures
    assert abs(peak - 2 * b.FALLBACK_PEAKS["bf16_tflops"]) < 1e-9 and "fallback" in kind
    t, src = b.dram_traffic("qgemm_tc2_kernel 3072x14336 bias+gelu", 27280)
    assert t and 1.6e9 < t < 2.3e9 and src                              # at least the algorithmic 1.69 GB
    assert b.dram_traffic("qgemm_tc2_kernel 3072x14336 bias+gelu", 3410) == (None, None)
    assert b.dram_traffic("no such kernel", 27280) == (None, None)
    # algorithmic bytes of the dominant linear and the operations of the pair
    assert b.gemm_bytes(27280, 3072, 14336) == 4 * 27280 * 3072 + 14336 * 3072 + 4 * 14336 + 4 * 27280 * 14336 + 4 * 14336
    assert b.ffn_ops(27280) == 2.0 * 27280 * 3072 * 14336 * 2


def test_both_arms_print_the_same_config(pkg):
    b = _bench()
    for world in (1, 2, 4, 8):
        shards = [pkg.sharding.row_shard(27280, world, r) for r in range(world)]
        cfg = b.workload_config(27280, shards, world)
        assert cfg["workload"] == "ffn_pair_720p" and cfg["rows_total"] == 27280
        per = cfg["rows_per_gpu"] if world > 1 else [cfg["rows_per_gpu"]]
        assert sum(per) == 27280 and max(per) == -(-107 // world) * 256 or world == 1
