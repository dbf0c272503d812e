#!/usr/bin/env python3
"""Benchmark of the int8 quantized-linear path (one JSON line on stdout).

Workload ("ffn_pair_720p"): the DiT FFN pair at the 720p/121-frame token count,
M = 27280 rows in total:  x[M,3072] -> int8 linear 3072->14336 (+bias, GELU-tanh)
-> int8 linear 14336->3072 (+bias).  One step = one pass of that pair through
sdq_ffn_pair: two activation-quantization launches and two tcgen05 GEMM launches
(plus the short pass that finishes a shared last wave, when one is used).  Weights are
synthetic N(0,0.02) bf16 packed to int8 by the GPU packer; activations N(0,1)*0.5.

  python bench.py [--gpus N] [--steps K] [--warmup W]          (torchrun for N > 1)
  python bench.py --impl reference ...   times the reference's CPU sd::qgemm instead

Multi-GPU: the M token rows are split over the ranks in whole 256-row tiles (strong
scaling: the total work is fixed), weights replicated, no collective in the data path.
`value` is the whole-job int8 throughput in TOPS (2*M*N*K per GEMM, the reference's
own formula, tests/test_core.cpp:174) over the slowest rank's time.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D_MODEL, D_FFN, M_720P = 3072, 14336, 27280
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
INT8_NOMINAL_TOPS = 4500.0
TRAFFIC_TABLE = os.path.join(ROOT, "self-evolve-diffusion-cpp_b200", "ncu_dram_traffic.json")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--rows", type=int, default=M_720P, help="token rows in total (split over the GPUs)")
    ap.add_argument("--workload", default="ffn_pair_720p", choices=["ffn_pair_720p", "sweep", "branch", "block", "fp32"])
    ap.add_argument("--blocks", type=int, default=30, help="branch workload: number of DiT blocks")
    ap.add_argument("--heads", type=int, default=24, help="fp32 workload: attention heads of 128")
    ap.add_argument("--qk-scale", type=float, default=1.0,
                    help="fp32 workload: factor on the standard-normal q and k (larger = more peaked softmax)")
    ap.add_argument("--with-attention", action="store_true",
                    help="block workload: also run the block's self- and cross-attention (sdq_sdpa) in the fused pattern")
    ap.add_argument("--pack-file-blocks", type=int, default=0,
                    help="branch workload: also write this many blocks as a .sdcpp file and time the load")
    ap.add_argument("--verify-blocks", type=int, default=30,
                    help="branch workload: blocks whose packed bytes and scales are compared with the CPU packer's")
    ap.add_argument("--audio", action="store_true", help="branch workload: run the audio branch after the video branch")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-peak-probe", action="store_true")
    ap.add_argument("--no-dropin", action="store_true", help="skip the drop-in library's end-to-end figure")
    ap.add_argument("--no-block", action="store_true", help="skip the whole-block secondary measurement")
    ap.add_argument("--no-parity", action="store_true", help="N > 1: skip the bit-equality check of the two splits")
    return ap.parse_args()


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def int8_peak(pk, pk_kind, region_seconds):
    """The tensor roofline of an int8 kernel: no int8 figure is measured on this pool, so it is
    twice the measured dense bf16 rate (the int8 pipe issues twice the operations per
    instruction) -- the burst figure for a timed region shorter than a second, the sustained
    (power-capped) one for a longer region."""
    burst = region_seconds < 1.0
    key = "bf16_tflops" if burst else "bf16_tflops_sustained"
    return 2.0 * float(pk.get(key, FALLBACK_PEAKS[key])), \
        "2 x dense bf16 %s, of %s" % ("burst" if burst else "sustained", pk_kind)


def dram_traffic(kernel, rows):
    """dram__bytes_read.sum + dram__bytes_write.sum per launch from the committed table of ncu
    captures (kernel, rows) -> bytes; None when no capture of this build matches."""
    try:
        for row in json.load(open(TRAFFIC_TABLE))["rows"]:
            if row["kernel"] == kernel and int(row["rows"]) == int(rows):
                return int(row["dram_bytes"]), row.get("source")
    except (OSError, ValueError, KeyError):
        pass
    return None, None


def ffn_ops(rows):
    return 2.0 * rows * D_MODEL * D_FFN * 2


def gemm_bytes(M, K, N, bias=True):
    """Algorithmic bytes of one quantized linear: fp32 A in, int8 W, scales, fp32 out."""
    return 4 * M * K + N * K + 4 * N + 4 * M * N + (4 * N if bias else 0)


def workload_config(rows_total, shards, world):
    """The `config` object both arms print (the reference arm runs the same workload on the host)."""
    per = [e - b for b, e in shards]
    return {"workload": "ffn_pair_720p", "rows_total": rows_total, "rows_per_gpu": per if world > 1 else per[0],
            "k_n": [D_MODEL, D_FFN],
            "parallelism": "rows split x%d in whole 256-row tiles, weights replicated, no collective" % world,
            "l2": "no flush: a step streams x, both weight matrices, the %d MB intermediate (written, then read) "
                  "and y through the 126 MB L2" % (max(per) * D_FFN * 4 // 1000000)}


# ------------------------------------------------------------------ clocks
class ClockSampler:
    """SM clock, power and throttle reasons of one GPU while the timed region runs: NVML polled
    every few milliseconds from a thread (read-only queries), nvidia-smi every 100 ms where the
    NVML binding is missing."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")
    BITS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index):
        self.rows, self.proc, self.nvml, self.stop_flag = [], None, None, False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index(index))
            self.max_sm = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.t = threading.Thread(target=self._poll, daemon=True)
            self.t.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    @staticmethod
    def _physical_index(index):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v for v in vis.split(",") if v.strip()]
            if index < len(ids) and ids[index].strip().isdigit():
                return int(ids[index])
        return index

    def _poll(self):
        nv = self.nvml
        while not self.stop_flag:
            try:
                sm = float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                watts = nv.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.rows.append((time.time(), sm, watts, mask))
            except Exception:
                pass
            time.sleep(0.004)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0, t1):
        if self.nvml:
            self.stop_flag = True
            self.t.join(timeout=1.0)
            inside = [r for r in self.rows if t0 <= r[0] <= t1] or self.rows[-3:]
            reasons = sorted(n for n, bit in self.BITS.items() if any(r[3] & bit for r in inside))
            return {"sm_mhz": float(np.median([r[1] for r in inside])) if inside else None,
                    "sm_max_mhz": self.max_sm, "reasons": reasons, "samples": len(inside),
                    "power_w": float(np.median([r[2] for r in inside])) if inside else None,
                    "how": "NVML polled every ~5 ms inside the timed region"}
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        inside = [r for (t, r) in self.rows if t0 - 0.05 <= t <= t1 + 0.15] or [r for _, r in self.rows[-3:]]
        sm, mx, reasons, watts = [], None, set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in inside:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
                watts.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm),
                "power_w": float(np.median(watts)) if watts else None,
                "how": "nvidia-smi every 100 ms around the timed region"}


# ------------------------------------------------------------------ reference arm (CPU)
def reference_throughput(A, w1, w2, b1, b2, rows, reps=1):
    """Seconds for the FFN pair on `rows` rows with the reference's own compiled sd::qgemm
    (all host threads); falls back to the oracle port where oracle/_ref is absent."""
    from oracle.binding import Oracle, Reference
    orc = Oracle()
    if Reference.available():
        ref, kind, cores = Reference(), "reference", None
        cores = ref.nthreads()
        qg = ref.qgemm
    else:
        kind, cores, qg = "port", orc.threads(), orc.qgemm
    best = 1e30
    for _ in range(reps):
        t0 = time.perf_counter()
        h = qg(A[:rows], w1[0], w1[1])
        h = orc.gelu_tanh(orc.bias_add(h, b1, inplace=True), inplace=True)
        y = qg(h, w2[0], w2[1])
        y = orc.bias_add(y, b2, inplace=True)
        best = min(best, time.perf_counter() - t0)
    return best, kind, cores


def host_problem(rows, seed=42):
    """Seeded host copy of the workload (weights packed by the oracle's packer arithmetic)."""
    from oracle.binding import Oracle
    orc = Oracle()
    rng = np.random.default_rng(seed)
    A = (rng.standard_normal((rows, D_MODEL)) * 0.5).astype(np.float32)

    def w(n, k):
        bits = orc.f32_to_bf16((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
        return orc.quant_rows_packer(orc.bf16_to_f32(bits))
    w1, w2 = w(D_FFN, D_MODEL), w(D_MODEL, D_FFN)
    b1 = (rng.standard_normal(D_FFN) * 0.02).astype(np.float32)
    b2 = (rng.standard_normal(D_MODEL) * 0.02).astype(np.float32)
    return A, w1, w2, b1, b2


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import __graft_entry__ as ge
    sharding = ge.load_package().sharding
    probe_rows = 64
    A, w1, w2, b1, b2 = host_problem(4096)
    t_probe, kind, cores = reference_throughput(A, w1, w2, b1, b2, probe_rows)
    # size a step so that warmup+steps take about two minutes of CPU time
    budget = float(os.environ.get("SDQ_BENCH_REF_BUDGET_S", "120")) / max(1, args.steps + args.warmup)
    rows = int(max(32, min(4096, probe_rows * budget / t_probe)))
    rows -= rows % 8
    for _ in range(args.warmup):
        reference_throughput(A, w1, w2, b1, b2, rows)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        reference_throughput(A, w1, w2, b1, b2, rows)
    dt = (time.perf_counter() - t0) / args.steps
    tops = ffn_ops(rows) / dt / 1e12
    sample = ("a RATE measured on a sample: the FFN pair on %d of the %d rows per step (the path is linear in the "
              "row count: every row is quantized and multiplied independently, src/core/qgemm.cpp:84-96), "
              "all host threads; ms_per_step is the time of that sample" % (rows, args.rows))
    shards = [sharding.row_shard(args.rows, args.gpus, r) for r in range(args.gpus)]
    line = {"impl": "reference", "metric": "int8_qgemm_throughput", "value": tops, "unit": "TOPS",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "s8",
            "data": "synthetic", "device": "host CPU",
            "config": workload_config(args.rows, shards, args.gpus),
            "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------ B200 arm
def multirank_parity(pkg, s, torch, dist, dev, sp, rank, world):
    """Both exact partitions of one linear, run over the real ranks before anything is timed:
    rows split (every rank its row tiles, no exchange; gathered here only to compare) and columns
    split with the exchange fused into the GEMM epilogue (sdq_qgemm_colsplit: every rank stores its
    column block into all ranks' result buffers).  Each is compared bit for bit with the same
    linear computed whole on this rank's own GPU.  Returns True only if every rank agrees."""
    import ctypes as C
    par, lib = pkg.parallel, s.lib
    g = torch.Generator(device=dev)
    g.manual_seed(1234)                                   # the same problem on every rank
    M, K, N = 2500, 1024, 2048
    A = torch.randn(M, K, device=dev, generator=g)
    q = torch.randint(-127, 128, (N, K), device=dev, dtype=torch.int8, generator=g)
    sc = torch.rand(N, device=dev, generator=g) * 1e-3 + 1e-4
    bias = torch.randn(N, device=dev, generator=g) * 0.02
    w = s.weight_wrap_device(q.data_ptr(), sc.data_ptr(), N, K)
    full = torch.empty(M, N, device=dev)
    s._ck(lib.sdq_qgemm(w, A.data_ptr(), M, full.data_ptr(), bias.data_ptr(), 0, sp))
    # rows
    r0, r1 = pkg.sharding.row_shard(M, world, rank)
    mine = torch.empty(max(r1 - r0, 0), N, device=dev)
    if r1 > r0:
        s._ck(lib.sdq_qgemm(w, A[r0:r1].data_ptr(), r1 - r0, mine.data_ptr(), bias.data_ptr(), 0, sp))
    s.sync(sp)
    rows_ok = bool(torch.equal(par.gather_rows(mine, M).view(torch.int32), full.view(torch.int32)))
    # columns, exchange fused into the epilogue
    n0, n1 = pkg.sharding.col_shard(N, world, rank)
    wq = q[n0:n1].contiguous()
    ws = sc[n0:n1].contiguous()
    bb = bias[n0:n1].contiguous()
    wblk = s.weight_wrap_device(wq.data_ptr(), ws.data_ptr(), n1 - n0, K)
    shared = par.SharedOutput(s, M * N * 4)
    par.qgemm_colsplit_fused(s, wblk, A.data_ptr(), M, N, shared, bias_ptr=bb.data_ptr(), stream=sp)
    s.sync(sp)
    dist.barrier()                                        # every rank's stores have landed
    got = torch.from_numpy(shared.local.to_numpy(np.float32, (M, N))).to(dev)
    cols_ok = bool(torch.equal(got.view(torch.int32), full.view(torch.int32)))
    shared.close()
    s.weight_release(wblk)
    s.weight_release(w)
    ok = torch.tensor([1.0 if (rows_ok and cols_ok) else 0.0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    return bool(ok.item() == 1.0), rows_ok, cols_ok


def dropin_e2e(rows, steps=2):
    """One FFN through libsd_b200.so the way the reference's caller runs it (sd::load_sdcpp views,
    sd::qgemm on host sd::Tensor objects with a fresh output each, bias and GELU passes on the
    host between the two): wall-clock per step from the bench_dropin program, with the page-locked
    tensor pool (the default) and with it switched off."""
    exe = os.path.join(ROOT, "self-evolve-diffusion-cpp_b200", "bench_dropin")
    if not os.path.exists(exe):
        return {"unavailable": "bench_dropin is not built"}
    out = {}
    for label, env in (("pinned_tensor_pool", {}), ("pageable_tensors", {"SD_PINNED_POOL_MB": "0"})):
        try:
            r = subprocess.run([exe, str(rows), str(steps)], capture_output=True, text=True, timeout=600,
                               env=dict(os.environ, **env))
            out[label] = json.loads(r.stdout.strip().splitlines()[-1]) if r.returncode == 0 else \
                {"failed": (r.stderr or r.stdout)[-300:]}
        except Exception as e:  # the figure is a secondary one: report, do not abort the bench line
            out[label] = {"failed": repr(e)}
    best = out.get("pinned_tensor_pool", {})
    if "ms_per_step" in best:
        out["value"], out["unit"], out["ms_per_step"] = best["tops"], "TOPS", best["ms_per_step"]
        out["h2d_bytes_per_step"], out["d2h_bytes_per_step"] = best["h2d_bytes_per_step"], best["d2h_bytes_per_step"]
    out["what"] = ("sd::qgemm of libsd_b200.so on host sd::Tensor buffers, FFN = qgemm -> host bias + GELU -> qgemm -> "
                   "host bias, output tensor allocated per call; wall clock, %d steps after one warm-up" % steps)
    return out


def run_b200(args):
    import ctypes as C

    import torch
    import torch.distributed as dist

    import __graft_entry__ as ge

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d: launch N>1 with torch.distributed.run" % (args.gpus, world))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = ge.load_package()
    s = pkg.Sdq(local)
    S = pkg.sdq
    lib = s.lib
    dev = torch.device("cuda", local)
    stream = torch.cuda.current_stream()
    sp = C.c_void_p(stream.cuda_stream)
    M_total = args.rows
    shards = [pkg.sharding.row_shard(M_total, world, r) for r in range(world)]
    M = shards[rank][1] - shards[rank][0]              # this rank's rows (strong scaling)

    def ck(rc):
        s._ck(rc)

    parity = None
    if world > 1 and not args.no_parity:
        parity = multirank_parity(pkg, s, torch, dist, dev, sp, rank, world)
        if not parity[0]:
            raise SystemExit("multi-rank parity failed on rank %d: rows %s, columns %s" % (rank, parity[1], parity[2]))

    # ---- synthetic problem, resident in HBM before any timing starts
    g = torch.Generator(device=dev)
    g.manual_seed(42)                                  # weights: the same on every rank (replicated)

    def packed(n, k):
        wb = (torch.randn(n, k, device=dev, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        q = torch.empty(n, k, device=dev, dtype=torch.int8)
        sc = torch.empty(n, device=dev, dtype=torch.float32)
        ck(lib.sdq_quantize_rows(wb.data_ptr(), S.BF16, n, k, S.MODE_PACKER, q.data_ptr(), sc.data_ptr(), 0, sp))
        return q, sc, s.weight_wrap_device(q.data_ptr(), sc.data_ptr(), n, k)
    q1, s1, w1 = packed(D_FFN, D_MODEL)
    q2, s2, w2 = packed(D_MODEL, D_FFN)
    b1 = torch.randn(D_FFN, device=dev, generator=g) * 0.02
    b2 = torch.randn(D_MODEL, device=dev, generator=g) * 0.02
    g.manual_seed(1000 + rank)                         # activations: this rank's rows
    Mb = max(M, 1)
    A = torch.randn(Mb, D_MODEL, device=dev, generator=g, dtype=torch.float32) * 0.5
    H = torch.empty(Mb, D_FFN, device=dev, dtype=torch.float32)
    Y = torch.empty(Mb, D_MODEL, device=dev, dtype=torch.float32)
    aq = torch.empty(Mb * D_FFN, device=dev, dtype=torch.int8)
    a_s = torch.empty(Mb, device=dev, dtype=torch.float32)

    def ev():
        return torch.cuda.Event(enable_timing=True)

    def step():
        # the pair as one call of the public entry point: nothing between its launches, so the
        # GEMMs' prologues overlap the quantize kernels' tails (programmatic dependent launch)
        ck(lib.sdq_ffn_pair(w1, b1.data_ptr(), w2, b2.data_ptr(), A.data_ptr(), M, H.data_ptr(), Y.data_ptr(), 0, sp))

    def marked_step(marks):
        # the same four kernels as separate calls with an event between them: per-kernel times
        def mark():
            e = ev()
            e.record(stream)
            marks.append(e)
        mark()
        ck(lib.sdq_quantize_activations(A.data_ptr(), M, D_MODEL, aq.data_ptr(), a_s.data_ptr(), sp))
        mark()
        ck(lib.sdq_qgemm_prequantized(w1, aq.data_ptr(), a_s.data_ptr(), M, H.data_ptr(), b1.data_ptr(),
                                      None, S.GELU_TANH, sp))
        mark()
        ck(lib.sdq_quantize_activations(H.data_ptr(), M, D_FFN, aq.data_ptr(), a_s.data_ptr(), sp))
        mark()
        ck(lib.sdq_qgemm_prequantized(w2, aq.data_ptr(), a_s.data_ptr(), M, Y.data_ptr(), b2.data_ptr(),
                                      None, 0, sp))
        mark()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warm = max(3, args.warmup)
    for _ in range(warm):
        step()
    s.sync(sp)
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    launches0 = s.launches()
    e0, e1 = ev(), ev()
    t_wall0 = time.time()
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    barrier()
    t_wall1 = time.time()
    launches = s.launches() - launches0
    s.sync(sp)                                   # also surfaces a device-side timeout
    ms_total = e0.elapsed_time(e1)
    t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    ms_step = ms_total / args.steps
    clocks = sampler.stop(t_wall0, t_wall1) if sampler else None

    # per-kernel durations from a separate pass (events between the launches), mean over its steps
    n_marked = max(3, min(args.steps, 20))
    marks_all = []
    for _ in range(n_marked):
        m = []
        marked_step(m)
        marks_all.append(m)
    barrier()
    names = ["act_quant_k3072", "gemm_up_3072x14336", "act_quant_k14336", "gemm_down_14336x3072"]
    kern_ms = {n: float(np.mean([m[i].elapsed_time(m[i + 1]) for m in marks_all])) for i, n in enumerate(names)}
    marked_step_ms = float(np.mean([m[0].elapsed_time(m[4]) for m in marks_all]))

    # ---- end to end through the host-pointer C ABI call: pinned host in, pinned host out
    e2e = None
    if not args.no_e2e:
        hA = torch.empty(Mb, D_MODEL, dtype=torch.float32, pin_memory=True)
        hA.copy_(A)
        hY = torch.empty(Mb, D_MODEL, dtype=torch.float32, pin_memory=True)

        def e2e_step():
            # the public call for the pair: host x in, host y out, copies inside the call
            ck(lib.sdq_ffn_pair(w1, b1.data_ptr(), w2, b2.data_ptr(), hA.data_ptr(), M, None, hY.data_ptr(),
                                S.A_HOST | S.OUT_HOST, sp))
        n_e2e = max(3, min(args.steps, 10))
        for _ in range(3):
            e2e_step()
        barrier()
        a0, a1 = ev(), ev()
        a0.record(stream)
        for _ in range(n_e2e):
            e2e_step()
        a1.record(stream)
        barrier()
        te = torch.tensor([a0.elapsed_time(a1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_ms = float(te.item()) / n_e2e
        e2e = {"value": ffn_ops(M_total) / (e2e_ms * 1e-3) / 1e12, "unit": "TOPS",
               "h2d_bytes_per_step": 4 * M_total * D_MODEL, "d2h_bytes_per_step": 4 * M_total * D_MODEL,
               "ms_per_step": e2e_ms, "steps": n_e2e,
               "what": "sdq_ffn_pair with pinned host x and y (chunked upload / arithmetic / download pipeline)"}
        assert torch.isfinite(hY).all()
        del hA, hY

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0

    pk, pk_kind = peaks()
    peak, peak_kind = int8_peak(pk, pk_kind, ms_total * 1e-3)
    dom = "gemm_up_3072x14336"
    dom_ops = 2.0 * M * D_MODEL * D_FFN
    achieved = dom_ops / (kern_ms[dom] * 1e-3) / 1e12
    traffic, traffic_src = dram_traffic("qgemm_tc2_kernel 3072x14336 bias+gelu", M)
    value = ffn_ops(M_total) / (ms_step * 1e-3) / 1e12
    hbm = float(pk.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    roofline = {"bound": "tensor", "kernel": "qgemm_tc2_kernel " + dom, "achieved": achieved, "peak": peak,
                "unit": "TFLOP/s", "unit_note": "tera int8 operations per second (2*M*N*K), i.e. TOPS",
                "frac": achieved / peak, "traffic": traffic, "traffic_source": traffic_src,
                "peak_kind": peak_kind,
                "step_frac": value / world / peak,
                "step_frac_what": "the whole FFN pair per GPU (both quantize launches included) over the same peak",
                "frac_of_2x_bf16_sustained": achieved / (2.0 * float(pk.get("bf16_tflops_sustained",
                                                                            FALLBACK_PEAKS["bf16_tflops_sustained"]))),
                "frac_of_nominal_int8_4500": achieved / INT8_NOMINAL_TOPS,
                "step_frac_of_nominal_int8_4500": value / world / INT8_NOMINAL_TOPS,
                "algorithmic_bytes": gemm_bytes(M, D_MODEL, D_FFN),
                "kernel_ms": kern_ms, "kernel_ms_from": "a separate pass of %d steps with an event between the "
                                                       "launches (%.4f ms per step there)" % (n_marked, marked_step_ms),
                "gemm_down_frac": 2.0 * M * D_MODEL * D_FFN / (kern_ms["gemm_down_14336x3072"] * 1e-3) / 1e12 / peak,
                "hbm_frac_act_quant_k14336": (5.0 * M * D_FFN + 4 * M) / (kern_ms["act_quant_k14336"] * 1e-3) / 1e9 / hbm,
                "hbm_frac_act_quant_k3072": (5.0 * M * D_MODEL + 4 * M) / (kern_ms["act_quant_k3072"] * 1e-3) / 1e9 / hbm}

    # the device's own MMA-issue-bound int8 rate, measured now (burst: one 2 ms launch on an
    # idle GPU; sustained: back-to-back launches for ~3 s, median of the last half)
    if not args.no_peak_probe:
        time.sleep(1.0)
        burst = max(s.int8_mma_probe(2000)[1] for _ in range(3))
        t_end, rates = time.time() + 3.0, []
        while time.time() < t_end:
            rates.append(s.int8_mma_probe(20000)[1])
        sustained = float(np.median(rates[len(rates) // 2:]))
        roofline["int8_mma_peak_measured"] = {"burst_tops": burst, "sustained_tops": sustained,
                                              "how": "tcgen05.mma kind::i8 128x256x32 issued back to back "
                                                     "from shared memory on all SMs (sdq_int8_mma_probe)"}
        roofline["frac_of_int8_mma_probe"] = achieved / (burst if ms_total < 1000.0 else sustained)

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        hostA, hw1, hw2, hb1, hb2 = host_problem(2048)
        tp, kind, cores = reference_throughput(hostA, hw1, hw2, hb1, hb2, 64)
        rows = int(max(64, min(2048, 64 * 12.0 / tp)))       # about 12 s of CPU work
        rows -= rows % 8
        tt, kind, cores = reference_throughput(hostA, hw1, hw2, hb1, hb2, rows)
        cpu = {"value": ffn_ops(rows) / tt / 1e12, "unit": "TOPS", "cores": cores, "kind": kind,
               "sample": "FFN pair on %d of %d rows, one pass, reference sd::qgemm on all host threads" % (rows, M_total)}

    line = {"metric": "int8_qgemm_throughput", "value": value, "unit": "TOPS", "n_gpus": world,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "s8",
            "data": "synthetic",
            "config": workload_config(M_total, shards, world),
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "roofline": roofline,
            "cpu_baseline": cpu}
    if parity is not None:
        line["multirank_parity"] = parity[0]
        line["multirank_parity_what"] = ("before timing, on the %d ranks: row split and column split with the exchange "
                                         "fused into the GEMM epilogue (peer stores), each bit-equal to the unsplit "
                                         "linear" % world)
    if world == 1 and not args.no_dropin:
        del A, H, Y, aq
        torch.cuda.empty_cache()
        line["e2e_dropin"] = dropin_e2e(M_total)
    if world == 1 and not args.no_block:
        line["block_720p"] = measure_block(pkg, s, torch, rows=M_total, steps=3, warmup=1, with_attention=True)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


# ------------------------------------------------------------------ shape sweep
SWEEP_KN = [(3072, 3072), (3072, 9216), (3072, 14336), (14336, 3072), (3072, 18432)]
SWEEP_M = [192, 1024, 4096, 16384, 27280, 54560]


def run_sweep(args):
    """Every DiT linear (K,N) over the token counts of the shape sweep; rows split over the
    ranks (total work fixed), whole sd::qgemm per point = quantize launch + GEMM launch.
    L2 is flushed (256 MiB write) before every timed call.  One JSON line, key "sweep"."""
    import ctypes as C

    import torch
    import torch.distributed as dist

    import __graft_entry__ as ge

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = ge.load_package()
    s = pkg.Sdq(local)
    S, lib = pkg.sdq, s.lib
    dev = torch.device("cuda", local)
    stream = torch.cuda.current_stream()
    sp = C.c_void_p(stream.cuda_stream)
    g = torch.Generator(device=dev)
    g.manual_seed(7 + rank)
    flush = torch.empty(256 << 20, device=dev, dtype=torch.uint8)
    pk, pk_kind = peaks()
    hbm = float(pk.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    tens, tens_kind = int8_peak(pk, pk_kind, 0.0)      # single calls on a flushed L2: the burst figure
    points = []
    for (K, N) in SWEEP_KN:
        wb = (torch.randn(N, K, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        q = torch.empty(N, K, device=dev, dtype=torch.int8)
        sc = torch.empty(N, device=dev, dtype=torch.float32)
        s._ck(lib.sdq_quantize_rows(wb.data_ptr(), S.BF16, N, K, S.MODE_PACKER, q.data_ptr(), sc.data_ptr(), 0, sp))
        w = s.weight_wrap_device(q.data_ptr(), sc.data_ptr(), N, K)
        for Mtot in SWEEP_M:
            r0, r1 = pkg.sharding.row_shard(Mtot, world, rank)
            M = r1 - r0
            A = torch.randn(max(M, 1), K, device=dev, generator=g)
            out = torch.empty(max(M, 1), N, device=dev)
            times = []
            for it in range(2 + args.steps):
                flush.zero_()
                if world > 1:
                    dist.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                s._ck(lib.sdq_qgemm(w, A.data_ptr(), M, out.data_ptr(), None, 0, sp))
                e1.record(stream)
                torch.cuda.synchronize()
                if it >= 2:
                    times.append(e0.elapsed_time(e1))
            t = torch.tensor([float(np.median(times))], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            ops = 2.0 * Mtot * N * K
            byts = gemm_bytes(Mtot, K, N, bias=False)
            t_tensor = ops / (tens * 1e12 * world) * 1e3
            t_hbm = byts / (hbm * 1e9 * world) * 1e3
            points.append({"K": K, "N": N, "M": Mtot, "ms": ms, "tops": ops / (ms * 1e-3) / 1e12,
                           "bound": "tensor" if t_tensor >= t_hbm else "hbm",
                           "frac_of_bound": max(t_tensor, t_hbm) / ms})
            del A, out
        s.weight_release(w)
        del wb, q, sc
    # column split + all-gather at the largest token count: every rank holds N/world weight
    # rows and all of A, computes out[:, n0:n1]; the blocks are all-gathered (NCCL) into [M, N]
    nsplit = []
    if world > 1:
        par = pkg.parallel
        Mtot = SWEEP_M[-1]
        for (K, N) in SWEEP_KN:
            n0, n1 = pkg.sharding.col_shard(N, world, rank)
            wb = (torch.randn(n1 - n0, K, device=dev, generator=g) * 0.02).to(torch.bfloat16)
            q = torch.empty(n1 - n0, K, device=dev, dtype=torch.int8)
            sc = torch.empty(n1 - n0, device=dev, dtype=torch.float32)
            s._ck(lib.sdq_quantize_rows(wb.data_ptr(), S.BF16, n1 - n0, K, S.MODE_PACKER, q.data_ptr(),
                                        sc.data_ptr(), 0, sp))
            w = s.weight_wrap_device(q.data_ptr(), sc.data_ptr(), n1 - n0, K)
            A = torch.randn(Mtot, K, device=dev, generator=g)
            block = torch.empty(Mtot, n1 - n0, device=dev)
            tg, ta = [], []
            for it in range(1 + args.steps):
                flush.zero_()
                dist.barrier()
                e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
                e0.record(stream)
                s._ck(lib.sdq_qgemm(w, A.data_ptr(), Mtot, block.data_ptr(), None, 0, sp))
                e1.record(stream)
                full = par.allgather_columns(block, N)
                e2.record(stream)
                torch.cuda.synchronize()
                if it >= 1:
                    tg.append(e0.elapsed_time(e1))
                    ta.append(e1.elapsed_time(e2))
                del full
            # fused form: the GEMM epilogue stores the block into every rank's [M, N] buffer;
            # timed to the end of a 1-element all-reduce that orders the ranks on the stream
            shared = par.SharedOutput(s, Mtot * N * 4)
            tok = torch.zeros(1, device=dev)
            tf = []
            for it in range(1 + args.steps):
                flush.zero_()
                dist.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                par.qgemm_colsplit_fused(s, w, A.data_ptr(), Mtot, N, shared, stream=sp)
                dist.all_reduce(tok)
                e1.record(stream)
                torch.cuda.synchronize()
                if it >= 1:
                    tf.append(e0.elapsed_time(e1))
            shared.close()
            t = torch.tensor([float(np.median(tg)), float(np.median(ta)), float(np.median(tf))], device=dev,
                             dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            nsplit.append({"K": K, "N": N, "M": Mtot, "gemm_ms": float(t[0]), "allgather_ms": float(t[1]),
                           "fused_peer_store_ms": float(t[2]),
                           "gathered_bytes_per_rank": 4 * Mtot * N * (world - 1) // world,
                           "tops_gemm_then_allgather": 2.0 * Mtot * N * K / (float(t[0] + t[1]) * 1e-3) / 1e12,
                           "tops_fused": 2.0 * Mtot * N * K / (float(t[2]) * 1e-3) / 1e12})
            s.weight_release(w)
            del wb, q, sc, A, block
    s.sync(sp)
    if rank == 0:
        total_ops = sum(2.0 * p["M"] * p["N"] * p["K"] for p in points)
        total_ms = sum(p["ms"] for p in points)
        print(json.dumps({"metric": "int8_qgemm_throughput", "value": total_ops / (total_ms * 1e-3) / 1e12,
                          "unit": "TOPS", "n_gpus": world, "steps": args.steps, "warmup": 2,
                          "ms_per_step": total_ms, "higher_is_better": True, "scaling": "strong",
                          "vs_baseline": None, "dtype": "s8", "data": "synthetic",
                          "config": {"workload": "dit_linear_shape_sweep", "points": len(points),
                                     "l2": "flushed with a 256 MiB write before every timed call",
                                     "peaks": "bound = max(2MNK / (" + tens_kind + "), bytes / HBM copy of " +
                                              pk_kind + ")"},
                          "sweep": points, "column_split_allgather": nsplit}))
    if world > 1:
        dist.destroy_process_group()
    return 0


# ------------------------------------------------------------------ whole branch
# linears of one DiT block (name, K, N, rows: None = this branch's tokens, "other" = the other
# branch's tokens, a number = that many rows), reference src/model/ovi_dit.cpp:490-536
BLOCK_LINEARS = [("self_attn.qkv", 3072, 9216, None), ("self_attn.o", 3072, 3072, None),
                 ("cross_attn.q", 3072, 3072, None), ("cross_attn.k", 3072, 3072, 512),
                 ("cross_attn.v", 3072, 3072, 512), ("cross_attn.o", 3072, 3072, None),
                 ("ffn.0", 3072, 14336, None), ("ffn.2", 14336, 3072, None)]
# the audio branch has the same linears on its own (few) tokens, and its fusion K/V projections
# read the VIDEO tokens (src/model/ovi_dit.cpp:229-256, :530-531)
AUDIO_BLOCK_LINEARS = BLOCK_LINEARS + [("cross_attn.k_fusion", 3072, 3072, "other"),
                                       ("cross_attn.v_fusion", 3072, 3072, "other")]
AUDIO_TOKENS = 157   # 5 s of 16 kHz audio at one latent per 512 samples


def run_branch(args):
    """A random-init 5B-parameter DiT branch: 30 blocks of int8 linears.  Phase 1 packs the bf16
    weights to the .sdcpp int8 layout on the GPU; the packed bytes and scales of the first
    --verify-blocks blocks (default: all) are compared with the CPU packer's byte for byte, and a
    SHA-256 over everything compared is printed for both sides.  Phase 2 runs every linear once at
    M = --rows video tokens (K/V projections at 512 text tokens).  With --audio the audio branch
    follows on the same ranks (its own 157 tokens, fusion K/V on the video tokens).  Rows are split
    over the ranks in whole tiles; no collective; one JSON line."""
    import ctypes as C
    import hashlib

    import torch
    import torch.distributed as dist

    import __graft_entry__ as ge

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = ge.load_package()
    s = pkg.Sdq(local)
    S, lib = pkg.sdq, s.lib
    dev = torch.device("cuda", local)
    stream = torch.cuda.current_stream()
    sp = C.c_void_p(stream.cuda_stream)
    g = torch.Generator(device=dev)
    g.manual_seed(5)                                   # the same weights on every rank (replicated)
    blocks = args.blocks

    def ev():
        return torch.cuda.Event(enable_timing=True)

    def local_rows(total):
        r0, r1 = pkg.sharding.row_shard(total, world, rank)
        return r1 - r0

    branches = [("video", BLOCK_LINEARS, args.rows, AUDIO_TOKENS)]
    if args.audio:
        branches.append(("audio", AUDIO_BLOCK_LINEARS, AUDIO_TOKENS, args.rows))
    M_max = max(local_rows(args.rows), 1)
    x = torch.randn(M_max, 3072, device=dev, generator=g)
    xf = torch.randn(M_max, 14336, device=dev, generator=g)
    xt = torch.randn(512, 3072, device=dev, generator=g)
    out = torch.empty(M_max * 14336, device=dev)
    orc = None
    results, load = [], None
    for (bname, linears, own_tokens, other_tokens) in branches:
        weights, pack_elems, verified = [], 0, 0
        sha_gpu, sha_cpu = hashlib.sha256(), hashlib.sha256()
        # the branch's bf16 weights, then ONE timed sweep of the packer over all of them (launches
        # back to back, as a packer run over a checkpoint makes them), then the comparison
        srcs = []
        for b in range(blocks):
            for (name, K, N, rows) in linears:
                wb = (torch.randn(N, K, device=dev, generator=g) * 0.02).to(torch.bfloat16)
                q = torch.empty(N, K, device=dev, dtype=torch.int8)
                sc = torch.empty(N, device=dev, dtype=torch.float32)
                srcs.append((b, name, K, N, rows, wb, q, sc))
                pack_elems += N * K
        torch.cuda.synchronize()
        e0, e1 = ev(), ev()
        e0.record(stream)
        for (b, name, K, N, rows, wb, q, sc) in srcs:
            s._ck(lib.sdq_quantize_rows(wb.data_ptr(), S.BF16, N, K, S.MODE_PACKER, q.data_ptr(), sc.data_ptr(), 0, sp))
        e1.record(stream)
        torch.cuda.synchronize()
        pack_ms = e0.elapsed_time(e1)
        for (b, name, K, N, rows, wb, q, sc) in srcs:
            if rank == 0 and b < args.verify_blocks:
                if orc is None:
                    from oracle.binding import Oracle
                    orc = Oracle()
                bits = wb.view(torch.int16).cpu().numpy().view(np.uint16)
                q_c, s_c = orc.quant_rows_packer(orc.bf16_to_f32(bits))
                q_g, s_g = q.cpu().numpy().tobytes(), sc.cpu().numpy().tobytes()
                if q_g != q_c.tobytes() or s_g != s_c.tobytes():
                    raise SystemExit("packed bytes of %s block %d %s differ from the CPU packer" % (bname, b, name))
                for h, parts in ((sha_gpu, (q_g, s_g)), (sha_cpu, (q_c.tobytes(), s_c.tobytes()))):
                    for part in parts:
                        h.update(part)
                verified += 1
            weights.append((K, N, rows, q, sc, s.weight_wrap_device(q.data_ptr(), sc.data_ptr(), N, K)))
        del srcs, wb
        torch.cuda.empty_cache()
        # optional: write the first blocks as a .sdcpp file and time open + validate + upload
        if rank == 0 and args.pack_file_blocks > 0 and load is None:
            import struct
            import tempfile
            nb = min(args.pack_file_blocks, blocks) * len(linears)
            path = os.path.join(tempfile.gettempdir(), "sdq_bench_branch.sdcpp")
            entries, off = [], 0
            for i in range(nb):
                K, N = weights[i][0], weights[i][1]
                entries.append(("blocks.%d.%s.weight" % (i // len(linears), linears[i % len(linears)][0]), N, K, off))
                off += N * K + 4 * N
            with open(path, "wb") as f:
                f.write(b"SDCP" + struct.pack("<II", 1, nb))
                for name, N, K, o in entries:
                    f.write(struct.pack("<I", len(name)) + name.encode() + struct.pack("<BI", 0, 2) + struct.pack("<qqQ", N, K, o))
                for i in range(nb):
                    f.write(weights[i][3].cpu().numpy().tobytes())
                    f.write(weights[i][4].cpu().numpy().tobytes())
            nbytes = os.path.getsize(path)
            times = []
            for _ in range(3):
                t0 = time.perf_counter()
                pack = s.open_pack(path, upload=True)
                s.sync(None)
                times.append(time.perf_counter() - t0)
                pinned = pack.pinned()
                n_ent = len(pack.entries())
                pack.close()
            os.remove(path)
            load = {"file_bytes": nbytes, "entries": n_ent, "seconds_best": min(times), "seconds_first": times[0],
                    "gb_per_s": nbytes / min(times) / 1e9, "mapping_page_locked": pinned}
        M_own, M_other = local_rows(own_tokens), local_rows(other_tokens)

        def forward():
            ops = 0.0
            for (K, N, rows, q, sc, w) in weights:
                if rows is None:
                    a, m, total = (x if K == 3072 else xf), M_own, own_tokens
                elif rows == "other":
                    a, m, total = x, M_other, other_tokens
                else:
                    a, m, total = xt, (rows if rank == 0 else 0), rows   # the text K/V rows are not worth splitting
                if m:
                    s._ck(lib.sdq_qgemm(w, a.data_ptr(), m, out.data_ptr(), None, 0, sp))
                ops += 2.0 * total * N * K
            return ops
        forward()
        s.sync(sp)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        n0 = s.launches()
        e0, e1 = ev(), ev()
        e0.record(stream)
        for _ in range(args.steps):
            ops = forward()
        e1.record(stream)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        s.sync(sp)
        t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        results.append({"branch": bname, "tokens": own_tokens, "ms": float(t.item()), "ops": ops,
                        "tops": ops / (float(t.item()) * 1e-3) / 1e12, "launches": (s.launches() - n0) // args.steps,
                        "int8_params": pack_elems, "pack_ms": pack_ms, "tensors_verified_against_cpu_packer": verified,
                        "sha256_gpu_packed": sha_gpu.hexdigest() if verified else None,
                        "sha256_cpu_packed": sha_cpu.hexdigest() if verified else None})
        for wt in weights:
            s.weight_release(wt[5])
        del weights
        torch.cuda.empty_cache()
    if rank == 0:
        pk, pk_kind = peaks()
        hbm = float(pk.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
        ms = sum(r["ms"] for r in results)
        ops = sum(r["ops"] for r in results)
        pack_elems = sum(r["int8_params"] for r in results)
        pack_ms = sum(r["pack_ms"] for r in results)
        pack_gbs = (3.0 * pack_elems) / (pack_ms * 1e-3) / 1e9
        print(json.dumps({"metric": "int8_qgemm_throughput", "value": ops / (ms * 1e-3) / 1e12, "unit": "TOPS",
                          "n_gpus": world, "steps": args.steps, "warmup": 1, "ms_per_step": ms,
                          "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "s8",
                          "data": "synthetic",
                          "config": {"workload": "dit_branch_all_linears", "blocks": blocks, "rows": args.rows,
                                     "branches": [r["branch"] for r in results], "int8_params": pack_elems,
                                     "parallelism": "each branch's rows split x%d in whole tiles, branches back to back, "
                                                    "weights replicated, no collective" % world},
                          "gpu_launches": sum(r["launches"] for r in results) * args.steps,
                          "branches": results,
                          "pack": {"elements": pack_elems, "ms": pack_ms, "gb_per_s": pack_gbs,
                                   "roofline": {"bound": "hbm", "achieved": pack_gbs, "peak": hbm, "unit": "GB/s",
                                                "frac": pack_gbs / hbm, "of": pk_kind},
                                   "tensors_verified_against_cpu_packer": sum(r["tensors_verified_against_cpu_packer"]
                                                                              for r in results)},
                          "pack_load": load}))
    if world > 1:
        dist.destroy_process_group()
    return 0


def measure_block(pkg, s, torch, rows, steps, warmup, with_attention):
    """One DiT block's int8 linears at M = rows tokens (K/V of the text cross-attention at 512
    rows) in three call patterns: (a) eight bare sdq_qgemm calls; (b) the reference's call pattern
    with every pass it runs around the linears -- layernorm, modulation, bias adds, GELU, gated and
    plain residual adds -- as separate elementwise passes (torch) around bare sdq_qgemm calls;
    (c) the same work through the fused entry points (layernorm + modulation + quantize once for
    q/k/v, bias / GELU / residual in the GEMM epilogues, sdq_ffn_block).  With attention, pattern
    (c) also runs the block's self-attention and text cross-attention (sdq_sdpa).  Returns the
    fields of the JSON line."""
    import ctypes as C

    import types
    args = types.SimpleNamespace(rows=rows, steps=steps, warmup=warmup, with_attention=with_attention)
    S, lib = pkg.sdq, s.lib
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream()
    sp = C.c_void_p(stream.cuda_stream)
    g = torch.Generator(device=dev)
    g.manual_seed(7)
    M, D, F, T = args.rows, D_MODEL, D_FFN, 512

    def p(t):
        return C.c_void_p(t.data_ptr())

    def weight(n, k):
        q = torch.randint(-127, 128, (n, k), device=dev, dtype=torch.int8, generator=g)
        sc = torch.rand(n, device=dev, generator=g) * 2e-4 + 1e-5
        return (q, sc, s.weight_wrap_device(q.data_ptr(), sc.data_ptr(), n, k),
                torch.randn(n, device=dev, generator=g) * 0.02)
    W = {name: weight(N, K) for (name, K, N, _) in BLOCK_LINEARS}
    x = torch.randn(M, D, device=dev, generator=g)
    att = torch.randn(M, D, device=dev, generator=g)        # stands in for the attention outputs
    ctx = torch.randn(T, D, device=dev, generator=g)
    e = torch.randn(6, D, device=dev, generator=g) * 0.1     # modulation table of the block
    ln3_w = 1 + torch.randn(D, device=dev, generator=g) * 0.1
    ln3_b = torch.randn(D, device=dev, generator=g) * 0.1
    qkv = torch.empty(M, 3 * D, device=dev)
    y = torch.empty(M, D, device=dev)
    kv = torch.empty(T, D, device=dev)
    hid = torch.empty(M, F, device=dev)
    aq = torch.empty(M, D, device=dev, dtype=torch.int8)
    a_s = torch.empty(M, device=dev)
    aqt = torch.empty(T, D, device=dev, dtype=torch.int8)
    a_st = torch.empty(T, device=dev)

    def lin(name, a, m, out, bias=False, flags=0):
        s._ck(lib.sdq_qgemm(W[name][2], p(a), m, p(out), p(W[name][3]) if bias else None, flags, sp))

    def pre(name, q8, sc, m, out, flags=0):
        s._ck(lib.sdq_qgemm_prequantized(W[name][2], p(q8), p(sc), m, p(out), p(W[name][3]), None, flags, sp))

    def bare():
        for name, a, m, out in (("self_attn.qkv", x, M, qkv), ("self_attn.o", att, M, y),
                                ("cross_attn.q", x, M, y), ("cross_attn.k", ctx, T, kv),
                                ("cross_attn.v", ctx, T, kv), ("cross_attn.o", att, M, y),
                                ("ffn.0", x, M, hid), ("ffn.2", hid, M, y)):
            lin(name, a, m, out)

    def lin_bias(name, a, m, out):
        lin(name, a, m, out)
        out.add_(W[name][3])                              # mlin's separate bias pass

    def unfused(xx):
        ln = torch.nn.functional.layer_norm
        h = ln(xx, (D,)) * (1 + e[1]) + e[0]
        lin_bias("self_attn.qkv", h, M, qkv)
        lin_bias("self_attn.o", att, M, y)
        xx.addcmul_(y, e[2])
        h = ln(xx, (D,), ln3_w, ln3_b)
        lin_bias("cross_attn.q", h, M, y)
        lin_bias("cross_attn.k", ctx, T, kv)
        lin_bias("cross_attn.v", ctx, T, kv)
        lin_bias("cross_attn.o", att, M, y)
        xx.add_(y)
        h = ln(xx, (D,)) * (1 + e[4]) + e[3]
        lin_bias("ffn.0", h, M, hid)
        hid.copy_(torch.nn.functional.gelu(hid, approximate="tanh"))
        lin_bias("ffn.2", hid, M, y)
        xx.addcmul_(y, e[5])

    heads = D // 128
    qs, ks, vs = [torch.empty(M, D, device=dev) for _ in range(3)] if args.with_attention else (None, None, None)
    kv2 = torch.empty(T, D, device=dev) if args.with_attention else None

    def fused(xx):
        eps = C.c_float(1e-6)
        s._ck(lib.sdq_layernorm_mod_quantize(p(xx), M, D, p(e[0]), p(e[1]), eps, p(aq), p(a_s), None, 0, sp))
        pre("self_attn.qkv", aq, a_s, M, qkv)
        if args.with_attention:      # self-attention over the M tokens.  The three copies stand in for
            # the caller's q/k RMSNorm and RoPE passes, which read the projections and write q, k, v
            qs.copy_(qkv[:, :D])
            ks.copy_(qkv[:, D:2 * D])
            vs.copy_(qkv[:, 2 * D:])
            s._ck(lib.sdq_sdpa(p(qs), p(ks), p(vs), M, M, D, heads, p(att), 0, sp))
        s._ck(lib.sdq_qgemm_residual(W["self_attn.o"][2], p(att), M, p(xx), p(e[2]), p(xx), p(W["self_attn.o"][3]), 0, sp))
        s._ck(lib.sdq_layernorm_mod_quantize(p(xx), M, D, p(ln3_b), p(ln3_w), eps, p(aq), p(a_s), None, S.LN_AFFINE, sp))
        pre("cross_attn.q", aq, a_s, M, y)
        s._ck(lib.sdq_quantize_activations(p(ctx), T, D, p(aqt), p(a_st), sp))
        pre("cross_attn.k", aqt, a_st, T, kv)
        pre("cross_attn.v", aqt, a_st, T, kv2 if args.with_attention else kv)
        if args.with_attention:      # cross-attention on the 512 text tokens
            s._ck(lib.sdq_sdpa(p(y), p(kv), p(kv2), M, T, D, heads, p(att), 0, sp))
        s._ck(lib.sdq_qgemm_residual(W["cross_attn.o"][2], p(att), M, p(xx), None, p(xx), p(W["cross_attn.o"][3]), 0, sp))
        s._ck(lib.sdq_ffn_block(W["ffn.0"][2], p(W["ffn.0"][3]), W["ffn.2"][2], p(W["ffn.2"][3]), p(xx), M,
                                p(e[3]), p(e[4]), p(e[5]), eps, 0, sp))

    def timed(fn):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        n0 = s.launches()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        s.sync(sp)
        return e0.elapsed_time(e1) / args.steps, (s.launches() - n0) // args.steps
    # the two in-place patterns agree within the GELU bound on the same input
    agree = None
    if not args.with_attention:    # (with attention the fused pattern computes more than the unfused one)
        xa, xb = x.clone(), x.clone()
        unfused(xa)
        fused(xb)
        torch.cuda.synchronize()
        agree = float((xa - xb).abs().max() / xa.abs().max())
    ops = sum(2.0 * (M if rows is None else rows) * N * K for (_, K, N, rows) in BLOCK_LINEARS)
    xw = x.clone()
    t_bare, l_bare = timed(bare)
    t_unf, l_unf = timed(lambda: unfused(xw))
    xw.copy_(x)
    t_fus, l_fus = timed(lambda: fused(xw))
    for (_, _, wh, _) in W.values():
        s.weight_release(wh)
    return ({"metric": "int8_qgemm_throughput", "value": ops / (t_fus * 1e-3) / 1e12, "unit": "TOPS",
                      "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": t_fus,
                      "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s8",
                      "data": "synthetic",
                      "config": {"workload": "dit_block_linears_fused_call_pattern", "rows": M,
                                 "l2": "inputs larger than L2 (x %d MB)" % (M * D * 4 // 1000000)},
                      "gpu_launches": l_fus * args.steps,
                      "patterns_ms": {"bare_linears": t_bare, "unfused_with_elementwise_passes": t_unf,
                                      "fused_entry_points": t_fus},
                      "launches_per_block": {"bare_linears": l_bare, "unfused_own_kernels": l_unf, "fused": l_fus},
                      "fused_pattern_includes_attention": bool(args.with_attention),
                      "fused_vs_unfused_max_rel_diff": agree})


def run_block(args):
    """--workload block: measure_block on one GPU, one JSON line."""
    import torch

    import __graft_entry__ as ge

    torch.cuda.set_device(0)
    pkg = ge.load_package()
    s = pkg.Sdq(0)
    print(json.dumps(measure_block(pkg, s, torch, args.rows, args.steps, args.warmup, args.with_attention)))
    return 0


def run_fp32(args):
    """The two fp32 kernels beside the int8 linears of a DiT block: exact-softmax attention
    (blk::sdpa) over --rows x --rows tokens with --heads heads of 128, and the fp32 sd::matmul
    at --rows x 3072 x 3072.  Times both with CUDA events, checks a sample of each result
    against float64, and times torch's fp32 attention / matmul next to them.  One GPU; one JSON
    line (value = attention TFLOP/s of algorithmic work, 4 * Lq * Lk * C)."""
    import ctypes as C

    import torch

    import __graft_entry__ as ge

    torch.cuda.set_device(0)
    pkg = ge.load_package()
    s = pkg.Sdq(0)
    lib = s.lib
    dev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream()
    sp = C.c_void_p(stream.cuda_stream)
    g = torch.Generator(device=dev)
    g.manual_seed(11)
    L, H = args.rows, args.heads
    Cc = H * 128

    def p(t):
        return C.c_void_p(t.data_ptr())

    def timed(fn, clocks=None):
        for _ in range(max(args.warmup, 1)):
            fn()
        torch.cuda.synchronize()
        sampler = ClockSampler(0) if clocks is not None else None
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_wall0 = time.time()
        e0.record(stream)
        for _ in range(args.steps):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        if sampler:
            clocks.update(sampler.stop(t_wall0, time.time()))
        return e0.elapsed_time(e1) / args.steps
    q, k, v = [torch.randn(L, Cc, device=dev, generator=g) for _ in range(3)]
    q *= args.qk_scale
    k *= args.qk_scale
    out = torch.empty(L, Cc, device=dev)
    n0 = s.launches()
    att_clocks = {}
    t_att = timed(lambda: s._ck(lib.sdq_sdpa(p(q), p(k), p(v), L, L, Cc, H, p(out), 0, sp)), att_clocks)
    att_launches = (s.launches() - n0) // (args.steps + max(args.warmup, 1))
    rows = min(L, 1024)                                   # float64 check: two heads, the first rows
    q64, k64, v64 = [x.view(L, H, 128).transpose(0, 1)[:2].double() for x in (q, k, v)]
    ref = torch.softmax(q64[:, :rows] @ k64.transpose(1, 2) / 128 ** 0.5, -1) @ v64

    def err_now():
        return float((out.view(L, H, 128).transpose(0, 1)[:2, :rows].double() - ref).abs().max() / ref.abs().max())
    variants = {}
    for name, fl in (("v_as_one_fp16", pkg.sdq.SDPA_V_FP16), ("k_as_one_fp16", pkg.sdq.SDPA_K_FP16),
                     ("k_and_v_as_one_fp16", pkg.sdq.SDPA_K_FP16 | pkg.sdq.SDPA_V_FP16)):
        t_var = timed(lambda: s._ck(lib.sdq_sdpa(p(q), p(k), p(v), L, L, Cc, H, p(out), fl, sp)))
        variants[name] = {"ms": t_var, "max_err_over_max_abs_vs_float64": err_now()}
    t_att_v16 = variants["v_as_one_fp16"]["ms"]
    s._ck(lib.sdq_sdpa(p(q), p(k), p(v), L, L, Cc, H, p(out), 0, sp))      # (out: the full-precision result again)
    torch.cuda.synchronize()
    err_att = err_now()
    torch.backends.cuda.matmul.allow_tf32 = False
    tq, tk, tv = [x.view(1, L, H, 128).transpose(1, 2) for x in (q, k, v)]
    t_att_torch = timed(lambda: torch.nn.functional.scaled_dot_product_attention(tq, tk, tv))
    del q64, k64, v64, ref
    M, K, N = L, D_MODEL, D_MODEL
    A = torch.randn(M, K, device=dev, generator=g)
    W = torch.randn(K, N, device=dev, generator=g) * 0.05
    o2 = torch.empty(M, N, device=dev)
    h = C.c_uint64(0)
    s._ck(lib.sdq_fweight_upload(p(W), K, N, 0, C.byref(h)))
    t_mm = timed(lambda: s._ck(lib.sdq_fmatmul(h.value, p(A), M, p(o2), None, 0, sp)))
    r64 = A[:rows].double() @ W.double()
    err_mm = float((o2[:rows].double() - r64).abs().max() / r64.abs().max())
    t_mm_torch = timed(lambda: torch.matmul(A, W, out=o2))
    att_flop, mm_flop = 4.0 * L * L * Cc, 2.0 * M * K * N
    pk, pk_kind = peaks()
    bf16 = float(pk.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    print(json.dumps({"metric": "fp32_attention_throughput", "value": att_flop / (t_att * 1e-3) / 1e12,
                      "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps, "warmup": max(args.warmup, 1),
                      "ms_per_step": t_att, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                      "dtype": "fp16x3 scores and P*V (two-term splits), f32 accumulate", "data": "synthetic",
                      "config": {"workload": "dit_attention_and_fp32_matmul", "tokens": L, "heads": H,
                                 "l2": "q, k, v %d MB each" % (L * Cc * 4 // 1000000)},
                      "gpu_launches": att_launches * args.steps, "clocks": att_clocks,
                      "attention": {"ms": t_att, "tflops": att_flop / (t_att * 1e-3) / 1e12,
                                    "max_err_over_max_abs_vs_float64": err_att, "torch_fp32_sdpa_ms": t_att_torch,
                                    "ms_with_v_as_one_fp16": t_att_v16, "reduced_operand_variants": variants,
                                    "frac_of_measured_bf16_peak": att_flop / (t_att * 1e-3) / 1e12 / bf16, "of": pk_kind,
                                    # 48 fp16 MMAs of 128x128x16 per 128 keys against 16 of plain fp16 attention
                                    "issued_fp16_tflops": 3.0 * att_flop / (t_att * 1e-3) / 1e12},
                      "matmul": {"shape": [M, K, N], "ms": t_mm, "tflops": mm_flop / (t_mm * 1e-3) / 1e12,
                                 "max_err_over_max_abs_vs_float64": err_mm, "torch_fp32_matmul_ms": t_mm_torch}}))
    return 0


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        sys.exit(run_reference(a))
    sys.exit({"sweep": run_sweep, "branch": run_branch, "block": run_block,
              "fp32": run_fp32}.get(a.workload, run_b200)(a))
