#!/usr/bin/env python
"""Benchmark of the aiehlc matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the hot path over one batch of seeded synthetic input.  The headline
workload is the int8 4096^3 GEMM with the fused srs epilogue (shift 8, cascade split-K 4); with N GPUs
every rank runs it on its own 4096 rows of a (4096 N)-row problem (B replicated, no collective).  One
JSON line is printed by rank 0.  Beside the headline the default run measures, with their own fixed step
counts and in the same line under "configs", every other configuration the metric is quoted on:

    N = 1 : cfg1 (64^3), cfg3 (bf16 8192^3, with the library GEMM beside it), cfg4 (the convolution:
            TOPS, us per call, GB/s; also larger batches and the allocation-free entry point), cfg5
            (65536 x 8192 x 8192 on one GPU) and "sustained": the headline GEMM for at least two seconds
            under the power cap, with the clocks sampled during the loop;
    N > 1 : cfg5 (the same 65536 x 8192 x 8192 product with its rows sharded over the ranks: strong
            scaling) and cfg5_splitk (split-K 8 over the ranks, the int32 partial sums exchanged once by
            the GEMM epilogue over peer memory and once by NCCL reduce-scatter, and whether both agree).

The reference arm (--impl reference) times the CPU golden loop restated in oracle/ on the host cores of
this machine, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

L2_BYTES = 126 * 1024 * 1024
NVLINK_GBS = 770.0   # measured peer-copy bandwidth between two B200 per direction (nominal 900)
# dram__bytes_read.sum + dram__bytes_write.sum per launch, from the ncu captures summarised in profiles/
NCU_TRAFFIC_BYTES = {"cfg2": 33.9e6, "cfg3": 1.229e9, "cfg4": 0.33e6, "cfg4_n128": 25.9e6, "shallow_k": 220.7e6,
                     "scatter_local": 1.151e9}

WORKLOADS = {
    "cfg2": dict(M=4096, N=4096, K=4096, kind="i8_srs", shift=8, splitk=4, scaling="weak",
                 desc="int8 GEMM 4096^3, A row-major, B [N][K], int32 accumulate in TMEM, srs shift 8 "
                      "half-even saturating to int8, cascade split-K 4"),
    "cfg1": dict(M=64, N=64, K=64, kind="i8_i32", scaling="weak", desc="int8 GEMM 64^3 -> int32 (one tile)"),
    "mm_i32": dict(M=4096, N=4096, K=4096, kind="mm_i32", scaling="weak",
                   desc="the reference's own kernel (int32 x int32 -> int32, uint32 wrap-around) at 4096^3, "
                        "as unsigned int8 limb GEMMs on the tensor cores"),
    "cfg3": dict(M=8192, N=8192, K=8192, kind="bf16", scaling="weak",
                 desc="bf16 GEMM 8192^3, fp32 accumulate, bf16 out"),
    "cfg4": dict(kind="conv", n=1, h=56, w=56, cin=64, cout=64, shift=6, scaling="weak",
                 desc="int8 conv2d NHWC 1x56x56x64, 3x3x64x64 HWIO, stride 1 pad 1, per-channel srs 6"),
    "cfg5": dict(M=65536, N=8192, K=8192, kind="i8_i32", scaling="strong",
                 desc="int8 GEMM 65536x8192x8192 -> int32, rows of A/C sharded over the GPUs"),
    "shallow_k": dict(M=16384, N=4096, K=512, kind="i8_i32", scaling="weak", bound="hbm",
                      desc="int8 GEMM 16384x4096x512 -> int32: 268 MB of results over 4 K blocks, the output stage "
                           "sets the pace (two groups of epilogue warps)"),
    "scatter_local": dict(M=16384, N=8192, K=2048, kind="i8_i32_scatter", shards=8, scaling="weak", bound="hbm",
                          desc="int8 GEMM 16384x8192x2048 added into 8 row shards of an int32 result, all shards in this "
                               "GPU's memory: the split-K exchange kernel (aiehlc_gemm_i8_i32_scatter_dev) without a wire"),
    "cfg5_splitk": dict(M=65536, N=8192, K=8192, kind="i8_i32_splitk", splitk=8, scaling="strong",
                        desc="int8 GEMM 65536x8192x8192 -> int32, split-K 8 over the GPUs, int32 partial sums "
                             "exchanged between the GPUs (how: splitk_exchange)"),
}


def load_peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return dict(hbm_gbs=float(d["hbm_gbs"]), bf16=float(d["bf16_tflops"]),
                        bf16_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
        except Exception:  # noqa: BLE001
            pass
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Polls SM clock, power and throttle reasons through NVML while a timed region runs."""

    def __init__(self, device_index: int, period_s: float = 0.001):
        self.idx = device_index
        self.period = period_s
        self.samples: list[int] = []
        self.power: list[float] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thr = None
        self._nvml = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001
            self._nvml = None
            return self
        self._thr = threading.Thread(target=self._run, daemon=True)
        self._thr.start()
        return self

    def _physical_index(self) -> int:
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            parts = [p for p in vis.split(",") if p.strip() != ""]
            try:
                return int(parts[self.idx])
            except Exception:  # noqa: BLE001
                return self.idx
        return self.idx

    def _run(self):
        n = self._nvml
        names = {
            "hw_slowdown": getattr(n, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(n, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(n, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(n, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        get_reasons = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(
            n, "nvmlDeviceGetCurrentClocksThrottleReasons", None)
        while not self._stop.is_set():
            try:
                self.samples.append(int(n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM)))
                self.power.append(n.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
                if get_reasons:
                    mask = int(get_reasons(self._h))
                    for k, bit in names.items():
                        if mask & bit:
                            self.reasons.add(k)
            except Exception:  # noqa: BLE001
                pass
            time.sleep(self.period)

    def stop(self) -> dict:
        self._stop.set()
        if self._thr:
            self._thr.join(timeout=1.0)
        if not self.samples:
            return self._smi_fallback()
        out = {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
               "reasons": sorted(self.reasons), "samples": len(self.samples)}
        if self.power:
            out["power_w_max"] = round(max(self.power), 1)
        return out

    def _smi_fallback(self) -> dict:
        try:
            out = subprocess.run(["nvidia-smi", "--query-gpu=clocks.sm,clocks.max.sm", "--format=csv,noheader,nounits",
                                  "-i", str(self._physical_index())], capture_output=True, text=True, timeout=10).stdout
            a, b = [float(v) for v in out.strip().split(",")]
            return {"sm_mhz": a, "sm_max_mhz": b, "reasons": [], "samples": 1, "note": "idle sample (NVML unavailable)"}
        except Exception:  # noqa: BLE001
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}


# --------------------------------------------------------------------------- CPU legs
def host_threads() -> int:
    """Host threads this process may use (launchers such as torchrun export OMP_NUM_THREADS=1)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_time_i8_srs(rows: int, n: int, k: int, shift: int, splitk: int, seed: int, reps: int = 1):
    """Times the oracle's GEMM+srs on `rows` rows of the workload; returns (seconds per rep, threads)."""
    from aiehlc_b200 import synth
    from oracle import oracle as O
    O.set_threads(host_threads())
    A = synth.int8_uniform(seed, (rows, k))
    B = synth.int8_uniform(seed + 1000, (n, k))
    O.gemm_i8_srs(A[:8], B[:64], shift=shift, splitk=splitk)  # page in / warm up
    t0 = time.perf_counter()
    for _ in range(reps):
        O.gemm_i8_srs(A, B, shift=shift, splitk=splitk)
    return (time.perf_counter() - t0) / reps, O.max_threads()


def _cpu_case(wl: dict, name: str):
    """(make(rows) -> zero-argument callable running the oracle on `rows` units, units in the workload,
    ops per unit, what a unit is) for the CPU golden restatement of a workload."""
    import numpy as np

    from aiehlc_b200 import synth
    from oracle import oracle as O
    kind = wl["kind"]
    if kind == "conv":
        h, w, cin, cout = wl["h"], wl["w"], wl["cin"], wl["cout"]
        wts = synth.int8_uniform(1004, (3, 3, cin, cout))
        sv = np.full(cout, wl["shift"], np.uint8)

        def make(imgs):
            x = synth.int8_uniform(4, (imgs, h, w, cin))
            return lambda: O.conv2d_i8_srs(x, wts, sv, pad=1)
        return make, wl["n"], 2.0 * h * w * cout * 9 * cin, "images"
    M, N, K = wl["M"], wl["N"], wl["K"]
    if kind == "bf16":
        B = synth.normal_bf16_bits(1003, (N, K))

        def make(rows):
            A = synth.normal_bf16_bits(3, (rows, K))
            return lambda: O.gemm_bf16(A, B)
    elif kind == "mm_i32":
        rng = np.random.default_rng(1)

        def make(rows):
            packed = rng.integers(-2**31, 2**31 - 1, size=(rows + N) * K, dtype=np.int64).astype(np.int32)
            return lambda: O.mm_i32(packed, rows, N, K)
    else:
        seed = {"cfg2": 2, "cfg1": 1}.get(name, 5)
        B = synth.int8_uniform(seed + 1000, (N, K))

        def make(rows):
            A = synth.int8_uniform(seed, (rows, K))
            if kind == "i8_srs":
                return lambda: O.gemm_i8_srs(A, B, shift=wl["shift"], splitk=wl["splitk"])
            return lambda: O.gemm_i8_i32(A, B)
    return make, M, 2.0 * N * K, "rows of A"


def reference_arm(args, name: str, wl: dict) -> dict:
    """CPU golden restatement (oracle/) on the host cores, a bounded sample of the workload per step."""
    from oracle import oracle as O
    if wl["kind"] == "i8_i32_splitk":
        return {"impl": "reference", "unavailable": "the split-K exchange between GPUs has no CPU counterpart: "
                                                    "time --workload cfg5 (the same product) instead"}
    O.set_threads(host_threads())
    make, units_total, ops_per_unit, unit_name = _cpu_case(wl, name)
    probe_units = min(units_total, 32 if unit_name == "rows of A" else 1)
    probe = make(probe_units)
    probe()
    t0 = time.perf_counter()
    probe()
    per_unit = (time.perf_counter() - t0) / probe_units
    total_steps = max(1, args.steps + args.warmup)
    budget_s = 90.0
    units = int(max(1, min(units_total, budget_s / total_steps / max(per_unit, 1e-9))))
    run = make(units)
    for _ in range(args.warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run()
    dt = time.perf_counter() - t0
    value = ops_per_unit * units * args.steps / dt / 1e12
    unit = "TFLOPS" if wl["kind"] == "bf16" else "TOPS"
    sample = f"{units} of {units_total} {unit_name} per step (everything else at full size), {args.steps} steps"
    threads = O.max_threads()
    return {
        "impl": "reference", "metric": metric_name(name, wl, unit), "value": value, "unit": unit,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": wl["scaling"], "vs_baseline": None, "dtype": dtype_of(wl["kind"]),
        "data": "synthetic",
        "config": {"workload": wl["desc"], "per_gpu": per_gpu_text(wl, args.gpus), "parallelism": f"row-shard x{args.gpus}",
                   "l2": "not applicable: CPU golden loop on the host cores", "tile_n": "not applicable",
                   "launch": f"oracle call per step on {threads} host threads; {sample}"},
        "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def metric_name(name: str, wl: dict, unit: str) -> str:
    return "int8 GEMM TOPS (srs epilogue), device-timed" if wl["kind"] == "i8_srs" else f"{name} {unit}, device-timed"


def dtype_of(kind: str) -> str:
    return "bf16" if kind == "bf16" else ("int32 via u8 limbs" if kind == "mm_i32" else "int8")


def per_gpu_text(wl: dict, world: int) -> str:
    if wl["kind"] == "conv":
        return f"M={wl['n'] * wl['h'] * wl['w']} N={wl['cout']} K={9 * wl['cin']}"
    m = wl["M"] if wl["scaling"] == "weak" or wl["kind"] == "i8_i32_splitk" else -(-wl["M"] // world)
    k = wl["K"] // world if wl["kind"] == "i8_i32_splitk" else wl["K"]
    return f"M={m} N={wl['N']} K={k}"


# --------------------------------------------------------------------------- GPU arm
GATE_HEAD = 8   # calls queued behind the closed gate before it opens (the same at every number of GPUs)


class StreamGate:
    """Holds a stream at a wait on a word of pinned host memory (a stream memory operation, no kernel spins)
    until the host writes it: work queued behind it starts when the host says so."""

    def __init__(self):
        import torch
        from cuda.bindings import driver as drv
        self._drv = drv
        self._flag = torch.zeros(1, dtype=torch.int32).pin_memory()
        err, dptr = drv.cuMemHostGetDevicePointer(self._flag.data_ptr(), 0)
        if err != drv.CUresult.CUDA_SUCCESS:
            raise RuntimeError(f"cuMemHostGetDevicePointer: {err}")
        self._dptr = dptr

    def close(self, stream):
        drv = self._drv
        self._flag[0] = 0
        (err,) = drv.cuStreamWaitValue32(stream.cuda_stream, self._dptr, 1,
                                         drv.CUstreamWaitValue_flags.CU_STREAM_WAIT_VALUE_EQ)
        if err != drv.CUresult.CUDA_SUCCESS:
            raise RuntimeError(f"cuStreamWaitValue32: {err}")

    def open(self):
        self._flag[0] = 1


class Env:
    """What every leg of the GPU arm shares: the rank's device, context, process group and side stream."""

    def __init__(self, args):
        import torch
        self.args = args
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist
        from aiehlc_b200.ops import Context
        self.ctx = Context(self.local_rank)
        if args.tile_n:
            self.ctx.set_tile_n(args.tile_n)
        self.peaks = load_peaks()
        # every leg runs on one side stream (calls are bound to the stream current at bind time)
        self.side = torch.cuda.Stream()
        torch.cuda.set_stream(self.side)
        self.gate = None
        self.gate_error = None
        try:
            self.gate = StreamGate()
        except Exception as exc:  # noqa: BLE001
            self.gate_error = f"{type(exc).__name__}: {exc}"[:160]
        self._symm = None

    def barrier(self):
        import torch
        if self.world > 1:
            self.dist.barrier(device_ids=[self.local_rank])
        torch.cuda.synchronize()

    def max_over_ranks(self, value: float) -> float:
        import torch
        t = torch.tensor([value], dtype=torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def gather(self, value: float) -> list:
        import torch
        t = torch.tensor([value], dtype=torch.float64, device=self.dev)
        if self.world == 1:
            return [float(t.item())]
        out = [torch.zeros_like(t) for _ in range(self.world)]
        self.dist.all_gather(out, t)
        return [float(o.item()) for o in out]


class Work:
    """One workload on this rank: step(i) issues step i; ops are this rank's share per step."""
    step = None
    ops_per_step = 0.0
    alg_bytes = 0
    unit = "TOPS"
    kind = ""
    dtype = "int8"
    per_gpu = ""
    l2_note = ""
    launch_bound = False
    extra: dict

    def __init__(self):
        self.extra = {}
        self.keep = []      # tensors that must stay alive while the steps run


def make_conv(env: Env, wl: dict, n: int | None = None) -> Work:
    import torch

    from aiehlc_b200 import synth
    n = n or wl["n"]
    h, w, cin, cout = wl["h"], wl["w"], wl["cin"], wl["cout"]
    dev, ctx = env.dev, env.ctx
    set_bytes = n * h * w * (cin + cout) + 9 * cin * cout + cout
    nsets = 8 if n == 1 else max(2, min(24, -(-2 * L2_BYTES // set_bytes)))
    wk = Work()
    wk.xs = [synth.int8_uniform_torch(4 + 10 * i, (n, h, w, cin), dev) for i in range(nsets)]
    wk.ws = [synth.int8_uniform_torch(1004 + 10 * i, (3, 3, cin, cout), dev) for i in range(nsets)]
    wk.sv = torch.full((cout,), wl["shift"], dtype=torch.uint8, device=dev)
    wk.ys = [torch.empty((n, h, w, cout), dtype=torch.int8, device=dev) for _ in range(nsets)]
    calls = [ctx.bound_conv2d_i8_srs(wk.xs[j], wk.ws[j], wk.sv, wk.ys[j], pad=1) for j in range(nsets)]
    wk.nsets = nsets
    wk.batch = n
    wk.step = lambda i: calls[i % nsets]()
    wk.ops_per_step = 2.0 * n * h * w * cout * 9 * cin
    wk.alg_bytes = set_bytes
    wk.kind, wk.unit, wk.dtype = "conv", "TOPS", "int8"
    wk.per_gpu = f"M={n * h * w} N={cout} K={9 * cin}"
    wk.l2_note = (f"rotating {nsets} input sets; operands are L2-resident by nature ({set_bytes / 1e6:.2f} MB per step)"
                  if nsets * set_bytes < L2_BYTES else f"rotating {nsets} input sets ({nsets * set_bytes / 1e6:.0f} MB) > 126 MB L2")
    wk.launch_bound = n * h * w <= 3136 * 8
    return wk


def make_gemm(env: Env, name: str, wl: dict, sets: int = 0) -> Work:
    import torch

    from aiehlc_b200 import shard, synth
    dev, ctx, rank, world = env.dev, env.ctx, env.rank, env.world
    kind = wl["kind"]
    M, N, K = wl["M"], wl["N"], wl["K"]
    if wl["scaling"] == "weak":
        m_local, row0 = M, rank * M          # every rank owns M rows of a (world*M)-row problem
    else:
        row0, m_local = shard.row_shard(M, world, rank)
    esize = 2 if kind == "bf16" else (4 if kind == "mm_i32" else 1)
    out_esize = {"i8_srs": 1, "i8_i32": 4, "bf16": 2, "mm_i32": 4, "i8_i32_scatter": 4}[kind]
    set_bytes = m_local * K * esize + N * K * esize + m_local * N * out_esize
    nsets = max(1, min(8, -(-2 * L2_BYTES // set_bytes))) if set_bytes < 2 * L2_BYTES else 1
    if sets > 0:
        nsets = sets
    wk = Work()
    As, Bs, Cs = [], [], []
    for i in range(nsets):
        if kind == "mm_i32":
            g = torch.Generator(device=dev).manual_seed(1 + i)   # the packed window of the examples: A words, then B words
            As.append(torch.randint(-2**31, 2**31 - 1, ((m_local + N) * K,), dtype=torch.int32, device=dev, generator=g))
            Bs.append(None)
            Cs.append(torch.empty((m_local, N), dtype=torch.int32, device=dev))
        elif kind == "bf16":
            As.append(synth.normal_bf16_torch(3 + 10 * i, (m_local, K), dev, start=row0 * K))
            Bs.append(synth.normal_bf16_torch(1003 + 10 * i, (N, K), dev))
            Cs.append(torch.empty((m_local, N), dtype=torch.bfloat16, device=dev))
        else:
            seed = {"cfg2": 2, "cfg1": 1}.get(name, 5)
            As.append(synth.int8_uniform_torch(seed + 10 * i, (m_local, K), dev, start=row0 * K))
            Bs.append(synth.int8_uniform_torch(seed + 1000 + 10 * i, (N, K), dev))
            Cs.append(torch.empty((m_local, N), dtype=torch.int8 if kind == "i8_srs" else torch.int32, device=dev))
    wk.keep = [As, Bs, Cs]
    # every argument of the C-ABI call is converted once, outside the timed region
    if kind == "i8_srs":
        calls = [ctx.bound_gemm_i8_srs(As[j], Bs[j], Cs[j], shift=wl["shift"], splitk=wl["splitk"]) for j in range(nsets)]
    elif kind == "mm_i32":
        calls = [(lambda j=j: ctx.mm_i32(As[j], m_local, N, K, out=Cs[j])) for j in range(nsets)]
    elif kind == "bf16":
        calls = [ctx.bound_gemm_bf16(As[j], Bs[j], Cs[j]) for j in range(nsets)]
    elif kind == "i8_i32_scatter":
        rows = m_local // wl["shards"]
        calls = [ctx.bound_gemm_i8_i32_scatter(As[j], Bs[j], [Cs[j][g * rows:(g + 1) * rows].data_ptr() for g in range(wl["shards"])],
                                               rows, N, first_shard=1) for j in range(nsets)]
    else:
        calls = [ctx.bound_gemm_i8_i32(As[j], Bs[j], Cs[j]) for j in range(nsets)]
    wk.nsets = nsets
    wk.step = lambda i: calls[i % nsets]()
    wk.ops_per_step = 2.0 * m_local * N * K
    wk.alg_bytes = set_bytes
    wk.kind, wk.unit, wk.dtype = kind, ("TFLOPS" if kind == "bf16" else "TOPS"), dtype_of(kind)
    wk.per_gpu = f"M={m_local} N={N} K={K}"
    wk.shape = (m_local, N, K)
    wk.l2_note = (f"rotating {nsets} input sets; operands are L2-resident by nature ({set_bytes / 1e3:.0f} KB per step)"
                  if nsets * set_bytes < L2_BYTES
                  else f"rotating {nsets} input sets ({nsets * set_bytes / 1e6:.0f} MB) > 126 MB L2" if nsets > 1
                  else f"one input set of {set_bytes / 1e6:.0f} MB > 126 MB L2" if set_bytes > L2_BYTES
                  else f"single input set of {set_bytes / 1e6:.1f} MB")
    wk.launch_bound = wk.ops_per_step < 1e9
    return wk


def timed(env: Env, wk: Work, steps: int, warmup: int, mode: str) -> dict:
    """W warm-up steps, then exactly `steps` steps between two CUDA events on the launching stream, a barrier
    and a device synchronisation on both sides; returns this rank's and the slowest rank's milliseconds.
    mode: "gate"  one C-ABI call per step; the stream is held at a gate while the first GATE_HEAD calls are
                  queued, so the host is ahead of the GPU when the clock starts -- the same at every N;
          "graph" the steps are recorded once and replayed as one CUDA graph (launch-bound workloads:
                  the timed region measures the GPU, not the interpreter);
          "plain" one call per step, no gate."""
    import torch
    ctx = env.ctx
    W = max(warmup, 3)
    for i in range(W):
        wk.step(i)
    ctx.sync()
    note = {}
    graph, graph_launches = None, 0
    if mode == "graph":
        torch.cuda.synchronize()
        try:
            graph = torch.cuda.CUDAGraph()
            c0 = ctx.launch_count
            with torch.cuda.graph(graph, stream=env.side, capture_error_mode="thread_local"):
                for i in range(steps):
                    wk.step(i)
            graph_launches = ctx.launch_count - c0
            graph.replay()           # microsecond kernels: a trial replay costs nothing
            torch.cuda.synchronize()
        except Exception as exc:  # noqa: BLE001  -- recording failed: issue the steps one by one instead
            graph, mode = None, "gate"
            note["graph_fallback"] = f"{type(exc).__name__}: {exc}"[:160]
            torch.cuda.synchronize()
    gate = env.gate if mode == "gate" else None
    if mode == "gate" and gate is None:
        note["gate_fallback"] = env.gate_error
    env.barrier()
    sampler = ClockSampler(env.local_rank).start()
    launches0 = ctx.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    env.barrier()
    head = min(GATE_HEAD, max(1, steps // 2))
    if gate is not None:
        try:
            gate.close(env.side)             # everything queued from here on waits for gate.open()
        except Exception as exc:  # noqa: BLE001  -- no gate on this system: plain call-by-call run
            note["gate_fallback"] = f"{type(exc).__name__}: {exc}"[:160]
            gate = None
    if gate is not None:
        try:
            e0.record()
            for i in range(steps):
                if i == head:
                    gate.open()
                wk.step(i)
        finally:
            gate.open()
    else:
        e0.record()
        if graph is not None:
            graph.replay()
        else:
            for i in range(steps):
                wk.step(i)
    e1.record()
    env.barrier()
    local_ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    launches = graph_launches if graph is not None else ctx.launch_count - launches0
    status = ctx.sync()
    max_ms = env.max_over_ranks(local_ms)
    launch = ("the steps replayed from one CUDA graph" if graph is not None else
              f"one C-ABI call per step, the first {head} queued behind a stream gate before the clock starts"
              if gate is not None else "one C-ABI call per step")
    return dict(local_ms=local_ms, max_ms=max_ms, clocks=clocks, launches=int(launches), status=int(status),
                launch=launch, steps=steps, warmup=W, note=note)


def roofline_of(env: Env, name: str, wl: dict, wk: Work, res: dict) -> dict:
    """Roofline of the dominant kernel on this rank: algorithmic ops (or bytes) per launch over the mean
    launch time, against the measured peak (burst for a short timed region, sustained for a long one)."""
    peaks = env.peaks
    per_launch_ms = res["local_ms"] / res["steps"]
    achieved = wk.ops_per_step / (per_launch_ms * 1e-3) / 1e12
    traffic = NCU_TRAFFIC_BYTES.get(name)
    if wk.kind == "conv":
        if wk.batch != wl["n"]:
            traffic = NCU_TRAFFIC_BYTES.get(f"{name}_n{wk.batch}")
        gbs = wk.alg_bytes / (per_launch_ms * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": gbs / peaks["hbm_gbs"], "traffic": traffic,
                "note": f"{per_launch_ms * 1e3:.1f} us per call, {res['launches'] // max(res['steps'], 1)} launch(es) "
                        f"per call, HWIO weights as given; {wk.alg_bytes} algorithmic bytes per call; peak {peaks['source']}"}
    sustained = res["local_ms"] > 250.0
    base = peaks["bf16_sustained"] if sustained else peaks["bf16"]
    which = "sustained" if sustained else "burst"
    peak = base * (1.0 if wk.dtype == "bf16" else 2.0)
    roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": wk.unit, "frac": achieved / peak,
                "traffic": traffic,
                "note": (f"peak = 2 x measured bf16 {which} (kind::i8 has twice the K per instruction)"
                         if wk.dtype != "bf16" else f"peak = measured bf16 {which}") +
                        f", of {peaks['source']}; timed region {res['local_ms']:.0f} ms"}
    if wl.get("bound") == "hbm":
        # a product over a shallow K: the result bytes, not the MMAs, bound the launch
        m, n, k = wk.shape
        gemm_bytes = m * k + n * k + m * n * 4 * (2 if wk.kind == "i8_i32_scatter" else 1)   # an add reads what it writes
        gbs = gemm_bytes / (per_launch_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": gbs / peaks["hbm_gbs"], "traffic": traffic,
                    "note": f"algorithmic bytes A + B + C(int32{', read and written' if wk.kind == 'i8_i32_scatter' else ''}) = "
                            f"{gemm_bytes / 1e6:.1f} MB per launch; peak {peaks['source']}"}
    if wk.kind == "mm_i32":
        # one int32 product costs ten int8 limb products (K + 2K + 3K + 4K bytes of depth)
        roofline["achieved"] = achieved * 10.0
        roofline["frac"] = achieved * 10.0 / roofline["peak"]
        roofline["note"] = ("int8 tensor work = 10 x 2MNK (four limb GEMMs of depth K, 2K, 3K, 4K); value counts the "
                            "int32 multiply-adds; " + roofline["note"])
    return roofline


def default_mode(wk: Work, requested: str) -> str:
    if requested in ("on", "graph"):
        return "graph"
    if requested in ("off", "plain"):
        return "plain"
    if requested == "gate":
        return "gate"
    return "graph" if wk.launch_bound else "gate"


def sub_record(env: Env, name: str, wl: dict, wk: Work, res: dict) -> dict:
    """A configuration measured beside the headline: value over the whole job, this rank's roofline."""
    total_ops = wk.ops_per_step * res["steps"] * (env.world if wl["scaling"] == "weak" else 1)
    if wl["scaling"] == "strong":
        total_ops = 2.0 * wl["M"] * wl["N"] * wl["K"] * res["steps"]
    rec = {"value": total_ops / (res["max_ms"] * 1e-3) / 1e12, "unit": wk.unit, "ms_per_step": res["max_ms"] / res["steps"],
           "steps": res["steps"], "warmup": res["warmup"], "scaling": wl["scaling"], "per_gpu": wk.per_gpu,
           "workload": wl["desc"], "l2": wk.l2_note, "launch": res["launch"], "gpu_launches": res["launches"],
           "roofline": roofline_of(env, name, wl, wk, res), "clocks": res["clocks"], "device_status": res["status"]}
    rec.update(res["note"])
    return rec


def release(*objs):
    import gc

    import torch
    for o in objs:
        if isinstance(o, Work):
            o.keep = []
            o.step = None
            for a in ("xs", "ws", "ys", "sv"):
                if hasattr(o, a):
                    setattr(o, a, None)
    gc.collect()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()


# ------------------------------------------------------------------------- legs beside the headline
def library_gemm(env: Env, kind: str, M: int, N: int, K: int, iters: int) -> float | str:
    """The library GEMM (cuBLASLt through torch) on the same shape in the same process, for context."""
    import torch
    try:
        if kind == "bf16":
            a = torch.randn((M, K), dtype=torch.bfloat16, device=env.dev)
            b = torch.randn((N, K), dtype=torch.bfloat16, device=env.dev)
            fn = lambda: torch.matmul(a, b.T)  # noqa: E731
        else:
            a = torch.randint(-128, 128, (M, K), dtype=torch.int8, device=env.dev)
            b = torch.randint(-128, 128, (N, K), dtype=torch.int8, device=env.dev)
            fn = lambda: torch._int_mm(a, b.T)  # noqa: E731
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return 2.0 * M * N * K / (e0.elapsed_time(e1) / iters * 1e-3) / 1e12
    except Exception as exc:  # noqa: BLE001
        return f"unavailable: {exc}"[:160]


def conv_side_legs(env: Env, wl: dict, wk: Work, steps: int) -> dict:
    """The same convolutions through the other two entry points, replayed from a graph like the main leg:
    weights re-laid once beforehand (one launch per call) and the allocation-free entry point."""
    import ctypes as C

    import torch

    from aiehlc_b200 import _capi
    ctx, out = env.ctx, {}
    nsets = wk.nsets
    n, h, w, cin = wk.xs[0].shape
    cout = wk.ws[0].shape[3]

    def replay_us(step):
        for j in range(nsets):
            step(j)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=env.side, capture_error_mode="thread_local"):
            for i in range(steps):
                step(i)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps * 1e3

    try:
        packed = [ctx.conv2d_pack_weights(wk.ws[j]) for j in range(nsets)]
        out["prepacked_weights_us_per_conv"] = replay_us(
            lambda i: ctx.conv2d_i8_srs_packed(wk.xs[i % nsets], packed[i % nsets], (3, 3), wk.sv, pad=1, out=wk.ys[i % nsets]))
        lib, p = _capi.load(), (lambda t: C.c_void_p(t.data_ptr()))
        stream = C.c_void_p(env.side.cuda_stream)

        def static_step(i):
            j = i % nsets
            _capi.check(lib.aiehlc_conv2d_i8_srs_static_dev(ctx._h, p(wk.xs[j]), p(wk.ws[j]), p(wk.ys[j]), n, h, w, cin, cout,
                                                            3, 3, 1, p(wk.sv), stream))
        out["static_us_per_conv"] = replay_us(static_step)
    except Exception as exc:  # noqa: BLE001
        out["side_legs_error"] = f"{type(exc).__name__}: {exc}"[:160]
    return out


def splitk_record(env: Env, wl: dict, steps: int, warmup: int) -> dict:
    """Split-K 8 over the ranks, both exchanges in one run: the GEMM epilogue adding every tile into its
    owner's row shard over peer memory (fused), and a full int32 partial matrix followed by NCCL
    reduce-scatter; checks once that both give the same bits."""
    import torch

    from aiehlc_b200 import shard, synth
    dist, dev, ctx, rank, world = env.dist, env.dev, env.ctx, env.rank, env.world
    M, N, K = wl["M"], wl["N"], wl["K"]
    k0, k_local = shard.k_range(K, wl["splitk"], world, rank)
    rec = {"workload": wl["desc"], "per_gpu": f"M={M} N={N} K={k_local}", "scaling": "strong", "steps": steps}
    a = synth.int8_uniform_torch(5, (M, K), dev)[:, k0:k0 + k_local].contiguous()
    b = synth.int8_uniform_torch(1005, (N, K), dev)[:, k0:k0 + k_local].contiguous()
    rows_out = M // world
    rs_out = torch.empty((rows_out, N), dtype=torch.int32, device=dev)
    partial = torch.empty((M, N), dtype=torch.int32, device=dev)
    nccl_call = ctx.bound_gemm_i8_i32(a, b, partial)
    wire_bytes = (world - 1) / world * M * N * 4            # int32 partial sums leaving this GPU per step
    ops_total = 2.0 * M * N * K

    def nccl_step(_i):
        nccl_call()
        dist.reduce_scatter_tensor(rs_out, partial, op=dist.ReduceOp.SUM)

    wk = Work()
    wk.step = nccl_step
    res = timed(env, wk, steps, warmup, "plain")
    rec["nccl_ms"] = res["max_ms"] / steps
    rec["nccl_tops"] = ops_total / (rec["nccl_ms"] * 1e-3) / 1e12
    fused_ok = True
    try:
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer mappings only
        import torch.distributed._symmetric_memory as symm
        sym_out = symm.empty((rows_out, N), dtype=torch.int32, device=dev)
        hdl = symm.rendezvous(sym_out, dist.group.WORLD)
        peer_ptrs = [int(p) for p in hdl.buffer_ptrs]
        fused_call = ctx.bound_gemm_i8_i32_scatter(a, b, peer_ptrs, rows_out, N, first_shard=rank + 1)
        tick = torch.zeros(1, dtype=torch.int32, device=dev)
    except Exception as exc:  # noqa: BLE001
        fused_ok = False
        rec["fused_unavailable"] = f"{type(exc).__name__}: {exc}"[:200]
    flags = torch.tensor([1 if fused_ok else 0], dtype=torch.int32, device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if int(flags.item()) == 1:
        def fused_step(_i):
            sym_out.zero_()
            dist.all_reduce(tick)        # stream-ordered: every shard is zero before anyone adds into it
            fused_call()
            dist.all_reduce(tick)        # ... and every contribution has landed before anyone reads

        wk2 = Work()
        wk2.step = fused_step
        res2 = timed(env, wk2, steps, warmup, "plain")
        rec["fused_ms"] = res2["max_ms"] / steps
        rec["fused_tops"] = ops_total / (rec["fused_ms"] * 1e-3) / 1e12
        rec["clocks"] = res2["clocks"]
        rec["device_status"] = res2["status"]
        rec["gpu_launches"] = res2["launches"]
        # once, outside the timed regions: the fused exchange gives what GEMM + NCCL reduce-scatter gives
        fused_step(0)
        nccl_step(0)
        torch.cuda.synchronize()
        same = torch.tensor([1 if torch.equal(rs_out, sym_out) else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        rec["matches_nccl"] = bool(int(same.item()))
        peak = env.peaks["bf16"] * 2.0
        t_math = (ops_total / world) / (peak * 1e12)
        t_wire = wire_bytes / (NVLINK_GBS * 1e9)
        rec["wire_GBps"] = wire_bytes / (rec["fused_ms"] * 1e-3) / 1e9
        rec["nccl_wire_GBps"] = wire_bytes / (rec["nccl_ms"] * 1e-3) / 1e9
        rec["value"], rec["unit"], rec["ms_per_step"] = rec["fused_tops"], "TOPS", rec["fused_ms"]
        rec["roofline"] = {"bound": "nvlink", "achieved": rec["wire_GBps"], "peak": NVLINK_GBS, "unit": "GB/s",
                           "frac": max(t_math, t_wire) / (rec["fused_ms"] * 1e-3), "traffic": None,
                           "note": f"target = max(math {t_math * 1e3:.2f} ms at the tensor peak, wire {t_wire * 1e3:.2f} ms: "
                                   f"{wire_bytes / 1e9:.2f} GB of int32 partial sums per GPU at the measured {NVLINK_GBS:.0f} "
                                   "GB/s peer-copy rate per direction); frac = target / measured step"}
        rec["exchange"] = ("fused: add-reducing tile stores into the owners' shards over peer memory, a tiny all-reduce "
                           "before (all shards zeroed) and after (all adds landed); nccl: GEMM into a full partial "
                           "matrix, then reduce_scatter_tensor")
    else:
        rec["value"], rec["unit"], rec["ms_per_step"] = rec["nccl_tops"], "TOPS", rec["nccl_ms"]
    return rec


def e2e_i8_srs(env: Env, wl: dict, steps: int) -> dict:
    """The headline metric through the host-buffer entry point: pinned host A, B -> device, GEMM + srs,
    C -> host, all inside the timed region.  Also a copy-only leg (the same bytes, no kernel) and every
    rank's own time, so that the line shows what the host's copy bandwidth allows at this N."""
    import torch

    from aiehlc_b200 import synth
    ctx, dev, rank, world = env.ctx, env.dev, env.rank, env.world
    M, N, K = wl["M"], wl["N"], wl["K"]
    a = torch.from_numpy(synth.int8_uniform(2, (M, K), start=rank * M * K)).pin_memory()
    b = torch.from_numpy(synth.int8_uniform(1002, (N, K))).pin_memory()
    c = torch.empty((M, N), dtype=torch.int8).pin_memory()
    an, bn, cn = a.numpy(), b.numpy(), c.numpy()
    for _ in range(3):
        ctx.gemm_i8_srs_host(an, bn, shift=wl["shift"], splitk=wl["splitk"], out=cn)
    env.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        ctx.gemm_i8_srs_host(an, bn, shift=wl["shift"], splitk=wl["splitk"], out=cn)
    torch.cuda.synchronize()
    dt_local = time.perf_counter() - t0
    per_rank = env.gather(dt_local / steps * 1e3)
    dt = max(per_rank) * 1e-3 * steps
    # the copies alone: A and B up on one stream, C down on another, as the entry point does
    da, db = torch.empty_like(a, device=dev), torch.empty_like(b, device=dev)
    dc = torch.empty((M, N), dtype=torch.int8, device=dev)
    s_up, s_dn = torch.cuda.Stream(), torch.cuda.Stream()

    def copies():
        with torch.cuda.stream(s_up):
            da.copy_(a, non_blocking=True)
            db.copy_(b, non_blocking=True)
        with torch.cuda.stream(s_dn):
            c.copy_(dc, non_blocking=True)
    for _ in range(2):
        copies()
    env.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        copies()
        s_up.synchronize()
        s_dn.synchronize()
    copy_ms = env.gather((time.perf_counter() - t0) / steps * 1e3)
    ops = 2.0 * M * N * K * steps * world
    h2d, d2h = int(an.nbytes + bn.nbytes), int(cn.nbytes)
    ms = max(per_rank)
    return {"value": ops / dt / 1e12, "unit": "TOPS", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "steps": steps, "ms_per_step": ms, "per_rank_ms": [round(v, 4) for v in per_rank],
            "h2d_GBps_per_rank": round(h2d / (ms * 1e-3) / 1e9, 1), "d2h_GBps_per_rank": round(d2h / (ms * 1e-3) / 1e9, 1),
            "copy_only_ms_per_rank": [round(v, 4) for v in copy_ms],
            "copy_only_note": "the same H2D and D2H bytes with no kernel, both directions at once: what the host's "
                              "links allow with this many ranks copying together",
            "api": "aiehlc_gemm_i8_srs_host (pinned host buffers, copies inside the timed region)"}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--tile-n", type=int, default=0)
    ap.add_argument("--no-cpu", action="store_true", help="skip the timed CPU baseline")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-lib", action="store_true", help="skip the library GEMM timings")
    ap.add_argument("--no-configs", action="store_true", help="only the headline workload, none of the other configurations")
    ap.add_argument("--sets", type=int, default=0, help="number of rotating input sets (0 = enough to exceed L2)")
    ap.add_argument("--sustained-seconds", type=float, default=2.2)
    ap.add_argument("--batch", type=int, default=0, help="cfg4: images per call (0 = the configuration's own 1)")
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off", "gate"],
                    help="gate (auto for GEMMs, at every number of GPUs): one call per step, the first ones queued "
                         "behind a stream gate before the clock starts; on (auto for the launch-bound cfg1 and cfg4): "
                         "the timed steps replayed from one CUDA graph; off: plain calls")
    args = ap.parse_args()
    name = args.workload
    wl = WORKLOADS[name]
    rank = int(os.environ.get("RANK", "0"))

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps(reference_arm(args, name, wl)), flush=True)
        return 0

    import torch
    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: bench.py needs a B200 (there is no CPU path)"}))
        return 1
    env = Env(args)
    world, dist = env.world, env.dist
    kind = wl["kind"]
    extra: dict = {}

    # ---------------------------------------------------------------- the headline workload
    if kind == "i8_i32_splitk":
        if world < 2:
            wl = dict(WORKLOADS["cfg5"])
            kind = wl["kind"]
            extra["note"] = "cfg5_splitk on one GPU is cfg5: there is nothing to exchange"
        else:
            rec = splitk_record(env, wl, args.steps, args.warmup)
            line = {"metric": metric_name(name, wl, "TOPS"), "value": rec["value"], "unit": "TOPS", "n_gpus": world,
                    "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": rec["ms_per_step"],
                    "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                    "config": {"workload": wl["desc"], "per_gpu": rec["per_gpu"], "parallelism": f"split-K x{world}",
                               "l2": "one input set > 126 MB L2", "tile_n": args.tile_n or "auto",
                               "launch": "one C-ABI call per step"},
                    "roofline": rec.get("roofline"), "clocks": rec.get("clocks"), "gpu_launches": rec.get("gpu_launches", 0),
                    "splitk": rec}
            if env.rank == 0:
                print(json.dumps(line), flush=True)
            dist.destroy_process_group()
            return 0
    if kind == "conv" and args.batch:
        wl = dict(wl, desc=wl["desc"].replace(f"NHWC {wl['n']}x", f"NHWC {args.batch}x"))
    wk = make_conv(env, wl, args.batch or None) if kind == "conv" else make_gemm(env, name, wl, args.sets)
    mode = default_mode(wk, args.graph)
    res = timed(env, wk, args.steps, args.warmup, mode)
    total_ops = wk.ops_per_step * res["steps"] * world
    if wl["scaling"] == "strong":
        total_ops = 2.0 * wl["M"] * wl["N"] * wl["K"] * res["steps"]
    value = total_ops / (res["max_ms"] * 1e-3) / 1e12
    roofline = roofline_of(env, name, wl, wk, res)
    extra.update(res["note"])
    if kind == "i8_srs" and world == 1:
        # the same steps with the caller's promise that no operand is written by the kernel just before (true here:
        # the inputs are resident buffers): loader and multiplier warps of launch i+1 start while launch i drains
        env.ctx.set_operands_ready(True)
        try:
            r2 = timed(env, wk, args.steps, args.warmup, mode)
            extra["with_operands_ready"] = {"value": wk.ops_per_step * r2["steps"] / (r2["max_ms"] * 1e-3) / 1e12, "unit": wk.unit,
                                            "ms_per_step": r2["max_ms"] / r2["steps"], "device_status": r2["status"],
                                            "what": "aiehlc_set_operands_ready(ctx, 1): off by default, not part of the headline"}
        finally:
            env.ctx.set_operands_ready(False)
    if kind == "i8_srs" and env.rank == 0 and not args.no_lib:
        extra["library_int8_tops"] = library_gemm(env, "int8", wl["M"], wl["N"], wl["K"], 50)
    if kind == "bf16" and env.rank == 0 and not args.no_lib:
        extra["library_bf16_tflops"] = library_gemm(env, "bf16", wl["M"], wl["N"], wl["K"], 10)
    if kind == "conv" and mode == "graph":
        extra.update(conv_side_legs(env, wl, wk, args.steps))

    line = {
        "metric": metric_name(name, wl, wk.unit), "value": value, "unit": wk.unit, "n_gpus": world, "steps": res["steps"],
        "warmup": res["warmup"], "ms_per_step": res["max_ms"] / res["steps"], "higher_is_better": True,
        "scaling": wl["scaling"], "vs_baseline": None, "dtype": wk.dtype, "data": "synthetic",
        "config": {"workload": wl["desc"], "per_gpu": wk.per_gpu, "parallelism": f"row-shard x{world}", "l2": wk.l2_note,
                   "tile_n": args.tile_n or "auto", "launch": res["launch"]},
        "roofline": roofline, "clocks": res["clocks"], "gpu_launches": res["launches"], "device_status": res["status"],
    }
    # ---------------------------------------------------------------- end to end through the host API
    if not args.no_e2e and kind == "i8_srs":
        line["e2e"] = e2e_i8_srs(env, wl, min(res["steps"], 20))
    if env.rank == 0 and world == 1 and not args.no_cpu and kind == "i8_srs":
        rows = 1024
        m_local, n_dim, k_dim = wk.shape
        sec, threads = cpu_time_i8_srs(rows, n_dim, k_dim, wl["shift"], wl["splitk"], seed=2)
        reps = int(max(1, min(16, 10.0 / max(sec, 1e-3))))       # the CPU leg runs roughly 10 s in total
        if reps > 1:
            sec, threads = cpu_time_i8_srs(rows, n_dim, k_dim, wl["shift"], wl["splitk"], seed=2, reps=reps)
        line["cpu_baseline"] = {"value": 2.0 * rows * n_dim * k_dim / sec / 1e12, "unit": "TOPS", "cores": threads,
                                "kind": "port", "sample": f"{rows} of {m_local} rows (full N, K) x {reps} repetitions, "
                                                          "oracle GEMM + srs with OpenMP"}

    # ---------------------------------------------------------------- the other configurations
    configs: dict = {}
    if name == "cfg2" and not args.no_configs:
        release()
        release(wk)
        wk = None
        plan = ([("cfg1", 2000), ("cfg3", 20), ("cfg4", 2000), ("cfg5", 5)] if world == 1 else [("cfg5", 10)])
        for cname, csteps in plan:
            try:
                cwl = WORKLOADS[cname]
                cwk = make_conv(env, cwl) if cwl["kind"] == "conv" else make_gemm(env, cname, cwl)
                cmode = default_mode(cwk, args.graph)
                r = timed(env, cwk, csteps, 3, cmode)
                rec = sub_record(env, cname, cwl, cwk, r)
                if cname == "cfg3" and not args.no_lib:
                    rec["library_bf16_tflops"] = library_gemm(env, "bf16", cwl["M"], cwl["N"], cwl["K"], 10)
                if cname == "cfg4":
                    rec["us_per_conv"] = rec["ms_per_step"] * 1e3
                    if cmode == "graph":
                        rec.update(conv_side_legs(env, cwl, cwk, csteps))
                    batches = {}
                    for nb in (8, 32, 128):
                        bwk = make_conv(env, cwl, nb)
                        br = timed(env, bwk, 40, 3, default_mode(bwk, args.graph))
                        per_ms = br["local_ms"] / br["steps"]
                        batches[f"n{nb}"] = {"value": bwk.ops_per_step / (per_ms * 1e-3) / 1e12, "unit": "TOPS",
                                             "us_per_call": per_ms * 1e3, "GBps": bwk.alg_bytes / (per_ms * 1e-3) / 1e9,
                                             "frac_of_hbm_peak": bwk.alg_bytes / (per_ms * 1e-3) / 1e9 / env.peaks["hbm_gbs"],
                                             "traffic": NCU_TRAFFIC_BYTES.get(f"cfg4_n{nb}"),
                                             "launch": br["launch"], "l2": bwk.l2_note}
                        release(bwk)
                    rec["batches"] = batches
                configs[cname] = rec
                release(cwk)
                cwk = None
            except Exception as exc:  # noqa: BLE001  -- a side leg must not cost the headline
                configs[cname] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
                release()
        if world == 1:
            # last, so that the burst figures above start from a cool GPU: the headline GEMM for seconds, not
            # milliseconds -- the clocks settle under the power cap
            try:
                swk = make_gemm(env, "cfg2", wl, args.sets)
                per_ms = res["local_ms"] / res["steps"]
                n_sus = max(100, int(args.sustained_seconds * 1e3 / per_ms * 1.15))
                r = timed(env, swk, n_sus, 3, "plain" if args.graph == "off" else "gate")
                rec = sub_record(env, "cfg2", wl, swk, r)
                rec["seconds"] = r["local_ms"] / 1e3
                configs["sustained"] = rec
                release(swk)
                swk = None
            except Exception as exc:  # noqa: BLE001
                configs["sustained"] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        if world > 1:
            try:
                configs["cfg5_splitk"] = splitk_record(env, WORKLOADS["cfg5_splitk"], 5, 3)
            except Exception as exc:  # noqa: BLE001
                configs["cfg5_splitk"] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    if configs:
        line["configs"] = configs
    line.update(extra)
    if env.rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
