#!/usr/bin/env python
"""Benchmark of the aiehlc matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the hot path over one batch of seeded synthetic input.  The default
workload is the int8 4096^3 GEMM with the fused srs epilogue (shift 8, cascade split-K 4), the
configuration the headline metric is quoted on; with N GPUs the GEMM is sharded by rows of A/C
(each rank owns 4096 rows, B replicated, no collective).  One JSON line is printed by rank 0.

The reference arm (--impl reference) times the CPU golden loop restated in oracle/ on the host
cores of this machine, on a bounded sample of the same workload.
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
NVLINK_GBS = 770.0   # measured peer-copy bandwidth per direction per GPU on this pool (nominal 900)
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the committed ncu captures (profiles/)
NCU_TRAFFIC_BYTES = {"cfg2": 33.7e6}

WORKLOADS = {
    # name: (M per GPU or total, N, K, description)
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
    """Polls SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, device_index: int, period_s: float = 0.002):
        self.idx = device_index
        self.period = period_s
        self.samples: list[int] = []
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
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}

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


def reference_arm(args, wl: dict) -> dict:
    """CPU golden restatement (oracle/) on the host cores, bounded sample per step."""
    n, k = wl["N"], wl["K"]
    shift, splitk = wl.get("shift", 8), wl.get("splitk", 1)
    probe_rows = 32
    t_probe, threads = cpu_time_i8_srs(probe_rows, n, k, shift, splitk, seed=2)
    per_row = t_probe / probe_rows
    total_steps = max(1, args.steps + args.warmup)
    budget_s = 90.0
    rows = int(max(16, min(wl["M"], budget_s / total_steps / per_row)))
    from aiehlc_b200 import synth
    from oracle import oracle as O
    O.set_threads(host_threads())
    A = synth.int8_uniform(2, (rows, k))
    B = synth.int8_uniform(1002, (n, k))
    for _ in range(args.warmup):
        O.gemm_i8_srs(A, B, shift=shift, splitk=splitk)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        O.gemm_i8_srs(A, B, shift=shift, splitk=splitk)
    dt = time.perf_counter() - t0
    ops = 2.0 * rows * n * k * args.steps
    tops = ops / dt / 1e12
    sample = f"{rows} of {wl['M']} rows of A per step (full N, K), {args.steps} steps"
    return {
        "impl": "reference", "metric": "int8 GEMM TOPS (srs epilogue), device-timed", "value": tops, "unit": "TOPS",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": wl["scaling"], "vs_baseline": None, "dtype": "int8",
        "data": "synthetic", "config": {"workload": wl["desc"], "sample": sample},
        "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


# --------------------------------------------------------------------------- GPU arm
GATE_HEAD = 128   # calls queued before the gate opens: far below the depth of a stream's launch queue


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
    ap.add_argument("--no-lib", action="store_true", help="skip the library int8 GEMM timing")
    ap.add_argument("--sets", type=int, default=0, help="number of rotating input sets (0 = enough to exceed L2)")
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off", "gate"],
                    help="on: replay the timed steps from one CUDA graph (auto: for the launch-bound workloads cfg1 and "
                         "cfg4 on one GPU); gate: one call per step, the first ones queued behind a stream gate before "
                         "the clock starts (auto: GEMM workloads on several GPUs)")
    ap.add_argument("--splitk-exchange", default="fused", choices=["fused", "nccl"],
                    help="cfg5_splitk: partial sums added into the owners' shards by the GEMM epilogue over peer "
                         "memory (fused), or a full partial matrix followed by NCCL reduce-scatter (nccl)")
    args = ap.parse_args()
    wl = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        if rank == 0:
            ref_wl = wl if wl["kind"] == "i8_srs" else WORKLOADS["cfg2"]
            print(json.dumps(reference_arm(args, ref_wl)), flush=True)
        return 0

    import torch
    from aiehlc_b200 import shard, synth
    from aiehlc_b200.ops import Context

    if not torch.cuda.is_available():
        print(json.dumps({"error": "no CUDA device: bench.py needs a B200 (there is no CPU path)"}))
        return 1
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    ctx = Context(local_rank)
    if args.tile_n:
        ctx.set_tile_n(args.tile_n)
    peaks = load_peaks()
    kind = wl["kind"]
    W, K_steps = max(args.warmup, 3), args.steps

    # launch-bound workloads: the K steps are recorded once and replayed as one CUDA graph, so the timed
    # region measures the GPU and not the interpreter issuing 5 us calls
    # ... and with several ranks, where one rank's interpreter falling behind would set the job's time
    # Several ranks run call by call as one GPU does (a graph replay loses the overlap of consecutive launches:
    # 50.3 against 48.0 us per step), but the stream is held at a gate until the first calls are queued, so that
    # the interpreter is ahead of the GPU when the clock starts; if the gate cannot be set up, a graph is used.
    use_gate = args.graph == "gate" or (args.graph == "auto" and world > 1 and wl["kind"] in ("i8_srs", "i8_i32", "bf16"))
    use_graph = args.graph == "on" or (args.graph == "auto" and args.workload in ("cfg1", "cfg4") and world == 1)
    gate, gate_fallback = None, None
    if use_gate:
        try:
            gate = StreamGate()
        except Exception as exc:  # noqa: BLE001
            use_gate, use_graph = False, True
            gate_fallback = f"{type(exc).__name__}: {exc}"[:160]
    if use_graph or use_gate:
        side = torch.cuda.Stream()
        torch.cuda.set_stream(side)        # calls are bound to the stream current at bind time

    # ---------------------------------------------------------------- build the per-rank workload
    extra = {}
    if gate_fallback:
        extra["gate_fallback"] = gate_fallback
    if kind == "conv":
        n, h, w, cin, cout = wl["n"], wl["h"], wl["w"], wl["cin"], wl["cout"]
        nsets = 8
        xs = [synth.int8_uniform_torch(4 + 10 * i, (n, h, w, cin), dev) for i in range(nsets)]
        ws = [synth.int8_uniform_torch(1004 + 10 * i, (3, 3, cin, cout), dev) for i in range(nsets)]
        sv = torch.full((cout,), wl["shift"], dtype=torch.uint8, device=dev)
        ys = [torch.empty((n, h, w, cout), dtype=torch.int8, device=dev) for _ in range(nsets)]
        ops_per_step = 2.0 * n * h * w * cout * 9 * cin
        alg_bytes = n * h * w * cin + 9 * cin * cout + n * h * w * cout + cout

        calls = [ctx.bound_conv2d_i8_srs(xs[j], ws[j], sv, ys[j], pad=1) for j in range(nsets)]

        def step(i):
            calls[i % nsets]()
        l2_note = f"rotating {nsets} input sets; operands are L2-resident by nature (0.44 MB per step)"
        unit, dtype = "TOPS", "int8"
        m_local, n_dim, k_dim = n * h * w, cout, 9 * cin
    else:
        M, N, K = wl["M"], wl["N"], wl["K"]
        if wl["scaling"] == "weak":
            m_local, row0 = M, rank * M          # every rank owns M rows of a (world*M)-row problem
        else:
            row0, m_local = shard.row_shard(M, world, rank)
        n_dim, k_dim = N, K
        if kind == "i8_i32_splitk":
            k0, k_local = shard.k_range(K, wl["splitk"], world, rank)
            m_local, row0 = M, 0
        else:
            k0, k_local = 0, K
        esize = 2 if kind == "bf16" else 1
        out_esize = {"i8_srs": 1, "i8_i32": 4, "i8_i32_splitk": 4, "bf16": 2, "mm_i32": 4}[kind]
        if kind == "mm_i32":
            esize = 4
        set_bytes = m_local * k_local * esize + N * k_local * esize + m_local * N * out_esize
        nsets = max(1, min(8, -(-2 * L2_BYTES // set_bytes))) if set_bytes < 2 * L2_BYTES else 1
        if kind == "i8_i32_splitk":
            nsets = 1
        if args.sets > 0:
            nsets = args.sets
        As, Bs, Cs = [], [], []
        for i in range(nsets):
            if kind == "mm_i32":
                # the packed window of the examples: A words, then B words
                g = torch.Generator(device=dev).manual_seed(1 + i)
                As.append(torch.randint(-2**31, 2**31 - 1, ((m_local + N) * K,), dtype=torch.int32, device=dev, generator=g))
                Bs.append(None)
                Cs.append(torch.empty((m_local, N), dtype=torch.int32, device=dev))
            elif kind == "bf16":
                As.append(synth.normal_bf16_torch(3 + 10 * i, (m_local, K), dev, start=row0 * K))
                Bs.append(synth.normal_bf16_torch(1003 + 10 * i, (N, K), dev))
                Cs.append(torch.empty((m_local, N), dtype=torch.bfloat16, device=dev))
            else:
                seed = {"cfg2": 2, "cfg1": 1}.get(args.workload, 5)
                a = synth.int8_uniform_torch(seed + 10 * i, (m_local, K), dev, start=row0 * K)
                b = synth.int8_uniform_torch(seed + 1000 + 10 * i, (N, K), dev)
                if k_local != K:
                    a = a[:, k0:k0 + k_local].contiguous()
                    b = b[:, k0:k0 + k_local].contiguous()
                As.append(a)
                Bs.append(b)
                Cs.append(torch.empty((m_local, N), dtype=torch.int8 if kind == "i8_srs" else torch.int32, device=dev))
        ops_per_step = 2.0 * m_local * N * k_local
        alg_bytes = set_bytes
        l2_note = (f"rotating {nsets} input sets; operands are L2-resident by nature ({set_bytes / 1e3:.0f} KB per step)"
                   if nsets * set_bytes < L2_BYTES
                   else f"rotating {nsets} input sets ({nsets * set_bytes / 1e6:.0f} MB) > 126 MB L2" if nsets > 1
                   else f"one input set of {set_bytes / 1e6:.0f} MB > 126 MB L2" if set_bytes > L2_BYTES
                   else f"single input set of {set_bytes / 1e6:.1f} MB")
        rs_out = None
        fused_call = None
        if kind == "i8_i32_splitk":
            rows_out = M // world
            rs_out = torch.empty((rows_out, N), dtype=torch.int32, device=dev)
            if world > 1 and args.splitk_exchange == "fused":
                # every rank's shard of C in memory all ranks can address; the epilogue adds into the owner's shard
                try:
                    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer mappings only
                    import torch.distributed._symmetric_memory as symm
                    sym_out = symm.empty((rows_out, N), dtype=torch.int32, device=dev)
                    hdl = symm.rendezvous(sym_out, dist.group.WORLD)
                    peer_ptrs = [int(p) for p in hdl.buffer_ptrs]
                    fused_call = ctx.bound_gemm_i8_i32_scatter(As[0], Bs[0], peer_ptrs, rows_out, N, first_shard=rank + 1)
                    tick = torch.zeros(1, dtype=torch.int32, device=dev)
                    extra["splitk_exchange"] = "fused: tile add-reductions into the owners' shards over peer memory"
                except Exception as exc:  # noqa: BLE001
                    fused_call = None
                    extra["splitk_exchange"] = f"nccl reduce-scatter (peer memory unavailable: {type(exc).__name__}: {exc})"[:200]
            elif world > 1:
                extra["splitk_exchange"] = "nccl reduce-scatter of a full int32 partial matrix"

        # every argument of the C-ABI call is converted once, outside the timed region
        if kind == "i8_srs":
            calls = [ctx.bound_gemm_i8_srs(As[j], Bs[j], Cs[j], shift=wl["shift"], splitk=wl["splitk"]) for j in range(nsets)]
        elif kind == "mm_i32":
            calls = [(lambda j=j: ctx.mm_i32(As[j], m_local, N, K, out=Cs[j])) for j in range(nsets)]
        elif kind == "bf16":
            calls = [ctx.bound_gemm_bf16(As[j], Bs[j], Cs[j]) for j in range(nsets)]
        else:
            calls = [ctx.bound_gemm_i8_i32(As[j], Bs[j], Cs[j]) for j in range(nsets)]

        def step(i):
            j = i % nsets
            if fused_call is not None:
                sym_out.zero_()
                dist.all_reduce(tick)        # stream-ordered: every shard is zero before anyone adds into it
                fused_call()
                dist.all_reduce(tick)        # ... and every contribution has landed before anyone reads
                return
            calls[j]()
            if kind == "i8_i32_splitk" and world > 1:
                dist.reduce_scatter_tensor(rs_out, Cs[j], op=dist.ReduceOp.SUM)

        if fused_call is not None:
            # once, outside the timed region: the fused exchange gives what GEMM + NCCL reduce-scatter gives
            step(0)
            calls[0]()
            dist.reduce_scatter_tensor(rs_out, Cs[0], op=dist.ReduceOp.SUM)
            same = torch.tensor([1 if torch.equal(rs_out, sym_out) else 0], dtype=torch.int32, device=dev)
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
            extra["splitk_exchange_matches_nccl"] = bool(int(same.item()))
        unit = "TFLOPS" if kind == "bf16" else "TOPS"
        dtype = "bf16" if kind == "bf16" else ("int32 via u8 limbs" if kind == "mm_i32" else "int8")

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize()

    # ---------------------------------------------------------------- warm-up, then the timed region
    for i in range(W):
        step(i)
    ctx.sync()
    graph, graph_launches = None, 0
    if use_graph:
        torch.cuda.synchronize()
        try:
            graph = torch.cuda.CUDAGraph()
            c0 = ctx.launch_count
            with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                for i in range(K_steps):
                    step(i)
            graph_launches = ctx.launch_count - c0
            if args.workload in ("cfg1", "cfg4"):
                graph.replay()           # microsecond kernels: a trial replay costs nothing
            # (the long-running workloads are not replayed beforehand: a whole extra pass would start the timed
            # one under the power cap, unlike the call-by-call form the single-GPU run uses)
            torch.cuda.synchronize()
        except Exception as exc:  # noqa: BLE001  -- recording failed: issue the steps one by one instead
            graph, use_graph = None, False
            extra["graph_fallback"] = f"{type(exc).__name__}: {exc}"[:160]
            torch.cuda.synchronize()
    barrier()
    sampler = ClockSampler(local_rank).start()
    launches0 = ctx.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    if gate is not None:
        try:
            gate.close(side)             # everything queued from here on waits for gate.open()
        except Exception as exc:  # noqa: BLE001  -- no gate on this system: plain call-by-call run
            extra["gate_fallback"] = f"{type(exc).__name__}: {exc}"[:160]
            gate = None
    if gate is not None:
        try:
            e0.record()
            head = min(K_steps, GATE_HEAD)
            for i in range(K_steps):
                if i == head:
                    gate.open()
                step(i)
        finally:
            gate.open()
    else:
        e0.record()
        if graph is not None:
            graph.replay()
        else:
            for i in range(K_steps):
                step(i)
    e1.record()
    barrier()
    elapsed_ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    launches = graph_launches if graph is not None else ctx.launch_count - launches0
    status = ctx.sync()
    t = torch.tensor([elapsed_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    max_ms = float(t.item())
    total_ops = ops_per_step * K_steps * world
    value = total_ops / (max_ms * 1e-3) / 1e12

    # roofline of the dominant kernel on this rank: algorithmic ops per launch / mean launch time
    per_launch_ms = elapsed_ms / K_steps
    achieved = ops_per_step / (per_launch_ms * 1e-3) / 1e12
    if kind == "conv":
        gbs = alg_bytes / (per_launch_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                    "note": f"latency-bound: {per_launch_ms * 1e3:.1f} us per conv ({launches // max(K_steps, 1)} launch(es) "
                            f"per step, HWIO weights as given); peak {peaks['source']}"}
    else:
        # burst peak for a short timed region, sustained (power-capped) peak once it runs for long
        sustained = elapsed_ms > 250.0
        base = peaks["bf16_sustained"] if sustained else peaks["bf16"]
        which = "sustained" if sustained else "burst"
        peak = base * (1.0 if dtype == "bf16" else 2.0)
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                    "traffic": NCU_TRAFFIC_BYTES.get(args.workload),
                    "note": (f"peak = 2 x measured bf16 {which} (kind::i8 has twice the K per instruction)"
                             if dtype != "bf16" else f"peak = measured bf16 {which}") +
                            f", of {peaks['source']}; timed region {elapsed_ms:.0f} ms"}
    if wl.get("bound") == "hbm" and kind != "conv":
        # a product over a shallow K: the result bytes, not the MMAs, bound the launch
        gemm_bytes = wl["M"] * wl["K"] + wl["N"] * wl["K"] + wl["M"] * wl["N"] * 4
        gbs = gemm_bytes / (per_launch_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": gbs / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES.get(args.workload),
                    "note": f"algorithmic bytes A + B + C(int32) = {gemm_bytes / 1e6:.1f} MB per launch; peak {peaks['source']}"}
    if kind == "mm_i32":
        # one int32 product costs ten int8 limb products (K + 2K + 3K + 4K bytes of depth)
        roofline["achieved"] = achieved * 10.0
        roofline["frac"] = achieved * 10.0 / roofline["peak"]
        roofline["note"] = ("int8 tensor work = 10 x 2MNK (four limb GEMMs of depth K, 2K, 3K, 4K); value counts the "
                            "int32 multiply-adds; " + roofline["note"])
    if kind == "i8_i32_splitk" and world > 1:
        # compute step followed by an exchange: the target time is the slower of the two legs
        wire_bytes = (world - 1) / world * wl["M"] * wl["N"] * 4            # int32 partial sums leaving this GPU
        t_math = ops_per_step / (peak * 1e12)
        t_wire = wire_bytes / (NVLINK_GBS * 1e9)
        gbs = wire_bytes / (per_launch_ms * 1e-3) / 1e9
        roofline = {"bound": "nvlink", "achieved": gbs, "peak": NVLINK_GBS, "unit": "GB/s",
                    "frac": max(t_math, t_wire) / (per_launch_ms * 1e-3), "traffic": None,
                    "note": f"target = max(math {t_math * 1e3:.2f} ms at the tensor peak, wire {t_wire * 1e3:.2f} ms: "
                            f"{wire_bytes / 1e9:.2f} GB of int32 partial sums per GPU at the measured {NVLINK_GBS:.0f} GB/s "
                            "peer-copy rate per direction); frac = target / measured step"}
    extra.update(extra_measurements(args, wl, ctx, dev, kind, rank))

    # ---------------------------------------------------------------- end-to-end through the host API
    e2e = None
    if not args.no_e2e and kind == "i8_srs":
        e2e = e2e_i8_srs(ctx, wl, m_local, rank, world, dist, dev, min(K_steps, 20))

    line = {
        "metric": "int8 GEMM TOPS (srs epilogue), device-timed" if kind == "i8_srs" else f"{args.workload} {unit}, device-timed",
        "value": value, "unit": unit, "n_gpus": world, "steps": K_steps, "warmup": W, "ms_per_step": max_ms / K_steps,
        "higher_is_better": True, "scaling": wl["scaling"], "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": {"workload": wl["desc"], "per_gpu": f"M={m_local} N={n_dim} K={k_dim}", "parallelism": f"row-shard x{world}",
                   "l2": l2_note, "tile_n": args.tile_n or "auto",
                   "launch": "the K steps replayed from one CUDA graph" if use_graph else
                             (f"one C-ABI call per step, the first {min(K_steps, GATE_HEAD)} queued behind a stream gate before the clock starts"
                              if gate is not None else "one C-ABI call per step")},
        "roofline": roofline, "clocks": clocks, "gpu_launches": int(launches), "device_status": int(status),
    }
    if e2e is not None:
        line["e2e"] = e2e
    if rank == 0 and world == 1 and not args.no_cpu and kind == "i8_srs":
        rows = 1024
        sec, threads = cpu_time_i8_srs(rows, n_dim, k_dim, wl["shift"], wl["splitk"], seed=2)
        # scale the sample so the CPU leg runs roughly 10 s in total
        reps = int(max(1, min(16, 10.0 / max(sec, 1e-3))))
        if reps > 1:
            sec, threads = cpu_time_i8_srs(rows, n_dim, k_dim, wl["shift"], wl["splitk"], seed=2, reps=reps)
        line["cpu_baseline"] = {"value": 2.0 * rows * n_dim * k_dim / sec / 1e12, "unit": "TOPS", "cores": threads,
                                "kind": "port", "sample": f"{rows} of {m_local} rows (full N, K) x {reps} repetitions, "
                                                          "oracle GEMM + srs with OpenMP"}
    if kind == "conv" and use_graph:
        # the same convolutions with weights re-laid once beforehand (one launch per convolution), for context
        packed = [ctx.conv2d_pack_weights(ws[j]) for j in range(nsets)]
        for j in range(nsets):
            ctx.conv2d_i8_srs_packed(xs[j], packed[j], (3, 3), sv, pad=1, out=ys[j])
        torch.cuda.synchronize()
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g2, stream=side, capture_error_mode="thread_local"):
            for i in range(K_steps):
                ctx.conv2d_i8_srs_packed(xs[i % nsets], packed[i % nsets], (3, 3), sv, pad=1, out=ys[i % nsets])
        g2.replay()
        torch.cuda.synchronize()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record()
        g2.replay()
        p1.record()
        torch.cuda.synchronize()
        extra["prepacked_weights_us_per_conv"] = p0.elapsed_time(p1) / K_steps * 1e3
    line.update(extra)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


def extra_measurements(args, wl, ctx, dev, kind, rank) -> dict:
    """Library int8 GEMM on the same shape, for context (not part of the metric)."""
    import torch
    out = {}
    if kind == "i8_srs" and rank == 0 and not args.no_lib:
        try:
            M, N, K = wl["M"], wl["N"], wl["K"]
            a = torch.randint(-128, 128, (M, K), dtype=torch.int8, device=dev)
            b = torch.randint(-128, 128, (N, K), dtype=torch.int8, device=dev)
            for _ in range(5):
                torch._int_mm(a, b.T)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(50):
                torch._int_mm(a, b.T)
            e1.record()
            torch.cuda.synchronize()
            out["library_int8_tops"] = 2.0 * M * N * K / (e0.elapsed_time(e1) / 50 * 1e-3) / 1e12
        except Exception as exc:  # noqa: BLE001
            out["library_int8_tops"] = f"unavailable: {exc}"
    return out


def e2e_i8_srs(ctx, wl, m_local, rank, world, dist, dev, steps) -> dict:
    """Same metric through the host-buffer entry point: pinned host A, B -> device, GEMM + srs, C -> host."""
    import numpy as np
    import torch
    from aiehlc_b200 import synth
    N, K = wl["N"], wl["K"]
    a = torch.from_numpy(synth.int8_uniform(2, (m_local, K), start=rank * m_local * K)).pin_memory()
    b = torch.from_numpy(synth.int8_uniform(1002, (N, K))).pin_memory()
    c = torch.empty((m_local, N), dtype=torch.int8).pin_memory()
    an, bn, cn = a.numpy(), b.numpy(), c.numpy()
    for _ in range(3):
        ctx.gemm_i8_srs_host(an, bn, shift=wl["shift"], splitk=wl["splitk"], out=cn)
    if world > 1:
        dist.barrier(device_ids=[dev.index])
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        ctx.gemm_i8_srs_host(an, bn, shift=wl["shift"], splitk=wl["splitk"], out=cn)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    tt = torch.tensor([dt], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    dt = float(tt.item())
    ops = 2.0 * m_local * N * K * steps * world
    return {"value": ops / dt / 1e12, "unit": "TOPS", "h2d_bytes_per_step": int(an.nbytes + bn.nbytes),
            "d2h_bytes_per_step": int(cn.nbytes), "steps": steps,
            "api": "aiehlc_gemm_i8_srs_host (pinned host buffers, copies inside the timed region)"}


if __name__ == "__main__":
    sys.exit(main())
