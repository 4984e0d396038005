"""Clock-stamp timelines of the kernels, from the measurement build of the library.

    AIEHLC_MEASURE=1 python -m aiehlc_b200.build                    # libaiehlc_b200_measure.so
    AIEHLC_MEASURE=1 python -m aiehlc_b200.measure gemm-pace        # the CTA-pair GEMM, tile by tile
    AIEHLC_MEASURE=1 python -m aiehlc_b200.measure conv-timeline    # the convolution kernels

The measurement build writes clock64() stamps of one CTA into a buffer given with aiehlc_set_trace and can leave
out part of a kernel (aiehlc_set_debug: 1 = no TMA loads, 2 = no MMAs; results are then meaningless, the timing is
the point).  The regular build has neither.  Needs a B200; prints SM cycles.
"""
from __future__ import annotations

import os
import sys


def _context():
    if os.environ.get("AIEHLC_MEASURE", "0") in ("", "0"):
        raise SystemExit("set AIEHLC_MEASURE=1: the stamps exist only in the measurement build")
    import torch

    from .ops import Context
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    return Context(0), torch.device("cuda", 0), torch


def gemm_pace(M: int = 4096, N: int = 4096, K: int = 4096) -> None:
    """Per work unit of one CTA pair of the int8 GEMM + srs: when its MMAs started, when the last was issued, when
    the accumulator was complete, when its output stage ended -- with everything on, with the TMA loads left out
    (the tensor core's pace on whatever is in shared memory) and with the MMAs left out (the loads' pace)."""
    ctx, dev, torch = _context()
    A = torch.randint(-128, 128, (M, K), dtype=torch.int8, device=dev)
    B = torch.randint(-128, 128, (N, K), dtype=torch.int8, device=dev)
    out = torch.empty((M, N), dtype=torch.int8, device=dev)

    def run():
        ctx.gemm_i8_srs(A, B, shift=8, out=out)

    k_blocks = K // 128
    for mode, what in ((0, "loads and MMAs"), (1, "MMAs only (no TMA loads)"), (2, "loads only (no MMAs)")):
        ctx.set_debug(mode)
        for cta in (40, 146):
            os.environ["AIEHLC_TRACE_CTA"] = str(cta)
            trace = torch.zeros(8 * 64, dtype=torch.int64, device=dev)
            for _ in range(5):
                run()
            ctx.set_trace(trace)
            run()
            torch.cuda.synchronize()
            ctx.set_trace(None)
            t = trace.view(-1, 8).cpu()
            t0 = int(t[0, 5])
            print(f"{what}: CTA {cta} (pair {cta // 2}), entry to exit {int(t[0, 6]) - t0} cycles")
            for i in range(t.shape[0]):
                if int(t[i, 0]) == 0:
                    break
                start, issued, _, ready, done = (int(v) - t0 for v in t[i, :5])
                print(f"    unit {i}: MMAs from {start:7d}, last issued {issued:7d}, accumulator complete {ready:7d}, "
                      f"output stage done {done:7d} | main loop {ready - start:6d} cycles = "
                      f"{(ready - start) / (4 * k_blocks):.0f} per MMA if the unit is a whole tile")
    ctx.set_debug(0)
    print("status word", ctx.sync())


def conv_timeline() -> None:
    """The 56 x 56 x 64 -> 64 layer, 3 x 3: the batch-1 kernel's chain of latencies (CTA 0) and, at batch 128, the
    persistent kernel's groups of four tiles (MMA warp) and its output stage (first output warp, even tiles)."""
    ctx, dev, torch = _context()
    from . import synth
    sv = torch.full((64,), 6, dtype=torch.uint8, device=dev)
    nsets = 8
    xs = [synth.int8_uniform_torch(4 + i, (1, 56, 56, 64), dev) for i in range(nsets)]
    ws = [synth.int8_uniform_torch(1004 + i, (3, 3, 64, 64), dev) for i in range(nsets)]
    y = torch.empty((1, 56, 56, 64), dtype=torch.int8, device=dev)
    for k in range(6):
        ctx.conv2d_i8_srs(xs[k % nsets], ws[k % nsets], sv, pad=1, out=y)
    for rep in range(3):
        trace = torch.zeros(64, dtype=torch.int64, device=dev)
        ctx.set_trace(trace)
        ctx.conv2d_i8_srs(xs[(rep + 3) % nsets], ws[(rep + 3) % nsets], sv, pad=1, out=y)
        torch.cuda.synchronize()
        ctx.set_trace(None)
        t = trace.cpu().tolist()
        t0 = t[0]
        print(f"batch 1, CTA 0: dependency wait over {t[1] - t0}, patch landed {t[2] - t0}, MMAs issued {t[3] - t0}, "
              f"accumulator complete {t[4] - t0}, output stage done {t[5] - t0}, exit {t[6] - t0}")
    n = 128
    x = synth.int8_uniform_torch(4, (n, 56, 56, 64), dev)
    y = torch.empty((n, 56, 56, 64), dtype=torch.int8, device=dev)
    for mode, what in ((2, "one tile per MMA group"), (3, "two tiles"), (4, "four tiles")):
        ctx.set_conv_persistent(mode)
        for _ in range(3):
            ctx.conv2d_i8_srs(x, ws[0], sv, pad=1, out=y)
        trace = torch.zeros(512, dtype=torch.int64, device=dev)
        ctx.set_trace(trace)
        ctx.conv2d_i8_srs(x, ws[0], sv, pad=1, out=y)
        torch.cuda.synchronize()
        ctx.set_trace(None)
        t = trace.view(-1, 4).cpu()
        t0 = int(t[0, 0])
        print(f"batch {n}, persistent form, {what}:")
        for i in range(26):
            a, b, c, d = (int(v) for v in t[i])
            parts = []
            if a:
                parts.append(f"group's MMAs from {a - t0:6d} to {b - t0:6d} ({b - a} cycles)")
            if c:
                parts.append(f"output stage {c - t0:6d} to {d - t0:6d} ({d - c} cycles)")
            if parts:
                print(f"    tile {i:2d}: " + ", ".join(parts))
    ctx.set_conv_persistent(1)
    print("status word", ctx.sync())


def main(argv) -> int:
    if len(argv) != 2 or argv[1] not in ("gemm-pace", "conv-timeline"):
        print(__doc__)
        return 2
    {"gemm-pace": gemm_pace, "conv-timeline": conv_timeline}[argv[1]]()
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
