"""The allocation-free convolution entry point (aiehlc_conv2d_i8_srs_static_dev).

It exists for callers that cannot allocate device memory at the time of the call -- a frozen
memory pool, a loop that must stay clear of the driver's allocator lock, a host that owns the whole
device -- so its weight scratch is a fixed array inside the library rather than a cudaMalloc'd
workspace.  This test calls it through the C ABI twice in a row, with different inputs, and checks
each result bit for bit against the regular entry point (integer path: no tolerance), plus the size
limit.  The file name sorts last so that a run stopping at the first failure has already run
everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from aiehlc_b200 import _capi, synth
from aiehlc_b200.ops import Context

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _run(lib, h, fn_name, x, w, sv, pad):
    n, hh, ww, cin = x.shape
    kh, kw, _, cout = w.shape
    y = torch.full((n, hh, ww, cout), 0x55, dtype=torch.int8, device=DEV)
    stream = C.c_void_p(torch.cuda.current_stream(0).cuda_stream)
    rc = getattr(lib, fn_name)(h, _ptr(x), _ptr(w), _ptr(y), n, hh, ww, cin, cout, kh, kw, pad, _ptr(sv), stream)
    return rc, y


def test_static_scratch_conv_matches_regular_entry_point_twice():
    lib = _capi.load()
    ctx = Context(0)
    try:
        cases = [
            ((1, 56, 56, 64), (3, 3, 64, 64), 1, 4),      # the benchmark convolution
            ((2, 9, 20, 128), (3, 3, 128, 48), 1, 14),    # other shape, other values: nothing may leak over
        ]
        for xs, ws, pad, seed in cases:
            x = torch.from_numpy(synth.int8_uniform(seed, xs)).to(DEV)
            w = torch.from_numpy(synth.int8_uniform(seed + 1000, ws)).to(DEV)
            sv = torch.from_numpy((np.arange(ws[3]) % 9 + 2).astype(np.uint8)).to(DEV)
            rc_ref, y_ref = _run(lib, ctx._h, "aiehlc_conv2d_i8_srs_dev", x, w, sv, pad)
            rc_new, y_new = _run(lib, ctx._h, "aiehlc_conv2d_i8_srs_static_dev", x, w, sv, pad)
            assert rc_ref == _capi.OK and rc_new == _capi.OK, lib.aiehlc_last_error()
            assert ctx.sync() == 0
            assert torch.equal(y_new, y_ref)
            assert not torch.all(y_new == 0x55)
        # weights beyond the fixed scratch are refused with a clear message, nothing is launched
        big_x = torch.zeros((1, 4, 4, 512), dtype=torch.int8, device=DEV)
        big_w = torch.zeros((3, 3, 512, 256), dtype=torch.int8, device=DEV)       # 1,179,648 bytes > 1 MiB
        sv = torch.zeros(256, dtype=torch.uint8, device=DEV)
        before = ctx.launch_count
        rc, _ = _run(lib, ctx._h, "aiehlc_conv2d_i8_srs_static_dev", big_x, big_w, sv, 1)
        assert rc == _capi.ERR_UNSUPPORTED and b"static scratch" in lib.aiehlc_last_error()
        assert ctx.launch_count == before
        rc, _ = _run(lib, ctx._h, "aiehlc_conv2d_i8_srs_dev", big_x, big_w, sv, 1)    # the regular one takes it
        assert rc == _capi.OK and ctx.sync() == 0
    finally:
        ctx.close()


@pytest.mark.parametrize("xs,ws,pad", [
    ((1, 10, 12, 24), (3, 3, 24, 16), 1),        # cin outside the tensor-core tiling: the CUDA-core kernel, no scratch
    ((1, 12, 12, 64), (5, 5, 64, 48), 2),        # 5 x 5 filter, weights re-laid into the static array
    ((2, 6, 6, 128), (3, 3, 128, 512), 1),       # more output channels than one MMA: several channel tiles
    ((1, 8, 8, 256), (1, 1, 256, 256), 0),       # 1 x 1 filter: per-tap form
    ((1, 5, 5, 512), (1, 1, 512, 2048), 0),         # weights of exactly 1 MiB: the limit itself is accepted
])
def test_static_scratch_conv_other_forms(xs, ws, pad):
    lib = _capi.load()
    assert ws[0] * ws[1] * ws[2] * ws[3] <= 1 << 20
    ctx = Context(0)
    try:
        x = torch.from_numpy(synth.int8_uniform(21, xs)).to(DEV)
        w = torch.from_numpy(synth.int8_uniform(1021, ws)).to(DEV)
        sv = torch.from_numpy((np.arange(ws[3]) % 11).astype(np.uint8)).to(DEV)
        rc_ref, y_ref = _run(lib, ctx._h, "aiehlc_conv2d_i8_srs_dev", x, w, sv, pad)
        rc_new, y_new = _run(lib, ctx._h, "aiehlc_conv2d_i8_srs_static_dev", x, w, sv, pad)
        assert rc_ref == _capi.OK and rc_new == _capi.OK, lib.aiehlc_last_error()
        assert ctx.sync() == 0
        assert torch.equal(y_new, y_ref)
        # the same tiling serves both entry points: what aiehlc_plan_conv2d says is what either runs
        gen = lib.aiehlc_workspace_generation(ctx._h)
        rc_new, y_again = _run(lib, ctx._h, "aiehlc_conv2d_i8_srs_static_dev", x, w, sv, pad)
        assert rc_new == _capi.OK and ctx.sync() == 0 and torch.equal(y_again, y_ref)
        assert lib.aiehlc_workspace_generation(ctx._h) == gen          # no workspace moved
    finally:
        ctx.close()


def test_static_scratch_conv_empty_batch_and_two_contexts():
    lib = _capi.load()
    a, b = Context(0), Context(0)
    try:
        x0 = torch.zeros((0, 8, 8, 64), dtype=torch.int8, device=DEV)
        w = torch.from_numpy(synth.int8_uniform(1031, (3, 3, 64, 48))).to(DEV)
        sv = torch.full((48,), 5, dtype=torch.uint8, device=DEV)
        before = a.launch_count
        rc, _ = _run(lib, a._h, "aiehlc_conv2d_i8_srs_static_dev", x0, w, sv, 1)
        assert rc == _capi.OK and a.launch_count == before             # n == 0: nothing to do, nothing launched
        # two contexts on one device share the one array: used one after the other (never overlapping),
        # each gets its own weights' result
        for seed, c in ((41, a), (42, b), (43, a)):
            x = torch.from_numpy(synth.int8_uniform(seed, (1, 9, 9, 64))).to(DEV)
            w = torch.from_numpy(synth.int8_uniform(seed + 1000, (3, 3, 64, 48))).to(DEV)
            rc_ref, y_ref = _run(lib, c._h, "aiehlc_conv2d_i8_srs_dev", x, w, sv, 1)
            torch.cuda.synchronize()
            rc_new, y_new = _run(lib, c._h, "aiehlc_conv2d_i8_srs_static_dev", x, w, sv, 1)
            torch.cuda.synchronize()
            assert rc_ref == _capi.OK and rc_new == _capi.OK, lib.aiehlc_last_error()
            assert torch.equal(y_new, y_ref)
    finally:
        a.close()
        b.close()


def test_a_small_static_call_does_not_lower_the_shared_memory_limit_of_later_calls():
    """The dynamic shared-memory limit of a kernel belongs to the device, not to a context: a call that
    needs little (from either entry point, from any context) must not leave a later, larger one without."""
    lib = _capi.load()
    a, b = Context(0), Context(0)
    try:
        big = ((2, 9, 20, 128), (3, 3, 128, 48))
        small = ((1, 6, 6, 32), (1, 1, 32, 16))
        outs = []
        for ctx_, name, (xs, ws) in ((a, "aiehlc_conv2d_i8_srs_dev", big), (b, "aiehlc_conv2d_i8_srs_static_dev", small),
                                     (b, "aiehlc_conv2d_i8_srs_dev", small), (a, "aiehlc_conv2d_i8_srs_dev", big),
                                     (b, "aiehlc_conv2d_i8_srs_static_dev", big)):
            x = torch.from_numpy(synth.int8_uniform(51, xs)).to(DEV)
            w = torch.from_numpy(synth.int8_uniform(1051, ws)).to(DEV)
            sv = torch.full((ws[3],), 6, dtype=torch.uint8, device=DEV)
            rc, y = _run(lib, ctx_._h, name, x, w, sv, ws[0] // 2)
            assert rc == _capi.OK, lib.aiehlc_last_error()
            torch.cuda.synchronize()
            assert ctx_.sync() == 0
            outs.append(y)
        assert torch.equal(outs[0], outs[3]) and torch.equal(outs[0], outs[4]) and torch.equal(outs[1], outs[2])
    finally:
        a.close()
        b.close()
