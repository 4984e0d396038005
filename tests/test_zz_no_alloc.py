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
