"""conv2d (bit-exact) and bf16 GEMM (tolerance) against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from aiehlc_b200 import synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
BF16_TOL = 1e-2   # max |got - ref| / max(|ref|, 1): the benchmark's stated tolerance


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


CONV_SHAPES = [(1, 56, 56, 64, 64),      # the benchmark configuration
               (2, 14, 14, 32, 48), (1, 20, 150, 128, 64), (1, 9, 9, 256, 32), (3, 5, 7, 64, 16),
               (1, 1, 1, 64, 64), (1, 130, 3, 32, 16), (1, 6, 6, 128, 272),
               (1, 8, 8, 24, 16), (2, 5, 5, 3, 8), (1, 4, 4, 64, 10)]   # the last three take the direct kernel


@pytest.mark.parametrize("halo,direct,wide", [(True, True, True), (True, False, True), (True, True, False),
                                              (True, False, False), (False, False, False)])
@pytest.mark.parametrize("shape", CONV_SHAPES)
def test_conv2d_matches_oracle(ctx, shape, halo, direct, wide):
    """The forms of the tensor-core kernel: the tile's input patch fetched once with all taps as views
    into it, with the HWIO weights consumed as they are (one launch) or re-laid first (two), and one
    activation box per tap."""
    n, h, w, cin, cout = shape
    x = synth.int8_uniform(4, (n, h, w, cin))
    wt = synth.int8_uniform(1004, (3, 3, cin, cout))
    sv = np.full(cout, 6, np.uint8)
    exp = O.conv2d_i8_srs(x, wt, sv, pad=1)
    ctx.set_conv_halo(halo)
    ctx.set_conv_hwio_direct(direct)
    ctx.set_conv_wide_n(wide)
    try:
        got = ctx.conv2d_i8_srs(_dev(x), _dev(wt), _dev(sv), pad=1).cpu().numpy()
        assert ctx.sync() == 0
    finally:
        ctx.set_conv_halo(True)
        ctx.set_conv_hwio_direct(True)
        ctx.set_conv_wide_n(False)
    assert np.array_equal(got, exp)


@pytest.mark.parametrize("n", [8, 32, 128])
def test_conv2d_batches_of_the_benchmark_layer(ctx, n):
    """The 56 x 56 x 64 -> 64 layer at batch 8, 32 and 128: images are independent, so every image of the batched
    call equals the single-image call on it (itself bit-exact against the oracle), in every form; two images
    per batch are also checked against the oracle directly."""
    x = synth.int8_uniform(40 + n, (n, 56, 56, 64))
    wt = synth.int8_uniform(1040 + n, (3, 3, 64, 64))
    sv = (np.arange(64) % 7 + 3).astype(np.uint8)
    dx, dw, dsv = _dev(x), _dev(wt), _dev(sv)
    got = ctx.conv2d_i8_srs(dx, dw, dsv, pad=1)
    for img in (0, n - 1):
        assert np.array_equal(got[img].cpu().numpy(), O.conv2d_i8_srs(x[img:img + 1], wt, sv, pad=1)[0])
    single = torch.cat([ctx.conv2d_i8_srs(dx[i:i + 1].contiguous(), dw, dsv, pad=1) for i in range(n)])
    assert torch.equal(got, single)
    try:
        for halo, direct, wide, persistent in ((True, True, True, True), (True, False, False, True), (False, False, False, True),
                                               (True, True, False, False)):
            ctx.set_conv_halo(halo)
            ctx.set_conv_hwio_direct(direct)
            ctx.set_conv_wide_n(wide)
            ctx.set_conv_persistent(persistent)
            assert torch.equal(ctx.conv2d_i8_srs(dx, dw, dsv, pad=1), got)
    finally:
        ctx.set_conv_halo(True)
        ctx.set_conv_hwio_direct(True)
        ctx.set_conv_wide_n(False)
        ctx.set_conv_persistent(True)
    assert ctx.sync() == 0


@pytest.mark.parametrize("shape,kh,pad", [((32, 56, 56, 64, 64), 3, 1),      # the benchmark layer at batch 32
                                          ((48, 28, 28, 32, 48), 3, 1),      # weights re-laid first (channel tile 48)
                                          ((6, 60, 60, 128, 272), 3, 1),     # 17 channel tiles of 16: the CTAs are split between them
                                          ((8, 40, 40, 64, 64), 5, 2),       # 5 x 5 filter
                                          ((4, 30, 300, 64, 32), 3, 1),      # images wider than a tile
                                          ((80, 17, 23, 128, 16), 3, 1),     # ragged tiles, few channels
                                          ((48, 28, 28, 64, 128), 3, 1),     # 128 channels: two tiles per MMA group at most
                                          ((48, 28, 28, 32, 256), 3, 1)])    # 256 channels: one accumulator pair fills TMEM
def test_conv2d_persistent_form_matches_one_tile_form(ctx, shape, kh, pad):
    """Many tiles per SM: CTAs keep the weights in shared memory and walk the tiles.  Same bits as the one-CTA-per-tile
    form (itself checked against the oracle shape by shape), launch after launch; the first and last image are
    also checked against the oracle directly."""
    from aiehlc_b200.ops import plan_conv2d
    n, h, w, cin, cout = shape
    x = synth.int8_uniform(31, (n, h, w, cin))
    wt = synth.int8_uniform(1031, (kh, kh, cin, cout))
    sv = (np.arange(cout) % 9 + 2).astype(np.uint8)
    if cout == 32:
        sv[5] = 31                        # a shift that needs 64-bit rounding
    dx, dw, dsv = _dev(x), _dev(wt), _dev(sv)
    try:
        ctx.set_conv_persistent(False)
        assert plan_conv2d(n, h, w, cin, cout, kh, kh, pad, ctx=ctx)["persistent"] == 0
        want = ctx.conv2d_i8_srs(dx, dw, dsv, pad=pad)
        ctx.set_conv_persistent(True)
        plan = plan_conv2d(n, h, w, cin, cout, kh, kh, pad, ctx=ctx)
        assert plan["persistent"] == 1 and plan["ctas"] <= ctx.sm_count, plan
        for mode in (2, 3, 4, 1):         # the MMAs of one tile at a time, of two, of four tiles interleaved, the default
            ctx.set_conv_persistent(mode)
            for _ in range(2):
                assert torch.equal(ctx.conv2d_i8_srs(dx, dw, dsv, pad=pad), want)
        packed = ctx.conv2d_pack_weights(dw)                      # weights re-laid by the caller: the K-major operand
        assert torch.equal(ctx.conv2d_i8_srs_packed(dx, packed, (kh, kh), dsv, pad=pad), want)
    finally:
        ctx.set_conv_persistent(True)
    for img in (0, n - 1):
        assert np.array_equal(want[img].cpu().numpy(), O.conv2d_i8_srs(x[img:img + 1], wt, sv, pad=pad)[0])
    assert ctx.sync() == 0


@pytest.mark.parametrize("shift", [0, 1, 6, 29, 30])
def test_conv2d_persistent_form_with_one_shift_for_every_channel(ctx, shift):
    """One shift for the whole channel tile keeps the rounding constants in registers (up to shift 29; above that
    the 64-bit form): same bits as the oracle and as the one-tile form."""
    n, h, w, cin, cout = 12, 56, 56, 64, 64
    x = synth.int8_uniform(77, (n, h, w, cin))
    wt = synth.int8_uniform(1077, (3, 3, cin, cout))
    sv = np.full(cout, shift, dtype=np.uint8)
    dx, dw, dsv = _dev(x), _dev(wt), _dev(sv)
    try:
        ctx.set_conv_persistent(False)
        want = ctx.conv2d_i8_srs(dx, dw, dsv, pad=1)
        ctx.set_conv_persistent(True)
        for _ in range(2):
            assert torch.equal(ctx.conv2d_i8_srs(dx, dw, dsv, pad=1), want)
    finally:
        ctx.set_conv_persistent(True)
    for img in (0, n - 1):
        assert np.array_equal(want[img].cpu().numpy(), O.conv2d_i8_srs(x[img:img + 1], wt, sv, pad=1)[0])
    assert ctx.sync() == 0


def test_conv2d_benchmark_shape_is_one_launch(ctx):
    x = _dev(synth.int8_uniform(4, (1, 56, 56, 64)))
    wt = _dev(synth.int8_uniform(1004, (3, 3, 64, 64)))
    sv = _dev(np.full(64, 6, np.uint8))
    ctx.conv2d_i8_srs(x, wt, sv, pad=1)
    before = ctx.launch_count
    ctx.conv2d_i8_srs(x, wt, sv, pad=1)
    assert ctx.launch_count == before + 1            # no weight re-layout pass
    ctx.set_conv_hwio_direct(False)
    try:
        before = ctx.launch_count
        ctx.conv2d_i8_srs(x, wt, sv, pad=1)
        assert ctx.launch_count == before + 2
    finally:
        ctx.set_conv_hwio_direct(True)


@pytest.mark.parametrize("kh,kw,pad,shape", [(5, 5, 2, (1, 12, 12, 64, 32)), (7, 7, 3, (2, 20, 20, 32, 16)),
                                             (3, 3, 1, (1, 10, 200, 64, 48)), (5, 5, 2, (1, 6, 300, 128, 32)),
                                             (3, 3, 1, (1, 3, 126, 256, 64)), (9, 9, 4, (1, 9, 9, 64, 16)),
                                             (1, 1, 0, (1, 8, 8, 256, 32))])
def test_conv2d_other_filters_through_the_patch_form(ctx, kh, kw, pad, shape):
    """Other filter sizes (same-size output: kh = kw = 2 * pad + 1), images wider than one tile (the patch
    form tiles the width in pieces of 128 - (kw - 1) pixels), several input-channel chunks, and the 1 x 1
    filter, which has no patch to share and takes the per-tap form."""
    n, h, w, cin, cout = shape
    x = synth.int8_uniform(6, (n, h, w, cin))
    wt = synth.int8_uniform(1006, (kh, kw, cin, cout))
    sv = ((np.arange(cout) * 5) % 12).astype(np.uint8)
    got = ctx.conv2d_i8_srs(_dev(x), _dev(wt), _dev(sv), pad=pad).cpu().numpy()
    assert ctx.sync() == 0
    assert np.array_equal(got, O.conv2d_i8_srs(x, wt, sv, pad=pad))


def test_conv2d_per_channel_shifts_5x5_and_host_entry(ctx):
    x = synth.int8_uniform(4, (1, 12, 12, 64))
    wt = synth.int8_uniform(1004, (5, 5, 64, 32))
    sv = (np.arange(32) % 14).astype(np.uint8)
    exp = O.conv2d_i8_srs(x, wt, sv, pad=2)
    assert np.array_equal(ctx.conv2d_i8_srs_host(x, wt, sv, pad=2), exp)
    x1 = synth.int8_uniform(4, (1, 10, 10, 32))
    w1 = synth.int8_uniform(1004, (1, 1, 32, 32))
    assert np.array_equal(ctx.conv2d_i8_srs_host(x1, w1, sv, pad=0), O.conv2d_i8_srs(x1, w1, sv, pad=0))


def test_conv2d_with_prepacked_weights(ctx):
    """Weights re-laid once, then one launch per convolution: same bits as the two-launch entry point."""
    x1 = synth.int8_uniform(4, (1, 56, 56, 64))
    x2 = synth.int8_uniform(5, (1, 56, 56, 64))
    wt = synth.int8_uniform(1004, (3, 3, 64, 64))
    sv = np.full(64, 6, np.uint8)
    packed = ctx.conv2d_pack_weights(_dev(wt))
    assert np.array_equal(packed.cpu().numpy(), np.ascontiguousarray(wt.reshape(9, 64, 64).transpose(0, 2, 1)))
    before = ctx.launch_count
    for x in (x1, x2):
        got = ctx.conv2d_i8_srs_packed(_dev(x), packed, (3, 3), _dev(sv), pad=1).cpu().numpy()
        assert np.array_equal(got, O.conv2d_i8_srs(x, wt, sv, pad=1))
    assert ctx.launch_count == before + 2 and ctx.sync() == 0
    from aiehlc_b200 import _capi
    with pytest.raises(_capi.AiehlcError):                     # direct-kernel shapes have no packed form
        ctx.conv2d_i8_srs_packed(_dev(synth.int8_uniform(4, (1, 4, 4, 24))), packed, (3, 3), _dev(sv), pad=1)


def _bf16_err(got_bits, ref32):
    got = synth.bf16_bits_to_f32(got_bits).astype(np.float64)
    return float(np.max(np.abs(got - ref32) / np.maximum(np.abs(ref32), 1.0)))


@pytest.mark.parametrize("shape", [(128, 128, 64), (256, 256, 512), (300, 200, 136), (64, 72, 8), (33, 17, 20),
                                   (1024, 1024, 1024)])
def test_gemm_bf16_within_tolerance(ctx, shape):
    M, N, K = shape
    A = synth.normal_bf16_bits(3, (M, K))
    B = synth.normal_bf16_bits(1003, (N, K))
    ref = O.gemm_bf16(A, B).astype(np.float64)
    got = ctx.gemm_bf16_host(A, B)
    assert _bf16_err(got, ref) <= BF16_TOL
    dA = _dev(A.view(np.int16)).view(torch.bfloat16)
    dB = _dev(B.view(np.int16)).view(torch.bfloat16)
    got_dev = ctx.gemm_bf16(dA, dB).view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got_dev, got)


def _bf16_tight(got_f64, ref_f64, K):
    """Second metric, scaled to the data: with N(0,1) operands the sums have a spread of sqrt(K), so 1e-2
    against max(|ref|, 1) is loose for outputs near zero.  A result rounded to bf16 (8 mantissa bits) from an
    fp32 accumulation must satisfy |got - ref| <= 2^-8 |ref| + 1e-3 sqrt(K); a lost K block (an error of about
    sqrt(128)) does not."""
    bound = np.abs(ref_f64) / 256.0 + 1e-3 * np.sqrt(K)
    return float(np.max(np.abs(got_f64 - ref_f64) / bound))


def test_gemm_bf16_8192_sampled(ctx):
    """bf16 8192^3: 64 full rows + 64 full columns + 4096 random elements against the fp32-accumulated
    oracle, tolerance 1e-2 (abs-or-rel with eps = 1), and the tighter data-scaled bound on the same samples."""
    M = N = K = 8192
    A = synth.normal_bf16_bits(3, (M, K))
    B = synth.normal_bf16_bits(1003, (N, K))
    dA = _dev(A.view(np.int16)).view(torch.bfloat16)
    dB = _dev(B.view(np.int16)).view(torch.bfloat16)
    C = ctx.gemm_bf16(dA, dB)
    assert ctx.sync() == 0
    rng = np.random.default_rng(3)
    rows = np.sort(rng.choice(M, 64, replace=False))
    cols = np.sort(rng.choice(N, 64, replace=False))
    got_rows = C[torch.from_numpy(rows).to(DEV)].view(torch.int16).cpu().numpy().view(np.uint16)
    ref_rows = O.gemm_bf16(A[rows], B).astype(np.float64)
    assert _bf16_err(got_rows, ref_rows) <= BF16_TOL
    assert _bf16_tight(synth.bf16_bits_to_f32(got_rows).astype(np.float64), ref_rows, K) <= 1.0
    got_cols = C[:, torch.from_numpy(cols).to(DEV)].contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    ref_cols = O.gemm_bf16(A, B[cols]).astype(np.float64)
    assert _bf16_err(got_cols, ref_cols) <= BF16_TOL
    assert _bf16_tight(synth.bf16_bits_to_f32(got_cols).astype(np.float64), ref_cols, K) <= 1.0
    ii, jj = rng.integers(0, M, 4096), rng.integers(0, N, 4096)
    a32 = synth.bf16_bits_to_f32(A[ii]).astype(np.float64)
    b32 = synth.bf16_bits_to_f32(B[jj]).astype(np.float64)
    ref = np.einsum("ik,ik->i", a32, b32)
    got = C[torch.from_numpy(ii).to(DEV), torch.from_numpy(jj).to(DEV)].float().cpu().numpy().astype(np.float64)
    assert float(np.max(np.abs(got - ref) / np.maximum(np.abs(ref), 1.0))) <= BF16_TOL
    assert _bf16_tight(got, ref, K) <= 1.0
