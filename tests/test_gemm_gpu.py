"""Parity of the CUDA GEMM path with the CPU oracle, through the C ABI.  Integer results are
compared bit for bit."""
import numpy as np
import pytest
import torch

from aiehlc_b200 import _capi, synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


# ---------------------------------------------------------------- the reference's own kernel (int32)
def test_perf_fixture_matches_reference_output(ctx, golden):
    packed = np.arange(1, 513, dtype=np.int32)                      # example/perf/aieml_perf.cc:141-144
    got = ctx.mm_i32(_dev(packed), 16, 16, 16).cpu().numpy()
    assert np.array_equal(got.ravel(), np.array(golden["aieml_perf"]["words_read_back"][:256], dtype=np.int32))
    assert np.array_equal(ctx.mm_i32_host(packed, 16, 16, 16), got)


def test_reference_fixtures_through_the_tensor_core_form(ctx, golden):
    """The reference's own 16 x 16 x 16 program output (and the 8 x 8 fixture) reproduced by the byte-limb
    GEMMs on the tensor cores, forced for these tiny sizes."""
    ctx.set_mm_i32_tensor(2)
    try:
        packed = np.arange(1, 513, dtype=np.int32)                      # example/perf/aieml_perf.cc:141-144
        got = ctx.mm_i32(_dev(packed), 16, 16, 16).cpu().numpy()
        assert np.array_equal(got.ravel(), np.array(golden["aieml_perf"]["words_read_back"][:256], dtype=np.int32))
        c8 = ctx.mm_i32_host(np.arange(0, 128, dtype=np.int32), 8, 8, 8)  # aieoob.c:83-86
        assert np.array_equal(c8, O.mm_i32(np.arange(0, 128, dtype=np.int32), 8, 8, 8))
        rng = np.random.default_rng(12)
        for (M, N, K) in [(1, 1, 1), (33, 17, 7), (100, 70, 33)]:
            inp = rng.integers(-2**31, 2**31 - 1, size=(M + N) * K, dtype=np.int64).astype(np.int32)
            assert np.array_equal(ctx.mm_i32_host(inp, M, N, K), O.mm_i32(inp, M, N, K))
        assert ctx.sync() == 0
    finally:
        ctx.set_mm_i32_tensor(1)


def test_mm_fixtures_known_answers(ctx):
    c = ctx.mm_i32_host(np.arange(0, 512, dtype=np.int32), 16, 16, 16)    # aieml_mm.cc:137-140
    assert (c[0, 0], c[0, 15], c[15, 0], c[15, 15], int(c.sum(dtype=np.int64))) == (31960, 60760, 1043800, 1994200, 200366080)
    c = ctx.mm_i32_host(np.arange(0, 128, dtype=np.int32), 8, 8, 8)       # aieoob.c:83-86
    assert np.array_equal(c, O.mm_i32(np.arange(0, 128, dtype=np.int32), 8, 8, 8))


@pytest.mark.parametrize("shape", [(16, 16, 16), (1, 1, 1), (100, 70, 33), (257, 129, 65)])
def test_mm_i32_wraparound(ctx, shape):
    M, N, K = shape
    rng = np.random.default_rng(7)
    inp = rng.integers(-2**31, 2**31 - 1, size=(M + N) * K, dtype=np.int64).astype(np.int32)
    assert np.array_equal(ctx.mm_i32_host(inp, M, N, K), O.mm_i32(inp, M, N, K))


@pytest.mark.parametrize("shape", [(512, 384, 1000), (300, 200, 4100), (1024, 1024, 1024), (130, 70, 8256), (256, 64, 64),
                                   (128, 64, 20000)])
def test_mm_i32_on_the_tensor_cores(ctx, shape):
    """Large int32 products run as int8 limb GEMMs on the tensor cores: full-range random words, and the
    all-ones words that make every limb product as large as it can get (K goes in ranges of 8192 columns: up to
    8256 no partial sum can reach 2^31), against the oracle and against the CUDA-core kernel."""
    M, N, K = shape
    rng = np.random.default_rng(11)
    inp = rng.integers(-2**31, 2**31 - 1, size=(M + N) * K, dtype=np.int64).astype(np.int32)
    d_in = _dev(inp)
    got = ctx.mm_i32(d_in, M, N, K)
    assert np.array_equal(got.cpu().numpy(), O.mm_i32(inp, M, N, K))
    ones = _dev(np.full((M + N) * K, -1, dtype=np.int32))                 # 0xFFFFFFFF everywhere
    got_ones = ctx.mm_i32(ones, M, N, K)
    assert bool((got_ones == K).all())                                    # (-1) * (-1) summed K times
    ctx.set_mm_i32_tensor(False)
    try:
        assert torch.equal(ctx.mm_i32(d_in, M, N, K), got)
    finally:
        ctx.set_mm_i32_tensor(True)
    assert ctx.sync() == 0


# ---------------------------------------------------------------- int8 -> int32
SHAPES = [(64, 64, 64),            # the single-tile configuration
          (128, 256, 128), (256, 512, 1024), (1024, 1024, 1024),
          (1, 1, 16), (1, 16, 1), (130, 70, 48), (300, 200, 400),        # ragged M, N
          (100, 60, 50), (33, 17, 7), (5, 3, 1),                         # K not a multiple of 16: repack path
          (127, 255, 4096), (129, 257, 144)]


@pytest.mark.parametrize("pair", [-1, 0, 1])
@pytest.mark.parametrize("tile_n", [0, 64, 128, 256])
@pytest.mark.parametrize("shape", SHAPES)
def test_gemm_i8_i32_matches_oracle(ctx, shape, tile_n, pair):
    """Every tile shape of both kernel families (one CTA per tile, CTA pair per tile)."""
    M, N, K = shape
    A = synth.int8_uniform(1, (M, K))
    B = synth.int8_uniform(1001, (N, K))
    ctx.set_tile_n(tile_n)
    ctx.set_cta_pair(pair)
    try:
        got = ctx.gemm_i8_i32(_dev(A), _dev(B)).cpu().numpy()
    finally:
        ctx.set_tile_n(0)
        ctx.set_cta_pair(-1)
    assert ctx.sync() == 0
    assert np.array_equal(got, O.gemm_i8_i32(A, B))


@pytest.mark.parametrize("offset", [0, 1, 2, 3, 8])
@pytest.mark.parametrize("K", [17, 19, 50, 333, 1001, 3000])
def test_operands_with_unaligned_rows_or_base(ctx, K, offset):
    """Row pitches and base addresses TMA cannot take (not multiples of 16 bytes): the operands are first
    copied to a pitched workspace, 16 bytes per thread from any byte alignment; same bytes as the oracle
    for int8 (int32 and srs results) and within the bf16 tolerance for bf16 (2-byte alignment)."""
    M, N = 150, 70
    A = synth.int8_uniform(21, (M, K))
    B = synth.int8_uniform(1021, (N, K))
    flat_a = torch.zeros(M * K + 64, dtype=torch.int8, device=DEV)
    flat_b = torch.zeros(N * K + 64, dtype=torch.int8, device=DEV)
    dA = flat_a[offset:offset + M * K].view(M, K)
    dB = flat_b[offset + 1:offset + 1 + N * K].view(N, K)
    dA.copy_(_dev(A)); dB.copy_(_dev(B))
    assert np.array_equal(ctx.gemm_i8_i32(dA, dB).cpu().numpy(), O.gemm_i8_i32(A, B))
    assert np.array_equal(ctx.gemm_i8_srs(dA, dB, shift=6).cpu().numpy(), O.gemm_i8_srs(A, B, shift=6))
    Ab = synth.normal_bf16_bits(22, (M, K))
    Bb = synth.normal_bf16_bits(1022, (N, K))
    flat = torch.zeros((M + N) * K + 64, dtype=torch.bfloat16, device=DEV)
    dAb = flat[offset:offset + M * K].view(M, K)
    dBb = flat[offset + M * K + 1:offset + M * K + 1 + N * K].view(N, K)
    dAb.copy_(_dev(Ab.view(np.int16)).view(torch.bfloat16)); dBb.copy_(_dev(Bb.view(np.int16)).view(torch.bfloat16))
    ref = O.gemm_bf16(Ab, Bb).astype(np.float64)
    gf = ctx.gemm_bf16(dAb, dBb).float().cpu().numpy().astype(np.float64)
    assert float(np.max(np.abs(gf - ref) / np.maximum(np.abs(ref), 1.0))) <= 1e-2      # the bf16 tolerance
    assert ctx.sync() == 0


def test_extreme_values_and_host_entry_point(ctx):
    M, N, K = 192, 160, 8192                                            # |acc| reaches 2^27
    A = np.full((M, K), -128, np.int8)
    B = np.full((N, K), -128, np.int8)
    B[::2] = 127
    assert np.array_equal(ctx.gemm_i8_i32_host(A, B), O.gemm_i8_i32(A, B))


def test_empty_and_zero_sizes(ctx):
    e = torch.empty((0, 64), dtype=torch.int8, device=DEV)
    b = _dev(synth.int8_uniform(1, (32, 64)))
    assert ctx.gemm_i8_i32(e, b).shape == (0, 32)
    a0 = torch.empty((8, 0), dtype=torch.int8, device=DEV)
    b0 = torch.empty((4, 0), dtype=torch.int8, device=DEV)
    assert not ctx.gemm_i8_i32(a0, b0).any()                             # empty contraction: zeros
    assert not ctx.gemm_i8_srs(a0, b0, shift=3).any()
    with pytest.raises(_capi.AiehlcError):
        ctx.gemm_i8_srs(b, b, shift=32)
    with pytest.raises(_capi.AiehlcError):
        ctx.gemm_i8_srs(b, b, shift=1, splitk=7)                         # 7 does not divide 64
    with pytest.raises(ValueError):
        ctx.gemm_i8_i32(b, _dev(synth.int8_uniform(1, (32, 48))))


# ---------------------------------------------------------------- srs epilogue, split-K, cascade
@pytest.mark.parametrize("pair", [0, 1])
@pytest.mark.parametrize("shape,shift", [((256, 256, 256), 8), ((300, 200, 400), 6), ((512, 384, 1024), 0),
                                         ((128, 128, 2048), 12), ((64, 48, 80), 1), ((96, 80, 72), 31),
                                         ((260, 520, 40000), 30), ((140, 100, 33000), 3)])
def test_gemm_i8_srs_matches_oracle(ctx, shape, shift, pair):
    M, N, K = shape
    ctx.set_cta_pair(pair)
    A = synth.int8_uniform(2, (M, K))
    B = synth.int8_uniform(1002, (N, K))
    exp = O.gemm_i8_srs(A, B, shift=shift)
    assert np.array_equal(ctx.gemm_i8_srs(_dev(A), _dev(B), shift=shift).cpu().numpy(), exp)
    assert np.array_equal(ctx.gemm_i8_srs_host(A, B, shift=shift), exp)
    sv = ((np.arange(N) * 7) % 13).astype(np.uint8)
    assert np.array_equal(ctx.gemm_i8_srs(_dev(A), _dev(B), shift_vec=_dev(sv)).cpu().numpy(),
                          O.gemm_i8_srs(A, B, shift_vec=sv))
    assert np.array_equal(ctx.gemm_i8_srs_host(A, B, shift_vec=sv), O.gemm_i8_srs(A, B, shift_vec=sv))
    ctx.set_cta_pair(-1)


def test_srs_rounding_ties_through_the_kernel(ctx):
    # rows of A select one value per row: C[i][j] = a_i * b_j with K = 16 -> products hit exact .5 ties
    K = 16
    A = np.zeros((128, K), np.int8)
    B = np.zeros((128, K), np.int8)
    A[:, 0] = np.arange(-64, 64)
    B[:, 0] = np.arange(-64, 64)[::-1]
    for s in (1, 2, 3, 7):
        assert np.array_equal(ctx.gemm_i8_srs_host(A, B, shift=s), O.gemm_i8_srs(A, B, shift=s))


@pytest.mark.parametrize("splitk", [1, 2, 4, 8])
def test_split_k_in_one_launch_and_as_cascade(ctx, splitk):
    M, N, K = 384, 320, 1024
    A = synth.int8_uniform(2, (M, K))
    B = synth.int8_uniform(1002, (N, K))
    unsplit = O.gemm_i8_srs(A, B, shift=8)
    assert np.array_equal(O.gemm_i8_srs(A, B, shift=8, splitk=splitk), unsplit)
    dA, dB = _dev(A), _dev(B)
    assert np.array_equal(ctx.gemm_i8_srs(dA, dB, shift=8, splitk=splitk).cpu().numpy(), unsplit)
    assert np.array_equal(ctx.gemm_i8_srs_cascade(dA, dB, splitk, shift=8).cpu().numpy(), unsplit)


@pytest.mark.parametrize("shape,tile_n,sms,k_per_load", [
    ((4096, 4096, 2048), 0, 0, 0),       # 256 tiles on 74 pairs: 3 full waves + 34 tail tiles
    ((2560, 2560, 4096), 0, 0, 0),       # 100 tiles: one full wave + 26
    ((2700, 2300, 2176), 0, 0, 0),       # ragged edges, 17 K blocks (odd): halves of 10 and 7
    ((2700, 2300, 2176), 0, 0, 1),       # ... one K block per tile load
    ((5000, 3000, 2064), 0, 0, 0),       # K not a whole number of 128-byte blocks
    ((2048, 1536, 2048), 128, 0, 0),     # 256 x 128 tiles: 96 of them
    ((1280, 1024, 2048), 0, 32, 0),      # 16 pairs (a launch limited to 32 SMs): 20 tiles
    ((1536, 1792, 8192), 0, 24, 0),      # 12 pairs, 42 tiles, a deep K: 64 blocks per tile
])
def test_tail_tiles_as_k_halves_are_bit_identical(ctx, shape, tile_n, sms, k_per_load):
    """A last wave at most half full runs as K halves: the upper halves first, the lower halves last, the partial
    sums added in the lower half's output stage.  Same bits as the oracle and as the whole-tile schedule, launch
    after launch (the deposit counters return to zero), for the int32, the accumulating and the srs output
    stages and both store forms."""
    from aiehlc_b200.ops import plan_gemm
    M, N, K = shape
    ctx.set_cta_pair(1)
    ctx.set_tile_n(tile_n)
    ctx.set_cta_limit(sms)
    ctx.set_k_per_load(k_per_load)
    ctx.set_split_tail(1)
    try:
        plan = plan_gemm(M, N, K, ctx=ctx)
        assert 0 < plan["split_k_tiles"] <= plan["slots"] // 2 and plan["narrow_tail_tiles"] == 0, plan
        assert 8 <= plan["split_k_at"] <= plan["k_blocks"] - 7
        A = synth.int8_uniform(6, (M, K))
        B = synth.int8_uniform(1006, (N, K))
        dA, dB = _dev(A), _dev(B)
        exp32 = O.gemm_i8_i32(A, B)
        sv = (np.arange(N) % 13 + 3).astype(np.uint8)
        exp8 = O.gemm_i8_srs(A, B, shift=9)
        exp8v = O.gemm_i8_srs(A, B, shift_vec=sv, acc_in=exp32)
        d32 = _dev(exp32)
        for rep in range(3):
            ctx.set_tma_store(rep)                  # 0: per-thread stores, 1: tile stores for int32, 2: for int8 too
            got = ctx.gemm_i8_i32(dA, dB)
            assert np.array_equal(got.cpu().numpy(), exp32)
            ctx.gemm_i8_i32(dA, dB, out=got, accumulate=True)
            assert np.array_equal(got.cpu().numpy(), 2 * exp32)
            assert np.array_equal(ctx.gemm_i8_srs(dA, dB, shift=9).cpu().numpy(), exp8)
            assert np.array_equal(ctx.gemm_i8_srs(dA, dB, shift_vec=_dev(sv), acc_in=d32).cpu().numpy(), exp8v)
        ctx.set_tma_store(1)
        ctx.set_split_tail(0)
        assert plan_gemm(M, N, K, ctx=ctx)["split_k_tiles"] == 0
        assert np.array_equal(ctx.gemm_i8_i32(dA, dB).cpu().numpy(), exp32)
        assert ctx.sync() == 0
    finally:
        ctx.set_tma_store(1)
        ctx.set_split_tail(3)
        ctx.set_k_per_load(0)
        ctx.set_cta_limit(0)
        ctx.set_tile_n(0)
        ctx.set_cta_pair(-1)


@pytest.mark.parametrize("k_per_load", [1, 2])
@pytest.mark.parametrize("shape", [(2304, 2304, 512), (2560, 2304, 384), (2500, 2400, 640), (2560, 2000, 272)])
def test_tail_tiles_cut_into_column_ranges(ctx, shape, k_per_load):
    """A thin last wave of 256-column pair tiles is cut into two 128-column ranges (narrower MMAs, a second
    tensor map for B): same bits as the oracle for int32 and srs results, same bits as the uncut schedule
    for bf16 (every element is still one accumulation over K in the same order)."""
    from aiehlc_b200.ops import plan_gemm
    M, N, K = shape
    ctx.set_cta_pair(1)
    ctx.set_tile_n(256)
    ctx.set_k_per_load(k_per_load)
    try:
        A = synth.int8_uniform(11, (M, K))
        B = synth.int8_uniform(1011, (N, K))
        dA, dB = _dev(A), _dev(B)
        Ab = _dev(synth.normal_bf16_bits(12, (M, K // 2)).view(np.int16)).view(torch.bfloat16)
        Bb = _dev(synth.normal_bf16_bits(1012, (N, K // 2)).view(np.int16)).view(torch.bfloat16)
        ctx.set_split_tail(0)
        whole = ctx.gemm_bf16(Ab, Bb)
        ctx.set_split_tail(2)
        assert plan_gemm(M, N, K, ctx=ctx)["narrow_tail_tiles"] > 0 and plan_gemm(M, N, K, ctx=ctx)["split_k_tiles"] == 0
        for _ in range(2):
            assert np.array_equal(ctx.gemm_i8_i32(dA, dB).cpu().numpy(), O.gemm_i8_i32(A, B))
            assert np.array_equal(ctx.gemm_i8_srs(dA, dB, shift=9).cpu().numpy(), O.gemm_i8_srs(A, B, shift=9))
        assert torch.equal(ctx.gemm_bf16(Ab, Bb), whole)
        assert ctx.sync() == 0
    finally:
        ctx.set_split_tail(3)
        ctx.set_k_per_load(0)
        ctx.set_tile_n(0)
        ctx.set_cta_pair(-1)


@pytest.mark.parametrize("tma_store", [0, 1, 2])
def test_both_store_paths(ctx, tma_store):
    """Results leave either through shared memory + TMA tile stores or through per-thread stores."""
    M, N, K = 520, 336, 272
    A = synth.int8_uniform(8, (M, K))
    B = synth.int8_uniform(1008, (N, K))
    ctx.set_tma_store(tma_store)
    try:
        dA, dB = _dev(A), _dev(B)
        acc = ctx.gemm_i8_i32(dA, dB)
        assert np.array_equal(acc.cpu().numpy(), O.gemm_i8_i32(A, B))
        ctx.gemm_i8_i32(dA, dB, out=acc, accumulate=True)                       # add-reduction form of the store
        assert np.array_equal(acc.cpu().numpy(), 2 * O.gemm_i8_i32(A, B))
        assert np.array_equal(ctx.gemm_i8_srs(dA, dB, shift=7).cpu().numpy(), O.gemm_i8_srs(A, B, shift=7))
        Ab = synth.normal_bf16_bits(3, (M, K))
        Bb = synth.normal_bf16_bits(1003, (N, K))
        got = ctx.gemm_bf16(_dev(Ab.view(np.int16)).view(torch.bfloat16), _dev(Bb.view(np.int16)).view(torch.bfloat16))
        ref = O.gemm_bf16(Ab, Bb).astype(np.float64)
        gf = got.float().cpu().numpy().astype(np.float64)
        assert float(np.max(np.abs(gf - ref) / np.maximum(np.abs(ref), 1.0))) <= 1e-2
        assert ctx.sync() == 0
    finally:
        ctx.set_tma_store(1)


@pytest.mark.parametrize("tma_store", [1, 2])
@pytest.mark.parametrize("groups", [1, 2])
@pytest.mark.parametrize("shape", [(512, 512, 512), (520, 336, 640), (300, 260, 192), (2304, 2304, 512), (2560, 2000, 272)])
def test_epilogue_warp_groups(ctx, shape, groups, tma_store):
    """CTA-pair kernel with one or two groups of epilogue warps (two: the warps of a TMEM lane quarter
    each drain half of a tile's columns, also of the 128-column ranges of a thin last wave), results
    leaving through tile stores or, for int8, per-thread stores: the oracle's bytes in every case."""
    M, N, K = shape
    A = synth.int8_uniform(13, (M, K))
    B = synth.int8_uniform(1013, (N, K))
    ctx.set_epilogue_groups(groups)
    ctx.set_tma_store(tma_store)
    ctx.set_cta_pair(1)
    try:
        dA, dB = _dev(A), _dev(B)
        exp32 = O.gemm_i8_i32(A, B)
        acc = ctx.gemm_i8_i32(dA, dB)
        assert np.array_equal(acc.cpu().numpy(), exp32)
        ctx.gemm_i8_i32(dA, dB, out=acc, accumulate=True)
        assert np.array_equal(acc.cpu().numpy(), exp32 * 2)
        assert np.array_equal(ctx.gemm_i8_srs(dA, dB, shift=8).cpu().numpy(), O.gemm_i8_srs(A, B, shift=8))
        Kb = K // 2
        Ab = synth.normal_bf16_bits(14, (M, Kb))
        Bb = synth.normal_bf16_bits(1014, (N, Kb))
        got = ctx.gemm_bf16(_dev(Ab.view(np.int16)).view(torch.bfloat16), _dev(Bb.view(np.int16)).view(torch.bfloat16))
        ref = O.gemm_bf16(Ab, Bb).astype(np.float64)
        gf = got.float().cpu().numpy().astype(np.float64)
        assert float(np.max(np.abs(gf - ref) / np.maximum(np.abs(ref), 1.0))) <= 1e-2      # the bf16 tolerance
        assert ctx.sync() == 0
    finally:
        ctx.set_epilogue_groups(0)
        ctx.set_tma_store(1)
        ctx.set_cta_pair(-1)


@pytest.mark.parametrize("k_per_load", [1, 2])
@pytest.mark.parametrize("shape", [(512, 512, 512), (520, 336, 640), (300, 520, 1152), (256, 256, 384), (1024, 384, 2176)])
def test_k_blocks_per_tile_load(ctx, shape, k_per_load):
    """CTA-pair kernel with one or two 128-byte K blocks per TMA tile load (odd and even block counts,
    split-K ranges that end inside a pair of blocks); both settings give the oracle's bytes."""
    M, N, K = shape
    A = synth.int8_uniform(9, (M, K))
    B = synth.int8_uniform(1009, (N, K))
    ctx.set_k_per_load(k_per_load)
    ctx.set_cta_pair(1)
    try:
        dA, dB = _dev(A), _dev(B)
        assert np.array_equal(ctx.gemm_i8_i32(dA, dB).cpu().numpy(), O.gemm_i8_i32(A, B))
        for splitk in (1, 2):
            assert np.array_equal(ctx.gemm_i8_srs(dA, dB, shift=8, splitk=splitk).cpu().numpy(),
                                  O.gemm_i8_srs(A, B, shift=8, splitk=splitk))
        Kb = K // 2                                                     # same K bytes per row as the int8 case
        Ab = synth.normal_bf16_bits(4, (M, Kb))
        Bb = synth.normal_bf16_bits(1004, (N, Kb))
        got = ctx.gemm_bf16(_dev(Ab.view(np.int16)).view(torch.bfloat16), _dev(Bb.view(np.int16)).view(torch.bfloat16))
        ref = O.gemm_bf16(Ab, Bb).astype(np.float64)
        gf = got.float().cpu().numpy().astype(np.float64)
        assert float(np.max(np.abs(gf - ref) / np.maximum(np.abs(ref), 1.0))) <= 1e-2      # the bf16 tolerance
        assert ctx.sync() == 0
    finally:
        ctx.set_k_per_load(0)
        ctx.set_cta_pair(-1)


@pytest.mark.parametrize("tile_stores", [0, 1])
@pytest.mark.parametrize("pair", [0, 1])
@pytest.mark.parametrize("M,N,K,rows_per_shard,group_m,first_shard",
                         [(1000, 520, 272, 256, 0, 0), (2304, 2304, 512, 1152, 0, 1), (640, 256, 1024, 128, 0, 3),
                          (300, 64, 96, 384, 0, 0),
                          (2048, 512, 256, 512, 2, 1), (4096, 256, 128, 512, 1, 5)])   # shard-interleaved tile order
def test_row_sharded_add_reduction_output(ctx, M, N, K, rows_per_shard, group_m, first_shard, pair, tile_stores):
    """GEMM whose epilogue adds into a row-sharded C (the fused split-K exchange; here every shard is
    local): zeroed shards receive the product, a second K slice adds to it, rows past M stay untouched;
    the visiting order (first_shard) never changes the result."""
    A = synth.int8_uniform(13, (M, K))
    B = synth.int8_uniform(1013, (N, K))
    n_shards = -(-M // rows_per_shard)
    shards = [torch.zeros((rows_per_shard, N), dtype=torch.int32, device=DEV) for _ in range(n_shards)]
    shards[-1] += 77                                                   # rows past M must keep this
    ctx.set_cta_pair(pair)
    ctx.set_group_m(group_m)
    ctx.set_shard_tile_stores(bool(tile_stores))
    try:
        half = K // 2 // 16 * 16
        dA, dB = _dev(A), _dev(B)
        exp = O.gemm_i8_i32(A, B)
        exp[(n_shards - 1) * rows_per_shard:] += 77
        for groups in ((1, 2) if pair else (0,)):                      # epilogue warp groups of the pair kernel
            ctx.set_epilogue_groups(groups)
            for sh in shards[:-1]:
                sh.zero_()
            shards[-1].fill_(77)
            ctx.gemm_i8_i32_scatter(dA[:, :half].contiguous(), dB[:, :half].contiguous(), shards, rows_per_shard, first_shard)
            ctx.gemm_i8_i32_scatter(dA[:, half:].contiguous(), dB[:, half:].contiguous(), shards, rows_per_shard, first_shard + 1)
            assert ctx.sync() == 0
            got = torch.cat(shards).cpu().numpy()
            assert np.array_equal(got[:M], exp)
            assert np.all(got[M:] == 77)
    finally:
        ctx.set_cta_pair(-1)
        ctx.set_group_m(0)
        ctx.set_shard_tile_stores(True)
        ctx.set_epilogue_groups(0)
    with pytest.raises(_capi.AiehlcError):
        ctx.gemm_i8_i32_scatter(dA, dB, shards, 100)                   # not a multiple of 128
    with pytest.raises(_capi.AiehlcError):
        ctx.gemm_i8_i32_scatter(dA, dB, shards[:1], 128)               # shards do not cover M


@pytest.mark.parametrize("shape", [(1024, 768, 512), (300, 520, 1152), (2304, 2304, 512)])
def test_sm_limit_changes_the_schedule_not_the_result(ctx, shape):
    """The Col x Row grid of the kernel-call form becomes a limit on the SMs a launch occupies: the planner
    sizes waves for that many CTAs; the bits stay the same."""
    from aiehlc_b200.ops import plan_gemm
    M, N, K = shape
    A, B = _dev(synth.int8_uniform(61, (M, K))), _dev(synth.int8_uniform(1061, (N, K)))
    want = ctx.gemm_i8_srs(A, B, shift=7)
    want32 = ctx.gemm_i8_i32(A, B)
    try:
        for sms in (1, 2, 16, 128, 1000):
            ctx.set_cta_limit(sms)
            plan = plan_gemm(M, N, K, ctx=ctx)
            assert plan["slots"] * (2 if plan["cta_pair"] else 1) <= min(sms, ctx.sm_count)
            assert torch.equal(ctx.gemm_i8_srs(A, B, shift=7), want)
            assert torch.equal(ctx.gemm_i8_i32(A, B), want32)
    finally:
        ctx.set_cta_limit(0)
    assert ctx.sync() == 0


@pytest.mark.parametrize("pair", [0, 1])
def test_operands_declared_ready_start_early_same_bits(ctx, pair):
    """With the caller's promise that operands are not written by the preceding kernel, loader and multiplier
    warps start while that kernel drains; the output stage still waits.  Back-to-back launches on rotating
    operands, a cascade whose partial sums come from the kernel just before, and operands the library re-pitches
    itself (where it must not start early): the same bits as without the promise."""
    ctx.set_cta_pair(pair)
    shapes = [(1024, 768, 1024), (2304, 2304, 512), (300, 520, 1152), (4096, 4096, 1024), (2560, 3072, 2048)]
    try:
        for (M, N, K) in shapes:
            sets = [(_dev(synth.int8_uniform(70 + i, (M, K))), _dev(synth.int8_uniform(1070 + i, (N, K)))) for i in range(4)]
            ctx.set_operands_ready(False)
            want = [(ctx.gemm_i8_i32(a, b), ctx.gemm_i8_srs(a, b, shift=7)) for a, b in sets]
            want_chain = ctx.gemm_i8_srs_cascade(sets[0][0], sets[0][1], stages=4, shift=9)
            ctx.set_operands_ready(True)
            for rep in range(5):
                got = []
                for a, b in sets:                      # launches queue up behind one another
                    got.append((ctx.gemm_i8_i32(a, b), ctx.gemm_i8_srs(a, b, shift=7)))
                for (g32, g8), (w32, w8) in zip(got, want):
                    assert torch.equal(g32, w32) and torch.equal(g8, w8)
                assert torch.equal(ctx.gemm_i8_srs_cascade(sets[0][0], sets[0][1], stages=4, shift=9), want_chain)
        # K = 1001: both operands are re-pitched by a kernel of the library right before the GEMM
        A, B = synth.int8_uniform(80, (384, 1001)), synth.int8_uniform(1080, (320, 1001))
        for rep in range(3):
            assert np.array_equal(ctx.gemm_i8_i32(_dev(A), _dev(B)).cpu().numpy(), O.gemm_i8_i32(A, B))
        rng = np.random.default_rng(5)
        inp = rng.integers(-2**31, 2**31 - 1, size=(512 + 384) * 1000, dtype=np.int64).astype(np.int32)
        assert np.array_equal(ctx.mm_i32(_dev(inp), 512, 384, 1000).cpu().numpy(), O.mm_i32(inp, 512, 384, 1000))
        assert ctx.sync() == 0
    finally:
        ctx.set_operands_ready(False)
        ctx.set_cta_pair(-1)


@pytest.mark.parametrize("pair", [0, 1])
def test_a_wait_that_runs_out_is_reported_and_the_context_survives(ctx, pair):
    """No GPU fault, no hang: the producer is told not to deliver (debug mode 3), the consumers' bounded
    waits run out after about a second, the kernel returns through its error exit, the host reads which
    wait gave up, and the next launch on the same context is correct again."""
    import ctypes as C
    import time
    M, N, K = 256, 256, 256
    A = synth.int8_uniform(14, (M, K))
    B = synth.int8_uniform(1014, (N, K))
    dA, dB = _dev(A), _dev(B)
    ctx.set_cta_pair(pair)
    try:
        ctx.set_debug(3)
        t0 = time.perf_counter()
        ctx.gemm_i8_i32(dA, dB)
        st = C.c_int32(0)
        rc = ctx._lib.aiehlc_sync(ctx._h, ctx._stream(), C.byref(st))
        waited = time.perf_counter() - t0
        assert rc == _capi.ERR_DEVICE and st.value in (101, 102, 104), (rc, st.value)   # which wait gave up first
        assert 0.3 < waited < 10.0, waited
        ctx.set_debug(0)
        assert ctx.sync() == 0                                                          # the word was cleared
        assert np.array_equal(ctx.gemm_i8_i32(dA, dB).cpu().numpy(), O.gemm_i8_i32(A, B))
        assert ctx.sync() == 0
    finally:
        ctx.set_debug(0)
        ctx.set_cta_pair(-1)


def test_accumulate_and_flush(ctx):
    M, N, K = 200, 136, 512
    A = synth.int8_uniform(2, (M, K))
    B = synth.int8_uniform(1002, (N, K))
    acc = ctx.gemm_i8_i32(_dev(A[:, :256].copy()), _dev(B[:, :256].copy()))
    ctx.gemm_i8_i32(_dev(A[:, 256:].copy()), _dev(B[:, 256:].copy()), out=acc, accumulate=True)
    assert np.array_equal(acc.cpu().numpy(), O.gemm_i8_i32(A, B))
    sv = ((np.arange(N) * 3) % 9).astype(np.uint8)
    assert np.array_equal(ctx.srs_i32_i8(acc, shift=5).cpu().numpy(), O.gemm_i8_srs(A, B, shift=5))
    assert np.array_equal(ctx.srs_i32_i8(acc, shift_vec=_dev(sv)).cpu().numpy(), O.gemm_i8_srs(A, B, shift_vec=sv))


# ---------------------------------------------------------------- full benchmark size
def test_cfg2_full_size_properties_and_sampled_rows(ctx):
    """int8 4096^3, srs shift 8, split-K 4: sampled rows bit-exact against the oracle, the whole
    matrix checked through size-independent properties."""
    M = N = K = 4096
    dA = synth.int8_uniform_torch(2, (M, K), DEV)
    dB = synth.int8_uniform_torch(1002, (N, K), DEV)
    c8 = ctx.gemm_i8_srs(dA, dB, shift=8, splitk=4)
    c32 = ctx.gemm_i8_i32(dA, dB)
    assert ctx.sync() == 0
    # (1) sampled rows, full width, against the oracle
    rows = np.r_[0:64, 2037:2101, 4032:4096]
    A_rows = synth.int8_uniform(2, (M, K))[rows]
    B = synth.int8_uniform(1002, (N, K))
    assert np.array_equal(c32[torch.from_numpy(rows).to(DEV)].cpu().numpy(), O.gemm_i8_i32(A_rows, B))
    assert np.array_equal(c8[torch.from_numpy(rows).to(DEV)].cpu().numpy(), O.gemm_i8_srs(A_rows, B, shift=8, splitk=4))
    # (2) the epilogue is consistent with the int32 result everywhere: srs(C32) == C8
    assert torch.equal(ctx.srs_i32_i8(c32, shift=8), c8)
    # (3) checksum of checksums: sum_j C[i][j] == A[i] . (sum_j B[j]) for every row i (exact in int64)
    colsum = dB.to(torch.float64).sum(dim=0)
    assert torch.equal(c32.to(torch.float64).sum(dim=1), dA.to(torch.float64) @ colsum)
    # (4) linearity in A: C(A with rows negated) == -C
    neg = ctx.gemm_i8_i32((-dA.clamp(min=-127)).contiguous(), dB)
    assert torch.equal(neg, -ctx.gemm_i8_i32(dA.clamp(min=-127).contiguous(), dB))
    # (5) cascade over 4 launches equals the single launch
    assert torch.equal(ctx.gemm_i8_srs_cascade(dA, dB, 4, shift=8), c8)


@pytest.mark.parametrize("shape", [(16384, 4096, 512), (8192, 8192, 1024)])
def test_shallow_k_large_outputs_sampled_rows_and_checksums(ctx, shape):
    """Large outputs over a shallow K (the output stage sets the pace; two groups of epilogue warps by
    default): sampled rows bit-exact against the oracle, every row through the checksum of checksums,
    srs consistent with the int32 result everywhere, one and two groups identical."""
    M, N, K = shape
    dA = synth.int8_uniform_torch(6, (M, K), DEV)
    dB = synth.int8_uniform_torch(1006, (N, K), DEV)
    c32 = ctx.gemm_i8_i32(dA, dB)
    c8 = ctx.gemm_i8_srs(dA, dB, shift=7)
    assert ctx.sync() == 0
    rows = np.r_[0:8, M // 2 - 4:M // 2 + 4, M - 8:M]
    B = synth.int8_uniform(1006, (N, K))
    A_rows = np.concatenate([synth.int8_uniform(6, (1, K), start=int(r) * K) for r in rows])
    sel = torch.from_numpy(rows).to(DEV)
    assert np.array_equal(c32[sel].cpu().numpy(), O.gemm_i8_i32(A_rows, B))
    assert np.array_equal(c8[sel].cpu().numpy(), O.gemm_i8_srs(A_rows, B, shift=7))
    colsum = dB.to(torch.float64).sum(dim=0)
    assert torch.equal(c32.to(torch.float64).sum(dim=1), dA.to(torch.float64) @ colsum)
    assert torch.equal(ctx.srs_i32_i8(c32, shift=7), c8)
    try:
        for groups in (1, 2):
            ctx.set_epilogue_groups(groups)
            assert torch.equal(ctx.gemm_i8_i32(dA, dB), c32), groups
            assert torch.equal(ctx.gemm_i8_srs(dA, dB, shift=7), c8), groups
        assert ctx.sync() == 0
    finally:
        ctx.set_epilogue_groups(0)


def test_cfg5_full_size_sampled_rows_and_checksums(ctx):
    """int8 65536 x 8192 x 8192 -> int32 (2.1 GB of results) at full size: sampled rows bit-exact against the
    oracle, every row through the checksum of checksums, and the row-sharded form (8 shards of 8192 rows,
    two K slices added into zeroed shards) equal to the single launch."""
    M, N, K = 65536, 8192, 8192
    dA = synth.int8_uniform_torch(5, (M, K), DEV)
    dB = synth.int8_uniform_torch(1005, (N, K), DEV)
    c32 = ctx.gemm_i8_i32(dA, dB)
    assert ctx.sync() == 0
    rows = np.r_[0:4, 8190:8194, 40000:40004, 65532:65536]            # across shard and tile boundaries
    B = synth.int8_uniform(1005, (N, K))
    A_rows = np.concatenate([synth.int8_uniform(5, (1, K), start=int(r) * K) for r in rows])
    assert np.array_equal(c32[torch.from_numpy(rows).to(DEV)].cpu().numpy(), O.gemm_i8_i32(A_rows, B))
    # sum_j C[i][j] == A[i] . (sum_j B[j]) for every row i: |values| < 2^53, exact in float64
    colsum = dB.to(torch.float64).sum(dim=0)
    want = torch.empty(M, dtype=torch.float64, device=DEV)
    for r0 in range(0, M, 8192):                                       # row blocks keep the temporaries small
        want[r0:r0 + 8192] = dA[r0:r0 + 8192].to(torch.float64) @ colsum
    got = torch.empty(M, dtype=torch.float64, device=DEV)
    for r0 in range(0, M, 8192):
        got[r0:r0 + 8192] = c32[r0:r0 + 8192].to(torch.float64).sum(dim=1)
    assert torch.equal(got, want)
    # the split-K exchange's form: two K slices added into 8 zeroed row shards
    shards = [torch.zeros((8192, N), dtype=torch.int32, device=DEV) for _ in range(8)]
    half = K // 2
    ctx.gemm_i8_i32_scatter(dA[:, :half].contiguous(), dB[:, :half].contiguous(), shards, 8192, first_shard=1)
    ctx.gemm_i8_i32_scatter(dA[:, half:].contiguous(), dB[:, half:].contiguous(), shards, 8192, first_shard=6)
    assert ctx.sync() == 0
    for g in range(8):
        assert torch.equal(shards[g], c32[g * 8192:(g + 1) * 8192]), g
