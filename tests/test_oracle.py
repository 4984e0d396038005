"""The CPU oracle against the reference's own fixtures and outputs (no GPU)."""
import numpy as np
import pytest

from aiehlc_b200 import synth
from oracle import oracle as O


def test_perf_fixture_matches_reference_program(golden):
    # in[i] = i + 1, 512 words (example/perf/aieml_perf.cc:141-144); the JSON holds what the
    # reference's own `perf` kernel produced, and its own golden loop agreed with it.
    g = golden["aieml_perf"]
    assert g["self_check_passed"]
    ref = np.array(g["words_read_back"], dtype=np.int32)
    assert ref.size == 512
    got = O.mm_i32(np.arange(1, 513, dtype=np.int32), 16, 16, 16)
    assert np.array_equal(got.ravel(), ref[:256])
    assert not ref[256:].any()  # the kernel writes 256 words of the 512-word window


def test_known_answers_of_reference_fixtures():
    c = O.mm_i32(np.arange(1, 513, dtype=np.int32), 16, 16, 16)            # aieml_perf.cc:141-144
    assert (c[0, 0], c[0, 15], c[15, 0], c[15, 15], int(c.sum(dtype=np.int64))) == (36312, 68952, 1051992, 2006232, 202463232)
    c = O.mm_i32(np.arange(0, 512, dtype=np.int32), 16, 16, 16)            # aieml_mm.cc:137-140
    assert (c[0, 0], c[0, 15], c[15, 0], c[15, 15], int(c.sum(dtype=np.int64))) == (31960, 60760, 1043800, 1994200, 200366080)
    c = O.mm_i32(np.arange(0, 128, dtype=np.int32), 8, 8, 8)               # example/other/aieoob.c:83-86
    a = np.arange(64).reshape(8, 8)
    b = np.arange(64, 128).reshape(8, 8)
    assert np.array_equal(c, a @ b.T)


def test_chain_constants_of_reference_programs(golden):
    assert golden["multi_tile"]["words_read_back"] == [26] * 20           # 15 + 1 + 10, multi_tile.cpp:148-158
    assert golden["seq_full_col"]["words_read_back"] == [23] * 20         # 15 + 8 tiles, seq_full_col.cpp:161-171
    assert golden["multi_kernel"]["words_read_back"] == [100 + i for i in range(20)] + [200 + i for i in range(20)]
    assert golden["tutorial_example"]["words_read_back"] == [100 + i for i in range(20)]
    assert all(p["self_check_passed"] for p in golden.values())


def test_mm_i32_wraps_like_uint32():
    rng = np.random.default_rng(1)
    inp = rng.integers(-2**31, 2**31 - 1, size=(40 + 24) * 9, dtype=np.int64).astype(np.int32)
    got = O.mm_i32(inp, 40, 24, 9)
    a = inp[:40 * 9].reshape(40, 9).astype(np.uint32)
    b = inp[40 * 9:].reshape(24, 9).astype(np.uint32)
    exp = np.zeros((40, 24), np.uint32)
    for k in range(9):
        exp += a[:, k:k + 1] * b[:, k][None, :]
    assert np.array_equal(got.view(np.uint32), exp)


@pytest.mark.parametrize("shape", [(64, 64, 64), (17, 5, 33), (1, 1, 1), (130, 70, 48)])
def test_gemm_i8_is_the_golden_loop_on_widened_operands(shape):
    M, N, K = shape
    A = synth.int8_uniform(1, (M, K))
    B = synth.int8_uniform(1001, (N, K))
    packed = np.concatenate([A.astype(np.int32).ravel(), B.astype(np.int32).ravel()])
    assert np.array_equal(O.gemm_i8_i32(A, B), O.mm_i32(packed, M, N, K))
    assert np.array_equal(O.gemm_i8_i32(A, B), A.astype(np.int64) @ B.astype(np.int64).T)


def _srs_py(x: int, s: int) -> int:
    """Independent statement with exact rationals: round half to even of x / 2^s, then saturate."""
    from fractions import Fraction
    q = Fraction(x, 1 << s)
    fl = q.numerator // q.denominator
    rem = q - fl
    if rem > Fraction(1, 2) or (rem == Fraction(1, 2) and fl % 2 == 1):
        fl += 1
    return max(-128, min(127, fl))


def test_srs_definition():
    for s in (0, 1, 2, 6, 8, 12, 31):
        for x in list(range(-600, 600)) + [2**31 - 1, -2**31, 127 << 8, (127 << 8) + 128, (-128 << 8) - 129,
                                           32767, 32768, 32769, -32768, -32896, 384, 640, -384, -640]:
            assert O.srs_i8(x, s) == _srs_py(x, s), (x, s)
    assert [O.srs_i8(v, 1) for v in (1, 3, 5, -1, -3)] == [0, 2, 2, 0, -2]   # ties go to the even neighbour
    assert O.srs_i8(10**9, 8) == 127 and O.srs_i8(-10**9, 8) == -128


def test_split_k_equals_unsplit_and_acc_in():
    A = synth.int8_uniform(2, (48, 256))
    B = synth.int8_uniform(1002, (40, 256))
    base = O.gemm_i8_srs(A, B, shift=8)
    for sk in (2, 4, 8):
        assert np.array_equal(O.gemm_i8_srs(A, B, shift=8, splitk=sk), base)
    part = O.gemm_i8_i32(A[:, :192], B[:, :192])
    assert np.array_equal(O.gemm_i8_srs(A[:, 192:], B[:, 192:], shift=8, acc_in=part), base)
    acc = O.gemm_i8_i32(A, B)
    assert np.array_equal(O.srs_i32_i8(acc, shift=8), base)
    sv = (np.arange(40) % 11).astype(np.uint8)
    assert np.array_equal(O.gemm_i8_srs(A, B, shift_vec=sv), O.srs_i32_i8(acc, shift_vec=sv))


def test_conv2d_against_im2col():
    x = synth.int8_uniform(4, (2, 7, 9, 8))
    w = synth.int8_uniform(1004, (3, 3, 8, 16))
    sv = np.full(16, 6, np.uint8)
    y = O.conv2d_i8_srs(x, w, sv, pad=1)
    xp = np.pad(x.astype(np.int64), ((0, 0), (1, 1), (1, 1), (0, 0)))
    cols = np.stack([xp[:, kh:kh + 7, kw:kw + 9, :] for kh in range(3) for kw in range(3)], axis=3)  # n,h,w,9,ci
    acc = cols.reshape(2 * 7 * 9, 72) @ w.astype(np.int64).reshape(72, 16)
    exp = O.srs_i32_i8(acc.astype(np.int32), shift_vec=sv).reshape(2, 7, 9, 16)
    assert np.array_equal(y, exp)


def test_bf16_reference_values():
    A = synth.normal_bf16_bits(3, (24, 200))
    B = synth.normal_bf16_bits(1003, (16, 200))
    c32, cb = O.gemm_bf16(A, B, want_bf16=True)
    exact = synth.bf16_bits_to_f32(A).astype(np.float64) @ synth.bf16_bits_to_f32(B).astype(np.float64).T
    assert np.max(np.abs(c32 - exact) / np.maximum(np.abs(exact), 1.0)) < 1e-4
    assert np.array_equal(cb, synth.f32_to_bf16_bits(c32))
