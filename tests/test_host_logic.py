"""Host-side logic that needs no GPU: seeded inputs, sharding, and the 2-rank split-K exchange on gloo."""
import os
import socket
import subprocess
import sys
import textwrap
from pathlib import Path

import numpy as np
import pytest

from aiehlc_b200 import shard, synth

ROOT = Path(__file__).resolve().parents[1]


def test_synth_is_counter_based_and_matches_its_torch_twin():
    a = synth.int8_uniform(5, (8, 32))
    assert np.array_equal(a[3:5], synth.int8_uniform(5, (2, 32), start=3 * 32))   # any shard on its own
    t = synth.int8_uniform_torch(5, (8, 32), "cpu")
    assert np.array_equal(t.numpy(), a)
    big = synth.int8_uniform(7, (256, 1024))
    assert big.min() == -128 and big.max() == 127 and abs(float(big.mean())) < 1.0
    x = synth.normal_f32(3, (512, 512))
    assert abs(float(x.mean())) < 0.01 and abs(float(x.std()) - 1.0) < 0.01


def test_bf16_rounding_is_nearest_even():
    import torch
    x = synth.normal_f32(9, (4096,))
    assert np.array_equal(synth.f32_to_bf16_bits(x), torch.from_numpy(x).bfloat16().view(torch.int16).numpy().view(np.uint16))
    assert np.array_equal(synth.bf16_bits_to_f32(synth.f32_to_bf16_bits(x)), torch.from_numpy(x).bfloat16().float().numpy())


@pytest.mark.parametrize("m,world", [(65536, 8), (65536, 1), (4096, 2), (10, 4), (3, 4), (0, 2)])
def test_row_shards_cover_m_exactly(m, world):
    spans = [shard.row_shard(m, world, r) for r in range(world)]
    assert spans[0][0] == 0 and sum(n for _, n in spans) == m
    for (f0, n0), (f1, _) in zip(spans, spans[1:]):
        assert f0 + n0 == f1
    assert max(n for _, n in spans) - min(n for _, n in spans) <= 1


def test_k_slices():
    assert [list(shard.k_slices(8, 2, r)) for r in range(2)] == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert shard.k_range(8192, 8, 8, 3) == (3072, 1024)
    assert shard.k_range(8192, 8, 2, 1) == (4096, 4096)
    with pytest.raises(ValueError):
        shard.k_slices(8, 3, 0)
    with pytest.raises(ValueError):
        shard.row_shard(8, 2, 2)


def test_gemm_planner_needs_no_gpu():
    """The tiling plan (counterpart of the compiler's creatematmul + broadcast analysis) is host logic."""
    from aiehlc_b200.ops import plan_gemm
    p = plan_gemm(4096, 4096, 4096)                     # the benchmark GEMM: 256 pair tiles on 74 CTA pairs
    assert (p["tile_m"], p["tile_n"], p["cta_pair"]) == (256, 256, 1)
    assert (p["grid_m"], p["grid_n"], p["tiles"], p["slots"], p["waves"]) == (16, 16, 256, 74, 4)
    assert abs(p["wave_efficiency"] - 256 / 296) < 1e-9
    assert p["k_blocks"] == 32 and p["tmem_columns"] == 512 and p["smem_bytes"] <= 227 * 1024
    # two 128-byte K blocks per tile load: three 64 KiB stages hold what six 32 KiB stages did
    assert p["tile_k_bytes"] == 256 and p["stages"] == 3
    assert (p["a_shared_by"], p["b_shared_by"]) == (16, 16)   # A rows serve a grid row, B rows a grid column
    # 3 full waves + 34 tiles: by default the 34 tail tiles run as 68 column ranges (measured faster than K halves)
    assert p["split_k_tiles"] == 0 and p["narrow_tail_tiles"] == 34
    p = plan_gemm(64, 64, 64)                           # one tile: a single CTA, the narrowest tile
    assert (p["tile_m"], p["tile_n"], p["cta_pair"], p["tiles"], p["waves"]) == (128, 64, 0, 1, 1)
    p = plan_gemm(8192, 8192, 8192, kind="bf16")
    assert p["k_blocks"] == 128 and p["tiles"] == 1024 and p["waves"] == 14
    from aiehlc_b200 import _capi
    with pytest.raises(_capi.AiehlcError):
        plan_gemm(0, 4, 4)


def test_k_halves_schedule_gives_every_pair_at_most_half_a_tile_more():
    """Host logic of the tail balancing along K (the unit order the kernels walk, restated): upper halves, one
    whole tile per pair, lower halves, the other whole tiles, dealt round-robin -- every tile's K range is covered
    exactly once, a lower half is the SECOND unit of its pair (its upper half, the first unit of another pair, is
    done by then), and no pair has more than full + 1/2 tile times of work."""
    # (tiles, pairs, K blocks) of a few launches; the cut is the planner's: an even number of blocks in the lower half
    for (T, P, nkb) in [(256, 74, 32), (100, 74, 32), (99, 74, 17), (256, 74, 16), (320, 74, 32), (20, 16, 16), (42, 12, 64)]:
        rem, cut = T % P, (nkb // 2 + 1) & ~1
        assert 0 < rem <= P // 2
        first = T - rem
        units = [(first + u, cut, nkb) for u in range(rem)] + [(t, 0, nkb) for t in range(P)] + \
                [(first + u, 0, cut) for u in range(rem)] + [(t, 0, nkb) for t in range(P, first)]
        cover = {}
        for t, a, b in units:
            cover.setdefault(t, []).append((a, b))
        assert all(sorted(v) in ([(0, nkb)], [(0, cut), (cut, nkb)]) for v in cover.values()) and len(cover) == T
        for pair in range(P):
            mine = units[pair::P]
            work = sum(b - a for _, a, b in mine)
            assert work <= (T // P) * nkb + max(cut, nkb - cut)
            halves = [(i, a) for i, (t, a, b) in enumerate(mine) if b - a < nkb]
            assert halves in ([], [(0, cut)], [(1, 0)])     # an upper half first, or a lower half second
        # the upper half of a tile is in the first round, its lower half in the second, on another pair
        where = {(t, a): i for i, (t, a, b) in enumerate(units) if b - a < nkb}
        for u in range(rem):
            up, lo = where[(first + u, cut)], where[(first + u, 0)]
            assert up < P <= lo < 2 * P and up % P != lo % P


def test_tile_visiting_order_needs_no_gpu():
    """The order the kernels walk the tile grid in (the function they call, run on the host): every tile
    exactly once; plain launches walk groups of 8 row-blocks column by column; launches with a row-sharded
    output put consecutive tiles on consecutive shards and use a slot count coprime with the shard count,
    so each persistent CTA pair cycles through all owners."""
    import numpy as np
    from aiehlc_b200.ops import plan_gemm, plan_tile_order
    M, N, K = 4096, 4096, 4096
    p = plan_gemm(M, N, K)
    rb, cb, slots = plan_tile_order(M, N, K)
    assert slots == 74 and len(rb) == p["tiles"] == 256
    assert len({(int(a), int(b)) for a, b in zip(rb, cb)}) == 256                 # a bijection onto the grid
    assert list(rb[:8]) == list(range(8)) and set(cb[:8]) == {0}                  # group of 8 row-blocks, column 0
    assert list(rb[8:16]) == list(range(8)) and set(cb[8:16]) == {1}
    # ragged grid: the last group has fewer row-blocks
    rb, cb, _ = plan_tile_order(2560 + 100, 1000, 512)
    grid = plan_gemm(2560 + 100, 1000, 512)
    assert len({(int(a), int(b)) for a, b in zip(rb, cb)}) == grid["tiles"] == grid["grid_m"] * grid["grid_n"]
    assert rb.max() == grid["grid_m"] - 1 and cb.max() == grid["grid_n"] - 1
    # split-K exchange over 8 owners: 65536 rows, 8192 per shard = 32 row-blocks of 256 rows each
    M, N, K, shards, rps = 65536, 8192, 1024, 8, 8192
    for first in (1, 5):
        rb, cb, slots = plan_tile_order(M, N, K, num_shards=shards, rows_per_shard=rps, first_shard=first)
        assert len(rb) == 256 * 32 and len({(int(a), int(b)) for a, b in zip(rb, cb)}) == len(rb)
        owner = rb // (rps // 256)
        assert list(owner[:16]) == [(first + t) % shards for t in range(16)]      # consecutive tiles, consecutive owners
        assert slots == 73 and np.gcd(slots, shards) == 1
        for s in (0, 36, 72):                                                     # every slot meets every owner in 8 rounds
            assert set(owner[s::slots][:shards]) == set(range(shards))
    # shards that do not hold whole groups of row-blocks: rows in plain order, still every tile once
    rb, cb, slots = plan_tile_order(1000, 520, 272, num_shards=4, rows_per_shard=256)
    assert len({(int(a), int(b)) for a, b in zip(rb, cb)}) == len(rb)
    from aiehlc_b200 import _capi
    with pytest.raises(_capi.AiehlcError):
        plan_tile_order(1000, 520, 272, num_shards=4, rows_per_shard=100)


def test_int32_product_as_byte_limb_products():
    """The arithmetic behind the tensor-core form of the reference's int32 kernel, in numpy: with unsigned
    bytes a_t, b_u of the operands, sum_k a*b mod 2^32 == sum_s 2^(8s) * sum_k sum_(t<=s) a_t * b_(s-t)  mod 2^32,
    and up to K = 8256 no group sum reaches 2^31 (so the int32 accumulator never overflows)."""
    import numpy as np
    from oracle import oracle as O
    rng = np.random.default_rng(5)
    M, N, K = 7, 5, 300
    inp = rng.integers(-2**31, 2**31 - 1, size=(M + N) * K, dtype=np.int64).astype(np.int32)
    A = inp[:M * K].reshape(M, K).view(np.uint32).astype(np.uint64)
    B = inp[M * K:].reshape(N, K).view(np.uint32).astype(np.uint64)
    limb = lambda x, t: (x >> np.uint64(8 * t)) & np.uint64(0xFF)
    total = np.zeros((M, N), dtype=np.uint64)
    for s in range(4):
        group = sum(limb(A, t) @ limb(B, s - t).T for t in range(s + 1))          # one int8 GEMM of depth (s+1) K
        assert int(group.max()) < 2**31
        total += (group << np.uint64(8 * s)) & np.uint64(0xFFFFFFFF)
    got = (total & np.uint64(0xFFFFFFFF)).astype(np.uint32).view(np.int32)
    assert np.array_equal(got, O.mm_i32(inp, M, N, K))
    assert 4 * 8256 * 255 * 255 < 2**31 <= 4 * 8257 * 255 * 255                   # the K limit of one range


def test_conv_planner_needs_no_gpu():
    """Which form a convolution takes and how it is tiled is host logic."""
    from aiehlc_b200.ops import plan_conv2d
    p = plan_conv2d(1, 56, 56, 64, 64)                       # the benchmark convolution
    assert p["form"] == 1 and (p["tile_rows"], p["tile_width"]) == (1, 56)
    assert (p["patch_rows"], p["patch_width"], p["m_rows_used"]) == (3, 58, 58)
    assert (p["cout_tile"], p["cin_chunk"], p["ctas"]) == (32, 64, 112)
    assert (p["tma_boxes_per_cta"], p["mmas_per_cta"]) == (2, 18) and p["smem_bytes"] <= 227 * 1024
    assert p["launches"] == 1                                # HWIO weights feed the tensor cores as they are
    p = plan_conv2d(8, 56, 56, 64, 64)                       # enough tiles: two image rows per CTA, all channels
    assert p["form"] == 1 and p["tile_rows"] == 2 and p["m_rows_used"] == 116 and p["cout_tile"] == 64
    p = plan_conv2d(1, 6, 300, 128, 32, 5, 5, 2)             # wider than a tile: pieces of 128 - (kw - 1) pixels
    assert p["form"] == 1 and p["tile_width"] == 124 and p["patch_width"] == 128 and p["patch_rows"] == 5
    p = plan_conv2d(1, 8, 8, 256, 32, 1, 1, 0)               # 1 x 1: nothing to share between taps
    assert p["form"] == 0 and p["tma_boxes_per_cta"] == 4 and p["mmas_per_cta"] == 8 and p["launches"] == 2
    p = plan_conv2d(4, 28, 28, 512, 512)                     # every tap's weights of a channel tile must fit
    assert p["form"] == 1 and 9 * p["cout_tile"] * p["cin_chunk"] <= 96 * 1024 and p["tma_boxes_per_cta"] == 8
    assert plan_conv2d(1, 8, 8, 24, 16)["form"] == 2         # 24 input channels: the CUDA-core kernel
    from aiehlc_b200 import _capi
    with pytest.raises(_capi.AiehlcError):
        plan_conv2d(1, 8, 8, 64, 64, 3, 3, 0)                # not a same-size filter


_WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np, torch, torch.distributed as dist
    sys.path.insert(0, os.environ["AIEHLC_ROOT"])
    from aiehlc_b200 import shard, synth
    from oracle import oracle as O
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    M, N, K, splitk = 64, 48, 256, 8
    A = synth.int8_uniform(5, (M, K)); B = synth.int8_uniform(1005, (N, K))
    full = O.gemm_i8_i32(A, B)
    # row-sharded: every rank computes its rows only, no exchange; the gather is for the check
    r0, nr = shard.row_shard(M, world, rank)
    mine = torch.from_numpy(O.gemm_i8_i32(A[r0:r0 + nr], B))
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine)
    assert np.array_equal(torch.cat(parts).numpy(), full)
    # split-K: rank-local partial over its K slices, then one reduce-scatter of int32 partials
    k0, nk = shard.k_range(K, splitk, world, rank)
    partial = torch.from_numpy(O.gemm_i8_i32(A[:, k0:k0 + nk], B[:, k0:k0 + nk]))
    # gloo has no reduce_scatter: all_reduce, then keep the own row block (same sums, same owner)
    dist.all_reduce(partial, op=dist.ReduceOp.SUM)
    out = partial[rank * (M // world):(rank + 1) * (M // world)]
    assert np.array_equal(out.numpy(), full[rank * (M // world):(rank + 1) * (M // world)])
    dist.barrier()
    dist.destroy_process_group()
    print("rank", rank, "ok")
""")


def test_two_rank_sharding_on_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, AIEHLC_ROOT=str(ROOT), OMP_NUM_THREADS="2")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)],
                         capture_output=True, text=True, env=env, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.count("ok") == 2


def test_reference_arm_prints_one_json_line():
    import json
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "2", "--warmup", "1"],
                         capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "TOPS" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["e2e"]["h2d_bytes_per_step"] == 0
