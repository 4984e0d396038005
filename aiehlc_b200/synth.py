"""Seeded synthetic inputs for the benchmark configurations.

A counter-based generator (splitmix64 of seed and element index) so that any shard of a large
operand can be produced independently, on the host (numpy) or on the device (torch), with the
same values.  Distributions follow the benchmark configurations: int8 uniform in [-128, 127];
N(0, 1) rounded to bf16.
"""
from __future__ import annotations

import numpy as np

_GOLDEN = 0x9E3779B97F4A7C15
_M1 = 0xBF58476D1CE4E5B9
_M2 = 0x94D049BB133111EB
_MASK = (1 << 64) - 1


def splitmix64_np(seed: int, start: int, count: int) -> np.ndarray:
    """uint64 stream element i = mix(seed + (start + i + 1) * golden)."""
    with np.errstate(over="ignore"):
        idx = np.arange(start + 1, start + 1 + count, dtype=np.uint64)
        z = np.uint64(seed & _MASK) + idx * np.uint64(_GOLDEN)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(_M1)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(_M2)
        z = z ^ (z >> np.uint64(31))
    return z


def int8_uniform(seed: int, shape, start: int = 0) -> np.ndarray:
    """int8 uniform over [-128, 127]: the low byte of the stream, reinterpreted."""
    n = int(np.prod(shape))
    z = splitmix64_np(seed, start, n)
    return (z & np.uint64(0xFF)).astype(np.uint8).view(np.int8).reshape(shape)


def normal_f32(seed: int, shape, start: int = 0) -> np.ndarray:
    """N(0,1) by Box-Muller on two 24-bit uniforms cut from one 64-bit word."""
    n = int(np.prod(shape))
    z = splitmix64_np(seed, start, n)
    u1 = ((z >> np.uint64(40)).astype(np.float64) + 1.0) / 16777216.0
    u2 = ((z >> np.uint64(16)) & np.uint64(0xFFFFFF)).astype(np.float64) / 16777216.0
    x = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return x.astype(np.float32).reshape(shape)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = u + np.uint64(0x7FFF) + ((u >> np.uint64(16)) & np.uint64(1))
    return (u >> np.uint64(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def normal_bf16_bits(seed: int, shape, start: int = 0) -> np.ndarray:
    return f32_to_bf16_bits(normal_f32(seed, shape, start))


# ------------------------------------------------------------------ device-side twins (torch)
def _splitmix64_torch(seed: int, start: int, count: int, device):
    import torch

    def s64(v: int) -> int:  # two's-complement view of a uint64 constant
        v &= _MASK
        return v - (1 << 64) if v >= (1 << 63) else v

    def lsr(x, s: int):  # logical shift right on int64 storage
        return (x >> s) & ((1 << (64 - s)) - 1)

    idx = torch.arange(start + 1, start + 1 + count, dtype=torch.int64, device=device)
    z = idx * s64(_GOLDEN) + s64(seed)
    z = (z ^ lsr(z, 30)) * s64(_M1)
    z = (z ^ lsr(z, 27)) * s64(_M2)
    z = z ^ lsr(z, 31)
    return z


def int8_uniform_torch(seed: int, shape, device, start: int = 0, chunk: int = 1 << 26):
    """Same values as int8_uniform(), produced on `device` in chunks (bounded scratch)."""
    import torch
    n = 1
    for s in shape:
        n *= int(s)
    out = torch.empty(n, dtype=torch.int8, device=device)
    for off in range(0, n, chunk):
        c = min(chunk, n - off)
        z = _splitmix64_torch(seed, start + off, c, device)
        out[off:off + c] = (z & 0xFF).to(torch.uint8).view(torch.int8)
    return out.view(*shape)


def normal_bf16_torch(seed: int, shape, device, start: int = 0, chunk: int = 1 << 25):
    """N(0,1) -> bf16 on `device` (same stream as normal_f32; transcendental rounding may differ
    from numpy by an ulp, so copy rather than regenerate when bit equality across sides matters)."""
    import math

    import torch
    n = 1
    for s in shape:
        n *= int(s)
    out = torch.empty(n, dtype=torch.bfloat16, device=device)
    for off in range(0, n, chunk):
        c = min(chunk, n - off)
        z = _splitmix64_torch(seed, start + off, c, device)
        u1 = (((z >> 40) & 0xFFFFFF).to(torch.float64) + 1.0) / 16777216.0
        u2 = ((z >> 16) & 0xFFFFFF).to(torch.float64) / 16777216.0
        x = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(2.0 * math.pi * u2)
        out[off:off + c] = x.to(torch.float32).to(torch.bfloat16)
    return out.view(*shape)
