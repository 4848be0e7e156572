"""Seeded synthetic inputs for the benchmark configurations.

Every generator is counter based - element i depends only on (seed, i) - so a shard can
produce its slice [start, start + n) on its own and the CPU checker sees the same bits.
Host arrays are numpy; callers copy them to the device.
"""
from __future__ import annotations

import numpy as np

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)


def _mix(idx: np.ndarray, seed: int) -> np.ndarray:
    """splitmix64 finaliser over (seed, index); works in place on a uint64 index array."""
    x = idx
    tmp = np.empty_like(x)
    with np.errstate(over="ignore"):
        x += np.uint64(1)
        x *= _GOLDEN
        x += np.uint64((seed * 0xD1B54A32D192ED03) & 0xFFFFFFFFFFFFFFFF)
        np.right_shift(x, np.uint64(30), out=tmp); x ^= tmp
        x *= np.uint64(0xBF58476D1CE4E5B9)
        np.right_shift(x, np.uint64(27), out=tmp); x ^= tmp
        x *= np.uint64(0x94D049BB133111EB)
        np.right_shift(x, np.uint64(31), out=tmp); x ^= tmp
    return x


def _fill(out: np.ndarray, start: int, fn, chunk: int = 1 << 18) -> np.ndarray:
    """Evaluates fn(index array) chunk by chunk (small chunks stay in cache)."""
    pos, n = 0, out.size
    while pos < n:
        c = min(chunk, n - pos)
        out[pos:pos + c] = fn(np.arange(start + pos, start + pos + c, dtype=np.uint64))
        pos += c
    return out


def uniform_int32(n: int, seed: int, lo: int = 0, hi: int = 16, start: int = 0) -> np.ndarray:
    """i.i.d. uniform integers in [lo, hi)."""
    span = np.uint64(hi - lo)
    return _fill(np.empty(n, np.int32), start, lambda i: ((_mix(i, seed) >> np.uint64(11)) % span).astype(np.int32) + lo)


def uniform_uint32(n: int, seed: int, start: int = 0) -> np.ndarray:
    """i.i.d. uniform over the full 32-bit range."""
    return _fill(np.empty(n, np.uint32), start, lambda i: (_mix(i, seed) >> np.uint64(32)).astype(np.uint32))


def uniform_float32(n: int, seed: int, start: int = 0) -> np.ndarray:
    """i.i.d. uniform in [0, 1) with 24 random mantissa bits."""
    return _fill(np.empty(n, np.float32), start,
                 lambda i: ((_mix(i, seed) >> np.uint64(40)).astype(np.float32) * np.float32(2.0 ** -24)))


def normal_float32(n: int, seed: int, start: int = 0) -> np.ndarray:
    """i.i.d. N(0, 1) by Box-Muller on two counter-based uniforms."""
    def gen(i):
        u1 = ((_mix(i.copy(), seed) >> np.uint64(11)).astype(np.float64) + 0.5) * 2.0 ** -53
        u2 = ((_mix(i.copy(), seed ^ 0x5DEECE66D) >> np.uint64(11)).astype(np.float64)) * 2.0 ** -53
        return (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)).astype(np.float32)
    return _fill(np.empty(n, np.float32), start, gen)


def zipf_uint64(n: int, seed: int, s: float = 1.1, support: int = 1 << 32, start: int = 0) -> np.ndarray:
    """Zipf(s)-distributed ranks over {0 .. support-1} (inverse CDF of the continuous
    power law, floored), passed through a 32-bit bijection so that the frequent keys are
    not neighbours; zero-extended to 64 bits (the upper four key bytes are constant)."""
    a = 1.0 - s

    def gen(i):
        u = ((_mix(i, seed) >> np.uint64(11)).astype(np.float64) + 0.5) * 2.0 ** -53
        rank = np.floor(((float(support) ** a - 1.0) * u + 1.0) ** (1.0 / a)) - 1.0
        r = np.clip(rank, 0, support - 1).astype(np.uint64)
        with np.errstate(over="ignore"):
            r = (r * np.uint64(0x9E3779B1)) & np.uint64(support - 1)   # odd multiplier: a bijection mod 2^k
            r ^= r >> np.uint64(15)
        return r
    return _fill(np.empty(n, np.uint64), start, gen)


# ---- the same generators evaluated on the device (torch int64 arithmetic wraps like uint64) ----
def _signed(v: int) -> int:
    v &= 0xFFFFFFFFFFFFFFFF
    return v - (1 << 64) if v >= (1 << 63) else v


def _lsr(x, k: int):
    return (x >> k) & ((1 << (64 - k)) - 1)


def _mix_torch(idx, seed: int):
    x = (idx + 1) * _signed(0x9E3779B97F4A7C15) + _signed(seed * 0xD1B54A32D192ED03)
    x = x ^ _lsr(x, 30)
    x = x * _signed(0xBF58476D1CE4E5B9)
    x = x ^ _lsr(x, 27)
    x = x * _signed(0x94D049BB133111EB)
    x = x ^ _lsr(x, 31)
    return x


def _fill_torch(n: int, start: int, device, dtype, fn, chunk: int = 1 << 24):
    import torch
    out = torch.empty(n, dtype=dtype, device=device)
    pos = 0
    while pos < n:
        c = min(chunk, n - pos)
        idx = torch.arange(start + pos, start + pos + c, dtype=torch.int64, device=device)
        out[pos:pos + c] = fn(idx)
        pos += c
    return out


def uniform_uint32_device(n: int, seed: int, device, start: int = 0):
    """Bit-identical to uniform_uint32, produced on `device`."""
    import torch
    return _fill_torch(n, start, device, torch.int32,
                       lambda i: _lsr(_mix_torch(i, seed), 32).to(torch.int32)).view(torch.uint32)


def uniform_int32_device(n: int, seed: int, device, lo: int = 0, hi: int = 16, start: int = 0):
    """Bit-identical to uniform_int32."""
    import torch
    return _fill_torch(n, start, device, torch.int32,
                       lambda i: (_lsr(_mix_torch(i, seed), 11) % (hi - lo)).to(torch.int32) + lo)


def uniform_float32_device(n: int, seed: int, device, start: int = 0):
    """Bit-identical to uniform_float32."""
    import torch
    return _fill_torch(n, start, device, torch.float32,
                       lambda i: _lsr(_mix_torch(i, seed), 40).to(torch.float32) * (2.0 ** -24))


def normal_float32_device(n: int, seed: int, device, start: int = 0):
    """Same construction as normal_float32; device libm may differ in the last bit."""
    import math
    import torch

    def gen(i):
        u1 = (_lsr(_mix_torch(i, seed), 11).to(torch.float64) + 0.5) * 2.0 ** -53
        u2 = _lsr(_mix_torch(i, seed ^ 0x5DEECE66D), 11).to(torch.float64) * 2.0 ** -53
        return (torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(2.0 * math.pi * u2)).to(torch.float32)
    return _fill_torch(n, start, device, torch.float32, gen)


def zipf_uint64_device(n: int, seed: int, device, s: float = 1.1, support: int = 1 << 32, start: int = 0):
    """Same construction as zipf_uint64; device pow may differ in the last bit."""
    import torch
    a = 1.0 - s

    def gen(i):
        u = (_lsr(_mix_torch(i, seed), 11).to(torch.float64) + 0.5) * 2.0 ** -53
        rank = torch.floor(((float(support) ** a - 1.0) * u + 1.0) ** (1.0 / a)) - 1.0
        r = rank.clamp(0, support - 1).to(torch.int64)
        r = (r * 0x9E3779B1) & (support - 1)
        r = r ^ (r >> 15)
        return r
    return _fill_torch(n, start, device, torch.int64, gen).view(torch.uint64)
