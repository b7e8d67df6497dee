"""Synthetic inputs keyed by the GLOBAL element index.

A value depends only on (seed, index of the element in the un-sharded tensor), never on which rank
produces it or on how many ranks there are, so that a job split over N GPUs works on exactly the
slabs a single GPU would see and its results can be compared bit for bit with the single-GPU ones.

Values are approximately N(0, 1): the sum of twelve 16-bit uniforms taken from three SplitMix64
outputs per element, centred and scaled by 2^-16 (Irwin-Hall). Only 64-bit integer arithmetic and
one exact float32 scaling are involved, so NumPy on any host and torch on any device give the same
bits. ``normal_np`` is the host form, ``normal_torch`` its twin for a torch device; both take the
global index of the first element and a count.
"""
from __future__ import annotations

import numpy as np

_GOLD = 0x9E3779B97F4A7C15
_M1 = 0xBF58476D1CE4E5B9
_M2 = 0x94D049BB133111EB


def _splitmix64_np(x):
    x = x + np.uint64(_GOLD)
    z = x
    z = (z ^ (z >> np.uint64(30))) * np.uint64(_M1)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(_M2)
    return z ^ (z >> np.uint64(31))


def normal_np(seed: int, start: int, count: int) -> np.ndarray:
    """float32 values of global elements [start, start + count)."""
    idx = np.arange(start, start + count, dtype=np.uint64)
    total = np.zeros(count, dtype=np.int64)
    with np.errstate(over="ignore"):
        for r in range(3):
            z = _splitmix64_np(idx * np.uint64(3) + np.uint64(r) + (np.uint64(seed) << np.uint64(40)))
            for s in (0, 16, 32, 48):
                total += ((z >> np.uint64(s)) & np.uint64(0xFFFF)).astype(np.int64)
    return (total - 393210).astype(np.float32) * np.float32(1.0 / 65536.0)


def _signed(c: int) -> int:
    return c - (1 << 64) if c >= (1 << 63) else c


def normal_torch(torch, seed: int, start: int, count: int, device, chunk: int = 1 << 24):
    """The same values as ``normal_np`` as a float32 torch tensor on ``device``. torch has no unsigned
    64-bit arithmetic; signed int64 wraps the same way, and a logical right shift is an arithmetic
    one followed by a mask of the bits that survive."""
    out = torch.empty(count, dtype=torch.float32, device=device)

    def shr(z, k):
        return (z >> k) & ((1 << (64 - k)) - 1)

    for c0 in range(0, count, chunk):
        n = min(chunk, count - c0)
        idx = torch.arange(start + c0, start + c0 + n, dtype=torch.int64, device=device)
        total = torch.zeros(n, dtype=torch.int64, device=device)
        for r in range(3):
            x = idx * 3 + (r + _signed((seed << 40) & ((1 << 64) - 1))) + _signed(_GOLD)
            z = (x ^ shr(x, 30)) * _signed(_M1)
            z = (z ^ shr(z, 27)) * _signed(_M2)
            z = z ^ shr(z, 31)
            for s in (0, 16, 32, 48):
                total += (z >> s) & 0xFFFF
        out[c0:c0 + n] = (total - 393210).to(torch.float32) * (1.0 / 65536.0)
    return out


def units_torch(torch, seed: int, unit_begin: int, unit_end: int, rows: int, dim: int, device, scale: float = 1.0,
                dtype=None):
    """(unit_end - unit_begin, rows, dim) slab of the global (units, rows, dim) tensor of stream
    ``seed``: what rank r of a job sharded over the leading axis holds."""
    per = rows * dim
    t = normal_torch(torch, seed, unit_begin * per, (unit_end - unit_begin) * per, device)
    if scale != 1.0:
        t = t * scale
    t = t.view(unit_end - unit_begin, rows, dim)
    return t.to(dtype) if dtype is not None else t
