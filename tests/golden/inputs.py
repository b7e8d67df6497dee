"""Bit-reproducible synthetic inputs for the golden vectors.

Values are approximately N(0, 1): the sum of twelve 16-bit uniforms from a
counter-based SplitMix64 stream, centred and scaled (Irwin-Hall). Only integer
arithmetic and one exact float32 scaling are involved, so every platform and
NumPy version yields the same bits; the fixtures therefore store outputs only.
"""
import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x):
    x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
    z = x
    z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
    z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
    return z ^ (z >> np.uint64(31))


def normal(seed: int, shape) -> np.ndarray:
    n = int(np.prod(shape))
    idx = np.arange(n, dtype=np.uint64)
    total = np.zeros(n, dtype=np.int64)
    with np.errstate(over="ignore"):
        for r in range(3):
            z = _splitmix64(idx * np.uint64(3) + np.uint64(r) + (np.uint64(seed) << np.uint64(40)))
            for s in (0, 16, 32, 48):
                total += ((z >> np.uint64(s)) & np.uint64(0xFFFF)).astype(np.int64)
    # mean 12*32767.5, variance 12*(65536^2-1)/12 ~= 65536^2
    centred = total - 393210
    return (centred.astype(np.float32) * np.float32(1.0 / 65536.0)).reshape(shape)
