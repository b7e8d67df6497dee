import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def bf16_round(x: np.ndarray) -> np.ndarray:
    """Round float32 values to the nearest bfloat16 (ties to even), returned as float32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).reshape(x.shape)


@pytest.fixture(scope="session")
def golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "attention_golden.npz"))


@pytest.fixture(scope="session")
def linear_golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "linear_golden.npz"))


def linear_golden_inputs(meta):
    """x, w, b (None when the case has no bias), upstream gradient of one linear_golden.npz case."""
    from inputs import normal

    m, k, n, seed, with_bias = (int(x) for x in meta)
    x = normal(seed, (m, k))
    w = normal(seed + 1, (k, n)) * np.float32(0.1)
    b = normal(seed + 2, (n,)) if with_bias else None
    return x, w, b, normal(seed + 3, (m, n))


@pytest.fixture(scope="session")
def softmax_golden():
    return np.load(os.path.join(ROOT, "tests", "golden", "softmax_golden.npz"))


def softmax_golden_inputs(meta):
    """Logits and one-hot targets of one softmax_golden.npz case."""
    from inputs import normal

    rows, cols, seed = (int(x) for x in meta)
    x = normal(seed, (rows, cols)) * np.float32(3.0)
    target = np.zeros((rows, cols), np.float32)
    target[np.arange(rows), (7 * np.arange(rows)) % cols] = 1.0
    return x, target


def golden_inputs(meta, with_dout=False):
    from inputs import normal

    B, H, Lq, Lk, D, causal, seed = (int(x) for x in meta)
    q = normal(seed, (B, H, Lq, D))
    k = normal(seed + 100, (B, H, Lk, D))
    v = normal(seed + 200, (B, H, Lk, D))
    out = [q, k, v]
    if with_dout:
        out.append(normal(seed + 300, (B, H, Lq, D)))
    return out, bool(causal)


def seeded(shape, seed, scale=1.0):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal(shape, dtype=np.float32) * np.float32(scale)).astype(np.float32)


class Guarded:
    """A device buffer with a poisoned band on each side, standing in for a memory checker: the
    kernels under test write into ``.t`` (a torch tensor view in the middle of a larger byte
    buffer whose first and last ``band`` bytes hold 0x7F) and ``check()`` asserts afterwards that no
    byte of either band changed, i.e. that nothing was written outside the tensor."""

    def __init__(self, torch, shape, dtype, device, band=32 * 1024):
        n = 1
        for s in shape:
            n *= int(s)
        es = torch.empty((), dtype=dtype).element_size()
        self.band = band
        self.raw = torch.full((2 * band + n * es,), 0x7F, dtype=torch.uint8, device=device)
        self.t = self.raw[band:band + n * es].view(dtype).view(*shape)
        self._torch = torch

    def check(self, name=""):
        lo, hi = self.raw[:self.band], self.raw[-self.band:]
        assert bool((lo == 0x7F).all()) and bool((hi == 0x7F).all()), f"write outside the tensor {name}"
