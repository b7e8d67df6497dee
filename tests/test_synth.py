"""CPU-only: the generator of synthetic inputs keyed by the global element index
(``ember_b200.synth``) gives the same bits on the host (NumPy) and through torch, agrees with the
generator the golden vectors were made with, and a slab generated on its own equals the same slab
cut out of the whole tensor (so inputs do not depend on how many ranks share a job)."""
import os
import sys

import numpy as np
import pytest

from ember_b200 import synth

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
torch = pytest.importorskip("torch")


@pytest.mark.parametrize("seed,start,count", [(1, 0, 1000), (7, 123456789, 4097), (500, (1 << 33) + 5, 300)])
def test_numpy_and_torch_twins_agree_bit_for_bit(seed, start, count):
    a = synth.normal_np(seed, start, count)
    b = synth.normal_torch(torch, seed, start, count, "cpu", chunk=1000).numpy()
    assert a.dtype == np.float32 and np.array_equal(a, b)
    assert abs(float(a.mean())) < 0.2 and 0.8 < float(a.std()) < 1.2


def test_matches_the_golden_vector_generator():
    from inputs import normal

    assert np.array_equal(normal(3, (5, 7, 11)).reshape(-1), synth.normal_np(3, 0, 5 * 7 * 11))


def test_a_slab_does_not_depend_on_the_sharding():
    units, rows, dim = 8, 6, 16
    whole = synth.units_torch(torch, 9, 0, units, rows, dim, "cpu", 0.5, torch.bfloat16)
    for world in (2, 4, 8):
        per = units // world
        for r in range(world):
            slab = synth.units_torch(torch, 9, r * per, (r + 1) * per, rows, dim, "cpu", 0.5, torch.bfloat16)
            assert torch.equal(slab, whole[r * per:(r + 1) * per])


def test_bench_checksum_sees_single_bit_changes_and_positions():
    """The 64-bit checksum bench.py uses for its one-GPU-vs-N identity checks: equal tensors agree, one
    flipped bit or two swapped elements do not."""
    import importlib.util

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    a = synth.units_torch(torch, 3, 0, 2, 16, 32, "cpu", 0.5, torch.bfloat16)
    b = a.clone()
    assert bench.unit_checksum(torch, a) == bench.unit_checksum(torch, b)
    b.view(torch.int16)[1, 3, 5] ^= 1
    assert bench.unit_checksum(torch, a) != bench.unit_checksum(torch, b)
    c = a.clone()
    c[0, 0, 0], c[0, 0, 1] = a[0, 0, 1].clone(), a[0, 0, 0].clone()
    if not torch.equal(c, a):
        assert bench.unit_checksum(torch, a) != bench.unit_checksum(torch, c)
    f = torch.arange(10, dtype=torch.float32)
    assert bench.unit_checksum(torch, f) == bench.unit_checksum(torch, f.clone())
