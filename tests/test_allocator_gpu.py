"""GPU tests of the stream-ordered allocator that replaces the reference's one cudaMalloc/cudaFree
per tensor (src/core/memory_gpu.cu:10-28, TODO.md:12): freed blocks are reused from the pool, a
failed allocation is a NULL / MemoryError with the context intact (src/tensor/tensor_api.c:28-31),
and a block released in a caller's stream order is not recycled before that stream is done with it."""
import ctypes

import numpy as np
import pytest

import ember_b200 as em
from ember_b200 import _lib

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def L():
    if not torch.cuda.is_available():
        pytest.skip("needs CUDA")
    lib = _lib.lib()
    _lib.check(lib.ember_set_device(0))
    return lib


def _stats(L):
    r, u = ctypes.c_size_t(0), ctypes.c_size_t(0)
    _lib.check(L.ember_pool_stats(ctypes.byref(r), ctypes.byref(u)))
    return r.value, u.value


def test_freed_blocks_are_reused_without_new_driver_allocations(L):
    sizes = [1 << 12, 3 << 20, 17 << 20, 1 << 16, 64 << 20, 5 << 10]
    # warm the pool with the largest working set of the loop below
    blocks = [L.alloc_memory(s) for s in sizes]
    assert all(blocks)
    for b in blocks:
        L.free_memory(b)
    L.sync_device()
    reserved0, used0 = _stats(L)
    rng = np.random.default_rng(0)
    for i in range(1000):
        n = int(rng.integers(1, len(sizes) + 1))
        held = [L.alloc_memory(sizes[int(j)]) for j in rng.permutation(len(sizes))[:n]]
        assert all(held)
        for b in held:
            L.free_memory(b)
    L.sync_device()
    reserved1, used1 = _stats(L)
    # 1000 rounds of up to 90 MB each came out of what the pool already held (a little slack for
    # fragmentation; without reuse the pool would have grown by tens of gigabytes)
    assert reserved1 <= reserved0 + sum(sizes), (reserved0, reserved1)
    assert used1 == used0                                  # and nothing leaked


def test_failed_allocation_is_null_and_memory_error_and_context_survives(L):
    assert L.alloc_memory(1 << 50) is None
    assert b"cudaMallocAsync" in L.ember_last_error()
    with pytest.raises(MemoryError):
        em.Tensor.empty((1 << 48,), "float32")
    # the context is still usable: a small attention call runs and is correct to float32 accuracy
    x = np.random.default_rng(1).standard_normal((1, 1, 8, 16)).astype(np.float32)
    o, _ = em.attention_forward(em.Tensor(x), em.Tensor(x), em.Tensor(x), None, False)
    assert np.isfinite(o.to_np()).all()


def test_free_in_a_callers_stream_order_protects_a_running_kernel(L):
    """A block is written and read by kernels queued behind long-running work on a caller's stream
    and released at once with ember_free_async on that stream. An allocation on the library stream
    that is filled immediately must not disturb them: either the pool hands out other memory, or it
    makes the library stream wait for the release. (free_memory would order the release on the
    library stream, which knows nothing of the caller's kernels.)"""
    s = torch.cuda.Stream()
    sp = ctypes.c_void_p(s.cuda_stream)
    n = 32 << 20                                            # elements
    ones = torch.full((n,), 1.0, dtype=torch.float32, device="cuda")
    twos = torch.full((n,), 2.0, dtype=torch.float32, device="cuda")
    got_a = torch.zeros((n,), dtype=torch.float32, device="cuda")
    got_b = torch.zeros((n,), dtype=torch.float32, device="cuda")
    busy = torch.empty(1 << 28, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    a = L.ember_alloc_async(2 * n, sp)
    assert a
    with torch.cuda.stream(s):
        for _ in range(20):                                 # a few milliseconds of work ahead of `a`'s users
            busy.mul_(1.0001)
    _lib.check(L.ember_f32_to_bf16(ones.data_ptr(), a, n, sp))     # writes `a` on the caller's stream
    _lib.check(L.ember_bf16_to_f32(a, got_a.data_ptr(), n, sp))    # reads it back
    _lib.check(L.ember_free_async(a, sp))
    b = L.alloc_memory(2 * n)                                      # library stream, idle: runs at once
    assert b
    _lib.check(L.ember_f32_to_bf16(twos.data_ptr(), b, n, None))
    _lib.check(L.ember_bf16_to_f32(b, got_b.data_ptr(), n, None))
    L.free_memory(b)
    s.synchronize()
    L.sync_device()
    assert bool((got_a == 1.0).all()) and bool((got_b == 2.0).all())
