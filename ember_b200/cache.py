"""Key/value cache for decode steps: preallocated (B, Hkv, capacity, D) tensors, rows appended in
place, single-query attention over the filled part with grouped-query heads. The reference has no
cache; a decode step there rebuilds K and V as new tensors on every token
(ember/tensor/tensor.py:163-197 only multiplies whole tensors). The C ABI underneath
(``ember_kv_cache_append``, ``ember_attention_decode_cache``) also takes per-sequence lengths and a
page table; this class covers the common case of sequences that grow in step.
"""
from __future__ import annotations

import math

from . import _core
from .tensor import Tensor, _DT


class KVCache:
    def __init__(self, batch: int, kv_heads: int, capacity: int, head_dim: int, dtype: str = "bfloat16"):
        self.batch, self.kv_heads, self.capacity, self.head_dim, self.dtype = batch, kv_heads, capacity, head_dim, dtype
        n = batch * kv_heads * capacity * head_dim
        self.k = Tensor._from_core(_core._Tensor(n, _DT[dtype]), (batch, kv_heads, capacity, head_dim), dtype)
        self.v = Tensor._from_core(_core._Tensor(n, _DT[dtype]), (batch, kv_heads, capacity, head_dim), dtype)
        self.length = 0

    def append(self, k_new: Tensor, v_new: Tensor) -> None:
        """k_new, v_new: (B, Hkv, n_new, D); written at rows [length, length + n_new)."""
        for name, t in (("k_new", k_new), ("v_new", v_new)):
            if not isinstance(t, Tensor):
                raise TypeError(f"KVCache.append: {name} must be a Tensor, got '{type(t).__name__}'")
        want = (self.batch, self.kv_heads, k_new.shape[2] if len(k_new.shape) == 4 else -1, self.head_dim)
        if k_new.shape != want or v_new.shape != want:
            raise ValueError(f"KVCache.append expects (B={self.batch}, Hkv={self.kv_heads}, n_new, D={self.head_dim}), "
                             f"got {k_new.shape} and {v_new.shape}")
        n_new = k_new.shape[2]
        if self.length + n_new > self.capacity:
            raise ValueError(f"KVCache.append: {n_new} more rows do not fit ({self.length} of {self.capacity} used)")
        _core._kv_append(self.k._core, self.v._core, k_new._core, v_new._core, self.batch, self.kv_heads, self.capacity,
                         self.head_dim, n_new, self.length)
        self.length += n_new

    def decode(self, q: Tensor, scale: float | None = None, num_splits: int = 0):
        """q: (B, Hq, D) or (B, Hq, 1, D), Hq a multiple (1, 2, 4, 8) of Hkv. Returns (out, lse)."""
        if not isinstance(q, Tensor):
            raise TypeError(f"KVCache.decode: q must be a Tensor, got '{type(q).__name__}'")
        if self.length == 0:
            raise ValueError("KVCache.decode: the cache is empty")
        if len(q.shape) not in (3, 4) or q.shape[0] != self.batch or q.shape[-1] != self.head_dim or \
                (len(q.shape) == 4 and q.shape[2] != 1) or q.shape[1] % self.kv_heads:
            raise ValueError(f"KVCache.decode expects q of shape (B={self.batch}, Hq, [1,] D={self.head_dim}) with Hq a "
                             f"multiple of {self.kv_heads}, got {q.shape}")
        if scale is None:
            scale = 1.0 / math.sqrt(self.head_dim)
        out, lse = _core._decode_cache(q._core, self.k._core, self.v._core, self.batch, q.shape[1], self.kv_heads, self.length,
                                       self.capacity, self.head_dim, float(scale), int(num_splits))
        return Tensor._from_core(out, q.shape, q.dtype), Tensor._from_core(lse, (self.batch, q.shape[1]), "float32")
