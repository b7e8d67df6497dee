"""Host-side mirror of the reference's tensor front-end for the attention path.

``Tensor`` carries shape and dtype in Python and an opaque device buffer underneath, as the
reference's does (ember/tensor/tensor.py:73-117: shape/strides live only in Python; the native
object holds ``d_ptr`` and ``size``, src/core/tensor_types.h:6-9). Only contiguous row-major
layout exists (ember/tensor/tensor_utils.py:85-94). dtype widens from the reference's single
``"float32"`` (ember/tensor/tensor.py:69) to ``"float32" | "bfloat16"``.

``attention`` is the new functional op, added the way the reference adds a non-element-wise
operator (docs/extending.md:83-88); it validates like ``Tensor.__matmul__``
(ember/tensor/tensor.py:163-197): TypeError for non-Tensor operands, ValueError for rank/shape
mismatches.
"""
from __future__ import annotations

import ctypes
import math

import numpy as np

from . import _lib
from ._lib import EMBER_BF16, EMBER_F32, EMBER_OP_BWD, EMBER_OP_DECODE, check

_DT = {"float32": EMBER_F32, "bfloat16": EMBER_BF16}
_ES = {"float32": 4, "bfloat16": 2}


class _Buffer:
    """Owns one device allocation (the ``_Tensor`` of src/tensor/tensor_api.c:21-41)."""

    __slots__ = ("ptr", "nbytes")

    def __init__(self, nbytes: int):
        self.nbytes = int(nbytes)
        self.ptr = _lib.lib().alloc_memory(self.nbytes)
        if not self.ptr:
            self.ptr = None
            raise MemoryError("Failed to allocate device memory: " + _lib.last_error())

    def __del__(self):
        if getattr(self, "ptr", None):
            try:
                _lib.lib().free_memory(self.ptr)
            except Exception:
                pass
            self.ptr = None


class Tensor:
    """A contiguous device tensor of float32 or bfloat16 elements."""

    def __init__(self, data, dtype: str = "float32"):
        arr = np.ascontiguousarray(np.asarray(data), dtype=np.float32)  # tensor.py:80-85: force f32
        if dtype not in _DT:
            raise TypeError(f"Unsupported dtype {dtype!r}")
        self.shape = tuple(arr.shape)
        self.dtype = "float32"
        self._core = _Buffer(max(arr.size, 1) * 4)
        if arr.size:
            _lib.lib().copy_to_device(self._core.ptr, arr.ctypes.data, arr.size * 4)
        if dtype == "bfloat16":
            b = self.to_bf16()
            self._core, self.dtype = b._core, b.dtype

    @classmethod
    def _from_core(cls, core: _Buffer, shape, dtype: str) -> "Tensor":
        t = cls.__new__(cls)
        t.shape, t.dtype, t._core = tuple(shape), dtype, core
        return t

    @classmethod
    def empty(cls, shape, dtype: str = "float32") -> "Tensor":
        n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
        return cls._from_core(_Buffer(max(n, 1) * _ES[dtype]), shape, dtype)

    @classmethod
    def from_np(cls, arr, dtype: str = "float32") -> "Tensor":
        return cls(arr, dtype)

    @property
    def size(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64)) if len(self.shape) else 1

    @property
    def ptr(self) -> int:
        return self._core.ptr

    def to_bf16(self) -> "Tensor":
        if self.dtype == "bfloat16":
            return self
        out = Tensor.empty(self.shape, "bfloat16")
        check(_lib.lib().ember_f32_to_bf16(self.ptr, out.ptr, self.size, None))
        return out

    def to_f32(self) -> "Tensor":
        if self.dtype == "float32":
            return self
        out = Tensor.empty(self.shape, "float32")
        check(_lib.lib().ember_bf16_to_f32(self.ptr, out.ptr, self.size, None))
        return out

    def to_np(self) -> np.ndarray:
        """Float32 NumPy copy (bf16 tensors are widened first); waits for the device."""
        t = self.to_f32()
        out = np.empty(self.shape, dtype=np.float32)
        if out.size:
            _lib.lib().copy_from_device(out.ctypes.data, t.ptr, out.size * 4)
        return out

    def __repr__(self):
        return f"Tensor(shape={self.shape}, dtype={self.dtype})"


def _check_qkv(q, k, v, fn):
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not isinstance(t, Tensor):
            raise TypeError(f"{fn}: {name} must be a Tensor, got '{type(t).__name__}'")
    if len(q.shape) < 2 or len(k.shape) < 2 or len(v.shape) < 2:
        raise ValueError(f"{fn} requires at least 2D operands, got {q.shape}, {k.shape}, {v.shape}")
    if q.shape[:-2] != k.shape[:-2] or k.shape != v.shape:
        raise ValueError(f"Batch dimensions must match for {fn}: {q.shape} vs {k.shape} vs {v.shape}")
    if q.shape[-1] != k.shape[-1]:
        raise ValueError(f"Shape mismatch: {q.shape} cannot attend over {k.shape}")
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError(f"{fn}: q, k and v must share a dtype, got {q.dtype}, {k.dtype}, {v.dtype}")
    bh = int(np.prod(q.shape[:-2], dtype=np.int64)) if len(q.shape) > 2 else 1
    return bh, q.shape[-2], k.shape[-2], q.shape[-1]


def attention_forward(q: Tensor, k: Tensor, v: Tensor, scale: float | None = None, causal: bool = False):
    """Fused softmax(q kT * scale [+ causal mask]) v. Returns (out, lse); lse is float32 of shape q.shape[:-1]."""
    bh, lq, lk, d = _check_qkv(q, k, v, "attention")
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    out = Tensor.empty(q.shape, q.dtype)
    lse = Tensor.empty(q.shape[:-1], "float32")
    check(_lib.lib().ember_attention_fwd(q.ptr, k.ptr, v.ptr, out.ptr, lse.ptr, bh, lq, lk, d, float(scale),
                                         int(bool(causal)), _DT[q.dtype], None))
    return out, lse


def attention(q: Tensor, k: Tensor, v: Tensor, scale: float | None = None, causal: bool = False) -> Tensor:
    """``ember.attention``: 4-D (B, H, L, D) operands (any number of leading batch dims)."""
    return attention_forward(q, k, v, scale, causal)[0]


def attention_backward(q: Tensor, k: Tensor, v: Tensor, out: Tensor, lse: Tensor, dout: Tensor,
                       scale: float | None = None, causal: bool = False):
    """Returns (dq, dk, dv) given the forward's inputs, output and log-sum-exp."""
    bh, lq, lk, d = _check_qkv(q, k, v, "attention_backward")
    for name, t, shp in (("out", out, q.shape), ("dout", dout, q.shape), ("lse", lse, q.shape[:-1])):
        if not isinstance(t, Tensor):
            raise TypeError(f"attention_backward: {name} must be a Tensor, got '{type(t).__name__}'")
        if t.shape != tuple(shp):
            raise ValueError(f"attention_backward: {name} has shape {t.shape}, expected {tuple(shp)}")
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    L = _lib.lib()
    dq, dk, dv = Tensor.empty(q.shape, q.dtype), Tensor.empty(k.shape, k.dtype), Tensor.empty(v.shape, v.dtype)
    nbytes = L.ember_attention_workspace_bytes(EMBER_OP_BWD, bh, lq, lk, d, _DT[q.dtype], 0)
    ws = _Buffer(nbytes)
    check(L.ember_attention_bwd(q.ptr, k.ptr, v.ptr, out.ptr, lse.ptr, dout.ptr, dq.ptr, dk.ptr, dv.ptr, bh, lq,
                                lk, d, float(scale), int(bool(causal)), _DT[q.dtype], ws.ptr, nbytes, None))
    return dq, dk, dv


def attention_decode(q: Tensor, k: Tensor, v: Tensor, scale: float | None = None, num_splits: int = 0):
    """Single-query decode: q has one row per (batch, head); returns (out, lse)."""
    bh, lq, lk, d = _check_qkv(q, k, v, "attention_decode")
    if lq != 1:
        raise ValueError(f"attention_decode needs exactly one query row, got {lq}")
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    L = _lib.lib()
    out = Tensor.empty(q.shape, q.dtype)
    lse = Tensor.empty(q.shape[:-1], "float32")
    nbytes = L.ember_attention_workspace_bytes(EMBER_OP_DECODE, bh, 1, lk, d, _DT[q.dtype], int(num_splits))
    ws = _Buffer(nbytes) if nbytes else None
    check(L.ember_attention_decode(q.ptr, k.ptr, v.ptr, out.ptr, lse.ptr, bh, lk, d, float(scale), _DT[q.dtype],
                                   int(num_splits), ws.ptr if ws else None, nbytes, None))
    return out, lse
