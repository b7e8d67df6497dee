"""Host-side mirror of the reference's tensor front-end for the attention path.

``Tensor`` carries shape and dtype in Python and an opaque native ``_Tensor`` underneath, as the
reference's does (ember/tensor/tensor.py:73-117: shape/strides live only in Python; the native
object holds ``d_ptr`` and ``size``, src/core/tensor_types.h:6-9). Only contiguous row-major
layout exists (ember/tensor/tensor_utils.py:85-94). dtype widens from the reference's single
``"float32"`` (ember/tensor/tensor.py:69) to ``"float32" | "bfloat16"``.

``attention`` is the new functional op, added the way the reference adds a non-element-wise
operator (docs/extending.md:83-88): a binding function in ``ember_b200._core`` (CPython extension,
csrc/tensor_api.c) called with the native objects and the extents as ints. It validates like
``Tensor.__matmul__`` (ember/tensor/tensor.py:163-197): TypeError for non-Tensor operands,
ValueError for rank/shape mismatches.
"""
from __future__ import annotations

import math

import numpy as np

from . import _core

_DT = {"float32": _core.F32, "bfloat16": _core.BF16}


class Tensor:
    """A contiguous device tensor of float32 or bfloat16 elements."""

    def __init__(self, data, dtype: str = "float32"):
        if dtype not in _DT:
            raise TypeError(f"Unsupported dtype {dtype!r}")
        arr = np.ascontiguousarray(np.asarray(data), dtype=np.float32)  # tensor.py:80-85: force f32
        self.shape = tuple(arr.shape)
        self.dtype = dtype
        self._core = _core._from_numpy(arr.reshape(-1), _DT[dtype])

    @classmethod
    def _from_core(cls, core, shape, dtype: str) -> "Tensor":
        t = cls.__new__(cls)
        t.shape, t.dtype, t._core = tuple(shape), dtype, core
        return t

    @classmethod
    def empty(cls, shape, dtype: str = "float32") -> "Tensor":
        n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
        return cls._from_core(_core._Tensor(n, _DT[dtype]), shape, dtype)

    @classmethod
    def from_np(cls, arr, dtype: str = "float32") -> "Tensor":
        return cls(arr, dtype)

    @property
    def size(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64)) if len(self.shape) else 1

    @property
    def ptr(self) -> int:
        """Device address of the buffer (for callers of the raw C ABI)."""
        return self._core._ptr()

    def view(self, offset: int, shape) -> "Tensor":
        """A tensor of the given shape over this tensor's elements from ``offset`` on (no copy; the
        view keeps the memory alive)."""
        n = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
        return Tensor._from_core(self._core._view(int(offset), n), shape, self.dtype)

    def to_bf16(self) -> "Tensor":
        return Tensor._from_core(_core._convert(self._core, _core.BF16), self.shape, "bfloat16")

    def to_f32(self) -> "Tensor":
        return Tensor._from_core(_core._convert(self._core, _core.F32), self.shape, "float32")

    def to_np(self) -> np.ndarray:
        """Float32 NumPy copy (bf16 tensors are widened on the device first); waits for the device."""
        out = np.empty(self.size, dtype=np.float32)
        self._core._copy_to_buffer(out)
        return out.reshape(self.shape)

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
    lead = q.shape[:-2]
    heads = lead[-1] if lead else 1
    batch = int(np.prod(lead[:-1], dtype=np.int64)) if len(lead) > 1 else 1
    return batch, heads, q.shape[-2], k.shape[-2], q.shape[-1]


def attention_forward(q: Tensor, k: Tensor, v: Tensor, scale: float | None = None, causal: bool = False):
    """Fused softmax(q kT * scale [+ causal mask]) v. Returns (out, lse); lse is float32 of shape q.shape[:-1]."""
    B, H, lq, lk, d = _check_qkv(q, k, v, "attention")
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    out, lse = _core._attention_fwd(q._core, k._core, v._core, B, H, lq, lk, d, float(scale), int(bool(causal)))
    return Tensor._from_core(out, q.shape, q.dtype), Tensor._from_core(lse, q.shape[:-1], "float32")


def attention(q: Tensor, k: Tensor, v: Tensor, scale: float | None = None, causal: bool = False) -> Tensor:
    """``ember.attention``: 4-D (B, H, L, D) operands (any number of leading batch dims)."""
    return attention_forward(q, k, v, scale, causal)[0]


def attention_backward(q: Tensor, k: Tensor, v: Tensor, out: Tensor, lse: Tensor, dout: Tensor,
                       scale: float | None = None, causal: bool = False, into=None):
    """Returns (dq, dk, dv) given the forward's inputs, output and log-sum-exp. ``into`` may supply
    the three result tensors (e.g. views of one buffer); they are then written instead of allocated."""
    B, H, lq, lk, d = _check_qkv(q, k, v, "attention_backward")
    for name, t, shp in (("out", out, q.shape), ("dout", dout, q.shape), ("lse", lse, q.shape[:-1])):
        if not isinstance(t, Tensor):
            raise TypeError(f"attention_backward: {name} must be a Tensor, got '{type(t).__name__}'")
        if t.shape != tuple(shp):
            raise ValueError(f"attention_backward: {name} has shape {t.shape}, expected {tuple(shp)}")
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    outs = tuple(t._core for t in into) if into is not None else None
    dq, dk, dv = _core._attention_bwd(q._core, k._core, v._core, out._core, lse._core, dout._core, B, H, lq, lk, d,
                                      float(scale), int(bool(causal)), outs)
    return (Tensor._from_core(dq, q.shape, q.dtype), Tensor._from_core(dk, k.shape, k.dtype),
            Tensor._from_core(dv, v.shape, v.dtype))


def attention_decode(q: Tensor, k: Tensor, v: Tensor, scale: float | None = None, num_splits: int = 0):
    """Single-query decode: q has one row per (batch, head); returns (out, lse)."""
    B, H, lq, lk, d = _check_qkv(q, k, v, "attention_decode")
    if lq != 1:
        raise ValueError(f"attention_decode needs exactly one query row, got {lq}")
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    out, lse = _core._attention_decode(q._core, k._core, v._core, B, H, lk, d, float(scale), int(num_splits))
    return Tensor._from_core(out, q.shape, q.dtype), Tensor._from_core(lse, q.shape[:-1], "float32")


def _check_linear(x, w, b, fn):
    for name, t in (("x", x), ("w", w)) + ((("b", b),) if b is not None else ()):
        if not isinstance(t, Tensor):
            raise TypeError(f"{fn}: {name} must be a Tensor, got '{type(t).__name__}'")
    if len(w.shape) != 2:
        raise ValueError(f"{fn}: w must be (in_features, out_features), got {w.shape}")
    if b is not None and b.size != w.shape[1]:
        raise ValueError(f"{fn}: bias has {b.size} elements, expected {w.shape[1]}")
    if x.dtype != w.dtype or (b is not None and b.dtype != w.dtype):
        raise TypeError(f"{fn}: x, w and bias must share a dtype")


def linear_forward(x: Tensor, w: Tensor, b: Tensor | None = None, *, x_heads: int = 0, y_heads: int = 0) -> Tensor:
    """``b + x @ w`` of the reference's Linear layer (ember/nn/layers.py:45-48) in one call.

    x is (..., in_features) and the result (..., out_features), unless a head-major layout is asked
    for: with ``x_heads`` > 0, x is (B, x_heads, L, D) as attention writes it and counts as the
    (B*L, x_heads*D) matrix; with ``y_heads`` > 0 (x then is (B, L, in_features)) the result is
    (parts, B, y_heads, L, D) with parts * y_heads * D == out_features, which is what a fused q/k/v
    projection hands to attention."""
    _check_linear(x, w, b, "linear")
    k, n = w.shape
    if x_heads:
        if len(x.shape) != 4 or x.shape[1] != x_heads or x.shape[1] * x.shape[3] != k:
            raise ValueError(f"linear: head-major x must be (B, {x_heads}, L, D) with {x_heads}*D == {k}, got {x.shape}")
        B, _, seq, dim = x.shape
        m, out_shape = B * seq, (B, seq, n)
    else:
        if len(x.shape) < 1 or x.shape[-1] != k:
            raise ValueError(f"Shape mismatch: {x.shape} cannot be multiplied with {w.shape}")
        m, out_shape = x.size // k, x.shape[:-1] + (n,)
        seq = dim = 0
    if y_heads:
        if x_heads or len(x.shape) != 3:
            raise ValueError(f"linear: a head-major result needs x of shape (B, L, in_features), got {x.shape}")
        B, seq = x.shape[0], x.shape[1]
        if n % y_heads:
            raise ValueError(f"linear: out_features={n} is not a multiple of y_heads={y_heads}")
        # parts is whatever makes the head dimension the one attention will see: the caller says it
        # through the weight's width, out_features = parts * y_heads * D with D = in_features / y_heads
        dim = k // y_heads
        if dim == 0 or n % (y_heads * dim):
            raise ValueError(f"linear: out_features={n} is not a multiple of y_heads*D={y_heads * dim}")
        out_shape = (n // (y_heads * dim), B, y_heads, seq, dim)
    y = _core._linear_fwd(x._core, w._core, b._core if b is not None else None, m, n, k, x_heads, y_heads, seq, dim)
    return Tensor._from_core(y, out_shape, x.dtype)


def linear_backward(x: Tensor, w: Tensor, grad_y: Tensor, *, x_heads: int = 0, y_heads: int = 0,
                    need_grad_x: bool = True, need_grad_b: bool = True):
    """Returns (grad_x | None, grad_w, grad_b | None) of the reference's Linear.backward
    (ember/nn/layers.py:50-56); layouts as in ``linear_forward`` (grad_x has x's, grad_y has y's)."""
    _check_linear(x, w, None, "linear_backward")
    if not isinstance(grad_y, Tensor):
        raise TypeError(f"linear_backward: grad_y must be a Tensor, got '{type(grad_y).__name__}'")
    k, n = w.shape
    seq = dim = 0
    if x_heads:
        B, _, seq, dim = x.shape
        m = B * seq
    else:
        m = x.size // k
    if y_heads:
        B, seq = x.shape[0], x.shape[1]
        dim = k // y_heads
    if grad_y.size != m * n:
        raise ValueError(f"linear_backward: grad_y has {grad_y.size} elements, expected {m * n}")
    dx, dw, db = _core._linear_bwd(x._core, w._core, grad_y._core, m, n, k, x_heads, y_heads, seq, dim,
                                   int(bool(need_grad_x)), int(bool(need_grad_b)))
    return (Tensor._from_core(dx, x.shape, x.dtype) if dx is not None else None, Tensor._from_core(dw, w.shape, w.dtype),
            Tensor._from_core(db, (n,), w.dtype) if db is not None else None)


def _rows_cols(a: Tensor, fn: str):
    if not isinstance(a, Tensor):
        raise TypeError(f"{fn} expects a Tensor, got '{type(a).__name__}'")
    if len(a.shape) < 1:
        raise ValueError(f"{fn} needs at least one axis")
    return a.size // a.shape[-1], a.shape[-1]


def softmax(a: Tensor, axis: int = -1) -> Tensor:
    """Numerically-stable softmax along the last axis (the reference's ``softmax``,
    ember/tensor/tensor.py:430-437, as one fused pass)."""
    if axis not in (-1, len(a.shape) - 1):
        raise ValueError("softmax: only the last axis is supported by the fused kernel")
    rows, cols = _rows_cols(a, "softmax()")
    return Tensor._from_core(_core._softmax(a._core, rows, cols, 0), a.shape, a.dtype)


def log_softmax(a: Tensor, axis: int = -1) -> Tensor:
    if axis not in (-1, len(a.shape) - 1):
        raise ValueError("log_softmax: only the last axis is supported by the fused kernel")
    rows, cols = _rows_cols(a, "log_softmax()")
    return Tensor._from_core(_core._softmax(a._core, rows, cols, 1), a.shape, a.dtype)
