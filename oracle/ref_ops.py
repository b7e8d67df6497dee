"""Attention composed from the REFERENCE's own compiled C operators. TEST INFRASTRUCTURE ONLY.

``_ref/libember_ref_ops.so`` is the reference's unmodified ``operators_cpu.c`` +
``memory_cpu.c`` compiled by the Makefile beside this file. This module calls
those C functions through ctypes in the order the reference's Python front-end
would (``Tensor.__matmul__`` -> ``matmul_batched``; ``* scale`` -> ``mul_scalar``;
``+ mask`` -> ``add_broadcasted`` with the strides ``calculate_broadcast`` yields;
``softmax`` -> ``max_axis``, ``sub_broadcasted``, ``exponent_tensor``, ``sum_axis``,
``truediv_broadcasted``), one (batch*head) slice at a time because the reference
counts elements in a C ``int``. Transposes are done in NumPy, as the reference
forces for tensors of rank > 2. It is the "reference" CPU baseline of the benchmark
and the pin the C restatement is checked against.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(_HERE, "_ref", "libember_ref_ops.so")
_f = ctypes.POINTER(ctypes.c_float)
_i = ctypes.POINTER(ctypes.c_int)
_LIB = None


def available() -> bool:
    return os.path.exists(SO)


def lib():
    global _LIB
    if _LIB is None:
        L = ctypes.CDLL(SO)
        L.matmul_batched.argtypes = [_f, _f, _f] + [ctypes.c_int] * 4
        L.mul_scalar.argtypes = [_f, ctypes.c_float, _f, ctypes.c_int]
        L.mul_tensor.argtypes = [_f, _f, _f, ctypes.c_int]
        for n in ("add", "sub", "truediv"):
            getattr(L, n + "_broadcasted").argtypes = [_f, _f, _f, _i, _i, _i, ctypes.c_int]
        L.exponent_tensor.argtypes = [_f, _f, ctypes.c_int]
        L.max_axis.argtypes = [_f, _f] + [ctypes.c_int] * 3
        L.sum_axis.argtypes = [_f, _f] + [ctypes.c_int] * 3
        L.log_tensor.argtypes = [_f, _f, ctypes.c_int]
        L.sub_tensor.argtypes = [_f, _f, _f, ctypes.c_int]
        L.truediv_scalar.argtypes = [_f, ctypes.c_float, _f, ctypes.c_int]
        L.sum.argtypes = [_f, ctypes.c_int]
        L.sum.restype = ctypes.c_float
        for n in ("matmul_batched", "mul_scalar", "mul_tensor", "add_broadcasted", "sub_broadcasted",
                  "truediv_broadcasted", "exponent_tensor", "max_axis", "sum_axis", "log_tensor", "sub_tensor",
                  "truediv_scalar"):
            getattr(L, n).restype = None
        _LIB = L
    return _LIB


def _p(a):
    return a.ctypes.data_as(_f)


def _ia(t):
    return (ctypes.c_int * len(t))(*t)


def _mm(a, b):
    n, k = a.shape
    m = b.shape[1]
    out = np.empty((n, m), np.float32)
    lib().matmul_batched(_p(a), _p(b), _p(out), 1, n, m, k)
    return out


def _bcast(name, a, b_col_or_mat, strides_b):
    """a: (lq, lk); second operand broadcast with the given element strides."""
    lq, lk = a.shape
    out = np.empty_like(a)
    getattr(lib(), name + "_broadcasted")(_p(a), _p(b_col_or_mat), _p(out), _ia((lq, lk)),
                                          _ia((lk, 1)), _ia(strides_b), 2)
    return out


def _softmax_rows(s):
    lq, lk = s.shape
    L = lib()
    mx = np.empty((lq, 1), np.float32)
    L.max_axis(_p(s), _p(mx), lq, 1, lk)
    sh = _bcast("sub", s, mx, (1, 0))
    e = np.empty_like(sh)
    L.exponent_tensor(_p(sh), _p(e), lq * lk)
    sm = np.empty((lq, 1), np.float32)
    L.sum_axis(_p(e), _p(sm), lq, 1, lk)
    return _bcast("truediv", e, sm, (1, 0)), mx, sm


def causal_mask(lq, lk):
    i = np.arange(lq)[:, None]
    j = np.arange(lk)[None, :]
    return np.where(j > i + (lk - lq), -np.inf, 0.0).astype(np.float32)


def _probs(q, k, scale, mask):
    L = lib()
    kt = np.ascontiguousarray(k.T)
    s = _mm(q, kt)
    s2 = np.empty_like(s)
    L.mul_scalar(_p(s), ctypes.c_float(scale), _p(s2), s.size)
    if mask is not None:
        s2 = _bcast("add", s2, mask, (mask.shape[1], 1))
    return _softmax_rows(s2)


def attention_fwd(q, k, v, scale=None, causal=False):
    q, k, v = (np.ascontiguousarray(x, np.float32) for x in (q, k, v))
    lq, d = q.shape[-2:]
    lk = k.shape[-2]
    if scale is None:
        scale = 1.0 / np.sqrt(d)
    q2, k2, v2 = q.reshape(-1, lq, d), k.reshape(-1, lk, d), v.reshape(-1, lk, d)
    out = np.empty_like(q2)
    lse = np.empty(q2.shape[:2], np.float32)
    mask = causal_mask(lq, lk) if causal else None
    for b in range(q2.shape[0]):
        p, mx, sm = _probs(q2[b], k2[b], float(scale), mask)
        out[b] = _mm(p, v2[b])
        lse[b] = (mx.astype(np.float64) + np.log(sm.astype(np.float64)))[:, 0]
    return out.reshape(q.shape), lse.reshape(q.shape[:-1])


def attention_bwd(q, k, v, dout, scale=None, causal=False):
    q, k, v, dout = (np.ascontiguousarray(x, np.float32) for x in (q, k, v, dout))
    lq, d = q.shape[-2:]
    lk = k.shape[-2]
    if scale is None:
        scale = 1.0 / np.sqrt(d)
    L = lib()
    q2, k2, v2, g2 = (x.reshape(-1, x.shape[-2], d) for x in (q, k, v, dout))
    dq, dk, dv = np.empty_like(q2), np.empty_like(k2), np.empty_like(v2)
    mask = causal_mask(lq, lk) if causal else None
    for b in range(q2.shape[0]):
        p, _, _ = _probs(q2[b], k2[b], float(scale), mask)
        dv[b] = _mm(np.ascontiguousarray(p.T), g2[b])
        dp = _mm(g2[b], np.ascontiguousarray(v2[b].T))
        prod = np.empty_like(p)
        L.mul_tensor(_p(dp), _p(p), _p(prod), p.size)
        delta = np.empty((lq, 1), np.float32)
        L.sum_axis(_p(prod), _p(delta), lq, 1, lk)
        t = _bcast("sub", dp, delta, (1, 0))
        t2 = np.empty_like(t)
        L.mul_tensor(_p(p), _p(t), _p(t2), t.size)
        ds = np.empty_like(t2)
        L.mul_scalar(_p(t2), ctypes.c_float(scale), _p(ds), t2.size)
        dq[b] = _mm(ds, k2[b])
        dk[b] = _mm(np.ascontiguousarray(ds.T), q2[b])
    return dq.reshape(q.shape), dk.reshape(k.shape), dv.reshape(v.shape)


def linear_fwd(x, w, b=None):
    """The reference's Linear.forward (ember/nn/layers.py:45-48) on its compiled C operators."""
    x, w = (np.ascontiguousarray(t, np.float32) for t in (x, w))
    y = _mm(x, w)
    if b is None:
        return y
    b2 = np.ascontiguousarray(b, np.float32).reshape(1, -1)
    m, n = y.shape
    out = np.empty_like(y)
    # b + (x @ w): the bias is the first operand, broadcast over the rows
    lib().add_broadcasted(_p(b2), _p(y), _p(out), _ia((m, n)), _ia((0, 1)), _ia((n, 1)), 2)
    return out


def linear_bwd(x, w, dy):
    """The reference's Linear.backward (ember/nn/layers.py:50-56): host transposes, C matmuls, sum over axis 0."""
    x, w, dy = (np.ascontiguousarray(t, np.float32) for t in (x, w, dy))
    m, n = dy.shape
    dw = _mm(np.ascontiguousarray(x.T), dy)
    db = np.empty((n,), np.float32)
    lib().sum_axis(_p(dy), _p(db), 1, n, m)
    dx = _mm(dy, np.ascontiguousarray(w.T))
    return dx, dw, db


def softmax(x):
    """ember.softmax(x, axis=-1) on the reference's compiled C operators (2-D input)."""
    x = np.ascontiguousarray(x, np.float32)
    p, _, _ = _softmax_rows(x.copy())
    return p


def cross_entropy_fwd(pred, target):
    """CrossEntropyLoss.forward (ember/loss/losses.py:42-51) op by op; returns (loss, probs)."""
    pred, target = (np.ascontiguousarray(t, np.float32) for t in (pred, target))
    rows, cols = pred.shape
    L = lib()
    mx = np.empty((rows, 1), np.float32)
    L.max_axis(_p(pred), _p(mx), rows, 1, cols)
    shifted = _bcast("sub", pred, mx, (1, 0))
    e = np.empty_like(shifted)
    L.exponent_tensor(_p(shifted), _p(e), e.size)
    sm = np.empty((rows, 1), np.float32)
    L.sum_axis(_p(e), _p(sm), rows, 1, cols)
    lg = np.empty_like(sm)
    L.log_tensor(_p(sm), _p(lg), rows)
    logp = _bcast("sub", shifted, lg, (1, 0))
    probs = np.empty_like(logp)
    L.exponent_tensor(_p(logp), _p(probs), probs.size)
    prod = np.empty_like(logp)
    L.mul_tensor(_p(target), _p(logp), _p(prod), prod.size)
    total = L.sum(_p(prod), prod.size)
    return -float(total) / rows, probs


def cross_entropy_bwd(probs, target):
    probs, target = (np.ascontiguousarray(t, np.float32) for t in (probs, target))
    d = np.empty_like(probs)
    lib().sub_tensor(_p(probs), _p(target), _p(d), d.size)
    g = np.empty_like(d)
    lib().truediv_scalar(_p(d), ctypes.c_float(float(probs.shape[0])), _p(g), d.size)
    return g
