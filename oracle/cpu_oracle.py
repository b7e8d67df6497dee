"""ctypes front-end of the C oracle (``attention_oracle.c``). TEST INFRASTRUCTURE ONLY.

``attention_fwd`` / ``attention_bwd`` take and return float32 NumPy arrays of
shape (B, H, L, D) (any number of leading batch dims). The arithmetic follows
the reference's composed path; see the header of ``attention_oracle.c`` for the
file:line of each step.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

_f32p = ctypes.POINTER(ctypes.c_float)


def build(force: bool = False) -> str:
    """Compile ``liboracle.so`` beside its source if missing or stale."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "attention_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "liboracle.so"])
    return so


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        L = ctypes.CDLL(build())
        L.oracle_attention_fwd.argtypes = [_f32p] * 6 + [ctypes.c_int] * 4 + [ctypes.c_float, ctypes.c_int]
        L.oracle_attention_fwd.restype = None
        L.oracle_attention_bwd.argtypes = [_f32p] * 7 + [ctypes.c_int] * 4 + [ctypes.c_float, ctypes.c_int]
        L.oracle_attention_bwd.restype = None
        L.oracle_linear_fwd.argtypes = [_f32p] * 4 + [ctypes.c_int] * 3
        L.oracle_linear_fwd.restype = None
        L.oracle_linear_bwd.argtypes = [_f32p] * 6 + [ctypes.c_int] * 3
        L.oracle_linear_bwd.restype = None
        L.oracle_softmax.argtypes = [_f32p, _f32p, ctypes.c_int, ctypes.c_int]
        L.oracle_softmax.restype = None
        L.oracle_cross_entropy_fwd.argtypes = [_f32p] * 3 + [ctypes.c_int] * 2
        L.oracle_cross_entropy_fwd.restype = ctypes.c_double
        L.oracle_cross_entropy_bwd.argtypes = [_f32p] * 3 + [ctypes.c_int] * 2
        L.oracle_cross_entropy_bwd.restype = None
        L.oracle_set_threads.argtypes = [ctypes.c_int]
        _LIB = L
    return _LIB


def set_threads(n: int) -> None:
    lib().oracle_set_threads(int(n))


def _p(a):
    return a.ctypes.data_as(_f32p) if a is not None else None


def _prep(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    return x


def attention_fwd(q, k, v, scale=None, causal=False, return_probs=False):
    """Returns (out, lse[, probs]). lse = rowmax + log(rowsum) of the scaled, masked scores."""
    q, k, v = _prep(q), _prep(k), _prep(v)
    lq, d = q.shape[-2:]
    lk = k.shape[-2]
    bh = int(np.prod(q.shape[:-2], dtype=np.int64))
    if scale is None:
        scale = 1.0 / np.sqrt(d)
    out = np.empty_like(q)
    lse = np.empty(q.shape[:-1], dtype=np.float32)
    probs = np.empty(q.shape[:-2] + (lq, lk), dtype=np.float32) if return_probs else None
    lib().oracle_attention_fwd(_p(q), _p(k), _p(v), _p(out), _p(lse), _p(probs), bh, lq, lk, d,
                               float(scale), int(bool(causal)))
    return (out, lse, probs) if return_probs else (out, lse)


def attention_bwd(q, k, v, dout, scale=None, causal=False):
    """Returns (dq, dk, dv) of the composed manual backward."""
    q, k, v, dout = _prep(q), _prep(k), _prep(v), _prep(dout)
    lq, d = q.shape[-2:]
    lk = k.shape[-2]
    bh = int(np.prod(q.shape[:-2], dtype=np.int64))
    if scale is None:
        scale = 1.0 / np.sqrt(d)
    dq, dk, dv = np.empty_like(q), np.empty_like(k), np.empty_like(v)
    lib().oracle_attention_bwd(_p(q), _p(k), _p(v), _p(dout), _p(dq), _p(dk), _p(dv), bh, lq, lk, d,
                               float(scale), int(bool(causal)))
    return dq, dk, dv


def linear_fwd(x, w, b=None):
    """y = b + x @ w of the reference's Linear layer; x (m,k), w (k,n), b (n) or None."""
    x, w = _prep(x), _prep(w)
    m, k = x.shape
    n = w.shape[1]
    bb = _prep(b).reshape(n) if b is not None else None
    y = np.empty((m, n), dtype=np.float32)
    lib().oracle_linear_fwd(_p(x), _p(w), _p(bb), _p(y), m, n, k)
    return y


def linear_bwd(x, w, dy):
    """Returns (grad_x, grad_w, grad_b) of the reference's Linear.backward."""
    x, w, dy = _prep(x), _prep(w), _prep(dy)
    m, k = x.shape
    n = w.shape[1]
    dx, dw, db = np.empty((m, k), np.float32), np.empty((k, n), np.float32), np.empty((n,), np.float32)
    lib().oracle_linear_bwd(_p(x), _p(w), _p(dy), _p(dx), _p(dw), _p(db), m, n, k)
    return dx, dw, db


def softmax(x):
    """Softmax over the last axis, as the reference composes it (ember/tensor/tensor.py:430-437)."""
    x = _prep(x)
    cols = x.shape[-1]
    y = np.empty_like(x)
    lib().oracle_softmax(_p(x), _p(y), x.size // cols, cols)
    return y


def cross_entropy_fwd(pred, target):
    """Returns (loss, probs) of the reference's CrossEntropyLoss.forward (ember/loss/losses.py:42-51)."""
    pred, target = _prep(pred), _prep(target)
    rows, cols = pred.shape
    probs = np.empty_like(pred)
    loss = lib().oracle_cross_entropy_fwd(_p(pred), _p(target), _p(probs), rows, cols)
    return float(loss), probs


def cross_entropy_bwd(probs, target):
    """(probs - target) / n of CrossEntropyLoss.backward (ember/loss/losses.py:53-56)."""
    probs, target = _prep(probs), _prep(target)
    rows, cols = probs.shape
    grad = np.empty_like(probs)
    lib().oracle_cross_entropy_bwd(_p(probs), _p(target), _p(grad), rows, cols)
    return grad
