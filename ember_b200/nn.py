"""Layers of the attention path. ``Attention`` follows the reference's manual-backward layer contract
(ember/nn/base.py:7-35: ``__call__`` caches input and output, ``forward``/``backward`` are
explicit, ``parameters``/``gradients``/``reset``), as ``Linear`` does for matmul
(ember/nn/layers.py:45-56); it has no parameters. ``Linear`` is the reference's layer of that name
as one fused call per direction, and ``MultiHeadAttention`` chains a fused q/k/v projection,
attention and the output projection with the (B, H, L, D) layout produced and consumed directly by
the projections, so that no transpose runs in between.
"""
from __future__ import annotations

import abc
import math

import numpy as np

from .tensor import Tensor, attention_backward, attention_forward, linear_backward, linear_forward


class Layer(abc.ABC):
    """The reference's layer contract (ember/nn/base.py:7-35): calling a layer runs ``forward`` and
    remembers the input and the output (``x``, ``y``) for the explicit ``backward``; ``training``
    defaults to True as it does there (base.py:11). Subclasses give ``forward``, ``backward``,
    ``parameters``, ``gradients`` and ``reset``."""

    x = None
    y = None

    def __call__(self, x, training: bool = True):
        self._training = training
        self.x = x
        self.y = self.forward(x, training)
        return self.y

    @abc.abstractmethod
    def forward(self, x, training: bool = True): ...

    @abc.abstractmethod
    def backward(self, grad_y): ...

    @abc.abstractmethod
    def parameters(self) -> list: ...

    @abc.abstractmethod
    def gradients(self) -> list: ...

    @abc.abstractmethod
    def reset(self) -> None: ...


class Sequential(Layer):
    """Layers applied one after the other, gradients walked back in reverse (the reference's
    container of the same name, ember/nn/base.py:50-75). ``Linear`` and ``MultiHeadAttention`` map
    one tensor to one tensor and compose here; ``Attention`` maps a (q, k, v) triple to one tensor and
    returns a triple from ``backward``, so it can only stand first."""

    def __init__(self, *layers: Layer):
        self.layers = tuple(layers)

    def forward(self, x, training: bool = True):
        for layer in self.layers:
            x = layer(x, training)
        return x

    def backward(self, grad_y):
        for layer in self.layers[::-1]:
            grad_y = layer.backward(grad_y)
        return grad_y

    def parameters(self) -> list:
        return [p for layer in self.layers for p in layer.parameters()]

    def gradients(self) -> list:
        return [g for layer in self.layers for g in layer.gradients()]

    def reset(self) -> None:
        self.x = self.y = None
        for layer in self.layers:
            layer.reset()


class Attention(Layer):
    """Scaled-dot-product attention over a ``(q, k, v)`` triple of (B, H, L, D) tensors."""

    def __init__(self, causal: bool = False, scale: float | None = None):
        self.causal = causal
        self.scale = scale
        self.x = None
        self.y = None
        self._lse = None

    def forward(self, x, training: bool = True) -> Tensor:
        q, k, v = x
        out, lse = attention_forward(q, k, v, self.scale, self.causal)
        self._lse = lse
        return out

    def backward(self, grad_y: Tensor):
        """Returns ``(dq, dk, dv)``, the gradient with respect to the cached input triple."""
        if self.x is None or self._lse is None:
            raise RuntimeError("Attention.backward called before forward")
        q, k, v = self.x
        return attention_backward(q, k, v, self.y, self._lse, grad_y, self.scale, self.causal)

    def parameters(self):
        return []

    def gradients(self):
        return []

    def reset(self):
        self.x = self.y = self._lse = None


class Linear(Layer):
    """``y = b + x @ w`` with w of shape (in_features, out_features), as the reference's Linear
    (ember/nn/layers.py:9-56). Weights start uniform in +-1/sqrt(in_features) and the bias at zero
    (layers.py:26-33); ``seed`` makes that reproducible."""

    def __init__(self, in_features: int, out_features: int, dtype: str = "float32", seed: int | None = None):
        self.in_features, self.out_features, self.dtype, self._seed = in_features, out_features, dtype, seed
        self.reset()

    def reset(self):
        self.x = self.y = None
        scale = 1.0 / math.sqrt(self.in_features)
        rng = np.random.default_rng(self._seed)
        self.w = Tensor(rng.uniform(-scale, scale, size=(self.in_features, self.out_features)).astype(np.float32), self.dtype)
        self.b = Tensor(np.zeros((self.out_features,), np.float32), self.dtype)
        self.grad_w = self.grad_b = None

    def parameters(self):
        return [self.w, self.b]

    def gradients(self):
        return [self.grad_w, self.grad_b]

    def forward(self, x: Tensor, training: bool = True) -> Tensor:
        self.x = x
        self.y = linear_forward(x, self.w, self.b)
        return self.y

    def backward(self, grad_y: Tensor) -> Tensor:
        assert self.x is not None, "forward() must run before backward()"
        grad_x, self.grad_w, self.grad_b = linear_backward(self.x, self.w, grad_y)
        return grad_x


class MultiHeadAttention(Layer):
    """Self-attention block over x of shape (B, L, E): q, k, v = split(x @ w_qkv + b_qkv) per head,
    attention, then the output projection. Parameters: w_qkv (E, 3E), b_qkv (3E), w_o (E, E), b_o (E).
    The q/k/v projection writes (3, B, H, L, D) and the output projection reads attention's
    (B, H, L, D) result as the (B*L, E) matrix, both inside the matrix-product kernels."""

    def __init__(self, embed_dim: int, num_heads: int, causal: bool = False, dtype: str = "float32",
                 seed: int | None = None):
        if embed_dim % num_heads:
            raise ValueError(f"embed_dim={embed_dim} is not a multiple of num_heads={num_heads}")
        self.embed_dim, self.num_heads, self.causal, self.dtype, self._seed = embed_dim, num_heads, causal, dtype, seed
        self.reset()

    def reset(self):
        e = self.embed_dim
        scale = 1.0 / math.sqrt(e)
        rng = np.random.default_rng(self._seed)
        mk = lambda shape: Tensor(rng.uniform(-scale, scale, size=shape).astype(np.float32), self.dtype)  # noqa: E731
        self.w_qkv, self.w_o = mk((e, 3 * e)), mk((e, e))
        self.b_qkv = Tensor(np.zeros((3 * e,), np.float32), self.dtype)
        self.b_o = Tensor(np.zeros((e,), np.float32), self.dtype)
        self.x = self.y = None
        self._qkv = self._o = self._lse = None
        self.grad_w_qkv = self.grad_b_qkv = self.grad_w_o = self.grad_b_o = None

    def parameters(self):
        return [self.w_qkv, self.b_qkv, self.w_o, self.b_o]

    def gradients(self):
        return [self.grad_w_qkv, self.grad_b_qkv, self.grad_w_o, self.grad_b_o]

    def _split(self, qkv: Tensor):
        _, B, H, L, D = qkv.shape
        n = B * H * L * D
        return tuple(qkv.view(i * n, (B, H, L, D)) for i in range(3))

    def forward(self, x: Tensor, training: bool = True) -> Tensor:
        if len(x.shape) != 3 or x.shape[-1] != self.embed_dim:
            raise ValueError(f"MultiHeadAttention expects (B, L, {self.embed_dim}), got {x.shape}")
        self.x = x
        self._qkv = linear_forward(x, self.w_qkv, self.b_qkv, y_heads=self.num_heads)
        q, k, v = self._split(self._qkv)
        self._o, self._lse = attention_forward(q, k, v, None, self.causal)
        self.y = linear_forward(self._o, self.w_o, self.b_o, x_heads=self.num_heads)
        return self.y

    def backward(self, grad_y: Tensor) -> Tensor:
        assert self.x is not None and self._o is not None, "forward() must run before backward()"
        H = self.num_heads
        grad_o, self.grad_w_o, self.grad_b_o = linear_backward(self._o, self.w_o, grad_y, x_heads=H)
        q, k, v = self._split(self._qkv)
        # the three gradients have to lie back to back, as the projection's (3, B, H, L, D) result does
        grad_qkv = Tensor.empty(self._qkv.shape, self._qkv.dtype)
        attention_backward(q, k, v, self._o, self._lse, grad_o, None, self.causal, into=self._split(grad_qkv))
        grad_x, self.grad_w_qkv, self.grad_b_qkv = linear_backward(self.x, self.w_qkv, grad_qkv, y_heads=H)
        return grad_x

    # ---- generation: the same block over a key/value cache -----------------------------------
    def prefill(self, x: Tensor, cache) -> Tensor:
        """forward(x) under the causal mask that also stores the keys and values of x's positions in
        ``cache`` (a ``KVCache`` with kv_heads == num_heads), ready for ``decode_step``."""
        if not self.causal:
            raise ValueError("prefill/decode_step need a causal MultiHeadAttention")
        y = self.forward(x, False)
        _, k, v = self._split(self._qkv)
        cache.append(k, v)
        return y

    def decode_step(self, x_t: Tensor, cache) -> Tensor:
        """One new position: x_t is (B, 1, E). Its key and value are appended to ``cache`` and its
        query attends over everything stored so far; returns (B, 1, E)."""
        if len(x_t.shape) != 3 or x_t.shape[1] != 1 or x_t.shape[2] != self.embed_dim:
            raise ValueError(f"decode_step expects (B, 1, {self.embed_dim}), got {x_t.shape}")
        B, H, D = x_t.shape[0], self.num_heads, self.embed_dim // self.num_heads
        qkv = linear_forward(x_t, self.w_qkv, self.b_qkv, y_heads=H)  # (3, B, H, 1, D)
        q, k, v = self._split(qkv)
        cache.append(k, v)
        o, _ = cache.decode(q.view(0, (B, H, D)))
        return linear_forward(o.view(0, (B, H, 1, D)), self.w_o, self.b_o, x_heads=H)
