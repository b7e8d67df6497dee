"""``Attention`` layer following the reference's manual-backward layer contract
(ember/nn/base.py:7-35: ``__call__`` caches input and output, ``forward``/``backward`` are
explicit, ``parameters``/``gradients``/``reset``), as ``Linear`` does for matmul
(ember/nn/layers.py:45-56). The layer has no parameters.
"""
from __future__ import annotations

from .tensor import Tensor, attention_backward, attention_forward


class Attention:
    """Scaled-dot-product attention over a ``(q, k, v)`` triple of (B, H, L, D) tensors."""

    def __init__(self, causal: bool = False, scale: float | None = None):
        self.causal = causal
        self.scale = scale
        self.x = None
        self.y = None
        self._lse = None

    def __call__(self, x, training: bool = False) -> Tensor:
        self.x = x
        self.y = self.forward(x, training)
        return self.y

    def forward(self, x, training: bool = False) -> Tensor:
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
