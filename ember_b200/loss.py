"""Losses of the attention path's callers. ``CrossEntropyLoss`` follows the reference's class of that
name (ember/loss/losses.py:30-56: logits and one-hot targets of shape (batch, classes), the mean over
the batch, ``forward`` returns a Python float and caches the softmax for ``backward``) with the
eight-operator chain replaced by one fused kernel per direction.
"""
from __future__ import annotations

from . import _core
from .tensor import Tensor


class CrossEntropyLoss:
    def __init__(self) -> None:
        self.probs: Tensor | None = None
        self.target: Tensor | None = None
        self.n: int = 0

    def forward(self, pred: Tensor, target: Tensor) -> float:
        for name, t in (("pred", pred), ("target", target)):
            if not isinstance(t, Tensor):
                raise TypeError(f"CrossEntropyLoss: {name} must be a Tensor, got '{type(t).__name__}'")
        if len(pred.shape) != 2 or pred.shape != target.shape:
            raise ValueError(f"CrossEntropyLoss expects pred and target of one (batch, classes) shape, got {pred.shape} and {target.shape}")
        self.n = pred.shape[0]
        self.target = target
        loss, probs = _core._cross_entropy_fwd(pred._core, target._core, pred.shape[0], pred.shape[1])
        self.probs = Tensor._from_core(probs, pred.shape, pred.dtype)
        return float(Tensor._from_core(loss, (1,), "float32").to_np()[0])

    def __call__(self, pred: Tensor, target: Tensor) -> float:
        return self.forward(pred, target)

    def backward(self) -> Tensor:
        assert self.probs is not None, "forward() must run before backward()"
        assert self.target is not None, "forward() must run before backward()"
        g = _core._cross_entropy_bwd(self.probs._core, self.target._core, self.probs.shape[0], self.probs.shape[1])
        return Tensor._from_core(g, self.probs.shape, self.probs.dtype)
