"""B200-native fused attention behind the reference's tensor / layer surface.

    import ember_b200 as em
    o = em.attention(em.Tensor(q), em.Tensor(k), em.Tensor(v), causal=True)
"""
from . import nn  # noqa: F401
from .tensor import (Tensor, attention, attention_backward, attention_decode,  # noqa: F401
                     attention_forward)

__all__ = ["Tensor", "attention", "attention_forward", "attention_backward", "attention_decode", "nn"]
