"""Flat re-export of the native binding, as the reference does in ember/_core/__init__.py:1-55."""
from ._tensor import (BF16, F32, _attention_bwd, _attention_decode, _attention_fwd, _convert,  # noqa: F401
                      _cross_entropy_bwd, _cross_entropy_fwd, _decode_cache, _from_numpy, _kv_append, _linear_bwd,
                      _linear_fwd, _softmax, _sync, _Tensor)
