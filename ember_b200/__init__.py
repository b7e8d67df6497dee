"""B200-native fused attention behind the reference's tensor / layer surface.

    import ember_b200 as em
    o = em.attention(em.Tensor(q), em.Tensor(k), em.Tensor(v), causal=True)

The public names are resolved on first use, so that ``python -m ember_b200.build`` can run in a
fresh checkout before the native libraries exist. There is no CPU fallback: using any of them
without the built CUDA library raises ImportError with the build command.
"""
import importlib

__all__ = ["Tensor", "attention", "attention_forward", "attention_backward", "attention_decode", "linear_forward",
           "linear_backward", "softmax", "log_softmax", "KVCache", "nn", "loss"]

_TENSOR_NAMES = {"Tensor", "attention", "attention_forward", "attention_backward", "attention_decode", "linear_forward",
                 "linear_backward", "softmax", "log_softmax"}


def __getattr__(name):
    if name in _TENSOR_NAMES:
        try:
            mod = importlib.import_module(".tensor", __name__)
        except ImportError as e:
            raise ImportError(
                f"ember_b200 native libraries are not built ({e}); run `python -m ember_b200.build` "
                "(needs nvcc and gcc; there is no CPU fallback for the attention path)") from e
        return getattr(mod, name)
    if name == "KVCache":
        return importlib.import_module(".cache", __name__).KVCache
    if name in ("nn", "loss", "cache", "tensor", "shard", "_lib", "_core", "build"):
        return importlib.import_module("." + name, __name__)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
