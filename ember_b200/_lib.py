"""Loader of the C-ABI CUDA library (``libember_b200.so``) and status -> exception mapping.

There is no CPU fallback: if the library is missing or CUDA is unusable the calls raise.
Exceptions follow the reference binding's conventions (src/tensor/tensor_api.c:196-199,
314-321: ValueError for shape/size mismatches; :28-31: MemoryError for failed allocation);
everything else the native layer reports becomes RuntimeError.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# EMBER_B200_LIB selects another build of the same library (the bounds-checked debug build, for one)
LIB_PATH = os.environ.get("EMBER_B200_LIB") or os.path.join(_HERE, "libember_b200.so")

EMBER_OK, EMBER_ERR_INVALID, EMBER_ERR_UNSUPPORTED, EMBER_ERR_CUDA = 0, 1, 2, 3
EMBER_ERR_TIMEOUT, EMBER_ERR_NOMEM, EMBER_ERR_WORKSPACE = 4, 5, 6
EMBER_F32, EMBER_BF16 = 0, 1
EMBER_OP_FWD, EMBER_OP_BWD, EMBER_OP_DECODE = 0, 1, 2

_vp, _i, _f, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t

SIGNATURES = {
    # name: (restype, argtypes) -- mirrors include/ember_b200.h
    "alloc_memory": (_vp, [_sz]),
    "free_memory": (None, [_vp]),
    "copy_to_device": (None, [_vp, _vp, _sz]),
    "copy_from_device": (None, [_vp, _vp, _sz]),
    "sync_device": (None, []),
    "ember_alloc_async": (_vp, [_sz, _vp]),
    "ember_free_async": (_i, [_vp, _vp]),
    "ember_pool_stats": (_i, [ctypes.POINTER(_sz), ctypes.POINTER(_sz)]),
    "ember_set_device": (_i, [_i]),
    "ember_get_device": (_i, [ctypes.POINTER(_i)]),
    "ember_stream": (_vp, []),
    "ember_f32_to_bf16": (_i, [_vp, _vp, _sz, _vp]),
    "ember_bf16_to_f32": (_i, [_vp, _vp, _sz, _vp]),
    "ember_status_string": (ctypes.c_char_p, [_i]),
    "ember_last_error": (ctypes.c_char_p, []),
    "ember_check_device_status": (_i, [_vp, ctypes.POINTER(_i)]),
    "ember_selftest_wait_timeout": (_i, [_vp]),
    "ember_attention_fwd": (_i, [_vp] * 5 + [_i] * 4 + [_f, _i, _i, _vp]),
    "ember_attention_bwd": (_i, [_vp] * 9 + [_i] * 4 + [_f, _i, _i, _vp, _sz, _vp]),
    "ember_set_deterministic": (_i, [_i]),
    "ember_get_deterministic": (_i, []),
    "ember_set_forward_block_rows": (_i, [_i]),
    "ember_attention_decode": (_i, [_vp] * 5 + [_i] * 3 + [_f, _i, _i, _vp, _sz, _vp]),
    "ember_attention_decode_static": (_i, [_vp] * 5 + [_i] * 3 + [_f, _i, _i, _vp]),
    "ember_attention_decode_static_capacity": (_sz, []),
    "ember_attention_workspace_bytes": (_sz, [_i] * 7),
    "ember_attention_decode_splits": (_i, [_i] * 4),
    "ember_attention_kernel_name": (ctypes.c_char_p, [_i] * 5),
    "ember_work_order_item": (_i, [_i, _i, _i, _sz, _i, _i, ctypes.POINTER(_i), ctypes.POINTER(_i)]),
    "ember_attention_fwd_host": (_i, [_vp] * 5 + [_i] * 4 + [ctypes.c_float, _i, _i]),
    "ember_comm_unique_id": (_i, [_vp]),
    "ember_comm_init": (_i, [ctypes.POINTER(_vp), _vp, _i, _i, _i]),
    "ember_comm_destroy": (_i, [_vp]),
    "ember_gather_outputs": (_i, [_vp, _vp, _sz, _vp, _vp]),
    "ember_linear_fwd": (_i, [_vp] * 4 + [ctypes.c_longlong] + [_i] * 7 + [_vp]),
    "ember_linear_bwd": (_i, [_vp] * 6 + [ctypes.c_longlong] + [_i] * 7 + [_vp]),
    "ember_linear_kernel_name": (ctypes.c_char_p, [_i, ctypes.c_longlong] + [_i] * 7),
    "ember_kv_cache_append": (_i, [_vp] * 4 + [_i] * 6 + [_vp, _vp, _i, _i, _i, _vp]),
    "ember_attention_decode_cache": (_i, [_vp] * 5 + [_i] * 6 + [ctypes.c_float, _i, _vp, _vp, _i, _i, _i, _vp, _sz, _vp]),
    "ember_attention_decode_cache_workspace_bytes": (_sz, [_i] * 6),
    "ember_attention_decode_cache_splits": (_i, [_i] * 3),
    "ember_softmax_fwd": (_i, [_vp, _vp, ctypes.c_longlong, _i, _i, _i, _vp]),
    "ember_cross_entropy_workspace_bytes": (_sz, [ctypes.c_longlong]),
    "ember_cross_entropy_fwd": (_i, [_vp] * 4 + [ctypes.c_longlong, _i, _i, _vp, _sz, _vp]),
    "ember_cross_entropy_bwd": (_i, [_vp] * 3 + [ctypes.c_longlong, _i, _i, _vp]),
}

_LIB = None


def lib() -> ctypes.CDLL:
    """The loaded library. Raises ImportError with build instructions if it is absent."""
    global _LIB
    if _LIB is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m ember_b200.build` "
                "(needs nvcc; there is no CPU fallback for the attention path)")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = L
    return _LIB


def last_error() -> str:
    return lib().ember_last_error().decode()


def check(status: int) -> None:
    """Raises the Python exception that corresponds to a non-zero ember_status."""
    if status == EMBER_OK:
        return
    L = lib()
    msg = f"{L.ember_status_string(status).decode()}: {last_error()}"
    if status == EMBER_ERR_INVALID:
        raise ValueError(msg)
    if status == EMBER_ERR_NOMEM:
        raise MemoryError(msg)
    raise RuntimeError(msg)
