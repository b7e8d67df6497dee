"""CPU-only: the C-ABI library loads and exports every symbol its header declares; host-side
argument validation mirrors the reference binding's exceptions. No compute call is made."""
import ctypes
import os
import re

import pytest

import ember_b200
from ember_b200 import _lib
from ember_b200.tensor import Tensor

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "ember_b200.h")).read()
    return re.findall(r"EMBER_API\s+[\w\s\*]+?\b(\w+)\s*\(", text)


def test_header_declares_the_attention_entry_points():
    names = _declared_symbols()
    for n in ("ember_attention_fwd", "ember_attention_bwd", "ember_attention_decode",
              "ember_attention_workspace_bytes", "alloc_memory", "free_memory", "copy_to_device",
              "copy_from_device", "sync_device"):
        assert n in names


def test_library_exports_every_declared_symbol():
    L = ctypes.CDLL(_lib.LIB_PATH)
    for n in _declared_symbols():
        assert hasattr(L, n), f"{n} declared in include/ember_b200.h but not exported"


def test_python_signatures_cover_the_header():
    assert set(_declared_symbols()) == set(_lib.SIGNATURES)


def test_status_strings():
    L = _lib.lib()
    assert L.ember_status_string(0) == b"ok"
    assert b"timed out" in L.ember_status_string(_lib.EMBER_ERR_TIMEOUT)


def test_workspace_sizes_need_no_gpu():
    L = _lib.lib()
    assert L.ember_attention_workspace_bytes(_lib.EMBER_OP_FWD, 8, 128, 128, 64, 0, 0) == 0
    assert L.ember_attention_workspace_bytes(_lib.EMBER_OP_BWD, 8, 128, 128, 64, 0, 0) >= 8 * 128 * 4
    one = L.ember_attention_workspace_bytes(_lib.EMBER_OP_DECODE, 8, 1, 4096, 128, 1, 1)
    four = L.ember_attention_workspace_bytes(_lib.EMBER_OP_DECODE, 8, 1, 4096, 128, 1, 4)
    assert one == 0 and four >= 8 * 4 * (128 + 2) * 4


def test_kernel_dispatch_names():
    L = _lib.lib()
    assert L.ember_attention_kernel_name(_lib.EMBER_OP_FWD, 4096, 4096, 128, _lib.EMBER_BF16) == b"sm100_tcgen05"
    assert L.ember_attention_kernel_name(_lib.EMBER_OP_FWD, 128, 128, 64, _lib.EMBER_F32) == b"simt_f32"
    # any multiple of 8 up to 128 runs on the tensor cores (zero-padded to 64 or 128 columns)
    assert L.ember_attention_kernel_name(_lib.EMBER_OP_FWD, 128, 128, 80, _lib.EMBER_BF16) == b"sm100_tcgen05"
    assert L.ember_attention_kernel_name(_lib.EMBER_OP_BWD, 128, 128, 24, _lib.EMBER_BF16) == b"sm100_tcgen05"
    assert L.ember_attention_kernel_name(_lib.EMBER_OP_FWD, 128, 128, 100, _lib.EMBER_BF16) == b"simt_f32"


def _fake(shape, dtype="float32"):
    return Tensor._from_core(None, shape, dtype)


def test_attention_rejects_non_tensor_operands():
    with pytest.raises(TypeError):
        ember_b200.attention(_fake((1, 1, 4, 8)), [[1.0]], _fake((1, 1, 4, 8)))


@pytest.mark.parametrize("qs,ks,vs", [
    ((1, 2, 4, 8), (1, 3, 4, 8), (1, 3, 4, 8)),   # batch dims differ
    ((1, 2, 4, 8), (1, 2, 4, 16), (1, 2, 4, 16)),  # head dim differs
    ((1, 2, 4, 8), (1, 2, 5, 8), (1, 2, 4, 8)),    # k/v lengths differ
    ((8,), (8,), (8,)),                            # rank < 2
])
def test_attention_rejects_mismatched_shapes(qs, ks, vs):
    with pytest.raises(ValueError):
        ember_b200.attention(_fake(qs), _fake(ks), _fake(vs))


def test_attention_rejects_mixed_dtypes():
    with pytest.raises(TypeError):
        ember_b200.attention(_fake((1, 1, 4, 8), "bfloat16"), _fake((1, 1, 4, 8)), _fake((1, 1, 4, 8)))


def test_decode_needs_one_query_row():
    with pytest.raises(ValueError):
        ember_b200.attention_decode(_fake((1, 1, 2, 8)), _fake((1, 1, 4, 8)), _fake((1, 1, 4, 8)))


def test_native_argument_checks_return_invalid_without_touching_the_gpu():
    L = _lib.lib()
    # negative extent and causal with lq > lk are rejected before any CUDA call
    assert L.ember_attention_fwd(1, 1, 1, 1, None, 1, -4, 4, 8, 1.0, 0, 0, None) == _lib.EMBER_ERR_INVALID
    assert L.ember_attention_fwd(16, 16, 16, 16, None, 1, 8, 4, 8, 1.0, 1, 0, None) == _lib.EMBER_ERR_INVALID
    assert b"lq <= lk" in L.ember_last_error()
    assert L.ember_attention_fwd(None, 16, 16, 16, None, 1, 4, 4, 8, 1.0, 0, 0, None) == _lib.EMBER_ERR_INVALID
    with pytest.raises(ValueError):
        _lib.check(_lib.EMBER_ERR_INVALID)
    with pytest.raises(MemoryError):
        _lib.check(_lib.EMBER_ERR_NOMEM)
    with pytest.raises(RuntimeError):
        _lib.check(_lib.EMBER_ERR_TIMEOUT)


def test_cpython_binding_surface_and_type_errors():
    import numpy as np

    from ember_b200 import _core

    for name in ("_Tensor", "_from_numpy", "_convert", "_attention_fwd", "_attention_bwd", "_attention_decode", "_sync"):
        assert hasattr(_core, name)
    assert (_core.F32, _core.BF16) == (_lib.EMBER_F32, _lib.EMBER_BF16)
    with pytest.raises(TypeError):  # "O!" parse failure, as in the reference binding
        _core._attention_fwd(1, 2, 3, 1, 1, 4, 4, 8, 1.0, 0)
    with pytest.raises(TypeError):  # only float32 host buffers are accepted (reference: format "f")
        _core._from_numpy(np.zeros(4, np.float64))
    with pytest.raises(ValueError):
        _core._from_numpy(np.zeros(4, np.float32), 7)


def test_work_order_visits_every_block_once_and_groups_units():
    """Host arithmetic of the CTA order: a bijection onto (unit, block rank); within a group the
    heaviest ranks come first; concurrently launched CTAs (consecutive indices) share few units."""
    import ctypes

    L = _lib.lib()
    u, r = ctypes.c_int(), ctypes.c_int()
    for units, blocks, touched, causal in ((128, 16, 4 << 20, 1), (128, 16, 4 << 20, 0), (64, 32, 8 << 20, 1),
                                           (7, 200, 100 << 20, 1), (149, 1, 64, 0), (13, 16, 2 << 20, 1), (1, 1, 1, 0)):
        seen, order = set(), []
        for idx in range(units * blocks):
            assert L.ember_work_order_item(units, blocks, 148, touched, causal, idx, ctypes.byref(u), ctypes.byref(r)) == 0
            assert 0 <= u.value < units and 0 <= r.value < blocks
            seen.add((u.value, r.value))
            order.append((u.value, r.value))
        assert len(seen) == units * blocks
        # a unit's blocks are taken heaviest first
        for unit in {0, units - 1}:
            ranks = [rk for (un, rk) in order if un == unit]
            assert ranks == sorted(ranks)
        if units * blocks >= 296:
            assert len({un for (un, _) in order[:148]}) <= max(148 // blocks + 1, (64 << 20) // max(touched, 1)) + 1
    assert L.ember_work_order_item(4, 4, 148, 1, 0, 16, ctypes.byref(u), ctypes.byref(r)) != 0
