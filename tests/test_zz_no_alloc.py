"""GPU test of ember_attention_decode_static, the decode entry point for callers that must not
allocate device memory (for example a serving loop that owns the whole device through its own
arena, or a path on which an allocation would stall the device). It keeps the split partials in a
fixed array inside the library instead of a caller-supplied workspace.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test. The test also passes when run alone in a fresh process, where its first call is
the one that resolves the array's device address.
"""
import numpy as np
import pytest

import ember_b200 as em
from conftest import bf16_round, seeded
from ember_b200 import _lib

pytestmark = pytest.mark.gpu


def _decode_both(B, H, Lk, D, splits, seed):
    L = _lib.lib()
    q, k, v = (bf16_round(seeded((B, H, n, D), seed + i, 0.5)) for i, n in enumerate((1, Lk, Lk)))
    tq, tk, tv = (em.Tensor(x, "bfloat16") for x in (q, k, v))
    ref_out, ref_lse = em.attention_decode(tq, tk, tv, None, splits)   # existing entry point
    out = em.Tensor.empty(tq.shape, "bfloat16")
    lse = em.Tensor.empty(tq.shape[:-1], "float32")
    # the library stream, so that the call is ordered after the uploads above
    rc = L.ember_attention_decode_static(tq.ptr, tk.ptr, tv.ptr, out.ptr, lse.ptr, B * H, Lk, D,
                                         1.0 / np.sqrt(D), _lib.EMBER_BF16, splits, L.ember_stream())
    _lib.check(rc)
    return out.to_np(), lse.to_np(), ref_out.to_np(), ref_lse.to_np()


def test_static_scratch_decode_matches_workspace_decode_twice_in_a_row():
    # two calls in a row with different shapes: the second one finds the first one's partials in
    # the shared array and must not be disturbed by them
    for (B, H, Lk, D, splits, seed) in ((2, 4, 4096, 128, 8, 10), (1, 3, 3000, 64, 5, 20)):
        out, lse, ref_out, ref_lse = _decode_both(B, H, Lk, D, splits, seed)
        assert np.abs(out - ref_out).max() <= 2e-2
        assert np.abs(lse - ref_lse).max() <= 2e-2


def test_static_scratch_decode_rejects_oversized_requests():
    L = _lib.lib()
    cap = L.ember_attention_decode_static_capacity()
    assert cap == 4 << 20
    B, H, Lk, D = 1, 2, 1024, 128
    q, k, v = (em.Tensor(seeded((B, H, n, D), 1, 0.5), "bfloat16") for n in (1, Lk, Lk))
    out = em.Tensor.empty(q.shape, "bfloat16")
    # 2^20 (batch*head) rows x 2 splits would need far more than the built-in scratch: rejected
    # before anything is launched (the pointers are never read).
    rc = L.ember_attention_decode_static(q.ptr, k.ptr, v.ptr, out.ptr, None, 1 << 20, Lk, D, 0.1,
                                         _lib.EMBER_BF16, 2, L.ember_stream())
    assert rc == _lib.EMBER_ERR_WORKSPACE
    assert b"built-in scratch" in L.ember_last_error()
    # the library's own split choice always fits
    rc = L.ember_attention_decode_static(q.ptr, k.ptr, v.ptr, out.ptr, None, B * H, Lk, D, 0.1,
                                         _lib.EMBER_BF16, 0, L.ember_stream())
    assert rc == _lib.EMBER_OK
    L.sync_device()
