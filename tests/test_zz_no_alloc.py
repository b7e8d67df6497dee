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
from oracle import cpu_oracle

pytestmark = pytest.mark.gpu


def _decode_both(B, H, Lk, D, splits, seed, dtype="bfloat16", stream="library"):
    L = _lib.lib()
    rnd = bf16_round if dtype == "bfloat16" else (lambda x: x)
    q, k, v = (rnd(seeded((B, H, n, D), seed + i, 0.5)) for i, n in enumerate((1, Lk, Lk)))
    tq, tk, tv = (em.Tensor(x, dtype) for x in (q, k, v))
    ref_out, ref_lse = em.attention_decode(tq, tk, tv, None, splits)   # existing entry point
    out = em.Tensor.empty(tq.shape, dtype)
    lse = em.Tensor.empty(tq.shape[:-1], "float32")
    if stream == "library":
        sp = L.ember_stream()      # ordered after the uploads above
    else:
        L.sync_device()            # NULL means the CUDA default stream here: the uploads must be done
        sp = None
    rc = L.ember_attention_decode_static(tq.ptr, tk.ptr, tv.ptr, out.ptr, lse.ptr, B * H, Lk, D,
                                         1.0 / np.sqrt(D), _lib.EMBER_BF16 if dtype == "bfloat16" else _lib.EMBER_F32,
                                         splits, sp)
    _lib.check(rc)
    if stream != "library":
        import ctypes
        cudart = ctypes.CDLL("libcudart.so.12")
        assert cudart.cudaDeviceSynchronize() == 0
    oracle_out, oracle_lse = cpu_oracle.attention_fwd(q, k, v, None, False)
    return out.to_np(), lse.to_np(), ref_out.to_np(), ref_lse.to_np(), oracle_out, oracle_lse


def test_static_scratch_decode_matches_workspace_decode_twice_in_a_row():
    # two calls in a row with different shapes: the second one finds the first one's partials in
    # the shared array and must not be disturbed by them. The same kernel with the same split count
    # runs behind both entry points, so the results are equal bit for bit; the oracle comparison is
    # at the tolerance of the storage type.
    for (B, H, Lk, D, splits, seed, dtype, tol) in ((2, 4, 4096, 128, 8, 10, "bfloat16", 2e-2),
                                                    (1, 3, 3000, 64, 5, 20, "bfloat16", 2e-2),
                                                    (2, 2, 2000, 64, 4, 30, "float32", 1e-3)):
        out, lse, ref_out, ref_lse, o_out, o_lse = _decode_both(B, H, Lk, D, splits, seed, dtype)
        assert np.array_equal(out, ref_out) and np.array_equal(lse, ref_lse)
        assert np.abs(out - o_out).max() <= tol and np.abs(lse - o_lse).max() <= tol


def test_static_scratch_decode_on_the_default_stream():
    out, lse, ref_out, ref_lse, o_out, o_lse = _decode_both(1, 4, 2048, 128, 4, 40, "bfloat16", stream="default")
    assert np.array_equal(out, ref_out) and np.array_equal(lse, ref_lse)
    assert np.abs(out - o_out).max() <= 2e-2


def test_static_scratch_decode_shrinks_its_own_split_choice_to_fit():
    # 4100 (batch*head) rows of d=128 over 600 keys: the library's split choice for the workspace
    # entry point (2 here) would need 4.1 MiB of partials, just more than the built-in 4 MiB, so the
    # static entry point lowers it; the VALUES must still be right. Inputs are made on the device
    # (torch) to keep the host out of it.
    torch = pytest.importorskip("torch")
    import ctypes
    L = _lib.lib()
    _lib.check(L.ember_set_device(0))
    BH, Lk, D = 4100, 600, 128
    cap = L.ember_attention_decode_static_capacity()
    auto = L.ember_attention_decode_splits(BH, Lk, D, _lib.EMBER_BF16)
    assert L.ember_attention_workspace_bytes(_lib.EMBER_OP_DECODE, BH, 1, Lk, D, _lib.EMBER_BF16, auto) > cap
    g = torch.Generator(device="cuda").manual_seed(50)
    q = (torch.randn((BH, 1, D), generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    k = (torch.randn((BH, Lk, D), generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    v = (torch.randn((BH, Lk, D), generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    out = torch.empty_like(q)
    lse = torch.empty((BH,), device="cuda", dtype=torch.float32)
    s = torch.cuda.Stream()
    torch.cuda.synchronize()
    _lib.check(L.ember_attention_decode_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), BH,
                                               Lk, D, 1.0 / np.sqrt(D), _lib.EMBER_BF16, 0, ctypes.c_void_p(s.cuda_stream)))
    s.synchronize()
    assert torch.isfinite(out.float()).all()
    for r in (0, 4099, 2050):
        ro, rl = cpu_oracle.attention_fwd(q[r].float().cpu().numpy(), k[r].float().cpu().numpy(), v[r].float().cpu().numpy(),
                                          None, False)
        assert np.abs(out[r].float().cpu().numpy() - ro).max() <= 2e-2 and abs(float(lse[r]) - float(rl[0])) <= 2e-2


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
