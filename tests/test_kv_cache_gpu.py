"""GPU parity of the key/value cache entry points: append in place, decode over a partly filled
cache with per-sequence lengths, grouped-query heads and a page table, against the CPU oracle run on
the equivalent dense problem (K/V heads repeated per query head, cut to each sequence's length)."""
import ctypes
import math

import numpy as np
import pytest

from ember_b200 import _lib
from oracle import cpu_oracle

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def env():
    if not torch.cuda.is_available():
        pytest.skip("needs CUDA")
    L = _lib.lib()
    _lib.check(L.ember_set_device(0))
    dev = torch.device("cuda", 0)
    s = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(s)
    return L, dev, ctypes.c_void_p(s.cuda_stream)


def _t(a, dev, bf16):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    return t.to(torch.bfloat16) if bf16 else t


def _round(a, bf16):
    return torch.from_numpy(a).to(torch.bfloat16).float().numpy() if bf16 else a


def _ptr(t):
    return t.data_ptr() if t is not None else None


def _oracle(q, k, v, lens, group):
    """q (B, Hq, D); k, v (B, Hkv, cap, D) dense; returns out (B, Hq, D), lse (B, Hq)."""
    B, Hq, D = q.shape
    out, lse = np.empty_like(q), np.empty((B, Hq), np.float32)
    for b in range(B):
        n = int(lens[b])
        for h in range(Hq):
            o, l = cpu_oracle.attention_fwd(q[b, h][None, :], k[b, h // group, :n], v[b, h // group, :n], None, False)
            out[b, h], lse[b, h] = o[0], l[0]
    return out, lse


def _decode(L, sp, dev, q, kc, vc, B, Hq, Hkv, lk, cap, D, bf16, lens=None, table=None, page=0, max_blocks=0, splits=0):
    dt = _lib.EMBER_BF16 if bf16 else _lib.EMBER_F32
    out = torch.empty_like(q)
    lse = torch.empty((B, Hq), device=dev, dtype=torch.float32)
    n = L.ember_attention_decode_cache_workspace_bytes(B, Hq, Hkv, lk, D, splits)
    ws = torch.empty(max(n, 256), device=dev, dtype=torch.uint8)
    _lib.check(L.ember_attention_decode_cache(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), lse.data_ptr(), B,
                                              Hq, Hkv, lk, cap, D, 1.0 / math.sqrt(D), dt, _ptr(lens), _ptr(table), page,
                                              max_blocks, splits, ws.data_ptr(), n, sp))
    torch.cuda.synchronize()
    where = ctypes.c_int(0)
    assert L.ember_check_device_status(sp, ctypes.byref(where)) == 0, where.value
    return out.float().cpu().numpy(), lse.cpu().numpy()


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("cfg", [
    # B, Hq, Hkv, capacity, D, splits
    (2, 4, 4, 300, 64, 0),
    (2, 8, 4, 700, 128, 3),
    (3, 8, 2, 1100, 128, 0),
    (1, 16, 2, 520, 64, 2),
    (2, 6, 3, 90, 32, 1),
])
def test_decode_over_cache_with_lengths_and_groups(env, cfg, bf16):
    L, dev, sp = env
    B, Hq, Hkv, cap, D, splits = cfg
    group = Hq // Hkv
    rng = np.random.default_rng(cap + D + Hq)
    q = _round(rng.standard_normal((B, Hq, D), dtype=np.float32) * 0.5, bf16)
    k = _round(rng.standard_normal((B, Hkv, cap, D), dtype=np.float32) * 0.5, bf16)
    v = _round(rng.standard_normal((B, Hkv, cap, D), dtype=np.float32) * 0.5, bf16)
    lens = np.array([max(1, cap - 37 * b - 5) for b in range(B)], np.int32)
    tq, tk, tv = _t(q, dev, bf16), _t(k, dev, bf16), _t(v, dev, bf16)
    tl = torch.from_numpy(lens).to(dev)
    tol = 2e-2 if bf16 else 1e-3
    ro, rl = _oracle(q, k, v, lens, group)
    o, l = _decode(L, sp, dev, tq, tk, tv, B, Hq, Hkv, cap, cap, D, bf16, lens=tl, splits=splits)
    assert np.abs(o - ro).max() <= tol and np.abs(l - rl).max() <= tol
    # without seq_lens every sequence uses lk keys
    lk = cap - 3
    ro, rl = _oracle(q, k, v, np.full(B, lk), group)
    o, l = _decode(L, sp, dev, tq, tk, tv, B, Hq, Hkv, lk, cap, D, bf16, splits=splits)
    assert np.abs(o - ro).max() <= tol and np.abs(l - rl).max() <= tol


@pytest.mark.parametrize("bf16", [False, True])
def test_append_then_decode_matches_dense(env, bf16):
    """Fill a cache in three appends (one with per-sequence positions), then decode."""
    L, dev, sp = env
    B, Hq, Hkv, cap, D = 2, 8, 2, 256, 128
    dt = _lib.EMBER_BF16 if bf16 else _lib.EMBER_F32
    rng = np.random.default_rng(3)
    k_full = _round(rng.standard_normal((B, Hkv, 200, D), dtype=np.float32) * 0.5, bf16)
    v_full = _round(rng.standard_normal((B, Hkv, 200, D), dtype=np.float32) * 0.5, bf16)
    td = torch.bfloat16 if bf16 else torch.float32
    kc = torch.zeros((B, Hkv, cap, D), device=dev, dtype=td)
    vc = torch.zeros_like(kc)
    pos = 0
    for n_new in (128, 71):
        kn, vn = (_t(np.ascontiguousarray(a[:, :, pos:pos + n_new]), dev, bf16) for a in (k_full, v_full))
        _lib.check(L.ember_kv_cache_append(kc.data_ptr(), vc.data_ptr(), kn.data_ptr(), vn.data_ptr(), B, Hkv, cap, D, n_new,
                                           pos, None, None, 0, 0, dt, sp))
        pos += n_new
    lens = torch.full((B,), pos, device=dev, dtype=torch.int32)
    kn, vn = (_t(np.ascontiguousarray(a[:, :, pos:pos + 1]), dev, bf16) for a in (k_full, v_full))
    _lib.check(L.ember_kv_cache_append(kc.data_ptr(), vc.data_ptr(), kn.data_ptr(), vn.data_ptr(), B, Hkv, cap, D, 1, 0, lens.data_ptr(),
                                       None, 0, 0, dt, sp))
    torch.cuda.synchronize()
    assert np.array_equal(kc[:, :, :200].float().cpu().numpy(), k_full)
    assert np.array_equal(vc[:, :, :200].float().cpu().numpy(), v_full)
    assert float(kc[:, :, 200:].float().abs().max()) == 0.0
    q = _round(rng.standard_normal((B, Hq, D), dtype=np.float32) * 0.5, bf16)
    o, l = _decode(L, sp, dev, _t(q, dev, bf16), kc, vc, B, Hq, Hkv, 200, cap, D, bf16)
    ro, rl = _oracle(q, k_full, v_full, np.full(B, 200), Hq // Hkv)
    tol = 2e-2 if bf16 else 1e-3
    assert np.abs(o - ro).max() <= tol and np.abs(l - rl).max() <= tol
    # a row that does not fit is reported, not written
    with pytest.raises(ValueError):
        _lib.check(L.ember_kv_cache_append(kc.data_ptr(), vc.data_ptr(), kn.data_ptr(), vn.data_ptr(), B, Hkv, cap, D, 1, cap,
                                           None, None, 0, 0, dt, sp))


@pytest.mark.parametrize("bf16", [False, True])
def test_paged_cache(env, bf16):
    L, dev, sp = env
    B, Hq, Hkv, D, page, max_blocks = 2, 8, 4, 128, 16, 20
    dt = _lib.EMBER_BF16 if bf16 else _lib.EMBER_F32
    rng = np.random.default_rng(9)
    lens = np.array([300, 171], np.int32)
    num_pages = B * max_blocks + 3
    perm = rng.permutation(num_pages)[:B * max_blocks].astype(np.int32).reshape(B, max_blocks)
    k = _round(rng.standard_normal((B, Hkv, page * max_blocks, D), dtype=np.float32) * 0.5, bf16)
    v = _round(rng.standard_normal((B, Hkv, page * max_blocks, D), dtype=np.float32) * 0.5, bf16)
    td = torch.bfloat16 if bf16 else torch.float32
    kp = torch.zeros((num_pages, Hkv, page, D), device=dev, dtype=td)
    vp = torch.zeros_like(kp)
    table = torch.from_numpy(perm).to(dev)
    # fill through the append entry point: 4 chunks per sequence starting at position 0
    pos = 0
    for n_new in (100, 100, 100, 20):
        kn, vn = (_t(np.ascontiguousarray(a[:, :, pos:pos + n_new]), dev, bf16) for a in (k, v))
        _lib.check(L.ember_kv_cache_append(kp.data_ptr(), vp.data_ptr(), kn.data_ptr(), vn.data_ptr(), B, Hkv, 0, D, n_new, pos,
                                           None, table.data_ptr(), page, max_blocks, dt, sp))
        pos += n_new
    q = _round(rng.standard_normal((B, Hq, D), dtype=np.float32) * 0.5, bf16)
    tl = torch.from_numpy(lens).to(dev)
    o, l = _decode(L, sp, dev, _t(q, dev, bf16), kp, vp, B, Hq, Hkv, 320, 0, D, bf16, lens=tl, table=table, page=page,
                   max_blocks=max_blocks, splits=2)
    ro, rl = _oracle(q, k, v, lens, Hq // Hkv)
    tol = 2e-2 if bf16 else 1e-3
    assert np.abs(o - ro).max() <= tol and np.abs(l - rl).max() <= tol


def test_group_of_one_equals_plain_decode(env):
    """q_heads == kv_heads and a full contiguous cache is ember_attention_decode's problem."""
    L, dev, sp = env
    B, H, lk, D = 2, 4, 777, 128
    g = torch.Generator(device=dev).manual_seed(1)
    q = (torch.randn((B, H, D), generator=g, device=dev) * 0.5).to(torch.bfloat16)
    k = (torch.randn((B, H, lk, D), generator=g, device=dev) * 0.5).to(torch.bfloat16)
    v = (torch.randn((B, H, lk, D), generator=g, device=dev) * 0.5).to(torch.bfloat16)
    o1, l1 = _decode(L, sp, dev, q, k, v, B, H, H, lk, lk, D, True)
    out = torch.empty_like(q)
    lse = torch.empty((B, H), device=dev, dtype=torch.float32)
    n = L.ember_attention_workspace_bytes(_lib.EMBER_OP_DECODE, B * H, 1, lk, D, 1, 0)
    ws = torch.empty(max(n, 256), device=dev, dtype=torch.uint8)
    _lib.check(L.ember_attention_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(), B * H, lk, D,
                                        1.0 / math.sqrt(D), 1, 0, ws.data_ptr(), n, sp))
    torch.cuda.synchronize()
    assert np.abs(o1 - out.float().cpu().numpy()).max() <= 1e-2
    assert np.abs(l1 - lse.cpu().numpy()).max() <= 1e-4


def test_unsupported_group_is_reported(env):
    L, dev, sp = env
    t = torch.zeros(4096, device=dev)
    with pytest.raises(RuntimeError):
        _lib.check(L.ember_attention_decode_cache(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), None, 1, 3, 1, 8, 8, 8,
                                                  1.0, _lib.EMBER_F32, None, None, 0, 0, 1, None, 0, sp))
    with pytest.raises(ValueError):
        _lib.check(L.ember_attention_decode_cache(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), None, 1, 3, 2, 8, 8, 8,
                                                  1.0, _lib.EMBER_F32, None, None, 0, 0, 1, None, 0, sp))


@pytest.mark.parametrize("cfg", [
    # B, Hq, Hkv, capacity, D, splits: grouped heads (tensor-core path for bf16) and one head per K/V head
    (2, 8, 2, 700, 128, 0),
    (2, 8, 2, 700, 128, 3),
    (3, 4, 4, 520, 64, 2),
])
def test_cache_rows_past_the_sequence_length_are_never_used(env, cfg):
    """The rows of a cache beyond seq_lens[b] were never written by the caller and may hold anything.
    Here they hold bf16 NaN and Inf bit patterns (written by the host; nothing faults): the result
    must be finite and equal to the oracle's on the filled part, on both kernel families."""
    L, dev, sp = env
    B, Hq, Hkv, cap, D, splits = cfg
    rng = np.random.default_rng(17 + cap + Hq)
    q = _round(rng.standard_normal((B, Hq, D), dtype=np.float32) * 0.5, True)
    k = _round(rng.standard_normal((B, Hkv, cap, D), dtype=np.float32) * 0.5, True)
    v = _round(rng.standard_normal((B, Hkv, cap, D), dtype=np.float32) * 0.5, True)
    lens = np.array([cap - 150 * b - 61 for b in range(B)], np.int32)   # none a multiple of 128
    tq, tk, tv = _t(q, dev, True), _t(k, dev, True), _t(v, dev, True)
    for b in range(B):
        n = int(lens[b])
        tk[b, :, n:] = float("nan")
        tv[b, :, n::2] = float("inf")
        tv[b, :, n + 1::2] = float("nan")
    tl = torch.from_numpy(lens).to(dev)
    ro, rl = _oracle(q, k, v, lens, Hq // Hkv)
    o, l = _decode(L, sp, dev, tq, tk, tv, B, Hq, Hkv, cap, cap, D, True, lens=tl, splits=splits)
    assert np.isfinite(o).all() and np.isfinite(l).all()
    assert np.abs(o - ro).max() <= 2e-2 and np.abs(l - rl).max() <= 2e-2


@pytest.mark.parametrize("cfg", [(2, 8, 2, 400, 128, 0), (2, 8, 2, 400, 128, 2), (2, 4, 4, 400, 64, 0), (2, 4, 4, 400, 64, 3)])
def test_an_empty_sequence_gives_zeros_and_minus_infinity(env, cfg):
    """seq_lens[b] == 0: that sequence's output rows are zeros and its lse is -inf; the others are
    unaffected."""
    L, dev, sp = env
    B, Hq, Hkv, cap, D, splits = cfg
    rng = np.random.default_rng(5)
    q = _round(rng.standard_normal((B, Hq, D), dtype=np.float32) * 0.5, True)
    k = _round(rng.standard_normal((B, Hkv, cap, D), dtype=np.float32) * 0.5, True)
    v = _round(rng.standard_normal((B, Hkv, cap, D), dtype=np.float32) * 0.5, True)
    lens = np.array([0, cap - 7], np.int32)
    tl = torch.from_numpy(lens).to(dev)
    o, l = _decode(L, sp, dev, _t(q, dev, True), _t(k, dev, True), _t(v, dev, True), B, Hq, Hkv, cap, cap, D, True, lens=tl,
                   splits=splits)
    assert (o[0] == 0).all() and np.isneginf(l[0]).all()
    ro, rl = _oracle(q[1:], k[1:], v[1:], lens[1:], Hq // Hkv)
    assert np.abs(o[1:] - ro).max() <= 2e-2 and np.abs(l[1:] - rl).max() <= 2e-2


def test_decode_with_more_than_65535_batch_heads(env):
    """batch*heads = 70 000 rows (a grid dimension of its own would stop at 65 535): sampled rows
    against the oracle, all rows finite."""
    L, dev, sp = env
    BH, Lk, D = 70000, 512, 64
    g = torch.Generator(device=dev).manual_seed(9)
    q = (torch.randn((BH, 1, D), generator=g, device=dev) * 0.5).to(torch.bfloat16)
    k = (torch.randn((BH, Lk, D), generator=g, device=dev) * 0.5).to(torch.bfloat16)
    v = (torch.randn((BH, Lk, D), generator=g, device=dev) * 0.5).to(torch.bfloat16)
    for splits in (1, 2):
        o = torch.empty_like(q)
        lse = torch.empty((BH,), device=dev, dtype=torch.float32)
        n = L.ember_attention_workspace_bytes(_lib.EMBER_OP_DECODE, BH, 1, Lk, D, 1, splits)
        ws = torch.empty(max(n, 256), device=dev, dtype=torch.uint8)
        _lib.check(L.ember_attention_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), BH, Lk, D,
                                            1.0 / math.sqrt(D), 1, splits, ws.data_ptr(), n, sp))
        torch.cuda.synchronize()
        assert torch.isfinite(o.float()).all() and torch.isfinite(lse).all()
        for r in (0, 65535, 65536, 69999):
            ro, rl = cpu_oracle.attention_fwd(q[r].float().cpu().numpy(), k[r].float().cpu().numpy(), v[r].float().cpu().numpy(),
                                              None, False)
            assert np.abs(o[r].float().cpu().numpy() - ro).max() <= 2e-2
            assert abs(float(lse[r]) - float(rl[0])) <= 2e-2
