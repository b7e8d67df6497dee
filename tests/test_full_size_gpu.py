"""GPU tests at the full sizes of the benchmark configurations. The CPU oracle is far too slow there (minutes per
(batch, head) slice), so parity is established in two ways: whole tensors against this library's
float32-arithmetic CUDA-core kernels (themselves pinned to the oracle and the golden vectors by the
small-shape tests), and one full (batch, head) slice against the CPU oracle."""
import ctypes
import math

import numpy as np
import pytest

from ember_b200 import _lib
from oracle import cpu_oracle

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _bf16(t):
    return t.to(torch.bfloat16)


def _rand(shape, seed, scale, dev):
    g = torch.Generator(device=dev).manual_seed(seed)
    return _bf16(torch.randn(shape, generator=g, device=dev) * scale)


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


def _fwd(L, sp, q, k, v, causal, dtype):
    BH, Lq, D = q.shape[0] * q.shape[1], q.shape[2], q.shape[3]
    Lk = k.shape[2]
    o = torch.empty_like(q)
    lse = torch.empty(q.shape[:3], device=q.device, dtype=torch.float32)
    _lib.check(L.ember_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), BH, Lq,
                                     Lk, D, 1.0 / math.sqrt(D), int(causal), dtype, sp))
    return o, lse


def _bwd(L, sp, q, k, v, o, lse, do, causal, dtype):
    BH, Lq, D = q.shape[0] * q.shape[1], q.shape[2], q.shape[3]
    Lk = k.shape[2]
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    n = L.ember_attention_workspace_bytes(_lib.EMBER_OP_BWD, BH, Lq, Lk, D, dtype, 0)
    ws = torch.empty(n, device=q.device, dtype=torch.uint8)
    _lib.check(L.ember_attention_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                     do.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), BH, Lq, Lk, D,
                                     1.0 / math.sqrt(D), int(causal), dtype, ws.data_ptr(), n, sp))
    return dq, dk, dv


def _no_fault(L, sp):
    where = ctypes.c_int(0)
    assert L.ember_check_device_status(sp, ctypes.byref(where)) == 0, where.value


def test_c2_causal_prefill_full_size(env):
    """B=4 H=32 L=4096 D=128 bf16 causal: tcgen05 kernel vs the float32-arithmetic kernel on the
    same bf16 inputs (float32 storage routes to the CUDA-core kernel), plus one slice vs the oracle."""
    L, dev, sp = env
    B, H, S, D = 4, 32, 4096, 128
    q, k, v = (_rand((B, H, S, D), s, 0.5, dev) for s in (1, 2, 3))
    o, lse = _fwd(L, sp, q, k, v, True, _lib.EMBER_BF16)
    of, lsef = _fwd(L, sp, q.float(), k.float(), v.float(), True, _lib.EMBER_F32)
    torch.cuda.synchronize()
    _no_fault(L, sp)
    assert torch.isfinite(o.float()).all()
    assert (o.float() - of).abs().max().item() <= 2e-2
    assert (lse - lsef).abs().max().item() <= 2e-2
    # the last (batch, head) slice against the CPU oracle
    qs, ks, vs = (t[-1, -1].float().cpu().numpy() for t in (q, k, v))
    ro, rl = cpu_oracle.attention_fwd(qs, ks, vs, None, True)
    assert np.abs(o[-1, -1].float().cpu().numpy() - ro).max() <= 2e-2
    assert np.abs(lse[-1, -1].cpu().numpy() - rl).max() <= 2e-2
    # property: with V = 1 every output is exactly 1 whatever the probabilities are
    ones = torch.ones_like(v)
    o1, _ = _fwd(L, sp, q, k, ones, True, _lib.EMBER_BF16)
    assert (o1.float() - 1.0).abs().max().item() <= 1e-2


def test_c3_causal_backward_full_size(env):
    """B=2 H=32 L=8192 D=128 bf16 causal: dQ/dK/dV of the tcgen05 kernels vs the float32-arithmetic
    kernels, tolerance 2e-2 of the largest reference magnitude per tensor."""
    L, dev, sp = env
    B, H, S, D = 2, 32, 8192, 128
    q, k, v = (_rand((B, H, S, D), s, 0.5, dev) for s in (4, 5, 6))
    do = _rand((B, H, S, D), 7, 1.0, dev)
    o, lse = _fwd(L, sp, q, k, v, True, _lib.EMBER_BF16)
    grads = _bwd(L, sp, q, k, v, o, lse, do, True, _lib.EMBER_BF16)
    qf, kf, vf, dof = q.float(), k.float(), v.float(), do.float()
    of, lsef = _fwd(L, sp, qf, kf, vf, True, _lib.EMBER_F32)
    refs = _bwd(L, sp, qf, kf, vf, of, lsef, dof, True, _lib.EMBER_F32)
    torch.cuda.synchronize()
    _no_fault(L, sp)
    for g, r, name in zip(grads, refs, ("dq", "dk", "dv")):
        err = (g.float() - r).abs().max().item()
        assert err <= 2e-2 * r.abs().max().item(), (name, err)
    # The last (batch, head) slice against the CPU oracle, on the rows the oracle can afford: the last
    # 512 query rows see every key, and under the causal mask the last 512 keys are seen by those
    # rows only. The oracle run on (those 512 queries, all 8192 keys) with the bottom-right aligned
    # mask therefore gives dQ of those rows and dK/dV of the last 512 keys of the full problem exactly
    # (about 5 Gflop on the host instead of 86 for the whole slice). The first 512 rows/keys likewise
    # give dQ[:512] from the oracle on the (512 x 512) top-left problem.
    R = 512
    qs, ks, vs, gs = (t[-1, -1].float().cpu().numpy() for t in (q, k, v, do))
    rdq, rdk, rdv = cpu_oracle.attention_bwd(qs[-R:], ks, vs, gs[-R:], None, True)
    got = [g[-1, -1].float().cpu().numpy() for g in grads]
    for name, a, b in (("dq", got[0][-R:], rdq), ("dk", got[1][-R:], rdk[-R:]), ("dv", got[2][-R:], rdv[-R:])):
        assert np.abs(a - b).max() <= 2e-2 * np.abs(b).max(), (name, np.abs(a - b).max(), np.abs(b).max())
    rdq0, _, _ = cpu_oracle.attention_bwd(qs[:R], ks[:R], vs[:R], gs[:R], None, True)
    assert np.abs(got[0][:R] - rdq0).max() <= 2e-2 * np.abs(rdq0).max()
    # linearity in dO: doubling the upstream gradient doubles every gradient bit for bit (scaling by
    # 2 is exact in every step), except where the value is a float32 denormal (around 1e-38: the first
    # causal rows, whose dS cancels to almost nothing)
    # That holds for dK and dV in both backward modes, and for dQ in the deterministic (two-kernel)
    # mode; the default single-pass kernel adds its dQ contributions in no fixed order, so there dQ is
    # linear to float32 rounding of the accumulator only.
    do2 = _bf16(do.float() * 2)
    g2 = _bwd(L, sp, q, k, v, o, lse, do2, True, _lib.EMBER_BF16)
    for name, a, b in zip(("dq", "dk", "dv"), grads, g2):
        a2 = _bf16(a.float() * 2)
        if name == "dq" and not L.ember_get_deterministic():
            # (rounding is relative to the partial sums, so the bound has a part relative to the largest value)
            af = a2.float()
            assert ((af - b.float()).abs() <= 2.0 ** -7 * af.abs() + 1e-3 * af.abs().max()).all()
            continue
        differs = a2 != b
        assert (b.float().abs()[differs] < 1e-30).all(), name
    before = L.ember_set_deterministic(1)
    try:
        d1 = _bwd(L, sp, q, k, v, o, lse, do, True, _lib.EMBER_BF16)
        d2 = _bwd(L, sp, q, k, v, o, lse, do2, True, _lib.EMBER_BF16)
        torch.cuda.synchronize()
    finally:
        L.ember_set_deterministic(before)
    for name, a, b, r in zip(("dq", "dk", "dv"), d1, d2, refs):
        assert ((a.float() - r).abs().max().item()) <= 2e-2 * r.abs().max().item(), name
        a2 = _bf16(a.float() * 2)
        differs = a2 != b
        assert (b.float().abs()[differs] < 1e-30).all(), name


def test_c5_long_sequence_units(env):
    """The multi-GPU sweep's longest shape (H=64 heads of D=128 at L=16384, bf16, causal), on three
    of its 128 (batch*head) units: forward and backward of the tcgen05 kernels against the
    float32-arithmetic kernels on all three (the first shape with more than 2^28 score elements per
    unit), and against the CPU oracle on the last 256 query rows / keys of the last unit."""
    L, dev, sp = env
    BH, S, D = 3, 16384, 128
    q, k, v = (_rand((1, BH, S, D), s, 0.5, dev) for s in (21, 22, 23))
    do = _rand((1, BH, S, D), 24, 1.0, dev)
    o, lse = _fwd(L, sp, q, k, v, True, _lib.EMBER_BF16)
    grads = _bwd(L, sp, q, k, v, o, lse, do, True, _lib.EMBER_BF16)
    qf, kf, vf, dof = q.float(), k.float(), v.float(), do.float()
    of, lsef = _fwd(L, sp, qf, kf, vf, True, _lib.EMBER_F32)
    refs = _bwd(L, sp, qf, kf, vf, of, lsef, dof, True, _lib.EMBER_F32)
    torch.cuda.synchronize()
    _no_fault(L, sp)
    assert (o.float() - of).abs().max().item() <= 2e-2
    assert (lse - lsef).abs().max().item() <= 2e-2
    for g, r, name in zip(grads, refs, ("dq", "dk", "dv")):
        err = (g.float() - r).abs().max().item()
        assert err <= 2e-2 * r.abs().max().item(), (name, err)
    R = 256
    qs, ks, vs, gs = (t[0, -1].float().cpu().numpy() for t in (q, k, v, do))
    ro, rl = cpu_oracle.attention_fwd(qs[-R:], ks, vs, None, True)
    assert np.abs(o[0, -1, -R:].float().cpu().numpy() - ro).max() <= 2e-2
    assert np.abs(lse[0, -1, -R:].cpu().numpy() - rl).max() <= 2e-2
    rdq, rdk, rdv = cpu_oracle.attention_bwd(qs[-R:], ks, vs, gs[-R:], None, True)
    got = [g[0, -1].float().cpu().numpy() for g in grads]
    for name, a, b in (("dq", got[0][-R:], rdq), ("dk", got[1][-R:], rdk[-R:]), ("dv", got[2][-R:], rdv[-R:])):
        assert np.abs(a - b).max() <= 2e-2 * np.abs(b).max(), (name, np.abs(a - b).max(), np.abs(b).max())


def test_c4_decode_full_size(env):
    """B=64 H=32 Lk=32768 D=128 bf16 decode (34 GB of cache): the library's split choice vs one
    split per row, and a sample of rows vs the CPU oracle."""
    L, dev, sp = env
    B, H, Lk, D = 64, 32, 32768, 128
    g = torch.Generator(device=dev).manual_seed(11)
    kc = torch.empty((B, H, Lk, D), device=dev, dtype=torch.bfloat16)
    vc = torch.empty((B, H, Lk, D), device=dev, dtype=torch.bfloat16)
    for t in (kc, vc):
        for b in range(B):
            t[b] = _bf16(torch.randn((H, Lk, D), generator=g, device=dev) * 0.5)
    q = _bf16(torch.randn((B, H, 1, D), generator=g, device=dev) * 0.5)

    def run(splits):
        o = torch.empty_like(q)
        lse = torch.empty((B, H), device=dev, dtype=torch.float32)
        n = L.ember_attention_workspace_bytes(_lib.EMBER_OP_DECODE, B * H, 1, Lk, D, 1, splits)
        ws = torch.empty(max(n, 256), device=dev, dtype=torch.uint8)
        _lib.check(L.ember_attention_decode(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                            B * H, Lk, D, 1.0 / math.sqrt(D), 1, splits, ws.data_ptr(), n, sp))
        torch.cuda.synchronize()
        return o, lse

    o_auto, l_auto = run(0)
    o_one, l_one = run(1)
    assert (o_auto.float() - o_one.float()).abs().max().item() <= 1e-2
    assert (l_auto - l_one).abs().max().item() <= 1e-4
    for (b, h) in ((0, 0), (63, 31), (17, 5)):
        ro, rl = cpu_oracle.attention_fwd(q[b, h].float().cpu().numpy(), kc[b, h].float().cpu().numpy(),
                                          vc[b, h].float().cpu().numpy(), None, False)
        assert np.abs(o_auto[b, h].float().cpu().numpy() - ro).max() <= 2e-2
        assert abs(float(l_auto[b, h]) - float(rl[0])) <= 2e-2
