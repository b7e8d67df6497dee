"""CPU-only: pins the C oracle against the reference's golden vectors, against the reference's
own compiled operators (when that build is present) and against float64 NumPy."""
import numpy as np
import pytest

from conftest import golden_inputs, linear_golden_inputs, seeded, softmax_golden_inputs
from oracle import cpu_oracle, ref_ops

CASES = ["c1_fwd_f32", "c1_causal", "ragged_causal", "ragged_noncausal", "decode", "d128"]


@pytest.mark.parametrize("name", CASES)
def test_oracle_matches_golden_bit_for_bit(golden, name):
    meta = golden[name + "/meta"]
    has_bwd = (name + "/dq") in golden.files
    (q, k, v, *rest), causal = golden_inputs(meta, with_dout=has_bwd)
    scale = float(golden[name + "/scale"])
    out, lse = cpu_oracle.attention_fwd(q, k, v, scale, causal)
    assert np.array_equal(out, golden[name + "/out"])
    np.testing.assert_allclose(lse, golden[name + "/lse"], rtol=0, atol=2e-6)
    if has_bwd:
        dq, dk, dv = cpu_oracle.attention_bwd(q, k, v, rest[0], scale, causal)
        assert np.array_equal(dq, golden[name + "/dq"])
        assert np.array_equal(dk, golden[name + "/dk"])
        assert np.array_equal(dv, golden[name + "/dv"])


@pytest.mark.skipif(not ref_ops.available(), reason="oracle/_ref not built (needs the reference checkout)")
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(2, 2, 64, 64, 64), (1, 3, 17, 33, 32), (1, 1, 1, 50, 16), (1, 2, 40, 72, 128)])
def test_oracle_matches_compiled_reference_ops(shape, causal):
    B, H, Lq, Lk, D = shape
    q, k, v, g = (seeded((B, H, L, D), s) for L, s in ((Lq, 1), (Lk, 2), (Lk, 3), (Lq, 4)))
    o1, l1 = cpu_oracle.attention_fwd(q, k, v, None, causal)
    o2, l2 = ref_ops.attention_fwd(q, k, v, None, causal)
    assert np.array_equal(o1, o2) and np.array_equal(l1, l2)
    for a, b in zip(cpu_oracle.attention_bwd(q, k, v, g, None, causal), ref_ops.attention_bwd(q, k, v, g, None, causal)):
        assert np.array_equal(a, b)


def _f64_attention(q, k, v, g, scale, causal):
    q, k, v, g = (x.astype(np.float64) for x in (q, k, v, g))
    s = np.einsum("...id,...jd->...ij", q, k) * scale
    if causal:
        Lq, Lk = s.shape[-2:]
        i, j = np.arange(Lq)[:, None], np.arange(Lk)[None, :]
        s = np.where(j > i + (Lk - Lq), -np.inf, s)
    m = s.max(-1, keepdims=True)
    e = np.exp(s - m)
    l = e.sum(-1, keepdims=True)
    p = e / l
    o = p @ v
    dv = np.swapaxes(p, -1, -2) @ g
    dp = g @ np.swapaxes(v, -1, -2)
    ds = p * (dp - (dp * p).sum(-1, keepdims=True)) * scale
    return o, (m + np.log(l))[..., 0], ds @ k, np.swapaxes(ds, -1, -2) @ q, dv


@pytest.mark.parametrize("causal", [False, True])
def test_oracle_close_to_float64(causal):
    B, H, Lq, Lk, D = 1, 2, 96, 160, 64
    q, k, v, g = (seeded((B, H, L, D), s) for L, s in ((Lq, 11), (Lk, 12), (Lk, 13), (Lq, 14)))
    scale = 1.0 / np.sqrt(D)
    o, lse = cpu_oracle.attention_fwd(q, k, v, scale, causal)
    dq, dk, dv = cpu_oracle.attention_bwd(q, k, v, g, scale, causal)
    ro, rl, rdq, rdk, rdv = _f64_attention(q, k, v, g, scale, causal)
    for a, b in ((o, ro), (lse, rl), (dq, rdq), (dk, rdk), (dv, rdv)):
        assert np.abs(a - b).max() < 2e-6


def test_oracle_threads_do_not_change_bits():
    q, k, v = (seeded((2, 3, 40, 32), s) for s in (1, 2, 3))
    a = cpu_oracle.attention_fwd(q, k, v, None, True)[0]
    cpu_oracle.set_threads(4)
    try:
        b = cpu_oracle.attention_fwd(q, k, v, None, True)[0]
    finally:
        cpu_oracle.set_threads(1)
    assert np.array_equal(a, b)


LINEAR_CASES = ["lin_small", "lin_tile", "lin_ragged", "lin_nobias"]


@pytest.mark.parametrize("name", LINEAR_CASES)
def test_linear_oracle_matches_golden_bit_for_bit(linear_golden, name):
    """The golden file was produced by the reference's own Linear layer (forward, backward, gradients)."""
    x, w, b, dy = linear_golden_inputs(linear_golden[name + "/meta"])
    y = cpu_oracle.linear_fwd(x, w, b)
    assert np.array_equal(y, linear_golden[name + "/y"])
    dx, dw, db = cpu_oracle.linear_bwd(x, w, dy)
    assert np.array_equal(dx, linear_golden[name + "/gx"])
    assert np.array_equal(dw, linear_golden[name + "/gw"])
    assert np.array_equal(db, linear_golden[name + "/gb"])


@pytest.mark.skipif(not ref_ops.available(), reason="oracle/_ref not built (needs the reference checkout)")
@pytest.mark.parametrize("mkn", [(1, 1, 1), (33, 65, 17), (64, 128, 96)])
def test_linear_oracle_matches_compiled_reference_ops(mkn):
    m, k, n = mkn
    x, w, b, dy = seeded((m, k), 1), seeded((k, n), 2, 0.1), seeded((n,), 3), seeded((m, n), 4)
    assert np.array_equal(cpu_oracle.linear_fwd(x, w, b), ref_ops.linear_fwd(x, w, b))
    for a, c in zip(cpu_oracle.linear_bwd(x, w, dy), ref_ops.linear_bwd(x, w, dy)):
        assert np.array_equal(a, c)


@pytest.mark.parametrize("name", ["sm_small", "sm_ragged", "sm_wide"])
def test_softmax_and_cross_entropy_oracle_match_golden_bit_for_bit(softmax_golden, name):
    """The golden file holds em.softmax and the reference's CrossEntropyLoss (loss, cached probs, gradient)."""
    x, target = softmax_golden_inputs(softmax_golden[name + "/meta"])
    assert np.array_equal(cpu_oracle.softmax(x), softmax_golden[name + "/softmax"])
    loss, probs = cpu_oracle.cross_entropy_fwd(x, target)
    assert loss == float(softmax_golden[name + "/loss"])
    assert np.array_equal(probs, softmax_golden[name + "/probs"])
    assert np.array_equal(cpu_oracle.cross_entropy_bwd(probs, target), softmax_golden[name + "/grad"])


@pytest.mark.skipif(not ref_ops.available(), reason="oracle/_ref not built (needs the reference checkout)")
def test_softmax_and_cross_entropy_oracle_match_compiled_reference_ops():
    x = seeded((40, 257), 9, 3.0)
    target = np.zeros_like(x)
    target[np.arange(40), np.arange(40) * 5 % 257] = 1.0
    assert np.array_equal(cpu_oracle.softmax(x), ref_ops.softmax(x))
    (l1, p1), (l2, p2) = cpu_oracle.cross_entropy_fwd(x, target), ref_ops.cross_entropy_fwd(x, target)
    assert l1 == l2 and np.array_equal(p1, p2)
    assert np.array_equal(cpu_oracle.cross_entropy_bwd(p1, target), ref_ops.cross_entropy_bwd(p2, target))
