"""GPU tests of the layer surface: Linear and MultiHeadAttention (projection -> attention ->
projection with head-major tensors in between) against the same chain composed on the CPU oracle."""
import numpy as np
import pytest

from conftest import bf16_round
from oracle import cpu_oracle

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def em():
    if not torch.cuda.is_available():
        pytest.skip("needs CUDA")
    import ember_b200

    return ember_b200


def _rel(a, b):
    return np.abs(a - b).max() / max(np.abs(b).max(), 1e-6)


def test_linear_layer_contract(em):
    """Same calls as the reference's Linear: __call__ caches, backward returns grad_x and fills the gradients."""
    layer = em.nn.Linear(96, 40, seed=3)
    assert [t.shape for t in layer.parameters()] == [(96, 40), (40,)]
    assert layer.gradients() == [None, None]
    rng = np.random.default_rng(0)
    x, g = rng.standard_normal((33, 96), dtype=np.float32), rng.standard_normal((33, 40), dtype=np.float32)
    w, b = layer.w.to_np(), layer.b.to_np()
    y = layer(em.Tensor(x), True)
    gx = layer.backward(em.Tensor(g))
    gw, gb = layer.gradients()
    ry = cpu_oracle.linear_fwd(x, w, b)
    rgx, rgw, rgb = cpu_oracle.linear_bwd(x, w, g)
    for got, ref in ((y, ry), (gx, rgx), (gw, rgw), (gb, rgb)):
        assert _rel(got.to_np(), ref) <= 1e-3
    layer.reset()
    assert layer.x is None and layer.gradients() == [None, None]
    with pytest.raises(ValueError):
        layer(em.Tensor(np.zeros((4, 95), np.float32)))
    with pytest.raises(TypeError):
        em.linear_forward(x, layer.w)


def _mha_oracle(x, wqkv, bqkv, wo, bo, H, causal, gy):
    B, L, E = x.shape
    D = E // H
    x2 = x.reshape(B * L, E)
    qkv = cpu_oracle.linear_fwd(x2, wqkv, bqkv)                       # (B*L, 3E)
    qkv_h = qkv.reshape(B, L, 3, H, D).transpose(2, 0, 3, 1, 4)       # (3, B, H, L, D)
    q, k, v = (np.ascontiguousarray(t) for t in qkv_h)
    o, _ = cpu_oracle.attention_fwd(q, k, v, None, causal)
    o2 = np.ascontiguousarray(o.transpose(0, 2, 1, 3)).reshape(B * L, E)
    y = cpu_oracle.linear_fwd(o2, wo, bo)
    g2 = gy.reshape(B * L, E)
    go2, gwo, gbo = cpu_oracle.linear_bwd(o2, wo, g2)
    go = np.ascontiguousarray(go2.reshape(B, L, H, D).transpose(0, 2, 1, 3))
    dq, dk, dv = cpu_oracle.attention_bwd(q, k, v, go, None, causal)
    gqkv = np.stack([dq, dk, dv]).transpose(1, 3, 0, 2, 4).reshape(B * L, 3 * E)
    gx, gwqkv, gbqkv = cpu_oracle.linear_bwd(x2, wqkv, np.ascontiguousarray(gqkv))
    return y.reshape(B, L, E), gx.reshape(B, L, E), gwqkv, gbqkv, gwo, gbo


@pytest.mark.parametrize("cfg", [
    # B, L, E, H, causal, dtype, tol
    (2, 48, 64, 4, False, "float32", 2e-3),
    (1, 130, 96, 3, True, "float32", 2e-3),
    (2, 128, 256, 2, True, "bfloat16", 4e-2),   # D = 128: tcgen05 attention and projections
    (2, 256, 256, 4, False, "bfloat16", 4e-2),  # D = 64
])
def test_multi_head_attention_matches_composed_oracle(em, cfg):
    B, L, E, H, causal, dtype, tol = cfg
    layer = em.nn.MultiHeadAttention(E, H, causal=causal, dtype=dtype, seed=7)
    rng = np.random.default_rng(11)
    layer.b_qkv = em.Tensor(rng.standard_normal((3 * E,), dtype=np.float32) * 0.1, dtype)
    layer.b_o = em.Tensor(rng.standard_normal((E,), dtype=np.float32) * 0.1, dtype)
    x = rng.standard_normal((B, L, E), dtype=np.float32)
    gy = rng.standard_normal((B, L, E), dtype=np.float32)
    if dtype == "bfloat16":
        x, gy = bf16_round(x), bf16_round(gy)
    wqkv, bqkv, wo, bo = (t.to_np() for t in layer.parameters())
    y = layer(em.Tensor(x, dtype), True)
    assert y.shape == (B, L, E)
    gx = layer.backward(em.Tensor(gy, dtype))
    ref = _mha_oracle(x, wqkv, bqkv, wo, bo, H, causal, gy)
    got = (y, gx) + tuple(layer.gradients())
    for name, g, r in zip(("y", "grad_x", "grad_w_qkv", "grad_b_qkv", "grad_w_o", "grad_b_o"), got, ref):
        assert g.shape == r.shape, name
        assert _rel(g.to_np(), r) <= tol, (name, _rel(g.to_np(), r))


def test_layers_subclass_layer_and_compose_in_sequential(em):
    """Linear and MultiHeadAttention are ``Layer`` subclasses (single tensor in, single tensor out)
    and compose in ``Sequential`` the way the reference's layers do (ember/nn/base.py:50-75):
    forward in order, backward in reverse, parameters and gradients concatenated; ``training``
    defaults to True as in the reference's ``Layer.__call__``."""
    nn = em.nn
    E, H, B, L = 64, 2, 2, 32
    lin1, mha, lin2 = nn.Linear(E, E, seed=1), nn.MultiHeadAttention(E, H, causal=True, seed=2), nn.Linear(E, 24, seed=3)
    net = nn.Sequential(lin1, mha, lin2)
    for layer in (lin1, mha, lin2, net, nn.Attention()):
        assert isinstance(layer, nn.Layer)
    rng = np.random.default_rng(4)
    x, g = rng.standard_normal((B, L, E), dtype=np.float32), rng.standard_normal((B, L, 24), dtype=np.float32)
    y = net(em.Tensor(x))
    assert net._training is True and lin1._training is True
    # the same three steps by hand
    h1 = lin1.forward(em.Tensor(x))
    h2 = mha.forward(h1)
    y2 = lin2.forward(h2)
    assert np.array_equal(y.to_np(), y2.to_np())
    gx = net.backward(em.Tensor(g))
    gx2 = lin1.backward(mha.backward(lin2.backward(em.Tensor(g))))
    assert np.array_equal(gx.to_np(), gx2.to_np())
    assert len(net.parameters()) == 2 + 4 + 2 and len(net.gradients()) == 8
    assert all(t is not None for t in net.gradients())
    net.reset()
    assert net.x is None and lin1.x is None and mha.x is None
    att = nn.Attention(causal=True)
    q = em.Tensor(rng.standard_normal((1, 2, 16, 32), dtype=np.float32))
    att((q, q, q))
    assert att._training is True
