"""GPU tests of the Python surface added around the attention path: softmax, log_softmax and the
CrossEntropyLoss class, with the reference's calling conventions (ember/tensor/tensor.py:430-437,
ember/loss/losses.py:30-56)."""
import numpy as np
import pytest

from oracle import cpu_oracle

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def em():
    if not torch.cuda.is_available():
        pytest.skip("needs CUDA")
    import ember_b200

    return ember_b200


def test_softmax_matches_reference_golden(em, softmax_golden):
    from conftest import softmax_golden_inputs

    for name in ("sm_small", "sm_ragged", "sm_wide"):
        x, _ = softmax_golden_inputs(softmax_golden[name + "/meta"])
        got = em.softmax(em.Tensor(x), axis=-1)
        assert got.shape == x.shape
        assert np.abs(got.to_np() - softmax_golden[name + "/softmax"]).max() <= 1e-3
        ls = em.log_softmax(em.Tensor(x)).to_np()
        assert np.abs(np.exp(ls) - softmax_golden[name + "/softmax"]).max() <= 1e-3
    with pytest.raises(TypeError):
        em.softmax(np.zeros((2, 2), np.float32))
    with pytest.raises(ValueError):
        em.softmax(em.Tensor(np.zeros((2, 3, 4), np.float32)), axis=0)
    assert em.softmax(em.Tensor(np.zeros((2, 3, 4), np.float32))).shape == (2, 3, 4)


def test_cross_entropy_loss_class_matches_reference_golden(em, softmax_golden):
    from conftest import softmax_golden_inputs

    for name in ("sm_small", "sm_ragged", "sm_wide"):
        x, target = softmax_golden_inputs(softmax_golden[name + "/meta"])
        loss_fn = em.loss.CrossEntropyLoss()
        loss = loss_fn.forward(em.Tensor(x), em.Tensor(target))
        assert isinstance(loss, float)
        assert abs(loss - float(softmax_golden[name + "/loss"])) <= 1e-3 * abs(float(softmax_golden[name + "/loss"]))
        assert np.abs(loss_fn.probs.to_np() - softmax_golden[name + "/probs"]).max() <= 1e-3
        g = loss_fn.backward()
        assert np.abs(g.to_np() - softmax_golden[name + "/grad"]).max() <= 1e-3 / x.shape[0]
    with pytest.raises(ValueError):
        em.loss.CrossEntropyLoss().forward(em.Tensor(np.zeros((2, 3), np.float32)), em.Tensor(np.zeros((2, 4), np.float32)))
    with pytest.raises(AssertionError):
        em.loss.CrossEntropyLoss().backward()


def test_classifier_head_training_step(em):
    """x -> MultiHeadAttention -> Linear -> CrossEntropyLoss and back: the gradient chain runs end to
    end and matches the same chain on the CPU oracle."""
    B, L, E, H, C = 2, 32, 64, 4, 10
    rng = np.random.default_rng(5)
    x = rng.standard_normal((B, L, E), dtype=np.float32)
    mha = em.nn.MultiHeadAttention(E, H, causal=True, seed=1)
    head = em.nn.Linear(E, C, seed=2)
    target = np.zeros((B * L, C), np.float32)
    target[np.arange(B * L), rng.integers(0, C, B * L)] = 1.0
    y = mha(em.Tensor(x))
    logits = head(em.Tensor(y.to_np().reshape(B * L, E)))
    loss_fn = em.loss.CrossEntropyLoss()
    loss = loss_fn.forward(logits, em.Tensor(target))
    g_logits = loss_fn.backward()
    g_y = head.backward(g_logits)
    g_x = mha.backward(em.Tensor(g_y.to_np().reshape(B, L, E)))
    assert g_x.shape == (B, L, E) and np.isfinite(g_x.to_np()).all()
    ref_loss, ref_probs = cpu_oracle.cross_entropy_fwd(logits.to_np(), target)
    assert abs(loss - ref_loss) <= 1e-3 * abs(ref_loss)
    ref_g = cpu_oracle.cross_entropy_bwd(ref_probs, target)
    assert np.abs(g_logits.to_np() - ref_g).max() <= 1e-5
    rgx, rgw, rgb = cpu_oracle.linear_bwd(y.to_np().reshape(B * L, E), head.w.to_np(), ref_g)
    assert np.abs(g_y.to_np() - rgx).max() <= 1e-3 * max(np.abs(rgx).max(), 1e-6)
    assert np.abs(head.grad_w.to_np() - rgw).max() <= 1e-3 * np.abs(rgw).max()


def test_kv_cache_class_grows_and_decodes(em):
    """Token-by-token decode over a growing cache equals causal attention over the whole sequence."""
    B, Hq, Hkv, L, D = 2, 8, 2, 40, 64
    rng = np.random.default_rng(2)
    q = rng.standard_normal((B, Hq, L, D), dtype=np.float32) * 0.5
    k = rng.standard_normal((B, Hkv, L, D), dtype=np.float32) * 0.5
    v = rng.standard_normal((B, Hkv, L, D), dtype=np.float32) * 0.5
    cache = em.KVCache(B, Hkv, 64, D, dtype="float32")
    cache.append(em.Tensor(k[:, :, :25]), em.Tensor(v[:, :, :25]))  # prefill
    outs = []
    for t in range(25, L):
        cache.append(em.Tensor(k[:, :, t:t + 1]), em.Tensor(v[:, :, t:t + 1]))
        o, lse = cache.decode(em.Tensor(np.ascontiguousarray(q[:, :, t])))
        assert o.shape == (B, Hq, D) and lse.shape == (B, Hq)
        outs.append(o.to_np())
    kr, vr = np.repeat(k, Hq // Hkv, axis=1), np.repeat(v, Hq // Hkv, axis=1)
    ref, _ = cpu_oracle.attention_fwd(q, kr, vr, None, True)
    got = np.stack(outs, axis=2)
    assert np.abs(got - ref[:, :, 25:]).max() <= 1e-3
    with pytest.raises(ValueError):
        cache.append(em.Tensor(k[:, :, :30]), em.Tensor(v[:, :, :30]))
    with pytest.raises(ValueError):
        cache.decode(em.Tensor(np.zeros((B, 3, D), np.float32)))


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-3), ("bfloat16", 5e-2)])
def test_generation_with_cache_matches_full_forward(em, dtype, tol):
    """prefill + decode_step token by token gives the rows the causal block gives on the whole sequence."""
    B, L, E, H, P = 2, 24, 128, 2, 16
    rng = np.random.default_rng(4)
    x = rng.standard_normal((B, L, E), dtype=np.float32)
    layer = em.nn.MultiHeadAttention(E, H, causal=True, dtype=dtype, seed=3)
    full = layer(em.Tensor(x, dtype), False).to_np()
    cache = em.KVCache(B, H, 32, E // H, dtype=dtype)
    y0 = layer.prefill(em.Tensor(np.ascontiguousarray(x[:, :P]), dtype), cache).to_np()
    assert np.abs(y0 - full[:, :P]).max() <= tol * max(1.0, np.abs(full).max())
    for t in range(P, L):
        yt = layer.decode_step(em.Tensor(np.ascontiguousarray(x[:, t:t + 1]), dtype), cache).to_np()
        assert yt.shape == (B, 1, E)
        assert np.abs(yt[:, 0] - full[:, t]).max() <= tol * max(1.0, np.abs(full).max())
    assert cache.length == L
