"""GPU parity of the fused softmax / log-softmax / softmax cross-entropy entry points against the
CPU oracle of the reference's compositions (ember/tensor/tensor.py:430-437, ember/loss/losses.py:42-56),
through the C-ABI. float32 storage: 1e-3 (observed ~1e-6); bf16 storage: 2e-2 (output rounding)."""
import ctypes

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


def _dev(a, dev, bf16):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    return t.to(torch.bfloat16) if bf16 else t


def _round(a, bf16):
    return torch.from_numpy(a).to(torch.bfloat16).float().numpy() if bf16 else a


SHAPES = [(1, 1), (5, 7), (33, 130), (64, 128), (300, 1000), (17, 2048), (9, 2056), (6, 5000), (4, 16384), (3, 40001),
          (3, 50000), (2, 70001)]


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("shape", SHAPES)
def test_softmax_and_log_softmax(env, shape, bf16):
    L, dev, sp = env
    rows, cols = shape
    rng = np.random.default_rng(rows * 131 + cols)
    x = _round(rng.standard_normal(shape, dtype=np.float32) * 4, bf16)
    x[0, cols // 2] = 30.0 if not bf16 else 30.0  # a dominant entry
    tx = _dev(x, dev, bf16)
    ty = torch.empty_like(tx)
    dt = _lib.EMBER_BF16 if bf16 else _lib.EMBER_F32
    ref = cpu_oracle.softmax(x)
    _lib.check(L.ember_softmax_fwd(tx.data_ptr(), ty.data_ptr(), rows, cols, dt, 0, sp))
    torch.cuda.synchronize()
    got = ty.float().cpu().numpy()
    tol = 2e-2 if bf16 else 1e-3
    assert np.abs(got - ref).max() <= tol
    assert np.abs(got.sum(-1) - 1).max() <= (2e-2 if bf16 else 1e-4)
    _lib.check(L.ember_softmax_fwd(tx.data_ptr(), ty.data_ptr(), rows, cols, dt, 1, sp))
    torch.cuda.synchronize()
    got = ty.float().cpu().numpy()
    with np.errstate(divide="ignore"):
        ref_log = np.log(ref.astype(np.float64))
    finite = np.isfinite(ref_log) & (ref_log > -80)
    assert np.abs(got[finite] - ref_log[finite]).max() <= tol * max(1.0, np.abs(ref_log[finite]).max())


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("shape", [(4, 7), (33, 130), (256, 1000), (64, 4096), (7, 32768), (5, 50000)])
def test_cross_entropy(env, shape, bf16):
    L, dev, sp = env
    rows, cols = shape
    rng = np.random.default_rng(rows + cols)
    pred = _round(rng.standard_normal(shape, dtype=np.float32) * 3, bf16)
    target = np.zeros(shape, np.float32)
    target[np.arange(rows), rng.integers(0, cols, rows)] = 1.0
    dt = _lib.EMBER_BF16 if bf16 else _lib.EMBER_F32
    tp, tt = _dev(pred, dev, bf16), _dev(target, dev, bf16)
    probs, grad = torch.empty_like(tp), torch.empty_like(tp)
    loss = torch.zeros(1, device=dev, dtype=torch.float32)
    n = L.ember_cross_entropy_workspace_bytes(rows)
    ws = torch.empty(n, device=dev, dtype=torch.uint8)
    _lib.check(L.ember_cross_entropy_fwd(tp.data_ptr(), tt.data_ptr(), probs.data_ptr(), loss.data_ptr(), rows, cols, dt,
                                         ws.data_ptr(), n, sp))
    _lib.check(L.ember_cross_entropy_bwd(probs.data_ptr(), tt.data_ptr(), grad.data_ptr(), rows, cols, dt, sp))
    torch.cuda.synchronize()
    ref_loss, ref_probs = cpu_oracle.cross_entropy_fwd(pred, target)
    tol = 2e-2 if bf16 else 1e-3
    assert abs(float(loss[0]) - ref_loss) <= 1e-3 * max(1.0, abs(ref_loss))  # the loss is float32 in both modes
    assert np.abs(probs.float().cpu().numpy() - ref_probs).max() <= tol
    ref_grad = cpu_oracle.cross_entropy_bwd(_round(ref_probs, bf16), target)
    assert np.abs(grad.float().cpu().numpy() - ref_grad).max() <= tol / rows + 1e-7


def test_cross_entropy_needs_workspace(env):
    L, dev, sp = env
    t = torch.zeros(64, device=dev)
    with pytest.raises(RuntimeError):
        _lib.check(L.ember_cross_entropy_fwd(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), 8, 8, _lib.EMBER_F32,
                                             None, 0, sp))
    with pytest.raises(ValueError):
        _lib.check(L.ember_softmax_fwd(t.data_ptr(), t.data_ptr(), 0, 8, _lib.EMBER_F32, 0, sp))
