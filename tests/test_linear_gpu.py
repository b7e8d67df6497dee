"""GPU parity of the Linear entry points (the projections either side of attention) against the
CPU oracle of the reference's Linear layer, through the C-ABI. float32 storage: tolerance 1e-3;
bf16 storage: 2e-2, both relative to the largest reference magnitude of the tensor (the oracle
gets the bf16-rounded inputs, so input rounding is not charged to the kernel)."""
import ctypes

import numpy as np
import pytest

from conftest import linear_golden_inputs
from ember_b200 import _lib
from oracle import cpu_oracle

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

F32_TOL, BF16_TOL = 1e-3, 2e-2


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


def _np(t):
    return t.float().cpu().numpy()


def _to_heads(a, parts, batch, heads, seq, dim):
    """(batch*seq, parts*heads*dim) row-major -> (parts, batch, heads, seq, dim)."""
    return np.ascontiguousarray(a.reshape(batch, seq, parts, heads, dim).transpose(2, 0, 3, 1, 4))


def _from_heads(a, parts, batch, heads, seq, dim):
    return np.ascontiguousarray(a.reshape(parts, batch, heads, seq, dim).transpose(1, 3, 0, 2, 4)).reshape(
        batch * seq, parts * heads * dim)


def _run(L, sp, dev, x, w, b, dy, bf16, x_heads=0, y_heads=0, seq=0, dim=0):
    """x, w, b, dy are logical row-major float32 arrays; returns logical row-major results."""
    m, k = x.shape
    n = w.shape[1]
    dtype = _lib.EMBER_BF16 if bf16 else _lib.EMBER_F32
    batch = m // seq if seq else 0
    xs = _to_heads(x, 1, batch, x_heads, seq, dim) if x_heads else x
    dys = _to_heads(dy, n // (y_heads * dim), batch, y_heads, seq, dim) if y_heads else dy
    tx, tw, tdy = _dev(xs, dev, bf16), _dev(w, dev, bf16), _dev(dys, dev, bf16)
    tb = _dev(b, dev, bf16) if b is not None else None
    ty = torch.empty(m * n, device=dev, dtype=tx.dtype)
    tdx, tdw, tdb = (torch.empty(c, device=dev, dtype=tx.dtype) for c in (m * k, k * n, n))
    _lib.check(L.ember_linear_fwd(tx.data_ptr(), tw.data_ptr(), tb.data_ptr() if tb is not None else None, ty.data_ptr(),
                                  m, n, k, dtype, x_heads, y_heads, seq, dim, sp))
    _lib.check(L.ember_linear_bwd(tx.data_ptr(), tw.data_ptr(), tdy.data_ptr(), tdx.data_ptr(), tdw.data_ptr(),
                                  tdb.data_ptr(), m, n, k, dtype, x_heads, y_heads, seq, dim, sp))
    torch.cuda.synchronize()
    where = ctypes.c_int(0)
    assert L.ember_check_device_status(sp, ctypes.byref(where)) == 0, where.value
    y, dx = _np(ty), _np(tdx)
    y = _from_heads(y, n // (y_heads * dim), batch, y_heads, seq, dim) if y_heads else y.reshape(m, n)
    dx = _from_heads(dx, 1, batch, x_heads, seq, dim) if x_heads else dx.reshape(m, k)
    return y, dx, _np(tdw).reshape(k, n), _np(tdb)


def _check(got, ref, tol):
    for g, r, name in zip(got, ref, ("y", "grad_x", "grad_w", "grad_b")):
        assert np.isfinite(g).all(), name
        assert np.abs(g - r).max() <= tol * max(np.abs(r).max(), 1e-6), (name, np.abs(g - r).max(), np.abs(r).max())


def _rounded(arrs, bf16):
    if not bf16:
        return arrs
    return [None if a is None else torch.from_numpy(a).to(torch.bfloat16).float().numpy() for a in arrs]


@pytest.mark.parametrize("name", ["lin_small", "lin_tile", "lin_ragged", "lin_nobias"])
def test_f32_matches_reference_golden(env, linear_golden, name):
    L, dev, sp = env
    x, w, b, dy = linear_golden_inputs(linear_golden[name + "/meta"])
    got = _run(L, sp, dev, x, w, b, dy, bf16=False)
    ref = [linear_golden[name + "/" + k] for k in ("y", "gx", "gw", "gb")]
    _check(got, ref, F32_TOL)


TC_SHAPES = [(128, 256, 64), (256, 512, 128), (384, 264, 200), (130, 72, 520), (1000, 1024, 328), (4096, 768, 512)]


@pytest.mark.parametrize("bias", [True, False])
@pytest.mark.parametrize("mnk", TC_SHAPES)
def test_bf16_tcgen05(env, mnk, bias):
    L, dev, sp = env
    m, n, k = mnk
    for prod in range(3):
        assert L.ember_linear_kernel_name(prod, m, n, k, _lib.EMBER_BF16, 0, 0, 0, 0) == b"sm100_tcgen05"
    rng = np.random.default_rng(m + n + k)
    x, w, dy = (rng.standard_normal(s, dtype=np.float32) * sc for s, sc in (((m, k), 1.0), ((k, n), 0.1), ((m, n), 1.0)))
    b = rng.standard_normal((n,), dtype=np.float32) if bias else None
    x, w, b, dy = _rounded([x, w, b, dy], True)
    got = _run(L, sp, dev, x, w, b, dy, bf16=True)
    ref = (cpu_oracle.linear_fwd(x, w, b),) + cpu_oracle.linear_bwd(x, w, dy)
    _check(got, ref, BF16_TOL)


def test_bf16_odd_shape_uses_cuda_cores(env):
    L, dev, sp = env
    m, n, k = 77, 50, 91  # not multiples of 8: no 16-byte rows for TMA
    assert L.ember_linear_kernel_name(0, m, n, k, _lib.EMBER_BF16, 0, 0, 0, 0) == b"simt_f32"
    rng = np.random.default_rng(5)
    x, w, b, dy = _rounded([rng.standard_normal(s, dtype=np.float32) for s in ((m, k), (k, n), (n,), (m, n))], True)
    got = _run(L, sp, dev, x, w, b, dy, bf16=True)
    _check(got, (cpu_oracle.linear_fwd(x, w, b),) + cpu_oracle.linear_bwd(x, w, dy), BF16_TOL)


HEAD_CASES = [
    # batch, seq, heads, dim, (x_heads?, y parts) : a fused q/k/v projection and an output projection
    (2, 128, 4, 64, False, 3),
    (2, 256, 2, 128, False, 3),
    (2, 128, 4, 64, True, 0),
    (1, 384, 3, 128, True, 0),
    (3, 40, 2, 32, False, 3),   # seq not a multiple of 128: CUDA-core path
    (3, 40, 2, 32, True, 0),
]


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("case", HEAD_CASES)
def test_head_major_layouts(env, case, bf16):
    """x head-major (what attention writes) or y head-major in 3 parts (what attention reads)."""
    L, dev, sp = env
    batch, seq, heads, dim, x_is_heads, parts = case
    e = heads * dim
    m, k = batch * seq, e
    n = parts * e if parts else e
    rng = np.random.default_rng(batch * seq + heads + dim)
    x, w, b, dy = _rounded([rng.standard_normal(s, dtype=np.float32) * sc
                            for s, sc in (((m, k), 1.0), ((k, n), 0.1), ((n,), 1.0), ((m, n), 1.0))], bf16)
    got = _run(L, sp, dev, x, w, b, dy, bf16, x_heads=heads if x_is_heads else 0, y_heads=heads if parts else 0,
               seq=seq, dim=dim)
    ref = (cpu_oracle.linear_fwd(x, w, b),) + cpu_oracle.linear_bwd(x, w, dy)
    _check(got, ref, BF16_TOL if bf16 else F32_TOL)
    if bf16 and seq % 128 == 0:
        dt = _lib.EMBER_BF16
        assert L.ember_linear_kernel_name(0, m, n, k, dt, heads if x_is_heads else 0, heads if parts else 0, seq, dim) == b"sm100_tcgen05"


def test_invalid_arguments_are_value_errors(env):
    L, dev, sp = env
    t = torch.zeros(64, device=dev)
    with pytest.raises(ValueError):
        _lib.check(L.ember_linear_fwd(t.data_ptr(), t.data_ptr(), None, t.data_ptr(), 0, 8, 8, _lib.EMBER_F32, 0, 0, 0, 0, sp))
    with pytest.raises(ValueError):  # k must equal x_heads * head_dim
        _lib.check(L.ember_linear_fwd(t.data_ptr(), t.data_ptr(), None, t.data_ptr(), 8, 8, 8, _lib.EMBER_F32, 2, 0, 4, 8, sp))
    with pytest.raises(ValueError):
        _lib.check(L.ember_linear_bwd(t.data_ptr(), t.data_ptr(), t.data_ptr(), None, None, None, 8, 8, 8,
                                      _lib.EMBER_F32, 0, 0, 0, 0, sp))
