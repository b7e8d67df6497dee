"""Exhaustive small-shape sweep of the tensor-core attention kernels against the CPU oracle, with
every output inside poisoned guard bands.

compute-sanitizer is not available where these tests run, so this file stands in for it on the
shapes where index arithmetic goes wrong first: every sequence length from 1 to 260 (below, at and
just above one and two 128-row tiles), with and without the causal mask, for both head dimensions
of the tcgen05 kernels, forward and backward, one (batch, head) unit each. Outputs are placed
directly between two 32 KB bands of 0x7F bytes which must be untouched afterwards.
Tolerances are those of the bf16 mode: 2e-2 on O and LSE, 2e-2 of the largest reference magnitude
on each gradient."""
import ctypes
import math

import numpy as np
import pytest

from conftest import Guarded, bf16_round, seeded
from ember_b200 import _lib
from oracle import cpu_oracle

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

LMAX = 260


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


@pytest.fixture(params=[128, 256])
def block_rows(request):
    """Both forms of the forward kernel (one or two query tiles per CTA); left to itself the library
    would take the one-tile form for every launch this small."""
    L = _lib.lib()
    before = L.ember_set_forward_block_rows(request.param)
    assert before >= 0
    yield request.param
    L.ember_set_forward_block_rows(before)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
def test_every_length_up_to_260(env, D, causal, block_rows):
    sweep(env, D, causal, range(1, LMAX + 1))


# Head dimensions the kernels pad to 64 / 128 columns, at the lengths around the tile boundaries and
# every ninth one between: a store into the padding of a row would hit the next row or a guard band.
PADDED_LENGTHS = sorted(set(range(1, LMAX + 1, 9)) | {63, 64, 65, 127, 128, 129, 191, 192, 193, 255, 256, 257, 260})


@pytest.mark.parametrize("D", [24, 80])
@pytest.mark.parametrize("causal", [False, True])
def test_padded_head_dims_over_lengths(env, D, causal, block_rows):
    sweep(env, D, causal, PADDED_LENGTHS)


def sweep(env, D, causal, lengths):
    L, dev, sp = env
    host = [bf16_round(seeded((LMAX, D), s, sc)) for s, sc in ((31, 0.5), (32, 0.5), (33, 0.5), (34, 1.0))]
    q, k, v, do = (torch.from_numpy(x).to(dev).to(torch.bfloat16) for x in host)
    scale = 1.0 / math.sqrt(D)
    bf, f32 = torch.bfloat16, torch.float32
    worst = 0.0
    for n in lengths:
        assert L.ember_attention_kernel_name(_lib.EMBER_OP_FWD, n, n, D, 1) == b"sm100_tcgen05"
        assert L.ember_attention_kernel_name(_lib.EMBER_OP_BWD, n, n, D, 1) == b"sm100_tcgen05"
        o, dq, dk, dv = (Guarded(torch, (n, D), bf, dev) for _ in range(4))
        lse = Guarded(torch, (n,), f32, dev)
        wsn = L.ember_attention_workspace_bytes(_lib.EMBER_OP_BWD, 1, n, n, D, 1, 0)
        ws = Guarded(torch, (wsn,), torch.uint8, dev)
        _lib.check(L.ember_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.t.data_ptr(), lse.t.data_ptr(), 1, n, n,
                                         D, scale, int(causal), 1, sp))
        _lib.check(L.ember_attention_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.t.data_ptr(), lse.t.data_ptr(),
                                         do.data_ptr(), dq.t.data_ptr(), dk.t.data_ptr(), dv.t.data_ptr(), 1, n, n, D, scale,
                                         int(causal), 1, ws.t.data_ptr(), wsn, sp))
        torch.cuda.synchronize()
        for name, g in (("o", o), ("lse", lse), ("dq", dq), ("dk", dk), ("dv", dv), ("workspace", ws)):
            g.check(f"{name} at L={n} D={D} causal={causal}")
        hq, hk, hv, hg = (x[:n] for x in host)
        ro, rl = cpu_oracle.attention_fwd(hq, hk, hv, None, causal)
        eo = np.abs(o.t.float().cpu().numpy() - ro).max()
        el = np.abs(lse.t.cpu().numpy() - rl).max()
        assert eo <= 2e-2 and el <= 2e-2, (n, eo, el)
        worst = max(worst, eo, el)
        for name, got, ref in zip(("dq", "dk", "dv"), (dq, dk, dv), cpu_oracle.attention_bwd(hq, hk, hv, hg, None, causal)):
            err = np.abs(got.t.float().cpu().numpy() - ref).max()
            assert err <= 2e-2 * max(np.abs(ref).max(), 1e-6), (name, n, err)
    where = ctypes.c_int(0)
    assert L.ember_check_device_status(sp, ctypes.byref(where)) == 0, where.value
