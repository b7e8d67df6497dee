"""GPU test of the bounds-checked debug build (``libember_b200_dbg.so``, -DEMBER_BOUNDS_CHECK): the
tensor-core attention kernels run with every global store checked against its tensor's extent, over
lengths below, at and above the tile sizes; no store may be reported, and the results match the oracle.
A child process loads the debug library through EMBER_B200_LIB (one process, one build of the library).
Skipped when the debug library has not been built (`python -m ember_b200.build --bounds`)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DBG = os.path.join(ROOT, "ember_b200", "libember_b200_dbg.so")

CODE = r"""
import ctypes, math, sys
import numpy as np
root = sys.argv[1]
sys.path.insert(0, root); sys.path.insert(0, root + "/tests")
import torch
from conftest import bf16_round, seeded
from ember_b200 import _lib
from oracle import cpu_oracle
L = _lib.lib()
assert _lib.LIB_PATH.endswith("_dbg.so")
_lib.check(L.ember_set_device(0))
dev = torch.device("cuda", 0)
st = torch.cuda.Stream(device=dev); torch.cuda.set_stream(st); sp = ctypes.c_void_p(st.cuda_stream)
for D in (64, 128):
    host = [bf16_round(seeded((700, D), s, sc)) for s, sc in ((1, 0.5), (2, 0.5), (3, 0.5), (4, 1.0))]
    q, k, v, do = (torch.from_numpy(x).to(dev).to(torch.bfloat16) for x in host)
    for n in (1, 17, 100, 127, 128, 129, 255, 256, 257, 260, 384, 513, 700):
        for causal in (0, 1):
            # both forms of the forward kernel: one query tile per CTA (odd passes) and two (even)
            assert L.ember_set_forward_block_rows(128 if (n + causal) % 2 else 256) >= 0
            o, dq, dk, dv = (torch.empty((n, D), device=dev, dtype=torch.bfloat16) for _ in range(4))
            lse = torch.empty((n,), device=dev, dtype=torch.float32)
            wsn = L.ember_attention_workspace_bytes(_lib.EMBER_OP_BWD, 1, n, n, D, 1, 0)
            ws = torch.empty(wsn, device=dev, dtype=torch.uint8)
            sc = 1.0 / math.sqrt(D)
            _lib.check(L.ember_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), 1, n, n, D, sc, causal, 1, sp))
            _lib.check(L.ember_attention_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), do.data_ptr(),
                                             dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), 1, n, n, D, sc, causal, 1, ws.data_ptr(), wsn, sp))
            where = ctypes.c_int(0)
            rc = L.ember_check_device_status(sp, ctypes.byref(where))
            assert rc == 0, (n, D, causal, where.value, L.ember_last_error())
            ro, rl = cpu_oracle.attention_fwd(host[0][:n], host[1][:n], host[2][:n], None, bool(causal))
            assert np.abs(o.float().cpu().numpy() - ro).max() <= 2e-2
            for got, ref in zip((dq, dk, dv), cpu_oracle.attention_bwd(host[0][:n], host[1][:n], host[2][:n], host[3][:n], None, bool(causal))):
                assert np.abs(got.float().cpu().numpy() - ref).max() <= 2e-2 * max(np.abs(ref).max(), 1e-6)
print("debug build ok")
"""


def test_bounds_checked_build_reports_no_store_outside_a_tensor():
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("needs CUDA")
    if not os.path.exists(DBG):
        pytest.skip("debug library not built (python -m ember_b200.build --bounds)")
    env = dict(os.environ, EMBER_B200_LIB=DBG)
    r = subprocess.run([sys.executable, "-c", CODE, ROOT], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "debug build ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
