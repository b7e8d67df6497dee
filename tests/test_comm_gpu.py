"""GPU test (two GPUs of one box) of the optional output gather: two ranks each run the forward on
their (batch*head) slab of the same seeded tensors and gather; the gathered tensor equals the
single-rank result bit for bit. Skipped with fewer than two GPUs. NVLS is off, as for every
multi-process GPU test here, and no kernel of the library reads peer memory."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, ret):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist

    import ember_b200 as em
    from conftest import bf16_round, seeded
    from ember_b200 import _lib
    from ember_b200.comm import Communicator

    _lib.check(_lib.lib().ember_set_device(rank))
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0))
    comm = Communicator(rank, world, store, timeout_s=60.0)
    B, H, L, D = 2, 4, 384, 128
    q, k, v = (bf16_round(seeded((B * H, L, D), s, 0.5)) for s in (1, 2, 3))   # every rank: the same whole tensors
    b, e = comm.slab(B * H)
    o_local, _ = em.attention_forward(*(em.Tensor(x[b:e][None], "bfloat16") for x in (q, k, v)), None, True)
    full = comm.gather(em.Tensor._from_core(o_local._core, (e - b, L, D), "bfloat16"))
    got = full.to_np()
    if rank == 0:
        o_ref, _ = em.attention_forward(*(em.Tensor(x[None], "bfloat16") for x in (q, k, v)), None, True)
        ret["equal"] = bool(np.array_equal(got, o_ref.to_np()[0]))
    comm.close()


def test_two_ranks_gather_equals_the_single_rank_result():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
        assert dict(ret) == {"equal": True}
