"""CPU-only: the host-side rendezvous of the optional output gather. A rank that never arrives is
detected on the host of the others (a TimeoutError naming it) before any communicator is built or
anything is launched; the failure is made on the host (a rank that simply does not check in)."""
import threading
import time

import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402

from ember_b200.comm import wait_for_ranks  # noqa: E402


def test_all_ranks_checking_in_passes():
    store = dist.HashStore()
    world = 3

    def rank(r):
        time.sleep(0.05 * r)
        store.set(f"ember_comm/rank{r}", b"1")

    ths = [threading.Thread(target=rank, args=(r,)) for r in range(world)]
    for t in ths:
        t.start()
    wait_for_ranks(store, world, timeout_s=5.0)
    for t in ths:
        t.join()


def test_a_rank_that_never_arrives_is_a_timeout_naming_it():
    store = dist.HashStore()
    store.set("ember_comm/rank0", b"1")
    store.set("ember_comm/rank2", b"1")
    t0 = time.monotonic()
    with pytest.raises(TimeoutError, match=r"ranks \[1\] of 3"):
        wait_for_ranks(store, 3, timeout_s=0.5)
    assert time.monotonic() - t0 < 5.0
