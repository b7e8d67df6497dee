"""CPU-only: the (batch*head) partition, single-process and as world_size-2 gloo ranks."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ember_b200.shard import shard_range, shard_sizes
from oracle import cpu_oracle


@pytest.mark.parametrize("bh,world", [(128, 1), (128, 2), (128, 8), (7, 4), (3, 8), (0, 2)])
def test_shards_tile_the_axis(bh, world):
    ranges = [shard_range(bh, r, world) for r in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == bh
    for (b0, e0), (b1, e1) in zip(ranges, ranges[1:]):
        assert e0 == b1
    sizes = shard_sizes(bh, world)
    assert sum(sizes) == bh and max(sizes) - min(sizes) <= 1


def test_bad_rank_raises():
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, H, L, D = 2, 3, 24, 16
        rng = np.random.default_rng(0)  # every rank generates the same un-sharded tensors
        q, k, v = (rng.standard_normal((B * H, L, D), dtype=np.float32) for _ in range(3))
        b, e = shard_range(B * H, rank, world)
        o_local = cpu_oracle.attention_fwd(q[b:e], k[b:e], v[b:e], None, True)[0]
        # optional result gather (not on the data path): equal-sized slabs -> all_gather
        parts = [torch.empty_like(torch.from_numpy(o_local)) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(o_local))
        full = torch.cat(parts).numpy()
        ref = cpu_oracle.attention_fwd(q, k, v, None, True)[0]
        ret[rank] = bool(np.array_equal(full, ref))
    finally:
        dist.destroy_process_group()


def test_two_ranks_reproduce_the_single_rank_result():
    world = 2
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}
