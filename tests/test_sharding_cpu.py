"""Host-side sharding logic: planner properties on one process, and a world_size-2 gloo run in which
each rank computes its own (batch, head) slices (CPU oracle standing in for the kernel) and the union
equals the unsharded result bit for bit."""
import math
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cfk_b200.sharding import element_offset, slice_range, strides, sub_calls


@pytest.mark.parametrize("B,H,W", [(2, 32, 1), (2, 32, 2), (2, 32, 4), (2, 32, 8), (3, 5, 4), (1, 3, 8), (4, 16, 3)])
def test_plan_covers_every_slice_once(B, H, W):
    seen = np.zeros(B * H, int)
    sizes = []
    for r in range(W):
        lo, hi = slice_range(B, H, W, r)
        sizes.append(hi - lo)
        covered = 0
        for c in sub_calls(B, H, W, r):
            assert 0 <= c.head_begin and c.head_begin + c.head_count <= H
            assert c.batch_count == 1 or (c.head_begin == 0 and c.head_count == H)
            for b in range(c.batch_begin, c.batch_begin + c.batch_count):
                for h in range(c.head_begin, c.head_begin + c.head_count):
                    seen[b * H + h] += 1
                    covered += 1
        assert covered == hi - lo
    assert (seen == 1).all()
    assert max(sizes) - min(sizes) <= 1


def test_offsets_and_strides():
    c = sub_calls(2, 8, 4, 1)[0]           # rank 1 of 4: batch 0, heads 4..7
    assert (c.batch_begin, c.batch_count, c.head_begin, c.head_count) == (0, 1, 4, 4)
    assert element_offset(c, seq=16, heads=8, head_dim=64) == 4 * 64
    assert strides(16, 8, 64) == (16 * 8 * 64, 8 * 64, 64)


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    from oracle.oracle import CfkOracle
    orc = CfkOracle()
    B, S, H, D = 2, 96, 3, 32
    q, k, v = (orc.fill((B, S, H, D), seed=3081 + i) for i in range(3))      # identical on every rank
    o = np.zeros((B, S, H, D), np.float32)
    for c in sub_calls(B, H, world, rank):
        part = orc.attention(q, k, v, 1.0 / math.sqrt(D), True,
                             b_range=(c.batch_begin, c.batch_begin + c.batch_count),
                             h_range=(c.head_begin, c.head_begin + c.head_count))["o"]
        o += part
    t = torch.from_numpy(o)
    dist.all_reduce(t)                      # test-side gather only; the data path itself has no collective
    if rank == 0:
        full = orc.attention(q, k, v, 1.0 / math.sqrt(D), True)["o"]
        np.save(os.path.join(out_dir, "ok.npy"), np.array([np.array_equal(t.numpy(), full)]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_union_equals_unsharded(tmp_path):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert np.load(tmp_path / "ok.npy")[0]
