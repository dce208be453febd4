"""Host-side multi-GPU logic on CPU: two gloo ranks (no GPU involved)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from machinelearning_b200 import sharding


def test_split_range_is_a_partition():
    for n in (0, 1, 7, 8, 32, 33):
        for world in (1, 2, 3, 8):
            spans = [sharding.split_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (a, b), (c, d) in zip(spans, spans[1:]):
                assert b == c and b - a >= d - c >= 0
    with pytest.raises(ValueError):
        sharding.split_range(4, 2, 2)


def test_plan_prefers_batch_then_kv_heads():
    assert sharding.plan(32, 12, 8, 3) == {"dim": "batch", "start": 12, "stop": 16}
    assert sharding.plan(8, 16, 8, 7) == {"dim": "batch", "start": 7, "stop": 8}
    p = sharding.plan(2, 4, 8, 5)
    assert p == {"dim": "kv_head", "batch": 1, "start": 1, "stop": 2}
    covered = sorted((sharding.plan(2, 4, 8, r)["batch"], sharding.plan(2, 4, 8, r)["start"])
                     for r in range(8))
    assert covered == [(b, h) for b in range(2) for h in range(4)]
    with pytest.raises(ValueError):
        sharding.plan(2, 3, 8, 0)


def test_take_shard_head_slices_follow_their_kv_head():
    B, T, H, Hkv, D = 2, 5, 8, 4, 4
    q = torch.arange(B * T * H * D, dtype=torch.float32).view(B, T, H, D)
    k = torch.arange(B * T * Hkv * D, dtype=torch.float32).view(B, T, Hkv, D)
    ql, kl, vl, dl = sharding.take_shard(q, k, k, q, sharding.plan(B, Hkv, 8, 5))
    assert ql.shape == (1, T, 2, D) and kl.shape == (1, T, 1, D)
    assert torch.equal(ql, q[1:2, :, 2:4]) and torch.equal(kl, k[1:2, :, 1:2])
    assert ql.is_contiguous() and kl.is_contiguous()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, B):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(B * 3 * 2, dtype=torch.float32).view(B, 3, 2)
        p = sharding.plan(B, 1, world, rank)
        local = full[p["start"]:p["stop"]] * 1.0
        got = sharding.gather_batch_shards(local, B)
        assert torch.equal(got, full)
        slow = sharding.max_over_ranks(10.0 + rank, "cpu")
        assert slow == 10.0 + world - 1
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("B", [4, 5])
def test_gather_and_slowest_rank_over_two_gloo_ranks(B):
    mp.spawn(_worker, args=(2, _free_port(), B), nprocs=2, join=True)
