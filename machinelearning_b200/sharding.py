"""Multi-GPU partitioning of the attention path: one process per GPU.

Every (batch, head) pair is independent in forward and backward (the reference
kernel indexes them as ``blockIdx.y = b * H + h``, ``flash_attn_cuda.cu:164-168``;
with GQA the unit for dK/dV is ``(b, hkv)``, ``:1017-1020``), so the path shards
with no collective inside it.  Batch is split first (contiguous slices of
``[B,T,H,D]``, no copy); KV-head groups are split only when there are fewer
batch elements than ranks.  Collectives appear only around the path: gathering
outputs and gradients for verification and taking the slowest rank's time.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def split_range(n: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous balanced share ``[start, stop)`` of ``n`` units for ``rank``."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world: {rank}/{world}")
    base, extra = divmod(n, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def plan(B: int, Hkv: int, world: int, rank: int) -> dict:
    """Which slice of the problem ``rank`` owns.

    ``{"dim": "batch", "start", "stop"}`` when ``B >= world``; otherwise ranks are
    spread over ``B * Hkv`` (batch, kv-head) units: ``{"dim": "kv_head", "batch":
    b, "start", "stop"}`` with a KV-head range inside one batch element (query
    heads follow their KV head: ``[start * group, stop * group)``).
    """
    if B >= world:
        s, e = split_range(B, world, rank)
        return {"dim": "batch", "start": s, "stop": e}
    if (B * Hkv) % world != 0 or world % B != 0:
        raise ValueError(f"cannot split B={B} x Hkv={Hkv} units evenly over {world} ranks")
    per_batch = world // B
    b, r = divmod(rank, per_batch)
    s, e = split_range(Hkv, per_batch, r)
    return {"dim": "kv_head", "batch": b, "start": s, "stop": e}


def take_shard(q, k, v, dout, plan_: dict):
    """Local (q, k, v, dout) for a plan; batch shards are views, head shards copies."""
    if plan_["dim"] == "batch":
        sl = slice(plan_["start"], plan_["stop"])
        return q[sl], k[sl], v[sl], dout[sl]
    group = q.shape[2] // k.shape[2]
    b = plan_["batch"]
    ks, ke = plan_["start"], plan_["stop"]
    hq = slice(ks * group, ke * group)
    return (q[b:b + 1, :, hq].contiguous(), k[b:b + 1, :, ks:ke].contiguous(),
            v[b:b + 1, :, ks:ke].contiguous(), dout[b:b + 1, :, hq].contiguous())


def gather_batch_shards(local: torch.Tensor, B: int, group=None) -> torch.Tensor:
    """All-gather batch shards (possibly uneven) back into a ``[B, ...]`` tensor."""
    world = dist.get_world_size(group)
    sizes = [split_range(B, world, r) for r in range(world)]
    longest = max(e - s for s, e in sizes)
    padded = local.new_zeros((longest,) + tuple(local.shape[1:]))
    padded[: local.shape[0]] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[: e - s] for p, (s, e) in zip(parts, sizes)], dim=0)


def max_over_ranks(value: float, device, group=None) -> float:
    """The slowest rank's figure (how every multi-GPU time here is reported)."""
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
