"""Multi-GPU partition of the decode hot path.

Every (batch item, KV head) pair is an independent unit: it owns its packed codes, scales
and softmax, and the query heads of a KV head travel with it. Units are block-assigned to
ranks, so attention needs no collective; the only exchange is one all-gather of each
layer's attention output. The reference has no distributed code; this is new.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class ShardPlan:
    """Which slice of ``[B, H_kv]`` a rank owns. Either whole batch items (``axis="batch"``)
    or, when there are fewer batch items than ranks, KV heads of every batch item
    (``axis="head"``). Ranks beyond the available units hold a replica of the last shard
    (``replica=True``) and contribute nothing to the gather."""

    axis: str
    lo: int
    hi: int
    world: int
    rank: int
    replica: bool = False

    @property
    def size(self) -> int:
        return self.hi - self.lo


def plan_shards(batch: int, n_kv_heads: int, world: int, rank: int) -> ShardPlan:
    """Block partition of the units over ``world`` ranks (even split required so that the
    gather is a plain all-gather)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"plan_shards: bad rank {rank} of {world}")
    if batch % world == 0:
        per = batch // world
        return ShardPlan("batch", rank * per, (rank + 1) * per, world, rank)
    if n_kv_heads % world == 0:
        per = n_kv_heads // world
        return ShardPlan("head", rank * per, (rank + 1) * per, world, rank)
    units = batch if batch >= n_kv_heads else n_kv_heads
    axis = "batch" if batch >= n_kv_heads else "head"
    if units >= world:
        raise ValueError(
            f"plan_shards: neither batch={batch} nor kv heads={n_kv_heads} divides evenly over {world} ranks")
    # fewer units than ranks: surplus ranks are replicas
    r = min(rank, units - 1)
    return ShardPlan(axis, r, r + 1, world, rank, replica=rank >= units)


def shard_kv(x: torch.Tensor, plan: ShardPlan) -> torch.Tensor:
    """This rank's slice of a ``[B, H_kv, ...]`` tensor."""
    return x[plan.lo : plan.hi] if plan.axis == "batch" else x[:, plan.lo : plan.hi]


def shard_queries(q: torch.Tensor, plan: ShardPlan, n_kv_heads: int) -> torch.Tensor:
    """This rank's slice of ``q [B, H_q, S_q, D]``: the query heads of its KV heads."""
    if plan.axis == "batch":
        return q[plan.lo : plan.hi]
    hpk = q.shape[1] // n_kv_heads
    return q[:, plan.lo * hpk : plan.hi * hpk]


def gather_layer_output(local: torch.Tensor, plan: ShardPlan, out: torch.Tensor | None = None,
                        group=None) -> torch.Tensor:
    """All-gather one layer's attention output along the sharded axis.

    ``local`` is ``[B_local, H_q, S_q, D]`` (batch shards) or ``[B, H_q_local, S_q, D]`` (head
    shards); the result is the full ``[B, H_q, S_q, D]``. With one rank it returns ``local``.
    """
    if plan.world == 1:
        return local
    if plan.axis == "batch":
        shape = (local.shape[0] * plan.world, *local.shape[1:])
        if out is None:
            out = torch.empty(shape, dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    # head shards: gather into [world, B, H_local, S_q, D], then put ranks next to heads
    flat = torch.empty((plan.world * local.shape[0], *local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, local.contiguous(), group=group)
    stacked = flat.view(plan.world, *local.shape)
    full = stacked.permute(1, 0, 2, 3, 4).reshape(local.shape[0], plan.world * local.shape[1], *local.shape[2:])
    if out is not None:
        out.copy_(full)
        return out
    return full


__all__ = ["ShardPlan", "plan_shards", "shard_kv", "shard_queries", "gather_layer_output"]
