"""The multi-GPU partition on CPU: plan arithmetic, and a world-size-2 gloo run that shards a
decode step by batch and by KV head, attends per rank with the oracle (standing in for the
kernels, which need a GPU) and checks the gathered output against the unsharded result."""

from __future__ import annotations

import math
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import kivi as o_kivi
from veloxquant_mlx_b200.sharding import gather_layer_output, plan_shards, shard_kv, shard_queries


def test_plan_covers_units_disjointly():
    for B, H, W in [(16, 8, 8), (16, 8, 2), (4, 8, 8), (1, 8, 4), (6, 8, 4)]:
        plans = [plan_shards(B, H, W, r) for r in range(W)]
        axis = plans[0].axis
        total = B if axis == "batch" else H
        covered = sorted(i for p in plans for i in range(p.lo, p.hi))
        assert covered == list(range(total)) and all(p.axis == axis and not p.replica for p in plans)
    assert plan_shards(16, 8, 8, 3).axis == "batch" and plan_shards(4, 8, 8, 3).axis == "head"
    # fewer units than ranks: surplus ranks replicate
    plans = [plan_shards(1, 3, 4, r) for r in range(4)]
    assert [p.replica for p in plans] == [False, False, False, True]
    with pytest.raises(ValueError):
        plan_shards(6, 9, 4, 0)
    with pytest.raises(ValueError):
        plan_shards(4, 4, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, B, H_q, H_kv, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        D, S, g = 32, 64, 32
        q, kc, ks, kz, vc, vs, vz = o_kivi.make_inputs(B, H_q, S, D, 2, g, seed=1, H_kv=H_kv)
        scale = 1.0 / math.sqrt(D)
        full = o_kivi.reference_attend(q, kc, ks, kz, vc, vs, vz, g, scale)
        plan = plan_shards(B, H_kv, world, rank)
        sl = lambda a: shard_kv(torch.from_numpy(a), plan).numpy()  # noqa: E731
        q_loc = shard_queries(torch.from_numpy(q), plan, H_kv).numpy()
        loc = o_kivi.reference_attend(q_loc, sl(kc), sl(ks), sl(kz), sl(vc), sl(vs), sl(vz), g, scale)
        got = gather_layer_output(torch.from_numpy(loc), plan).numpy()
        ok = got.shape == full.shape and np.allclose(got, full, atol=1e-6)
        ret[rank] = (plan.axis, bool(ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("B,H_q,H_kv,axis", [(4, 8, 2, "batch"), (1, 8, 4, "head"), (3, 8, 2, "head")])
def test_world_size_2_gloo_gather_matches_unsharded(B, H_q, H_kv, axis):
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), B, H_q, H_kv, ret), nprocs=world, join=True)
    assert dict(ret) == {0: (axis, True), 1: (axis, True)}
