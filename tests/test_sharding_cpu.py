"""The multi-GPU partition on CPU: plan arithmetic over the flattened (batch, kv head) units,
and gloo runs (world sizes 2 and 4) that shard a decode step, attend per rank with the oracle
(standing in for the kernels, which need a GPU) and check the gathered output against the
unsharded result -- even splits, uneven splits, and fewer units than ranks (replica ranks)."""

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
    for B, H, W in [(16, 8, 8), (16, 8, 2), (4, 8, 8), (1, 8, 4), (6, 8, 4), (6, 2, 4), (5, 3, 4), (3, 1, 2)]:
        plans = [plan_shards(B, H, W, r) for r in range(W)]
        covered = sorted(i for p in plans if not p.replica for i in range(p.lo, p.hi))
        assert covered == list(range(B * H)), (B, H, W)
        sizes = [p.owned for p in plans]
        assert max(sizes) - min(sizes) <= 1 and all(p.units == B * H for p in plans)
        assert [p.block(r) for p in plans[:1] for r in range(W)] == [(p.lo, p.hi) for p in plans]
    # the two benchmark partitions: 128 units -> 16 per GPU; 32 units -> 4 per GPU
    assert plan_shards(16, 8, 8, 3).size == 16 and plan_shards(4, 8, 8, 3).size == 4
    # units that neither axis divides evenly still split: 12 units over 4 ranks, 3 each
    assert [plan_shards(6, 2, 4, r).size for r in range(4)] == [3, 3, 3, 3]
    # fewer units than ranks: surplus ranks replicate the last unit and own no output rows
    plans = [plan_shards(1, 3, 4, r) for r in range(4)]
    assert [p.replica for p in plans] == [False, False, False, True]
    assert (plans[3].lo, plans[3].hi, plans[3].owned, plans[3].size) == (2, 3, 0, 1)
    with pytest.raises(ValueError):
        plan_shards(4, 4, 2, 2)
    with pytest.raises(ValueError):
        plan_shards(0, 4, 2, 0)


def test_shard_views_take_the_right_units():
    B, H_kv, hpk, D = 3, 2, 4, 8
    kv = torch.arange(B * H_kv * 5 * D, dtype=torch.float32).reshape(B, H_kv, 5, D)
    q = torch.arange(B * H_kv * hpk * D, dtype=torch.float32).reshape(B, H_kv * hpk, 1, D)
    plan = plan_shards(B, H_kv, 4, 1)  # 6 units over 4 ranks: sizes 2, 2, 1, 1; rank 1 owns units 2, 3
    assert (plan.lo, plan.hi) == (2, 4)
    loc = shard_kv(kv, plan)
    assert loc.shape == (2, 1, 5, D) and torch.equal(loc[0, 0], kv[1, 0]) and torch.equal(loc[1, 0], kv[1, 1])
    ql = shard_queries(q, plan)
    assert ql.shape == (2, hpk, 1, D) and torch.equal(ql[0], q[1, :hpk]) and torch.equal(ql[1], q[1, hpk:])
    with pytest.raises(ValueError):
        shard_kv(kv[:2], plan)


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
        q_loc = shard_queries(torch.from_numpy(q), plan).numpy()
        loc = o_kivi.reference_attend(q_loc, sl(kc), sl(ks), sl(kz), sl(vc), sl(vs), sl(vz), g, scale)
        got = gather_layer_output(torch.from_numpy(loc), plan).numpy()
        ok = got.shape == full.shape and np.allclose(got, full, atol=1e-6)
        ret[rank] = (plan.size, plan.replica, bool(ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,B,H_q,H_kv,sizes", [
    (2, 4, 8, 2, [4, 4]),          # whole batch items per rank
    (2, 1, 8, 4, [2, 2]),          # kv heads of one batch item
    (2, 3, 8, 2, [3, 3]),          # a rank's block spans parts of two batch items
    (2, 3, 3, 1, [2, 1]),          # uneven blocks
    (4, 1, 6, 3, [1, 1, 1, 1]),    # fewer units than ranks: rank 3 is a replica
])
def test_gloo_gather_matches_unsharded(world, B, H_q, H_kv, sizes):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), B, H_q, H_kv, ret), nprocs=world, join=True)
    units = B * H_kv
    want = {r: (sizes[r], r >= units, True) for r in range(world)}
    assert dict(ret) == want
