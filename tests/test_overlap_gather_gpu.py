"""Launch arrangements around the decode attention, on the GPU:

* ``overlap_previous`` (programmatic dependent launch of the main kernel): back-to-back calls
  that share one workspace must give exactly the results of the same calls made one at a time;
* the peer exchange: the merge step publishes its rows into every rank's gathered tensor and
  raises an arrival word; the consumer-side wait returns; rounds are counted on the device so
  a captured graph can be replayed. Ranks are emulated on one GPU by making the calls of both
  ranks one after the other on one stream (every word a wait polls was raised by an earlier
  launch); a real two-process, two-GPU run follows when two GPUs are visible;
* the bounded device waits: made to run out through the library's self-test knobs (a barrier
  that nothing arms, a small poll limit), they must surface as ``VQ_ERR_TIMEOUT`` exactly once.
  Nothing here faults or hangs the GPU;
* steady-state decode through the cache allocates no device memory.
"""

from __future__ import annotations

import ctypes as C
import math
import os
import socket

import numpy as np
import pytest
import torch

from oracle import kivi as o_kivi

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCALE = 1.0 / math.sqrt(128)


def _cache(bits=4, residual=128, capacity=None):
    from veloxquant_mlx_b200.cache import KVCacheConfig, KVCacheFactory

    return KVCacheFactory.create(KVCacheConfig(method="kivi", head_dim=128, bit_width_inlier=bits, capacity=capacity,
                                               residual_length=residual, fused_sdpa_memory_bound=True))


def _filled(seed, B, H_kv, S, bits=4, dtype=torch.float16, dev=DEV):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    k = torch.randn((B, H_kv, S, 128), generator=g, device=dev, dtype=torch.float32).to(dtype)
    v = torch.randn((B, H_kv, S, 128), generator=g, device=dev, dtype=torch.float32).to(dtype)
    c = _cache(bits)
    c.update_and_fetch(k, v)
    return c, k, v


@pytest.mark.parametrize("B,H_kv,H_q,S", [(1, 2, 8, 700), (4, 8, 32, 4096 + 40)])
def test_overlapped_back_to_back_calls_equal_isolated_calls(B, H_kv, H_q, S):
    """50 rounds of two calls on different caches through ONE workspace, each allowed to start
    before the previous call has finished: bit-identical to the isolated calls."""
    c, _, _ = _filled(1, B, H_kv, S)
    d, _, _ = _filled(2, B, H_kv, S)
    g = torch.Generator(device=DEV)
    g.manual_seed(3)
    q = torch.randn((B, H_q, 1, 128), generator=g, device=DEV, dtype=torch.float16)
    # (the isolated calls carry the flag too: it also selects the split plan, i.e. the summation order)
    want_c = c.fused_sdpa(q, SCALE, overlap_previous=True).clone()
    torch.cuda.synchronize()
    want_d = d.fused_sdpa(q, SCALE, overlap_previous=True).clone()
    torch.cuda.synchronize()
    assert not torch.equal(want_c, want_d)
    plain = c.fused_sdpa(q, SCALE).float()
    assert float((plain - want_c.float()).abs().max()) < 1e-3
    oc, od = torch.empty_like(q), torch.empty_like(q)
    for _ in range(50):
        oc.fill_(float("nan"))
        od.fill_(float("nan"))
        torch.cuda.synchronize()
        c.fused_sdpa(q, SCALE, out=oc, overlap_previous=True)
        d.fused_sdpa(q, SCALE, out=od, overlap_previous=True)
        c.fused_sdpa(q, SCALE, out=oc, overlap_previous=True)
        torch.cuda.synchronize()
        assert torch.equal(oc, want_c) and torch.equal(od, want_d)
    c.check_status()


def test_overlapped_calls_in_a_replayed_graph():
    caches = [_filled(10 + i, 2, 2, 1000 + 32 * i)[0] for i in range(4)]
    q = torch.randn((2, 8, 1, 128), device=DEV, dtype=torch.float16)
    want = []
    for c in caches:
        want.append(c.fused_sdpa(q, SCALE, overlap_previous=True).clone())
        torch.cuda.synchronize()
    outs = [torch.empty_like(q) for _ in caches]

    def step():
        for c, o in zip(caches, outs):
            c.fused_sdpa(q, SCALE, out=o, overlap_previous=True)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for _ in range(5):
        for o in outs:
            o.zero_()
        graph.replay()
        torch.cuda.synchronize()
        for o, w in zip(outs, want):
            assert torch.equal(o, w)


def _emulated_gathers(world, B, H_kv, hpk, dtype):
    """PeerGather structures of `world` ranks whose buffers all live on this GPU."""
    from veloxquant_mlx_b200 import _lib
    from veloxquant_mlx_b200.sharding import plan_shards

    units = B * H_kv
    outs = [torch.zeros((units * hpk, 128), dtype=dtype, device=DEV) for _ in range(world)]
    flags = [torch.zeros(32, dtype=torch.int32, device=DEV) for _ in range(world)]
    states = [torch.zeros(4, dtype=torch.int32, device=DEV) for _ in range(world)]
    plans = [plan_shards(B, H_kv, world, r) for r in range(world)]
    structs = []
    for r in range(world):
        pg = _lib.PeerGather()
        pg.world, pg.rank, pg.n_sources = world, r, min(units, world)
        pg.row_offset = plans[r].lo * hpk
        for p in range(world):
            pg.out[p] = outs[p].data_ptr()
            pg.flags[p] = flags[p].data_ptr()
        pg.state = states[r].data_ptr()
        for p in range(world):
            pg.arrivals[p] = plans[p].owned * -(-hpk // 4)
        structs.append(pg)
    return plans, structs, outs, flags, states


@pytest.mark.parametrize("world,B,H_kv,H_q,dtype,S", [
    (2, 2, 2, 8, torch.float16, 1500), (4, 3, 2, 16, torch.bfloat16, 1500), (3, 1, 4, 8, torch.float32, 1500),
    # long and large enough that every rank's launch takes the eight-head kernel, whose CTAs arrive
    # with the weight of the four-head chunks they stand for (5 heads per kv head: weight 2)
    (2, 6, 8, 40, torch.float16, 16384 + 200)])
def test_peer_exchange_emulated_ranks_gather_the_unsharded_output(world, B, H_kv, H_q, dtype, S):
    from veloxquant_mlx_b200 import _lib
    from veloxquant_mlx_b200 import kernels as vk
    from veloxquant_mlx_b200.sharding import shard_kv, shard_queries, unshard_output

    hpk = H_q // H_kv
    act = torch.float16 if dtype == torch.float32 else dtype
    full, k, v = _filled(5, B, H_kv, S, dtype=act)
    units = B * H_kv
    plans, structs, outs, flags, states = _emulated_gathers(world, B, H_kv, hpk, dtype)
    shards = []
    for r in range(world):
        c = _cache()
        c.update_and_fetch(shard_kv(k, plans[r]).contiguous(), shard_kv(v, plans[r]).contiguous())
        shards.append(c)
    for rnd in range(3):
        g = torch.Generator(device=DEV)
        g.manual_seed(20 + rnd)
        q = torch.randn((B, H_q, 1, 128), generator=g, device=DEV, dtype=torch.float32).to(act)
        want = full.fused_sdpa(q, SCALE).to(dtype)
        for o in outs:
            o.zero_()
        for r in range(world):
            q_loc = shard_queries(q, plans[r]).contiguous()
            loc = torch.empty(q_loc.shape, dtype=dtype, device=DEV)
            shards[r].fused_sdpa(q_loc, SCALE, out=loc, gather=structs[r], overlap_previous=True)
        for r in range(world):
            _lib.check(_lib.lib().vq_peer_gather_wait(C.byref(structs[r]), torch.cuda.current_stream().cuda_stream), "wait")
        torch.cuda.synchronize()
        vk.attend_status()
        for r in range(world):
            got = unshard_output(outs[r].view(units, hpk, 1, 128), plans[r])
            err = (got.float() - want.float()).abs()
            assert bool((err <= 2e-3 + 1e-2 * want.float().abs()).all()), f"rank {r} round {rnd}: {err.max().item():.3e}"
            assert torch.equal(outs[r], outs[0])
        assert [int(s[2]) for s in states] == [rnd + 1] * world
        # every rank's word r holds (rounds so far) x (rank r's four-head chunks that write rows)
        assert all(int(f[r]) == (rnd + 1) * plans[r].owned * -(-hpk // 4) for f in flags for r in range(world))


def test_peer_wait_that_nothing_satisfies_times_out_and_is_reported_once():
    """The consumer-side wait for a rank that never publishes gives up (after about a second)
    and the status call reports it; the GPU stays usable."""
    from veloxquant_mlx_b200 import VQLibraryError, _lib
    from veloxquant_mlx_b200 import kernels as vk

    plans, structs, outs, flags, states = _emulated_gathers(2, 1, 2, 4, torch.float16)
    vk.attend_status()
    _lib.check(_lib.lib().vq_peer_gather_wait(C.byref(structs[0]), torch.cuda.current_stream().cuda_stream), "wait")
    with pytest.raises(VQLibraryError, match="VQ_ERR_TIMEOUT.*did not arrive"):
        vk.attend_status()
    vk.attend_status()
    assert torch.zeros(1, device=DEV).item() == 0.0


def test_attend_bounded_wait_self_test_reports_timeout_once():
    from veloxquant_mlx_b200 import VQLibraryError
    from veloxquant_mlx_b200 import kernels as vk

    c, _, _ = _filled(7, 1, 2, 640)
    q = torch.randn((1, 8, 1, 128), device=DEV, dtype=torch.float16)
    want = c.fused_sdpa(q, SCALE).clone()
    c.check_status()
    assert vk.tune("attend_wait_test", 1) == 0
    got = c.fused_sdpa(q, SCALE)
    with pytest.raises(VQLibraryError, match="VQ_ERR_TIMEOUT"):
        c.check_status()
    c.check_status()                       # cleared by the report
    assert torch.equal(got, want)          # the self-test waits on an extra barrier only
    assert torch.equal(c.fused_sdpa(q, SCALE), want)
    c.check_status()                       # one-shot: the next launch is a normal one


def test_vq_search_bounded_wait_self_test_reports_timeout_once():
    from veloxquant_mlx_b200 import VQLibraryError
    from veloxquant_mlx_b200 import kernels as vk
    from veloxquant_mlx_b200 import vecinfer as vi

    x = torch.randn(8192, 8, device=DEV).to(torch.float16)
    cb = torch.randn(256, 8, device=DEV)
    want = vi.quantize_vq(x, cb, 8, index_dtype=torch.uint8)
    vk.quantize_status()
    prev = vk.tune("vq_search", 1)
    try:
        vk.tune("vq_wait_test", 1)
        got = vi.quantize_vq(x, cb, 8, index_dtype=torch.uint8)
        with pytest.raises(VQLibraryError, match="VQ_ERR_TIMEOUT"):
            vk.quantize_status()
        vk.quantize_status()
        assert torch.equal(got, want)
    finally:
        vk.tune("vq_search", prev)


@pytest.mark.parametrize("bits", [2, 4])
def test_causal_multi_row_attention_over_the_packed_cache(bits):
    B, H_kv, H_q, S, S_q, g = 2, 2, 8, 300, 7, 32
    c, k, v = _filled(31, B, H_kv, S, bits=bits)
    gen = torch.Generator(device=DEV)
    gen.manual_seed(5)
    q = torch.randn((B, H_q, S_q, 128), generator=gen, device=DEV, dtype=torch.float16)
    nq = c._n_quantized
    levels = (1 << bits) - 1
    kc, ks, kz = o_kivi.quant_keys(k[:, :, :nq].cpu().numpy(), g, levels)
    vc, vs, vz = o_kivi.quant_values(v[:, :, :nq].cpu().numpy(), g, levels)
    for causal in (True, False):
        got = c.fused_sdpa(q, SCALE, causal=causal).float().cpu().numpy()
        ref = o_kivi.reference_attend(q.cpu().numpy(), kc, ks, kz, vc, vs, vz, g, SCALE, k_res=k[:, :, nq:].cpu().numpy(),
                                      v_res=v[:, :, nq:].cpu().numpy(), causal=causal)
        err = np.abs(got - ref)
        assert np.all(err <= 2e-3 + 1e-2 * np.abs(ref)), f"causal={causal}: {err.max():.3e}"
    # the last row of a causal call sees everything: it equals a single-row decode call
    last = c.fused_sdpa(q[:, :, -1:].contiguous(), SCALE).float()
    full = c.fused_sdpa(q, SCALE, causal=True).float()[:, :, -1:]
    assert float((last - full).abs().max()) < 2e-3
    with pytest.raises(ValueError, match="query rows"):
        c.fused_sdpa(torch.zeros(B, H_q, S + 1, 128, device=DEV, dtype=torch.float16), SCALE)


def test_steady_state_decode_allocates_nothing_and_matches_a_prefill():
    """300 single-token appends (9 flushes, one move of the window back to the buffer's front)
    with attention after each: no allocation from torch's allocator, and the packed store ends
    up identical to a one-shot prefill of the same tokens."""
    B, H_kv, H_q, S0, n_dec = 2, 2, 8, 384, 300
    g = torch.Generator(device=DEV)
    g.manual_seed(11)
    k = torch.randn((B, H_kv, S0 + n_dec, 128), generator=g, device=DEV, dtype=torch.float16)
    v = torch.randn((B, H_kv, S0 + n_dec, 128), generator=g, device=DEV, dtype=torch.float16)
    q = torch.randn((B, H_q, 1, 128), generator=g, device=DEV, dtype=torch.float16)
    c = _cache(capacity=1024)  # (the packed store doubles when full: pre-sized here, as a serving loop would)
    c.update_and_fetch(k[:, :, :S0], v[:, :, :S0])
    out = torch.empty_like(q)
    kt = torch.empty((B, H_kv, 1, 128), device=DEV, dtype=torch.float16)
    vt = torch.empty_like(kt)
    for t in range(S0, S0 + 40):  # warm-up: first flush, workspace, residual buffer in place
        kt.copy_(k[:, :, t : t + 1]); vt.copy_(v[:, :, t : t + 1])
        c.update_and_fetch(kt, vt)
        c.fused_sdpa(q, SCALE, out=out)
    torch.cuda.synchronize()
    before = torch.cuda.memory_stats()["allocation.all.allocated"]
    free_before = torch.cuda.mem_get_info()[0]
    moved = 0
    for t in range(S0 + 40, S0 + n_dec):
        kt.copy_(k[:, :, t : t + 1]); vt.copy_(v[:, :, t : t + 1])
        lo = c._res_lo
        c.update_and_fetch(kt, vt)
        moved += int(c._res_lo < lo and c._res_lo == 0)
        c.fused_sdpa(q, SCALE, out=out)
    torch.cuda.synchronize()
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == before
    assert torch.cuda.mem_get_info()[0] == free_before
    assert moved >= 1 and c._n_quantized == ((S0 + n_dec - 128) // 32) * 32
    one = _cache()
    one.update_and_fetch(k, v)
    nq = one._n_quantized
    assert c._n_quantized == nq and c._n_res == one._n_res
    for a, b in ((c._k_codes, one._k_codes), (c._v_codes, one._v_codes), (c._v_scale, one._v_scale), (c._v_zero, one._v_zero)):
        assert torch.equal(a[:, :, :nq], b[:, :, :nq])
    assert torch.equal(c._k_scale[:, :, : nq // 32], one._k_scale[:, :, : nq // 32])
    assert torch.equal(c.fused_sdpa(q, SCALE), one.fused_sdpa(q, SCALE))
    st = c.state
    assert torch.equal(st[6], k[:, :, nq:]) and torch.equal(st[7], v[:, :, nq:])


def test_state_loads_into_a_cache_that_already_holds_a_larger_capacity():
    big, _, _ = _filled(40, 1, 2, 3000)
    small, ks, vs = _filled(41, 1, 2, 500)
    q = torch.randn((1, 8, 1, 128), device=DEV, dtype=torch.float16)
    want = small.fused_sdpa(q, SCALE).clone()
    big.state = small.state
    assert big.offset == 500 and torch.equal(big.fused_sdpa(q, SCALE), want)


# ---------------------------------------------------------------------------------------------
# two processes, two GPUs
def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _two_gpu_worker(rank, world, port, ret):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from veloxquant_mlx_b200 import kernels as vk
        from veloxquant_mlx_b200.sharding import PeerExchange, gather_layer_output, plan_shards, shard_kv, shard_queries

        B, H_kv, H_q, S, L = 3, 2, 8, 2100, 3
        hpk = H_q // H_kv
        plan = plan_shards(B, H_kv, world, rank)
        px = PeerExchange(plan, L, hpk, 128, torch.float16, dev)
        fulls, shards = [], []
        for l in range(L):
            full, k, v = _filled(100 + l, B, H_kv, S, dev=dev)
            c = _cache()
            c.update_and_fetch(shard_kv(k, plan).contiguous(), shard_kv(v, plan).contiguous())
            fulls.append(full)
            shards.append(c)
        ok = True
        for rnd in range(3):
            g = torch.Generator(device=dev)
            g.manual_seed(50 + rnd)
            q = torch.randn((B, H_q, 1, 128), generator=g, device=dev, dtype=torch.float16)
            q_loc = shard_queries(q, plan).contiguous()
            for l in range(L):
                loc = torch.empty_like(q_loc)
                shards[l].fused_sdpa(q_loc, SCALE, out=loc, gather=px.layer(l))
                px.wait(l)
                want = fulls[l].fused_sdpa(q, SCALE).float()
                got = px.output(l).float()
                ok &= bool(((got - want).abs() <= 2e-3 + 1e-2 * want.abs()).all())
                ok &= torch.equal(px.output(l), gather_layer_output(loc, plan))
        torch.cuda.synchronize()
        vk.attend_status()
        px.close()
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_sharded_attention_gathers_the_unsharded_output():
    import torch.multiprocessing as mp

    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_two_gpu_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert dict(ret) == {0: True, 1: True}


def test_overlapped_decode_loop_equals_the_plain_loop():
    """update_and_fetch + fused_sdpa per layer, every call allowed to start under the previous
    one (the append copies its rows after a wait, the attention reads them after its own): the
    same outputs as the plain loop (up to the split plan's summation order) and bit-identical
    stores, across two quantize-on-append flushes; flush steps fall back to plain launches."""
    L, B, H_kv, H_q, S0, n_dec = 4, 2, 2, 8, 1000, 70
    g = torch.Generator(device=DEV)
    g.manual_seed(21)
    kv = torch.randn((2, L, B, H_kv, S0 + n_dec, 128), generator=g, device=DEV, dtype=torch.float16)
    qs = torch.randn((n_dec, L, B, H_q, 1, 128), generator=g, device=DEV, dtype=torch.float16)
    plain = [_cache(capacity=2048) for _ in range(L)]
    fast = [_cache(capacity=2048) for _ in range(L)]
    for l in range(L):
        for c in (plain[l], fast[l]):
            c.update_and_fetch(kv[0, l, :, :, :S0], kv[1, l, :, :, :S0])
    out_p = torch.empty((L, B, H_q, 1, 128), device=DEV, dtype=torch.float16)
    out_f = torch.empty_like(out_p)
    flushes = 0
    for t in range(n_dec):
        nq = fast[0]._n_quantized
        for l in range(L):
            k1, v1 = kv[0, l, :, :, S0 + t : S0 + t + 1].contiguous(), kv[1, l, :, :, S0 + t : S0 + t + 1].contiguous()
            plain[l].update_and_fetch(k1, v1)
            plain[l].fused_sdpa(qs[t, l], SCALE, out=out_p[l])
        torch.cuda.synchronize()
        # (inputs of the overlapped calls are complete here: nothing they read is produced by the
        # kernels right before them)
        for l in range(L):
            k1, v1 = kv[0, l, :, :, S0 + t : S0 + t + 1].contiguous(), kv[1, l, :, :, S0 + t : S0 + t + 1].contiguous()
            torch.cuda.synchronize()
            fast[l].update_and_fetch(k1, v1, overlap_previous=True)
            fast[l].fused_sdpa(qs[t, l], SCALE, out=out_f[l], overlap_previous=True)
        torch.cuda.synchronize()
        flushes += int(fast[0]._n_quantized != nq)
        assert float((out_p.float() - out_f.float()).abs().max()) < 1e-3, f"step {t}"
    assert flushes == 2
    for a, b in zip(plain, fast):
        nq = a._n_quantized
        assert nq == b._n_quantized and a._n_res == b._n_res
        assert torch.equal(a._k_codes[:, :, :nq], b._k_codes[:, :, :nq]) and torch.equal(a._v_scale[:, :, :nq], b._v_scale[:, :, :nq])
        for x, y in zip(a.state, b.state):
            assert torch.equal(x, y)
    fast[0].check_status()
