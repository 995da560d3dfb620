"""Multi-GPU partition of the decode hot path (one process per GPU, one node).

Every (batch item, KV head) pair is an independent unit: it owns its packed codes, scales
and softmax, and the query heads of a KV head travel with it. The ``B * H_kv`` units are
flattened (batch-major) and block-assigned to ranks, so attention needs no collective; the
only exchange is the delivery of each layer's attention output to every rank. Two ways to
do that are provided:

* :func:`gather_layer_output` -- an NCCL (or gloo) all-gather of the ranks' row blocks;
* :class:`PeerExchange` -- no collective call at all: the merge step of the attention kernel
  stores its rows straight into every rank's gathered tensor through peer-mapped pointers
  (CUDA IPC over NVLink) and raises an arrival word; a one-CTA kernel with a bounded wait is
  the consumer side (``vq_peer_gather_wait``).

A rank's shard is handed to the kernels as ``[units_local, 1, ...]`` tensors (batch axis =
this rank's units, one KV head each), which is exactly how the kernels index anyway: a
query row is ``unit * heads_per_kv + head``. The reference has no distributed code; this
module is new.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import _lib


@dataclass(frozen=True)
class ShardPlan:
    """The run of flattened ``(batch, kv head)`` units ``[lo, hi)`` a rank owns.

    ``units = batch * n_kv_heads`` are split into ``world`` contiguous blocks whose sizes
    differ by at most one (the first ``units % world`` ranks get one more). With fewer units
    than ranks the surplus ranks are *replicas*: they hold (and may compute on) a copy of the
    last unit but own no rows of the gathered output (``replica=True``, ``rows == 0``).
    """

    lo: int
    hi: int
    units: int
    n_kv_heads: int
    world: int
    rank: int
    replica: bool = False

    @property
    def size(self) -> int:
        """Units this rank computes on (a replica computes on one)."""
        return self.hi - self.lo

    @property
    def owned(self) -> int:
        """Units whose output rows this rank contributes to the gather."""
        return 0 if self.replica else self.hi - self.lo

    def block(self, rank: int) -> tuple[int, int]:
        """``(lo, hi)`` of the units OWNED by ``rank`` (empty for a replica)."""
        n = min(self.units, self.world)
        if rank >= n:
            return self.units, self.units
        base, extra = divmod(self.units, n)
        lo = rank * base + min(rank, extra)
        return lo, lo + base + (1 if rank < extra else 0)

    @property
    def max_owned(self) -> int:
        return max(self.block(r)[1] - self.block(r)[0] for r in range(self.world))


def plan_shards(batch: int, n_kv_heads: int, world: int, rank: int) -> ShardPlan:
    """Block partition of the ``batch * n_kv_heads`` flattened units over ``world`` ranks."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"plan_shards: bad rank {rank} of {world}")
    if batch < 1 or n_kv_heads < 1:
        raise ValueError(f"plan_shards: batch={batch} and kv heads={n_kv_heads} must be >= 1")
    units = batch * n_kv_heads
    probe = ShardPlan(0, 0, units, n_kv_heads, world, rank)
    lo, hi = probe.block(rank)
    if rank >= units:  # fewer units than ranks: a replica of the last unit
        return ShardPlan(units - 1, units, units, n_kv_heads, world, rank, replica=True)
    return ShardPlan(lo, hi, units, n_kv_heads, world, rank)


def shard_kv(x: torch.Tensor, plan: ShardPlan) -> torch.Tensor:
    """This rank's units of a ``[B, H_kv, ...]`` tensor, as ``[units_local, 1, ...]``."""
    if x.shape[0] * x.shape[1] != plan.units:
        raise ValueError(f"shard_kv: tensor has {x.shape[0]}x{x.shape[1]} units, the plan {plan.units}")
    return x.reshape(plan.units, 1, *x.shape[2:])[plan.lo : plan.hi]


def shard_queries(q: torch.Tensor, plan: ShardPlan, n_kv_heads: int | None = None) -> torch.Tensor:
    """This rank's slice of ``q [B, H_q, S_q, D]``: the query heads of its units, as
    ``[units_local, heads_per_kv, S_q, D]``."""
    n_kv_heads = plan.n_kv_heads if n_kv_heads is None else n_kv_heads
    B, H_q = q.shape[0], q.shape[1]
    if B * n_kv_heads != plan.units or H_q % n_kv_heads:
        raise ValueError(f"shard_queries: q {tuple(q.shape)} does not match {plan.units} units of {n_kv_heads} kv heads")
    hpk = H_q // n_kv_heads
    return q.reshape(plan.units, hpk, *q.shape[2:])[plan.lo : plan.hi]


def unshard_output(flat: torch.Tensor, plan: ShardPlan) -> torch.Tensor:
    """``[units, heads_per_kv, S_q, D]`` (all ranks' rows in unit order) -> ``[B, H_q, S_q, D]``."""
    B = plan.units // plan.n_kv_heads
    return flat.reshape(B, plan.n_kv_heads * flat.shape[1], *flat.shape[2:])


def gather_layer_output(local: torch.Tensor, plan: ShardPlan, out: torch.Tensor | None = None,
                        group=None) -> torch.Tensor:
    """All-gather one layer's attention output with a collective call.

    ``local`` is this rank's ``[units_local, heads_per_kv, S_q, D]``; the result is the full
    ``[B, H_q, S_q, D]``. Blocks of unequal size are padded to the largest block for the
    collective and trimmed afterwards; replicas contribute nothing. With one rank the input
    is only reshaped.
    """
    if plan.world == 1:
        full = unshard_output(local, plan)
        if out is not None:
            out.copy_(full)
            return out
        return full
    m = plan.max_owned
    send = local[: plan.owned]
    if plan.owned < m:
        pad = torch.zeros((m - plan.owned, *local.shape[1:]), dtype=local.dtype, device=local.device)
        send = torch.cat([send, pad], dim=0)
    flat = torch.empty((plan.world * m, *local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, send.contiguous(), group=group)
    if plan.units == plan.world * m:
        rows = flat
    else:
        parts = []
        for r in range(plan.world):
            lo, hi = plan.block(r)
            parts.append(flat[r * m : r * m + (hi - lo)])
        rows = torch.cat(parts, dim=0)
    full = unshard_output(rows, plan)
    if out is not None:
        out.copy_(full)
        return out
    return full


class PeerExchange:
    """Per-layer gathered output tensors that every rank's attention kernel writes directly.

    Each rank allocates one buffer holding, per layer, the gathered output
    ``[units, heads_per_kv, S_q, D]`` and an arrival array ``uint32[world]``; the buffers are
    exchanged as CUDA IPC handles over the process group and mapped once. ``layer(l)`` is the
    ``PeerGather`` structure to pass as ``gather=`` to ``kernels.kivi_decode_attend`` (or
    ``KIVIKVCache.fused_sdpa``); ``wait(l)`` enqueues the consumer-side wait; ``output(l)``
    is the full ``[B, H_q, S_q, D]`` tensor, valid on the stream after ``wait(l)``.

    Every rank must make the same sequence of calls per layer. Nothing here uses multicast
    or the bulk-copy engine on peer memory: plain stores, then a flag with a bounded wait
    (``kernels.attend_status()`` raises if a wait ran out).
    """

    _FLAG_STRIDE = 128  # bytes between the arrival arrays of two layers
    # A device allocation may be mapped only once per process, and two exchange buffers can lie in
    # one allocation of the peer's caching allocator: handle -> [mapped base, users]
    _MAPPED: dict = {}

    def __init__(self, plan: ShardPlan, n_layers: int, heads_per_kv: int, head_dim: int, dtype: torch.dtype,
                 device: torch.device, s_q: int = 1, group=None) -> None:
        if plan.world > _lib.VQ_MAX_PEERS:
            raise ValueError(f"PeerExchange: at most {_lib.VQ_MAX_PEERS} ranks, got {plan.world}")
        if plan.world * 4 > self._FLAG_STRIDE:
            raise ValueError("PeerExchange: too many ranks for the arrival array")
        self.plan, self.n_layers, self.group = plan, n_layers, group
        self.hpk, self.D, self.s_q, self.dtype, self.device = heads_per_kv, head_dim, s_q, dtype, device
        es = torch.empty((), dtype=dtype).element_size()
        self._rows = plan.units * heads_per_kv * s_q
        self._layer_bytes = -(-self._rows * head_dim * es // 256) * 256
        out_bytes = n_layers * self._layer_bytes
        self._flags_off = out_bytes
        total = out_bytes + n_layers * self._FLAG_STRIDE
        self.buffer = torch.zeros(total, dtype=torch.uint8, device=device)
        self.state = torch.zeros((n_layers, 4), dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        lib = _lib.lib()
        self._opened: list = []
        if plan.world == 1:
            peer_ptrs = [self.buffer.data_ptr()]
        else:
            handle = (C.c_ubyte * 64)()
            off = C.c_int64(0)
            with _lib.on_device(device):
                _lib.check(lib.vq_peer_export(self.buffer.data_ptr(), handle, C.byref(off)), "PeerExchange")
            mine = (bytes(handle), int(off.value))
            everyone = [None] * plan.world
            dist.all_gather_object(everyone, mine, group=group)
            peer_ptrs = []
            for r, (h, o) in enumerate(everyone):
                if r == plan.rank:
                    peer_ptrs.append(self.buffer.data_ptr())
                    continue
                key = (device.index, r, h)
                entry = self._MAPPED.get(key)
                if entry is None:
                    base = C.c_void_p()
                    hb = (C.c_ubyte * 64).from_buffer_copy(h)
                    with _lib.on_device(device):
                        _lib.check(lib.vq_peer_open(hb, C.byref(base)), "PeerExchange")
                    entry = self._MAPPED[key] = [base.value, 0]
                entry[1] += 1
                self._opened.append(key)
                peer_ptrs.append(entry[0] + o)
            # nobody may publish into a buffer that its owner has not zeroed and mapped yet
            dist.barrier(group=group)
        self._peer_ptrs = peer_ptrs
        self._structs = [self._make(l) for l in range(n_layers)]

    def _make(self, l: int) -> _lib.PeerGather:
        pg = _lib.PeerGather()
        pg.world, pg.rank = self.plan.world, self.plan.rank
        pg.n_sources = min(self.plan.units, self.plan.world)
        pg.row_offset = self.plan.lo * self.hpk * self.s_q
        for r, base in enumerate(self._peer_ptrs):
            pg.out[r] = base + l * self._layer_bytes
            pg.flags[r] = base + self._flags_off + l * self._FLAG_STRIDE
        pg.state = self.state[l].data_ptr()
        n_chunks = -(-self.hpk // 4)   # CTAs per unit that write rows (four query heads each)
        for r in range(self.plan.world):
            lo, hi = self.plan.block(r)
            pg.arrivals[r] = (hi - lo) * n_chunks * self.s_q
        return pg

    def layer(self, l: int) -> _lib.PeerGather:
        if self.plan.replica:
            raise RuntimeError("PeerExchange.layer: a replica rank owns no rows of the gathered output")
        return self._structs[l]

    def wait(self, l: int) -> None:
        """Enqueue, on the current stream, the bounded wait for all ranks' rows of layer ``l``."""
        with _lib.on_device(self.device):
            _lib.check(_lib.lib().vq_peer_gather_wait(C.byref(self._structs[l]), _lib.stream_ptr(self.device)),
                       "PeerExchange.wait")

    def output(self, l: int) -> torch.Tensor:
        es = torch.empty((), dtype=self.dtype).element_size()
        raw = self.buffer[l * self._layer_bytes : l * self._layer_bytes + self._rows * self.D * es]
        flat = raw.view(self.dtype).view(self.plan.units, self.hpk, self.s_q, self.D)
        return unshard_output(flat, self.plan)

    def __enter__(self) -> "PeerExchange":
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    def close(self) -> None:
        """Unmap the peers' buffers (after a barrier: nobody may still be writing into ours)."""
        if self.plan.world > 1:
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
        lib = _lib.lib()
        for key in self._opened:
            entry = self._MAPPED[key]
            entry[1] -= 1
            if entry[1] == 0:
                with _lib.on_device(self.device):
                    lib.vq_peer_close(entry[0])
                del self._MAPPED[key]
        self._opened = []


__all__ = ["ShardPlan", "plan_shards", "shard_kv", "shard_queries", "unshard_output", "gather_layer_output",
           "PeerExchange"]
