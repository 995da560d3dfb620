"""Per-operation timings of the hot path on one GPU, at the sizes the headline configurations
use. ``bench.py`` measures the decode step; this module times the other operations one at a
time (quantize-on-append kernels, the coded-cache attends) so that each has a measured rate
and a command a profiler can wrap:

    python -m veloxquant_mlx_b200.microbench                 # every operation
    python -m veloxquant_mlx_b200.microbench --op vq_quantize --dtype float16 --iters 20

Each line is JSON: operation, shape, microseconds per call (CUDA events, after 3 warm-up calls,
inputs larger than L2 or re-created so that nothing is served from cache where that matters),
algorithmic bytes or useful FLOPs per call and the resulting rate.
"""

from __future__ import annotations

import argparse
import json

import torch

from . import kernels as k
from . import rabitq as rq
from . import vecinfer as vi

_DT = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}


_USE_GRAPH = False


def _time_us(fn, iters: int) -> float:
    """Microseconds per call. With ``--graph`` the call is captured once into a CUDA graph and the
    graph is replayed, which takes the Python and launch overhead out of short operations."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    run = fn
    if _USE_GRAPH:
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        with torch.cuda.graph(g):
            fn()
        run = g.replay
        run()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        run()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


def _line(op, shape, us, *, nbytes=None, flops=None, **extra):
    rec = {"op": op, "shape": shape, "us": round(us, 2)}
    if nbytes is not None:
        rec.update(bytes=int(nbytes), GBps=round(nbytes / us / 1e3, 1))
    if flops is not None:
        rec.update(useful_flops=int(flops), TFLOPs=round(flops / us / 1e6, 2))
    rec.update(extra)
    print(json.dumps(rec), flush=True)


def op_kivi_quantize(a):
    """Quantize + pack of one layer's K and V at the decode workload's prefill shape."""
    B, H, S, D = a.batch, 8, a.ctx, 128
    x = torch.randn(B, H, S, D, device="cuda", dtype=_DT[a.dtype] if a.dtype != "float32" else torch.bfloat16)
    for bits in (4, 2):
        for axis, name in ((-2, "keys"), (-1, "values")):
            us = _time_us(lambda: k.kivi_quantize(x, axis, 32, bits), a.iters)
            n = x.numel()
            nb = n * x.element_size() + n * bits // 8 + (n // 32) * 8
            _line("kivi_quantize", f"{name} b={bits} [{B},{H},{S},{D}] {x.dtype}", us, nbytes=nb)


def op_vq_quantize(a):
    dt = _DT[a.dtype]
    k.tune("vq_search", a.search)
    for S in (4096, 65536):
        keys = torch.randn(8, S, 128, device="cuda").to(dt)
        cb = torch.randn(256, 8, device="cuda")
        us = _time_us(lambda: vi.quantize_vq(keys, cb, 8, index_dtype=torch.uint8), a.iters)
        n = 8 * S * 16
        _line("vq_quantize", f"[8,{S},128] {a.dtype} sub_dim=8 n_c=256 search={a.search}", us, flops=2 * n * 256 * 8,
              nbytes=keys.numel() * keys.element_size() + n)
    k.tune("vq_search", 0)


def op_vq_encode(a):
    keys = torch.randn(1, 8, 4096, 128, device="cuda").to(_DT[a.dtype])
    cb = torch.randn(256, 8, device="cuda")
    H = vi.walsh_hadamard_matrix(128, device="cuda")
    sm = torch.rand(8, 128, device="cuda") + 0.5
    us = _time_us(lambda: vi.vecinfer_encode_decode_metal(keys, cb, 8, H, sm), a.iters)
    _line("vq_encode_decode_keys", "[1,8,4096,128] sub_dim=8 n_c=256", us, flops=2 * 8 * 4096 * 16 * 256 * 8)
    us = _time_us(lambda: vi.vecinfer_encode_decode_simple_metal(keys, cb, 8), a.iters)
    _line("vq_encode_decode_values", "[1,8,4096,128] sub_dim=8 n_c=256", us, flops=2 * 8 * 4096 * 16 * 256 * 8)


def op_vq_attend(a):
    S = 4096
    keys = torch.randn(1, 8, S, 128, device="cuda", dtype=torch.float16)
    cb = torch.randn(256, 8, device="cuda")
    kidx = vi.quantize_vq(keys, cb, 8, index_dtype=torch.uint8)
    v = torch.randn(1, 8, S, 128, device="cuda", dtype=torch.float16)
    q = torch.randn(1, 32, 1, 128, device="cuda", dtype=torch.float16)
    us = _time_us(lambda: vi.fused_sdpa_vq(q, kidx, cb, v, None, 0.088), a.iters)
    _line("vq_attend", f"H_q=32 H_kv=8 S={S} dense f16 values", us, nbytes=kidx.numel() + v.numel() * 2)
    # a serving shape (batch 8, 16 384 keys): the staged tensor-core kernel with the score table in shared memory
    B, S = 8, 16384
    v = torch.randn(B, 8, S, 128, device="cuda", dtype=torch.float16)
    kidx = vi.quantize_vq(v, cb, 8, index_dtype=torch.uint8)
    q = torch.randn(B, 32, 1, 128, device="cuda", dtype=torch.float16)
    us = _time_us(lambda: vi.fused_sdpa_vq(q, kidx, cb, v, None, 0.088), a.iters)
    _line("vq_attend", f"B={B} H_q=32 H_kv=8 S={S} dense f16 values", us, nbytes=kidx.numel() + v.numel() * 2)


def op_rabitq(a):
    B, H, S, D = 8, 8, 16384, 128
    keys = torch.randn(B * H * S, D, device="cuda", dtype=torch.float16)
    diag = torch.from_numpy(rq.make_hadamard_diagonal(D)).to("cuda")
    us = _time_us(lambda: rq.rabitq_encode(keys, diag), a.iters)
    _line("rabitq_encode", f"[{B * H * S},{D}] f16", us, nbytes=keys.numel() * 2 + keys.shape[0] * (D // 8 + 4))
    bits, mag = rq.rabitq_encode(keys, diag)
    v = torch.randn(B, H, S, D, device="cuda", dtype=torch.float16)
    q = torch.randn(B, 32, 1, D, device="cuda", dtype=torch.float16)
    qs = torch.full((B, 32, 1), 0.01, device="cuda")
    us = _time_us(lambda: rq.rabitq_fused_attend(q, qs, bits.view(B, H, S, D // 8), mag.view(B, H, S), None, v, None), a.iters)
    _line("rabitq_attend", f"B={B} H_q=32 H_kv={H} S={S} dense f16 values", us, nbytes=B * H * S * (D // 8 + 4 + 2 * D))


def op_rvq(a):
    """TurboQuant-RVQ quantize+pack and unpack+decode of 1 Mi rotated key vectors (head_dim 128)."""
    from . import rvq

    N, D = 8 * 8 * 16384, 128
    for bits in (2, 4):
        q = rvq.TurboQuantRVQ(D, bits, use_hadamard=True)
        y = (torch.randn(N, D, device="cuda") / D ** 0.5).to(torch.float16)
        c1, c2 = q._codebook1, q._codebook2
        us = _time_us(lambda: rvq.rvq_quant_pack(y, c1.centroids, c1.boundaries, c2.boundaries, bits), a.iters)
        nw = rvq.n_words_for(D, bits)
        _line("rvq_quant_pack", f"[{N},{D}] f16 b={bits}", us, nbytes=N * D * 2 + 2 * N * nw * 4)
        p1, p2 = rvq.rvq_quant_pack(y, c1.centroids, c1.boundaries, c2.boundaries, bits)
        norms = torch.ones(N, device="cuda", dtype=torch.bfloat16)
        diag = q._rot("cuda")
        us = _time_us(lambda: rvq.rvq_unpack_decode(p1, p2, norms, c1.centroids, c2.centroids, diag, bits, D), a.iters)
        _line("rvq_unpack_decode", f"[{N},{D}] b={bits} -> f16", us, nbytes=N * D * 2 + 2 * N * nw * 4 + N * 2)


def op_skvq(a):
    """SKVQ clipped group quantize+pack (clip-factor search / one factor, with and without a channel
    permutation) and unpack+dequantize of 1 Mi rows (head_dim 128, groups of 32)."""
    from . import skvq

    n_bh, n_tok, D = 64, 16384, 128
    x = torch.randn(n_bh, n_tok, D, device="cuda", dtype=_DT[a.dtype])
    perm = torch.stack([torch.randperm(D, device="cuda") for _ in range(8)]).to(torch.int32)
    for bits in (2, 4):
        out = skvq.quantize_pack(x, bits, 32)
        nb = x.numel() * x.element_size() + x.numel() * bits // 8 + 2 * (x.numel() // 32) * 4
        for label, alphas, p in (("search5", skvq.DEFAULT_ALPHA_GRID, None), ("search5+perm", skvq.DEFAULT_ALPHA_GRID, perm),
                                 ("fixed", (0.94,), None)):
            us = _time_us(lambda: skvq.quantize_pack(x, bits, 32, alphas, perm=p, out=out), a.iters)
            _line("skvq_quant_pack", f"[{n_bh * n_tok},{D}] {a.dtype} b={bits} {label}", us, nbytes=nb)
        y = torch.empty_like(x)
        inv = torch.argsort(perm.long(), dim=-1).to(torch.int32)
        for label, ip in (("", None), ("+perm", inv)):
            us = _time_us(lambda: skvq.unpack_dequant(*out, bits, 32, n_tok, x.dtype, inv_perm=ip, out=y), a.iters)
            _line("skvq_unpack_dequant", f"[{n_bh * n_tok},{D}] b={bits} -> {a.dtype} {label}", us, nbytes=nb)


def op_kivi_attend(a):
    """Decode attention over a KIVI cache at the small benchmark shapes (config 1 and config 5, one layer)."""
    from .cache import KVCacheConfig, KVCacheFactory

    for name, B, Hq, Hkv, S, bits in (("config1", 1, 32, 8, 4096, 2), ("config5", 4, 40, 8, 16384 + 256, 2)):
        cache = KVCacheFactory.create(KVCacheConfig(method="kivi", bit_width_inlier=bits, fused_sdpa_memory_bound=True))
        kk = torch.randn(B, Hkv, S, 128, device="cuda", dtype=torch.float16)
        vv = torch.randn(B, Hkv, S, 128, device="cuda", dtype=torch.float16)
        cache.update_and_fetch(kk, vv)
        q = torch.randn(B, Hq, 1, 128, device="cuda", dtype=torch.float16)
        out = torch.empty_like(q)
        us = _time_us(lambda: cache.fused_sdpa(q, 128 ** -0.5, out=out), a.iters)
        nq = cache._n_quantized
        R = S - nq
        nb = B * (Hkv * (2 * nq * 128 * bits // 8 + (nq // 32) * 128 * 8 + nq * 4 * 8 + 2 * R * 128 * 2) + 2 * Hq * 128 * 2)
        _line("kivi_attend", f"{name}: B={B} H_q={Hq} H_kv={Hkv} S={S} b={bits}", us, nbytes=nb)


OPS = {"kivi_attend": op_kivi_attend, "kivi_quantize": op_kivi_quantize, "vq_quantize": op_vq_quantize, "vq_encode": op_vq_encode,
       "vq_attend": op_vq_attend, "rabitq": op_rabitq, "rvq": op_rvq, "skvq": op_skvq}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--op", choices=sorted(OPS) + ["all"], default="all")
    ap.add_argument("--dtype", choices=sorted(_DT), default="float16")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--batch", type=int, default=4, help="batch of the kivi_quantize shape")
    ap.add_argument("--ctx", type=int, default=32768, help="context of the kivi_quantize shape")
    ap.add_argument("--search", type=int, default=0, choices=range(5),
                    help="vq_quantize: 0 choose, 1 tcgen05, 2 mma.sync, 3 exact, 4 tcgen05 with the two-pass epilogue")
    ap.add_argument("--graph", action="store_true", help="time CUDA-graph replays (GPU time without launch overhead)")
    a = ap.parse_args(argv)
    global _USE_GRAPH
    _USE_GRAPH = a.graph
    if not torch.cuda.is_available():
        raise SystemExit("microbench needs a CUDA device")
    for name in (sorted(OPS) if a.op == "all" else [a.op]):
        OPS[name](a)


if __name__ == "__main__":
    main()
