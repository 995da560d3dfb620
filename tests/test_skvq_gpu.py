"""SKVQ on the GPU: the packed quantizer / dequantizer against the oracle and the golden vectors,
and the cache against the oracle's dense model, following the reference's own tests
(veloxquant_mlx/tests/quantizers/test_skvq.py, tests/cache/test_skvq_cache.py)."""

import os

import numpy as np
import pytest
import torch

from oracle import bitpack as o_bitpack
from oracle import skvq as o_skvq

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _s():
    from veloxquant_mlx_b200 import skvq

    return skvq


def _het_scales(d, seed=3):
    rng = np.random.default_rng(seed)
    scales = np.logspace(-2, 1, d)
    rng.shuffle(scales)
    return scales


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


# ------------------------------------------------------------------------------- quantizer
@pytest.mark.parametrize("tag", list("abcde"))
def test_quantizer_matches_golden_vectors(tag):
    """Codes, lo, scale (searched and fixed clip factor), permutation and permuted round trip equal
    the outputs of the reference's module run over NumPy, bit for bit."""
    s = _s()
    z = np.load(os.path.join(GOLDEN, "skvq.npz"))
    x = z[f"{tag}_x"]
    bits, gs = (int(v) for v in z[f"{tag}_meta"])
    xt = _t(x)
    for suffix, alphas in (("", s.DEFAULT_ALPHA_GRID), ("_a90", (0.9,))):
        codes, lo, scale = s.clipped_group_quant(xt, bits, gs, alphas)
        assert codes.dtype == torch.uint8 and lo.dtype == torch.float32
        np.testing.assert_array_equal(codes.cpu().numpy(), z[f"{tag}_codes{suffix}"])
        np.testing.assert_array_equal(lo.cpu().numpy(), z[f"{tag}_lo{suffix}"])
        np.testing.assert_array_equal(scale.cpu().numpy(), z[f"{tag}_scale{suffix}"])
    perm = s.channel_permutation(xt)
    np.testing.assert_array_equal(perm.cpu().numpy(), z[f"{tag}_perm"])
    np.testing.assert_array_equal(s.invert_permutation(perm).cpu().numpy(), z[f"{tag}_inv"])
    rt = s.skvq_round_trip(xt, perm, bits, gs)
    assert rt.dtype == xt.dtype
    np.testing.assert_array_equal(rt.cpu().numpy(), z[f"{tag}_rt"])


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("bits", [1, 2, 3, 4, 5, 6, 7, 8])
@pytest.mark.parametrize("gs,D", [(8, 64), (16, 64), (32, 128), (64, 128), (32, 256)])
def test_packed_quantizer_bit_exact_vs_oracle(dt, bits, gs, D):
    """Every width and group size: packed bytes = the oracle's codes packed LSB-first, (lo, scale)
    equal, and the dequantizer restores the oracle's reconstruction; with and without a per-head
    permutation, from a strided source and into an offset of a larger buffer."""
    s = _s()
    rng = np.random.default_rng(bits * 1000 + gs + D)
    n_bh, n_tok, H = 6, 37, 3
    x = rng.standard_normal((n_bh, 50, D)) * _het_scales(D)[None, None, :]
    x[rng.random(x.shape) < 0.03] *= 20.0
    x[0, 0, :gs] = 0.5                                    # constant group
    xt = _t(x.astype(np.float32)).to(dt)
    x32 = xt.float().cpu().numpy()[:, :n_tok]
    perm = np.stack([rng.permutation(D) for _ in range(H)]).astype(np.int32)
    for p in (None, perm):
        xp = x32 if p is None else np.take_along_axis(x32, np.broadcast_to(p[np.arange(n_bh) % H][:, None, :], x32.shape), axis=-1)
        codes, lo, scale = o_skvq.clipped_group_quant(xp.reshape(-1, D), bits, gs)
        G = D // gs
        bufs = (torch.zeros((n_bh, 64, D * bits // 8), dtype=torch.uint8, device=DEV),
                torch.zeros((n_bh, 64, G), dtype=torch.float32, device=DEV), torch.zeros((n_bh, 64, G), dtype=torch.float32, device=DEV))
        s.quantize_pack(xt[:, :n_tok], bits, gs, perm=None if p is None else _t(p), out=bufs, tok_offset=5)
        got = bufs[0][:, 5:5 + n_tok].cpu().numpy()
        np.testing.assert_array_equal(got.reshape(-1, D * bits // 8), o_bitpack.pack(codes, bits).reshape(-1, D * bits // 8))
        np.testing.assert_array_equal(bufs[1][:, 5:5 + n_tok].cpu().numpy().reshape(-1, G), lo)
        np.testing.assert_array_equal(bufs[2][:, 5:5 + n_tok].cpu().numpy().reshape(-1, G), scale)
        assert int(bufs[0][:, :5].sum()) == 0 and int(bufs[0][:, 5 + n_tok:].sum()) == 0
        recon = o_skvq.clipped_group_dequant(codes, lo, scale, gs, D).reshape(n_bh, n_tok, D)
        inv = None
        if p is not None:
            inv = np.argsort(p, axis=-1, kind="stable").astype(np.int32)
            recon = np.take_along_axis(recon, np.broadcast_to(inv[np.arange(n_bh) % H][:, None, :], recon.shape), axis=-1)
        packed = tuple(b[:, 5:5 + n_tok].contiguous() for b in bufs)
        out = s.unpack_dequant(*packed, bits, gs, n_tok, dt, inv_perm=None if inv is None else _t(inv))
        want = torch.from_numpy(recon).to(dt)
        assert torch.equal(out.cpu(), want)


def test_quantizer_properties_and_guards():
    """alpha = 1 equals plain min/max (up to a step on boundary elements); the search is never worse per
    group; errors fall with the width; reordering wins on heterogeneous channels; the reference's guards."""
    s = _s()
    rng = np.random.default_rng(6)
    x = rng.standard_normal((128, 32)).astype(np.float32)
    x[rng.random((128, 32)) < 0.03] *= 20.0
    xt = _t(x)

    def per_group_mse(alphas, bits=2):
        c, lo, sc = s.clipped_group_quant(xt, bits, 8, alphas)
        r = s.clipped_group_dequant(c, lo, sc, 8, 32)
        return ((r - xt) ** 2).reshape(128, 4, 8).mean(-1)

    assert bool((per_group_mse(s.DEFAULT_ALPHA_GRID) <= per_group_mse((1.0,)) + 1e-9).all())
    errs = [float(per_group_mse(s.DEFAULT_ALPHA_GRID, b).mean()) for b in (2, 3, 4, 6, 8)]
    assert all(a > b for a, b in zip(errs, errs[1:]))
    het = _t((rng.standard_normal((256, 64)) * _het_scales(64)[None, :]).astype(np.float32))
    perm = s.channel_permutation(het)
    e_perm = float(((s.skvq_round_trip(het, perm, 2, 16) - het) ** 2).mean())
    e_id = float(((s.skvq_round_trip(het, None, 2, 16) - het) ** 2).mean())
    assert e_perm < e_id
    back = s.apply_permutation(s.apply_permutation(het, perm), s.invert_permutation(perm))
    assert torch.equal(back, het)
    half = het.half()
    assert s.skvq_round_trip(half, perm, 4, 16).dtype == torch.float16
    with pytest.raises(ValueError, match=r"bits=0 must be in \[1, 8\]"):
        s.clipped_group_quant(xt, 0, 8)
    with pytest.raises(ValueError, match="group_size=0 must be >= 1"):
        s.clipped_group_quant(xt, 2, 0)
    with pytest.raises(ValueError, match="alphas must be non-empty"):
        s.clipped_group_quant(xt, 2, 8, ())
    with pytest.raises(ValueError, match=r"alpha=1.5 must be in \(0, 1\]"):
        s.clipped_group_quant(xt, 2, 8, (1.5,))
    with pytest.raises(ValueError, match="ragged last group"):
        s.clipped_group_quant(xt[:, :30].contiguous(), 2, 8)
    assert s.skvq_compressed_bytes(10, 64, 2, 16) == 10 * 64 * 2 // 8 + 10 * 4 * 4 and s.skvq_fp16_bytes(10, 64) == 1280


# ------------------------------------------------------------------------------------ cache
def _kv(B, H, S, D, seed=0, channel_scales=None, dt=np.float16):
    rng = np.random.default_rng(seed)
    k = rng.standard_normal((B, H, S, D)).astype(np.float32)
    v = rng.standard_normal((B, H, S, D)).astype(np.float32)
    if channel_scales is not None:
        cs = channel_scales.astype(np.float32)[None, None, None, :]
        k, v = k * cs, v * cs
    return k.astype(dt), v.astype(dt)


def _make(**cfg):
    from veloxquant_mlx_b200.cache import KVCacheConfig, KVCacheFactory

    base = {"method": "skvq", "head_dim": 64, "skvq_window": 16, "skvq_n_sink": 4, "skvq_group_size": 16,
            "skvq_bits_key": 2, "skvq_bits_value": 2}
    base.update(cfg)
    return KVCacheFactory.create(KVCacheConfig(**base))


def _model(**cfg):
    base = dict(head_dim=64, bits_k=2, bits_v=2, group_size=16, window=16, n_sink=4)
    base.update(cfg)
    return o_skvq.SKVQCacheModel(**base)


def test_cache_defaults_factory_and_short_sequence_passthrough():
    from veloxquant_mlx_b200.cache import KVCacheConfig, KVCacheFactory, SKVQKVCache

    c = KVCacheFactory.create(KVCacheConfig(method="skvq", head_dim=64))
    assert isinstance(c, SKVQKVCache) and (c._bits_k, c._bits_v) == (4, 4)
    c = _make()
    assert not hasattr(c, "bits") and c.assigned_avg_bits == 16.0 and not c.is_trimmable()
    k, v = _kv(1, 2, 10, 64, seed=1)
    ko, vo = c.update_and_fetch(_t(k), _t(v))
    assert ko.dtype == torch.float16 and np.array_equal(ko.cpu().numpy(), k) and np.array_equal(vo.cpu().numpy(), v)
    assert c.quantized_tokens == 0 and c.compressed_key_bytes == 0 and c.offset == 10
    with pytest.raises(AttributeError):
        c.merge


@pytest.mark.parametrize("het", [False, True])
@pytest.mark.parametrize("cfg", [{}, {"skvq_reorder": False}, {"skvq_clip_search": False, "skvq_clip_alpha": 0.9},
                                 {"skvq_bits_key": 4, "skvq_bits_value": 3, "skvq_n_sink": 0},
                                 {"head_dim": 128, "skvq_group_size": 32, "skvq_window": 32, "skvq_n_sink": 5}])
def test_cache_equals_the_dense_model_prefill_and_decode(het, cfg):
    """Prefill of 3 chunks + 5, then token-by-token decode across two more chunk boundaries: what
    ``update_and_fetch`` returns equals the oracle's dense model after every call, bit for bit
    (frontier in whole chunks, sink rows exact, permutations from the first chunk only), and one
    prefill of all tokens gives the same final state as the streamed run."""
    D = cfg.get("head_dim", 64)
    r = cfg.get("skvq_window", 16)
    B, H, S0, n_dec = 2, 3, 3 * r + 5, 2 * r + 3
    k, v = _kv(B, H, S0 + n_dec, D, seed=7, channel_scales=_het_scales(D) if het else None)
    names = {"skvq_bits_key": "bits_k", "skvq_bits_value": "bits_v", "skvq_group_size": "group_size", "skvq_window": "window",
             "skvq_n_sink": "n_sink", "skvq_reorder": "reorder", "skvq_clip_search": "clip_search", "skvq_clip_alpha": "clip_alpha",
             "head_dim": "head_dim"}
    c, m = _make(**cfg), _model(**{names[a]: b for a, b in cfg.items()})
    ko, vo = c.update_and_fetch(_t(k[:, :, :S0]), _t(v[:, :, :S0]))
    mk, mv = m.update_and_fetch(k[:, :, :S0], v[:, :, :S0])
    assert c.quantized_tokens == 3 * r == m.q_end
    np.testing.assert_array_equal(ko.cpu().numpy(), mk)
    np.testing.assert_array_equal(vo.cpu().numpy(), mv)
    if m.perm_k is not None:
        np.testing.assert_array_equal(c.key_perms.cpu().numpy(), m.perm_k)
        np.testing.assert_array_equal(c.value_perms.cpu().numpy(), m.perm_v)
    else:
        assert c.key_perms is None
    for t in range(S0, S0 + n_dec):
        ko, vo = c.update_and_fetch(_t(k[:, :, t:t + 1]), _t(v[:, :, t:t + 1]))
        mk, mv = m.update_and_fetch(k[:, :, t:t + 1], v[:, :, t:t + 1])
        if (t + 1) % r == 0 or t == S0 + n_dec - 1:
            np.testing.assert_array_equal(ko.cpu().numpy(), mk)
            np.testing.assert_array_equal(vo.cpu().numpy(), mv)
    assert c.compressed_key_bytes == m.compressed_key_bytes and c.compressed_value_bytes == m.compressed_value_bytes
    one = _make(**cfg)
    k1, v1 = one.update_and_fetch(_t(k), _t(v))
    assert torch.equal(k1, ko) and torch.equal(v1, vo)
    n_sink = cfg.get("skvq_n_sink", 4)
    if n_sink:
        assert np.array_equal(ko[:, :, :n_sink].cpu().numpy(), k[:, :, :n_sink])
    q = slice(max(n_sink, 1), 5 * r)
    assert not np.array_equal(ko[:, :, q].cpu().numpy(), k[:, :, q])


def test_cache_accounting_guards_and_compression():
    from veloxquant_mlx_b200.cache import QuantizerConfigError
    from veloxquant_mlx_b200.skvq import skvq_compressed_bytes

    B, H, D, r, n_sink, gs = 1, 2, 64, 16, 4, 16
    c = _make()
    k, v = _kv(B, H, 2 * r + 3, D, seed=12)
    c.update_and_fetch(_t(k), _t(v))
    expect = (skvq_compressed_bytes(r - n_sink, D, 2, gs) + skvq_compressed_bytes(r, D, 2, gs)) * B * H
    assert c.compressed_key_bytes == expect == c.compressed_value_bytes
    assert c.fp16_key_bytes == B * H * (2 * r + 3) * D * 2
    assert c.residual_fp16_bytes == (3 + n_sink) * D * 2 * 2 * B * H
    assert c.perm_bytes == 2 * H * D * 4 and 2.0 < c.assigned_avg_bits < 16.0 and c.tokens_seen == 2 * r + 3
    big = _make(skvq_window=32, skvq_n_sink=4, skvq_max_ctx=4096)
    k, v = _kv(1, 2, 1024, 64, seed=13)
    big.update_and_fetch(_t(k), _t(v))
    ratio = (big.compressed_key_bytes + big.compressed_value_bytes + big.residual_fp16_bytes + big.perm_bytes) / (
        big.fp16_key_bytes + big.fp16_value_bytes)
    assert ratio < 0.35
    # resident bytes: 2-bit codes + float32 (lo, scale) per 16 channels = 6 bits per element, + window, sinks, permutations
    assert big.nbytes < 0.45 * (big.fp16_key_bytes + big.fp16_value_bytes)
    capped = _make(skvq_max_ctx=32)
    k, v = _kv(1, 2, 33, 64, seed=15)
    with pytest.raises(ValueError, match="skvq_max_ctx"):
        capped.update_and_fetch(_t(k), _t(v))
    for bad, pat in (({"skvq_bits_key": 0}, "skvq_bits_key"), ({"skvq_bits_value": 9}, "skvq_bits_value"),
                     ({"skvq_group_size": 0}, "skvq_group_size"), ({"skvq_window": 1}, "skvq_window"),
                     ({"skvq_n_sink": 16}, "skvq_n_sink"), ({"skvq_clip_alpha": 0.0}, "skvq_clip_alpha"),
                     ({"skvq_group_size": 24}, "8, 16, 32 or 64")):
        with pytest.raises(QuantizerConfigError, match=pat):
            _make(**bad)


def test_cache_attention_persistence_and_standalone_protocol(tmp_path):
    """``fused_sdpa`` = attention over the dense view; save / load restores a cache that continues
    bit-identically; the one-vector-per-call protocol runs on top."""
    from veloxquant_mlx_b200.cache import KVCacheConfig
    from veloxquant_mlx_b200.persistence import load_prompt_cache, save_prompt_cache

    B, H, D = 2, 2, 64
    k, v = _kv(B, H, 70, D, seed=21, channel_scales=_het_scales(D))
    c = _make()
    ko, vo = c.update_and_fetch(_t(k[:, :, :50]), _t(v[:, :, :50]))
    q = torch.randn(B, 4, 1, D, device=DEV, dtype=torch.float16)
    want = torch.nn.functional.scaled_dot_product_attention(q, ko.repeat_interleave(2, 1), vo.repeat_interleave(2, 1), scale=0.125)
    torch.testing.assert_close(c.fused_sdpa(q, 0.125), want, atol=2e-3, rtol=1e-2)
    path = str(tmp_path / "skvq.safetensors")
    save_prompt_cache(path, [c])
    cfg = KVCacheConfig(method="skvq", head_dim=64, skvq_window=16, skvq_n_sink=4, skvq_group_size=16, skvq_bits_key=2, skvq_bits_value=2)
    (d,) = load_prompt_cache(path, cfg, device=DEV)
    assert d.offset == 50 and d.quantized_tokens == 48 and d.compressed_key_bytes == c.compressed_key_bytes
    a = c.update_and_fetch(_t(k[:, :, 50:]), _t(v[:, :, 50:]))
    b = d.update_and_fetch(_t(k[:, :, 50:]), _t(v[:, :, 50:]))
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    one = _make(skvq_window=4, skvq_n_sink=1, skvq_group_size=16)
    rows = torch.randn(9, 2, D, device=DEV, dtype=torch.float16)
    for kk, vv in rows:
        one.append(kk, vv)
    assert len(one) == 9 and one.quantized_tokens == 8 and one.memory_bytes() > 0
    assert one.attend(rows[0, 0]).shape == (D,)
    one.reset()
    assert len(one) == 0 and one.quantized_tokens == 0
