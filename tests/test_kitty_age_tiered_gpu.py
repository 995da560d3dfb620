"""Kitty and AgeTieredKV on the GPU: quantizer functions against the golden vectors (the reference's
modules run over NumPy) and the caches against the oracle's dense models."""

import os

import numpy as np
import pytest
import torch

from oracle import age_tiered as o_age
from oracle import kitty as o_kitty

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _make(method, **cfg):
    from veloxquant_mlx_b200.cache import KVCacheConfig, KVCacheFactory

    return KVCacheFactory.create(KVCacheConfig(method=method, **cfg))


def test_quantizer_functions_match_golden_vectors():
    from veloxquant_mlx_b200 import age_tiered as at
    from veloxquant_mlx_b200 import kitty
    from veloxquant_mlx_b200 import quant_utils as qu

    z = np.load(os.path.join(GOLDEN, "group_quant.npz"))
    for tag in "abcd":
        x = z[f"gq_{tag}_x"]
        b, gs = (int(v) for v in z[f"gq_{tag}_meta"])
        codes, scale, zero = qu._group_quant_codes_batched(_t(x), b, gs)
        np.testing.assert_array_equal(codes.cpu().numpy(), z[f"gq_{tag}_codes"])
        np.testing.assert_array_equal(scale.cpu().numpy(), z[f"gq_{tag}_scale"])
        np.testing.assert_array_equal(zero.cpu().numpy(), z[f"gq_{tag}_zero"])
        np.testing.assert_array_equal(qu._group_quant_dequant_batched(_t(x), b, gs).cpu().numpy(), z[f"gq_{tag}_rt"])
    mask = kitty.hi_mask_from_variance_batched(_t(z["kitty_var"]), 0.25)
    np.testing.assert_array_equal(mask.cpu().numpy(), z["kitty_mask"])
    np.testing.assert_array_equal(kitty.quantize_mixed_channels_batched(_t(z["kitty_x"]), mask).cpu().numpy(), z["kitty_out"])
    kx = _t(z["kitty_x"]).float()
    np.testing.assert_allclose(kitty.compute_running_variance(kx.sum(1)[0], (kx ** 2).sum(1)[0], 96).cpu().numpy(),
                               z["kitty_running_var"], rtol=1e-5)
    # explicit index lists == the mask form; channels in neither list pass through
    hi, lo = kitty.rank_channels_by_sensitivity(_t(z["kitty_x"][0]), 0.25)
    assert hi == np.nonzero(z["kitty_mask"][0])[0].tolist() and sorted(hi + lo) == list(range(64))
    one = kitty.quantize_mixed_channels(_t(z["kitty_x"][0]), hi, lo)
    np.testing.assert_array_equal(one.cpu().numpy(), z["kitty_out"][0])
    tiers = at.default_age_tiers(8, 4, 2)
    assert at.assign_age_tiers([200 - (i + 1) for i in range(200)], 40, 120) == list(z["age_tok_tier"])
    out = at.age_tier_quantize_batched(_t(z["age_x"]), list(z["age_group_tier"]), tiers, 32)
    np.testing.assert_array_equal(out.cpu().numpy(), z["age_out"])
    assert [at.age_tiered_bytes({0: 40, 1: 80, 2: 80}, tiers, 32), at.full_fp16_bytes(200, 32)] == list(z["age_bytes"])


def _het(d, seed):
    s = np.logspace(-1, 1, d)
    np.random.default_rng(seed).shuffle(s)
    return s


def test_kitty_cache_equals_the_dense_model():
    """Prefill block, a second multi-token block, then single tokens: returned keys equal the oracle's
    model bit for bit (ranking from the block, then from running statistics; one-token blocks come
    back exactly), values untouched, accounting and trim as the reference."""
    B, H, D = 2, 3, 64
    rng = np.random.default_rng(3)
    k = (rng.standard_normal((B, H, 120, D)) * _het(D, 1)[None, None, None, :]).astype(np.float16)
    v = rng.standard_normal((B, H, 120, D)).astype(np.float16)
    c, m = _make("kitty", head_dim=D), o_kitty.KittyCacheModel(D)
    assert not hasattr(c, "bits") and c.assigned_avg_bits == 2.5
    for lo, hi in [(0, 70), (70, 110)] + [(t, t + 1) for t in range(110, 120)]:
        ko, vo = c.update_and_fetch(_t(k[:, :, lo:hi]), _t(v[:, :, lo:hi]))
        mk, mv = m.update_and_fetch(k[:, :, lo:hi], v[:, :, lo:hi])
        np.testing.assert_array_equal(ko.cpu().numpy(), mk)
        np.testing.assert_array_equal(vo.cpu().numpy(), mv)
    assert np.array_equal(ko[:, :, 110:].cpu().numpy(), k[:, :, 110:])           # one-token groups are exact
    assert not np.array_equal(ko[:, :, :70].cpu().numpy(), k[:, :, :70])
    assert (c.compressed_key_bytes, c.fp16_key_bytes, c.value_fp16_bytes) == (m.compressed_key_bytes, m.fp16_key_bytes, m.value_fp16_bytes)
    q = torch.randn(B, 6, 1, D, device=DEV, dtype=torch.float16)
    want = torch.nn.functional.scaled_dot_product_attention(q, ko.repeat_interleave(2, 1), vo.repeat_interleave(2, 1), scale=0.125)
    torch.testing.assert_close(c.fused_sdpa(q, 0.125), want)
    before = c.fp16_key_bytes
    assert c.trim(5) == 5 and c.offset == 115 and c.fp16_key_bytes == before - B * H * 5 * D * 2 and c._n_keys == 115
    from veloxquant_mlx_b200.cache import QuantizerConfigError
    with pytest.raises(QuantizerConfigError, match="kitty_hi_fraction"):
        _make("kitty", head_dim=D, kitty_hi_fraction=1.5)


@pytest.mark.parametrize("dt", [np.float16, "bfloat16"])
def test_age_tiered_cache_equals_the_dense_model(dt):
    """Prefill past both boundaries, then decode across group and tier boundaries: the returned
    tensors equal the oracle's recompute-everything-from-raw model bit for bit after every call, while
    the cache holds raw rows only for the groups that are not final."""
    B, H, D, gs = 2, 2, 32, 8
    rng = np.random.default_rng(5)
    k32 = rng.standard_normal((B, H, 150, D)).astype(np.float32)
    v32 = rng.standard_normal((B, H, 150, D)).astype(np.float32)
    if dt == "bfloat16":
        kt, vt = torch.from_numpy(k32).to(torch.bfloat16), torch.from_numpy(v32).to(torch.bfloat16)
        k, v = kt.float().numpy(), vt.float().numpy()      # the model works on the bf16 values ...
    else:
        k, v = k32.astype(np.float16), v32.astype(np.float16)
        kt, vt = torch.from_numpy(k), torch.from_numpy(v)
    c = _make("age_tiered", head_dim=D, age_recent_boundary=20, age_mid_boundary=50, age_group_size=gs)
    m = o_age.AgeTieredCacheModel(D, 20, 50, (8, 4, 2), gs)
    for lo, hi in [(0, 93)] + [(t, t + 1) for t in range(93, 130)] + [(130, 150)]:
        ko, vo = c.update_and_fetch(kt[:, :, lo:hi].to(DEV), vt[:, :, lo:hi].to(DEV))
        mk, mv = m.update_and_fetch(k[:, :, lo:hi], v[:, :, lo:hi])
        if dt == "bfloat16":   # ... and rounds float16 results to bfloat16 as the cache's storage does
            mk = torch.from_numpy(mk.astype(np.float32)).to(torch.bfloat16).float().numpy()
            mv = torch.from_numpy(mv.astype(np.float32)).to(torch.bfloat16).float().numpy()
        np.testing.assert_array_equal(ko.float().cpu().numpy(), mk.astype(np.float32))
        np.testing.assert_array_equal(vo.float().cpu().numpy(), mv.astype(np.float32))
    assert c.offset == 150 and c.tokens_kept == 150 and c.tokens_seen == B * H * 150
    assert c.age_tiered_bytes == m.age_tiered_bytes and c.full_seq_bytes == m.full_seq_bytes and c.compression_ratio > 1.0
    assert c.tokens_recent == 20 * B * H and c.tokens_mid == 30 * B * H and c.tokens_old == 100 * B * H
    # final groups: first token (index 8g) has age 150 - (8g + 1) >= 50 for g <= 12 -> 13 whole groups packed; the rest raw
    assert c._n_final == 104 and c._raw_k.shape[1] == 46 and not c.is_trimmable()
    # resident: 2-bit codes + float32 (scale, zero) per 8 tokens and channel for the final groups, raw 16-bit rows for the rest
    assert c.nbytes == 2 * B * H * D * (104 * 2 // 8 + (104 // gs) * 8 + 46 * 2) < c.full_seq_bytes
    q = torch.randn(B, 4, 1, D, device=DEV, dtype=ko.dtype)
    want = torch.nn.functional.scaled_dot_product_attention(q, ko.repeat_interleave(2, 1), vo.repeat_interleave(2, 1), scale=0.2)
    torch.testing.assert_close(c.fused_sdpa(q, 0.2), want)
    from veloxquant_mlx_b200.cache import QuantizerConfigError
    with pytest.raises(QuantizerConfigError, match="age_mid_boundary"):
        _make("age_tiered", head_dim=D, age_recent_boundary=64, age_mid_boundary=32)
    with pytest.raises(QuantizerConfigError, match="age_bits_old"):
        _make("age_tiered", head_dim=D, age_bits_old=0)


@pytest.mark.parametrize("method,cfg", [("kitty", dict(kitty_group_size=8)),
                                        ("age_tiered", dict(age_recent_boundary=20, age_mid_boundary=50, age_group_size=8))])
def test_saved_and_restored_caches_continue_bit_identically(method, cfg, tmp_path):
    """``save_prompt_cache`` / ``load_prompt_cache`` of a Kitty and an AgeTieredKV cache mid-sequence:
    the restored cache returns exactly what the uninterrupted one returns for the tokens that follow."""
    from veloxquant_mlx_b200.cache import KVCacheConfig
    from veloxquant_mlx_b200.persistence import load_prompt_cache, save_prompt_cache

    B, H, D = 2, 2, 32
    rng = np.random.default_rng(9)
    k = (rng.standard_normal((B, H, 130, D)) * _het(D, 2)[None, None, None, :]).astype(np.float16)
    v = rng.standard_normal((B, H, 130, D)).astype(np.float16)
    c = _make(method, head_dim=D, **cfg)
    c.update_and_fetch(_t(k[:, :, :90]), _t(v[:, :, :90]))
    c.update_and_fetch(_t(k[:, :, 90:91]), _t(v[:, :, 90:91]))
    path = str(tmp_path / f"{method}.safetensors")
    save_prompt_cache(path, [c])
    (d,) = load_prompt_cache(path, KVCacheConfig(method=method, head_dim=D, **cfg), device=DEV)
    assert d.offset == 91
    q = torch.randn(B, 4, 1, D, device=DEV, dtype=torch.float16)
    assert torch.equal(c.fused_sdpa(q, 0.2), d.fused_sdpa(q, 0.2))
    for lo, hi in [(91, 92), (92, 120), (120, 121), (121, 130)]:
        a = c.update_and_fetch(_t(k[:, :, lo:hi]), _t(v[:, :, lo:hi]))
        b = d.update_and_fetch(_t(k[:, :, lo:hi]), _t(v[:, :, lo:hi]))
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
