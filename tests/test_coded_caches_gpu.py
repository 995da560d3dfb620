"""VecInfer and RaBitQ caches on the GPU against the oracle (reference semantics:
tests/cache/test_vecinfer_fused_sdpa.py:189-540, test_vecinfer_gqa_smooth.py:67-109,
test_vecinfer_memory_bound_state.py)."""

from __future__ import annotations

import math
import warnings

import numpy as np
import pytest
import torch

from oracle import rabitq as o_rq
from oracle import vq as o_vq

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _make(method, **kw):
    from veloxquant_mlx_b200.cache import KVCacheConfig, KVCacheFactory

    kw.setdefault("head_dim", 128)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", UserWarning)
        return KVCacheFactory.create(KVCacheConfig(method=method, **kw))


def _kv(B, H, S, D, seed, scale=0.3):
    rng = np.random.default_rng(seed)
    k = torch.from_numpy((rng.standard_normal((B, H, S, D)) * scale).astype(np.float32)).half().to(DEV)
    v = torch.from_numpy((rng.standard_normal((B, H, S, D)) * scale).astype(np.float32)).half().to(DEV)
    return k, v


def _codebooks(seed, sub_k=8, sub_v=8, n=256):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((n, sub_k)).astype(np.float32) * 0.3,
            rng.standard_normal((n, sub_v)).astype(np.float32) * 0.3)


@pytest.mark.parametrize("causal,window,S_q", [(True, 0, 1), (False, 0, 1), (True, 64, 1), (True, 0, 8)])
@pytest.mark.parametrize("H_q,H_kv", [(4, 4), (32, 8)])
def test_vecinfer_fused_matches_reference_sdpa(causal, window, S_q, H_q, H_kv):
    D, S = 128, 300
    cbk, cbv = _codebooks(1)
    lam = np.random.default_rng(2).uniform(0.5, 2.0, (H_kv, D)).astype(np.float32)
    c = _make("vecinfer", key_sub_dim=8, value_sub_dim=8, key_codebook_bits=8, value_codebook_bits=8,
              key_codebook=cbk, value_codebook=cbv, smooth_factors=lam, fused_sdpa=True, fused_sdpa_memory_bound=True)
    k, v = _kv(1, H_kv, S, D, seed=3)
    ko, vo = c.update_and_fetch(k, v)
    assert ko.shape[2] == 0 and c.offset == S and not hasattr(c, "bits")
    q = torch.from_numpy((np.random.default_rng(4).standard_normal((1, H_q, S_q, D)) * 0.3).astype(np.float32)).half().to(DEV)
    out = c.fused_sdpa(q, 1.0 / math.sqrt(D), causal=causal, sliding_window=window)
    assert out.dtype == torch.float16
    # oracle: same transforms in float32, indices from the oracle's quantizer
    k_t = o_vq.dual_transform_keys_wht(k.float().cpu().numpy(), lam)
    kidx = o_vq.quantize_vq(k_t, cbk, 8)
    vidx = o_vq.quantize_vq(v.cpu().numpy(), cbv, 8)
    q_t = o_vq.dual_transform_queries_wht(q.float().cpu().numpy(), lam)
    # the fixed-order butterfly is the dense transform up to float32 rounding
    H = o_vq.walsh_hadamard_matrix(D)
    np.testing.assert_allclose(k_t, o_vq.apply_dual_transform_keys(k.float().cpu().numpy(), lam, H), atol=2e-6)
    ref = o_vq.reference_sdpa(q_t, kidx, cbk, vidx, 1.0 / math.sqrt(D), v_codebook=cbv, causal=causal, sliding_window=window)
    got_idx = c._v_idx[:, :, :S].cpu().numpy().astype(np.int32)
    np.testing.assert_array_equal(got_idx, vidx)
    # the transform has a fixed summation order (native butterfly = oracle): every index is equal
    np.testing.assert_array_equal(c._k_idx[:, :, :S].cpu().numpy().astype(np.int32), kidx)
    err = np.abs(out.float().cpu().numpy() - ref)
    assert err.max() < 1e-2


def test_vecinfer_standard_mode_state_trim_growth_and_cap():
    D = 64
    cbk, cbv = _codebooks(5, 4, 8, 16)
    kw = dict(head_dim=D, key_sub_dim=4, value_sub_dim=8, key_codebook_bits=4, value_codebook_bits=4,
              key_codebook=cbk, value_codebook=cbv)
    c = _make("vecinfer", **kw)
    k, v = _kv(2, 2, 40, D, seed=6)
    ko, vo = c.update_and_fetch(k, v)
    assert ko.shape == k.shape and ko.dtype == torch.float16
    vref = o_vq.dequantize_vq(o_vq.quantize_vq(v.cpu().numpy(), cbv, 8), cbv)
    np.testing.assert_array_equal(vo.float().cpu().numpy(), vref.astype(np.float16).astype(np.float32))
    for t in range(300):  # growth past the initial 256-row capacity
        c.update_and_fetch(k[:, :, :1], v[:, :, :1])
    assert c.offset == 340 and c._k_idx.shape[2] == 512 and c.nbytes == 2 * 2 * 340 * (16 + 8)
    d = _make("vecinfer", **kw)
    d.state = c.state
    q = torch.randn(2, 4, 1, D, device=DEV, dtype=torch.float16)
    assert d.offset == 340 and torch.equal(c.fused_sdpa(q, 0.125), d.fused_sdpa(q, 0.125))
    assert c.trim(100) == 100 and c.offset == 240
    with pytest.raises(AttributeError, match="does not support merge"):
        c.merge
    assert not hasattr(c, "merge")
    capped = _make("vecinfer", fused_sdpa=True, fused_sdpa_memory_bound=True, fused_sdpa_max_ctx=32, **kw)
    with pytest.raises(RuntimeError, match="fused_sdpa_max_ctx"):
        capped.update_and_fetch(k, v)
    with pytest.raises(RuntimeError, match="requires fused_sdpa=True"):
        _make("vecinfer", fused_sdpa_memory_bound=True, **kw)


def test_vecinfer_smooth_rows_rules_and_random_codebook_warning():
    from veloxquant_mlx_b200.cache import KVCacheConfig, KVCacheFactory, QuantizerConfigError

    D = 64
    with pytest.warns(UserWarning, match="random N"):
        KVCacheFactory.create(KVCacheConfig(method="vecinfer", head_dim=D))
    with pytest.raises(QuantizerConfigError, match="finite and >"):
        _make("vecinfer", head_dim=D, smooth_factors=np.zeros(D, np.float32))
    k, v = _kv(1, 2, 8, D, seed=7)
    sm8 = np.random.default_rng(8).uniform(0.5, 2, (8, D)).astype(np.float32)  # per query head, GQA 4:1
    c = _make("vecinfer", head_dim=D, smooth_factors=sm8)
    c.update_and_fetch(k, v)
    np.testing.assert_allclose(c._smooth.cpu().numpy(), sm8.reshape(2, 4, D).mean(1), rtol=1e-6)
    bad = _make("vecinfer", head_dim=D, smooth_factors=sm8[:3])
    with pytest.raises(QuantizerConfigError, match="3 rows"):
        bad.update_and_fetch(k, v)


def test_rabitq_cache_matches_oracle_and_composes():
    B, H_kv, H_q, D, S = 2, 2, 8, 128, 700
    c = _make("rabitq", head_dim=D, seed=7)
    k, v = _kv(B, H_kv, S, D, seed=9, scale=1.0)
    c.update_and_fetch(k[:, :, :650], v[:, :, :650])
    for t in range(650, S):
        c.update_and_fetch(k[:, :, t : t + 1], v[:, :, t : t + 1])
    assert c.offset == S and c.assigned_avg_bits == 1.0
    diag = o_rq.make_hadamard_diagonal(D, seed=7)
    bits, mag, _ = o_rq.encode_hadamard(k.cpu().numpy().reshape(-1, D), diag)
    np.testing.assert_array_equal(c._bits[:, :, :S].cpu().numpy().reshape(-1, D // 8), bits)
    np.testing.assert_allclose(c._mag[:, :, :S].cpu().numpy().reshape(-1), mag, rtol=1e-4)
    q = torch.randn(B, H_q, 1, D, device=DEV, dtype=torch.float16)
    scale = 1.0 / math.sqrt(D)
    out = c.fused_sdpa(q, scale)
    assert out.dtype == torch.float16 and out.shape == q.shape
    q_rot = o_rq.wht_butterfly(q.float().cpu().numpy() * diag) / np.sqrt(np.float32(D))
    q_scale = np.abs(q_rot).mean(-1).astype(np.float32) * np.float32(scale)
    ref = o_rq.reference_attend(q_rot, q_scale, bits.reshape(B, H_kv, S, D // 8), mag.reshape(B, H_kv, S),
                                np.zeros((B, H_kv, S), np.float32), v.cpu().numpy())
    err = np.abs(out.float().cpu().numpy() - ref)
    assert np.all(err <= 2e-3 + 1e-2 * np.abs(ref)), err.max()
    d = _make("rabitq", head_dim=D, seed=7)
    d.state = c.state
    # the restored cache holds exact-size buffers, which take the plain-load kernel: same math, other summation order
    torch.testing.assert_close(d.fused_sdpa(q, scale).float(), out.float(), atol=2e-3, rtol=1e-2)
    assert c.trim(10) == 10 and c.offset == S - 10


@pytest.mark.parametrize("D", [32, 64, 128, 256])
@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16, torch.float32])
def test_dual_transform_butterfly_is_bit_identical_to_the_oracle(D, dt):
    """Smooth + Walsh-Hadamard butterfly (keys: divide, queries: multiply; per-head factors,
    GQA repetition on the query side, one shared factor row, no factors)."""
    from veloxquant_mlx_b200 import vecinfer as vi

    rng = np.random.default_rng(D)
    B, H_kv, H_q, S = 2, 2, 6, 37
    k = torch.from_numpy(rng.standard_normal((B, H_kv, S, D)).astype(np.float32)).to(dt).to(DEV)
    q = torch.from_numpy(rng.standard_normal((B, H_q, 3, D)).astype(np.float32)).to(dt).to(DEV)
    for lam in (rng.uniform(0.5, 2.0, (H_kv, D)).astype(np.float32), rng.uniform(0.5, 2.0, (D,)).astype(np.float32),
                rng.uniform(0.5, 2.0, (1, D)).astype(np.float32), None):
        lt = None if lam is None else torch.from_numpy(lam).to(DEV)
        got_k = vi.dual_transform_keys_wht(k, lt)
        got_q = vi.dual_transform_queries_wht(q, lt)
        assert got_k.dtype == torch.float32 and got_k.shape == k.shape
        np.testing.assert_array_equal(got_k.cpu().numpy(), o_vq.dual_transform_keys_wht(k.float().cpu().numpy(), lam))
        np.testing.assert_array_equal(got_q.cpu().numpy(), o_vq.dual_transform_queries_wht(q.float().cpu().numpy(), lam))
    with pytest.raises(ValueError, match="must be 32, 64, 128 or 256"):
        vi.dual_transform_keys_wht(torch.zeros(2, 48, device=DEV))
    assert vi.wht_entry(128) == float(o_vq.walsh_hadamard_matrix(128)[0, 0])
