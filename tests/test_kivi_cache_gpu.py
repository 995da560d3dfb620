"""Packed KIVI cache on the GPU against the oracle and the reference cache's semantics
(tests/cache/test_kivi_cache.py:40-221, tests/cache/test_trim_rollback.py:27-48)."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from oracle import kivi as o_kivi

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _make(**kw):
    from veloxquant_mlx_b200.cache import KVCacheConfig, KVCacheFactory

    kw.setdefault("head_dim", 128)
    return KVCacheFactory.create(KVCacheConfig(method="kivi", **kw))


def _kv(B, H, S, D, seed=0, dtype=torch.float16):
    rng = np.random.default_rng(seed)
    k = torch.from_numpy(rng.standard_normal((B, H, S, D)).astype(np.float32)).to(dtype).to(DEV)
    v = torch.from_numpy(rng.standard_normal((B, H, S, D)).astype(np.float32)).to(dtype).to(DEV)
    return k, v


def _reference_view(k_all, v_all, n_q, g, levels):
    """What the reference cache holds: rows < n_q round-tripped group by group, rest exact."""
    k32, v32 = k_all.float().cpu().numpy(), v_all.float().cpu().numpy()
    ko, vo = k32.copy(), v32.copy()
    if n_q:
        ko[:, :, :n_q] = o_kivi.quant_dequant_along(k_all[:, :, :n_q].cpu().numpy(), -2, g, levels).astype(np.float32)
        vo[:, :, :n_q] = o_kivi.quant_dequant_along(v_all[:, :, :n_q].cpu().numpy(), -1, g, levels).astype(np.float32)
    return ko, vo


def test_shape_dtype_and_no_bits_attribute():
    c = _make()
    k, v = _kv(1, 4, 64, 128)
    ko, vo = c.update_and_fetch(k, v)
    assert ko.shape == (1, 4, 64, 128) and vo.shape == (1, 4, 64, 128) and ko.dtype == torch.float16
    assert not hasattr(c, "bits") and hasattr(c, "assigned_avg_bits")
    with pytest.raises(NotImplementedError):
        c.merge()


def test_residual_window_exact_and_aged_tokens_lossy():
    c = _make(residual_length=64)
    k, v = _kv(1, 2, 32, 128, seed=1)
    ko, vo = c.update_and_fetch(k, v)
    assert torch.equal(ko, k) and torch.equal(vo, v) and c.compressed_key_bytes == 0
    c = _make(residual_length=16)
    k, v = _kv(1, 2, 80, 128, seed=2)
    ko, vo = c.update_and_fetch(k, v)
    assert torch.equal(ko[:, :, -16:], k[:, :, -16:])
    assert (ko[:, :, :64].float() - k[:, :, :64].float()).abs().mean() > 0
    assert c.compressed_key_bytes > 0 and c.residual_fp16_bytes > 0 and c._n_quantized == 64
    rk, rv = _reference_view(k, v, 64, 32, 3)
    np.testing.assert_array_equal(ko.float().cpu().numpy(), rk)
    np.testing.assert_array_equal(vo.float().cpu().numpy(), rv)


@pytest.mark.parametrize("b", [2, 4])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_prefill_equals_streamed_and_group_aligned_flush(b, dtype):
    B, H, D, S = 2, 2, 128, 300
    k, v = _kv(B, H, S, D, seed=b, dtype=dtype)
    one = _make(bit_width_inlier=b, residual_length=64)
    ko, vo = one.update_and_fetch(k, v)
    streamed = _make(bit_width_inlier=b, residual_length=64)
    streamed.update_and_fetch(k[:, :, :77], v[:, :, :77])
    for t in range(77, S):
        ks, vs = streamed.update_and_fetch(k[:, :, t : t + 1], v[:, :, t : t + 1])
        assert streamed._n_quantized % 32 == 0
        assert streamed.offset - streamed._n_quantized < 64 + 32
    assert one._n_quantized == streamed._n_quantized == ((S - 64) // 32) * 32
    assert ko.dtype == dtype and torch.equal(ko, ks) and torch.equal(vo, vs)
    nq = one._n_quantized
    for name in ("_k_codes", "_v_codes", "_v_scale", "_v_zero"):
        assert torch.equal(getattr(one, name)[:, :, :nq], getattr(streamed, name)[:, :, :nq]), name
    for name in ("_k_scale", "_k_zero"):
        assert torch.equal(getattr(one, name)[:, :, : nq // 32], getattr(streamed, name)[:, :, : nq // 32]), name
    assert one.compressed_key_bytes == streamed.compressed_key_bytes
    assert one.nbytes == streamed.nbytes and one.assigned_avg_bits == float(b)


def test_decode_tokens_age_out_with_small_groups():
    c = _make(residual_length=4, kivi_group_size=4)
    k, v = _kv(1, 1, 10, 128, seed=7)
    c.update_and_fetch(k, v)
    assert c._n_quantized == 4 and c.offset == 10
    sizes = []
    for t in range(12):
        k1, v1 = _kv(1, 1, 1, 128, seed=100 + t)
        c.update_and_fetch(k1, v1)
        sizes.append(c.residual_fp16_bytes)
    assert max(sizes) <= (4 + 4) * 128 * 2 * 2 and c.offset == 22


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16, torch.float32])
def test_append_kernel_copies_both_tensors_and_declines_odd_layouts(dt):
    from veloxquant_mlx_b200 import kernels as k
    g = torch.Generator(device=DEV).manual_seed(5)
    B, H, cap, D = 3, 2, 40, 128
    k_res = torch.zeros(B, H, cap, D, device=DEV, dtype=dt)
    v_res = torch.zeros(B, H, cap, D, device=DEV, dtype=dt)
    want_k, want_v = k_res.clone(), v_res.clone()
    pos = 0
    for S in (1, 5, 1, 16):
        big = torch.randn(2, B, H, S + 3, D, device=DEV, dtype=torch.float32, generator=g).to(dt)
        keys, values = big[0, :, :, 1:S + 1], big[1, :, :, 1:S + 1]  # evenly spaced slabs, not contiguous
        assert k.kivi_append(keys, values, k_res, v_res, pos)
        want_k[:, :, pos:pos + S], want_v[:, :, pos:pos + S] = keys, values
        pos += S
    assert torch.equal(k_res, want_k) and torch.equal(v_res, want_v)
    # layouts the kernel does not take are declined, nothing is written
    odd = torch.randn(B, H, 1, D + 8, device=DEV, dtype=torch.float32).to(dt)[..., 4:D + 4]  # rows not 16-byte aligned / strided
    before = k_res.clone()
    assert not k.kivi_append(odd, odd, k_res, v_res, pos)
    assert not k.kivi_append(keys[:, :, :1].transpose(0, 1), values[:, :, :1].transpose(0, 1), k_res.transpose(0, 1), v_res.transpose(0, 1), pos)
    assert not k.kivi_append(keys, values, k_res, v_res, cap - 1)  # would run past the buffer
    assert torch.equal(k_res, before)


def test_append_of_two_slices_of_one_buffer_equals_separate_tensors():
    """K and V that arrive as two slices of one tensor (a fused projection's output) are appended
    by one copy; the cache contents must not depend on that."""
    a, b = _make(residual_length=8, kivi_group_size=4), _make(residual_length=8, kivi_group_size=4)
    for t in range(15):
        buf = torch.randn(3, 2, 2, 1, 128, device=DEV, dtype=torch.float16,
                          generator=torch.Generator(device=DEV).manual_seed(40 + t))
        k, v = buf[1], buf[2]                   # same storage, fixed offset
        a.update_and_fetch(k, v)
        b.update_and_fetch(k.clone(), v.clone())  # two storages
        if t == 3:  # a pair in reversed order (values before keys) must take the two-copy path
            a.update_and_fetch(buf[2], buf[1])
            b.update_and_fetch(buf[2].clone(), buf[1].clone())
    ka, va = a._materialize()
    kb, vb = b._materialize()
    assert torch.equal(ka, kb) and torch.equal(va, vb) and a.offset == b.offset == 16


@pytest.mark.parametrize("b", [2, 4])
@pytest.mark.parametrize("memory_bound", [False, True])
def test_fused_sdpa_matches_oracle(b, memory_bound):
    B, H_kv, H_q, D, S = 2, 2, 8, 128, 517
    k, v = _kv(B, H_kv, S, D, seed=11 + b)
    c = _make(bit_width_inlier=b, residual_length=128, fused_sdpa_memory_bound=memory_bound)
    ko, vo = c.update_and_fetch(k, v)
    if memory_bound:
        assert ko.shape[2] == 0 and vo.shape[2] == 0
    q = torch.randn(B, H_q, 1, D, device=DEV, dtype=torch.float16)
    out = c.fused_sdpa(q, 1.0 / math.sqrt(D))
    nq = c._n_quantized
    assert nq == ((S - 128) // 32) * 32 and c.offset == S
    levels = (1 << b) - 1
    kc, ks, kz = o_kivi.quant_keys(k[:, :, :nq].cpu().numpy(), 32, levels)
    vc, vs, vz = o_kivi.quant_values(v[:, :, :nq].cpu().numpy(), 32, levels)
    ref = o_kivi.reference_attend(q.cpu().numpy(), kc, ks, kz, vc, vs, vz, 32, 1.0 / math.sqrt(D),
                                  k_res=k[:, :, nq:].cpu().numpy(), v_res=v[:, :, nq:].cpu().numpy())
    err = np.abs(out.float().cpu().numpy() - ref)
    assert err.max() < 2e-3
    # several query rows: the tail-aligned causal mask, so the last row equals the decode call
    two = c.fused_sdpa(torch.cat([q, q], dim=2), 1.0 / math.sqrt(D))
    assert two.shape == (B, H_q, 2, D) and float((two[:, :, 1:].float() - out.float()).abs().max()) < 2e-3
    with pytest.raises(ValueError, match="sliding_window"):
        c.fused_sdpa(q, 0.1, sliding_window=4)


def test_trim_rolls_back_frontier_and_matches_reference_buffer_semantics():
    g, R, b = 32, 32, 2
    full_k, full_v = _kv(1, 2, 656, 128, seed=21)
    c = _make(bit_width_inlier=b, residual_length=R)
    c.update_and_fetch(full_k[:, :, :256], full_v[:, :, :256])
    assert c._n_quantized == 224
    assert c.trim(200) == 200 and c.offset == 56
    assert c._n_quantized == 32 and c._n_quantized <= c.offset
    # rows 32..55 were quantized before the trim: they come back once-rounded, not exact
    kv_now, _ = c._materialize()
    rk, _ = _reference_view(full_k[:, :, :256], full_v[:, :, :256], 224, g, 3)
    np.testing.assert_array_equal(kv_now.float().cpu().numpy(), rk[:, :, :56])
    new_k, new_v = full_k[:, :, 256:], full_v[:, :, 256:]
    ko, _ = c.update_and_fetch(new_k, new_v)
    assert (ko[:, :, 56:224].float() - new_k[:, :, :168].float()).abs().max() > 0
    fresh = _make(bit_width_inlier=b, residual_length=R)
    fresh.update_and_fetch(torch.cat([full_k[:, :, :56], new_k], 2), torch.cat([full_v[:, :, :56], new_v], 2))
    assert c._n_quantized == fresh._n_quantized and c.offset == fresh.offset
    assert c.compressed_key_bytes == fresh.compressed_key_bytes
    assert c.compressed_value_bytes == fresh.compressed_value_bytes
    assert c.fp16_key_bytes == fresh.fp16_key_bytes
    # trimming inside the residual only shortens it
    n0 = c._n_quantized
    assert c.trim(5) == 5 and c._n_quantized == n0


def test_state_round_trip_and_compression_ratio():
    c = _make(bit_width_inlier=2, residual_length=16)
    k, v = _kv(1, 4, 256, 128, seed=3)
    c.update_and_fetch(k, v)
    total = c.compressed_key_bytes + c.compressed_value_bytes + c.residual_fp16_bytes
    assert (c.fp16_key_bytes + c.fp16_value_bytes) / total > 1.5
    assert c.effective_compression_ratio > 1.5
    d = _make(bit_width_inlier=2, residual_length=16)
    d.state = c.state
    assert d.offset == c.offset and d._n_quantized == c._n_quantized
    q = torch.randn(1, 8, 1, 128, device=DEV, dtype=torch.float16)
    assert torch.equal(c.fused_sdpa(q, 0.1), d.fused_sdpa(q, 0.1))
    assert not c.empty() and c.size() == 256 and len(c) == 256
