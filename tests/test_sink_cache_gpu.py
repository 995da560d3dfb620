"""Sink-protected KIVI cache on the GPU: its dense view against the oracle's (bit for bit), its
fused attention against dense attention over that view, and the reference tests' properties
(``veloxquant_mlx/tests/cache/test_sink_cache.py``)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle.kivi_sink import SinkProtectedOracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _make(**kw):
    from veloxquant_mlx_b200.cache import KVCacheConfig, KVCacheFactory

    base = dict(method="kivi_sink", head_dim=128, bit_width_inlier=2, residual_length=8, kivi_group_size=32, n_sink_tokens=5)
    base.update(kw)
    return KVCacheFactory.create(KVCacheConfig(**base))


def _kv(B=1, H=4, S=64, D=128, sinks=((0, 7, 20),), scale=25.0, seed=0, dtype=np.float16):
    rng = np.random.default_rng(seed)
    K = rng.standard_normal((B, H, S, D)).astype(np.float32)
    V = rng.standard_normal((B, H, S, D)).astype(np.float32)
    for b, ps in enumerate(sinks):
        for p in ps:
            K[b, :, p] *= scale
    return K.astype(dtype), V.astype(dtype)


def _t(x):
    return torch.from_numpy(x).to(DEV)


def _dense_attend(q, k, v, scale, hpk):
    """float64 softmax attention of q [B,Hq,1,D] over dense k, v [B,Hkv,S,D]."""
    k = np.repeat(k.astype(np.float64), hpk, axis=1)
    v = np.repeat(v.astype(np.float64), hpk, axis=1)
    s = np.einsum("bhqd,bhkd->bhqk", q.astype(np.float64), k) * scale
    s -= s.max(-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(-1, keepdims=True)
    return np.einsum("bhqk,bhkd->bhqd", p, v)


def test_planted_sinks_detected_preserved_and_view_matches_oracle():
    K, V = _kv()
    c = _make(n_sink_tokens=3)
    ko, vo = c.update_and_fetch(_t(K), _t(V))
    o = SinkProtectedOracle(128, 2, 32, 8, 3)
    rk, rv = o.update_and_fetch(K, V)
    assert set(c.sink_positions) == {0, 7, 20} == set(o.sink_positions_for(0))
    np.testing.assert_array_equal(ko.cpu().numpy(), rk)
    np.testing.assert_array_equal(vo.cpu().numpy(), rv)
    assert not torch.equal(ko[:, :, 30], _t(K)[:, :, 30])


def test_zero_sinks_equals_plain_kivi():
    from veloxquant_mlx_b200.cache import KVCacheConfig, KVCacheFactory

    K, V = _kv(sinks=((),))
    a, av = _make(n_sink_tokens=0).update_and_fetch(_t(K), _t(V))
    b, bv = KVCacheFactory.create(KVCacheConfig(method="kivi", head_dim=128, bit_width_inlier=2, residual_length=8,
                                                kivi_group_size=32)).update_and_fetch(_t(K), _t(V))
    assert torch.equal(a, b) and torch.equal(av, bv)


def test_byte_accounting_no_double_count():
    c = _make(n_sink_tokens=3)
    K, V = _kv()
    c.update_and_fetch(_t(K), _t(V))
    B, H, D = 1, 4, 128
    fp16_tok = D * 2 * 2 * H * B
    assert c.offset - c._n_quantized == 32
    assert c.residual_fp16_bytes == 32 * fp16_tok
    assert c.sink_fp16_bytes == 3 * fp16_tok
    assert c.fp16_key_bytes == H * B * 64 * D * 2
    # 29 compressed tokens: the reference's formula (sink_cache.py:231-241)
    assert c.compressed_key_bytes == -(-29 * D * 2 // 8) * H * B + 1 * D * 2 * 2 * H * B
    assert c.compressed_value_bytes == -(-29 * D * 2 // 8) * H * B + 29 * 4 * 2 * 2 * H * B
    total = c.compressed_key_bytes + c.compressed_value_bytes + c.sink_fp16_bytes + c.residual_fp16_bytes
    assert total < c.fp16_key_bytes + c.fp16_value_bytes


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_per_batch_sinks_small_head_dim_view_matches_oracle(dtype):
    """Batch element 1 alone has an outlier at position 5 (the reference's regression test for
    per-batch tracking), on a shape the fused attention does not cover: the dense view is what counts."""
    c = _make(head_dim=8, n_sink_tokens=2, kivi_group_size=4, residual_length=4)
    rng = np.random.default_rng(1)
    K = rng.standard_normal((2, 1, 20, 8)).astype(np.float32)
    K[1, 0, 5] = 50.0
    V = rng.standard_normal((2, 1, 20, 8)).astype(np.float32)
    K, V = K.astype(dtype), V.astype(dtype)
    ko, vo = c.update_and_fetch(_t(K), _t(V))
    o = SinkProtectedOracle(8, 2, 4, 4, 2)
    rk, rv = o.update_and_fetch(K, V)
    assert 5 in c.sink_positions_for(1)
    np.testing.assert_array_equal(ko.cpu().numpy(), rk)
    np.testing.assert_array_equal(vo.cpu().numpy(), rv)
    assert torch.equal(ko[1, :, 5], _t(K)[1, :, 5]) and not torch.equal(ko[0, :, 5], _t(K)[0, :, 5])


@pytest.mark.parametrize("bits", [2, 4])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_streamed_decode_view_and_fused_attention(bits, dtype):
    """Prefill, then token-by-token decode across several flushes with different sinks per batch
    element (some arriving during decode): the dense view equals the oracle's at every checked
    step, and the fused attention equals dense attention over that view."""
    B, H, Hq, D, S0, steps = 2, 2, 8, 128, 150, 80
    npdt = np.float16 if dtype is torch.float16 else np.float32
    K, V = _kv(B, H, S0 + steps, D, sinks=((0, 3, 160), (1, 77, 200)), seed=3, dtype=np.float32)
    Kt, Vt = torch.from_numpy(K).to(dtype), torch.from_numpy(V).to(dtype)
    Kn, Vn = Kt.float().numpy().astype(npdt), Vt.float().numpy().astype(npdt)  # what the cache is given
    if dtype is torch.bfloat16:
        Kn, Vn = Kt.float().numpy(), Vt.float().numpy()
    c = _make(bit_width_inlier=bits, residual_length=16, n_sink_tokens=3, fused_sdpa_memory_bound=False)
    o = SinkProtectedOracle(D, bits, 32, 16, 3)
    c.update_and_fetch(Kt[:, :, :S0].to(DEV), Vt[:, :, :S0].to(DEV))
    o.update_and_fetch(Kn[:, :, :S0], Vn[:, :, :S0])
    rng = np.random.default_rng(7)
    scale = 1.0 / np.sqrt(D)
    for t in range(S0, S0 + steps):
        ko, vo = c.update_and_fetch(Kt[:, :, t : t + 1].to(DEV), Vt[:, :, t : t + 1].to(DEV))
        rk, rv = o.update_and_fetch(Kn[:, :, t : t + 1], Vn[:, :, t : t + 1])
        if t % 9 == 0 or t == S0 + steps - 1:
            if dtype is torch.float16:
                np.testing.assert_array_equal(ko.cpu().numpy(), rk)
                np.testing.assert_array_equal(vo.cpu().numpy(), rv)
            else:
                # the oracle rounds its float32 round trip to the buffer dtype (float32 here): compare
                # after the same bf16 rounding the cache applies
                rk_b = torch.from_numpy(rk).to(torch.bfloat16).float().numpy()
                rv_b = torch.from_numpy(rv).to(torch.bfloat16).float().numpy()
                np.testing.assert_array_equal(ko.float().cpu().numpy(), rk_b)
                np.testing.assert_array_equal(vo.float().cpu().numpy(), rv_b)
            q = rng.standard_normal((B, Hq, 1, D)).astype(np.float32)
            got = c.fused_sdpa(torch.from_numpy(q).to(dtype).to(DEV), scale).float().cpu().numpy()
            qn = torch.from_numpy(q).to(dtype).float().numpy()
            want = _dense_attend(qn, ko.float().cpu().numpy(), vo.float().cpu().numpy(), scale, Hq // H)
            err = np.abs(got - want)
            assert (err <= 2e-3 + 1e-2 * np.abs(want)).all(), f"t={t}: max err {err.max():.3e}"
    assert set(c.sink_positions_for(0)) == set(o.sink_positions_for(0))
    assert set(c.sink_positions_for(1)) == set(o.sink_positions_for(1))
    c.check_status()


def test_memory_bound_decode_loop_with_output_buffer():
    """The serving form: sentinels from update_and_fetch, attention into a caller's buffer (the
    host fast path re-uses the argument structure, which carries the sinks)."""
    B, H, Hq, D = 2, 2, 8, 128
    K, V = _kv(B, H, 400, D, sinks=((0, 5), (2, 9)), seed=11)
    c = _make(bit_width_inlier=4, residual_length=32, n_sink_tokens=2, fused_sdpa_memory_bound=True)
    o = SinkProtectedOracle(D, 4, 32, 32, 2)
    c.update_and_fetch(_t(K[:, :, :300]), _t(V[:, :, :300]))
    o.update_and_fetch(K[:, :, :300], V[:, :, :300])
    q = torch.empty(B, Hq, 1, D, dtype=torch.float16, device=DEV)
    out = torch.empty_like(q)
    rng = np.random.default_rng(2)
    scale = 1.0 / np.sqrt(D)
    for t in range(300, 400):
        ks, _ = c.update_and_fetch(_t(K[:, :, t : t + 1]), _t(V[:, :, t : t + 1]))
        assert ks.shape[2] == 0
        rk, rv = o.update_and_fetch(K[:, :, t : t + 1], V[:, :, t : t + 1])
        qn = rng.standard_normal((B, Hq, 1, D)).astype(np.float16)
        q.copy_(_t(qn))
        c.fused_sdpa(q, scale, out=out)
        if t % 7 == 0:
            want = _dense_attend(qn.astype(np.float32), rk.astype(np.float32), rv.astype(np.float32), scale, Hq // H)
            err = np.abs(out.float().cpu().numpy() - want)
            assert (err <= 2e-3 + 1e-2 * np.abs(want)).all(), f"t={t}: max err {err.max():.3e}"


def test_trim_into_the_quantized_region_and_continue():
    K, V = _kv(1, 2, 200, 128, sinks=((0, 40, 70),), seed=5)
    c = _make(residual_length=8, n_sink_tokens=3)
    o = SinkProtectedOracle(128, 2, 32, 8, 3)
    c.update_and_fetch(_t(K[:, :, :100]), _t(V[:, :, :100]))
    o.update_and_fetch(K[:, :, :100], V[:, :, :100])
    assert c._n_quantized == 64 == o.n_quantized
    assert c.trim(50) == 50 == o.trim(50)
    assert c._n_quantized == 32 == o.n_quantized
    assert set(c.sink_positions) == set(o.sink_positions_for(0))
    ko, vo = c.update_and_fetch(_t(K[:, :, 100:200]), _t(V[:, :, 100:200]))
    rk, rv = o.update_and_fetch(K[:, :, 100:200], V[:, :, 100:200])
    np.testing.assert_array_equal(ko.cpu().numpy(), rk)
    np.testing.assert_array_equal(vo.cpu().numpy(), rv)
    q = np.random.default_rng(0).standard_normal((1, 8, 1, 128)).astype(np.float16)
    got = c.fused_sdpa(_t(q), 0.09).float().cpu().numpy()
    want = _dense_attend(q.astype(np.float32), rk.astype(np.float32), rv.astype(np.float32), 0.09, 4)
    assert (np.abs(got - want) <= 2e-3 + 1e-2 * np.abs(want)).all()


def test_state_round_trip_through_a_file(tmp_path):
    from veloxquant_mlx_b200.cache import KVCacheConfig
    from veloxquant_mlx_b200.persistence import load_prompt_cache, save_prompt_cache

    K, V = _kv(2, 2, 180, 128, sinks=((0, 33), (4, 90)), seed=8)
    cfg = KVCacheConfig(method="kivi_sink", head_dim=128, bit_width_inlier=4, residual_length=16, n_sink_tokens=2)
    c = _make(bit_width_inlier=4, residual_length=16, n_sink_tokens=2)
    c.update_and_fetch(_t(K[:, :, :150]), _t(V[:, :, :150]))
    path = str(tmp_path / "sink.safetensors")
    save_prompt_cache(path, [c])
    (d,) = load_prompt_cache(path, cfg)
    assert d.sink_positions_for(0) == c.sink_positions_for(0) and d.sink_positions_for(1) == c.sink_positions_for(1)
    q = _t(np.random.default_rng(1).standard_normal((2, 8, 1, 128)).astype(np.float16))
    for t in range(150, 180):
        a = c.update_and_fetch(_t(K[:, :, t : t + 1]), _t(V[:, :, t : t + 1]))
        b = d.update_and_fetch(_t(K[:, :, t : t + 1]), _t(V[:, :, t : t + 1]))
        assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    assert torch.equal(c.fused_sdpa(q, 0.09), d.fused_sdpa(q, 0.09))
    assert c.sink_fp16_bytes == d.sink_fp16_bytes


def test_many_query_rows_are_refused_once_sinks_are_packed():
    K, V = _kv()
    c = _make(n_sink_tokens=3)
    c.update_and_fetch(_t(K), _t(V))
    with pytest.raises(ValueError, match="one query row"):
        c.fused_sdpa(torch.zeros(1, 4, 2, 128, dtype=torch.float16, device=DEV), 0.1)
