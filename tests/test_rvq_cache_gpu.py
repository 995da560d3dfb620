"""Packed TurboQuant-RVQ cache on the GPU: stored streams and dequantized keys against the
oracle pipeline bit for bit, and the behaviour the reference's cache tests pin
(``veloxquant_mlx/tests/metal/test_rvq_quant_pack.py:97-117``, growth, trim, state)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import rvq as o_rvq

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _make(**kw):
    from veloxquant_mlx_b200.cache import KVCacheConfig, KVCacheFactory

    base = dict(method="turboquant_rvq", head_dim=128, bit_width_inlier=2, seed=0)
    base.update(kw)
    return KVCacheFactory.create(KVCacheConfig(**base))


def _oracle_encode_decode(keys16: np.ndarray, cache):
    """The cache's pipeline in NumPy: float32 norm, unit direction in fp16, randomized Hadamard in
    float32 (butterfly order), two-stage quantize + pack, decode, bf16 norm."""
    q = cache._quantizer
    D = keys16.shape[-1]
    k32 = keys16.reshape(-1, D).astype(np.float32)
    norms = np.sqrt((k32 * k32).sum(-1, keepdims=True, dtype=np.float32))
    unit = (k32 / np.maximum(norms, np.float32(1e-4))).astype(np.float16)
    y = (o_rvq.wht_butterfly(unit.astype(np.float32) * q._diag_np) * (np.float32(1.0) / np.sqrt(np.float32(D)))).astype(np.float16)
    _, _, p1, p2 = o_rvq.rvq_quant_pack(y, q._codebook1.centroids, q._codebook1.boundaries, q._codebook2.boundaries, q._b)
    nb = torch.from_numpy(norms).to(torch.bfloat16).float().numpy().reshape(-1)
    k_hat = o_rvq.rvq_unpack_decode(p1, p2, nb, q._codebook1.centroids, q._codebook2.centroids, q._diag_np, q._b, D)
    return p1, p2, nb, k_hat


@pytest.mark.parametrize("bits", [1, 2, 4])
def test_prefill_streams_and_keys_match_the_oracle(bits):
    B, H, S, D = 2, 4, 40, 128
    rng = np.random.default_rng(5)
    keys = (rng.standard_normal((B, H, S, D)) * 3).astype(np.float16)
    vals = rng.standard_normal((B, H, S, D)).astype(np.float16)
    c = _make(bit_width_inlier=bits)
    k_hat, v = c.update_and_fetch(torch.from_numpy(keys).to(DEV), torch.from_numpy(vals).to(DEV))
    p1, p2, nb, want = _oracle_encode_decode(keys, c)
    nw = c._n_words
    np.testing.assert_array_equal(c._packed1.view(torch.int32)[:, :, :S].cpu().numpy().view(np.uint32).reshape(-1, nw), p1)
    np.testing.assert_array_equal(c._packed2.view(torch.int32)[:, :, :S].cpu().numpy().view(np.uint32).reshape(-1, nw), p2)
    np.testing.assert_array_equal(c._norms[:, :, :S].float().cpu().numpy().reshape(-1), nb)
    np.testing.assert_array_equal(k_hat.cpu().numpy().reshape(-1, D), want)
    assert torch.equal(v, torch.from_numpy(vals).to(DEV)) and k_hat.dtype == torch.float16
    assert c.offset == S and c._packed1.shape[2] == 512   # ceil((256 + 40 - 1) / 256) * 256, as the reference grows
    assert c.compressed_key_bytes == (2 * nw * 4 + 2) * H * B * S and c.fp16_key_bytes == H * B * S * D * 2
    assert c.nbytes == B * H * S * (2 * nw * 4 + 2 + D * 2)
    assert c.assigned_bits == bits and not hasattr(c, "bits")
    cos = torch.nn.functional.cosine_similarity(k_hat.float(), torch.from_numpy(keys).to(DEV).float(), dim=-1)
    assert float(cos.mean()) > {1: 0.90, 2: 0.97, 4: 0.995}[bits]


def test_streamed_appends_equal_one_shot_and_buffers_grow_in_steps():
    B, H, D = 1, 2, 128
    rng = np.random.default_rng(1)
    keys = torch.from_numpy(rng.standard_normal((B, H, 600, D)).astype(np.float16)).to(DEV)
    vals = torch.from_numpy(rng.standard_normal((B, H, 600, D)).astype(np.float16)).to(DEV)
    one = _make()
    k1, v1 = one.update_and_fetch(keys, vals)
    assert one._packed1.shape[2] == 1024   # ceil((256 + 600 - 1) / 256) * 256
    st = _make()
    st.update_and_fetch(keys[:, :, :250], vals[:, :, :250])
    assert st._packed1.shape[2] == 512
    for t in range(250, 600):
        k2, v2 = st.update_and_fetch(keys[:, :, t : t + 1], vals[:, :, t : t + 1])
    assert st._packed1.shape[2] == 768
    assert torch.equal(k1, k2) and torch.equal(v1, v2) and st.offset == 600
    # bf16 keys take the same path (unit direction in fp16) and come back in bf16
    kb = _make().update_and_fetch(keys.to(torch.bfloat16), vals.to(torch.bfloat16))[0]
    assert kb.dtype == torch.bfloat16 and kb.shape == k1.shape


def test_trim_state_and_file_round_trip(tmp_path):
    from veloxquant_mlx_b200.cache import KVCacheConfig, TurboQuantRVQKVCache
    from veloxquant_mlx_b200.persistence import load_prompt_cache, save_prompt_cache

    B, H, D = 2, 2, 128
    keys = torch.randn(B, H, 300, D, device=DEV, dtype=torch.float16)
    vals = torch.randn(B, H, 300, D, device=DEV, dtype=torch.float16)
    c = _make(seed=7)
    c.update_and_fetch(keys[:, :, :200], vals[:, :, :200])
    assert c.is_trimmable() and c.trim(50) == 50 and c.offset == 150 and c.trim(0) == 0
    assert c.compressed_key_bytes == int((2 * c._n_words * 4 + 2) * H * B * 200 * (150 / 200))
    assert c.meta_state == ("128", "2", "7", "150")
    d = TurboQuantRVQKVCache.from_state(c.state, c.meta_state)
    path = str(tmp_path / "rvq.safetensors")
    save_prompt_cache(path, [c])
    (e,) = load_prompt_cache(path, KVCacheConfig(method="turboquant_rvq", head_dim=128, bit_width_inlier=2, seed=7))
    outs = [x.update_and_fetch(keys[:, :, 200:], vals[:, :, 200:]) for x in (c, d, e)]
    for ko, vo in outs[1:]:
        assert torch.equal(ko, outs[0][0]) and torch.equal(vo, outs[0][1])
    assert outs[0][0].shape[2] == 250
    with pytest.raises(TypeError):
        TurboQuantRVQKVCache.from_state(c.state)
    with pytest.raises(AttributeError):
        c.merge


def test_attention_over_dequantized_keys_and_standalone_protocol():
    B, H, Hq, D = 1, 2, 8, 128
    keys = torch.randn(B, H, 100, D, device=DEV, dtype=torch.float16)
    vals = torch.randn(B, H, 100, D, device=DEV, dtype=torch.float16)
    c = _make()
    k_hat, v = c.update_and_fetch(keys, vals)
    q = torch.randn(B, Hq, 1, D, device=DEV, dtype=torch.float16)
    got = c.fused_sdpa(q, D ** -0.5)
    kk, vv = k_hat.repeat_interleave(4, dim=1).float(), v.repeat_interleave(4, dim=1).float()
    p = torch.softmax((q.float() @ kk.transpose(-1, -2)) * D ** -0.5, dim=-1)
    assert float((got.float() - p @ vv).abs().max()) < 2e-3
    s = _make(head_dim=128)
    for t in range(5):
        s.append_key(keys[0, 0, t])
        s.append_value(vals[0, 0, t])
    assert len(s) == 5 and s.memory_bytes() == s.nbytes and s.attend(q[0, 0, 0]).shape == (D,)
    s.reset()
    assert len(s) == 0


def test_configuration_errors():
    from veloxquant_mlx_b200.cache import QuantizerConfigError

    with pytest.raises(QuantizerConfigError):
        _make(bit_width_inlier=5)
    with pytest.raises(QuantizerConfigError):
        _make(head_dim=96)
    with pytest.raises(TypeError):
        from veloxquant_mlx_b200.cache import KVCacheConfig, TurboQuantRVQKVCache
        TurboQuantRVQKVCache(KVCacheConfig(method="turboquant_rvq", bit_width_inlier=[2, 2]))
    c = _make()
    with pytest.raises(QuantizerConfigError):
        c.update_and_fetch(torch.zeros(1, 1, 1, 64, device=DEV, dtype=torch.float16), torch.zeros(1, 1, 1, 64, device=DEV, dtype=torch.float16))
