"""Tiled attention of many query rows over sign-bit keys, against the oracle's restatement of
the reference's ``_reference_prefill`` (tests/metal/test_rabitq_prefill.py:32-53) and against
the golden outputs that function produced. Tolerance: the reference's own (atol = rtol = 2e-2,
which covers half-precision weight and value tiles with float32 accumulation)."""

from __future__ import annotations

import os

import numpy as np
import pytest
import torch

from oracle import bitpack as o_bitpack
from oracle import rabitq as o_rabitq

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "rabitq.npz")


def _inputs(B, H, H_kv, S_q, S_kv, D, seed):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((B, H, S_q, D)).astype(np.float16)
    k_bits = rng.integers(0, 256, (B, H_kv, S_kv, D // 8), dtype=np.uint8)
    k_mag = rng.uniform(0.05, 0.15, (B, H_kv, S_kv)).astype(np.float32)
    k_const = rng.uniform(-0.2, 0.2, (B, H_kv, S_kv)).astype(np.float32)
    v_idx = rng.integers(0, 16, (B, H_kv, S_kv, D), dtype=np.uint8)
    v_cents = np.sort(rng.standard_normal(16)).astype(np.float32)
    return q, 1.0 / np.sqrt(D), k_bits, k_mag, k_const, v_idx, v_cents


def _run(q, scale, k_bits, k_mag, k_const, v_idx, v_cents, causal=False, dense=None):
    from veloxquant_mlx_b200 import rabitq as rq

    t = lambda a: None if a is None else torch.from_numpy(a).to(DEV)  # noqa: E731
    if dense is None:
        packed = rq.rabitq_pack_values(t(v_idx))
        out = rq.rabitq_prefill_attend(t(q), scale, t(k_bits), t(k_mag), t(k_const), packed, t(v_cents), causal=causal)
    else:
        out = rq.rabitq_prefill_attend(t(q), scale, t(k_bits), t(k_mag), t(k_const), dense, None, causal=causal)
    torch.cuda.synchronize()
    return out.float().cpu().numpy()


@pytest.mark.parametrize("tag", ["pre_B1_H1_Sq8_S33_D64_c0", "pre_B2_H2_Sq33_S200_D128_c0", "pre_B1_H2_Sq40_S40_D128_c1",
                                 "pre_B2_H1_Sq5_S77_D64_c1"])
def test_prefill_matches_the_reference_functions_outputs(tag):
    z = np.load(GOLDEN)
    g = lambda n: z[f"{tag}_{n}"]  # noqa: E731
    got = _run(g("q"), float(g("scale")[0]), g("k_bits"), g("k_mag"), g("k_const"), g("v_idx"), g("v_cents"), causal=tag.endswith("c1"))
    np.testing.assert_allclose(got, g("out"), atol=2e-2, rtol=2e-2)
    assert float(np.abs(got - g("out")).max()) < 4e-3  # far inside the reference's tolerance


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("S_q", [1, 8, 33, 256])
@pytest.mark.parametrize("S_kv", [8, 33, 2048])
@pytest.mark.parametrize("BH", [(1, 1), (2, 2)])
def test_prefill_attend_parity(D, S_q, S_kv, BH):
    B, H = BH
    args = _inputs(B, H, H, S_q, S_kv, D, seed=D + S_q + S_kv + B * H)
    got = _run(*args)
    assert got.shape == (B, H, S_q, D)
    np.testing.assert_allclose(got, o_rabitq.reference_prefill(*args), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("S_q,S_kv", [(1, 64), (40, 40), (33, 200), (256, 300), (70, 2048)])
@pytest.mark.parametrize("H,H_kv", [(2, 2), (8, 2), (5, 1)])
def test_causal_and_grouped_query_heads(S_q, S_kv, H, H_kv):
    args = _inputs(2, H, H_kv, S_q, S_kv, 128, seed=S_q + S_kv + H)
    got = _run(*args, causal=True)
    ref = o_rabitq.reference_prefill(*args, causal=True)
    np.testing.assert_allclose(got, ref, atol=2e-2, rtol=2e-2)
    # the first row of a causal call over exactly S_q slots sees one slot: its value row
    if S_q == S_kv:
        v_hat = args[6][args[5]]
        rep = H // H_kv
        np.testing.assert_allclose(got[:, :, 0], np.repeat(v_hat[:, :, 0], rep, axis=1), atol=2e-3)


@pytest.mark.parametrize("dt", [torch.float16, torch.bfloat16])
def test_dense_values_and_no_constants(dt):
    q, scale, k_bits, k_mag, _, _, _ = _inputs(2, 8, 2, 50, 333, 128, seed=5)
    v = torch.randn((2, 2, 333, 128), device=DEV, dtype=torch.float32).to(dt)
    got = _run(q, scale, k_bits, k_mag, None, None, None, causal=True, dense=v)
    ref = o_rabitq.reference_prefill(q, scale, k_bits, k_mag, None, v.float().cpu().numpy(), None, causal=True)
    np.testing.assert_allclose(got, ref, atol=2e-2, rtol=2e-2)


def test_argument_errors():
    from veloxquant_mlx_b200 import rabitq as rq

    q, scale, k_bits, k_mag, k_const, v_idx, v_cents = _inputs(1, 2, 2, 4, 16, 128, seed=1)
    t = lambda a: torch.from_numpy(a).to(DEV)  # noqa: E731
    packed = rq.rabitq_pack_values(t(v_idx))
    with pytest.raises(ValueError, match="q must be 4D"):
        rq.rabitq_prefill_attend(t(q)[0], scale, t(k_bits), t(k_mag), t(k_const), packed, t(v_cents))
    with pytest.raises(ValueError, match="nibble-packed"):
        rq.rabitq_prefill_attend(t(q), scale, t(k_bits), t(k_mag), t(k_const), t(v_idx), t(v_cents))
    with pytest.raises(ValueError, match="k_mag must be"):
        rq.rabitq_prefill_attend(t(q), scale, t(k_bits), t(k_mag)[:, :, :5], t(k_const), packed, t(v_cents))
    with pytest.raises(ValueError, match="<= 16 entries"):
        rq.rabitq_prefill_attend(t(q), scale, t(k_bits), t(k_mag), t(k_const), packed, torch.zeros(17, device=DEV))
    with pytest.raises(ValueError, match="causal attention of"):
        rq.rabitq_prefill_attend(torch.zeros(1, 2, 32, 128, device=DEV, dtype=torch.float16), scale, t(k_bits), t(k_mag),
                                 t(k_const), packed, t(v_cents), causal=True)
    with pytest.raises(ValueError, match="64 or 128"):
        rq.rabitq_prefill_attend(torch.zeros(1, 2, 4, 256, device=DEV, dtype=torch.float16), scale, t(k_bits), t(k_mag),
                                 t(k_const), packed, t(v_cents))


def test_cache_attends_a_prompt_chunk_causally():
    """``RaBitQKVCache.fused_sdpa`` with several query rows: rotated queries, exact dots with the
    decoded keys, tail-aligned causal mask; equals the oracle on the cache's own stored bits."""
    from veloxquant_mlx_b200.cache import KVCacheConfig, KVCacheFactory

    B, H_kv, H_q, S, S_q, D = 2, 2, 8, 300, 37, 128
    g = torch.Generator(device=DEV).manual_seed(9)
    k = torch.randn((B, H_kv, S, D), generator=g, device=DEV, dtype=torch.float16)
    v = torch.randn((B, H_kv, S, D), generator=g, device=DEV, dtype=torch.float16)
    q = torch.randn((B, H_q, S_q, D), generator=g, device=DEV, dtype=torch.float16)
    c = KVCacheFactory.create(KVCacheConfig(method="rabitq", head_dim=D))
    c.update_and_fetch(k, v)
    got = c.fused_sdpa(q, 0.088, causal=True).float().cpu().numpy()
    q_rot = ((q.float() * c._diag) @ c._H).half().cpu().numpy()
    ref = o_rabitq.reference_prefill(q_rot, 0.088, c._bits[:, :, :S].cpu().numpy(), c._mag[:, :, :S].cpu().numpy(), None,
                                     v.float().cpu().numpy(), None, causal=True)
    np.testing.assert_allclose(got, ref, atol=2e-2, rtol=2e-2)
    assert c.fused_sdpa(q, 0.088, causal=False).shape == (B, H_q, S_q, D)
    with pytest.raises(ValueError, match="query rows"):
        c.fused_sdpa(torch.zeros(B, H_q, S + 1, D, device=DEV, dtype=torch.float16), 0.088)
