"""GPU parity for the RaBitQ path through the C ABI against the CPU oracle and the golden
fixtures produced by the reference's own test functions. Mirrors tests/metal/test_rabitq_encode.py,
test_rabitq_attend.py, test_rabitq_values.py of the reference.

Sign bits and packed bytes: bit-exact. Magnitudes: rtol 1e-4 (as the reference's test; the
L1 sum is reduced in a different order). Attention: atol = rtol = 1e-2 as in the reference,
plus |got-ref| <= 2e-3 + 1e-2*|ref|.
"""

from __future__ import annotations

import os

import numpy as np
import pytest
import torch

from oracle import bitpack as o_bitpack
from oracle import rabitq as o_rq

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _r():
    from veloxquant_mlx_b200 import rabitq

    return rabitq


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


@pytest.mark.parametrize("D", [8, 16, 32, 64, 128, 256])
@pytest.mark.parametrize("N", [1, 33, 512])
def test_encode_bits_exact_mag_close(D, N):
    rng = np.random.default_rng(D + N)
    keys = rng.standard_normal((N, D)).astype(np.float16)
    diag = rng.choice([-1.0, 1.0], size=D).astype(np.float32)
    bits, mag = _r().rabitq_encode(_t(keys), _t(diag))
    obits, omag, _ = o_rq.encode_hadamard(keys, diag)
    assert bits.dtype == torch.uint8 and bits.shape == (N, D // 8) and mag.dtype == torch.float32
    np.testing.assert_array_equal(bits.cpu().numpy(), obits)
    np.testing.assert_allclose(mag.cpu().numpy(), omag, rtol=1e-4)


def test_encode_matches_golden_and_config4_shape():
    z = np.load(os.path.join(GOLDEN, "rabitq.npz"))
    r = _r()
    for N, D in [(1, 8), (33, 64), (64, 128), (17, 256)]:
        tag = f"enc_N{N}_D{D}"
        bits, mag = r.rabitq_encode(_t(z[f"{tag}_keys"]), _t(z[f"{tag}_diag"]))
        np.testing.assert_array_equal(bits.cpu().numpy(), z[f"{tag}_bits"])
        np.testing.assert_allclose(mag.cpu().numpy(), z[f"{tag}_mag"], rtol=1e-4)
    # benchmark config 4: keys fp16 [8, 16384, 128] (one batch item), seeded rotation
    rng = np.random.default_rng(4)
    keys = rng.standard_normal((8 * 16384, 128)).astype(np.float16)
    diag = r.make_hadamard_diagonal(128, seed=42)
    np.testing.assert_array_equal(diag, z["diag_d128_s42"])
    bits, mag = r.rabitq_encode(_t(keys), _t(diag))
    obits, omag, _ = o_rq.encode_hadamard(keys, diag)
    np.testing.assert_array_equal(bits.cpu().numpy(), obits)
    np.testing.assert_allclose(mag.cpu().numpy(), omag, rtol=1e-4)
    # the "sign bits packed into uint32" view is the same bytes on a little-endian machine
    assert bits.view(torch.int32).shape == (8 * 16384, 4)
    # dense QR rotation (the variant benchmark config 4 words): rotate with a GEMM, then pack
    rot = r.make_rotation_matrix(128, seed=42).astype(np.float32)
    np.testing.assert_array_equal(rot, z["rot_d128_s42"])
    y = (_t(keys[:4096]).float() @ _t(rot).T).contiguous()
    b2, m2 = r.rabitq_encode_rotated(y)
    np.testing.assert_array_equal(b2.cpu().numpy(), o_rq.pack_signs(y.cpu().numpy()))
    np.testing.assert_allclose(m2.cpu().numpy(), np.abs(y.cpu().numpy()).sum(1) / 128, rtol=1e-4)
    for bad, msg in [((4, 12), "divisible by 8"), ((4, 24), "power of two")]:
        with pytest.raises(ValueError, match=msg):
            r.rabitq_encode(torch.zeros(bad, device=DEV, dtype=torch.float16), torch.ones(bad[1], device=DEV))


@pytest.mark.parametrize("shape", [(6,), (4, 64), (1, 2, 33, 128), (2, 2, 7, 256)])
def test_pack_values_and_hamming(shape):
    rng = np.random.default_rng(sum(shape))
    v_idx = rng.integers(0, 16, shape, dtype=np.uint8)
    packed = _r().rabitq_pack_values(_t(v_idx))
    assert packed.shape == (*shape[:-1], shape[-1] // 2)
    np.testing.assert_array_equal(packed.cpu().numpy(), o_bitpack.pack_nibbles(v_idx))
    masked = np.array([[0xFF, 0x01, 0x12, 0x03]], dtype=np.uint8)
    np.testing.assert_array_equal(_r().rabitq_pack_values(_t(masked)).cpu().numpy(), o_bitpack.pack_nibbles(masked))
    with pytest.raises(ValueError, match="even"):
        _r().rabitq_pack_values(torch.zeros((4, 7), dtype=torch.uint8, device=DEV))
    bits = rng.integers(0, 256, (97, 16), dtype=np.uint8)
    qb = rng.integers(0, 256, 16, dtype=np.uint8)
    cx = rng.standard_normal(97).astype(np.float32)
    s = _r().rabitq_hamming_score(_t(qb), _t(bits), _t(cx), 0.25)      # (the reference's order: constants, then the scale)
    np.testing.assert_array_equal(s.cpu().numpy(), o_rq.hamming_score(qb, bits, 0.25, cx))


def _attend_inputs(B, H, S_q, S_kv, D, seed, H_kv=None):
    H_kv = H_kv or H
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((B, H, S_q, D)).astype(np.float16)
    q_scale = (rng.uniform(0.05, 0.15, (B, H, S_q)) / np.sqrt(D)).astype(np.float32)
    k_bits = rng.integers(0, 256, (B, H_kv, S_kv, D // 8), dtype=np.uint8)
    k_mag = rng.uniform(0.5, 1.5, (B, H_kv, S_kv)).astype(np.float32)
    k_const = rng.uniform(-0.2, 0.2, (B, H_kv, S_kv)).astype(np.float32)
    v_idx = rng.integers(0, 16, (B, H_kv, S_kv, D), dtype=np.uint8)
    v_cents = np.sort(rng.standard_normal(16)).astype(np.float32)
    return q, q_scale, k_bits, k_mag, k_const, v_idx, v_cents


@pytest.mark.parametrize("D", [64, 128, 256])
@pytest.mark.parametrize("S_kv", [1, 33, 256, 3000])
@pytest.mark.parametrize("S_q", [1, 8])
@pytest.mark.parametrize("BH", [(1, 1), (2, 2)])
def test_attend_parity_and_packed_equals_unpacked(D, S_kv, S_q, BH):
    B, H = BH
    ins = _attend_inputs(B, H, S_q, S_kv, D, seed=D + S_kv + S_q + B * H)
    ref = o_rq.reference_attend(*ins)
    r = _r()
    targs = [_t(a) for a in ins]
    out = r.rabitq_fused_attend(*targs)
    assert out.shape == (B, H, S_q, D) and out.dtype == torch.float16
    got = out.float().cpu().numpy()
    np.testing.assert_allclose(got, ref, atol=1e-2, rtol=1e-2)
    assert np.all(np.abs(got - ref) <= 2e-3 + 1e-2 * np.abs(ref))
    packed = r.rabitq_fused_attend(*targs[:5], r.rabitq_pack_values(targs[5]), targs[6])
    assert torch.equal(out, packed)  # bit-identical, as the reference requires


@pytest.mark.parametrize("D", [64, 256])
@pytest.mark.parametrize("H,H_kv", [(6, 2), (12, 2)])
def test_attend_parity_grouped_heads_every_head_dim(D, H, H_kv):
    """3 and 6 query heads per kv head (the 4- and 8-head instantiations) at the narrowest and the
    widest head_dim: every head keeps its own accumulators, nibble-coded and dense values."""
    B, S = 2, 700
    ins = _attend_inputs(B, H, 1, S, D, seed=D + H, H_kv=H_kv)
    ref = o_rq.reference_attend(*ins)
    r = _r()
    got = r.rabitq_fused_attend(*[_t(a) for a in ins]).float().cpu().numpy()
    assert np.all(np.abs(got - ref) <= 2e-3 + 1e-2 * np.abs(ref)), np.abs(got - ref).max()
    v = np.random.default_rng(D).standard_normal((B, H_kv, S, D)).astype(np.float16)
    ref = o_rq.reference_attend(*ins[:5], v)
    got = r.rabitq_fused_attend(*[_t(a) for a in ins[:5]], _t(v), None).float().cpu().numpy()
    assert np.all(np.abs(got - ref) <= 2e-3 + 1e-2 * np.abs(ref)), np.abs(got - ref).max()


def test_attend_golden_fixture_gqa_dense_values_and_errors():
    z = np.load(os.path.join(GOLDEN, "rabitq.npz"))
    r = _r()
    for tag in ["att_B1_H1_Sq1_S33_D64", "att_B2_H2_Sq1_S256_D128", "att_B1_H2_Sq4_S64_D256"]:
        g = lambda k: _t(z[f"{tag}_{k}"])  # noqa: E731
        out = r.rabitq_fused_attend(g("q"), g("q_scale"), g("k_bits"), g("k_mag"), g("k_const"), g("v_idx"), g("v_cents"))
        np.testing.assert_allclose(out.float().cpu().numpy(), z[f"{tag}_out"], atol=1e-2, rtol=1e-2)
    # benchmark config 4 form: 32 query heads over 8 kv heads, fp16 values, no k_const,
    # buffers larger than the live context
    B, H, H_kv, S, cap, D = 2, 32, 8, 2000, 2048, 128
    q, q_scale, k_bits, k_mag, _, _, _ = _attend_inputs(B, H, 1, cap, D, seed=9, H_kv=H_kv)
    v = np.random.default_rng(10).standard_normal((B, H_kv, cap, D)).astype(np.float16)
    out = r.rabitq_fused_attend(_t(q), _t(q_scale), _t(k_bits), _t(k_mag), None, _t(v), None, s_kv=S)
    ref = o_rq.reference_attend(q, q_scale, k_bits[:, :, :S], k_mag[:, :, :S], np.zeros((B, H_kv, S), np.float32), v[:, :, :S])
    got = out.float().cpu().numpy()
    assert np.all(np.abs(got - ref) <= 2e-3 + 1e-2 * np.abs(ref)), np.abs(got - ref).max()
    ins = [_t(a) for a in _attend_inputs(1, 2, 1, 16, 64, seed=1)]
    with pytest.raises(ValueError, match="q must be 4D"):
        r.rabitq_fused_attend(ins[0][0], *ins[1:])
    with pytest.raises(ValueError, match="k_mag must be"):
        r.rabitq_fused_attend(ins[0], ins[1], ins[2], ins[3][:, :, :5], *ins[4:])
    with pytest.raises(ValueError, match="at most 16"):
        r.rabitq_fused_attend(*ins[:6], torch.zeros(17, device=DEV))
    with pytest.raises(ValueError, match="v_idx must be"):
        r.rabitq_fused_attend(*ins[:5], ins[5][..., :7], ins[6])


def test_encode_then_attend_composes():
    """Keys encoded on the device feed the attention: sign bits + magnitude estimate the
    rotated inner product (reference: tests/metal/test_rabitq_encode.py:125-164)."""
    r = _r()
    rng = np.random.default_rng(3)
    B, H, S, D = 1, 2, 128, 128
    keys = rng.standard_normal((B * H * S, D)).astype(np.float16)
    diag = r.make_hadamard_diagonal(D, seed=7)
    bits, mag = r.rabitq_encode(_t(keys), _t(diag))
    q = rng.standard_normal((B, H, 1, D)).astype(np.float16)
    q_scale = np.full((B, H, 1), 0.01, np.float32)
    v = rng.standard_normal((B, H, S, D)).astype(np.float16)
    out = r.rabitq_fused_attend(_t(q), _t(q_scale), bits.view(B, H, S, D // 8), mag.view(B, H, S), None, _t(v), None)
    ref = o_rq.reference_attend(q, q_scale, bits.cpu().numpy().reshape(B, H, S, D // 8),
                                mag.cpu().numpy().reshape(B, H, S), np.zeros((B, H, S), np.float32), v)
    assert np.all(np.abs(out.float().cpu().numpy() - ref) <= 2e-3 + 1e-2 * np.abs(ref))


@pytest.mark.parametrize("dt", ["float16", "bfloat16"])
@pytest.mark.parametrize("H,H_kv,S_q", [(8, 8, 1), (8, 2, 2), (16, 2, 1)])
@pytest.mark.parametrize("S,cap", [(32, 32), (1000, 1024), (4097, 4352)])
def test_staged_kernel_dense_values(dt, H, H_kv, S_q, S, cap):
    """Buffers that hold whole 32-key tiles take the bulk-copy staged kernel (head_dim 128, dense
    16-bit values); the same data in buffers that do not must give the same answer."""
    r = _r()
    B, D = 2, 128
    tdt = torch.float16 if dt == "float16" else torch.bfloat16
    q, q_scale, k_bits, k_mag, k_const, _, _ = _attend_inputs(B, H, S_q, cap, D, seed=S + H + S_q, H_kv=H_kv)
    v = torch.from_numpy(np.random.default_rng(S).standard_normal((B, H_kv, cap, D)).astype(np.float32)).to(tdt)
    for kc in (k_const, None):
        out = r.rabitq_fused_attend(_t(q), _t(q_scale), _t(k_bits), _t(k_mag), None if kc is None else _t(kc),
                                    v.to(DEV), None, s_kv=S)
        ref = o_rq.reference_attend(q, q_scale, k_bits[:, :, :S], k_mag[:, :, :S],
                                    np.zeros((B, H_kv, S), np.float32) if kc is None else kc[:, :, :S],
                                    v[:, :, :S].float().numpy())
        got = out.float().cpu().numpy()
        assert np.all(np.abs(got - ref) <= 2e-3 + 1e-2 * np.abs(ref)), np.abs(got - ref).max()
        # exact-size buffers with an odd length cannot be staged
        if S % 4:
            plain = r.rabitq_fused_attend(_t(q), _t(q_scale), _t(k_bits[:, :, :S].copy()), _t(k_mag[:, :, :S].copy()),
                                          None if kc is None else _t(kc[:, :, :S].copy()), v[:, :, :S].contiguous().to(DEV), None)
            torch.testing.assert_close(out.float(), plain.float(), atol=2e-3, rtol=1e-2)
    from veloxquant_mlx_b200._lib import lib
    assert lib().vq_kivi_attend_status() == 0
