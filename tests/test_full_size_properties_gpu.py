"""Parity at the full benchmark sizes through properties that do not need the oracle to run at
that size: quantize -> dequantize error bounds, exact reconstruction of constant groups,
softmax weights summing to one (constant values come back exactly), identical inputs in
different batch slots giving identical outputs, independence from the context split count,
and agreement of a strided sample of (batch, head) units with the oracle."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import bitpack as o_bp
from oracle import kivi as o_kivi

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _layer(B, H_kv, S, D, dtype, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    k = torch.randn(B, H_kv, S, D, device=DEV, dtype=torch.float32, generator=g)
    v = torch.randn(B, H_kv, S, D, device=DEV, dtype=torch.float32, generator=g)
    k[..., [3, 40, 77, 120]] *= 20.0  # the outlier recipe of the reference's own tests
    v[..., [5, 60]] *= 20.0
    return k.to(dtype), v.to(dtype)


@pytest.mark.parametrize("name,B,H_q,H_kv,S,bits,dtype", [
    ("config3", 16, 32, 8, 32768, 4, torch.bfloat16),   # Llama-3.1-8B-shaped decode layer
    ("config5", 4, 40, 8, 16640, 2, torch.float16),     # Qwen2.5-32B-shaped layer after 256 decode steps
])
def test_full_size_layer_properties(name, B, H_q, H_kv, S, bits, dtype):
    from veloxquant_mlx_b200 import kernels as k

    D, g, R = 128, 32, 128
    levels = (1 << bits) - 1
    keys, values = _layer(B, H_kv, S, D, dtype, seed=len(name))
    n_q = o_kivi.quantization_boundary(S, R, g)
    kc, ks, kz = k.kivi_quantize(keys[:, :, :n_q], -2, g, bits)
    vc, vs, vz = k.kivi_quantize(values[:, :, :n_q], -1, g, bits)
    sb = k.storage_bits(bits)

    # 1. round trip: |x - x_hat| <= scale/2 (+ rounding of x_hat to the 16-bit type)
    k_hat = k.scalar_decode_once(kc, ks, kz, g, "K", store_bits=sb, out_dtype=torch.float32)
    err = (k_hat - keys[:, :, :n_q].float()).abs()
    bound = ks.repeat_interleave(g, dim=2) * 0.5 * (1 + 1e-5) + 1e-6
    assert bool((err <= bound).all()), float((err - bound).max())
    v_hat = k.scalar_decode_once(vc, vs, vz, g, "V", store_bits=sb, out_dtype=torch.float32)
    errv = (v_hat - values[:, :, :n_q].float()).abs()
    boundv = vs.repeat_interleave(g, dim=3) * 0.5 * (1 + 1e-5) + 1e-6
    assert bool((errv <= boundv).all())
    # scale and zero follow from the group extrema exactly
    kmin = keys[:, :, :n_q].float().reshape(B, H_kv, n_q // g, g, D).amin(3)
    kmax = keys[:, :, :n_q].float().reshape(B, H_kv, n_q // g, g, D).amax(3)
    assert torch.equal(kz, kmin)
    # (tensor / tensor: a true IEEE divide; a Python-scalar divisor would become a reciprocal multiply)
    assert torch.equal(ks, torch.clamp(torch.div(kmax - kmin, torch.full_like(kmax, float(levels))), min=1e-8))

    # 2. a strided sample of units against the oracle, bit for bit
    for b, h in ((0, 0), (B - 1, H_kv - 1), (B // 2, 3)):
        oc, os_, oz = o_kivi.quant_keys(keys[b, h, :n_q].float().cpu().numpy()[None, None], g, levels)
        np.testing.assert_array_equal(o_bp.unpack(kc[b, h].cpu().numpy(), sb, D), oc[0, 0])
        np.testing.assert_array_equal(ks[b, h].cpu().numpy(), os_[0, 0])
        ov, ovs, ovz = o_kivi.quant_values(values[b, h, :n_q].float().cpu().numpy()[None, None], g, levels)
        np.testing.assert_array_equal(o_bp.unpack(vc[b, h].cpu().numpy(), sb, D), ov[0, 0])
        np.testing.assert_array_equal(vz[b, h].cpu().numpy(), ovz[0, 0])

    # 3. attention: output of the sampled units against the oracle on the same codes
    q = torch.randn(B, H_q, 1, D, device=DEV, dtype=dtype)
    scale = D ** -0.5
    k_res, v_res = keys[:, :, n_q:].contiguous(), values[:, :, n_q:].contiguous()
    out = k.kivi_decode_attend(q, kc, ks, kz, vc, vs, vz, g, scale, store_bits=sb, k_res=k_res, v_res=v_res)
    hpk = H_q // H_kv
    for b, h in ((0, 0), (B - 1, H_kv - 1)):
        k_full = np.concatenate([o_kivi.dequant_keys(o_bp.unpack(kc[b, h].cpu().numpy(), sb, D)[None, None], ks[b, h].cpu().numpy()[None, None],
                                                     kz[b, h].cpu().numpy()[None, None], g)[0, 0], k_res[b, h].float().cpu().numpy()])
        v_full = np.concatenate([o_kivi.dequant_values(o_bp.unpack(vc[b, h].cpu().numpy(), sb, D)[None, None], vs[b, h].cpu().numpy()[None, None],
                                                       vz[b, h].cpu().numpy()[None, None], g)[0, 0], v_res[b, h].float().cpu().numpy()])
        qh = q[b, h * hpk:(h + 1) * hpk, 0].float().cpu().numpy()
        s = (qh @ k_full.T) * np.float32(scale)
        w = np.exp(s - s.max(-1, keepdims=True))
        ref = (w / w.sum(-1, keepdims=True)) @ v_full
        got = out[b, h * hpk:(h + 1) * hpk, 0].float().cpu().numpy()
        assert np.all(np.abs(got - ref) <= 2e-3 + 1e-2 * np.abs(ref)), np.abs(got - ref).max()

    # 4. the split count does not matter
    out1 = k.kivi_decode_attend(q, kc, ks, kz, vc, vs, vz, g, scale, store_bits=sb, k_res=k_res, v_res=v_res, n_splits=3)
    torch.testing.assert_close(out1.float(), out.float(), atol=2e-3, rtol=1e-2)

    # 5. identical units in different batch slots give identical outputs
    for t in (kc, ks, kz, vc, vs, vz, k_res, v_res):
        t[B - 1].copy_(t[0])
    q[B - 1].copy_(q[0])
    out2 = k.kivi_decode_attend(q, kc, ks, kz, vc, vs, vz, g, scale, store_bits=sb, k_res=k_res, v_res=v_res)
    assert torch.equal(out2[0], out2[B - 1])

    # 6. constant values come back exactly: the weights sum to one, a constant group has codes 0
    const = torch.full_like(values[:, :, :n_q], 0.75)
    cc, cs, cz = k.kivi_quantize(const, -1, g, bits)
    assert int(cc.max()) == 0 and bool((cz == 0.75).all())
    out3 = k.kivi_decode_attend(q, kc, ks, kz, cc, cs, cz, g, scale, store_bits=sb,
                                k_res=k_res, v_res=torch.full_like(v_res, 0.75))
    torch.testing.assert_close(out3.float(), torch.full_like(out3, 0.75).float(), atol=2e-3, rtol=0)
    from veloxquant_mlx_b200._lib import lib
    assert lib().vq_kivi_attend_status() == 0


def test_full_size_rabitq_config4_properties():
    """benchmark config 4 at full size: batch 8, 8 KV heads, 16384 keys of dim 128, 32 query heads."""
    from oracle import rabitq as o_rq
    from veloxquant_mlx_b200 import rabitq as rq

    B, H_q, H_kv, S, D = 8, 32, 8, 16384, 128
    g = torch.Generator(device=DEV).manual_seed(4)
    keys = torch.randn(B * H_kv * S, D, device=DEV, dtype=torch.float16, generator=g)
    diag_np = rq.make_hadamard_diagonal(D, seed=42)
    diag = torch.from_numpy(diag_np).to(DEV)
    bits, mag = rq.rabitq_encode(keys, diag)
    # sample rows against the oracle, bit for bit
    idx = torch.arange(0, B * H_kv * S, 4099, device=DEV)
    obits, omag, _ = o_rq.encode_hadamard(keys[idx].cpu().numpy(), diag_np)
    np.testing.assert_array_equal(bits[idx].cpu().numpy(), obits)
    np.testing.assert_allclose(mag[idx].cpu().numpy(), omag, rtol=1e-4)
    # magnitude = mean |rotated key| >= 0, and the rotation keeps the norm: sum y^2 = sum k^2, so
    # mean|y| <= sqrt(mean k^2)
    rms = keys.float().pow(2).mean(1).sqrt()
    assert bool((mag >= 0).all()) and bool((mag <= rms * (1 + 1e-3)).all())
    # sign bits of -k are the complement of those of k wherever y != 0 (the transform is linear)
    nb, _ = rq.rabitq_encode(-keys[:65536], diag)
    assert int((nb ^ bits[:65536]).to(torch.int32).ne(255).sum()) < 65536 * 16 * 1e-3

    v = torch.randn(B, H_kv, S, D, device=DEV, dtype=torch.float16, generator=g)
    q = torch.randn(B, H_q, 1, D, device=DEV, dtype=torch.float16, generator=g)
    qs = torch.full((B, H_q, 1), 0.01, device=DEV)
    kb, km = bits.view(B, H_kv, S, D // 8), mag.view(B, H_kv, S)
    out = rq.rabitq_fused_attend(q, qs, kb, km, None, v, None)
    hpk = H_q // H_kv
    for b, h in ((0, 0), (B - 1, H_kv - 1)):
        ref = o_rq.reference_attend(q[b:b + 1, h * hpk:(h + 1) * hpk].cpu().numpy(), qs[b:b + 1, h * hpk:(h + 1) * hpk].cpu().numpy(),
                                    kb[b:b + 1, h:h + 1].cpu().numpy(), km[b:b + 1, h:h + 1].cpu().numpy(),
                                    np.zeros((1, 1, S), np.float32), v[b:b + 1, h:h + 1].cpu().numpy())
        got = out[b:b + 1, h * hpk:(h + 1) * hpk].float().cpu().numpy()
        assert np.all(np.abs(got - ref) <= 2e-3 + 1e-2 * np.abs(ref)), np.abs(got - ref).max()
    # split count does not matter; constant values come back; identical slots give identical rows
    out1 = rq.rabitq_fused_attend(q, qs, kb, km, None, v, None, n_splits=5)
    torch.testing.assert_close(out1.float(), out.float(), atol=2e-3, rtol=1e-2)
    outc = rq.rabitq_fused_attend(q, qs, kb, km, None, torch.full_like(v, -1.5), None)
    torch.testing.assert_close(outc.float(), torch.full_like(outc, -1.5).float(), atol=2e-3, rtol=0)
    kb2, km2, v2, q2, qs2 = kb.clone(), km.clone(), v.clone(), q.clone(), qs.clone()
    for t in (kb2, km2, v2, q2, qs2):
        t[B - 1].copy_(t[0])
    out2 = rq.rabitq_fused_attend(q2, qs2, kb2, km2, None, v2, None)
    assert torch.equal(out2[0], out2[B - 1])
    from veloxquant_mlx_b200._lib import lib
    assert lib().vq_kivi_attend_status() == 0


def test_full_size_skvq_properties():
    """1 Mi rows of 128 channels (a 16K-token prefill of 64 (batch, head) blocks) through the SKVQ
    kernels: with one clip factor of 1 every element is reconstructed to within half a step and every
    group uses both end codes; the searched factor is never worse per group; a permuted round trip
    equals the plain round trip of the pre-permuted rows; a sample of rows equals the oracle."""
    from oracle import skvq as o_skvq
    from veloxquant_mlx_b200 import skvq

    n_bh, n_tok, D, gs, bits = 64, 16384, 128, 32, 4
    g = torch.Generator(device=DEV).manual_seed(11)
    x = torch.randn(n_bh, n_tok, D, device=DEV, dtype=torch.float32, generator=g)
    x[..., [3, 40, 77, 120]] *= 20.0
    x = x.to(torch.float16)
    x32 = x.float()
    packed, lo, scale = skvq.quantize_pack(x, bits, gs, (1.0,))
    rt1 = skvq.unpack_dequant(packed, lo, scale, bits, gs, n_tok, torch.float32)
    step = scale.repeat_interleave(gs, dim=-1)
    assert bool(((rt1 - x32).abs() <= 0.5 * step * (1 + 1e-5) + 1e-6).all())
    codes = skvq.unpack_dequant(packed, torch.zeros_like(lo), torch.ones_like(scale), bits, gs, n_tok, torch.float32)
    cg = codes.reshape(n_bh, n_tok, D // gs, gs)
    assert bool((cg.amin(-1) == 0).all()) and bool((cg.amax(-1) == 15).all())
    e1 = ((rt1 - x32) ** 2).reshape(n_bh, n_tok, D // gs, gs).sum(-1)
    del rt1, codes, cg, step
    packed5 = skvq.quantize_pack(x, bits, gs)
    rt5 = skvq.unpack_dequant(*packed5, bits, gs, n_tok, torch.float32)
    e5 = ((rt5 - x32) ** 2).reshape(n_bh, n_tok, D // gs, gs).sum(-1)
    assert bool((e5 <= e1 * (1 + 1e-5) + 1e-9).all()) and float(e5.sum()) < float(e1.sum())
    del e1, e5, rt5
    perm = torch.stack([torch.randperm(D, generator=torch.Generator().manual_seed(h)) for h in range(8)]).to(torch.int32).to(DEV)
    inv = torch.argsort(perm.long(), dim=-1).to(torch.int32)
    pp = skvq.quantize_pack(x, bits, gs, perm=perm)
    a = skvq.unpack_dequant(*pp, bits, gs, n_tok, torch.float16, inv_perm=inv)
    xp = torch.gather(x, 2, perm.long()[torch.arange(n_bh, device=DEV) % 8][:, None, :].expand(n_bh, n_tok, D))
    b = skvq.unpack_dequant(*skvq.quantize_pack(xp, bits, gs), bits, gs, n_tok, torch.float16)
    b = torch.gather(b, 2, inv.long()[torch.arange(n_bh, device=DEV) % 8][:, None, :].expand(n_bh, n_tok, D))
    assert torch.equal(a, b)
    rows = x[5::16, 100::4000].reshape(-1, D).cpu().numpy()
    oc, olo, osc = o_skvq.clipped_group_quant(rows, bits, gs)
    got = tuple(t[5::16, 100::4000] for t in packed5)
    np.testing.assert_array_equal(got[0].reshape(-1, D * bits // 8).cpu().numpy(), o_bp.pack(oc, bits))
    np.testing.assert_array_equal(got[1].reshape(-1, D // gs).cpu().numpy(), olo)
    np.testing.assert_array_equal(got[2].reshape(-1, D // gs).cpu().numpy(), osc)
