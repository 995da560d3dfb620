"""GPU parity for the KIVI path, through the C ABI, against the CPU oracle and the
committed golden fixtures. Mirrors the reference's own parametrisations:
tests/metal/test_kivi_quant.py, tests/metal/test_scalar_attend.py, tests/metal/test_worker_kernel_parity.py.

Tolerance: integer outputs (codes, packed bytes) and float32 scale/zero are bit-exact;
attention outputs satisfy |got - ref| <= 2e-3 + 1e-2*|ref| (and max-abs < 2e-3 on the
reference's N(0,1) cases, as its own tests require).
"""

from __future__ import annotations

import math
import os

import numpy as np
import pytest
import torch

from oracle import bitpack as o_bitpack
from oracle import kivi as o_kivi

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DEV = "cuda:0"

_TORCH_DT = {"float16": torch.float16, "float32": torch.float32, "bfloat16": torch.bfloat16}


def _k():
    from veloxquant_mlx_b200 import kernels

    return kernels


def _np_cast(x32: np.ndarray, dt: str):
    """float32 ndarray -> (torch tensor on GPU in dtype dt, the same values as float32 ndarray)."""
    t = torch.from_numpy(x32).to(_TORCH_DT[dt])
    return t.to(DEV), t.to(torch.float32).numpy()


def _assert_attn_close(got: np.ndarray, ref: np.ndarray, strict=True):
    err = np.abs(got - ref)
    bound = 2e-3 + 1e-2 * np.abs(ref)
    assert np.all(err <= bound), f"max err {err.max():.3e}, worst excess {(err - bound).max():.3e}"
    if strict:
        assert err.max() < 2e-3, f"max|abs|={err.max():.3e}"


# ----------------------------------------------------------------- quant round trip
@pytest.mark.parametrize("dt", ["float16", "float32", "bfloat16"])
@pytest.mark.parametrize("b", [1, 2, 4, 8])
@pytest.mark.parametrize("g", [4, 32, 128])
@pytest.mark.parametrize("axis", [-1, -2])
def test_quant_dequant_bit_exact(dt, b, g, axis):
    rng = np.random.default_rng(b * 100 + g)
    levels = (1 << b) - 1
    for shape in [(1, 2, 64, 128), (2, 1, 33, 64), (1, 1, 7, 32), (1, 2, 200, 96), (1, 1, 50, 128)]:
        xt, x32 = _np_cast(rng.standard_normal(shape).astype(np.float32), dt)
        got = _k().kivi_group_quant_dequant(xt, axis, g, levels)
        assert got.dtype == xt.dtype and got.shape == xt.shape
        want32 = o_kivi.quant_dequant_along(x32, axis, g, levels)
        want = torch.from_numpy(want32).to(_TORCH_DT[dt])
        assert torch.equal(got.cpu(), want), f"shape={shape}"


def test_quant_dequant_special_values():
    k = _k()
    # round-half-even on integer data (reference: test_kivi_quant.py:121-127)
    x = torch.tensor(np.tile(np.array([0, 1, 2, 3], np.float32), 8).reshape(1, 1, 1, 32), device=DEV)
    got = k.kivi_group_quant_dequant(x, -1, 32, 2).cpu().numpy()
    np.testing.assert_array_equal(got, o_kivi.quant_dequant_along(x.cpu().numpy(), -1, 32, 2))
    # eps floor on a constant group
    c = torch.full((1, 1, 32, 8), 3.5, device=DEV)
    assert torch.equal(k.kivi_group_quant_dequant(c, -2, 32, 3), c)
    # group of one is lossless
    r = torch.randn(1, 2, 9, 16, device=DEV, dtype=torch.float16)
    assert torch.equal(k.kivi_group_quant_dequant(r, -1, 1, 3), r)
    assert torch.equal(k.kivi_group_quant_dequant(r, -2, 1, 3), r)
    # no-FMA reconstruction at b=8 (reference: test_kivi_quant.py:130-137)
    big = np.random.default_rng(0).standard_normal((1, 4, 256, 128)).astype(np.float32)
    got = k.kivi_group_quant_dequant(torch.from_numpy(big).to(DEV), -2, 32, 255).cpu().numpy()
    np.testing.assert_array_equal(got, o_kivi.quant_dequant_along(big, -2, 32, 255))
    # empty input returns as is; slices of a larger buffer are read through their strides
    e = torch.empty(1, 1, 0, 8, device=DEV)
    assert k.kivi_group_quant_dequant(e, -1, 4, 3).shape == e.shape
    buf = torch.randn(2, 3, 100, 64, device=DEV, dtype=torch.float16)
    sl = buf[:, :, 32:96, :]
    got = k.kivi_group_quant_dequant(sl, -2, 32, 3).cpu().numpy()
    np.testing.assert_array_equal(got, o_kivi.quant_dequant_along(sl.cpu().numpy(), -2, 32, 3))


# ----------------------------------------------------------------- codes + params
@pytest.mark.parametrize("dt", ["float16", "bfloat16", "float32"])
@pytest.mark.parametrize("b,g,shape", [
    (2, 32, (1, 8, 256, 128)), (4, 32, (2, 2, 96, 128)), (1, 4, (1, 2, 33, 32)), (8, 128, (1, 1, 200, 128)),
    (3, 32, (1, 2, 50, 96)), (4, 32, (1, 2, 50, 64)), (2, 16, (1, 1, 40, 256)),
])
def test_quantize_pack_bit_exact(dt, b, g, shape):
    rng = np.random.default_rng(b + g)
    levels = (1 << b) - 1
    xt, x32 = _np_cast(rng.standard_normal(shape).astype(np.float32) * 3.0, dt)
    k = _k()
    sb = k.storage_bits(b)
    # keys
    kc, ks, kz = k.kivi_quantize(xt, -2, g, b)
    oc, os_, oz = o_kivi.quant_keys(x32, g, levels)
    np.testing.assert_array_equal(kc.cpu().numpy(), o_bitpack.pack(oc, sb))
    np.testing.assert_array_equal(ks.cpu().numpy(), os_)
    np.testing.assert_array_equal(kz.cpu().numpy(), oz)
    # values
    vc, vs, vz = k.kivi_quantize(xt, -1, g, b)
    oc, os_, oz = o_kivi.quant_values(x32, g, levels)
    np.testing.assert_array_equal(vc.cpu().numpy(), o_bitpack.pack(oc, sb))
    np.testing.assert_array_equal(vs.cpu().numpy(), os_)
    np.testing.assert_array_equal(vz.cpu().numpy(), oz)
    # one code per byte (the reference's own layout)
    uc, _, _ = k.kivi_quantize(xt, -1, g, b, store_bits=8)
    np.testing.assert_array_equal(uc.cpu().numpy(), oc)
    # decode-once reproduces code*scale+zero
    deq = k.scalar_decode_once(vc, vs, vz, g, "V", store_bits=sb, out_dtype=torch.float32)
    np.testing.assert_array_equal(deq.cpu().numpy(), o_kivi.dequant_values(oc, os_, oz, g))
    deq = k.scalar_decode_once(kc, ks, kz, g, "K", store_bits=sb, out_dtype=torch.float32)
    oc, os_, oz = o_kivi.quant_keys(x32, g, levels)
    np.testing.assert_array_equal(deq.cpu().numpy(), o_kivi.dequant_keys(oc, os_, oz, g))


def test_quantize_matches_golden_fixture():
    z = np.load(os.path.join(GOLDEN, "kivi.npz"))
    k = _k()
    for name in [str(n) for n in z["names"]]:
        B, H, S_kv, D, b, g, seed, H_kv = [int(v) for v in z[f"{name}_meta"]]
        H_kv = H if H_kv < 0 else H_kv
        rng = np.random.default_rng(seed)
        rng.standard_normal((B, H, 1, D))
        kf = rng.standard_normal((B, H_kv, S_kv, D)).astype(np.float32)
        vf = rng.standard_normal((B, H_kv, S_kv, D)).astype(np.float32)
        kc, ks, kz = k.kivi_quantize(torch.from_numpy(kf).to(DEV), -2, g, b, store_bits=8)
        vc, vs, vz = k.kivi_quantize(torch.from_numpy(vf).to(DEV), -1, g, b, store_bits=8)
        for got, key in [(kc, "kc"), (ks, "ks"), (kz, "kz"), (vc, "vc"), (vs, "vs"), (vz, "vz")]:
            np.testing.assert_array_equal(got.cpu().numpy(), z[f"{name}_{key}"], err_msg=f"{name}:{key}")


def test_quantize_into_cache_buffers_at_offset():
    k = _k()
    B, H, D, g, b, cap = 2, 2, 128, 32, 4, 256
    x = torch.randn(B, H, 64, D, device=DEV, dtype=torch.float16)
    codes = torch.zeros(B, H, cap, D // 2, dtype=torch.uint8, device=DEV)
    ks = torch.zeros(B, H, cap // g, D, device=DEV)
    kz = torch.zeros_like(ks)
    k.kivi_quantize_into(x, -2, g, b, codes=codes, scale=ks, zero=kz, tok_offset=96)
    oc, os_, oz = o_kivi.quant_keys(x.cpu().numpy(), g, 15)
    np.testing.assert_array_equal(codes[:, :, 96:160].cpu().numpy(), o_bitpack.pack(oc, 4))
    np.testing.assert_array_equal(ks[:, :, 3:5].cpu().numpy(), os_)
    assert codes[:, :, :96].abs().sum() == 0 and codes[:, :, 160:].abs().sum() == 0
    with pytest.raises(RuntimeError):
        k.kivi_quantize_into(x, -2, g, b, codes=codes, scale=ks, zero=kz, tok_offset=224)


# ----------------------------------------------------------------- bit pack
@pytest.mark.parametrize("b", [1, 2, 4])
def test_bit_pack_roundtrip_and_known_answer(b):
    k = _k()
    rng = np.random.default_rng(b)
    vals = rng.integers(0, 1 << b, 4096, dtype=np.uint8)
    packed = k.turboquant_bit_pack(torch.from_numpy(vals).to(DEV), b)
    np.testing.assert_array_equal(packed.cpu().numpy(), o_bitpack.pack(vals, b))
    back = k.turboquant_bit_unpack(packed, 4096, b)
    np.testing.assert_array_equal(back.cpu().numpy(), vals)
    if b == 2:
        ka = k.turboquant_bit_pack(torch.tensor([0, 1, 2, 3, 0, 1, 2, 3], dtype=torch.uint8, device=DEV), 2)
        assert ka.cpu().tolist() == [228, 228]
    with pytest.raises(ValueError):
        k.turboquant_bit_pack(torch.zeros(3, dtype=torch.uint8, device=DEV), b if b > 1 else 2)
    with pytest.raises(ValueError):
        k.turboquant_bit_unpack(packed[:1], 4096, b)


# ----------------------------------------------------------------- attend
def _to_dev(*arrs):
    return [torch.from_numpy(np.ascontiguousarray(a)).to(DEV) for a in arrs]


def _attend_unpacked(q, kc, ks, kz, vc, vs, vz, g, scale, **kw):
    tq, tkc, tks, tkz, tvc, tvs, tvz = _to_dev(q, kc, ks, kz, vc, vs, vz)
    out = _k().scalar_fused_decode_attend(tq, tkc, tks, tkz, tvc, tvs, tvz, g, scale, **kw)
    assert out.dtype == torch.float16
    return out.float().cpu().numpy()


@pytest.mark.parametrize("S_kv", [64, 512, 2048])
@pytest.mark.parametrize("nsg", [None, 1, 2, 4, 8])
def test_scalar_attend_parity(S_kv, nsg):
    B, H, D, b, g = 1, 4, 128, 2, 32
    scale = 1.0 / math.sqrt(D)
    ins = o_kivi.make_inputs(B, H, S_kv, D, b, g)
    ref = o_kivi.reference_attend(*ins, g, scale)
    got = _attend_unpacked(*ins, g, scale, nsg=nsg)
    assert got.shape == ref.shape
    _assert_attn_close(got, ref)


@pytest.mark.parametrize("b", [2, 3, 4])
def test_scalar_attend_bitwidths(b):
    B, H, D, g, S_kv = 1, 4, 128, 32, 1024
    scale = 1.0 / math.sqrt(D)
    ins = o_kivi.make_inputs(B, H, S_kv, D, b, g, seed=b)
    _assert_attn_close(_attend_unpacked(*ins, g, scale), o_kivi.reference_attend(*ins, g, scale))


@pytest.mark.parametrize("H_q,H_kv", [(8, 2), (32, 4), (32, 8), (16, 1)])
@pytest.mark.parametrize("S_kv", [64, 512, 2048])
def test_scalar_attend_gqa_parity(H_q, H_kv, S_kv):
    D, b, g = 128, 2, 32
    scale = 1.0 / math.sqrt(D)
    ins = o_kivi.make_inputs(1, H_q, S_kv, D, b, g, H_kv=H_kv)
    _assert_attn_close(_attend_unpacked(*ins, g, scale), o_kivi.reference_attend(*ins, g, scale))


def test_scalar_attend_batch_and_golden_fixture():
    z = np.load(os.path.join(GOLDEN, "kivi.npz"))
    for name in [str(n) for n in z["names"]]:
        B, H, S_kv, D, b, g, seed, H_kv = [int(v) for v in z[f"{name}_meta"]]
        g_ = lambda key: z[f"{name}_{key}"]  # noqa: E731
        got = _attend_unpacked(g_("q"), g_("kc"), g_("ks"), g_("kz"), g_("vc"), g_("vs"), g_("vz"),
                               g, 1.0 / math.sqrt(D))
        _assert_attn_close(got, g_("out"))


@pytest.mark.parametrize("D", [32, 64, 96, 256])
@pytest.mark.parametrize("S_q", [1, 3])
def test_scalar_attend_head_dims_and_query_rows(D, S_q):
    rng = np.random.default_rng(D + S_q)
    B, H, H_kv, S_kv, b, g = 2, 4, 2, 100, 4, 32
    q = rng.standard_normal((B, H, S_q, D)).astype(np.float16)
    kf = rng.standard_normal((B, H_kv, S_kv, D)).astype(np.float32)
    vf = rng.standard_normal((B, H_kv, S_kv, D)).astype(np.float32)
    kc, ks, kz = o_kivi.quant_keys(kf, g, 15)
    vc, vs, vz = o_kivi.quant_values(vf, g, 15)
    scale = 1.0 / math.sqrt(D)
    ref = o_kivi.reference_attend(q, kc, ks, kz, vc, vs, vz, g, scale)
    _assert_attn_close(_attend_unpacked(q, kc, ks, kz, vc, vs, vz, g, scale), ref)


@pytest.mark.parametrize("b", [1, 2, 4])
@pytest.mark.parametrize("n_res", [0, 1, 37, 159])
@pytest.mark.parametrize("dt", ["float16", "bfloat16"])
def test_packed_attend_with_residual_tail(b, n_res, dt):
    """Packed codes + unquantized tail in one call (general kernel forced)."""
    rng = np.random.default_rng(b * 7 + n_res)
    B, H, H_kv, D, g, n_quant = 2, 8, 2, 128, 32, 192
    levels = (1 << b) - 1
    k = _k()
    qt, q32 = _np_cast(rng.standard_normal((B, H, 1, D)).astype(np.float32), dt)
    kt, k32 = _np_cast(rng.standard_normal((B, H_kv, n_quant + n_res, D)).astype(np.float32), dt)
    vt, v32 = _np_cast(rng.standard_normal((B, H_kv, n_quant + n_res, D)).astype(np.float32), dt)
    kc, ks, kz = k.kivi_quantize(kt[:, :, :n_quant], -2, g, b)
    vc, vs, vz = k.kivi_quantize(vt[:, :, :n_quant], -1, g, b)
    k_res = kt[:, :, n_quant:].contiguous() if n_res else None
    v_res = vt[:, :, n_quant:].contiguous() if n_res else None
    scale = 1.0 / math.sqrt(D)
    out = k.kivi_decode_attend(qt, kc, ks, kz, vc, vs, vz, g, scale, store_bits=b, k_res=k_res,
                               v_res=v_res, variant=1)
    assert out.dtype == qt.dtype
    okc, oks, okz = o_kivi.quant_keys(k32[:, :, :n_quant], g, levels)
    ovc, ovs, ovz = o_kivi.quant_values(v32[:, :, :n_quant], g, levels)
    ref = o_kivi.reference_attend(q32, okc, oks, okz, ovc, ovs, ovz, g, scale,
                                  k_res=k32[:, :, n_quant:], v_res=v32[:, :, n_quant:])
    _assert_attn_close(out.float().cpu().numpy(), ref, strict=(dt == "float16"))


def test_predecoded_attend_and_validation_errors():
    k = _k()
    rng = np.random.default_rng(0)
    q = torch.from_numpy(rng.standard_normal((1, 8, 1, 64)).astype(np.float16)).to(DEV)
    kh = torch.from_numpy(rng.standard_normal((1, 2, 300, 64)).astype(np.float16)).to(DEV)
    vh = torch.from_numpy(rng.standard_normal((1, 2, 300, 64)).astype(np.float16)).to(DEV)
    out = k.scalar_predecoded_attend(q, kh, vh, 0.125)
    ref = o_kivi.reference_attend(q.cpu().numpy(), None, None, None, None, None, None, 1, 0.125,
                                  k_res=kh.cpu().numpy(), v_res=vh.cpu().numpy())
    _assert_attn_close(out.float().cpu().numpy(), ref)
    ins = _to_dev(*o_kivi.make_inputs(1, 4, 64, 128, 2, 32))
    with pytest.raises(ValueError, match="q must be 4D"):
        k.scalar_fused_decode_attend(ins[0][0], *ins[1:], 32, 0.1)
    with pytest.raises(ValueError, match="nsg=.* must be in 1..32"):
        k.scalar_fused_decode_attend(*ins, 32, 0.1, nsg=33)
    with pytest.raises(ValueError, match="multiple of"):
        k.scalar_fused_decode_attend(ins[0][:, :3], *ins[1:], 32, 0.1)
    with pytest.raises(ValueError, match="batch mismatch"):
        k.scalar_fused_decode_attend(torch.cat([ins[0], ins[0]]), *ins[1:], 32, 0.1)
    bigq = torch.zeros(1, 34, 1, 128, dtype=torch.float16, device=DEV)
    one = [t[:, :1].contiguous() for t in ins[1:]]
    with pytest.raises(ValueError, match="exceeds the supported maximum"):
        k.scalar_fused_decode_attend(bigq[:, :17 * 1], *[t for t in one], 32, 0.1)


# ----------------------------------------------------------------- tensor-core kernel
def _packed_case(rng, B, H, H_kv, n_quant, n_res, b, dt, outliers=False):
    D, g = 128, 32
    k = _k()
    kf = rng.standard_normal((B, H_kv, n_quant + n_res, D)).astype(np.float32)
    vf = rng.standard_normal((B, H_kv, n_quant + n_res, D)).astype(np.float32)
    if outliers:  # 4 fixed outlier channels per head, x20 (reference: tests/allocators/test_vecinfer.py:67-77)
        for h in range(H_kv):
            ch = rng.choice(D, size=4, replace=False)
            kf[:, h, :, ch] *= 20.0
            vf[:, h, :, ch] *= 20.0
    qt, q32 = _np_cast(rng.standard_normal((B, H, 1, D)).astype(np.float32), dt)
    kt, k32 = _np_cast(kf, dt)
    vt, v32 = _np_cast(vf, dt)
    kc, ks, kz = k.kivi_quantize(kt[:, :, :n_quant], -2, g, b)
    vc, vs, vz = k.kivi_quantize(vt[:, :, :n_quant], -1, g, b)
    levels = (1 << b) - 1
    okc, oks, okz = o_kivi.quant_keys(k32[:, :, :n_quant], g, levels)
    ovc, ovs, ovz = o_kivi.quant_values(v32[:, :, :n_quant], g, levels)
    np.testing.assert_array_equal(kc.cpu().numpy(), o_bitpack.pack(okc, b))
    np.testing.assert_array_equal(vc.cpu().numpy(), o_bitpack.pack(ovc, b))
    ref = o_kivi.reference_attend(q32, okc, oks, okz, ovc, ovs, ovz, g, 1.0 / math.sqrt(D),
                                  k_res=k32[:, :, n_quant:], v_res=v32[:, :, n_quant:])
    k_res = kt[:, :, n_quant:].contiguous() if n_res else None
    v_res = vt[:, :, n_quant:].contiguous() if n_res else None
    return (qt, kc, ks, kz, vc, vs, vz, k_res, v_res), ref


@pytest.mark.parametrize("b", [2, 4])
@pytest.mark.parametrize("H,H_kv", [(4, 4), (8, 4), (8, 2), (8, 1), (12, 2)])
@pytest.mark.parametrize("n_quant,n_res", [(32, 0), (128, 5), (160, 128), (1024 + 96, 37), (4096 - 128, 128)])
def test_mma_attend_parity(b, H, H_kv, n_quant, n_res):
    rng = np.random.default_rng(b + H + n_quant)
    (qt, kc, ks, kz, vc, vs, vz, k_res, v_res), ref = _packed_case(rng, 2, H, H_kv, n_quant, n_res, b, "float16")
    k = _k()
    out = k.kivi_decode_attend(qt, kc, ks, kz, vc, vs, vz, 32, 1.0 / math.sqrt(128), store_bits=b,
                               k_res=k_res, v_res=v_res, variant=2)
    _assert_attn_close(out.float().cpu().numpy(), ref)
    from veloxquant_mlx_b200 import _lib
    _lib.check(_lib.lib().vq_kivi_attend_status(), "status")
    # the general kernel agrees too, and an explicit split count changes nothing material
    out1 = k.kivi_decode_attend(qt, kc, ks, kz, vc, vs, vz, 32, 1.0 / math.sqrt(128), store_bits=b,
                                k_res=k_res, v_res=v_res, variant=1)
    _assert_attn_close(out1.float().cpu().numpy(), ref)
    out3 = k.kivi_decode_attend(qt, kc, ks, kz, vc, vs, vz, 32, 1.0 / math.sqrt(128), store_bits=b,
                                k_res=k_res, v_res=v_res, variant=2, n_splits=3)
    _assert_attn_close(out3.float().cpu().numpy(), ref)


@pytest.mark.parametrize("b", [2, 4])
@pytest.mark.parametrize("B,H,H_kv", [(3, 40, 8), (4, 48, 6), (12, 14, 2)])
def test_mma_attend_parity_more_than_four_heads_long_context(b, B, H, H_kv):
    """5, 8 and 7 query heads per kv head over a context long and wide enough (512 groups or more,
    12288 unit-groups or more) that the launch takes the eight-head kernel; plain and overlapped
    launches, automatic and explicit splits."""
    rng = np.random.default_rng(b + H)
    (qt, kc, ks, kz, vc, vs, vz, k_res, v_res), ref = _packed_case(rng, B, H, H_kv, 16384 + 32, 37, b, "bfloat16")
    k = _k()
    for kw in ({}, {"n_splits": 3}, {"overlap_previous": True}):
        out = k.kivi_decode_attend(qt, kc, ks, kz, vc, vs, vz, 32, 1.0 / math.sqrt(128), store_bits=b,
                                   k_res=k_res, v_res=v_res, variant=2, **kw)
        _assert_attn_close(out.float().cpu().numpy(), ref, strict=False)
    from veloxquant_mlx_b200 import _lib
    _lib.check(_lib.lib().vq_kivi_attend_status(), "status")


@pytest.mark.parametrize("n_res", [1, 3, 4, 17, 33, 255])
@pytest.mark.parametrize("dt", ["float16", "bfloat16", "float32"])
def test_mma_attend_tail_kernel_edges(n_res, dt):
    """The unquantized tail is spread over the warps of a unit's CTAs (row r goes to warp
    r mod 4*splits): tail lengths below, at and far above the warp count, all three residual
    dtypes, 8 query heads per KV head. (The max-abs bound is asked of float16 outputs only: a
    bfloat16 output of magnitude 0.5..1 is itself rounded by up to 2^-9.)"""
    rng = np.random.default_rng(1000 + n_res)
    (qt, kc, ks, kz, vc, vs, vz, k_res, v_res), ref = _packed_case(rng, 2, 16, 2, 96, n_res, 4, dt)
    out = _k().kivi_decode_attend(qt, kc, ks, kz, vc, vs, vz, 32, 1.0 / math.sqrt(128), store_bits=4,
                                  k_res=k_res, v_res=v_res, variant=2)
    _assert_attn_close(out.float().cpu().numpy(), ref, strict=(dt != "bfloat16"))
    from veloxquant_mlx_b200 import _lib
    _lib.check(_lib.lib().vq_kivi_attend_status(), "status")


def test_back_to_back_calls_with_different_inputs_do_not_interfere():
    """Calls on different caches issued back to back without synchronisation (their scratch
    buffers are handed from one call to the next by the allocator) must each return what the same
    call returns in isolation, bit for bit."""
    k = _k()
    cases = [_packed_case(np.random.default_rng(300 + i), 2, 8, 2, 1024 + 32 * i, 40 + 9 * i, 4, "float16")[0] for i in range(4)]

    def call(a):
        qt, kc, ks, kz, vc, vs, vz, k_res, v_res = a
        return k.kivi_decode_attend(qt, kc, ks, kz, vc, vs, vz, 32, 1.0 / math.sqrt(128), store_bits=4,
                                    k_res=k_res, v_res=v_res, variant=2)

    alone = []
    for a in cases:
        o = call(a)
        torch.cuda.synchronize()
        alone.append(o.clone())
    for _ in range(20):
        outs = [call(a) for a in cases]
    torch.cuda.synchronize()
    for o, r in zip(outs, alone):
        assert torch.equal(o, r)
    from veloxquant_mlx_b200 import _lib
    _lib.check(_lib.lib().vq_kivi_attend_status(), "status")


def test_mma_attend_replayed_from_a_cuda_graph():
    """Captured into a CUDA graph and replayed several times back to back (every replay finds the
    tickets of the previous one and carries the same ticket epoch), the output must be that of
    the plain call, bit for bit, also after the query changed in place."""
    rng = np.random.default_rng(77)
    (qt, kc, ks, kz, vc, vs, vz, k_res, v_res), ref = _packed_case(rng, 2, 8, 2, 2048, 100, 4, "float16")
    k = _k()
    out = torch.empty_like(qt)
    call = lambda: k.kivi_decode_attend(qt, kc, ks, kz, vc, vs, vz, 32, 1.0 / math.sqrt(128), store_bits=4,
                                        k_res=k_res, v_res=v_res, variant=2, out=out)
    call()
    eager = out.clone()
    _assert_attn_close(eager.float().cpu().numpy(), ref)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        call()
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        call()
    out.zero_()
    for _ in range(5):
        g.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    qt.mul_(-0.5)  # same buffers, new contents
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    replayed = out.clone()
    call()
    assert torch.equal(replayed, out)
    from veloxquant_mlx_b200 import _lib
    _lib.check(_lib.lib().vq_kivi_attend_status(), "status")


@pytest.mark.parametrize("b", [2, 4])
@pytest.mark.parametrize("dt", ["float16", "bfloat16"])
def test_mma_attend_config1_with_outlier_channels(b, dt):
    """benchmark config 1 shape: B=1, 8 kv heads, 32 q heads, S=4096, residual 128, outliers x20."""
    rng = np.random.default_rng(0)
    args, ref = _packed_case(rng, 1, 32, 8, 4096 - 128, 128, b, dt, outliers=True)
    qt, kc, ks, kz, vc, vs, vz, k_res, v_res = args
    out = _k().kivi_decode_attend(qt, kc, ks, kz, vc, vs, vz, 32, 1.0 / math.sqrt(128), store_bits=b,
                                  k_res=k_res, v_res=v_res, variant=2)
    assert out.dtype == qt.dtype
    _assert_attn_close(out.float().cpu().numpy(), ref, strict=False)


def test_mma_attend_in_capacity_buffers():
    """Codes live in larger pre-allocated buffers; only the first n_quant rows are attended."""
    rng = np.random.default_rng(3)
    k = _k()
    B, H, H_kv, D, g, b, cap, n_quant, n_res = 2, 8, 2, 128, 32, 4, 512, 320, 40
    (qt, kc, ks, kz, vc, vs, vz, k_res, v_res), ref = _packed_case(rng, B, H, H_kv, n_quant, n_res, b, "float16")
    def grow(t, n):
        out = torch.zeros(t.shape[0], t.shape[1], n, t.shape[3], dtype=t.dtype, device=t.device)
        out[:, :, :t.shape[2]] = t
        return out
    KC, VC, VS, VZ = grow(kc, cap), grow(vc, cap), grow(vs, cap), grow(vz, cap)
    KS, KZ = grow(ks, cap // g), grow(kz, cap // g)
    KR, VR = grow(k_res, 160), grow(v_res, 160)
    for variant in (1, 2):
        out = k.kivi_decode_attend(qt, KC, KS, KZ, VC, VS, VZ, g, 1.0 / math.sqrt(D), store_bits=b,
                                   n_quant=n_quant, k_res=KR, v_res=VR, n_res=n_res, variant=variant)
        _assert_attn_close(out.float().cpu().numpy(), ref)


def test_mma_variant_rejects_unsupported_shapes():
    k = _k()
    ins = _to_dev(*o_kivi.make_inputs(1, 4, 64, 64, 2, 32))
    with pytest.raises(ValueError, match="tensor-core kernel unavailable"):
        k.kivi_decode_attend(*ins, 32, 0.1, store_bits=8, variant=2)
