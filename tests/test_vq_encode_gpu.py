"""One-launch VecInfer quantize-on-append (smooth -> WHT -> nearest centroid -> gather -> inverse
WHT -> smooth), the layer-batched KIVI attend and the split-partial merge, against the oracle.
Indices and the float16 round trip are bit-exact: the kernel keeps the oracle's operation order."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import kivi as o_kivi
from oracle import vq as o_vq

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
_DT = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}


def _inputs(seed, B, Hn, S, D, sub_dim, n_c, dt):
    rng = np.random.default_rng(seed)
    x = torch.from_numpy(rng.standard_normal((B, Hn, S, D)).astype(np.float32)).to(_DT[dt])
    cb = rng.standard_normal((n_c, sub_dim)).astype(np.float32)
    return x, cb, rng


@pytest.mark.parametrize("dt", ["float16", "bfloat16", "float32"])
@pytest.mark.parametrize("shape", [(1, 2, 37, 128, 8, 256), (2, 3, 9, 64, 4, 16), (1, 1, 8, 32, 2, 5),
                                   (1, 4, 5, 256, 16, 64)])
@pytest.mark.parametrize("smooth_rows", [None, 1, "H", "2H"])
def test_encode_decode_keys_matches_oracle(dt, shape, smooth_rows):
    from veloxquant_mlx_b200 import vecinfer as vi

    B, Hn, S, D, sub_dim, n_c = shape
    x, cb, rng = _inputs(sum(shape) + len(dt), B, Hn, S, D, sub_dim, n_c, dt)
    H = o_vq.walsh_hadamard_matrix(D)
    smooth = None
    if smooth_rows is not None:
        rows = {1: 1, "H": Hn, "2H": 2 * Hn}[smooth_rows]
        smooth = (np.abs(rng.standard_normal((rows, D))) + 0.25).astype(np.float32)
        smooth[0, 3] = 0.0  # factors <= 1e-8 leave the element undivided
        if rows == 1 and D >= 64:
            smooth = smooth[0]  # the 1-D form
    want_hat, want_idx = o_vq.encode_decode_keys(x.float().numpy(), cb, sub_dim, H, smooth)
    hat, idx = vi.vecinfer_encode_decode_metal(
        x.to(DEV), torch.from_numpy(cb).to(DEV), sub_dim, torch.from_numpy(H).to(DEV),
        None if smooth is None else torch.from_numpy(smooth).to(DEV))
    assert hat.dtype == torch.float16 and idx.dtype == torch.int32
    np.testing.assert_array_equal(idx.cpu().numpy(), want_idx)
    np.testing.assert_array_equal(hat.cpu().numpy().view(np.uint16), want_hat.view(np.uint16))
    only_idx = vi.vecinfer_encode_keys(x.to(DEV), torch.from_numpy(cb).to(DEV), sub_dim, torch.from_numpy(H).to(DEV),
                                       None if smooth is None else torch.from_numpy(smooth).to(DEV),
                                       index_dtype=torch.uint8 if n_c <= 256 else torch.int32)
    np.testing.assert_array_equal(only_idx.cpu().numpy().astype(np.int32), want_idx)


@pytest.mark.parametrize("dt", ["float16", "float32"])
def test_encode_decode_values_matches_oracle_and_flat_search(dt):
    from veloxquant_mlx_b200 import vecinfer as vi

    x, cb, _ = _inputs(5, 2, 2, 19, 128, 8, 256, dt)
    want_hat, want_idx = o_vq.encode_decode_values(x.float().numpy(), cb, 8)
    hat, idx = vi.vecinfer_encode_decode_simple_metal(x.to(DEV), torch.from_numpy(cb).to(DEV), 8)
    assert idx.dtype == torch.uint32 and hat.dtype == torch.float16
    np.testing.assert_array_equal(idx.cpu().numpy(), want_idx)
    np.testing.assert_array_equal(hat.cpu().numpy().view(np.uint16), want_hat.view(np.uint16))
    flat = vi.vecinfer_quantize_metal(x.to(DEV), torch.from_numpy(cb).to(DEV), 8)
    np.testing.assert_array_equal(flat.cpu().numpy(), want_idx.astype(np.int32))
    back = vi.vecinfer_dequant_metal(flat, torch.from_numpy(cb).to(DEV), out_dtype=torch.float16)
    np.testing.assert_array_equal(back.cpu().numpy().view(np.uint16), want_hat.view(np.uint16))


def test_stacked_codebooks_and_empty_input():
    from veloxquant_mlx_b200 import vecinfer as vi

    rng = np.random.default_rng(11)
    x = torch.from_numpy(rng.standard_normal((1, 2, 6, 32)).astype(np.float32))
    cbs = rng.standard_normal((8, 16, 4)).astype(np.float32)  # one codebook per sub-space
    hat, idx = vi._encode_decode("t", x.to(DEV), torch.from_numpy(cbs).to(DEV), 4, None, None, False, torch.int32)
    want = o_vq.quantize_vq(x.numpy(), cbs, 4)
    np.testing.assert_array_equal(idx.cpu().numpy(), want)
    np.testing.assert_array_equal(hat.float().cpu().numpy(), o_vq.dequantize_vq(want, cbs).astype(np.float16).astype(np.float32))
    e_hat, e_idx = vi.vecinfer_encode_decode_simple_metal(torch.zeros(1, 2, 0, 32, device=DEV), torch.from_numpy(cbs[0]).to(DEV), 4)
    assert e_hat.shape == (1, 2, 0, 32) and e_idx.shape == (1, 2, 0, 8)


def test_argument_errors():
    from veloxquant_mlx_b200 import vecinfer as vi

    cb = torch.zeros(4, 8, device=DEV)
    H = torch.eye(128, device=DEV)
    with pytest.raises(ValueError, match="keys must be 4D"):
        vi.vecinfer_encode_decode_metal(torch.zeros(2, 3, 128, device=DEV), cb, 8, H)
    with pytest.raises(ValueError, match="not divisible by sub_dim"):
        vi.vecinfer_encode_decode_metal(torch.zeros(1, 1, 2, 100, device=DEV), cb, 8, H)
    with pytest.raises(ValueError, match="> 512"):
        vi.vecinfer_encode_decode_simple_metal(torch.zeros(1, 1, 2, 1024, device=DEV), cb, 8)
    with pytest.raises(ValueError, match="codebook must be non-empty"):
        vi.vecinfer_encode_decode_simple_metal(torch.zeros(1, 1, 2, 128, device=DEV), torch.zeros(4, 4, device=DEV), 8)


@pytest.mark.parametrize("bits,store_bits", [(2, 2), (4, 4), (4, 8)])
def test_layer_batched_attend_equals_per_layer(bits, store_bits):
    from veloxquant_mlx_b200 import kernels as k

    NL, B, H_kv, H_q, S, D, g = 3, 2, 2, 8, 160, 128, 32
    rng = np.random.default_rng(bits + store_bits)
    q = torch.from_numpy(rng.standard_normal((NL, B, H_q, 1, D)).astype(np.float32)).half().to(DEV)
    packs = []
    for layer in range(NL):
        kk = torch.from_numpy(rng.standard_normal((B, H_kv, S, D)).astype(np.float32)).half().to(DEV)
        vv = torch.from_numpy(rng.standard_normal((B, H_kv, S, D)).astype(np.float32)).half().to(DEV)
        if store_bits == 8:
            kc, ks, kz = k.kivi_quantize(kk, -2, g, bits, store_bits=8)
            vc, vs, vz = k.kivi_quantize(vv, -1, g, bits, store_bits=8)
        else:
            kc, ks, kz = k.kivi_quantize(kk, -2, g, bits)
            vc, vs, vz = k.kivi_quantize(vv, -1, g, bits)
        packs.append((kc, ks, kz, vc, vs, vz))
    stacked = [torch.stack([p[i] for p in packs]) for i in range(6)]
    scale = 1.0 / np.sqrt(D)
    got = k.scalar_fused_decode_attend_batched(q, *stacked, g, scale, store_bits=store_bits)
    assert got.shape == (NL, B, H_q, 1, D) and got.dtype == torch.float16
    for layer in range(NL):
        one = k.scalar_fused_decode_attend(q[layer], *packs[layer], g, scale, store_bits=store_bits)
        assert torch.equal(got[layer], one)  # the folded call uses one layer's split count: bit-identical
        kc, ks, kz, vc, vs, vz = (t.cpu().numpy() for t in packs[layer])
        from oracle import bitpack as o_bp
        ref = o_kivi.reference_attend(q[layer].float().cpu().numpy(), o_bp.unpack(kc, store_bits, D), ks, kz,
                                      o_bp.unpack(vc, store_bits, D), vs, vz, g, scale)
        err = np.abs(got[layer].float().cpu().numpy() - ref)
        assert (err <= 2e-3 + 1e-2 * np.abs(ref)).all()
    with pytest.raises(ValueError, match="q must be 5D"):
        k.scalar_fused_decode_attend_batched(q[0], *stacked, g, scale)
    with pytest.raises(ValueError, match="NL mismatch"):
        k.scalar_fused_decode_attend_batched(q[:2], *stacked, g, scale)


def test_lse_merge_combines_two_halves_of_a_context():
    from veloxquant_mlx_b200 import kernels as k

    rng = np.random.default_rng(3)
    rows, n_splits, D = 5, 4, 96
    scores = rng.standard_normal((rows, n_splits, 40)).astype(np.float32) * 3
    vals = rng.standard_normal((rows, n_splits, 40, D)).astype(np.float32)
    scores[2, 1] = -np.inf  # a split that saw no slot
    m = scores.max(-1)
    with np.errstate(invalid="ignore"):
        p = np.where(np.isinf(m)[..., None], 0.0, np.exp(scores - m[..., None])).astype(np.float32)
    part_o = np.einsum("rsn,rsnd->rsd", p, vals).astype(np.float32)
    part_ml = np.stack([m, p.sum(-1)], -1).astype(np.float32)
    flat_s = scores.reshape(rows, -1)
    w = np.exp(flat_s - flat_s.max(-1, keepdims=True))
    want = (w / w.sum(-1, keepdims=True))[:, None, :] @ vals.reshape(rows, -1, D)
    got = k.lse_merge(torch.from_numpy(part_o).to(DEV), torch.from_numpy(part_ml).to(DEV), out_dtype=torch.float32)
    np.testing.assert_allclose(got.cpu().numpy(), want[:, 0], rtol=2e-5, atol=2e-6)
    with pytest.raises(ValueError, match="part_o"):
        k.lse_merge(torch.zeros(2, 3, device=DEV), torch.zeros(2, 3, 2, device=DEV))
