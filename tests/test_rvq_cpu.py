"""TurboQuant-RVQ host pieces: the Lloyd-Max codebooks against fixtures computed by the
reference's own ``math/lloyd_max.py`` (``tests/golden/rvq.npz``), the packing layout, and the
oracle's quantize / decode round trip."""

from __future__ import annotations

import os

import numpy as np
import pytest
import torch

from oracle import rvq as o_rvq

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "rvq.npz"))


@pytest.mark.parametrize("b", [1, 2, 3, 4])
def test_codebooks_match_the_reference_lloyd_max(b):
    from veloxquant_mlx_b200 import rvq

    for d in (64, 128, 256):
        cb = rvq.gaussian_codebook(b, d)
        ref = GOLD[f"gauss_b{b}_d{d}"]
        np.testing.assert_allclose(cb.centroids32, ref.astype(np.float32), rtol=0, atol=1e-9)
        np.testing.assert_array_equal(cb.centroids, ref.astype(np.float32).astype(np.float16))
        ref32 = np.sort(ref.astype(np.float32))
        np.testing.assert_array_equal(cb.boundaries, ((ref32[:-1] + ref32[1:]) / np.float32(2)).astype(np.float16))
        scale = float(GOLD[f"scale_b{b}_d{d}"])
        q = rvq.TurboQuantRVQ(d, b, use_hadamard=True)
        assert q._residual_scale == scale
        np.testing.assert_array_equal(q._codebook2.centroids, GOLD[f"laplace_b{b}_d{d}"].astype(np.float32).astype(np.float16))
    for d in (8, 16, 32):
        np.testing.assert_array_equal(rvq.beta_codebook(b, d).centroids, GOLD[f"beta_b{b}_d{d}"].astype(np.float32).astype(np.float16))


def test_lloyd_max_rejects_bad_arguments():
    from veloxquant_mlx_b200 import rvq

    with pytest.raises(ValueError):
        rvq.lloyd_max(lambda x: np.ones_like(x), (1.0, 0.0), 4)
    with pytest.raises(ValueError):
        rvq.lloyd_max(lambda x: np.ones_like(x), (0.0, 1.0), 0)
    c, b = rvq.lloyd_max(lambda x: np.ones_like(x), (0.0, 1.0), 4)   # uniform density: equal cells
    np.testing.assert_allclose(c, [0.125, 0.375, 0.625, 0.875], atol=1e-6)
    assert b[0] == -np.inf and b[-1] == np.inf


@pytest.mark.parametrize("bits", [1, 2, 3, 4])
@pytest.mark.parametrize("d", [8, 13, 32, 100, 128])
def test_pack_layout_and_round_trip(bits, d):
    from veloxquant_mlx_b200 import rvq

    rng = np.random.default_rng(bits * 100 + d)
    idx = rng.integers(0, 1 << bits, (5, d)).astype(np.uint8)
    packed = o_rvq.pack_indices(idx, bits)
    assert packed.dtype == np.uint32 and packed.shape == (5, rvq.n_words_for(d, bits))
    np.testing.assert_array_equal(o_rvq.unpack_indices(packed, bits, d), idx)
    t = rvq.pack_indices(torch.from_numpy(idx), bits)
    np.testing.assert_array_equal(t.view(torch.int32).numpy().view(np.uint32), packed)
    np.testing.assert_array_equal(rvq.unpack_indices(t, bits, d).numpy(), idx)
    # element i of a word sits in bits [i*bits, (i+1)*bits)
    epw = 32 // bits
    for i in range(min(d, epw)):
        assert (int(packed[0, 0]) >> (i * bits)) & ((1 << bits) - 1) == idx[0, i]


def test_known_answer_two_bit_word():
    idx = np.array([[0, 1, 2, 3] * 4], dtype=np.uint8)
    assert o_rvq.pack_indices(idx, 2)[0, 0] == 0xE4E4E4E4


def test_oracle_quantize_counts_boundaries_and_rounds_the_residual():
    c1 = np.array([-1.0, -0.25, 0.25, 1.0], np.float16)
    b1 = np.array([-0.625, 0.0, 0.625], np.float16)
    b2 = np.array([-0.1, 0.0, 0.1], np.float16)
    y = np.array([[-2.0, -0.625, 0.0, 1e-3, 0.7, np.nan, 0.3, 0.35]], np.float16)
    idx1, idx2, p1, p2 = o_rvq.rvq_quant_pack(y, c1, b1, b2, 2)
    # a value equal to a boundary does not exceed it; NaN exceeds nothing
    assert idx1.tolist() == [[0, 0, 1, 2, 3, 0, 2, 2]]
    assert idx2[0, 7] == 3 and idx2[0, 6] == 2      # residuals 0.1 (just above fp16(0.1)) and 0.05
    np.testing.assert_array_equal(o_rvq.unpack_indices(p1, 2, 8), idx1)


def test_oracle_decode_inverts_the_rotation():
    from veloxquant_mlx_b200 import rvq
    from veloxquant_mlx_b200.rabitq import make_hadamard_diagonal

    d, bits = 128, 4
    rng = np.random.default_rng(0)
    x = rng.standard_normal((64, d)).astype(np.float32)
    x /= np.linalg.norm(x, axis=1, keepdims=True)
    diag = make_hadamard_diagonal(d, seed=3)
    y = (o_rvq.wht_butterfly(x * diag) / np.sqrt(np.float32(d))).astype(np.float16)
    c1, c2 = rvq.gaussian_codebook(bits, d), rvq.TurboQuantRVQ(d, bits, use_hadamard=True)._codebook2
    _, _, p1, p2 = o_rvq.rvq_quant_pack(y, c1.centroids, c1.boundaries, c2.boundaries, bits)
    rec = o_rvq.rvq_unpack_decode(p1, p2, np.ones(64, np.float32), c1.centroids, c2.centroids, diag, bits, d).astype(np.float32)
    cos = (rec * x).sum(1) / np.linalg.norm(rec, axis=1)
    assert cos.min() > 0.995


def test_packing_and_norm_helpers_match_the_reference_cache_functions_run_over_numpy():
    """``_pack_indices`` / ``_unpack_indices`` / ``_unit_fp16_from_fp16`` / ``_rescale_fp16`` of
    ``cache/turboquant_rvq_cache.py:65-126``, extracted and executed with NumPy answering ``mx``
    (tests/golden/rvq.npz): the oracle's and the package's packing reproduce the words bit for bit
    (1-4 bits, a ragged last word); the unit direction / norm split and the saturating rescale of the
    cache agree with theirs (norms to float32 rounding, unit vectors and rescaled rows to a float16 step)."""
    from veloxquant_mlx_b200 import rvq

    z = GOLD
    for bits in (1, 2, 3, 4):
        for d in (64, 128, 20):
            idx, words = z[f"pack_b{bits}_d{d}_idx"], z[f"pack_b{bits}_d{d}_words"]
            assert np.array_equal(o_rvq.pack_indices(idx, bits), words)
            assert np.array_equal(o_rvq.unpack_indices(words, bits, d), idx)
            got = rvq.pack_indices(torch.from_numpy(idx), bits)
            assert got.dtype == torch.uint32 and np.array_equal(got.view(torch.int32).numpy().view(np.uint32), words)
            assert np.array_equal(rvq.unpack_indices(got, bits, d).numpy(), idx)
    k = torch.from_numpy(z["cache_k"])
    k32 = k.float()
    norms = torch.linalg.vector_norm(k32, dim=-1, keepdim=True)          # what TurboQuantRVQKVCache.update_and_fetch computes
    unit = (k32 / norms.clamp_min(1e-4)).to(torch.float16)
    np.testing.assert_allclose(norms.numpy(), z["cache_norms"], rtol=2e-7)
    np.testing.assert_allclose(unit.float().numpy(), z["cache_unit"].astype(np.float32), rtol=2.0 ** -10, atol=2.0 ** -24)
    assert float((unit.numpy() == z["cache_unit"]).mean()) > 0.99
    assert float(z["cache_norms"].max()) > 65504.0                         # the case the float32 norm exists for
    resc = (torch.from_numpy(z["cache_unit"]).float() * torch.from_numpy(z["cache_norms"])).clamp(-65504.0, 65504.0).to(torch.float16)
    assert np.array_equal(resc.numpy(), z["cache_rescaled"])


def test_quantizer_tables_and_host_encode_match_the_reference_quantizer_run_over_numpy():
    """``rvq_reference.npz`` holds what the reference's ``TurboQuantRVQ`` built and returned when run
    over a NumPy stand-in: this package's quantizer builds the same tables, and its host-side
    two-stage encode maps the reference's rotated input to the reference's indices."""
    from veloxquant_mlx_b200 import rvq

    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "rvq_reference.npz"))
    for d, b in z["quantizer_cases"]:
        t = f"q_d{d}_b{b}_"
        q = rvq.TurboQuantRVQ(int(d), int(b), seed=3, use_hadamard=True)
        np.testing.assert_array_equal(q._codebook1.centroids, z[t + "c1"])
        np.testing.assert_array_equal(q._codebook1.boundaries, z[t + "b1"])
        np.testing.assert_array_equal(q._codebook2.centroids, z[t + "c2"])
        np.testing.assert_array_equal(q._codebook2.boundaries, z[t + "b2"])
        np.testing.assert_array_equal(q._diag_np, z[t + "diag"])
        y = torch.from_numpy(z[t + "rotated"])
        idx1 = q._codebook1.quantize(y)
        r1 = y - q._codebook1.dequantize(idx1).to(y.dtype)
        np.testing.assert_array_equal(idx1.numpy(), z[t + "idx1"])
        np.testing.assert_array_equal(q._codebook2.quantize(r1).numpy(), z[t + "idx2"])
        # the rotation itself (matrix form on the host) agrees to float16 rounding
        rot = q.rotate(torch.from_numpy(z[t + "x"])).float().numpy()
        np.testing.assert_allclose(rot, z[t + "rotated"].astype(np.float32), atol=2.0 ** -10, rtol=0)
