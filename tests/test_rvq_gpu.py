"""TurboQuant-RVQ kernels on the GPU against the oracle: quantize+pack bit for bit (the
reference's bar, ``veloxquant_mlx/tests/metal/test_rvq_quant_pack.py:50-66``), unpack+decode bit
for bit against the restated Metal arithmetic (``tests/metal/test_rvq_unpack_decode.py``)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import rvq as o_rvq

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _u32(t):
    return t.cpu().view(torch.int32).numpy().view(np.uint32)


def _tables(d, bits):
    from veloxquant_mlx_b200 import rvq

    q = rvq.TurboQuantRVQ(d, bits, seed=d + bits, use_hadamard=True)
    return q, q._codebook1, q._codebook2


@pytest.mark.parametrize("D", [8, 16, 32, 64, 128, 256])
@pytest.mark.parametrize("bits", [1, 2, 3, 4])
@pytest.mark.parametrize("N", [1, 5, 33])
def test_quant_pack_bit_exact(D, bits, N):
    from veloxquant_mlx_b200 import rvq

    q, c1, c2 = _tables(D, bits)
    rng = np.random.default_rng(D * 100 + bits * 10 + N)
    y = (rng.standard_normal((N, D)) / np.sqrt(D)).astype(np.float16)
    p1, p2 = rvq.rvq_quant_pack(torch.from_numpy(y).to(DEV), c1.centroids, c1.boundaries, c2.boundaries, bits)
    _, _, r1, r2 = o_rvq.rvq_quant_pack(y, c1.centroids, c1.boundaries, c2.boundaries, bits)
    assert p1.dtype == torch.uint32 and tuple(p1.shape) == r1.shape
    np.testing.assert_array_equal(_u32(p1), r1)
    np.testing.assert_array_equal(_u32(p2), r2)


def test_quant_pack_large_edges_and_odd_width():
    from veloxquant_mlx_b200 import rvq

    for D, bits in ((128, 2), (128, 3), (100, 4), (1024, 1)):
        q, c1, c2 = _tables(128 if D == 100 else D, bits)
        rng = np.random.default_rng(D + bits)
        y = (rng.standard_normal((20001, D)) / np.sqrt(D)).astype(np.float16)
        # values exactly on boundaries, special values, huge values
        y[0, : (1 << bits) - 1] = c1.boundaries
        y[1, :4] = np.array([np.nan, np.inf, -np.inf, 0.0], np.float16)
        y[2] = 60000.0
        y[3, : 1 << bits] = c1.centroids
        p1, p2 = rvq.rvq_quant_pack(torch.from_numpy(y).to(DEV), c1.centroids, c1.boundaries, c2.boundaries, bits)
        _, _, r1, r2 = o_rvq.rvq_quant_pack(y, c1.centroids, c1.boundaries, c2.boundaries, bits)
        np.testing.assert_array_equal(_u32(p1), r1)
        np.testing.assert_array_equal(_u32(p2), r2)


@pytest.mark.parametrize("bits", [1, 2, 3, 4])
def test_code_table_covers_every_float16_pattern(bits):
    """The 65 536-entry table against the oracle on all bit patterns (NaNs, infinities, denormals
    included), and the table path against the comparing path on the same input."""
    from veloxquant_mlx_b200 import rvq

    q, c1, c2 = _tables(128, bits)
    table = rvq.rvq_code_table(c1.centroids, c1.boundaries, c2.boundaries, bits, DEV).cpu().numpy()
    y = np.arange(65536, dtype=np.uint16).view(np.float16).reshape(512, 128)
    with np.errstate(invalid="ignore", over="ignore"):
        idx1, idx2, _, _ = o_rvq.rvq_quant_pack(y, c1.centroids, c1.boundaries, c2.boundaries, bits)
    np.testing.assert_array_equal(table & 15, idx1.reshape(-1))
    np.testing.assert_array_equal(table >> 4, idx2.reshape(-1))
    x = torch.from_numpy(y).to(DEV).repeat(20, 1)
    a = rvq.rvq_quant_pack(x, c1.centroids, c1.boundaries, c2.boundaries, bits, use_table=True)
    b = rvq.rvq_quant_pack(x, c1.centroids, c1.boundaries, c2.boundaries, bits, use_table=False)
    assert torch.equal(a[0].view(torch.int32), b[0].view(torch.int32)) and torch.equal(a[1].view(torch.int32), b[1].view(torch.int32))


@pytest.mark.parametrize("D,bits", [(128, 2), (64, 1), (256, 4), (32, 3)])
def test_encode_pack_equals_packing_the_unfused_codes(D, bits):
    """``encode_pack`` against ``pack_indices(encode())``: the reference's parity test."""
    from veloxquant_mlx_b200 import rvq

    q = rvq.TurboQuantRVQ(D, bits, seed=1, use_hadamard=True)
    x = torch.randn(777, D, device=DEV, dtype=torch.float16)
    idx1, idx2 = q.encode(x)
    p1, p2 = q.encode_pack(x)
    assert torch.equal(p1.view(torch.int32), rvq.pack_indices(idx1, bits).view(torch.int32))
    assert torch.equal(p2.view(torch.int32), rvq.pack_indices(idx2, bits).view(torch.int32))


@pytest.mark.parametrize("D", [8, 32, 64, 128, 256, 1024])
@pytest.mark.parametrize("bits", [1, 2, 3, 4])
def test_unpack_decode_matches_the_restated_kernel(D, bits):
    from veloxquant_mlx_b200 import rvq
    from veloxquant_mlx_b200.rabitq import make_hadamard_diagonal

    c1 = rvq.gaussian_codebook(bits, max(D, 64))
    c2 = rvq.laplacian_codebook(bits, 0.05)
    rng = np.random.default_rng(D + bits)
    N = 301
    nw = rvq.n_words_for(D, bits)
    i1 = rng.integers(0, 1 << bits, (N, D)).astype(np.uint8)
    i2 = rng.integers(0, 1 << bits, (N, D)).astype(np.uint8)
    p1, p2 = o_rvq.pack_indices(i1, bits), o_rvq.pack_indices(i2, bits)
    assert p1.shape == (N, nw)
    norms = (rng.random(N) * 20 + 0.1).astype(np.float32)
    norms[0] = 1e6   # saturates
    diag = make_hadamard_diagonal(D, seed=5)
    want = o_rvq.rvq_unpack_decode(p1, p2, norms, c1.centroids, c2.centroids, diag, bits, D)
    tp1 = torch.from_numpy(p1.view(np.int32)).to(DEV).view(torch.uint32)
    tp2 = torch.from_numpy(p2.view(np.int32)).to(DEV).view(torch.uint32)
    got = rvq.rvq_unpack_decode(tp1, tp2, torch.from_numpy(norms).to(DEV), c1.centroids, c2.centroids, diag, bits, D)
    assert got.dtype == torch.float16 and tuple(got.shape) == (N, D)
    np.testing.assert_array_equal(got.cpu().numpy(), want)
    assert np.abs(want[0]).max() == 65504.0
    # bf16 norms, and the streams read in place from an over-allocated [BH, cap, n_words] buffer
    BH, cap, seq = 7, 43, 29
    b1 = torch.from_numpy(p1.view(np.int32)).to(DEV).view(torch.uint32).reshape(BH, cap, nw)
    b2 = torch.from_numpy(p2.view(np.int32)).to(DEV).view(torch.uint32).reshape(BH, cap, nw)
    nb = torch.from_numpy(norms).to(DEV).to(torch.bfloat16).reshape(BH, cap, 1)
    got3 = rvq.rvq_unpack_decode(b1, b2, nb, c1.centroids, c2.centroids, diag, bits, D, seq_len=seq)
    rows = (np.arange(BH)[:, None] * cap + np.arange(seq)[None, :]).reshape(-1)
    want3 = o_rvq.rvq_unpack_decode(p1[rows], p2[rows], nb.float().cpu().numpy().reshape(-1)[rows], c1.centroids, c2.centroids, diag, bits, D)
    np.testing.assert_array_equal(got3.cpu().numpy(), want3)


def test_round_trip_quality_and_fused_decode():
    from veloxquant_mlx_b200 import rvq

    D = 128
    x = torch.randn(4096, D, device=DEV, dtype=torch.float32)
    norms = x.norm(dim=1)
    xu = (x / norms[:, None]).to(torch.float16)
    floors = {1: 0.90, 2: 0.97, 3: 0.99, 4: 0.995}
    for bits, floor in floors.items():
        q = rvq.TurboQuantRVQ(D, bits, seed=0, use_hadamard=True)
        assert q.supports_fused_decode
        p1, p2 = q.encode_pack(xu)
        rec = q.decode_packed(p1, p2, norms).float()
        cos = torch.nn.functional.cosine_similarity(rec, x, dim=1)
        assert float(cos.mean()) > floor, (bits, float(cos.mean()))
        # the unfused decode agrees with the fused one up to the float16 roundings on the way
        idx1, idx2 = q.encode(xu)
        rec2 = q.decode(idx1, idx2).float() * norms[:, None]
        assert float((rec2 - rec).abs().max()) < 2e-2 * float(norms.max())


def test_wrappers_reject_bad_arguments():
    from veloxquant_mlx_b200 import rvq

    q, c1, c2 = _tables(128, 2)
    y = torch.zeros(4, 128, dtype=torch.float16, device=DEV)
    with pytest.raises(ValueError, match="2D"):
        rvq.rvq_quant_pack(y[0], c1.centroids, c1.boundaries, c2.boundaries, 2)
    with pytest.raises(ValueError, match="bits"):
        rvq.rvq_quant_pack(y, c1.centroids, c1.boundaries, c2.boundaries, 5)
    with pytest.raises(ValueError, match="float16"):
        rvq.rvq_quant_pack(y.float(), c1.centroids, c1.boundaries, c2.boundaries, 2)
    with pytest.raises(ValueError, match="boundaries"):
        rvq.rvq_quant_pack(y, c1.centroids, c1.boundaries[:2], c2.boundaries, 2)
    p1, p2 = rvq.rvq_quant_pack(y, c1.centroids, c1.boundaries, c2.boundaries, 2)
    n = torch.ones(4, device=DEV)
    with pytest.raises(ValueError, match="power of two"):
        rvq.rvq_unpack_decode(p1, p2, n, c1.centroids, c2.centroids, q._diag_np, 2, 100)
    with pytest.raises(ValueError, match="seq_len requires"):
        rvq.rvq_unpack_decode(p1, p2, n, c1.centroids, c2.centroids, q._diag_np, 2, 128, seq_len=2)
    with pytest.raises(ValueError, match="words per row"):
        rvq.rvq_unpack_decode(p1[:, :4], p2[:, :4], n, c1.centroids, c2.centroids, q._diag_np, 2, 128)
    with pytest.raises(ValueError, match="norms"):
        rvq.rvq_unpack_decode(p1, p2, n[:3], c1.centroids, c2.centroids, q._diag_np, 2, 128)
    assert rvq.rvq_unpack_decode(p1[:0], p2[:0], n[:0], c1.centroids, c2.centroids, q._diag_np, 2, 128).shape == (0, 128)
