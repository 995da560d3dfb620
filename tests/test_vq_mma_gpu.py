"""The tensor-core nearest-centroid search must return exactly the indices of the reference
evaluation order: random data, float32 codebooks that halves cannot represent, exact ties on
an integer lattice, duplicated centroids, near-ties one ulp apart, rows and codebooks outside
the half-precision range, non-finite rows, ragged sizes. Inputs have >= 1024 sub-vectors so
that vq_vq_quantize picks the tensor-core kernel (smaller calls run the CUDA-core search)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import vq as o_vq

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
_DT = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}


def _check(x32, cb32, sub_dim, dt="float32", index_dtype=torch.int32):
    from veloxquant_mlx_b200 import vecinfer as vi

    t = torch.from_numpy(np.ascontiguousarray(x32)).to(_DT[dt])
    want = o_vq.quantize_vq(t.float().numpy(), cb32, sub_dim)
    got = vi.quantize_vq(t.to(DEV), torch.from_numpy(cb32).to(DEV), sub_dim, index_dtype=index_dtype)
    got = got.cpu().numpy().astype(np.int64)
    bad = np.argwhere(got != want)
    assert bad.size == 0, f"{len(bad)} of {want.size} indices differ, first at {bad[0]}: {got[tuple(bad[0])]} vs {want[tuple(bad[0])]}"


@pytest.mark.parametrize("dt", ["float16", "bfloat16", "float32"])
@pytest.mark.parametrize("sub_dim,n_c", [(8, 256), (8, 100), (8, 2), (4, 256), (4, 37), (8, 1024)])
def test_random_float32_codebooks(dt, sub_dim, n_c):
    rng = np.random.default_rng(n_c + sub_dim)
    x = rng.standard_normal((4111, 2 * sub_dim)).astype(np.float32)  # ragged: not a multiple of 64 rows
    x[:, 3] *= 20.0
    cb = rng.standard_normal((n_c, sub_dim)).astype(np.float32)
    _check(x, cb, sub_dim, dt)
    if n_c <= 256:
        _check(x[:1500], cb, sub_dim, dt, torch.uint8)


@pytest.mark.parametrize("sub_dim", [4, 8])
def test_exact_ties_duplicates_and_near_ties(sub_dim):
    rng = np.random.default_rng(sub_dim)
    # integer lattice: many sub-vectors are equidistant from several centroids -> lowest index
    x = rng.integers(-2, 3, (2048, sub_dim)).astype(np.float32)
    cb = rng.integers(-2, 3, (64, sub_dim)).astype(np.float32)
    cb[40] = cb[7]   # duplicates
    cb[41] = cb[7]
    _check(x, cb, sub_dim, "float16")
    _check(x, cb, sub_dim, "float32")
    # near-ties: centroid pairs that differ by one float32 ulp in one coordinate
    cb2 = rng.standard_normal((128, sub_dim)).astype(np.float32)
    cb2[64:] = cb2[:64]
    cb2[64:, 0] = np.nextafter(cb2[:64, 0], np.float32(np.inf))
    x2 = (cb2[rng.integers(0, 128, 4096)] + 1e-3 * rng.standard_normal((4096, sub_dim))).astype(np.float32)
    _check(x2, cb2, sub_dim, "float32")
    _check(x2, cb2, sub_dim, "bfloat16")
    # sub-vectors exactly on a centroid, and midpoints of centroid pairs
    mid = (0.5 * (cb2[:64] + cb2[rng.permutation(64)])).astype(np.float32)
    _check(np.concatenate([cb2, mid, x2[:1024]]), cb2, sub_dim, "float32")


def test_out_of_range_rows_and_codebooks():
    rng = np.random.default_rng(9)
    x = rng.standard_normal((2048, 8)).astype(np.float32)
    cb = rng.standard_normal((256, 8)).astype(np.float32)
    xb = x.copy()
    xb[5] *= 1e6          # beyond half range: that row is searched in float32
    xb[70, 2] = np.inf
    xb[71, 0] = np.nan    # NaN distances never win: index 0
    xb[900] = 0.0
    _check(xb, cb, 8, "float32")
    _check(x, np.zeros((16, 8), np.float32), 8)          # all-zero codebook: every row ties
    _check(x * 1e-3, cb * 1e-3, 8)                       # codebook below the half-precision window
    _check(x * 1e4, cb * 1e4, 8)                         # and above it
    cbn = cb.copy()
    cbn[3, 1] = np.nan
    cbn[9, 0] = np.inf
    _check(x, cbn, 8)
    _check(x.astype(np.float32) * 3e4, cb, 8, "float16")  # large but representable halves


@pytest.mark.parametrize("dt", ["float16", "float32"])
@pytest.mark.parametrize("sub_dim", [4, 8])
def test_one_codebook_per_sub_space(dt, sub_dim):
    rng = np.random.default_rng(17 + sub_dim)
    D = 64
    x = rng.standard_normal((2, 3, 211, D)).astype(np.float32)
    cbs = rng.standard_normal((D // sub_dim, 200, sub_dim)).astype(np.float32)
    cbs[3, 50] = cbs[3, 20]  # a duplicate inside one sub-space
    _check(x, cbs, sub_dim, dt)
    _check(x, cbs, sub_dim, dt, torch.uint8)


def test_cache_sized_call_matches_small_calls():
    from veloxquant_mlx_b200 import vecinfer as vi

    rng = np.random.default_rng(1)
    keys = torch.from_numpy(rng.standard_normal((8, 1024, 128)).astype(np.float32)).half().to(DEV)
    cb = torch.from_numpy(rng.standard_normal((256, 8)).astype(np.float32)).to(DEV)
    big = vi.quantize_vq(keys, cb, 8, index_dtype=torch.uint8)
    # 32-token slices have 512 sub-vectors each: below the tensor-core threshold
    small = torch.cat([vi.quantize_vq(keys[:, i : i + 32].contiguous(), cb, 8, index_dtype=torch.uint8)
                       for i in range(0, 1024, 32)], dim=1)
    assert torch.equal(big, small)
