"""Each nearest-centroid search pinned through ``vq_tune(VQ_KNOB_VQ_SEARCH, ...)`` -- tcgen05 +
tensor memory, warp-level MMAs, exact CUDA-core search -- must return exactly the indices of
the reference evaluation order (``oracle.vq.quantize_vq``) on the same inputs."""

from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

_MODES = {"tc5": 1, "mma": 2, "exact": 3, "tc5_two_pass": 4}


@pytest.fixture
def pinned_search():
    from veloxquant_mlx_b200 import kernels as k

    def pin(mode):
        k.tune("vq_search", _MODES[mode])

    yield pin
    k.tune("vq_search", 0)


def _check(x32, cb, tag, dt):
    from oracle import vq as o_vq
    from veloxquant_mlx_b200 import kernels as k
    from veloxquant_mlx_b200 import vecinfer as vi

    x = torch.from_numpy(x32).to(dt)
    tag = f"{tag} [{dt}]"
    got = vi.quantize_vq(x.cuda(), torch.from_numpy(cb).cuda(), 8,
                         index_dtype=torch.uint8 if cb.shape[-2] <= 256 else torch.int32)
    k.quantize_status()
    want = o_vq.quantize_vq(x.float().numpy(), cb, 8)
    bad = int((got.cpu().numpy().astype(np.int32) != want).sum())
    assert bad == 0, f"{tag}: {bad} of {want.size} indices differ"


@pytest.mark.parametrize("mode", ["tc5", "mma", "exact", "tc5_two_pass"])
def test_pinned_search_matches_the_reference_order(mode, pinned_search):
    pinned_search(mode)
    rng = np.random.default_rng(0)
    for dt in (torch.float16, torch.bfloat16):
        for n_rows, n_c in ((1000, 256), (5000, 256), (4096, 64), (777, 16), (3000, 144), (70000, 256)):
            x = rng.standard_normal((n_rows, 8)).astype(np.float32)
            x[:, 3] *= 20.0
            _check(x, rng.standard_normal((n_c, 8)).astype(np.float32), f"random {n_rows}x{n_c}", dt)
        # exact ties on an integer lattice, duplicated centroids, 1-ulp near-ties
        x = rng.integers(-2, 3, (4096, 8)).astype(np.float32)
        cb = rng.integers(-2, 3, (64, 8)).astype(np.float32)
        cb[40] = cb[7]
        cb[41] = cb[7]
        _check(x, cb, "lattice", dt)
        cb2 = rng.standard_normal((128, 8)).astype(np.float32)
        cb2[64:] = cb2[:64]
        cb2[64:, 0] = np.nextafter(cb2[:64, 0], np.float32(np.inf))
        x2 = (cb2[rng.integers(0, 128, 4096)] + 1e-3 * rng.standard_normal((4096, 8))).astype(np.float32)
        _check(x2, cb2, "near-ties", dt)
        # 256 centroids (the single-pass epilogue's 8 x 16 grid per half row): duplicates that share a
        # grid column, a grid row, or sit in the two halves; then 1-ulp near-ties of every centroid
        cb3 = rng.integers(-3, 4, (256, 8)).astype(np.float32)
        cb3[23] = cb3[7]          # same grid column (7 and 7 + 16)
        cb3[41] = cb3[40]         # same grid row
        cb3[130] = cb3[2]         # lower and upper half
        cb3[255] = cb3[128]
        x3 = rng.integers(-3, 4, (8192, 8)).astype(np.float32)
        x3[:256] = cb3            # every centroid is hit exactly
        _check(x3, cb3, "lattice 256", dt)
        cb4 = rng.standard_normal((256, 8)).astype(np.float32)
        cb4[128:] = cb4[:128]
        cb4[128:, 0] = np.nextafter(cb4[:128, 0], np.float32(np.inf))
        cb4[64:128] = cb4[:64]
        cb4[64:128, 1] = np.nextafter(cb4[:64, 1], np.float32(-np.inf))
        x4 = (cb4[rng.integers(0, 256, 8192)] + 1e-3 * rng.standard_normal((8192, 8))).astype(np.float32)
        _check(x4, cb4, "near-ties 256", dt)
        # rows and codebooks outside the half-precision window fall back to the reference order
        xb = rng.standard_normal((2048, 8)).astype(np.float32)
        xb[5] *= 3e4
        xb[70, 2] = np.inf
        xb[71, 0] = np.nan
        xb[900] = 0
        cbr = rng.standard_normal((256, 8)).astype(np.float32)
        _check(xb, cbr, "bad rows", dt)
        _check(xb, cbr * 100, "large codebook", dt)
        _check(xb, np.zeros((16, 8), np.float32), "zero codebook", dt)
        # one codebook per sub-space (the second benchmark configuration's wording): 16 sub-spaces of dim 8
        xs = rng.standard_normal((2, 300, 128)).astype(np.float32)
        cbs = rng.standard_normal((16, 256, 8)).astype(np.float32)
        cbs[5, 100] = cbs[5, 3]
        _check(xs, cbs, "per-sub-space codebooks", dt)


@pytest.mark.parametrize("mode", ["tc5", "mma", "exact", "tc5_two_pass"])
def test_every_search_matches_the_reference_function_golden_vectors(mode, pinned_search):
    """Indices equal those of the reference's ``quantize_vq`` (``allocators/vecinfer.py:281-318``)
    executed over NumPy (tests/golden/vq.npz), bit for bit, at sub-vector sizes 2, 4 and 8, with a
    duplicated centroid and an exact hit; the gather restores the reference's reconstruction."""
    import os

    from veloxquant_mlx_b200 import kernels as k
    from veloxquant_mlx_b200 import vecinfer as vi

    pinned_search(mode)
    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "vq.npz"))
    for tag, sub in (("s2", 2), ("s4", 4), ("s4big", 4), ("s8", 8)):
        x, cb, idx = z[f"q_{tag}_x"], z[f"q_{tag}_cb"], z[f"q_{tag}_idx"]
        got = vi.quantize_vq(torch.from_numpy(x).cuda(), torch.from_numpy(cb).cuda(), sub)
        k.quantize_status()
        np.testing.assert_array_equal(got.cpu().numpy(), idx, err_msg=f"{tag} [{mode}]")
        deq = vi.dequantize_vq(got, torch.from_numpy(cb).cuda())
        np.testing.assert_array_equal(deq.cpu().numpy(), z[f"q_{tag}_deq"])
