"""Each nearest-centroid search pinned with VQ_VQ_SEARCH -- tc5 (tcgen05 + tensor memory), mma
(warp-level MMAs), exact (CUDA cores) -- must return exactly the indices of the reference
evaluation order on the same inputs. The switch is read once per process, so each mode is
checked in a child process."""

from __future__ import annotations

import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_CHILD = r"""
import sys
import numpy as np, torch
sys.path.insert(0, %r)
from veloxquant_mlx_b200 import vecinfer as vi
from veloxquant_mlx_b200._lib import lib
from oracle import vq as o_vq
rng = np.random.default_rng(0)
DT = torch.float16
def check(x32, cb, tag):
    x = torch.from_numpy(x32).to(DT)
    tag = f"{tag} [{DT}]"
    got = vi.quantize_vq(x.cuda(), torch.from_numpy(cb).cuda(), 8, index_dtype=torch.uint8 if cb.shape[-2] <= 256 else torch.int32)
    assert lib().vq_vq_quantize_status() == 0, tag
    want = o_vq.quantize_vq(x.float().numpy(), cb, 8)
    bad = int((got.cpu().numpy().astype(np.int32) != want).sum())
    assert bad == 0, f"{tag}: {bad} of {want.size} indices differ"
for DT in (torch.float16, torch.bfloat16):
    for n_rows, n_c in ((1000, 256), (5000, 256), (4096, 64), (777, 16), (3000, 144), (70000, 256)):
        x = rng.standard_normal((n_rows, 8)).astype(np.float32); x[:, 3] *= 20.0
        check(x, rng.standard_normal((n_c, 8)).astype(np.float32), f"random {n_rows}x{n_c}")
    # exact ties on an integer lattice, duplicated centroids, 1-ulp near-ties
    x = rng.integers(-2, 3, (4096, 8)).astype(np.float32)
    cb = rng.integers(-2, 3, (64, 8)).astype(np.float32); cb[40] = cb[7]; cb[41] = cb[7]
    check(x, cb, "lattice")
    cb2 = rng.standard_normal((128, 8)).astype(np.float32); cb2[64:] = cb2[:64]
    cb2[64:, 0] = np.nextafter(cb2[:64, 0], np.float32(np.inf))
    x2 = (cb2[rng.integers(0, 128, 4096)] + 1e-3 * rng.standard_normal((4096, 8))).astype(np.float32)
    check(x2, cb2, "near-ties")
    # rows and codebooks outside the half-precision window fall back to the reference order
    xb = rng.standard_normal((2048, 8)).astype(np.float32); xb[5] *= 3e4; xb[70, 2] = np.inf; xb[71, 0] = np.nan; xb[900] = 0
    cbr = rng.standard_normal((256, 8)).astype(np.float32)
    check(xb, cbr, "bad rows")
    check(xb, cbr * 100, "large codebook")
    check(xb, np.zeros((16, 8), np.float32), "zero codebook")
    # one codebook per sub-space (the second benchmark configuration's wording): 16 sub-spaces of dim 8
    xs = rng.standard_normal((2, 300, 128)).astype(np.float32)
    cbs = rng.standard_normal((16, 256, 8)).astype(np.float32); cbs[5, 100] = cbs[5, 3]
    check(xs, cbs, "per-sub-space codebooks")
print("search ok")
"""


@pytest.mark.parametrize("mode", ["tc5", "mma", "exact"])
def test_pinned_search_matches_the_reference_order(mode):
    env = dict(os.environ, VQ_VQ_SEARCH=mode)
    out = subprocess.run([sys.executable, "-c", _CHILD % ROOT], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "search ok" in out.stdout, out.stdout[-2000:] + out.stderr[-4000:]
