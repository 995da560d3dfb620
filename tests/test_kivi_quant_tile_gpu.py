"""The tuned quantize kernel (head_dim 128, group 32, f16/bf16) must be bit-identical to the
oracle, including the cases its reciprocal shortcut could get wrong: quotients that land on
exact halves (round-half-even), constant groups (scale floored at eps), huge and tiny ranges."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import bitpack as o_bitpack
from oracle import kivi as o_kivi

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
_DT = {"float16": torch.float16, "bfloat16": torch.bfloat16}


def _check(x32, dt, b, axis):
    from veloxquant_mlx_b200 import kernels as k

    t = torch.from_numpy(x32).to(_DT[dt])
    xs = t.float().numpy()
    codes, scale, zero = k.kivi_quantize(t.to(DEV), axis, 32, b)
    oc, os_, oz = (o_kivi.quant_keys if axis == -2 else o_kivi.quant_values)(xs, 32, (1 << b) - 1)
    np.testing.assert_array_equal(scale.cpu().numpy(), os_)
    np.testing.assert_array_equal(zero.cpu().numpy(), oz)
    got = o_bitpack.unpack(codes.cpu().numpy(), k.storage_bits(b), 128)
    bad = np.argwhere(got != oc)
    assert bad.size == 0, f"{len(bad)} codes differ, first at {bad[0]}: {got[tuple(bad[0])]} vs {oc[tuple(bad[0])]}"


@pytest.mark.parametrize("dt", ["float16", "bfloat16"])
@pytest.mark.parametrize("b", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("axis", [-2, -1])
def test_random_and_outlier_data(dt, b, axis):
    rng = np.random.default_rng(b * 10 + (axis == -1))
    x = rng.standard_normal((2, 3, 256, 128)).astype(np.float32)
    x[..., [3, 40, 77, 120]] *= 20.0
    _check(x, dt, b, axis)
    if axis == -1:  # values take any token count (ragged last tile)
        _check(x[:, :, :77], dt, b, axis)


@pytest.mark.parametrize("b", [2, 4, 8])
@pytest.mark.parametrize("axis", [-2, -1])
def test_exact_half_quotients_and_degenerate_groups(b, axis):
    levels = (1 << b) - 1
    rng = np.random.default_rng(b)
    # integer data whose range is 2*levels: every odd value sits exactly on k + 0.5
    x = rng.integers(0, 2 * levels + 1, (1, 2, 64, 128)).astype(np.float32)
    x[:, :, 0, :] = 0
    x[:, :, 1, :] = 2 * levels
    x[:, :, :, 0] = 0
    x[:, :, :, 1] = 2 * levels
    _check(x, "float16", b, axis)
    # multiples of 1/3 of the step, constant groups, one huge and one tiny group
    y = (rng.integers(0, 3 * levels + 1, (1, 2, 64, 128)) / 3.0).astype(np.float32)
    y[0, 0, :32, :] = 3.5
    y[0, 1, 32:, :64] *= 1e3
    y[0, 1, :32, 64:] *= 1e-4
    _check(y, "float16", b, axis)
    _check(y, "bfloat16", b, axis)


def test_slices_of_cache_buffers_take_the_same_path():
    from veloxquant_mlx_b200 import kernels as k

    buf = torch.randn(2, 2, 300, 128, device=DEV, dtype=torch.float16)
    sl = buf[:, :, 40:168]
    codes, scale, zero = k.kivi_quantize(sl, -2, 32, 4)
    oc, os_, oz = o_kivi.quant_keys(sl.cpu().numpy(), 32, 15)
    np.testing.assert_array_equal(codes.cpu().numpy(), o_bitpack.pack(oc, 4))
    np.testing.assert_array_equal(scale.cpu().numpy(), os_)
