"""The shared group-quantization core of the reference's sibling methods
(``quantizers/_quant_utils.py``) on the KIVI quantize kernel: codes, scales and zero-points
bit-identical to the oracle (``oracle.kivi.quant_keys``, pinned to the reference's NumPy twin),
the padded tail as the reference returns it, batched == looped."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import kivi as o_kivi

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("N,D,b,gs", [(64, 128, 2, 32), (100, 64, 4, 32), (33, 16, 3, 8), (7, 8, 8, 32), (256, 128, 1, 64)])
@pytest.mark.parametrize("dt", [torch.float16, torch.float32])
def test_group_quant_codes_match_the_oracle(N, D, b, gs, dt):
    from veloxquant_mlx_b200 import quant_utils as qu

    rng = np.random.default_rng(N + D + b)
    x = torch.from_numpy(rng.standard_normal((N, D)).astype(np.float32)).to(dt).to(DEV)
    codes, scale, zero = qu._group_quant_codes(x, b, gs)
    n_groups = -(-N // gs)
    assert codes.shape == (n_groups, gs, D) and codes.dtype == torch.float32 and scale.shape == (n_groups, 1, D)
    oc, os_, oz = o_kivi.quant_keys(x.float().cpu().numpy()[None, None], gs, (1 << b) - 1)
    flat = codes.reshape(n_groups * gs, D).cpu().numpy()
    np.testing.assert_array_equal(flat[:N], oc[0, 0].astype(np.float32))
    np.testing.assert_array_equal(flat[N:], np.broadcast_to(flat[N - 1], (n_groups * gs - N, D)))  # padded tail
    np.testing.assert_array_equal(scale[:, 0].cpu().numpy(), os_[0, 0])
    np.testing.assert_array_equal(zero[:, 0].cpu().numpy(), oz[0, 0])
    rec = qu._group_dequant_codes(codes, scale, zero, N, gs)
    ref = o_kivi.dequant_keys(oc, os_, oz, gs)[0, 0]
    np.testing.assert_array_equal(rec.cpu().numpy(), ref)
    rt = qu._group_quant_dequant(x, b, gs)
    assert rt.dtype == torch.float16
    np.testing.assert_array_equal(rt.float().cpu().numpy(), ref.astype(np.float16).astype(np.float32))


def test_batched_functions_equal_a_loop_over_rows():
    from veloxquant_mlx_b200 import quant_utils as qu

    x = torch.randn(5, 70, 32, device=DEV, dtype=torch.float16)
    codes, scale, zero = qu._group_quant_codes_batched(x, 4, 32)
    assert codes.shape == (5, 3, 32, 32) and scale.shape == (5, 3, 1, 32)
    for i in range(5):
        c1, s1, z1 = qu._group_quant_codes(x[i], 4, 32)
        assert torch.equal(codes[i], c1) and torch.equal(scale[i], s1) and torch.equal(zero[i], z1)
    rec = qu._group_dequant_codes_batched(codes, scale, zero, 70, 32)
    assert rec.shape == (5, 70, 32)
    rt = qu._group_quant_dequant_batched(x, 4, 32)
    assert torch.equal(rt, rec.to(torch.float16))
    with pytest.raises(ValueError, match="must be 3D"):
        qu._group_quant_codes_batched(x[0], 4, 32)
    with pytest.raises(ValueError, match=r"b=9"):
        qu._group_quant_codes(x[0], 9, 32)
