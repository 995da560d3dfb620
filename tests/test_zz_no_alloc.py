"""The allocation-free decode-attention entry point, ``vq_kivi_decode_attend_static``.

Some users of this library run where device memory cannot be allocated once serving has
started: the memory pool was sized and handed out up front, or a host runtime owns every
allocation. For them the library offers a variant of the fused KIVI decode attention whose
scratch (the per-split partial results) sits in a fixed 8 MiB array inside the library
instead of a caller-provided workspace.

This file checks, through the C ABI, that the variant gives the same answer as the regular
entry point -- twice in a row with different inputs, because the built-in array is shared
by all calls and keeps the previous call's contents -- and that it refuses a problem too
large for the array with a clear error. The comparison is with the regular entry point, not
with the CPU oracle: the regular entry point is what the other test files check against the
oracle, and here only the scratch memory differs. It is named to be collected last, so a run that
stops at the first failure has already run every other test.
"""

from __future__ import annotations

import ctypes as C
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _case(seed, B, H, H_kv, n_quant, n_res, bits):
    from veloxquant_mlx_b200 import kernels as k

    g = torch.Generator(device=DEV)
    g.manual_seed(seed)
    D, group = 128, 32
    q = torch.randn((B, H, 1, D), generator=g, device=DEV, dtype=torch.float16)
    kv = torch.randn((2, B, H_kv, n_quant + n_res, D), generator=g, device=DEV, dtype=torch.float16)
    kc, ks, kz = k.kivi_quantize(kv[0][:, :, :n_quant], -2, group, bits)
    vc, vs, vz = k.kivi_quantize(kv[1][:, :, :n_quant], -1, group, bits)
    k_res = kv[0][:, :, n_quant:].contiguous()
    v_res = kv[1][:, :, n_quant:].contiguous()
    return q, kc, ks, kz, vc, vs, vz, k_res, v_res


def _run(case, bits, static, variant=0, n_splits=0):
    from veloxquant_mlx_b200 import kernels as k

    q, kc, ks, kz, vc, vs, vz, k_res, v_res = case
    out = torch.full(q.shape, float("nan"), dtype=q.dtype, device=q.device)  # caller-owned output
    k.kivi_decode_attend(q, kc, ks, kz, vc, vs, vz, 32, 1.0 / math.sqrt(128), store_bits=bits,
                         k_res=k_res, v_res=v_res, out=out, static_scratch=static, variant=variant,
                         n_splits=n_splits)
    torch.cuda.synchronize()
    return out.float().cpu().numpy()


@pytest.mark.parametrize("bits,variant", [(4, 0), (2, 0), (4, 1)])
def test_static_scratch_matches_workspace_entry_point_twice_in_a_row(bits, variant):
    # two different problems back to back: the second call finds the first call's partials
    # still in the built-in array and must not be affected by them
    cases = [_case(1, 2, 8, 2, 1024, 40, bits), _case(2, 1, 4, 4, 256, 0, bits)]
    for case in cases:
        want = _run(case, bits, static=False, variant=variant)
        got = _run(case, bits, static=True, variant=variant)
        assert np.isfinite(got).all()
        # same kernels, same split plan: the tolerance of the other attention tests is kept
        # as the bound, although the two results are expected to coincide
        err = np.abs(got - want)
        assert np.all(err <= 2e-3 + 1e-2 * np.abs(want)), f"max err {err.max():.3e}"
    # and once more on the first problem, after the second one overwrote the array
    want = _run(cases[0], bits, static=False, variant=variant)
    got = _run(cases[0], bits, static=True, variant=variant)
    assert np.all(np.abs(got - want) <= 2e-3 + 1e-2 * np.abs(want))


def test_static_scratch_rejects_oversized_problems_with_a_clear_error():
    from veloxquant_mlx_b200 import VQLibraryError

    # 256 splits x (16 batch x 8 heads) rows x 130 floats = 17 MB, beyond the 8 MiB array
    case = _case(3, 16, 8, 8, 2048, 0, 4)
    with pytest.raises(VQLibraryError, match="VQ_ERR_CAPACITY.*built-in"):
        _run(case, 4, static=True, variant=1, n_splits=256)
    # the regular entry point handles the same call
    assert np.isfinite(_run(case, 4, static=False, variant=1, n_splits=256)).all()


def test_static_entry_point_allocates_nothing_after_its_first_call():
    """Neither torch's allocator nor the driver hands out memory for a call after the first one
    on the device (the first one resolves the array's address, which under lazy module loading
    is also when the driver sets the array aside)."""
    case = _case(4, 2, 8, 2, 512, 16, 4)
    _run(case, 4, static=True)  # first call on the device: one-time address look-up
    torch.cuda.synchronize()
    before = torch.cuda.memory_stats()["allocation.all.allocated"]
    free_before = torch.cuda.mem_get_info()[0]
    from veloxquant_mlx_b200 import kernels as k

    q, kc, ks, kz, vc, vs, vz, k_res, v_res = case
    out = torch.empty_like(q)
    mid = torch.cuda.memory_stats()["allocation.all.allocated"]
    k.kivi_decode_attend(q, kc, ks, kz, vc, vs, vz, 32, 0.1, store_bits=4, k_res=k_res, v_res=v_res,
                         out=out, static_scratch=True)
    torch.cuda.synchronize()
    after = torch.cuda.memory_stats()["allocation.all.allocated"]
    assert mid == before + 1 and after == mid
    # the driver's own view of free device memory: cudaMalloc inside the library, or a module
    # loaded by the call, would show here and not in torch's counters (out comes from torch's
    # cache, already reserved, so it does not move this figure either)
    assert torch.cuda.mem_get_info()[0] == free_before
