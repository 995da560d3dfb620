"""The native caches against traces of the reference's own cache classes (``cache/kivi_cache.py``,
``sink_cache.py``, ``skvq_cache.py``, ``kitty_cache.py``, ``age_tiered_cache.py``), which
``tests/golden/make_golden.py`` executed unmodified over NumPy stand-ins for ``mlx.core`` and for the
``mlx_lm`` container class they derive from (``tests/golden/cache_traces.npz``)."""

import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _make(method, **cfg):
    from veloxquant_mlx_b200.cache import KVCacheConfig, KVCacheFactory

    return KVCacheFactory.create(KVCacheConfig(method=method, **cfg))


@pytest.mark.parametrize("method,tag,trimmable,cfg", [
    ("kivi", "kivi", True, dict(bit_width_inlier=2, kivi_group_size=8, residual_length=16)),
    ("kivi_sink", "sink", True, dict(bit_width_inlier=2, kivi_group_size=8, residual_length=16, n_sink_tokens=2)),
    ("skvq", "skvq", False, dict(skvq_bits_key=2, skvq_bits_value=3, skvq_group_size=8, skvq_window=16, skvq_n_sink=3)),
    ("kitty", "kitty", True, dict(kitty_group_size=8)),
    ("age_tiered", "age", False, dict(age_recent_boundary=20, age_mid_boundary=50, age_group_size=8)),
])
def test_native_caches_replay_the_reference_classes_traces(method, tag, trimmable, cfg):
    """The recorded call script (prefill, single tokens, a block, a trim, more tokens) on the native
    caches: what ``update_and_fetch`` returns equals, bit for bit, what the reference's own cache
    classes returned when make_golden.py executed them over the NumPy stand-ins."""
    z = np.load(os.path.join(GOLDEN, "cache_traces.npz"))
    c = _make(method, head_dim=32, **cfg)
    k, v = z["k"], z["v"]
    checked = 0
    for i, (op, a, b) in enumerate(z["script"].tolist()):
        if op == 1:
            if trimmable:
                assert c.trim(a) == a
            continue
        ko, vo = c.update_and_fetch(_t(k[:, :, a:b]), _t(v[:, :, a:b]))
        if f"{tag}_k_{i}" in z:
            np.testing.assert_array_equal(ko.cpu().numpy(), z[f"{tag}_k_{i}"], err_msg=f"{tag} keys after call {i}")
            np.testing.assert_array_equal(vo.cpu().numpy(), z[f"{tag}_v_{i}"], err_msg=f"{tag} values after call {i}")
            assert c.offset == int(z[f"{tag}_c_{i}"][0])
            checked += 1
    assert checked >= 10
