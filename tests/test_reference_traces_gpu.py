"""The native caches against traces of the reference's own cache classes (``cache/kivi_cache.py``,
``sink_cache.py``, ``skvq_cache.py``, ``kitty_cache.py``, ``age_tiered_cache.py``), which
``tests/golden/make_golden.py`` executed unmodified over NumPy stand-ins for ``mlx.core`` and for the
``mlx_lm`` container class they derive from (``tests/golden/cache_traces.npz``; the TurboQuant-RVQ
class's trace is in ``tests/golden/rvq_reference.npz``)."""

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


def test_native_vecinfer_cache_replays_the_reference_class_trace():
    """VecInfer (standard path, per-head smooth factors, 256-entry codebooks): the value reconstructions
    equal the reference class's bit for bit (no transform on that side); the key reconstructions agree to
    one float16 step, and all but a sliver exactly -- the reference rotates with a dense ``@ H`` (whatever
    order the matrix product takes), this package with the butterfly, so the float32 values behind the
    float16 rounding differ in their last bits."""
    z = np.load(os.path.join(GOLDEN, "cache_traces.npz"))
    c = _make("vecinfer", head_dim=32, key_sub_dim=4, value_sub_dim=8, key_codebook_bits=8, value_codebook_bits=8,
              smooth_factors=_t(z["vecinfer_smooth"]), key_codebook=_t(z["vecinfer_cb_k"]), value_codebook=_t(z["vecinfer_cb_v"]))
    k, v = z["k"], z["v"]
    checked, same, total = 0, 0, 0
    for i, (op, a, b) in enumerate(z["script"].tolist()):
        if op == 1:
            assert c.trim(a) == a
            continue
        ko, vo = c.update_and_fetch(_t(k[:, :, a:b]), _t(v[:, :, a:b]))
        if f"vecinfer_k_{i}" in z:
            want_k, want_v = z[f"vecinfer_k_{i}"], z[f"vecinfer_v_{i}"]
            np.testing.assert_array_equal(vo.cpu().numpy(), want_v)
            got = ko.float().cpu().numpy()
            np.testing.assert_allclose(got, want_k.astype(np.float32), rtol=2.0 ** -10, atol=2.0 ** -14)
            same += int((got == want_k.astype(np.float32)).sum())
            total += got.size
            assert c.offset == int(z[f"vecinfer_c_{i}"][0])
            checked += 1
    assert checked >= 10 and same / total > 0.995


def test_native_rvq_cache_replays_the_reference_class_trace():
    """TurboQuant-RVQ (``cache/turboquant_rvq_cache.py`` executed over the stand-ins,
    ``tests/golden/rvq_reference.npz``; one key with a norm past 65504, one zero key, a trim): values,
    offsets, buffer growth and byte counters equal the reference class's; the decoded keys and the stored
    code words equal it row for row, where a row may differ only if the float32 norm's summation order
    (a library reduction here, NumPy's there) moved a coordinate across a code boundary -- at most a
    sliver of rows, each then within one code step."""
    z = np.load(os.path.join(GOLDEN, "rvq_reference.npz"))
    B, H, D, T, bits, seed = (int(x) for x in z["cache_dims"])
    c = _make("turboquant_rvq", head_dim=D, bit_width_inlier=bits, seed=seed)
    k, v = z["cache_k"], z["cache_v"]
    checked, same, total = 0, 0, 0
    for i, (op, a, b) in enumerate(z["cache_script"].tolist()):
        if op == 1:
            assert c.trim(a) == a
            continue
        ko, vo = c.update_and_fetch(_t(k[:, :, a:b]), _t(v[:, :, a:b]))
        if f"cache_k_{i}" in z:
            want = z[f"cache_k_{i}"].astype(np.float32)
            got = ko.float().cpu().numpy()
            assert ko.dtype == torch.float16 and got.shape == want.shape and np.isfinite(got).all()
            np.testing.assert_array_equal(vo.cpu().numpy(), z[f"cache_v_{i}"])
            rows_same = (got == want).all(-1)
            err = np.linalg.norm(got - want, axis=-1) / np.maximum(np.linalg.norm(want, axis=-1), 1e-30)
            assert float(err.max()) <= 0.25
            same += int(rows_same.sum())
            total += rows_same.size
            assert [c.offset, c._packed1.shape[2], c.compressed_key_bytes, c.fp16_key_bytes, c.nbytes] == z[f"cache_c_{i}"].tolist()
            checked += 1
    assert checked >= 5 and same / total >= 0.98
    p1, p2, norms, _ = c.state
    words_same = (p1.cpu().numpy().view(np.uint32) == z["cache_state_p1"]).all(-1) & (p2.cpu().numpy().view(np.uint32) == z["cache_state_p2"]).all(-1)
    assert float(words_same.mean()) >= 0.98
    np.testing.assert_allclose(norms.float().cpu().numpy(), z["cache_state_norms"], rtol=2.0 ** -7, atol=0)
    assert [int(s) for s in c.meta_state] == z["cache_meta_state"].tolist()
