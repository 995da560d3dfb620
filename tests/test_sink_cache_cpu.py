"""The sink-protected cache's oracle against the properties the reference's own tests assert
(``veloxquant_mlx/tests/cache/test_sink_cache.py:56-160``), and the parts of the product class
that need no GPU (factory dispatch, configuration errors)."""

from __future__ import annotations

import numpy as np
import pytest

from oracle import kivi as o_kivi
from oracle.kivi_sink import SinkProtectedOracle, neighbour_sources


def _kv_with_sinks(B=1, S=64, H=4, D=128, sink_pos=(0, 7, 20), scale=25.0, seed=0):
    rng = np.random.default_rng(seed)
    K = rng.standard_normal((B, H, S, D)).astype(np.float16)
    V = rng.standard_normal((B, H, S, D)).astype(np.float16)
    for p in sink_pos:
        K[:, :, p, :] *= scale
    return K, V


def test_neighbour_rule_left_first_then_right():
    assert neighbour_sources([3], 8) == {3: 2}
    assert neighbour_sources([0], 8) == {0: 1}
    assert neighbour_sources([0, 1, 2], 8) == {0: 3, 1: 3, 2: 3}
    assert neighbour_sources([4, 5], 8) == {4: 3, 5: 3}
    assert neighbour_sources([7], 8) == {7: 6}
    assert neighbour_sources([0, 1], 2) == {0: 0, 1: 1}   # nothing to copy from


def test_planted_sinks_detected_and_preserved():
    o = SinkProtectedOracle(128, 2, 32, 8, n_sink=3)
    K, V = _kv_with_sinks()
    ko, vo = o.update_and_fetch(K, V)
    assert set(o.sink_positions_for(0)) == {0, 7, 20}
    for p in (0, 7, 20):
        assert np.array_equal(ko[:, :, p], K[:, :, p]) and np.array_equal(vo[:, :, p], V[:, :, p])
    assert not np.array_equal(ko[:, :, 30], K[:, :, 30])
    assert o.n_quantized == 32 and np.array_equal(ko[:, :, 32:], K[:, :, 32:])


def test_zero_sinks_is_plain_kivi():
    K, V = _kv_with_sinks(sink_pos=())
    o = SinkProtectedOracle(128, 2, 32, 8, n_sink=0)
    ko, vo = o.update_and_fetch(K, V)
    np.testing.assert_array_equal(ko[:, :, :32], o_kivi.quant_dequant_along(K[:, :, :32], -2, 32, 3))
    np.testing.assert_array_equal(vo[:, :, :32], o_kivi.quant_dequant_along(V[:, :, :32], -1, 32, 3))


def test_sinks_are_excluded_from_the_group_parameters():
    """A 25x key row must not widen its group's scale: the other rows' error stays that of a
    block without the sink."""
    K, V = _kv_with_sinks(S=64, sink_pos=(7,))
    o = SinkProtectedOracle(128, 2, 32, 8, n_sink=1)
    ko, _ = o.update_and_fetch(K, V)
    plain = SinkProtectedOracle(128, 2, 32, 8, n_sink=0)
    kp, _ = plain.update_and_fetch(K, V)
    rows = [r for r in range(32) if r != 7]
    err_s = np.abs(ko[:, :, rows].astype(np.float32) - K[:, :, rows].astype(np.float32)).mean()
    err_p = np.abs(kp[:, :, rows].astype(np.float32) - K[:, :, rows].astype(np.float32)).mean()
    assert err_s < 0.3 * err_p


def test_sinks_tracked_independently_per_batch_element():
    o = SinkProtectedOracle(8, 2, 4, 4, n_sink=2)
    rng = np.random.default_rng(1)
    K = rng.standard_normal((2, 1, 20, 8)).astype(np.float32)
    K[1, 0, 5, :] = 50.0
    K = K.astype(np.float16)
    V = rng.standard_normal((2, 1, 20, 8)).astype(np.float16)
    ko, _ = o.update_and_fetch(K, V)
    assert 5 in o.sink_positions_for(1)
    assert np.array_equal(ko[1, :, 5], K[1, :, 5]) and not np.array_equal(ko[0, :, 5], K[0, :, 5])


def test_streamed_decode_matches_one_shot_when_sinks_come_first():
    """Sinks that are among the first tokens are selected the same way by a prefill and by a
    token-by-token run (the case the reference's note calls fully effective)."""
    K, V = _kv_with_sinks(S=100, sink_pos=(0, 3), seed=4)
    a = SinkProtectedOracle(128, 2, 32, 16, n_sink=2)
    ka, va = a.update_and_fetch(K, V)
    b = SinkProtectedOracle(128, 2, 32, 16, n_sink=2)
    b.update_and_fetch(K[:, :, :10], V[:, :, :10])
    for t in range(10, 100):
        kb, vb = b.update_and_fetch(K[:, :, t : t + 1], V[:, :, t : t + 1])
    np.testing.assert_array_equal(ka, kb)
    np.testing.assert_array_equal(va, vb)


def test_trim_drops_candidates_and_snaps_the_frontier():
    K, V = _kv_with_sinks(S=100, sink_pos=(0, 90), seed=5)
    o = SinkProtectedOracle(128, 2, 32, 8, n_sink=2)
    o.update_and_fetch(K, V)
    assert o.n_quantized == 64 and set(o.sink_positions_for(0)) == {0, 90}
    assert o.trim(50) == 50
    assert o.offset == 50 and o.n_quantized == 32 and o.sink_positions_for(0) == [0]


def test_factory_dispatch_and_configuration_errors():
    from veloxquant_mlx_b200 import kernels
    from veloxquant_mlx_b200.cache import KIVIKVCache, KVCacheConfig, KVCacheFactory, QuantizerConfigError, SinkProtectedKVCache

    assert issubclass(SinkProtectedKVCache, KIVIKVCache)
    if not kernels.kivi_available():
        with pytest.raises(RuntimeError):
            KVCacheFactory.create(KVCacheConfig(method="kivi_sink"))
        return
    c = KVCacheFactory.create(KVCacheConfig(method="kivi_sink", n_sink_tokens=3))
    assert isinstance(c, SinkProtectedKVCache) and not hasattr(c, "bits")
    with pytest.raises(QuantizerConfigError):
        KVCacheFactory.create(KVCacheConfig(method="kivi_sink", n_sink_tokens=-1))
