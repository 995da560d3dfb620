"""Host-side configuration surface (no GPU): options read-through, explicit-field priority,
factory validation. Mirrors the reference's tests/cache/test_kvcache_config_options.py:29-107
and tests/cache/test_cache_factory.py:46-99."""

from __future__ import annotations

import warnings

import pytest

from veloxquant_mlx_b200.cache import (KIVIOptions, KVCacheBuilder, KVCacheConfig, KVCacheFactory,
                                       QuantizerConfigError, VecInferOptions)


def test_options_populate_flat_fields():
    cfg = KVCacheConfig(method="kivi", options=KIVIOptions(kivi_group_size=64))
    assert cfg.kivi_group_size == 64
    cfg = KVCacheConfig(method="vecinfer", options=VecInferOptions(key_sub_dim=8, residual_length=32))
    assert cfg.key_sub_dim == 8 and cfg.residual_length == 32 and cfg.value_sub_dim == 8


def test_explicit_flat_kwarg_beats_options_even_when_equal_to_default():
    cfg = KVCacheConfig(method="kivi", kivi_group_size=32, options=KIVIOptions(kivi_group_size=64))
    assert cfg.kivi_group_size == 32
    cfg = KVCacheConfig(method="kivi", residual_length=128, options=VecInferOptions(residual_length=16))
    assert cfg.residual_length == 128


def test_flat_setter_warns_after_construction():
    cfg = KVCacheConfig(method="kivi")
    with pytest.warns(DeprecationWarning, match="KIVIOptions"):
        cfg.kivi_group_size = 16
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        cfg.head_dim = 64  # not an options-backed field: silent


def test_factory_rejects_observers_outlier_bits_and_lists():
    with pytest.raises(QuantizerConfigError, match="observers"):
        KVCacheFactory.create(KVCacheConfig(method="kivi", observers=[object()]))
    with pytest.raises(QuantizerConfigError, match="bit_width_outlier"):
        KVCacheFactory.create(KVCacheConfig(method="kivi", bit_width_outlier=4))
    with pytest.raises(QuantizerConfigError, match="single int"):
        KVCacheFactory.create(KVCacheConfig(method="kivi", bit_width_inlier=[2, 4]))
    with pytest.raises(QuantizerConfigError, match="sliding_window"):
        KVCacheFactory.create(KVCacheConfig(method="kivi", sliding_window=64))


def test_unknown_method_lists_every_choice():
    with pytest.raises(QuantizerConfigError) as ei:
        KVCacheFactory.create(KVCacheConfig(method="no_such_method"))
    msg = str(ei.value)
    assert "unknown method 'no_such_method'" in msg and "kivi" in msg


def test_config_error_is_a_value_error_and_repr():
    assert issubclass(QuantizerConfigError, ValueError)
    assert "method='kivi'" in repr(KVCacheConfig(method="kivi", head_dim=64))


def test_no_cpu_path():
    # without a CUDA device (or with use_metal_kernels=False) construction fails loudly
    import torch

    with pytest.raises(RuntimeError, match="use_metal_kernels=False"):
        KVCacheFactory.create(KVCacheConfig(method="kivi", use_metal_kernels=False))
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="not available"):
            KVCacheFactory.create(KVCacheConfig(method="kivi"))


def test_builder_layer_lists_validate():
    with pytest.raises(QuantizerConfigError, match="2 entries for 3 layers"):
        KVCacheBuilder.for_layers(3, KVCacheConfig(method="kivi", bit_width_inlier=[2, 4]))


def test_named_bit_width_inlier_warns_for_methods_that_ignore_it():
    """The reference warns when the caller names ``bit_width_inlier`` for a method that never reads
    it, pointing at the method's own bit-width fields (``cache/base.py:930-955``); a copy made by
    ``dataclasses.replace`` names every field and does not warn."""
    import dataclasses
    import warnings

    from veloxquant_mlx_b200.cache import KVCacheConfig

    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        KVCacheConfig(method="kivi", bit_width_inlier=4)
        KVCacheConfig(method="turboquant_rvq", bit_width_inlier=3)
        KVCacheConfig(method="skvq")
        assert not w
        c = KVCacheConfig(method="skvq", bit_width_inlier=2)
        assert len(w) == 1 and issubclass(w[0].category, UserWarning)
        assert "ignores bit_width_inlier=2" in str(w[0].message) and "skvq_bits_key, skvq_bits_value" in str(w[0].message)
        dataclasses.replace(c, head_dim=64)
        assert len(w) == 1
        KVCacheConfig(method="vecinfer", bit_width_inlier=3)
        assert len(w) == 2 and "own bit-width field" not in str(w[1].message)


def _config_namespace():
    import types

    from veloxquant_mlx_b200 import cache as c

    return types.SimpleNamespace(KVCacheConfig=c.KVCacheConfig, KVCacheFactory=c.KVCacheFactory, VecInferOptions=c.VecInferOptions,
                                 KIVIOptions=c.KIVIOptions, SKVQOptions=c.SKVQOptions, KittyOptions=c.KittyOptions,
                                 AgeTieredKVOptions=c.AgeTieredKVOptions, KVCacheBuilder=c.KVCacheBuilder, PlainCache=c.DenseKVCache)


def _load_config_scenarios():
    import importlib.util
    import json
    import os

    here = os.path.join(os.path.dirname(__file__), "golden")
    spec = importlib.util.spec_from_file_location("config_scenarios", os.path.join(here, "config_scenarios.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    with open(os.path.join(here, "config_traces.json")) as fh:
        return mod, json.load(fh)


def test_configuration_layer_matches_the_reference_config_layer_scenario_by_scenario():
    """Defaults of every shared field (the default method included), options read-through, an
    explicitly named flat field beating the options object, the deprecation warning on assigning an
    options-owned flat field, the ignored-bit-width warning, ``repr``, positional construction and the
    factory's refusals (unknown method, list-form width, observers, outlier width): the same scenarios
    (tests/golden/config_scenarios.py) were run by make_golden.py against the reference's own
    ``cache/base.py`` + ``cache/options.py``; every record (values, warnings, errors) must be equal."""
    import json

    mod, ref = _load_config_scenarios()
    mine = json.loads(json.dumps(mod.scenarios(_config_namespace()), default=str))
    assert set(mine) == set(ref["config"]) and len(mine) >= 19
    for name, record in ref["config"].items():
        assert mine[name] == record, name


@pytest.mark.gpu
def test_cache_construction_matches_the_reference_classes_scenario_by_scenario():
    """Class created per method and every constructor refusal (negative sink count, window of 1, sinks
    past the window, zero bits, clip factor above 1, hi fraction above 1, boundaries out of order, 17
    bits, list-form width, a sliding window on a protocol cache): same class names, same error types
    and messages as the reference's cache classes executed by make_golden.py."""
    import json

    mod, ref = _load_config_scenarios()
    mine = json.loads(json.dumps(mod.construction_scenarios(_config_namespace()), default=str))
    assert set(mine) == set(ref["construction"]) and len(mine) >= 15
    for name, record in ref["construction"].items():
        assert mine[name] == record, (name, mine[name], record)


def test_builder_plans_a_model_layer_by_layer_as_the_reference_builder_does():
    """``KVCacheBuilder.for_model`` over stand-in models, against the reference's own builder run by
    make_golden.py on the same models (``cache/base.py:1242-1433``): where the layers are found, the
    per-layer head_dim and its three sources in their order of precedence, seeds by layer index, a
    list-form width spread over the attention layers only, what a layer without attention receives (the
    model's own slot, looked up on the class; a plain cache when the hook is missing, fails with a
    warning, or returns the wrong length), and the error for a list of the wrong length."""
    import json

    mod, ref = _load_config_scenarios()
    mine = json.loads(json.dumps(mod.builder_scenarios(_config_namespace()), default=str))
    assert set(mine) == set(ref["builder"]) and len(mine) >= 15
    for name, record in ref["builder"].items():
        assert mine[name] == record, (name, mine[name], record)


def test_dense_cache_for_unquantized_layers_grows_trims_and_restores():
    import torch

    from veloxquant_mlx_b200.cache import DenseKVCache

    k, v = torch.randn(1, 2, 300, 8), torch.randn(1, 2, 300, 4)
    d = DenseKVCache()
    assert d.empty() and d.nbytes == 0 and d.state == (None, None)
    a, b = d.update_and_fetch(k[:, :, :250], v[:, :, :250])
    assert d.keys.shape[2] == 512 and a.shape[2] == 250
    for t in range(250, 300):
        a, b = d.update_and_fetch(k[:, :, t:t + 1], v[:, :, t:t + 1])
    assert torch.equal(a, k) and torch.equal(b, v) and d.offset == d.size() == 300
    assert d.nbytes == 300 * 2 * (8 + 4) * 4 and d.is_trimmable()
    assert d.trim(5) == 5 and d.trim(1000) == 295 and d.offset == 0
    a, b = d.update_and_fetch(k[:, :, :3], v[:, :, :3])
    assert torch.equal(a, k[:, :, :3])
    e = DenseKVCache()
    e.state = d.state
    assert e.offset == 3 and torch.equal(e.state[1], v[:, :, :3])
    a, b = e.update_and_fetch(k[:, :, 3:4], v[:, :, 3:4])           # a restored cache grows from its live rows
    assert torch.equal(a, k[:, :, :4]) and torch.equal(b, v[:, :, :4])
    e.reset()
    assert e.empty() and e.offset == 0
