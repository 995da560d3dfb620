"""Configuration scenarios run against BOTH the reference's ``cache/base.py`` (by make_golden.py, over
stand-ins for ``mlx_lm`` and the cache modules) and this package's ``cache.py`` (by
tests/test_cache_config.py): each returns a JSON-able record of what the configuration layer did
(field values, warnings, errors), so the two can be compared entry by entry."""

import dataclasses
import warnings

SHARED_FIELDS = ["method", "head_dim", "bit_width_inlier", "bit_width_outlier", "seed", "sliding_window", "key_sub_dim",
                 "value_sub_dim", "key_codebook_bits", "value_codebook_bits", "residual_length", "kivi_group_size",
                 "fused_sdpa", "fused_sdpa_max_ctx", "fused_sdpa_memory_bound", "n_sink_tokens", "skvq_bits_key",
                 "skvq_bits_value", "skvq_group_size", "skvq_window", "skvq_n_sink", "skvq_reorder", "skvq_clip_search",
                 "skvq_clip_alpha", "skvq_max_ctx", "kitty_hi_fraction", "kitty_hi_bit", "kitty_lo_bit", "kitty_group_size",
                 "age_recent_boundary", "age_mid_boundary", "age_bits_recent", "age_bits_mid", "age_bits_old", "age_group_size"]


def _fields(cfg):
    return {name: getattr(cfg, name) for name in SHARED_FIELDS}


def _record(fn):
    """Run ``fn``; report its result, the warnings it raised (category + the part of the message
    that names the field / method) and the exception (type name + first 60 characters, without the
    list of registered methods)."""
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        try:
            result, error = fn(), None
        except Exception as e:  # noqa: BLE001
            result, error = None, [type(e).__name__, str(e).split(" Choices:")[0][:60]]
    warns = sorted([x.category.__name__, str(x.message).split(" is deprecated")[0].split(": only")[0][:80]] for x in w
                   if issubclass(x.category, (DeprecationWarning, UserWarning)) and "random N(0,1)" not in str(x.message))
    return {"result": result, "warnings": warns, "error": error}


def scenarios(ns):
    """``ns``: an object with ``KVCacheConfig``, ``KVCacheFactory``, ``VecInferOptions``, ``KIVIOptions``,
    ``SKVQOptions``, ``KittyOptions``, ``AgeTieredKVOptions``. Returns ``{name: record}``."""
    C, F = ns.KVCacheConfig, ns.KVCacheFactory
    out = {}
    out["defaults"] = _record(lambda: _fields(C()))
    out["repr"] = _record(lambda: repr(C(method="kivi", head_dim=64, bit_width_inlier=4, seed=7)))
    out["options_read_through_skvq"] = _record(lambda: _fields(C(method="skvq", options=ns.SKVQOptions(skvq_window=64, skvq_bits_key=2))))
    out["explicit_kwarg_wins"] = _record(lambda: _fields(C(method="skvq", skvq_window=128, options=ns.SKVQOptions(skvq_window=64))))
    out["options_vecinfer"] = _record(lambda: _fields(C(method="vecinfer", options=ns.VecInferOptions(key_sub_dim=8, residual_length=32))))
    out["options_kivi_group"] = _record(lambda: _fields(C(method="kivi", options=ns.KIVIOptions(kivi_group_size=64))))
    out["options_kitty"] = _record(lambda: _fields(C(method="kitty", options=ns.KittyOptions(kitty_hi_bit=8))))
    out["options_age"] = _record(lambda: _fields(C(method="age_tiered", options=ns.AgeTieredKVOptions(age_mid_boundary=256))))
    out["foreign_options_fill_their_fields"] = _record(lambda: _fields(C(method="kivi", options=ns.SKVQOptions(skvq_n_sink=1))))

    def set_flat():
        c = C(method="skvq")
        c.skvq_window = 5
        c.head_dim = 32          # not an options-owned field: silent
        return [c.skvq_window, c.head_dim]

    out["setattr_deprecation"] = _record(set_flat)
    out["inlier_bits_named_for_skvq"] = _record(lambda: _fields(C(method="skvq", bit_width_inlier=2))["bit_width_inlier"])
    out["inlier_bits_named_for_vecinfer"] = _record(lambda: C(method="vecinfer", bit_width_inlier=3).bit_width_inlier)
    out["inlier_bits_named_for_kivi"] = _record(lambda: C(method="kivi", bit_width_inlier=3).bit_width_inlier)
    out["replace_does_not_warn"] = _record(lambda: dataclasses.replace(C(method="kitty"), head_dim=64).head_dim)
    out["positional_method"] = _record(lambda: _fields(C("kivi_sink", 64))["head_dim"])
    out["factory_unknown_method"] = _record(lambda: F.create(C(method="no_such_method")))
    out["factory_list_bits"] = _record(lambda: F.create(C(method="kivi", bit_width_inlier=[2, 4])))
    out["factory_observers"] = _record(lambda: F.create(C(method="kivi", observers=[object()])))
    out["factory_outlier_bits"] = _record(lambda: F.create(C(method="kivi", bit_width_outlier=3)))
    return out


def construction_scenarios(ns):
    """Scenarios that construct a cache (this package needs a CUDA device for them)."""
    C, F = ns.KVCacheConfig, ns.KVCacheFactory
    out = {}
    out["factory_sliding_window_on_protocol_cache"] = _record(lambda: type(F.create(C(method="kivi", head_dim=32, sliding_window=16))).__name__)
    for method, kw in (("kivi", {}), ("kivi_sink", {}), ("skvq", {}), ("kitty", {}), ("age_tiered", {})):
        out[f"factory_{method}"] = _record(lambda m=method, k=kw: type(F.create(C(method=m, head_dim=32, **k))).__name__)
    for method, kw, tag in (("kivi_sink", {"n_sink_tokens": -1}, "negative_sinks"), ("skvq", {"skvq_window": 1}, "window_1"),
                            ("skvq", {"skvq_n_sink": 200}, "sinks_past_window"), ("skvq", {"skvq_bits_key": 0}, "bits_0"),
                            ("skvq", {"skvq_clip_alpha": 1.5}, "alpha"), ("kitty", {"kitty_hi_fraction": 2.0}, "hi_fraction"),
                            ("age_tiered", {"age_recent_boundary": 0}, "recent_0"),
                            ("age_tiered", {"age_recent_boundary": 64, "age_mid_boundary": 32}, "mid_below_recent"),
                            ("age_tiered", {"age_bits_mid": 17}, "bits_17"), ("kivi", {"bit_width_inlier": [2]}, "kivi_list")):
        out[f"factory_{method}_{tag}"] = _record(lambda m=method, k=kw: type(F.create(C(method=m, head_dim=32, **k))).__name__)
    return out
