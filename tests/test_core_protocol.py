"""The standalone cache protocol (``KVCache``) and ``EncodedVector``, as the reference's
``core/abstractions.py:120-189`` and ``core/context.py:72-138`` define them."""

from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from veloxquant_mlx_b200.core import EncodedVector, KVCache, StandaloneProtocol


def test_kvcache_is_abstract_and_has_the_reference_surface():
    with pytest.raises(TypeError):
        KVCache()
    for name in ("append_key", "append_value", "attend", "memory_bytes", "reset", "append", "__len__"):
        assert hasattr(KVCache, name)

    class Tiny(KVCache):
        def __init__(self):
            self.k, self.v = [], []

        def append_key(self, k):
            self.k.append(k)

        def append_value(self, v):
            self.v.append(v)

        def attend(self, q):
            return q

        def memory_bytes(self):
            return 0

        def __len__(self):
            return len(self.v)

    t = Tiny()
    t.append(1, 2)
    assert len(t) == 1 and repr(t) == "Tiny(size=1)"
    with pytest.raises(NotImplementedError):
        t.reset()


def test_encoded_vector_counts_every_array_and_nested_encodings():
    inner = EncodedVector("turboquant_mse", 2, 4, indices=np.zeros((2, 4), np.uint8))
    ev = EncodedVector("composite", 2, 8, indices=torch.zeros(2, 8, dtype=torch.uint8), norm=torch.zeros(2, dtype=torch.float16),
                       signs=np.zeros((2, 16), np.int8), angles=[np.zeros((2, 4), np.float16), np.zeros((2, 2), np.float16)],
                       outlier_idx=np.arange(3, dtype=np.int32), inlier_encoded=inner)
    assert ev.memory_bytes() == 16 + 4 + 32 + 16 + 8 + 12 + 8
    assert EncodedVector("empty", 0, 8).memory_bytes() == 0
    assert "composite" in repr(ev)


def test_every_cache_class_is_a_kvcache():
    from veloxquant_mlx_b200.cache import KIVIKVCache, RaBitQKVCache, VecInferKVCache

    for cls in (KIVIKVCache, RaBitQKVCache, VecInferKVCache):
        assert issubclass(cls, KVCache) and issubclass(cls, StandaloneProtocol)


def test_standalone_protocol_argument_errors_need_no_gpu():
    class Fake(StandaloneProtocol):
        _head_dim = 8
        offset = 0
        nbytes = 0

        def _reset_tokens(self):
            self.offset = 0

    f = Fake()
    with pytest.raises(RuntimeError, match="append_key comes first"):
        f.append_value(torch.zeros(8))
    with pytest.raises(ValueError, match="expected d=8"):
        f.append_key(torch.zeros(4))
    with pytest.raises(ValueError, match="shape"):
        f.append_key(torch.zeros(2, 8))
    f.append_key(torch.zeros(8))
    with pytest.raises(RuntimeError, match="still waits"):
        f.append_key(torch.zeros(8))
    assert torch.equal(f.attend(torch.ones(8)), torch.zeros(8)) and f.memory_bytes() == 0
    f.reset()
    assert f._pending_key is None


@pytest.mark.gpu
@pytest.mark.parametrize("method", ["kivi", "rabitq", "vecinfer"])
def test_standalone_calls_equal_the_batched_protocol(method):
    import warnings

    from veloxquant_mlx_b200.cache import KVCacheConfig, KVCacheFactory

    d, n = 128, 200
    kw = dict(method=method, head_dim=d)
    if method == "kivi":
        kw.update(bit_width_inlier=4, residual_length=64)
    if method == "vecinfer":
        kw.update(key_sub_dim=8, value_sub_dim=8, key_codebook_bits=8, value_codebook_bits=8, fused_sdpa=True)
    g = torch.Generator(device="cuda:0").manual_seed(3)
    k = torch.randn((n, d), generator=g, device="cuda:0", dtype=torch.float16)
    v = torch.randn((n, d), generator=g, device="cuda:0", dtype=torch.float16)
    q = torch.randn((d,), generator=g, device="cuda:0", dtype=torch.float16)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        one, many = KVCacheFactory.create(KVCacheConfig(**kw)), KVCacheFactory.create(KVCacheConfig(**kw))
    assert isinstance(one, KVCache) and len(one) == 0 and one.memory_bytes() == 0
    assert torch.equal(one.attend(q), torch.zeros_like(q))
    for t in range(n):
        one.append(k[t], v[t])
        many.update_and_fetch(k[t].view(1, 1, 1, d), v[t].view(1, 1, 1, d))
    assert len(one) == n and one.memory_bytes() == many.nbytes > 0
    want = many.fused_sdpa(q.view(1, 1, 1, d), 1.0 / math.sqrt(d)).view(d)
    got = one.attend(q)
    assert got.shape == (d,) and got.dtype == q.dtype and torch.equal(got, want)
    one.reset()
    assert len(one) == 0 and torch.equal(one.attend(q), torch.zeros_like(q))
    one.append(k[0], v[0])          # still usable after reset: the quantizer state was kept
    assert len(one) == 1
    if method != "vecinfer":        # one token: the output is that token's value (kept exact by these two caches)
        assert float((one.attend(q).float() - v[0].float()).abs().max()) < 1e-2


def test_vecinfer_byte_counters_follow_the_reference_class_trace():
    """The counters behind ``compressed_key_bytes`` / ``compressed_value_bytes`` / ``fp16_key_bytes`` /
    ``fp16_value_bytes`` over the recorded call script (appends and a trim) against what the reference's
    ``VecInferKVCache`` held after each call when it was executed over the NumPy stand-ins
    (``tests/golden/cache_traces.npz``); the accounting is host arithmetic and needs no device."""
    import os

    import numpy as np

    import veloxquant_mlx_b200.cache  # noqa: F401  (the package's import order: the registry first)
    from veloxquant_mlx_b200.cache_coded import VecInferKVCache, _VQByteAccounting

    assert issubclass(VecInferKVCache, _VQByteAccounting)
    for name in ("compressed_key_bytes", "fp16_key_bytes", "compressed_value_bytes", "fp16_value_bytes", "codebook_bytes"):
        assert isinstance(getattr(VecInferKVCache, name), property)

    class Counters(_VQByteAccounting):
        _key_sub_dim, _value_sub_dim, _key_bits, _value_bits = 4, 8, 8, 8      # the trace's configuration

    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "cache_traces.npz"))
    B, H, _, D = z["k"].shape
    c, offset, checked = Counters(), 0, 0
    c._reset_bytes()
    for i, (op, a, b) in enumerate(z["script"].tolist()):
        if op == 1:
            c._scale_bytes((offset - a) / offset)          # what trim(a) does after lowering the offset
            offset -= a
            continue
        c._account_bytes(B, H, b - a, D)
        offset += b - a
        if f"vecinfer_c_{i}" in z:
            want = z[f"vecinfer_c_{i}"].tolist()            # offset, key bytes, value bytes, fp16 key bytes, tokens seen
            assert [offset, c.compressed_key_bytes, c.compressed_value_bytes, c.fp16_key_bytes, c._tokens_seen] == want, i
            assert c.fp16_value_bytes == c.fp16_key_bytes
            checked += 1
    assert checked >= 10 and c.codebook_bytes == 256 * 4 * 2 + 256 * 8 * 2


def test_cache_classes_define_the_public_surface_of_the_reference_classes():
    """``tests/golden/class_surfaces.json``: the public properties, setters and method parameter lists the
    reference's cache classes define themselves, read from its source. Each class here has every
    property as a property (with a setter where the reference has one) and every method with the same
    parameters in the same order. ``merge`` is a property that raises ``AttributeError`` wherever the
    reference makes it one, so that ``hasattr(cache, "merge")`` is false. One name is left out:
    ``TurboQuantRVQKVCache.make_mask``, which forwards to the mask builder of the reference's serving
    framework; here the model library builds the masks."""
    import inspect
    import json
    import os

    from veloxquant_mlx_b200 import cache as c

    with open(os.path.join(os.path.dirname(__file__), "golden", "class_surfaces.json")) as fh:
        ref = json.load(fh)
    left_out = {("TurboQuantRVQKVCache", "make_mask")}
    assert len(ref) == 7
    for cls_name, spec in ref.items():
        cls = getattr(c, cls_name)
        for name in spec["properties"]:
            assert isinstance(inspect.getattr_static(cls, name), property), (cls_name, name)
        for name in spec["setters"]:
            assert inspect.getattr_static(cls, name).fset is not None, (cls_name, name)
        for name, sig in spec["methods"].items():
            if (cls_name, name) in left_out:
                continue
            fn = inspect.getattr_static(cls, name)
            fn = fn.__func__ if isinstance(fn, (classmethod, staticmethod)) else fn
            params = list(inspect.signature(fn).parameters.values())[1:]          # without self / cls
            names = [p.name for p in params if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
            if not sig["var_positional"]:
                assert names[:len(sig["positional"])] == sig["positional"], (cls_name, name, names)
            assert set(sig["keyword_only"]) <= {p.name for p in params}, (cls_name, name)
        if "merge" in spec["properties"]:
            obj = object.__new__(cls)
            assert not hasattr(obj, "merge"), cls_name


def test_kivi_byte_counters_follow_the_reference_class_trace():
    """``KIVIKVCache``'s own accounting methods (host arithmetic) driven through the recorded call script
    with the reference's flush policy: the frontier, compressed key / value bytes, fp16 bytes, residual
    bytes and token count equal what the reference's ``KIVIKVCache`` held after each recorded call, the
    trim's roll-back included (``tests/golden/cache_traces.npz``; group 8, residual 16, 2 bits)."""
    import os

    import numpy as np

    from oracle import kivi as o_kivi
    from veloxquant_mlx_b200.cache import KIVIKVCache

    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "cache_traces.npz"))
    B, H, _, D = z["k"].shape
    g, R = 8, 16
    c = object.__new__(KIVIKVCache)                      # the accounting needs no device
    c._group_size, c._b, c._shape_bhd = g, 2, (B, H, D)
    c.offset = c._n_quantized = 0
    c._key_bytes_compressed = c._value_bytes_compressed = 0
    c._key_bytes_fp16 = c._value_bytes_fp16 = c._residual_fp16_bytes = c._tokens_seen = 0
    checked = 0
    for i, (op, a, b) in enumerate(z["script"].tolist()):
        if op == 1:                                      # trim(a): the frontier snaps down to a group multiple
            new_offset = c.offset - a
            n_rolled = 0
            if new_offset < c._n_quantized:
                new_nq = (new_offset // g) * g
                n_rolled, c._n_quantized = c._n_quantized - new_nq, new_nq
            c.offset = new_offset
            c._rollback_bytes(a, n_rolled)
            continue
        S = b - a
        c.offset += S
        boundary = o_kivi.quantization_boundary(c.offset, R, g)
        n_flush = max(boundary - c._n_quantized, 0)
        c._n_quantized += n_flush
        c._account_bytes(B, H, S, D, n_flush)
        if f"kivi_c_{i}" in z:
            want = z[f"kivi_c_{i}"].tolist()   # offset, frontier, key bytes, value bytes, fp16 key bytes, residual bytes, tokens
            got = [c.offset, c._n_quantized, c.compressed_key_bytes, c.compressed_value_bytes, c.fp16_key_bytes,
                   c.residual_fp16_bytes, c._tokens_seen]
            assert got == want, (i, got, want)
            checked += 1
    assert checked >= 10
