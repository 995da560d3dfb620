"""Model-level integration: the mask recogniser (the semantics pinned by the reference's
``metal/fused_sdpa.py:332-396``), the SDPA dispatch rule (``metal/fused_sdpa.py:399-416``) and
the Hugging Face Transformers cache adapter, driven by a small randomly initialised Llama.
The plumbing runs on CPU with a dense stand-in cache; with a GPU the real caches are used."""

from __future__ import annotations

import warnings

import pytest
import torch

from veloxquant_mlx_b200 import integration as I


def _q(B=2, H=4, N=3, D=8):
    return torch.zeros(B, H, N, D)


def _causal(N, S, window=0, dtype=torch.bool):
    q = torch.arange(S - N, S)[:, None]
    k = torch.arange(S)[None, :]
    vis = k <= q
    if window:
        vis &= k > q - window
    if dtype == torch.bool:
        return vis
    return torch.where(vis, torch.zeros((), dtype=dtype), torch.full((), float("-inf"), dtype=dtype))


def test_mask_none_and_causal_string():
    assert I._memory_bound_mask_parameters(None, _q(), 10) == (False, 0)
    assert I._memory_bound_mask_parameters("causal", _q(), 10) == (True, 0)
    with pytest.raises(ValueError, match="cannot be represented"):
        I._memory_bound_mask_parameters("sliding", _q(), 10)


@pytest.mark.parametrize("dtype", [torch.bool, torch.float32, torch.float16])
@pytest.mark.parametrize("shape", ["2d", "3d", "4d-broadcast", "4d-full"])
def test_tail_aligned_causal_and_window_masks_are_recognised(dtype, shape):
    N, S = 3, 10
    for window, want in ((0, (True, 0)), (4, (True, 4)), (S, (True, 0))):
        m = _causal(N, S, window if window != S else 0, dtype)
        if shape == "3d":
            m = m[None]
        elif shape == "4d-broadcast":
            m = m[None, None]
        elif shape == "4d-full":
            m = m[None, None].expand(2, 4, N, S).contiguous()
        assert I._memory_bound_mask_parameters(m, _q(N=N), S) == want
    full = torch.ones(N, S, dtype=torch.bool) if dtype == torch.bool else torch.zeros(N, S, dtype=dtype)
    assert I._memory_bound_mask_parameters(full, _q(N=N), S) == (False, 0)
    # one query row (decode): everything visible, or a trailing window
    row = _causal(1, S, 0, dtype)
    assert I._memory_bound_mask_parameters(row, _q(N=1), S) == (False, 0)
    assert I._memory_bound_mask_parameters(_causal(1, S, 5, dtype), _q(N=1), S) == (True, 5)


def test_masks_the_kernel_cannot_represent_raise_instead_of_being_ignored():
    N, S = 3, 10
    good = _causal(N, S)
    hole = good.clone(); hole[1, 2] = False
    padded = good.clone(); padded[:, 0] = False                      # left padding
    per_head = good[None, None].expand(2, 4, N, S).clone(); per_head[0, 1, 2, 5] = False
    per_batch = good[None, None].expand(2, 1, N, S).clone(); per_batch[1, 0, :, :2] = False
    bias = torch.zeros(N, S); bias[0, 0] = -1.5                       # a finite bias is not a mask
    shifted = torch.ones(N, S, dtype=torch.bool).tril(0)             # top-left aligned causal
    nothing = torch.zeros(N, S, dtype=torch.bool)
    for bad in (hole, padded, per_head, per_batch, bias, shifted, nothing, torch.zeros(N, S, dtype=torch.int32),
                torch.ones(5, S, dtype=torch.bool), torch.ones(N, S + 1, dtype=torch.bool), torch.ones(1, 1, 1, N, S, dtype=torch.bool)):
        with pytest.raises(ValueError, match="cannot be represented"):
            I._memory_bound_mask_parameters(bad, _q(N=N), S)
    with pytest.raises(ValueError):
        I._memory_bound_mask_parameters(torch.ones(4, 2, dtype=torch.bool), _q(N=4), 2)   # more queries than keys


class _DenseCache:
    """Dense stand-in with this package's cache interface (for the plumbing tests on CPU)."""

    def __init__(self, memory_bound):
        self._memory_bound, self.k, self.v, self.offset, self.calls = memory_bound, None, None, 0, []

    def update_and_fetch(self, k, v):
        self.k = k if self.k is None else torch.cat([self.k, k], 2)
        self.v = v if self.v is None else torch.cat([self.v, v], 2)
        self.offset = self.k.shape[2]
        if self._memory_bound:
            z = k.new_zeros((k.shape[0], k.shape[1], 0, k.shape[3]))
            return z, z
        return self.k, self.v

    def fused_sdpa(self, q, scale, *, causal=True, sliding_window=0):
        self.calls.append((q.shape[2], causal, sliding_window))
        return I._dense_sdpa(q, self.k, self.v, scale, "causal" if causal and q.shape[2] > 1 else None)

    def reset(self):
        self.k = self.v = None
        self.offset = 0

    def trim(self, n):
        self.k, self.v = self.k[:, :, :-n], self.v[:, :, :-n]
        self.offset -= n
        return n


def test_dispatch_rule_memory_bound_never_falls_back_to_the_sentinels():
    q = torch.randn(1, 4, 1, 8)
    c = _DenseCache(True)
    c.update_and_fetch(torch.randn(1, 2, 5, 8), torch.randn(1, 2, 5, 8))
    z = torch.zeros(1, 2, 0, 8)
    out = I.fused_sdpa_dispatch(q, z, z, c, 0.3, None)
    assert out.shape == (1, 4, 1, 8) and c.calls == [(1, False, 0)]
    with pytest.raises(ValueError, match="attention sinks"):
        I.fused_sdpa_dispatch(q, z, z, c, 0.3, None, sinks=torch.zeros(4))
    hole = torch.ones(1, 5, dtype=torch.bool); hole[0, 2] = False
    with pytest.raises(ValueError, match="cannot be represented"):
        I.fused_sdpa_dispatch(q, z, z, c, 0.3, hole)
    c.fused_sdpa = None
    with pytest.raises(RuntimeError, match="callable fused_sdpa"):
        I.fused_sdpa_dispatch(q, z, z, c, 0.3, None)
    # a cache that keeps real K/V takes the original attention, with the caller's arguments
    seen = {}
    d = _DenseCache(False)
    k, v = d.update_and_fetch(torch.randn(1, 2, 5, 8), torch.randn(1, 2, 5, 8))
    I.fused_sdpa_dispatch(q, k, v, d, 0.3, "causal", original=lambda *a, **kw: seen.update(kw) or a[0])
    assert seen["cache"] is d and seen["mask"] == "causal" and seen["scale"] == 0.3 and d.calls == []


def test_attention_function_refuses_orphaned_sentinels():
    q = torch.randn(1, 4, 1, 8)
    z = torch.zeros(1, 2, 0, 8)
    with pytest.raises(RuntimeError, match="zero-length keys"):
        I.veloxquant_attention(None, q, z, z, None, scaling=0.3)


def _tiny_llama():
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=100, hidden_size=512, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=128, max_position_embeddings=512, pad_token_id=0, eos_token_id=None)
    return cfg, LlamaForCausalLM(cfg).eval()


def test_transformers_adapter_generates_like_the_dynamic_cache_cpu():
    from transformers.cache_utils import Cache, DynamicCache

    cfg, model = _tiny_llama()
    ids = torch.randint(1, 100, (2, 12))
    am = torch.ones_like(ids)
    with torch.no_grad(), warnings.catch_warnings():
        warnings.simplefilter("ignore")
        ref = model.generate(ids, attention_mask=am, max_new_tokens=6, do_sample=False, past_key_values=DynamicCache(config=cfg))
        Layer = I.make_cache_layer_class()
        I.patch_hf_for_fused_sdpa(model)
        for mb in (False, True):
            fakes = [_DenseCache(mb) for _ in range(2)]
            cache = Cache(layers=[Layer(c) for c in fakes])
            out = model.generate(ids, attention_mask=am, max_new_tokens=6, do_sample=False, past_key_values=cache)
            assert torch.equal(out, ref), f"memory_bound={mb}"
            assert cache.get_seq_length() == 17
            if mb:   # one causal prefill call of 12 rows, then single-row decode calls, in every layer
                assert all(f.calls[0] == (12, True, 0) and set(f.calls[1:]) == {(1, False, 0)} for f in fakes)
            cache.crop(10)
            assert cache.get_seq_length() == 10


@pytest.mark.gpu
@pytest.mark.parametrize("method,memory_bound", [("kivi", False), ("kivi", True), ("rabitq", True), ("kivi_sink", False), ("skvq", False),
                                                 ("kitty", False), ("age_tiered", False), ("turboquant_rvq", False)])
def test_transformers_model_decodes_over_the_compressed_caches(method, memory_bound):
    """A randomly initialised Llama generates with this package's caches through
    ``patch_model_kv_cache`` + ``patch_hf_for_fused_sdpa``; with 8-bit KIVI the logits stay close
    to the uncompressed run, and a fresh cache is built per ``make_cache()`` call."""
    from transformers.cache_utils import DynamicCache

    from veloxquant_mlx_b200.cache import KVCacheConfig

    cfg, model = _tiny_llama()
    model = model.to("cuda:0").half()
    ids = torch.randint(1, 100, (2, 200), device="cuda:0")
    with torch.no_grad(), warnings.catch_warnings():
        warnings.simplefilter("ignore")
        ref = model(ids, past_key_values=DynamicCache(config=cfg), use_cache=True)
        kw = dict(method=method, head_dim=128, fused_sdpa_memory_bound=memory_bound)
        if method in ("kivi", "kivi_sink"):
            kw.update(bit_width_inlier=8, residual_length=32)
        if method == "skvq":
            kw.update(skvq_bits_key=8, skvq_bits_value=8, skvq_window=32)
        if method == "turboquant_rvq":
            kw.update(bit_width_inlier=4)
        if method not in ("kivi", "kivi_sink", "rabitq"):
            kw.pop("fused_sdpa_memory_bound")
        first = I.patch_model_kv_cache(model, KVCacheConfig(**kw))
        I.patch_hf_for_fused_sdpa(model)
        assert model.make_cache() is not first and len(first.layers) == 2
        cache = model.make_cache()
        fused_calls = []
        if memory_bound:   # the packed store must be what is attended over, in every layer
            for layer in cache.layers:
                inner = layer.cache.fused_sdpa
                layer.cache.fused_sdpa = (lambda f: lambda q, *a, **k: (fused_calls.append(q.shape[2]), f(q, *a, **k))[1])(inner)
        out = model(ids, past_key_values=cache, use_cache=True)
        assert cache.get_seq_length() == 200
        assert fused_calls == ([200, 200] if memory_bound else [])
        if method in ("kivi", "kivi_sink", "skvq"):
            assert float((out.logits.float() - ref.logits.float()).abs().max()) < 0.08
        if method == "kivi":
            assert cache.layers[0].cache._n_quantized == 160
        if method == "skvq":
            assert cache.layers[0].cache.quantized_tokens == 192
        if method == "age_tiered":
            assert cache.layers[0].cache.tokens_mid == 2 * 2 * (200 - 128)
        step = model(ids[:, -1:], past_key_values=cache, use_cache=True)
        assert step.logits.shape == (2, 1, 100) and cache.get_seq_length() == 201 and torch.isfinite(step.logits).all()
        assert fused_calls == ([200, 200, 1, 1] if memory_bound else [])
        if method == "rabitq":
            # sign-bit keys are a coarse estimate, but the attention must see the values: the
            # logits follow the uncompressed run far more closely than a run without attention would
            ref_step = ref.logits[:, -1].float()
            got = out.logits[:, -1].float()
            cos = torch.nn.functional.cosine_similarity(got, ref_step, dim=-1)
            assert float(cos.min()) > 0.5, cos
        gen = model.generate(ids[:, :50], attention_mask=torch.ones_like(ids[:, :50]), max_new_tokens=8, do_sample=False,
                             past_key_values=model.make_cache())
        assert gen.shape == (2, 58)


def test_mask_recogniser_agrees_with_the_reference_function_on_every_recorded_mask():
    """237 masks -- all-visible, tail-aligned causal, trailing windows of several widths, boolean /
    additive float32 / float16 / -1e9 / integer forms, every broadcastable shape, and masks with holes,
    per-head differences, shifts, wrong shapes, biases, random patterns -- through the reference's
    ``_memory_bound_mask_parameters`` (``metal/fused_sdpa.py:332-396``, executed over NumPy by
    tests/golden/make_golden.py): the same ``(causal, window)`` or the same refusal for every one."""
    import os

    import numpy as np

    from veloxquant_mlx_b200.integration import _memory_bound_mask_parameters

    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "masks.npz"))
    B, H, KV = (int(x) for x in z["dims"])
    accepted = 0
    for i in range(int(z["n_cases"][0])):
        ok, causal, window, N = (int(x) for x in z[f"r{i}"])
        q = torch.zeros(B, H, N, 8)
        try:
            got = _memory_bound_mask_parameters(torch.from_numpy(z[f"m{i}"]), q, KV)
            res = (1, int(got[0]), int(got[1]))
        except ValueError:
            res = (0, 0, 0)
        assert res == (ok, causal, window), (i, z[f"m{i}"].shape, z[f"m{i}"].dtype)
        accepted += ok
    assert 100 < accepted < 200


def test_hf_cache_is_planned_from_the_model_layer_by_layer():
    """``make_hf_cache(model, config)`` asks ``KVCacheBuilder.for_model``: the head_dim of every layer is
    read from the model's attention modules (not from the configuration's default), seeds follow the layer
    index, an instance-level ``make_cache`` hook installed by an earlier patch is not called back. The
    factory is replaced by a recorder, so this needs no device."""
    from transformers import LlamaConfig, LlamaForCausalLM

    from veloxquant_mlx_b200 import cache as c

    cfg = LlamaConfig(vocab_size=50, hidden_size=128, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=32, max_position_embeddings=64)
    model = LlamaForCausalLM(cfg).eval()
    model.make_cache = lambda: 1 / 0
    seen = []

    class Recorded(c.DenseKVCache):
        def __init__(self, config):
            super().__init__()
            seen.append((config.method, config.head_dim, config.bit_width_inlier, config.seed))

    original = c.KVCacheFactory.create
    c.KVCacheFactory.create = staticmethod(Recorded)
    try:
        hf = I.make_hf_cache(model, c.KVCacheConfig(method="kivi", bit_width_inlier=[2, 4, 8], seed=5))
        by_count = I.make_hf_cache(2, c.KVCacheConfig(method="kivi", head_dim=64, seed=1))
    finally:
        c.KVCacheFactory.create = staticmethod(original)
    assert seen == [("kivi", 32, 2, 5), ("kivi", 32, 4, 6), ("kivi", 32, 8, 7), ("kivi", 64, 2, 1), ("kivi", 64, 2, 2)]
    assert len(hf.layers) == 3 and len(by_count.layers) == 2 and hf.get_seq_length() == 0
    # the adapter drives any cache of the list through the same calls: a prefill and a step on the stand-ins
    ids = torch.randint(1, 50, (1, 9))
    with torch.no_grad(), warnings.catch_warnings():
        warnings.simplefilter("ignore")
        out = model(ids, past_key_values=hf, use_cache=True)
        model(ids[:, -1:], past_key_values=hf, use_cache=True)
    assert hf.get_seq_length() == 10 and torch.isfinite(out.logits).all()
