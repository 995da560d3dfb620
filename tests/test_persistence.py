"""Persistence format and prefix-cache reuse (reference: ``state`` / ``meta_state`` of
``cache/vecinfer_cache.py:542-609`` and ``cache/turboquant_rvq_cache.py:380-425``,
``integration/prefix_cache.py``). The LRU logic runs on CPU with a stand-in cache; the file
round trip and the reuse of real caches need the GPU."""

from __future__ import annotations

import copy
import math
import warnings

import pytest
import torch

from veloxquant_mlx_b200.persistence import PrefixCache, load_prompt_cache, save_prompt_cache


class _Toy:
    """Stand-in cache: remembers how many tokens it holds."""

    def __init__(self, n=0):
        self.n = n

    def trim(self, k):
        k = min(k, self.n)
        self.n -= k
        return k

    def is_trimmable(self):
        return True

    @property
    def nbytes(self):
        return 10 * self.n


def _toy_prefix_cache(**kw):
    return PrefixCache(None, 2, factory=lambda: [_Toy(), _Toy()], cloner=lambda cs: [copy.copy(c) for c in cs], **kw)


def test_prefix_cache_miss_hit_extend_and_trim():
    pc = _toy_prefix_cache()
    caches, rest = pc.fetch([1, 2, 3, 4])
    assert [c.n for c in caches] == [0, 0] and rest == [1, 2, 3, 4] and pc.misses == 1
    pc.insert([1, 2, 3, 4, 5, 6], [_Toy(6), _Toy(6)])
    # a prompt that extends the stored sequence: everything stored is reused
    caches, rest = pc.fetch([1, 2, 3, 4, 5, 6, 7, 8])
    assert [c.n for c in caches] == [6, 6] and rest == [7, 8] and pc.hits == 1
    # a prompt that diverges after 3 tokens: the copy is cut back to the shared prefix
    caches, rest = pc.fetch([1, 2, 3, 9, 9])
    assert [c.n for c in caches] == [3, 3] and rest == [9, 9]
    # the same sequence again: at least the last token is left for the model
    caches, rest = pc.fetch([1, 2, 3, 4, 5, 6])
    assert [c.n for c in caches] == [5, 5] and rest == [6]
    # snapshots are copies: what fetch hands out never changes the stored entry
    caches[0].trim(5)
    assert pc.fetch([1, 2, 3, 4, 5, 6, 7])[0][0].n == 6
    # other model key: nothing shared
    assert pc.fetch([1, 2, 3], model_key="other")[1] == [1, 2, 3]


def test_prefix_cache_lru_eviction_by_count_and_bytes():
    pc = _toy_prefix_cache(max_size=2)
    pc.insert([1, 1], [_Toy(2), _Toy(2)])
    pc.insert([2, 2], [_Toy(2), _Toy(2)])
    pc.fetch([1, 1, 5])                       # touches the first entry
    pc.insert([3, 3], [_Toy(2), _Toy(2)])     # evicts the least recently used: [2, 2]
    assert len(pc) == 2 and pc.fetch([2, 2, 5])[1] == [2, 2, 5] and pc.fetch([1, 1, 5])[1] == [5]
    pc = _toy_prefix_cache(max_bytes=100)
    pc.insert([1] * 4, [_Toy(4), _Toy(4)])    # 80 bytes
    pc.insert([2] * 4, [_Toy(4), _Toy(4)])    # 160 bytes in all: the older entry goes
    assert len(pc) == 1 and pc.nbytes == 80


@pytest.mark.gpu
@pytest.mark.parametrize("method", ["kivi", "vecinfer", "rabitq"])
def test_file_round_trip_restores_an_identical_cache(method, tmp_path):
    from veloxquant_mlx_b200.cache import KVCacheConfig, KVCacheFactory

    dev, D, L = "cuda:0", 128, 3
    kw = dict(method=method, head_dim=D)
    if method == "kivi":
        kw.update(bit_width_inlier=2, residual_length=64, fused_sdpa_memory_bound=True)
    if method == "vecinfer":
        kw.update(key_sub_dim=8, value_sub_dim=8, key_codebook_bits=8, value_codebook_bits=8, fused_sdpa=True,
                  fused_sdpa_memory_bound=True)
    cfg = KVCacheConfig(**kw)
    g = torch.Generator(device=dev).manual_seed(1)
    kv = torch.randn((2, L, 2, 2, 333, D), generator=g, device=dev, dtype=torch.float16)
    q = torch.randn((2, 8, 1, D), generator=g, device=dev, dtype=torch.float16)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        caches = [KVCacheFactory.create(cfg) for _ in range(L)]
        for l, c in enumerate(caches):
            c.update_and_fetch(kv[0, l, :, :, :300], kv[1, l, :, :, :300])
        path = str(tmp_path / "prompt.safetensors")
        save_prompt_cache(path, caches, metadata={"model": "toy", "tokens": 300})
        loaded, meta = load_prompt_cache(path, cfg, device=dev, return_metadata=True)
    assert meta == {"model": "toy", "tokens": 300} and len(loaded) == L
    scale = 1.0 / math.sqrt(D)
    for l, (a, b) in enumerate(zip(caches, loaded)):
        assert b.offset == a.offset == 300 and b.meta_state == a.meta_state and b.nbytes == a.nbytes
        for x, y in zip(a.state, b.state):
            assert (x is None and y is None) or torch.equal(x, y)
        assert torch.equal(a.fused_sdpa(q, scale), b.fused_sdpa(q, scale))
        # decoding on after the restore is the same as never having stopped
        for t in range(300, 333):
            a.update_and_fetch(kv[0, l, :, :, t : t + 1], kv[1, l, :, :, t : t + 1])
            b.update_and_fetch(kv[0, l, :, :, t : t + 1], kv[1, l, :, :, t : t + 1])
        assert torch.equal(a.fused_sdpa(q, scale), b.fused_sdpa(q, scale))
    with pytest.raises(ValueError, match="saved by method"):
        load_prompt_cache(path, KVCacheConfig(method="rabitq" if method != "rabitq" else "kivi", head_dim=D), device=dev)


@pytest.mark.gpu
def test_empty_caches_round_trip(tmp_path):
    from veloxquant_mlx_b200.cache import KVCacheConfig, KVCacheFactory

    cfg = KVCacheConfig(method="kivi", head_dim=128)
    path = str(tmp_path / "empty.safetensors")
    save_prompt_cache(path, [KVCacheFactory.create(cfg) for _ in range(2)])
    loaded = load_prompt_cache(path, cfg, device="cuda:0")
    assert [c.offset for c in loaded] == [0, 0] and all(c.empty() for c in loaded)


@pytest.mark.gpu
def test_prefix_reuse_with_kivi_caches_equals_a_fresh_prefill():
    """A stored 200-token entry serves a prompt that shares its first 150 tokens: the copy is
    trimmed (KIVI re-opens the partly trimmed group) and fed the rest; the result must equal a
    cache that saw the new prompt from scratch, bit for bit in its packed store."""
    from veloxquant_mlx_b200.cache import KVCacheConfig, KVCacheFactory

    dev, D = "cuda:0", 128
    cfg = KVCacheConfig(method="kivi", head_dim=D, bit_width_inlier=4, residual_length=32, fused_sdpa_memory_bound=True)
    g = torch.Generator(device=dev).manual_seed(2)
    # "token embeddings": K/V rows are a function of (position, token id) only, as in a model's first layer
    table = torch.randn((2, 50, 1, 2, 1, D), generator=g, device=dev, dtype=torch.float16)

    def feed(cache, tokens):
        for t in tokens:
            cache.update_and_fetch(table[0, t], table[1, t])

    stored = list(range(40)) * 5            # 200 tokens
    new = stored[:150] + [41, 42, 43, 44] * 10
    pc = PrefixCache(cfg, 1)
    caches, rest = pc.fetch(stored)
    assert rest == stored
    feed(caches[0], stored)
    pc.insert(stored, caches)
    got, rest = pc.fetch(new)
    assert rest == new[150:] and got[0].offset == 150
    feed(got[0], rest)
    want = KVCacheFactory.create(cfg)
    feed(want, new)
    assert got[0].offset == want.offset and got[0]._n_quantized == want._n_quantized
    q = torch.randn((1, 8, 1, D), generator=g, device=dev, dtype=torch.float16)
    # rows of the re-opened group were rounded once before they were quantized again (the
    # reference's trim rule), so the two stores agree except in that group
    lo = (150 // 32) * 32
    assert torch.equal(got[0]._k_codes[:, :, :lo], want._k_codes[:, :, :lo])
    out_a, out_b = got[0].fused_sdpa(q, 0.088).float(), want.fused_sdpa(q, 0.088).float()
    assert float((out_a - out_b).abs().max()) < 2e-2
    # the stored entry is untouched and still serves its own continuation
    again, rest = pc.fetch(stored + [7])
    assert rest == [7] and again[0].offset == 200
