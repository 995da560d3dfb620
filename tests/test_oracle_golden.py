"""The oracle against fixtures produced by executing the reference's own code
(``tests/golden/make_golden.py``) and against the reference's known answers."""

from __future__ import annotations

import math
import os

import numpy as np
import pytest

from oracle import bitpack, kivi, rabitq, vq

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name):
    return np.load(os.path.join(GOLDEN, name))


# ----------------------------------------------------------------- bit packing
def test_bitpack_known_answer():
    # reference: tests/metal/test_worker_kernel_parity.py:18-30
    got = bitpack.pack(np.array([0, 1, 2, 3, 0, 1, 2, 3], dtype=np.uint8), 2)
    assert got.tolist() == [228, 228]
    assert _load("bitpack.npz")["known_answer_2bit"].tolist() == [228, 228]


@pytest.mark.parametrize("b", [1, 2, 3, 4])
@pytest.mark.parametrize("n", [8, 13, 64, 257])
def test_bitpack_matches_reference_module(b, n):
    z = _load("bitpack.npz")
    vals, packed = z[f"b{b}_n{n}_vals"], z[f"b{b}_n{n}_packed"]
    np.testing.assert_array_equal(bitpack.pack(vals, b), packed)
    np.testing.assert_array_equal(bitpack.unpack(packed, b, n), vals)


@pytest.mark.parametrize("b", range(1, 9))
def test_bitpack_roundtrip_any_width(b):
    rng = np.random.default_rng(b)
    vals = rng.integers(0, 1 << b, (3, 5, 77), dtype=np.uint8)
    np.testing.assert_array_equal(bitpack.unpack(bitpack.pack(vals, b), b, 77), vals)


# ------------------------------------------------------------------------ KIVI
def _kivi_cases():
    z = _load("kivi.npz")
    return [str(n) for n in z["names"]]


@pytest.mark.parametrize("name", _kivi_cases())
def test_kivi_quant_bit_exact_with_reference_numpy(name):
    z = _load("kivi.npz")
    B, H, S_kv, D, b, g, seed, H_kv = [int(v) for v in z[f"{name}_meta"]]
    H_kv = H if H_kv < 0 else H_kv
    # regenerate the inputs exactly as the reference's _make_inputs does
    rng = np.random.default_rng(seed)
    levels = (1 << b) - 1
    q = rng.standard_normal((B, H, 1, D)).astype(np.float16)
    kf = rng.standard_normal((B, H_kv, S_kv, D)).astype(np.float32)
    vf = rng.standard_normal((B, H_kv, S_kv, D)).astype(np.float32)
    np.testing.assert_array_equal(q, z[f"{name}_q"])
    kc, ks, kz = kivi.quant_keys(kf, g, levels)
    vc, vs, vz = kivi.quant_values(vf, g, levels)
    for got, key in [(kc, "kc"), (ks, "ks"), (kz, "kz"), (vc, "vc"), (vs, "vs"), (vz, "vz")]:
        want = z[f"{name}_{key}"]
        assert got.dtype == want.dtype and got.shape == want.shape
        np.testing.assert_array_equal(got, want)
    out = kivi.reference_attend(q, kc, ks, kz, vc, vs, vz, g, 1.0 / math.sqrt(D))
    np.testing.assert_allclose(out, z[f"{name}_out"], rtol=0, atol=1e-6)


def test_kivi_special_values():
    z = _load("kivi.npz")
    const = np.full((1, 1, 32, 8), 3.5, dtype=np.float32)
    c, s, zz = kivi.quant_keys(const, 32, 3)
    np.testing.assert_array_equal(c, z["const_kc"])
    np.testing.assert_array_equal(s, z["const_ks"])
    np.testing.assert_array_equal(zz, z["const_kz"])
    assert np.all(s == np.float32(1e-8)) and np.all(c == 0)
    c, s, zz = kivi.quant_values(z["halfeven_in"], 32, 2)
    np.testing.assert_array_equal(c, z["halfeven_vc"])
    # 1/1.5 -> 0.667 -> 1 ; 2/1.5 -> 1.33 -> 1 ; exact halves round to even
    assert set(np.unique(c)) <= {0, 1, 2}


def test_kivi_group_of_one_is_lossless():
    # reference: tests/metal/test_kivi_quant.py:151-159
    rng = np.random.default_rng(5)
    x = rng.standard_normal((1, 2, 9, 16)).astype(np.float16)
    np.testing.assert_array_equal(kivi.quant_dequant_along(x, -1, 1, 3), x)
    np.testing.assert_array_equal(kivi.quant_dequant_along(x, -2, 1, 3), x)


def test_kivi_pack_codes_layout():
    codes = np.arange(16, dtype=np.uint8).reshape(1, 16) % 4
    packed = kivi.pack_codes(codes, 2)
    assert packed.shape == (1, 4)
    assert packed[0, 0] == (0 | 1 << 2 | 2 << 4 | 3 << 6)
    assert kivi.storage_bits(3) == 4 and kivi.storage_bits(5) == 8


def test_kivi_boundary_rule():
    # reference: cache/kivi_cache.py:206-225 ; tests/cache/test_kivi_cache.py:187-199
    assert kivi.quantization_boundary(100, 128, 32) == 0
    assert kivi.quantization_boundary(128 + 31, 128, 32) == 0
    assert kivi.quantization_boundary(128 + 32, 128, 32) == 32
    assert kivi.quantization_boundary(4096, 128, 32) == 3968


# ---------------------------------------------------------------------- RaBitQ
@pytest.mark.parametrize("N,D", [(1, 8), (33, 64), (64, 128), (17, 256)])
def test_rabitq_encode_matches_reference_numpy(N, D):
    z = _load("rabitq.npz")
    tag = f"enc_N{N}_D{D}"
    bits, mag, _ = rabitq.encode_hadamard(z[f"{tag}_keys"], z[f"{tag}_diag"])
    np.testing.assert_array_equal(bits, z[f"{tag}_bits"])
    np.testing.assert_allclose(mag, z[f"{tag}_mag"], rtol=1e-6)


@pytest.mark.parametrize("tag", ["att_B1_H1_Sq1_S33_D64", "att_B2_H2_Sq1_S256_D128", "att_B1_H2_Sq4_S64_D256"])
def test_rabitq_attend_matches_reference_numpy(tag):
    z = _load("rabitq.npz")
    g = lambda k: z[f"{tag}_{k}"]  # noqa: E731
    out = rabitq.reference_attend(g("q"), g("q_scale"), g("k_bits"), g("k_mag"), g("k_const"),
                                  g("v_idx"), g("v_cents"))
    np.testing.assert_allclose(out, g("out"), rtol=1e-5, atol=1e-6)
    np.testing.assert_array_equal(bitpack.pack_nibbles(g("v_idx")), g("v_packed"))


def test_rabitq_signs_and_rotation_match_reference_modules():
    z = _load("rabitq.npz")
    np.testing.assert_array_equal(rabitq.pack_signs(z["signs_in"]), z["signs_out"])
    for d, seed in [(64, 42), (128, 42), (128, 7)]:
        np.testing.assert_array_equal(rabitq.make_hadamard_diagonal(d, seed), z[f"diag_d{d}_s{seed}"])
    np.testing.assert_array_equal(rabitq.make_rotation_matrix(24, 42), z["rot_d24_s42"])
    np.testing.assert_array_equal(rabitq.make_rotation_matrix(128, 42).astype(np.float32), z["rot_d128_s42"])


def test_rabitq_hamming_score():
    rng = np.random.default_rng(0)
    bits = rng.integers(0, 256, (9, 16), dtype=np.uint8)
    qb = rng.integers(0, 256, 16, dtype=np.uint8)
    cx = rng.standard_normal(9).astype(np.float32)
    s = rabitq.hamming_score(qb, bits, 0.25, cx)
    want = np.array([bin(int.from_bytes(bytes(a ^ b for a, b in zip(row, qb)), "little")).count("1")
                     for row in bits], dtype=np.float32) * np.float32(0.25) + cx
    np.testing.assert_array_equal(s, want)


# -------------------------------------------------------------------- VecInfer
@pytest.mark.parametrize("d", [1, 2, 8, 128])
def test_vq_wht_matches_reference_function(d):
    np.testing.assert_array_equal(vq.walsh_hadamard_matrix(d), _load("vq.npz")[f"wht_{d}"])


def test_vq_quantize_sequential_order_and_ties():
    cb = np.array([[0, 0], [1, 1], [1, 1], [2, 2]], dtype=np.float32)
    x = np.array([[1, 1, 0.5, 0.5, 9, 9]], dtype=np.float32)
    idx = vq.quantize_vq(x, cb, 2)
    assert idx.dtype == np.int32
    # exact hit -> first of the duplicated centroids; midpoint tie -> lowest index
    assert idx.tolist() == [[1, 0, 3]]
    rng = np.random.default_rng(3)
    x = rng.standard_normal((4, 50, 64)).astype(np.float16)
    cb = rng.standard_normal((256, 8)).astype(np.float16)
    idx = vq.quantize_vq(x, cb, 8)
    # brute-force python loop on a few entries, same canonical order
    xf, cf = x.astype(np.float32), cb.astype(np.float32)
    for (a, b, j) in [(0, 0, 0), (3, 49, 7), (2, 17, 3)]:
        best, bi = np.float32(np.inf), 0
        for c in range(256):
            dist = np.float32(0)
            for i in range(8):
                d = np.float32(xf[a, b, j * 8 + i] - cf[c, i])
                dist = np.float32(dist + np.float32(d * d))
            if dist < best:
                best, bi = dist, c
        assert idx[a, b, j] == bi


def test_vq_lut_equals_explicit_dot_and_dual_transform_invariance():
    # reference: tests/allocators/test_vecinfer.py:133-153 and :35-54
    rng = np.random.default_rng(1)
    D, sub = 64, 8
    cb = rng.standard_normal((16, sub)).astype(np.float32)
    q = rng.standard_normal((2, 3, D)).astype(np.float32)
    idx = rng.integers(0, 16, (5, D // sub))
    lut = vq.compute_query_lut(q, cb, sub)
    k_hat = vq.dequantize_vq(idx, cb)
    want = np.einsum("abd,sd->abs", q, k_hat)
    got = lut[:, :, np.arange(D // sub), idx].sum(-1)  # [2,3,5]
    np.testing.assert_allclose(got, want, rtol=1e-4, atol=1e-4)
    H = vq.walsh_hadamard_matrix(D)
    np.testing.assert_allclose(H @ H.T, np.eye(D), atol=1e-5)
    lam = rng.uniform(0.5, 2.0, (4, D)).astype(np.float32)
    K = rng.standard_normal((1, 4, 7, D)).astype(np.float32)
    Q = rng.standard_normal((1, 8, 1, D)).astype(np.float32)  # GQA 2:1
    Kt = vq.apply_dual_transform_keys(K, lam, H)
    Qt = vq.apply_dual_transform_queries(Q, lam, H)
    s0 = np.einsum("bhqd,bhsd->bhqs", Q, np.repeat(K, 2, axis=1))
    s1 = np.einsum("bhqd,bhsd->bhqs", Qt, np.repeat(Kt, 2, axis=1))
    np.testing.assert_allclose(s0, s1, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("tag", ["pre_B1_H1_Sq8_S33_D64_c0", "pre_B2_H2_Sq33_S200_D128_c0", "pre_B1_H2_Sq40_S40_D128_c1",
                                 "pre_B2_H1_Sq5_S77_D64_c1"])
def test_rabitq_prefill_matches_reference_numpy(tag):
    """``oracle.rabitq.reference_prefill`` against the outputs of the reference's own
    ``_reference_prefill`` (tests/metal/test_rabitq_prefill.py), executed by make_golden.py."""
    z = _load("rabitq.npz")
    g = lambda n: z[f"{tag}_{n}"]  # noqa: E731
    out = rabitq.reference_prefill(g("q"), float(g("scale")[0]), g("k_bits"), g("k_mag"), g("k_const"), g("v_idx"), g("v_cents"),
                                   causal=tag.endswith("c1"))
    np.testing.assert_allclose(out, g("out"), rtol=0, atol=1e-6)
    assert np.array_equal(bitpack.pack(g("v_idx"), 4), g("v_packed"))


@pytest.mark.parametrize("tag", list("abcde"))
def test_skvq_oracle_matches_the_reference_module_run_over_numpy(tag):
    """``oracle.skvq`` against ``quantizers/skvq.py`` executed whole with NumPy standing in for
    ``mlx.core`` (make_golden.py): codes, lo, scale with and without the clip search, the channel
    permutation and the permuted round trip, bit for bit."""
    from oracle import skvq

    z = _load("skvq.npz")
    x = z[f"{tag}_x"]
    bits, gs = (int(v) for v in z[f"{tag}_meta"])
    assert tuple(z["alpha_grid"]) == skvq.DEFAULT_ALPHA_GRID
    for suffix, alphas in (("", skvq.DEFAULT_ALPHA_GRID), ("_a90", (0.9,))):
        codes, lo, scale = skvq.clipped_group_quant(x, bits, gs, alphas)
        assert np.array_equal(codes, z[f"{tag}_codes{suffix}"])
        assert np.array_equal(lo, z[f"{tag}_lo{suffix}"]) and np.array_equal(scale, z[f"{tag}_scale{suffix}"])
    perm = skvq.channel_permutation(x)
    assert np.array_equal(perm, z[f"{tag}_perm"]) and np.array_equal(skvq.invert_permutation(perm), z[f"{tag}_inv"])
    rt = skvq.skvq_round_trip(x, perm, bits, gs)
    assert rt.dtype == x.dtype and np.array_equal(rt, z[f"{tag}_rt"])
    assert [skvq.skvq_compressed_bytes(123, 128, 4, 32), skvq.skvq_compressed_bytes(11, 64, 3, 16),
            skvq.skvq_fp16_bytes(77, 128)] == [int(v) for v in z["bytes"]]


def test_skvq_oracle_properties_of_the_reference_tests():
    """alpha = 1 is plain min/max quantization up to one step on isolated boundary elements; the
    searched clip factor is never worse per group (quantizers test_skvq.py:100-138)."""
    from oracle import skvq

    rng = np.random.default_rng(6)
    x = rng.standard_normal((128, 32)).astype(np.float32)
    x[rng.random((128, 32)) < 0.03] *= 20.0
    codes, lo, scale = skvq.clipped_group_quant(x, 2, 8, (1.0,))
    xg = x.reshape(128, 4, 8)
    gmin, gmax = xg.min(-1, keepdims=True), xg.max(-1, keepdims=True)
    ref_scale = np.maximum((gmax - gmin) / 3.0, 1e-8)
    ref_codes = np.clip(np.round((xg - gmin) / ref_scale), 0, 3)
    got = codes.astype(np.float64).reshape(128, 4, 8)
    assert np.mean(got == ref_codes) > 0.999 and np.max(np.abs(got - ref_codes)) <= 1.0

    def per_group_mse(alphas):
        c, lo, sc = skvq.clipped_group_quant(x, 2, 8, alphas)
        r = skvq.clipped_group_dequant(c, lo, sc, 8, 32)
        return ((r - x) ** 2).reshape(128, 4, 8).mean(-1)

    assert np.all(per_group_mse(skvq.DEFAULT_ALPHA_GRID) <= per_group_mse((1.0,)) + 1e-9)


def test_group_quant_core_kitty_and_age_tiered_oracles_match_the_reference_modules_run_over_numpy():
    """``oracle.kivi.quant_keys`` / ``dequant_keys`` against ``quantizers/_quant_utils.py``, and
    ``oracle.kitty`` / ``oracle.age_tiered`` against ``quantizers/kitty.py`` / ``age_tiered.py``, all
    executed whole with NumPy standing in for ``mlx.core`` (make_golden.py), bit for bit."""
    from oracle import age_tiered, kitty

    z = _load("group_quant.npz")
    for tag in "abcd":
        x = z[f"gq_{tag}_x"]
        b, gs = (int(v) for v in z[f"gq_{tag}_meta"])
        N, S, D = x.shape
        ng = -(-S // gs)
        c, s, zz = kivi.quant_keys(x.astype(np.float32)[None], gs, (1 << b) - 1)
        assert np.array_equal(c[0].astype(np.float32), z[f"gq_{tag}_codes"].reshape(N, ng * gs, D)[:, :S])
        assert np.array_equal(s[0].reshape(N, ng, 1, D), z[f"gq_{tag}_scale"])
        assert np.array_equal(zz[0].reshape(N, ng, 1, D), z[f"gq_{tag}_zero"])
        assert np.array_equal(kitty.group_quant_dequant_batched(x, b, gs), z[f"gq_{tag}_rt"])
    mask = kitty.hi_mask_from_variance_batched(z["kitty_var"], 0.25)
    assert np.array_equal(mask, z["kitty_mask"]) and int(mask.sum(1)[0]) == 16
    assert np.array_equal(kitty.quantize_mixed_channels_batched(z["kitty_x"], mask), z["kitty_out"])
    kx = z["kitty_x"].astype(np.float32)
    assert np.array_equal(kitty.compute_running_variance(kx.sum(1)[0], (kx ** 2).sum(1)[0], 96), z["kitty_running_var"])
    assert np.array_equal(age_tiered.assign_age_tiers([200 - (i + 1) for i in range(200)], 40, 120), z["age_tok_tier"])
    assert np.array_equal(age_tiered.age_tier_quantize_batched(z["age_x"], list(z["age_group_tier"]), (8, 4, 2), 32), z["age_out"])
    assert [age_tiered.age_tiered_bytes({0: 40, 1: 80, 2: 80}, (8, 4, 2), 32), age_tiered.full_fp16_bytes(200, 32)] == list(z["age_bytes"])


def _replay(tag, model, z, trimmable, counters):
    """Feed the recorded call script to an oracle cache model and compare what it returns, and its
    counters, with what the reference's cache CLASS returned when make_golden.py executed it over the
    NumPy stand-ins (``mlx.core`` answered by NumPy, a minimal container for its ``mlx_lm`` base class)."""
    k, v = z["k"], z["v"]
    checked = 0
    for i, (op, a, b) in enumerate(z["script"].tolist()):
        if op == 1:
            if trimmable:
                assert model.trim(a) == a
            continue
        ko, vo = model.update_and_fetch(k[:, :, a:b], v[:, :, a:b])
        if f"{tag}_k_{i}" in z:
            assert np.array_equal(ko, z[f"{tag}_k_{i}"]), (tag, i)
            assert np.array_equal(vo, z[f"{tag}_v_{i}"]), (tag, i)
            got = [int(c(model)) for c in counters]
            assert got == z[f"{tag}_c_{i}"].tolist()[: len(got)], (tag, i, got, z[f"{tag}_c_{i}"].tolist())
            checked += 1
    assert checked >= 10
    return model


def test_cache_policies_match_the_reference_classes_run_over_numpy():
    """KIVI (residual window, group-aligned frontier, trim), sink-protected KIVI, SKVQ, Kitty and
    AgeTieredKV: the oracle's cache models against traces of the reference's own classes
    (``cache/kivi_cache.py``, ``sink_cache.py``, ``skvq_cache.py``, ``kitty_cache.py``,
    ``age_tiered_cache.py``) executed unmodified: returned keys / values bit for bit at every
    recorded call (a prefill, single tokens, a block, a trim, more tokens), frontier and byte counters."""
    from oracle import age_tiered, kitty, kivi_sink, skvq

    z = _load("cache_traces.npz")
    _replay("kivi", kivi_sink.SinkProtectedOracle(32, 2, group=8, residual_length=16, n_sink=0), z, True,
            [lambda m: m.offset, lambda m: m.n_quantized])
    s = _replay("sink", kivi_sink.SinkProtectedOracle(32, 2, group=8, residual_length=16, n_sink=2), z, True,
                [lambda m: m.offset, lambda m: m.n_quantized])
    assert [s.sink_positions_for(0), s.sink_positions_for(1)] == z["sink_positions"].tolist()
    m = _replay("skvq", skvq.SKVQCacheModel(32, bits_k=2, bits_v=3, group_size=8, window=16, n_sink=3), z, False,
                [lambda m: m.offset, lambda m: m.q_end, lambda m: m.compressed_key_bytes, lambda m: m.compressed_value_bytes])
    assert np.array_equal(m.perm_k, z["skvq_perm_k"]) and np.array_equal(m.perm_v, z["skvq_perm_v"])
    _replay("kitty", kitty.KittyCacheModel(32, 0.25, 4, 2, 8), z, True,
            [lambda m: m.keys.shape[2], lambda m: m.n_keys, lambda m: m.compressed_key_bytes, lambda m: m.fp16_key_bytes,
             lambda m: m.value_fp16_bytes])
    _replay("age", age_tiered.AgeTieredCacheModel(32, 20, 50, (8, 4, 2), 8), z, False,
            [lambda m: m.raw_k.shape[1], lambda m: m.age_tiered_bytes, lambda m: m.full_seq_bytes])


@pytest.mark.parametrize("tag,sub", [("s2", 2), ("s4", 4), ("s4big", 4), ("s8", 8)])
def test_quantize_vq_oracle_matches_the_reference_function_run_over_numpy(tag, sub):
    """``oracle.vq.quantize_vq`` / ``dequantize_vq`` against ``allocators/vecinfer.py:281-335`` executed
    with NumPy answering ``mx`` (make_golden.py). Below 8 elements NumPy sums a row in order, the
    order of the reference's Metal kernel and of the oracle: bit for bit. At sub_dim 8 NumPy sums as
    a tree; the indices still agree on these vectors (a difference could only be a near-tie)."""
    z = _load("vq.npz")
    x, cb, idx = z[f"q_{tag}_x"], z[f"q_{tag}_cb"], z[f"q_{tag}_idx"]
    got = vq.quantize_vq(x, cb, sub)
    assert got.dtype == idx.dtype == np.int32 and np.array_equal(got, idx)
    assert int(idx.reshape(-1)[5]) == 3                      # the duplicated centroid: lower index wins
    assert np.array_equal(vq.dequantize_vq(idx, cb), z[f"q_{tag}_deq"])


@pytest.mark.parametrize("tag", list("abcde"))
def test_vq_reference_sdpa_matches_the_reference_function_run_over_numpy(tag):
    """``oracle.vq.reference_sdpa`` (attention in the transformed space: dual-transformed queries
    against dequantized key codes) against the reference's ``_reference_sdpa``
    (tests/cache/test_vecinfer_fused_sdpa.py:69-115: dequantize, rotate back, smooth, masked softmax in
    the original space), executed with NumPy answering ``mx``: causal, tail-aligned multi-row,
    trailing window, grouped heads, per-head / shared / no smooth factors. Equal to 2e-6."""
    z = _load("vq.npz")
    g = lambda n: z[f"sdpa_{tag}_{n}"]  # noqa: E731
    smooth = z[f"sdpa_{tag}_smooth"] if f"sdpa_{tag}_smooth" in z else np.ones(64, np.float32)
    causal, window = (int(x) for x in g("flags"))
    q_t = vq.apply_dual_transform_queries(g("q").astype(np.float32), smooth, vq.walsh_hadamard_matrix(64))
    out = vq.reference_sdpa(q_t, g("k_idx"), g("cb_k"), g("v_idx"), 0.125, v_codebook=g("cb_v"), causal=bool(causal),
                            sliding_window=window)
    np.testing.assert_allclose(out, g("out"), rtol=0, atol=2e-6)


def _rvq_midpoints(centroids64):
    """Voronoi boundaries as the reference's ``ScalarCodebook`` holds them: midpoints of the float32
    centroids, rounded to float16 (``codebooks/scalar_codebook.py:57-60``)."""
    c = np.asarray(centroids64).astype(np.float32)
    return ((c[:-1] + c[1:]) / np.float32(2.0)).astype(np.float16)


def test_rvq_oracle_matches_the_reference_quantizer_run_over_numpy():
    """``rvq_reference.npz``: ``TurboQuantRVQ.encode`` / ``decode`` executed unmodified over the NumPy
    stand-in. From the reference's rotated input both index streams are reproduced bit for bit, and so
    are the rotation and the decoded vectors (the stand-in's Hadamard butterfly is this oracle's)."""
    from oracle import rvq

    z = np.load(os.path.join(GOLDEN, "rvq_reference.npz"))
    codebooks = np.load(os.path.join(GOLDEN, "rvq.npz"))
    for d, b in z["quantizer_cases"]:
        t = f"q_d{d}_b{b}_"
        c1, b1, c2, b2, diag = (z[t + k] for k in ("c1", "b1", "c2", "b2", "diag"))
        # the tables the quantizer built are the float16 roundings of the pinned Lloyd-Max codebooks
        np.testing.assert_array_equal(c1, codebooks[f"gauss_b{b}_d{d}"].astype(np.float16))
        np.testing.assert_array_equal(c2, codebooks[f"laplace_b{b}_d{d}"].astype(np.float16))
        np.testing.assert_array_equal(b1, _rvq_midpoints(codebooks[f"gauss_b{b}_d{d}"]))
        np.testing.assert_array_equal(b2, _rvq_midpoints(codebooks[f"laplace_b{b}_d{d}"]))
        np.testing.assert_array_equal(diag, rabitq.make_hadamard_diagonal(int(d), 3))
        i1, i2, w1, w2 = rvq.rvq_quant_pack(z[t + "rotated"], c1, b1, b2, int(b))
        np.testing.assert_array_equal(i1, z[t + "idx1"])
        np.testing.assert_array_equal(i2, z[t + "idx2"])
        assert len(np.unique(i2)) == 2 ** b                    # the residual stage is exercised
        np.testing.assert_array_equal(rvq.rotate(z[t + "x"], diag), z[t + "rotated"])
        got = rvq.rvq_unpack_decode(w1, w2, np.ones(len(i1), np.float32), c1, c2, diag, int(b), int(d))
        np.testing.assert_array_equal(got, z[t + "decoded"])


def test_rvq_cache_model_matches_the_reference_class_run_over_numpy():
    """The reference's ``TurboQuantRVQKVCache`` over a call script (prefill, single tokens, a block, a
    trim, more tokens; one key with a norm past 65504 and one zero key): returned keys and values,
    offsets, buffer growth and byte counters, then the stored state."""
    from oracle import rvq

    z = np.load(os.path.join(GOLDEN, "rvq_reference.npz"))
    codebooks = np.load(os.path.join(GOLDEN, "rvq.npz"))
    B, H, D, T, bits, seed = (int(x) for x in z["cache_dims"])
    c1 = codebooks[f"gauss_b{bits}_d{D}"].astype(np.float16)
    c2 = codebooks[f"laplace_b{bits}_d{D}"].astype(np.float16)
    m = rvq.RVQCacheModel(D, bits, rabitq.make_hadamard_diagonal(D, seed), c1, _rvq_midpoints(codebooks[f"gauss_b{bits}_d{D}"]),
                          c2, _rvq_midpoints(codebooks[f"laplace_b{bits}_d{D}"]))
    k, v = z["cache_k"], z["cache_v"]
    checked = 0
    for i, (op, a, b) in enumerate(z["cache_script"]):
        if op == 1:
            assert m.trim(int(a)) == a
            continue
        ko, vo = m.update_and_fetch(k[:, :, a:b], v[:, :, a:b])
        if f"cache_k_{i}" in z.files:
            np.testing.assert_array_equal(ko, z[f"cache_k_{i}"])
            np.testing.assert_array_equal(vo, z[f"cache_v_{i}"])
            assert [m.offset, m.p1.shape[2], m.compressed_key_bytes, m.fp16_key_bytes, m.nbytes] == list(z[f"cache_c_{i}"])
            checked += 1
    assert checked >= 5 and np.isfinite(ko.astype(np.float32)).all()
    n = m.offset
    np.testing.assert_array_equal(m.p1[:, :, :n], z["cache_state_p1"])
    np.testing.assert_array_equal(m.p2[:, :, :n], z["cache_state_p2"])
    np.testing.assert_array_equal(m.norms[:, :, :n], z["cache_state_norms"])
    assert float(z["cache_state_norms"].max()) > 65504.0 and float(z["cache_state_norms"].min()) == 0.0
    assert list(z["cache_meta_state"]) == [D, bits, seed, n]


def test_kivi_oracle_matches_the_reference_quantizer_class_run_over_numpy():
    """``kivi_quantizer.npz``: the reference's ``KIVIQuantizer`` (``quantizers/kivi.py:103-196``) executed
    unmodified over the NumPy stand-in, both grouping axes, ragged last groups, one-value groups: codes,
    scales, zero points and the float16 reconstruction, bit for bit."""
    z = np.load(os.path.join(GOLDEN, "kivi_quantizer.npz"))
    assert len(z["cases"]) == 12
    for axis, n, d, b, g in z["cases"].tolist():
        t = f"{'token' if axis else 'channel'}_n{n}_d{d}_b{b}_g{g}_"
        x = z[t + "x"][None, None]
        levels = (1 << b) - 1
        if axis == 0:
            c, s, zp = kivi.quant_keys(x, g, levels)
            rec = kivi.dequant_keys(c, s, zp, g)
            assert s.shape == (1, 1, -(-n // g), d)
        else:
            c, s, zp = kivi.quant_values(x, g, levels)
            rec = kivi.dequant_values(c, s, zp, g)
            assert s.shape == (1, 1, n, -(-d // g))
        np.testing.assert_array_equal(c[0, 0], z[t + "codes"])
        np.testing.assert_array_equal(s[0, 0], z[t + "scale"])
        np.testing.assert_array_equal(zp[0, 0], z[t + "zero"])
        assert z[t + "scale"].dtype == np.float32 and z[t + "codes"].dtype == np.uint8
        np.testing.assert_array_equal(rec[0, 0].astype(np.float16), z[t + "decoded"])
        ip = (rec[0, 0].astype(np.float16).astype(np.float32) @ z[t + "q"].astype(np.float32)).astype(np.float16)
        np.testing.assert_allclose(ip.astype(np.float32), z[t + "ip"].astype(np.float32), rtol=2e-3, atol=2e-3)
        assert s.min() >= np.float32(1e-8) and (axis == 1 or s.min() == np.float32(1e-8))   # the constant channel: eps-floored scale
    assert "NaN or Inf" in str(z["nonfinite_message"])


def _vq_transform_cases(z):
    """(tag, expected outcome, function kind, input, smooth) for every row of the fixture's table."""
    for row in z["table"]:
        tag, res = str(row).split(":")
        short, xn, sn = tag.split("_")
        if sn == "badwidth":
            sm = np.ones((2, 33), np.float32)
        elif sn == "smooth3d":
            sm = np.ones((1, 2, 32), np.float32)
        else:
            sm = z["in_" + sn]
        yield tag, res, short, z["in_" + xn], sm


def test_vq_dual_transform_and_lut_match_the_reference_functions_run_over_numpy():
    """``vq_transform.npz``: ``apply_dual_transform_keys`` / ``_queries`` / ``compute_query_lut``
    (``allocators/vecinfer.py:93-184``, ``:341-359``) executed over the NumPy stand-in on every way the
    smooth factors broadcast (one vector, a row per head, query groups of a KV head, the averaged
    fallback for mismatched head counts, 2-D / 3-D / 4-D inputs, float16) and the shapes they reject."""
    z = np.load(os.path.join(GOLDEN, "vq_transform.npz"))
    H = z["H"]
    np.testing.assert_array_equal(vq.walsh_hadamard_matrix(32).astype(np.float32), H)
    fns = {"keys": vq.apply_dual_transform_keys, "queries": vq.apply_dual_transform_queries}
    n_ok = n_rejected = 0
    for tag, res, short, x, sm in _vq_transform_cases(z):
        if res == "ValueError":
            with pytest.raises(ValueError):
                fns[short](x, sm, H)
            n_rejected += 1
            continue
        got, want = fns[short](x, sm, H), z[tag]
        assert got.dtype == want.dtype and got.shape == want.shape, tag
        tol = 1e-5 if want.dtype == np.float32 else 2e-2
        np.testing.assert_allclose(got.astype(np.float32), want.astype(np.float32), rtol=0, atol=tol, err_msg=tag)
        n_ok += 1
    assert n_ok == 48 and n_rejected == 4
    for name in ("q4", "q3"):
        got = vq.compute_query_lut(z["in_" + name], z["lut_codebook"], 4)
        assert got.shape == z["lut_" + name].shape
        np.testing.assert_allclose(got, z["lut_" + name], rtol=0, atol=1e-6)
    with pytest.raises(ValueError, match="not divisible"):
        vq.compute_query_lut(z["in_q4"], np.ones((16, 5), np.float32), 5)
    assert "not divisible by sub_dim=5" in str(z["lut_bad"])
