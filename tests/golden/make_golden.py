"""Generate the golden fixtures in this folder by EXECUTING reference code.

Run once, in a container that has the reference checkout (it cannot travel to
the GPU box, so the resulting ``.npz`` files are committed)::

    python tests/golden/make_golden.py --reference /path/to/VeloxQuant-MLX

What is executed from the reference, unmodified:

* ``veloxquant_mlx/dsa/bit_pack.py`` and ``veloxquant_mlx/math/rotation.py``
  are MLX-free and are loaded whole with ``importlib``.
* The reference's test files hold the authors' own NumPy statements of the
  kernels' math, but import ``mlx`` at module top. Their pure-NumPy functions
  (``_quant_keys``, ``_quant_values``, ``_reference_attend``, ``_make_inputs``,
  ``_wht_butterfly``, ``_reference_encode``, ``_pack_np`` ...) are pulled out
  of the parsed source by name and executed as they stand, with only ``np``
  and ``math`` in scope.
* ``walsh_hadamard_matrix`` and ``_pack_signs`` are pulled the same way from
  ``allocators/vecinfer.py`` / ``quantizers/rabitq.py`` (both NumPy-only
  bodies inside MLX-importing modules).
* ``veloxquant_mlx/math/lloyd_max.py`` and ``math/distributions.py`` are MLX-free
  and loaded whole (``core/constants.py``, which ``lloyd_max`` imports by its package
  path, is loaded the same way and registered under that path first); the
  Lloyd-Max codebooks of TurboQuant-RVQ are computed with them, using the
  supports of ``codebooks/strategies.py:38-94`` and the ``_laplacian_pdf`` of
  ``quantizers/turboquant_rvq.py``.

* ``veloxquant_mlx/quantizers/skvq.py`` is loaded whole with a NumPy stand-in registered as
  ``mlx.core`` (the functions it calls -- min, max, mean, round, clip, argmin, argsort, take ...
  -- answered by NumPy in float32): the file's own arithmetic runs unmodified; what the stand-in
  decides is the order of the error mean and ``round``'s tie rule (NumPy's).

* ``quantizers/_quant_utils.py``, ``quantizers/kitty.py`` and ``quantizers/age_tiered.py`` are loaded
  whole over the same stand-in (``_quant_utils`` registered under its package path first).
* Extracted by name and executed over the same stand-in: ``quantize_vq`` / ``dequantize_vq``
  (``allocators/vecinfer.py``), ``_reference_sdpa`` (``tests/cache/test_vecinfer_fused_sdpa.py``),
  ``_memory_bound_mask_parameters`` (``metal/fused_sdpa.py``), and the helper functions of
  ``cache/turboquant_rvq_cache.py`` (word packing, norm split, rescale).
* The cache CLASSES ``cache/kivi_cache.py``, ``sink_cache.py``, ``skvq_cache.py``, ``kitty_cache.py``,
  ``age_tiered_cache.py``, ``vecinfer_cache.py`` and the configuration layer ``cache/base.py`` +
  ``cache/options.py`` are loaded whole over the stand-in with stubs for their other imports: a
  minimal container (``_GrowingKV``, written here) for the ``mlx_lm`` class they derive from,
  ``metal_available() = False``, the real ``core/exceptions.py``, ``core/context.py``,
  ``core/abstractions.py``. Their traces over a call script go to ``cache_traces.npz``; the scenario
  records of ``config_scenarios.py`` to ``config_traces.json``.

* ``quantizers/turboquant_rvq.py`` and ``cache/turboquant_rvq_cache.py`` are loaded whole with the
  package modules they import (``core/constants.py``, ``exceptions.py``, ``context.py``,
  ``abstractions.py``, ``registry.py``, ``dsa/avl_tree.py``, ``math/distributions.py``,
  ``lloyd_max.py``, ``rotation.py``, ``codebooks/scalar_codebook.py``, ``base.py``,
  ``strategies.py``, ``preconditioners/rotation.py``) over the stand-in, extended with a float32
  butterfly for ``hadamard_transform``, ``searchsorted`` and ``ml_dtypes``'s ``bfloat16``; the
  quantizer's outputs and the cache class's trace go to ``rvq_reference.npz``.

* ``quantizers/kivi.py`` (the ``KIVIQuantizer`` class) is loaded whole over the stand-in with the
  ``core/`` modules it imports; its ``encode`` / ``decode`` / ``estimate_inner_product`` outputs on
  both grouping axes go to ``kivi_quantizer.npz``.

* ``apply_dual_transform_keys`` / ``apply_dual_transform_queries`` / ``compute_query_lut``
  (``allocators/vecinfer.py``) are extracted by name and executed over the stand-in on every
  smooth-factor broadcasting convention; outputs and the accept / reject table go to
  ``vq_transform.npz``.

* The parameter lists of the kernel wrappers (``metal/_*.py``, ``metal/fused_sdpa.py``) and of the
  VecInfer functions are read from the parsed source, without executing them, into
  ``wrapper_signatures.json``; the public properties, setters and method parameter lists of the
  cache classes the same way into ``class_surfaces.json``.
* The kernel-wrapper modules themselves (``metal/_kivi_quant.py``, ``_scalar_attend.py``,
  ``_rabitq*.py``, ``_rvq_*.py``, ``_vecinfer.py``, ``fused_sdpa.py``, with ``_kernel_utils.py``) are
  loaded whole over the stand-in, whose kernel launcher only raises, and called with the arguments of
  ``wrapper_scenarios.py`` that they must refuse before any launch; ``wrapper_refusals.json`` records
  the exception types and messages.

Nothing here imports the oracle: the fixtures are the reference's outputs and
the oracle is checked against them by ``tests/test_oracle_golden.py``.
"""

from __future__ import annotations

import argparse
import ast
import importlib.util
import math
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def load_module(path: str, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    import sys
    sys.modules[name] = mod   # (dataclasses look their module up while the body runs)
    spec.loader.exec_module(mod)
    return mod


def extract_functions(path: str, names, extra_ns=None):
    """Exec the named top-level ``def``s of ``path`` with np/math in scope."""
    with open(path, "r", encoding="utf-8") as fh:
        tree = ast.parse(fh.read(), filename=path)
    wanted = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    missing = set(names) - {n.name for n in wanted}
    if missing:
        raise RuntimeError(f"{path}: functions not found: {sorted(missing)}")
    mod = ast.Module(body=wanted, type_ignores=[])
    ns = {"np": np, "math": math, "__name__": "ref_extract"}
    if extra_ns:
        ns.update(extra_ns)
    exec(compile(mod, path, "exec"), ns)
    return ns


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of a checkout of the reference project")
    args = ap.parse_args()
    R = args.reference
    pkg = os.path.join(R, "veloxquant_mlx")

    # ---------------- bit packing (whole module) ----------------
    bp = load_module(os.path.join(pkg, "dsa", "bit_pack.py"), "ref_bit_pack")
    rng = np.random.default_rng(1234)
    out = {}
    for b in (1, 2, 3, 4):
        for n in (8, 13, 64, 257):
            vals = rng.integers(0, 1 << b, n, dtype=np.uint8)
            packed = bp.BitPackBuffer(b).pack(vals)
            out[f"b{b}_n{n}_vals"] = vals
            out[f"b{b}_n{n}_packed"] = packed
    ka = bp.BitPackBuffer(2).pack(np.array([0, 1, 2, 3, 0, 1, 2, 3], dtype=np.uint8))
    assert ka.tolist() == [228, 228]
    out["known_answer_2bit"] = ka
    np.savez_compressed(os.path.join(HERE, "bitpack.npz"), **out)

    # ---------------- KIVI quant + attend (test-file NumPy functions) ----------------
    tsa = os.path.join(pkg, "tests", "metal", "test_scalar_attend.py")
    ns = extract_functions(tsa, ["_quant_keys", "_quant_values", "_reference_attend", "_make_inputs"])
    out = {}
    cases = [
        # name, B, H, S_kv, D, b, g, seed, H_kv
        ("mha_b2", 1, 4, 64, 128, 2, 32, 0, None),
        ("mha_b3", 1, 4, 96, 128, 3, 32, 3, None),
        ("mha_b4", 1, 2, 64, 64, 4, 32, 4, None),
        ("gqa_b2", 2, 8, 160, 128, 2, 32, 0, 2),
        ("ragged_b4", 1, 2, 50, 96, 4, 32, 7, None),
        ("g4_b1", 1, 2, 33, 32, 1, 4, 9, None),
        ("g128_b8", 1, 1, 200, 128, 8, 128, 11, None),
    ]
    names = []
    for name, B, H, S_kv, D, b, g, seed, H_kv in cases:
        q, kc, ks, kz, vc, vs, vz = ns["_make_inputs"](B, H, S_kv, D, b, g, seed=seed, H_kv=H_kv)
        ref = ns["_reference_attend"](q, kc, ks, kz, vc, vs, vz, g, 1.0 / math.sqrt(D))
        for k, v in dict(q=q, kc=kc, ks=ks, kz=kz, vc=vc, vs=vs, vz=vz, out=ref).items():
            out[f"{name}_{k}"] = v
        out[f"{name}_meta"] = np.array([B, H, S_kv, D, b, g, seed, -1 if H_kv is None else H_kv])
        names.append(name)
    out["names"] = np.array(names)
    # special values the reference's own tests pin (tests/metal/test_kivi_quant.py:121-159)
    const = np.full((1, 1, 32, 8), 3.5, dtype=np.float32)
    c, s, z = ns["_quant_keys"](const, 32, 3)
    out["const_kc"], out["const_ks"], out["const_kz"] = c, s, z
    integer_tile = np.tile(np.array([0, 1, 2, 3], dtype=np.float32), 8).reshape(1, 1, 1, 32)
    c, s, z = ns["_quant_values"](integer_tile, 32, 2)  # half-even case: levels=2
    out["halfeven_vc"], out["halfeven_vs"], out["halfeven_vz"] = c, s, z
    out["halfeven_in"] = integer_tile
    np.savez_compressed(os.path.join(HERE, "kivi.npz"), **out)

    # ---------------- RaBitQ ----------------
    tre = os.path.join(pkg, "tests", "metal", "test_rabitq_encode.py")
    ns_e = extract_functions(tre, ["_wht_butterfly", "_reference_encode", "_make_inputs"])
    tra = os.path.join(pkg, "tests", "metal", "test_rabitq_attend.py")
    ns_a = extract_functions(tra, ["_reference_attend", "_make_inputs"])
    trv = os.path.join(pkg, "tests", "metal", "test_rabitq_values.py")
    ns_v = extract_functions(trv, ["_pack_np"])
    ns_s = extract_functions(os.path.join(pkg, "quantizers", "rabitq.py"), ["_pack_signs"])
    rot = load_module(os.path.join(pkg, "math", "rotation.py"), "ref_rotation")
    out = {}
    for N, D, seed in [(1, 8, 0), (33, 64, 1), (64, 128, 2), (17, 256, 3)]:
        keys, diag = ns_e["_make_inputs"](N, D, seed=seed)
        bits, mag = ns_e["_reference_encode"](keys, diag)
        tag = f"enc_N{N}_D{D}"
        out[f"{tag}_keys"], out[f"{tag}_diag"] = keys, diag
        out[f"{tag}_bits"], out[f"{tag}_mag"] = bits, mag
    for B, H, S_q, S_kv, D, seed in [(1, 1, 1, 33, 64, 5), (2, 2, 1, 256, 128, 6), (1, 2, 4, 64, 256, 99)]:
        q, q_scale, k_bits, k_mag, k_const, v_idx, v_cents = ns_a["_make_inputs"](B, H, S_q, S_kv, D, seed=seed)
        ref = ns_a["_reference_attend"](q, q_scale, k_bits, k_mag, k_const, v_idx, v_cents)
        tag = f"att_B{B}_H{H}_Sq{S_q}_S{S_kv}_D{D}"
        for k, v in dict(q=q, q_scale=q_scale, k_bits=k_bits, k_mag=k_mag, k_const=k_const,
                         v_idx=v_idx, v_cents=v_cents, out=ref, v_packed=ns_v["_pack_np"](v_idx)).items():
            out[f"{tag}_{k}"] = v
    trp = os.path.join(pkg, "tests", "metal", "test_rabitq_prefill.py")
    ns_p = extract_functions(trp, ["_reference_prefill", "_make_inputs"])
    for B, H, S_q, S_kv, D, seed, causal in [(1, 1, 8, 33, 64, 11, False), (2, 2, 33, 200, 128, 12, False),
                                             (1, 2, 40, 40, 128, 13, True), (2, 1, 5, 77, 64, 14, True)]:
        q, scale, k_bits, k_mag, k_const, v_idx, v_cents = ns_p["_make_inputs"](B, H, S_q, S_kv, D, seed=seed)
        ref = ns_p["_reference_prefill"](q, scale, k_bits, k_mag, k_const, v_idx, v_cents, causal=causal)
        tag = f"pre_B{B}_H{H}_Sq{S_q}_S{S_kv}_D{D}_c{int(causal)}"
        for k, v in dict(q=q, scale=scale, k_bits=k_bits, k_mag=k_mag, k_const=k_const, v_idx=v_idx, v_cents=v_cents,
                         out=ref, v_packed=ns_v["_pack_np"](v_idx)).items():
            out[f"{tag}_{k}"] = v
    resid = np.random.default_rng(8).standard_normal((5, 64)).astype(np.float32)
    out["signs_in"], out["signs_out"] = resid, ns_s["_pack_signs"](resid)
    for d, seed in [(64, 42), (128, 42), (128, 7)]:
        out[f"diag_d{d}_s{seed}"] = rot.make_hadamard_diagonal(d, seed=seed)
    out["rot_d24_s42"] = rot.make_rotation_matrix(24, seed=42)
    out["rot_d128_s42"] = rot.make_rotation_matrix(128, seed=42).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "rabitq.npz"), **out)

    # ---------------- VecInfer pieces that are NumPy in the reference ----------------
    ns_w = extract_functions(os.path.join(pkg, "allocators", "vecinfer.py"), ["walsh_hadamard_matrix"],
                             extra_ns={"mx": _MxShim()})
    out = {}
    for d in (1, 2, 8, 128):
        out[f"wht_{d}"] = np.asarray(ns_w["walsh_hadamard_matrix"](d))
    # quantize_vq / dequantize_vq (allocators/vecinfer.py:281-335): the module's own array-API path,
    # executed with NumPy answering ``mx``. NumPy sums a contiguous row of fewer than 8 float32 in
    # order, which is also the order of the reference's Metal kernel; at sub_dim 8 it sums as a tree.
    import sys
    import types

    ns_q = extract_functions(os.path.join(pkg, "allocators", "vecinfer.py"), ["quantize_vq", "dequantize_vq"],
                             extra_ns={"mx": _mx_numpy_module()})
    rng = np.random.default_rng(281)
    for tag, sub, n_c, shape in [("s2", 2, 16, (3, 50, 16)), ("s4", 4, 256, (2, 4, 64, 64)), ("s4big", 4, 4096, (1, 2, 40, 128)),
                                 ("s8", 8, 256, (2, 300, 128))]:
        x = rng.standard_normal(shape).astype(np.float16)
        cb = rng.standard_normal((n_c, sub)).astype(np.float16)
        cb[7] = cb[3]                                        # a duplicated centroid: the lower index must win
        x.reshape(-1, sub)[5] = cb[3]                        # an exact hit on it
        idx = np.asarray(ns_q["quantize_vq"](x, cb, sub))
        out[f"q_{tag}_x"], out[f"q_{tag}_cb"], out[f"q_{tag}_idx"] = x, cb, idx
        out[f"q_{tag}_deq"] = np.asarray(ns_q["dequantize_vq"](idx, cb))
    # _reference_sdpa (tests/cache/test_vecinfer_fused_sdpa.py:69-115): the reference's dense statement of
    # attention over VQ keys and values (dequantize, rotate back, smooth, masked softmax), same stand-in
    shim = _mx_numpy_module()
    ns_s = extract_functions(os.path.join(pkg, "tests", "cache", "test_vecinfer_fused_sdpa.py"), ["_reference_sdpa"],
                             extra_ns={"mx": shim, "dequantize_vq": ns_q["dequantize_vq"]})
    Hm = np.asarray(ns_w["walsh_hadamard_matrix"](64), np.float32)
    for tag, B, H_q, H_kv, S_q, S_kv, causal, window, smooth_kind in [
            ("a", 1, 4, 4, 1, 200, True, 0, "none"), ("b", 2, 8, 2, 1, 333, True, 0, "per_head"),
            ("c", 1, 4, 2, 8, 64, True, 0, "shared"), ("d", 2, 4, 4, 3, 150, True, 40, "per_head"),
            ("e", 1, 2, 2, 5, 90, False, 0, "none")]:
        q = rng.standard_normal((B, H_q, S_q, 64)).astype(np.float16)
        cb_k = rng.standard_normal((256, 8)).astype(np.float16)
        cb_v = rng.standard_normal((256, 8)).astype(np.float16)
        k_idx = rng.integers(0, 256, (B, H_kv, S_kv, 8)).astype(np.int32)
        v_idx = rng.integers(0, 256, (B, H_kv, S_kv, 8)).astype(np.int32)
        smooth = {"none": None, "per_head": rng.uniform(0.5, 2.0, (H_kv, 64)).astype(np.float32),
                  "shared": rng.uniform(0.5, 2.0, (64,)).astype(np.float32)}[smooth_kind]
        o = ns_s["_reference_sdpa"](q, k_idx, cb_k, v_idx, cb_v, smooth, Hm, 0.125, causal=causal, sliding_window=window)
        for name, arr in (("q", q), ("cb_k", cb_k), ("cb_v", cb_v), ("k_idx", k_idx), ("v_idx", v_idx), ("out", np.asarray(o)),
                          ("flags", np.asarray([int(causal), window]))):
            out[f"sdpa_{tag}_{name}"] = arr
        if smooth is not None:
            out[f"sdpa_{tag}_smooth"] = smooth
    np.savez_compressed(os.path.join(HERE, "vq.npz"), **out)
    # ---------------- TurboQuant-RVQ codebooks (whole modules) ----------------

    consts = load_module(os.path.join(pkg, "core", "constants.py"), "veloxquant_mlx.core.constants")
    for name in ("veloxquant_mlx", "veloxquant_mlx.core"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["veloxquant_mlx.core.constants"] = consts
    lm = load_module(os.path.join(pkg, "math", "lloyd_max.py"), "ref_lloyd_max")
    dist = load_module(os.path.join(pkg, "math", "distributions.py"), "ref_distributions")
    ns_l = extract_functions(os.path.join(pkg, "quantizers", "turboquant_rvq.py"), ["_laplacian_pdf"])
    out = {}
    for b in (1, 2, 3, 4):
        for d in (64, 128, 256):
            sigma = 1.0 / math.sqrt(d)
            c, _ = lm.lloyd_max(lambda x, s=sigma: dist.gaussian_pdf(x, sigma=s), (-6.0 * sigma, 6.0 * sigma), n_levels=2 ** b)
            out[f"gauss_b{b}_d{d}"] = c
            # the default residual scale of TurboQuantRVQ.__init__ for (d, b)
            sigma_q = math.sqrt((math.sqrt(3.0 * math.pi) / 2.0) * (4.0 ** -b) / d)
            scale = max(sigma_q / math.sqrt(2.0), 1e-6)
            c2, _ = lm.lloyd_max(ns_l["_laplacian_pdf"](scale), (-8.0 * scale, 8.0 * scale), n_levels=2 ** b)
            out[f"laplace_b{b}_d{d}"] = c2
            out[f"scale_b{b}_d{d}"] = np.float64(scale)
        for d in (8, 16, 32):
            c, _ = lm.lloyd_max(lambda x, dd=d: dist.beta_pdf(x, dd), (-1.0 + 1e-6, 1.0 - 1e-6), n_levels=2 ** b)
            out[f"beta_b{b}_d{d}"] = c
    # the mask recogniser of the fused attention dispatch (metal/fused_sdpa.py:332-396), same stand-in
    ns_m = extract_functions(os.path.join(pkg, "metal", "fused_sdpa.py"), ["_memory_bound_mask_parameters"],
                             extra_ns={"mx": _mx_numpy_module()})
    rng_m = np.random.default_rng(332)
    cases = []

    def tail_mask(n, kv, width=None):
        qp = np.arange(kv - n, kv)[:, None]
        kp = np.arange(kv)[None, :]
        vis = kp <= qp
        if width:
            vis &= kp > qp - width
        return vis

    def additive(vis, neg=-np.inf, dt=np.float32):
        return np.where(vis, 0.0, neg).astype(dt)

    Bm, Hm_, Nm, KV = 2, 3, 4, 11
    base = [tail_mask(Nm, KV), tail_mask(Nm, KV, 5), tail_mask(Nm, KV, 1), tail_mask(Nm, KV, KV), np.ones((Nm, KV), bool),
            tail_mask(1, KV), tail_mask(1, KV, 3), np.ones((1, KV), bool), np.zeros((Nm, KV), bool)]
    for vis in base:
        n = vis.shape[0]
        for form in (vis, additive(vis), additive(vis, dt=np.float16), additive(vis, neg=-1e9), vis.astype(np.int32)):
            for shape in ((n, KV), (1, 1, n, KV), (Bm, 1, n, KV), (1, Hm_, n, KV), (Bm, Hm_, n, KV)):
                cases.append((np.broadcast_to(form, shape).copy(), n))
    hole = tail_mask(Nm, KV)
    hole[2, 1] = False                                                 # a padding hole
    per_head = np.broadcast_to(tail_mask(Nm, KV), (Bm, Hm_, Nm, KV)).copy()
    per_head[1, 2] = tail_mask(Nm, KV, 5)                              # one head with its own window
    shifted = np.roll(tail_mask(Nm, KV), 1, axis=1)                    # causal, but not tail-aligned
    cases += [(hole, Nm), (additive(hole), Nm), (per_head, Nm), (shifted, Nm), (tail_mask(Nm, KV)[:, :KV - 1], Nm),
              (tail_mask(Nm, KV)[None, None, None], Nm), (np.ones((KV,), bool), Nm), (tail_mask(Nm, KV)[-1], Nm),
              (np.ones((Nm, 1), bool), Nm), (additive(tail_mask(Nm, KV)) + np.float32(0.5), Nm),
              (rng_m.random((Nm, KV)) < 0.5, Nm), (np.ones((3, Hm_, Nm, KV), bool), Nm)]
    out_m = {"n_cases": np.asarray([len(cases)]), "dims": np.asarray([Bm, Hm_, KV])}
    for i, (mask, n) in enumerate(cases):
        q = np.zeros((Bm, Hm_, n, 8), np.float16)
        try:
            causal, window = ns_m["_memory_bound_mask_parameters"](mask, q, KV)
            res = [1, int(bool(causal)), int(window)]
        except ValueError:
            res = [0, 0, 0]
        out_m[f"m{i}"], out_m[f"r{i}"] = mask, np.asarray(res + [n])
    np.savez_compressed(os.path.join(HERE, "masks.npz"), **out_m)

    # helper functions of cache/turboquant_rvq_cache.py (:65-126): unit direction + norm, rescale with
    # float16 saturation, bit-packing of the code streams; executed with NumPy answering ``mx``
    from functools import partial

    shim = _mx_numpy_module()
    ns_r = extract_functions(os.path.join(pkg, "cache", "turboquant_rvq_cache.py"),
                             ["_unit_fp16_from_fp16", "_rescale_fp16", "_pack_indices", "_unpack_indices"],
                             extra_ns={"mx": shim, "partial": partial, "Any": object, "_WORD_BITS": 32})
    rng_r = np.random.default_rng(747)
    kk = (rng_r.standard_normal((5, 7, 64)) * 10.0 ** rng_r.uniform(-3, 4.5, (5, 7, 1))).astype(np.float16)   # norms past 65504 too
    unit, norms = ns_r["_unit_fp16_from_fp16"](kk)
    out["cache_k"], out["cache_unit"], out["cache_norms"] = kk, np.asarray(unit), np.asarray(norms)
    out["cache_rescaled"] = np.asarray(ns_r["_rescale_fp16"](np.asarray(unit), np.asarray(norms)))
    for bits in (1, 2, 3, 4):
        for d in (64, 128, 20):
            idx = rng_r.integers(0, 1 << bits, (3, 4, d)).astype(np.uint8)
            packed = np.asarray(ns_r["_pack_indices"](idx, bits))
            out[f"pack_b{bits}_d{d}_idx"], out[f"pack_b{bits}_d{d}_words"] = idx, packed.astype(np.uint32)
            assert np.array_equal(np.asarray(ns_r["_unpack_indices"](packed.astype(np.uint32), bits, d)), idx)
    np.savez_compressed(os.path.join(HERE, "rvq.npz"), **out)

    # ---------------- SKVQ quantizer (whole module, NumPy standing in for mlx.core) ----------------
    mlx_pkg = types.ModuleType("mlx")
    mlx_pkg.core = _mx_numpy_module()
    saved = {k: sys.modules.get(k) for k in ("mlx", "mlx.core")}
    sys.modules["mlx"], sys.modules["mlx.core"] = mlx_pkg, mlx_pkg.core
    try:
        skvq = load_module(os.path.join(pkg, "quantizers", "skvq.py"), "ref_skvq")
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
    out = {"alpha_grid": np.asarray(skvq.DEFAULT_ALPHA_GRID, np.float64)}
    rng = np.random.default_rng(2405)
    for tag, n, d, bits, gs, dt in [("a", 64, 32, 2, 8, np.float32), ("b", 48, 128, 4, 32, np.float16),
                                    ("c", 40, 64, 3, 16, np.float16), ("d", 33, 128, 1, 64, np.float32),
                                    ("e", 24, 128, 8, 32, np.float16)]:
        scales = np.logspace(-2, 1, d)
        rng.shuffle(scales)
        x = (rng.standard_normal((n, d)) * scales[None, :]).astype(np.float32)
        x[rng.random((n, d)) < 0.03] *= 20.0                       # sparse outliers: where clipping wins
        x[0, :gs] = 0.75                                           # a constant group (range 0 -> scale = eps)
        x = x.astype(dt)
        codes, lo, scale = skvq.clipped_group_quant(x, bits, gs)
        perm = skvq.channel_permutation(x)
        out[f"{tag}_x"], out[f"{tag}_meta"] = x, np.asarray([bits, gs])
        out[f"{tag}_codes"], out[f"{tag}_lo"], out[f"{tag}_scale"] = np.asarray(codes), np.asarray(lo), np.asarray(scale)
        out[f"{tag}_perm"] = np.asarray(perm)
        out[f"{tag}_inv"] = np.asarray(skvq.invert_permutation(perm))
        out[f"{tag}_rt"] = np.asarray(skvq.skvq_round_trip(x, perm, bits, gs))
        c1, lo1, s1 = skvq.clipped_group_quant(x, bits, gs, alphas=(0.9,))
        out[f"{tag}_codes_a90"], out[f"{tag}_lo_a90"], out[f"{tag}_scale_a90"] = np.asarray(c1), np.asarray(lo1), np.asarray(s1)
    out["bytes"] = np.asarray([skvq.skvq_compressed_bytes(123, 128, 4, 32), skvq.skvq_compressed_bytes(11, 64, 3, 16),
                               skvq.skvq_fp16_bytes(77, 128)])
    np.savez_compressed(os.path.join(HERE, "skvq.npz"), **out)

    # ------- shared group-quant core, Kitty and AgeTiered quantizers (whole modules over the same stand-in) -------
    saved = {k: sys.modules.get(k) for k in ("mlx", "mlx.core", "veloxquant_mlx.quantizers", "veloxquant_mlx.quantizers._quant_utils")}
    sys.modules["mlx"], sys.modules["mlx.core"] = mlx_pkg, mlx_pkg.core
    try:
        qu = load_module(os.path.join(pkg, "quantizers", "_quant_utils.py"), "veloxquant_mlx.quantizers._quant_utils")
        sys.modules.setdefault("veloxquant_mlx.quantizers", types.ModuleType("veloxquant_mlx.quantizers"))
        sys.modules["veloxquant_mlx.quantizers._quant_utils"] = qu
        kitty = load_module(os.path.join(pkg, "quantizers", "kitty.py"), "ref_kitty")
        age = load_module(os.path.join(pkg, "quantizers", "age_tiered.py"), "ref_age_tiered")
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
    out = {}
    rng = np.random.default_rng(256)
    for tag, n, s_len, d, b, gs, dt in [("a", 3, 70, 32, 2, 32, np.float16), ("b", 2, 64, 128, 4, 32, np.float16),
                                        ("c", 4, 5, 16, 8, 8, np.float32), ("d", 1, 33, 64, 3, 16, np.float16)]:
        x = (rng.standard_normal((n, s_len, d)) * np.logspace(-1, 1, d)[None, None, :]).astype(dt)
        codes, scale, zero = qu._group_quant_codes_batched(x, b, gs)
        out[f"gq_{tag}_x"], out[f"gq_{tag}_meta"] = x, np.asarray([b, gs])
        out[f"gq_{tag}_codes"], out[f"gq_{tag}_scale"], out[f"gq_{tag}_zero"] = np.asarray(codes), np.asarray(scale), np.asarray(zero)
        out[f"gq_{tag}_rt"] = np.asarray(qu._group_quant_dequant_batched(x, b, gs))
    # Kitty: channel ranking and the mixed-precision round trip (per-row masks)
    kx = (rng.standard_normal((6, 96, 64)) * rng.permutation(np.logspace(-1, 1, 64))[None, None, :]).astype(np.float16)
    var = np.var(kx.astype(np.float32), axis=1)
    mask = kitty.hi_mask_from_variance_batched(var, 0.25)
    out["kitty_x"], out["kitty_var"], out["kitty_mask"] = kx, var, np.asarray(mask)
    out["kitty_out"] = np.asarray(kitty.quantize_mixed_channels_batched(kx, mask, hi_bit=4, lo_bit=2, group_size=32))
    out["kitty_running_var"] = np.asarray(kitty.compute_running_variance(kx.astype(np.float32).sum(1)[0], (kx.astype(np.float32) ** 2).sum(1)[0], 96))
    # AgeTiered: three tiers over position-aligned groups, last group ragged
    ax = rng.standard_normal((4, 200, 32)).astype(np.float16)
    tiers = age.default_age_tiers(8, 4, 2)
    ages = [200 - (i + 1) for i in range(200)]
    tok_tier = age.assign_age_tiers(ages, 40, 120)
    group_tier = [tok_tier[g * 32] for g in range(7)]
    out["age_x"], out["age_tok_tier"], out["age_group_tier"] = ax, np.asarray(tok_tier), np.asarray(group_tier)
    out["age_out"] = np.asarray(age.age_tier_quantize_batched(ax, group_tier, tiers, 32))
    out["age_bytes"] = np.asarray([age.age_tiered_bytes({age.RECENT: 40, age.MID: 80, age.OLD: 80}, tiers, 32), age.full_fp16_bytes(200, 32)])
    np.savez_compressed(os.path.join(HERE, "group_quant.npz"), **out)

    # ------- the cache classes themselves, over the same stand-in plus a minimal container base class -------
    names = ["mlx", "mlx.core", "mlx_lm", "mlx_lm.models", "mlx_lm.models.cache", "veloxquant_mlx.core.exceptions",
             "veloxquant_mlx.metal", "veloxquant_mlx.metal.kernels", "veloxquant_mlx.cache", "veloxquant_mlx.cache.kivi_cache",
             "veloxquant_mlx.quantizers", "veloxquant_mlx.quantizers._quant_utils", "veloxquant_mlx.quantizers.skvq",
             "veloxquant_mlx.quantizers.kitty", "veloxquant_mlx.quantizers.age_tiered", "veloxquant_mlx.metal.fused_sdpa",
             "veloxquant_mlx.allocators", "veloxquant_mlx.allocators.vecinfer", "veloxquant_mlx.core.context",
             "veloxquant_mlx.core.abstractions", "veloxquant_mlx.cache.options", "veloxquant_mlx.cache.sliding_window_cache",
             "veloxquant_mlx.cache.sink_cache", "veloxquant_mlx.cache.skvq_cache", "veloxquant_mlx.cache.kitty_cache",
             "veloxquant_mlx.cache.age_tiered_cache", "veloxquant_mlx.cache.base", "veloxquant_mlx.metal._warmup"]
    saved = {k: sys.modules.get(k) for k in names}
    try:
        sys.modules["mlx"], sys.modules["mlx.core"] = mlx_pkg, mlx_pkg.core
        for name in ("mlx_lm", "mlx_lm.models", "veloxquant_mlx.cache", "veloxquant_mlx.quantizers"):
            sys.modules[name] = types.ModuleType(name)
        base = types.ModuleType("mlx_lm.models.cache")
        base.KVCache = _GrowingKV
        sys.modules["mlx_lm.models.cache"] = base
        load_module(os.path.join(pkg, "core", "exceptions.py"), "veloxquant_mlx.core.exceptions")
        metal = types.ModuleType("veloxquant_mlx.metal")
        metal.metal_available = lambda: False               # the classes then take their own array path
        metal_k = types.ModuleType("veloxquant_mlx.metal.kernels")
        metal_k.kivi_group_quant_dequant = None
        sys.modules["veloxquant_mlx.metal"], sys.modules["veloxquant_mlx.metal.kernels"] = metal, metal_k
        for mod in ("_quant_utils", "skvq", "kitty", "age_tiered"):
            load_module(os.path.join(pkg, "quantizers", mod + ".py"), "veloxquant_mlx.quantizers." + mod)
        kivi_c = load_module(os.path.join(pkg, "cache", "kivi_cache.py"), "veloxquant_mlx.cache.kivi_cache")
        sink_c = load_module(os.path.join(pkg, "cache", "sink_cache.py"), "ref_sink_cache")
        skvq_c = load_module(os.path.join(pkg, "cache", "skvq_cache.py"), "ref_skvq_cache")
        kitty_c = load_module(os.path.join(pkg, "cache", "kitty_cache.py"), "ref_kitty_cache")
        age_c = load_module(os.path.join(pkg, "cache", "age_tiered_cache.py"), "ref_age_tiered_cache")
        out = {}
        rng = np.random.default_rng(77)
        B, H, D, T = 2, 2, 32, 120
        scales = rng.permutation(np.logspace(-1, 1, D))
        k = (rng.standard_normal((B, H, T, D)) * scales[None, None, None, :]).astype(np.float16)
        v = rng.standard_normal((B, H, T, D)).astype(np.float16)
        k[0, :, 3] *= 6.0
        k[1, :, 17] *= 6.0                                   # one outstanding key norm per sequence (a sink)
        out["k"], out["v"] = k, v
        # calls: a prefill, single tokens, a block, a trim (where the class allows it), more tokens
        script = [("put", 0, 45)] + [("put", t, t + 1) for t in range(45, 75)] + [("put", 75, 90), ("trim", 11, 0)] + \
                 [("put", t, t + 1) for t in range(79, 100)] + [("put", 100, 120)]
        out["script"] = np.asarray([[{"put": 0, "trim": 1}[op], a, b] for op, a, b in script])

        def run(tag, cache, counters, trimmable):
            for i, (op, a, b) in enumerate(script):
                if op == "trim":
                    if not trimmable:
                        continue
                    assert cache.trim(a) == a
                    continue
                ko, vo = cache.update_and_fetch(k[:, :, a:b], v[:, :, a:b])
                if b - a > 1 or b % 8 == 0 or b == 120:
                    out[f"{tag}_k_{i}"], out[f"{tag}_v_{i}"] = np.array(ko), np.array(vo)
                    out[f"{tag}_c_{i}"] = np.asarray([int(getattr(cache, c)) for c in counters], dtype=np.int64)

        cfg = types.SimpleNamespace(head_dim=D, bit_width_inlier=2, kivi_group_size=8, residual_length=16, use_metal_kernels=None,
                                    n_sink_tokens=2, skvq_bits_key=2, skvq_bits_value=3, skvq_group_size=8, skvq_window=16,
                                    skvq_n_sink=3, skvq_reorder=True, skvq_clip_search=True, skvq_clip_alpha=1.0, skvq_max_ctx=None,
                                    kitty_hi_fraction=0.25, kitty_hi_bit=4, kitty_lo_bit=2, kitty_group_size=8,
                                    age_recent_boundary=20, age_mid_boundary=50, age_bits_recent=8, age_bits_mid=4, age_bits_old=2,
                                    age_group_size=8)
        run("kivi", kivi_c.KIVIKVCache(cfg), ["offset", "_n_quantized", "_key_bytes_compressed", "_value_bytes_compressed",
                                              "_key_bytes_fp16", "_residual_fp16_bytes", "_tokens_seen"], True)
        sink = sink_c.SinkProtectedKVCache(cfg)
        run("sink", sink, ["offset", "_n_quantized", "_key_bytes_compressed", "_value_bytes_compressed", "_sink_fp16_bytes",
                           "_residual_fp16_bytes", "_tokens_seen"], True)
        out["sink_positions"] = np.asarray([sink.sink_positions_for(0), sink.sink_positions_for(1)])
        skc = skvq_c.SKVQKVCache(cfg)
        run("skvq", skc, ["offset", "_q_end", "_compressed_key_bytes", "_compressed_value_bytes", "_fp16_key_bytes",
                          "residual_fp16_bytes", "perm_bytes"], False)
        out["skvq_perm_k"], out["skvq_perm_v"] = np.asarray(skc.key_perms), np.asarray(skc.value_perms)
        run("kitty", kitty_c.KittyKVCache(cfg), ["offset", "_n_keys", "_compressed_key_bytes", "_fp16_key_bytes", "_value_fp16_bytes"], True)
        run("age", age_c.AgeTieredKVCache(cfg), ["offset", "age_tiered_bytes", "full_seq_bytes", "tokens_recent", "tokens_mid", "tokens_old"], False)
        # VecInfer (standard path: every block smoothed, rotated, VQ-coded and reconstructed on its own)
        fs = types.ModuleType("veloxquant_mlx.metal.fused_sdpa")
        fs.supports_shape = lambda **kw: False
        fs.is_patched = lambda: False
        sys.modules["veloxquant_mlx.metal.fused_sdpa"] = fs
        sys.modules["veloxquant_mlx.allocators"] = types.ModuleType("veloxquant_mlx.allocators")
        load_module(os.path.join(pkg, "allocators", "vecinfer.py"), "veloxquant_mlx.allocators.vecinfer")
        vi_c = load_module(os.path.join(pkg, "cache", "vecinfer_cache.py"), "ref_vecinfer_cache")
        vcfg = types.SimpleNamespace(head_dim=D, key_sub_dim=4, value_sub_dim=8, key_codebook_bits=8, value_codebook_bits=8,
                                     residual_length=128, seed=42, use_metal_kernels=None, fused_sdpa=False,
                                     fused_sdpa_memory_bound=False, fused_sdpa_max_ctx=None,
                                     smooth_factors=rng.uniform(0.5, 2.0, (H, D)).astype(np.float32),
                                     key_codebook=rng.standard_normal((256, 4)).astype(np.float32),
                                     value_codebook=rng.standard_normal((256, 8)).astype(np.float32))
        out["vecinfer_smooth"], out["vecinfer_cb_k"], out["vecinfer_cb_v"] = vcfg.smooth_factors, vcfg.key_codebook, vcfg.value_codebook
        run("vecinfer", vi_c.VecInferKVCache(vcfg), ["offset", "_key_bytes_compressed", "_value_bytes_compressed", "_key_bytes_fp16",
                                                     "_tokens_seen"], True)
        np.savez_compressed(os.path.join(HERE, "cache_traces.npz"), **out)

        # ------- the configuration layer itself (cache/base.py, cache/options.py), same stand-ins -------
        import json

        import config_scenarios

        for mod in ("context", "abstractions"):
            load_module(os.path.join(pkg, "core", mod + ".py"), "veloxquant_mlx.core." + mod)
        opts = load_module(os.path.join(pkg, "cache", "options.py"), "veloxquant_mlx.cache.options")
        sw = types.ModuleType("veloxquant_mlx.cache.sliding_window_cache")
        sw.SlidingWindowKVCache = type("SlidingWindowKVCache", (), {"__init__": lambda self, cache, window_size: None})
        sys.modules["veloxquant_mlx.cache.sliding_window_cache"] = sw
        for name, path in (("sink_cache", "sink_cache.py"), ("skvq_cache", "skvq_cache.py"), ("kitty_cache", "kitty_cache.py"),
                           ("age_tiered_cache", "age_tiered_cache.py")):
            load_module(os.path.join(pkg, "cache", path), "veloxquant_mlx.cache." + name)
        base_m = load_module(os.path.join(pkg, "cache", "base.py"), "veloxquant_mlx.cache.base")
        ns_cfg = types.SimpleNamespace(KVCacheConfig=base_m.KVCacheConfig, KVCacheFactory=base_m.KVCacheFactory,
                                       VecInferOptions=opts.VecInferOptions, KIVIOptions=opts.KIVIOptions, SKVQOptions=opts.SKVQOptions,
                                       KittyOptions=opts.KittyOptions, AgeTieredKVOptions=opts.AgeTieredKVOptions,
                                       KVCacheBuilder=base_m.KVCacheBuilder, PlainCache=_GrowingKV)
        warm = types.ModuleType("veloxquant_mlx.metal._warmup")          # (kernel pre-compilation: nothing to do here)
        warm.warmup_for_config = lambda cfg: None
        sys.modules["veloxquant_mlx.metal._warmup"] = warm
        with open(os.path.join(HERE, "config_traces.json"), "w") as fh:
            json.dump({"config": config_scenarios.scenarios(ns_cfg), "construction": config_scenarios.construction_scenarios(ns_cfg),
                       "builder": config_scenarios.builder_scenarios(ns_cfg)},
                      fh, indent=1, sort_keys=True, default=str)
    finally:
        for key, val in saved.items():
            if val is None:
                sys.modules.pop(key, None)
            else:
                sys.modules[key] = val
    _rvq_reference_section(pkg)
    _kivi_quantizer_section(pkg)
    _vq_transform_section(pkg)
    _wrapper_signatures_section(pkg)
    _class_surfaces_section(pkg)
    _wrapper_refusals_section(pkg)
    print("golden fixtures written to", HERE)


def _rvq_reference_section(pkg: str) -> None:
    """``quantizers/turboquant_rvq.py`` (``TurboQuantRVQ.encode`` / ``decode``) and the cache class of
    ``cache/turboquant_rvq_cache.py``, loaded whole with everything they import from the package
    (``codebooks/``, ``preconditioners/rotation.py``, ``math/``, ``dsa/avl_tree.py``, ``core/``) over
    the NumPy stand-in. Two ``mlx.core`` functions have no NumPy namesake and are written here:
    ``hadamard_transform`` (float32 butterfly, strides ascending, times ``1/sqrt(n)``) and
    ``searchsorted``; ``bfloat16`` is ``ml_dtypes``'s. Writes ``rvq_reference.npz``."""
    import sys
    import types

    import ml_dtypes

    mx = _mx_numpy_module()
    mx.bfloat16 = ml_dtypes.bfloat16

    def hadamard_transform(a, scale=None):
        x = np.asarray(a, dtype=np.float32).copy()
        n = x.shape[-1]
        h = 1
        while h < n:
            y = x.reshape(*x.shape[:-1], n // (2 * h), 2, h)
            lo, hi = y[..., 0, :] + y[..., 1, :], y[..., 0, :] - y[..., 1, :]
            x = np.stack([lo, hi], axis=-2).reshape(*x.shape[:-1], n).astype(np.float32)
            h *= 2
        return (x * np.float32(1.0 / np.sqrt(np.float32(n)) if scale is None else scale)).astype(np.float32)

    mx.hadamard_transform = hadamard_transform
    mx.searchsorted = lambda a, v, side="left": np.searchsorted(a, v, side=side)
    mlx_pkg = types.ModuleType("mlx")
    mlx_pkg.core = mx
    packages = ["veloxquant_mlx", "veloxquant_mlx.core", "veloxquant_mlx.dsa", "veloxquant_mlx.codebooks", "veloxquant_mlx.math",
                "veloxquant_mlx.preconditioners", "veloxquant_mlx.quantizers", "veloxquant_mlx.cache", "mlx_lm", "mlx_lm.models"]
    files = [("core/constants.py", "core.constants"), ("core/exceptions.py", "core.exceptions"), ("core/context.py", "core.context"),
             ("core/abstractions.py", "core.abstractions"), ("core/registry.py", "core.registry"), ("dsa/avl_tree.py", "dsa.avl_tree"),
             ("math/distributions.py", "math.distributions"), ("math/lloyd_max.py", "math.lloyd_max"), ("math/rotation.py", "math.rotation"),
             ("codebooks/scalar_codebook.py", "codebooks.scalar_codebook"), ("codebooks/base.py", "codebooks.base"),
             ("codebooks/strategies.py", "codebooks.strategies"), ("preconditioners/rotation.py", "preconditioners.rotation"),
             ("quantizers/turboquant_rvq.py", "quantizers.turboquant_rvq"), ("cache/turboquant_rvq_cache.py", "cache.turboquant_rvq_cache")]
    names = ["mlx", "mlx.core", "mlx_lm.models.cache", "veloxquant_mlx.metal"] + packages + ["veloxquant_mlx." + n for _, n in files]
    saved = {k: sys.modules.get(k) for k in names}
    try:
        sys.modules["mlx"], sys.modules["mlx.core"] = mlx_pkg, mx
        for name in packages:
            sys.modules[name] = types.ModuleType(name)

        class _SteppedKV(_GrowingKV):
            step = 256                                           # the growth step of the class the reference derives from

        base = types.ModuleType("mlx_lm.models.cache")
        base.KVCache, base.create_attention_mask = _SteppedKV, None
        sys.modules["mlx_lm.models.cache"] = base
        metal = types.ModuleType("veloxquant_mlx.metal")
        metal.metal_available = lambda: False                    # the classes then take their own array path
        sys.modules["veloxquant_mlx.metal"] = metal
        mods = {n: load_module(os.path.join(pkg, *rel.split("/")), "veloxquant_mlx." + n) for rel, n in files}
        rvq, cache_m = mods["quantizers.turboquant_rvq"], mods["cache.turboquant_rvq_cache"]

        out = {}
        cases = [(64, 1), (64, 4), (128, 2), (128, 3), (128, 4), (256, 2)]
        out["quantizer_cases"] = np.asarray(cases)
        for d, b in cases:
            q = rvq.TurboQuantRVQ(d=d, b=b, seed=3, use_hadamard=True)
            x = np.random.default_rng(1000 * d + b).standard_normal((96, d)).astype(np.float32)
            x = (x / np.linalg.norm(x, axis=-1, keepdims=True)).astype(np.float16)
            ev = q.encode(x)
            t = f"q_d{d}_b{b}_"
            out[t + "x"], out[t + "rotated"] = x, np.asarray(q._rotation.apply(x))
            out[t + "idx1"], out[t + "idx2"] = np.asarray(ev.indices), np.asarray(ev.signs).astype(np.uint8)
            out[t + "decoded"] = np.asarray(q.decode(ev))
            out[t + "diag"] = np.asarray(q._rotation._D, dtype=np.float32)
            out[t + "c1"], out[t + "b1"] = np.asarray(q._codebook1.centroids_mx()), np.asarray(q._codebook1.boundaries_mx())
            out[t + "c2"], out[t + "b2"] = np.asarray(q._codebook2.centroids_mx()), np.asarray(q._codebook2.boundaries_mx())

        # the cache class over a call script: a prefill, single tokens, a block, a trim, more tokens
        rng = np.random.default_rng(251)
        B, H, D, T, bits, seed = 2, 2, 64, 120, 2, 5
        k = (rng.standard_normal((B, H, T, D)) * 10.0 ** rng.uniform(-2, 2, (B, H, T, 1))).astype(np.float16)
        k[1, 0, 9] = (np.sign(k[1, 0, 9].astype(np.float32)) * 30000.0).astype(np.float16)     # a norm past 65504
        k[0, 1, 50] = 0                                                                          # a zero key
        v = rng.standard_normal((B, H, T, D)).astype(np.float16)
        script = [("put", 0, 45)] + [("put", t, t + 1) for t in range(45, 75)] + [("put", 75, 90), ("trim", 11, 0)] + \
                 [("put", t, t + 1) for t in range(79, 100)] + [("put", 100, 120)]
        out["cache_dims"], out["cache_k"], out["cache_v"] = np.asarray([B, H, D, T, bits, seed]), k, v
        out["cache_script"] = np.asarray([[{"put": 0, "trim": 1}[op], a, b] for op, a, b in script])
        cfg = types.SimpleNamespace(head_dim=D, bit_width_inlier=bits, seed=seed, use_metal_kernels=None)
        cache = cache_m.TurboQuantRVQKVCache(cfg)
        for i, (op, a, b) in enumerate(script):
            if op == "trim":
                assert cache.trim(a) == a
                continue
            ko, vo = cache.update_and_fetch(k[:, :, a:b], v[:, :, a:b])
            if b - a > 1 or b % 32 == 0:
                out[f"cache_k_{i}"], out[f"cache_v_{i}"] = np.array(ko), np.array(vo)
                out[f"cache_c_{i}"] = np.asarray([cache.offset, cache._packed1.shape[2], cache.compressed_key_bytes, cache.fp16_key_bytes,
                                                  cache.nbytes], dtype=np.int64)
        p1, p2, norms, vals = cache.state
        out["cache_state_p1"], out["cache_state_p2"] = np.asarray(p1).astype(np.uint32), np.asarray(p2).astype(np.uint32)
        out["cache_state_norms"] = np.asarray(norms).astype(np.float32)
        out["cache_meta_state"] = np.asarray([int(s) for s in cache.meta_state])
        np.savez_compressed(os.path.join(HERE, "rvq_reference.npz"), **out)
    finally:
        for key, val in saved.items():
            if val is None:
                sys.modules.pop(key, None)
            else:
                sys.modules[key] = val


def _kivi_quantizer_section(pkg: str) -> None:
    """``quantizers/kivi.py`` (``KIVIQuantizer.encode`` / ``decode``, both axes, ragged last groups),
    loaded whole over the NumPy stand-in with the ``core/`` modules it imports. Writes
    ``kivi_quantizer.npz``."""
    import sys
    import types

    mx = _mx_numpy_module()
    mlx_pkg = types.ModuleType("mlx")
    mlx_pkg.core = mx
    packages = ["veloxquant_mlx", "veloxquant_mlx.core", "veloxquant_mlx.quantizers"]
    files = [("core/constants.py", "core.constants"), ("core/exceptions.py", "core.exceptions"), ("core/context.py", "core.context"),
             ("core/abstractions.py", "core.abstractions"), ("core/registry.py", "core.registry"), ("quantizers/kivi.py", "quantizers.kivi")]
    names = ["mlx", "mlx.core"] + packages + ["veloxquant_mlx." + n for _, n in files]
    saved = {k: sys.modules.get(k) for k in names}
    try:
        sys.modules["mlx"], sys.modules["mlx.core"] = mlx_pkg, mx
        for name in packages:
            sys.modules[name] = types.ModuleType(name)
        mods = {n: load_module(os.path.join(pkg, *rel.split("/")), "veloxquant_mlx." + n) for rel, n in files}
        kivi = mods["quantizers.kivi"]
        rng = np.random.default_rng(103)
        out = {}
        cases = []
        for axis in ("channel", "token"):
            for n, d, b, g in [(64, 32, 2, 32), (70, 40, 2, 32), (45, 24, 4, 8), (33, 16, 1, 16), (12, 8, 8, 5), (7, 64, 3, 1)]:
                cases.append([0 if axis == "channel" else 1, n, d, b, g])
                x = (rng.standard_normal((n, d)) * rng.uniform(0.2, 3.0, (1, d))).astype(np.float16)
                x[n // 2, :] = x[n // 2, 0]                      # a constant row (one-value groups on the token axis)
                x[:, d // 2] = 1.5                               # a constant channel (one-value groups on the channel axis)
                q = kivi.KIVIQuantizer(d=d, b=b, group_size=g, axis=axis)
                ev = q.encode(x)
                t = f"{axis}_n{n}_d{d}_b{b}_g{g}_"
                out[t + "x"], out[t + "codes"] = x, np.asarray(ev.indices)
                out[t + "scale"], out[t + "zero"] = np.asarray(ev.norm), np.asarray(ev.residual_norm)
                out[t + "decoded"] = np.asarray(q.decode(ev))
                qv = rng.standard_normal(d).astype(np.float16)
                out[t + "q"], out[t + "ip"] = qv, np.asarray(q.estimate_inner_product(qv, ev))
        out["cases"] = np.asarray(cases)
        bad = np.ones((4, 8), np.float16)
        bad[1, 2] = np.inf
        try:
            kivi.KIVIQuantizer(d=8).encode(bad)
            raise AssertionError("an infinite input was accepted")
        except mods["core.exceptions"].QuantizerConfigError as e:
            out["nonfinite_message"] = np.asarray(str(e))
        np.savez_compressed(os.path.join(HERE, "kivi_quantizer.npz"), **out)
    finally:
        for key, val in saved.items():
            if val is None:
                sys.modules.pop(key, None)
            else:
                sys.modules[key] = val


def _vq_transform_section(pkg: str) -> None:
    """``apply_dual_transform_keys`` / ``apply_dual_transform_queries`` / ``compute_query_lut`` /
    ``walsh_hadamard_matrix`` (``allocators/vecinfer.py:60-184``, ``:341-359``) extracted by name and
    executed over the NumPy stand-in, over every broadcasting convention of the smooth factors (one
    vector, one row per head, grouped query heads, mismatched head counts) and the shapes they
    reject. Writes ``vq_transform.npz``."""
    mx = _mx_numpy_module()
    ns = extract_functions(os.path.join(pkg, "allocators", "vecinfer.py"),
                           ["walsh_hadamard_matrix", "apply_dual_transform_keys", "apply_dual_transform_queries", "compute_query_lut"],
                           extra_ns={"mx": mx})
    rng = np.random.default_rng(616)
    D, Hkv, Hq, B, S = 32, 2, 6, 2, 5
    Hm = np.asarray(ns["walsh_hadamard_matrix"](D), dtype=np.float32)
    out = {"H": Hm}
    smooth = {"vec": rng.uniform(0.5, 2.0, D).astype(np.float32), "kv": rng.uniform(0.5, 2.0, (Hkv, D)).astype(np.float32),
              "q": rng.uniform(0.5, 2.0, (Hq, D)).astype(np.float32), "five": rng.uniform(0.5, 2.0, (5, D)).astype(np.float32)}
    xs = {"k4": rng.standard_normal((B, Hkv, S, D)).astype(np.float32), "k3": rng.standard_normal((Hkv, S, D)).astype(np.float32),
          "k2": rng.standard_normal((S, D)).astype(np.float32), "q4": rng.standard_normal((B, Hq, S, D)).astype(np.float32),
          "q3": rng.standard_normal((Hq, 1, D)).astype(np.float32), "k4h": rng.standard_normal((B, Hkv, S, D)).astype(np.float16)}
    for name, arr in list(smooth.items()) + list(xs.items()):
        out["in_" + name] = arr
    table = []
    for fn_name, short in (("apply_dual_transform_keys", "keys"), ("apply_dual_transform_queries", "queries")):
        for xn, x in xs.items():
            for sn, sm in smooth.items():
                tag = f"{short}_{xn}_{sn}"
                try:
                    out[tag] = np.asarray(ns[fn_name](x, sm, Hm))
                    table.append(tag + ":ok")
                except ValueError:
                    table.append(tag + ":ValueError")
    for fn_name, short in (("apply_dual_transform_keys", "keys"), ("apply_dual_transform_queries", "queries")):
        for tag, x, sm in ((f"{short}_k4_badwidth", xs["k4"], np.ones((Hkv, D + 1), np.float32)),
                           (f"{short}_k4_smooth3d", xs["k4"], np.ones((1, Hkv, D), np.float32))):
            try:
                ns[fn_name](x, sm, Hm)
                table.append(tag + ":ok")
            except ValueError:
                table.append(tag + ":ValueError")
    out["table"] = np.asarray(table)
    cb = rng.standard_normal((16, 4)).astype(np.float32)
    out["lut_codebook"] = cb
    out["lut_q4"] = np.asarray(ns["compute_query_lut"](xs["q4"], cb, 4))
    out["lut_q3"] = np.asarray(ns["compute_query_lut"](xs["q3"], cb, 4))
    try:
        ns["compute_query_lut"](xs["q4"], rng.standard_normal((16, 5)).astype(np.float32), 5)
        out["lut_bad"] = np.asarray("ok")
    except ValueError as e:
        out["lut_bad"] = np.asarray(str(e))
    np.savez_compressed(os.path.join(HERE, "vq_transform.npz"), **out)


WRAPPER_FILES = {
    "metal/_kivi_quant.py": ["kivi_group_quant_dequant"],
    "metal/_scalar_attend.py": ["scalar_fused_decode_attend", "scalar_fused_decode_attend_batched", "scalar_decode_once",
                                "scalar_predecoded_attend"],
    "metal/_bit_packing.py": ["turboquant_bit_pack", "turboquant_bit_unpack"],
    "metal/_rabitq.py": ["rabitq_hamming_score"], "metal/_rabitq_attend.py": ["rabitq_fused_attend"],
    "metal/_rabitq_encode.py": ["rabitq_encode"], "metal/_rabitq_prefill.py": ["rabitq_prefill_attend"],
    "metal/_rabitq_values.py": ["rabitq_pack_values"], "metal/_rvq_quant_pack.py": ["rvq_quant_pack"],
    "metal/_rvq_unpack_decode.py": ["rvq_unpack_decode"],
    "metal/_vecinfer.py": ["vecinfer_quantize_metal", "vecinfer_dequant_metal", "vecinfer_encode_decode_metal",
                           "vecinfer_encode_decode_simple_metal"],
    "metal/fused_sdpa.py": ["metal_fused_sdpa", "supports_shape"],
    "allocators/vecinfer.py": ["quantize_vq", "dequantize_vq", "compute_query_lut", "apply_dual_transform_keys",
                               "apply_dual_transform_queries", "walsh_hadamard_matrix"],
}


def _wrapper_signatures_section(pkg: str) -> None:
    """The parameter lists of the reference's kernel wrappers and VecInfer functions on this path, read
    from the parsed source (nothing is executed): positional names in order, keyword-only names, how
    many positionals carry a default. Writes ``wrapper_signatures.json``."""
    import json

    out = {}
    for rel, names in WRAPPER_FILES.items():
        with open(os.path.join(pkg, *rel.split("/")), "r", encoding="utf-8") as fh:
            tree = ast.parse(fh.read())
        found = {n.name: n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names}
        missing = set(names) - set(found)
        if missing:
            raise RuntimeError(f"{rel}: functions not found: {sorted(missing)}")
        for name, node in found.items():
            a = node.args
            out[name] = {"file": rel, "positional": [x.arg for x in a.posonlyargs + a.args], "keyword_only": [x.arg for x in a.kwonlyargs],
                         "n_defaults": len(a.defaults)}
    with open(os.path.join(HERE, "wrapper_signatures.json"), "w") as fh:
        json.dump(out, fh, indent=1, sort_keys=True)


CACHE_CLASS_FILES = {
    "cache/kivi_cache.py": "KIVIKVCache", "cache/sink_cache.py": "SinkProtectedKVCache", "cache/vecinfer_cache.py": "VecInferKVCache",
    "cache/turboquant_rvq_cache.py": "TurboQuantRVQKVCache", "cache/skvq_cache.py": "SKVQKVCache",
    "cache/kitty_cache.py": "KittyKVCache", "cache/age_tiered_cache.py": "AgeTieredKVCache",
}


def _class_surfaces_section(pkg: str) -> None:
    """The public surface the reference's cache classes define themselves (what they inherit from their
    serving framework's container is not in the checkout), read from the parsed source: per class its
    public properties, which of them have a setter, and its public methods with their parameter lists.
    Writes ``class_surfaces.json``."""
    import json

    out = {}
    for rel, cls_name in CACHE_CLASS_FILES.items():
        with open(os.path.join(pkg, *rel.split("/")), "r", encoding="utf-8") as fh:
            tree = ast.parse(fh.read())
        node = next(n for n in tree.body if isinstance(n, ast.ClassDef) and n.name == cls_name)
        rec = {"file": rel, "properties": [], "setters": [], "methods": {}}
        for n in node.body:
            if isinstance(n, ast.Assign) and isinstance(n.value, ast.Call) and getattr(n.value.func, "id", "") == "property":
                rec["properties"] += [t.id for t in n.targets if isinstance(t, ast.Name) and not t.id.startswith("_")]
            if not isinstance(n, ast.FunctionDef) or n.name.startswith("_"):
                continue
            decorators = [ast.unparse(d) for d in n.decorator_list]
            if "property" in decorators:
                rec["properties"].append(n.name)
            elif any(d.endswith(".setter") for d in decorators):
                rec["setters"].append(n.name)
            else:
                a = n.args
                rec["methods"][n.name] = {"positional": [x.arg for x in a.posonlyargs + a.args][0 if "staticmethod" in decorators else 1:],
                                          "keyword_only": [x.arg for x in a.kwonlyargs], "var_positional": a.vararg is not None}
        out[cls_name] = rec
    with open(os.path.join(HERE, "class_surfaces.json"), "w") as fh:
        json.dump(out, fh, indent=1, sort_keys=True)


def _wrapper_refusals_section(pkg: str) -> None:
    """The reference's kernel wrappers (``metal/_*.py``, ``metal/fused_sdpa.py``), loaded whole over the
    NumPy stand-in with a kernel launcher that is never reached, on the calls of
    ``wrapper_scenarios.py`` that they must refuse: exception types and messages go to
    ``wrapper_refusals.json``."""
    import json
    import sys
    import types

    import wrapper_scenarios

    mx = _mx_numpy_module()

    def metal_kernel(**kw):
        def launch(**k):
            raise RuntimeError("kernel launcher reached")
        return launch

    mx.fast = types.SimpleNamespace(metal_kernel=metal_kernel)
    mlx_pkg = types.ModuleType("mlx")
    mlx_pkg.core = mx
    modules = {rel: "veloxquant_mlx." + rel[:-3].replace("/", ".") for rel in WRAPPER_FILES if rel.startswith("metal/")}
    names = ["mlx", "mlx.core", "veloxquant_mlx", "veloxquant_mlx.metal", "veloxquant_mlx.metal._kernel_utils"] + list(modules.values())
    saved = {k: sys.modules.get(k) for k in names}
    try:
        sys.modules["mlx"], sys.modules["mlx.core"] = mlx_pkg, mx
        for name in ("veloxquant_mlx", "veloxquant_mlx.metal"):
            sys.modules[name] = types.ModuleType(name)
        load_module(os.path.join(pkg, "metal", "_kernel_utils.py"), "veloxquant_mlx.metal._kernel_utils")
        ns = types.SimpleNamespace()
        for rel, mod_name in modules.items():
            mod = load_module(os.path.join(pkg, *rel.split("/")), mod_name)
            for fn_name in WRAPPER_FILES[rel]:
                setattr(ns, fn_name, getattr(mod, fn_name))
        records = wrapper_scenarios.refusal_scenarios(ns, lambda a: a)
        assert all(r[0] != "accepted" and "launcher" not in r[1] for r in records.values()), records
        with open(os.path.join(HERE, "wrapper_refusals.json"), "w") as fh:
            json.dump(records, fh, indent=1, sort_keys=True)
    finally:
        for key, val in saved.items():
            if val is None:
                sys.modules.pop(key, None)
            else:
                sys.modules[key] = val


class _GrowingKV:
    """Minimal stand-in for the container class the reference's caches derive from (``mlx_lm``'s
    ``KVCache``, a dependency that is not part of the reference checkout): rows are appended along
    axis 2, ``keys`` / ``values`` hold at least ``offset`` rows, ``trim`` lowers ``offset``. Written
    for this script; it allocates exactly, where the original grows in steps."""

    def __init__(self):
        self.keys = self.values = None
        self.offset = 0

    def update_and_fetch(self, keys, values):
        if self.keys is None:
            self.keys, self.values = np.array(keys), np.array(values)
        else:
            self.keys = np.concatenate([self.keys[..., : self.offset, :], keys], axis=2)
            self.values = np.concatenate([self.values[..., : self.offset, :], values], axis=2)
        self.offset += keys.shape[2]
        return self.keys[..., : self.offset, :], self.values[..., : self.offset, :]

    def trim(self, n):
        n = min(self.offset, n)
        self.offset -= n
        return n

    def is_trimmable(self):
        return True


def _mx_numpy_module():
    """A module object that answers the ``mlx.core`` names ``quantizers/skvq.py`` uses with NumPy
    (float32 arrays stay float32: Python scalars are weak). ``argsort`` is stable, as MLX's is said
    to be (skvq.py:88-89)."""
    import types

    m = types.ModuleType("mlx.core")
    m.float32, m.uint8, m.int32, m.float16 = np.float32, np.uint8, np.int32, np.float16
    class _IsNdarray(type):
        def __instancecheck__(cls, obj):
            return isinstance(obj, np.ndarray)

    class array(metaclass=_IsNdarray):
        """``mx.array`` is a constructor and a type: calls copy into a NumPy array (as an MLX array of an
        array is a copy), ``isinstance(x, mx.array)`` holds for NumPy arrays."""

        def __new__(cls, a, dtype=None):
            return np.array(a, dtype=dtype)

    m.array = array
    m.min = lambda a, axis=None, keepdims=False: np.min(a, axis=axis, keepdims=keepdims)
    m.max = lambda a, axis=None, keepdims=False: np.max(a, axis=axis, keepdims=keepdims)
    m.mean = lambda a, axis=None, keepdims=False: np.mean(a, axis=axis, keepdims=keepdims)
    m.maximum, m.clip, m.round, m.square = np.maximum, np.clip, np.round, np.square
    m.argmin = lambda a, axis=None: np.argmin(a, axis=axis)
    m.argsort = lambda a, axis=-1: np.argsort(a, axis=axis, kind="stable")
    m.broadcast_to, m.take_along_axis, m.concatenate, m.take = np.broadcast_to, np.take_along_axis, np.concatenate, np.take
    m.var = lambda a, axis=None, keepdims=False: np.var(a, axis=axis, keepdims=keepdims)
    m.sum = lambda a, axis=None, keepdims=False: np.sum(a, axis=axis, keepdims=keepdims)
    m.where, m.stack, m.zeros_like, m.arange = np.where, np.stack, np.zeros_like, np.arange
    m.eval = lambda *a: None
    m.compile = lambda f=None, **kw: f
    m.bool_, m.floating, m.issubdtype, m.all = np.bool_, np.floating, np.issubdtype, np.all
    m.moveaxis, m.swapaxes = np.moveaxis, np.swapaxes
    m.repeat = lambda a, repeats, axis=None: np.repeat(a, repeats, axis=axis)

    def softmax(a, axis=-1):
        e = np.exp(a - np.max(a, axis=axis, keepdims=True))
        return e / np.sum(e, axis=axis, keepdims=True)

    m.softmax = softmax
    m.linalg = types.SimpleNamespace(norm=np.linalg.norm)
    m.bfloat16 = object()        # (NumPy has no bfloat16: compares unequal to every dtype)
    m.uint32, m.int8, m.uint16 = np.uint32, np.int8, np.uint16
    m.logical_not, m.logical_and, m.isfinite, m.abs, m.sqrt, m.matmul = np.logical_not, np.logical_and, np.isfinite, np.abs, np.sqrt, np.matmul
    m.zeros = lambda shape, dtype=np.float32: np.zeros(shape, dtype=dtype)
    m.ones = lambda shape, dtype=np.float32: np.ones(shape, dtype=dtype)
    return m


class _NdView(np.ndarray):
    """ndarray with MLX's ``astype`` spelling; used only so that
    ``mx.array(H).astype(dtype)`` at the end of ``walsh_hadamard_matrix`` runs."""

    def astype(self, dtype, *a, **k):  # noqa: D401
        return np.asarray(self, dtype=np.float32)


class _MxShim:
    """Just enough of ``mx`` for ``walsh_hadamard_matrix``'s final cast: the
    matrix itself is built with NumPy inside the reference function."""

    float32 = np.float32

    @staticmethod
    def array(a):
        return np.asarray(a).view(_NdView)


if __name__ == "__main__":
    main()
