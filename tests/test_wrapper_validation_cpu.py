"""Argument validation of the kernel wrappers happens on the host, before any pointer reaches
the native library: a wrong-shaped output or a too-short parameter buffer must be a
``ValueError``, never an out-of-bounds device access. None of these calls needs a GPU (the
checks come before the device check)."""

from __future__ import annotations

import pytest
import torch

from veloxquant_mlx_b200 import kernels as k

B, H_q, H_kv, D, g, bits, cap = 2, 8, 2, 128, 32, 4, 64


def _attend_inputs():
    rb = D * bits // 8
    return dict(
        q=torch.zeros(B, H_q, 1, D, dtype=torch.float16),
        k_codes=torch.zeros(B, H_kv, cap, rb, dtype=torch.uint8),
        k_scale=torch.ones(B, H_kv, cap // g, D), k_zero=torch.zeros(B, H_kv, cap // g, D),
        v_codes=torch.zeros(B, H_kv, cap, rb, dtype=torch.uint8),
        v_scale=torch.ones(B, H_kv, cap, D // g), v_zero=torch.zeros(B, H_kv, cap, D // g),
    )


def _call(t, **kw):
    return k.kivi_decode_attend(t["q"], t["k_codes"], t["k_scale"], t["k_zero"], t["v_codes"], t["v_scale"],
                                t["v_zero"], g, 0.1, store_bits=bits, **kw)


def test_well_formed_cpu_call_reaches_the_device_check_only():
    from veloxquant_mlx_b200 import VQLibraryError

    with pytest.raises(VQLibraryError, match="must be a CUDA tensor"):
        _call(_attend_inputs())


@pytest.mark.parametrize("mutate,match", [
    (lambda t: t.update(out=torch.zeros(B, H_q, 1, D // 2, dtype=torch.float16)), "out must be a contiguous"),
    (lambda t: t.update(out=torch.zeros(B, H_q, 2, D, dtype=torch.float16)[:, :, :1]), "out must be a contiguous"),
    (lambda t: t.update(out=torch.zeros(B, H_q, 1, D, dtype=torch.int32)), "unsupported out dtype"),
    (lambda t: t.update(k_scale=t["k_scale"][:, :, :1], k_zero=t["k_zero"][:, :, :1]), "k_scale/k_zero"),
    (lambda t: t.update(k_zero=t["k_zero"][:, :, :1]), "k_scale/k_zero"),
    (lambda t: t.update(k_scale=t["k_scale"][..., :64], k_zero=t["k_zero"][..., :64]), "k_scale/k_zero"),
    (lambda t: t.update(v_scale=t["v_scale"][:, :, :32], v_zero=t["v_zero"][:, :, :32]), "v_scale/v_zero"),
    (lambda t: t.update(v_scale=t["v_scale"][..., :2], v_zero=t["v_zero"][..., :2]), "v_scale/v_zero"),
    (lambda t: t.update(v_codes=t["v_codes"][:1]), "v_codes shape"),
    (lambda t: t.update(v_codes=t["v_codes"][..., :32]), "v_codes shape"),
    (lambda t: t.update(k_scale=t["k_scale"].double()), "k_scale must be a float32"),
    (lambda t: t.update(k_codes=t["k_codes"].to(torch.int8)), "must be uint8"),
    (lambda t: t.update(gather=object()), "gather must be"),
])
def test_decode_attend_rejects_malformed_buffers_before_any_launch(mutate, match):
    t = _attend_inputs()
    extra = {}
    probe = dict(t)
    mutate(probe)
    for key in ("out", "gather"):
        if key in probe:
            extra[key] = probe.pop(key)
    with pytest.raises(ValueError, match=match):
        _call(probe, **extra)


def test_decode_attend_rejects_bad_residual_rows():
    t = _attend_inputs()
    res = torch.zeros(B, H_kv, 16, D, dtype=torch.float16)
    with pytest.raises(ValueError, match="exceed the residual buffers"):
        _call(t, k_res=res, v_res=res, n_res=10, res_offset=8)
    with pytest.raises(ValueError, match="k_res / v_res must be"):
        _call(t, k_res=res[:1], v_res=res[:1])


def test_quantize_into_rejects_buffers_of_another_batch_or_head_count():
    x = torch.zeros(B, H_kv, 32, D, dtype=torch.float16)
    codes = torch.zeros(B, H_kv, 64, D * bits // 8, dtype=torch.uint8)
    scale = torch.zeros(B, H_kv, 2, D)
    with pytest.raises(ValueError, match="leading"):
        k.kivi_quantize_into(x, -2, g, bits, codes=codes[:1], scale=scale, zero=scale.clone())
    with pytest.raises(ValueError, match="leading"):
        k.kivi_quantize_into(x, -2, g, bits, codes=codes, scale=scale[:, :1].contiguous(), zero=scale[:, :1].clone())
    with pytest.raises(ValueError, match="contiguous uint8"):
        k.kivi_quantize_into(x, -2, g, bits, codes=codes[..., :32], scale=scale, zero=scale.clone())


def test_dual_transforms_and_lut_follow_the_reference_functions_on_every_smooth_convention():
    """The host-side ``apply_dual_transform_keys`` / ``_queries`` / ``compute_query_lut`` on CPU tensors
    against the reference's own functions executed over a NumPy stand-in
    (``tests/golden/vq_transform.npz``): same outputs, dtypes and shapes on every way the smooth factors
    broadcast, and a ``ValueError`` on every shape the reference rejects."""
    import os

    import numpy as np

    from veloxquant_mlx_b200 import vecinfer as vi

    z = np.load(os.path.join(os.path.dirname(__file__), "golden", "vq_transform.npz"))
    H = torch.from_numpy(z["H"])
    assert torch.equal(vi.walsh_hadamard_matrix(32), H)
    fns = {"keys": vi.apply_dual_transform_keys, "queries": vi.apply_dual_transform_queries}
    n_ok = n_rejected = 0
    for row in z["table"]:
        tag, res = str(row).split(":")
        short, xn, sn = tag.split("_")
        sm = {"badwidth": np.ones((2, 33), np.float32), "smooth3d": np.ones((1, 2, 32), np.float32)}.get(sn)
        sm = torch.from_numpy(z["in_" + sn] if sm is None else sm)
        x = torch.from_numpy(z["in_" + xn])
        if res == "ValueError":
            with pytest.raises(ValueError):
                fns[short](x, sm, H)
            n_rejected += 1
            continue
        got, want = fns[short](x, sm, H).numpy(), z[tag]
        assert got.dtype == want.dtype and got.shape == want.shape, tag
        np.testing.assert_allclose(got.astype(np.float32), want.astype(np.float32), rtol=0,
                                   atol=1e-5 if want.dtype == np.float32 else 2e-2, err_msg=tag)
        n_ok += 1
    assert n_ok == 48 and n_rejected == 4
    cb = torch.from_numpy(z["lut_codebook"])
    for name in ("q4", "q3"):
        np.testing.assert_allclose(vi.compute_query_lut(torch.from_numpy(z["in_" + name]), cb, 4).numpy(), z["lut_" + name], rtol=0, atol=1e-6)
    with pytest.raises(ValueError) as e:
        vi.compute_query_lut(torch.from_numpy(z["in_q4"]), torch.ones(16, 5), 5)
    assert str(e.value) == str(z["lut_bad"])


def test_every_wrapper_takes_the_reference_wrappers_arguments_in_their_order():
    """``tests/golden/wrapper_signatures.json`` holds the parameter lists of the reference's kernel
    wrappers and VecInfer functions on this path, read from its source. Each one exists here under the
    same name, is importable from the single ``kernels`` module as in the reference
    (``metal/kernels.py``), takes the same positional parameters in the same order (extra parameters
    may only follow, with defaults), knows every keyword-only name, and requires no argument the
    reference gives a default."""
    import inspect
    import json
    import os

    from veloxquant_mlx_b200 import integration, vecinfer

    with open(os.path.join(os.path.dirname(__file__), "golden", "wrapper_signatures.json")) as fh:
        ref = json.load(fh)
    assert len(ref) == 26
    for name, spec in ref.items():
        if spec["file"].startswith("metal/_") or name == "metal_fused_sdpa":
            fn = getattr(k, name)                                   # the reference's one import point
        else:
            fn = getattr(vecinfer, name, None) or getattr(integration, name)
        params = list(inspect.signature(fn).parameters.values())
        positional = [p for p in params if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
        names = [p.name for p in positional]
        n = len(spec["positional"])
        assert names[:n] == spec["positional"], (name, names, spec["positional"])
        required = n - spec["n_defaults"]
        assert all(p.default is not p.empty for p in positional[required:]), (name, "a required argument the reference defaults")
        accepted = {p.name for p in params}
        assert set(spec["keyword_only"]) <= accepted, (name, spec["keyword_only"])
        assert all(p.default is not p.empty for p in params if p.kind == p.KEYWORD_ONLY), name
    assert k.rvq_quant_pack.__module__.endswith(".rvq") and k.rabitq_encode.__module__.endswith(".rabitq")
    with pytest.raises(AttributeError):
        k.no_such_wrapper
    assert vecinfer.supports_shape(256, 16, 128) and vecinfer.supports_shape(n_centroids=256, n_sub=32, head_dim=256)
    assert not vecinfer.supports_shape(256, 16, 100) and not vecinfer.supports_shape(256, 16, 512)
    assert not vecinfer.supports_shape(4096, 32, 128) and not vecinfer.supports_shape(0, 16, 128)
    with pytest.raises(ValueError, match="one constant per candidate"):
        k.rabitq_hamming_score(torch.zeros(2, dtype=torch.uint8), torch.zeros(5, 2, dtype=torch.uint8), 0.25, torch.zeros(5))


def test_wrappers_refuse_what_the_reference_wrappers_refuse_with_the_same_words():
    """31 calls the reference's wrappers refuse before any launch (wrong ranks, head counts that do not
    group, widths a sub-vector does not divide, table sizes that do not fit the bit width, ...), recorded
    by make_golden.py from the reference's own wrapper modules executed over a NumPy stand-in
    (``tests/golden/wrapper_refusals.json``): the wrappers here raise the same exception type with the
    same message on CPU tensors, i.e. before the device is looked at."""
    import importlib.util
    import json
    import os

    here = os.path.join(os.path.dirname(__file__), "golden")
    spec = importlib.util.spec_from_file_location("wrapper_scenarios", os.path.join(here, "wrapper_scenarios.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    with open(os.path.join(here, "wrapper_refusals.json")) as fh:
        ref = json.load(fh)
    mine = mod.refusal_scenarios(k, torch.from_numpy)
    assert set(mine) == set(ref) and len(ref) == 31
    for name, record in ref.items():
        assert mine[name] == record, (name, mine[name], record)
