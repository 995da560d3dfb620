"""Calls the kernel wrappers must REFUSE, run against BOTH the reference's wrappers (by make_golden.py,
over a NumPy stand-in for ``mlx.core`` whose kernel launcher is never reached) and this package's (by
tests/test_wrapper_validation_cpu.py, on CPU tensors: every check comes before the device check). Each
scenario records the exception type and message, so the two can be compared entry by entry."""

import numpy as np


def _attempt(fn, *args, **kwargs):
    try:
        fn(*args, **kwargs)
    except Exception as e:  # noqa: BLE001
        return [type(e).__name__, str(e)]
    return ["accepted", ""]


def refusal_scenarios(ns, arr):
    """``ns``: an object carrying the wrappers by their reference names; ``arr(ndarray)`` makes the
    side's array type. Returns ``{name: [exception type, message]}``."""
    f16, f32, u8, u32 = np.float16, np.float32, np.uint8, np.uint32
    z = lambda shape, dt: arr(np.zeros(shape, dt))  # noqa: E731
    out = {}

    # ---- scalar_fused_decode_attend / _batched ------------------------------------------------
    B, Hq, Hkv, D, g, S = 2, 8, 2, 64, 32, 64

    def attend_args(**o):
        d = dict(q=z((B, Hq, 1, D), f16), k_codes=z((B, Hkv, S, D), u8), k_scale=z((B, Hkv, S // g, D), f32),
                 k_zero=z((B, Hkv, S // g, D), f32), v_codes=z((B, Hkv, S, D), u8), v_scale=z((B, Hkv, S, D // g), f32),
                 v_zero=z((B, Hkv, S, D // g), f32))
        d.update(o)
        return [d[k] for k in ("q", "k_codes", "k_scale", "k_zero", "v_codes", "v_scale", "v_zero")]

    bad = {"q_3d": dict(q=z((Hq, 1, D), f16)), "codes_3d": dict(k_codes=z((Hkv, S, D), u8)), "d_512": dict(q=z((B, Hq, 1, 512), f16)),
           "batch": dict(k_codes=z((3, Hkv, S, D), u8)), "head_dim": dict(k_codes=z((B, Hkv, S, 32), u8)),
           "kv_heads": dict(v_codes=z((B, 4, S, D), u8)), "gqa": dict(q=z((B, 7, 1, D), f16)),
           "heads_per_kv": dict(q=z((B, Hkv * 64, 1, D), f16))}
    for tag, o in bad.items():
        out["attend_" + tag] = _attempt(ns.scalar_fused_decode_attend, *attend_args(**o), g, 0.1)
    for nsg in (0, 33):
        out[f"attend_nsg_{nsg}"] = _attempt(ns.scalar_fused_decode_attend, *attend_args(), g, 0.1, nsg)

    # ---- kivi_group_quant_dequant -------------------------------------------------------------
    x = z((1, 2, 64, 32), f16)
    out["kivi_axis"] = _attempt(ns.kivi_group_quant_dequant, x, 0, 32, 3)
    out["kivi_group_0"] = _attempt(ns.kivi_group_quant_dequant, x, -1, 0, 3)
    out["kivi_levels_0"] = _attempt(ns.kivi_group_quant_dequant, x, -1, 32, 0)

    # ---- rabitq ---------------------------------------------------------------------------------
    out["rabitq_encode_1d"] = _attempt(ns.rabitq_encode, z((128,), f16), z((128,), f32))
    out["rabitq_encode_d_100"] = _attempt(ns.rabitq_encode, z((4, 100), f16), z((100,), f32))
    out["rabitq_encode_diag"] = _attempt(ns.rabitq_encode, z((4, 128), f16), z((64,), f32))
    out["rabitq_values_odd"] = _attempt(ns.rabitq_pack_values, z((4, 7), u8))
    out["rabitq_hamming_q_2d"] = _attempt(ns.rabitq_hamming_score, z((1, 16), u8), z((5, 16), u8), z((5,), f32), z((1,), f32))
    out["rabitq_hamming_bits_1d"] = _attempt(ns.rabitq_hamming_score, z((16,), u8), z((80,), u8), z((5,), f32), z((1,), f32))
    out["rabitq_hamming_width"] = _attempt(ns.rabitq_hamming_score, z((8,), u8), z((5, 16), u8), z((5,), f32), z((1,), f32))

    # ---- rvq ------------------------------------------------------------------------------------
    c, b = z((4,), f16), z((3,), f16)
    out["rvq_pack_1d"] = _attempt(ns.rvq_quant_pack, z((128,), f16), c, b, b, 2)
    out["rvq_pack_bits_3"] = _attempt(ns.rvq_quant_pack, z((4, 128), f16), c, b, b, 3)
    out["rvq_pack_bits_0"] = _attempt(ns.rvq_quant_pack, z((4, 128), f16), c, b, b, 0)
    out["rvq_pack_tables"] = _attempt(ns.rvq_quant_pack, z((4, 128), f16), z((3,), f16), b, b, 2)
    out["rvq_decode_d_96"] = _attempt(ns.rvq_unpack_decode, z((4, 6), u32), z((4, 6), u32), z((4,), f32), c, c, z((96,), f32), 2, 96)
    out["rvq_decode_words"] = _attempt(ns.rvq_unpack_decode, z((4, 7), u32), z((4, 7), u32), z((4,), f32), c, c, z((128,), f32), 2, 128)

    # ---- vecinfer -------------------------------------------------------------------------------
    cb = z((16, 4), f32)
    out["vq_quantize_width"] = _attempt(ns.vecinfer_quantize_metal, z((8, 30), f16), cb, 4)
    out["vq_quantize_sub_dim"] = _attempt(ns.vecinfer_quantize_metal, z((8, 32), f16), cb, 8)
    out["vq_quantize_codebook_1d"] = _attempt(ns.vecinfer_quantize_metal, z((8, 32), f16), z((16,), f32), 4)
    q = z((1, 2, 1, 32), f32)
    ki, vi = z((1, 2, 10, 8), u32), z((1, 2, 10, 4), u32)
    vcb = z((16, 8), f32)
    out["vq_sdpa_k_width"] = _attempt(ns.metal_fused_sdpa, q, z((1, 2, 10, 7), u32), cb, vi, vcb, 0.1)
    out["vq_sdpa_gqa"] = _attempt(ns.metal_fused_sdpa, z((1, 3, 1, 32), f32), ki, cb, vi, vcb, 0.1)
    return out
