"""ctypes binding of ``libvqb200.so`` (the C ABI declared in ``include/vqb200.h``).

There is no CPU fallback: if the shared library is missing, or a call returns a
non-zero status, an exception is raised.
"""

from __future__ import annotations

import ctypes as C
import os
import threading

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libvqb200.so")

VQ_F16, VQ_BF16, VQ_F32 = 0, 1, 2

_DTYPE_CODE = {torch.float16: VQ_F16, torch.bfloat16: VQ_BF16, torch.float32: VQ_F32}

_STATUS_NAME = {
    0: "VQ_OK", -1: "VQ_ERR_SHAPE", -2: "VQ_ERR_DTYPE", -3: "VQ_ERR_ALIGN",
    -4: "VQ_ERR_CAPACITY", -5: "VQ_ERR_ARCH", -6: "VQ_ERR_TIMEOUT", -7: "VQ_ERR_CUDA",
}


class KiviQuantArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("dtype", C.c_int32), ("axis", C.c_int32),
        ("n_bh", C.c_int64), ("n_tok", C.c_int64), ("head_dim", C.c_int64),
        ("x_stride_bh", C.c_int64),
        ("levels", C.c_int32), ("store_bits", C.c_int32), ("group", C.c_int32), ("eps", C.c_float),
        ("codes", C.c_void_p), ("codes_stride_bh", C.c_int64),
        ("scale", C.c_void_p), ("zero", C.c_void_p), ("param_stride_bh", C.c_int64),
        ("recon", C.c_void_p), ("recon_stride_bh", C.c_int64),
    ]


class KiviDequantArgs(C.Structure):
    _fields_ = [
        ("codes", C.c_void_p), ("codes_stride_bh", C.c_int64),
        ("scale", C.c_void_p), ("zero", C.c_void_p), ("param_stride_bh", C.c_int64),
        ("axis", C.c_int32), ("store_bits", C.c_int32), ("group", C.c_int32),
        ("n_bh", C.c_int64), ("n_tok", C.c_int64), ("head_dim", C.c_int64),
        ("out", C.c_void_p), ("out_dtype", C.c_int32), ("out_stride_bh", C.c_int64),
    ]


class KiviAttendArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("out", C.c_void_p),
        ("q_dtype", C.c_int32), ("out_dtype", C.c_int32),
        ("B", C.c_int32), ("H_q", C.c_int32), ("H_kv", C.c_int32), ("S_q", C.c_int32), ("D", C.c_int32),
        ("store_bits", C.c_int32), ("group", C.c_int32), ("n_quant", C.c_int32), ("n_res", C.c_int32),
        ("scale", C.c_float),
        ("k_codes", C.c_void_p), ("k_codes_stride_bh", C.c_int64),
        ("k_scale", C.c_void_p), ("k_zero", C.c_void_p), ("k_param_stride_bh", C.c_int64),
        ("v_codes", C.c_void_p), ("v_codes_stride_bh", C.c_int64),
        ("v_scale", C.c_void_p), ("v_zero", C.c_void_p), ("v_param_stride_bh", C.c_int64),
        ("k_res", C.c_void_p), ("v_res", C.c_void_p), ("res_dtype", C.c_int32), ("res_stride_bh", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64),
        ("n_splits", C.c_int32), ("variant", C.c_int32),
        ("flags", C.c_int32), ("reserved", C.c_int32), ("gather", C.c_void_p), ("sinks", C.c_void_p),
    ]


VQ_ATTEND_OVERLAP_PREVIOUS = 1
VQ_ATTEND_CAUSAL = 2
VQ_MAX_PEERS = 16
(VQ_KNOB_ATTEND_STAGES, VQ_KNOB_ATTEND_WAVES, VQ_KNOB_VQ_SEARCH, VQ_KNOB_ATTEND_WAIT_TEST,
 VQ_KNOB_VQ_WAIT_TEST) = range(5)


class KiviSinks(C.Structure):
    _fields_ = [
        ("k", C.c_void_p), ("v", C.c_void_p), ("k_dead", C.c_void_p), ("count", C.c_void_p),
        ("stride_bh", C.c_int64), ("max_rows", C.c_int32), ("reserved", C.c_int32),
    ]


class PeerGather(C.Structure):
    _fields_ = [
        ("world", C.c_int32), ("rank", C.c_int32), ("n_sources", C.c_int32), ("reserved", C.c_int32),
        ("row_offset", C.c_int64),
        ("out", C.c_void_p * VQ_MAX_PEERS), ("flags", C.c_void_p * VQ_MAX_PEERS), ("state", C.c_void_p),
        ("arrivals", C.c_int32 * VQ_MAX_PEERS),
    ]


class VqAttendArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("out", C.c_void_p), ("q_dtype", C.c_int32), ("out_dtype", C.c_int32),
        ("B", C.c_int32), ("H_q", C.c_int32), ("H_kv", C.c_int32), ("S_q", C.c_int32), ("S_kv", C.c_int32),
        ("D", C.c_int32), ("kv_stride_tok", C.c_int64), ("scale", C.c_float),
        ("causal", C.c_int32), ("sliding_window", C.c_int32),
        ("k_indices", C.c_void_p), ("k_index_bytes", C.c_int32), ("k_codebook", C.c_void_p),
        ("k_n_centroids", C.c_int32), ("k_sub_dim", C.c_int32), ("k_stacked", C.c_int32),
        ("v_mode", C.c_int32), ("v", C.c_void_p), ("v_dtype", C.c_int32), ("v_index_bytes", C.c_int32),
        ("v_codebook", C.c_void_p), ("v_n_centroids", C.c_int32), ("v_sub_dim", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64), ("n_splits", C.c_int32),
    ]


class RabitqAttendArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("out", C.c_void_p), ("q_dtype", C.c_int32), ("out_dtype", C.c_int32),
        ("B", C.c_int32), ("H_q", C.c_int32), ("H_kv", C.c_int32), ("S_q", C.c_int32), ("S_kv", C.c_int32),
        ("D", C.c_int32), ("kv_stride_tok", C.c_int64),
        ("q_scale", C.c_void_p), ("k_bits", C.c_void_p), ("k_mag", C.c_void_p), ("k_const", C.c_void_p),
        ("v_mode", C.c_int32), ("v", C.c_void_p), ("v_dtype", C.c_int32),
        ("v_cents", C.c_void_p), ("n_cents", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64), ("n_splits", C.c_int32),
    ]


class RabitqPrefillArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("out", C.c_void_p), ("q_dtype", C.c_int32), ("out_dtype", C.c_int32),
        ("B", C.c_int32), ("H_q", C.c_int32), ("H_kv", C.c_int32), ("S_q", C.c_int32), ("S_kv", C.c_int32),
        ("D", C.c_int32), ("kv_stride_tok", C.c_int64), ("scale", C.c_float), ("causal", C.c_int32),
        ("k_bits", C.c_void_p), ("k_mag", C.c_void_p), ("k_const", C.c_void_p),
        ("v_mode", C.c_int32), ("v_dtype", C.c_int32), ("v", C.c_void_p), ("v_cents", C.c_void_p),
        ("n_cents", C.c_int32), ("reserved", C.c_int32),
    ]


class VqEncodeArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("x_dtype", C.c_int32), ("n_tok", C.c_int64), ("D", C.c_int32), ("sub_dim", C.c_int32),
        ("tok_per_head", C.c_int64), ("n_heads", C.c_int32), ("codebook", C.c_void_p),
        ("n_centroids", C.c_int32), ("stacked_codebooks", C.c_int32), ("H", C.c_void_p),
        ("smooth", C.c_void_p), ("smooth_rows", C.c_int32), ("x_hat", C.c_void_p), ("hat_dtype", C.c_int32),
        ("indices", C.c_void_p), ("index_bytes", C.c_int32),
    ]


class SkvqQuantArgs(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("x_stride_bh", C.c_int64), ("perm", C.c_void_p), ("codes", C.c_void_p), ("lo", C.c_void_p),
        ("scale", C.c_void_p), ("q_stride_bh", C.c_int64), ("alphas", C.c_float * 8), ("n_alphas", C.c_int32),
        ("x_dtype", C.c_int32), ("n_bh", C.c_int32), ("n_heads", C.c_int32), ("n_tok", C.c_int32), ("D", C.c_int32),
        ("bits", C.c_int32), ("group_size", C.c_int32),
    ]


class SkvqDequantArgs(C.Structure):
    _fields_ = [
        ("codes", C.c_void_p), ("lo", C.c_void_p), ("scale", C.c_void_p), ("q_stride_bh", C.c_int64),
        ("inv_perm", C.c_void_p), ("out", C.c_void_p), ("out_stride_bh", C.c_int64), ("out_dtype", C.c_int32),
        ("n_bh", C.c_int32), ("n_heads", C.c_int32), ("n_tok", C.c_int32), ("D", C.c_int32), ("bits", C.c_int32),
        ("group_size", C.c_int32), ("reserved", C.c_int32),
    ]


# name -> (restype, argtypes); every symbol include/vqb200.h declares.
SIGNATURES = {
    "vq_version": (C.c_int32, []),
    "vq_last_error": (C.c_char_p, []),
    "vq_tune": (C.c_int32, [C.c_int32, C.c_int32]),
    "vq_peer_gather_wait": (C.c_int32, [C.POINTER(PeerGather), C.c_void_p]),
    "vq_peer_export": (C.c_int32, [C.c_void_p, C.c_void_p, C.POINTER(C.c_int64)]),
    "vq_peer_open": (C.c_int32, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "vq_peer_close": (C.c_int32, [C.c_void_p]),
    "vq_kivi_quantize": (C.c_int32, [C.POINTER(KiviQuantArgs), C.c_void_p]),
    "vq_kivi_quantize_pack": (C.c_int32, [C.POINTER(KiviQuantArgs), C.c_void_p]),
    "vq_kivi_quant_dequant": (C.c_int32, [C.POINTER(KiviQuantArgs), C.c_void_p]),
    "vq_kivi_append": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                   C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "vq_kivi_dequant": (C.c_int32, [C.POINTER(KiviDequantArgs), C.c_void_p]),
    "vq_predecoded_attend": (C.c_int32, [C.POINTER(KiviAttendArgs), C.c_void_p]),
    "vq_lse_merge": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_void_p, C.c_int32,
                                 C.c_void_p]),
    "vq_vq_encode_decode_keys": (C.c_int32, [C.POINTER(VqEncodeArgs), C.c_void_p]),
    "vq_vq_encode_decode_values": (C.c_int32, [C.POINTER(VqEncodeArgs), C.c_void_p]),
    "vq_kivi_attend_workspace_bytes": (C.c_int64, [C.POINTER(KiviAttendArgs)]),
    "vq_kivi_attend_splits": (C.c_int32, [C.POINTER(KiviAttendArgs)]),
    "vq_kivi_decode_attend": (C.c_int32, [C.POINTER(KiviAttendArgs), C.c_void_p]),
    "vq_kivi_attend_status": (C.c_int32, []),
    "vq_kivi_decode_attend_static": (C.c_int32, [C.POINTER(KiviAttendArgs), C.c_void_p]),
    "vq_vq_quantize": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_void_p, C.c_int32, C.c_int32,
                                   C.c_void_p, C.c_int32, C.c_void_p]),
    "vq_vq_quantize_status": (C.c_int32, []),
    "vq_vq_dequant": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int64, C.c_void_p, C.c_int32, C.c_int32, C.c_int32,
                                  C.c_void_p, C.c_int32, C.c_void_p]),
    "vq_vq_dual_transform": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_int64, C.c_int32, C.c_void_p,
                                         C.c_int32, C.c_int32, C.c_float, C.c_void_p, C.c_void_p]),
    "vq_vq_attend_workspace_bytes": (C.c_int64, [C.POINTER(VqAttendArgs)]),
    "vq_vq_decode_attend": (C.c_int32, [C.POINTER(VqAttendArgs), C.c_void_p]),
    "vq_rabitq_encode": (C.c_int32, [C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_void_p, C.c_int32,
                                     C.c_void_p, C.c_void_p, C.c_void_p]),
    "vq_rabitq_pack_values": (C.c_int32, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "vq_rabitq_hamming_score": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_float,
                                            C.c_void_p, C.c_void_p, C.c_void_p]),
    "vq_rabitq_attend_workspace_bytes": (C.c_int64, [C.POINTER(RabitqAttendArgs)]),
    "vq_rabitq_decode_attend": (C.c_int32, [C.POINTER(RabitqAttendArgs), C.c_void_p]),
    "vq_rabitq_prefill_attend": (C.c_int32, [C.POINTER(RabitqPrefillArgs), C.c_void_p]),
    "vq_rvq_quant_pack": (C.c_int32, [C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                      C.c_void_p, C.c_void_p, C.c_void_p]),
    "vq_rvq_build_table": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p]),
    "vq_rvq_unpack_decode": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p,
                                         C.c_int32, C.c_int32, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "vq_skvq_quantize_pack": (C.c_int32, [C.POINTER(SkvqQuantArgs), C.c_void_p]),
    "vq_skvq_unpack_dequant": (C.c_int32, [C.POINTER(SkvqDequantArgs), C.c_void_p]),
    "vq_bit_pack": (C.c_int32, [C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p]),
    "vq_bit_unpack": (C.c_int32, [C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_void_p]),
}

_lib = None
_lock = threading.Lock()


class VQLibraryError(RuntimeError):
    """The native library is missing or a native call failed."""


def lib() -> C.CDLL:
    """Load (once) and return the bound library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise VQLibraryError(
                    f"{LIB_PATH} not found: build it with `python -m veloxquant_mlx_b200.build` "
                    "(there is no CPU fallback)"
                )
            handle = C.CDLL(LIB_PATH)
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(handle, name)
                fn.restype = res
                fn.argtypes = args
            _lib = handle
    return _lib


def check(status: int, what: str) -> None:
    """Raise on a non-zero vq_status: ValueError for argument problems, RuntimeError otherwise."""
    if status == 0:
        return
    msg = lib().vq_last_error().decode("utf-8", "replace")
    text = f"{what}: {_STATUS_NAME.get(status, status)}: {msg}"
    if status in (-1, -2, -3):
        raise ValueError(text)
    raise VQLibraryError(text)


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dt]
    except KeyError:
        raise ValueError(f"unsupported dtype {dt}; expected float16, bfloat16 or float32") from None


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr(device: torch.device) -> int:
    """The current stream of ``device`` as a raw ``cudaStream_t`` value. (Through the raw accessor
    where PyTorch has it: building a ``torch.cuda.Stream`` object per kernel launch costs several
    microseconds, more than the launch itself.)"""
    if _raw_stream is not None:
        idx = device.index
        return _raw_stream(torch.cuda.current_device() if idx is None else idx)
    return torch.cuda.current_stream(device).cuda_stream


class _NoGuard:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def on_device(device: torch.device):
    """Context that makes ``device`` current for a library call; free when it already is (the
    device guard object costs more than a kernel launch)."""
    idx = device.index
    if idx is None or idx == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(idx)


def require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise VQLibraryError(
            f"{name} must be a CUDA tensor: this package runs on sm_100a only and has no CPU path"
        )
