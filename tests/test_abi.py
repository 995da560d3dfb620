"""The C-ABI library loads and exports every symbol that include/vqb200.h declares.
No compute call is made here (no GPU needed)."""

from __future__ import annotations

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built_lib():
    from veloxquant_mlx_b200 import build

    return build.build()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "vqb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vq_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_symbols():
    syms = _declared_symbols()
    assert "vq_kivi_decode_attend" in syms and "vq_kivi_quantize" in syms and len(syms) >= 8


def test_library_exports_every_declared_symbol(built_lib):
    handle = ctypes.CDLL(built_lib)
    for name in _declared_symbols():
        assert hasattr(handle, name), f"{name} declared in vqb200.h but not exported"


def test_binding_table_matches_header(built_lib):
    from veloxquant_mlx_b200 import _lib

    assert sorted(_lib.SIGNATURES) == _declared_symbols()
    lib = _lib.lib()
    assert lib.vq_version() >= 100
    assert isinstance(lib.vq_last_error(), bytes)


def test_struct_sizes_match_header(built_lib, tmp_path):
    """Compile a tiny C program against the header and compare sizeof() with ctypes."""
    import subprocess

    from veloxquant_mlx_b200 import _lib

    src = tmp_path / "sz.c"
    src.write_text(
        '#include <stdio.h>\n#include "vqb200.h"\nint main(){printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\\n",'
        "sizeof(vq_kivi_quant_args),sizeof(vq_kivi_dequant_args),sizeof(vq_kivi_attend_args),"
        "sizeof(vq_vq_attend_args),sizeof(vq_rabitq_attend_args),sizeof(vq_vq_encode_args),"
        "sizeof(vq_peer_gather),sizeof(vq_rabitq_prefill_args),sizeof(vq_kivi_sinks),"
        "sizeof(vq_skvq_quant_args),sizeof(vq_skvq_dequant_args));return 0;}\n"
    )
    exe = tmp_path / "sz"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()
    got = [ctypes.sizeof(t) for t in (_lib.KiviQuantArgs, _lib.KiviDequantArgs, _lib.KiviAttendArgs,
                                      _lib.VqAttendArgs, _lib.RabitqAttendArgs, _lib.VqEncodeArgs, _lib.PeerGather,
                                      _lib.RabitqPrefillArgs, _lib.KiviSinks, _lib.SkvqQuantArgs, _lib.SkvqDequantArgs)]
    assert [int(v) for v in out] == got


def test_cpu_tensor_is_rejected_loudly(built_lib):
    import torch

    from veloxquant_mlx_b200 import VQLibraryError, kernels

    with pytest.raises(VQLibraryError):
        kernels.kivi_group_quant_dequant(torch.zeros(1, 1, 32, 8), -1, 32, 3)
    with pytest.raises(ValueError, match="axis must be -1 or -2"):
        kernels.kivi_group_quant_dequant(torch.zeros(1, 1, 32, 8), 0, 32, 3)
