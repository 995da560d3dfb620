"""Build libvqb200.so in-tree with nvcc for sm_100a.

    python -m veloxquant_mlx_b200.build [--force] [--verbose]

The shared library is written next to this file so that it travels with a source
snapshot; nothing is installed into site-packages.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libvqb200.so")
OBJ_DIR = os.path.join(HERE, "build")

# (source, extra flags). The quantizers are compiled without FMA contraction so that
# code*scale+zero stays two separately rounded float32 operations.
SOURCES = [
    ("api.cu", []),
    ("bitpack.cu", []),
    ("kivi_quant.cu", ["-fmad=false"]),
    ("kivi_quant_tile.cu", ["-fmad=false"]),
    ("kivi_attend.cu", []),
    ("kivi_attend_mma.cu", []),
    ("kivi_attend_static.cu", []),
    ("peer_gather.cu", []),
    ("vq_quant.cu", ["-fmad=false"]),
    ("vq_encode.cu", ["-fmad=false"]),
    ("vq_transform.cu", ["-fmad=false"]),
    ("vq_quant_mma.cu", []),
    ("vq_quant_tc5.cu", []),
    ("rabitq.cu", ["-fmad=false"]),
    ("coded_attend.cu", []),
    ("rabitq_prefill.cu", []),
    ("rvq.cu", []),
    ("skvq.cu", ["-fmad=false"]),
]

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]


def nvcc_path() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
    return cand


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    nvcc = nvcc_path()
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(os.path.dirname(HERE), "include", "vqb200.h"))
    objs = []
    for src, extra in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _stale(o, [s] + headers):
            cmd = [nvcc, *ARCH, *COMMON, *extra, "-c", s, "-o", o]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
                print(" ".join(cmd), flush=True)
            subprocess.run(cmd, check=True)
    if force or _stale(OUT, objs):
        cmd = [nvcc, *ARCH, "-shared", "-o", OUT, *objs]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
    sys.exit(0)
