"""B200-native compressed-KV hot path: quantize-on-append and fused dequant-SDPA decode.

Hand-written sm_100a CUDA kernels behind a C ABI (``libvqb200.so``, declared in
``include/vqb200.h``), called through ``ctypes`` with ``torch.Tensor`` containers, behind
the reference's ``KVCacheConfig(method=...)`` / cache / kernel-wrapper interface for the
KIVI, VecInfer and RaBitQ paths. There is no CPU fallback.
"""

from . import kernels, rabitq, vecinfer  # noqa: F401
from ._lib import VQLibraryError, lib  # noqa: F401

__version__ = "0.1.0"
