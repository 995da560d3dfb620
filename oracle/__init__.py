"""CPU oracle for the compressed-KV hot path (TEST INFRASTRUCTURE, not product).

Every function here is a NumPy restatement of the reference's algorithm for
quantize-on-append and fused dequant-SDPA decode (KIVI group-affine codes,
VecInfer ``quantize_vq`` indices, RaBitQ sign bits). Each function cites the
reference file:line it follows (paths are relative to the reference project's
root).

Only the test suite, the smoke check and the CPU-baseline leg of the benchmark
may import this package; it is the checker, never the thing measured as the
product and never a fallback for a missing CUDA extension.

Pinning status (what anchors these restatements to the reference itself):

* ``bitpack``  -- pinned: fixtures produced by executing the reference's own
  ``dsa/bit_pack.py`` plus its known-answer vector
  ``[0,1,2,3,0,1,2,3] @ 2 bit -> [228, 228]``.
* ``kivi``     -- pinned: fixtures produced by executing the NumPy functions
  ``_quant_keys/_quant_values/_reference_attend`` that the reference ships in
  ``veloxquant_mlx/tests/metal/test_scalar_attend.py``; the reference's own
  tests pin those bit-for-bit to its MLX path and Metal kernels.
* ``rabitq``   -- pinned: fixtures from the reference's ``_wht_butterfly/
  _reference_encode/_reference_attend/_pack_np`` test functions and from
  ``math/rotation.py`` executed here.
* ``vq``       -- ``quantize_vq`` and the attention oracle are pinned by the
  reference's own functions executed with NumPy answering ``mlx.core``
  (``tests/golden/vq.npz``). What stays open ("parity unpinned" at the bit
  level) is MLX's own reduction order, which is not installable here; the
  oracle fixes the summation order of ``vecinfer_quantize.metal`` (sequential
  over the sub-vector, unfused multiply/add, lowest index wins ties).
* ``rvq``      -- pinned: codebooks from the reference's Lloyd-Max modules;
  the quantizer's ``encode`` / ``decode`` and the cache class executed over
  the same stand-in (``tests/golden/rvq_reference.npz``), bit for bit.
* ``skvq``, ``kitty``, ``age_tiered``, ``kivi_sink`` -- pinned: the
  reference's quantizer modules and cache classes executed over the stand-in
  (``tests/golden/skvq.npz``, ``group_quant.npz``, ``cache_traces.npz``).
"""

from . import bitpack, kivi, rabitq, vq  # noqa: F401
