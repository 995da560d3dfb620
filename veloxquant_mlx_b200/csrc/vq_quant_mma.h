// Internal interface between vq_vq_quantize and the tensor-core search.
#pragma once
#include "common.cuh"

namespace vq {
// True when the tensor-core search can take this call (sub_dim 4 or 8, 2..2048 centroids,
// enough rows; one shared codebook or one per sub-space). VQ_VQ_SEARCH=exact|mma|tc5 in the environment pins the choice.
bool vq_quantize_mma_supported(const void *x, int32_t x_dtype, int64_t n, int32_t sub_dim, int32_t n_c, int32_t n_sub);
int32_t vq_quantize_mma_launch(const void *x, int32_t x_dtype, int64_t n, int32_t sub_dim, const float *cb, int32_t n_c,
                               int32_t n_sub, void *indices, int32_t index_bytes, cudaStream_t st);
// tcgen05 + tensor-memory search (vq_quant_tc5.cu): f16 or bf16 input, sub_dim 8, 16..256 centroids in
// multiples of 16, one shared codebook or one per sub-space, >= 4096 sub-vectors. Tried first.
bool vq_quantize_tc5_supported(const void *x, int32_t x_dtype, int64_t n, int32_t sub_dim, int32_t n_c, int32_t n_sub);
int32_t vq_quantize_tc5_launch(const void *x, int32_t x_dtype, int64_t n, const float *cb, int32_t n_c, int32_t n_sub,
                               void *indices, int32_t index_bytes, cudaStream_t st);
// Reads and clears the "a bounded wait gave up" flag of that kernel (synchronises the device).
int32_t vq_quantize_tc5_take_timeout(int *flag);
}  // namespace vq
