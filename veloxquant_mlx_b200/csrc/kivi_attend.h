// Internal interface between the attend entry point and the tensor-core kernel.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace vq {
// NULL when the tensor-core kernel can run `a`; otherwise a static string saying why not.
const char *kivi_attend_mma_supported(const vq_kivi_attend_args &a);
// Context splits the tensor-core kernel will use for `a` (for workspace sizing).
int kivi_attend_mma_splits(const vq_kivi_attend_args &a, const DeviceInfo &di);
// Workspace bytes of the tensor-core kernel for `a` with `n_splits` context splits.
int64_t kivi_attend_mma_workspace(const vq_kivi_attend_args &a, int n_splits);
// Reads and clears the device-side "a bounded wait gave up" flag (synchronises the device).
int32_t kivi_attend_mma_take_timeout(int *flag);
// The same flag of the staged RaBitQ attend kernel (coded_attend.cu).
int32_t coded_attend_take_timeout(int *flag);
// The same flag of the peer-arrival wait kernel (peer_gather.cu).
int32_t peer_gather_take_timeout(int *flag);
// A per-(batch, kv head) array of `rows` rows of `row_bytes` bytes (slabs `stride_bh_bytes` apart) as a
// rank-3 byte tensor map whose boxes of `box_rows` x `box_bytes` (<= 128) are stored with the 128-byte
// swizzle. Encodings are cached per `slot` (0..3: one per use) and thread.
int32_t make_rows_map(int slot, const void *base, int64_t row_bytes, int64_t rows, int64_t stride_bh_bytes, int32_t n_bh,
                      int32_t box_bytes, int32_t box_rows, CUtensorMap *map);
int32_t kivi_attend_mma_launch(const vq_kivi_attend_args &a, const DeviceInfo &di, cudaStream_t st);
// Combine per-split partial softmaxes written as part_o[(row*n_splits+s)*D + d] (natural-exp
// domain, unnormalised) and part_ml[(row*n_splits+s)*2 + {0: max, 1: sum}] into out[row*D + d].
int32_t launch_split_merge(const float *part_o, const float *part_ml, int n_splits, int D, void *out,
                           int out_dtype, int64_t rows, cudaStream_t st);
}  // namespace vq
