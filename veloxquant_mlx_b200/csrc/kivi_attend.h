// Internal interface between the attend entry point and the tensor-core kernel.
#pragma once
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
int32_t kivi_attend_mma_launch(const vq_kivi_attend_args &a, const DeviceInfo &di, cudaStream_t st);
// Combine per-split partial softmaxes written as part_o[(row*n_splits+s)*D + d] (natural-exp
// domain, unnormalised) and part_ml[(row*n_splits+s)*2 + {0: max, 1: sum}] into out[row*D + d].
int32_t launch_split_merge(const float *part_o, const float *part_ml, int n_splits, int D, void *out,
                           int out_dtype, int64_t rows, cudaStream_t st);
}  // namespace vq
