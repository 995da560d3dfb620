// Internal interface between the attend entry point and the tensor-core kernel.
#pragma once
#include "common.cuh"

namespace vq {
// NULL when the tensor-core kernel can run `a`; otherwise a static string saying why not.
const char *kivi_attend_mma_supported(const vq_kivi_attend_args &a);
// Context splits the tensor-core kernel will use for `a` (for workspace sizing).
int kivi_attend_mma_splits(const vq_kivi_attend_args &a, const DeviceInfo &di);
// Reads and clears the device-side "a bounded wait gave up" flag (synchronises the device).
int32_t kivi_attend_mma_take_timeout(int *flag);
int32_t kivi_attend_mma_launch(const vq_kivi_attend_args &a, const DeviceInfo &di, cudaStream_t st);
}  // namespace vq
