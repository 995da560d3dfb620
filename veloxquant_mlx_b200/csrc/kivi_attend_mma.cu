// Placeholder until the tensor-core kernel lands.
#include "kivi_attend.h"
namespace vq {
const char *kivi_attend_mma_supported(const vq_kivi_attend_args &) { return "not built"; }
int kivi_attend_mma_splits(const vq_kivi_attend_args &, const DeviceInfo &) { return 1; }
int32_t kivi_attend_mma_launch(const vq_kivi_attend_args &, const DeviceInfo &, cudaStream_t) {
    return fail(VQ_ERR_SHAPE, "tensor-core kernel not built");
}
}  // namespace vq
