// vq_kivi_decode_attend_static: the fused KIVI decode attention for callers that cannot
// allocate device memory.
//
// Who that is: code running where cudaMalloc is off the table -- a serving loop whose
// memory pool is fully handed out and frozen before the first request, a plugin hosted by
// a runtime that owns every allocation and gives guests no allocator, or a latency-critical
// path where an allocation (a synchronising call that can also fail under memory pressure)
// is not acceptable. The regular entry point leaves the split-partials workspace to the
// caller; this one needs no workspace argument at all. The partial (max, sum, output)
// records of the context splits go into a fixed array that is part of the library image.
//
// The array below is part of this library's device image: kStaticScratchBytes per GPU, held
// until process exit once its module is loaded on that GPU. In host code its name is only a
// handle for the runtime, not an address a kernel could use, so the device address is looked
// up with cudaGetSymbolAddress, once per device, and that pointer is what the kernels receive.
// This translation unit holds nothing but the array, so under CUDA's default lazy module
// loading the look-up is what loads its module on a device: the driver sets the 8 MiB aside
// at that moment, and the look-up can fail when the device is out of memory. That is why the
// first call per device belongs before the caller freezes its memory; it is the only call
// that can take device memory.
#include <mutex>

#include "common.cuh"

namespace vq {
namespace {

constexpr size_t kStaticScratchBytes = VQ_KIVI_STATIC_SCRATCH_BYTES;  // 8 MiB per GPU

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch on the CURRENT device; resolved on first use there.
int32_t static_scratch_ptr(void **out) {
    static void *ptrs[64];
    static bool have[64];
    static std::mutex mu;
    int dev = 0;
    VQ_CHECK_CUDA(cudaGetDevice(&dev));
    VQ_REQUIRE(dev >= 0 && dev < 64, VQ_ERR_CUDA, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!have[dev]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr)
            return fail(VQ_ERR_CUDA, "vq_kivi_decode_attend_static: cudaGetSymbolAddress failed on device %d: %s",
                        dev, cudaGetErrorString(e));
        ptrs[dev] = p;
        have[dev] = true;
    }
    *out = ptrs[dev];
    return VQ_OK;
}

}  // namespace
}  // namespace vq

extern "C" int32_t vq_kivi_decode_attend_static(const vq_kivi_attend_args *args, void *stream) {
    using namespace vq;
    VQ_REQUIRE(args != nullptr, VQ_ERR_SHAPE, "vq_kivi_decode_attend_static: args is NULL");
    vq_kivi_attend_args a = *args;
    a.workspace = nullptr;
    a.workspace_bytes = 0;
    const int64_t need = vq_kivi_attend_workspace_bytes(&a);
    VQ_REQUIRE(need <= (int64_t)kStaticScratchBytes, VQ_ERR_CAPACITY,
               "vq_kivi_decode_attend_static: this call needs %lld bytes of split scratch but the built-in "
               "array holds %lld; lower n_splits or the batch, or use vq_kivi_decode_attend with a workspace",
               (long long)need, (long long)kStaticScratchBytes);
    void *ptr = nullptr;
    const int32_t rc = static_scratch_ptr(&ptr);
    if (rc != VQ_OK) return rc;
    // Nothing in the scratch has to start at zero: every partial record the merge reads is
    // written earlier in the same call, so stale contents of a previous call are never seen.
    a.workspace = ptr;
    a.workspace_bytes = (int64_t)kStaticScratchBytes;
    return vq_kivi_decode_attend(&a, stream);
}
