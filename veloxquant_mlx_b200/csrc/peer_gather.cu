// Sharded decode across the GPUs of one node: the consumer side of the per-layer output
// exchange, and the inter-process mapping of the exchange buffers.
//
// The producer side is the merging CTAs of the decode attend kernel (kivi_attend_mma.cu): they store
// their output rows into every rank's gathered tensor through peer-mapped pointers and then
// each of those CTAs adds 1 to word `rank` of every rank's arrival array. Here:
//   - peer_gather_wait_kernel: one CTA, thread r polls arrival word r of THIS rank until it
//     reaches (the round this rank is waiting for) x (rank r's arrivals per round). The poll count is bounded; a wait that runs
//     out raises a device flag (reported by vq_kivi_attend_status) and the kernel returns, so
//     a missing peer can never hang the GPU.
//   - vq_peer_export / vq_peer_open / vq_peer_close: CUDA IPC handles, so that one process per
//     GPU can map the other processes' buffers. Only plain loads and stores ever touch the
//     mapped memory (no multicast, no bulk-copy engine).
#include <cstring>

#include "common.cuh"
#include "kivi_attend.h"

namespace vq {
namespace {

constexpr uint32_t kPeerSpinLimit = 1u << 20;  // x ~0.5-1 us of sleep per poll: about a second

__device__ int g_peer_timeout = 0;

struct Arrivals { int32_t n[VQ_MAX_PEERS]; };

__global__ void __launch_bounds__(32) peer_gather_wait_kernel(const uint32_t *flags, uint32_t *state, int n_sources,
                                                               const __grid_constant__ Arrivals per_round) {
    // whatever follows on the stream may become resident; it must not read the gathered rows
    // before this grid has completed
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ uint32_t want;
    if (threadIdx.x == 0) {
        want = state[2] + 1u;  // rounds are counted on the device so that a captured graph can be replayed
        state[2] = want;
    }
    __syncthreads();
    bool ok = true;
    if ((int)threadIdx.x < n_sources) {
        ok = false;
        const uint32_t *f = flags + threadIdx.x;
        const uint32_t need = want * (uint32_t)per_round.n[threadIdx.x];  // (modulo 2^32, like the word itself)
        for (uint32_t i = 0; i < kPeerSpinLimit; ++i) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if ((int32_t)(v - need) >= 0) { ok = true; break; }
            __nanosleep(400);
        }
    }
    if (!ok) atomicExch(&g_peer_timeout, 1);
    // the grid that published this rank's own rows (and everything before it) has completed
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

}  // namespace

int32_t peer_gather_take_timeout(int *flag) {
    int zero = 0;
    VQ_CHECK_CUDA(cudaMemcpyFromSymbol(flag, g_peer_timeout, sizeof(int)));
    if (*flag) VQ_CHECK_CUDA(cudaMemcpyToSymbol(g_peer_timeout, &zero, sizeof(int)));
    return VQ_OK;
}

}  // namespace vq

extern "C" int32_t vq_peer_gather_wait(const vq_peer_gather *g, void *stream) {
    using namespace vq;
    VQ_REQUIRE(g != nullptr, VQ_ERR_SHAPE, "vq_peer_gather_wait: gather is NULL");
    VQ_REQUIRE(g->world >= 1 && g->world <= VQ_MAX_PEERS && g->rank >= 0 && g->rank < g->world, VQ_ERR_SHAPE,
               "vq_peer_gather_wait: rank %d of %d is out of range", g->rank, g->world);
    VQ_REQUIRE(g->n_sources >= 1 && g->n_sources <= g->world, VQ_ERR_SHAPE,
               "vq_peer_gather_wait: n_sources=%d must be in 1..world=%d", g->n_sources, g->world);
    VQ_REQUIRE(g->state != nullptr && g->flags[g->rank] != nullptr, VQ_ERR_SHAPE, "vq_peer_gather_wait: NULL buffer");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    Arrivals per_round;
    for (int r = 0; r < VQ_MAX_PEERS; ++r) {
        VQ_REQUIRE(r >= g->n_sources || g->arrivals[r] >= 1, VQ_ERR_SHAPE, "vq_peer_gather_wait: arrivals[%d]=%d must be >= 1", r, g->arrivals[r]);
        per_round.n[r] = g->arrivals[r];
    }
    VQ_CHECK_CUDA(cudaLaunchKernelEx(&cfg, peer_gather_wait_kernel, (const uint32_t *)g->flags[g->rank], g->state, (int)g->n_sources, per_round));
    return VQ_OK;
}

extern "C" int32_t vq_peer_export(const void *ptr, void *handle, int64_t *offset) {
    using namespace vq;
    VQ_REQUIRE(ptr && handle && offset, VQ_ERR_SHAPE, "vq_peer_export: NULL argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    cudaPointerAttributes attr;
    VQ_CHECK_CUDA(cudaPointerGetAttributes(&attr, ptr));
    VQ_REQUIRE(attr.type == cudaMemoryTypeDevice, VQ_ERR_SHAPE, "vq_peer_export: not a device pointer");
    cudaIpcMemHandle_t h;
    VQ_CHECK_CUDA(cudaIpcGetMemHandle(&h, const_cast<void *>(ptr)));
    // The handle names the whole allocation; a peer that opens it gets the allocation's base.
    // Opening our own handle is not allowed, so the base is found by asking the driver for the
    // address range that contains ptr.
    using RangeFn = int (*)(unsigned long long *, size_t *, unsigned long long);
    static RangeFn range_fn = [] {
        void *fp = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fp, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            fp = nullptr;
        return (RangeFn)fp;
    }();
    VQ_REQUIRE(range_fn != nullptr, VQ_ERR_CUDA, "vq_peer_export: the driver does not export cuMemGetAddressRange");
    unsigned long long base = 0;
    size_t size = 0;
    const int r = range_fn(&base, &size, (unsigned long long)reinterpret_cast<uintptr_t>(ptr));
    VQ_REQUIRE(r == 0, VQ_ERR_CUDA, "vq_peer_export: cuMemGetAddressRange failed (%d)", r);
    memcpy(handle, &h, sizeof(h));
    *offset = (int64_t)(reinterpret_cast<uintptr_t>(ptr) - (uintptr_t)base);
    return VQ_OK;
}

extern "C" int32_t vq_peer_open(const void *handle, void **base) {
    using namespace vq;
    VQ_REQUIRE(handle && base, VQ_ERR_SHAPE, "vq_peer_open: NULL argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void *p = nullptr;
    VQ_CHECK_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *base = p;
    return VQ_OK;
}

extern "C" int32_t vq_peer_close(void *base) {
    using namespace vq;
    VQ_REQUIRE(base != nullptr, VQ_ERR_SHAPE, "vq_peer_close: NULL argument");
    VQ_CHECK_CUDA(cudaIpcCloseMemHandle(base));
    return VQ_OK;
}
