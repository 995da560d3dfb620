// VecInfer product VQ: nearest-centroid search and codebook gather.
//
// vq_vq_quantize sends the serving shapes to the tensor-core search (vq_quant_mma.cu), which
// returns the same indices; everything else runs vq_quantize_kernel, the exact search: float32 squared distances accumulated in the
// canonical order (sequential over the sub-vector, product and sum rounded separately --
// this file is compiled with -fmad=false), strict '<' so the lowest index wins ties. One
// thread owns one sub-vector (its sub_dim values stay in registers); the codebook is staged
// in shared memory as float32 and every lane of a warp reads the same centroid row
// (a broadcast, no bank conflicts). Work per sub-vector: n_c * sub_dim * 3 float ops.
#include <algorithm>

#include "common.cuh"
#include "vq_quant_mma.h"

namespace vq {

template <typename T, int SUB>
__global__ void __launch_bounds__(256)
vq_quantize_kernel(const T *__restrict__ x, int64_t n, const float *__restrict__ codebook, int n_c,
                   int n_sub, void *__restrict__ indices, int index_bytes) {
    extern __shared__ float sh_cb[];  // [n_c][SUB] of the codebook this CTA uses
    // With stacked codebooks a CTA handles sub-vectors of one sub-space only: blockIdx.y.
    const int sub_space = n_sub > 0 ? blockIdx.y : 0;
    const float *cb = codebook + (int64_t)sub_space * n_c * SUB;
    for (int i = threadIdx.x; i < n_c * SUB; i += blockDim.x) sh_cb[i] = cb[i];
    __syncthreads();
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t count = n_sub > 0 ? (n + n_sub - 1 - sub_space) / n_sub : n;  // sub-vectors of this sub-space
    for (int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < count; j += stride) {
        const int64_t vec = n_sub > 0 ? j * n_sub + sub_space : j;
        float xv[SUB];
#pragma unroll
        for (int i = 0; i < SUB; ++i) xv[i] = to_f32<T>(x[vec * SUB + i]);
        float best = INFINITY;
        uint32_t best_idx = 0;
        for (int c = 0; c < n_c; ++c) {
            float dist = 0.f;
#pragma unroll
            for (int i = 0; i < SUB; ++i) {
                const float d = __fsub_rn(xv[i], sh_cb[c * SUB + i]);
                dist = __fadd_rn(dist, __fmul_rn(d, d));
            }
            if (dist < best) { best = dist; best_idx = (uint32_t)c; }
        }
        if (index_bytes == 1) reinterpret_cast<uint8_t *>(indices)[vec] = (uint8_t)best_idx;
        else if (index_bytes == 2) reinterpret_cast<uint16_t *>(indices)[vec] = (uint16_t)best_idx;
        else reinterpret_cast<uint32_t *>(indices)[vec] = best_idx;
    }
}

template <typename T>
__global__ void vq_dequant_kernel(const void *__restrict__ indices, int index_bytes, int64_t n,
                                  const float *__restrict__ codebook, int n_c, int sub_dim, int n_sub,
                                  T *__restrict__ out) {
    const int64_t total = n * sub_dim;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t vec = i / sub_dim;
        const int comp = (int)(i % sub_dim);
        uint32_t idx;
        if (index_bytes == 1) idx = reinterpret_cast<const uint8_t *>(indices)[vec];
        else if (index_bytes == 2) idx = reinterpret_cast<const uint16_t *>(indices)[vec];
        else idx = reinterpret_cast<const uint32_t *>(indices)[vec];
        idx = min(idx, (uint32_t)(n_c - 1));
        const int64_t base = n_sub > 0 ? (int64_t)(vec % n_sub) * n_c * sub_dim : 0;
        out[i] = from_f32<T>(codebook[base + (int64_t)idx * sub_dim + comp]);
    }
}

template <typename T>
static int32_t launch_quantize(const void *x, int64_t n, int sub_dim, const float *cb, int n_c, int n_sub,
                               void *indices, int index_bytes, cudaStream_t st) {
    const size_t smem = (size_t)n_c * sub_dim * sizeof(float);
    const int64_t per_space = n_sub > 0 ? ceil_div(n, n_sub) : n;
    const unsigned gx = (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(per_space, 256), 148 * 8));
    dim3 grid(gx, n_sub > 0 ? n_sub : 1);
#define VQ_Q(SUB)                                                                                         \
    case SUB:                                                                                             \
        if (smem > 48 * 1024)                                                                             \
            VQ_CHECK_CUDA(cudaFuncSetAttribute(vq_quantize_kernel<T, SUB>,                                 \
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));  \
        vq_quantize_kernel<T, SUB><<<grid, 256, smem, st>>>((const T *)x, n, cb, n_c, n_sub, indices, index_bytes); \
        break;
    switch (sub_dim) {
        VQ_Q(1) VQ_Q(2) VQ_Q(4) VQ_Q(8) VQ_Q(16)
        default: return fail(VQ_ERR_SHAPE, "vq_vq_quantize: sub_dim must be 1, 2, 4, 8 or 16, got %d", sub_dim);
    }
#undef VQ_Q
    VQ_CHECK_LAUNCH("vq_quantize_kernel");
    return VQ_OK;
}

}  // namespace vq

extern "C" int32_t vq_vq_quantize(const void *x, int32_t x_dtype, int64_t n, int32_t sub_dim,
                                  const float *codebook, int32_t n_centroids, int32_t n_sub, void *indices,
                                  int32_t index_bytes, void *stream) {
    using namespace vq;
    VQ_REQUIRE(n >= 0, VQ_ERR_SHAPE, "vq_vq_quantize: n must be >= 0");
    VQ_REQUIRE(n_centroids >= 1 && n_centroids <= 65536, VQ_ERR_SHAPE, "vq_vq_quantize: n_centroids=%d out of range", n_centroids);
    VQ_REQUIRE(index_bytes == 1 || index_bytes == 2 || index_bytes == 4, VQ_ERR_SHAPE, "vq_vq_quantize: index_bytes must be 1, 2 or 4");
    VQ_REQUIRE(index_bytes == 4 || n_centroids <= (1 << (8 * index_bytes)), VQ_ERR_SHAPE,
               "vq_vq_quantize: %d centroids do not fit %d-byte indices", n_centroids, index_bytes);
    VQ_REQUIRE(n_sub >= 0 && n_sub <= 65535, VQ_ERR_SHAPE, "vq_vq_quantize: bad n_sub");
    VQ_REQUIRE((size_t)n_centroids * sub_dim * 4 <= 200 * 1024, VQ_ERR_CAPACITY, "vq_vq_quantize: codebook of %d x %d floats does not fit shared memory", n_centroids, sub_dim);
    if (n == 0) return VQ_OK;
    VQ_REQUIRE(x && codebook && indices, VQ_ERR_SHAPE, "vq_vq_quantize: NULL argument");
    cudaStream_t st = (cudaStream_t)stream;
    if (vq_quantize_tc5_supported(x, x_dtype, n, sub_dim, n_centroids, n_sub))
        return vq_quantize_tc5_launch(x, x_dtype, n, codebook, n_centroids, n_sub, indices, index_bytes, st);
    if (vq_quantize_mma_supported(x, x_dtype, n, sub_dim, n_centroids, n_sub))
        return vq_quantize_mma_launch(x, x_dtype, n, sub_dim, codebook, n_centroids, n_sub, indices, index_bytes, st);
    switch (x_dtype) {
        case VQ_F16: return launch_quantize<__half>(x, n, sub_dim, codebook, n_centroids, n_sub, indices, index_bytes, st);
        case VQ_BF16: return launch_quantize<__nv_bfloat16>(x, n, sub_dim, codebook, n_centroids, n_sub, indices, index_bytes, st);
        case VQ_F32: return launch_quantize<float>(x, n, sub_dim, codebook, n_centroids, n_sub, indices, index_bytes, st);
        default: return fail(VQ_ERR_DTYPE, "vq_vq_quantize: unknown dtype %d", x_dtype);
    }
}

extern "C" int32_t vq_vq_dequant(const void *indices, int32_t index_bytes, int64_t n, const float *codebook,
                                 int32_t n_centroids, int32_t sub_dim, int32_t n_sub, void *out,
                                 int32_t out_dtype, void *stream) {
    using namespace vq;
    VQ_REQUIRE(n >= 0 && sub_dim >= 1 && n_centroids >= 1, VQ_ERR_SHAPE, "vq_vq_dequant: bad sizes");
    VQ_REQUIRE(index_bytes == 1 || index_bytes == 2 || index_bytes == 4, VQ_ERR_SHAPE, "vq_vq_dequant: index_bytes must be 1, 2 or 4");
    if (n == 0) return VQ_OK;
    const int64_t total = n * sub_dim;
    const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(total, 256), 148 * 32);
    cudaStream_t st = (cudaStream_t)stream;
    switch (out_dtype) {
        case VQ_F16: vq_dequant_kernel<__half><<<blocks, 256, 0, st>>>(indices, index_bytes, n, codebook, n_centroids, sub_dim, n_sub, (__half *)out); break;
        case VQ_BF16: vq_dequant_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(indices, index_bytes, n, codebook, n_centroids, sub_dim, n_sub, (__nv_bfloat16 *)out); break;
        case VQ_F32: vq_dequant_kernel<float><<<blocks, 256, 0, st>>>(indices, index_bytes, n, codebook, n_centroids, sub_dim, n_sub, (float *)out); break;
        default: return fail(VQ_ERR_DTYPE, "vq_vq_dequant: unknown dtype %d", out_dtype);
    }
    VQ_CHECK_LAUNCH("vq_dequant_kernel");
    return VQ_OK;
}

extern "C" int32_t vq_vq_quantize_status(void) {
    using namespace vq;
    int flag = 0;
    int32_t rc = vq_quantize_tc5_take_timeout(&flag);
    if (rc != VQ_OK) return rc;
    if (flag) return fail(VQ_ERR_TIMEOUT, "vq_vq_quantize: a bounded wait on an MMA-completion barrier gave up");
    return VQ_OK;
}
