// VecInfer dual transform with a defined summation order: smooth (divide for keys, multiply for
// queries), then the orthonormal Walsh-Hadamard transform as a Sylvester butterfly, then one
// multiplication by the matrix's common entry magnitude c = (1/sqrt 2)^log2(D).
//
// The reference writes the transform as a matrix product with the dense Hadamard matrix
// (allocators/vecinfer.py:93-184), whose float32 summation order is whatever the matmul of its
// framework does. Here the order is fixed: every butterfly pair is (lower + upper,
// lower - upper), strides 1, 2, 4, ... -- the order of the CPU oracle -- so that the VQ indices
// computed from the transformed keys are reproducible bit for bit, and no library GEMM sits on
// the append path. 7 add stages per element instead of a D-term dot product.
//
// Layout: one warp per row, a lane holds EPL = D / 32 consecutive elements; the stages with
// stride < EPL pair registers, the five widest stages cross lanes through shuffles.
#include <algorithm>

#include "common.cuh"

namespace vq {
namespace {

template <typename T, int EPL>
__device__ __forceinline__ void load_row(const T *p, float (&v)[EPL]) {
#pragma unroll
    for (int j = 0; j < EPL; ++j) v[j] = to_f32<T>(p[j]);
}

template <typename T, int EPL>
__global__ void __launch_bounds__(128)
vq_dual_transform_kernel(const T *__restrict__ x, int64_t n_rows, int64_t tok_per_head, int n_heads,
                         const float *__restrict__ smooth, int smooth_rows, int divide, float c,
                         float *__restrict__ out) {
    constexpr int D = 32 * EPL;
    const int lane = threadIdx.x & 31;
    const int64_t warp_id = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int64_t n_warps = (int64_t)gridDim.x * 4;
    for (int64_t row = warp_id; row < n_rows; row += n_warps) {
        float v[EPL];
        load_row<T, EPL>(x + row * D + EPL * lane, v);
        if (smooth != nullptr) {
            const int head = (int)((row / tok_per_head) % n_heads);
            const float *s = smooth + (int64_t)(head % smooth_rows) * D + EPL * lane;
#pragma unroll
            for (int j = 0; j < EPL; ++j) v[j] = divide ? __fdiv_rn(v[j], s[j]) : __fmul_rn(v[j], s[j]);
        }
#pragma unroll
        for (int st = 1; st < EPL; st <<= 1) {
#pragma unroll
            for (int j = 0; j < EPL; ++j) {
                if ((j & st) == 0) {
                    const float a = v[j], b = v[j + st];
                    v[j] = __fadd_rn(a, b);
                    v[j + st] = __fsub_rn(a, b);
                }
            }
        }
#pragma unroll
        for (int m = 1; m < 32; m <<= 1) {
            const bool upper = lane & m;
#pragma unroll
            for (int j = 0; j < EPL; ++j) {
                const float other = __shfl_xor_sync(0xffffffffu, v[j], m);
                v[j] = upper ? __fsub_rn(other, v[j]) : __fadd_rn(v[j], other);
            }
        }
#pragma unroll
        for (int j = 0; j < EPL; ++j) out[row * D + EPL * lane + j] = __fmul_rn(v[j], c);
    }
}

template <typename T>
int32_t launch_t(const void *x, int64_t n_rows, int D, int64_t tok_per_head, int n_heads, const float *smooth,
                 int smooth_rows, int divide, float c, float *out, int sm_count, cudaStream_t st) {
    const unsigned blocks = (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(n_rows, 4), (int64_t)sm_count * 16));
#define VQ_T(EPL)                                                                                                  \
    case 32 * EPL:                                                                                                 \
        vq_dual_transform_kernel<T, EPL><<<blocks, 128, 0, st>>>((const T *)x, n_rows, tok_per_head, n_heads, smooth, \
                                                                 smooth_rows, divide, c, out);                      \
        break;
    switch (D) {
        VQ_T(1) VQ_T(2) VQ_T(4) VQ_T(8)
        default: return fail(VQ_ERR_SHAPE, "vq_vq_dual_transform: D=%d must be 32, 64, 128 or 256", D);
    }
#undef VQ_T
    VQ_CHECK_LAUNCH("vq_dual_transform_kernel");
    return VQ_OK;
}

}  // namespace
}  // namespace vq

extern "C" int32_t vq_vq_dual_transform(const void *x, int32_t x_dtype, int64_t n_rows, int32_t D, int64_t tok_per_head,
                                        int32_t n_heads, const float *smooth, int32_t smooth_rows, int32_t divide, float c,
                                        float *out, void *stream) {
    using namespace vq;
    VQ_REQUIRE(n_rows >= 0, VQ_ERR_SHAPE, "vq_vq_dual_transform: n_rows=%lld", (long long)n_rows);
    if (n_rows == 0) return VQ_OK;
    VQ_REQUIRE(x && out, VQ_ERR_SHAPE, "vq_vq_dual_transform: NULL argument");
    VQ_REQUIRE(x_dtype >= 0 && x_dtype <= 2, VQ_ERR_DTYPE, "vq_vq_dual_transform: unknown dtype %d", x_dtype);
    if (smooth)
        VQ_REQUIRE(smooth_rows >= 1 && n_heads >= 1 && tok_per_head >= 1, VQ_ERR_SHAPE,
                   "vq_vq_dual_transform: smooth needs smooth_rows, n_heads and tok_per_head >= 1");
    DeviceInfo di;
    int32_t rc = device_info(&di);
    if (rc != VQ_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t tph = tok_per_head > 0 ? tok_per_head : 1;
    const int nh = n_heads > 0 ? n_heads : 1;
    switch (x_dtype) {
        case VQ_F16: return launch_t<__half>(x, n_rows, D, tph, nh, smooth, smooth_rows, divide, c, out, di.sm_count, st);
        case VQ_BF16: return launch_t<__nv_bfloat16>(x, n_rows, D, tph, nh, smooth, smooth_rows, divide, c, out, di.sm_count, st);
        default: return launch_t<float>(x, n_rows, D, tph, nh, smooth, smooth_rows, divide, c, out, di.sm_count, st);
    }
}
