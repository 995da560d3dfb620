// VecInfer quantize-on-append in one launch: smooth divide -> H x (dense Walsh-Hadamard
// matvec) -> nearest centroid -> codebook gather -> H^T c -> smooth multiply, and the plain
// quantize + gather used for values.
//
// Every floating-point step keeps the order of the reference's one-dispatch kernel: the two
// matvecs accumulate c = 0..D-1 in order from 0.0 with the product and the sum rounded
// separately (this file is compiled with -fmad=false), the distance is the sequential sum of
// the exact search, ties go to the lowest centroid index.
//
// One CTA works on kTok tokens at a time with D threads (rounded up to a warp multiple):
//   phase A  thread d loads element d of each token, divides by its smooth factor
//   phase B  thread r accumulates output r of all kTok tokens: one conflict-free read of the
//            transposed H (shared memory) and two broadcast float4 reads (token values are
//            stored [D][kTok]) feed kTok multiply-adds
//   phase C  one thread per (token, sub-vector) scans the codebook (shared memory, broadcast)
//   phase D-F gather, H^T matvec (H itself is the conflict-free layout here), smooth multiply
#include <algorithm>

#include "common.cuh"

namespace vq {
namespace {

constexpr int kTok = 8;  // the matvec loops read a token row as two float4

struct EncParams {
    const void *x;
    int x_dtype;
    int64_t n_tok;
    int D, sub_dim, n_sub, n_c;
    int64_t tok_per_head;
    int n_heads;
    const float *codebook;
    int stacked;  // codebooks: 0 = one shared, else n_sub of them
    const float *H;
    const float *smooth;
    int smooth_rows;
    void *x_hat;
    int hat_dtype;
    void *indices;
    int index_bytes;
    int h_in_smem;
};

template <int SUB>
__global__ void __launch_bounds__(512)
vq_encode_decode_kernel(const EncParams p) {
    extern __shared__ float sh[];
    const int D = p.D, n_sub = p.n_sub, n_c = p.n_c;
    const int n_books = p.stacked ? n_sub : 1;
    float *sh_cb = sh;                                   // [n_books][n_c][SUB]
    float *buf_a = sh_cb + (((size_t)n_books * n_c * SUB + 3) & ~(size_t)3);  // [D][kTok], rows 16-byte aligned
    float *buf_b = buf_a + kTok * D;                     // [D][kTok]
    uint32_t *sh_idx = reinterpret_cast<uint32_t *>(buf_b + kTok * D);  // [kTok][n_sub]
    float *sh_ht = reinterpret_cast<float *>(sh_idx + kTok * n_sub);     // [D][D], Ht[c][r] = H[r][c]
    const int tid = threadIdx.x;
    const bool transform = p.H != nullptr;

    for (int i = tid; i < n_books * n_c * SUB; i += blockDim.x) sh_cb[i] = p.codebook[i];
    if (transform && p.h_in_smem)
        for (int i = tid; i < D * D; i += blockDim.x) {
            const int r = i / D, c = i % D;
            sh_ht[c * D + r] = p.H[i];
        }
    __syncthreads();

    const int64_t n_iter = (p.n_tok + kTok - 1) / kTok;
    for (int64_t it = blockIdx.x; it < n_iter; it += gridDim.x) {
        const int64_t tok0 = it * kTok;
        const int n_here = (int)min((int64_t)kTok, p.n_tok - tok0);

        // phase A: load (+ smooth divide)
        if (tid < D) {
#pragma unroll
            for (int t = 0; t < kTok; ++t) {
                float v = 0.f;
                if (t < n_here) {
                    v = load_as_f32(p.x, p.x_dtype, (tok0 + t) * D + tid);
                    if (p.smooth) {
                        const int h = (int)(((tok0 + t) / p.tok_per_head) % p.n_heads);
                        const float s = p.smooth[(int64_t)(h % p.smooth_rows) * D + tid];
                        if (s > 1e-8f) v = __fdiv_rn(v, s);
                    }
                }
                buf_a[tid * kTok + t] = v;
            }
        }
        __syncthreads();

        // phase B: y = H x
        const float *src = buf_a;
        if (transform) {
            if (tid < D) {
                float acc[kTok];
#pragma unroll
                for (int t = 0; t < kTok; ++t) acc[t] = 0.f;
                for (int c = 0; c < D; ++c) {
                    const float hv = p.h_in_smem ? sh_ht[c * D + tid] : __ldg(p.H + (int64_t)tid * D + c);
                    float xs[kTok];
                    *reinterpret_cast<float4 *>(xs) = *reinterpret_cast<const float4 *>(buf_a + c * kTok);
                    *reinterpret_cast<float4 *>(xs + 4) = *reinterpret_cast<const float4 *>(buf_a + c * kTok + 4);
#pragma unroll
                    for (int t = 0; t < kTok; ++t) acc[t] = __fadd_rn(acc[t], __fmul_rn(hv, xs[t]));
                }
#pragma unroll
                for (int t = 0; t < kTok; ++t) buf_b[tid * kTok + t] = acc[t];
            }
            __syncthreads();
            src = buf_b;
        }

        // phase C: nearest centroid, one thread per (token, sub-vector)
        for (int j = tid; j < n_here * n_sub; j += blockDim.x) {
            const int t = j / n_sub, s = j % n_sub;
            float xv[SUB];
#pragma unroll
            for (int i = 0; i < SUB; ++i) xv[i] = src[(s * SUB + i) * kTok + t];
            const float *cb = sh_cb + (size_t)(p.stacked ? s : 0) * n_c * SUB;
            float best = INFINITY;
            uint32_t best_idx = 0;
            for (int c = 0; c < n_c; ++c) {
                float dist = 0.f;
#pragma unroll
                for (int i = 0; i < SUB; ++i) {
                    const float d = __fsub_rn(xv[i], cb[c * SUB + i]);
                    dist = __fadd_rn(dist, __fmul_rn(d, d));
                }
                if (dist < best) { best = dist; best_idx = (uint32_t)c; }
            }
            sh_idx[t * n_sub + s] = best_idx;
            if (p.indices) {
                const int64_t o = (tok0 + t) * n_sub + s;
                if (p.index_bytes == 1) reinterpret_cast<uint8_t *>(p.indices)[o] = (uint8_t)best_idx;
                else if (p.index_bytes == 2) reinterpret_cast<uint16_t *>(p.indices)[o] = (uint16_t)best_idx;
                else reinterpret_cast<uint32_t *>(p.indices)[o] = best_idx;
            }
        }
        __syncthreads();

        if (p.x_hat) {
            // phase D: gather the winners
            if (tid < D) {
                const int s = tid / SUB, comp = tid % SUB;
                const float *cb = sh_cb + (size_t)(p.stacked ? s : 0) * n_c * SUB;
#pragma unroll
                for (int t = 0; t < kTok; ++t)
                    buf_a[tid * kTok + t] = t < n_here ? cb[sh_idx[t * n_sub + s] * SUB + comp] : 0.f;
            }
            __syncthreads();
            if (tid < D) {
                float acc[kTok];
                if (transform) {
                    // phase E: H^T c -- element (c, tid) of H, consecutive over threads
#pragma unroll
                    for (int t = 0; t < kTok; ++t) acc[t] = 0.f;
                    for (int c = 0; c < D; ++c) {
                        const float hv = __ldg(p.H + (int64_t)c * D + tid);
                        float xs[kTok];
                        *reinterpret_cast<float4 *>(xs) = *reinterpret_cast<const float4 *>(buf_a + c * kTok);
                        *reinterpret_cast<float4 *>(xs + 4) = *reinterpret_cast<const float4 *>(buf_a + c * kTok + 4);
#pragma unroll
                        for (int t = 0; t < kTok; ++t) acc[t] = __fadd_rn(acc[t], __fmul_rn(hv, xs[t]));
                    }
                } else {
#pragma unroll
                    for (int t = 0; t < kTok; ++t) acc[t] = buf_a[tid * kTok + t];
                }
                // phase F + store
#pragma unroll
                for (int t = 0; t < kTok; ++t) {
                    if (t >= n_here) continue;
                    float v = acc[t];
                    if (p.smooth) {
                        const int h = (int)(((tok0 + t) / p.tok_per_head) % p.n_heads);
                        v = __fmul_rn(v, p.smooth[(int64_t)(h % p.smooth_rows) * D + tid]);
                    }
                    store_from_f32(p.x_hat, p.hat_dtype, (tok0 + t) * D + tid, v);
                }
            }
        }
        __syncthreads();
    }
}

int32_t launch(const vq_vq_encode_args &a, bool keys, cudaStream_t st) {
    const char *who = keys ? "vq_vq_encode_decode_keys" : "vq_vq_encode_decode_values";
    VQ_REQUIRE(a.n_tok >= 0, VQ_ERR_SHAPE, "%s: n_tok must be >= 0", who);
    VQ_REQUIRE(a.D >= 1 && a.D <= 512, VQ_ERR_SHAPE, "%s: D=%d > 512 or < 1", who, a.D);
    VQ_REQUIRE(a.sub_dim >= 1 && a.D % a.sub_dim == 0, VQ_ERR_SHAPE, "%s: D=%d not divisible by sub_dim=%d", who, a.D, a.sub_dim);
    VQ_REQUIRE(a.n_centroids >= 1 && a.n_centroids <= 65536, VQ_ERR_SHAPE, "%s: n_centroids=%d out of range", who, a.n_centroids);
    VQ_REQUIRE(a.index_bytes == 1 || a.index_bytes == 2 || a.index_bytes == 4, VQ_ERR_SHAPE, "%s: index_bytes must be 1, 2 or 4", who);
    VQ_REQUIRE(a.index_bytes == 4 || a.n_centroids <= (1 << (8 * a.index_bytes)), VQ_ERR_SHAPE,
               "%s: %d centroids do not fit %d-byte indices", who, a.n_centroids, a.index_bytes);
    VQ_REQUIRE(a.x_dtype >= 0 && a.x_dtype <= 2 && a.hat_dtype >= 0 && a.hat_dtype <= 2, VQ_ERR_DTYPE, "%s: bad dtype", who);
    if (a.n_tok == 0) return VQ_OK;
    VQ_REQUIRE(a.x && a.codebook && (a.indices || a.x_hat), VQ_ERR_SHAPE, "%s: NULL argument", who);
    EncParams p{};
    p.x = a.x; p.x_dtype = a.x_dtype; p.n_tok = a.n_tok; p.D = a.D; p.sub_dim = a.sub_dim;
    p.n_sub = a.D / a.sub_dim; p.n_c = a.n_centroids;
    p.tok_per_head = a.tok_per_head > 0 ? a.tok_per_head : 1; p.n_heads = a.n_heads > 0 ? a.n_heads : 1;
    p.codebook = a.codebook; p.stacked = a.stacked_codebooks ? 1 : 0;
    p.H = keys ? a.H : nullptr;
    p.smooth = keys ? a.smooth : nullptr;
    p.smooth_rows = a.smooth_rows > 0 ? a.smooth_rows : 1;
    p.x_hat = a.x_hat; p.hat_dtype = a.hat_dtype; p.indices = a.indices; p.index_bytes = a.index_bytes;
    if (keys && a.smooth) VQ_REQUIRE(a.n_heads >= 1 && a.tok_per_head >= 1, VQ_ERR_SHAPE, "%s: smooth needs n_heads and tok_per_head", who);

    DeviceInfo di;
    int32_t rc = device_info(&di);
    if (rc != VQ_OK) return rc;
    const int n_books = p.stacked ? p.n_sub : 1;
    size_t smem = ((((size_t)n_books * p.n_c * p.sub_dim + 3) & ~(size_t)3) + 2 * (size_t)kTok * p.D + (size_t)kTok * p.n_sub) * 4;
    VQ_REQUIRE(smem <= di.smem_optin, VQ_ERR_CAPACITY, "%s: codebook of %d x %d x %d floats does not fit shared memory", who, n_books, p.n_c, p.sub_dim);
    const size_t with_h = smem + (size_t)p.D * p.D * 4;
    p.h_in_smem = (p.H && with_h <= di.smem_optin) ? 1 : 0;
    if (p.h_in_smem) smem = with_h;
    const int threads = (int)std::min<int64_t>(512, ceil_div(std::max(p.D, 32), 32) * 32);
    const int per_sm = (int)std::max<size_t>(1, std::min<size_t>(4, di.smem_optin / (smem + 1024)));
    const unsigned blocks = (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(a.n_tok, kTok), (int64_t)di.sm_count * per_sm));
#define VQ_E(SUB)                                                                                              \
    case SUB:                                                                                                  \
        if (smem > 48 * 1024)                                                                                  \
            VQ_CHECK_CUDA(cudaFuncSetAttribute(vq_encode_decode_kernel<SUB>,                                   \
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));       \
        vq_encode_decode_kernel<SUB><<<blocks, threads, smem, st>>>(p);                                        \
        break;
    switch (p.sub_dim) {
        VQ_E(1) VQ_E(2) VQ_E(4) VQ_E(8) VQ_E(16)
        default: return fail(VQ_ERR_SHAPE, "%s: sub_dim must be 1, 2, 4, 8 or 16, got %d", who, p.sub_dim);
    }
#undef VQ_E
    VQ_CHECK_LAUNCH("vq_encode_decode_kernel");
    return VQ_OK;
}

}  // namespace
}  // namespace vq

extern "C" int32_t vq_vq_encode_decode_keys(const vq_vq_encode_args *args, void *stream) {
    VQ_REQUIRE(args != nullptr, VQ_ERR_SHAPE, "vq_vq_encode_decode_keys: args is NULL");
    return vq::launch(*args, true, (cudaStream_t)stream);
}

extern "C" int32_t vq_vq_encode_decode_values(const vq_vq_encode_args *args, void *stream) {
    VQ_REQUIRE(args != nullptr, VQ_ERR_SHAPE, "vq_vq_encode_decode_values: args is NULL");
    return vq::launch(*args, false, (cudaStream_t)stream);
}
