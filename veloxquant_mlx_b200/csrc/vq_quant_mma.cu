// VecInfer nearest-centroid search on the tensor cores, with the exact answer.
//
// The exact search (vq_quant.cu) spends n_c * sub_dim * 3 float ops per sub-vector on the
// CUDA cores. Here the tensor cores rank the centroids first:
//     s[j][c] = x_j . c  -  |c|^2 / 2          (largest s  <=>  smallest |x_j - c|^2)
// as m16n8k16 f16 MMAs with float32 accumulation: 16 sub-vectors on M, 8 centroids on N. Each
// float32 centroid is split into two halves (c = hi + lo) that share the K = 16 axis of one
// MMA with a repeated x, so the products are exact and the ranking error is a few float32
// ulps; -|c|^2/2 enters as the accumulator's initial value. f32/bf16 inputs are split the
// same way (x = hi + lo).
//
// Exactness. The reference result is defined by a particular float32 evaluation order
// (sequential sum of squared differences, first minimum wins). Its rounding and the MMA's
// differ, so for every sub-vector the kernel finds ALL centroids whose score is within
//     delta = 2^-16 * (|x|^2 + max|c|^2)
// of the best score. Error budget, relative to |x|^2 + max|c|^2: the MMA adds at most ~20
// terms with float32 rounding (2^-23 each) to exact products of halves, the centroid's hi+lo
// split leaves 2^-22: below 2^-18.7; the reference's own sum of squared differences is within
// 2^-19.7 in these units. Two scores are compared, so orders can differ only within
// 2 * (2^-18.7 + 2^-19.7) = 2^-17.1: delta is twice that. Pass 1 takes the row maximum (two 3-input max per MMA); pass 2 repeats the same
// MMAs (bit-identical scores) and counts/identifies scores >= max - delta. One candidate:
// it is the answer. Several (near-ties, duplicate centroids), or a row that the half-precision
// operands cannot represent (|x| > 2^15, non-finite), or a codebook outside [2^-4, 2^12]:
// the warp runs the reference evaluation order over all centroids for that row.
//
// Why not tcgen05: the bound is not the MMA rate but the compare/select work per score on
// the half-rate integer/compare pipe (1.5 instructions per score, two passes). The tensor pipe
// is already busy ~80 % of the time with warp-level MMAs at 8 cycles each.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "common.cuh"
#include "vq_quant_mma.h"

namespace vq {
namespace {

constexpr int kMT = 4;        // m-tiles (16 sub-vectors each) a warp carries through the codebook
constexpr int kWarpsQ = 8;

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ void split_h2(float x0, float x1, uint32_t &hi, uint32_t &lo) {
    hi = pack_h2(x0, x1);
    const float2 h = __half22float2(*reinterpret_cast<__half2 *>(&hi));
    lo = pack_h2(x0 - h.x, x1 - h.y);
}
__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                        const float (&c)[4]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Two neighbouring elements as loaded (kept raw while they are prefetched) and as floats.
template <typename T> struct Raw { using type = uint32_t; };
template <> struct Raw<float> { using type = float2; };
template <typename T>
__device__ __forceinline__ typename Raw<T>::type load_raw(const T *p) {
    return __ldg(reinterpret_cast<const typename Raw<T>::type *>(p));
}
template <typename T>
__device__ __forceinline__ float2 raw_to_f32(typename Raw<T>::type r);
template <>
__device__ __forceinline__ float2 raw_to_f32<float>(float2 r) { return r; }
template <>
__device__ __forceinline__ float2 raw_to_f32<__half>(uint32_t r) { return __half22float2(*reinterpret_cast<__half2 *>(&r)); }
template <>
__device__ __forceinline__ float2 raw_to_f32<__nv_bfloat16>(uint32_t r) {
    return make_float2(__uint_as_float(r << 16), __uint_as_float(r & 0xffff0000u));
}

// The reference evaluation order for one sub-vector, spread over the warp: lane l takes
// centroids l, l+32, ...; (distance, index) pairs are then reduced with "smaller distance,
// then smaller index", which is what a sequential strict '<' scan returns.
template <typename T, int SUB>
__device__ uint32_t exact_row(const T *xrow, const float *__restrict__ cb, int n_c, int lane) {
    float xv[SUB];
#pragma unroll
    for (int i = 0; i < SUB; ++i) xv[i] = to_f32<T>(xrow[i]);
    float best = INFINITY;
    uint32_t best_idx = 0xffffffffu;
    for (int c = lane; c < n_c; c += 32) {
        float dist = 0.f;
#pragma unroll
        for (int i = 0; i < SUB; ++i) {
            const float d = __fsub_rn(xv[i], __ldg(cb + (int64_t)c * SUB + i));
            dist = __fadd_rn(dist, __fmul_rn(d, d));
        }
        // a NaN distance never wins a strict '<' in the sequential scan
        if (dist < best) { best = dist; best_idx = (uint32_t)c; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, best_idx, o);
        if (ob < best || (ob == best && oi < best_idx)) { best = ob; best_idx = oi; }
    }
    // every distance NaN/inf-free comparison failed (all NaN, or all +inf): the scan keeps index 0
    return best_idx == 0xffffffffu ? 0u : best_idx;
}

template <int SUB, bool SPLIT>
struct Shape {
    static constexpr int NM = (SUB == 8 && SPLIT) ? 2 : 1;  // MMAs per (m-tile, n-tile)
};

// T: input dtype; SUB: 4 or 8. SPLIT = the input needs hi + lo halves (anything but f16).
template <typename T, int SUB>
__global__ void __launch_bounds__(kWarpsQ * 32, 2)
vq_quantize_mma_kernel(const T *__restrict__ x, int64_t n_vec, const float *__restrict__ cb_all, int n_c, int n_sub,
                       void *__restrict__ indices, int index_bytes) {
    // With one codebook per sub-space (n_sub > 0) a CTA works on sub-space blockIdx.y only:
    // its rows are the sub-vectors sub, sub + n_sub, sub + 2 n_sub, ...
    const int sub = n_sub > 0 ? blockIdx.y : 0;
    const int64_t vstride = n_sub > 0 ? n_sub : 1;
    const int64_t n = n_sub > 0 ? (n_vec + n_sub - 1 - sub) / n_sub : n_vec;  // rows of this sub-space
    const float *__restrict__ cb = cb_all + (int64_t)sub * n_c * SUB;
    constexpr bool SPLIT = !std::is_same<T, __half>::value;
    constexpr int NM = Shape<SUB, SPLIT>::NM;
    extern __shared__ __align__(16) uint8_t smem[];
    const int n_tiles = ((n_c + 31) / 32) * 4;  // 8 centroids each; padded to whole groups of 4 tiles
    uint2 *sh_b = reinterpret_cast<uint2 *>(smem);                             // [n_tiles][NM][32]
    // accumulator start values -|c|^2/2 as ready-made register quads: [n_tiles][lane % 4]
    float4 *sh_c = reinterpret_cast<float4 *>(sh_b + (size_t)n_tiles * NM * 32);
    __shared__ float sh_cmax2;
    __shared__ int sh_cb_bad;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, c = lane & 3;

    // ---- prologue: B fragments (hi/lo halves of the centroids) and -|c|^2/2 -------------
    if (tid == 0) { sh_cmax2 = 0.f; sh_cb_bad = 0; }
    __syncthreads();
    for (int i = tid; i < n_tiles * 32; i += blockDim.x) {
        const int nt = i >> 5, l = i & 31, gg = l >> 2, cc = l & 3;
        const int cen = nt * 8 + gg;
        const int pi = (2 * cc) % SUB;
        float c0 = 0.f, c1 = 0.f;
        if (cen < n_c) { c0 = cb[(int64_t)cen * SUB + pi]; c1 = cb[(int64_t)cen * SUB + pi + 1]; }
        uint32_t hi, lo;
        split_h2(c0, c1, hi, lo);
        if constexpr (SUB == 8 && !SPLIT) {
            sh_b[(size_t)nt * 32 + l] = make_uint2(hi, lo);
        } else if constexpr (SUB == 8 && SPLIT) {
            sh_b[((size_t)nt * 2 + 0) * 32 + l] = make_uint2(hi, hi);
            sh_b[((size_t)nt * 2 + 1) * 32 + l] = make_uint2(lo, lo);
        } else if constexpr (SUB == 4 && !SPLIT) {
            sh_b[(size_t)nt * 32 + l] = make_uint2(cc < 2 ? hi : lo, 0u);
        } else {
            sh_b[(size_t)nt * 32 + l] = make_uint2(hi, lo);
        }
    }
    for (int i = tid; i < n_tiles * 8; i += blockDim.x) {
        float h = -3.0e38f;  // padding centroids can never be within delta of a real one
        if (i < n_c) {
            float s2 = 0.f, mx = 0.f;
            bool bad = false;
#pragma unroll
            for (int k = 0; k < SUB; ++k) {
                const float v = cb[(int64_t)i * SUB + k];
                s2 = fmaf(v, v, s2);
                mx = fmaxf(mx, fabsf(v));
                bad |= !(fabsf(v) <= 4096.f);
            }
            h = -0.5f * s2;
            atomicMax(reinterpret_cast<int *>(&sh_cmax2), __float_as_int(mx * mx));  // non-negative floats order as ints
            if (bad) sh_cb_bad = 1;
        }
        // centroid i is column i % 8 of tile i / 8: element (i & 1) of the pair held by lane c = (i % 8) / 2
        float *quad = reinterpret_cast<float *>(sh_c + (i >> 3) * 4 + ((i & 7) >> 1));
        quad[i & 1] = h;
        quad[2 + (i & 1)] = h;
    }
    __syncthreads();
    const float cmax2 = sh_cmax2;
    // Outside this range the half-precision operands lose their error bound: every row then
    // takes the reference-order scan (correct, just not fast).
    const bool cb_ok = !sh_cb_bad && cmax2 >= 0.00390625f;

    const int pi = (2 * c) % SUB;  // this lane's element pair of a sub-vector
    const int64_t n_chunks = (n + 16 * kMT - 1) / (16 * kMT);
    const int64_t chunk_step = (int64_t)gridDim.x * kWarpsQ;
    using RawT = typename Raw<T>::type;
    RawT raw[kMT][2];  // the next chunk's elements, in flight while the current chunk is searched
    auto fetch = [&](int64_t chunk) {
        const int64_t r0 = chunk * (16 * kMT);
#pragma unroll
        for (int mt = 0; mt < kMT; ++mt)
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int64_t row = max((int64_t)0, min(r0 + mt * 16 + g + 8 * r, n - 1));
                raw[mt][r] = load_raw<T>(x + (row * vstride + sub) * SUB + pi);
            }
    };
    int64_t chunk = (int64_t)blockIdx.x * kWarpsQ + warp;
    if (chunk < n_chunks) fetch(chunk);
    for (; chunk < n_chunks; chunk += chunk_step) {
        const int64_t row0 = chunk * (16 * kMT);
        uint32_t a[kMT][4];
        float thr[kMT][2];
        bool bad_row[kMT][2];
#pragma unroll
        for (int mt = 0; mt < kMT; ++mt) {
            float xn[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const float2 v = raw_to_f32<T>(raw[mt][r]);
                uint32_t hi, lo;
                if constexpr (SPLIT) split_h2(v.x, v.y, hi, lo);
                else { hi = pack_h2(v.x, v.y); lo = hi; }
                if constexpr (SUB == 8) {
                    a[mt][r] = hi;
                    a[mt][2 + r] = lo;  // f16: the same x again, against the low halves of c
                } else {
                    a[mt][r] = (SPLIT && c >= 2) ? lo : hi;
                    a[mt][2 + r] = a[mt][r];
                }
                // The MMA wants four consecutive registers. Equal values would share one
                // register and be copied into place before every MMA: make the copy once.
                asm volatile("mov.b32 %0, %1;" : "=r"(a[mt][2 + r]) : "r"(a[mt][2 + r]));
                const bool own = SUB == 8 || c < 2;
                float s2 = own ? fmaf(v.x, v.x, v.y * v.y) : 0.f;
                float bad = !(fabsf(v.x) <= 32768.f && fabsf(v.y) <= 32768.f) ? 1.f : 0.f;
                s2 += __shfl_xor_sync(0xffffffffu, s2, 1);
                s2 += __shfl_xor_sync(0xffffffffu, s2, 2);
                bad += __shfl_xor_sync(0xffffffffu, bad, 1);
                bad += __shfl_xor_sync(0xffffffffu, bad, 2);
                xn[r] = s2;
                bad_row[mt][r] = bad != 0.f || !cb_ok;
            }
            thr[mt][0] = xn[0];
            thr[mt][1] = xn[1];
        }
        if (chunk + chunk_step < n_chunks) fetch(chunk + chunk_step);

        // ---- pass 1: row maxima ----------------------------------------------------------
        float best[kMT][2];
#pragma unroll
        for (int mt = 0; mt < kMT; ++mt) best[mt][0] = best[mt][1] = -INFINITY;
        const uint2 *pb = sh_b + lane;
        const float4 *pc = sh_c + c;
        for (int q = 0; q < n_tiles; q += 4, pb += 4 * NM * 32, pc += 16) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                uint2 b[NM];
#pragma unroll
                for (int m = 0; m < NM; ++m) b[m] = pb[(u * NM + m) * 32];
                const float4 ci = pc[u * 4];
                const float cinit[4] = {ci.x, ci.y, ci.z, ci.w};
#pragma unroll
                for (int mt = 0; mt < kMT; ++mt) {
                    float d[4];
                    mma_f16(d, a[mt], b[0].x, b[0].y, cinit);
                    if constexpr (NM == 2) mma_f16(d, a[mt], b[1].x, b[1].y, d);
                    best[mt][0] = max3(best[mt][0], d[0], d[1]);
                    best[mt][1] = max3(best[mt][1], d[2], d[3]);
                }
            }
        }
#pragma unroll
        for (int mt = 0; mt < kMT; ++mt)
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float m = best[mt][r];
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
                thr[mt][r] = m - 1.52587890625e-05f * (thr[mt][r] + cmax2);
            }

        // ---- pass 2: the same scores again; count and name those within delta of the best --
        // 65536 * hits + sum of hit indices, kept in float so that the predicated adds run on
        // the FMA pipe (exact for one hit: < 2^24; two or more hits only need to be >= 131072)
        float acc[kMT][2];
#pragma unroll
        for (int mt = 0; mt < kMT; ++mt) acc[mt][0] = acc[mt][1] = 0.f;
        float kq = (float)(65536 + 2 * c);
        pb = sh_b + lane;
        pc = sh_c + c;
        for (int q = 0; q < n_tiles; q += 4, pb += 4 * NM * 32, pc += 16, kq += 32.f) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                uint2 b[NM];
#pragma unroll
                for (int m = 0; m < NM; ++m) b[m] = pb[(u * NM + m) * 32];
                const float4 ci = pc[u * 4];
                const float cinit[4] = {ci.x, ci.y, ci.z, ci.w};
                const float k0 = kq + (float)(8 * u), k1 = kq + (float)(8 * u + 1);
#pragma unroll
                for (int mt = 0; mt < kMT; ++mt) {
                    float d[4];
                    mma_f16(d, a[mt], b[0].x, b[0].y, cinit);
                    if constexpr (NM == 2) mma_f16(d, a[mt], b[1].x, b[1].y, d);
                    if (d[0] >= thr[mt][0]) acc[mt][0] += k0;
                    if (d[1] >= thr[mt][0]) acc[mt][0] += k1;
                    if (d[2] >= thr[mt][1]) acc[mt][1] += k0;
                    if (d[3] >= thr[mt][1]) acc[mt][1] += k1;
                }
            }
        }

        // ---- results ---------------------------------------------------------------------
#pragma unroll
        for (int mt = 0; mt < kMT; ++mt)
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                float v = acc[mt][r];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                const int64_t row = row0 + mt * 16 + g + 8 * r;
                const bool live = row < n;
                const bool slow = live && (bad_row[mt][r] || !(v >= 65536.f && v < 131072.f));
                uint32_t slow_mask = __ballot_sync(0xffffffffu, slow && c == 0);
                uint32_t idx = (uint32_t)((int)v - 65536) & 0xffffu;
                while (slow_mask) {
                    const int src = __ffs(slow_mask) - 1;
                    slow_mask &= slow_mask - 1;
                    const int64_t srow = row0 + mt * 16 + (src >> 2) + 8 * r;
                    const uint32_t e = exact_row<T, SUB>(x + (srow * vstride + sub) * SUB, cb, n_c, lane);
                    if (lane == src) idx = e;
                }
                if (live && c == 0) {
                    const int64_t o = row * vstride + sub;
                    if (index_bytes == 1) reinterpret_cast<uint8_t *>(indices)[o] = (uint8_t)idx;
                    else if (index_bytes == 2) reinterpret_cast<uint16_t *>(indices)[o] = (uint16_t)idx;
                    else reinterpret_cast<uint32_t *>(indices)[o] = idx;
                }
            }
    }
}

template <typename T, int SUB>
int32_t launch(const void *x, int64_t n, const float *cb, int n_c, int n_sub, void *indices, int index_bytes, cudaStream_t st) {
    constexpr bool SPLIT = !std::is_same<T, __half>::value;
    constexpr int NM = Shape<SUB, SPLIT>::NM;
    DeviceInfo di;
    int32_t rc = device_info(&di);
    if (rc != VQ_OK) return rc;
    const int n_tiles = ((n_c + 31) / 32) * 4;
    const size_t smem = (size_t)n_tiles * NM * 32 * sizeof(uint2) + (size_t)n_tiles * 4 * sizeof(float4);
    if (smem > 48 * 1024)
        VQ_CHECK_CUDA(cudaFuncSetAttribute(vq_quantize_mma_kernel<T, SUB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int ny = n_sub > 0 ? n_sub : 1;
    const int64_t n_chunks = ceil_div(ceil_div(n, ny), 16 * kMT);
    const int64_t fill = std::max<int64_t>(1, ceil_div((int64_t)di.sm_count * 2, ny));  // CTAs per sub-space for two per SM
    const unsigned blocks = (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(n_chunks, kWarpsQ), fill));
    vq_quantize_mma_kernel<T, SUB><<<dim3(blocks, ny), kWarpsQ * 32, smem, st>>>((const T *)x, n, cb, n_c, n_sub, indices, index_bytes);
    VQ_CHECK_LAUNCH("vq_quantize_mma_kernel");
    return VQ_OK;
}

template <typename T>
int32_t launch_sub(const void *x, int64_t n, int sub_dim, const float *cb, int n_c, int n_sub, void *indices,
                   int index_bytes, cudaStream_t st) {
    return sub_dim == 8 ? launch<T, 8>(x, n, cb, n_c, n_sub, indices, index_bytes, st)
                        : launch<T, 4>(x, n, cb, n_c, n_sub, indices, index_bytes, st);
}

}  // namespace

bool vq_quantize_mma_supported(const void *x, int32_t x_dtype, int64_t n, int32_t sub_dim, int32_t n_c, int32_t n_sub) {
    const int mode = knob_get(VQ_KNOB_VQ_SEARCH);  // 0 choose; 1 tcgen05 / 2 mma.sync / 3 exact pin one search
    if (mode == 1 || mode == 3 || mode == 4) return false;
    if (n_sub < 0 || n_sub > 65535 || (sub_dim != 4 && sub_dim != 8)) return false;
    if (n_c < 2 || n_c > 2048) return false;
    if (x_dtype != VQ_F16 && x_dtype != VQ_BF16 && x_dtype != VQ_F32) return false;
    if (!is_aligned(x, x_dtype == VQ_F32 ? 8 : 4)) return false;
    const bool forced = mode == 2;
    return forced || n >= 1024;  // tiny inputs: the prologue would dominate
}

int32_t vq_quantize_mma_launch(const void *x, int32_t x_dtype, int64_t n, int32_t sub_dim, const float *cb, int32_t n_c,
                               int32_t n_sub, void *indices, int32_t index_bytes, cudaStream_t st) {
    switch (x_dtype) {
        case VQ_F16: return launch_sub<__half>(x, n, sub_dim, cb, n_c, n_sub, indices, index_bytes, st);
        case VQ_BF16: return launch_sub<__nv_bfloat16>(x, n, sub_dim, cb, n_c, n_sub, indices, index_bytes, st);
        default: return launch_sub<float>(x, n, sub_dim, cb, n_c, n_sub, indices, index_bytes, st);
    }
}

}  // namespace vq
