// Two-stage scalar residual quantization of rotated key vectors (TurboQuant-RVQ), packed.
//
// vq_rvq_quant_pack: per coordinate y (fp16 after the rotation)
//     idx1 = #{k : y > boundaries1[k]}                 stage-1 code (sorted Voronoi boundaries)
//     r1   = half(y - centroids1[idx1])                the residual, rounded to fp16
//     idx2 = #{k : r1 > boundaries2[k]}                stage-2 code
// and both code streams are written as uint32 words of 32 / bits codes each, first code in the
// low bits, the last word of a row zero-padded: the layout and the comparisons of the
// reference's fused kernel (veloxquant_mlx/metal/src/rvq_quant_pack.metal, wrapper
// metal/_rvq_quant_pack.py:83-149) and of its unfused path (ScalarCodebook.quantize,
// codebooks/scalar_codebook.py:77-95, then _pack_indices, cache/turboquant_rvq_cache.py:82-106),
// which the reference pins to each other bit for bit. One thread produces one word of each
// stream: it reads its 32 / bits consecutive coordinates (8 to 64 bytes), so neighbouring
// threads read neighbouring memory and nothing is staged. HBM-bound: 2 bytes in, bits / 4 out
// per coordinate.
// Both codes are a function of the coordinate's 16 bits alone (the residual is rounded to fp16
// before the second comparison), so a caller that quantizes many vectors with one pair of
// codebooks first builds the 65 536-entry table y -> idx1 | idx2 << 4 (vq_rvq_build_table) and
// passes it in: the kernel then keeps the table in shared memory and spends one byte load per
// coordinate instead of 2 * (2^bits - 1) comparisons, which is what lets it run at the speed
// of its memory traffic.
//
// vq_rvq_unpack_decode: the inverse used on every fetch of the reference's cache
// (metal/src/rvq_unpack_decode.metal, wrapper metal/_rvq_unpack_decode.py:78-183): unpack both
// streams, y = half(c1[idx1] + c2[idx2]), h = WHT(y) / sqrt(D) in float32 with the butterfly order
// (stride 1, 2, 4, ...; lower = self + partner, upper = partner - self), x = half(h * diag),
// out = half(clamp(x * norm, +-65504)). One warp per vector, D / 32 consecutive coordinates per
// lane: the first stages run inside a lane, the rest through shuffles. Rows are read in place
// from a cache buffer of `cap` slots per (batch, head) of which the first `seq` are live.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace vq {
namespace {

constexpr int kMaxLevels = 16;  // bits <= 4

struct RvqTables {
    float c1[kMaxLevels];
    float b1[kMaxLevels];  // 2^bits - 1 used
    float b2[kMaxLevels];
};

template <int BITS>
__global__ void __launch_bounds__(256)
rvq_quant_pack_kernel(const __half *__restrict__ y, int64_t n_rows, int D, int n_words, const __grid_constant__ RvqTables t,
                      uint32_t *__restrict__ packed1, uint32_t *__restrict__ packed2) {
    constexpr int EPW = 32 / BITS;
    constexpr int NB = (1 << BITS) - 1;
    const int64_t total = n_rows * n_words;
    const bool whole = D % EPW == 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        // (rows that are whole words form one contiguous run of words: no division)
        const __half *src;
        int n_el = EPW;
        if (whole) {
            src = y + i * EPW;
        } else {
            const int64_t row = i / n_words;
            const int d0 = (int)(i - row * n_words) * EPW;
            src = y + row * D + d0;
            n_el = min(EPW, D - d0);
        }
        uint32_t w1 = 0u, w2 = 0u;
        // 16-byte loads where the word's coordinates allow it (EPW * 2 bytes is 64, 32 or 16 for 1, 2, 4 bits)
        if ((EPW % 8) == 0 && n_el == EPW && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
#pragma unroll
            for (int v = 0; v < EPW / 8; ++v) {
                const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(src) + v);
                const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const __half hv = __ushort_as_half((unsigned short)((u[e >> 1] >> (16 * (e & 1))) & 0xffffu));
                    const float yv = __half2float(hv);
                    int idx1 = 0;
#pragma unroll
                    for (int k = 0; k < NB; ++k) idx1 += yv > t.b1[k];
                    float cq = t.c1[0];
#pragma unroll
                    for (int k = 1; k <= NB; ++k) cq = idx1 == k ? t.c1[k] : cq;
                    const float r1 = __half2float(__float2half_rn(yv - cq));
                    int idx2 = 0;
#pragma unroll
                    for (int k = 0; k < NB; ++k) idx2 += r1 > t.b2[k];
                    w1 |= (uint32_t)idx1 << ((8 * v + e) * BITS);
                    w2 |= (uint32_t)idx2 << ((8 * v + e) * BITS);
                }
            }
        } else {
            for (int e = 0; e < n_el; ++e) {
                const float yv = __half2float(src[e]);
                int idx1 = 0;
#pragma unroll
                for (int k = 0; k < NB; ++k) idx1 += yv > t.b1[k];
                const float r1 = __half2float(__float2half_rn(yv - t.c1[idx1]));
                int idx2 = 0;
#pragma unroll
                for (int k = 0; k < NB; ++k) idx2 += r1 > t.b2[k];
                w1 |= (uint32_t)idx1 << (e * BITS);
                w2 |= (uint32_t)idx2 << (e * BITS);
            }
        }
        packed1[i] = w1;
        packed2[i] = w2;
    }
}

// table[y bits] = idx1 | idx2 << 4 for every float16 bit pattern.
template <int BITS>
__global__ void __launch_bounds__(256)
rvq_build_table_kernel(const __grid_constant__ RvqTables t, uint8_t *__restrict__ table) {
    constexpr int NB = (1 << BITS) - 1;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 65536) return;
    const float yv = __half2float(__ushort_as_half((unsigned short)i));
    int idx1 = 0;
#pragma unroll
    for (int k = 0; k < NB; ++k) idx1 += yv > t.b1[k];
    float c = t.c1[0];
#pragma unroll
    for (int k = 1; k <= NB; ++k) c = idx1 == k ? t.c1[k] : c;
    const float r1 = __half2float(__float2half_rn(yv - c));
    int idx2 = 0;
#pragma unroll
    for (int k = 0; k < NB; ++k) idx2 += r1 > t.b2[k];
    table[i] = (uint8_t)(idx1 | (idx2 << 4));
}

// One thread produces one word of each stream from the table in shared memory.
template <int BITS>
__global__ void __launch_bounds__(512)
rvq_quant_pack_lut_kernel(const __half *__restrict__ y, int64_t n_rows, int D, int n_words, const uint8_t *__restrict__ table,
                          uint32_t *__restrict__ packed1, uint32_t *__restrict__ packed2) {
    extern __shared__ __align__(16) uint8_t lut[];
    constexpr int EPW = 32 / BITS;
    for (int i = threadIdx.x; i < 65536 / 16; i += blockDim.x)
        reinterpret_cast<uint4 *>(lut)[i] = __ldg(reinterpret_cast<const uint4 *>(table) + i);
    __syncthreads();
    const int64_t total = n_rows * n_words;
    const bool whole = D % EPW == 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        // (rows that are whole words form one contiguous run of words: no division)
        const __half *src;
        int n_el = EPW;
        if (whole) {
            src = y + i * EPW;
        } else {
            const int64_t row = i / n_words;
            const int d0 = (int)(i - row * n_words) * EPW;
            src = y + row * D + d0;
            n_el = min(EPW, D - d0);
        }
        uint32_t w1 = 0u, w2 = 0u;
        if ((EPW % 8) == 0 && n_el == EPW && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
#pragma unroll
            for (int v = 0; v < EPW / 8; ++v) {
                const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(src) + v);
                const uint32_t u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const uint32_t code = lut[(u[e >> 1] >> (16 * (e & 1))) & 0xffffu];
                    w1 |= (code & 15u) << ((8 * v + e) * BITS);
                    w2 |= (code >> 4) << ((8 * v + e) * BITS);
                }
            }
        } else {
            for (int e = 0; e < n_el; ++e) {
                const uint32_t code = lut[__half_as_ushort(src[e])];
                w1 |= (code & 15u) << (e * BITS);
                w2 |= (code >> 4) << (e * BITS);
            }
        }
        packed1[i] = w1;
        packed2[i] = w2;
    }
}

struct RvqDecodeTables {
    float c1[kMaxLevels];
    float c2[kMaxLevels];
};

// EPL = D / 32 consecutive coordinates per lane (D >= 32), or one coordinate in the first D lanes (D < 32).
template <int BITS, int EPL>
__global__ void __launch_bounds__(256)
rvq_unpack_decode_kernel(const uint32_t *__restrict__ packed1, const uint32_t *__restrict__ packed2, const void *__restrict__ norms,
                         int norms_dtype, const __grid_constant__ RvqDecodeTables t, const float *__restrict__ diag, int D, int n_words,
                         int64_t n_out, int64_t seq, int64_t cap, float inv_sqrt_d, __half *__restrict__ out) {
    constexpr int EPW = 32 / BITS;
    constexpr uint32_t MASK = (1u << BITS) - 1u;
    // the two centroid tables in shared memory (a lookup by a per-lane index from the constant
    // bank would be serialised; 16 floats sit in 16 banks)
    __shared__ float sc1[kMaxLevels], sc2[kMaxLevels];
    if (threadIdx.x < kMaxLevels) { sc1[threadIdx.x] = t.c1[threadIdx.x]; sc2[threadIdx.x] = t.c2[threadIdx.x]; }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const bool live = EPL > 1 || lane < D;
    const int lanes = EPL > 1 ? 32 : D;
    float dg[EPL];
#pragma unroll
    for (int e = 0; e < EPL; ++e) dg[e] = live ? __ldg(diag + lane * EPL + e) : 0.f;
#pragma unroll 2
    for (int64_t n = warp0; n < n_out; n += n_warps) {
        int64_t row = n;
        if (seq != cap) {
            if (n_out < (1ll << 31)) {
                const uint32_t bh = (uint32_t)n / (uint32_t)seq;
                row = (int64_t)bh * cap + ((uint32_t)n - bh * (uint32_t)seq);
            } else {
                const int64_t bh = n / seq;
                row = bh * cap + (n - bh * seq);
            }
        }
        float v[EPL];
        if (live) {
            // this lane's coordinates lane*EPL .. +EPL-1 come from one or more whole words, or share one
            uint32_t w1 = 0u, w2 = 0u;
            int cur = -1;
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                const int d = lane * EPL + e;
                const int w = d / EPW, shift = (d % EPW) * BITS;
                if (w != cur) {
                    w1 = __ldg(packed1 + row * n_words + w);
                    w2 = __ldg(packed2 + row * n_words + w);
                    cur = w;
                }
                // (two fp16 values: their float sum is exact, so one rounding gives the fp16 sum)
                v[e] = __half2float(__float2half_rn(sc1[(w1 >> shift) & MASK] + sc2[(w2 >> shift) & MASK]));
            }
        } else {
#pragma unroll
            for (int e = 0; e < EPL; ++e) v[e] = 0.f;
        }
        // butterfly, strides ascending: inside the lane first, then across lanes
#pragma unroll
        for (int s = 1; s < EPL; s <<= 1) {
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                if ((e & s) == 0) {
                    const float lo = v[e], hi = v[e | s];
                    v[e] = lo + hi;
                    v[e | s] = lo - hi;
                }
            }
        }
        for (int s = 1; s < lanes; s <<= 1) {
            const float sgn = (lane & s) ? -1.f : 1.f;  // upper lane: partner - self; lower: self + partner
#pragma unroll
            for (int e = 0; e < EPL; ++e) v[e] = fmaf(sgn, v[e], __shfl_xor_sync(0xffffffffu, v[e], s));
        }
        if (live) {
            const float nrm = load_as_f32(norms, norms_dtype, row);
            __half res[EPL];
            // (diag is +-1: half(h * diag) = diag * half(h), and the sign can ride on the norm)
            if constexpr (EPL >= 2) {
#pragma unroll
                for (int e = 0; e < EPL; e += 2) {
                    const float2 xu = __half22float2(__floats2half2_rn(__fmul_rn(v[e], inv_sqrt_d), __fmul_rn(v[e + 1], inv_sqrt_d)));
                    const float k0 = fminf(fmaxf(__fmul_rn(xu.x, __fmul_rn(dg[e], nrm)), -65504.f), 65504.f);
                    const float k1 = fminf(fmaxf(__fmul_rn(xu.y, __fmul_rn(dg[e + 1], nrm)), -65504.f), 65504.f);
                    *reinterpret_cast<__half2 *>(res + e) = __floats2half2_rn(k0, k1);
                }
            } else {
                const float xu = __half2float(__float2half_rn(__fmul_rn(v[0], inv_sqrt_d)));
                res[0] = __float2half_rn(fminf(fmaxf(__fmul_rn(xu, __fmul_rn(dg[0], nrm)), -65504.f), 65504.f));
            }
            __half *dst = out + n * D + lane * EPL;
            if constexpr (EPL >= 8) {
#pragma unroll
                for (int e = 0; e < EPL; e += 8) *reinterpret_cast<uint4 *>(dst + e) = *reinterpret_cast<const uint4 *>(res + e);
            } else if constexpr (EPL == 4) {
                *reinterpret_cast<uint2 *>(dst) = *reinterpret_cast<const uint2 *>(res);
            } else if constexpr (EPL == 2) {
                *reinterpret_cast<uint32_t *>(dst) = *reinterpret_cast<const uint32_t *>(res);
            } else {
                dst[0] = res[0];
            }
        }
    }
}

// D >= 32: a lane holds 32 consecutive coordinates (D / 32 lanes per vector, 32 / (D / 32) vectors
// per warp), so five butterfly stages run in registers and only log2(D / 32) need shuffles: the
// shuffle unit, not the memory, is what the 32-lanes-per-vector layout above saturates.
template <int BITS>
__global__ void __launch_bounds__(256)
rvq_unpack_decode_wide_kernel(const uint32_t *__restrict__ packed1, const uint32_t *__restrict__ packed2,
                              const void *__restrict__ norms, int norms_dtype, const __grid_constant__ RvqDecodeTables t,
                              const float *__restrict__ diag, int D, int n_words, int64_t n_out, int64_t seq, int64_t cap,
                              float inv_sqrt_d, __half *__restrict__ out) {
    constexpr int EPW = 32 / BITS;
    constexpr uint32_t MASK = (1u << BITS) - 1u;
    __shared__ float sc1[kMaxLevels], sc2[kMaxLevels];
    if (threadIdx.x < kMaxLevels) { sc1[threadIdx.x] = t.c1[threadIdx.x]; sc2[threadIdx.x] = t.c2[threadIdx.x]; }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int lpr = D >> 5, rpw = 32 / lpr;
    const int sub = lane % lpr, rin = lane / lpr;
    const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t base = warp0 * rpw; base < n_out; base += n_warps * rpw) {
        const int64_t n = base + rin;
        const bool live = n < n_out;
        int64_t row = n;
        if (live && seq != cap) {
            if (n_out < (1ll << 31)) {
                const uint32_t bh = (uint32_t)n / (uint32_t)seq;
                row = (int64_t)bh * cap + ((uint32_t)n - bh * (uint32_t)seq);
            } else {
                const int64_t bh = n / seq;
                row = bh * cap + (n - bh * seq);
            }
        }
        float v[32];
        if (live) {
            uint32_t w1 = 0u, w2 = 0u;
            int cur = -1;
            const uint32_t *r1 = packed1 + row * n_words, *r2 = packed2 + row * n_words;
#pragma unroll
            for (int e = 0; e < 32; ++e) {
                const int d = sub * 32 + e;
                const int w = d / EPW, shift = (d % EPW) * BITS;
                if (w != cur) { w1 = __ldg(r1 + w); w2 = __ldg(r2 + w); cur = w; }
                v[e] = sc1[(w1 >> shift) & MASK] + sc2[(w2 >> shift) & MASK];
            }
            // (two fp16 values: their float sum is exact, so one rounding gives the fp16 sum)
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
                const float2 r = __half22float2(__floats2half2_rn(v[e], v[e + 1]));
                v[e] = r.x; v[e + 1] = r.y;
            }
        } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = 0.f;
        }
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
                if ((e & s) == 0) {
                    const float lo = v[e], hi = v[e | s];
                    v[e] = lo + hi;
                    v[e | s] = lo - hi;
                }
            }
        }
        for (int s = 1; s < lpr; s <<= 1) {
            const float sgn = (sub & s) ? -1.f : 1.f;  // upper chunk: partner - self; lower: self + partner
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = fmaf(sgn, v[e], __shfl_xor_sync(0xffffffffu, v[e], s));
        }
        if (live) {
            const float nrm = load_as_f32(norms, norms_dtype, row);
            const float4 *dgp = reinterpret_cast<const float4 *>(diag + sub * 32);
            uint4 *dst = reinterpret_cast<uint4 *>(out + n * D + sub * 32);
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
                const float4 da = __ldg(dgp + e / 4), db = __ldg(dgp + e / 4 + 1);
                const float dg[8] = {da.x, da.y, da.z, da.w, db.x, db.y, db.z, db.w};
                __half2 res[4];
#pragma unroll
                for (int i = 0; i < 8; i += 2) {
                    // (diag is +-1: half(h * diag) = diag * half(h), and the sign can ride on the norm)
                    const float2 xu = __half22float2(__floats2half2_rn(__fmul_rn(v[e + i], inv_sqrt_d), __fmul_rn(v[e + i + 1], inv_sqrt_d)));
                    const float k0 = fminf(fmaxf(__fmul_rn(xu.x, __fmul_rn(dg[i], nrm)), -65504.f), 65504.f);
                    const float k1 = fminf(fmaxf(__fmul_rn(xu.y, __fmul_rn(dg[i + 1], nrm)), -65504.f), 65504.f);
                    res[i / 2] = __floats2half2_rn(k0, k1);
                }
                dst[e / 8] = *reinterpret_cast<const uint4 *>(res);
            }
        }
    }
}

int32_t check_bits(int32_t bits, const char *who) {
    VQ_REQUIRE(bits >= 1 && bits <= 4, VQ_ERR_SHAPE, "%s: bits must be 1-4, got %d", who, bits);
    return VQ_OK;
}

}  // namespace
}  // namespace vq

static void fill_tables(vq::RvqTables &t, const float *centroids1, const float *boundaries1, const float *boundaries2, int bits) {
    const int levels = 1 << bits;
    for (int i = 0; i < levels; ++i) t.c1[i] = centroids1[i];
    for (int i = 0; i < levels - 1; ++i) { t.b1[i] = boundaries1[i]; t.b2[i] = boundaries2[i]; }
}

extern "C" int32_t vq_rvq_build_table(const float *centroids1, const float *boundaries1, const float *boundaries2, int32_t bits,
                                      uint8_t *table, void *stream) {
    using namespace vq;
    int32_t rc = check_bits(bits, "rvq_build_table");
    if (rc != VQ_OK) return rc;
    VQ_REQUIRE(centroids1 && boundaries1 && boundaries2 && table, VQ_ERR_SHAPE, "rvq_build_table: NULL argument");
    VQ_REQUIRE(is_aligned(table, 16), VQ_ERR_ALIGN, "rvq_build_table: the table must be 16-byte aligned");
    DeviceInfo di;
    rc = device_info(&di);
    if (rc != VQ_OK) return rc;
    RvqTables t = {};
    fill_tables(t, centroids1, boundaries1, boundaries2, bits);
    cudaStream_t st = (cudaStream_t)stream;
    switch (bits) {
        case 1: rvq_build_table_kernel<1><<<256, 256, 0, st>>>(t, table); break;
        case 2: rvq_build_table_kernel<2><<<256, 256, 0, st>>>(t, table); break;
        case 3: rvq_build_table_kernel<3><<<256, 256, 0, st>>>(t, table); break;
        default: rvq_build_table_kernel<4><<<256, 256, 0, st>>>(t, table); break;
    }
    VQ_CHECK_LAUNCH("rvq_build_table_kernel");
    return VQ_OK;
}

extern "C" int32_t vq_rvq_quant_pack(const void *rotated, int64_t n_rows, int32_t D, const float *centroids1,
                                     const float *boundaries1, const float *boundaries2, const uint8_t *table, int32_t bits,
                                     uint32_t *packed1, uint32_t *packed2, void *stream) {
    using namespace vq;
    int32_t rc = check_bits(bits, "rvq_quant_pack");
    if (rc != VQ_OK) return rc;
    VQ_REQUIRE(n_rows >= 0 && D >= 1 && D <= 1024, VQ_ERR_SHAPE, "rvq_quant_pack: D=%d must be in 1..1024", D);
    if (n_rows == 0) return VQ_OK;
    VQ_REQUIRE(rotated && packed1 && packed2, VQ_ERR_SHAPE, "rvq_quant_pack: NULL argument");
    VQ_REQUIRE(table || (centroids1 && boundaries1 && boundaries2), VQ_ERR_SHAPE, "rvq_quant_pack: neither a table nor the codebooks were given");
    VQ_REQUIRE(is_aligned(rotated, 2) && is_aligned(packed1, 4) && is_aligned(packed2, 4) && is_aligned(table, 16), VQ_ERR_ALIGN,
               "rvq_quant_pack: misaligned buffer");
    DeviceInfo di;
    rc = device_info(&di);
    if (rc != VQ_OK) return rc;
    const int epw = 32 / bits;
    const int n_words = (D + epw - 1) / epw;
    const int64_t total = n_rows * n_words;
    cudaStream_t st = (cudaStream_t)stream;
    const __half *y = (const __half *)rotated;
    if (table != nullptr && total >= 65536) {
        // every CTA keeps the 64 KB table in shared memory, three CTAs per SM (smaller inputs: filling
        // the table would cost more than it saves)
        const size_t smem = 65536;
        const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(total, 512), (int64_t)di.sm_count * 3);
#define VQ_RVQ_LUT(B)                                                                                                       \
    do {                                                                                                                    \
        VQ_CHECK_CUDA(cudaFuncSetAttribute(rvq_quant_pack_lut_kernel<B>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        rvq_quant_pack_lut_kernel<B><<<blocks, 512, smem, st>>>(y, n_rows, D, n_words, table, packed1, packed2);            \
    } while (0)
        switch (bits) {
            case 1: VQ_RVQ_LUT(1); break;
            case 2: VQ_RVQ_LUT(2); break;
            case 3: VQ_RVQ_LUT(3); break;
            default: VQ_RVQ_LUT(4); break;
        }
#undef VQ_RVQ_LUT
        VQ_CHECK_LAUNCH("rvq_quant_pack_lut_kernel");
        return VQ_OK;
    }
    VQ_REQUIRE(centroids1 && boundaries1 && boundaries2, VQ_ERR_SHAPE, "rvq_quant_pack: the codebooks are needed for inputs below 65536 words");
    // the codebooks are host arrays (a handful of floats): they travel as kernel arguments
    RvqTables t = {};
    fill_tables(t, centroids1, boundaries1, boundaries2, bits);
    const unsigned blocks = (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(total, 256), (int64_t)di.sm_count * 16));
    switch (bits) {
        case 1: rvq_quant_pack_kernel<1><<<blocks, 256, 0, st>>>(y, n_rows, D, n_words, t, packed1, packed2); break;
        case 2: rvq_quant_pack_kernel<2><<<blocks, 256, 0, st>>>(y, n_rows, D, n_words, t, packed1, packed2); break;
        case 3: rvq_quant_pack_kernel<3><<<blocks, 256, 0, st>>>(y, n_rows, D, n_words, t, packed1, packed2); break;
        default: rvq_quant_pack_kernel<4><<<blocks, 256, 0, st>>>(y, n_rows, D, n_words, t, packed1, packed2); break;
    }
    VQ_CHECK_LAUNCH("rvq_quant_pack_kernel");
    return VQ_OK;
}

extern "C" int32_t vq_rvq_unpack_decode(const uint32_t *packed1, const uint32_t *packed2, const void *norms, int32_t norms_dtype,
                                        const float *centroids1, const float *centroids2, const float *diag, int32_t bits,
                                        int32_t D, int64_t n_bh, int64_t seq, int64_t cap, void *out, void *stream) {
    using namespace vq;
    int32_t rc = check_bits(bits, "rvq_unpack_decode");
    if (rc != VQ_OK) return rc;
    VQ_REQUIRE(D >= 1 && D <= 1024 && (D & (D - 1)) == 0, VQ_ERR_SHAPE, "rvq_unpack_decode: d=%d must be a power of two <= 1024", D);
    VQ_REQUIRE(n_bh >= 0 && seq >= 0 && seq <= cap, VQ_ERR_SHAPE, "rvq_unpack_decode: seq_len=%lld must be in [0, %lld]", (long long)seq, (long long)cap);
    VQ_REQUIRE(norms_dtype >= 0 && norms_dtype <= 2, VQ_ERR_DTYPE, "rvq_unpack_decode: bad norms dtype");
    const int64_t n_out = n_bh * seq;
    if (n_out == 0) return VQ_OK;
    VQ_REQUIRE(packed1 && packed2 && norms && centroids1 && centroids2 && diag && out, VQ_ERR_SHAPE, "rvq_unpack_decode: NULL argument");
    DeviceInfo di;
    rc = device_info(&di);
    if (rc != VQ_OK) return rc;
    RvqDecodeTables t = {};
    for (int i = 0; i < (1 << bits); ++i) { t.c1[i] = centroids1[i]; t.c2[i] = centroids2[i]; }
    const int epw = 32 / bits;
    const int n_words = (D + epw - 1) / epw;
    const float inv_sqrt_d = 1.0f / sqrtf((float)D);
    cudaStream_t st = (cudaStream_t)stream;
    __half *o = (__half *)out;
    if (D >= 32) {
        VQ_REQUIRE(is_aligned(out, 16) && is_aligned(diag, 16), VQ_ERR_ALIGN, "rvq_unpack_decode: out and diag must be 16-byte aligned");
        const int rpw = 32 / (D / 32);
        const unsigned blocks = (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(n_out, 8 * rpw), (int64_t)di.sm_count * 8));
#define VQ_RVQ_WIDE(B) \
    rvq_unpack_decode_wide_kernel<B><<<blocks, 256, 0, st>>>(packed1, packed2, norms, norms_dtype, t, diag, D, n_words, n_out, seq, cap, inv_sqrt_d, o)
        switch (bits) {
            case 1: VQ_RVQ_WIDE(1); break;
            case 2: VQ_RVQ_WIDE(2); break;
            case 3: VQ_RVQ_WIDE(3); break;
            default: VQ_RVQ_WIDE(4); break;
        }
#undef VQ_RVQ_WIDE
        VQ_CHECK_LAUNCH("rvq_unpack_decode_wide_kernel");
        return VQ_OK;
    }
    const unsigned blocks = (unsigned)std::max<int64_t>(1, std::min<int64_t>(ceil_div(n_out, 8), (int64_t)di.sm_count * 16));
#define VQ_RVQ_DEC(B) \
    rvq_unpack_decode_kernel<B, 1><<<blocks, 256, 0, st>>>(packed1, packed2, norms, norms_dtype, t, diag, D, n_words, n_out, seq, cap, inv_sqrt_d, o)
    switch (bits) {
        case 1: VQ_RVQ_DEC(1); break;
        case 2: VQ_RVQ_DEC(2); break;
        case 3: VQ_RVQ_DEC(3); break;
        default: VQ_RVQ_DEC(4); break;
    }
#undef VQ_RVQ_DEC
    VQ_CHECK_LAUNCH("rvq_unpack_decode_kernel");
    return VQ_OK;
}
