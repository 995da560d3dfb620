// RaBitQ 1-bit key encode (randomized Hadamard rotation + sign bits + L1 magnitude),
// 4-bit value packing and the packed Hamming score.
//
// Encode: one warp per key row. The row (D <= 1024, a power of two) sits in shared memory;
// the Sylvester butterfly pairs element i+j with i+j+stride exactly as the reference's
// sequential loop does (lower = a+b, upper = a-b), so every stage is the same float32
// operation on the same operands and the result is bit-identical however the pairs are
// spread over lanes. Sign bits are packed with ballots (32 bits = 4 output bytes).
#include <algorithm>
#include <type_traits>

#include "common.cuh"

namespace vq {

constexpr int kEncWarps = 4;

template <typename T>
__global__ void __launch_bounds__(kEncWarps * 32)
rabitq_encode_kernel(const T *__restrict__ keys, int64_t n, int D, const float *__restrict__ diag,
                     int rotate, uint8_t *__restrict__ bits, float *__restrict__ mag) {
    extern __shared__ float sh[];  // [kEncWarps][D]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float *buf = sh + (size_t)warp * D;
    const float inv_norm_den = sqrtf((float)D);
    const int n_bytes = D / 8;
    for (int64_t row = (int64_t)blockIdx.x * kEncWarps + warp; row < n; row += (int64_t)gridDim.x * kEncWarps) {
        for (int i = lane; i < D; i += 32) {
            float v = to_f32<T>(keys[row * D + i]);
            if (rotate) v = __fmul_rn(v, diag[i]);
            buf[i] = v;
        }
        __syncwarp();
        if (rotate) {
            for (int stride = 1; stride < D; stride <<= 1) {
                // pair p (0..D/2-1): lower index = (p / stride) * 2 * stride + p % stride
                for (int p = lane; p < D / 2; p += 32) {
                    const int lo = (p / stride) * 2 * stride + (p % stride);
                    const float a = buf[lo], b = buf[lo + stride];
                    buf[lo] = __fadd_rn(a, b);
                    buf[lo + stride] = __fsub_rn(a, b);
                }
                __syncwarp();
            }
        }
        float l1 = 0.f;
        for (int i0 = 0; i0 < D; i0 += 32) {
            const int i = i0 + lane;
            float y = 0.f;
            bool live = i < D;
            if (live) {
                y = buf[i];
                if (rotate) y = __fdiv_rn(y, inv_norm_den);
                l1 += fabsf(y);
            }
            const uint32_t ballot = __ballot_sync(0xffffffffu, live && y >= 0.f);
            if (lane < 4 && i0 / 8 + lane < n_bytes) bits[row * n_bytes + i0 / 8 + lane] = (uint8_t)(ballot >> (8 * lane));
        }
        l1 = warp_sum(l1);
        if (lane == 0) mag[row] = l1 / (float)D;
        __syncwarp();
    }
}

// Register-resident variant for D = 32 * EPL (32, 64, 128, 256): lane l holds elements
// EPL*l .. EPL*l + EPL-1. Butterfly stages with stride < EPL pair registers of one lane;
// larger strides pair lane l with lane l ^ (stride / EPL) through a shuffle. Every pair is
// still (lower + upper, lower - upper), so the result is bit-identical to the shared-memory
// kernel and to the reference's sequential loop.
// EPL consecutive elements as floats with the widest aligned load (the caller guarantees a
// 16-byte aligned base; rows are D elements apart, so EPL * sizeof(T) divides every offset).
template <typename T, int EPL>
__device__ __forceinline__ void load_epl(const T *p, float (&v)[EPL]) {
    if constexpr (sizeof(T) == 4) {
        if constexpr (EPL % 4 == 0) {
#pragma unroll
            for (int i = 0; i < EPL / 4; ++i) {
                const float4 f = __ldg(reinterpret_cast<const float4 *>(p) + i);
                v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
            }
        } else if constexpr (EPL == 2) {
            const float2 f = __ldg(reinterpret_cast<const float2 *>(p));
            v[0] = f.x; v[1] = f.y;
        } else {
            v[0] = __ldg(reinterpret_cast<const float *>(p));
        }
    } else {
        uint32_t w[(EPL + 1) / 2];
        if constexpr (EPL == 8) { const uint4 t = __ldg(reinterpret_cast<const uint4 *>(p)); w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w; }
        else if constexpr (EPL == 4) { const uint2 t = __ldg(reinterpret_cast<const uint2 *>(p)); w[0] = t.x; w[1] = t.y; }
        else if constexpr (EPL == 2) { w[0] = __ldg(reinterpret_cast<const uint32_t *>(p)); }
        else { v[0] = to_f32<T>(*p); return; }
#pragma unroll
        for (int i = 0; i < EPL / 2; ++i) {
            if constexpr (std::is_same<T, __half>::value) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
                v[2 * i] = f.x; v[2 * i + 1] = f.y;
            } else {
                v[2 * i] = __uint_as_float(w[i] << 16); v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            }
        }
    }
}

template <typename T, int EPL>
__global__ void __launch_bounds__(128)
rabitq_encode_reg_kernel(const T *__restrict__ keys, int64_t n, const float *__restrict__ diag, int rotate,
                         uint8_t *__restrict__ bits, float *__restrict__ mag) {
    constexpr int D = 32 * EPL;
    constexpr int R = EPL <= 4 ? 4 : 2;  // rows a warp carries at once: loads in flight and independent butterfly chains
    const int lane = threadIdx.x & 31;
    const int64_t warp_id = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int64_t n_warps = (int64_t)gridDim.x * 4;
    float dg[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) dg[j] = rotate ? diag[EPL * lane + j] : 1.f;
    const float den = sqrtf((float)D);
    const float rden = __frcp_rn(den);
    for (int64_t row0 = warp_id * R; row0 < n; row0 += n_warps * R) {
        float v[R][EPL];
#pragma unroll
        for (int r = 0; r < R; ++r) load_epl<T, EPL>(keys + min(row0 + r, n - 1) * D + EPL * lane, v[r]);
        if (rotate) {
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int j = 0; j < EPL; ++j) v[r][j] = __fmul_rn(v[r][j], dg[j]);
#pragma unroll
            for (int s = 1; s < EPL; s <<= 1) {
#pragma unroll
                for (int r = 0; r < R; ++r)
#pragma unroll
                    for (int j = 0; j < EPL; ++j) {
                        if ((j & s) == 0) {
                            const float a = v[r][j], b2 = v[r][j + s];
                            v[r][j] = __fadd_rn(a, b2);
                            v[r][j + s] = __fsub_rn(a, b2);
                        }
                    }
            }
#pragma unroll
            for (int m = 1; m < 32; m <<= 1) {
                const bool upper = lane & m;
#pragma unroll
                for (int r = 0; r < R; ++r)
#pragma unroll
                    for (int j = 0; j < EPL; ++j) {
                        const float other = __shfl_xor_sync(0xffffffffu, v[r][j], m);
                        v[r][j] = upper ? __fsub_rn(other, v[r][j]) : __fadd_rn(v[r][j], other);
                    }
            }
            // v / sqrt(D), correctly rounded without the divide: rc = RN(1/den), t0 = RN(v*rc),
            // r = v - den*t0 (exact in one fma), RN(t0 + r*rc) is the IEEE quotient (Markstein).
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int j = 0; j < EPL; ++j) {
                    const float t0 = __fmul_rn(v[r][j], rden);
                    v[r][j] = __fmaf_rn(__fmaf_rn(-den, t0, v[r][j]), rden, t0);
                }
        }
        constexpr int LPW = 32 / EPL;  // lanes per 32-bit output word
#pragma unroll
        for (int r = 0; r < R; ++r) {
            float l1 = 0.f;
            uint32_t mine = 0;
#pragma unroll
            for (int j = 0; j < EPL; ++j) {
                l1 += fabsf(v[r][j]);
                mine |= (v[r][j] >= 0.f ? 1u : 0u) << j;
            }
            uint32_t word = mine << (EPL * (lane % LPW));
#pragma unroll
            for (int m = 1; m < LPW; m <<= 1) word |= __shfl_xor_sync(0xffffffffu, word, m);
            l1 = warp_sum(l1);
            if (row0 + r < n) {
                if (lane % LPW == 0) reinterpret_cast<uint32_t *>(bits + (row0 + r) * (D / 8))[lane / LPW] = word;
                if (lane == 0) mag[row0 + r] = l1 / (float)D;
            }
        }
    }
}

// D = 32 * LPR with 32 consecutive elements per lane: LPR lanes share a key row, a warp carries
// 32 / LPR rows. The five butterfly stages with stride < 32 pair registers of one lane, only
// the log2(LPR) widest stages cross lanes (2 of 7 stages at D = 128, against 5 of 7 with four
// elements per lane), and a lane's 32 sign bits are one whole output word. Every pair is
// still (lower + upper, lower - upper): bit-identical to the sequential Sylvester loop.
template <typename T, int LPR>
__global__ void __launch_bounds__(128)
rabitq_encode_wide_kernel(const T *__restrict__ keys, int64_t n, const float *__restrict__ diag,
                          uint8_t *__restrict__ bits, float *__restrict__ mag) {
    constexpr int D = 32 * LPR, RPW = 32 / LPR;
    const int lane = threadIdx.x & 31;
    const int part = lane % LPR, rsub = lane / LPR;  // which 32 elements of which of the warp's rows
    const int64_t warp_id = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int64_t n_warps = (int64_t)gridDim.x * 4;
    float dg[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) dg[j] = diag[32 * part + j];
    const float den = sqrtf((float)D), rden = __frcp_rn(den);
    for (int64_t row0 = warp_id * RPW; row0 < n; row0 += n_warps * RPW) {
        const int64_t row = min(row0 + rsub, n - 1);
        float v[32];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float t[8];
            load_epl<T, 8>(keys + row * D + 32 * part + 8 * k, t);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[8 * k + j] = __fmul_rn(t[j], dg[8 * k + j]);
        }
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                if ((j & s) == 0) {
                    const float a = v[j], b2 = v[j + s];
                    v[j] = __fadd_rn(a, b2);
                    v[j + s] = __fsub_rn(a, b2);
                }
            }
        }
#pragma unroll
        for (int m = 1; m < LPR; m <<= 1) {
            const bool upper = part & m;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float other = __shfl_xor_sync(0xffffffffu, v[j], m);
                v[j] = upper ? __fsub_rn(other, v[j]) : __fadd_rn(v[j], other);
            }
        }
        float l1 = 0.f;
        uint32_t word = 0;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const float t0 = __fmul_rn(v[j], rden);
            const float y = __fmaf_rn(__fmaf_rn(-den, t0, v[j]), rden, t0);  // v / sqrt(D), correctly rounded
            l1 += fabsf(y);
            word |= (y >= 0.f ? 1u : 0u) << j;
        }
#pragma unroll
        for (int m = 1; m < LPR; m <<= 1) l1 += __shfl_xor_sync(0xffffffffu, l1, m);
        if (row0 + rsub < n) {
            reinterpret_cast<uint32_t *>(bits + (row0 + rsub) * (D / 8))[part] = word;
            if (part == 0) mag[row0 + rsub] = l1 / (float)D;
        }
    }
}

__global__ void rabitq_pack_values_kernel(const uint8_t *__restrict__ v_idx, int64_t n_out,
                                          uint8_t *__restrict__ packed) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_out;
         i += (int64_t)gridDim.x * blockDim.x)
        packed[i] = (uint8_t)((v_idx[2 * i] & 0xF) | ((v_idx[2 * i + 1] & 0xF) << 4));
}

__global__ void rabitq_hamming_kernel(const uint8_t *__restrict__ q_bits, const uint8_t *__restrict__ bits,
                                      int64_t n, int n_bytes, float scale, const float *__restrict__ cx,
                                      float *__restrict__ score) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (int64_t)gridDim.x * blockDim.x) {
        int ham = 0;
        for (int j = 0; j < n_bytes; ++j) ham += __popc((uint32_t)(q_bits[j] ^ bits[i * n_bytes + j]));
        score[i] = __fadd_rn(__fmul_rn((float)ham, scale), cx ? cx[i] : 0.f);
    }
}

}  // namespace vq

extern "C" int32_t vq_rabitq_encode(const void *keys, int32_t dtype, int64_t n, int32_t D, const float *diag,
                                    int32_t rotate, uint8_t *bits, float *mag, void *stream) {
    using namespace vq;
    VQ_REQUIRE(n >= 0, VQ_ERR_SHAPE, "rabitq_encode: n must be >= 0");
    VQ_REQUIRE(D >= 8 && D <= 1024 && D % 8 == 0, VQ_ERR_SHAPE, "rabitq_encode: D=%d must be a multiple of 8 in 8..1024", D);
    VQ_REQUIRE(!rotate || (D & (D - 1)) == 0, VQ_ERR_SHAPE, "rabitq_encode: D=%d must be a power of 2 for the Hadamard rotation", D);
    VQ_REQUIRE(!rotate || diag != nullptr, VQ_ERR_SHAPE, "rabitq_encode: diag is NULL");
    if (n == 0) return VQ_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if ((D == 64 || D == 128 || D == 256) && rotate && is_aligned(bits, 4) && is_aligned(keys, 16)) {
        const int rpw = 32 / (D / 32);
        const unsigned rb = (unsigned)std::min<int64_t>(ceil_div(n, 4 * rpw), 148 * 16);
#define VQ_ENCW(TT)                                                                                              \
    switch (D) {                                                                                                 \
        case 64: rabitq_encode_wide_kernel<TT, 2><<<rb, 128, 0, st>>>((const TT *)keys, n, diag, bits, mag); break;  \
        case 128: rabitq_encode_wide_kernel<TT, 4><<<rb, 128, 0, st>>>((const TT *)keys, n, diag, bits, mag); break; \
        default: rabitq_encode_wide_kernel<TT, 8><<<rb, 128, 0, st>>>((const TT *)keys, n, diag, bits, mag); break;  \
    }
        switch (dtype) {
            case VQ_F16: VQ_ENCW(__half); break;
            case VQ_BF16: VQ_ENCW(__nv_bfloat16); break;
            case VQ_F32: VQ_ENCW(float); break;
            default: return fail(VQ_ERR_DTYPE, "rabitq_encode: unknown dtype %d", dtype);
        }
#undef VQ_ENCW
        VQ_CHECK_LAUNCH("rabitq_encode_wide_kernel");
        return VQ_OK;
    }
    if ((D == 32 || D == 64 || D == 128 || D == 256) && is_aligned(bits, 4) && is_aligned(keys, 16)) {
        const unsigned rb = (unsigned)std::min<int64_t>(ceil_div(n, 16), 148 * 16);
#define VQ_ENC(TT, EPL) rabitq_encode_reg_kernel<TT, EPL><<<rb, 128, 0, st>>>((const TT *)keys, n, diag, rotate, bits, mag)
#define VQ_ENC_D(TT)                                                                   \
    switch (D) {                                                                       \
        case 32: VQ_ENC(TT, 1); break;                                                 \
        case 64: VQ_ENC(TT, 2); break;                                                 \
        case 128: VQ_ENC(TT, 4); break;                                                \
        default: VQ_ENC(TT, 8); break;                                                 \
    }
        switch (dtype) {
            case VQ_F16: VQ_ENC_D(__half); break;
            case VQ_BF16: VQ_ENC_D(__nv_bfloat16); break;
            case VQ_F32: VQ_ENC_D(float); break;
            default: return fail(VQ_ERR_DTYPE, "rabitq_encode: unknown dtype %d", dtype);
        }
#undef VQ_ENC_D
#undef VQ_ENC
        VQ_CHECK_LAUNCH("rabitq_encode_reg_kernel");
        return VQ_OK;
    }
    const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(n, kEncWarps), 148 * 16);
    const size_t smem = (size_t)kEncWarps * D * sizeof(float);
    switch (dtype) {
        case VQ_F16: rabitq_encode_kernel<__half><<<blocks, kEncWarps * 32, smem, st>>>((const __half *)keys, n, D, diag, rotate, bits, mag); break;
        case VQ_BF16: rabitq_encode_kernel<__nv_bfloat16><<<blocks, kEncWarps * 32, smem, st>>>((const __nv_bfloat16 *)keys, n, D, diag, rotate, bits, mag); break;
        case VQ_F32: rabitq_encode_kernel<float><<<blocks, kEncWarps * 32, smem, st>>>((const float *)keys, n, D, diag, rotate, bits, mag); break;
        default: return fail(VQ_ERR_DTYPE, "rabitq_encode: unknown dtype %d", dtype);
    }
    VQ_CHECK_LAUNCH("rabitq_encode_kernel");
    return VQ_OK;
}

extern "C" int32_t vq_rabitq_pack_values(const uint8_t *v_idx, int64_t n_out, uint8_t *packed, void *stream) {
    using namespace vq;
    VQ_REQUIRE(n_out >= 0, VQ_ERR_SHAPE, "rabitq_pack_values: n_out must be >= 0");
    if (n_out == 0) return VQ_OK;
    const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(n_out, 256), 148 * 16);
    rabitq_pack_values_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(v_idx, n_out, packed);
    VQ_CHECK_LAUNCH("rabitq_pack_values_kernel");
    return VQ_OK;
}

extern "C" int32_t vq_rabitq_hamming_score(const uint8_t *q_bits, const uint8_t *bits, int64_t n, int32_t n_bytes,
                                           float scale, const float *cx, float *score, void *stream) {
    using namespace vq;
    VQ_REQUIRE(n >= 0 && n_bytes >= 1, VQ_ERR_SHAPE, "rabitq_hamming_score: bad sizes");
    if (n == 0) return VQ_OK;
    const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(n, 256), 148 * 16);
    rabitq_hamming_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(q_bits, bits, n, n_bytes, scale, cx, score);
    VQ_CHECK_LAUNCH("rabitq_hamming_kernel");
    return VQ_OK;
}
