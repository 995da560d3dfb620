// KIVI quantize + pack, tuned for the serving shape: head_dim 128, group 32, f16/bf16 input,
// 2/4/8-bit containers. HBM-bound streaming pass (read 2 B per element, write sb/8 B plus the
// group parameters); the general kernels in kivi_quant.cu cover every other shape.
//
// One warp owns one tile of 32 tokens x 128 channels. Lane l loads rows 2i + (l >> 4),
// i = 0..15, as 16-byte vectors of the 8 channels 8*(l & 15) .. +7, so every load
// instruction of the warp covers two whole 256-byte rows and the tile is read exactly once
// (it stays in registers as packed halves between the min/max pass and the code pass).
//   keys   (axis 0): a lane sees 16 of the 32 tokens of its 8 channels; one xor-16 exchange
//                    completes each channel's min/max. Codes of a row's 8 channels are packed
//                    in-lane into one word: no cross-lane packing.
//   values (axis 1): a row's 32-channel group is 4 neighbouring lanes: two xor shuffles.
// Extrema are taken on the packed 16-bit values (min/max do not round), two per instruction.
// Rounding is bit-identical to the reference's float32 divide + round-half-even: the correctly
// rounded quotient comes from a reciprocal and two fused multiply-adds (see codes8_fast), the
// rounding from a magic-number add. This file is compiled with -fmad=false; the fused
// operations it uses are explicit.
#include "common.cuh"
#include "kivi_quant_tile.h"

namespace vq {
namespace {

constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23: x + kMagic rounds x to the nearest-even integer

// a / b correctly rounded (== __fdiv_rn) from rb = RN(1/b): t0 = RN(a*rb), r = a - b*t0 (exact
// in one fma), RN(t0 + r*rb). Used where the divisor is shared by many quotients.
__device__ __forceinline__ float div_by(float a, float b, float rb) {
    const float t0 = __fmul_rn(a, rb);
    const float q = __fmaf_rn(__fmaf_rn(-b, t0, a), rb, t0);
    return fabsf(t0) < INFINITY ? q : t0;  // an infinite or NaN quotient stays what the divide gives
}

// ---- packed (two elements per register) min / max and widening -----------------------------
template <typename T> struct Pk;
template <> struct Pk<__half> {
    using t2 = __half2;
    static __device__ __forceinline__ float2 widen(uint32_t w) { return __half22float2(*reinterpret_cast<const __half2 *>(&w)); }
};
template <> struct Pk<__nv_bfloat16> {
    using t2 = __nv_bfloat162;
    static __device__ __forceinline__ float2 widen(uint32_t w) {
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    }
};
template <typename T>
__device__ __forceinline__ uint32_t pmin(uint32_t a, uint32_t b) {
    using t2 = typename Pk<T>::t2;
    t2 r = __hmin2(*reinterpret_cast<const t2 *>(&a), *reinterpret_cast<const t2 *>(&b));
    return *reinterpret_cast<uint32_t *>(&r);
}
template <typename T>
__device__ __forceinline__ uint32_t pmax(uint32_t a, uint32_t b) {
    using t2 = typename Pk<T>::t2;
    t2 r = __hmax2(*reinterpret_cast<const t2 *>(&a), *reinterpret_cast<const t2 *>(&b));
    return *reinterpret_cast<uint32_t *>(&r);
}

// Codes of 8 neighbouring channels of one row, packed into `SB`-bit fields (LSB first).
// The IEEE quotient (v - min) / scale is produced without the divide instruction: with
// rc = RN(1/scale) (correctly rounded), t0 = RN(d*rc), r = d - scale*t0 (exact, one fma),
// RN(t0 + r*rc) is the correctly rounded quotient (Markstein's theorem; cross-checked against
// the divide on 8e10 operand pairs of this range, ties included). It is rounded to the
// nearest-even integer by the magic-number add; the integer then sits in the low mantissa
// bits of that sum and is shifted into place by an integer multiply-add. 0 <= quotient <=
// levels for finite input, so no clamp; `odd` reports a non-finite or out-of-range quotient
// (non-finite input), for which the caller falls back to the clamped divide.
template <int SB>
__device__ __forceinline__ uint64_t codes8_fast(const float (&v)[8], const float (&mn)[8], const float (&sc)[8],
                                                const float (&rc)[8], float levels, bool &odd) {
    uint32_t lo = 0, hi = 0;
    bool bad = false;
    const float lim = levels + 0.25f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float d = __fsub_rn(v[j], mn[j]);
        const float t0 = __fmul_rn(d, rc[j]);
        const float r = __fmaf_rn(-sc[j], t0, d);
        const float t = __fmaf_rn(r, rc[j], t0);
        bad |= !(t < lim);  // NaN too; a finite quotient is at most levels * (1 + 2^-22)
        const uint32_t bits = __float_as_uint(__fadd_rn(t, kMagic));  // 0x4B400000 + code
        if (SB == 8 && j >= 4) hi += bits << (8 * (j - 4));
        else lo += bits << (SB * j);
    }
    odd = bad;
    // remove the exponent bits that rode along (modulo 2^32, like the sums above)
    uint32_t c_lo = 0, c_hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        if (SB == 8 && j >= 4) c_hi += 0x4B400000u << (8 * (j - 4));
        else c_lo += 0x4B400000u << (SB * j);
    }
    return ((uint64_t)(hi - c_hi) << 32) | (uint32_t)(lo - c_lo);
}

template <int SB>
__device__ __forceinline__ uint64_t codes8_exact(const float (&v)[8], const float (&mn)[8], const float (&sc)[8], float levels) {
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float q = fminf(fmaxf(rintf(__fdiv_rn(__fsub_rn(v[j], mn[j]), sc[j])), 0.0f), levels);
        const uint32_t c = (uint32_t)q;
        if (SB == 8 && j >= 4) hi |= c << (8 * (j - 4));
        else lo |= c << (SB * j);
    }
    return ((uint64_t)hi << 32) | lo;
}

template <int SB>
__device__ __forceinline__ void store_packed(uint8_t *row, int cl, uint64_t w) {
    if constexpr (SB == 4) reinterpret_cast<uint32_t *>(row)[cl] = (uint32_t)w;
    else if constexpr (SB == 2) reinterpret_cast<uint16_t *>(row)[cl] = (uint16_t)w;
    else reinterpret_cast<uint2 *>(row)[cl] = make_uint2((uint32_t)w, (uint32_t)(w >> 32));
}

template <typename T, int SB, int AXIS>
__global__ void __launch_bounds__(128, 4)
kivi_quant_tile_kernel(const T *__restrict__ x, int64_t x_stride_bh, int64_t n_tok, int64_t tiles_per_bh,
                       int64_t n_tiles, float levels, float eps, uint8_t *__restrict__ codes,
                       int64_t codes_stride_bh, float *__restrict__ scale, float *__restrict__ zero,
                       int64_t param_stride_bh) {
    constexpr int D = 128, RB = D * SB / 8;
    const int lane = threadIdx.x & 31;
    const int64_t tile_id = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (tile_id >= n_tiles) return;
    const int64_t bh = tile_id / tiles_per_bh, tile = tile_id % tiles_per_bh;
    const int64_t tok0 = tile * 32;
    const int hf = lane >> 4, cl = lane & 15;
    const float rlev = __frcp_rn(levels);
    const T *xb = x + bh * x_stride_bh + tok0 * D + 8 * cl;
    uint8_t *cb = codes + bh * codes_stride_bh + tok0 * RB;

    uint4 raw[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int row = 2 * i + hf;
        raw[i] = (tok0 + row < n_tok) ? __ldg(reinterpret_cast<const uint4 *>(xb + (int64_t)row * D)) : make_uint4(0, 0, 0, 0);
    }

    if constexpr (AXIS == 0) {
        // per-channel extrema over this lane's 16 rows, two channels per register
        uint32_t mnp[4] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w}, mxp[4] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w};
#pragma unroll
        for (int i = 1; i < 16; ++i) {
            const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) { mnp[k] = pmin<T>(mnp[k], w[k]); mxp[k] = pmax<T>(mxp[k], w[k]); }
        }
        float mn[8], sc[8], rc[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t on = __shfl_xor_sync(0xffffffffu, mnp[k], 16), ox = __shfl_xor_sync(0xffffffffu, mxp[k], 16);
            const float2 fn = Pk<T>::widen(pmin<T>(mnp[k], on)), fx = Pk<T>::widen(pmax<T>(mxp[k], ox));
            mn[2 * k] = fn.x; mn[2 * k + 1] = fn.y;
            sc[2 * k] = fmaxf(div_by(__fsub_rn(fx.x, fn.x), levels, rlev), eps);
            sc[2 * k + 1] = fmaxf(div_by(__fsub_rn(fx.y, fn.y), levels, rlev), eps);
            rc[2 * k] = __frcp_rn(sc[2 * k]);
            rc[2 * k + 1] = __frcp_rn(sc[2 * k + 1]);
        }
        if (hf == 0) {
            float4 *ps = reinterpret_cast<float4 *>(scale + bh * param_stride_bh + tile * D + 8 * cl);
            float4 *pz = reinterpret_cast<float4 *>(zero + bh * param_stride_bh + tile * D + 8 * cl);
            ps[0] = make_float4(sc[0], sc[1], sc[2], sc[3]); ps[1] = make_float4(sc[4], sc[5], sc[6], sc[7]);
            pz[0] = make_float4(mn[0], mn[1], mn[2], mn[3]); pz[1] = make_float4(mn[4], mn[5], mn[6], mn[7]);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
            float v[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) { const float2 f = Pk<T>::widen(w[k]); v[2 * k] = f.x; v[2 * k + 1] = f.y; }
            bool odd;
            uint64_t packed = codes8_fast<SB>(v, mn, sc, rc, levels, odd);
            if (odd) packed = codes8_exact<SB>(v, mn, sc, levels);
            store_packed<SB>(cb + (int64_t)(2 * i + hf) * RB, cl, packed);
        }
    }
}

// Values (one scale per token row and 32-channel group): a lane owns whole groups, so the
// extrema need no exchange between lanes and the scale arithmetic is done once per 32
// elements. Lane l takes group l % 4 of rows l / 4 + 8 i (i = 0..3) of the warp's 32-row tile:
// 64 contiguous input bytes, RB / 4 contiguous code bytes, one scale and one zero each.
template <typename T, int SB>
__global__ void __launch_bounds__(128, 4)
kivi_quant_tile_values_kernel(const T *__restrict__ x, int64_t x_stride_bh, int64_t n_tok, int64_t tiles_per_bh,
                              int64_t n_tiles, float levels, float eps, uint8_t *__restrict__ codes,
                              int64_t codes_stride_bh, float *__restrict__ scale, float *__restrict__ zero,
                              int64_t param_stride_bh) {
    constexpr int D = 128, RB = D * SB / 8;
    const int lane = threadIdx.x & 31;
    const int64_t tile_id = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (tile_id >= n_tiles) return;
    const int64_t bh = tile_id / tiles_per_bh, tile = tile_id % tiles_per_bh;
    const int64_t tok0 = tile * 32;
    const int gq = lane & 3, r0 = lane >> 2;
    const float rlev = __frcp_rn(levels);
    const T *xb = x + bh * x_stride_bh + tok0 * D + 32 * gq;
    uint8_t *cb = codes + bh * codes_stride_bh + tok0 * RB + gq * (RB / 4);

    uint4 raw[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = r0 + 8 * i;
        const bool live = tok0 + row < n_tok;
#pragma unroll
        for (int k = 0; k < 4; ++k)
            raw[i][k] = live ? __ldg(reinterpret_cast<const uint4 *>(xb + (int64_t)row * D) + k) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = r0 + 8 * i;
        uint32_t pn = raw[i][0].x, px = raw[i][0].x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t w[4] = {raw[i][k].x, raw[i][k].y, raw[i][k].z, raw[i][k].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) { pn = pmin<T>(pn, w[e]); px = pmax<T>(px, w[e]); }
        }
        const float2 fn = Pk<T>::widen(pn), fx = Pk<T>::widen(px);
        const float mn1 = fminf(fn.x, fn.y), mx1 = fmaxf(fx.x, fx.y);
        const float sc1 = fmaxf(div_by(__fsub_rn(mx1, mn1), levels, rlev), eps);
        const float rc1 = __frcp_rn(sc1);
        if (tok0 + row < n_tok) {
            const int64_t pidx = bh * param_stride_bh + (tok0 + row) * 4 + gq;
            scale[pidx] = sc1;
            zero[pidx] = mn1;
            float mn[8], sc[8], rc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) { mn[j] = mn1; sc[j] = sc1; rc[j] = rc1; }
            uint64_t packed[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t w[4] = {raw[i][k].x, raw[i][k].y, raw[i][k].z, raw[i][k].w};
                float v[8];
#pragma unroll
                for (int e = 0; e < 4; ++e) { const float2 f = Pk<T>::widen(w[e]); v[2 * e] = f.x; v[2 * e + 1] = f.y; }
                bool odd;
                packed[k] = codes8_fast<SB>(v, mn, sc, rc, levels, odd);
                if (odd) packed[k] = codes8_exact<SB>(v, mn, sc, levels);
            }
            uint8_t *dst = cb + (int64_t)row * RB;
            if constexpr (SB == 4) {
                *reinterpret_cast<uint4 *>(dst) = make_uint4((uint32_t)packed[0], (uint32_t)packed[1], (uint32_t)packed[2], (uint32_t)packed[3]);
            } else if constexpr (SB == 2) {
                *reinterpret_cast<uint2 *>(dst) = make_uint2((uint32_t)packed[0] | ((uint32_t)packed[1] << 16),
                                                             (uint32_t)packed[2] | ((uint32_t)packed[3] << 16));
            } else {
                reinterpret_cast<uint4 *>(dst)[0] = make_uint4((uint32_t)packed[0], (uint32_t)(packed[0] >> 32), (uint32_t)packed[1], (uint32_t)(packed[1] >> 32));
                reinterpret_cast<uint4 *>(dst)[1] = make_uint4((uint32_t)packed[2], (uint32_t)(packed[2] >> 32), (uint32_t)packed[3], (uint32_t)(packed[3] >> 32));
            }
        }
    }
}

template <typename T, int SB>
int32_t launch_tile(const vq_kivi_quant_args &a, cudaStream_t st) {
    const int64_t tiles_per_bh = ceil_div(a.n_tok, 32);
    const int64_t n_tiles = a.n_bh * tiles_per_bh;
    const int64_t blocks = ceil_div(n_tiles, 4);
    VQ_REQUIRE(blocks < (1ll << 31), VQ_ERR_SHAPE, "vq_kivi_quantize: tensor too large for one launch");
    if (a.axis == 0)
        kivi_quant_tile_kernel<T, SB, 0><<<(unsigned)blocks, 128, 0, st>>>(
            (const T *)a.x, a.x_stride_bh, a.n_tok, tiles_per_bh, n_tiles, (float)a.levels, a.eps, a.codes,
            a.codes_stride_bh, a.scale, a.zero, a.param_stride_bh);
    else
        kivi_quant_tile_values_kernel<T, SB><<<(unsigned)blocks, 128, 0, st>>>(
            (const T *)a.x, a.x_stride_bh, a.n_tok, tiles_per_bh, n_tiles, (float)a.levels, a.eps, a.codes,
            a.codes_stride_bh, a.scale, a.zero, a.param_stride_bh);
    VQ_CHECK_LAUNCH("kivi_quant_tile_kernel");
    return VQ_OK;
}

template <typename T>
int32_t launch_bits(const vq_kivi_quant_args &a, cudaStream_t st) {
    switch (a.store_bits) {
        case 2: return launch_tile<T, 2>(a, st);
        case 4: return launch_tile<T, 4>(a, st);
        default: return launch_tile<T, 8>(a, st);
    }
}

}  // namespace

bool kivi_quant_tile_supported(const vq_kivi_quant_args &a) {
    if (a.head_dim != 128 || a.group != 32) return false;
    if (a.dtype != VQ_F16 && a.dtype != VQ_BF16) return false;
    if (!a.codes || !a.scale || !a.zero || a.recon) return false;
    if (a.store_bits != 2 && a.store_bits != 4 && a.store_bits != 8) return false;
    if (a.axis == 0 && a.n_tok % 32) return false;
    if (!is_aligned(a.x, 16) || a.x_stride_bh % 8) return false;
    const int rb = 128 * a.store_bits / 8;
    if (!is_aligned(a.codes, 16) || a.codes_stride_bh % 16 || rb % 8) return false;
    if (!is_aligned(a.scale, 16) || !is_aligned(a.zero, 16) || a.param_stride_bh % 4) return false;
    return true;
}

int32_t kivi_quant_tile_launch(const vq_kivi_quant_args &a, cudaStream_t st) {
    return a.dtype == VQ_F16 ? launch_bits<__half>(a, st) : launch_bits<__nv_bfloat16>(a, st);
}

}  // namespace vq
