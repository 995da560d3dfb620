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
// Rounding is bit-identical to the reference's float32 divide: the quotient is first
// estimated with a correctly rounded reciprocal; only if the estimate lies within 2e-4 of a
// half-integer (where a 2-ulp estimate error could flip round-half-even) is the IEEE divide
// executed. Compiled with -fmad=false.
#include "common.cuh"
#include "kivi_quant_tile.h"

namespace vq {
namespace {

template <typename T>
__device__ __forceinline__ void unpack8(const uint4 &r, float (&v)[8]);
template <>
__device__ __forceinline__ void unpack8<__half>(const uint4 &r, float (&v)[8]) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        v[2 * i] = f.x;
        v[2 * i + 1] = f.y;
    }
}
template <>
__device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4 &r, float (&v)[8]) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

__device__ __forceinline__ float code_of(float v, float gmin, float scale, float rcp, float levels) {
    const float d = __fsub_rn(v, gmin);
    const float t = __fmul_rn(d, rcp);
    float q = rintf(t);
    if (fabsf(fabsf(__fsub_rn(t, q)) - 0.5f) < 2e-4f) q = rintf(__fdiv_rn(d, scale));  // near a tie: exact divide
    return fminf(fmaxf(q, 0.0f), levels);
}

template <int SB>
__device__ __forceinline__ void store_codes(uint8_t *row, int cl, const float (&q)[8]) {
    if constexpr (SB == 4) {
        uint32_t w = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) w |= ((uint32_t)q[j]) << (4 * j);
        reinterpret_cast<uint32_t *>(row)[cl] = w;
    } else if constexpr (SB == 2) {
        uint32_t w = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) w |= ((uint32_t)q[j]) << (2 * j);
        reinterpret_cast<uint16_t *>(row)[cl] = (uint16_t)w;
    } else {
        uint32_t w0 = 0, w1 = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            w0 |= ((uint32_t)q[j]) << (8 * j);
            w1 |= ((uint32_t)q[4 + j]) << (8 * j);
        }
        reinterpret_cast<uint2 *>(row)[cl] = make_uint2(w0, w1);
    }
}

template <typename T, int SB, int AXIS>
__global__ void __launch_bounds__(128)
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
    const T *xb = x + bh * x_stride_bh + tok0 * D + 8 * cl;
    uint8_t *cb = codes + bh * codes_stride_bh + tok0 * RB;

    uint4 raw[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int row = 2 * i + hf;
        raw[i] = (tok0 + row < n_tok) ? __ldg(reinterpret_cast<const uint4 *>(xb + (int64_t)row * D)) : make_uint4(0, 0, 0, 0);
    }

    if constexpr (AXIS == 0) {
        float mn[8], mx[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { mn[j] = INFINITY; mx[j] = -INFINITY; }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float v[8];
            unpack8<T>(raw[i], v);
#pragma unroll
            for (int j = 0; j < 8; ++j) { mn[j] = fminf(mn[j], v[j]); mx[j] = fmaxf(mx[j], v[j]); }
        }
        float sc[8], rc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            mn[j] = fminf(mn[j], __shfl_xor_sync(0xffffffffu, mn[j], 16));
            mx[j] = fmaxf(mx[j], __shfl_xor_sync(0xffffffffu, mx[j], 16));
            sc[j] = fmaxf(__fdiv_rn(__fsub_rn(mx[j], mn[j]), levels), eps);
            rc[j] = __frcp_rn(sc[j]);
        }
        if (hf == 0) {
            float4 *ps = reinterpret_cast<float4 *>(scale + bh * param_stride_bh + tile * D + 8 * cl);
            float4 *pz = reinterpret_cast<float4 *>(zero + bh * param_stride_bh + tile * D + 8 * cl);
            ps[0] = make_float4(sc[0], sc[1], sc[2], sc[3]); ps[1] = make_float4(sc[4], sc[5], sc[6], sc[7]);
            pz[0] = make_float4(mn[0], mn[1], mn[2], mn[3]); pz[1] = make_float4(mn[4], mn[5], mn[6], mn[7]);
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float v[8], q[8];
            unpack8<T>(raw[i], v);
#pragma unroll
            for (int j = 0; j < 8; ++j) q[j] = code_of(v[j], mn[j], sc[j], rc[j], levels);
            store_codes<SB>(cb + (int64_t)(2 * i + hf) * RB, cl, q);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int row = 2 * i + hf;
            float v[8], q[8];
            unpack8<T>(raw[i], v);
            float mn = v[0], mx = v[0];
#pragma unroll
            for (int j = 1; j < 8; ++j) { mn = fminf(mn, v[j]); mx = fmaxf(mx, v[j]); }
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, 2));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float sc = fmaxf(__fdiv_rn(__fsub_rn(mx, mn), levels), eps);
            const float rc = __frcp_rn(sc);
            if (tok0 + row < n_tok) {
                if ((cl & 3) == 0) {
                    const int64_t pidx = bh * param_stride_bh + (tok0 + row) * 4 + (cl >> 2);
                    scale[pidx] = sc;
                    zero[pidx] = mn;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) q[j] = code_of(v[j], mn, sc, rc, levels);
                store_codes<SB>(cb + (int64_t)row * RB, cl, q);
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
        kivi_quant_tile_kernel<T, SB, 1><<<(unsigned)blocks, 128, 0, st>>>(
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
    if (!is_aligned(a.codes, 8) || a.codes_stride_bh % 8 || rb % 8) return false;
    if (!is_aligned(a.scale, 16) || !is_aligned(a.zero, 16) || a.param_stride_bh % 4) return false;
    return true;
}

int32_t kivi_quant_tile_launch(const vq_kivi_quant_args &a, cudaStream_t st) {
    return a.dtype == VQ_F16 ? launch_bits<__half>(a, st) : launch_bits<__nv_bfloat16>(a, st);
}

}  // namespace vq
