// SKVQ: clipped group quantization with a per-group clip-factor search, packed, and its inverse
// (reference: veloxquant_mlx/quantizers/skvq.py:103-182; the channel gathers of :98-100 folded in).
//
// One thread owns one (token, channel group): the group's GS values live in registers, so the
// min / max, the five candidate windows and their reconstruction errors need no shuffles. The
// error sums follow a fixed order (eight partial sums over the elements 8 apart, then a tree),
// every product and sum is rounded separately (this file is compiled with -fmad=false; the fused
// operations of the quotient below are explicit), the first minimum wins. HBM traffic is small
// next to the arithmetic: ~13 instructions per element and candidate, so the search runs at the
// instruction rate, the single-candidate form near the copy rate.
#include <type_traits>

#include "common.cuh"

namespace vq {
namespace {

constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23: x + kMagic - kMagic rounds x to the nearest-even integer
constexpr float kEps = 1e-8f;

struct QuantParams {
    const void *x; int64_t x_stride_bh;
    const int32_t *perm;
    uint8_t *codes; float *lo; float *scale; int64_t q_stride_bh;
    float alphas[8]; int n_alphas;
    int n_bh, n_heads, n_tok, D, bits;
};

// clip((v - lo) / scale, 0, levels) + kMagic: the IEEE quotient from rc = RN(1/scale) as t0 = RN(d*rc),
// r = d - scale*t0 (exact in one fma), RN(t0 + r*rc) (Markstein), clamped BEFORE the rounding (the
// bounds are integers, so clamp and round-to-nearest-even commute), then rounded by the magic-number
// add: the sum's low mantissa bits hold the code. For finite input of sane magnitude (range below
// 1e30) the quotient is finite; `exact_div` selects the divide for the rest.
template <bool EXACT_DIV>
__device__ __forceinline__ float code_plus_magic(float v, float lo, float scale, float rc, float levels) {
    const float d = __fsub_rn(v, lo);
    float q;
    if (EXACT_DIV) {
        q = __fdiv_rn(d, scale);
    } else {
        const float t0 = __fmul_rn(d, rc);
        q = __fmaf_rn(__fmaf_rn(-scale, t0, d), rc, t0);
    }
    return __fadd_rn(fminf(fmaxf(q, 0.0f), levels), kMagic);
}

// 1, 2, 4, 8 bits with whole words per group: 32/BITS codes fill a word exactly. The float bits
// (0x4B400000 + code) are shift-added as they are (compile-time shifts); the exponent bits that
// rode along sum to a constant that is taken off once per word (all modulo 2^32).
template <int GS, int BITS, bool EXACT_DIV>
__device__ __forceinline__ void pack_pow2(const float (&v)[GS], float lo, float scale, float rc, float levels, uint32_t *d32) {
    constexpr int PER = 32 / BITS;
    if constexpr (GS % PER == 0) {
        uint32_t ride = 0;
#pragma unroll
        for (int k = 0; k < PER; ++k) ride += 0x4B400000u << (k * BITS);
#pragma unroll
        for (int j0 = 0; j0 < GS; j0 += PER) {
            uint32_t w = 0;
#pragma unroll
            for (int k = 0; k < PER; ++k)
                w += __float_as_uint(code_plus_magic<EXACT_DIV>(v[j0 + k], lo, scale, rc, levels)) << (k * BITS);
            *d32++ = w - ride;
        }
    }
}

// The search and the packing of one group whose values, minimum, maximum and range are known.
template <int GS, bool EXACT_DIV>
__device__ __forceinline__ void quantize_group(const QuantParams &p, const float (&v)[GS], float gmin, float gmax, float rng,
                                               int bh, int tok, int g, int G) {
    const float mid = __fmul_rn(__fadd_rn(gmax, gmin), 0.5f);
    const float levels = (float)((1 << p.bits) - 1);

    float best_err = 0.f, best_lo = 0.f, best_scale = 0.f;
    for (int a = 0; a < p.n_alphas; ++a) {
        const float ar = __fmul_rn(p.alphas[a], rng);
        const float lo = __fsub_rn(mid, __fmul_rn(ar, 0.5f));
        const float scale = fmaxf(__fdiv_rn(ar, levels), kEps);
        if (p.n_alphas == 1) { best_lo = lo; best_scale = scale; break; }
        const float rc = __frcp_rn(scale);
        float r[8];
#pragma unroll
        for (int j = 0; j < GS; ++j) {
            const float c = __fsub_rn(code_plus_magic<EXACT_DIV>(v[j], lo, scale, rc, levels), kMagic);
            const float e = __fsub_rn(__fadd_rn(__fmul_rn(c, scale), lo), v[j]);
            const float sq = __fmul_rn(e, e);
            if (j < 8) r[j] = sq;
            else r[j & 7] = __fadd_rn(r[j & 7], sq);
        }
        const float err = __fadd_rn(__fadd_rn(__fadd_rn(r[0], r[1]), __fadd_rn(r[2], r[3])),
                                    __fadd_rn(__fadd_rn(r[4], r[5]), __fadd_rn(r[6], r[7])));
        if (a == 0 || err < best_err) { best_err = err; best_lo = lo; best_scale = scale; }
    }

    // codes of the chosen window, appended LSB-first; a group is GS*bits/8 whole bytes
    const int64_t qrow = (int64_t)bh * p.q_stride_bh + tok;
    p.lo[qrow * G + g] = best_lo;
    p.scale[qrow * G + g] = best_scale;
    const float rc = __frcp_rn(best_scale);
    const int group_bytes = GS * p.bits / 8;
    uint8_t *dst = p.codes + qrow * ((int64_t)p.D * p.bits / 8) + (int64_t)g * group_bytes;
    uint64_t acc = 0;
    int nb = 0;
    if ((group_bytes & 3) == 0 && (p.bits & (p.bits - 1)) == 0) {
        uint32_t *d32 = reinterpret_cast<uint32_t *>(dst);
        switch (p.bits) {
            case 1: pack_pow2<GS, 1, EXACT_DIV>(v, best_lo, best_scale, rc, levels, d32); break;
            case 2: pack_pow2<GS, 2, EXACT_DIV>(v, best_lo, best_scale, rc, levels, d32); break;
            case 4: pack_pow2<GS, 4, EXACT_DIV>(v, best_lo, best_scale, rc, levels, d32); break;
            default: pack_pow2<GS, 8, EXACT_DIV>(v, best_lo, best_scale, rc, levels, d32); break;
        }
    } else if ((group_bytes & 3) == 0) {
        uint32_t *d32 = reinterpret_cast<uint32_t *>(dst);
#pragma unroll
        for (int j = 0; j < GS; ++j) {
            const float cm = code_plus_magic<EXACT_DIV>(v[j], best_lo, best_scale, rc, levels);
            acc |= (uint64_t)(__float_as_uint(cm) & 0xFFu) << nb;   // (the code: low mantissa bits of code + 1.5 * 2^23)
            nb += p.bits;
            if (nb >= 32) { *d32++ = (uint32_t)acc; acc >>= 32; nb -= 32; }
        }
    } else {
#pragma unroll
        for (int j = 0; j < GS; ++j) {
            const float cm = code_plus_magic<EXACT_DIV>(v[j], best_lo, best_scale, rc, levels);
            acc |= (uint64_t)(__float_as_uint(cm) & 0xFFu) << nb;   // (the code: low mantissa bits of code + 1.5 * 2^23)
            nb += p.bits;
            while (nb >= 8) { *dst++ = (uint8_t)acc; acc >>= 8; nb -= 8; }
        }
    }
}

template <typename T, int GS>
__global__ void __launch_bounds__(128) skvq_quant_kernel(const QuantParams p) {
    const int G = p.D / GS;
    const int64_t n_groups = (int64_t)p.n_bh * p.n_tok * G;
    const int64_t gi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gi >= n_groups) return;
    const int g = (int)(gi % G);
    const int64_t row = gi / G;
    const int tok = (int)(row % p.n_tok);
    const int bh = (int)(row / p.n_tok);
    const T *src = reinterpret_cast<const T *>(p.x) + (int64_t)bh * p.x_stride_bh + (int64_t)tok * p.D;

    float v[GS];
    if (p.perm) {
        const int32_t *pm = p.perm + (int64_t)(bh % p.n_heads) * p.D + g * GS;
#pragma unroll
        for (int j = 0; j < GS; ++j) v[j] = to_f32<T>(src[__ldg(pm + j)]);
    } else {
        // 16-byte vector loads of the group's contiguous channels
        constexpr int PER = 16 / (int)sizeof(T);
        const uint4 *s4 = reinterpret_cast<const uint4 *>(src + g * GS);
#pragma unroll
        for (int j = 0; j < GS / PER; ++j) {
            const uint4 w = __ldg(s4 + j);
            const T *e = reinterpret_cast<const T *>(&w);
#pragma unroll
            for (int i = 0; i < PER; ++i) v[j * PER + i] = to_f32<T>(e[i]);
        }
    }
    float gmin = v[0], gmax = v[0];
#pragma unroll
    for (int j = 1; j < GS; ++j) { gmin = fminf(gmin, v[j]); gmax = fmaxf(gmax, v[j]); }
    const float rng = __fsub_rn(gmax, gmin);
    // (a range of 1e30 or more, or NaN: the quotients may leave the finite range; plain divides)
    if (rng < 1e30f) quantize_group<GS, false>(p, v, gmin, gmax, rng, bh, tok, g, G);
    else quantize_group<GS, true>(p, v, gmin, gmax, rng, bh, tok, g, G);
}

struct DequantParams {
    const uint8_t *codes; const float *lo; const float *scale; int64_t q_stride_bh;
    const int32_t *inv_perm;
    void *out; int64_t out_stride_bh; int out_dtype;
    int n_bh, n_heads, n_tok, D, bits, gs;
};

// General form, one thread per output element: channel c of the output is stored channel
// inv_perm[c] (any D, any group size). The serving shapes take the row kernel below.
__global__ void __launch_bounds__(256) skvq_dequant_kernel(const DequantParams p) {
    const int64_t total = (int64_t)p.n_bh * p.n_tok * p.D;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int c = (int)(i % p.D);
    const int64_t row = i / p.D;
    const int tok = (int)(row % p.n_tok);
    const int bh = (int)(row / p.n_tok);
    const int j = p.inv_perm ? __ldg(p.inv_perm + (int64_t)(bh % p.n_heads) * p.D + c) : c;
    const int64_t qrow = (int64_t)bh * p.q_stride_bh + tok;
    const uint8_t *src = p.codes + qrow * ((int64_t)p.D * p.bits / 8);
    const int bit = j * p.bits;
    uint32_t w = src[bit >> 3];
    if ((bit & 7) + p.bits > 8) w |= (uint32_t)src[(bit >> 3) + 1] << 8;
    const float code = (float)((w >> (bit & 7)) & ((1u << p.bits) - 1u));
    const int G = p.D / p.gs;
    const float val = __fadd_rn(__fmul_rn(code, p.scale[qrow * G + j / p.gs]), p.lo[qrow * G + j / p.gs]);
    store_from_f32(p.out, p.out_dtype, (int64_t)bh * p.out_stride_bh + (int64_t)tok * p.D + c, val);
}

// Row form (D = 32 * CPL, CPL = 2, 4 or 8; packed rows and parameter rows 4-byte aligned): a warp
// owns a token row. Its lanes load the row's packed words (at most 64) and its (lo, scale) pairs
// once, coalesced; every lane then picks the codes of its CPL consecutive OUTPUT channels out of
// the other lanes' registers by shuffle -- which is also the inverse channel gather -- and stores
// them as one vector. Four rows per warp are in flight (eight measured slower: fewer resident warps). blockIdx.y = (batch, head) block, so the
// head's permutation entries are loaded once per thread.
// float(c) for 0 <= c < 2^23 without the conversion unit: c in the mantissa of 2^23, minus 2^23 (exact)
__device__ __forceinline__ float small_uint_as_float(uint32_t c) { return __fsub_rn(__uint_as_float(0x4B000000u | c), 8388608.0f); }

constexpr int kDqWarps = 4, kDqRowsPerWarp = 8;

__device__ __forceinline__ uint32_t bit_field(uint32_t w, int pos, int len) {
    uint32_t r;
    asm("bfe.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(w), "r"(pos), "r"(len));
    return r;
}

template <typename T, int CPL>
__device__ __forceinline__ void store_row_piece(T *dst, const float (&v)[CPL]) {
    if constexpr (sizeof(T) == 4) {
#pragma unroll
        for (int i = 0; i < CPL; i += 4) *reinterpret_cast<float4 *>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
    } else {
        uint32_t pk[CPL / 2];
#pragma unroll
        for (int i = 0; i < CPL / 2; ++i) {
            if constexpr (sizeof(T) == 2 && std::is_same<T, __half>::value) {
                const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
                pk[i] = *reinterpret_cast<const uint32_t *>(&h);
            } else {
                const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                pk[i] = *reinterpret_cast<const uint32_t *>(&h);
            }
        }
        if constexpr (CPL == 2) *reinterpret_cast<uint32_t *>(dst) = pk[0];
        else if constexpr (CPL == 4) *reinterpret_cast<uint2 *>(dst) = make_uint2(pk[0], pk[1]);
        else *reinterpret_cast<uint4 *>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    }
}

// ONE_WORD: no permutation and a lane's CPL codes inside one packed word (1, 2, 4 bits; 8 while
// CPL <= 4): one word shuffle and one (lo, scale) shuffle pair per row. Otherwise every code is
// fetched by its own shuffles (two words where a code may straddle: 3, 5, 6, 7 bits; a second
// register where the row has more than 32 words).
// GATHER (with ONE_WORD): a permutation is undone through shared memory -- the row is decoded in
// stored order, rounded to the output type, parked in the warp's slice, and every lane picks its
// output channels from there (four 2- or 4-byte reads instead of three shuffles per code).
template <typename T, int CPL, bool ONE_WORD, bool GATHER>
__global__ void __launch_bounds__(kDqWarps * 32) skvq_dequant_rows_kernel(const DequantParams p) {
    __shared__ __align__(16) T park[GATHER ? kDqWarps * 32 * CPL : 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int bh = blockIdx.y;
    constexpr int D = 32 * CPL;
    const int G = D / p.gs;
    const int n_words = D * p.bits / 32;   // <= 64
    const bool wide = n_words > 32, straddle = (p.bits & (p.bits - 1)) != 0;
    int bit[CPL], grp[CPL];
#pragma unroll
    for (int i = 0; i < CPL; ++i) {
        const int c = lane * CPL + i;
        const int j = (!ONE_WORD && p.inv_perm) ? __ldg(p.inv_perm + (int64_t)(bh % p.n_heads) * D + c) : c;
        bit[i] = j * p.bits;
        grp[i] = j / p.gs;
    }
    int from[CPL];  // GATHER: stored channel of each of this lane's output channels
#pragma unroll
    for (int i = 0; i < CPL; ++i) from[i] = GATHER ? __ldg(p.inv_perm + (int64_t)(bh % p.n_heads) * D + lane * CPL + i) : 0;
    T *mine = park + (GATHER ? warp * 32 * CPL : 0);
    const int tok0 = (blockIdx.x * kDqWarps + warp) * kDqRowsPerWarp;
    const int64_t q0 = (int64_t)bh * p.q_stride_bh;
    const uint32_t *codes = reinterpret_cast<const uint32_t *>(p.codes) + q0 * n_words + lane;
    const float *lo_p = p.lo + q0 * G + lane, *sc_p = p.scale + q0 * G + lane;
    T *out = reinterpret_cast<T *>(p.out) + (int64_t)bh * p.out_stride_bh + lane * CPL;
    const bool has_w0 = lane < n_words, has_w1 = lane + 32 < n_words, has_g = lane < G;
    constexpr int R = 4;  // rows in flight
    const int t_end = min(tok0 + kDqRowsPerWarp, p.n_tok);
    for (int t0 = tok0; t0 < t_end; t0 += R) {
        uint32_t w0[R], w1[R];
        float lo[R], sc[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int tok = min(t0 + r, p.n_tok - 1);
            w0[r] = has_w0 ? __ldg(codes + tok * n_words) : 0u;
            w1[r] = (!ONE_WORD && has_w1) ? __ldg(codes + tok * n_words + 32) : 0u;
            lo[r] = has_g ? __ldg(lo_p + tok * G) : 0.f;
            sc[r] = has_g ? __ldg(sc_p + tok * G) : 0.f;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            float v[CPL];
            if constexpr (ONE_WORD) {
                const uint32_t w = __shfl_sync(0xffffffffu, w0[r], bit[0] >> 5);
                const float l = __shfl_sync(0xffffffffu, lo[r], grp[0]), sc1 = __shfl_sync(0xffffffffu, sc[r], grp[0]);
#pragma unroll
                for (int i = 0; i < CPL; ++i)
                    v[i] = __fadd_rn(__fmul_rn(small_uint_as_float(bit_field(w, (bit[0] & 31) + i * p.bits, p.bits)), sc1), l);
            } else {
#pragma unroll
                for (int i = 0; i < CPL; ++i) {
                    const int wi = bit[i] >> 5, sh = bit[i] & 31;
                    uint32_t wlo = __shfl_sync(0xffffffffu, w0[r], wi & 31), whi = 0u;
                    if (wide) {
                        const uint32_t a1 = __shfl_sync(0xffffffffu, w1[r], wi & 31);
                        wlo = wi < 32 ? wlo : a1;
                    }
                    if (straddle) {
                        whi = __shfl_sync(0xffffffffu, w0[r], (wi + 1) & 31);
                        if (wide) {
                            const uint32_t b1 = __shfl_sync(0xffffffffu, w1[r], (wi + 1) & 31);
                            whi = wi + 1 < 32 ? whi : b1;
                        }
                    }
                    const uint32_t code = bit_field(__funnelshift_r(wlo, whi, sh), 0, p.bits);
                    const float l = __shfl_sync(0xffffffffu, lo[r], grp[i]), sc1 = __shfl_sync(0xffffffffu, sc[r], grp[i]);
                    v[i] = __fadd_rn(__fmul_rn(small_uint_as_float(code), sc1), l);
                }
            }
            if constexpr (GATHER) {
                __syncwarp();  // the previous row's reads are done
                store_row_piece<T, CPL>(mine + lane * CPL, v);
                __syncwarp();
                __align__(16) T g[CPL];
#pragma unroll
                for (int i = 0; i < CPL; ++i) g[i] = mine[from[i]];
                if (t0 + r < p.n_tok) {
                    T *dst = out + (int64_t)(t0 + r) * D;
                    if constexpr (sizeof(T) * CPL == 4) *reinterpret_cast<uint32_t *>(dst) = *reinterpret_cast<const uint32_t *>(g);
                    else if constexpr (sizeof(T) * CPL == 8) *reinterpret_cast<uint2 *>(dst) = *reinterpret_cast<const uint2 *>(g);
                    else {
#pragma unroll
                        for (int i = 0; i < (int)(sizeof(T) * CPL / 16); ++i)
                            reinterpret_cast<uint4 *>(dst)[i] = reinterpret_cast<const uint4 *>(g)[i];
                    }
                }
            } else {
                if (t0 + r < p.n_tok) store_row_piece<T, CPL>(out + (int64_t)(t0 + r) * D, v);
            }
        }
    }
}

template <typename T, int CPL>
void launch_dequant_rows_cpl(const DequantParams &p, dim3 grid, cudaStream_t st) {
    const bool pow2 = (p.bits & (p.bits - 1)) == 0;
    const bool one_word = pow2 && CPL * p.bits <= 32;
    if (one_word && p.inv_perm == nullptr) skvq_dequant_rows_kernel<T, CPL, true, false><<<grid, kDqWarps * 32, 0, st>>>(p);
    else if (one_word) skvq_dequant_rows_kernel<T, CPL, true, true><<<grid, kDqWarps * 32, 0, st>>>(p);
    else skvq_dequant_rows_kernel<T, CPL, false, false><<<grid, kDqWarps * 32, 0, st>>>(p);
}

template <typename T>
int32_t launch_dequant_rows(const DequantParams &p, cudaStream_t st) {
    dim3 grid((unsigned)ceil_div(p.n_tok, kDqWarps * kDqRowsPerWarp), (unsigned)p.n_bh);
    switch (p.D / 32) {
        case 2: launch_dequant_rows_cpl<T, 2>(p, grid, st); break;
        case 4: launch_dequant_rows_cpl<T, 4>(p, grid, st); break;
        default: launch_dequant_rows_cpl<T, 8>(p, grid, st); break;
    }
    VQ_CHECK_LAUNCH("skvq_dequant_rows_kernel");
    return VQ_OK;
}

template <typename T>
int32_t launch_quant(const QuantParams &p, int gs, cudaStream_t st) {
    const int64_t n_groups = (int64_t)p.n_bh * p.n_tok * (p.D / gs);
    const unsigned blocks = (unsigned)ceil_div(n_groups, 128);
    switch (gs) {
        case 8: skvq_quant_kernel<T, 8><<<blocks, 128, 0, st>>>(p); break;
        case 16: skvq_quant_kernel<T, 16><<<blocks, 128, 0, st>>>(p); break;
        case 32: skvq_quant_kernel<T, 32><<<blocks, 128, 0, st>>>(p); break;
        default: skvq_quant_kernel<T, 64><<<blocks, 128, 0, st>>>(p); break;
    }
    VQ_CHECK_LAUNCH("skvq_quant_kernel");
    return VQ_OK;
}

}  // namespace
}  // namespace vq

extern "C" int32_t vq_skvq_quantize_pack(const vq_skvq_quant_args *args, void *stream) {
    using namespace vq;
    VQ_REQUIRE(args != nullptr, VQ_ERR_SHAPE, "vq_skvq_quantize_pack: args is NULL");
    const vq_skvq_quant_args &a = *args;
    VQ_REQUIRE(a.bits >= 1 && a.bits <= 8, VQ_ERR_SHAPE, "skvq: bits=%d must be in [1, 8] (uint8 codes)", a.bits);
    VQ_REQUIRE(a.group_size == 8 || a.group_size == 16 || a.group_size == 32 || a.group_size == 64, VQ_ERR_SHAPE,
               "skvq: group_size=%d must be 8, 16, 32 or 64 here", a.group_size);
    VQ_REQUIRE(a.D >= a.group_size && a.D % a.group_size == 0 && a.D <= 1024, VQ_ERR_SHAPE,
               "skvq: D=%d must be a multiple of group_size=%d (at most 1024)", a.D, a.group_size);
    VQ_REQUIRE(a.n_alphas >= 1 && a.n_alphas <= 8, VQ_ERR_SHAPE, "skvq: alphas must hold 1 to 8 values");
    for (int i = 0; i < a.n_alphas; ++i)
        VQ_REQUIRE(a.alphas[i] > 0.f && a.alphas[i] <= 1.f, VQ_ERR_SHAPE, "skvq: alpha=%g must be in (0, 1]", (double)a.alphas[i]);
    VQ_REQUIRE(a.n_bh >= 0 && a.n_tok >= 0 && a.n_heads >= 1, VQ_ERR_SHAPE, "skvq: bad sizes");
    if (a.n_bh == 0 || a.n_tok == 0) return VQ_OK;
    VQ_REQUIRE(a.x && a.codes && a.lo && a.scale, VQ_ERR_SHAPE, "skvq: NULL argument");
    VQ_REQUIRE(a.x_dtype == VQ_F16 || a.x_dtype == VQ_BF16 || a.x_dtype == VQ_F32, VQ_ERR_DTYPE, "skvq: unsupported dtype %d", a.x_dtype);
    const size_t es = dtype_size(a.x_dtype);
    VQ_REQUIRE(a.perm || (is_aligned(a.x, 16) && (a.x_stride_bh * es) % 16 == 0 && ((size_t)a.D * es) % 16 == 0 &&
                          ((size_t)a.group_size * es) % 16 == 0),
               VQ_ERR_ALIGN, "skvq: rows must be 16-byte aligned");
    const int group_bytes = a.group_size * a.bits / 8;
    VQ_REQUIRE((group_bytes & 3) != 0 || (is_aligned(a.codes, 4) && ((int64_t)a.D * a.bits / 8) % 4 == 0), VQ_ERR_ALIGN,
               "skvq: packed rows must be 4-byte aligned");
    QuantParams p{};
    p.x = a.x; p.x_stride_bh = a.x_stride_bh; p.perm = a.perm;
    p.codes = a.codes; p.lo = a.lo; p.scale = a.scale; p.q_stride_bh = a.q_stride_bh;
    for (int i = 0; i < a.n_alphas; ++i) p.alphas[i] = a.alphas[i];
    p.n_alphas = a.n_alphas; p.n_bh = a.n_bh; p.n_heads = a.n_heads; p.n_tok = a.n_tok; p.D = a.D; p.bits = a.bits;
    cudaStream_t st = (cudaStream_t)stream;
    if (a.x_dtype == VQ_F16) return launch_quant<__half>(p, a.group_size, st);
    if (a.x_dtype == VQ_BF16) return launch_quant<__nv_bfloat16>(p, a.group_size, st);
    return launch_quant<float>(p, a.group_size, st);
}

extern "C" int32_t vq_skvq_unpack_dequant(const vq_skvq_dequant_args *args, void *stream) {
    using namespace vq;
    VQ_REQUIRE(args != nullptr, VQ_ERR_SHAPE, "vq_skvq_unpack_dequant: args is NULL");
    const vq_skvq_dequant_args &a = *args;
    VQ_REQUIRE(a.bits >= 1 && a.bits <= 8, VQ_ERR_SHAPE, "skvq: bits=%d must be in [1, 8] (uint8 codes)", a.bits);
    VQ_REQUIRE(a.group_size >= 1 && a.D >= 1 && a.D % a.group_size == 0 && ((int64_t)a.D * a.bits) % 8 == 0, VQ_ERR_SHAPE,
               "skvq: D=%d must be a multiple of group_size=%d and D*bits of 8", a.D, a.group_size);
    VQ_REQUIRE(a.n_bh >= 0 && a.n_tok >= 0 && a.n_heads >= 1, VQ_ERR_SHAPE, "skvq: bad sizes");
    if (a.n_bh == 0 || a.n_tok == 0) return VQ_OK;
    VQ_REQUIRE(a.codes && a.lo && a.scale && a.out, VQ_ERR_SHAPE, "skvq: NULL argument");
    VQ_REQUIRE(a.out_dtype == VQ_F16 || a.out_dtype == VQ_BF16 || a.out_dtype == VQ_F32, VQ_ERR_DTYPE, "skvq: unsupported dtype %d", a.out_dtype);
    DequantParams p{};
    p.codes = a.codes; p.lo = a.lo; p.scale = a.scale; p.q_stride_bh = a.q_stride_bh; p.inv_perm = a.inv_perm;
    p.out = a.out; p.out_stride_bh = a.out_stride_bh; p.out_dtype = a.out_dtype;
    p.n_bh = a.n_bh; p.n_heads = a.n_heads; p.n_tok = a.n_tok; p.D = a.D; p.bits = a.bits; p.gs = a.group_size;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t es = dtype_size(a.out_dtype);
    const bool rows_ok = (a.D == 64 || a.D == 128 || a.D == 256) && a.n_bh <= 65535 && ((int64_t)a.D * a.bits / 8) % 4 == 0 &&
                         is_aligned(a.codes, 4) && is_aligned(a.out, 16) && ((size_t)a.out_stride_bh * es) % 16 == 0;
    if (rows_ok) {
        if (a.out_dtype == VQ_F16) return launch_dequant_rows<__half>(p, st);
        if (a.out_dtype == VQ_BF16) return launch_dequant_rows<__nv_bfloat16>(p, st);
        return launch_dequant_rows<float>(p, st);
    }
    const int64_t total = (int64_t)a.n_bh * a.n_tok * a.D;
    skvq_dequant_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, st>>>(p);
    VQ_CHECK_LAUNCH("skvq_dequant_kernel");
    return VQ_OK;
}
