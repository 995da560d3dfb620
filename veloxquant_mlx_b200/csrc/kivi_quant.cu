// KIVI asymmetric group quantization: codes + (scale, zero) and/or the round-tripped tensor.
//
// Two layouts, because keys and values group along opposite axes of a row-major
// [tokens, head_dim] tile:
//   keys   (axis 0): one thread per (slab, token group, channel); a warp covers 32 adjacent
//                    channels, so every load is coalesced although each thread walks its
//                    group with a stride of head_dim. Codes of neighbouring channels are
//                    merged into 32-bit words with a warp OR-reduction before the store.
//   values (axis 1): one thread per (slab, token, run of channel groups that ends on a
//                    byte boundary); the thread owns whole output bytes.
// All arithmetic is float32 with IEEE division and round-half-even; this file is compiled
// with -fmad=false so that q*scale+min is two separately rounded operations.
#include <algorithm>

#include "common.cuh"
#include "kivi_quant_tile.h"

namespace vq {

__device__ __forceinline__ float quant_code(float v, float gmin, float scale, float levels) {
    float q = rintf(__fdiv_rn(__fsub_rn(v, gmin), scale));
    return fminf(fmaxf(q, 0.0f), levels);
}

template <typename T>
__global__ void kivi_quant_channel_kernel(const T *__restrict__ x, int64_t x_stride_bh, int64_t n_tok,
                                          int64_t D, int group, float levels, float eps, int sb,
                                          uint8_t *__restrict__ codes, int64_t codes_stride_bh,
                                          float *__restrict__ scale_out, float *__restrict__ zero_out,
                                          int64_t param_stride_bh, T *__restrict__ recon,
                                          int64_t recon_stride_bh, int word_stores) {
    const int64_t n_groups = (n_tok + group - 1) / group;
    const int64_t bh = blockIdx.x / n_groups;
    const int64_t grp = blockIdx.x % n_groups;
    const int64_t s0 = grp * group;
    const int64_t s1 = min(s0 + (int64_t)group, n_tok);
    const int cpw = 32 / sb;  // codes per 32-bit word
    const int64_t row_bytes = D * sb / 8;
    const T *xb = x + bh * x_stride_bh;
    const int lane = threadIdx.x & 31;

    // Loop bound is padded to a multiple of 32 so that whole warps stay in the shuffles.
    const int64_t d_end = (D + 31) / 32 * 32;
    for (int64_t d = threadIdx.x; d < d_end; d += blockDim.x) {
        const bool live = d < D;
        float gmin = INFINITY, gmax = -INFINITY;
        if (live) {
            for (int64_t s = s0; s < s1; ++s) {
                float v = to_f32<T>(xb[s * D + d]);
                gmin = fminf(gmin, v);
                gmax = fmaxf(gmax, v);
            }
        }
        const float sc = fmaxf(__fdiv_rn(__fsub_rn(gmax, gmin), levels), eps);
        if (live && scale_out) {
            scale_out[bh * param_stride_bh + grp * D + d] = sc;
            zero_out[bh * param_stride_bh + grp * D + d] = gmin;
        }
        for (int64_t s = s0; s < s1; ++s) {
            float q = 0.0f;
            if (live) {
                float v = to_f32<T>(xb[s * D + d]);
                q = quant_code(v, gmin, sc, levels);
                if (recon) {
                    float prod = __fmul_rn(q, sc);
                    recon[bh * recon_stride_bh + s * D + d] = from_f32<T>(__fadd_rn(prod, gmin));
                }
            }
            if (codes) {
                uint32_t w = ((uint32_t)q) << ((lane % cpw) * sb);
                for (int o = 1; o < cpw; o <<= 1) w |= __shfl_xor_sync(0xffffffffu, w, o);
                if (live && (lane % cpw) == 0) {
                    uint8_t *row = codes + bh * codes_stride_bh + s * row_bytes;
                    const int64_t byte0 = (d / cpw) * 4;
                    if (word_stores) {
                        *reinterpret_cast<uint32_t *>(row + byte0) = w;
                    } else {
                        for (int k = 0; k < 4 && byte0 + k < row_bytes; ++k) row[byte0 + k] = (uint8_t)(w >> (8 * k));
                    }
                }
            }
        }
    }
}

template <typename T>
__global__ void kivi_quant_token_kernel(const T *__restrict__ x, int64_t x_stride_bh, int64_t n_bh,
                                        int64_t n_tok, int64_t D, int group, int groups_per_thread,
                                        float levels, float eps, int sb, uint8_t *__restrict__ codes,
                                        int64_t codes_stride_bh, float *__restrict__ scale_out,
                                        float *__restrict__ zero_out, int64_t param_stride_bh,
                                        T *__restrict__ recon, int64_t recon_stride_bh) {
    const int64_t n_groups = (D + group - 1) / group;
    const int64_t runs = (n_groups + groups_per_thread - 1) / groups_per_thread;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (tid >= n_bh * n_tok * runs) return;
    const int64_t run = tid % runs;
    const int64_t tok = (tid / runs) % n_tok;
    const int64_t bh = tid / (runs * n_tok);
    const T *row = x + bh * x_stride_bh + tok * D;
    const int64_t row_bytes = D * sb / 8;
    uint8_t *crow = codes ? codes + bh * codes_stride_bh + tok * row_bytes : nullptr;

    uint32_t acc = 0;  // bits waiting to be flushed as whole bytes
    int nbits = 0;
    int64_t byte_pos = (run * groups_per_thread * (int64_t)group * sb) / 8;
    const int64_t g_begin = run * groups_per_thread;
    const int64_t g_end = min(g_begin + (int64_t)groups_per_thread, n_groups);
    for (int64_t gi = g_begin; gi < g_end; ++gi) {
        const int64_t d0 = gi * group;
        const int64_t d1 = min(d0 + (int64_t)group, D);
        float gmin = INFINITY, gmax = -INFINITY;
        for (int64_t d = d0; d < d1; ++d) {
            float v = to_f32<T>(row[d]);
            gmin = fminf(gmin, v);
            gmax = fmaxf(gmax, v);
        }
        const float sc = fmaxf(__fdiv_rn(__fsub_rn(gmax, gmin), levels), eps);
        if (scale_out) {
            scale_out[bh * param_stride_bh + tok * n_groups + gi] = sc;
            zero_out[bh * param_stride_bh + tok * n_groups + gi] = gmin;
        }
        for (int64_t d = d0; d < d1; ++d) {
            float q = quant_code(to_f32<T>(row[d]), gmin, sc, levels);
            if (recon) {
                float prod = __fmul_rn(q, sc);
                recon[bh * recon_stride_bh + tok * D + d] = from_f32<T>(__fadd_rn(prod, gmin));
            }
            if (crow) {
                acc |= ((uint32_t)q) << nbits;
                nbits += sb;
                if (nbits >= 8) {
                    crow[byte_pos++] = (uint8_t)acc;
                    acc >>= 8;
                    nbits -= 8;
                }
            }
        }
    }
    if (crow && nbits > 0 && byte_pos < row_bytes) crow[byte_pos] = (uint8_t)acc;
}

template <typename T>
__global__ void kivi_dequant_kernel(const uint8_t *__restrict__ codes, int64_t codes_stride_bh,
                                    const float *__restrict__ scale, const float *__restrict__ zero,
                                    int64_t param_stride_bh, int axis, int sb, int group, int64_t n_bh,
                                    int64_t n_tok, int64_t D, T *__restrict__ out, int64_t out_stride_bh) {
    const int64_t total = n_bh * n_tok * D;
    const int64_t row_bytes = D * sb / 8;
    const int64_t n_vgroups = (D + group - 1) / group;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t d = i % D;
        const int64_t tok = (i / D) % n_tok;
        const int64_t bh = i / (D * n_tok);
        const uint32_t c = load_code(codes + bh * codes_stride_bh + tok * row_bytes, (int)d, sb);
        const int64_t p = (axis == 0) ? bh * param_stride_bh + (tok / group) * D + d
                                      : bh * param_stride_bh + tok * n_vgroups + d / group;
        const float prod = __fmul_rn((float)c, scale[p]);
        out[bh * out_stride_bh + tok * D + d] = from_f32<T>(__fadd_rn(prod, zero[p]));
    }
}

static int gcd_int(int a, int b) { return b == 0 ? a : gcd_int(b, a % b); }

template <typename T>
static int32_t launch_quant(const vq_kivi_quant_args &a, cudaStream_t st) {
    const float levels = (float)a.levels;
    const int sb = a.store_bits;
    if (a.axis == 0) {
        const int64_t n_groups = ceil_div(a.n_tok, a.group);
        const int64_t blocks = a.n_bh * n_groups;
        VQ_REQUIRE(blocks < (1ll << 31), VQ_ERR_SHAPE, "vq_kivi_quantize: too many (slab, group) tiles");
        const int64_t row_bytes = a.head_dim * sb / 8;
        const int word_stores = a.codes && is_aligned(a.codes, 4) && row_bytes % 4 == 0 &&
                                a.codes_stride_bh % 4 == 0;
        int threads = (int)std::min<int64_t>(256, ceil_div(a.head_dim, 32) * 32);
        kivi_quant_channel_kernel<T><<<(unsigned)blocks, threads, 0, st>>>(
            (const T *)a.x, a.x_stride_bh, a.n_tok, a.head_dim, a.group, levels, a.eps, sb, a.codes,
            a.codes_stride_bh, a.scale, a.zero, a.param_stride_bh, (T *)a.recon, a.recon_stride_bh,
            word_stores);
        VQ_CHECK_LAUNCH("kivi_quant_channel_kernel");
    } else {
        const int gbits = (int)(((int64_t)a.group * sb) % 8);
        const int gpt = 8 / gcd_int(8, gbits == 0 ? 8 : gbits);
        const int64_t n_groups = ceil_div(a.head_dim, a.group);
        const int64_t runs = ceil_div(n_groups, gpt);
        const int64_t total = a.n_bh * a.n_tok * runs;
        const int threads = 128;
        const int64_t blocks = ceil_div(total, threads);
        VQ_REQUIRE(blocks < (1ll << 31), VQ_ERR_SHAPE, "vq_kivi_quantize: tensor too large for one launch");
        kivi_quant_token_kernel<T><<<(unsigned)blocks, threads, 0, st>>>(
            (const T *)a.x, a.x_stride_bh, a.n_bh, a.n_tok, a.head_dim, a.group, gpt, levels, a.eps, sb,
            a.codes, a.codes_stride_bh, a.scale, a.zero, a.param_stride_bh, (T *)a.recon,
            a.recon_stride_bh);
        VQ_CHECK_LAUNCH("kivi_quant_token_kernel");
    }
    return VQ_OK;
}

}  // namespace vq

extern "C" int32_t vq_kivi_quantize(const vq_kivi_quant_args *args, void *stream) {
    using namespace vq;
    VQ_REQUIRE(args != nullptr, VQ_ERR_SHAPE, "vq_kivi_quantize: args is NULL");
    const vq_kivi_quant_args &a = *args;
    VQ_REQUIRE(a.axis == 0 || a.axis == 1, VQ_ERR_SHAPE, "vq_kivi_quantize: axis must be 0 or 1, got %d", a.axis);
    VQ_REQUIRE(a.group >= 1, VQ_ERR_SHAPE, "vq_kivi_quantize: group must be >= 1, got %d", a.group);
    VQ_REQUIRE(a.levels >= 1 && a.levels <= 255, VQ_ERR_SHAPE, "vq_kivi_quantize: levels must be in 1..255, got %d", a.levels);
    VQ_REQUIRE(a.n_bh >= 0 && a.n_tok >= 0 && a.head_dim >= 1, VQ_ERR_SHAPE, "vq_kivi_quantize: negative size");
    VQ_REQUIRE((a.scale == nullptr) == (a.zero == nullptr), VQ_ERR_SHAPE, "vq_kivi_quantize: scale and zero must both be given or both NULL");
    if (a.codes) {
        const int sb = a.store_bits;
        VQ_REQUIRE(sb == 1 || sb == 2 || sb == 4 || sb == 8, VQ_ERR_SHAPE, "vq_kivi_quantize: store_bits must be 1, 2, 4 or 8, got %d", sb);
        VQ_REQUIRE(a.levels < (1 << sb), VQ_ERR_SHAPE, "vq_kivi_quantize: levels=%d does not fit %d-bit containers", a.levels, sb);
        VQ_REQUIRE((a.head_dim * sb) % 8 == 0, VQ_ERR_SHAPE, "vq_kivi_quantize: head_dim*store_bits must be a multiple of 8");
    }
    if (a.n_bh == 0 || a.n_tok == 0) return VQ_OK;
    VQ_REQUIRE(a.x != nullptr, VQ_ERR_SHAPE, "vq_kivi_quantize: x is NULL");
    cudaStream_t st = (cudaStream_t)stream;
    if (kivi_quant_tile_supported(a)) return kivi_quant_tile_launch(a, st);
    switch (a.dtype) {
        case VQ_F16: return launch_quant<__half>(a, st);
        case VQ_BF16: return launch_quant<__nv_bfloat16>(a, st);
        case VQ_F32: return launch_quant<float>(a, st);
        default: return fail(VQ_ERR_DTYPE, "vq_kivi_quantize: unknown dtype %d", a.dtype);
    }
}

extern "C" int32_t vq_kivi_dequant(const vq_kivi_dequant_args *args, void *stream) {
    using namespace vq;
    VQ_REQUIRE(args != nullptr, VQ_ERR_SHAPE, "vq_kivi_dequant: args is NULL");
    const vq_kivi_dequant_args &a = *args;
    const int sb = a.store_bits;
    VQ_REQUIRE(a.axis == 0 || a.axis == 1, VQ_ERR_SHAPE, "vq_kivi_dequant: axis must be 0 or 1");
    VQ_REQUIRE(sb == 1 || sb == 2 || sb == 4 || sb == 8, VQ_ERR_SHAPE, "vq_kivi_dequant: store_bits must be 1, 2, 4 or 8");
    VQ_REQUIRE(a.group >= 1 && a.head_dim >= 1 && (a.head_dim * sb) % 8 == 0, VQ_ERR_SHAPE, "vq_kivi_dequant: bad group/head_dim");
    const int64_t total = a.n_bh * a.n_tok * a.head_dim;
    if (total == 0) return VQ_OK;
    const int threads = 256;
    const unsigned blocks = (unsigned)std::min<int64_t>(ceil_div(total, threads), 148 * 32);
    cudaStream_t st = (cudaStream_t)stream;
#define VQ_DEQ(T)                                                                                   \
    kivi_dequant_kernel<T><<<blocks, threads, 0, st>>>(a.codes, a.codes_stride_bh, a.scale, a.zero, \
                                                       a.param_stride_bh, a.axis, sb, a.group,      \
                                                       a.n_bh, a.n_tok, a.head_dim, (T *)a.out,     \
                                                       a.out_stride_bh)
    switch (a.out_dtype) {
        case VQ_F16: VQ_DEQ(__half); break;
        case VQ_BF16: VQ_DEQ(__nv_bfloat16); break;
        case VQ_F32: VQ_DEQ(float); break;
        default: return fail(VQ_ERR_DTYPE, "vq_kivi_dequant: unknown dtype %d", a.out_dtype);
    }
#undef VQ_DEQ
    VQ_CHECK_LAUNCH("kivi_dequant_kernel");
    return VQ_OK;
}

extern "C" int32_t vq_kivi_quantize_pack(const vq_kivi_quant_args *args, void *stream) {
    using namespace vq;
    VQ_REQUIRE(args != nullptr, VQ_ERR_SHAPE, "vq_kivi_quantize_pack: args is NULL");
    VQ_REQUIRE(args->codes && args->scale && args->zero, VQ_ERR_SHAPE, "vq_kivi_quantize_pack: codes, scale and zero are required");
    vq_kivi_quant_args a = *args;
    a.recon = nullptr;
    return vq_kivi_quantize(&a, stream);
}

namespace vq {
// One thread per 16-byte chunk of a new row, keys and values alike.
__global__ void __launch_bounds__(256)
kivi_append_kernel(const uint4 *__restrict__ k_new, const uint4 *__restrict__ v_new, int64_t new_stride_bh,
                   uint4 *__restrict__ k_res, uint4 *__restrict__ v_res, int64_t res_stride_bh, int64_t n_bh,
                   int64_t n_new, int64_t tok_offset, int row_chunks) {
    // Launched as a programmatic dependent (flags & VQ_ATTEND_OVERLAP_PREVIOUS) this grid may
    // start while the work before it still runs. What follows it may start as well (the
    // trigger), e.g. the attention over the same cache, which reads these rows only after its
    // own wait. The rows are loaded at once and written after the wait, i.e. after everything
    // before this grid has finished. (Both instructions do nothing after a plain launch.)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int64_t per_slab = n_new * row_chunks;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = i < n_bh * per_slab;
    const int64_t s = live ? i / per_slab : 0, off = live ? i % per_slab : 0;  // strides are in 16-byte chunks here
    const int64_t src = s * new_stride_bh + off, dst = s * res_stride_bh + tok_offset * row_chunks + off;
    uint4 kv = make_uint4(0, 0, 0, 0), vv = kv;
    if (live) { kv = k_new[src]; vv = v_new[src]; }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (live) {
        k_res[dst] = kv;
        v_res[dst] = vv;
    }
}
}  // namespace vq

extern "C" int32_t vq_kivi_append(const void *k_new, const void *v_new, int64_t new_stride_bh, void *k_res, void *v_res,
                                  int64_t res_stride_bh, int64_t n_bh, int64_t n_new, int64_t tok_offset,
                                  int32_t head_dim, int32_t dtype, int32_t flags, void *stream) {
    using namespace vq;
    VQ_REQUIRE(k_new && v_new && k_res && v_res, VQ_ERR_SHAPE, "vq_kivi_append: a buffer is NULL");
    VQ_REQUIRE(dtype == VQ_F16 || dtype == VQ_BF16 || dtype == VQ_F32, VQ_ERR_DTYPE, "vq_kivi_append: bad dtype %d", dtype);
    VQ_REQUIRE(n_bh >= 0 && n_new >= 0 && tok_offset >= 0 && head_dim >= 1, VQ_ERR_SHAPE, "vq_kivi_append: negative size");
    const int64_t es = dtype == VQ_F32 ? 4 : 2;
    VQ_REQUIRE((head_dim * es) % 16 == 0 && (new_stride_bh * es) % 16 == 0 && (res_stride_bh * es) % 16 == 0 &&
                   is_aligned(k_new, 16) && is_aligned(v_new, 16) && is_aligned(k_res, 16) && is_aligned(v_res, 16),
               VQ_ERR_ALIGN, "vq_kivi_append: rows, strides and pointers must be multiples of 16 bytes");
    const int row_chunks = (int)(head_dim * es / 16);
    const int64_t total = n_bh * n_new * row_chunks;
    if (total == 0) return VQ_OK;
    VQ_REQUIRE(ceil_div(total, 256) < (1ll << 31), VQ_ERR_SHAPE, "vq_kivi_append: block too large for one launch");
    VQ_REQUIRE((flags & ~VQ_ATTEND_OVERLAP_PREVIOUS) == 0, VQ_ERR_SHAPE, "vq_kivi_append: unknown bits in flags (%d)", flags);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ceil_div(total, 256));
    cfg.blockDim = dim3(256);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (flags & VQ_ATTEND_OVERLAP_PREVIOUS) ? 1 : 0;
    VQ_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kivi_append_kernel, (const uint4 *)k_new, (const uint4 *)v_new, new_stride_bh * es / 16,
                                     (uint4 *)k_res, (uint4 *)v_res, res_stride_bh * es / 16, n_bh, n_new, tok_offset, row_chunks));
    return VQ_OK;
}

extern "C" int32_t vq_kivi_quant_dequant(const vq_kivi_quant_args *args, void *stream) {
    using namespace vq;
    VQ_REQUIRE(args != nullptr, VQ_ERR_SHAPE, "vq_kivi_quant_dequant: args is NULL");
    VQ_REQUIRE(args->recon != nullptr, VQ_ERR_SHAPE, "vq_kivi_quant_dequant: recon is required");
    return vq_kivi_quantize(args, stream);
}
