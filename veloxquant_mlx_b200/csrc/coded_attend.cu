// Decode attention over keys that are scored without being reconstructed:
//   VecInfer : score = scale * sum_s lut[s][idx[t][s]],  lut[s][c] = q_sub[s] . codebook[c]
//   RaBitQ   : score = (D - 2*popcount(sign(q) ^ bits[t])) * q_scale * k_mag[t] + k_const[t]
// Both read a few bytes per key (16 B at D=128) so the value stream dominates the traffic.
//
// One CTA per (context split, kv head x query row, batch); one warp per query head of the
// kv head (GQA heads share the CTA so the value rows they all read hit L1). Within a warp a
// lane owns one key of a 32-key tile for scoring, then owns D/32 output channels for the
// value accumulation (the tile's weights are broadcast with shuffles). Online softmax per
// warp; context splits are merged by the shared split-merge kernel.
#include <algorithm>

#include "common.cuh"
#include "kivi_attend.h"

namespace vq {

namespace {

constexpr int kMaxWarps = 16;
constexpr int kMaxDpl = 8;  // D <= 256

enum { KEY_VQ = 0, KEY_RABITQ = 1 };
enum { V_DENSE = 0, V_VQ = 1, V_CENT_BYTE = 2, V_CENT_NIBBLE = 3 };

struct CodedParams {
    const void *q; void *out; int q_dtype, out_dtype;
    int B, H_q, H_kv, S_q, S_kv, D;
    int64_t stride_tok;
    float scale; int causal, window;
    int key_mode;
    const void *k_codes; int k_index_bytes; const float *k_codebook; int k_nc, k_sub, k_stacked;
    const float *q_scale, *k_mag, *k_const;
    int v_mode; const void *v; int v_dtype, v_index_bytes; const float *v_codebook; int v_nc, v_sub;
    int n_splits, heads_per_cta, n_head_chunks;
    float *part_o, *part_ml;
};

__device__ __forceinline__ uint32_t load_index(const void *p, int bytes, int64_t i) {
    if (bytes == 1) return reinterpret_cast<const uint8_t *>(p)[i];
    if (bytes == 2) return reinterpret_cast<const uint16_t *>(p)[i];
    return reinterpret_cast<const uint32_t *>(p)[i];
}

__global__ void __launch_bounds__(kMaxWarps * 32)
coded_attend_kernel(const CodedParams p) {
    extern __shared__ float sh_lut[];  // VQ: [warps][n_sub * n_c]; RaBitQ: unused
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int split = blockIdx.x;
    int y = blockIdx.y;
    const int hc = y % p.n_head_chunks; y /= p.n_head_chunks;
    const int sq = y % p.S_q;
    const int hkv = y / p.S_q;
    const int b = blockIdx.z;
    const int hpk = p.H_q / p.H_kv;
    const int hp = hc * p.heads_per_cta + warp;  // head within the kv group
    const bool head_live = hp < hpk;
    const int hq = hkv * hpk + (head_live ? hp : 0);
    const int D = p.D, dpl = D / 32;
    const int64_t bh = (int64_t)b * p.H_kv + hkv;
    const int64_t qrow = ((int64_t)b * p.H_q + hq) * p.S_q + sq;

    // ---- per-warp query state -----------------------------------------------------------
    const int n_sub = p.key_mode == KEY_VQ ? D / p.k_sub : 0;
    float *lut = sh_lut + (size_t)warp * n_sub * p.k_nc;
    uint32_t qbits[8];  // RaBitQ: sign bits of q, 32 per word
    float qs = 0.f;
    if (p.key_mode == KEY_VQ) {
        if (head_live) {
            for (int i = lane; i < n_sub * p.k_nc; i += 32) {
                const int s = i / p.k_nc, c = i % p.k_nc;
                const float *cb = p.k_codebook + ((int64_t)(p.k_stacked ? s : 0) * p.k_nc + c) * p.k_sub;
                float dot = 0.f;
                for (int e = 0; e < p.k_sub; ++e) dot += load_as_f32(p.q, p.q_dtype, qrow * D + s * p.k_sub + e) * cb[e];
                lut[i] = dot;
            }
        }
        __syncwarp();
    } else {
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            float v = (32 * w + lane < D) ? load_as_f32(p.q, p.q_dtype, qrow * D + 32 * w + lane) : -1.f;
            qbits[w] = __ballot_sync(0xffffffffu, v >= 0.f);
        }
        qs = p.q_scale[qrow];
    }

    const int chunk = (p.S_kv + p.n_splits - 1) / p.n_splits;
    const int t_begin = split * chunk;
    const int t_end = min(p.S_kv, t_begin + chunk);
    const int q_abs = p.S_kv - p.S_q + sq;

    float m_run = -INFINITY, l_run = 0.f, acc[kMaxDpl];
#pragma unroll
    for (int i = 0; i < kMaxDpl; ++i) acc[i] = 0.f;

    if (head_live) {
        for (int tile = t_begin; tile < t_end; tile += 32) {
            const int t = tile + lane;
            bool valid = t < t_end;
            if (valid && p.causal && t > q_abs) valid = false;
            if (valid && p.window > 0 && q_abs + 1 > p.window && t + p.window < q_abs + 1) valid = false;
            float score = -INFINITY;
            if (valid) {
                const int64_t tok = bh * p.stride_tok + t;
                if (p.key_mode == KEY_VQ) {
                    float s = 0.f;
                    for (int sub = 0; sub < n_sub; ++sub) {
                        uint32_t c = load_index(p.k_codes, p.k_index_bytes, tok * n_sub + sub);
                        c = min(c, (uint32_t)(p.k_nc - 1));
                        s += lut[sub * p.k_nc + c];
                    }
                    score = s * p.scale;
                } else {
                    const uint32_t *kb = reinterpret_cast<const uint32_t *>(
                        reinterpret_cast<const uint8_t *>(p.k_codes) + tok * (D / 8));
                    int ham = 0;
                    if ((D & 31) == 0) {
#pragma unroll
                        for (int w = 0; w < 8; ++w)
                            if (32 * w < D) ham += __popc(qbits[w] ^ kb[w]);
                    } else {
                        const uint8_t *kbb = reinterpret_cast<const uint8_t *>(kb);
                        for (int j = 0; j < D / 8; ++j)
                            ham += __popc(((qbits[j >> 2] >> (8 * (j & 3))) & 0xffu) ^ (uint32_t)kbb[j]);
                    }
                    score = ((float)D - 2.0f * (float)ham) * qs * p.k_mag[tok] + (p.k_const ? p.k_const[tok] : 0.f);
                }
            }
            const float tile_max = warp_max(score);
            if (tile_max == -INFINITY) continue;  // whole tile masked
            const float m_new = fmaxf(m_run, tile_max);
            const float factor = (m_run == -INFINITY) ? 0.f : __expf(m_run - m_new);
            m_run = m_new;
            const float w = valid ? __expf(score - m_new) : 0.f;
            l_run = l_run * factor + warp_sum(w);
#pragma unroll
            for (int i = 0; i < kMaxDpl; ++i) acc[i] *= factor;
            const int n_in_tile = min(32, t_end - tile);
            for (int l = 0; l < n_in_tile; ++l) {
                const float wl = __shfl_sync(0xffffffffu, w, l);
                if (wl == 0.f) continue;
                const int64_t tok = bh * p.stride_tok + tile + l;
#pragma unroll
                for (int i = 0; i < kMaxDpl; ++i) {
                    if (i < dpl) {
                        const int dim = lane * dpl + i;
                        float vv;
                        if (p.v_mode == V_DENSE) {
                            vv = load_as_f32(p.v, p.v_dtype, tok * D + dim);
                        } else if (p.v_mode == V_VQ) {
                            const int nsv = D / p.v_sub;
                            uint32_t c = load_index(p.v, p.v_index_bytes, tok * nsv + dim / p.v_sub);
                            c = min(c, (uint32_t)(p.v_nc - 1));
                            vv = p.v_codebook[(int64_t)c * p.v_sub + dim % p.v_sub];
                        } else if (p.v_mode == V_CENT_BYTE) {
                            vv = p.v_codebook[reinterpret_cast<const uint8_t *>(p.v)[tok * D + dim] & 0xF];
                        } else {
                            const uint32_t byte = reinterpret_cast<const uint8_t *>(p.v)[tok * (D / 2) + (dim >> 1)];
                            vv = p.v_codebook[(dim & 1) ? (byte >> 4) : (byte & 0xFu)];
                        }
                        acc[i] = fmaf(wl, vv, acc[i]);
                    }
                }
            }
        }
        if (p.n_splits == 1) {
            const float inv = 1.0f / fmaxf(l_run, 1e-20f);
#pragma unroll
            for (int i = 0; i < kMaxDpl; ++i)
                if (i < dpl) store_from_f32(p.out, p.out_dtype, qrow * D + lane * dpl + i, acc[i] * inv);
        } else {
#pragma unroll
            for (int i = 0; i < kMaxDpl; ++i)
                if (i < dpl) p.part_o[(qrow * p.n_splits + split) * D + lane * dpl + i] = acc[i];
            if (lane == 0) {
                p.part_ml[(qrow * p.n_splits + split) * 2] = m_run;
                p.part_ml[(qrow * p.n_splits + split) * 2 + 1] = l_run;
            }
        }
    }
}

int pick_splits(int requested, int S_kv, int64_t ctas, int sm_count) {
    if (requested > 0) return std::min(requested, 256);
    int64_t want = ceil_div((int64_t)sm_count * 4, std::max<int64_t>(ctas, 1));
    want = std::min<int64_t>(want, ceil_div(S_kv, 256));
    return (int)std::max<int64_t>(1, std::min<int64_t>(want, 256));
}

int32_t launch_coded(CodedParams &p, void *workspace, int64_t workspace_bytes, int requested_splits,
                     const char *who, cudaStream_t st) {
    DeviceInfo di;
    int32_t rc = device_info(&di);
    if (rc != VQ_OK) return rc;
    VQ_REQUIRE(p.B >= 1 && p.H_q >= 1 && p.H_kv >= 1 && p.S_q >= 1 && p.S_kv >= 1, VQ_ERR_SHAPE, "%s: sizes must be >= 1", who);
    VQ_REQUIRE(p.H_q % p.H_kv == 0, VQ_ERR_SHAPE, "%s: H_q=%d must be a multiple of H_kv=%d.", who, p.H_q, p.H_kv);
    VQ_REQUIRE(p.D % 32 == 0 && p.D <= 256, VQ_ERR_SHAPE, "%s: D=%d must be a multiple of 32 and <= 256", who, p.D);
    const int hpk = p.H_q / p.H_kv;
    size_t lut_bytes = 0;
    if (p.key_mode == KEY_VQ) lut_bytes = (size_t)(p.D / p.k_sub) * p.k_nc * sizeof(float);
    int heads_per_cta = std::min(hpk, kMaxWarps);
    if (lut_bytes) heads_per_cta = (int)std::max<size_t>(1, std::min<size_t>(heads_per_cta, (160 * 1024) / lut_bytes));
    VQ_REQUIRE(lut_bytes <= 200 * 1024, VQ_ERR_CAPACITY, "%s: lookup table of %zu bytes does not fit shared memory", who, lut_bytes);
    p.heads_per_cta = heads_per_cta;
    p.n_head_chunks = (int)ceil_div(hpk, heads_per_cta);
    const int64_t gy = (int64_t)p.H_kv * p.S_q * p.n_head_chunks;
    VQ_REQUIRE(gy <= 65535 && p.B <= 65535, VQ_ERR_SHAPE, "%s: grid too large", who);
    p.n_splits = pick_splits(requested_splits, p.S_kv, gy * p.B, di.sm_count);
    const int64_t rows = (int64_t)p.B * p.H_q * p.S_q;
    if (p.n_splits > 1) {
        const int64_t need = rows * p.n_splits * ((int64_t)p.D + 2) * (int64_t)sizeof(float);
        VQ_REQUIRE(workspace != nullptr && workspace_bytes >= need, VQ_ERR_CAPACITY,
                   "%s: workspace of %lld bytes needed, %lld given", who, (long long)need, (long long)workspace_bytes);
        p.part_o = (float *)workspace;
        p.part_ml = p.part_o + rows * p.n_splits * p.D;
    }
    const size_t smem = lut_bytes * heads_per_cta;
    if (smem > 48 * 1024)
        VQ_CHECK_CUDA(cudaFuncSetAttribute(coded_attend_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid(p.n_splits, (unsigned)gy, p.B);
    coded_attend_kernel<<<grid, heads_per_cta * 32, smem, st>>>(p);
    VQ_CHECK_LAUNCH("coded_attend_kernel");
    if (p.n_splits > 1) return launch_split_merge(p.part_o, p.part_ml, p.n_splits, p.D, p.out, p.out_dtype, rows, st);
    return VQ_OK;
}

int64_t coded_workspace(int B, int H_q, int S_q, int D, int n_splits) {
    if (B < 1 || H_q < 1 || S_q < 1 || D < 1) return 0;
    const int64_t splits = n_splits > 0 ? std::min(n_splits, 256) : 256;
    return (int64_t)B * H_q * S_q * splits * ((int64_t)D + 2) * (int64_t)sizeof(float) + 256;
}

}  // namespace
}  // namespace vq

extern "C" int64_t vq_vq_attend_workspace_bytes(const vq_vq_attend_args *a) {
    return a ? vq::coded_workspace(a->B, a->H_q, a->S_q, a->D, a->n_splits) : 0;
}

extern "C" int32_t vq_vq_decode_attend(const vq_vq_attend_args *args, void *stream) {
    using namespace vq;
    VQ_REQUIRE(args != nullptr, VQ_ERR_SHAPE, "vq_vq_decode_attend: args is NULL");
    const vq_vq_attend_args &a = *args;
    VQ_REQUIRE(a.k_sub_dim >= 1 && a.D % a.k_sub_dim == 0, VQ_ERR_SHAPE, "fused_sdpa: D=%d must equal n_sub*sub_dim (sub_dim=%d).", a.D, a.k_sub_dim);
    VQ_REQUIRE(a.k_n_centroids >= 1, VQ_ERR_SHAPE, "fused_sdpa: bad centroid count");
    VQ_REQUIRE(a.v_mode == 0 || a.v_mode == 1, VQ_ERR_SHAPE, "fused_sdpa: v_mode must be 0 or 1");
    if (a.v_mode == 1)
        VQ_REQUIRE(a.v_sub_dim >= 1 && a.D % a.v_sub_dim == 0 && a.v_n_centroids >= 1 && a.v_codebook, VQ_ERR_SHAPE,
                   "fused_sdpa: D=%d must equal n_sub_v*sub_dim_v (sub_dim_v=%d).", a.D, a.v_sub_dim);
    VQ_REQUIRE(a.q && a.out && a.k_indices && a.k_codebook && a.v, VQ_ERR_SHAPE, "fused_sdpa: NULL argument");
    CodedParams p{};
    p.q = a.q; p.out = a.out; p.q_dtype = a.q_dtype; p.out_dtype = a.out_dtype;
    p.B = a.B; p.H_q = a.H_q; p.H_kv = a.H_kv; p.S_q = a.S_q; p.S_kv = a.S_kv; p.D = a.D;
    p.stride_tok = a.kv_stride_tok; p.scale = a.scale; p.causal = a.causal; p.window = a.sliding_window;
    p.key_mode = KEY_VQ;
    p.k_codes = a.k_indices; p.k_index_bytes = a.k_index_bytes; p.k_codebook = a.k_codebook;
    p.k_nc = a.k_n_centroids; p.k_sub = a.k_sub_dim; p.k_stacked = a.k_stacked;
    p.v_mode = a.v_mode == 0 ? V_DENSE : V_VQ; p.v = a.v; p.v_dtype = a.v_dtype; p.v_index_bytes = a.v_index_bytes;
    p.v_codebook = a.v_codebook; p.v_nc = a.v_n_centroids; p.v_sub = a.v_sub_dim;
    return launch_coded(p, a.workspace, a.workspace_bytes, a.n_splits, "fused_sdpa", (cudaStream_t)stream);
}

extern "C" int64_t vq_rabitq_attend_workspace_bytes(const vq_rabitq_attend_args *a) {
    return a ? vq::coded_workspace(a->B, a->H_q, a->S_q, a->D, a->n_splits) : 0;
}

extern "C" int32_t vq_rabitq_decode_attend(const vq_rabitq_attend_args *args, void *stream) {
    using namespace vq;
    VQ_REQUIRE(args != nullptr, VQ_ERR_SHAPE, "vq_rabitq_decode_attend: args is NULL");
    const vq_rabitq_attend_args &a = *args;
    VQ_REQUIRE(a.v_mode == 0 || a.v_mode == 2 || a.v_mode == 3, VQ_ERR_SHAPE, "rabitq_fused_attend: v_mode must be 0, 2 or 3");
    VQ_REQUIRE(a.v_mode == 0 || (a.v_cents && a.n_cents >= 1 && a.n_cents <= 16), VQ_ERR_SHAPE, "rabitq_fused_attend: v_cents must hold 1..16 entries");
    VQ_REQUIRE(a.q && a.out && a.q_scale && a.k_bits && a.k_mag && a.v, VQ_ERR_SHAPE, "rabitq_fused_attend: NULL argument");
    VQ_REQUIRE(a.D % 8 == 0, VQ_ERR_SHAPE, "rabitq_fused_attend: D must be a multiple of 8");
    VQ_REQUIRE(is_aligned(a.k_bits, 4) && (a.D / 8) % 4 == 0, VQ_ERR_ALIGN, "rabitq_fused_attend: k_bits must be 4-byte aligned with D a multiple of 32");
    CodedParams p{};
    p.q = a.q; p.out = a.out; p.q_dtype = a.q_dtype; p.out_dtype = a.out_dtype;
    p.B = a.B; p.H_q = a.H_q; p.H_kv = a.H_kv; p.S_q = a.S_q; p.S_kv = a.S_kv; p.D = a.D;
    p.stride_tok = a.kv_stride_tok; p.scale = 1.f; p.causal = 0; p.window = 0;
    p.key_mode = KEY_RABITQ;
    p.k_codes = a.k_bits; p.q_scale = a.q_scale; p.k_mag = a.k_mag; p.k_const = a.k_const;
    p.v_mode = a.v_mode == 0 ? V_DENSE : (a.v_mode == 2 ? V_CENT_BYTE : V_CENT_NIBBLE);
    p.v = a.v; p.v_dtype = a.v_dtype; p.v_codebook = a.v_cents; p.v_nc = a.n_cents;
    return launch_coded(p, a.workspace, a.workspace_bytes, a.n_splits, "rabitq_fused_attend", (cudaStream_t)stream);
}
