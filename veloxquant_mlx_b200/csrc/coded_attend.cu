// Decode attention over keys that are scored without being reconstructed:
//   VecInfer : score = scale * sum_s lut[s][idx[t][s]],  lut[s][c] = q_sub[s] . codebook[c]
//   RaBitQ   : score = (D - 2*popcount(sign(q) ^ bits[t])) * q_scale * k_mag[t] + k_const[t]
// Both read a few bytes per key (16 B at D=128) so the value stream dominates the traffic.
//
// One CTA per (context split, kv head x query row, batch) handles every query head of the kv
// head (GQA): a key code is loaded once and scored against all heads, a value row is loaded
// once and accumulated into all heads. A lane owns one key of a 32-key tile for scoring,
// then D/32 output channels for the value accumulation (weights broadcast with shuffles).
// Online softmax per warp and head; warps, then context splits, are merged afterwards.
#include <algorithm>

#include "common.cuh"
#include <cuda.h>

#include "kivi_attend.h"

namespace vq {

namespace {


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

constexpr int kWarpsC = 8;    // warps per CTA; each takes every 8th 32-key tile of the split
constexpr int kHeadsC = 8;    // query heads of one kv head handled by one CTA

// Fetch DPL consecutive value channels [lane*DPL, +DPL) of token `tok` as floats.
template <int DPL>
__device__ __forceinline__ void load_v_row(const CodedParams &p, int64_t tok, int lane, float (&v)[DPL]) {
    const int D = p.D;
    if (p.v_mode == V_DENSE) {
        if (p.v_dtype == VQ_F32) {
#pragma unroll
            for (int i = 0; i < DPL; ++i) v[i] = reinterpret_cast<const float *>(p.v)[tok * D + lane * DPL + i];
        } else if constexpr (DPL % 2 == 0) {
            const uint32_t *src = reinterpret_cast<const uint32_t *>(reinterpret_cast<const uint16_t *>(p.v) + tok * D + lane * DPL);
#pragma unroll
            for (int i = 0; i < DPL / 2; ++i) {
                const uint32_t w = src[i];
                if (p.v_dtype == VQ_F16) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w));
                    v[2 * i] = f.x; v[2 * i + 1] = f.y;
                } else {
                    v[2 * i] = __uint_as_float(w << 16); v[2 * i + 1] = __uint_as_float(w & 0xffff0000u);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < DPL; ++i) v[i] = load_as_f32(p.v, p.v_dtype, tok * D + lane * DPL + i);
        }
    } else if (p.v_mode == V_VQ) {
        const int nsv = D / p.v_sub;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int dim = lane * DPL + i;
            uint32_t c = load_index(p.v, p.v_index_bytes, tok * nsv + dim / p.v_sub);
            c = min(c, (uint32_t)(p.v_nc - 1));
            v[i] = p.v_codebook[(int64_t)c * p.v_sub + dim % p.v_sub];
        }
    } else if (p.v_mode == V_CENT_BYTE) {
#pragma unroll
        for (int i = 0; i < DPL; ++i) v[i] = p.v_codebook[reinterpret_cast<const uint8_t *>(p.v)[tok * D + lane * DPL + i] & 0xF];
    } else {
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int dim = lane * DPL + i;
            const uint32_t byte = reinterpret_cast<const uint8_t *>(p.v)[tok * (D / 2) + (dim >> 1)];
            v[i] = p.v_codebook[(dim & 1) ? (byte >> 4) : (byte & 0xFu)];
        }
    }
}

// Value-row access specialised at compile time so that the loads of several rows can be issued
// back to back before any of them is used (a run-time switch per row serialises them).
enum { VM_GENERIC = 0, VM_F16 = 1, VM_BF16 = 2, VM_NIBBLE = 3, VM_VQ8 = 4 };

// Raw 32-bit words one lane holds for one value row.
template <int DPL, int VM>
struct VRaw {
    static constexpr int N = (VM == VM_F16 || VM == VM_BF16) ? DPL / 2 : 1;
    uint32_t r[N];
};

template <int DPL, int VM>
__device__ __forceinline__ VRaw<DPL, VM> load_v_raw(const CodedParams &p, int64_t tok, int lane) {
    VRaw<DPL, VM> o;
    if constexpr (VM == VM_F16 || VM == VM_BF16) {
        const uint16_t *src = reinterpret_cast<const uint16_t *>(p.v) + tok * (DPL * 32) + lane * DPL;
        if constexpr (DPL == 2) o.r[0] = __ldg(reinterpret_cast<const uint32_t *>(src));
        else if constexpr (DPL == 4) { const uint2 t = __ldg(reinterpret_cast<const uint2 *>(src)); o.r[0] = t.x; o.r[1] = t.y; }
        else { const uint4 t = __ldg(reinterpret_cast<const uint4 *>(src)); o.r[0] = t.x; o.r[1] = t.y; o.r[2] = t.z; o.r[3] = t.w; }
    } else if constexpr (VM == VM_NIBBLE) {
        const uint8_t *src = reinterpret_cast<const uint8_t *>(p.v) + tok * (DPL * 16) + lane * (DPL / 2);
        if constexpr (DPL == 2) o.r[0] = __ldg(src);
        else if constexpr (DPL == 4) o.r[0] = __ldg(reinterpret_cast<const uint16_t *>(src));
        else o.r[0] = __ldg(reinterpret_cast<const uint32_t *>(src));
    } else {  // VM_VQ8: this lane's DPL channels lie inside one sub-vector
        const int nsv = (DPL * 32) / p.v_sub;
        o.r[0] = __ldg(reinterpret_cast<const uint8_t *>(p.v) + tok * nsv + (lane * DPL) / p.v_sub);
    }
    return o;
}

template <int DPL, int VM>
__device__ __forceinline__ void decode_v(const CodedParams &p, const VRaw<DPL, VM> &raw, const float *sh_vlut, int lane,
                                         float (&v)[DPL]) {
    if constexpr (VM == VM_F16) {
#pragma unroll
        for (int i = 0; i < DPL / 2; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&raw.r[i]));
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    } else if constexpr (VM == VM_BF16) {
#pragma unroll
        for (int i = 0; i < DPL / 2; ++i) {
            v[2 * i] = __uint_as_float(raw.r[i] << 16); v[2 * i + 1] = __uint_as_float(raw.r[i] & 0xffff0000u);
        }
    } else if constexpr (VM == VM_NIBBLE) {
#pragma unroll
        for (int i = 0; i < DPL; ++i) v[i] = sh_vlut[(raw.r[0] >> (4 * i)) & 0xFu];
    } else {
        const uint32_t c = min(raw.r[0], (uint32_t)(p.v_nc - 1));
        const float *row = sh_vlut + c * p.v_sub + (lane * DPL) % p.v_sub;
#pragma unroll
        for (int i = 0; i < DPL; ++i) v[i] = row[i];
    }
}

// Warp maximum of finite-or-minus-infinity floats in one reduction instruction: floats order like
// their bit patterns read as sign-magnitude integers, which one XOR turns into two's complement.
__device__ __forceinline__ float st_warp_max(float x) {
    int i = __float_as_int(x);
    i ^= (i >> 31) & 0x7fffffff;
    i = __reduce_max_sync(0xffffffffu, i);
    i ^= (i >> 31) & 0x7fffffff;
    return __int_as_float(i);
}

__device__ __forceinline__ bool is_aligned_dev(const void *ptr, unsigned a) { return (reinterpret_cast<uintptr_t>(ptr) & (a - 1)) == 0; }

// lut[head][sub][c] = q_sub[head][sub] . codebook[c] for sub-vectors of KS = 4 or 8 floats.
template <int KS, int NH>
__device__ __forceinline__ void build_lut_vec(const CodedParams &p, float *lut, const float *sh_q, int nh, int n_sub, int lut_stride, int D) {
    for (int c = threadIdx.x; c < p.k_nc; c += blockDim.x) {
        float cbr[KS];
        for (int s = 0; s < n_sub; ++s) {
            if (s == 0 || p.k_stacked) {
                const float4 *cb = reinterpret_cast<const float4 *>(p.k_codebook + ((int64_t)(p.k_stacked ? s : 0) * p.k_nc + c) * KS);
#pragma unroll
                for (int e = 0; e < KS / 4; ++e) {
                    const float4 t = __ldg(cb + e);
                    cbr[4 * e] = t.x; cbr[4 * e + 1] = t.y; cbr[4 * e + 2] = t.z; cbr[4 * e + 3] = t.w;
                }
            }
            float dot[NH];
#pragma unroll
            for (int hp = 0; hp < NH; ++hp) {
                // (rows past nh hold whatever the buffer held: computed, never stored)
                const float4 *qv = reinterpret_cast<const float4 *>(sh_q + (hp < nh ? hp : 0) * D + s * KS);
                float acc = 0.f;
#pragma unroll
                for (int e = 0; e < KS / 4; ++e) {
                    const float4 t = qv[e];
                    acc = fmaf(t.x, cbr[4 * e], acc); acc = fmaf(t.y, cbr[4 * e + 1], acc);
                    acc = fmaf(t.z, cbr[4 * e + 2], acc); acc = fmaf(t.w, cbr[4 * e + 3], acc);
                }
                dot[hp] = acc;
            }
#pragma unroll
            for (int hp = 0; hp < NH; ++hp)
                if (hp < nh) lut[hp * lut_stride + s * p.k_nc + c] = dot[hp];
        }
    }
}

// One CTA: (context split, kv head x query row x head chunk, batch). All (<= 8) query heads of
// the kv head are handled together: a key's code is loaded once and scored against every
// head, a value row is loaded once and accumulated into every head. Warps take alternate
// 32-key tiles of the split; value rows are fetched eight at a time so that eight
// independent loads are in flight per lane.
// EAGER (small grids: about one CTA per SM, every load's latency exposed): a warp requests all 32
// value rows of its tile before it scores the keys, so the rows arrive under the score / softmax work
// instead of in four batches after it (64 more registers; two CTAs per SM).
template <int DPL, int VM, int NH, bool EAGER = false>
__global__ void __launch_bounds__(kWarpsC * 32, (NH <= 4 && DPL <= 4 && VM != VM_GENERIC && !EAGER) ? 3 : 2)
coded_attend_kernel(const CodedParams p, int key_floats, int vlut_floats) {
    extern __shared__ __align__(16) float smem[];
    const int lane = threadIdx.x & 31, warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // (known warp-uniform)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the merge kernel may become resident
    const int split = blockIdx.x;
    int y = blockIdx.y;
    const int hc = y % p.n_head_chunks; y /= p.n_head_chunks;
    const int sq = y % p.S_q;
    const int hkv = y / p.S_q;
    const int b = blockIdx.z;
    const int hpk = p.H_q / p.H_kv;
    const int h0 = hc * kHeadsC;
    const int nh = min(NH, hpk - h0);  // NH = 4 is launched only when hpk <= 4
    const int D = p.D;
    const int64_t bh = (int64_t)b * p.H_kv + hkv;
    const int n_sub = p.key_mode == KEY_VQ ? D / p.k_sub : 0;
    const int lut_stride = n_sub * p.k_nc;

    // shared: VQ lookup tables [nh][n_sub*n_c] | RaBitQ: query sign words [nh][8] and scales [nh]
    float *lut = smem;
    uint32_t *sh_qbits = reinterpret_cast<uint32_t *>(smem);
    float *sh_qs = smem + NH * 8;
    float *sh_vlut = smem + key_floats;                              // value centroids / codebook
    float *sh_w = sh_vlut + vlut_floats + warp * (32 * NH);     // this warp's softmax weights [key][head]
    if constexpr (VM == VM_NIBBLE || VM == VM_VQ8) {
        const int n = VM == VM_NIBBLE ? p.v_nc : p.v_nc * p.v_sub;
        for (int i = threadIdx.x; i < vlut_floats; i += blockDim.x) sh_vlut[i] = i < n ? p.v_codebook[i] : 0.f;
    }
    if (p.key_mode == KEY_VQ) {
        // Query rows to shared memory first; then thread c holds centroid c in registers and
        // fills lut[head][sub][c] for every head and sub-space (writes are conflict-free, the
        // query values are broadcast reads).
        float *sh_q = lut + nh * lut_stride;  // [nh][D]
        for (int i = threadIdx.x; i < nh * D; i += blockDim.x) {
            const int hp = i / D, d = i % D;
            const int64_t qrow = ((int64_t)b * p.H_q + hkv * hpk + h0 + hp) * p.S_q + sq;
            sh_q[i] = load_as_f32(p.q, p.q_dtype, qrow * D + d);
        }
        __syncthreads();
        for (int c = threadIdx.x; c < p.k_nc && p.k_sub > 16; c += blockDim.x) {  // wide sub-vectors: no register copy
            for (int s = 0; s < n_sub; ++s) {
                const float *cb = p.k_codebook + ((int64_t)(p.k_stacked ? s : 0) * p.k_nc + c) * p.k_sub;
                for (int hp = 0; hp < nh; ++hp) {
                    float dot = 0.f;
                    for (int e = 0; e < p.k_sub; ++e) dot += sh_q[hp * D + s * p.k_sub + e] * cb[e];
                    lut[hp * lut_stride + s * p.k_nc + c] = dot;
                }
            }
        }
        // sub-vectors of 4 or 8 (16-byte aligned codebook rows): the centroid as vector loads, the query
        // sub-vector as broadcast vector reads, all heads' dot products as independent chains
        const bool vec_cb = (p.k_sub == 8 || p.k_sub == 4) && is_aligned_dev(p.k_codebook, 16) && lut_stride % 4 == 0;
        if (vec_cb && p.k_sub == 8) build_lut_vec<8, NH>(p, lut, sh_q, nh, n_sub, lut_stride, D);
        if (vec_cb && p.k_sub == 4) build_lut_vec<4, NH>(p, lut, sh_q, nh, n_sub, lut_stride, D);
        for (int c = threadIdx.x; c < p.k_nc && p.k_sub <= 16 && !vec_cb; c += blockDim.x) {
            float cbr[16];
            for (int s = 0; s < n_sub; ++s) {
                if (s == 0 || p.k_stacked) {
                    const float *cb = p.k_codebook + ((int64_t)(p.k_stacked ? s : 0) * p.k_nc + c) * p.k_sub;
#pragma unroll
                    for (int e = 0; e < 16; ++e) cbr[e] = e < p.k_sub ? cb[e] : 0.f;
                }
                for (int hp = 0; hp < nh; ++hp) {
                    const float *qs_ = sh_q + hp * D + s * p.k_sub;
                    float dot = 0.f;
#pragma unroll
                    for (int e = 0; e < 16; ++e)
                        if (e < p.k_sub) dot += qs_[e] * cbr[e];
                    lut[hp * lut_stride + s * p.k_nc + c] = dot;
                }
            }
        }
    } else if (warp < nh) {
        const int64_t qrow = ((int64_t)b * p.H_q + hkv * hpk + h0 + warp) * p.S_q + sq;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            const float v = (32 * w + lane < D) ? load_as_f32(p.q, p.q_dtype, qrow * D + 32 * w + lane) : -1.f;
            const uint32_t bits = __ballot_sync(0xffffffffu, v >= 0.f);
            if (lane == 0) sh_qbits[warp * 8 + w] = bits;
        }
        if (lane == 0) sh_qs[warp] = p.q_scale[qrow];
    }
    __syncthreads();

    const int chunk = (p.S_kv + p.n_splits - 1) / p.n_splits;
    const int t_begin = split * chunk;
    const int t_end = min(p.S_kv, t_begin + chunk);
    const int q_abs = p.S_kv - p.S_q + sq;
    const int n_words = D / 32;
    const bool idx16 = p.key_mode == KEY_VQ && n_sub == 16 && p.k_index_bytes == 1 && is_aligned_dev(p.k_codes, 16);

    float m_run[NH], l_run[NH], acc[NH][DPL];  // acc[head][this lane's DPL channels]
#pragma unroll
    for (int h = 0; h < NH; ++h) {
        m_run[h] = -INFINITY; l_run[h] = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[h][i] = 0.f;
    }

    for (int tile = t_begin + 32 * warp; tile < t_end; tile += 32 * kWarpsC) {
        const int t = tile + lane;
        bool valid = t < t_end;
        if (valid && p.causal && t > q_abs) valid = false;
        if (valid && p.window > 0 && q_abs + 1 > p.window && t + p.window < q_abs + 1) valid = false;
        const int64_t tok = bh * p.stride_tok + (valid ? t : t_begin);
        float w[NH];
        VRaw<DPL, VM> early[EAGER ? 32 : 1];
        if constexpr (EAGER) {
            const int n_in = min(32, t_end - tile);
#pragma unroll
            for (int j = 0; j < 32; ++j) early[j] = load_v_raw<DPL, VM>(p, bh * p.stride_tok + tile + min(j, n_in - 1), lane);
        }
        // ---- scores of this lane's key against every head ---------------------------------
        if (p.key_mode == KEY_VQ) {
#pragma unroll
            for (int h = 0; h < NH; ++h) w[h] = 0.f;
            if (idx16) {
                // sixteen one-byte indices per key: the whole row in one 16-byte load
                const uint4 iv = __ldg(reinterpret_cast<const uint4 *>(static_cast<const uint8_t *>(p.k_codes) + tok * 16));
                const uint32_t wd[4] = {iv.x, iv.y, iv.z, iv.w};
#pragma unroll
                for (int sub = 0; sub < 16; ++sub) {
                    const uint32_t c = min((wd[sub >> 2] >> (8 * (sub & 3))) & 0xFFu, (uint32_t)(p.k_nc - 1));
                    const float *row = lut + sub * p.k_nc + c;
#pragma unroll
                    for (int h = 0; h < NH; ++h)
                        if (h < nh) w[h] += row[h * lut_stride];
                }
            } else {
                for (int sub = 0; sub < n_sub; ++sub) {
                    uint32_t c = load_index(p.k_codes, p.k_index_bytes, tok * n_sub + sub);
                    c = min(c, (uint32_t)(p.k_nc - 1));
                    const float *row = lut + sub * p.k_nc + c;
#pragma unroll
                    for (int h = 0; h < NH; ++h)
                        if (h < nh) w[h] += row[h * lut_stride];
                }
            }
#pragma unroll
            for (int h = 0; h < NH; ++h) w[h] = valid ? w[h] * p.scale : -INFINITY;
        } else {
            const uint32_t *kb = reinterpret_cast<const uint32_t *>(reinterpret_cast<const uint8_t *>(p.k_codes) + tok * (D / 8));
            uint32_t kw[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) kw[i] = i < n_words ? kb[i] : 0u;
            const float km = p.k_mag[tok];
            const float kc = p.k_const ? p.k_const[tok] : 0.f;
#pragma unroll
            for (int h = 0; h < NH; ++h) {
                int ham = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (i < n_words) ham += __popc(sh_qbits[(h < nh ? h : 0) * 8 + i] ^ kw[i]);
                const float s = ((float)D - 2.0f * (float)ham) * sh_qs[h < nh ? h : 0] * km + kc;
                w[h] = valid ? s : -INFINITY;
            }
        }
        // ---- online softmax per head ------------------------------------------------------
        bool any_live = false;
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            if (h < nh) {
                const float tile_max = st_warp_max(w[h]);      // (one reduction instruction)
                if (tile_max == -INFINITY) { w[h] = 0.f; continue; }
                any_live = true;
                const float m_new = fmaxf(m_run[h], tile_max);
                const float factor = (m_run[h] == -INFINITY) ? 0.f : __expf(m_run[h] - m_new);
                m_run[h] = m_new;
                w[h] = valid ? __expf(w[h] - m_new) : 0.f;
                l_run[h] = l_run[h] * factor + w[h];           // (this lane's share: summed over the warp after the loop)
#pragma unroll
                for (int i = 0; i < DPL; ++i) acc[h][i] *= factor;
            } else {
                w[h] = 0.f;
            }
        }
        if (!any_live) continue;
        // ---- values: eight rows in flight, each accumulated into every head ----------------
        const int n_in_tile = min(32, t_end - tile);
        if constexpr (VM == VM_GENERIC) {
            for (int l0 = 0; l0 < n_in_tile; l0 += 8) {
                float vrow[8][DPL];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int tl = min(l0 + j, n_in_tile - 1);  // rows past the end get weight 0
                    load_v_row<DPL>(p, bh * p.stride_tok + tile + tl, lane, vrow[j]);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
#pragma unroll
                    for (int h = 0; h < NH; ++h) {
                        if (h < nh) {
                            const float wl = (l0 + j < n_in_tile) ? __shfl_sync(0xffffffffu, w[h], l0 + j) : 0.f;
#pragma unroll
                            for (int i = 0; i < DPL; ++i) acc[h][i] = fmaf(wl, vrow[j][i], acc[h][i]);
                        }
                    }
                }
            }
        } else {
            // weights to shared memory: one broadcast 16-byte read per row and four heads
            // instead of one shuffle per row and head
            __syncwarp();
            *reinterpret_cast<float4 *>(sh_w + lane * NH) = make_float4(w[0], w[1], w[2], w[3]);
            if constexpr (NH == 8) *reinterpret_cast<float4 *>(sh_w + lane * NH + 4) = make_float4(w[4], w[5], w[6], w[7]);
            __syncwarp();
            if constexpr (EAGER) {
                static_assert(NH == 4, "the eager form is instantiated for four heads");
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    float v[DPL];
                    decode_v<DPL, VM>(p, early[j], sh_vlut, lane, v);
                    const float4 wa = *reinterpret_cast<const float4 *>(sh_w + j * NH);   // (0 for rows past the tile's end)
                    const float wl4[4] = {wa.x, wa.y, wa.z, wa.w};
#pragma unroll
                    for (int h = 0; h < 4; ++h)
#pragma unroll
                        for (int i = 0; i < DPL; ++i) acc[h][i] = fmaf(wl4[h], v[i], acc[h][i]);
                }
                continue;
            }
            // Two batches of R rows are in flight: the next batch is requested before the
            // current one is consumed.
            constexpr int R = 8;
            const int64_t tok0 = bh * p.stride_tok + tile;
            VRaw<DPL, VM> raw[R], nxt[R];
#pragma unroll
            for (int j = 0; j < R; ++j) raw[j] = load_v_raw<DPL, VM>(p, tok0 + min(j, n_in_tile - 1), lane);
            // (with three CTAs per SM the register budget has no room for the second batch:
            // there the next batch is requested after the current one is consumed)
            constexpr bool kAhead = !(NH <= 4 && DPL <= 4);
#pragma unroll(kAhead ? 4 : 1)
            for (int l0 = 0; l0 < 32; l0 += R) {
                if (l0 >= n_in_tile) break;
                if (kAhead && l0 + R < 32 && l0 + R < n_in_tile) {
#pragma unroll
                    for (int j = 0; j < R; ++j) nxt[j] = load_v_raw<DPL, VM>(p, tok0 + min(l0 + R + j, n_in_tile - 1), lane);
                }
#pragma unroll
                for (int j = 0; j < R; ++j) {
                    float v[DPL];
                    decode_v<DPL, VM>(p, raw[j], sh_vlut, lane, v);
                    // rows past the end of the tile belong to lanes whose weight is already 0
                    const int wr = l0 + j;
                    const float4 wa = *reinterpret_cast<const float4 *>(sh_w + wr * NH);
                    const float wl4[4] = {wa.x, wa.y, wa.z, wa.w};
#pragma unroll
                    for (int h = 0; h < 4; ++h)
#pragma unroll
                        for (int i = 0; i < DPL; ++i) acc[h][i] = fmaf(wl4[h], v[i], acc[h][i]);
                    if constexpr (NH == 8) if (nh > 4) {
                        const float4 wb = *reinterpret_cast<const float4 *>(sh_w + wr * NH + 4);
                        const float wh4[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                        for (int h = 0; h < 4; ++h)
#pragma unroll
                            for (int i = 0; i < DPL; ++i) acc[4 + h][i] = fmaf(wh4[h], v[i], acc[4 + h][i]);
                    }
                }
                if (kAhead) {
#pragma unroll
                    for (int j = 0; j < R; ++j) raw[j] = nxt[j];
                } else if (l0 + R < 32 && l0 + R < n_in_tile) {
#pragma unroll
                    for (int j = 0; j < R; ++j) raw[j] = load_v_raw<DPL, VM>(p, tok0 + min(l0 + R + j, n_in_tile - 1), lane);
                }
            }
        }
    }

    // ---- merge the warps of this CTA -------------------------------------------------------
#pragma unroll
    for (int h = 0; h < NH; ++h) l_run[h] = warp_sum(l_run[h]);
    __syncthreads();  // the lookup tables are dead: reuse shared memory
    float *red_o = smem;                                   // [warps][heads][D]
    float *red_m = red_o + kWarpsC * NH * D;          // [warps][heads]
    float *red_l = red_m + kWarpsC * NH;
#pragma unroll
    for (int h = 0; h < NH; ++h) {
        if (h < nh) {
#pragma unroll
            for (int i = 0; i < DPL; ++i) red_o[(warp * NH + h) * D + lane * DPL + i] = acc[h][i];
            if (lane == 0) { red_m[warp * NH + h] = m_run[h]; red_l[warp * NH + h] = l_run[h]; }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nh * D; i += blockDim.x) {
        const int h = i / D, d = i % D;
        float gm = -INFINITY;
        for (int wq = 0; wq < kWarpsC; ++wq) gm = fmaxf(gm, red_m[wq * NH + h]);
        float gl = 0.f, o = 0.f;
        for (int wq = 0; wq < kWarpsC; ++wq) {
            const float mw = red_m[wq * NH + h];
            const float f = (mw == -INFINITY) ? 0.f : __expf(mw - gm);
            gl += red_l[wq * NH + h] * f;
            o += red_o[(wq * NH + h) * D + d] * f;
        }
        const int64_t qrow = ((int64_t)b * p.H_q + hkv * hpk + h0 + h) * p.S_q + sq;
        if (p.n_splits == 1) {
            store_from_f32(p.out, p.out_dtype, qrow * D + d, o / fmaxf(gl, 1e-20f));
        } else {
            p.part_o[(qrow * p.n_splits + split) * D + d] = o;
            if (d == 0) {
                p.part_ml[(qrow * p.n_splits + split) * 2] = gm;
                p.part_ml[(qrow * p.n_splits + split) * 2 + 1] = gl;
            }
        }
    }
}

// ---- RaBitQ over dense 16-bit values, head_dim 128: staged through shared memory ------------
// The same attention as coded_attend_kernel for the serving shape, with the key bits, key
// magnitudes (and constants) and the value rows of each 32-key tile brought in by the bulk
// async-copy engine: every warp runs its own two-stage cp.async.bulk + mbarrier pipeline
// (3 linear pieces and two tensor boxes per tile, 8.7-8.9 KB), so HBM reads stay in flight while the warp
// scores and accumulates. Waits are bounded; a timeout raises a device flag that
// vq_kivi_attend_status() reports.
//
// The weighted value sum runs on the tensor cores: O^T[channel, head] += V^T[channel, key] . P[key, head]
// as m16n8k16 MMAs with the value rows as the A operand (read from shared memory by transposing
// ldmatrix loads; the rows arrive through a tensor map with the 128-byte swizzle, which spreads
// the eight rows of a load over all banks) and the softmax weights as the small B operand. With
// up to four heads per CTA each weight occupies two of the eight columns as a (high, low) pair of
// halves, so the products carry ~22 bits of the weight; with eight heads it is one rounded
// half / bfloat16 per weight.
// three warps per CTA: four CTAs (57 KB of stages each) share an SM, and the 592 CTA slots divide typical
// (batch x kv head x split) grids better than 444 slots of four warps did (measured 51 vs 53 us at B=8, 8 kv heads, 16K keys)
constexpr int kStWarps = 3, kStStages = 2;
// one warp, one stage: key bits | magnitudes | constants | value rows (two swizzled halves of 32 x 128 bytes)
constexpr int kStMag = 512, kStConst = 640, kStV = 1024, kStBytes = 1024 + 32 * 256;
constexpr uint32_t kStSpin = 1u << 18;
__device__ int g_coded_timeout = 0;

__device__ __forceinline__ uint32_t st_smem_u32(const void *ptr) { return (uint32_t)__cvta_generic_to_shared(ptr); }
__device__ __forceinline__ bool st_mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kStSpin; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void st_bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void st_tensor_g2s(uint32_t dst, const CUtensorMap *map, int x, int y, int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void st_ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <bool BF16>
__device__ __forceinline__ void st_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (BF16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// Two weights as one B-operand register in the value dtype: the high halves (rounded weights) or,
// for the low column of a head, what the rounding left over.
template <bool BF16>
__device__ __forceinline__ uint32_t st_pack_weights(float x0, float x1, bool low) {
    if constexpr (BF16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
        if (low) h = __floats2bfloat162_rn(x0 - __low2float(h), x1 - __high2float(h));
        return *reinterpret_cast<uint32_t *>(&h);
    } else {
        __half2 h = __floats2half2_rn(x0, x1);
        if (low) h = __floats2half2_rn(x0 - __low2float(h), x1 - __high2float(h));
        return *reinterpret_cast<uint32_t *>(&h);
    }
}

// W = warps per CTA. VQ != 0: the keys are sixteen one-byte codebook indices (the 512-byte "bits" piece of
// a stage carries them) scored through a lookup table lut[sub][centroid][head] of 64 KB that the CTA builds
// first: one CTA of eight warps per SM instead of four CTAs of three. VQ == 2: the values are sixteen
// one-byte indices as well (a second 512-byte piece); the warp expands them through a float16 copy of the
// value codebook into the stage's value tile, in the layout the swizzled tensor copy would have left.
template <bool VBF16, int NH, int W, int VQ>
__global__ void __launch_bounds__(W * 32, VQ ? 1 : 4)
rabitq_attend_staged_kernel(const CodedParams p, const __grid_constant__ CUtensorMap v_map) {
    extern __shared__ __align__(1024) uint8_t st_raw[];
    constexpr int D = 128;
    const int lane = threadIdx.x & 31, warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // (known warp-uniform)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the merge kernel may become resident
    const int split = blockIdx.x;
    int y = blockIdx.y;
    const int hc = y % p.n_head_chunks; y /= p.n_head_chunks;
    const int sq = y % p.S_q;
    const int hkv = y / p.S_q;
    const int b = blockIdx.z;
    const int hpk = p.H_q / p.H_kv;
    const int h0 = hc * kHeadsC;
    const int nh = min(NH, hpk - h0);
    const int64_t bh = (int64_t)b * p.H_kv + hkv;

    // shared: stages (1024-byte aligned: the swizzle pattern repeats every 1024 bytes) | barriers |
    // query sign words [NH][4] | query scales [NH] | weights [warp][32][NH]
    constexpr int kStagesAll = W * kStStages * kStBytes;
    uint8_t *stages = st_raw + (size_t)warp * kStStages * kStBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(st_raw + kStagesAll);
    uint32_t *sh_qbits = reinterpret_cast<uint32_t *>(st_raw + kStagesAll + 64);
    float *sh_qs = reinterpret_cast<float *>(st_raw + kStagesAll + 64 + NH * 16);
    float *sh_w = reinterpret_cast<float *>(st_raw + kStagesAll + 256) + warp * (32 * NH);
    // VQ: query rows [NH][128] and the table [16][256] x float4 (one entry = the four heads' partial scores)
    float *sh_q = reinterpret_cast<float *>(st_raw + kStagesAll + 256) + W * (32 * NH);
    float4 *lutv = reinterpret_cast<float4 *>(sh_q + NH * D);
    constexpr bool VV = VQ == 2;
    __half *sh_vcb = reinterpret_cast<__half *>(lutv + 16 * 256);   // VV: value centroids [256][8] as halves
    const uint32_t wbar0 = st_smem_u32(bars) + 8u * (warp * kStStages);
    const int g = lane >> 2, c = lane & 3;
    if (st_smem_u32(st_raw) & 1023u) {  // the swizzled addressing below assumes this; never seen
        if (threadIdx.x == 0) atomicExch(&g_coded_timeout, 2);
        return;
    }

    if (threadIdx.x == 0) {
        for (int i = 0; i < W * kStStages; ++i)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(st_smem_u32(bars) + 8u * i));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if constexpr (VQ) {
        static_assert(NH == 4, "the table entry holds four heads");
        for (int i = threadIdx.x; i < NH * D; i += W * 32) {
            const int h = i / D, d = i % D;
            const int64_t qrow = ((int64_t)b * p.H_q + hkv * hpk + h0 + h) * p.S_q + sq;
            sh_q[i] = h < nh ? load_as_f32(p.q, p.q_dtype, qrow * D + d) : 0.f;
        }
        if constexpr (VV) {
            for (int i = threadIdx.x; i < 256 * 8; i += W * 32)
                sh_vcb[i] = __float2half_rn(p.v_codebook[(int64_t)min(i >> 3, p.v_nc - 1) * 8 + (i & 7)]);
        }
        __syncthreads();
        for (int cc = threadIdx.x; cc < 256; cc += W * 32) {
            const int cen = min(cc, p.k_nc - 1);
            float cbr[8];
            for (int sub = 0; sub < 16; ++sub) {
                if (sub == 0 || p.k_stacked) {
                    const float4 *cb = reinterpret_cast<const float4 *>(p.k_codebook + ((int64_t)(p.k_stacked ? sub : 0) * p.k_nc + cen) * 8);
                    const float4 t0 = __ldg(cb), t1 = __ldg(cb + 1);
                    cbr[0] = t0.x; cbr[1] = t0.y; cbr[2] = t0.z; cbr[3] = t0.w; cbr[4] = t1.x; cbr[5] = t1.y; cbr[6] = t1.z; cbr[7] = t1.w;
                }
                float dot[4];
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    const float4 *qv = reinterpret_cast<const float4 *>(sh_q + h * D + sub * 8);
                    const float4 u0 = qv[0], u1 = qv[1];
                    float acc1 = u0.x * cbr[0];
                    acc1 = fmaf(u0.y, cbr[1], acc1); acc1 = fmaf(u0.z, cbr[2], acc1); acc1 = fmaf(u0.w, cbr[3], acc1);
                    acc1 = fmaf(u1.x, cbr[4], acc1); acc1 = fmaf(u1.y, cbr[5], acc1); acc1 = fmaf(u1.z, cbr[6], acc1); acc1 = fmaf(u1.w, cbr[7], acc1);
                    dot[h] = acc1;
                }
                lutv[sub * 256 + cc] = make_float4(dot[0], dot[1], dot[2], dot[3]);
            }
        }
    } else {
        for (int h = warp; h < nh; h += W) {
            const int64_t qrow = ((int64_t)b * p.H_q + hkv * hpk + h0 + h) * p.S_q + sq;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float v = load_as_f32(p.q, p.q_dtype, qrow * D + 32 * w + lane);
                const uint32_t bits = __ballot_sync(0xffffffffu, v >= 0.f);
                if (lane == 0) sh_qbits[h * 4 + w] = bits;
            }
            if (lane == 0) sh_qs[h] = p.q_scale[qrow];
        }
    }
    __syncthreads();

    // this CTA's keys: whole 32-key tiles; warp w takes tiles w, w + 4, ...
    const int chunk = (((p.S_kv + p.n_splits - 1) / p.n_splits) + 31) & ~31;
    const int t_begin = split * chunk;
    const int t_end = min(p.S_kv, t_begin + chunk);
    const int n_tiles = t_begin < t_end ? (t_end - t_begin + 31) / 32 : 0;
    const int n_local = warp < n_tiles ? (n_tiles - warp + W - 1) / W : 0;
    const uint8_t *kb_g = reinterpret_cast<const uint8_t *>(p.k_codes) + bh * p.stride_tok * 16;
    const uint8_t *vb_g = VV ? reinterpret_cast<const uint8_t *>(p.v) + bh * p.stride_tok * 16 : nullptr;
    const float *km_g = VQ ? nullptr : p.k_mag + bh * p.stride_tok;
    const float *kc_g = (!VQ && p.k_const) ? p.k_const + bh * p.stride_tok : nullptr;

    auto issue = [&](int j) {  // lane 0 only
        const int64_t tile = t_begin + 32 * (warp + W * j);
        const int stage = j % kStStages;
        const uint32_t bar = wbar0 + 8u * stage;
        const uint32_t dst = st_smem_u32(stages + (size_t)stage * kStBytes);
        const uint32_t bytes = VV ? 1024u : 512 + (VQ ? 0 : 128) + (kc_g ? 128 : 0) + 32 * 256;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
        st_bulk_g2s(dst, kb_g + tile * 16, 512, bar);
        if constexpr (VV) {
            st_bulk_g2s(dst + 512, vb_g + tile * 16, 512, bar);   // the value indices (the value tile is built by the warp)
            return;
        }
        if constexpr (!VQ) st_bulk_g2s(dst + kStMag, km_g + tile, 128, bar);
        if (kc_g) st_bulk_g2s(dst + kStConst, kc_g + tile, 128, bar);
        // the value rows: channels 0-63 and 64-127 as two swizzled boxes; rows past the context read as zeros
        st_tensor_g2s(dst + kStV, &v_map, 0, (int)tile, (int)bh, bar);
        st_tensor_g2s(dst + kStV + 4096, &v_map, 128, (int)tile, (int)bh, bar);
    };
    if (lane == 0)
        for (int j = 0; j < kStStages - 1 && j < n_local; ++j) issue(j);

    // acc[mt]: channels 16*mt + g (regs 0, 1) and + 8 (regs 2, 3); columns 2c, 2c+1 = the (high, low)
    // weight columns of head c (NH = 4) or heads 2c, 2c+1 (NH = 8)
    float m_run[NH], l_run[NH], acc[8][4];
#pragma unroll
    for (int h = 0; h < NH; ++h) { m_run[h] = -INFINITY; l_run[h] = 0.f; }
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;
    // this lane's rows of the transposing loads: matrix lane / 8 = (keys 0-7 | 8-15) x (channel chunk even | odd)
    const uint32_t lm_tok = (uint32_t)(8 * (lane >> 4) + (lane & 7)), lm_chunk = (uint32_t)((lane >> 3) & 1);
    bool timed_out = false;
    for (int j = 0; j < n_local; ++j) {
        __syncwarp();  // every lane is done with the stage that is refilled next
        if (lane == 0 && j + kStStages - 1 < n_local) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue(j + kStStages - 1);
        }
        const int stage = j % kStStages;
        if (!timed_out && !st_mbar_wait(wbar0 + 8u * stage, (uint32_t)((j / kStStages) & 1))) timed_out = true;
        const uint8_t *st = stages + (size_t)stage * kStBytes;
        const int tile = t_begin + 32 * (warp + W * j);
        const bool valid = tile + lane < t_end;
        // ---- scores of this lane's key against every head ---------------------------------
        const uint4 kw = *reinterpret_cast<const uint4 *>(st + lane * 16);
        float w[NH];
        if constexpr (VQ) {
            // sixteen table reads of 16 bytes: one entry holds this centroid's partial score for all four heads
            const uint32_t wd[4] = {kw.x, kw.y, kw.z, kw.w};
            float4 sacc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int sub = 0; sub < 16; ++sub) {
                const uint32_t cen = (wd[sub >> 2] >> (8 * (sub & 3))) & 0xFFu;
                const float4 e = lutv[sub * 256 + cen];
                sacc.x += e.x; sacc.y += e.y; sacc.z += e.z; sacc.w += e.w;
            }
            w[0] = valid ? sacc.x * p.scale : -INFINITY; w[1] = valid ? sacc.y * p.scale : -INFINITY;
            w[2] = valid ? sacc.z * p.scale : -INFINITY; w[3] = valid ? sacc.w * p.scale : -INFINITY;
        } else {
            const float km = reinterpret_cast<const float *>(st + kStMag)[lane];
            const float kc = kc_g ? reinterpret_cast<const float *>(st + kStConst)[lane] : 0.f;
#pragma unroll
            for (int h = 0; h < NH; ++h) {
                const uint32_t *qb = sh_qbits + (h < nh ? h : 0) * 4;
                const int ham = __popc(qb[0] ^ kw.x) + __popc(qb[1] ^ kw.y) + __popc(qb[2] ^ kw.z) + __popc(qb[3] ^ kw.w);
                const float s = ((float)D - 2.0f * (float)ham) * sh_qs[h < nh ? h : 0] * km + kc;
                w[h] = valid ? s : -INFINITY;
            }
        }
        // ---- online softmax per head ------------------------------------------------------
        float factor[NH];
#pragma unroll
        for (int h = 0; h < NH; ++h) {
            if (h < nh) {
                const float tile_max = st_warp_max(w[h]);  // at least lane 0 of a tile is valid
                const float m_new = fmaxf(m_run[h], tile_max);
                factor[h] = (m_run[h] == -INFINITY) ? 0.f : __expf(m_run[h] - m_new);
                m_run[h] = m_new;
                w[h] = valid ? __expf(w[h] - m_new) : 0.f;
                l_run[h] = l_run[h] * factor[h] + w[h];  // (this lane's share: summed over the warp after the loop)
            } else {
                w[h] = 0.f;
                factor[h] = 1.f;
            }
        }
        {
            // rescale this lane's columns (the maxima settle after a few tiles: skipped when nothing moved)
            bool moved = false;
#pragma unroll
            for (int h = 0; h < NH; ++h) moved |= factor[h] != 1.f;
            if (moved) {  // (factor is the same in every lane)
                float f0, f1;
                if constexpr (NH == 4) {
                    f0 = f1 = c == 0 ? factor[0] : c == 1 ? factor[1] : c == 2 ? factor[2] : factor[3];
                } else {
                    f0 = c == 0 ? factor[0] : c == 1 ? factor[2] : c == 2 ? factor[4] : factor[6];
                    f1 = c == 0 ? factor[1] : c == 1 ? factor[3] : c == 2 ? factor[5] : factor[7];
                }
#pragma unroll
                for (int mt = 0; mt < 8; ++mt) { acc[mt][0] *= f0; acc[mt][1] *= f1; acc[mt][2] *= f0; acc[mt][3] *= f1; }
            }
        }
        // ---- the weights as the B operand: column g = head g / 2, high or low half (NH = 4); head g (NH = 8)
        __syncwarp();
        *reinterpret_cast<float4 *>(sh_w + lane * NH) = make_float4(w[0], w[1], w[2], w[3]);
        if constexpr (NH == 8) *reinterpret_cast<float4 *>(sh_w + lane * NH + 4) = make_float4(w[4], w[5], w[6], w[7]);
        __syncwarp();
        uint32_t pb[2][2];
        {
            const int hh = NH == 4 ? (g >> 1) : g;
            const bool low = NH == 4 && (g & 1);
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
                const float *wp = sh_w + (16 * ks + 2 * c) * NH + hh;
                pb[ks][0] = st_pack_weights<VBF16>(wp[0], wp[NH], low);
                pb[ks][1] = st_pack_weights<VBF16>(wp[8 * NH], wp[9 * NH], low);
            }
        }
        if constexpr (VV) {
            // this lane's key: sixteen centroids of 8 channels = sixteen 16-byte chunks of its 256-byte value
            // row, stored where the 128-byte-swizzled tensor copy would have put them
            const uint4 vw = *reinterpret_cast<const uint4 *>(st + 512 + lane * 16);
            const uint32_t vd[4] = {vw.x, vw.y, vw.z, vw.w};
            uint8_t *vt = const_cast<uint8_t *>(st) + kStV + lane * 128;
#pragma unroll
            for (int sub = 0; sub < 16; ++sub) {
                const uint32_t cen = min((vd[sub >> 2] >> (8 * (sub & 3))) & 0xFFu, (uint32_t)(p.v_nc - 1));
                const uint4 val = *reinterpret_cast<const uint4 *>(sh_vcb + cen * 8);
                *reinterpret_cast<uint4 *>(vt + (sub >> 3) * 4096 + (((sub & 7) ^ (lane & 7)) << 4)) = val;
            }
            __syncwarp();
        }
        // ---- O^T += V^T . P on the tensor cores ---------------------------------------------
        const uint32_t v_base = st_smem_u32(st + kStV);
#pragma unroll
        for (int mt = 0; mt < 8; ++mt) {
            // 16-byte chunk (8 channels) 2*mt + lm_chunk of the 256-byte row: half (mt / 4), chunk within it
            const uint32_t chunk = (uint32_t)(2 * (mt & 3)) + lm_chunk;
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
                const uint32_t tok = 16u * ks + lm_tok;
                uint32_t a[4];
                st_ldmatrix_x4_trans(a, v_base + (uint32_t)(mt >> 2) * 4096u + tok * 128u + ((chunk ^ (tok & 7u)) << 4));
                st_mma<VBF16>(acc[mt], a, pb[ks][0], pb[ks][1]);
            }
        }
    }
    if (timed_out && lane == 0) atomicExch(&g_coded_timeout, 1);
#pragma unroll
    for (int h = 0; h < NH; ++h) l_run[h] = warp_sum(l_run[h]);

    // ---- merge the warps of this CTA (the stages are drained: reuse them) ----------------------
    __syncthreads();
    float *red_o = reinterpret_cast<float *>(st_raw);  // [warps][heads][D]
    float *red_m = red_o + W * NH * D;
    float *red_l = red_m + W * NH;
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
        const int d0 = 16 * mt + g;
        if constexpr (NH == 4) {  // the high and the low weight column of head c
            red_o[(warp * NH + c) * D + d0] = acc[mt][0] + acc[mt][1];
            red_o[(warp * NH + c) * D + d0 + 8] = acc[mt][2] + acc[mt][3];
        } else {
            red_o[(warp * NH + 2 * c) * D + d0] = acc[mt][0];
            red_o[(warp * NH + 2 * c + 1) * D + d0] = acc[mt][1];
            red_o[(warp * NH + 2 * c) * D + d0 + 8] = acc[mt][2];
            red_o[(warp * NH + 2 * c + 1) * D + d0 + 8] = acc[mt][3];
        }
    }
    if (lane == 0) {
#pragma unroll
        for (int h = 0; h < NH; ++h) { red_m[warp * NH + h] = m_run[h]; red_l[warp * NH + h] = l_run[h]; }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nh * D; i += blockDim.x) {
        const int h = i / D, d = i % D;
        float gm = -INFINITY;
        for (int wq = 0; wq < W; ++wq) gm = fmaxf(gm, red_m[wq * NH + h]);
        float gl = 0.f, o = 0.f;
        for (int wq = 0; wq < W; ++wq) {
            const float mw = red_m[wq * NH + h];
            const float f = (mw == -INFINITY) ? 0.f : __expf(mw - gm);
            gl += red_l[wq * NH + h] * f;
            o += red_o[(wq * NH + h) * D + d] * f;
        }
        const int64_t qrow = ((int64_t)b * p.H_q + hkv * hpk + h0 + h) * p.S_q + sq;
        if (p.n_splits == 1) {
            store_from_f32(p.out, p.out_dtype, qrow * D + d, o / fmaxf(gl, 1e-20f));
        } else {
            p.part_o[(qrow * p.n_splits + split) * D + d] = o;
            if (d == 0) {
                p.part_ml[(qrow * p.n_splits + split) * 2] = gm;
                p.part_ml[(qrow * p.n_splits + split) * 2 + 1] = gl;
            }
        }
    }
}

// Can `p` take the staged kernel? Whole tiles are copied, so the buffers must hold the context
// rounded up to 32 keys, and every copied piece must start on a 16-byte boundary.
bool staged_ok(const CodedParams &p) {
    if (p.D != 128) return false;
    // values: dense 16-bit rows, or (with VQ keys) sixteen one-byte indices into at most 256 centroids of 8
    const bool vq_values = p.key_mode == KEY_VQ && p.v_mode == V_VQ && p.v_index_bytes == 1 && p.v_sub == 8 && p.v_nc <= 256;
    if (!vq_values && (p.v_mode != V_DENSE || (p.v_dtype != VQ_F16 && p.v_dtype != VQ_BF16))) return false;
    if (p.stride_tok % 4 || p.stride_tok < (((int64_t)p.S_kv + 31) & ~(int64_t)31)) return false;
    if (!is_aligned(p.k_codes, 16) || !is_aligned(p.v, 16)) return false;
    if (p.key_mode == KEY_VQ) {
        // sixteen one-byte indices per key, up to 256 centroids of 8, at most four heads per kv head, and
        // enough keys per CTA to pay for the table (a short context takes the plain kernel)
        // (the staged kernel applies no mask: one query row, or several without a causal mask, and no window)
        return p.k_sub == 8 && p.k_index_bytes == 1 && p.k_nc <= 256 && p.H_q / p.H_kv <= 4 && is_aligned(p.k_codebook, 16) &&
               p.window == 0 && (!p.causal || p.S_q == 1) && (int64_t)p.S_kv * p.B * p.H_kv * p.S_q >= (int64_t)1 << 18;
    }
    if (!is_aligned(p.k_mag, 16)) return false;
    if (p.k_const && !is_aligned(p.k_const, 16)) return false;
    return true;
}
constexpr int kVqStWarps = 8;   // warps of the lookup-table form (one CTA per SM)

// Split count for a kernel that keeps `per_sm` CTAs of this kind resident per SM: the count
// that minimises (waves of CTAs) x (keys per CTA + a fixed set-up cost in keys), so that the
// last wave is not mostly idle. `unit` = keys per indivisible piece of a split.
int pick_splits_waves(int requested, int S_kv, int64_t ctas, int sm_count, int per_sm, int unit) {
    if (requested > 0) return std::min(requested, 256);
    const int64_t slots = (int64_t)sm_count * per_sm;
    const int max_splits = (int)std::max<int64_t>(1, std::min<int64_t>(256, ceil_div(S_kv, 8 * unit)));
    int best = 1;
    int64_t best_cost = INT64_MAX;
    for (int n = 1; n <= max_splits; ++n) {
        const int64_t per_cta = ceil_div(ceil_div(S_kv, n), unit) * unit + 96;
        const int64_t cost = ceil_div(ctas * n, slots) * per_cta;
        if (cost < best_cost) { best_cost = cost; best = n; }
    }
    return best;
}

int pick_splits(int requested, int S_kv, int64_t ctas, int sm_count) {
    if (requested > 0) return std::min(requested, 256);
    // About four CTAs per SM (finer splits cost more in set-up and in the merge than they win
    // back in the last wave: measured), at least one 32-key tile per warp.
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
    VQ_REQUIRE(lut_bytes * std::min(hpk, kHeadsC) <= 200 * 1024, VQ_ERR_CAPACITY,
               "%s: lookup tables of %zu bytes per head do not fit shared memory", who, lut_bytes);
    p.heads_per_cta = kHeadsC;
    p.n_head_chunks = (int)ceil_div(hpk, kHeadsC);
    const int64_t gy = (int64_t)p.H_kv * p.S_q * p.n_head_chunks;
    VQ_REQUIRE(gy <= 65535 && p.B <= 65535, VQ_ERR_SHAPE, "%s: grid too large", who);
    p.n_splits = !staged_ok(p)           ? pick_splits(requested_splits, p.S_kv, gy * p.B, di.sm_count)
                 : p.key_mode == KEY_VQ ? pick_splits_waves(requested_splits, p.S_kv, gy * p.B, di.sm_count, 1, 32 * kVqStWarps)
                                        : pick_splits_waves(requested_splits, p.S_kv, gy * p.B, di.sm_count, 4, 32);
    const int64_t rows = (int64_t)p.B * p.H_q * p.S_q;
    if (p.n_splits > 1) {
        const int64_t need = rows * p.n_splits * ((int64_t)p.D + 2) * (int64_t)sizeof(float);
        VQ_REQUIRE(workspace != nullptr && workspace_bytes >= need, VQ_ERR_CAPACITY,
                   "%s: workspace of %lld bytes needed, %lld given", who, (long long)need, (long long)workspace_bytes);
        p.part_o = (float *)workspace;
        p.part_ml = p.part_o + rows * p.n_splits * p.D;
    }
    if (staged_ok(p) && p.key_mode == KEY_VQ) {
        constexpr int Wv = kVqStWarps;
        static_assert((size_t)Wv * kStStages * kStBytes >= ((size_t)Wv * 4 * 128 + 2 * Wv * 4) * sizeof(float), "the warp merge reuses the stages");
        const bool vv = p.v_mode == V_VQ;
        const size_t st_smem = (size_t)Wv * kStStages * kStBytes + 256 + (size_t)Wv * 32 * 4 * 4 + 4 * 128 * 4 + 16 * 256 * 16 + (vv ? 256 * 8 * 2 : 0);
        VQ_REQUIRE(st_smem <= di.smem_optin, VQ_ERR_CAPACITY, "%s: %zu bytes of shared memory needed", who, st_smem);
        dim3 sgrid(p.n_splits, (unsigned)gy, p.B);
        CUtensorMap v_map = {};
        if (vv) {   // coded values: no tensor copies, the value tile is built in shared memory
            VQ_CHECK_CUDA(cudaFuncSetAttribute(rabitq_attend_staged_kernel<false, 4, Wv, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)st_smem));
            rabitq_attend_staged_kernel<false, 4, Wv, 2><<<sgrid, Wv * 32, st_smem, st>>>(p, v_map);
            VQ_CHECK_LAUNCH("staged lookup-table attention kernel");
            if (p.n_splits > 1) return launch_split_merge(p.part_o, p.part_ml, p.n_splits, p.D, p.out, p.out_dtype, rows, st);
            return VQ_OK;
        }
        rc = make_rows_map(3, p.v, 256, p.S_kv, p.stride_tok * 256, p.B * p.H_kv, 128, 32, &v_map);
        if (rc != VQ_OK) return rc;
        if (p.v_dtype == VQ_BF16) {
            VQ_CHECK_CUDA(cudaFuncSetAttribute(rabitq_attend_staged_kernel<true, 4, Wv, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)st_smem));
            rabitq_attend_staged_kernel<true, 4, Wv, 1><<<sgrid, Wv * 32, st_smem, st>>>(p, v_map);
        } else {
            VQ_CHECK_CUDA(cudaFuncSetAttribute(rabitq_attend_staged_kernel<false, 4, Wv, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)st_smem));
            rabitq_attend_staged_kernel<false, 4, Wv, 1><<<sgrid, Wv * 32, st_smem, st>>>(p, v_map);
        }
        VQ_CHECK_LAUNCH("staged lookup-table attention kernel");
        if (p.n_splits > 1) return launch_split_merge(p.part_o, p.part_ml, p.n_splits, p.D, p.out, p.out_dtype, rows, st);
        return VQ_OK;
    }
    if (staged_ok(p)) {
        const int nh_s = hpk <= 4 ? 4 : kHeadsC;
        static_assert((size_t)kStWarps * kStStages * kStBytes >= ((size_t)kStWarps * 8 * 128 + 2 * kStWarps * 8) * sizeof(float),
                      "the warp merge reuses the stages");
        const size_t st_smem = (size_t)kStWarps * kStStages * kStBytes + 256 + (size_t)kStWarps * 32 * nh_s * 4;
        dim3 sgrid(p.n_splits, (unsigned)gy, p.B);
        // the value rows as [batch * kv head][key][256 bytes], boxes of 32 keys x 128 bytes
        CUtensorMap v_map;
        rc = make_rows_map(3, p.v, 256, p.S_kv, p.stride_tok * 256, p.B * p.H_kv, 128, 32, &v_map);
        if (rc != VQ_OK) return rc;
#define VQ_STAGED(BF, NHT)                                                                                      \
    do {                                                                                                        \
        VQ_CHECK_CUDA(cudaFuncSetAttribute(rabitq_attend_staged_kernel<BF, NHT, kStWarps, 0>,                \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)st_smem));         \
        rabitq_attend_staged_kernel<BF, NHT, kStWarps, 0><<<sgrid, kStWarps * 32, st_smem, st>>>(p, v_map); \
    } while (0)
        if (p.v_dtype == VQ_BF16) { if (nh_s == 4) VQ_STAGED(true, 4); else VQ_STAGED(true, 8); }
        else { if (nh_s == 4) VQ_STAGED(false, 4); else VQ_STAGED(false, 8); }
#undef VQ_STAGED
        VQ_CHECK_LAUNCH("rabitq_attend_staged_kernel");
        if (p.n_splits > 1) return launch_split_merge(p.part_o, p.part_ml, p.n_splits, p.D, p.out, p.out_dtype, rows, st);
        return VQ_OK;
    }
    // Specialised value access where the row layout allows vector loads.
    const int dpl = p.D / 32;
    const bool vec_ok = dpl == 2 || dpl == 4 || dpl == 8;
    int vm = VM_GENERIC;
    int vlut_floats = 0;
    if (vec_ok && p.v_mode == V_DENSE && (p.v_dtype == VQ_F16 || p.v_dtype == VQ_BF16) && is_aligned(p.v, 16)) {
        vm = p.v_dtype == VQ_F16 ? VM_F16 : VM_BF16;
    } else if (vec_ok && p.v_mode == V_CENT_NIBBLE && is_aligned(p.v, 4)) {
        vm = VM_NIBBLE;
        vlut_floats = 16;
    } else if (vec_ok && p.v_mode == V_VQ && p.v_index_bytes == 1 && p.v_sub % dpl == 0 &&
               (size_t)p.v_nc * p.v_sub * 4 <= 64 * 1024) {
        vm = VM_VQ8;
        vlut_floats = (p.v_nc * p.v_sub + 3) & ~3;
    }
    const int nh_t = hpk <= 4 ? 4 : kHeadsC;  // heads per CTA the kernel is instantiated for
    const size_t vq_key_bytes = p.key_mode == KEY_VQ ? lut_bytes * std::min(hpk, kHeadsC) + (size_t)nh_t * p.D * 4 : 0;
    const int key_floats = (int)((std::max(vq_key_bytes, (size_t)(nh_t * 9 * 4)) / 4 + 3) & ~(size_t)3);
    const size_t main_bytes = ((size_t)key_floats + vlut_floats + (size_t)kWarpsC * 32 * nh_t) * sizeof(float);
    VQ_REQUIRE(main_bytes <= di.smem_optin, VQ_ERR_CAPACITY, "%s: lookup tables of %zu bytes do not fit shared memory", who, main_bytes);
    const size_t red_bytes = ((size_t)kWarpsC * nh_t * p.D + 2 * kWarpsC * nh_t) * sizeof(float);
    const size_t smem = std::max(red_bytes, main_bytes);
    dim3 grid(p.n_splits, (unsigned)gy, p.B);
#define VQ_CODED_VM_N(DPL, VM, NHT)                                                                             \
    do {                                                                                                   \
        if (smem > 48 * 1024)                                                                              \
            VQ_CHECK_CUDA(cudaFuncSetAttribute(coded_attend_kernel<DPL, VM, NHT>,                                \
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));   \
        coded_attend_kernel<DPL, VM, NHT><<<grid, kWarpsC * 32, smem, st>>>(p, key_floats, vlut_floats);        \
    } while (0)
#define VQ_CODED_VM(DPL, VM)                                                                               \
    do {                                                                                                   \
        if (hpk <= 4) VQ_CODED_VM_N(DPL, VM, 4);                                                           \
        else VQ_CODED_VM_N(DPL, VM, 8);                                                                    \
    } while (0)
#define VQ_CODED_FAST(DPL)                                                                                 \
    case DPL:                                                                                              \
        switch (vm) {                                                                                      \
            case VM_F16: VQ_CODED_VM(DPL, VM_F16); break;                                                  \
            case VM_BF16: VQ_CODED_VM(DPL, VM_BF16); break;                                                \
            case VM_NIBBLE: VQ_CODED_VM(DPL, VM_NIBBLE); break;                                            \
            case VM_VQ8: VQ_CODED_VM(DPL, VM_VQ8); break;                                                  \
            default: VQ_CODED_VM(DPL, VM_GENERIC); break;                                                  \
        }                                                                                                  \
        break;
#define VQ_CODED_GEN(DPL) case DPL: VQ_CODED_VM(DPL, VM_GENERIC); break;
    // small grids (at most two CTAs per SM), head_dim 128, dense 16-bit values, up to four heads per kv head: the eager form
    if (gy * p.B * p.n_splits <= 2 * (int64_t)di.sm_count && dpl == 4 && hpk <= 4 && (vm == VM_F16 || vm == VM_BF16)) {
        if (smem > 48 * 1024) {
            VQ_CHECK_CUDA(cudaFuncSetAttribute(coded_attend_kernel<4, VM_F16, 4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            VQ_CHECK_CUDA(cudaFuncSetAttribute(coded_attend_kernel<4, VM_BF16, 4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        }
        if (vm == VM_F16) coded_attend_kernel<4, VM_F16, 4, true><<<grid, kWarpsC * 32, smem, st>>>(p, key_floats, vlut_floats);
        else coded_attend_kernel<4, VM_BF16, 4, true><<<grid, kWarpsC * 32, smem, st>>>(p, key_floats, vlut_floats);
        VQ_CHECK_LAUNCH("coded_attend_kernel");
        if (p.n_splits > 1) return launch_split_merge(p.part_o, p.part_ml, p.n_splits, p.D, p.out, p.out_dtype, rows, st);
        return VQ_OK;
    }
    switch (dpl) {
        VQ_CODED_GEN(1) VQ_CODED_FAST(2) VQ_CODED_GEN(3) VQ_CODED_FAST(4) VQ_CODED_GEN(5) VQ_CODED_GEN(6)
        VQ_CODED_GEN(7) VQ_CODED_FAST(8)
        default: return fail(VQ_ERR_SHAPE, "%s: unsupported head_dim %d", who, p.D);
    }
#undef VQ_CODED_GEN
#undef VQ_CODED_FAST
#undef VQ_CODED_VM
#undef VQ_CODED_VM_N
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

int32_t coded_attend_take_timeout(int *flag) {
    int zero = 0;
    VQ_CHECK_CUDA(cudaMemcpyFromSymbol(flag, g_coded_timeout, sizeof(int)));
    if (*flag) VQ_CHECK_CUDA(cudaMemcpyToSymbol(g_coded_timeout, &zero, sizeof(int)));
    return VQ_OK;
}

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
