// Tiled attention of many query rows over sign-bit keys (RaBitQ): the matmul-shaped companion
// of the decode kernel, for prompt chunks and multi-turn prefill.
//
// Score model (the reference's, metal/_rabitq_prefill.py:16-21): an exact dot with the decoded
// key, k_hat[j] = signs(k_bits[j]) * k_mag[j]:
//     score[i][j] = (q[i] . k_hat[j]) * scale + k_const[j]
// softmax over the slots (all, or with the tail-aligned causal mask: query row r of S_q sits at
// slot S_kv - S_q + r), then the weighted sum of the values: nibble-packed indices into a
// <= 16-entry scalar codebook (the reference form) or a dense f16/bf16 tensor.
//
// Mapping: both products run on the tensor cores as m16n8k16 f16 MMAs with float32
// accumulation. Signs are +-1, so k_mag[j] * scale is taken out of the dot and applied to the
// float32 score; the B operand of Q.K^T is built straight from the packed bits (two +-1.0
// halves per register: 0xBC00BC00 with the two sign bits flipped in), no decoded key tile ever
// exists. The softmax weights leave the score accumulators as the A operand of P.V (the usual
// register reuse); V tiles are staged once per CTA in shared memory as halves (nibbles decoded
// there) and read with transposing ldmatrix. The query rows of all query heads that share a KV
// head are stacked into one row axis (row = head * S_q + position), so a KV tile is decoded
// once for the whole group. One CTA = 4 warps x 16 rows; it walks the KV slots in tiles of 32.
#include <algorithm>

#include "common.cuh"

namespace vq {
namespace {

constexpr int kPfWarps = 4;
constexpr int kPfRows = 16 * kPfWarps;  // query rows per CTA
constexpr int kPfTile = 32;             // KV slots per tile
constexpr int kVPad = 8;                // halves of padding per staged V row (keeps ldmatrix rows on distinct banks)

struct PrefillParams {
    vq_rabitq_prefill_args a;
    int hpk;      // query heads per kv head
    int n_rows;   // hpk * S_q
};

__device__ __forceinline__ void pf_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pf_pack(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
// Two consecutive sign bits (bit p and p+1 of w) as a pair of halves: 1 -> +1.0, 0 -> -1.0.
__device__ __forceinline__ uint32_t sign_pair(uint32_t w, int p) {
    const uint32_t x = w >> p;
    return 0xBC00BC00u ^ ((x & 1u) << 15) ^ ((x & 2u) << 30);
}

template <int D>
__global__ void __launch_bounds__(kPfWarps * 32)
rabitq_prefill_kernel(const __grid_constant__ PrefillParams p) {
    constexpr int KB = D / 16;           // k-blocks of the Q.K^T product
    constexpr int NB = D / 8;            // 8-channel blocks of the output
    constexpr int VROW = D + kVPad;      // halves per staged V row
    __shared__ __align__(16) uint8_t sh_bits[kPfTile * (D / 8)];
    __shared__ float sh_mag[kPfTile], sh_const[kPfTile];
    __shared__ __align__(16) __half sh_v[kPfTile * VROW];
    __shared__ float sh_cents[16];

    const vq_rabitq_prefill_args &a = p.a;
    const int b = blockIdx.z, hkv = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, c = lane & 3;
    const int row0 = blockIdx.x * kPfRows + warp * 16;  // first row of this warp
    const int64_t bh = (int64_t)b * a.H_kv + hkv;
    const int q_align = a.S_kv - a.S_q;

    if (tid < 16) sh_cents[tid] = (a.v_mode == 3 && tid < a.n_cents) ? a.v_cents[tid] : 0.f;

    // ---- this warp's 16 query rows as A fragments (kept in registers for the whole kernel) ----
    // fragment kb: a0 = (row g, k 2c..2c+1), a1 = (row g+8, same k), a2 = (row g, k 2c+8..9), a3 = (row g+8, ...)
    uint32_t qa[KB][4];
    int q_abs[2];  // slot index at which rows g / g+8 sit (for the causal mask)
    bool live[2];
    int64_t out_off[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = row0 + g + 8 * r;
        live[r] = row < p.n_rows;
        const int hp = live[r] ? row / a.S_q : 0, pos = live[r] ? row % a.S_q : 0;
        q_abs[r] = q_align + pos;
        out_off[r] = ((((int64_t)b * a.H_q + hkv * p.hpk + hp) * a.S_q) + pos) * D;
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int d = kb * 16 + 2 * c + 8 * hf;
                const float x0 = live[r] ? load_as_f32(a.q, a.q_dtype, out_off[r] + d) : 0.f;
                const float x1 = live[r] ? load_as_f32(a.q, a.q_dtype, out_off[r] + d + 1) : 0.f;
                qa[kb][r + 2 * hf] = pf_pack(x0, x1);
            }
        }
    }

    float o[NB][4];
#pragma unroll
    for (int i = 0; i < NB; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float sc_log2 = a.scale * 1.4426950408889634f;  // scores kept in the log2 domain

    // slots any row of this CTA may see
    int kv_hi = a.S_kv;
    if (a.causal) {
        const int first = blockIdx.x * kPfRows, last = min(p.n_rows, first + kPfRows) - 1;
        const int max_pos = (first / a.S_q != last / a.S_q) ? a.S_q - 1 : last % a.S_q;
        kv_hi = min(a.S_kv, q_align + max_pos + 1);
    }

    for (int t0 = 0; t0 < kv_hi; t0 += kPfTile) {
        __syncthreads();  // the previous tile is consumed
        // ---- stage the tile: sign bits, magnitudes, constants, values as halves ----
        for (int i = tid; i < kPfTile * (D / 8) / 4; i += blockDim.x) {
            const int key = i / (D / 32), w = i % (D / 32);
            const int slot = t0 + key;
            uint32_t v = 0;
            if (slot < a.S_kv) v = reinterpret_cast<const uint32_t *>(a.k_bits + (bh * a.kv_stride_tok + slot) * (D / 8))[w];
            reinterpret_cast<uint32_t *>(sh_bits)[i] = v;
        }
        if (tid < kPfTile) {
            const int slot = t0 + tid;
            sh_mag[tid] = slot < a.S_kv ? a.k_mag[bh * a.kv_stride_tok + slot] * sc_log2 : 0.f;
            sh_const[tid] = (slot < a.S_kv && a.k_const) ? a.k_const[bh * a.kv_stride_tok + slot] * 1.4426950408889634f : 0.f;
        }
        if (a.v_mode == 3) {  // nibble-packed codebook indices: one byte -> two channels
            for (int i = tid; i < kPfTile * (D / 2); i += blockDim.x) {
                const int key = i / (D / 2), j = i % (D / 2);
                const int slot = t0 + key;
                float lo = 0.f, hi = 0.f;
                if (slot < a.S_kv) {
                    const uint32_t byte = static_cast<const uint8_t *>(a.v)[(bh * a.kv_stride_tok + slot) * (D / 2) + j];
                    lo = sh_cents[byte & 15u];
                    hi = sh_cents[byte >> 4];
                }
                *reinterpret_cast<__half2 *>(sh_v + key * VROW + 2 * j) = __floats2half2_rn(lo, hi);
            }
        } else {  // dense f16 / bf16 rows: 8 elements per thread and step
            for (int i = tid; i < kPfTile * (D / 8); i += blockDim.x) {
                const int key = i / (D / 8), j = i % (D / 8);
                const int slot = t0 + key;
                uint4 raw = make_uint4(0, 0, 0, 0);
                if (slot < a.S_kv) raw = reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(a.v) + (bh * a.kv_stride_tok + slot) * D)[j];
                if (a.v_dtype == VQ_BF16) {
                    uint32_t *wd = reinterpret_cast<uint32_t *>(&raw);
#pragma unroll
                    for (int u = 0; u < 4; ++u) wd[u] = pf_pack(__uint_as_float(wd[u] << 16), __uint_as_float(wd[u] & 0xffff0000u));
                }
                *reinterpret_cast<uint4 *>(sh_v + key * VROW + 8 * j) = raw;
            }
        }
        __syncthreads();

        // ---- S = Q . signs^T for the tile's 4 blocks of 8 slots ----
        float s[kPfTile / 8][4];
#pragma unroll
        for (int nb = 0; nb < kPfTile / 8; ++nb) {
            s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
            const uint32_t *kw = reinterpret_cast<const uint32_t *>(sh_bits + (nb * 8 + g) * (D / 8));  // slot nb*8 + g
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                const uint32_t w = kw[kb >> 1] >> (16 * (kb & 1));  // the 16 sign bits of dims kb*16 .. kb*16+15
                pf_mma(s[nb], qa[kb][0], qa[kb][1], qa[kb][2], qa[kb][3], sign_pair(w, 2 * c), sign_pair(w, 2 * c + 8));
            }
        }
        // ---- scale, bias, mask; online softmax for rows g and g+8 ----
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nb = 0; nb < kPfTile / 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = nb * 8 + 2 * c + (e & 1), r = e >> 1;
                const int slot = t0 + key;
                const bool ok = slot < a.S_kv && (!a.causal || slot <= q_abs[r]);
                s[nb][e] = ok ? fmaf(s[nb][e], sh_mag[key], sh_const[key]) : -INFINITY;
                tmax[r] = fmaxf(tmax[r], s[nb][e]);
            }
        }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
            tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
            const float mn = fmaxf(m_run[r], tmax[r]);
            corr[r] = (mn == -INFINITY) ? 1.f : exp2f(m_run[r] - mn);  // (a tile may be fully masked for a row)
            m_run[r] = mn;
        }
        float tsum[2] = {0.f, 0.f};
#pragma unroll
        for (int nb = 0; nb < kPfTile / 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = e >> 1;
                const float w = (m_run[r] == -INFINITY) ? 0.f : exp2f(s[nb][e] - m_run[r]);
                s[nb][e] = w;
                tsum[r] += w;
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * corr[r] + tsum[r];  // (lane-partial sums: reduced at the end)
#pragma unroll
        for (int i = 0; i < NB; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[0];
            o[i][2] *= corr[1]; o[i][3] *= corr[1];
        }
        // ---- O += P . V: the weights of slot blocks (2j, 2j+1) are the A fragment of k-block j ----
#pragma unroll
        for (int j = 0; j < kPfTile / 16; ++j) {
            const uint32_t a0 = pf_pack(s[2 * j][0], s[2 * j][1]), a1 = pf_pack(s[2 * j][2], s[2 * j][3]);
            const uint32_t a2 = pf_pack(s[2 * j + 1][0], s[2 * j + 1][1]), a3 = pf_pack(s[2 * j + 1][2], s[2 * j + 1][3]);
            // B fragment of channel block i: rows = slots 16j .. 16j+15, columns = channels 8i .. 8i+7;
            // one transposing ldmatrix.x4 fetches two channel blocks
#pragma unroll
            for (int i = 0; i < NB; i += 2) {
                const int m = lane >> 3, rr = lane & 7;  // matrix m: slots 16j + 8*(m&1) + rr, channels 8*(i + (m>>1))
                const uint32_t addr = (uint32_t)__cvta_generic_to_shared(sh_v + (16 * j + 8 * (m & 1) + rr) * VROW + 8 * (i + (m >> 1)));
                uint32_t v0, v1, v2, v3;
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3) : "r"(addr));
                pf_mma(o[i], a0, a1, a2, a3, v0, v1);
                pf_mma(o[i + 1], a0, a1, a2, a3, v2, v3);
            }
        }
    }

    // ---- normalise and store ----
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        if (!live[r]) continue;
        const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
#pragma unroll
        for (int i = 0; i < NB; ++i) {
            const int d = 8 * i + 2 * c;
            store_from_f32(a.out, a.out_dtype, out_off[r] + d, o[i][2 * r] * inv);
            store_from_f32(a.out, a.out_dtype, out_off[r] + d + 1, o[i][2 * r + 1] * inv);
        }
    }
}

}  // namespace
}  // namespace vq

extern "C" int32_t vq_rabitq_prefill_attend(const vq_rabitq_prefill_args *args, void *stream) {
    using namespace vq;
    const char *fn = "rabitq_prefill_attend";
    VQ_REQUIRE(args != nullptr, VQ_ERR_SHAPE, "%s: args is NULL", fn);
    const vq_rabitq_prefill_args &a = *args;
    DeviceInfo di;
    int32_t rc = device_info(&di);
    if (rc != VQ_OK) return rc;
    VQ_REQUIRE(a.B >= 1 && a.H_q >= 1 && a.H_kv >= 1 && a.S_q >= 1 && a.S_kv >= 1, VQ_ERR_SHAPE, "%s: sizes must be >= 1", fn);
    VQ_REQUIRE(a.H_q % a.H_kv == 0, VQ_ERR_SHAPE, "%s: H_q=%d must be a multiple of H_kv=%d", fn, a.H_q, a.H_kv);
    VQ_REQUIRE(a.D == 64 || a.D == 128, VQ_ERR_SHAPE, "%s: D=%d must be 64 or 128", fn, a.D);
    VQ_REQUIRE(!a.causal || a.S_q <= a.S_kv, VQ_ERR_SHAPE, "%s: causal mask with S_q=%d query rows over %d slots", fn, a.S_q, a.S_kv);
    VQ_REQUIRE(a.kv_stride_tok >= a.S_kv, VQ_ERR_SHAPE, "%s: kv_stride_tok=%lld is smaller than S_kv=%d", fn, (long long)a.kv_stride_tok, a.S_kv);
    VQ_REQUIRE(a.q && a.out && a.k_bits && a.k_mag && a.v, VQ_ERR_SHAPE, "%s: NULL argument", fn);
    VQ_REQUIRE(a.q_dtype >= 0 && a.q_dtype <= 2 && a.out_dtype >= 0 && a.out_dtype <= 2, VQ_ERR_DTYPE, "%s: bad q/out dtype", fn);
    VQ_REQUIRE(a.v_mode == 0 || a.v_mode == 3, VQ_ERR_SHAPE, "%s: v_mode must be 0 (dense) or 3 (nibble-packed)", fn);
    if (a.v_mode == 0)
        VQ_REQUIRE((a.v_dtype == VQ_F16 || a.v_dtype == VQ_BF16) && is_aligned(a.v, 16), VQ_ERR_DTYPE,
                   "%s: dense values must be f16 or bf16 and 16-byte aligned", fn);
    else
        VQ_REQUIRE(a.v_cents && a.n_cents >= 1 && a.n_cents <= 16, VQ_ERR_SHAPE, "%s: v_cents must hold 1..16 entries", fn);
    VQ_REQUIRE(is_aligned(a.k_bits, 4), VQ_ERR_ALIGN, "%s: k_bits must be 4-byte aligned", fn);
    PrefillParams p;
    p.a = a;
    p.hpk = a.H_q / a.H_kv;
    p.n_rows = p.hpk * a.S_q;
    const int64_t gx = ceil_div(p.n_rows, kPfRows);
    VQ_REQUIRE(gx < (1ll << 31) && a.H_kv <= 65535 && a.B <= 65535, VQ_ERR_SHAPE, "%s: grid too large", fn);
    dim3 grid((unsigned)gx, a.H_kv, a.B);
    if (a.D == 128) rabitq_prefill_kernel<128><<<grid, kPfWarps * 32, 0, (cudaStream_t)stream>>>(p);
    else rabitq_prefill_kernel<64><<<grid, kPfWarps * 32, 0, (cudaStream_t)stream>>>(p);
    VQ_CHECK_LAUNCH("rabitq_prefill_kernel");
    return VQ_OK;
}
