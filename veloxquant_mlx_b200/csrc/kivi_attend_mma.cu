// Fused dequant + single-query attention over packed 2-/4-bit KIVI codes for the serving
// shape (head_dim 128, group 32, one query row, <= 8 query heads per KV head).
//
// Why tensor cores: with the query heads of one KV head packed together, every KV token
// costs 2*128*heads multiply-adds; at B200's HBM rate that is several times what the FP32
// pipes sustain, so QK^T and PV run as m16n8k16 f16 MMAs with the KV tokens (QK^T) and the
// head_dim rows (PV) on the M axis and the packed query heads on the 8-wide N axis.
//
// Exactness: the A operands are the RAW integer codes, produced in registers from the
// packed words by one AND each (see unpack_word: exact halves, no int->float conversion).
// The group scales never touch the codes in half precision; they are folded, in float32,
// into the small B operands instead:
//     q.K_hat[t]  = sum_d code[t,d] * (q[d]*k_scale[G,d])  +  sum_d q[d]*k_zero[G,d]
//     P.V_hat[:,d] = sum_t code[t,d] * (P[t]*v_scale[t,g(d)]) + sum_t P[t]*v_zero[t,g(d)]
// and each float32 B value is split into a high and a low half (x = hi + lo) that occupy
// the 4 + 4 columns of the N = 8 tile, so products are exact and sums are float32. The two
// zero-point terms are plain float32 FMAs. Up to 4 query heads fit one CTA this way; a KV
// head with 5..8 query heads is covered by two CTAs (the second read hits L2).
// Warp-level MMAs are used (not tcgen05) because the A operand is born in registers.
//
// Data movement: each warp owns a contiguous run of 32-token groups of one (batch, kv head).
// Per group six contiguous pieces (K codes, V codes, K scale/zero, V scale/zero) are fetched
// by the bulk async-copy engine (completion on an mbarrier) into the warp's own 2- to 4-stage
// shared-memory ring, so HBM reads stay in flight while the warp unpacks. Five pieces are
// linear copies (cp.async.bulk). The V codes go through a tensor map (cp.async.bulk.tensor)
// that views the packed rows as 128-byte lines and stores them with the 128-byte swizzle: the
// transposing ldmatrix reads of V (8 token rows, one 16-byte segment each) then fall on 8
// different bank groups instead of 2 (rows are only 64 or 32 bytes apart), which took a
// quarter of the kernel's shared-memory wavefronts away.
// The context is split across CTAs; each writes an unnormalised partial (m, l, o) and takes a
// ticket; the CTA that takes a unit's last ticket merges the unit's partials and writes the
// output rows (and, in a sharded run, publishes them to the peers). The unquantized tail
// (residual window) is spread over all warps of all of a unit's CTAs, a few rows each, after
// their packed groups. One launch per call: nothing of a call sits resident and blocked, so a
// call launched with VQ_ATTEND_OVERLAP_PREVIOUS streams in behind the previous one without
// displacing its CTAs (this kernel takes the whole register file at 4 CTAs per SM).
#include <cuda.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <random>
#include <type_traits>

#include "kivi_attend.h"

namespace vq {

namespace {

constexpr int kD = 128;
constexpr int kGroup = 32;     // tokens per pipeline stage of one warp = one K scale group
constexpr int kWarps = 4;
constexpr int kMaxHeads = 8;   // query heads per kv head
constexpr int kChunkHeads = 4; // query heads per CTA (hi/lo halves fill the 8 MMA columns)
constexpr uint32_t kSpinLimit = 1u << 18;
constexpr uint32_t kSelfTestSpinLimit = 1u << 10;

__device__ int g_attend_timeout = 0;

template <int BITS>
struct Cfg {
    static constexpr int RB = kD * BITS / 8;     // bytes per packed row: 64 / 32
    static constexpr int CPW = 32 / BITS;        // codes per 32-bit word: 8 / 16
    static constexpr int NH = CPW / 2;           // half2 registers per unpacked word: 4 / 8
    static constexpr int KW = 32 / CPW;          // words of one thread's 32-channel K chunk: 4 / 2
    static constexpr int CU = 16 / BITS;         // codes per 16-bit unit: 4 / 8
    static constexpr int NSEG = RB / 16;         // 16-byte segments per row: 4 / 2
    static constexpr int KC_OFF = 0;
    static constexpr int VC_OFF = kGroup * RB;
    // (K scale and K zero tiles are swizzled and start on 1024-byte boundaries: same offsets in both)
    static constexpr int KS_OFF = 2 * kGroup * RB;
    static constexpr int VS_OFF = KS_OFF + 512;
    static constexpr int KZ_OFF = VS_OFF + 512;
    static constexpr int VZ_OFF = KZ_OFF + 512;
    static constexpr int STAGE_BYTES = VZ_OFF + 512;  // one warp, one stage: 6144 / 4096
    static constexpr int VROWS = kGroup * RB / 128;   // 128-byte lines of one group's V codes: 16 / 8
    // stages first (1024-byte aligned, as the swizzle pattern repeats every 1024 bytes), barriers after
    static constexpr int smem_bytes(int stages) { return kWarps * stages * STAGE_BYTES + 256; }
};

// ---- PTX helpers ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait: returns false (and the caller records a timeout) instead of spinning forever.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit = kSpinLimit) {
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
// Tiled copy of one box of a rank-3 tensor map (x: bytes within a 128-byte line, always 0 here;
// y: line; z: (batch, kv head)).
__device__ __forceinline__ void tensor_g2s(uint32_t dst, const CUtensorMap *map, int x, int y, int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}
// Byte offset inside a 128-byte-swizzled tile (tile base 1024-byte aligned) of linear offset `lin`:
// the 16-byte chunk index (bits 4-6) is XORed with the line index modulo 8 (bits 7-9).
__device__ __forceinline__ uint32_t swz128(uint32_t lin) { return lin ^ (((lin >> 7) & 7u) << 4); }
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ float2 unpack_h2(uint32_t v) {
    return __half22float2(*reinterpret_cast<__half2 *>(&v));
}
// x = hi + lo with hi = half(x), lo = half(x - hi): ~22 significant bits in two halves.
__device__ __forceinline__ void split_h2(float x0, float x1, uint32_t &hi, uint32_t &lo) {
    hi = pack_h2(x0, x1);
    const float2 h = unpack_h2(hi);
    lo = pack_h2(x0 - h.x, x1 - h.y);
}
// (hi, lo) halves of one value in one register = the column pair (2c, 2c+1): hi is x truncated
// to 11 significant bits (one AND; exactly a half in the normal range), lo = half(x - hi), so
// x = hi + lo holds to the half precision of lo (~22 significant bits).
__device__ __forceinline__ uint32_t split_pack_trunc(float x) {
    const float h = __uint_as_float(__float_as_uint(x) & 0xffffe000u);
    return pack_h2(h, x - h);
}
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(a));
    return r;
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

// Unpack one 32-bit word into half2 registers by masking alone. A half whose bit pattern is
// below 2048 (exponent field 0 or 1) has the value pattern * 2^-24: the subnormal range and
// the first normal binade lie on one straight line. So a code left in place at bit offset s
// of a 16-bit half IS the half-precision number code * 2^s * 2^-24, exactly, with no
// conversion and no magic-number subtract; the tensor cores take subnormal inputs as they
// are. Register i pairs the i-th code of the low 16 bits with the i-th code of the high 16
// bits; code_weight<BITS>(i) = 2^s is folded into the other MMA operand or the final scale.
template <int BITS>
__device__ __forceinline__ void unpack_word(uint32_t w, uint32_t (&h)[32 / BITS / 2]);

template <>
__device__ __forceinline__ void unpack_word<4>(uint32_t w, uint32_t (&h)[4]) {
    const uint32_t w8 = w >> 8;
    h[0] = w & 0x000f000fu;
    h[1] = w & 0x00f000f0u;
    h[2] = w8 & 0x000f000fu;
    h[3] = w8 & 0x00f000f0u;
}
template <>
__device__ __forceinline__ void unpack_word<2>(uint32_t w, uint32_t (&h)[8]) {
    const uint32_t w8 = w >> 8;
    h[0] = w & 0x00030003u;
    h[1] = w & 0x000c000cu;
    h[2] = w & 0x00300030u;
    h[3] = w & 0x00c000c0u;
    h[4] = w8 & 0x00030003u;
    h[5] = w8 & 0x000c000cu;
    h[6] = w8 & 0x00300030u;
    h[7] = w8 & 0x00c000c0u;
}
// 2^s of unpacked register i (depends only on i modulo 4 in both widths).
template <int BITS>
__host__ __device__ constexpr float code_weight(int i) {
    return BITS == 4 ? ((i & 1) ? 16.f : 1.f) : (float)(1 << (2 * (i & 3)));
}
constexpr float kTwo24 = 16777216.f;

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct Params {
    alignas(64) CUtensorMap v_map;   // V codes as [batch*kv head][lines of 128 bytes][128], swizzled boxes of one group
    alignas(64) CUtensorMap ks_map;  // K scales as [batch*kv head][4 lines per group][32 floats], swizzled boxes of one group
    alignas(64) CUtensorMap kz_map;  // K zeros, likewise
    vq_kivi_attend_args a;
    int hpk;
    int n_chunks;       // ceil(hpk / 4)
    int n_splits;       // context splits = partial records per (batch, kv head, query head)
    int groups_total;     // n_quant / 32
    int groups_per_warp;  // consecutive groups owned by one warp
    float *part_o;      // [B*H_kv][n_splits][hpk][128]
    float *part_ml;     // [B*H_kv][n_splits][hpk][2]
    unsigned long long *tickets;  // [B*H_kv][n_chunks]: (epoch << 16) | arrivals of the current call
    unsigned long long epoch;     // 48 bits that tell this call's tickets from whatever the workspace held before
    int wait_test;      // self-test: every warp also waits (briefly) on a barrier that nothing arms
    vq_peer_gather gather;  // world == 0: the output rows are not published to peers
    vq_kivi_sinks sinks;    // count == nullptr: no protected tokens
    int wide;               // eight query heads per CTA (kivi_attend_mma8_kernel) instead of four
};

// ---- helpers for the unquantized tail ----------------------------------------------------------
// Four consecutive elements of a residual row (dtype known at run time) as float32.
__device__ __forceinline__ void load_res4(const void *base, int32_t dt, int64_t elem, float (&d)[4]) {
    if (dt == VQ_F32) {
        const float4 v = *reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(base) + elem);
        d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
    } else {
        const uint2 raw = *reinterpret_cast<const uint2 *>(reinterpret_cast<const uint16_t *>(base) + elem);
        if (dt == VQ_F16) {
            const float2 lo = __half22float2(*reinterpret_cast<const __half2 *>(&raw.x));
            const float2 hi = __half22float2(*reinterpret_cast<const __half2 *>(&raw.y));
            d[0] = lo.x; d[1] = lo.y; d[2] = hi.x; d[3] = hi.y;
        } else {
            d[0] = __uint_as_float(raw.x << 16); d[1] = __uint_as_float(raw.x & 0xffff0000u);
            d[2] = __uint_as_float(raw.y << 16); d[3] = __uint_as_float(raw.y & 0xffff0000u);
        }
    }
}
// Four consecutive output elements of a row, in the output dtype.
__device__ __forceinline__ void store_out4(void *base, int32_t dt, int64_t elem, const float (&v)[4]) {
    if (dt == VQ_F32) {
        *reinterpret_cast<float4 *>(reinterpret_cast<float *>(base) + elem) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
        uint2 raw;
        if (dt == VQ_F16) {
            raw.x = pack_h2(v[0], v[1]);
            raw.y = pack_h2(v[2], v[3]);
        } else {
            const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
            raw.x = *reinterpret_cast<const uint32_t *>(&lo);
            raw.y = *reinterpret_cast<const uint32_t *>(&hi);
        }
        *reinterpret_cast<uint2 *>(reinterpret_cast<uint16_t *>(base) + elem) = raw;
    }
}

// The end of a CTA's work, after its partial record is written: take a ticket for the (batch, kv
// head, head chunk); the CTA that takes the last one merges the unit's partials, writes the
// output rows and, in a sharded run, publishes them. CH = query heads per CTA.
template <int CH>
__device__ __forceinline__ void ticket_merge_publish(const Params &p, uint64_t *bars, int64_t bh, int b, int hkv, int h0,
                                                     int hpk, int n_heads, int tid, int lane, int warp) {
    const vq_kivi_attend_args &a = p.a;
    // ---- ticket: the CTA that arrives last for this (batch, kv head, head chunk) merges ----------
    // The ticket word is (epoch << 16) | arrivals. Whatever the workspace held before this call
    // (another call's partials, a fresh allocation's old contents) has other upper 48 bits and
    // counts as zero arrivals: the epoch is a per-call 48-bit hash, so stray data matches it with
    // probability 2^-48. The merging CTA leaves 0 behind (epoch 0 is never issued), so in a steady
    // decode loop every ticket is found at 0, and a captured launch can be replayed with its epoch.
    int *sh_last = reinterpret_cast<int *>(bars) + 48;  // (behind the barriers, inside their 256 bytes)
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        unsigned long long *t = p.tickets + bh * p.n_chunks + (h0 / CH);
        unsigned long long cur = *reinterpret_cast<volatile unsigned long long *>(t), want;
        for (;;) {
            want = ((cur >> 16) == p.epoch) ? cur + 1ull : ((p.epoch << 16) | 1ull);
            const unsigned long long seen = atomicCAS(t, cur, want);
            if (seen == cur) break;
            cur = seen;  // (another CTA of this unit got in between: at most n_splits - 1 retries)
        }
        *sh_last = ((uint32_t)(want & 0xffffull) == (uint32_t)p.n_splits);
    }
    __syncthreads();
    if (!*sh_last) return;
    __threadfence();
    // Warp w merges query heads h0 + w, h0 + w + 4, ...: lane holds channels 4*lane .. 4*lane+3; the (max, sum) pair
    // of a part is one broadcast load. Loads bypass L1 (the partials were written by other SMs).
    for (int hw = warp; hw < n_heads; hw += kWarps) {
        const int64_t rec0 = bh * p.n_splits * hpk + h0 + hw;  // record of part s: rec0 + s * hpk
        float m = -INFINITY, l = 0.f, acc[4] = {0.f, 0.f, 0.f, 0.f};
        constexpr int kBatch = 8;
        for (int s0 = 0; s0 < p.n_splits; s0 += kBatch) {
            float2 ml[kBatch];
            float4 po[kBatch];
#pragma unroll
            for (int j = 0; j < kBatch; ++j) {
                const int s = min(s0 + j, p.n_splits - 1);
                const int64_t rec = rec0 + (int64_t)s * hpk;
                ml[j] = __ldcg(reinterpret_cast<const float2 *>(p.part_ml + rec * 2));
                po[j] = __ldcg(reinterpret_cast<const float4 *>(p.part_o + rec * kD + 4 * lane));
            }
#pragma unroll
            for (int j = 0; j < kBatch; ++j) {
                if (s0 + j < p.n_splits && ml[j].x != -INFINITY) {
                    const float mn = fmaxf(m, ml[j].x);
                    const float f = exp2f(m - mn), wgt = exp2f(ml[j].x - mn);
                    l = l * f + ml[j].y * wgt;
                    acc[0] = acc[0] * f + po[j].x * wgt; acc[1] = acc[1] * f + po[j].y * wgt;
                    acc[2] = acc[2] * f + po[j].z * wgt; acc[3] = acc[3] * f + po[j].w * wgt;
                    m = mn;
                }
            }
        }
        const float inv = 1.f / l;
        const float res[4] = {acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv};
        const int64_t row = (int64_t)b * a.H_q + hkv * hpk + h0 + hw;
        store_out4(a.out, a.out_dtype, row * kD + 4 * lane, res);
        if (p.gather.world > 0) {
            // publish the row to every rank's gathered tensor (plain stores to peer-mapped memory)
            const int64_t grow = p.gather.row_offset + row;
            for (int pr = 0; pr < p.gather.world; ++pr) store_out4(p.gather.out[pr], a.out_dtype, grow * kD + 4 * lane, res);
        }
    }
    if (p.gather.world > 0) {
        // Arrival: once the CTA's rows are stored, thread r fences system-wide (the barrier puts
        // every thread's stores before that fence) and adds 1 to this rank's word on rank r. One
        // fence latency per layer; the waiting side knows how many four-head chunks each rank sends per round.
        // (Counting the CTAs locally first and raising a flag from the last one cost a second fence;
        // a release store per rank cost one fence each: 22 us per layer at 8 ranks.)
        const vq_peer_gather &pg = p.gather;
        __syncthreads();
        if (tid < pg.world) {
            __threadfence_system();
            // (a CTA of the eight-head kernel counts as the four-head CTAs it stands for, so the count a
            // waiting rank expects does not depend on which kernel the sender's launch picked)
            asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(pg.flags[tid] + pg.rank),
                         "r"((uint32_t)(n_heads + kChunkHeads - 1) / kChunkHeads) : "memory");
        }
    }
    if (tid == 0) p.tickets[bh * p.n_chunks + (h0 / CH)] = 0ull;
}

// ---- main kernel ----------------------------------------------------------------------------
// Lane roles (g = lane / 4, c = lane % 4):
//   as a B-operand column (n = g): query head g / 2, high half if g is even, low half otherwise;
//   as an accumulator column pair (cols 2c, 2c+1): the high and the low half of head c, so
//   a lane adds its two columns and owns ONE head for its rows: no exchange between lanes for
//   the hi + lo sums, and the softmax of a head is computed once (by the 8 lanes g of column c).
// SINKS: the call carries protected tokens (extra tail rows); a separate instantiation so that
// the plain kernel's register allocation (at the limit of four CTAs per SM) is not touched.
template <int BITS, int STAGES, bool SINKS>
__global__ void __launch_bounds__(kWarps * 32, 4)
kivi_attend_mma_kernel(const __grid_constant__ Params p) {
    using C = Cfg<BITS>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const vq_kivi_attend_args &a = p.a;
    const int b = blockIdx.z, hkv = blockIdx.y;
    // whatever follows on the stream (the next call, launched as a programmatic dependent) may be
    // made resident as soon as every CTA of this grid has started
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int split = blockIdx.x / p.n_chunks;
    const int h0 = (blockIdx.x % p.n_chunks) * kChunkHeads;  // first head of this CTA's chunk
    const int tid = threadIdx.x, lane = tid & 31;
    // (read through a shuffle so that the compiler knows the warp index is the same in all lanes:
    // the pipeline's addresses, barriers and loop counters then live in uniform registers)
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int g = lane >> 2, c = lane & 3;
    const int hd = g >> 1, half_id = g & 1;
    const int hpk = p.hpk;
    const int64_t bh = (int64_t)b * a.H_kv + hkv;

    uint8_t *stages = smem_raw;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw + kWarps * STAGES * C::STAGE_BYTES);
    const uint32_t bar0 = smem_u32(bars);
    if (smem_u32(stages) & 1023u) {  // the swizzled addressing below assumes this; never seen
        if (tid == 0) atomicExch(&g_attend_timeout, 2);
        return;
    }

    // Each warp owns a contiguous run of 32-token groups and runs its own copy pipeline:
    // no CTA-wide synchronisation until the final merge.
    const int grp_begin = min(p.groups_total, (split * kWarps + warp) * p.groups_per_warp);
    const int grp_end = min(p.groups_total, grp_begin + p.groups_per_warp);
    const int n_local = grp_end - grp_begin;
    const uint32_t wbar0 = bar0 + 8u * (warp * STAGES);
    uint8_t *wstages = stages + (size_t)warp * STAGES * C::STAGE_BYTES;

    // Where this warp's first group starts in each of the three linearly copied arrays (the other
    // three pieces go through tensor maps and are addressed by group number).
    constexpr uint32_t code_bytes = kGroup * C::RB;
    const uint8_t *kc_w = a.k_codes + bh * a.k_codes_stride_bh + (int64_t)grp_begin * code_bytes;
    const float *vs_w = a.v_scale + bh * a.v_param_stride_bh + (int64_t)grp_begin * (kGroup * 4);
    const float *vz_w = a.v_zero + bh * a.v_param_stride_bh + (int64_t)grp_begin * (kGroup * 4);
    auto issue_group = [&](auto stage_c, int local_idx) {  // called by lane 0 only; stage_c = local_idx % STAGES
        constexpr int stage = decltype(stage_c)::value;
        const int grp = grp_begin + local_idx;
        const uint32_t bar = wbar0 + 8u * stage;
        const uint32_t dst = smem_u32(wstages + (size_t)stage * C::STAGE_BYTES);
        mbar_expect_tx(bar, 2 * code_bytes + 4 * 512);
        bulk_g2s(dst + C::KC_OFF, kc_w + (uint32_t)local_idx * code_bytes, code_bytes, bar);
        tensor_g2s(dst + C::VC_OFF, &p.v_map, 0, grp * C::VROWS, (int)bh, bar);
        tensor_g2s(dst + C::KS_OFF, &p.ks_map, 0, grp * 4, (int)bh, bar);
        tensor_g2s(dst + C::KZ_OFF, &p.kz_map, 0, grp * 4, (int)bh, bar);
        bulk_g2s(dst + C::VS_OFF, vs_w + (uint32_t)local_idx * (kGroup * 4), 512, bar);
        bulk_g2s(dst + C::VZ_OFF, vz_w + (uint32_t)local_idx * (kGroup * 4), 512, bar);
    };

    if (tid == 0) {
        for (int s = 0; s < kWarps * STAGES + 1; ++s) mbar_init(bar0 + 8u * s, 1);  // the last one is never armed
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (lane == 0) {
        if (0 < STAGES - 1 && 0 < n_local) issue_group(std::integral_constant<int, 0>{}, 0);
        if (1 < STAGES - 1 && 1 < n_local) issue_group(std::integral_constant<int, 1 % STAGES>{}, 1);
        if (2 < STAGES - 1 && 2 < n_local) issue_group(std::integral_constant<int, 2 % STAGES>{}, 2);
    }
    // This warp's first residual row is read only after its packed groups: ask for its lines now
    // (4 lanes: the two 128-byte halves of the K row and of the V row at 16-bit width).
    if (lane < 4 && split * kWarps + warp < a.n_res) {
        const size_t es = a.res_dtype == VQ_F32 ? 4 : 2;
        const uint8_t *base = static_cast<const uint8_t *>((lane & 2) ? a.v_res : a.k_res) +
                              ((size_t)bh * a.res_stride_bh + (size_t)(split * kWarps + warp) * kD) * es;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(base + (lane & 1) * (kD * es / 2)));
    }

    // This lane's 16 query channels (head hd) are channels 32c + 16*half_id + [0, 16), handled
    // as four blocks of 4. Unpacked K register (pair p, element e) couples the blocks
    // blk(p, 0) and blk(p, 1). The four lanes c of a quarter-warp read chunks that are 128 bytes
    // apart, which in a linear tile is the same bank for all four; the scale and zero tiles are
    // therefore fetched through a tensor map with the 128-byte swizzle (16-byte block j of line
    // c sits at j ^ c), and sc_off0 is where this lane finds its block 0. qd is pre-divided by
    // the code weight of its element so that (code * weight) * (q * scale / weight) needs no fix-up.
    // Block L is at sc_off0 ^ 16L: L only touches the two bits that hold c.
    const uint32_t sc_off0 = (uint32_t)(128 * c + 16 * ((4 * half_id) ^ c));
    float qd[16];
    {
        const bool live = h0 + hd < hpk;
        const int64_t qbase = ((int64_t)b * a.H_q + hkv * hpk + h0 + hd) * kD + 32 * c + 16 * half_id;
#pragma unroll
        for (int i = 0; i < 16; ++i)
            qd[i] = live ? load_as_f32(a.q, a.q_dtype, qbase + i) / code_weight<BITS>(i & 3) : 0.f;
    }
    // 2-bit only: byte selector that regroups ldmatrix output so that one register holds
    // 4 channels of each of two neighbouring channel groups (see the PV section).
    const uint32_t v_sel = (g & 1) ? 0x7351u : 0x6240u;
    const int v_src = ((g >> 1) << 2) | c;

    // ldmatrix row address of this lane inside the swizzled V tile: token 16*mt + 8*(mi&1) + r,
    // 16-byte segment sb + (mi>>1); sb is 0 or 2, i.e. bit 5 of the linear offset (clear in the lane's
    // part), so it is XORed in after the swizzle rather than added
    // (4-bit: the second m-tile is 1024 bytes on, which leaves the XORed bits alone as well)
    // (4-bit: the second m-tile is 1024 bytes on, which leaves the XORed bits alone as well)
    const uint32_t v_lin = (uint32_t)((8 * ((lane >> 3) & 1) + (lane & 7)) * C::RB + 16 * (lane >> 4));
    const uint32_t v_off0 = swz128(v_lin);
    const uint32_t v_off1 = (BITS == 4) ? v_off0 + 16 * C::RB : swz128(v_lin + 16 * C::RB);
    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    // sum_t P[t, head c] * v_zero[t, group] over this lane's tokens, for the four channel groups
    float oz[4] = {0.f, 0.f, 0.f, 0.f};
    float m_run = -INFINITY, l_run = 0.f;  // of head c
    const float sc = a.scale * 1.4426950408889634f;  // scores kept in the log2 domain
    bool timed_out = false;

    // One group of 32 tokens from pipeline stage `stage` (a compile-time value, so that every
    // shared-memory address of the body is this lane's fixed offset plus a constant).
    auto body = [&](auto stage_c, const int it) {
        constexpr int stage = decltype(stage_c)::value;
        __syncwarp();  // every lane is done reading the stage that is refilled next
        if (lane == 0 && it + STAGES - 1 < n_local) {
            // order the lanes' generic-proxy reads before the async-proxy overwrite
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue_group(std::integral_constant<int, (stage + STAGES - 1) % STAGES>{}, it + STAGES - 1);
        }
        // After a timeout the warp stops waiting (later waits would only repeat it); its
        // result is garbage and the host learns of it through vq_kivi_attend_status().
        if (!timed_out && !mbar_wait(wbar0 + 8u * stage, (uint32_t)((it / STAGES) & 1))) timed_out = true;
        const uint8_t *st = wstages + (size_t)stage * C::STAGE_BYTES;

        // ---- B operand of QK^T for this group: q*k_scale split into hi/lo halves ----------
        // Lanes g and g^1 share a head; each computes both halves for 16 of the 32 channels
        // of chunk c and they swap what the other needs.
        uint32_t qf[16];
        float ck;
        {
            float x[16];
            float cp[4] = {0.f, 0.f, 0.f, 0.f};  // per element index: sum q/weight * k_zero
#pragma unroll
            for (int L = 0; L < 4; ++L) {
                const float4 s4 = *reinterpret_cast<const float4 *>(st + C::KS_OFF + (sc_off0 ^ (16u * L)));
                const float4 z4 = *reinterpret_cast<const float4 *>(st + C::KZ_OFF + (sc_off0 ^ (16u * L)));
                x[4 * L + 0] = qd[4 * L + 0] * s4.x; x[4 * L + 1] = qd[4 * L + 1] * s4.y;
                x[4 * L + 2] = qd[4 * L + 2] * s4.z; x[4 * L + 3] = qd[4 * L + 3] * s4.w;
                cp[0] = fmaf(qd[4 * L + 0], z4.x, cp[0]); cp[1] = fmaf(qd[4 * L + 1], z4.y, cp[1]);
                cp[2] = fmaf(qd[4 * L + 2], z4.z, cp[2]); cp[3] = fmaf(qd[4 * L + 3], z4.w, cp[3]);
            }
            float cpart = cp[0] * code_weight<BITS>(0) + cp[1] * code_weight<BITS>(1) +
                          cp[2] * code_weight<BITS>(2) + cp[3] * code_weight<BITS>(3);
            uint32_t own_hi[8], own_lo[8], recv[8];
#pragma unroll
            for (int pt = 0; pt < 2; ++pt) {
                // the two blocks that unpacked register pair pt couples
                const int L0 = (BITS == 4) ? 2 * pt : pt, L1 = (BITS == 4) ? 2 * pt + 1 : pt + 2;
#pragma unroll
                for (int e = 0; e < 4; ++e) split_h2(x[4 * L0 + e], x[4 * L1 + e], own_hi[4 * pt + e], own_lo[4 * pt + e]);
            }
#pragma unroll
            for (int ii = 0; ii < 8; ++ii) {
                const uint32_t send = half_id ? own_hi[ii] : own_lo[ii];
                recv[ii] = __shfl_xor_sync(0xffffffffu, send, 4);
            }
#pragma unroll
            for (int ii = 0; ii < 8; ++ii) {
                qf[ii] = half_id ? recv[ii] : own_hi[ii];
                qf[8 + ii] = half_id ? own_lo[ii] : recv[ii];
            }
            // zero-point term sum_d q[d]*k_zero[d] of head hd: reduce over c and the half pair
            cpart += __shfl_xor_sync(0xffffffffu, cpart, 1);
            cpart += __shfl_xor_sync(0xffffffffu, cpart, 2);
            cpart += __shfl_xor_sync(0xffffffffu, cpart, 4);
            ck = __shfl_sync(0xffffffffu, cpart, 8 * c);  // head c is computed by lanes g = 2c, 2c+1
        }

        // ---- S = codes . (q*k_scale)  for this warp's 32 tokens -----------------------------
        float s_acc[2][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            s_acc[mt][0] = s_acc[mt][1] = s_acc[mt][2] = s_acc[mt][3] = 0.f;
            uint32_t kw[2][C::KW];  // [row g / g+8][word]
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int tok = 16 * mt + g + 8 * r;
                const uint8_t *src = st + C::KC_OFF + tok * C::RB + c * (C::KW * 4);
                if constexpr (C::KW == 4) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(src);
                    kw[r][0] = v.x; kw[r][1] = v.y; kw[r][2] = v.z; kw[r][3] = v.w;
                } else {
                    const uint2 v = *reinterpret_cast<const uint2 *>(src);
                    kw[r][0] = v.x; kw[r][1] = v.y;
                }
            }
#pragma unroll
            for (int w = 0; w < C::KW; ++w) {
                uint32_t x0[C::NH], x1[C::NH];
                unpack_word<BITS>(kw[0][w], x0);
                unpack_word<BITS>(kw[1][w], x1);
#pragma unroll
                for (int jj = 0; jj < C::NH / 2; ++jj)
                    mma_f16(s_acc[mt], x0[2 * jj], x1[2 * jj], x0[2 * jj + 1], x1[2 * jj + 1],
                            qf[w * C::NH + 2 * jj], qf[w * C::NH + 2 * jj + 1]);
            }
        }

        // ---- online softmax of head c over this lane's four tokens and the 8 lanes g ---------
        float pr[2][2];  // [m-tile][token g / g + 8]
        {
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                // high-half + low-half column; the MMA saw codes * 2^-24: undo that and add the
                // zero-point term
                pr[mt][0] = fmaf(s_acc[mt][0] + s_acc[mt][1], sc * kTwo24, ck * sc);
                pr[mt][1] = fmaf(s_acc[mt][2] + s_acc[mt][3], sc * kTwo24, ck * sc);
            }
            float v = fmaxf(fmaxf(pr[0][0], pr[0][1]), fmaxf(pr[1][0], pr[1][1]));
            v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
            v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
            v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
            const float mn = fmaxf(m_run, v);
            const float corr = fast_exp2(m_run - mn);
            m_run = mn;
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                pr[mt][0] = fast_exp2(pr[mt][0] - mn);
                pr[mt][1] = fast_exp2(pr[mt][1] - mn);
            }
            l_run = l_run * corr + ((pr[0][0] + pr[0][1]) + (pr[1][0] + pr[1][1]));
            // The running maxima settle after the first few groups; skip the rescale of the
            // 36 accumulators whenever no lane's maximum moved (warp-uniform branch).
            if (__any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    o[i][0] *= corr; o[i][1] *= corr; o[i][2] *= corr; o[i][3] *= corr;
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) oz[j] *= corr;
            }
        }

        // ---- O^T += codes^T . (P*v_scale), and the zero-point term in float32 ---------------
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            const int t0 = 16 * mt;
            const uint32_t v_off = mt ? v_off1 : v_off0;
            uint32_t pbw[4][2];  // [channel group][tokens 0-7 / 8-15 of the m-tile]
            {
                // P[token, head c] times the token's four value scales, each product split into
                // (hi, lo) = this lane's column pair; the 8x8 transpose turns the P tile
                // (tokens x columns) into the B operand (tokens on K, columns on N).
                const float4 sa = *reinterpret_cast<const float4 *>(st + C::VS_OFF + (t0 + g) * 16);
                const float4 sbv = *reinterpret_cast<const float4 *>(st + C::VS_OFF + (t0 + g + 8) * 16);
                const float4 za = *reinterpret_cast<const float4 *>(st + C::VZ_OFF + (t0 + g) * 16);
                const float4 zb = *reinterpret_cast<const float4 *>(st + C::VZ_OFF + (t0 + g + 8) * 16);
                const float sa4[4] = {sa.x, sa.y, sa.z, sa.w}, sb4[4] = {sbv.x, sbv.y, sbv.z, sbv.w};
                const float za4[4] = {za.x, za.y, za.z, za.w}, zb4[4] = {zb.x, zb.y, zb.z, zb.w};
                const float pa = pr[mt][0], pb = pr[mt][1];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    oz[j] = fmaf(pa, za4[j], fmaf(pb, zb4[j], oz[j]));
                    // The (hi, lo) pair keeps the products exact. One rounded half per product measured
                    // 5 % faster at 2 bits, but with value channels scaled x20 its 2^-11 relative
                    // rounding reached 1.1e-2 absolute: outside the tolerance, so it is not offered.
                    const float xa = pa * sa4[j], xb = pb * sb4[j];
                    pbw[j][0] = movmatrix_trans(split_pack_trunc(xa));
                    pbw[j][1] = movmatrix_trans(split_pack_trunc(xb));
                }
            }
#pragma unroll
            for (int sb = 0; sb < C::NSEG; sb += 2) {
                uint32_t R[4];  // [segment sb + i/2][token block i%2]
                ldmatrix_x4_trans(R, smem_u32(st + C::VC_OFF) + (v_off ^ (16 * sb)));
                if constexpr (BITS == 2) {
                    // A 16-bit unit holds 8 channels, so the 8 lanes of a column span two
                    // channel groups. Regroup bytes so each lane holds channels 4g..4g+3 of
                    // the first group in bits 0-7 and of the second group in bits 8-15.
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t lo = __shfl_sync(0xffffffffu, R[i], v_src);
                        const uint32_t hi = __shfl_sync(0xffffffffu, R[i], v_src + 16);
                        R[i] = __byte_perm(lo, hi, v_sel);
                    }
                }
#pragma unroll
                for (int si = 0; si < 2; ++si) {
                    const int seg = sb + si;
                    uint32_t e0[C::CU], e1[C::CU];
                    unpack_word<BITS>(R[2 * si + 0], e0);  // tokens (2c, 2c+1)
                    unpack_word<BITS>(R[2 * si + 1], e1);  // tokens (2c+8, 2c+9)
#pragma unroll
                    for (int u = 0; u < C::CU / 2; ++u) {
                        // channel group of the 16 rows of this MMA
                        const int gd = (BITS == 4) ? seg : 2 * seg + (u >> 1);
                        mma_f16(o[seg * (C::CU / 2) + u], e0[2 * u], e0[2 * u + 1], e1[2 * u], e1[2 * u + 1],
                                pbw[gd][0], pbw[gd][1]);
                    }
                }
            }
        }
    };
    {
        int it = 0;
        for (; it + STAGES <= n_local; it += STAGES) {
            body(std::integral_constant<int, 0>{}, it);
            body(std::integral_constant<int, 1>{}, it + 1);
            if constexpr (STAGES > 2) body(std::integral_constant<int, 2>{}, it + 2);
            if constexpr (STAGES > 3) body(std::integral_constant<int, 3>{}, it + 3);
        }
        if (it < n_local) body(std::integral_constant<int, 0>{}, it++);
        if constexpr (STAGES > 2) { if (it < n_local) body(std::integral_constant<int, 1>{}, it++); }
        if constexpr (STAGES > 3) { if (it < n_local) body(std::integral_constant<int, 2>{}, it++); }
    }

    // Self-test of the bounded wait: a barrier that nothing arms never completes its phase.
    if (p.wait_test && !mbar_wait(bar0 + 8u * (kWarps * STAGES), 0u, kSelfTestSpinLimit)) timed_out = true;
    if (timed_out) {
        if (lane == 0) atomicExch(&g_attend_timeout, 1);
        // copies announced to a barrier that gave up may still be landing: give them time before
        // the stages are reused below and the CTA leaves
        if (!p.wait_test)
            for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }

    // Launched as a programmatic dependent (VQ_ATTEND_OVERLAP_PREVIOUS), this grid runs beside
    // the end of the previous work on the stream. Everything above touched only q and the packed
    // store; what follows reads the residual rows (which a vq_kivi_append right before this call
    // may just have written) and writes partials and tickets into a buffer that the previous
    // call's last CTAs may still be reading: it waits for the work before this grid to finish.
    // (Returns at once after a plain launch.)
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- the unquantized tail: residual row r belongs to warp r mod (splits * 4) of the unit ----
    // CUDA cores, a lane holds 4 consecutive channels of the row; heads of this CTA's chunk only.
    float tm[kChunkHeads], tl[kChunkHeads], to[kChunkHeads][4];
#pragma unroll
    for (int hp = 0; hp < kChunkHeads; ++hp) {
        tm[hp] = -INFINITY;
        tl[hp] = 0.f;
        to[hp][0] = to[hp][1] = to[hp][2] = to[hp][3] = 0.f;
    }
    {
        // With protected tokens (SINKS), this batch element's side rows follow the residual rows,
        // twice: their exact rows (weight +1), then the dequantized keys of the slots they left
        // in the packed store (weight -1, no value: those slots' value scales are 0, so all they
        // added above is their share of the softmax sum, and this takes it out again).
        int n_sink = 0;
        if constexpr (SINKS) n_sink = min(p.sinks.count[b], p.sinks.max_rows);
        const int n_tail = a.n_res + 2 * n_sink;
        int r = split * kWarps + warp;
        if (r < n_tail) {
            const int r_stride = p.n_splits * kWarps;
            float qt[kChunkHeads][4];
#pragma unroll
            for (int hp = 0; hp < kChunkHeads; ++hp) {
                const bool live = h0 + hp < hpk;
                const int64_t qb = ((int64_t)b * a.H_q + hkv * hpk + h0 + hp) * kD + 4 * lane;
#pragma unroll
                for (int i = 0; i < 4; ++i) qt[hp][i] = live ? load_as_f32(a.q, a.q_dtype, qb + i) * sc : 0.f;
            }
            const int64_t rbase = bh * a.res_stride_bh + 4 * lane;
            for (; r < n_tail; r += r_stride) {
                float kd[4], vd[4];
                bool dead = false;
                if (!SINKS || r < a.n_res) {
                    load_res4(a.k_res, a.res_dtype, rbase + (int64_t)r * kD, kd);
                    load_res4(a.v_res, a.res_dtype, rbase + (int64_t)r * kD, vd);
                } else {
                    const int rs = r - a.n_res;  // a protected token's row: exact first, then dead
                    dead = rs >= n_sink;
                    const int64_t e = bh * p.sinks.stride_bh + (int64_t)(dead ? rs - n_sink : rs) * kD + 4 * lane;
                    load_res4(dead ? p.sinks.k_dead : p.sinks.k, dead ? VQ_F32 : a.res_dtype, e, kd);
                    if (dead) vd[0] = vd[1] = vd[2] = vd[3] = 0.f;
                    else load_res4(p.sinks.v, a.res_dtype, e, vd);
                }
#pragma unroll
                for (int hp = 0; hp < kChunkHeads; ++hp) {
                    const float sv = warp_sum(qt[hp][0] * kd[0] + qt[hp][1] * kd[1] + qt[hp][2] * kd[2] + qt[hp][3] * kd[3]);
                    const float mn = fmaxf(tm[hp], sv);
                    const float f = fast_exp2(tm[hp] - mn), wgt = fast_exp2(sv - mn);
                    tl[hp] = tl[hp] * f + ((SINKS && dead) ? -wgt : wgt);
                    tm[hp] = mn;
#pragma unroll
                    for (int i = 0; i < 4; ++i) to[hp][i] = to[hp][i] * f + wgt * vd[i];
                }
            }
        }
    }

    // ---- merge the four warps (packed part and tail part of each), write this split's partial ----
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 4);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 8);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 16);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float z = oz[j];
        z += __shfl_xor_sync(0xffffffffu, z, 4);
        z += __shfl_xor_sync(0xffffffffu, z, 8);
        z += __shfl_xor_sync(0xffffffffu, z, 16);
        oz[j] = z;
    }
    __syncthreads();  // all stages are drained: reuse them for the reduction
    constexpr int kSlots = 2 * kWarps;  // per warp: its packed groups, its tail rows
    float *red_o = reinterpret_cast<float *>(stages);               // [8 slots][4 heads][128]
    float *red_z = red_o + kSlots * kChunkHeads * kD;               // [8][4][4 groups]
    float *red_m = red_z + kSlots * kChunkHeads * 4;                // [8][4]
    float *red_l = red_m + kSlots * kChunkHeads;                    // [8][4]
    // channel of accumulator rows g / g+8 of MMA i
    auto chan = [&](int i) {
        const int seg = i / (C::CU / 2), u = i % (C::CU / 2);
        if constexpr (BITS == 4) return 32 * seg + 4 * g + 2 * u;
        else return 64 * seg + 32 * (u >> 1) + 4 * g + 2 * (u & 1);
    };
    {
        // Accumulator rows saw codes * weight * 2^-24 (see unpack_word): undo per row; the two
        // columns of a row are the high- and low-half contributions of head c.
        float *base = red_o + (warp * kChunkHeads + c) * kD;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int u = i % (C::CU / 2);
            const float f0 = kTwo24 / code_weight<BITS>(2 * u), f1 = kTwo24 / code_weight<BITS>(2 * u + 1);
            const int d0 = chan(i);
            base[d0] = (o[i][0] + o[i][1]) * f0;
            base[d0 + 1] = (o[i][2] + o[i][3]) * f1;
        }
        if (g == 0) {
            red_m[warp * kChunkHeads + c] = m_run;
            red_l[warp * kChunkHeads + c] = l_run;
#pragma unroll
            for (int j = 0; j < 4; ++j) red_z[(warp * kChunkHeads + c) * 4 + j] = oz[j];
        }
        // the tail slot of this warp
#pragma unroll
        for (int hp = 0; hp < kChunkHeads; ++hp) {
            const int slot = (kWarps + warp) * kChunkHeads + hp;
            *reinterpret_cast<float4 *>(red_o + slot * kD + 4 * lane) = make_float4(to[hp][0], to[hp][1], to[hp][2], to[hp][3]);
            if (lane == 0) { red_m[slot] = tm[hp]; red_l[slot] = tl[hp]; }
            if (lane < 4) red_z[slot * 4 + lane] = 0.f;
        }
    }
    __syncthreads();
    const int n_heads = min(kChunkHeads, hpk - h0);
    for (int i = tid; i < n_heads * kD; i += blockDim.x) {
        const int hp = i / kD, d = i % kD;
        float gm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kSlots; ++w) gm = fmaxf(gm, red_m[w * kChunkHeads + hp]);
        float gl = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < kSlots; ++w) {
            const float mw = red_m[w * kChunkHeads + hp];
            const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - gm);
            gl += red_l[w * kChunkHeads + hp] * f;
            acc += (red_o[(w * kChunkHeads + hp) * kD + d] + red_z[(w * kChunkHeads + hp) * 4 + (d >> 5)]) * f;
        }
        const int64_t rec = (bh * p.n_splits + split) * hpk + h0 + hp;
        p.part_o[rec * kD + d] = acc;
        if (d == 0) { p.part_ml[rec * 2] = gm; p.part_ml[rec * 2 + 1] = gl; }
    }

    ticket_merge_publish<kChunkHeads>(p, bars, bh, b, hkv, h0, hpk, n_heads, tid, lane, warp);
}

// ---- the same kernel for 5..8 query heads per kv head --------------------------------------------
// With four heads a CTA spends the eight MMA columns on (high, low) halves of each head's B
// operand; a kv head with more query heads then needs two CTAs, i.e. the unpack of every code
// twice. Here the eight columns are eight heads, and every A fragment (unpacked once) feeds two
// MMAs into the same accumulators: one with the high halves of the B operand, one with the low
// halves (hi + lo contributions simply add). Per 32-token group that is the unpack once, 64 MMAs
// instead of 2 x 32, and the per-head B-operand and softmax work of eight heads instead of
// 2 x 4: about half the instructions of two four-head CTAs. It costs registers (the B operands of
// eight heads in both halves): three CTAs per SM instead of four.
// Lane roles (g = lane / 4, c = lane % 4): as a B-operand column, head g for the 32 channels of
// chunk c; as an accumulator column pair (cols 2c, 2c+1), heads 2c and 2c+1 for its rows.
constexpr int kWideHeads = 8;

template <int BITS>
__global__ void __launch_bounds__(kWarps * 32, 3)
kivi_attend_mma8_kernel(const __grid_constant__ Params p) {
    using C = Cfg<BITS>;
    constexpr int STAGES = 2;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const vq_kivi_attend_args &a = p.a;
    const int b = blockIdx.z, hkv = blockIdx.y;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int split = blockIdx.x / p.n_chunks;
    const int h0 = (blockIdx.x % p.n_chunks) * kWideHeads;
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int g = lane >> 2, c = lane & 3;
    const int hpk = p.hpk;
    const int64_t bh = (int64_t)b * a.H_kv + hkv;

    uint8_t *stages = smem_raw;
    constexpr int kStageArea = kWarps * STAGES * C::STAGE_BYTES;
    constexpr int kRedArea = (2 * kWarps * kWideHeads * (kD + 4 + 2)) * 4;
    constexpr int kArea = kStageArea > kRedArea ? kStageArea : kRedArea;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem_raw + kArea);
    const uint32_t bar0 = smem_u32(bars);
    if (smem_u32(stages) & 1023u) {
        if (tid == 0) atomicExch(&g_attend_timeout, 2);
        return;
    }
    const int grp_begin = min(p.groups_total, (split * kWarps + warp) * p.groups_per_warp);
    const int grp_end = min(p.groups_total, grp_begin + p.groups_per_warp);
    const int n_local = grp_end - grp_begin;
    const uint32_t wbar0 = bar0 + 8u * (warp * STAGES);
    uint8_t *wstages = stages + (size_t)warp * STAGES * C::STAGE_BYTES;

    constexpr uint32_t code_bytes = kGroup * C::RB;
    const uint8_t *kc_w = a.k_codes + bh * a.k_codes_stride_bh + (int64_t)grp_begin * code_bytes;
    const float *vs_w = a.v_scale + bh * a.v_param_stride_bh + (int64_t)grp_begin * (kGroup * 4);
    const float *vz_w = a.v_zero + bh * a.v_param_stride_bh + (int64_t)grp_begin * (kGroup * 4);
    auto issue_group = [&](auto stage_c, int local_idx) {  // lane 0 only; stage_c = local_idx % STAGES
        constexpr int stage = decltype(stage_c)::value;
        const int grp = grp_begin + local_idx;
        const uint32_t bar = wbar0 + 8u * stage;
        const uint32_t dst = smem_u32(wstages + (size_t)stage * C::STAGE_BYTES);
        mbar_expect_tx(bar, 2 * code_bytes + 4 * 512);
        bulk_g2s(dst + C::KC_OFF, kc_w + (uint32_t)local_idx * code_bytes, code_bytes, bar);
        tensor_g2s(dst + C::VC_OFF, &p.v_map, 0, grp * C::VROWS, (int)bh, bar);
        tensor_g2s(dst + C::KS_OFF, &p.ks_map, 0, grp * 4, (int)bh, bar);
        tensor_g2s(dst + C::KZ_OFF, &p.kz_map, 0, grp * 4, (int)bh, bar);
        bulk_g2s(dst + C::VS_OFF, vs_w + (uint32_t)local_idx * (kGroup * 4), 512, bar);
        bulk_g2s(dst + C::VZ_OFF, vz_w + (uint32_t)local_idx * (kGroup * 4), 512, bar);
    };
    if (tid == 0) {
        for (int s = 0; s < kWarps * STAGES + 1; ++s) mbar_init(bar0 + 8u * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (lane == 0 && n_local > 0) issue_group(std::integral_constant<int, 0>{}, 0);
    if (lane < 4 && split * kWarps + warp < a.n_res) {
        const size_t es = a.res_dtype == VQ_F32 ? 4 : 2;
        const uint8_t *base = static_cast<const uint8_t *>((lane & 2) ? a.v_res : a.k_res) +
                              ((size_t)bh * a.res_stride_bh + (size_t)(split * kWarps + warp) * kD) * es;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(base + (lane & 1) * (kD * es / 2)));
    }

    // B-operand register r = w * NH + i of this lane (word w of its 32-channel chunk, unpacked
    // register i) pairs the chunk's channels CPW*w + i and CPW*w + CPW/2 + i (the i-th code of the
    // word's low and of its high 16 bits); both are pre-divided by the register's code weight.
    constexpr int NR = C::KW * C::NH;  // 16
    float qa[NR], qb[NR];
    {
        const bool live = h0 + g < hpk;
        const int64_t qbase = ((int64_t)b * a.H_q + hkv * hpk + h0 + g) * kD + 32 * c;
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const int w = r / C::NH, i = r % C::NH;
            const float inv = 1.f / code_weight<BITS>(i);
            qa[r] = live ? load_as_f32(a.q, a.q_dtype, qbase + C::CPW * w + i) * inv : 0.f;
            qb[r] = live ? load_as_f32(a.q, a.q_dtype, qbase + C::CPW * w + C::CPW / 2 + i) * inv : 0.f;
        }
    }
    const uint32_t v_sel = (g & 1) ? 0x7351u : 0x6240u;
    const int v_src = ((g >> 1) << 2) | c;
    const uint32_t v_lin = (uint32_t)((8 * ((lane >> 3) & 1) + (lane & 7)) * C::RB + 16 * (lane >> 4));
    const uint32_t v_off0 = swz128(v_lin);
    const uint32_t v_off1 = (BITS == 4) ? v_off0 + 16 * C::RB : swz128(v_lin + 16 * C::RB);
    float o[8][4];  // [MMA][row g: heads 2c, 2c+1 | row g+8: heads 2c, 2c+1]
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float oz[4][2];
#pragma unroll
    for (int j = 0; j < 4; ++j) oz[j][0] = oz[j][1] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float sc = a.scale * 1.4426950408889634f;
    bool timed_out = false;

    auto body = [&](auto stage_c, const int it) {
        constexpr int stage = decltype(stage_c)::value;
        __syncwarp();
        if (lane == 0 && it + 1 < n_local) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            issue_group(std::integral_constant<int, (stage + 1) % STAGES>{}, it + 1);
        }
        if (!timed_out && !mbar_wait(wbar0 + 8u * stage, (uint32_t)((it / STAGES) & 1))) timed_out = true;
        const uint8_t *st = wstages + (size_t)stage * C::STAGE_BYTES;

        // ---- B operand of QK^T: q * k_scale of head g over chunk c, as high and low halves ----
        uint32_t qh[NR], ql[NR];
        float ck0, ck1;
        {
            // (the tiles arrive 128-byte swizzled: 16-byte block j of line c sits at j ^ c)
            float ks[32], kz[32];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float4 s4 = *reinterpret_cast<const float4 *>(st + C::KS_OFF + 128 * c + 16 * (j ^ c));
                const float4 z4 = *reinterpret_cast<const float4 *>(st + C::KZ_OFF + 128 * c + 16 * (j ^ c));
                ks[4 * j] = s4.x; ks[4 * j + 1] = s4.y; ks[4 * j + 2] = s4.z; ks[4 * j + 3] = s4.w;
                kz[4 * j] = z4.x; kz[4 * j + 1] = z4.y; kz[4 * j + 2] = z4.z; kz[4 * j + 3] = z4.w;
            }
            float cp[4] = {0.f, 0.f, 0.f, 0.f};  // per code weight: sum q / weight * k_zero
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const int w = r / C::NH, i = r % C::NH;
                const int fa = C::CPW * w + i, fb = fa + C::CPW / 2;
                const float xa = qa[r] * ks[fa], xb = qb[r] * ks[fb];
                cp[i & 3] = fmaf(qa[r], kz[fa], fmaf(qb[r], kz[fb], cp[i & 3]));
                split_h2(xa, xb, qh[r], ql[r]);
            }
            float cpart = cp[0] * code_weight<BITS>(0) + cp[1] * code_weight<BITS>(1) +
                          cp[2] * code_weight<BITS>(2) + cp[3] * code_weight<BITS>(3);
            cpart += __shfl_xor_sync(0xffffffffu, cpart, 1);
            cpart += __shfl_xor_sync(0xffffffffu, cpart, 2);
            // this lane's accumulator columns are heads 2c and 2c+1: their zero-point terms sit in quads 2c, 2c+1
            ck0 = __shfl_sync(0xffffffffu, cpart, 8 * c);
            ck1 = __shfl_sync(0xffffffffu, cpart, 8 * c + 4);
        }

        // ---- S = codes . (q*k_scale): every unpacked fragment feeds a high-half and a low-half MMA ----
        float s_acc[2][4];
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            s_acc[mt][0] = s_acc[mt][1] = s_acc[mt][2] = s_acc[mt][3] = 0.f;
            uint32_t kw[2][C::KW];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const int tok = 16 * mt + g + 8 * r;
                const uint8_t *src = st + C::KC_OFF + tok * C::RB + c * (C::KW * 4);
                if constexpr (C::KW == 4) {
                    const uint4 v = *reinterpret_cast<const uint4 *>(src);
                    kw[r][0] = v.x; kw[r][1] = v.y; kw[r][2] = v.z; kw[r][3] = v.w;
                } else {
                    const uint2 v = *reinterpret_cast<const uint2 *>(src);
                    kw[r][0] = v.x; kw[r][1] = v.y;
                }
            }
#pragma unroll
            for (int w = 0; w < C::KW; ++w) {
                uint32_t x0[C::NH], x1[C::NH];
                unpack_word<BITS>(kw[0][w], x0);
                unpack_word<BITS>(kw[1][w], x1);
#pragma unroll
                for (int jj = 0; jj < C::NH / 2; ++jj) {
                    mma_f16(s_acc[mt], x0[2 * jj], x1[2 * jj], x0[2 * jj + 1], x1[2 * jj + 1],
                            qh[w * C::NH + 2 * jj], qh[w * C::NH + 2 * jj + 1]);
                    mma_f16(s_acc[mt], x0[2 * jj], x1[2 * jj], x0[2 * jj + 1], x1[2 * jj + 1],
                            ql[w * C::NH + 2 * jj], ql[w * C::NH + 2 * jj + 1]);
                }
            }
        }

        // ---- online softmax of heads 2c, 2c+1 over this lane's four tokens and the 8 lanes g ----
        float pr[2][2][2];  // [m-tile][token g / g + 8][head 2c / 2c + 1]
        {
            const float k0 = ck0 * sc, k1 = ck1 * sc, f = sc * kTwo24;
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
                pr[mt][0][0] = fmaf(s_acc[mt][0], f, k0); pr[mt][0][1] = fmaf(s_acc[mt][1], f, k1);
                pr[mt][1][0] = fmaf(s_acc[mt][2], f, k0); pr[mt][1][1] = fmaf(s_acc[mt][3], f, k1);
            }
            float corr[2];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                float v = fmaxf(fmaxf(pr[0][0][hh], pr[0][1][hh]), fmaxf(pr[1][0][hh], pr[1][1][hh]));
                v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
                v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 8));
                v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 16));
                const float mn = fmaxf(m_run[hh], v);
                corr[hh] = fast_exp2(m_run[hh] - mn);
                m_run[hh] = mn;
#pragma unroll
                for (int mt = 0; mt < 2; ++mt) {
                    pr[mt][0][hh] = fast_exp2(pr[mt][0][hh] - mn);
                    pr[mt][1][hh] = fast_exp2(pr[mt][1][hh] - mn);
                }
                l_run[hh] = l_run[hh] * corr[hh] + ((pr[0][0][hh] + pr[0][1][hh]) + (pr[1][0][hh] + pr[1][1][hh]));
            }
            if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    o[i][0] *= corr[0]; o[i][1] *= corr[1]; o[i][2] *= corr[0]; o[i][3] *= corr[1];
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) { oz[j][0] *= corr[0]; oz[j][1] *= corr[1]; }
            }
        }

        // ---- O^T += codes^T . (P*v_scale) (high and low halves), zero-point term in float32 ----
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            const int t0 = 16 * mt;
            const uint32_t v_off = mt ? v_off1 : v_off0;
            uint32_t pbh[4][2], pbl[4][2];  // [channel group][tokens 0-7 / 8-15 of the m-tile]
            {
                const float4 sa = *reinterpret_cast<const float4 *>(st + C::VS_OFF + (t0 + g) * 16);
                const float4 sbv = *reinterpret_cast<const float4 *>(st + C::VS_OFF + (t0 + g + 8) * 16);
                const float4 za = *reinterpret_cast<const float4 *>(st + C::VZ_OFF + (t0 + g) * 16);
                const float4 zb = *reinterpret_cast<const float4 *>(st + C::VZ_OFF + (t0 + g + 8) * 16);
                const float sa4[4] = {sa.x, sa.y, sa.z, sa.w}, sb4[4] = {sbv.x, sbv.y, sbv.z, sbv.w};
                const float za4[4] = {za.x, za.y, za.z, za.w}, zb4[4] = {zb.x, zb.y, zb.z, zb.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh)
                        oz[j][hh] = fmaf(pr[mt][0][hh], za4[j], fmaf(pr[mt][1][hh], zb4[j], oz[j][hh]));
                    // element pair (row = token, columns 2c, 2c+1 = heads 2c, 2c+1); the 8x8 transpose makes it
                    // the B operand (tokens on K, heads on N). High halves are truncations (one AND each).
#pragma unroll
                    for (int r = 0; r < 2; ++r) {
                        const float x0 = pr[mt][r][0] * (r ? sb4[j] : sa4[j]), x1 = pr[mt][r][1] * (r ? sb4[j] : sa4[j]);
                        const float h0f = __uint_as_float(__float_as_uint(x0) & 0xffffe000u);
                        const float h1f = __uint_as_float(__float_as_uint(x1) & 0xffffe000u);
                        pbh[j][r] = movmatrix_trans(pack_h2(h0f, h1f));
                        pbl[j][r] = movmatrix_trans(pack_h2(x0 - h0f, x1 - h1f));
                    }
                }
            }
#pragma unroll
            for (int sb = 0; sb < C::NSEG; sb += 2) {
                uint32_t R[4];
                ldmatrix_x4_trans(R, smem_u32(st + C::VC_OFF) + (v_off ^ (16 * sb)));
                if constexpr (BITS == 2) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t lo = __shfl_sync(0xffffffffu, R[i], v_src);
                        const uint32_t hi = __shfl_sync(0xffffffffu, R[i], v_src + 16);
                        R[i] = __byte_perm(lo, hi, v_sel);
                    }
                }
#pragma unroll
                for (int si = 0; si < 2; ++si) {
                    const int seg = sb + si;
                    uint32_t e0[C::CU], e1[C::CU];
                    unpack_word<BITS>(R[2 * si + 0], e0);
                    unpack_word<BITS>(R[2 * si + 1], e1);
#pragma unroll
                    for (int u = 0; u < C::CU / 2; ++u) {
                        const int gd = (BITS == 4) ? seg : 2 * seg + (u >> 1);
                        mma_f16(o[seg * (C::CU / 2) + u], e0[2 * u], e0[2 * u + 1], e1[2 * u], e1[2 * u + 1], pbh[gd][0], pbh[gd][1]);
                        mma_f16(o[seg * (C::CU / 2) + u], e0[2 * u], e0[2 * u + 1], e1[2 * u], e1[2 * u + 1], pbl[gd][0], pbl[gd][1]);
                    }
                }
            }
        }
    };
    {
        int it = 0;
        for (; it + STAGES <= n_local; it += STAGES) {
            body(std::integral_constant<int, 0>{}, it);
            body(std::integral_constant<int, 1>{}, it + 1);
        }
        if (it < n_local) body(std::integral_constant<int, 0>{}, it);
    }
    if (p.wait_test && !mbar_wait(bar0 + 8u * (kWarps * STAGES), 0u, kSelfTestSpinLimit)) timed_out = true;
    if (timed_out) {
        if (lane == 0) atomicExch(&g_attend_timeout, 1);
        if (!p.wait_test)
            for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }

    // ---- this warp's packed part into its slot of the reduction area (frees the accumulators) ----
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 4);
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 8);
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 16);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float z = oz[j][hh];
            z += __shfl_xor_sync(0xffffffffu, z, 4);
            z += __shfl_xor_sync(0xffffffffu, z, 8);
            z += __shfl_xor_sync(0xffffffffu, z, 16);
            oz[j][hh] = z;
        }
    }
    __syncthreads();  // all stages are drained: reuse them for the reduction
    constexpr int kSlots = 2 * kWarps;
    float *red_o = reinterpret_cast<float *>(stages);              // [8 slots][8 heads][128]
    float *red_z = red_o + kSlots * kWideHeads * kD;               // [8][8][4 groups]
    float *red_m = red_z + kSlots * kWideHeads * 4;                // [8][8]
    float *red_l = red_m + kSlots * kWideHeads;                    // [8][8]
    auto chan = [&](int i) {
        const int seg = i / (C::CU / 2), u = i % (C::CU / 2);
        if constexpr (BITS == 4) return 32 * seg + 4 * g + 2 * u;
        else return 64 * seg + 32 * (u >> 1) + 4 * g + 2 * (u & 1);
    };
    {
        float *base0 = red_o + (warp * kWideHeads + 2 * c) * kD, *base1 = base0 + kD;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int u = i % (C::CU / 2);
            const float f0 = kTwo24 / code_weight<BITS>(2 * u), f1 = kTwo24 / code_weight<BITS>(2 * u + 1);
            const int d0 = chan(i);
            base0[d0] = o[i][0] * f0; base1[d0] = o[i][1] * f0;
            base0[d0 + 1] = o[i][2] * f1; base1[d0 + 1] = o[i][3] * f1;
        }
        if (g == 0) {
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int slot = warp * kWideHeads + 2 * c + hh;
                red_m[slot] = m_run[hh];
                red_l[slot] = l_run[hh];
#pragma unroll
                for (int j = 0; j < 4; ++j) red_z[slot * 4 + j] = oz[j][hh];
            }
        }
    }

    // (see the four-head kernel: everything above touched only q and the packed store)
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- the unquantized tail, two passes of four heads (the registers of one pass are reused) ----
    const int n_heads = min(kWideHeads, hpk - h0);
#pragma unroll 1
    for (int hq = 0; hq < kWideHeads; hq += 4) {
        float tm[4], tl[4], to[4][4];
#pragma unroll
        for (int hp = 0; hp < 4; ++hp) {
            tm[hp] = -INFINITY;
            tl[hp] = 0.f;
            to[hp][0] = to[hp][1] = to[hp][2] = to[hp][3] = 0.f;
        }
        int r = split * kWarps + warp;
        if (r < a.n_res && hq < n_heads) {
            const int r_stride = p.n_splits * kWarps;
            float qt[4][4];
#pragma unroll
            for (int hp = 0; hp < 4; ++hp) {
                const bool live = h0 + hq + hp < hpk;
                const int64_t qb = ((int64_t)b * a.H_q + hkv * hpk + h0 + hq + hp) * kD + 4 * lane;
#pragma unroll
                for (int i = 0; i < 4; ++i) qt[hp][i] = live ? load_as_f32(a.q, a.q_dtype, qb + i) * sc : 0.f;
            }
            const int64_t rbase = bh * a.res_stride_bh + 4 * lane;
            for (; r < a.n_res; r += r_stride) {
                float kd[4], vd[4];
                load_res4(a.k_res, a.res_dtype, rbase + (int64_t)r * kD, kd);
                load_res4(a.v_res, a.res_dtype, rbase + (int64_t)r * kD, vd);
#pragma unroll
                for (int hp = 0; hp < 4; ++hp) {
                    const float sv = warp_sum(qt[hp][0] * kd[0] + qt[hp][1] * kd[1] + qt[hp][2] * kd[2] + qt[hp][3] * kd[3]);
                    const float mn = fmaxf(tm[hp], sv);
                    const float f = fast_exp2(tm[hp] - mn), wgt = fast_exp2(sv - mn);
                    tl[hp] = tl[hp] * f + wgt;
                    tm[hp] = mn;
#pragma unroll
                    for (int i = 0; i < 4; ++i) to[hp][i] = to[hp][i] * f + wgt * vd[i];
                }
            }
        }
#pragma unroll
        for (int hp = 0; hp < 4; ++hp) {
            const int slot = (kWarps + warp) * kWideHeads + hq + hp;
            *reinterpret_cast<float4 *>(red_o + slot * kD + 4 * lane) = make_float4(to[hp][0], to[hp][1], to[hp][2], to[hp][3]);
            if (lane == 0) { red_m[slot] = tm[hp]; red_l[slot] = tl[hp]; }
            if (lane < 4) red_z[slot * 4 + lane] = 0.f;
        }
    }
    __syncthreads();
    for (int i = tid; i < n_heads * kD; i += blockDim.x) {
        const int hp = i / kD, d = i % kD;
        float gm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kSlots; ++w) gm = fmaxf(gm, red_m[w * kWideHeads + hp]);
        float gl = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < kSlots; ++w) {
            const float mw = red_m[w * kWideHeads + hp];
            const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - gm);
            gl += red_l[w * kWideHeads + hp] * f;
            acc += (red_o[(w * kWideHeads + hp) * kD + d] + red_z[(w * kWideHeads + hp) * 4 + (d >> 5)]) * f;
        }
        const int64_t rec = (bh * p.n_splits + split) * hpk + h0 + hp;
        p.part_o[rec * kD + d] = acc;
        if (d == 0) { p.part_ml[rec * 2] = gm; p.part_ml[rec * 2 + 1] = gl; }
    }
    ticket_merge_publish<kWideHeads>(p, bars, bh, b, hkv, h0, hpk, n_heads, tid, lane, warp);
}

constexpr int kMaxSplits = 512;  // (a ticket counts arrivals in 16 bits)

// Pipeline depth and waves-per-launch are tunables (vq_tune: VQ_KNOB_ATTEND_STAGES = 2..4,
// VQ_KNOB_ATTEND_WAVES = 1..32).
int tuned_stages() { return knob_get(VQ_KNOB_ATTEND_STAGES); }
int tuned_waves() { return knob_get(VQ_KNOB_ATTEND_WAVES); }

int smem_for(int bits, int stages) {
    return bits == 4 ? Cfg<4>::smem_bytes(stages) : Cfg<2>::smem_bytes(stages);
}

// Context splits per (batch, kv head, head chunk). A CTA has fixed costs (pipeline fill, its few
// residual rows, the partial write and the ticket), so it wants a long run of groups; the GPU
// wants enough CTAs. Measured on B200 (32K context, 8 kv heads, 4 query heads each):
//   plain launches (a call runs alone): about 32 groups per warp, and at least ~256 CTAs per
//     launch -- batch 16: 8 splits, batch 8 and 4: 9, batch 2: 16, batch 1: 20;
//   calls that overlap their predecessor: CTAs of two or three calls are resident together, so a
//     launch need not fill the GPU by itself and longer CTAs win -- about 64 groups per warp
//     (32 when there are only a few units): batch 16: 3-4 splits, batch 8: 2-4, batch 4: 2-5,
//     batch 2: 5-9, batch 1: 5-8. Shorter contexts take proportionally shorter runs (16 at least).
// More than four query heads per kv head go to the eight-head kernel when the context is long and
// the launch is large (not with protected tokens: those rows exist in the four-head kernel only).
// Measured per layer, eight-head against two four-head chunks: 200 / 231 us (8 heads per kv head,
// batch 16, 32K context), 114 / 125 us (5 heads, batch 16, 16K), 35 / 40 us (5 heads, batch 4,
// 16K); but 289 / 266 us at batch 64 with an 8K context (one short CTA per unit and its larger
// fixed cost), and 21.5 / 20.3 us and 17.9 / 13.7 us on a half and an eighth of the batch-4 launch
// (too few CTAs: the four-head kernel's twice as many fill the GPU better).
bool wide_heads(const vq_kivi_attend_args &a) {
    const int64_t groups = a.n_quant / kGroup;
    return a.H_q / a.H_kv > kChunkHeads && a.sinks == nullptr && groups >= 512 &&
           (int64_t)a.B * a.H_kv * groups >= 12288;
}
int head_chunks(const vq_kivi_attend_args &a) {
    return (int)ceil_div(a.H_q / a.H_kv, wide_heads(a) ? kWideHeads : kChunkHeads);
}

int choose_splits(const vq_kivi_attend_args &a, const DeviceInfo &di) {
    (void)di;
    const int tiles = (int)ceil_div(a.n_quant, kGroup * kWarps);  // CTA-sized pieces of the context
    if (tiles <= 1) return std::max(tiles, 0);
    if (a.n_splits > 0) return std::min(std::min(a.n_splits, tiles), kMaxSplits);
    const int n_chunks = head_chunks(a);
    const int64_t units = (int64_t)a.B * a.H_kv * n_chunks;
    const int64_t groups = a.n_quant / kGroup;
    const int64_t cap = std::min<int64_t>(std::max(1, tiles / 4), kMaxSplits);  // >= 4 groups per warp
    int64_t want;
    if (a.flags & VQ_ATTEND_OVERLAP_PREVIOUS) {
        // (the run of groups a warp takes grows with the launch's total work, units x groups,
        // normalised to the 32K context the figures above were measured at: a launch of half the
        // context and half the units -- one rank's share of a sharded 16K-token batch -- at 64 groups
        // per warp was 64 CTAs that took as long as the unsharded launch)
        const int64_t scaled = (2 * units * groups + 512) / 1024;
        const int64_t per_warp = std::min<int64_t>(64, std::max<int64_t>(groups >= 768 ? 32 : 16, scaled));
        want = (groups + 2 * per_warp) / (4 * per_warp);  // rounded to nearest
    } else {
        const int64_t fill = ceil_div((int64_t)64 * tuned_waves() * 2, units);  // 256 CTAs at the default setting
        want = std::max<int64_t>(ceil_div(groups, 4 * 32), fill);
    }
    return (int)std::max<int64_t>(1, std::min(want, cap));
}

template <int BITS, int STAGES, bool SINKS>
int32_t launch_one(const Params &p, dim3 grid, cudaStream_t st) {
    const int smem = smem_for(BITS, STAGES);
    VQ_CHECK_CUDA(cudaFuncSetAttribute(kivi_attend_mma_kernel<BITS, STAGES, SINKS>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    // A plain (fully serialised) launch unless the caller set VQ_ATTEND_OVERLAP_PREVIOUS: then the
    // grid is a programmatic dependent of whatever precedes it on the stream (the previous call's
    // kernel triggers at its start) and only its residual rows and merge wait for that work.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kWarps * 32);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (p.a.flags & VQ_ATTEND_OVERLAP_PREVIOUS) ? 1 : 0;
    VQ_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kivi_attend_mma_kernel<BITS, STAGES, SINKS>, p));
    return VQ_OK;
}

template <int BITS>
int32_t launch_wide(const Params &p, dim3 grid, cudaStream_t st) {
    using C = Cfg<BITS>;
    constexpr int stage_area = kWarps * 2 * C::STAGE_BYTES, red_area = (2 * kWarps * kWideHeads * (kD + 4 + 2)) * 4;
    const int smem = (stage_area > red_area ? stage_area : red_area) + 256;
    VQ_CHECK_CUDA(cudaFuncSetAttribute(kivi_attend_mma8_kernel<BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kWarps * 32);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (p.a.flags & VQ_ATTEND_OVERLAP_PREVIOUS) ? 1 : 0;
    VQ_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kivi_attend_mma8_kernel<BITS>, p));
    return VQ_OK;
}

template <int BITS>
int32_t launch_bits(const Params &p, dim3 grid, cudaStream_t st) {
    if (p.wide) return launch_wide<BITS>(p, grid, st);
    if (p.sinks.count != nullptr) return launch_one<BITS, 2, true>(p, grid, st);  // (the stage knob applies to the plain kernel)
    switch (tuned_stages()) {
        case 3: return launch_one<BITS, 3, false>(p, grid, st);
        case 4: return launch_one<BITS, 4, false>(p, grid, st);
        default: return launch_one<BITS, 2, false>(p, grid, st);
    }
}

}  // namespace

const char *kivi_attend_mma_supported(const vq_kivi_attend_args &a) {
    if (a.D != kD) return "head_dim must be 128";
    if (a.S_q != 1) return "one query row per call";
    if (a.n_quant <= 0) return "no packed tokens";
    if (a.group != 32) return "group size must be 32";
    if (a.store_bits != 2 && a.store_bits != 4) return "codes must be stored in 2 or 4 bits";
    if (a.H_q / a.H_kv > kMaxHeads) return "more than 8 query heads per kv head";
    if (a.n_quant % 32) return "packed token count must be a multiple of the group size";
    if (a.B > 65535 || a.H_kv > 65535) return "grid too large";
    const int rb = kD * a.store_bits / 8;
    if (!is_aligned(a.k_codes, 16) || !is_aligned(a.v_codes, 16) || a.k_codes_stride_bh % 16 ||
        a.v_codes_stride_bh % 16 || rb % 16)
        return "code buffers must be 16-byte aligned";
    if (!is_aligned(a.k_scale, 16) || !is_aligned(a.k_zero, 16) || !is_aligned(a.v_scale, 16) ||
        !is_aligned(a.v_zero, 16) || a.k_param_stride_bh % 4 || a.v_param_stride_bh % 4)
        return "scale/zero buffers must be 16-byte aligned";
    if ((a.n_res > 0 || a.sinks != nullptr) && a.res_dtype != VQ_F16 && a.res_dtype != VQ_BF16 && a.res_dtype != VQ_F32)
        return "bad residual dtype";
    if (a.n_res > 0 && (!is_aligned(a.k_res, 16) || !is_aligned(a.v_res, 16) || a.res_stride_bh % 8))
        return "residual buffers must be 16-byte aligned";
    return nullptr;
}

int kivi_attend_mma_splits(const vq_kivi_attend_args &a, const DeviceInfo &di) { return choose_splits(a, di); }

// Workspace of a launch with `n_splits` context splits: the partial records, then one 64-bit
// ticket per (batch, kv head, head chunk).
int64_t kivi_attend_mma_workspace(const vq_kivi_attend_args &a, int n_splits) {
    const int hpk = a.H_q / a.H_kv;
    const int64_t recs = (int64_t)a.B * a.H_kv * n_splits * hpk;
    const int64_t part_bytes = recs * (kD + 2) * (int64_t)sizeof(float);
    return ((part_bytes + 15) & ~(int64_t)15) + (int64_t)a.B * a.H_kv * ceil_div(hpk, kChunkHeads) * 8;
}

int32_t kivi_attend_mma_take_timeout(int *flag) {
    int zero = 0;
    VQ_CHECK_CUDA(cudaMemcpyFromSymbol(flag, g_attend_timeout, sizeof(int)));
    if (*flag) VQ_CHECK_CUDA(cudaMemcpyToSymbol(g_attend_timeout, &zero, sizeof(int)));
    return VQ_OK;
}

// The driver's tensor-map encoder, looked up once through the runtime (no link against libcuda).
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            ptr = nullptr;
        return (EncodeTiledFn)ptr;
    }();
    return fn;
}

int32_t make_rows_map(int slot, const void *base, int64_t row_bytes, int64_t rows, int64_t stride_bh_bytes, int32_t n_bh,
                      int32_t box_bytes, int32_t box_rows, CUtensorMap *map) {
    // An encoding depends on nothing but these values, so entries never go stale. A decode
    // step calls with one set of buffers per layer: 64 direct-mapped entries per use and thread
    // keep all of them (the driver call costs more than the rest of this function's caller).
    struct Key { const void *ptr; int64_t row_bytes, rows, stride; int32_t n_bh, box_bytes, box_rows; };
    constexpr int kEntries = 64;
    struct Entry { Key key; CUtensorMap map; };
    thread_local Entry cache[4][kEntries] = {};
    const Key key = {base, row_bytes, rows, stride_bh_bytes, n_bh, box_bytes, box_rows};
    const uintptr_t h = reinterpret_cast<uintptr_t>(base) >> 8;
    Entry &e = cache[slot][(h ^ (h >> 6) ^ (h >> 12) ^ (h >> 18)) % kEntries];
    const Key &lk = e.key;
    if (key.ptr == lk.ptr && key.row_bytes == lk.row_bytes && key.rows == lk.rows && key.stride == lk.stride &&
        key.n_bh == lk.n_bh && key.box_bytes == lk.box_bytes && key.box_rows == lk.box_rows) {
        *map = e.map;
        return VQ_OK;
    }
    EncodeTiledFn enc = encode_tiled_fn();
    VQ_REQUIRE(enc != nullptr, VQ_ERR_CUDA, "the driver does not export cuTensorMapEncodeTiled");
    const cuuint64_t dims[3] = {(cuuint64_t)row_bytes, (cuuint64_t)rows, (cuuint64_t)n_bh};
    // (the stride of a dimension of extent 1 is not used for addressing but is still checked)
    const cuuint64_t strides[2] = {(cuuint64_t)row_bytes, (cuuint64_t)std::max<int64_t>(stride_bh_bytes, row_bytes)};
    const cuuint32_t box[3] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    VQ_REQUIRE(r == CUDA_SUCCESS, VQ_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    e.key = key;
    e.map = *map;
    return VQ_OK;
}

// 128-byte lines: the V codes (a unit's rows are contiguous, so a line holds 2 (4-bit) or 4 (2-bit)
// token rows; one box = one 32-token group) and the K scales / zeros (4 lines of 32 floats per group).
static int32_t make_line_map(int slot, const void *base, int64_t lines, int64_t stride_bh_bytes, int32_t n_bh,
                             int32_t box_lines, CUtensorMap *map) {
    return make_rows_map(slot, base, 128, lines, stride_bh_bytes, n_bh, 128, box_lines, map);
}

int32_t kivi_attend_mma_launch(const vq_kivi_attend_args &a, const DeviceInfo &di, cudaStream_t st) {
    Params p;
    {
        const int rb = kD * a.store_bits / 8;
        const int32_t n_bh = a.B * a.H_kv;
        const int64_t groups = a.n_quant / kGroup;
        int32_t rc = make_line_map(0, a.v_codes, a.n_quant * rb / 128, a.v_codes_stride_bh, n_bh, kGroup * rb / 128, &p.v_map);
        if (rc == VQ_OK) rc = make_line_map(1, a.k_scale, groups * 4, a.k_param_stride_bh * 4, n_bh, 4, &p.ks_map);
        if (rc == VQ_OK) rc = make_line_map(2, a.k_zero, groups * 4, a.k_param_stride_bh * 4, n_bh, 4, &p.kz_map);
        if (rc != VQ_OK) return rc;
    }
    p.a = a;
    p.a.gather = nullptr;  // (host pointers: the kernel gets copies of the structs instead)
    p.a.sinks = nullptr;
    p.sinks = vq_kivi_sinks{};
    if (a.sinks != nullptr) {
        const vq_kivi_sinks &sk = *a.sinks;
        VQ_REQUIRE(sk.reserved == 0 && sk.max_rows >= 0 && sk.max_rows <= 4096, VQ_ERR_SHAPE,
                   "vq_kivi_decode_attend: sinks.max_rows=%d must be in 0..4096 (reserved must be 0)", sk.max_rows);
        if (sk.max_rows > 0) {
            VQ_REQUIRE(sk.k && sk.v && sk.k_dead && sk.count, VQ_ERR_SHAPE, "vq_kivi_decode_attend: a sinks pointer is NULL");
            VQ_REQUIRE(is_aligned(sk.k, 16) && is_aligned(sk.v, 16) && is_aligned(sk.k_dead, 16) && sk.stride_bh % 8 == 0 &&
                           sk.stride_bh >= (int64_t)sk.max_rows * kD,
                       VQ_ERR_ALIGN, "vq_kivi_decode_attend: sinks rows must be 16-byte aligned, slabs >= max_rows rows apart");
            p.sinks = sk;
        }
    }
    p.wait_test = knob_take(VQ_KNOB_ATTEND_WAIT_TEST);
    p.gather = vq_peer_gather{};
    if (a.gather != nullptr) {
        const vq_peer_gather &pg = *a.gather;
        VQ_REQUIRE(pg.world >= 1 && pg.world <= VQ_MAX_PEERS && pg.rank >= 0 && pg.rank < pg.world, VQ_ERR_SHAPE,
                   "vq_kivi_decode_attend: gather rank %d of %d is out of range", pg.rank, pg.world);
        VQ_REQUIRE(pg.rank < pg.n_sources && pg.n_sources <= pg.world, VQ_ERR_SHAPE,
                   "vq_kivi_decode_attend: gather rank %d is not one of the %d publishing ranks", pg.rank, pg.n_sources);
        VQ_REQUIRE(pg.state != nullptr && pg.row_offset >= 0, VQ_ERR_SHAPE, "vq_kivi_decode_attend: gather state is NULL");
        for (int r = 0; r < pg.world; ++r)
            VQ_REQUIRE(pg.out[r] != nullptr && pg.flags[r] != nullptr && is_aligned(pg.out[r], 16), VQ_ERR_ALIGN,
                       "vq_kivi_decode_attend: gather buffers of rank %d must be non-NULL and 16-byte aligned", r);
        p.gather = pg;
    }
    p.hpk = a.H_q / a.H_kv;
    p.wide = wide_heads(a);
    p.n_chunks = head_chunks(a);
    p.n_splits = choose_splits(a, di);
    p.groups_total = a.n_quant / kGroup;
    p.groups_per_warp = (int)ceil_div(p.groups_total, (int64_t)p.n_splits * kWarps);
    // a split count that leaves trailing splits empty is trimmed
    p.n_splits = (int)ceil_div(p.groups_total, (int64_t)p.groups_per_warp * kWarps);
    const int64_t recs = (int64_t)a.B * a.H_kv * p.n_splits * p.hpk;
    const int64_t part_bytes = recs * (kD + 2) * (int64_t)sizeof(float);
    const int64_t need = kivi_attend_mma_workspace(a, p.n_splits);
    VQ_REQUIRE(a.workspace != nullptr && a.workspace_bytes >= need, VQ_ERR_CAPACITY,
               "vq_kivi_decode_attend: workspace of %lld bytes needed, %lld given", (long long)need,
               (long long)a.workspace_bytes);
    VQ_REQUIRE(is_aligned(a.workspace, 16), VQ_ERR_ALIGN, "vq_kivi_decode_attend: workspace must be 16-byte aligned");
    p.part_o = (float *)a.workspace;
    p.part_ml = p.part_o + recs * kD;
    p.tickets = reinterpret_cast<unsigned long long *>(static_cast<uint8_t *>(a.workspace) + ((part_bytes + 15) & ~(int64_t)15));
    // a fresh non-zero 48-bit epoch per call: a process-wide counter, salted once per process and
    // mixed (splitmix64), so that small integers or floats left in the workspace cannot equal it
    static const uint64_t salt = [] { std::random_device rd; return ((uint64_t)rd() << 32) ^ rd(); }();
    static std::atomic<uint64_t> next_epoch{1};
    do {
        uint64_t z = (next_epoch.fetch_add(1, std::memory_order_relaxed) ^ salt) + 0x9e3779b97f4a7c15ull;
        z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
        z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
        p.epoch = (z ^ (z >> 31)) >> 16;
    } while (p.epoch == 0);

    dim3 grid(p.n_splits * p.n_chunks, a.H_kv, a.B);
    return a.store_bits == 4 ? launch_bits<4>(p, grid, st) : launch_bits<2>(p, grid, st);
}

}  // namespace vq
