// VecInfer nearest-centroid search on the 5th-generation tensor cores (tcgen05 + TMEM), with
// the exact answer. f16 or bf16 input, sub_dim 8, 16..256 centroids (a multiple of 16), one shared
// codebook or one per sub-space; vq_quant_mma.cu covers the other shapes with warp-level MMAs.
//
// Per 128-row tile one CTA issues two 128 x N x 16 MMAs into a 128-lane x N-column float32
// accumulator in tensor memory:
//     D  = [x | x] . [c_hi | c_lo]^T          (centroid = hi + lo halves: exact products)
//     D += [1 1 1 0 ...] . [h_0 h_1 h_2 0 ...]^T,   h = -|c|^2/2 as the sum of three halves
// so D[row][c] = x_row . c - |c|^2/2, largest for the nearest centroid. Operands sit in shared
// memory in the canonical K-major layout (8-row x 16-byte core matrices, no swizzle); a row of
// x is 16 bytes, so a tile of x is already a stack of core matrices and is brought in with
// one 16-byte cp.async per row. Two threads (one per warpgroup) then own each row and half of its
// columns each. What they must learn from their 128 scores: the column of the best one, and
// whether any other score lies within
//     delta = 2^-16 * (|x|^2 + max|c|^2)
// of it (twice the worst-case difference between this evaluation and the reference's
// sequential float32 one: see vq_quant_mma.cu). One candidate: the answer. Otherwise (near-ties,
// duplicates, a row or a codebook outside the half-precision window) the warp runs the
// reference evaluation order for that row.
//
// With 256 centroids the scores leave tensor memory once (pass_grid): the thread views its 128
// columns as an 8 x 16 grid and keeps the 16 column maxima and the 8 row maxima, one max3 per
// two scores each, i.e. one instruction per score. Two different columns differ in their grid row
// or their grid column, so "exactly one row maximum and exactly one column maximum reach
// best - delta" holds exactly when one score does, and then the two name its place. The 24 maxima
// are counted against the threshold afterwards (48 instructions per thread instead of 256). The
// two halves of a row never wait for each other: each reports (its maximum, its verdict against
// its own maximum) and the half with the larger maximum is believed unless the two maxima are
// within delta of each other.
// Other centroid counts read the accumulator twice, 32 columns per load with the next load in
// flight: pass 1 takes the maximum, pass 2 counts and names the scores within delta of it.
// Two CTAs share an SM (256 accumulator columns each), so one CTA's MMAs run under the other's
// epilogue.
//
// Every wait on the MMA-completion barrier is bounded; on a timeout the CTA raises a device
// flag, skips the tile and still frees its tensor memory before it exits.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "common.cuh"
#include "vq_quant_mma.h"

namespace vq {
namespace {

constexpr int kRows = 128;           // rows (sub-vectors) per tile = accumulator lanes
constexpr int kSub = 8;
constexpr uint32_t kSpin = 1u << 20;

__device__ int g_tc5_timeout = 0;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Shared-memory matrix descriptor, K-major, no swizzle: core matrices of 8 rows x 16 bytes;
// `lbo` = bytes between core matrices that are neighbours along K, `sbo` = along M/N.
__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;  // descriptor version of this architecture
    return d;         // base offset 0, layout type 0 (no swizzle)
}

// Instruction descriptor for kind::f16: f16 x f16 -> f32, both operands K-major, M x N.
// (operand format field: 0 = f16, 1 = bf16)
__device__ __forceinline__ uint32_t make_idesc(int M, int N, bool bf16) {
    const uint32_t fmt = bf16 ? 1u : 0u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit = kSpin) {
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// 32 consecutive accumulator columns of this thread's lane (asynchronous: see tmem_ld_wait).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// The registers written by earlier tmem_ld32 calls may be read after this. The loaded values
// are threaded through the statement so that no use of them can be scheduled ahead of it.
__device__ __forceinline__ void tmem_ld_wait(float (&v)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+f"(v[0]), "+f"(v[1]), "+f"(v[2]), "+f"(v[3]), "+f"(v[4]), "+f"(v[5]), "+f"(v[6]), "+f"(v[7]), "+f"(v[8]),
                   "+f"(v[9]), "+f"(v[10]), "+f"(v[11]), "+f"(v[12]), "+f"(v[13]), "+f"(v[14]), "+f"(v[15]), "+f"(v[16]),
                   "+f"(v[17]), "+f"(v[18]), "+f"(v[19]), "+f"(v[20]), "+f"(v[21]), "+f"(v[22]), "+f"(v[23]), "+f"(v[24]),
                   "+f"(v[25]), "+f"(v[26]), "+f"(v[27]), "+f"(v[28]), "+f"(v[29]), "+f"(v[30]), "+f"(v[31])
                 :
                 : "memory");
}

// acc += k when v >= thr, as exactly one compare and one predicated add.
__device__ __forceinline__ void add_if_ge(float &acc, float v, float thr, float k) {
    asm("{\n\t.reg .pred p;\n\tsetp.ge.f32 p, %1, %2;\n\t@p add.f32 %0, %0, %3;\n\t}" : "+f"(acc) : "f"(v), "f"(thr), "f"(k));
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// The reference evaluation order for one row, spread over the warp (see vq_quant_mma.cu).
template <typename T>
__device__ uint32_t exact_row8(const T *xrow, const float *__restrict__ cb, int n_c, int lane) {
    float xv[kSub];
#pragma unroll
    for (int i = 0; i < kSub; ++i) xv[i] = to_f32<T>(xrow[i]);
    float best = INFINITY;
    uint32_t best_idx = 0xffffffffu;
    for (int c = lane; c < n_c; c += 32) {
        float dist = 0.f;
#pragma unroll
        for (int i = 0; i < kSub; ++i) {
            const float d = __fsub_rn(xv[i], __ldg(cb + (int64_t)c * kSub + i));
            dist = __fadd_rn(dist, __fmul_rn(d, d));
        }
        if (dist < best) { best = dist; best_idx = (uint32_t)c; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, best_idx, o);
        if (ob < best || (ob == best && oi < best_idx)) { best = ob; best_idx = oi; }
    }
    return best_idx == 0xffffffffu ? 0u : best_idx;
}

struct Tc5Smem {
    // every operand region starts on a 128-byte boundary
    uint8_t a[2][2][kRows * 16];   // [stage][K chunk]: the tile of x, twice (K = 16 = x | x)
    uint8_t a2[2][kRows * 16];     // [K chunk]: rows of (1 1 1 0 0 0 0 0 | 0 ...); bf16: four ones, chunk 0 only
    uint8_t b1[2][256 * 16];       // [K chunk]: centroid piece 0 | piece 1
    uint8_t b2[2][256 * 16];       // [K chunk]: (h0 h1 h2 0 ...) | 0; bf16: centroid piece 2 | (h0 h1 h2 h3 0 ...)
    float xch_m[2][kRows];         // row maxima of the two column halves
    float xch_acc[kRows];          // pass-2 results of the upper column half (single pass: its column-maxima verdict)
    float xch_base[kRows];         // (single pass: its row-maxima verdict)
    uint64_t bar;
    uint64_t idle_bar;             // never armed (self-test of the bounded wait)
    uint32_t tmem_base;
    float cmax2;
    int cb_bad;
    int timeout;
};

constexpr int kThreads = 2 * kRows;  // two warpgroups: each owns one half of the columns of every row

// Row maximum over this thread's (up to four) 32-column chunks [c_lo, c_hi). One load is in
// flight while the previous chunk is consumed.
__device__ __forceinline__ float pass_max(uint32_t taddr, int c_lo, int c_hi) {
    float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    if (c_lo >= c_hi) return -INFINITY;
    float va[32], vb[32];
    tmem_ld32(taddr + c_lo, va);
    tmem_ld_wait(va);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int c0 = c_lo + 32 * k;
        if (c0 >= c_hi) break;
        float (&cur)[32] = (k & 1) ? vb : va;
        float (&nxt)[32] = (k & 1) ? va : vb;
        const bool more = c0 + 32 < c_hi;
        if (more) tmem_ld32(taddr + c0 + 32, nxt);
        if (c0 + 32 <= c_hi) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) m4[(i >> 1) & 3] = max3(m4[(i >> 1) & 3], cur[i], cur[i + 1]);
        } else {  // the column count is a multiple of 16: a last half chunk
#pragma unroll
            for (int i = 0; i < 16; i += 2) m4[(i >> 1) & 3] = max3(m4[(i >> 1) & 3], cur[i], cur[i + 1]);
        }
        if (more) tmem_ld_wait(nxt);
    }
    return fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
}

// acc = 65536 * hits + sum of the hits' columns within their 32-column chunks (exact below
// 2^24); base = sum of the chunk offsets of chunks with a hit. With exactly one hit in the row
// its column is (acc - 65536) + base. Per score: one compare and one predicated add of a constant.
__device__ __forceinline__ void pass_count(uint32_t taddr, int c_lo, int c_hi, float thr, float &acc, float &base) {
    acc = 0.f;
    base = 0.f;
    if (c_lo >= c_hi) return;
    float va[32], vb[32];
    tmem_ld32(taddr + c_lo, va);
    tmem_ld_wait(va);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int c0 = c_lo + 32 * k;
        if (c0 >= c_hi) break;
        float (&cur)[32] = (k & 1) ? vb : va;
        float (&nxt)[32] = (k & 1) ? va : vb;
        const bool more = c0 + 32 < c_hi;
        if (more) tmem_ld32(taddr + c0 + 32, nxt);
        float a4[4] = {0.f, 0.f, 0.f, 0.f};
        if (c0 + 32 <= c_hi) {
#pragma unroll
            for (int i = 0; i < 32; ++i) add_if_ge(a4[i & 3], cur[i], thr, 65536.f + (float)i);
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) add_if_ge(a4[i & 3], cur[i], thr, 65536.f + (float)i);
        }
        const float a = (a4[0] + a4[1]) + (a4[2] + a4[3]);
        acc += a;
        if (a >= 65536.f) base += (float)c0;
        if (more) tmem_ld_wait(nxt);
    }
}

// Keeps the values of an array that an earlier tmem_ld32 filled from being read before the
// tcgen05.wait::ld that precedes this statement (both are volatile: they keep their order).
__device__ __forceinline__ void tmem_pin(float (&v)[32]) {
    asm volatile(""
                 : "+f"(v[0]), "+f"(v[1]), "+f"(v[2]), "+f"(v[3]), "+f"(v[4]), "+f"(v[5]), "+f"(v[6]), "+f"(v[7]), "+f"(v[8]),
                   "+f"(v[9]), "+f"(v[10]), "+f"(v[11]), "+f"(v[12]), "+f"(v[13]), "+f"(v[14]), "+f"(v[15]), "+f"(v[16]),
                   "+f"(v[17]), "+f"(v[18]), "+f"(v[19]), "+f"(v[20]), "+f"(v[21]), "+f"(v[22]), "+f"(v[23]), "+f"(v[24]),
                   "+f"(v[25]), "+f"(v[26]), "+f"(v[27]), "+f"(v[28]), "+f"(v[29]), "+f"(v[30]), "+f"(v[31])
                 :
                 : "memory");
}

// Maximum of 16 values in 8 instructions.
__device__ __forceinline__ float max16(const float *c) {
    float m = max3(c[0], c[1], c[2]);
#pragma unroll
    for (int i = 3; i < 15; i += 2) m = max3(m, c[i], c[i + 1]);
    return fmaxf(m, c[15]);
}

// One 32-column chunk = grid rows b0 and b0 + 1: their maxima, and the running column maxima.
template <bool FIRST>
__device__ __forceinline__ void grid_chunk(const float (&cur)[32], float (&P)[16], float &q0, float &q1) {
    q0 = max16(cur);
    q1 = max16(cur + 16);
#pragma unroll
    for (int j = 0; j < 16; ++j) P[j] = FIRST ? fmaxf(cur[j], cur[16 + j]) : max3(P[j], cur[j], cur[16 + j]);
}

// The single pass over this thread's 128 columns [c_lo, c_lo + 128), seen as 8 rows of 16:
// P[j] = maximum of grid column j, Q[k] = maximum of grid row k. Two loads are in flight at a time.
__device__ __forceinline__ void pass_grid(uint32_t taddr, int c_lo, float (&P)[16], float (&Q)[8]) {
    float va[32], vb[32];
    tmem_ld32(taddr + c_lo, va);
    tmem_ld32(taddr + c_lo + 32, vb);
    tmem_ld_wait(va);
    tmem_pin(vb);
    grid_chunk<true>(va, P, Q[0], Q[1]);
    tmem_ld32(taddr + c_lo + 64, va);
    grid_chunk<false>(vb, P, Q[2], Q[3]);
    tmem_ld32(taddr + c_lo + 96, vb);
    tmem_ld_wait(va);
    tmem_pin(vb);
    grid_chunk<false>(va, P, Q[4], Q[5]);
    grid_chunk<false>(vb, P, Q[6], Q[7]);
}

// Verdict of one half against its own maximum m: ap = 65536 * (column maxima >= m - d) + their
// grid columns, aq = 65536 * (row maxima >= m - d) + 16 * their grid rows. One score within d of
// the best: both counts are 1 and the score's column is (ap - 65536) + (aq - 65536).
__device__ __forceinline__ void grid_verdict(const float (&P)[16], const float (&Q)[8], float d, float &m, float &ap, float &aq) {
    m = fmaxf(max3(Q[0], Q[1], Q[2]), max3(Q[3], Q[4], Q[5]));
    m = max3(m, Q[6], Q[7]);
    const float thr = m - d;
    float a4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 16; ++j) add_if_ge(a4[j & 3], P[j], thr, 65536.f + (float)j);
    ap = (a4[0] + a4[1]) + (a4[2] + a4[3]);
    float b4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < 8; ++k) add_if_ge(b4[k & 3], Q[k], thr, 65536.f + 16.f * (float)k);
    aq = (b4[0] + b4[1]) + (b4[2] + b4[3]);
}

// T = __half: operands in f16, centroid = 2 pieces (K slots: x|x against c0|c1, then 1 1 1 against
// the three pieces of h). T = __nv_bfloat16: operands in bf16, whose 8-bit mantissa needs 3
// pieces per centroid and 4 for h: x|x against c0|c1, then x|1 1 1 1 against c2|h0 h1 h2 h3.
// ONEPASS: 256 centroids, the single-pass epilogue (pass_grid); otherwise the two-pass one.
template <typename T, bool ONEPASS>
__global__ void __launch_bounds__(kThreads, 2)
vq_quantize_tc5_kernel(const T *__restrict__ x, int64_t n_vec, const float *__restrict__ cb_all, int n_c, int n_sub,
                       void *__restrict__ indices, int index_bytes, int wait_test) {
    // With one codebook per sub-space (n_sub > 0) a CTA works on sub-space blockIdx.y only: its
    // rows are the sub-vectors sub, sub + n_sub, ... (row i is sub-vector i * vstride + sub).
    const int sub = n_sub > 0 ? blockIdx.y : 0;
    const int64_t vstride = n_sub > 0 ? n_sub : 1;
    const int64_t n = n_sub > 0 ? (n_vec + n_sub - 1 - sub) / n_sub : n_vec;
    const float *__restrict__ cb = cb_all + (int64_t)sub * n_c * kSub;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    Tc5Smem &sm = *reinterpret_cast<Tc5Smem *>(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = tid & (kRows - 1);   // this thread's row of the tile = its accumulator lane
    const int half = tid >> 7;         // which half of the columns it reads
    const int N = n_c;                 // a multiple of 16, <= 256

    // ---- one-time set-up: operand tiles that do not change, barrier, tensor memory ----------
    if (tid == 0) { sm.cmax2 = 0.f; sm.cb_bad = 0; sm.timeout = 0; }
    __syncthreads();
    for (int i = tid; i < 2 * kRows * 16 / 4; i += kThreads) reinterpret_cast<uint32_t *>(sm.a2)[i] = 0u;
    for (int i = tid; i < 2 * 256 * 16 / 4; i += kThreads) reinterpret_cast<uint32_t *>(sm.b2)[i] = 0u;
    __syncthreads();
    constexpr bool BF = std::is_same<T, __nv_bfloat16>::value;
    if (tid < kRows) {
        // a2 chunk 0: every row starts with three (bf16: four) ones
        T *row = reinterpret_cast<T *>(sm.a2[0] + tid * 16);
        row[0] = row[1] = row[2] = from_f32<T>(1.f);
        if (BF) row[3] = from_f32<T>(1.f);
    }
    for (int c = tid; c < N; c += kThreads) {
        float s2 = 0.f, mx = 0.f;
        bool bad = false;
        T *p0 = reinterpret_cast<T *>(sm.b1[0] + c * 16);
        T *p1 = reinterpret_cast<T *>(sm.b1[1] + c * 16);
        T *p2 = reinterpret_cast<T *>(sm.b2[0] + c * 16);  // bf16 only: third piece
#pragma unroll
        for (int k = 0; k < kSub; ++k) {
            const float v = cb[(int64_t)c * kSub + k];
            s2 = fmaf(v, v, s2);
            mx = fmaxf(mx, fabsf(v));
            bad |= !(fabsf(v) <= 64.f);
            const T a0 = from_f32<T>(v);
            const float r1 = v - to_f32<T>(a0);
            const T a1 = from_f32<T>(r1);
            p0[k] = a0;
            p1[k] = a1;
            if (BF) p2[k] = from_f32<T>(r1 - to_f32<T>(a1));
        }
        float h = -0.5f * s2;
        // f16: h pieces in K chunk 0 of the second MMA; bf16: in its chunk 1 (chunk 0 holds c2)
        T *hrow = reinterpret_cast<T *>(sm.b2[BF ? 1 : 0] + c * 16);
#pragma unroll
        for (int k = 0; k < (BF ? 4 : 3); ++k) {
            const T hk = from_f32<T>(h);
            hrow[k] = hk;
            h -= to_f32<T>(hk);
        }
        atomicMax(reinterpret_cast<int *>(&sm.cmax2), __float_as_int(mx * mx));
        if (bad) sm.cb_bad = 1;
    }
    if (tid == 0) {
        const uint32_t bar = smem_u32(&sm.bar);
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&sm.idle_bar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;" ::"r"(smem_u32(&sm.tmem_base)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // generic-proxy writes of the operand tiles must be visible to the tensor core's reads
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sm.tmem_base;
    const float cmax2 = sm.cmax2;
    const bool cb_ok = !sm.cb_bad && cmax2 >= 0.00390625f;

    // K-direction step = distance between the two K chunks of a tile; M/N-direction step = one
    // 128-byte core matrix (8 rows of 16 bytes)
    const uint32_t lbo_a = (uint32_t)(kRows * 16), sbo_a = 128u;
    const uint32_t lbo_b = (uint32_t)(256 * 16), sbo_b = 128u;
    const uint32_t bar = smem_u32(&sm.bar);

    // columns of this thread: the lower or the upper half (in whole 32-column chunks)
    const int n_split = min(N, 128);
    const int c_lo = half ? n_split : 0, c_hi = half ? N : n_split;
    // a warp may only touch the 32 accumulator lanes of its quarter: warp % 4
    const uint32_t taddr = tmem + ((uint32_t)((warp & 3) * 32) << 16);

    const int64_t n_tiles = (n + kRows - 1) / kRows;
    auto fetch = [&](int64_t tile, int stage) {
        if (tid < kRows) {
            const int64_t row = min(tile * kRows + tid, n - 1);
            const T *src = x + (row * vstride + sub) * kSub;
            const uint32_t d0 = smem_u32(sm.a[stage][0] + tid * 16), d1 = smem_u32(sm.a[stage][1] + tid * 16);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d0), "l"(src) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d1), "l"(src) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // Per tile: [barrier A] MMAs of this tile issued | results of the previous tile written, next
    // tile of x requested, row norms | [barrier B] MMAs done | pass 1 | [barrier C] | pass 2.
    // The MMAs therefore run under the previous tile's result handling.
    int64_t tile = blockIdx.x;
    if (tile < n_tiles) fetch(tile, 0);
    uint32_t phase = 0;
    bool timed_out = false;
    // results of the previous tile, finished after barrier A of the next one
    float prev_acc = 0.f, prev_base = 0.f, prev_m = 0.f, prev_d = 0.f;
    bool prev_bad = false, have_prev = false;
    int64_t prev_tile = 0;
    auto finish_prev = [&]() {
        if (!have_prev || half != 0) return;
        const int64_t row = prev_tile * kRows + r;
        bool slow;
        uint32_t idx;
        if constexpr (ONEPASS) {
            // the half with the larger maximum holds the best score; the other half holds a
            // candidate too when the maxima are within delta (also true when either is NaN)
            const float m1 = sm.xch_m[1][r];
            const bool upper = m1 > prev_m;
            const float ap = upper ? sm.xch_acc[r] : prev_acc, aq = upper ? sm.xch_base[r] : prev_base;
            const bool both = !(fabsf(prev_m - m1) > prev_d);
            const bool one = ap >= 65536.f && ap < 131072.f && aq >= 65536.f && aq < 131072.f;
            slow = prev_bad || both || !one;
            idx = (uint32_t)((int)ap + (int)aq - 131072 + (upper ? 128 : 0)) & 0xffffu;
        } else {
            const float acc = prev_acc + sm.xch_acc[r], base = prev_base + sm.xch_base[r];
            slow = prev_bad || !(acc >= 65536.f && acc < 131072.f);
            idx = (uint32_t)((int)acc - 65536 + (int)base) & 0xffffu;
        }
        // rows that need the reference order: the whole warp works on each in turn
        uint32_t slow_mask = __ballot_sync(0xffffffffu, slow && row < n && !timed_out);
        while (slow_mask) {
            const int src = __ffs(slow_mask) - 1;
            slow_mask &= slow_mask - 1;
            const int64_t srow = prev_tile * kRows + warp * 32 + src;
            const uint32_t e = exact_row8(x + (srow * vstride + sub) * kSub, cb, n_c, lane);
            if (lane == src) idx = e;
        }
        if (row < n && !timed_out) {
            const int64_t o = row * vstride + sub;
            if (index_bytes == 1) reinterpret_cast<uint8_t *>(indices)[o] = (uint8_t)idx;
            else if (index_bytes == 2) reinterpret_cast<uint16_t *>(indices)[o] = (uint16_t)idx;
            else reinterpret_cast<uint32_t *>(indices)[o] = idx;
        }
    };
    for (int it = 0; tile < n_tiles; tile += gridDim.x, ++it) {
        const int stage = it & 1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();  // A: this tile of x is in place; pass 2 of the previous tile has released tensor memory
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // (descriptors are rebuilt here, by the one thread that uses them, rather than kept in
            // every thread's registers across the epilogue)
            const uint64_t desc_a2 = make_desc(smem_u32(sm.a2[0]), lbo_a, sbo_a);
            const uint64_t desc_b1 = make_desc(smem_u32(sm.b1[0]), lbo_b, sbo_b);
            const uint64_t desc_b2 = make_desc(smem_u32(sm.b2[0]), lbo_b, sbo_b);
            const uint32_t idesc = make_idesc(kRows, N, BF);
            const uint64_t desc_a = make_desc(smem_u32(sm.a[stage][0]), lbo_a, sbo_a);
            mma_f16_ss(tmem, desc_a, desc_b1, idesc, 0u);
            if (BF) {
                // second MMA of the bf16 form: x again (against c2) | the constant ones (against h)
                const uint32_t a0 = smem_u32(sm.a[stage][0]);
                mma_f16_ss(tmem, make_desc(a0, smem_u32(sm.a2[0]) - a0, sbo_a), desc_b2, idesc, 1u);
            } else {
                mma_f16_ss(tmem, desc_a2, desc_b2, idesc, 1u);
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
        }
        finish_prev();
        if (tile + gridDim.x < n_tiles) fetch(tile + gridDim.x, stage ^ 1);

        // this thread's row: squared norm and range check from the shared-memory copy
        float xn = 0.f;
        bool bad = !cb_ok;
        {
            const uint4 raw = *reinterpret_cast<const uint4 *>(sm.a[stage][0] + r * 16);
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float2 f;
                if (BF) f = make_float2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xffff0000u));
                else f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
                xn = fmaf(f.x, f.x, fmaf(f.y, f.y, xn));
                bad |= !(fabsf(f.x) <= 32768.f && fabsf(f.y) <= 32768.f);
            }
        }
        // One thread polls the completion barrier; the others block on the CTA barrier, which
        // costs no issue slots (256 spinning threads took a fifth of the SM's issue slots away
        // from the other CTA's epilogue).
        if (tid == 0) {
            if (!timed_out && !mbar_wait(bar, phase)) sm.timeout = 1;
        }
        phase ^= 1u;
        __syncthreads();  // B
        timed_out = sm.timeout != 0;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

        // bf16: ~30 float32 roundings per score instead of ~20: the margin is doubled
        const float delta = (BF ? 3.0517578125e-05f : 1.52587890625e-05f) * (xn + cmax2);
        float acc = 0.f, base = 0.f;
        if constexpr (ONEPASS) {
            // ---- the single pass: 24 maxima of this half, then its verdict ----------------------
            float m = 0.f;
            if (!timed_out) {
                float P[16], Q[8];
                pass_grid(taddr, c_lo, P, Q);
                grid_verdict(P, Q, delta, m, acc, base);
            }
            if (half) { sm.xch_m[1][r] = m; sm.xch_acc[r] = acc; sm.xch_base[r] = base; }
            prev_m = m; prev_d = delta;
        } else {
            // ---- pass 1: the row's best score (each half of the columns, then exchanged) --------
            sm.xch_m[half][r] = timed_out ? 0.f : pass_max(taddr, c_lo, c_hi);
            __syncthreads();  // C
            const float m = fmaxf(sm.xch_m[0][r], sm.xch_m[1][r]);
            const float thr = m - delta;
            // ---- pass 2: count and name the scores within delta of it --------------------------
            if (!timed_out) pass_count(taddr, c_lo, c_hi, thr, acc, base);
            if (half) { sm.xch_acc[r] = acc; sm.xch_base[r] = base; }
        }
        prev_acc = acc; prev_base = base; prev_bad = bad; prev_tile = tile; have_prev = true;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    finish_prev();
    if (timed_out && lane == 0) atomicExch(&g_tc5_timeout, 1);
    // Self-test of the bounded wait, after all the work: a barrier that nothing arms never
    // completes its phase, so this wait runs out and the flag is raised (indices stay valid).
    if (wait_test && tid == 0 && !mbar_wait(smem_u32(&sm.idle_bar), 0u, 1u << 10)) atomicExch(&g_tc5_timeout, 1);
    // ---- release tensor memory on every path ---------------------------------------------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" ::"r"(tmem) : "memory");
    }
}

}  // namespace

bool vq_quantize_tc5_supported(const void *x, int32_t x_dtype, int64_t n, int32_t sub_dim, int32_t n_c, int32_t n_sub) {
    // 0 choose; 1 tcgen05 / 2 mma.sync / 3 exact pin one search; 4 = tcgen05 with the two-pass epilogue
    const int mode = knob_get(VQ_KNOB_VQ_SEARCH);
    if (mode == 2 || mode == 3) return false;
    if ((x_dtype != VQ_F16 && x_dtype != VQ_BF16) || sub_dim != kSub || n_sub < 0 || n_sub > 65535) return false;
    if (n_c < 16 || n_c > 256 || n_c % 16) return false;
    if (!is_aligned(x, 16)) return false;
    const bool forced = mode == 1 || mode == 4;
    return forced ? n >= 1 : n >= 4096;  // small inputs: the CUDA-core search has no set-up cost
}

int32_t vq_quantize_tc5_launch(const void *x, int32_t x_dtype, int64_t n, const float *cb, int32_t n_c, int32_t n_sub,
                               void *indices, int32_t index_bytes, cudaStream_t st) {
    DeviceInfo di;
    int32_t rc = device_info(&di);
    if (rc != VQ_OK) return rc;
    // Two CTAs per SM: each holds 256 of the SM's 512 accumulator columns. The shared-memory
    // request is padded so that a third CTA (which would wait for columns) cannot be resident.
    const size_t smem = std::max(sizeof(Tc5Smem) + 128, (size_t)80 * 1024);
    // 256 centroids take the single-pass epilogue (knob value 4 pins the two-pass one, to measure it)
    const bool onepass = n_c == 256 && knob_get(VQ_KNOB_VQ_SEARCH) != 4;
    VQ_CHECK_CUDA(cudaFuncSetAttribute(vq_quantize_tc5_kernel<__half, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    VQ_CHECK_CUDA(cudaFuncSetAttribute(vq_quantize_tc5_kernel<__nv_bfloat16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    VQ_CHECK_CUDA(cudaFuncSetAttribute(vq_quantize_tc5_kernel<__half, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    VQ_CHECK_CUDA(cudaFuncSetAttribute(vq_quantize_tc5_kernel<__nv_bfloat16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int ny = n_sub > 0 ? n_sub : 1;
    const int64_t n_tiles = ceil_div(ceil_div(n, ny), kRows);
    const int64_t fill = std::max<int64_t>(1, ceil_div((int64_t)di.sm_count * 2, ny));  // CTAs per sub-space for two per SM
    const unsigned blocks = (unsigned)std::max<int64_t>(1, std::min<int64_t>(n_tiles, fill));
    const int wait_test = knob_take(VQ_KNOB_VQ_WAIT_TEST);
    const dim3 grid(blocks, ny);
    if (x_dtype == VQ_BF16) {
        const auto *xp = (const __nv_bfloat16 *)x;
        if (onepass) vq_quantize_tc5_kernel<__nv_bfloat16, true><<<grid, kThreads, smem, st>>>(xp, n, cb, n_c, n_sub, indices, index_bytes, wait_test);
        else vq_quantize_tc5_kernel<__nv_bfloat16, false><<<grid, kThreads, smem, st>>>(xp, n, cb, n_c, n_sub, indices, index_bytes, wait_test);
    } else {
        const auto *xp = (const __half *)x;
        if (onepass) vq_quantize_tc5_kernel<__half, true><<<grid, kThreads, smem, st>>>(xp, n, cb, n_c, n_sub, indices, index_bytes, wait_test);
        else vq_quantize_tc5_kernel<__half, false><<<grid, kThreads, smem, st>>>(xp, n, cb, n_c, n_sub, indices, index_bytes, wait_test);
    }
    VQ_CHECK_LAUNCH("vq_quantize_tc5_kernel");
    return VQ_OK;
}

int32_t vq_quantize_tc5_take_timeout(int *flag) {
    VQ_CHECK_CUDA(cudaDeviceSynchronize());
    int zero = 0;
    VQ_CHECK_CUDA(cudaMemcpyFromSymbol(flag, g_tc5_timeout, sizeof(int)));
    VQ_CHECK_CUDA(cudaMemcpyToSymbol(g_tc5_timeout, &zero, sizeof(int)));
    return VQ_OK;
}

}  // namespace vq
