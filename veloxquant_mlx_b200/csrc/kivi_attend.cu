// Fused dequant + softmax attention over packed KIVI codes: entry point, the general
// CUDA-core kernel (any container width, group size, head_dim <= 256, any query length)
// and the split merge. The tensor-core kernel for the serving shape lives in
// kivi_attend_mma.cu and is selected here when its preconditions hold.
#include <algorithm>

#include "common.cuh"
#include "kivi_attend.h"

namespace vq {

constexpr int kGenWarps = 4;
constexpr int kGenHeads = 4;   // query heads of one KV head handled per CTA
constexpr int kGenMaxDS = 8;   // ceil(256 / 32)

// One CTA: one (batch, kv head, query row, chunk of <= 4 query heads, context split).
// Warp w walks tokens start+w, start+w+4, ...; lanes split head_dim.
__global__ void __launch_bounds__(kGenWarps * 32)
kivi_attend_general_kernel(const vq_kivi_attend_args a, int n_splits, int n_head_chunks,
                           float *__restrict__ part_o, float *__restrict__ part_ml) {
    __shared__ float sh_q[kGenHeads][256];
    __shared__ float sh_o[kGenWarps][kGenHeads][256];
    __shared__ float sh_m[kGenWarps][kGenHeads];
    __shared__ float sh_l[kGenWarps][kGenHeads];

    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the merge kernel may become resident
    const int split = blockIdx.x;
    const int hpk = a.H_q / a.H_kv;
    int y = blockIdx.y;
    const int hc = y % n_head_chunks; y /= n_head_chunks;
    const int sq = y % a.S_q;
    const int hkv = y / a.S_q;
    const int b = blockIdx.z;
    const int D = a.D;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h0 = hc * kGenHeads;                      // first head (within the kv group)
    const int nh = min(kGenHeads, hpk - h0);
    const int64_t bh = (int64_t)b * a.H_kv + hkv;

    for (int i = threadIdx.x; i < nh * D; i += blockDim.x) {
        const int hp = i / D, d = i % D;
        const int hq = hkv * hpk + h0 + hp;
        sh_q[hp][d] = load_as_f32(a.q, a.q_dtype, (((int64_t)b * a.H_q + hq) * a.S_q + sq) * D + d);
    }
    __syncthreads();

    // slots this query row sees: all of them, or (tail-aligned causal mask) those up to its own
    const int total = (a.flags & VQ_ATTEND_CAUSAL) ? a.n_quant + a.n_res - a.S_q + sq + 1 : a.n_quant + a.n_res;
    const int chunk = (total + n_splits - 1) / n_splits;
    const int t_begin = split * chunk;
    const int t_end = min(total, t_begin + chunk);
    const int sb = a.store_bits;
    const int64_t row_bytes = (int64_t)D * sb / 8;
    const int gv = (D + a.group - 1) / a.group;
    const int nd = (D + 31) / 32;

    float run_m[kGenHeads], run_l[kGenHeads], acc[kGenHeads][kGenMaxDS];
#pragma unroll
    for (int hp = 0; hp < kGenHeads; ++hp) {
        run_m[hp] = -INFINITY;
        run_l[hp] = 0.f;
#pragma unroll
        for (int i = 0; i < kGenMaxDS; ++i) acc[hp][i] = 0.f;
    }

    for (int t = t_begin + warp; t < t_end; t += kGenWarps) {
        float kd[kGenMaxDS], vd[kGenMaxDS];
        if (t < a.n_quant) {
            const uint8_t *krow = a.k_codes + bh * a.k_codes_stride_bh + (int64_t)t * row_bytes;
            const uint8_t *vrow = a.v_codes + bh * a.v_codes_stride_bh + (int64_t)t * row_bytes;
            const int64_t kp = bh * a.k_param_stride_bh + (int64_t)(t / a.group) * D;
            const int64_t vp = bh * a.v_param_stride_bh + (int64_t)t * gv;
#pragma unroll
            for (int i = 0; i < kGenMaxDS; ++i) {
                const int d = lane + 32 * i;
                kd[i] = vd[i] = 0.f;
                if (i < nd && d < D) {
                    kd[i] = (float)load_code(krow, d, sb) * a.k_scale[kp + d] + a.k_zero[kp + d];
                    vd[i] = (float)load_code(vrow, d, sb) * a.v_scale[vp + d / a.group] + a.v_zero[vp + d / a.group];
                }
            }
        } else {
            const int64_t r = bh * a.res_stride_bh + (int64_t)(t - a.n_quant) * D;
#pragma unroll
            for (int i = 0; i < kGenMaxDS; ++i) {
                const int d = lane + 32 * i;
                kd[i] = vd[i] = 0.f;
                if (i < nd && d < D) {
                    kd[i] = load_as_f32(a.k_res, a.res_dtype, r + d);
                    vd[i] = load_as_f32(a.v_res, a.res_dtype, r + d);
                }
            }
        }
#pragma unroll
        for (int hp = 0; hp < kGenHeads; ++hp) {
            if (hp < nh) {
                float dot = 0.f;
#pragma unroll
                for (int i = 0; i < kGenMaxDS; ++i)
                    if (i < nd) dot += sh_q[hp][(lane + 32 * i) < D ? lane + 32 * i : 0] * kd[i];
                const float s = warp_sum(dot) * a.scale;
                const float m_new = fmaxf(run_m[hp], s);
                const float factor = __expf(run_m[hp] - m_new);
                const float w = __expf(s - m_new);
                run_l[hp] = run_l[hp] * factor + w;
                run_m[hp] = m_new;
#pragma unroll
                for (int i = 0; i < kGenMaxDS; ++i) acc[hp][i] = acc[hp][i] * factor + w * vd[i];
            }
        }
    }

    // merge the warps of this CTA
    for (int hp = 0; hp < nh; ++hp) {
        if (lane == 0) { sh_m[warp][hp] = run_m[hp]; sh_l[warp][hp] = run_l[hp]; }
        for (int i = 0; i < nd; ++i) {
            const int d = lane + 32 * i;
            if (d < D) sh_o[warp][hp][d] = acc[hp][i];
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nh * D; i += blockDim.x) {
        const int hp = i / D, d = i % D;
        float gm = -INFINITY;
        for (int w = 0; w < kGenWarps; ++w) gm = fmaxf(gm, sh_m[w][hp]);
        float gl = 0.f, o = 0.f;
        for (int w = 0; w < kGenWarps; ++w) {
            const float f = (sh_m[w][hp] == -INFINITY) ? 0.f : __expf(sh_m[w][hp] - gm);
            gl += sh_l[w][hp] * f;
            o += sh_o[w][hp][d] * f;
        }
        const int hq = hkv * hpk + h0 + hp;
        const int64_t row = ((int64_t)b * a.H_q + hq) * a.S_q + sq;
        if (n_splits == 1) {
            store_from_f32(a.out, a.out_dtype, row * D + d, o / gl);
        } else {
            part_o[(row * n_splits + split) * D + d] = o;
            if (d == 0) {
                part_ml[(row * n_splits + split) * 2 + 0] = gm;
                part_ml[(row * n_splits + split) * 2 + 1] = gl;
            }
        }
    }
}

// Combine the per-split partial softmaxes: one CTA per output row. The split weights
// exp(m_s - M) are computed once into shared memory (n_splits <= 256); the sum over splits is
// unrolled so that several independent loads are in flight (the loop is latency-bound).
__global__ void __launch_bounds__(128)
kivi_attend_merge_kernel(const float *__restrict__ part_o, const float *__restrict__ part_ml,
                         int n_splits, int D, void *__restrict__ out, int out_dtype) {
    __shared__ float sh_w[256];
    __shared__ float sh_red[4];
    const int64_t row = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float *ml = part_ml + row * n_splits * 2;
    const float *po = part_o + row * n_splits * D;
    // the partials are complete and visible only after the grid that wrote them has finished
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // One round trip to memory: the (max, sum) pairs of this thread's splits (at most two) and
    // the first 8 partial rows of its first output column are requested together.
    float2 mls[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int s = tid + 128 * i;
        mls[i] = s < n_splits ? make_float2(ml[2 * s], ml[2 * s + 1]) : make_float2(-INFINITY, 0.f);
    }
    float first[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) first[u] = (u < n_splits && tid < D) ? po[(int64_t)u * D + tid] : 0.f;
    float m = warp_max(fmaxf(mls[0].x, mls[1].x));
    if (lane == 0) sh_red[warp] = m;
    __syncthreads();
    const float gm = fmaxf(fmaxf(sh_red[0], sh_red[1]), fmaxf(sh_red[2], sh_red[3]));
    __syncthreads();
    float l = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int s = tid + 128 * i;
        if (s < n_splits) {
            const float w = (mls[i].x == -INFINITY) ? 0.f : __expf(mls[i].x - gm);
            sh_w[s] = w;
            l += mls[i].y * w;
        }
    }
    l = warp_sum(l);
    if (lane == 0) sh_red[warp] = l;
    __syncthreads();
    const float gl = (sh_red[0] + sh_red[1]) + (sh_red[2] + sh_red[3]);
    for (int d = tid; d < D; d += 128) {
        float acc = 0.f;
        int s = 0;
        if (d == tid) {  // the rows requested up front
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (u < n_splits) acc = fmaf(first[u], sh_w[u], acc);
            s = min(8, n_splits);
        }
        for (; s + 8 <= n_splits; s += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = po[(int64_t)(s + u) * D + d];
#pragma unroll
            for (int u = 0; u < 8; ++u) acc = fmaf(v[u], sh_w[s + u], acc);
        }
        for (; s < n_splits; ++s) acc = fmaf(po[(int64_t)s * D + d], sh_w[s], acc);
        store_from_f32(out, out_dtype, row * D + d, acc / gl);
    }
}

int32_t launch_split_merge(const float *part_o, const float *part_ml, int n_splits, int D, void *out,
                           int out_dtype, int64_t rows, cudaStream_t st) {
    VQ_REQUIRE(rows < (1ll << 31), VQ_ERR_SHAPE, "split merge: too many output rows");
    VQ_REQUIRE(n_splits <= 256, VQ_ERR_SHAPE, "split merge: at most 256 splits, got %d", n_splits);
    // Launched as a programmatic dependent of whatever precedes it in the stream (the kernel that
    // writes the partials): its CTAs may become resident while that grid drains; the kernel's
    // first instruction waits for the grid's completion.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)rows);
    cfg.blockDim = dim3(128);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    VQ_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kivi_attend_merge_kernel, part_o, part_ml, n_splits, D, out, out_dtype));
    return VQ_OK;
}

static int32_t validate(const vq_kivi_attend_args &a) {
    VQ_REQUIRE(a.B >= 1 && a.H_q >= 1 && a.H_kv >= 1 && a.S_q >= 1, VQ_ERR_SHAPE, "vq_kivi_decode_attend: B, H_q, H_kv, S_q must be >= 1");
    VQ_REQUIRE(a.D >= 1 && a.D <= 256, VQ_ERR_SHAPE, "vq_kivi_decode_attend: D=%d must be in 1..256", a.D);
    VQ_REQUIRE(a.H_q % a.H_kv == 0, VQ_ERR_SHAPE, "vq_kivi_decode_attend: H_q=%d must be a multiple of H_kv=%d", a.H_q, a.H_kv);
    VQ_REQUIRE(a.H_q / a.H_kv <= 16, VQ_ERR_SHAPE, "vq_kivi_decode_attend: heads_per_kv=%d exceeds the supported maximum of 16", a.H_q / a.H_kv);
    VQ_REQUIRE(a.n_quant >= 0 && a.n_res >= 0 && a.n_quant + a.n_res >= 1, VQ_ERR_SHAPE, "vq_kivi_decode_attend: nothing to attend over");
    VQ_REQUIRE(a.q && a.out, VQ_ERR_SHAPE, "vq_kivi_decode_attend: q/out is NULL");
    VQ_REQUIRE(a.q_dtype >= 0 && a.q_dtype <= 2 && a.out_dtype >= 0 && a.out_dtype <= 2, VQ_ERR_DTYPE, "vq_kivi_decode_attend: bad q/out dtype");
    if (a.n_quant > 0) {
        const int sb = a.store_bits;
        VQ_REQUIRE(sb == 1 || sb == 2 || sb == 4 || sb == 8, VQ_ERR_SHAPE, "vq_kivi_decode_attend: store_bits must be 1, 2, 4 or 8, got %d", sb);
        VQ_REQUIRE(a.group >= 1, VQ_ERR_SHAPE, "vq_kivi_decode_attend: group must be >= 1");
        VQ_REQUIRE(((int64_t)a.D * sb) % 8 == 0, VQ_ERR_SHAPE, "vq_kivi_decode_attend: D*store_bits must be a multiple of 8");
        VQ_REQUIRE(a.k_codes && a.v_codes && a.k_scale && a.k_zero && a.v_scale && a.v_zero, VQ_ERR_SHAPE, "vq_kivi_decode_attend: a quantized tensor is NULL");
    }
    if (a.n_res > 0) {
        VQ_REQUIRE(a.k_res && a.v_res, VQ_ERR_SHAPE, "vq_kivi_decode_attend: residual tensor is NULL");
        VQ_REQUIRE(a.res_dtype >= 0 && a.res_dtype <= 2, VQ_ERR_DTYPE, "vq_kivi_decode_attend: bad residual dtype");
    }
    return VQ_OK;
}

static int general_splits(const vq_kivi_attend_args &a, int sm_count) {
    if (a.n_splits > 0) return std::min(a.n_splits, 256);
    const int total = a.n_quant + a.n_res;
    const int hpk = a.H_q / a.H_kv;
    const int64_t ctas = (int64_t)a.B * a.H_kv * a.S_q * ceil_div(hpk, kGenHeads);
    int64_t want = ceil_div((int64_t)sm_count * 4, ctas);
    want = std::min<int64_t>(want, ceil_div(total, 64));
    return (int)std::max<int64_t>(1, std::min<int64_t>(want, 256));
}

}  // namespace vq

extern "C" int64_t vq_kivi_attend_workspace_bytes(const vq_kivi_attend_args *args) {
    using namespace vq;
    if (!args) return 0;
    const vq_kivi_attend_args &a = *args;
    if (a.B < 1 || a.H_q < 1 || a.S_q < 1 || a.D < 1) return 0;
    // Room for the split count of whichever kernel the call will pick (+1 part for the tail).
    DeviceInfo di;
    if (device_info(&di) != VQ_OK) { di.sm_count = 148; di.smem_optin = 227 * 1024; }
    const int64_t rows = (int64_t)a.B * a.H_q * a.S_q;
    int64_t need = rows * general_splits(a, di.sm_count) * ((int64_t)a.D + 2) * (int64_t)sizeof(float);
    if (a.variant != 1 && a.H_kv >= 1 && a.H_q % a.H_kv == 0 && kivi_attend_mma_supported(a) == nullptr)
        need = std::max<int64_t>(need, kivi_attend_mma_workspace(a, kivi_attend_mma_splits(a, di)));
    return need + 256;
}

extern "C" int32_t vq_kivi_attend_splits(const vq_kivi_attend_args *args) {
    using namespace vq;
    if (!args) return 0;
    const vq_kivi_attend_args &a = *args;
    if (a.B < 1 || a.H_q < 1 || a.H_kv < 1 || a.S_q < 1 || a.D < 1 || a.H_q % a.H_kv) return 0;
    DeviceInfo di;
    if (device_info(&di) != VQ_OK) { di.sm_count = 148; di.smem_optin = 227 * 1024; }
    if (a.variant != 1 && kivi_attend_mma_supported(a) == nullptr) return kivi_attend_mma_splits(a, di);
    return general_splits(a, di.sm_count);
}

extern "C" int32_t vq_kivi_attend_status(void) {
    using namespace vq;
    int flag = 0, flag2 = 0, flag3 = 0;
    int32_t rc = kivi_attend_mma_take_timeout(&flag);
    if (rc != VQ_OK) return rc;
    rc = coded_attend_take_timeout(&flag2);
    if (rc != VQ_OK) return rc;
    rc = peer_gather_take_timeout(&flag3);
    if (rc != VQ_OK) return rc;
    if (flag3) return fail(VQ_ERR_TIMEOUT, "vq_peer_gather_wait: a peer's output rows did not arrive within the poll limit");
    if (flag) return fail(VQ_ERR_TIMEOUT, "vq_kivi_decode_attend: a bounded wait on a bulk-copy barrier gave up");
    if (flag2) return fail(VQ_ERR_TIMEOUT, "vq_rabitq_decode_attend: a bounded wait on a bulk-copy barrier gave up");
    return VQ_OK;
}

extern "C" int32_t vq_kivi_decode_attend(const vq_kivi_attend_args *args, void *stream) {
    using namespace vq;
    VQ_REQUIRE(args != nullptr, VQ_ERR_SHAPE, "vq_kivi_decode_attend: args is NULL");
    const vq_kivi_attend_args &a = *args;
    int32_t rc = validate(a);
    if (rc != VQ_OK) return rc;
    DeviceInfo di;
    rc = device_info(&di);
    if (rc != VQ_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;

    VQ_REQUIRE(a.reserved == 0 && (a.flags & ~(VQ_ATTEND_OVERLAP_PREVIOUS | VQ_ATTEND_CAUSAL)) == 0, VQ_ERR_SHAPE,
               "vq_kivi_decode_attend: unknown bits in flags (%d) or reserved (%d)", a.flags, a.reserved);
    VQ_REQUIRE(!(a.flags & VQ_ATTEND_CAUSAL) || a.S_q <= a.n_quant + a.n_res, VQ_ERR_SHAPE,
               "vq_kivi_decode_attend: causal mask with S_q=%d query rows over %d slots", a.S_q, a.n_quant + a.n_res);
    if (a.variant != 1) {
        const char *why = kivi_attend_mma_supported(a);
        if (why == nullptr) return kivi_attend_mma_launch(a, di, st);
        VQ_REQUIRE(a.variant != 2, VQ_ERR_SHAPE, "vq_kivi_decode_attend: tensor-core kernel unavailable: %s", why);
    }

    VQ_REQUIRE(a.sinks == nullptr, VQ_ERR_SHAPE,
               "vq_kivi_decode_attend: protected tokens (sinks) need the tensor-core kernel: %s",
               a.variant == 1 ? "variant 1 was forced" : kivi_attend_mma_supported(a));
    VQ_REQUIRE(a.gather == nullptr, VQ_ERR_SHAPE,
               "vq_kivi_decode_attend: publishing to peers (gather) needs the tensor-core kernel: %s",
               a.variant == 1 ? "variant 1 was forced" : kivi_attend_mma_supported(a));
    const int n_splits = general_splits(a, di.sm_count);
    const int64_t rows = (int64_t)a.B * a.H_q * a.S_q;
    float *part_o = nullptr, *part_ml = nullptr;
    if (n_splits > 1) {
        const int64_t need = rows * n_splits * ((int64_t)a.D + 2) * (int64_t)sizeof(float);
        VQ_REQUIRE(a.workspace != nullptr && a.workspace_bytes >= need, VQ_ERR_CAPACITY,
                   "vq_kivi_decode_attend: workspace of %lld bytes needed, %lld given", (long long)need, (long long)a.workspace_bytes);
        VQ_REQUIRE(is_aligned(a.workspace, 16), VQ_ERR_ALIGN, "vq_kivi_decode_attend: workspace must be 16-byte aligned");
        part_o = (float *)a.workspace;
        part_ml = part_o + rows * n_splits * a.D;
    }
    const int hpk = a.H_q / a.H_kv;
    const int n_head_chunks = (int)ceil_div(hpk, kGenHeads);
    const int64_t gy = (int64_t)a.H_kv * a.S_q * n_head_chunks;
    VQ_REQUIRE(gy <= 65535 && a.B <= 65535, VQ_ERR_SHAPE, "vq_kivi_decode_attend: grid too large (H_kv*S_q*chunks=%lld, B=%d)", (long long)gy, a.B);
    dim3 grid(n_splits, (unsigned)gy, a.B);
    kivi_attend_general_kernel<<<grid, kGenWarps * 32, 0, st>>>(a, n_splits, n_head_chunks, part_o, part_ml);
    VQ_CHECK_LAUNCH("kivi_attend_general_kernel");
    if (n_splits > 1) {
        kivi_attend_merge_kernel<<<(unsigned)rows, 128, 0, st>>>(part_o, part_ml, n_splits, a.D, a.out, a.out_dtype);
        VQ_CHECK_LAUNCH("kivi_attend_merge_kernel");
    }
    return VQ_OK;
}

extern "C" int32_t vq_predecoded_attend(const vq_kivi_attend_args *args, void *stream) {
    using namespace vq;
    VQ_REQUIRE(args != nullptr, VQ_ERR_SHAPE, "vq_predecoded_attend: args is NULL");
    VQ_REQUIRE(args->n_res >= 1 && args->k_res && args->v_res, VQ_ERR_SHAPE, "vq_predecoded_attend: k_res/v_res with n_res >= 1 rows are required");
    vq_kivi_attend_args a = *args;
    a.n_quant = 0;
    return vq_kivi_decode_attend(&a, stream);
}

extern "C" int32_t vq_lse_merge(const float *part_o, const float *part_ml, int64_t rows, int32_t n_splits,
                                int32_t D, void *out, int32_t out_dtype, void *stream) {
    using namespace vq;
    VQ_REQUIRE(rows >= 0 && n_splits >= 1 && D >= 1, VQ_ERR_SHAPE, "vq_lse_merge: bad sizes (rows=%lld, n_splits=%d, D=%d)", (long long)rows, n_splits, D);
    VQ_REQUIRE(out_dtype >= 0 && out_dtype <= 2, VQ_ERR_DTYPE, "vq_lse_merge: unknown dtype %d", out_dtype);
    if (rows == 0) return VQ_OK;
    VQ_REQUIRE(part_o && part_ml && out, VQ_ERR_SHAPE, "vq_lse_merge: NULL argument");
    return launch_split_merge(part_o, part_ml, n_splits, D, out, out_dtype, rows, (cudaStream_t)stream);
}
