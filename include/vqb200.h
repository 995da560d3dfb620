/*
 * vqb200.h -- C ABI of libvqb200.so: the compressed-KV hot path for NVIDIA B200 (sm_100a).
 *
 * Quantize-on-append (KIVI group-affine codes, VecInfer product-VQ indices, RaBitQ sign
 * bits) and fused dequant + single-query attention over the packed codes.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer owned by the caller unless stated otherwise; the
 *     library never allocates. Scratch memory is passed in as `workspace`, sized by the
 *     matching `*_workspace_bytes` query. Successive calls on one stream may share a workspace.
 *   - Every call is asynchronous on `stream` (a cudaStream_t passed as void*; NULL = the
 *     legacy default stream) and returns a vq_status (0 = ok, negative = error). After a
 *     non-zero return `vq_last_error()` holds a thread-local, human-readable reason.
 *   - Tensors are row-major and contiguous in their trailing axes; leading (batch*head)
 *     slabs are addressed through explicit strides so a caller can hand in slices of
 *     larger pre-allocated cache buffers.
 *   - Packed codes: element i of a row occupies bits [i*sb, (i+1)*sb) of the row's
 *     little-endian bit stream (sb = container width 1, 2, 4 or 8), i.e. consecutive
 *     channels of head_dim are packed LSB first. This is the reference's convention:
 *     veloxquant_mlx/dsa/bit_pack.py:120-139,198-220 and metal/src/bit_pack.metal:8-19.
 *
 * Each entry point names the reference interface it replaces (paths relative to the
 * reference project root).
 */
#ifndef VQB200_H
#define VQB200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum vq_status {
    VQ_OK = 0,
    VQ_ERR_SHAPE = -1,    /* bad dimension / unsupported size */
    VQ_ERR_DTYPE = -2,    /* unknown dtype code */
    VQ_ERR_ALIGN = -3,    /* pointer or stride not aligned as required */
    VQ_ERR_CAPACITY = -4, /* workspace too small / static limit exceeded */
    VQ_ERR_ARCH = -5,     /* device is not sm_100 */
    VQ_ERR_TIMEOUT = -6,  /* a bounded device-side wait gave up */
    VQ_ERR_CUDA = -7      /* CUDA runtime error (see vq_last_error) */
} vq_status;

typedef enum vq_dtype { VQ_F16 = 0, VQ_BF16 = 1, VQ_F32 = 2 } vq_dtype;

/* Library version: major*10000 + minor*100 + patch. */
int32_t vq_version(void);
/* Thread-local message for the last non-zero status returned on this thread. */
const char *vq_last_error(void);

/* Process-wide tuning and self-test knobs (for measurement sweeps and the library's own tests;
 * the defaults are what the kernels were tuned with). Returns the previous value, or
 * INT32_MIN for an unknown knob or a value out of range. No counterpart in the reference. */
typedef enum vq_knob {
    VQ_KNOB_ATTEND_STAGES = 0,   /* bulk-copy pipeline depth of the decode attend: 2..4 (2) */
    VQ_KNOB_ATTEND_WAVES = 1,    /* waves of CTAs the split count aims at: 1..32 (2) */
    VQ_KNOB_VQ_SEARCH = 2,       /* vq_vq_quantize search: 0 choose, 1 tcgen05, 2 mma.sync, 3 exact, 4 tcgen05 with the two-pass epilogue */
    VQ_KNOB_ATTEND_WAIT_TEST = 3,/* 1: in the NEXT vq_kivi_decode_attend (tensor-core kernel) every warp
                                    also waits, with 1024 polls, on a barrier that nothing arms: the
                                    bounded wait runs out, the kernel finishes normally and
                                    vq_kivi_attend_status reports VQ_ERR_TIMEOUT once (one-shot
                                    self-test of that path; nothing faults or hangs) */
    VQ_KNOB_VQ_WAIT_TEST = 4     /* 1: the same for the NEXT tcgen05 vq_vq_quantize launch and
                                    vq_vq_quantize_status */
} vq_knob;
int32_t vq_tune(int32_t knob, int32_t value);

/* ------------------------------------------------------------------------------------
 * KIVI asymmetric group quantization
 * ---------------------------------------------------------------------------------- */

/* One tensor [n_bh, n_tok, head_dim] -> codes + per-group (scale, zero), and/or the
 * round-tripped reconstruction.
 *
 * axis = 0: per-CHANNEL (KIVI keys): groups of `group` consecutive tokens per channel;
 *           scale/zero rows are [n_bh][ceil(n_tok/group)][head_dim].
 * axis = 1: per-TOKEN (KIVI values): groups of `group` consecutive channels per token;
 *           scale/zero rows are [n_bh][n_tok][ceil(head_dim/group)].
 * Math (float32, in this order): min, max, scale = max((max-min)/levels, eps),
 * q = clamp(rint((x-min)/scale), 0, levels) (round-half-even), zero = min. A ragged final
 * group is padded with its last live element. recon = T(q*scale + min) with the product
 * and the sum rounded separately.
 *
 * Replaces KIVIQuantizer._quantize_groups (veloxquant_mlx/quantizers/kivi.py:103-128),
 * KIVIKVCache._quant_dequant_along (veloxquant_mlx/cache/kivi_cache.py:151-201) and
 * kivi_group_quant_dequant (veloxquant_mlx/metal/_kivi_quant.py:138-207). */
typedef struct vq_kivi_quant_args {
    const void *x;            /* input, dtype `dtype` */
    int32_t dtype;            /* vq_dtype */
    int32_t axis;             /* 0 keys / per-channel, 1 values / per-token */
    int64_t n_bh, n_tok, head_dim;
    int64_t x_stride_bh;      /* elements between slabs of x; rows are head_dim apart */
    int32_t levels;           /* 2^b - 1, 1..255 */
    int32_t store_bits;       /* container width of one stored code: 1, 2, 4 or 8 */
    int32_t group;            /* >= 1 */
    float eps;                /* floor on scale (reference: 1e-8) */
    uint8_t *codes;           /* may be NULL; rows of head_dim*store_bits/8 bytes */
    int64_t codes_stride_bh;  /* bytes between slabs */
    float *scale;             /* may be NULL (then zero must be NULL too) */
    float *zero;
    int64_t param_stride_bh;  /* floats between slabs of scale / zero */
    void *recon;              /* may be NULL; same dtype and row layout as x */
    int64_t recon_stride_bh;  /* elements between slabs */
} vq_kivi_quant_args;
int32_t vq_kivi_quantize(const vq_kivi_quant_args *args, void *stream);
/* The two uses of vq_kivi_quantize under the names of the reference operations they stand
 * for. vq_kivi_quantize_pack is quantize-on-append into the packed store: codes, scale and
 * zero are required, recon is ignored (the reference has no packed KIVI store; its harness
 * keeps one code per byte: benchmark_scripts/benchmark_real_model_scalar_attend.py:155-182).
 * vq_kivi_quant_dequant is the round trip of kivi_group_quant_dequant
 * (veloxquant_mlx/metal/_kivi_quant.py:138-207): recon is required, codes/scale/zero are
 * written too when given. */
int32_t vq_kivi_quantize_pack(const vq_kivi_quant_args *args, void *stream);
int32_t vq_kivi_quant_dequant(const vq_kivi_quant_args *args, void *stream);
/* Store the incoming block of a KIVI cache update: n_new rows per slab of keys AND values are
 * copied behind the rows already held in the unquantized residual buffers, in one launch (the
 * reference's cache stores the block through its parent class before it quantizes what aged
 * out: veloxquant_mlx/cache/kivi_cache.py:250). Row r of slab s is read at
 * k_new + (s*new_stride_bh + r*head_dim) elements and written to
 * k_res + (s*res_stride_bh + (tok_offset + r)*head_dim) elements; likewise for the values.
 * dtype: VQ_F16, VQ_BF16 or VQ_F32. Rows must be multiples of 16 bytes, the four pointers
 * 16-byte aligned and both strides multiples of 16 bytes (VQ_ERR_ALIGN otherwise).
 * flags: 0, or VQ_ATTEND_OVERLAP_PREVIOUS: the copy may start while the preceding work on the
 * stream still runs (its loads of k_new / v_new then must not depend on that work); its stores
 * wait for that work to finish, and a vq_kivi_decode_attend with the same flag that follows
 * may start at once (it reads the residual rows only after this copy has completed). */
int32_t vq_kivi_append(const void *k_new, const void *v_new, int64_t new_stride_bh, void *k_res, void *v_res,
                       int64_t res_stride_bh, int64_t n_bh, int64_t n_new, int64_t tok_offset, int32_t head_dim,
                       int32_t dtype, int32_t flags, void *stream);

/* Flat dequantization code*scale+zero of one K (axis 0) or V (axis 1) tensor to
 * f16/bf16/f32. Replaces scalar_decode_once (veloxquant_mlx/metal/_scalar_attend.py:650-699,
 * metal/src/scalar_affine_decode_once.metal). */
typedef struct vq_kivi_dequant_args {
    const uint8_t *codes;
    int64_t codes_stride_bh;
    const float *scale;
    const float *zero;
    int64_t param_stride_bh;
    int32_t axis, store_bits, group;
    int64_t n_bh, n_tok, head_dim;
    void *out;
    int32_t out_dtype;
    int64_t out_stride_bh;
} vq_kivi_dequant_args;
int32_t vq_kivi_dequant(const vq_kivi_dequant_args *args, void *stream);

/* Fused dequant + softmax attention over packed KIVI codes, with an optional
 * unquantized tail (the residual window) attended in the same call.
 *   out[b,h,sq,:] = softmax_s( scale * q[b,h,sq,:] . K_hat[b,hk,s,:] ) . V_hat[b,hk,s,:]
 * with hk = h / (H_q/H_kv) (contiguous GQA blocks), K_hat = code*k_scale+k_zero for
 * s < n_quant and the tail rows after that. No mask (every query row sees every slot) unless
 * VQ_ATTEND_CAUSAL is set in `flags`.
 *
 * Replaces scalar_fused_decode_attend (veloxquant_mlx/metal/_scalar_attend.py:370-493,
 * metal/src/scalar_affine_attend.metal:8-175) and scalar_predecoded_attend
 * (_scalar_attend.py:702-779) when n_quant == 0. */
/* Protected ("sink") tokens of a sink-protected KIVI store (the reference's SinkProtectedKVCache,
 * veloxquant_mlx/cache/sink_cache.py:117-190, keeps the highest-key-norm tokens in fp16 inside its
 * dequantized buffer). Here such a token keeps a slot in the packed store, quantized from a copy
 * of a neighbouring row (as the reference does before it computes the group parameters) with its
 * value scale and zero-point set to 0, so the slot adds nothing to P.V; what its key still adds
 * to the softmax sum is taken out again through k_dead, and the token's exact rows come in as
 * extra tail rows. Batch element b has count[b] <= max_rows protected rows; per (b, kv head) a
 * slab of rows [max_rows..][D], stride_bh elements apart: k and v in the residual's dtype
 * (res_dtype must be set even when n_res is 0), k_dead in float32. */
typedef struct vq_kivi_sinks {
    const void *k;            /* exact key rows */
    const void *v;            /* exact value rows */
    const float *k_dead;      /* dequantized key of the slot each row left behind in the packed store */
    const int32_t *count;     /* [B], device memory */
    int64_t stride_bh;        /* elements */
    int32_t max_rows;
    int32_t reserved;         /* must be 0 */
} vq_kivi_sinks;

typedef struct vq_kivi_attend_args {
    const void *q;            /* [B, H_q, S_q, D] contiguous */
    void *out;                /* [B, H_q, S_q, D] contiguous */
    int32_t q_dtype, out_dtype;
    int32_t B, H_q, H_kv, S_q, D;
    int32_t store_bits;       /* 1, 2, 4 or 8 */
    int32_t group;
    int32_t n_quant;          /* packed tokens attended */
    int32_t n_res;            /* tail tokens attended */
    float scale;
    const uint8_t *k_codes;   /* [B*H_kv] slabs of rows D*store_bits/8 bytes */
    int64_t k_codes_stride_bh;
    const float *k_scale;     /* [B*H_kv] slabs of rows [token group][D] */
    const float *k_zero;
    int64_t k_param_stride_bh;
    const uint8_t *v_codes;
    int64_t v_codes_stride_bh;
    const float *v_scale;     /* [B*H_kv] slabs of rows [token][ceil(D/group)] */
    const float *v_zero;
    int64_t v_param_stride_bh;
    const void *k_res;        /* [B*H_kv] slabs of rows [token][D], dtype res_dtype */
    const void *v_res;
    int32_t res_dtype;
    int64_t res_stride_bh;    /* elements */
    void *workspace;          /* >= vq_kivi_attend_workspace_bytes(args) */
    int64_t workspace_bytes;
    int32_t n_splits;         /* context splits per (b, kv head); 0 = choose */
    int32_t variant;          /* 0 = choose; 1 = force the general CUDA-core kernel;
                                 2 = force the tensor-core kernel (error if unsupported) */
    int32_t flags;            /* VQ_ATTEND_* bits, 0 = none */
    int32_t reserved;         /* must be 0 */
    const struct vq_peer_gather *gather; /* NULL, or where the output rows are also published
                                 to the other ranks of a sharded run (see vq_peer_gather) */
    const struct vq_kivi_sinks *sinks;   /* NULL, or the protected tokens (tensor-core kernel only) */
} vq_kivi_attend_args;
/* The attention kernel may begin while the work that precedes this call on the stream is still
 * running (programmatic dependent launch): its prologue and its pass over the packed cache then
 * hide the previous kernels' drain, e.g. the previous layer's vq_kivi_decode_attend. The caller
 * promises that q, the codes, the scales and the zero-points of this call were complete before
 * that preceding work was launched. The residual rows, `workspace` and `out` are exempt: the
 * kernel touches them only after the preceding work has finished, so the residual rows may come
 * from a vq_kivi_append issued right before, and back-to-back calls may share one workspace.
 * Tensor-core kernel only; ignored by the general kernel. */
#define VQ_ATTEND_OVERLAP_PREVIOUS 1
/* Tail-aligned causal mask for S_q > 1: query row r sits at slot n_quant + n_res - S_q + r and
 * sees the slots up to its own (the mask of metal_fused_sdpa, veloxquant_mlx/metal/
 * fused_sdpa.py:200-299, applied to the KIVI store; S_q <= n_quant + n_res). General kernel. */
#define VQ_ATTEND_CAUSAL 2
int64_t vq_kivi_attend_workspace_bytes(const vq_kivi_attend_args *args);
/* Context splits vq_kivi_decode_attend would use for `args` (its n_splits honoured when > 0). A
 * caller that folds several layers into the batch axis passes the count of ONE layer as
 * n_splits, so that every layer is summed in exactly the order of a per-layer call (the
 * reference pins its batched kernel to its per-layer kernel bit for bit:
 * tests/metal/test_scalar_attend.py:660-707). 0 for unusable sizes. */
int32_t vq_kivi_attend_splits(const vq_kivi_attend_args *args);
int32_t vq_kivi_decode_attend(const vq_kivi_attend_args *args, void *stream);
/* Synchronises the device, then reports (and clears) whether any earlier
 * vq_kivi_decode_attend, vq_rabitq_decode_attend or vq_peer_gather_wait kernel abandoned a
 * bounded device-side wait: VQ_ERR_TIMEOUT if so (its output is then invalid), VQ_OK otherwise. No counterpart in the reference (its
 * kernels have no device-side waits). */
int32_t vq_kivi_attend_status(void);

/* Attention over already-decoded K/V rows only: vq_kivi_decode_attend with n_quant taken as
 * 0, so just k_res / v_res ([B*H_kv] slabs of n_res rows) are read. Replaces
 * scalar_predecoded_attend (veloxquant_mlx/metal/_scalar_attend.py:702-779,
 * metal/src/scalar_predecoded_attend.metal). */
int32_t vq_predecoded_attend(const vq_kivi_attend_args *args, void *stream);

/* Merge of split softmax partials, the last step of every split decode attend here:
 *   part_o  float32 [rows][n_splits][D]   sum_s exp(score_s - m) * v_s over the split's slots
 *   part_ml float32 [rows][n_splits][2]   (m = max score of the split or -inf if it saw no
 *                                          slot, l = sum_s exp(score_s - m))
 *   out[row, :] = sum_j part_o[row][j] * exp(m_j - M) / sum_j l_j * exp(m_j - M), M = max_j m_j
 * n_splits <= 256. Lets a caller that spreads one context over several calls (or devices) combine them. The
 * reference merges its SIMD-group partials inside the kernel
 * (metal/src/scalar_affine_attend.metal:120-175); it has no separate entry point. */
int32_t vq_lse_merge(const float *part_o, const float *part_ml, int64_t rows, int32_t n_splits,
                     int32_t D, void *out, int32_t out_dtype, void *stream);

/* ------------------------------------------------------------------------------------
 * Sharded decode: publishing a rank's output rows to its peers
 *
 * (batch, kv head) units are independent, so a decode step sharded over several GPUs of one
 * node needs no collective inside attention; each rank only has to deliver its rows of the
 * layer's output [B*H_q*S_q, D] to every rank. With `gather` set, the merge step of
 * vq_kivi_decode_attend stores its rows straight into every rank's copy of the gathered tensor
 * (plain stores to peer-mapped addresses over NVLink; no multicast, no bulk-copy engine); each of
 * its CTAs that wrote rows then fences once and adds 1 to this rank's arrival word on every rank.
 * vq_peer_gather_wait is the consumer side: a one-CTA kernel that returns once every publishing
 * rank's word has reached (rounds so far) x (that rank's arrivals per round), or gives up after a
 * bounded number of polls (vq_kivi_attend_status then reports VQ_ERR_TIMEOUT). Rounds are counted
 * on the device (`state`), so a captured CUDA graph can be replayed; the words only ever grow
 * (compared modulo 2^32). The reference has no multi-device code; there is no counterpart.
 * ---------------------------------------------------------------------------------- */
#define VQ_MAX_PEERS 16
typedef struct vq_peer_gather {
    int32_t world, rank;          /* 1 <= world <= VQ_MAX_PEERS: every rank receives the rows */
    int32_t n_sources;            /* ranks 0..n_sources-1 publish rows (ranks beyond hold replicas
                                     and publish nothing); 1 <= n_sources <= world */
    int32_t reserved;             /* must be 0 */
    int64_t row_offset;           /* first row of this call's rows inside the gathered tensor */
    void *out[VQ_MAX_PEERS];      /* base of the gathered tensor on each rank (own entry included),
                                     out_dtype, rows of D elements, 16-byte aligned */
    uint32_t *flags[VQ_MAX_PEERS];/* arrival words on each rank: uint32[world]; this rank adds
                                     to entry `rank` of every array */
    uint32_t *state;              /* this rank's round counter (word 2 of uint32[4]), zeroed once by
                                     the caller together with its `flags` array */
    int32_t arrivals[VQ_MAX_PEERS]; /* what each publishing rank adds to its word per round: its
                                     (batch, kv head) units x ceil(query heads per kv head / 4),
                                     i.e. the CTAs of its call that write rows; read by the wait */
} vq_peer_gather;
/* Waits on `stream` until the rows of the next round have arrived from every publishing rank
 * in this rank's gathered tensor. Call it once per vq_kivi_decode_attend that was given the same `gather`. */
int32_t vq_peer_gather_wait(const vq_peer_gather *gather, void *stream);
/* Inter-process handle of the device allocation that contains `ptr` (cudaIpcGetMemHandle) and
 * the offset of `ptr` inside it, for a peer process to map. `handle` receives 64 bytes. The
 * memory must come from cudaMalloc (PyTorch's default allocator qualifies). */
int32_t vq_peer_export(const void *ptr, void *handle, int64_t *offset);
/* Maps a peer process's allocation into this process (cudaIpcOpenMemHandle, peer access
 * enabled lazily): `*base` is its first byte. Open each allocation once per process. */
int32_t vq_peer_open(const void *handle, void **base);
int32_t vq_peer_close(void *base);

/* The same operation as vq_kivi_decode_attend for callers that cannot allocate device
 * memory (a frozen memory pool, a host runtime that owns all allocations, a path where a
 * synchronising, fallible cudaMalloc is not acceptable). It has no counterpart in the
 * reference. `workspace` / `workspace_bytes` in `args` are ignored: the split partials go
 * into an array built into the library (VQ_KIVI_STATIC_SCRATCH_BYTES, 8 MiB per GPU, held
 * until the process exits). After its one-time set-up on a device the call allocates nothing;
 * it returns VQ_ERR_CAPACITY, with the needed and available sizes in vq_last_error(), when
 * vq_kivi_attend_workspace_bytes(args) exceeds that capacity.
 *  - The FIRST call on each device looks up the array's device address (done with that device
 *    current). With CUDA's default lazy module loading this look-up is also the moment the
 *    driver loads the array's module on that device and sets aside its 8 MiB, so that first
 *    call can fail with VQ_ERR_CUDA (out of memory). Make it once per device while device
 *    memory may still be taken -- before the memory pool is frozen, before the first request,
 *    and before any stream capture. Every later call on that device allocates nothing.
 *  - All calls on a device share the one array. Calls must not overlap on the GPU (issue
 *    them on one stream, or order them with events): overlapping calls race on it. Nothing
 *    in it needs clearing between calls; every record read is written by the same call. */
#define VQ_KIVI_STATIC_SCRATCH_BYTES (8u << 20)
int32_t vq_kivi_decode_attend_static(const vq_kivi_attend_args *args, void *stream);

/* ------------------------------------------------------------------------------------
 * Bit packing of flat uint8 code arrays, b in {1, 2, 4}
 * Replaces bit_pack / bit_unpack (veloxquant_mlx/metal/_bit_packing.py:87-148,
 * metal/src/bit_pack.metal, bit_unpack.metal).
 * ---------------------------------------------------------------------------------- */
int32_t vq_bit_pack(const uint8_t *codes, int64_t n, int32_t bits, uint8_t *packed, void *stream);
int32_t vq_bit_unpack(const uint8_t *packed, int64_t n, int32_t bits, uint8_t *codes, void *stream);

/* ------------------------------------------------------------------------------------
 * VecInfer product VQ
 * ---------------------------------------------------------------------------------- */

/* Nearest-centroid indices of n sub-vectors. Distances are float32 in the order of
 * vecinfer_quantize.metal: dist = 0; for i in 0..sub_dim-1: d = x_i - c_i; dist = dist + d*d
 * (product and sum rounded separately); strict '<' so the lowest index wins ties.
 * x is [n, sub_dim] contiguous (dtype x_dtype). codebook is float32 [n_c, sub_dim], or with
 * n_sub > 0 a stack [n_sub, n_c, sub_dim] where sub-vector i uses codebook i % n_sub.
 * indices are written index_bytes (1, 2 or 4) wide, little endian unsigned.
 * Replaces quantize_vq (veloxquant_mlx/allocators/vecinfer.py:281-318) and
 * vecinfer_quantize_metal (metal/_vecinfer.py:181-222, metal/src/vecinfer_quantize.metal). */
int32_t vq_vq_quantize(const void *x, int32_t x_dtype, int64_t n, int32_t sub_dim,
                       const float *codebook, int32_t n_centroids, int32_t n_sub,
                       void *indices, int32_t index_bytes, void *stream);

/* Synchronises the device, then reports (and clears) whether an earlier vq_vq_quantize kernel
 * abandoned a bounded device-side wait: VQ_ERR_TIMEOUT if so (its indices are then invalid),
 * VQ_OK otherwise. No counterpart in the reference. */
int32_t vq_vq_quantize_status(void);

/* Codebook gather: out[i, :] = codebook[min(indices[i], n_c-1), :] (stacked codebooks as
 * above). Replaces dequantize_vq (allocators/vecinfer.py:321-335) and vecinfer_dequant_metal
 * (metal/_vecinfer.py:144-178, metal/src/vecinfer_dequant.metal). */
int32_t vq_vq_dequant(const void *indices, int32_t index_bytes, int64_t n, const float *codebook,
                      int32_t n_centroids, int32_t sub_dim, int32_t n_sub, void *out,
                      int32_t out_dtype, void *stream);

/* Quantize-on-append in one launch.
 * keys:   x [n_tok, D] -> (optional) smooth divide where smooth > 1e-8 -> y = H x as a
 *         sequential float32 matvec (c = 0..D-1, product and sum rounded separately) ->
 *         nearest centroid per sub-vector (as vq_vq_quantize) -> indices; and, when x_hat is
 *         given, gather -> H^T c -> smooth multiply -> x_hat (the round-tripped keys).
 *         Token t belongs to head (t / tok_per_head) % n_heads and uses smooth row
 *         head % smooth_rows. H may be NULL (no rotation), smooth may be NULL.
 * values: indices of x itself and x_hat = gathered centroids; H and smooth are ignored.
 * Either output may be NULL. D <= 512; sub_dim in {1, 2, 4, 8, 16}.
 * Replaces vecinfer_encode_decode_metal (veloxquant_mlx/metal/_vecinfer.py:225-293,
 * metal/src/vecinfer_encode_decode_full.metal) and vecinfer_encode_decode_simple_metal
 * (_vecinfer.py:296-345, metal/src/vecinfer_encode_decode_simple.metal). */
typedef struct vq_vq_encode_args {
    const void *x;            /* [n_tok, D] contiguous */
    int32_t x_dtype;
    int64_t n_tok;
    int32_t D, sub_dim;
    int64_t tok_per_head;     /* tokens per (batch, head) slab of x */
    int32_t n_heads;
    const float *codebook;    /* [n_c, sub_dim] or [D/sub_dim][n_c][sub_dim] */
    int32_t n_centroids;
    int32_t stacked_codebooks;/* 0 = one shared codebook, 1 = one per sub-space */
    const float *H;           /* [D, D] row-major or NULL */
    const float *smooth;      /* [smooth_rows, D] or NULL */
    int32_t smooth_rows;
    void *x_hat;              /* [n_tok, D], dtype hat_dtype, or NULL */
    int32_t hat_dtype;
    void *indices;            /* [n_tok, D/sub_dim], index_bytes wide, or NULL */
    int32_t index_bytes;
} vq_vq_encode_args;
int32_t vq_vq_encode_decode_keys(const vq_vq_encode_args *args, void *stream);
int32_t vq_vq_encode_decode_values(const vq_vq_encode_args *args, void *stream);

/* The dual transform with a defined float32 order: y = WHT(x / smooth) * c for keys
 * (divide != 0), y = WHT(x * smooth) * c for queries, where WHT is the unnormalised Sylvester
 * butterfly (pairs (lower + upper, lower - upper), strides 1, 2, 4, ...) and c the common entry
 * magnitude of the orthonormal Walsh-Hadamard matrix. x is [n_rows, D] (dtype x_dtype), out
 * float32 [n_rows, D]; row r belongs to head (r / tok_per_head) % n_heads and uses smooth row
 * head % smooth_rows; smooth may be NULL. D is 32, 64, 128 or 256. Replaces
 * apply_dual_transform_keys / _queries (veloxquant_mlx/allocators/vecinfer.py:93-184), which
 * multiply by the dense matrix in an unspecified summation order. */
int32_t vq_vq_dual_transform(const void *x, int32_t x_dtype, int64_t n_rows, int32_t D, int64_t tok_per_head,
                             int32_t n_heads, const float *smooth, int32_t smooth_rows, int32_t divide, float c,
                             float *out, void *stream);

/* Attention over VQ-coded keys scored through a per-query lookup table
 * lut[s][c] = q_sub[s] . codebook[c], score = scale * sum_s lut[s][idx[s]]; values are either
 * VQ-coded (indices + codebook: the reference form) or a dense tensor. Tail-aligned causal
 * mask (query row r sits at position S_kv - S_q + r) and optional trailing window.
 * h_kv = h_q * H_kv / H_q. Replaces metal_fused_sdpa (veloxquant_mlx/metal/fused_sdpa.py:200-299,
 * metal/src/fused_sdpa.metal). */
typedef struct vq_vq_attend_args {
    const void *q;            /* [B, H_q, S_q, D], already dual-transformed */
    void *out;                /* [B, H_q, S_q, D] */
    int32_t q_dtype, out_dtype;
    int32_t B, H_q, H_kv, S_q, S_kv, D;
    int64_t kv_stride_tok;    /* token capacity between (b, kv head) slabs of k/v arrays */
    float scale;
    int32_t causal, sliding_window;
    const void *k_indices;    /* [B*H_kv][cap][n_sub], k_index_bytes wide */
    int32_t k_index_bytes;
    const float *k_codebook;  /* [n_c, sub_dim] or [k_stacked = n_sub][n_c][sub_dim] */
    int32_t k_n_centroids, k_sub_dim, k_stacked;
    int32_t v_mode;           /* 0 = dense values (v_dtype), 1 = VQ indices + codebook */
    const void *v;            /* dense [B*H_kv][cap][D] or indices [B*H_kv][cap][D/v_sub_dim] */
    int32_t v_dtype, v_index_bytes;
    const float *v_codebook;  /* [n_c_v, v_sub_dim] */
    int32_t v_n_centroids, v_sub_dim;
    void *workspace;
    int64_t workspace_bytes;
    int32_t n_splits;         /* 0 = choose */
} vq_vq_attend_args;
int64_t vq_vq_attend_workspace_bytes(const vq_vq_attend_args *args);
int32_t vq_vq_decode_attend(const vq_vq_attend_args *args, void *stream);

/* ------------------------------------------------------------------------------------
 * RaBitQ 1-bit keys
 * ---------------------------------------------------------------------------------- */

/* keys [n, D] -> sign bits u8 [n, D/8] (element 8j+t at byte j bit t, >= 0 -> 1) and
 * mag[n] = sum|y| / D.  rotate = 1: y = WHT(keys * diag) / sqrt(D) with the Sylvester
 * butterfly (D a power of two <= 1024); rotate = 0: y = keys (already rotated, e.g. by a
 * dense QR rotation). Replaces rabitq_encode (veloxquant_mlx/metal/_rabitq_encode.py:83-128,
 * metal/src/rabitq_encode.metal) and _pack_signs (quantizers/rabitq.py:64-70). */
int32_t vq_rabitq_encode(const void *keys, int32_t dtype, int64_t n, int32_t D, const float *diag,
                         int32_t rotate, uint8_t *bits, float *mag, void *stream);

/* Two 4-bit indices per byte, low nibble = even element; n_out = n_in / 2 bytes.
 * Replaces rabitq_pack_values (metal/_rabitq_values.py:64-95). */
int32_t vq_rabitq_pack_values(const uint8_t *v_idx, int64_t n_out, uint8_t *packed, void *stream);

/* score[i] = popcount(q_bits ^ bits[i]) * scale + cx[i]. Replaces rabitq_hamming_score
 * (metal/_rabitq.py:63-103). */
int32_t vq_rabitq_hamming_score(const uint8_t *q_bits, const uint8_t *bits, int64_t n, int32_t n_bytes,
                                float scale, const float *cx, float *score, void *stream);

/* Attention over sign-bit keys: score = (D - 2*popcount(sign(q) ^ k_bits)) * q_scale * k_mag
 * + k_const, softmax over all slots (no mask), values from a <= 16-entry scalar codebook
 * (one index per byte or nibble-packed: the reference form) or a dense tensor. H_q may be a
 * multiple of H_kv (contiguous blocks). Replaces rabitq_fused_attend
 * (veloxquant_mlx/metal/_rabitq_attend.py:112-216, metal/src/rabitq_attend.metal). */
typedef struct vq_rabitq_attend_args {
    const void *q;            /* [B, H_q, S_q, D] */
    void *out;
    int32_t q_dtype, out_dtype;
    int32_t B, H_q, H_kv, S_q, S_kv, D;
    int64_t kv_stride_tok;
    const float *q_scale;     /* [B, H_q, S_q] */
    const uint8_t *k_bits;    /* [B*H_kv][cap][D/8] */
    const float *k_mag;       /* [B*H_kv][cap] */
    const float *k_const;     /* [B*H_kv][cap] or NULL (= 0) */
    int32_t v_mode;           /* 0 dense (v_dtype), 2 codebook index per byte, 3 nibble-packed */
    const void *v;
    int32_t v_dtype;
    const float *v_cents;     /* [<= 16] */
    int32_t n_cents;
    void *workspace;
    int64_t workspace_bytes;
    int32_t n_splits;
} vq_rabitq_attend_args;
int64_t vq_rabitq_attend_workspace_bytes(const vq_rabitq_attend_args *args);
int32_t vq_rabitq_decode_attend(const vq_rabitq_attend_args *args, void *stream);

/* Attention of MANY query rows over sign-bit keys (prompt chunks, multi-turn prefill): tiled on
 * the tensor cores. Score model: the exact dot with the decoded key,
 *   score[i][j] = (q[i] . (signs(k_bits[j]) * k_mag[j])) * scale + k_const[j]
 * (not the popcount estimator of the decode kernel), softmax over all slots or, with
 * causal != 0, the slots up to the query's own (row r of S_q sits at slot S_kv - S_q + r).
 * Values: nibble-packed indices into a <= 16-entry codebook (v_mode 3: the reference form) or a
 * dense f16 / bf16 tensor (v_mode 0). H_q may be a multiple of H_kv (contiguous blocks).
 * D is 64 or 128. No workspace. Replaces rabitq_prefill_attend
 * (veloxquant_mlx/metal/_rabitq_prefill.py:116-196, metal/src/rabitq_prefill.metal). */
typedef struct vq_rabitq_prefill_args {
    const void *q;            /* [B, H_q, S_q, D] */
    void *out;                /* [B, H_q, S_q, D] */
    int32_t q_dtype, out_dtype;
    int32_t B, H_q, H_kv, S_q, S_kv, D;
    int64_t kv_stride_tok;    /* token capacity between (b, kv head) slabs of the k/v arrays */
    float scale;
    int32_t causal;
    const uint8_t *k_bits;    /* [B*H_kv][cap][D/8] */
    const float *k_mag;       /* [B*H_kv][cap] */
    const float *k_const;     /* [B*H_kv][cap] or NULL (= 0) */
    int32_t v_mode;           /* 0 dense (v_dtype f16 / bf16), 3 nibble-packed codebook indices */
    int32_t v_dtype;
    const void *v;            /* dense [B*H_kv][cap][D] or nibbles [B*H_kv][cap][D/2] */
    const float *v_cents;     /* [<= 16] */
    int32_t n_cents;
    int32_t reserved;
} vq_rabitq_prefill_args;
int32_t vq_rabitq_prefill_attend(const vq_rabitq_prefill_args *args, void *stream);

/* ------------------------------------------------------------------------------------
 * TurboQuant-RVQ: two-stage scalar residual quantization of rotated key vectors, packed.
 * ------------------------------------------------------------------------------------ */
/* rvq_quant_pack (veloxquant_mlx/metal/_rvq_quant_pack.py:83-149, src/rvq_quant_pack.metal):
 * rotated [n_rows, D] float16 (device); centroids1 [2^bits], boundaries1 / boundaries2
 * [2^bits - 1] are HOST arrays (sorted, float16-representable values, as ScalarCodebook holds
 * them); packed1 / packed2 [n_rows, ceil(D / (32 / bits))] uint32 (device): code i of a word in
 * bits [i*bits, (i+1)*bits), last word zero-padded. bits 1..4, D <= 1024. Bit-identical to
 * ScalarCodebook.quantize + _pack_indices of both stages. */
int32_t vq_rvq_quant_pack(const void *rotated, int64_t n_rows, int32_t D, const float *centroids1,
                          const float *boundaries1, const float *boundaries2, const uint8_t *table, int32_t bits,
                          uint32_t *packed1, uint32_t *packed2, void *stream);
/* Both codes depend on nothing but the coordinate's 16 bits, so the whole two-stage quantizer is a
 * 65 536-entry table: table[bits of y] = idx1 | idx2 << 4 (device memory, 16-byte aligned, 64 KiB).
 * Built once per pair of codebooks and passed to vq_rvq_quant_pack as `table` (may be NULL there:
 * the kernel then compares against the boundaries; with a table the codebook pointers may be NULL
 * for inputs of at least 65 536 words). No counterpart in the reference. */
int32_t vq_rvq_build_table(const float *centroids1, const float *boundaries1, const float *boundaries2, int32_t bits,
                           uint8_t *table, void *stream);
/* rvq_unpack_decode (veloxquant_mlx/metal/_rvq_unpack_decode.py:78-183, src/rvq_unpack_decode.metal):
 * the packed streams are read in place from buffers of `cap` rows per (batch, head) of which the
 * first `seq` are live; norms [n_bh * cap] in norms_dtype; centroids1 / centroids2 [2^bits] are
 * HOST arrays, diag [D] (+-1) is a device array; out [n_bh * seq, D] float16, rows ordered
 * (batch-head, token). D a power of two <= 1024. */
int32_t vq_rvq_unpack_decode(const uint32_t *packed1, const uint32_t *packed2, const void *norms, int32_t norms_dtype,
                             const float *centroids1, const float *centroids2, const float *diag, int32_t bits,
                             int32_t D, int64_t n_bh, int64_t seq, int64_t cap, void *out, void *stream);

/* ---- SKVQ: clipped group quantization along the channel axis (per-token groups) -------------- */
/* clipped_group_quant (veloxquant_mlx/quantizers/skvq.py:103-165) with the channel gather of
 * apply_permutation (:98-100) folded in, codes bit-packed LSB-first along the row (the layout of
 * vq_bit_pack). For every group of `group_size` channels of a token and every clip factor alpha:
 * lo = mid - alpha*range/2, scale = max(alpha*range/(2^bits-1), 1e-8),
 * code = clip(rint((x - lo)/scale), 0, 2^bits-1); the alpha with the smallest squared
 * reconstruction error wins (first on ties; error sums in a fixed order: eight partial sums over
 * the elements 8 apart, then a tree) and is folded into the stored (lo, scale). float32 arithmetic,
 * every product and sum rounded separately. group_size 8, 16, 32 or 64 dividing D (the
 * reference pads a ragged last group; not offered here). */
typedef struct vq_skvq_quant_args {
    const void *x;        /* [n_bh][n_tok][D] in x_dtype; (batch, head) blocks x_stride_bh ELEMENTS apart */
    int64_t x_stride_bh;
    const int32_t *perm;  /* device [n_heads][D] or NULL: stored channel j = x[..., perm[bh % n_heads][j]] */
    uint8_t *codes;       /* [n_bh][>= n_tok][D*bits/8]; blocks q_stride_bh ROWS apart (also lo, scale) */
    float *lo;            /* [n_bh][>= n_tok][D/group_size] */
    float *scale;
    int64_t q_stride_bh;
    float alphas[8];      /* clip factors, each in (0, 1]; one value = no search */
    int32_t n_alphas, x_dtype, n_bh, n_heads, n_tok, D, bits, group_size;
} vq_skvq_quant_args;
int32_t vq_skvq_quantize_pack(const vq_skvq_quant_args *args, void *stream);
/* clipped_group_dequant (skvq.py:168-182) + the inverse gather: out[..., c] = code*scale + lo of
 * stored channel inv_perm[bh % n_heads][c] (c itself when inv_perm is NULL), rounded to out_dtype. */
typedef struct vq_skvq_dequant_args {
    const uint8_t *codes;
    const float *lo;
    const float *scale;
    int64_t q_stride_bh;
    const int32_t *inv_perm;
    void *out;            /* [n_bh][n_tok][D]; blocks out_stride_bh ELEMENTS apart */
    int64_t out_stride_bh;
    int32_t out_dtype, n_bh, n_heads, n_tok, D, bits, group_size, reserved;
} vq_skvq_dequant_args;
int32_t vq_skvq_unpack_dequant(const vq_skvq_dequant_args *args, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* VQB200_H */
