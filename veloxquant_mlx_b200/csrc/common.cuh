// Shared helpers for libvqb200: status/error plumbing, dtype loads/stores, small device utilities.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/vqb200.h"

namespace vq {

// Thread-local message buffer behind vq_last_error().
char *last_error_buf();
int32_t fail(int32_t code, const char *fmt, ...);

#define VQ_CHECK_CUDA(expr)                                                                  \
    do {                                                                                     \
        cudaError_t _e = (expr);                                                             \
        if (_e != cudaSuccess)                                                               \
            return vq::fail(VQ_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e));    \
    } while (0)

#define VQ_CHECK_LAUNCH(name)                                                                \
    do {                                                                                     \
        cudaError_t _e = cudaGetLastError();                                                 \
        if (_e != cudaSuccess)                                                               \
            return vq::fail(VQ_ERR_CUDA, "launch of %s failed: %s", name,                    \
                            cudaGetErrorString(_e));                                         \
    } while (0)

#define VQ_REQUIRE(cond, code, ...)                                                          \
    do {                                                                                     \
        if (!(cond)) return vq::fail(code, __VA_ARGS__);                                     \
    } while (0)

inline bool is_aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline size_t dtype_size(int32_t dt) { return dt == VQ_F32 ? 4 : 2; }

// Cached per-device facts (read-only after first use).
struct DeviceInfo {
    int sm_count;
    int cc_major;
    int cc_minor;
    size_t smem_optin;
};
int32_t device_info(DeviceInfo *out);

// Current value of a vq_knob (see vq_tune); knob_take also puts the default back (one-shot knobs).
int knob_get(int knob);
int knob_take(int knob);

// ---- typed element access --------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float load_as_f32(const void *p, int32_t dt, int64_t i) {
    if (dt == VQ_F16) return __half2float(reinterpret_cast<const __half *>(p)[i]);
    if (dt == VQ_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]);
    return reinterpret_cast<const float *>(p)[i];
}
__device__ __forceinline__ void store_from_f32(void *p, int32_t dt, int64_t i, float v) {
    if (dt == VQ_F16) reinterpret_cast<__half *>(p)[i] = __float2half_rn(v);
    else if (dt == VQ_BF16) reinterpret_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<float *>(p)[i] = v;
}

// Code i of a packed row (container width SB bits, LSB first).
__device__ __forceinline__ uint32_t load_code(const uint8_t *row, int i, int sb) {
    if (sb == 8) return row[i];
    const int per = 8 / sb;
    const uint32_t byte = row[i / per];
    return (byte >> ((i % per) * sb)) & ((1u << sb) - 1u);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

}  // namespace vq
