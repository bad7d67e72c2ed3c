// Shared device / host helpers of the qvb8_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/qvb8_b200.h"

#define QV_API extern "C" __attribute__((visibility("default")))

namespace qv {

// ---------------------------------------------------------------------------------------------------------------
// host: status + thread-local message

inline char *err_buf() {
    static thread_local char buf[512] = {0};
    return buf;
}

inline int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err_buf(), 512, fmt, ap);
    va_end(ap);
    return code;
}

inline int cuda_status(const char *what) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(QVB8_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return QVB8_OK;
}

inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// Common argument checks of every entry point that takes a pack.
inline int check_pack(const qvb8_pack *w, const char *who) {
    if (!w) return fail(QVB8_ERR_ARG, "%s: null pack", who);
    if (w->Q < 0 || w->P < 0 || w->Q > 0x7fffffff || w->P > 0x7fffffff)
        return fail(QVB8_ERR_ARG, "%s: Q=%lld P=%lld out of range", who, (long long)w->Q, (long long)w->P);
    if (w->Q > 0 && (!w->min_s || !w->tau_s || !w->nbits || !w->bit_off))
        return fail(QVB8_ERR_ARG, "%s: null row metadata", who);
    if (w->Q > 0 && w->P > 0 && (!w->ids || w->ids_bytes < 8))
        return fail(QVB8_ERR_ARG, "%s: ids buffer missing or shorter than its 8 pad bytes", who);
    if (w->n_esc < 0 || (w->n_esc > 0 && (!w->esc_idx || !w->esc_vals)))
        return fail(QVB8_ERR_ARG, "%s: escape table inconsistent", who);
    return QVB8_OK;
}

inline int check_device(const char *who) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return fail(QVB8_ERR_CUDA, "%s: no current CUDA device", who);
    }
    static thread_local int cached_dev = -1, cached_major = 0;
    if (cached_dev != dev) {
        int major = 0;
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        cached_dev = dev;
        cached_major = major;
    }
    if (cached_major != 10)
        return fail(QVB8_ERR_DEVICE, "%s: built for sm_100a, the current device is compute capability %d.x", who,
                    cached_major);
    return QVB8_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// device: ids

// One nb-bit id starting at absolute bit `bit` of an LSB-first stream, read byte-wise so that any base alignment
// works.  An id is at most 14 bits wide, so it spans at most three bytes; four are read (the buffer carries 8 pad
// bytes).
__device__ __forceinline__ uint32_t field_bytes(const uint8_t *__restrict__ ids, int64_t bit, int nb) {
    const uint8_t *p = ids + (bit >> 3);
    const uint32_t w = (uint32_t)__ldg(p) | ((uint32_t)__ldg(p + 1) << 8) | ((uint32_t)__ldg(p + 2) << 16) |
                       ((uint32_t)__ldg(p + 3) << 24);
    return (w >> (uint32_t)(bit & 7)) & ((1u << nb) - 1u);
}

// Exact uint -> float for values below 2^23 without the conversion pipe: place the integer in the mantissa of 2^23
// and subtract 2^23.
__device__ __forceinline__ float small_u2f(uint32_t i) { return __uint_as_float(i | 0x4B000000u) - 8388608.0f; }

// Restored fp32 weight of an id: ONE fused multiply-add, the value every certificate of the format is stated on.
__device__ __forceinline__ float band(uint32_t id, float ts, float m) { return __fmaf_rn((float)id, ts, m); }

// ---------------------------------------------------------------------------------------------------------------
// device: activations

// Saturating narrowing to fp16: values beyond +-65504 clamp, a NaN stays a NaN (comparisons, not fmin/fmax).
__device__ __forceinline__ __half sat_half(float v) {
    return __float2half_rn(v > 65504.0f ? 65504.0f : (v < -65504.0f ? -65504.0f : v));
}

template <int XT>
__device__ __forceinline__ float load_x(const void *__restrict__ X, int64_t i) {
    if constexpr (XT == QVB8_F16) return __half2float(__ldg(reinterpret_cast<const __half *>(X) + i));
    else if constexpr (XT == QVB8_BF16) return __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16 *>(X) + i));
    else return __ldg(reinterpret_cast<const float *>(X) + i);
}

// ---------------------------------------------------------------------------------------------------------------
// device: dense outputs

template <typename T> __device__ __forceinline__ T narrow(float v);
template <> __device__ __forceinline__ __half narrow<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ float narrow<float>(float v) { return v; }

}  // namespace qv
