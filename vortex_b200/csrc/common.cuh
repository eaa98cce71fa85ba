// Shared device/host helpers of the vortex_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/vortex_b200.h"

namespace vtx {

// ---- error plumbing -------------------------------------------------------
int fail(int code, const char* fmt, ...);   // records the message for vtx_last_error, returns code
// cudaGetLastError -> VTX_ERR_LAUNCH; adds the kernels the caller just launched to the count vtx_launch_count() reports
int check_launch(const char* what, long long launches = 1);

#define VTX_REQUIRE(cond, code, ...)            \
    do {                                        \
        if (!(cond)) return ::vtx::fail((code), __VA_ARGS__); \
    } while (0)

constexpr int kNumSMs = 148;

// Polls (each followed by a short sleep) of a global-memory flag before a kernel that waits for another block gives
// up, records a code in the device status word and carries on; vtx_debug_set_flag_poll_limit changes it.
int flag_poll_limit();

// ---- dtype helpers --------------------------------------------------------
template <typename T> struct DTypeCode;
template <> struct DTypeCode<float> { static constexpr int value = VTX_F32; };
template <> struct DTypeCode<__nv_bfloat16> { static constexpr int value = VTX_BF16; };
template <> struct DTypeCode<__half> { static constexpr int value = VTX_F16; };

__host__ __device__ inline int dtype_size(int64_t code) { return code == VTX_F32 ? 4 : 2; }

template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

// Round through the I/O type and come back to fp32 (identity for fp32).
template <typename T> __device__ __forceinline__ float round_io(float x) { return to_f32<T>(from_f32<T>(x)); }

// Parameter (weights, biases, masks, caches) of run-time dtype.
__device__ __forceinline__ float ld_param(const void* p, int64_t dtype, int64_t i) {
    if (dtype == VTX_F32) return static_cast<const float*>(p)[i];
    if (dtype == VTX_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    return __half2float(static_cast<const __half*>(p)[i]);
}

// Raw bits of parameter i and their value, kept apart so that a thread can issue every load of its set-up before it
// uses the first result (one memory round trip instead of one per parameter: ld_param's dtype branches end a basic
// block at every call).
__device__ __forceinline__ uint32_t ld_raw(const void* p, bool wide, int64_t i) {
    return wide ? static_cast<const uint32_t*>(p)[i] : (uint32_t) static_cast<const unsigned short*>(p)[i];
}
__device__ __forceinline__ float cvt_raw(uint32_t raw, int64_t dtype) {
    return dtype == VTX_F32 ? __uint_as_float(raw)
           : dtype == VTX_BF16 ? __uint_as_float(raw << 16) : __half2float(__ushort_as_half((unsigned short)raw));
}

// ---- q / k / v channel map -------------------------------------------------
struct QkvMap {
    int layout;
    int flip;
    int64_t D;
    int64_t hd;  // channels per head (column split)
    __host__ __device__ inline void get(int64_t d, int64_t& cq, int64_t& ck, int64_t& cv) const {
        if (layout == VTX_QKV_INTERLEAVED) {
            cq = 3 * d; ck = 3 * d + 1; cv = 3 * d + 2;
        } else if (layout == VTX_QKV_COLUMN_SPLIT) {
            int64_t n = d / hd, j = d - n * hd;
            cq = n * 3 * hd + j; ck = cq + hd; cv = cq + 2 * hd;
        } else {
            cq = d; ck = D + d; cv = 2 * D + d;
        }
        if (flip) { int64_t t = cq; cq = ck; ck = t; }
    }
};

// Dispatch a templated launcher on the I/O dtype code.
#define VTX_DISPATCH_IO(code, T, ...)                                   \
    switch (code) {                                                     \
        case VTX_F32:  { using T = float;          __VA_ARGS__; break; } \
        case VTX_BF16: { using T = __nv_bfloat16;  __VA_ARGS__; break; } \
        case VTX_F16:  { using T = __half;         __VA_ARGS__; break; } \
        default: return ::vtx::fail(VTX_ERR_BAD_ARG, "unknown io dtype %lld", (long long)(code)); \
    }

inline bool valid_dtype(int64_t c) { return c == VTX_F32 || c == VTX_BF16 || c == VTX_F16; }

template <typename T> __host__ __device__ inline T ceil_div(T a, T b) { return (a + b - 1) / b; }

}  // namespace vtx
