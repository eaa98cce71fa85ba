// Hyena-X forward: o = fir(h_q, q) * fir(h_k, k) * fir(h_v, v) on (batch, channel, time) tensors, depthwise causal
// filters of up to 16 taps (cross-correlation order: the last tap meets the current sample).  Memory-bound
// (3 reads + 1 write per element): a thread produces eight consecutive samples of one channel from three 16-byte
// loads per input (the current vector and the two before it, which hold the filter history), keeps the window in
// registers and rounds where the reference's tensors of the I/O dtype round (each FIR output, the first product).
#include "common.cuh"

namespace vtx {

constexpr int HX_MAX_TAPS = 16;
constexpr int HX_VEC = 8;            // samples per thread (16 bytes of bf16 / fp16)

// two fp32 -> one 32-bit word of the 2-byte I/O dtype (first value in the low half)
template <typename T> __device__ __forceinline__ uint32_t pack_pair(float a, float b);
template <> __device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float a, float b) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
    return r;
}
template <> __device__ __forceinline__ uint32_t pack_pair<__half>(float a, float b) {
    const __half2 hh = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&hh);
}
template <> __device__ __forceinline__ uint32_t pack_pair<float>(float, float) { return 0; }

// eight 2-byte elements of a 16-byte vector -> fp32 (no address-taken temporaries: they would live in local memory)
template <typename T> __device__ __forceinline__ void unpack8(const uint4& r, float* o);
template <> __device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4& r, float* o) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { o[2 * i] = __uint_as_float(w[i] << 16); o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
template <> __device__ __forceinline__ void unpack8<__half>(const uint4& r, float* o) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        o[2 * i] = f.x; o[2 * i + 1] = f.y;
    }
}
template <> __device__ __forceinline__ void unpack8<float>(const uint4&, float*) {}

template <typename T>
__global__ void __launch_bounds__(256) hyena_x_kernel(vtx_hyena_x_params p) {
    const int64_t nvec = (p.L + HX_VEC - 1) / HX_VEC;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= p.B * p.D * nvec) return;
    const int64_t row = idx / nvec, t0 = (idx % nvec) * HX_VEC;    // row = b * D + d
    const int64_t d = row % p.D;
    const int Lh = (int)p.Lh;
    const void* src[3] = {p.q, p.k, p.v};
    float z[3][HX_VEC];
#pragma unroll
    for (int x = 0; x < 3; ++x) {
        const T* in = static_cast<const T*>(src[x]) + row * p.L;
        // window: samples t0 - 16 .. t0 + 7 (zeros before the sequence start and after its end)
        float win[HX_MAX_TAPS + HX_VEC];
        const bool vec_ok = sizeof(T) == 2 && (p.L % HX_VEC) == 0 && (reinterpret_cast<uintptr_t>(in) % 16) == 0;
#pragma unroll
        for (int blk = 0; blk < 3; ++blk) {
            const int64_t tb = t0 + (blk - 2) * HX_VEC;
            if (vec_ok) {
                // L is a multiple of the vector length: a block lies wholly inside the sequence or wholly outside
                if (tb >= 0 && tb < p.L) {
                    unpack8<T>(*reinterpret_cast<const uint4*>(in + tb), &win[blk * HX_VEC]);
                } else {
#pragma unroll
                    for (int i = 0; i < HX_VEC; ++i) win[blk * HX_VEC + i] = 0.f;
                }
            } else {
#pragma unroll
                for (int i = 0; i < HX_VEC; ++i) {
                    const int64_t t = tb + i;
                    win[blk * HX_VEC + i] = (t >= 0 && t < p.L) ? to_f32<T>(in[t]) : 0.f;
                }
            }
        }
        float w[HX_MAX_TAPS];       // w[j] multiplies the sample j steps back
        const int64_t hoff = (x * p.D + d) * Lh;
        if (sizeof(T) == 2 && Lh == HX_MAX_TAPS && p.h_dtype == p.io_dtype && (reinterpret_cast<uintptr_t>(p.h) % 16) == 0) {
            // the channel's sixteen taps as two 16-byte loads
            float t[HX_MAX_TAPS];
            const uint4* hv = reinterpret_cast<const uint4*>(static_cast<const T*>(p.h) + hoff);
            unpack8<T>(__ldg(hv), &t[0]);
            unpack8<T>(__ldg(hv + 1), &t[8]);
#pragma unroll
            for (int j = 0; j < HX_MAX_TAPS; ++j) w[j] = t[HX_MAX_TAPS - 1 - j];
        } else {
#pragma unroll
            for (int j = 0; j < HX_MAX_TAPS; ++j) w[j] = j < Lh ? ld_param(p.h, p.h_dtype, hoff + (Lh - 1 - j)) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < HX_VEC; ++i) {
            float acc = 0.f;
#pragma unroll
            for (int j = HX_MAX_TAPS - 1; j >= 0; --j) acc = fmaf(w[j], win[2 * HX_VEC + i - j], acc);
            z[x][i] = round_io<T>(acc);
        }
    }
    T* out = static_cast<T*>(p.y) + row * p.L;
    float of[HX_VEC];
#pragma unroll
    for (int i = 0; i < HX_VEC; ++i) of[i] = round_io<T>(z[0][i] * z[1][i]) * z[2][i];
    if (sizeof(T) == 2 && t0 + HX_VEC <= p.L && (reinterpret_cast<uintptr_t>(out + t0) % 16) == 0) {
        uint32_t w4[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) w4[i] = pack_pair<T>(of[2 * i], of[2 * i + 1]);
        *reinterpret_cast<uint4*>(out + t0) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
    } else {
#pragma unroll
        for (int i = 0; i < HX_VEC; ++i)
            if (t0 + i < p.L) out[t0 + i] = from_f32<T>(of[i]);
    }
}

}  // namespace vtx

extern "C" int vtx_hyena_x_fwd(const vtx_hyena_x_params* p, void* stream) {
    using namespace vtx;
    VTX_REQUIRE(p && p->q && p->k && p->v && p->h && p->y, VTX_ERR_BAD_ARG, "hyena_x: null pointer");
    VTX_REQUIRE(p->B > 0 && p->D > 0 && p->L > 0 && p->Lh > 0, VTX_ERR_BAD_ARG, "hyena_x: sizes must be positive");
    VTX_REQUIRE(p->Lh <= HX_MAX_TAPS, VTX_ERR_UNSUPPORTED, "hyena_x: filter length %lld > %d", (long long)p->Lh, HX_MAX_TAPS);
    VTX_REQUIRE(valid_dtype(p->io_dtype), VTX_ERR_BAD_ARG, "hyena_x: bad io dtype");
    const int64_t n = p->B * p->D * ((p->L + HX_VEC - 1) / HX_VEC);
    VTX_REQUIRE(n < ((int64_t)1 << 39), VTX_ERR_UNSUPPORTED, "hyena_x: problem too large");
    VTX_DISPATCH_IO(p->io_dtype, T,
                    hyena_x_kernel<T><<<(unsigned)ceil_div<int64_t>(n, 256), 256, 0, (cudaStream_t)stream>>>(*p));
    return check_launch("hyena_x");
}
