// Gate -> grouped causal FIR -> gate on channel-first tensors, fp32 math on
// CUDA cores.  General path: any filter length, any I/O dtype, either tap
// convention.  One CTA owns one (batch, channel) row and a tile of GT output
// samples; k*v for the tile and its K-1 halo is staged in shared memory, and
// every thread slides a register window over it to produce GR consecutive
// outputs (GR FMAs per shared-memory word loaded).
#include "common.cuh"

namespace vtx {

constexpr int GR = 8;                 // outputs per thread
constexpr int GTHREADS = 128;
constexpr int GT = GR * GTHREADS;     // outputs per CTA
constexpr int GCG_MAX_K = 8192;

template <typename T>
__global__ void __launch_bounds__(GTHREADS) gcg_kernel(vtx_gcg_params p) {
    extern __shared__ float smem[];
    const int K = (int)p.K;
    const int Kp = (K + GR - 1) / GR * GR;   // taps padded with zeros to a multiple of GR
    float* hs = smem;                        // [Kp]   taps in cross-correlation order
    float* kv = smem + Kp;                   // [GT + Kp + GR]  kv[i] = sample t0 - (Kp-1) + i

    const int64_t L = p.L;
    const int64_t t0 = (int64_t)blockIdx.x * GT;
    const int64_t d = blockIdx.y, b = blockIdx.z;
    const int64_t g = d / (p.D / p.G);
    const int64_t hn = d / p.head_dim, hj = d % p.head_dim;
    const T* q = static_cast<const T*>(p.q) + b * p.q_stride_b + hn * p.q_stride_h + hj * p.q_stride_d;
    const T* k = static_cast<const T*>(p.k) + b * p.k_stride_b + hn * p.k_stride_h + hj * p.k_stride_d;
    const T* v = static_cast<const T*>(p.v) + b * p.v_stride_b + hn * p.v_stride_h + hj * p.v_stride_d;

    // y[t] = sum_m hs[m] * x[t - (Kp-1) + m]; padded taps sit at the front (oldest samples).
    for (int m = threadIdx.x; m < Kp; m += GTHREADS) {
        int j = m - (Kp - K);                // index into the K real taps, cross-correlation order
        float w = 0.f;
        if (j >= 0) {
            int src = p.taps == VTX_TAPS_CONV ? (K - 1 - j) : j;
            // the FFT path cuts the filter to the sequence length (taps beyond L never meet data anyway)
            w = ld_param(p.h, p.h_dtype, g * K + src);
        }
        hs[m] = w;
    }
    const int n_stage = GT + Kp + GR;
    for (int i = threadIdx.x; i < n_stage; i += GTHREADS) {
        int64_t t = t0 - (Kp - 1) + i;
        float x = 0.f;
        if (t >= 0 && t < L) {
            x = to_f32<T>(k[t]) * to_f32<T>(v[t]);
            if (p.round_kv) x = round_io<T>(x);
        }
        kv[i] = x;
    }
    __syncthreads();

    const int base = threadIdx.x * GR;
    float acc[GR];
#pragma unroll
    for (int r = 0; r < GR; ++r) acc[r] = 0.f;
    float win[2 * GR];
#pragma unroll
    for (int r = 0; r < GR; ++r) win[r] = kv[base + r];
    for (int m0 = 0; m0 < Kp; m0 += GR) {
#pragma unroll
        for (int r = 0; r < GR; ++r) win[GR + r] = kv[base + m0 + GR + r];
#pragma unroll
        for (int mm = 0; mm < GR; ++mm) {
            float w = hs[m0 + mm];
#pragma unroll
            for (int r = 0; r < GR; ++r) acc[r] = fmaf(w, win[r + mm], acc[r]);
        }
#pragma unroll
        for (int r = 0; r < GR; ++r) win[r] = win[GR + r];
    }

    float bias = 0.f;
    if (p.bias_mode != VTX_BIAS_NONE) bias = ld_param(p.bias, p.bias_dtype, d);
    T* y = static_cast<T*>(p.y) + b * p.y_stride_b + d * p.y_stride_d;
#pragma unroll
    for (int r = 0; r < GR; ++r) {
        int64_t t = t0 + base + r;
        if (t >= L) break;
        float x = kv[base + r + Kp - 1];
        float z;
        if (p.taps == VTX_TAPS_CONV) {
            // fp32 sum of the filter output and the skip term, one rounding (engine.py:78,187)
            z = round_io<T>(p.bias_mode == VTX_BIAS_GATED ? fmaf(bias, x, acc[r]) : acc[r] + bias);
        } else {
            z = round_io<T>(acc[r]);
            if (p.bias_mode == VTX_BIAS_GATED) z = round_io<T>(z + round_io<T>(bias * x));
            else if (p.bias_mode == VTX_BIAS_ADD) z = round_io<T>(z + bias);
        }
        if (p.mask) z *= ld_param(p.mask, p.mask_dtype, b * L + t);
        y[t * p.y_stride_l] = from_f32<T>(to_f32<T>(q[t]) * z);
    }

    if (p.state && K > 1 && t0 + GT >= L) {
        const int64_t ns = L < K - 1 ? L : K - 1;
        T* st = static_cast<T*>(p.state) + (b * p.D + d) * ns;
        for (int s = threadIdx.x; s < ns; s += GTHREADS) {
            int64_t ts = L - ns + s;
            st[s] = from_f32<T>(kv[ts - t0 + (Kp - 1)]);
        }
    }
}

bool gcg_tc_shape(const vtx_gcg_params* p);                    // gcg_tc.cu (tcgen05 path)
int gcg_tc_fwd(const vtx_gcg_params* p, cudaStream_t stream);

}  // namespace vtx

extern "C" int vtx_gcg_fwd(const vtx_gcg_params* p, void* stream) {
    using namespace vtx;
    VTX_REQUIRE(p && p->q && p->k && p->v && p->h && p->y, VTX_ERR_BAD_ARG, "gcg: null pointer");
    VTX_REQUIRE(p->B > 0 && p->L > 0 && p->D > 0 && p->G > 0 && p->K > 0, VTX_ERR_BAD_ARG,
                "gcg: sizes must be positive");
    VTX_REQUIRE(p->D % p->G == 0, VTX_ERR_BAD_ARG, "gcg: D=%lld not a multiple of G=%lld", (long long)p->D,
                (long long)p->G);
    VTX_REQUIRE(p->head_dim > 0 && p->D % p->head_dim == 0, VTX_ERR_BAD_ARG, "gcg: head_dim must divide D");
    VTX_REQUIRE(p->K <= GCG_MAX_K, VTX_ERR_UNSUPPORTED, "gcg: filter length %lld > %d", (long long)p->K, GCG_MAX_K);
    VTX_REQUIRE(p->B <= 65535 && p->D <= 65535, VTX_ERR_UNSUPPORTED, "gcg: B or D too large for one launch");
    VTX_REQUIRE(p->bias_mode == VTX_BIAS_NONE || p->bias, VTX_ERR_BAD_ARG, "gcg: bias mode set without a bias");
    VTX_REQUIRE(valid_dtype(p->h_dtype), VTX_ERR_BAD_ARG, "gcg: bad filter dtype");
    // Kernel choice: bf16 I/O with bf16 filters of up to 128 taps shared by blocks of 16 channels (time-contiguous,
    // 16-byte aligned operands) runs as a blocked-Toeplitz contraction on tensor cores; the kernel below takes the rest.
    if (gcg_tc_shape(p)) return gcg_tc_fwd(p, (cudaStream_t)stream);
    const int Kp = (int)((p->K + GR - 1) / GR * GR);
    const size_t smem = sizeof(float) * (size_t)(Kp + GT + Kp + GR);
    dim3 grid((unsigned)ceil_div<int64_t>(p->L, GT), (unsigned)p->D, (unsigned)p->B);
    cudaStream_t s = (cudaStream_t)stream;
    VTX_DISPATCH_IO(p->io_dtype, T, {
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(gcg_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return fail(VTX_ERR_LAUNCH, "gcg: shared memory opt-in: %s", cudaGetErrorString(e));
        }
        gcg_kernel<T><<<grid, GTHREADS, smem, s>>>(*p);
    });
    return check_launch("gcg");
}
