// Backward of the gate -> grouped causal FIR -> gate operator on channel-last operands [B, L, D] (the reference's
// (bs, l, g, dg) tensors with the group axes merged): replaces two_pass_bwd_grouped (vortex/ops/hyena_se/bwd.py:11-330,
// kernels bwd_kernels.py:239,468) and its restatement gcg_two_pass_chunked_bwd (ref_bwd.py:31-115).
//
// Forward (ref_fwd.py:80-127):  z = B * x,  y2[t] = sum_k h[g, k] z[t - (hl-1) + k],  y = C * y2.
// With the lag j = hl-1-k and w[j] = h[g, hl-1-j]:
//   dC      = dy * y2                                   (y2 saved by the forward)
//   g2      = dy * C
//   dz[t]   = sum_j w[j] g2[t + j]                      (the same filter, run against time)
//   dx      = dz * B,   dB = dz * x
//   dw[j]   = sum over batch, time and the group's channels of g2[t] z[t - j]
// Two kernels on the fp32 pipe (fp32 accumulation, one rounding on the way out):
//   data    a block owns 128 outputs of 32 channels; g2 with its K-1 rows of look-ahead sits in shared memory, a thread
//           owns 16 consecutive samples of one channel and walks the taps 16 at a time with its window in registers
//           (256 FMAs per 47 shared loads);
//   filter  a block owns 256 rows of up to 16 channels of one group; a thread owns 8 taps of one channel with a sliding
//           window of z in registers (64 FMAs per 23 shared loads), the channels are summed by shuffles and the
//           block's partial sums are added to an fp32 [G, K] accumulator with atomics (the order of those additions
//           is not fixed: the last bits of dh can differ from run to run).
#include "common.cuh"

namespace vtx {
namespace gbw {

constexpr int TT = 128;        // outputs per block (data kernel)
constexpr int CT = 32;         // channels per block (data kernel)
constexpr int TPT = 16;        // outputs per thread
constexpr int KMAX = 128;
constexpr int DROWS = TT + KMAX - 1 + 1;       // g2 rows a block may touch (padded taps reach one row further)
constexpr int DATA_SMEM = (DROWS * CT + KMAX * CT + 2 * TT * CT) * 4;      // x and B tiles sized for fp32 I/O

// 16 bytes of a row as floats
template <typename T> struct Vec { static constexpr int N = 16 / sizeof(T); };
template <typename T>
__device__ __forceinline__ void ld16(const T* p, float (&v)[Vec<T>::N]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < Vec<T>::N; ++i) v[i] = to_f32<T>(e[i]);
}
template <typename T>
__device__ __forceinline__ void st16(T* p, const float (&v)[Vec<T>::N]) {
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < Vec<T>::N; ++i) e[i] = from_f32<T>(v[i]);
    *reinterpret_cast<uint4*>(p) = raw;
}

// VEC: every row piece is 16-byte aligned (checked by the host): the block's inputs are then fetched as 16-byte vectors
// with all loads of a pass in flight, dC leaves from that pass, and x and B wait in shared memory for the epilogue, so
// that no global load stands between the arithmetic and the stores.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) gcg_bwd_data_kernel(vtx_gcg_bwd_params p) {
    extern __shared__ float sm[];
    float* g2 = sm;                     // [rows][CT]
    float* ws = sm + DROWS * CT;        // [Kpad][CT]: w[j] of the channel's group
    T* xs = reinterpret_cast<T*>(ws + KMAX * CT);      // [TT][CT] in the I/O dtype (VEC)
    T* bs = xs + TT * CT;                               // [TT][CT] (VEC)
    const int tid = threadIdx.x, c = tid % CT, s = tid / CT;       // s: which 16 outputs of the 128
    const int64_t t0 = (int64_t)blockIdx.x * TT, c0 = (int64_t)blockIdx.y * CT, b = blockIdx.z;
    const int K = (int)p.K, Kpad = (K + 15) / 16 * 16, rows = TT + Kpad - 1;
    const int64_t dg = p.D / p.G;
    const T* dy = static_cast<const T*>(p.dy) + b * p.dy_stride_b;
    const T* Cg = static_cast<const T*>(p.C) + b * p.c_stride_b;
    const bool cok = c0 + c < p.D;
    if (VEC) {
        constexpr int NV = Vec<T>::N, TPR = CT / NV, RPP = 256 / TPR;      // threads per row, rows per pass
        const int vc = (tid % TPR) * NV, vr = tid / TPR;
        const T* xg = static_cast<const T*>(p.x) + b * p.x_stride_b + c0 + vc;
        const T* bg = static_cast<const T*>(p.Bg) + b * p.b_stride_b + c0 + vc;
        const T* yg = static_cast<const T*>(p.y2) + b * p.y2_stride_b + c0 + vc;
        T* dCg = static_cast<T*>(p.dC) + b * p.L * p.D + c0 + vc;
        const bool vok = c0 + vc < p.D;      // D is a multiple of NV: a vector is inside or outside as a whole
#pragma unroll 2
        for (int r = vr; r < rows; r += RPP) {
            const int64_t t = t0 + r;
            float a[NV], cc[NV], g[NV];
#pragma unroll
            for (int i = 0; i < NV; ++i) a[i] = cc[i] = 0.f;
            const bool in = vok && t < p.L;
            if (in) { ld16<T>(dy + t * p.dy_stride_l + c0 + vc, a); ld16<T>(Cg + t * p.c_stride_l + c0 + vc, cc); }
#pragma unroll
            for (int i = 0; i < NV; ++i) g[i] = a[i] * cc[i];
#pragma unroll
            for (int i = 0; i < NV; i += 4)
                *reinterpret_cast<float4*>(g2 + r * CT + vc + i) = make_float4(g[i], g[i + 1], g[i + 2], g[i + 3]);
            if (r < TT) {
                uint4 xr = make_uint4(0, 0, 0, 0), br = xr;
                if (in) {
                    xr = *reinterpret_cast<const uint4*>(xg + t * p.x_stride_l);
                    br = *reinterpret_cast<const uint4*>(bg + t * p.b_stride_l);
                    float yv[NV];
                    ld16<T>(yg + t * p.y2_stride_l, yv);
#pragma unroll
                    for (int i = 0; i < NV; ++i) yv[i] *= a[i];
                    st16<T>(dCg + t * p.D, yv);
                }
                *reinterpret_cast<uint4*>(xs + r * CT + vc) = xr;
                *reinterpret_cast<uint4*>(bs + r * CT + vc) = br;
            }
        }
    } else {
        for (int r = s; r < rows; r += 8) {
            const int64_t t = t0 + r;
            float v = 0.f;
            if (cok && t < p.L) v = to_f32<T>(dy[t * p.dy_stride_l + c0 + c]) * to_f32<T>(Cg[t * p.c_stride_l + c0 + c]);
            g2[r * CT + c] = v;
        }
    }
    for (int j = s; j < Kpad; j += 8) {
        float w = 0.f;
        if (cok && j < K) w = ld_param(p.h, p.h_dtype, ((c0 + c) / dg) * K + (K - 1 - j));
        ws[j * CT + c] = w;
    }
    __syncthreads();
    float acc[TPT];
#pragma unroll
    for (int i = 0; i < TPT; ++i) acc[i] = 0.f;
    const float* gcol = g2 + (s * TPT) * CT + c;
    for (int jb = 0; jb < Kpad; jb += 16) {
        float win[TPT + 15], w[16];
#pragma unroll
        for (int m = 0; m < TPT + 15; ++m) win[m] = gcol[(jb + m) * CT];
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) w[jj] = ws[(jb + jj) * CT + c];
#pragma unroll
        for (int jj = 0; jj < 16; ++jj)
#pragma unroll
            for (int i = 0; i < TPT; ++i) acc[i] = fmaf(w[jj], win[i + jj], acc[i]);
    }
    if (!cok) return;
    const T* x = static_cast<const T*>(p.x) + b * p.x_stride_b + c0 + c;
    const T* Bg = static_cast<const T*>(p.Bg) + b * p.b_stride_b + c0 + c;
    const T* y2 = static_cast<const T*>(p.y2) + b * p.y2_stride_b + c0 + c;
    T* dx = static_cast<T*>(p.dx) + b * p.L * p.D + c0 + c;
    T* dB = static_cast<T*>(p.dB) + b * p.L * p.D + c0 + c;
    T* dC = static_cast<T*>(p.dC) + b * p.L * p.D + c0 + c;
    if (VEC) {
#pragma unroll
        for (int i = 0; i < TPT; ++i) {
            const int64_t t = t0 + s * TPT + i;
            if (t >= p.L) break;
            dx[t * p.D] = from_f32<T>(acc[i] * to_f32<T>(bs[(s * TPT + i) * CT + c]));
            dB[t * p.D] = from_f32<T>(acc[i] * to_f32<T>(xs[(s * TPT + i) * CT + c]));
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < TPT; ++i) {
        const int64_t t = t0 + s * TPT + i;
        if (t >= p.L) break;
        const float xv = to_f32<T>(x[t * p.x_stride_l]), bv = to_f32<T>(Bg[t * p.b_stride_l]);
        dx[t * p.D] = from_f32<T>(acc[i] * bv);
        dB[t * p.D] = from_f32<T>(acc[i] * xv);
        dC[t * p.D] = from_f32<T>(to_f32<T>(dy[t * p.dy_stride_l + c0 + c]) * to_f32<T>(y2[t * p.y2_stride_l]));
    }
}

constexpr int FT = 256;        // rows per block (filter kernel)
constexpr int FC = 16;         // channels per block, all of one group
constexpr int ZP = 18;         // row pitch of the z tile in floats: rows 8 apart fall on different banks
constexpr int FILT_SMEM = (FT * FC + (FT + KMAX) * ZP) * 4;

template <typename T, bool VEC>
__global__ void __launch_bounds__(256) gcg_bwd_filter_kernel(vtx_gcg_bwd_params p, int cw) {
    extern __shared__ float sm[];
    float* g2 = sm;                   // [FT][FC]
    float* zs = sm + FT * FC;         // [FT + KMAX][ZP]: row r holds z at time t0 - KMAX + r
    const int tid = threadIdx.x, c = tid % FC, jb = tid / FC;      // jb: taps 8 jb .. 8 jb + 7 (lags)
    const int64_t t0 = (int64_t)blockIdx.x * FT, c0 = (int64_t)blockIdx.y * cw, b = blockIdx.z;
    const int K = (int)p.K;
    const int64_t dg = p.D / p.G;
    const bool cok = c < cw;
    const T* dy = static_cast<const T*>(p.dy) + b * p.dy_stride_b;
    const T* Cg = static_cast<const T*>(p.C) + b * p.c_stride_b;
    const T* x = static_cast<const T*>(p.x) + b * p.x_stride_b;
    const T* Bg = static_cast<const T*>(p.Bg) + b * p.b_stride_b;
    if (VEC) {        // cw == 16: a row piece is 16 channels, fetched as 16-byte vectors
        constexpr int NV = Vec<T>::N, TPR = FC / NV, RPP = 256 / TPR;
        const int vc = (tid % TPR) * NV, vr = tid / TPR;
#pragma unroll 2
        for (int r = vr; r < FT; r += RPP) {
            const int64_t t = t0 + r;
            float a[NV], cc[NV];
#pragma unroll
            for (int i = 0; i < NV; ++i) a[i] = cc[i] = 0.f;
            if (t < p.L) { ld16<T>(dy + t * p.dy_stride_l + c0 + vc, a); ld16<T>(Cg + t * p.c_stride_l + c0 + vc, cc); }
#pragma unroll
            for (int i = 0; i < NV; i += 4)
                *reinterpret_cast<float4*>(g2 + r * FC + vc + i) = make_float4(a[i] * cc[i], a[i + 1] * cc[i + 1], a[i + 2] * cc[i + 2], a[i + 3] * cc[i + 3]);
        }
#pragma unroll 2
        for (int r = vr; r < FT + KMAX; r += RPP) {
            const int64_t t = t0 - KMAX + r;
            float a[NV], cc[NV];
#pragma unroll
            for (int i = 0; i < NV; ++i) a[i] = cc[i] = 0.f;
            if (t >= 0 && t < p.L) { ld16<T>(x + t * p.x_stride_l + c0 + vc, a); ld16<T>(Bg + t * p.b_stride_l + c0 + vc, cc); }
#pragma unroll
            for (int i = 0; i < NV; ++i) zs[r * ZP + vc + i] = a[i] * cc[i];
        }
    } else {
        for (int r = jb; r < FT; r += 16) {
            const int64_t t = t0 + r;
            float v = 0.f;
            if (cok && t < p.L) v = to_f32<T>(dy[t * p.dy_stride_l + c0 + c]) * to_f32<T>(Cg[t * p.c_stride_l + c0 + c]);
            g2[r * FC + c] = v;
        }
        for (int r = jb; r < FT + KMAX; r += 16) {
            const int64_t t = t0 - KMAX + r;
            float v = 0.f;
            if (cok && t >= 0 && t < p.L) v = to_f32<T>(x[t * p.x_stride_l + c0 + c]) * to_f32<T>(Bg[t * p.b_stride_l + c0 + c]);
            zs[r * ZP + c] = v;
        }
    }
    __syncthreads();
    // acc[i]: lag j = 8 jb + i.  Rows in blocks of 8: a[u] = g2[t0 + 8 k + u], window zw[m] = z[t0 + 8 k + m - 7 - 8 jb],
    // so that g2[t] z[t - j] = a[u] zw[u - i + 7].
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    if (8 * jb < K) {
        for (int k = 0; k < FT / 8; ++k) {
            float a[8], zw[15];
#pragma unroll
            for (int u = 0; u < 8; ++u) a[u] = g2[(8 * k + u) * FC + c];
            const float* zr = zs + (KMAX + 8 * k - 7 - 8 * jb) * ZP + c;
#pragma unroll
            for (int m = 0; m < 15; ++m) zw[m] = zr[m * ZP];
#pragma unroll
            for (int u = 0; u < 8; ++u)
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] = fmaf(a[u], zw[u - i + 7], acc[i]);
        }
    }
    // sum over the block's channels (the 16 lanes of a half-warp), then one atomic per lag
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float v = acc[i];
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        const int j = 8 * jb + i;
        if (c == 0 && j < K) atomicAdd(p.dh32 + (c0 / dg) * K + (K - 1 - j), v);
    }
}

}  // namespace gbw
}  // namespace vtx

extern "C" int vtx_gcg_bwd(const vtx_gcg_bwd_params* p, void* stream) {
    using namespace vtx;
    using namespace vtx::gbw;
    VTX_REQUIRE(p && p->dy && p->x && p->Bg && p->C && p->y2 && p->h && p->dx && p->dB && p->dC && p->dh32, VTX_ERR_BAD_ARG,
                "gcg_bwd: null pointer");
    VTX_REQUIRE(p->B > 0 && p->L > 0 && p->D > 0 && p->G > 0 && p->K > 0, VTX_ERR_BAD_ARG, "gcg_bwd: sizes must be positive");
    VTX_REQUIRE(p->D % p->G == 0, VTX_ERR_BAD_ARG, "gcg_bwd: D not a multiple of G");
    VTX_REQUIRE(p->K <= KMAX, VTX_ERR_UNSUPPORTED, "gcg_bwd: filter length %lld > %d", (long long)p->K, KMAX);
    VTX_REQUIRE(valid_dtype(p->io_dtype) && valid_dtype(p->h_dtype), VTX_ERR_BAD_ARG, "gcg_bwd: bad dtype");
    VTX_REQUIRE(p->B <= 65535, VTX_ERR_UNSUPPORTED, "gcg_bwd: batch too large");
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t dg = p->D / p->G;
    int cw = 16;                       // channels per block of the filter kernel: a power of two that divides dg
    while (dg % cw) cw /= 2;
    const dim3 gd((unsigned)ceil_div<int64_t>(p->L, TT), (unsigned)ceil_div<int64_t>(p->D, CT), (unsigned)p->B);
    const dim3 gf((unsigned)ceil_div<int64_t>(p->L, FT), (unsigned)(p->D / cw), (unsigned)p->B);
    VTX_REQUIRE(gd.y <= 65535 && gf.y <= 65535, VTX_ERR_UNSUPPORTED, "gcg_bwd: too many channel tiles");
    static bool attr_set[64][3] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    // 16-byte vectors: every base, every row pitch and the channel count on 16-byte boundaries
    const int64_t es = dtype_size(p->io_dtype), nv = 16 / es;
    auto al = [&](const void* q, int64_t sb, int64_t sl) {
        return reinterpret_cast<uintptr_t>(q) % 16 == 0 && (sb * es) % 16 == 0 && (sl * es) % 16 == 0;
    };
    const bool vec = p->D % nv == 0 && al(p->dy, p->dy_stride_b, p->dy_stride_l) && al(p->x, p->x_stride_b, p->x_stride_l) &&
                     al(p->Bg, p->b_stride_b, p->b_stride_l) && al(p->C, p->c_stride_b, p->c_stride_l) &&
                     al(p->y2, p->y2_stride_b, p->y2_stride_l) && al(p->dC, p->L * p->D, p->D);
    VTX_DISPATCH_IO(p->io_dtype, T, {
        const int ti = p->io_dtype == VTX_F32 ? 0 : p->io_dtype == VTX_BF16 ? 1 : 2;
        if (dev < 0 || dev >= 64 || !attr_set[dev][ti]) {
            cudaFuncSetAttribute(gcg_bwd_data_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, DATA_SMEM);
            cudaFuncSetAttribute(gcg_bwd_data_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, DATA_SMEM);
            cudaFuncSetAttribute(gcg_bwd_filter_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, FILT_SMEM);
            cudaFuncSetAttribute(gcg_bwd_filter_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, FILT_SMEM);
            if (dev >= 0 && dev < 64) attr_set[dev][ti] = true;
        }
        const int dsm = (DROWS * CT + KMAX * CT) * 4 + (vec ? 2 * TT * CT * (int)sizeof(T) : 0);
        if (vec) gcg_bwd_data_kernel<T, true><<<gd, 256, dsm, s>>>(*p);
        else gcg_bwd_data_kernel<T, false><<<gd, 256, dsm, s>>>(*p);
        if (vec && cw == 16) gcg_bwd_filter_kernel<T, true><<<gf, 256, FILT_SMEM, s>>>(*p, cw);
        else gcg_bwd_filter_kernel<T, false><<<gf, 256, FILT_SMEM, s>>>(*p, cw);
    });
    return check_launch("gcg_bwd", 2);
}
