// Featurizer: depthwise causal FIR (K <= 8) over the packed projection
// channels, channel-last in -> channel-first out (a fused transpose), plus the
// FIR cache (the last K-1 input samples).
//
// General kernel: one CTA owns a [64 time x 64 channel] tile.  Rows (time) are read with the
// channel index fastest, staged in shared memory together with K-1 halo rows,
// and written back with the time index fastest, so both sides are coalesced.
//
// 16-bit I/O with 16-byte aligned rows on both sides takes the TMA kernel further down: a [128 time x 64 channel]
// tile comes in as one box (its K-1 halo rows included, zeros before the sequence), every thread filters eight
// consecutive samples of one channel and writes them as one 16-byte vector into a [channel][time] tile laid out
// with the 128-byte swizzle (conflict-free for lanes on neighbouring channels), and two boxes of whole 128-byte
// rows along time carry the tile out.  Six CTAs per SM keep ~200 KB in flight; both directions move full lines.
#include "tma.cuh"
#include "umma.cuh"

namespace vtx {

VTX_DEFINE_STATUS_READER()

constexpr int FT = 64;   // time steps per tile
constexpr int FC = 64;   // channels per tile
constexpr int FK = 8;    // longest featurizer filter

template <typename T>
__global__ void __launch_bounds__(256) featurizer_kernel(vtx_featurizer_params p) {
    __shared__ float tile[FT + FK - 1][FC + 1];
    const int K = (int)p.K;
    const int64_t L = p.L, C = p.C;
    const int64_t t0 = (int64_t)blockIdx.x * FT;
    const int64_t c0 = (int64_t)blockIdx.y * FC;
    const int64_t b = blockIdx.z;
    const T* u = static_cast<const T*>(p.u) + b * p.u_stride_b;

    const int lane_c = threadIdx.x % FC, row0 = threadIdx.x / FC;
    for (int r = row0; r < FT + K - 1; r += 256 / FC) {
        int64_t t = t0 - (K - 1) + r, c = c0 + lane_c;
        float x = 0.f;
        if (t >= 0 && t < L && c < C) x = to_f32<T>(u[t * p.u_stride_l + c * p.u_stride_c]);
        tile[r][lane_c] = x;
    }
    __syncthreads();

    const int lt = threadIdx.x % FT, cc0 = threadIdx.x / FT;
    const int64_t t = t0 + lt;
    T* z = static_cast<T*>(p.z) + b * C * L;
    float m = 1.f;
    if (p.mask && t < L) m = ld_param(p.mask, p.mask_dtype, b * L + t);
    for (int cc = cc0; cc < FC; cc += 256 / FT) {
        int64_t c = c0 + cc;
        if (c >= C || t >= L) continue;
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < FK; ++j)
            if (j < K) acc = fmaf(ld_param(p.w, p.w_dtype, c * K + j), tile[lt + j][cc], acc);
        acc = round_io<T>(acc);
        if (p.bias) acc = round_io<T>(acc + ld_param(p.bias, p.bias_dtype, c));
        if (p.mask) acc = acc * m;
        z[c * L + t] = from_f32<T>(acc);
    }

    // FIR cache: the tile that holds the last sample also holds (in its halo) the K-1 before it.
    if (p.state && K > 1 && t0 + FT >= L) {
        const int64_t ns = L < K - 1 ? L : K - 1;
        T* st = static_cast<T*>(p.state) + b * C * ns;
        for (int i = threadIdx.x; i < FC * ns; i += 256) {
            int cc = i / (int)ns, s = i % (int)ns;
            int64_t c = c0 + cc;
            if (c >= C) continue;
            int64_t ts = L - ns + s;
            st[c * ns + s] = from_f32<T>(tile[ts - t0 + (K - 1)][cc]);
        }
    }
}


constexpr int FTT = 128;                  // time steps per tile of the TMA kernel
constexpr int FT_IN = (FTT + FK - 1) * FC * 2;           // input box: rows of 64 channels (128 bytes), 16-bit elements
constexpr int FT_OUT = FC * FTT * 2;                      // two [64 channels][64 samples] halves, 128-byte swizzle
constexpr int FT_SMEM = 1024 + FT_OUT + (FT_IN + 127) / 128 * 128 + FC * FK * 4 + 16;
static_assert(FT_SMEM <= 48 * 1024, "fits the default dynamic shared memory limit");

// two 16-bit elements in one word <-> a packed fp32 pair (low half = first element)
template <typename T> __device__ __forceinline__ umma::f32x2 unpack2(uint32_t w);
template <> __device__ __forceinline__ umma::f32x2 unpack2<__nv_bfloat16>(uint32_t w) { return umma::pk2(umma::bf_lo(w), umma::bf_hi(w)); }
template <> __device__ __forceinline__ umma::f32x2 unpack2<__half>(uint32_t w) {
    float lo, hi;
    asm("{\n\t.reg .f16 l, h;\n\tmov.b32 {l, h}, %2;\n\tcvt.f32.f16 %0, l;\n\tcvt.f32.f16 %1, h;\n\t}" : "=f"(lo), "=f"(hi) : "r"(w));
    return umma::pk2(lo, hi);
}
template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) { return umma::pack_bf16(lo, hi); }
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// PLAIN3: three taps, no bias, no mask (the featurizer of every shipped model configuration): a thread filters eight
// samples of a channel PAIR with packed fp32 arithmetic, one rounding on the way out.
template <typename T, bool PLAIN3>
__global__ void __launch_bounds__(256) featurizer_tma_kernel(const __grid_constant__ CUtensorMap tm_in,
                                                            const __grid_constant__ CUtensorMap tm_out,
                                                            vtx_featurizer_params p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sm_u = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* sm = reinterpret_cast<uint8_t*>(__cvta_shared_to_generic(sm_u));
    constexpr int OFF_IN = FT_OUT, OFF_W = FT_OUT + (FT_IN + 127) / 128 * 128, OFF_BAR = OFF_W + FC * FK * 4;
    const T* in = reinterpret_cast<const T*>(sm + OFF_IN);
    float* ws = reinterpret_cast<float*>(sm + OFF_W);
    const uint32_t bar = sm_u + OFF_BAR;
    const int K = (int)p.K, tid = threadIdx.x;
    const int64_t L = p.L, C = p.C;
    // (channel tiles are the fastest grid dimension: CTAs that run together read neighbouring pieces of the same rows)
    const int64_t t0 = (int64_t)blockIdx.y * FTT, c0 = (int64_t)blockIdx.x * FC, b = blockIdx.z;
    if (tid == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
        mbar_expect_tx(bar, (uint32_t)((FTT + K - 1) * FC * 2));
        tma_load_3d(sm_u + OFF_IN, &tm_in, bar, (int)c0, (int)(t0 - (K - 1)), (int)b);
    }
    for (int i = tid; i < FC * K; i += 256) {
        const int64_t c = c0 + i / K;
        ws[(i / K) * FK + i % K] = c < C ? ld_param(p.w, p.w_dtype, c * K + i % K) : 0.f;
    }
    __syncthreads();
    if (!mbar_wait(bar, 0, 51)) return;
    if (PLAIN3) {
        // task = (channel pair, block of 8 samples); the lanes of a warp cover the 64 channels of a row
        using namespace umma;
#pragma unroll 1
        for (int task = tid; task < (FC / 2) * (FTT / 8); task += 256) {
            const int cp = task % (FC / 2), t8 = task / (FC / 2);
            f32x2 wv[3];
#pragma unroll
            for (int j = 0; j < 3; ++j) wv[j] = pk2(ws[(2 * cp) * FK + j], ws[(2 * cp + 1) * FK + j]);
            const uint32_t src = sm_u + OFF_IN + (uint32_t)(t8 * 8 * FC * 2 + cp * 4);
            f32x2 x[10];
#pragma unroll
            for (int i = 0; i < 10; ++i) {
                uint32_t w;
                asm volatile("ld.shared.b32 %0, [%1];" : "=r"(w) : "r"(src + (uint32_t)(i * FC * 2)));
                x[i] = unpack2<T>(w);
            }
            float lo[8], hi[8];
#pragma unroll
            for (int e = 0; e < 8; ++e)        // same order of operations as the general kernel: identical bits
                up2(fma2(wv[2], x[e + 2], fma2(wv[1], x[e + 1], mul2(wv[0], x[e]))), lo[e], hi[e]);
            const uint32_t dst = sm_u + (uint32_t)((t8 / 8) * (FT_OUT / 2));
            const int r0 = 2 * cp, r1 = 2 * cp + 1;
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + (uint32_t)(r0 * 128 + (((t8 % 8) ^ (r0 & 7)) << 4))),
                         "r"(pack2<T>(lo[0], lo[1])), "r"(pack2<T>(lo[2], lo[3])), "r"(pack2<T>(lo[4], lo[5])), "r"(pack2<T>(lo[6], lo[7])) : "memory");
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + (uint32_t)(r1 * 128 + (((t8 % 8) ^ (r1 & 7)) << 4))),
                         "r"(pack2<T>(hi[0], hi[1])), "r"(pack2<T>(hi[2], hi[3])), "r"(pack2<T>(hi[4], hi[5])), "r"(pack2<T>(hi[6], hi[7])) : "memory");
        }
    } else
    // task = (channel, block of 8 samples); lanes run along channels
    for (int task = tid; task < FC * (FTT / 8); task += 256) {
        const int cc = task % FC, t8 = task / FC;
        const int64_t c = c0 + cc;
        float x[8 + FK - 1];
#pragma unroll
        for (int i = 0; i < 8 + FK - 1; ++i) x[i] = i < 8 + K - 1 ? to_f32<T>(in[(t8 * 8 + i) * FC + cc]) : 0.f;
        float wv[FK];
#pragma unroll
        for (int j = 0; j < FK; ++j) wv[j] = ws[cc * FK + j];
        const float bias = (p.bias && c < C) ? ld_param(p.bias, p.bias_dtype, c) : 0.f;
        alignas(16) T out[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < FK; ++j)
                if (j < K) acc = fmaf(wv[j], x[e + j], acc);
            acc = round_io<T>(acc);
            if (p.bias) acc = round_io<T>(acc + bias);
            if (p.mask) {
                const int64_t t = t0 + t8 * 8 + e;
                acc = acc * (t < L ? ld_param(p.mask, p.mask_dtype, b * L + t) : 0.f);
            }
            out[e] = from_f32<T>(acc);
        }
        *reinterpret_cast<uint4*>(sm + (t8 / 8) * (FT_OUT / 2) + cc * 128 + (((t8 % 8) ^ (cc & 7)) << 4)) =
            *reinterpret_cast<const uint4*>(out);
    }
    // FIR cache: the tile that holds the last sample also holds (in its halo) the K-1 before it
    if (p.state && K > 1 && t0 + FTT >= L) {
        const int64_t ns = L < K - 1 ? L : K - 1;
        T* st = static_cast<T*>(p.state) + b * C * ns;
        for (int i = tid; i < FC * ns; i += 256) {
            const int cc = i / (int)ns, s = i % (int)ns;
            if (c0 + cc < C) st[(c0 + cc) * ns + s] = in[(L - ns + s - t0 + (K - 1)) * FC + cc];
        }
    }
    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf)
            if (t0 + hf * 64 < L) tma_store_3d(&tm_out, sm_u + hf * (FT_OUT / 2), (int)(t0 + hf * 64), (int)c0, (int)b);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");     // the tile has left shared memory: the CTA may go
    }
}

}  // namespace vtx

extern "C" int vtx_featurizer_fwd(const vtx_featurizer_params* p, void* stream) {
    using namespace vtx;
    VTX_REQUIRE(p && p->u && p->w && p->z, VTX_ERR_BAD_ARG, "featurizer: null pointer");
    VTX_REQUIRE(p->B > 0 && p->L > 0 && p->C > 0, VTX_ERR_BAD_ARG, "featurizer: B, L, C must be positive");
    VTX_REQUIRE(p->K >= 1 && p->K <= FK, VTX_ERR_UNSUPPORTED, "featurizer: filter length %lld not in [1, %d]",
                (long long)p->K, FK);
    VTX_REQUIRE(p->B <= 65535 && ceil_div<int64_t>(p->C, FC) <= 65535, VTX_ERR_UNSUPPORTED,
                "featurizer: B or C too large for one launch");
    VTX_REQUIRE(valid_dtype(p->w_dtype) && (!p->bias || valid_dtype(p->bias_dtype)) &&
                    (!p->mask || valid_dtype(p->mask_dtype)),
                VTX_ERR_BAD_ARG, "featurizer: bad parameter dtype");
    const bool tma_ok = p->io_dtype != VTX_F32 && p->u_stride_c == 1 && reinterpret_cast<uintptr_t>(p->u) % 16 == 0 &&
                        p->u_stride_l % 8 == 0 && (p->B == 1 || p->u_stride_b % 8 == 0) && p->u_stride_l > 0 &&
                        reinterpret_cast<uintptr_t>(p->z) % 16 == 0 && p->L % 8 == 0 && p->L < ((int64_t)1 << 31) - 256 &&
                        p->C < ((int64_t)1 << 31) && ceil_div<int64_t>(p->L, FTT) <= 65535;
    if (tma_ok) {
        CUtensorMap tm_in, tm_out;
        if (int rc = make_tmap_3d(&tm_in, p->u, p->io_dtype, p->C, p->L, p->B, p->u_stride_l, p->u_stride_b, FC,
                                  FTT + (int)p->K - 1, 0, "featurizer"))
            return rc;
        if (int rc = make_tmap_3d(&tm_out, p->z, p->io_dtype, p->L, p->C, p->B, p->L, p->C * p->L, 64, FC, 128, "featurizer"))
            return rc;
        dim3 grid((unsigned)ceil_div<int64_t>(p->C, FC), (unsigned)ceil_div<int64_t>(p->L, FTT), (unsigned)p->B);
        const bool plain3 = p->K == 3 && !p->bias && !p->mask;
        cudaStream_t st = (cudaStream_t)stream;
        if (p->io_dtype == VTX_BF16) {
            if (plain3) featurizer_tma_kernel<__nv_bfloat16, true><<<grid, 256, FT_SMEM, st>>>(tm_in, tm_out, *p);
            else featurizer_tma_kernel<__nv_bfloat16, false><<<grid, 256, FT_SMEM, st>>>(tm_in, tm_out, *p);
        } else {
            if (plain3) featurizer_tma_kernel<__half, true><<<grid, 256, FT_SMEM, st>>>(tm_in, tm_out, *p);
            else featurizer_tma_kernel<__half, false><<<grid, 256, FT_SMEM, st>>>(tm_in, tm_out, *p);
        }
        return check_launch("featurizer");
    }
    dim3 grid((unsigned)ceil_div<int64_t>(p->L, FT), (unsigned)ceil_div<int64_t>(p->C, FC), (unsigned)p->B);
    VTX_DISPATCH_IO(p->io_dtype, T, featurizer_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>(*p));
    return check_launch("featurizer");
}
