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

template <typename T>
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
    const int64_t t0 = (int64_t)blockIdx.x * FTT, c0 = (int64_t)blockIdx.y * FC, b = blockIdx.z;
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
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
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
                        p->C < ((int64_t)1 << 31) && ceil_div<int64_t>(p->L, FTT) < ((int64_t)1 << 31);
    if (tma_ok) {
        CUtensorMap tm_in, tm_out;
        if (int rc = make_tmap_3d(&tm_in, p->u, p->io_dtype, p->C, p->L, p->B, p->u_stride_l, p->u_stride_b, FC,
                                  FTT + (int)p->K - 1, 0, "featurizer"))
            return rc;
        if (int rc = make_tmap_3d(&tm_out, p->z, p->io_dtype, p->L, p->C, p->B, p->L, p->C * p->L, 64, FC, 128, "featurizer"))
            return rc;
        dim3 grid((unsigned)ceil_div<int64_t>(p->L, FTT), (unsigned)ceil_div<int64_t>(p->C, FC), (unsigned)p->B);
        if (p->io_dtype == VTX_BF16) {
            featurizer_tma_kernel<__nv_bfloat16><<<grid, 256, FT_SMEM, (cudaStream_t)stream>>>(tm_in, tm_out, *p);
        } else {
            featurizer_tma_kernel<__half><<<grid, 256, FT_SMEM, (cudaStream_t)stream>>>(tm_in, tm_out, *p);
        }
        return check_launch("featurizer");
    }
    dim3 grid((unsigned)ceil_div<int64_t>(p->L, FT), (unsigned)ceil_div<int64_t>(p->C, FC), (unsigned)p->B);
    VTX_DISPATCH_IO(p->io_dtype, T, featurizer_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>(*p));
    return check_launch("featurizer");
}
