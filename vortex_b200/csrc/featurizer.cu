// Featurizer: depthwise causal FIR (K <= 8) over the packed projection
// channels, channel-last in -> channel-first out (a fused transpose), plus the
// FIR cache (the last K-1 input samples).
//
// One CTA owns a [64 time x 64 channel] tile.  Rows (time) are read with the
// channel index fastest, staged in shared memory together with K-1 halo rows,
// and written back with the time index fastest, so both sides are coalesced.
#include "common.cuh"

namespace vtx {

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
    dim3 grid((unsigned)ceil_div<int64_t>(p->L, FT), (unsigned)ceil_div<int64_t>(p->C, FC), (unsigned)p->B);
    VTX_DISPATCH_IO(p->io_dtype, T, featurizer_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>(*p));
    return check_launch("featurizer");
}
