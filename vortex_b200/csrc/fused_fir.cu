// Fused Hyena short-filter block on the channel-last projection output:
//   featurizer FIR (3 taps) -> q/k/v selection -> k*v -> grouped FIR (K <= 16) -> q gate
// in ONE pass over HBM (3 reads + 1 write per hidden channel and token).
//
// Bandwidth-bound design.  The unit of work is a warp task: one batch element,
// a slab of 64 hidden channels (192 packed columns) and a segment of the time
// axis.  A CTA is a single warp that runs its own TMA pipeline: lane 0 issues
// cp.async.bulk.tensor loads of [ROWS x 192] boxes (rows = time) into a ring of
// shared-memory stages guarded by mbarriers, all lanes consume.  Each lane owns
// two adjacent hidden channels and walks down the time axis keeping the
// featurizer history and the k*v window in registers, so nothing is re-read
// and every shared-memory word is touched once.  The halo at the start of a
// segment ((3-1) + (K-1) rows) is recomputed, not communicated; rows before
// the sequence start come back from TMA as zeros.  Stores are 4-byte (8-byte
// for fp32) per lane, 128 B per warp and row.
//
// The caches (last 2 projection rows, last K-1 values of k*v) are produced by
// a second, tiny kernel that recomputes the few rows it needs.
#include "tma.cuh"

namespace vtx {

VTX_DEFINE_STATUS_READER()

constexpr int FF_CH = 64;        // hidden channels per warp task
constexpr int FF_STAGES = 3;
constexpr int FF_STAGE_BYTES = 6144;
constexpr int FF_K3 = 3;

struct FusedArgs {
    const void* w3; int64_t w3_dtype;
    const void* b3; int64_t b3_dtype;
    const void* h;  int64_t h_dtype;
    const void* bias; int64_t bias_dtype;
    void* y; int64_t y_stride_b, y_stride_l;
    int64_t B, L, D, G, K;
    int64_t nslab, nseg, seg_len;
    int layout, flip, taps, bias_mode;
    int64_t hd;       // channels per head (column split)
    int64_t hist;     // rows before u[b][0] that hold the sequence's earlier samples (chunked prefill), 0 or >= K + 1
};

// Packed-column base of the q, k, v planes of a slab (plane layouts only).
__device__ __forceinline__ void plane_cols(const FusedArgs& a, int64_t d0, int64_t (&col)[3]) {
    if (a.layout == VTX_QKV_COLUMN_SPLIT) {
        int64_t n = d0 / a.hd, j = d0 - n * a.hd;
        col[0] = n * 3 * a.hd + j; col[1] = col[0] + a.hd; col[2] = col[0] + 2 * a.hd;
    } else {
        col[0] = d0; col[1] = a.D + d0; col[2] = 2 * a.D + d0;
    }
    if (a.flip) { int64_t t = col[0]; col[0] = col[1]; col[1] = t; }
}

template <typename T> struct Pair;   // two adjacent elements
template <> struct Pair<float> { using type = float2; };
template <> struct Pair<__nv_bfloat16> { using type = __nv_bfloat162; };
template <> struct Pair<__half> { using type = __half2; };

__device__ __forceinline__ float2 pair_to_f32(float2 x) { return x; }
__device__ __forceinline__ float2 pair_to_f32(__nv_bfloat162 x) { return __bfloat1622float2(x); }
__device__ __forceinline__ float2 pair_to_f32(__half2 x) { return __half22float2(x); }
template <typename T> __device__ __forceinline__ typename Pair<T>::type pair_from_f32(float a, float b);
template <> __device__ __forceinline__ float2 pair_from_f32<float>(float a, float b) { return make_float2(a, b); }
template <> __device__ __forceinline__ __nv_bfloat162 pair_from_f32<__nv_bfloat16>(float a, float b) {
    return __floats2bfloat162_rn(a, b);
}
template <> __device__ __forceinline__ __half2 pair_from_f32<__half>(float a, float b) { return __floats2half2_rn(a, b); }

// INTERLEAVED: stage = [ROWS][192]; lane reads 6 consecutive elements (q0 k0 v0 q1 k1 v1).
// planes     : stage = [3][ROWS][64]; lane reads 2 consecutive elements of each plane.
template <typename T, bool INTERLEAVED, int KMAX>
__global__ void __launch_bounds__(32) fused_fir_kernel(const __grid_constant__ CUtensorMap tmap, FusedArgs a) {
    constexpr int ROWS = FF_STAGE_BYTES / (3 * FF_CH * (int)sizeof(T));
    using P = typename Pair<T>::type;
    extern __shared__ uint8_t smem_raw[];
    // stages first (128-byte aligned for TMA), then the barriers
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + FF_STAGES * FF_STAGE_BYTES);
    const int lane = threadIdx.x;

    // task decode: neighbouring CTAs take neighbouring slabs of the same rows
    int64_t task = blockIdx.x;
    const int64_t slab = task % a.nslab; task /= a.nslab;
    const int64_t seg = task % a.nseg;
    const int64_t b = task / a.nseg;
    const int64_t d0 = slab * FF_CH;
    const int K = (int)a.K;
    const int halo = (FF_K3 - 1) + (K - 1);
    const int64_t ts = seg * a.seg_len;
    const int64_t te = ts + a.seg_len < a.L ? ts + a.seg_len : a.L;
    const int64_t row0 = ts - halo;
    const int nstages = (int)((te - row0 + ROWS - 1) / ROWS);
    const int64_t tmin = a.hist > 2 ? -(a.hist - 2) : 0;      // first sample whose featurizer output is complete

    int64_t pcol[3] = {0, 0, 0};
    if (!INTERLEAVED) plane_cols(a, d0, pcol);

    auto issue = [&](int s) {
        const int slot = s % FF_STAGES;
        const uint32_t bar = smem_u32(&bars[slot]);
        const uint32_t dst = smem_u32(base + slot * FF_STAGE_BYTES);
        const int r = (int)(row0 + (int64_t)s * ROWS + a.hist);      // the tensor map starts a.hist rows before u
        mbar_expect_tx(bar, FF_STAGE_BYTES);
        if (INTERLEAVED) {
            tma_load_3d(dst, &tmap, bar, (int)(3 * d0), r, (int)b);
        } else {
#pragma unroll
            for (int pl = 0; pl < 3; ++pl)
                tma_load_3d(dst + pl * (FF_STAGE_BYTES / 3), &tmap, bar, (int)pcol[pl], r, (int)b);
        }
    };

    if (lane == 0) {
        tma_prefetch_desc(&tmap);
        for (int s = 0; s < FF_STAGES; ++s) mbar_init(smem_u32(&bars[s]), 1);
        fence_mbar_init();
        fence_proxy_async_smem();
        for (int s = 0; s < FF_STAGES && s < nstages; ++s) issue(s);
    }

    // ---- per-lane constants: two hidden channels dA = d0 + 2*lane, dB = dA + 1 --------------------
    const int64_t dA = d0 + 2 * lane;
    float w3[2][3][FF_K3], b3[2][3], h[2][KMAX], bias[2];
    {
        // interleaved: parameters by raw position in the triple, the flip is applied when q and k
        // are picked (iq/ik below); planes: the flip already swapped the q and k planes
        QkvMap map{a.layout, INTERLEAVED ? 0 : a.flip, a.D, a.hd};
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int64_t d = dA + c < a.D ? dA + c : a.D - 1;   // clamp: lanes past D compute but never store
            int64_t pc[3];
            map.get(d, pc[0], pc[1], pc[2]);
#pragma unroll
            for (int s = 0; s < 3; ++s) {
#pragma unroll
                for (int j = 0; j < FF_K3; ++j) w3[c][s][j] = ld_param(a.w3, a.w3_dtype, pc[s] * FF_K3 + j);
                b3[c][s] = a.b3 ? ld_param(a.b3, a.b3_dtype, pc[s]) : 0.f;
            }
            const int64_t g = d / (a.D / a.G);
            // taps in cross-correlation order, zero-padded at the old end: y[t] = sum_m h[m] kv[t-(KMAX-1)+m]
#pragma unroll
            for (int m = 0; m < KMAX; ++m) {
                int j = m - (KMAX - K);
                h[c][m] = j >= 0 ? ld_param(a.h, a.h_dtype, g * K + (a.taps == VTX_TAPS_CONV ? K - 1 - j : j)) : 0.f;
            }
            bias[c] = a.bias_mode != VTX_BIAS_NONE ? ld_param(a.bias, a.bias_dtype, d) : 0.f;
        }
    }
    float xh[2][3][FF_K3 - 1];     // featurizer history, oldest first
    float kvw[2][KMAX - 1];        // k*v window, oldest first
#pragma unroll
    for (int c = 0; c < 2; ++c) {
#pragma unroll
        for (int s = 0; s < 3; ++s)
#pragma unroll
            for (int j = 0; j < FF_K3 - 1; ++j) xh[c][s][j] = 0.f;
#pragma unroll
        for (int j = 0; j < KMAX - 1; ++j) kvw[c][j] = 0.f;
    }
    // with flip_x1x2 the interleaved triple is (k, q, v); planes were already swapped through pcol/map
    const bool swap_qk = INTERLEAVED && a.flip;

    T* y = static_cast<T*>(a.y) + b * a.y_stride_b + dA;
    const bool store_pair = dA + 1 < a.D;
    const bool store_one = dA < a.D;
    __syncwarp();

    for (int s = 0; s < nstages; ++s) {
        const int slot = s % FF_STAGES;
        if (!mbar_wait(smem_u32(&bars[slot]), (uint32_t)((s / FF_STAGES) & 1), 1)) return;
        const T* st = reinterpret_cast<const T*>(base + slot * FF_STAGE_BYTES);
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            const int64_t t = row0 + (int64_t)s * ROWS + r;
            float x[2][3];
            if (INTERLEAVED) {
                const P* row = reinterpret_cast<const P*>(st + r * 3 * FF_CH) + 3 * lane;
                float2 e0 = pair_to_f32(row[0]), e1 = pair_to_f32(row[1]), e2 = pair_to_f32(row[2]);
                x[0][0] = e0.x; x[0][1] = e0.y; x[0][2] = e1.x; x[1][0] = e1.y; x[1][1] = e2.x; x[1][2] = e2.y;
            } else {
#pragma unroll
                for (int pl = 0; pl < 3; ++pl) {
                    float2 e = pair_to_f32(reinterpret_cast<const P*>(st + (pl * ROWS + r) * FF_CH)[lane]);
                    x[0][pl] = e.x; x[1][pl] = e.y;
                }
            }
            float out[2];
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                float z[3];
#pragma unroll
                for (int sx = 0; sx < 3; ++sx) {
                    float acc = fmaf(w3[c][sx][FF_K3 - 1], x[c][sx], b3[c][sx]);
#pragma unroll
                    for (int j = 0; j < FF_K3 - 1; ++j) acc = fmaf(w3[c][sx][j], xh[c][sx][j], acc);
#pragma unroll
                    for (int j = 0; j < FF_K3 - 2; ++j) xh[c][sx][j] = xh[c][sx][j + 1];
                    xh[c][sx][FF_K3 - 2] = x[c][sx];
                    z[sx] = acc;
                }
                const float zq = swap_qk ? z[1] : z[0], zk = swap_qk ? z[0] : z[1];
                float kv = t >= tmin ? zk * z[2] : 0.f;
                float acc = h[c][KMAX - 1] * kv;
#pragma unroll
                for (int m = 0; m < KMAX - 1; ++m) acc = fmaf(h[c][m], kvw[c][m], acc);
#pragma unroll
                for (int m = 0; m < KMAX - 2; ++m) kvw[c][m] = kvw[c][m + 1];
                kvw[c][KMAX - 2] = kv;
                if (a.bias_mode == VTX_BIAS_GATED) acc = fmaf(bias[c], kv, acc);
                else if (a.bias_mode == VTX_BIAS_ADD) acc += bias[c];
                out[c] = zq * acc;
            }
            if (t >= ts && t < te) {
                T* yr = y + t * a.y_stride_l;
                if (store_pair) *reinterpret_cast<P*>(yr) = pair_from_f32<T>(out[0], out[1]);
                else if (store_one) yr[0] = from_f32<T>(out[0]);
            }
        }
        __syncwarp();
        if (lane == 0 && s + FF_STAGES < nstages) issue(s + FF_STAGES);
    }
}

// Caches after prefill: fir_state[b, c, :] = u[b, L-n3:L, c] (n3 = min(L, 2)),
// inner_state[b, d, :] = round(kv[b, d, L-ns:L]) (ns = min(L, K-1)); thread per (b, d).
template <typename T>
__global__ void fused_state_kernel(const T* __restrict__ u, int64_t u_stride_b, int64_t u_stride_l, FusedArgs a,
                                   T* fir_state, T* inner_state) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.B * a.D) return;
    const int64_t b = i / a.D, d = i % a.D;
    QkvMap map{a.layout, a.flip, a.D, a.hd};
    int64_t pc[3];
    map.get(d, pc[0], pc[1], pc[2]);
    const T* ub = u + b * u_stride_b;
    // with history rows before u the caches are always full (negative times index those rows)
    if (fir_state) {
        const int64_t n3 = (a.hist > 0 || a.L >= FF_K3 - 1) ? FF_K3 - 1 : a.L;
        for (int s = 0; s < 3; ++s)
            for (int64_t j = 0; j < n3; ++j)
                fir_state[(b * 3 * a.D + pc[s]) * n3 + j] = ub[(a.L - n3 + j) * u_stride_l + pc[s]];
    }
    if (inner_state) {
        const int64_t ns = (a.hist > 0 || a.L >= a.K - 1) ? a.K - 1 : a.L;
        for (int64_t j = 0; j < ns; ++j) {
            const int64_t t = a.L - ns + j;
            float z[3];
            for (int s = 1; s < 3; ++s) {
                float acc = a.b3 ? ld_param(a.b3, a.b3_dtype, pc[s]) : 0.f;
                for (int jj = 0; jj < FF_K3; ++jj) {
                    int64_t tt = t - (FF_K3 - 1) + jj;
                    if (tt >= -a.hist) acc = fmaf(ld_param(a.w3, a.w3_dtype, pc[s] * FF_K3 + jj), to_f32<T>(ub[tt * u_stride_l + pc[s]]), acc);
                }
                z[s] = acc;
            }
            inner_state[(b * a.D + d) * ns + j] = from_f32<T>(z[1] * z[2]);
        }
    }
}

template <typename T, bool INTERLEAVED>
static int launch_fused(const vtx_fused_fir_params* p, const FusedArgs& a, const CUtensorMap& tmap, cudaStream_t s) {
    const size_t smem = FF_STAGES * FF_STAGE_BYTES + FF_STAGES * sizeof(uint64_t) + 128;
    const int64_t ntask = a.B * a.nslab * a.nseg;
    if (a.K <= 8) fused_fir_kernel<T, INTERLEAVED, 8><<<(unsigned)ntask, 32, smem, s>>>(tmap, a);
    else fused_fir_kernel<T, INTERLEAVED, 16><<<(unsigned)ntask, 32, smem, s>>>(tmap, a);
    if (int rc = check_launch("fused_fir")) return rc;
    if (p->fir_state || p->inner_state) {
        fused_state_kernel<T><<<(unsigned)ceil_div<int64_t>(a.B * a.D, 128), 128, 0, s>>>(
            static_cast<const T*>(p->u), p->u_stride_b, p->u_stride_l, a, static_cast<T*>(p->fir_state),
            static_cast<T*>(p->inner_state));
        return check_launch("fused_fir state");
    }
    return VTX_OK;
}

int fused_mr_tc_fwd(const vtx_fused_fir_params* p, cudaStream_t stream);   // fused_mr.cu (tcgen05 path)

}  // namespace vtx

extern "C" int vtx_fused_fir_fwd(const vtx_fused_fir_params* p, void* stream) {
    using namespace vtx;
    VTX_REQUIRE(p && p->u && p->w3 && p->h && p->y, VTX_ERR_BAD_ARG, "fused_fir: null pointer");
    VTX_REQUIRE(p->B > 0 && p->L > 0 && p->D > 0 && p->G > 0 && p->K > 0, VTX_ERR_BAD_ARG,
                "fused_fir: sizes must be positive");
    VTX_REQUIRE(p->D % p->G == 0, VTX_ERR_BAD_ARG, "fused_fir: D not a multiple of G");
    VTX_REQUIRE(p->K3 == FF_K3, VTX_ERR_UNSUPPORTED, "fused_fir: featurizer length %lld (only 3 is fused)",
                (long long)p->K3);
    VTX_REQUIRE(valid_dtype(p->io_dtype), VTX_ERR_BAD_ARG, "fused_fir: bad io dtype");
    VTX_REQUIRE(p->u_hist_rows == 0 || p->u_hist_rows >= p->K + 1, VTX_ERR_BAD_ARG,
                "fused_fir: u_hist_rows must be 0 or at least K + 1 = %lld", (long long)(p->K + 1));
    VTX_REQUIRE(p->bias_mode == VTX_BIAS_NONE || p->bias, VTX_ERR_BAD_ARG, "fused_fir: bias mode set without a bias");
    VTX_REQUIRE(p->B <= 65535, VTX_ERR_UNSUPPORTED, "fused_fir: batch too large");
    // Kernel choice: the tensor-core kernel (bf16, groups of 16 channels, up to 128 taps) is the faster one for every
    // filter length it takes; the CUDA-core kernel below covers the other dtypes and group sizes up to 16 taps.
    const bool tc_shape = p->io_dtype == VTX_BF16 && p->D == p->G * 16 && p->K <= 128 && !p->b3 && p->bias_mode != VTX_BIAS_ADD &&
                          (reinterpret_cast<uintptr_t>(p->y) % 32) == 0 && (p->y_stride_l % 16) == 0 && (p->y_stride_b % 16) == 0 &&
                          (p->layout != VTX_QKV_COLUMN_SPLIT || (p->num_heads > 0 && p->D % p->num_heads == 0 && (p->D / p->num_heads) % 16 == 0));
    if (tc_shape || p->K > 16) return fused_mr_tc_fwd(p, (cudaStream_t)stream);

    const int64_t es = dtype_size(p->io_dtype);
    FusedArgs a{};
    a.w3 = p->w3; a.w3_dtype = p->w3_dtype; a.b3 = p->b3; a.b3_dtype = p->b3_dtype;
    a.h = p->h; a.h_dtype = p->h_dtype; a.bias = p->bias; a.bias_dtype = p->bias_dtype;
    a.y = p->y; a.y_stride_b = p->y_stride_b; a.y_stride_l = p->y_stride_l;
    a.B = p->B; a.L = p->L; a.D = p->D; a.G = p->G; a.K = p->K;
    a.layout = (int)p->layout; a.flip = p->flip_x1x2 != 0; a.taps = (int)p->taps; a.bias_mode = (int)p->bias_mode;
    a.hd = p->D;
    a.hist = p->u_hist_rows;
    if (p->layout == VTX_QKV_COLUMN_SPLIT) {
        VTX_REQUIRE(p->num_heads > 0 && p->D % p->num_heads == 0, VTX_ERR_BAD_ARG,
                    "fused_fir: column split needs num_heads dividing D");
        a.hd = p->D / p->num_heads;
        VTX_REQUIRE(a.hd % FF_CH == 0, VTX_ERR_UNSUPPORTED, "fused_fir: column split needs head size %% %d == 0", FF_CH);
    }
    VTX_REQUIRE(p->layout == VTX_QKV_INTERLEAVED || (p->D * es) % 16 == 0, VTX_ERR_ALIGNMENT,
                "fused_fir: D*itemsize must be a multiple of 16 bytes for this q/k/v layout");
    VTX_REQUIRE((reinterpret_cast<uintptr_t>(p->y) % (2 * es)) == 0 && (p->y_stride_l % 2) == 0 &&
                    (p->y_stride_b % 2) == 0,
                VTX_ERR_ALIGNMENT, "fused_fir: y rows must be aligned to two elements");
    a.nslab = ceil_div<int64_t>(p->D, FF_CH);
    const int rows = FF_STAGE_BYTES / (3 * FF_CH * (int)es);
    // segment length: enough warp tasks for several waves of 12 resident warps per SM (short tail),
    // at least 4 stages of rows each, at most 512 rows
    int64_t seg = 512;
    while (seg > 4 * rows && p->B * a.nslab * ceil_div<int64_t>(p->L, seg) < (int64_t)kNumSMs * 48) seg /= 2;
    a.seg_len = seg;
    a.nseg = ceil_div<int64_t>(p->L, seg);
    VTX_REQUIRE(a.B * a.nslab * a.nseg < (int64_t)1 << 31, VTX_ERR_UNSUPPORTED, "fused_fir: too many tasks");

    const bool inter = p->layout == VTX_QKV_INTERLEAVED;
    CUtensorMap tmap;
    // the tensor map starts at the first history row
    const char* u_first = static_cast<const char*>(p->u) - p->u_hist_rows * p->u_stride_l * es;
    if (int rc = make_tmap_3d(&tmap, u_first, p->io_dtype, 3 * p->D, p->L + p->u_hist_rows, p->B, p->u_stride_l, p->u_stride_b,
                              inter ? 3 * FF_CH : FF_CH, rows, 0, "fused_fir"))
        return rc;
    cudaStream_t s = (cudaStream_t)stream;
    VTX_DISPATCH_IO(p->io_dtype, T, {
        return inter ? launch_fused<T, true>(p, a, tmap, s) : launch_fused<T, false>(p, a, tmap, s);
    });
    return VTX_OK;
}
