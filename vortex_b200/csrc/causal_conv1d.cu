// Short depthwise causal convolution (2..4 taps) of the reference's conv extension, forward and decode update:
// causal_conv1d_fwd (vortex/ops/conv/csrc/causal_conv1d.cpp:130-236, causal_conv1d_fwd.cu:44-135,208-346) and
// causal_conv1d_update (causal_conv1d.cpp:382-470, causal_conv1d_update.cu:24-100).
//   out[b,d,t] = act(bias[d] + sum_w weight[d,w] * xx[b,d,t-(W-1)+w]),   xx = [initial_states | x]
// Both tensor layouts of the reference go through one kernel each, by strides: with time contiguous a thread owns TS
// consecutive samples of one channel (lanes along time), with channels contiguous a lane owns a channel and walks TS
// samples (lanes along channels); either way a warp's accesses are contiguous.  fp32 arithmetic, one final rounding.
#include "common.cuh"
#include <initializer_list>

namespace vtx {
namespace cc1d {

constexpr int TS = 8;          // samples per thread
constexpr int MAXW = 4;

template <typename T, bool CHANNEL_LAST>
__global__ void __launch_bounds__(256) fwd_kernel(vtx_causal_conv1d_params p) {
    const int64_t nblk = ceil_div<int64_t>(p.L, (int64_t)TS);
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.B * p.D * nblk) return;
    int64_t b, d, tb;
    if (CHANNEL_LAST) { d = i % p.D; tb = (i / p.D) % nblk; b = i / (p.D * nblk); }
    else { tb = i % nblk; d = (i / nblk) % p.D; b = i / (nblk * p.D); }
    const int W = (int)p.W;
    const int64_t t0 = tb * TS;
    const T* x = static_cast<const T*>(p.x) + b * p.x_stride_b + d * p.x_stride_d;
    const T* ini = p.initial_states ? static_cast<const T*>(p.initial_states) + b * p.is_stride_b + d * p.is_stride_d : nullptr;
    const int32_t* sid = p.seq_idx ? p.seq_idx + b * p.L : nullptr;
    float w[MAXW];
#pragma unroll
    for (int j = 0; j < MAXW; ++j) w[j] = j < W ? ld_param(p.weight, p.weight_dtype, d * W + j) : 0.f;
    const float bias = p.bias ? ld_param(p.bias, p.bias_dtype, d) : 0.f;
    // window xx[t0-(W-1) .. t0+TS): negative times come from the initial states (or are zero)
    float xv[TS + MAXW - 1];
    int sv[TS + MAXW - 1];
#pragma unroll
    for (int k = 0; k < TS + MAXW - 1; ++k) {
        const int64_t t = t0 - (MAXW - 1) + k;
        float v = 0.f;
        int s = -1;
        if (t >= 0 && t < p.L) {
            v = to_f32<T>(x[t * p.x_stride_l]);
            if (sid) s = sid[t];
        } else if (t < 0 && t >= -(W - 1) && ini) {
            v = to_f32<T>(ini[(W - 1 + t) * p.is_stride_l]);
        }
        xv[k] = v; sv[k] = s;
    }
    T* out = static_cast<T*>(p.out) + b * p.out_stride_b + d * p.out_stride_d;
#pragma unroll
    for (int k = 0; k < TS; ++k) {
        const int64_t t = t0 + k;
        if (t >= p.L) break;
        float acc = bias;
#pragma unroll
        for (int j = 0; j < MAXW; ++j) {
            // tap j of W reaches back W-1-j samples: window slot k + (MAXW-1) - (W-1-j)
            if (j < W) {
                const int slot = k + (MAXW - 1) - (W - 1 - j);
                const bool on = !sid || sv[slot] == sv[k + MAXW - 1];
                acc = on ? fmaf(w[j], xv[slot], acc) : acc;
            }
        }
        if (p.silu) acc = acc / (1.f + expf(-acc));
        out[t * p.out_stride_l] = from_f32<T>(acc);
    }
    // final states: the last W-1 samples of [initial_states | x]; written by the thread that owns the last block
    if (p.final_states && tb == nblk - 1) {
        T* fs = static_cast<T*>(p.final_states) + b * p.fs_stride_b + d * p.fs_stride_d;
        for (int j = 0; j < W - 1; ++j) {
            const int64_t t = p.L - (W - 1) + j;
            float v = 0.f;
            if (t >= 0) v = to_f32<T>(x[t * p.x_stride_l]);
            else if (ini && t >= -(W - 1)) v = to_f32<T>(ini[(W - 1 + t) * p.is_stride_l]);
            fs[j * p.fs_stride_l] = from_f32<T>(v);
        }
    }
}


// ---- vectorised kernels: 16-byte accesses; taken when sizes, strides and addresses allow (else the kernel above) ----
template <typename T> struct Vec16 {
    static constexpr int N = 16 / (int)sizeof(T);
    T e[N];
};
template <typename T> __device__ __forceinline__ void ld16(const T* p, float (&f)[16 / sizeof(T)]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    Vec16<T> v;
    *reinterpret_cast<uint4*>(&v) = raw;
#pragma unroll
    for (int i = 0; i < Vec16<T>::N; ++i) f[i] = to_f32<T>(v.e[i]);
}
template <typename T> __device__ __forceinline__ void st16(T* p, const float (&f)[16 / sizeof(T)]) {
    Vec16<T> v;
#pragma unroll
    for (int i = 0; i < Vec16<T>::N; ++i) v.e[i] = from_f32<T>(f[i]);
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&v);
}
__device__ __forceinline__ float act(float a, bool silu) { return silu ? __fdividef(a, 1.f + __expf(-a)) : a; }

// Channel-last: a thread owns V = 16 bytes of channels and walks CLT samples with the W-1 rows before them in
// registers; a warp reads and writes 512 contiguous bytes per row.  Rows stay in their I/O dtype while in flight (U
// rows of 16 bytes per thread) and are widened at use, which keeps enough loads in flight for the memory system.
constexpr int CLT = 32;
template <typename T, int W, bool SEQ>
__global__ void __launch_bounds__(256, 2) fwd_cl_kernel(vtx_causal_conv1d_params p) {
    constexpr int V = Vec16<T>::N;
    const int64_t nv = p.D / V, nblk = ceil_div<int64_t>(p.L, (int64_t)CLT);
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.B * nblk * nv) return;
    const int64_t d = (i % nv) * V, tb = (i / nv) % nblk, b = i / (nv * nblk);
    const int64_t t0 = tb * CLT;
    const T* x = static_cast<const T*>(p.x) + b * p.x_stride_b + d;
    T* out = static_cast<T*>(p.out) + b * p.out_stride_b + d;
    const int32_t* sid = SEQ ? p.seq_idx + b * p.L : nullptr;
    float w[W][V], bias[V];
#pragma unroll
    for (int c = 0; c < V; ++c) {
#pragma unroll
        for (int j = 0; j < W; ++j) w[j][c] = ld_param(p.weight, p.weight_dtype, (d + c) * W + j);
        bias[c] = p.bias ? ld_param(p.bias, p.bias_dtype, d + c) : 0.f;
    }
    // rows t0-(W-1) .. t0-1, widened once
    float h[W - 1][V];
    int hs[W - 1];
#pragma unroll
    for (int j = 0; j < W - 1; ++j) {
        const int64_t t = t0 - (W - 1) + j;
        hs[j] = -1;
        if (t >= 0) {
            ld16<T>(x + t * p.x_stride_l, h[j]);
            if (SEQ) hs[j] = sid[t];
        } else {
#pragma unroll
            for (int c = 0; c < V; ++c)
                h[j][c] = p.initial_states ? to_f32<T>(static_cast<const T*>(p.initial_states)[b * p.is_stride_b + (d + c) * p.is_stride_d + (W - 1 + t) * p.is_stride_l]) : 0.f;
        }
    }
    const bool silu = p.silu != 0;
    const int nt = (int)((p.L - t0) < CLT ? (p.L - t0) : CLT);
    constexpr int U = 8;                       // rows in flight
    for (int k0 = 0; k0 < nt; k0 += U) {
        Vec16<T> xr[U];
        int xs[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            xs[u] = 0;
            if (k0 + u < nt) {
                *reinterpret_cast<uint4*>(&xr[u]) = *reinterpret_cast<const uint4*>(x + (t0 + k0 + u) * p.x_stride_l);
                if (SEQ) xs[u] = sid[t0 + k0 + u];
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (k0 + u < nt) {
                float cur[V], y[V];
#pragma unroll
                for (int c = 0; c < V; ++c) {
                    cur[c] = to_f32<T>(xr[u].e[c]);
                    float acc = fmaf(w[W - 1][c], cur[c], bias[c]);
#pragma unroll
                    for (int j = 0; j < W - 1; ++j) {
                        const bool on = !SEQ || hs[j] == xs[u];
                        acc = on ? fmaf(w[j][c], h[j][c], acc) : acc;
                    }
                    y[c] = act(acc, silu);
                }
                st16<T>(out + (t0 + k0 + u) * p.out_stride_l, y);
#pragma unroll
                for (int j = 0; j + 1 < W - 1; ++j) {
                    hs[j] = hs[j + 1];
#pragma unroll
                    for (int c = 0; c < V; ++c) h[j][c] = h[j + 1][c];
                }
                hs[W - 2] = xs[u];
#pragma unroll
                for (int c = 0; c < V; ++c) h[W - 2][c] = cur[c];
            }
        }
    }
    // after the walk h holds the last W-1 samples of [initial_states | x] when this is the last block
    if (p.final_states && tb == nblk - 1) {
#pragma unroll
        for (int j = 0; j < W - 1; ++j)
#pragma unroll
            for (int c = 0; c < V; ++c)
                static_cast<T*>(p.final_states)[b * p.fs_stride_b + (d + c) * p.fs_stride_d + j * p.fs_stride_l] = from_f32<T>(h[j][c]);
    }
}

// Time-last: a warp owns TLV x 32 consecutive 16-byte vectors of one channel's row; a thread takes the vectors
// lane, lane + 32, ... (coalesced 512-byte accesses, TLV loads in flight).  The W-1 samples before a vector come from
// the previous lane by shuffle (lane 31 hands over its previous vector); only the first lane of a warp fetches them
// from memory, and the first vector of a row takes the initial states.  No seq_idx on this path.
constexpr int TLV = 4;
template <typename T, int W>
__global__ void __launch_bounds__(256) fwd_tl_kernel(vtx_causal_conv1d_params p) {
    constexpr int V = Vec16<T>::N;
    const int64_t nv = p.L / V, nch = ceil_div<int64_t>(nv, (int64_t)(32 * TLV));
    const int64_t wid = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / 32;
    if (wid >= p.B * p.D * nch) return;                  // whole warps leave together
    const int lane = threadIdx.x & 31;
    const int64_t ch = wid % nch, d = (wid / nch) % p.D, b = wid / (nch * p.D);
    const T* x = static_cast<const T*>(p.x) + b * p.x_stride_b + d * p.x_stride_d;
    T* out = static_cast<T*>(p.out) + b * p.out_stride_b + d * p.out_stride_d;
    const int64_t v0 = ch * (32 * TLV) + lane;           // this thread's vectors: v0 + 32 k
    Vec16<T> raw[TLV];
#pragma unroll
    for (int k = 0; k < TLV; ++k)
        if (v0 + 32 * k < nv) *reinterpret_cast<uint4*>(&raw[k]) = *reinterpret_cast<const uint4*>(x + (v0 + 32 * k) * V);
        else *reinterpret_cast<uint4*>(&raw[k]) = make_uint4(0, 0, 0, 0);
    float w[W];
#pragma unroll
    for (int j = 0; j < W; ++j) w[j] = ld_param(p.weight, p.weight_dtype, d * W + j);
    const float bias = p.bias ? ld_param(p.bias, p.bias_dtype, d) : 0.f;
    const bool silu = p.silu != 0;
    // samples before the warp's first vector
    float first[W - 1];
#pragma unroll
    for (int j = 0; j < W - 1; ++j) {
        first[j] = 0.f;
        if (lane == 0) {
            if (ch > 0) first[j] = to_f32<T>(x[v0 * V - (W - 1) + j]);
            else if (p.initial_states)
                first[j] = to_f32<T>(static_cast<const T*>(p.initial_states)[b * p.is_stride_b + d * p.is_stride_d + j * p.is_stride_l]);
        }
    }
#pragma unroll
    for (int k = 0; k < TLV; ++k) {
        float xv[V + W - 1];
#pragma unroll
        for (int c = 0; c < V; ++c) xv[W - 1 + c] = to_f32<T>(raw[k].e[c]);
#pragma unroll
        for (int j = 0; j < W - 1; ++j) {
            // what the next lane needs: the tail of this vector; lane 31 hands over the tail of its previous vector
            const float mine = to_f32<T>(raw[k].e[V - (W - 1) + j]);
            const float prev = k > 0 ? to_f32<T>(raw[k > 0 ? k - 1 : 0].e[V - (W - 1) + j]) : 0.f;
            const float got = __shfl_sync(0xffffffffu, lane == 31 ? prev : mine, (lane + 31) & 31);
            xv[j] = (lane == 0 && k == 0) ? first[j] : got;
        }
        if (v0 + 32 * k < nv) {
            float y[V];
#pragma unroll
            for (int c = 0; c < V; ++c) {
                float acc = bias;
#pragma unroll
                for (int j = 0; j < W; ++j) acc = fmaf(w[j], xv[c + j], acc);
                y[c] = act(acc, silu);
            }
            st16<T>(out + (v0 + 32 * k) * V, y);
            if (p.final_states && v0 + 32 * k == nv - 1) {
#pragma unroll
                for (int j = 0; j < W - 1; ++j)
                    static_cast<T*>(p.final_states)[b * p.fs_stride_b + d * p.fs_stride_d + j * p.fs_stride_l] = from_f32<T>(xv[V + j]);
            }
        }
    }
}

template <typename T>
static bool vec_ok(const void* ptr, std::initializer_list<int64_t> strides) {
    constexpr int64_t V = 16 / sizeof(T);
    if (reinterpret_cast<uintptr_t>(ptr) % 16) return false;
    for (int64_t s : strides) if (s % V) return false;
    return true;
}

template <typename T, int W>
static void launch_fast(const vtx_causal_conv1d_params& p, bool cl, cudaStream_t s) {
    constexpr int64_t V = 16 / sizeof(T);
    if (cl) {
        const int64_t n = p.B * ceil_div<int64_t>(p.L, (int64_t)CLT) * (p.D / V);
        const unsigned blocks = (unsigned)ceil_div<int64_t>(n, 256);
        if (p.seq_idx) fwd_cl_kernel<T, W, true><<<blocks, 256, 0, s>>>(p);
        else fwd_cl_kernel<T, W, false><<<blocks, 256, 0, s>>>(p);
    } else {
        const int64_t warps = p.B * p.D * ceil_div<int64_t>(p.L / V, (int64_t)(32 * TLV));
        fwd_tl_kernel<T, W><<<(unsigned)ceil_div<int64_t>(warps, 8), 256, 0, s>>>(p);
    }
}

// Decode update: thread = (batch, channel); the new samples are few (usually one).
template <typename T>
__global__ void __launch_bounds__(128) update_kernel(vtx_causal_conv1d_update_params p) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.B * p.D) return;
    const int64_t b = i / p.D, d = i % p.D;
    const int W = (int)p.W;
    const int64_t SL = p.state_len, Lq = p.L;
    const int64_t sb = p.conv_state_indices ? (int64_t)p.conv_state_indices[b] : b;
    T* st = static_cast<T*>(p.conv_state) + sb * p.cs_stride_b + d * p.cs_stride_d;
    const T* x = static_cast<const T*>(p.x) + b * p.x_stride_b + d * p.x_stride_d;
    T* out = static_cast<T*>(p.out) + b * p.out_stride_b + d * p.out_stride_d;
    float w[MAXW];
#pragma unroll
    for (int j = 0; j < MAXW; ++j) w[j] = j < W ? ld_param(p.weight, p.weight_dtype, d * W + j) : 0.f;
    const float bias = p.bias ? ld_param(p.bias, p.bias_dtype, d) : 0.f;
    // the W-1 samples before the first new one
    float h[MAXW - 1] = {0.f, 0.f, 0.f};
    const int64_t pos = p.cache_seqlens ? (int64_t)p.cache_seqlens[b] : 0;
#pragma unroll
    for (int j = 0; j < MAXW - 1; ++j) {
        if (j < W - 1) {
            int64_t idx = p.cache_seqlens ? (((pos - (W - 1) + j) % SL) + SL) % SL : SL - (W - 1) + j;
            h[(MAXW - 1) - (W - 1) + j] = to_f32<T>(st[idx * p.cs_stride_l]);
        }
    }
    if (!p.cache_seqlens && Lq < SL) {
        // shift register: keep the last SL - Lq old samples (read before written: the walk goes forward)
        for (int64_t k = 0; k < SL - Lq; ++k) st[k * p.cs_stride_l] = st[(k + Lq) * p.cs_stride_l];
    }
    for (int64_t t = 0; t < Lq; ++t) {
        const T xt = x[t * p.x_stride_l];
        const float xf = to_f32<T>(xt);
        float acc = bias;
        // h holds the MAXW-1 samples before xf; tap j of W reaches back W-1-j
#pragma unroll
        for (int j = 0; j < MAXW; ++j) {
            if (j < W) {
                const int back = W - 1 - j;
                const float v = back == 0 ? xf : h[(MAXW - 1) - back];
                acc = fmaf(w[j], v, acc);
            }
        }
        h[0] = h[1]; h[1] = h[2]; h[2] = xf;
        if (p.silu) acc = acc / (1.f + expf(-acc));
        out[t * p.out_stride_l] = from_f32<T>(acc);
        if (p.cache_seqlens) st[((pos + t) % SL) * p.cs_stride_l] = xt;
        else if (t >= Lq - SL) st[(SL - Lq + t) * p.cs_stride_l] = xt;
    }
}

// States of packed sequences (causal_conv1d_varlen.py:8-39): states[b, c, state_len - 1 - r] = x[end_b - 1 - r, c]
// for the last state_len rows of sequence b, zero where that row belongs to an earlier sequence.  Thread = (b, s, c)
// with c fastest: rows of x and of the reference's [batch, state_len, dim] memory are read and written contiguously.
template <typename T>
__global__ void __launch_bounds__(256) varlen_states_kernel(vtx_varlen_states_params p) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.batch * p.state_len * p.dim) return;
    const int64_t c = i % p.dim, s = (i / p.dim) % p.state_len, b = i / (p.dim * p.state_len);
    const int64_t end = p.cu_seqlens[b + 1], begin = p.cu_seqlens[b];
    const int64_t row = end - p.state_len + s;
    T v = from_f32<T>(0.f);
    if (row >= begin && row >= 0 && row < p.total) v = static_cast<const T*>(p.x)[row * p.x_stride_t + c * p.x_stride_c];
    static_cast<T*>(p.states)[b * p.st_stride_b + c * p.st_stride_c + s * p.st_stride_l] = v;
}

}  // namespace cc1d
}  // namespace vtx

extern "C" int vtx_causal_conv1d_varlen_states(const vtx_varlen_states_params* p, void* stream) {
    using namespace vtx;
    using namespace vtx::cc1d;
    VTX_REQUIRE(p && p->x && p->cu_seqlens && p->states, VTX_ERR_BAD_ARG, "varlen_states: null pointer");
    VTX_REQUIRE(p->batch > 0 && p->dim > 0 && p->state_len > 0 && p->total >= 0, VTX_ERR_BAD_ARG,
                "varlen_states: sizes must be positive");
    const int64_t n = p->batch * p->state_len * p->dim;
    VTX_REQUIRE(ceil_div<int64_t>(n, 256) < ((int64_t)1 << 31), VTX_ERR_UNSUPPORTED, "varlen_states: problem too large");
    cudaStream_t s = (cudaStream_t)stream;
    VTX_DISPATCH_IO(p->io_dtype, T, { varlen_states_kernel<T><<<(unsigned)ceil_div<int64_t>(n, 256), 256, 0, s>>>(*p); });
    return check_launch("causal_conv1d_varlen_states");
}

extern "C" int vtx_causal_conv1d_fwd(const vtx_causal_conv1d_params* p, void* stream) {
    using namespace vtx;
    using namespace vtx::cc1d;
    VTX_REQUIRE(p && p->x && p->weight && p->out, VTX_ERR_BAD_ARG, "causal_conv1d: null pointer");
    VTX_REQUIRE(p->B > 0 && p->D > 0 && p->L > 0, VTX_ERR_BAD_ARG, "causal_conv1d: sizes must be positive");
    VTX_REQUIRE(p->W >= 2 && p->W <= MAXW, VTX_ERR_UNSUPPORTED, "causal_conv1d: only widths between 2 and 4 (got %lld)", (long long)p->W);
    VTX_REQUIRE(valid_dtype(p->weight_dtype) && (!p->bias || valid_dtype(p->bias_dtype)), VTX_ERR_BAD_ARG,
                "causal_conv1d: bad parameter dtype");
    const bool cl = p->x_stride_d == 1 && p->x_stride_l != 1;
    VTX_REQUIRE(!p->seq_idx || cl || p->L == 1 || p->x_stride_l == 1, VTX_ERR_BAD_ARG, "causal_conv1d: bad strides");
    const int64_t n = p->B * p->D * ceil_div<int64_t>(p->L, (int64_t)TS);
    VTX_REQUIRE(ceil_div<int64_t>(n, 256) < ((int64_t)1 << 31), VTX_ERR_UNSUPPORTED, "causal_conv1d: problem too large");
    const unsigned blocks = (unsigned)ceil_div<int64_t>(n, 256);
    cudaStream_t s = (cudaStream_t)stream;
    VTX_DISPATCH_IO(p->io_dtype, T, {
        constexpr int64_t V = 16 / sizeof(T);
        const bool fast_cl = cl && p->out_stride_d == 1 && p->D % V == 0 && p->B * p->L * (p->D / V) < ((int64_t)1 << 38) &&
                             vec_ok<T>(p->x, {p->x_stride_b, p->x_stride_l}) && vec_ok<T>(p->out, {p->out_stride_b, p->out_stride_l});
        const bool fast_tl = !cl && p->x_stride_l == 1 && p->out_stride_l == 1 && !p->seq_idx && p->L % V == 0 &&
                             p->B * p->D * (p->L / V) < ((int64_t)1 << 38) &&
                             vec_ok<T>(p->x, {p->x_stride_b, p->x_stride_d}) && vec_ok<T>(p->out, {p->out_stride_b, p->out_stride_d});
        if (fast_cl || fast_tl) {
            if (p->W == 2) launch_fast<T, 2>(*p, cl, s);
            else if (p->W == 3) launch_fast<T, 3>(*p, cl, s);
            else launch_fast<T, 4>(*p, cl, s);
        } else if (cl) {
            fwd_kernel<T, true><<<blocks, 256, 0, s>>>(*p);
        } else {
            fwd_kernel<T, false><<<blocks, 256, 0, s>>>(*p);
        }
    });
    return check_launch("causal_conv1d_fwd");
}

extern "C" int vtx_causal_conv1d_update(const vtx_causal_conv1d_update_params* p, void* stream) {
    using namespace vtx;
    using namespace vtx::cc1d;
    VTX_REQUIRE(p && p->x && p->weight && p->out && p->conv_state, VTX_ERR_BAD_ARG, "causal_conv1d_update: null pointer");
    VTX_REQUIRE(p->B > 0 && p->D > 0 && p->L > 0, VTX_ERR_BAD_ARG, "causal_conv1d_update: sizes must be positive");
    VTX_REQUIRE(p->W >= 2 && p->W <= MAXW, VTX_ERR_UNSUPPORTED, "causal_conv1d_update: only widths between 2 and 4 (got %lld)", (long long)p->W);
    VTX_REQUIRE(p->state_len >= p->W - 1, VTX_ERR_BAD_ARG, "causal_conv1d_update: conv_state shorter than width - 1");
    VTX_REQUIRE(valid_dtype(p->weight_dtype) && (!p->bias || valid_dtype(p->bias_dtype)), VTX_ERR_BAD_ARG,
                "causal_conv1d_update: bad parameter dtype");
    const unsigned blocks = (unsigned)ceil_div<int64_t>(p->B * p->D, 128);
    cudaStream_t s = (cudaStream_t)stream;
    VTX_DISPATCH_IO(p->io_dtype, T, { update_kernel<T><<<blocks, 128, 0, s>>>(*p); });
    return check_launch("causal_conv1d_update");
}
