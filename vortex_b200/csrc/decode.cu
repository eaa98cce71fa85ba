// Decode-time (one token) kernels: FIR shift-register step, modal IIR step,
// and the whole per-layer sequence in one launch.  All of them are pure HBM
// streaming over the caches; a row (one batch element, one channel) is served
// by LPR cooperating lanes so that long rows (Hyena-MR: 127 cached samples)
// are read and rewritten coalesced, with a shuffle reduction over the taps.
#include "common.cuh"

namespace vtx {

// Row and channel indices fit 32 bits (checked by the host): their quotients are taken as 32-bit divisions, which cost
// a tenth of the 64-bit ones -- the one-token kernels are short enough for a few 64-bit divisions per thread to be most
// of their instructions (the 128-tap tile kernel executed 1385 instructions per tile with them, eight per tile).
__device__ __forceinline__ int div32(int64_t a, int64_t b) { return (int)((unsigned)a / (unsigned)b); }
__device__ __forceinline__ QkvMap qkv_map(const vtx_decode_layer_params& p) {
    return QkvMap{(int)p.layout, (int)p.flip_x1x2, p.D, p.num_heads > 0 ? (int64_t)div32(p.D, p.num_heads) : p.D};
}

// Sum over the LPR lanes of a row.  The mask names only the lanes of this row's group, so the
// groups of a warp may diverge from one another (e.g. when the last rows of a launch are absent).
template <int LPR>
__device__ __forceinline__ float group_sum(float x) {
    if (LPR > 1) {
        const unsigned group = (threadIdx.x % 32) / LPR;
        const unsigned mask = LPR == 32 ? 0xffffffffu : (((1u << LPR) - 1u) << (group * LPR));
#pragma unroll
        for (int o = LPR / 2; o > 0; o >>= 1) x += __shfl_xor_sync(mask, x, o);
    }
    return x;
}

// One FIR step on a row.  Returns the filter output (before bias) on every lane of the group.
//   state_in [c] (any dtype), taps w [K] of the row's group, new sample u.
//   state_out fp32 [min(c+1, K-1)].
template <int LPR>
__device__ __forceinline__ float fir_row_step(const void* state_in, int64_t sdt, int64_t row_off, int c, int K,
                                              const void* w, int64_t wdt, int64_t w_off, bool flip, float u,
                                              float* state_out, int lane) {
    const bool grow = c < K - 1;
    const int c_out = grow ? c + 1 : c;
    float acc = 0.f;
    for (int i = lane; i < c; i += LPR) {
        float s = ld_param(state_in, sdt, row_off + i);
        float tap = ld_param(w, wdt, w_off + (flip ? c - i : i));
        acc = fmaf(s, tap, acc);
        int o = grow ? i : i - 1;
        if (o >= 0) state_out[o] = s;
    }
    acc = group_sum<LPR>(acc);
    float tap_u = ld_param(w, wdt, w_off + (flip ? 0 : c));
    if (lane == 0 && c_out > 0) state_out[c_out - 1] = u;
    return fmaf(tap_u, u, acc);
}

template <typename T, int LPR>
__global__ void __launch_bounds__(256) step_fir_kernel(vtx_step_fir_params p) {
    const int lane = threadIdx.x % LPR;
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / LPR;
    if (row >= p.B * p.C) return;   // whole groups leave together (blockDim % LPR == 0)
    const int64_t ch = row - (int64_t)div32(row, p.C) * p.C;
    const int c = (int)p.c, K = (int)p.K;
    const int c_out = c < K - 1 ? c + 1 : c;
    const float u = to_f32<T>(static_cast<const T*>(p.u)[row]);
    float y = fir_row_step<LPR>(p.state_in, p.state_dtype, row * c, c, K, p.w, p.w_dtype,
                                (int64_t)div32(ch, div32(p.C, p.Gw)) * K, p.flip_filter != 0, u, p.state_out + row * c_out, lane);
    if (lane == 0) {
        if (p.bias_mode != VTX_BIAS_NONE) {
            float b = ld_param(p.bias, p.bias_dtype, ch);
            y = p.bias_mode == VTX_BIAS_GATED ? fmaf(b, u, y) : y + b;
        }
        static_cast<T*>(p.y)[row] = from_f32<T>(y);
    }
}

// sigma <- p sigma + kv for the 16 lanes of a row; returns sum_s Re(R sigma) on every lane.
__device__ __forceinline__ float iir_row_step(const vtx_modal_params& m, int64_t g, const float* st_in,
                                              float* st_out, float kv, int lane) {
    float part = 0.f;
    if (lane < m.S) {
        const int64_t gi = g * m.S + lane;
        float mag = expf(static_cast<const float*>(m.log_poles)[gi]);
        float rr = static_cast<const float*>(m.res_re)[gi];
        if (m.theta) {
            float sn, cs;
            sincosf(static_cast<const float*>(m.theta)[gi], &sn, &cs);
            float pr = mag * cs, pi = mag * sn;
            float ri = m.res_im ? static_cast<const float*>(m.res_im)[gi] : 0.f;
            float2 s = reinterpret_cast<const float2*>(st_in)[lane];
            float nr = fmaf(pr, s.x, fmaf(-pi, s.y, kv));
            float ni = fmaf(pr, s.y, pi * s.x);
            reinterpret_cast<float2*>(st_out)[lane] = make_float2(nr, ni);
            part = rr * nr - ri * ni;
        } else {
            float s = fmaf(mag, st_in[lane], kv);
            st_out[lane] = s;
            part = rr * s;
        }
    }
    return group_sum<16>(part);
}

template <typename T>
__global__ void __launch_bounds__(256) step_iir_kernel(vtx_step_iir_params p) {
    const int lane = threadIdx.x % 16;
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / 16;
    if (row >= p.B * p.D) return;
    const int64_t d = row - (int64_t)div32(row, p.D) * p.D;
    const int64_t ss = p.modal.S * (p.modal.theta ? 2 : 1);
    float q = to_f32<T>(static_cast<const T*>(p.q)[row]);
    float kv = round_io<T>(to_f32<T>(static_cast<const T*>(p.k)[row]) * to_f32<T>(static_cast<const T*>(p.v)[row]));
    float res = iir_row_step(p.modal, div32(d, div32(p.D, p.modal.G)), p.state_in + row * ss, p.state_out + row * ss, kv, lane);
    if (lane == 0) {
        // D * x1v is a product of two I/O-dtype tensors in the reference (rounded there) unless D is fp32
        float skip = p.bias ? ld_param(p.bias, p.bias_dtype, d) * kv : 0.f;
        if (p.bias && p.bias_dtype != VTX_F32) skip = round_io<T>(skip);
        p.y[row] = q * (res + skip);
    }
}

// Whole layer.  LPR lanes per (batch, hidden channel); MODE 0 = FIR inner filter, 1 = modal IIR.
template <typename T, int LPR, int MODE>
__global__ void __launch_bounds__(256) decode_layer_kernel(vtx_decode_layer_params p) {
    const int lane = threadIdx.x % LPR;
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / LPR;
    if (row >= p.B * p.D) return;
    const int64_t b = div32(row, p.D), d = row - b * p.D;
    const QkvMap map = qkv_map(p);
    int64_t ch[3];
    map.get(d, ch[0], ch[1], ch[2]);
    const int K3 = (int)p.K3, c3 = K3 - 1;
    const T* u = static_cast<const T*>(p.u) + b * 3 * p.D;
    float z[3];
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        // featurizer step (engine.step_fir, not flipped, full cache): taps w3[c, :], newest last
        const int64_t c = ch[i], so = (b * 3 * p.D + c) * c3;
        float x = to_f32<T>(u[c]);
        float acc = ld_param(p.w3, p.w3_dtype, c * K3 + c3) * x;
        for (int j = 0; j < c3; ++j) {
            float s = ld_param(p.fir_state_in, p.fir_state_dtype, so + j);
            acc = fmaf(s, ld_param(p.w3, p.w3_dtype, c * K3 + j), acc);
            if (lane == 0 && j > 0) p.fir_state_out[so + j - 1] = s;
        }
        if (lane == 0 && c3 > 0) p.fir_state_out[so + c3 - 1] = x;
        if (p.b3) acc += ld_param(p.b3, p.b3_dtype, c);
        z[i] = round_io<T>(acc);
    }
    const float q = z[0];
    const float kv = round_io<T>(z[1] * z[2]);
    const float bias = p.bias ? ld_param(p.bias, p.bias_dtype, d) : 0.f;
    float y;
    if (MODE == 0) {
        const int K = (int)p.K, c = K - 1;
        float f = fir_row_step<LPR>(p.inner_state_in, p.inner_state_dtype, row * c, c, K, p.h, p.h_dtype,
                                    (int64_t)div32(d, div32(p.D, p.G)) * K, p.flip_filter != 0, kv, p.inner_state_out + row * c, lane);
        if (p.bias_mode == VTX_BIAS_GATED) f = fmaf(bias, kv, f);
        else if (p.bias_mode == VTX_BIAS_ADD) f += bias;
        y = round_io<T>(f) * q;
    } else {
        const int64_t ss = p.modal.S * (p.modal.theta ? 2 : 1);
        float res = iir_row_step(p.modal, div32(d, div32(p.D, p.modal.G)), p.iir_state_in + row * ss,
                                 p.iir_state_out + row * ss, kv, lane);
        float skip = bias * kv;
        if (p.bias && p.bias_dtype != VTX_F32) skip = round_io<T>(skip);
        y = q * (res + skip);
    }
    if (lane == 0) static_cast<T*>(p.y)[row] = from_f32<T>(y);
}

// ---- tiled layer kernels (fp32 caches, i.e. every decode step but the first after a prefill) -------------------
// A tile of RW consecutive hidden channels of one batch element is owned by one warp (long FIR rows) or half-warp
// (modal rows).  Lane r < RW takes the featurizer step of row r once (instead of every lane of a row repeating it);
// then the lanes stream the RW cache rows together, with all their loads issued before the first use: a decode step
// is pure cache traffic, so what counts is bytes in flight per SM.

// featurizer step of hidden channel d of batch element b: new q and k*v, featurizer cache shifted (K3 == 3)
template <typename T>
__device__ __forceinline__ void featurizer_step3(const vtx_decode_layer_params& p, int64_t b, int64_t d, float& q, float& kv) {
    const QkvMap map = qkv_map(p);
    int64_t ch[3];
    map.get(d, ch[0], ch[1], ch[2]);
    const T* u = static_cast<const T*>(p.u) + b * 3 * p.D;
    const float* fin = static_cast<const float*>(p.fir_state_in);
    float z[3];
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        const int64_t c = ch[i], so = (b * 3 * p.D + c) * 2;
        const float2 st = *reinterpret_cast<const float2*>(fin + so);
        const float x = to_f32<T>(u[c]);
        float acc = ld_param(p.w3, p.w3_dtype, c * 3 + 2) * x;
        acc = fmaf(st.x, ld_param(p.w3, p.w3_dtype, c * 3), acc);
        acc = fmaf(st.y, ld_param(p.w3, p.w3_dtype, c * 3 + 1), acc);
        *reinterpret_cast<float2*>(p.fir_state_out + so) = make_float2(st.y, x);
        if (p.b3) acc += ld_param(p.b3, p.b3_dtype, c);
        z[i] = round_io<T>(acc);
    }
    q = z[0];
    kv = round_io<T>(z[1] * z[2]);
}

// FIR layer, full fp32 inner cache of c = K-1 <= 128 samples per row, RW rows per warp.
template <typename T, int RW>
__global__ void __launch_bounds__(256) decode_fir_tile_kernel(vtx_decode_layer_params p) {
    const int lane = threadIdx.x % 32;
    const int64_t tile = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / 32;
    const int64_t row0 = tile * RW;
    if (row0 >= p.B * p.D) return;
    const int64_t b = div32(row0, p.D), d0 = row0 - b * p.D;
    float q_own = 0.f, kv_own = 0.f;
    if (lane < RW) featurizer_step3<T>(p, b, d0 + lane, q_own, kv_own);
    const int K = (int)p.K, c = K - 1;
    const bool flip = p.flip_filter != 0;
    const int cpg = div32(p.D, p.G);
    int g_row = div32(d0, cpg), g_rem = (int)d0 - g_row * cpg;      // group of row r, and the row's place in it
    const float* sin_ = static_cast<const float*>(p.inner_state_in) + row0 * c;
    float* sout = p.inner_state_out + row0 * c;
    // all cache loads of the tile first
    float s[RW][4];
#pragma unroll
    for (int r = 0; r < RW; ++r)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = lane + 32 * j;
            s[r][j] = i < c ? sin_[r * c + i] : 0.f;
        }
    // Per row: the lane's partial dot product over its (up to) four samples, and the shifted samples on their way out.
    float tap[4], tap_u[RW], part[RW], tap_u_cur = 0.f;
    int64_t g_have = -1;
#pragma unroll
    for (int r = 0; r < RW; ++r) {
        const int64_t g = g_row;
        if (++g_rem == cpg) { g_rem = 0; ++g_row; }
        if (g != g_have) {          // taps of the row's group (usually the same for the whole tile)
            g_have = g;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int i = lane + 32 * j;
                tap[j] = i < c ? ld_param(p.h, p.h_dtype, g * K + (flip ? c - i : i)) : 0.f;
            }
            tap_u_cur = ld_param(p.h, p.h_dtype, g * K + (flip ? 0 : c));
        }
        tap_u[r] = tap_u_cur;
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = lane + 32 * j;
            acc = fmaf(s[r][j], tap[j], acc);
            if (i >= 1 && i < c) sout[r * c + i - 1] = s[r][j];
        }
        part[r] = acc;
    }
    // Sum every row's partials over the 32 lanes with a folding exchange: each step halves the number of rows a lane
    // still carries (RW / 2 + RW / 4 + ... shuffles) instead of a five-step butterfly per row; lane l ends up with the
    // total of row l % RW (for RW == 8: after three folds over lane bits 4, 3, 2, then two plain steps over bits 1, 0).
    static_assert(RW == 8, "the fold below is written for eight rows per warp");
    {
        const bool hi4 = lane & 16, hi3 = lane & 8, hi2 = lane & 4;
        float q4[4], q2[2], q1;
#pragma unroll
        for (int r = 0; r < 4; ++r) {       // fold lane bit 4: lower half keeps rows 0..3, upper half rows 4..7
            const float give = hi4 ? part[r] : part[r + 4], keep = hi4 ? part[r + 4] : part[r];
            q4[r] = keep + __shfl_xor_sync(0xffffffffu, give, 16);
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {       // fold lane bit 3
            const float give = hi3 ? q4[r] : q4[r + 2], keep = hi3 ? q4[r + 2] : q4[r];
            q2[r] = keep + __shfl_xor_sync(0xffffffffu, give, 8);
        }
        {                                   // fold lane bit 2
            const float give = hi2 ? q2[0] : q2[1], keep = hi2 ? q2[1] : q2[0];
            q1 = keep + __shfl_xor_sync(0xffffffffu, give, 4);
        }
        q1 += __shfl_xor_sync(0xffffffffu, q1, 2);
        q1 += __shfl_xor_sync(0xffffffffu, q1, 1);
        // row held by this lane: bit 4 -> +4, bit 3 -> +2, bit 2 -> +1
        const int r = (hi4 ? 4 : 0) + (hi3 ? 2 : 0) + (hi2 ? 1 : 0);
        // the row's new sample and gate sit on lane r (featurizer step above)
        const float kv = __shfl_sync(0xffffffffu, kv_own, r), q = __shfl_sync(0xffffffffu, q_own, r);
        float tu = tap_u[0];
#pragma unroll
        for (int x = 1; x < RW; ++x)
            if (r == x) tu = tap_u[x];
        if ((lane & 3) == 0) {              // one lane per row finishes it
            const int64_t d = d0 + r;
            sout[r * c + c - 1] = kv;
            float f = fmaf(tu, kv, q1);
            if (p.bias_mode != VTX_BIAS_NONE) {
                const float bias = ld_param(p.bias, p.bias_dtype, d);
                f = p.bias_mode == VTX_BIAS_GATED ? fmaf(bias, kv, f) : f + bias;
            }
            static_cast<T*>(p.y)[row0 + r] = from_f32<T>(round_io<T>(f) * q);
        }
    }
}

// The 128-tap layer (Evo 2's medium filter: 127 cached samples per row) with everything the general tile kernel works
// out at run time fixed at compile time: the row pitch (load and store offsets become immediates), which lanes have a
// fourth sample, one filter for the whole tile (groups are whole tiles).  The featurizer step of the tile's 24 packed
// channels is done by 24 lanes, one channel each (the general kernel lets 8 lanes do three channels in turn).
// An instruction count a quarter of the general kernel's 1385 per tile, which had the kernel bound by issue.
template <typename T>
__global__ void __launch_bounds__(256) decode_fir127_kernel(vtx_decode_layer_params p) {
    constexpr int RW = 8, C = 127, K = 128;
    const int lane = threadIdx.x % 32;
    const int64_t tile = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / 32;
    const int64_t row0 = tile * RW;
    if (row0 >= p.B * p.D) return;
    const int64_t b = div32(row0, p.D), d0 = row0 - b * p.D;
    const float* sin_ = static_cast<const float*>(p.inner_state_in) + row0 * C + lane;
    float* sout = p.inner_state_out + row0 * C + lane;
    // all cache loads of the tile first
    float s[RW][4];
#pragma unroll
    for (int r = 0; r < RW; ++r) {
#pragma unroll
        for (int j = 0; j < 3; ++j) s[r][j] = sin_[r * C + 32 * j];
        s[r][3] = lane < 31 ? sin_[r * C + 96] : 0.f;
    }
    // featurizer step: lane < 24 takes packed channel (lane % 3) of row (lane / 3)
    float z = 0.f;
    if (lane < 3 * RW) {
        const QkvMap map = qkv_map(p);
        int64_t ch[3];
        map.get(d0 + lane / 3, ch[0], ch[1], ch[2]);
        const int part = lane % 3;
        const int64_t c = part == 0 ? ch[0] : part == 1 ? ch[1] : ch[2], so = (b * 3 * p.D + c) * 2;
        const float2 st = *reinterpret_cast<const float2*>(static_cast<const float*>(p.fir_state_in) + so);
        const float x = to_f32<T>(static_cast<const T*>(p.u)[b * 3 * p.D + c]);
        float acc = ld_param(p.w3, p.w3_dtype, c * 3 + 2) * x;
        acc = fmaf(st.x, ld_param(p.w3, p.w3_dtype, c * 3), acc);
        acc = fmaf(st.y, ld_param(p.w3, p.w3_dtype, c * 3 + 1), acc);
        *reinterpret_cast<float2*>(p.fir_state_out + so) = make_float2(st.y, x);
        if (p.b3) acc += ld_param(p.b3, p.b3_dtype, c);
        z = round_io<T>(acc);
    }
    // the tile's filter: sample i of a row meets tap i (or c - i when the taps are stored flipped)
    const bool flip = p.flip_filter != 0;
    const int64_t hb = (int64_t)div32(d0, div32(p.D, p.G)) * K;
    float tap[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = lane + 32 * j;
        tap[j] = i < C ? ld_param(p.h, p.h_dtype, hb + (flip ? C - i : i)) : 0.f;
    }
    const float tu = ld_param(p.h, p.h_dtype, hb + (flip ? 0 : C));
    float part[RW];
#pragma unroll
    for (int r = 0; r < RW; ++r) {
        part[r] = fmaf(s[r][3], tap[3], fmaf(s[r][2], tap[2], fmaf(s[r][1], tap[1], s[r][0] * tap[0])));
        if (lane >= 1) sout[r * C - 1] = s[r][0];
        sout[r * C + 31] = s[r][1];
        sout[r * C + 63] = s[r][2];
        if (lane < 31) sout[r * C + 95] = s[r][3];
    }
    // fold the eight rows' partial sums over the 32 lanes (as in the general kernel): lane l ends with the total of
    // row (bit 4 -> +4, bit 3 -> +2, bit 2 -> +1)
    const bool hi4 = lane & 16, hi3 = lane & 8, hi2 = lane & 4;
    float q4[4], q2[2], q1;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const float give = hi4 ? part[r] : part[r + 4], keep = hi4 ? part[r + 4] : part[r];
        q4[r] = keep + __shfl_xor_sync(0xffffffffu, give, 16);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const float give = hi3 ? q4[r] : q4[r + 2], keep = hi3 ? q4[r + 2] : q4[r];
        q2[r] = keep + __shfl_xor_sync(0xffffffffu, give, 8);
    }
    {
        const float give = hi2 ? q2[0] : q2[1], keep = hi2 ? q2[1] : q2[0];
        q1 = keep + __shfl_xor_sync(0xffffffffu, give, 4);
    }
    q1 += __shfl_xor_sync(0xffffffffu, q1, 2);
    q1 += __shfl_xor_sync(0xffffffffu, q1, 1);
    const int r = (hi4 ? 4 : 0) + (hi3 ? 2 : 0) + (hi2 ? 1 : 0);
    // the row's featurizer outputs sit on lanes 3 r (q), 3 r + 1 (k), 3 r + 2 (v)
    const float q = __shfl_sync(0xffffffffu, z, 3 * r), kk = __shfl_sync(0xffffffffu, z, 3 * r + 1),
                v = __shfl_sync(0xffffffffu, z, 3 * r + 2);
    if ((lane & 3) == 0) {
        const float kv = round_io<T>(kk * v);
        (p.inner_state_out + row0 * C)[r * C + C - 1] = kv;
        float f = fmaf(tu, kv, q1);
        if (p.bias_mode != VTX_BIAS_NONE) {
            const float bias = ld_param(p.bias, p.bias_dtype, d0 + r);
            f = p.bias_mode == VTX_BIAS_GATED ? fmaf(bias, kv, f) : f + bias;
        }
        static_cast<T*>(p.y)[row0 + r] = from_f32<T>(round_io<T>(f) * q);
    }
}

// Short FIR layer (K == 7: six cached samples per row), four consecutive rows per thread: the thread's 24 cache
// values are contiguous and 16-byte aligned, so they move as six 16-byte loads and six 16-byte stores.
template <typename T>
__global__ void __launch_bounds__(256) decode_fir7_kernel(vtx_decode_layer_params p) {
    constexpr int K = 7, c = 6, RT = 4;
    const int64_t row0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * RT;
    if (row0 >= p.B * p.D) return;
    const int64_t b = div32(row0, p.D), d0 = row0 - b * p.D;
    const float4* sin4 = reinterpret_cast<const float4*>(static_cast<const float*>(p.inner_state_in) + row0 * c);
    float4 v[6];
#pragma unroll
    for (int j = 0; j < 6; ++j) v[j] = sin4[j];
    float s[RT * c];
#pragma unroll
    for (int j = 0; j < 6; ++j) { s[4 * j] = v[j].x; s[4 * j + 1] = v[j].y; s[4 * j + 2] = v[j].z; s[4 * j + 3] = v[j].w; }
    const bool flip = p.flip_filter != 0;
    const int cpg = div32(p.D, p.G);
    int g_row = div32(d0, cpg), g_rem = (int)d0 - g_row * cpg;
    float o[RT * c];
#pragma unroll
    for (int r = 0; r < RT; ++r) {
        const int64_t d = d0 + r, g = g_row;
        if (++g_rem == cpg) { g_rem = 0; ++g_row; }
        float q, kv;
        featurizer_step3<T>(p, b, d, q, kv);
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < c; ++i) {
            acc = fmaf(s[r * c + i], ld_param(p.h, p.h_dtype, g * K + (flip ? c - i : i)), acc);
            if (i >= 1) o[r * c + i - 1] = s[r * c + i];
        }
        o[r * c + c - 1] = kv;
        float f = fmaf(ld_param(p.h, p.h_dtype, g * K + (flip ? 0 : c)), kv, acc);
        if (p.bias_mode != VTX_BIAS_NONE) {
            const float bias = ld_param(p.bias, p.bias_dtype, d);
            f = p.bias_mode == VTX_BIAS_GATED ? fmaf(bias, kv, f) : f + bias;
        }
        static_cast<T*>(p.y)[row0 + r] = from_f32<T>(round_io<T>(f) * q);
    }
    float4* sout4 = reinterpret_cast<float4*>(p.inner_state_out + row0 * c);
#pragma unroll
    for (int j = 0; j < 6; ++j) sout4[j] = make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
}

// The same layer for interleaved q/k/v (Evo 2's layout): the 12 packed channels of the thread's four hidden channels are
// neighbours, so their featurizer caches are six 16-byte vectors in and out, and every load of the thread (caches,
// tokens, raw parameter bits) is issued before the first use: one memory round trip, a few hundred instructions less
// than four calls of the general featurizer step.  Needs groups that are whole quads of channels.
template <typename T>
__global__ void __launch_bounds__(64) decode_fir7i_kernel(vtx_decode_layer_params p) {
    constexpr int K = 7, c = 6, RT = 4;
    const int64_t row0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * RT;
    if (row0 >= p.B * p.D) return;
    const int64_t b = div32(row0, p.D), d0 = row0 - b * p.D, c0 = b * 3 * p.D + 3 * d0;      // first packed channel
    const float4* sin4 = reinterpret_cast<const float4*>(static_cast<const float*>(p.inner_state_in) + row0 * c);
    const float4* fin4 = reinterpret_cast<const float4*>(static_cast<const float*>(p.fir_state_in) + c0 * 2);
    float4 v[6], f[6];
#pragma unroll
    for (int j = 0; j < 6; ++j) { v[j] = sin4[j]; f[j] = fin4[j]; }
    T ur[12];
#pragma unroll
    for (int i = 0; i < 12; ++i) ur[i] = static_cast<const T*>(p.u)[c0 + i];
    const bool w_wide = p.w3_dtype == VTX_F32, h_wide = p.h_dtype == VTX_F32;
    uint32_t wr[36], hr[K], br[12], dr[RT];
    const int64_t w0 = (3 * d0) * 3, hb = (int64_t)div32(d0, div32(p.D, p.G)) * K;
#pragma unroll
    for (int i = 0; i < 36; ++i) wr[i] = ld_raw(p.w3, w_wide, w0 + i);
#pragma unroll
    for (int i = 0; i < K; ++i) hr[i] = ld_raw(p.h, h_wide, hb + i);
#pragma unroll
    for (int i = 0; i < 12; ++i) br[i] = p.b3 ? ld_raw(p.b3, p.b3_dtype == VTX_F32, 3 * d0 + i) : 0u;
#pragma unroll
    for (int r = 0; r < RT; ++r) dr[r] = p.bias_mode != VTX_BIAS_NONE ? ld_raw(p.bias, p.bias_dtype == VTX_F32, d0 + r) : 0u;

    const float fs[24] = {f[0].x, f[0].y, f[0].z, f[0].w, f[1].x, f[1].y, f[1].z, f[1].w, f[2].x, f[2].y, f[2].z, f[2].w,
                          f[3].x, f[3].y, f[3].z, f[3].w, f[4].x, f[4].y, f[4].z, f[4].w, f[5].x, f[5].y, f[5].z, f[5].w};
    float z[12], fo[24];
#pragma unroll
    for (int i = 0; i < 12; ++i) {
        const float x = to_f32<T>(ur[i]);
        float acc = cvt_raw(wr[3 * i + 2], p.w3_dtype) * x;
        acc = fmaf(fs[2 * i], cvt_raw(wr[3 * i], p.w3_dtype), acc);
        acc = fmaf(fs[2 * i + 1], cvt_raw(wr[3 * i + 1], p.w3_dtype), acc);
        if (p.b3) acc += cvt_raw(br[i], p.b3_dtype);
        z[i] = round_io<T>(acc);
        fo[2 * i] = fs[2 * i + 1];
        fo[2 * i + 1] = x;
    }
    float4* fout4 = reinterpret_cast<float4*>(p.fir_state_out + c0 * 2);
#pragma unroll
    for (int j = 0; j < 6; ++j) fout4[j] = make_float4(fo[4 * j], fo[4 * j + 1], fo[4 * j + 2], fo[4 * j + 3]);

    const float s[RT * c] = {v[0].x, v[0].y, v[0].z, v[0].w, v[1].x, v[1].y, v[1].z, v[1].w, v[2].x, v[2].y, v[2].z, v[2].w,
                             v[3].x, v[3].y, v[3].z, v[3].w, v[4].x, v[4].y, v[4].z, v[4].w, v[5].x, v[5].y, v[5].z, v[5].w};
    const bool flip = p.flip_filter != 0, swap = p.flip_x1x2 != 0;
    float tap[K];
#pragma unroll
    for (int i = 0; i < K; ++i) tap[i] = cvt_raw(hr[i], p.h_dtype);
    float o[RT * c], y[RT];
#pragma unroll
    for (int r = 0; r < RT; ++r) {
        const float q = swap ? z[3 * r + 1] : z[3 * r], k = swap ? z[3 * r] : z[3 * r + 1];
        const float kv = round_io<T>(k * z[3 * r + 2]);
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < c; ++i) {
            acc = fmaf(s[r * c + i], flip ? tap[c - i] : tap[i], acc);
            if (i >= 1) o[r * c + i - 1] = s[r * c + i];
        }
        o[r * c + c - 1] = kv;
        float fv = fmaf(flip ? tap[0] : tap[c], kv, acc);
        if (p.bias_mode != VTX_BIAS_NONE) {
            const float bias = cvt_raw(dr[r], p.bias_dtype);
            fv = p.bias_mode == VTX_BIAS_GATED ? fmaf(bias, kv, fv) : fv + bias;
        }
        y[r] = round_io<T>(fv) * q;
    }
#pragma unroll
    for (int r = 0; r < RT; ++r) static_cast<T*>(p.y)[row0 + r] = from_f32<T>(y[r]);
    float4* sout4 = reinterpret_cast<float4*>(p.inner_state_out + row0 * c);
#pragma unroll
    for (int j = 0; j < 6; ++j) sout4[j] = make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
}

// Modal layer, RW rows per half-warp (lane = pole).  A block of 16 half-warps covers GPB channel groups of BPB batch
// elements; the groups' pole and residue parameters (expf, sincosf) are evaluated once per block into shared memory
// instead of once per tile.
template <typename T, int RW, bool CPLX>
__global__ void __launch_bounds__(256) decode_iir_tile_kernel(vtx_decode_layer_params p, int tiles_per_group, int gpb) {
    __shared__ float4 prm[16][16];                // [group of the block][pole]: p_re, p_im, R_re, R_im
    const int lane = threadIdx.x % 16, hw = threadIdx.x / 16;
    const unsigned mask = 0xffffu << (threadIdx.x % 32 - lane);
    const int S = (int)p.modal.S;
    const int64_t cpg = div32(p.D, p.modal.G);
    // block -> (batch slab, first group): blockIdx.x = slab * (G / gpb) + group block
    const int64_t gblocks = div32(p.modal.G, gpb), slab = div32(blockIdx.x, gblocks), g0 = ((int64_t)blockIdx.x - slab * gblocks) * gpb;
    for (int i = threadIdx.x; i < gpb * 16; i += blockDim.x) {
        const int gl = i / 16, sp = i % 16;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (sp < S) {
            const int64_t gi = (g0 + gl) * S + sp;
            const float mag = expf(static_cast<const float*>(p.modal.log_poles)[gi]);
            v.z = static_cast<const float*>(p.modal.res_re)[gi];
            if (CPLX) {
                float sn, cs;
                sincosf(static_cast<const float*>(p.modal.theta)[gi], &sn, &cs);
                v.x = mag * cs; v.y = mag * sn;
                v.w = p.modal.res_im ? static_cast<const float*>(p.modal.res_im)[gi] : 0.f;
            } else {
                v.x = mag;
            }
        }
        prm[gl][sp] = v;
    }
    __syncthreads();
    // half-warp hw -> tile: group gl = (hw / tiles_per_group) % gpb, tile within the group, batch element within the slab
    const int tpb = gpb * tiles_per_group;            // tiles of one batch element in this block
    const int gl = (hw % tpb) / tiles_per_group, tg = hw % tiles_per_group;
    const int64_t b = slab * (16 / tpb) + hw / tpb;
    if (b >= p.B) return;
    const int64_t d0 = (g0 + gl) * cpg + (int64_t)tg * RW, row0 = b * p.D + d0;
    float q_own = 0.f, kv_own = 0.f;
    if (lane < RW) featurizer_step3<T>(p, b, d0 + lane, q_own, kv_own);
    const int64_t ss = S * (CPLX ? 2 : 1);
    const float* st_in = p.iir_state_in + row0 * ss;
    float* st_out = p.iir_state_out + row0 * ss;
    float2 s[RW];
#pragma unroll
    for (int r = 0; r < RW; ++r) {
        s[r] = make_float2(0.f, 0.f);
        if (lane < S) {
            if (CPLX) s[r] = reinterpret_cast<const float2*>(st_in + r * ss)[lane];
            else s[r].x = st_in[r * ss + lane];
        }
    }
    const float4 pm = prm[gl][lane];
    const float pr = pm.x, pi = pm.y, rr = pm.z, ri = pm.w;
#pragma unroll
    for (int r = 0; r < RW; ++r) {
        const int64_t d = d0 + r;
        const float kv = __shfl_sync(mask, kv_own, r, 16), q = __shfl_sync(mask, q_own, r, 16);
        float part = 0.f;
        if (lane < S) {
            if (CPLX) {
                const float nr = fmaf(pr, s[r].x, fmaf(-pi, s[r].y, kv));
                const float ni = fmaf(pr, s[r].y, pi * s[r].x);
                reinterpret_cast<float2*>(st_out + r * ss)[lane] = make_float2(nr, ni);
                part = rr * nr - ri * ni;
            } else {
                const float n = fmaf(pr, s[r].x, kv);
                st_out[r * ss + lane] = n;
                part = rr * n;
            }
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) part += __shfl_xor_sync(mask, part, o, 16);
        if (lane == 0) {
            const float bias = p.bias ? ld_param(p.bias, p.bias_dtype, d) : 0.f;
            float skip = bias * kv;
            if (p.bias && p.bias_dtype != VTX_F32) skip = round_io<T>(skip);
            static_cast<T*>(p.y)[row0 + r] = from_f32<T>(q * (part + skip));
        }
    }
}

// Modal layer with real poles when the modal systems are not shared by whole tiles of 8 channels (Evo 2: one system
// per channel): four lanes per row, each with four of the row's 16 states as one 16-byte load and store; the row's
// poles and residues are read the same way.  Three of the four lanes do one packed channel of the featurizer each.
template <typename T>
__global__ void __launch_bounds__(256) decode_iir_quad_kernel(vtx_decode_layer_params p) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t row = tid >> 2;
    const int part = (int)(tid & 3);
    if (row >= p.B * p.D) return;                  // rows are whole quads: a quad leaves together
    const unsigned mask = 0xfu << ((threadIdx.x & 31) & ~3);
    const int64_t b = div32(row, p.D), d = row - b * p.D, g = div32(d, div32(p.D, p.modal.G));
    // state and parameters first: the longest latencies
    const float4 s = reinterpret_cast<const float4*>(p.iir_state_in + row * 16)[part];
    const float4 lp = reinterpret_cast<const float4*>(static_cast<const float*>(p.modal.log_poles) + g * 16)[part];
    const float4 rr = reinterpret_cast<const float4*>(static_cast<const float*>(p.modal.res_re) + g * 16)[part];
    float z = 0.f;
    const uint32_t draw = (part == 0 && p.bias) ? ld_raw(p.bias, p.bias_dtype == VTX_F32, d) : 0u;
    if (part < 3) {
        const QkvMap map = qkv_map(p);
        int64_t ch[3];
        map.get(d, ch[0], ch[1], ch[2]);
        const int64_t c = part == 0 ? ch[0] : part == 1 ? ch[1] : ch[2], so = (b * 3 * p.D + c) * 2;
        // every load of the featurizer step before the first use (raw parameter bits: no dtype branch in between)
        const float2 st = *reinterpret_cast<const float2*>(static_cast<const float*>(p.fir_state_in) + so);
        const T xr = static_cast<const T*>(p.u)[b * 3 * p.D + c];
        const bool wide = p.w3_dtype == VTX_F32;
        const uint32_t w0 = ld_raw(p.w3, wide, c * 3), w1 = ld_raw(p.w3, wide, c * 3 + 1), w2 = ld_raw(p.w3, wide, c * 3 + 2);
        const uint32_t b3r = p.b3 ? ld_raw(p.b3, p.b3_dtype == VTX_F32, c) : 0u;
        const float x = to_f32<T>(xr);
        float acc = cvt_raw(w2, p.w3_dtype) * x;
        acc = fmaf(st.x, cvt_raw(w0, p.w3_dtype), acc);
        acc = fmaf(st.y, cvt_raw(w1, p.w3_dtype), acc);
        *reinterpret_cast<float2*>(p.fir_state_out + so) = make_float2(st.y, x);
        if (p.b3) acc += cvt_raw(b3r, p.b3_dtype);
        z = round_io<T>(acc);
    }
    const float q = __shfl_sync(mask, z, 0, 4), k = __shfl_sync(mask, z, 1, 4), v = __shfl_sync(mask, z, 2, 4);
    const float kv = round_io<T>(k * v);
    float4 n;
    n.x = fmaf(expf(lp.x), s.x, kv);
    n.y = fmaf(expf(lp.y), s.y, kv);
    n.z = fmaf(expf(lp.z), s.z, kv);
    n.w = fmaf(expf(lp.w), s.w, kv);
    reinterpret_cast<float4*>(p.iir_state_out + row * 16)[part] = n;
    float sum = fmaf(rr.x, n.x, fmaf(rr.y, n.y, fmaf(rr.z, n.z, rr.w * n.w)));
    sum += __shfl_xor_sync(mask, sum, 1, 4);
    sum += __shfl_xor_sync(mask, sum, 2, 4);
    if (part == 0) {
        const float bias = p.bias ? cvt_raw(draw, p.bias_dtype) : 0.f;
        float skip = bias * kv;
        if (p.bias && p.bias_dtype != VTX_F32) skip = round_io<T>(skip);
        static_cast<T*>(p.y)[row] = from_f32<T>(q * (sum + skip));
    }
}

}  // namespace vtx

extern "C" int vtx_step_fir(const vtx_step_fir_params* p, void* stream) {
    using namespace vtx;
    VTX_REQUIRE(p && p->u && p->w && p->y, VTX_ERR_BAD_ARG, "step_fir: null pointer");
    VTX_REQUIRE(p->B > 0 && p->C > 0 && p->K > 0 && p->Gw > 0, VTX_ERR_BAD_ARG, "step_fir: sizes must be positive");
    VTX_REQUIRE(p->B * p->C < ((int64_t)1 << 31), VTX_ERR_UNSUPPORTED, "step_fir: more than 2^31 rows");
    VTX_REQUIRE(p->C % p->Gw == 0, VTX_ERR_BAD_ARG, "step_fir: C not a multiple of the filter count");
    VTX_REQUIRE(p->c >= 0 && p->c <= p->K - 1, VTX_ERR_BAD_ARG, "step_fir: cache length %lld outside [0, K-1]",
                (long long)p->c);
    VTX_REQUIRE(p->c == 0 || p->state_in, VTX_ERR_BAD_ARG, "step_fir: null state_in");
    VTX_REQUIRE(p->K == 1 || p->state_out, VTX_ERR_BAD_ARG, "step_fir: null state_out");
    VTX_REQUIRE((const void*)p->state_out != p->state_in || !p->state_in, VTX_ERR_BAD_ARG,
                "step_fir: state_out aliases state_in");
    VTX_REQUIRE(p->bias_mode == VTX_BIAS_NONE || p->bias, VTX_ERR_BAD_ARG, "step_fir: bias mode set without a bias");
    const int64_t rows = p->B * p->C;
    cudaStream_t s = (cudaStream_t)stream;
    VTX_DISPATCH_IO(p->io_dtype, T, {
        if (p->c > 16) step_fir_kernel<T, 32><<<(unsigned)ceil_div<int64_t>(rows * 32, 256), 256, 0, s>>>(*p);
        else step_fir_kernel<T, 1><<<(unsigned)ceil_div<int64_t>(rows, 256), 256, 0, s>>>(*p);
    });
    return check_launch("step_fir");
}

extern "C" int vtx_step_iir(const vtx_step_iir_params* p, void* stream) {
    using namespace vtx;
    VTX_REQUIRE(p && p->q && p->k && p->v && p->y && p->state_in && p->state_out, VTX_ERR_BAD_ARG,
                "step_iir: null pointer");
    VTX_REQUIRE(p->B > 0 && p->D > 0, VTX_ERR_BAD_ARG, "step_iir: sizes must be positive");
    VTX_REQUIRE(p->B * p->D < ((int64_t)1 << 31), VTX_ERR_UNSUPPORTED, "step_iir: more than 2^31 rows");
    VTX_REQUIRE(p->modal.log_poles && p->modal.res_re && p->modal.G > 0 && p->modal.S > 0, VTX_ERR_BAD_ARG,
                "step_iir: bad modal parameters");
    VTX_REQUIRE(p->D % p->modal.G == 0, VTX_ERR_BAD_ARG, "step_iir: D not a multiple of the number of modal systems");
    VTX_REQUIRE(p->modal.S <= 16, VTX_ERR_UNSUPPORTED, "step_iir: state size %lld > 16", (long long)p->modal.S);
    const int64_t rows = p->B * p->D;
    VTX_DISPATCH_IO(p->io_dtype, T,
                    step_iir_kernel<T><<<(unsigned)ceil_div<int64_t>(rows * 16, 256), 256, 0, (cudaStream_t)stream>>>(*p));
    return check_launch("step_iir");
}

extern "C" int vtx_decode_layer(const vtx_decode_layer_params* p, void* stream) {
    using namespace vtx;
    VTX_REQUIRE(p && p->u && p->w3 && p->y, VTX_ERR_BAD_ARG, "decode_layer: null pointer");
    VTX_REQUIRE(p->B > 0 && p->D > 0 && p->K3 >= 1 && p->K3 <= 8 && p->K >= 0, VTX_ERR_BAD_ARG,
                "decode_layer: bad sizes");
    VTX_REQUIRE(p->B * p->D < ((int64_t)1 << 29), VTX_ERR_UNSUPPORTED, "decode_layer: more than 2^29 rows");
    VTX_REQUIRE(p->K3 == 1 || (p->fir_state_in && p->fir_state_out), VTX_ERR_BAD_ARG, "decode_layer: null fir state");
    VTX_REQUIRE((const void*)p->fir_state_out != p->fir_state_in, VTX_ERR_BAD_ARG,
                "decode_layer: fir_state_out aliases fir_state_in");
    VTX_REQUIRE(p->layout != VTX_QKV_COLUMN_SPLIT || (p->num_heads > 0 && p->D % p->num_heads == 0), VTX_ERR_BAD_ARG,
                "decode_layer: column split needs num_heads dividing D");
    const int64_t rows = p->B * p->D;
    cudaStream_t s = (cudaStream_t)stream;
    if (p->K > 0) {
        VTX_REQUIRE(p->h && p->G > 0 && p->D % p->G == 0, VTX_ERR_BAD_ARG, "decode_layer: bad filter arguments");
        VTX_REQUIRE(p->K == 1 || (p->inner_state_in && p->inner_state_out), VTX_ERR_BAD_ARG,
                    "decode_layer: null inner state");
        VTX_REQUIRE((const void*)p->inner_state_out != p->inner_state_in, VTX_ERR_BAD_ARG,
                    "decode_layer: inner_state_out aliases inner_state_in");
        VTX_REQUIRE(p->bias_mode == VTX_BIAS_NONE || p->bias, VTX_ERR_BAD_ARG, "decode_layer: bias mode without a bias");
        // tiled kernel: full fp32 caches (every step but the first after a prefill), 3-tap featurizer, 18..129 taps
        const bool tiled = p->K > 17 && p->K <= 129 && p->K3 == 3 && p->D % 8 == 0 && p->fir_state_dtype == VTX_F32 &&
                           p->inner_state_dtype == VTX_F32;
        const bool short7 = p->K == 7 && p->K3 == 3 && p->D % 4 == 0 && p->fir_state_dtype == VTX_F32 &&
                            p->inner_state_dtype == VTX_F32 && reinterpret_cast<uintptr_t>(p->inner_state_in) % 16 == 0 &&
                            reinterpret_cast<uintptr_t>(p->inner_state_out) % 16 == 0;
        VTX_DISPATCH_IO(p->io_dtype, T, {
            const bool inter7 = short7 && p->layout == VTX_QKV_INTERLEAVED && (p->D / p->G) % 4 == 0 &&
                                reinterpret_cast<uintptr_t>(p->fir_state_in) % 16 == 0 &&
                                reinterpret_cast<uintptr_t>(p->fir_state_out) % 16 == 0;
            // (64-thread blocks: at ~140 registers per thread that is what lets B=64 x 4096 channels be resident at once)
            if (inter7) decode_fir7i_kernel<T><<<(unsigned)ceil_div<int64_t>(rows / 4, 64), 64, 0, s>>>(*p);
            else if (short7) decode_fir7_kernel<T><<<(unsigned)ceil_div<int64_t>(rows / 4, 256), 256, 0, s>>>(*p);
            else if (tiled && p->K == 128 && (p->D / p->G) % 8 == 0)
                decode_fir127_kernel<T><<<(unsigned)ceil_div<int64_t>(rows / 8 * 32, 256), 256, 0, s>>>(*p);
            else if (tiled) decode_fir_tile_kernel<T, 8><<<(unsigned)ceil_div<int64_t>(rows / 8 * 32, 256), 256, 0, s>>>(*p);
            else if (p->K > 17) decode_layer_kernel<T, 32, 0><<<(unsigned)ceil_div<int64_t>(rows * 32, 256), 256, 0, s>>>(*p);
            else decode_layer_kernel<T, 1, 0><<<(unsigned)ceil_div<int64_t>(rows, 256), 256, 0, s>>>(*p);
        });
    } else {
        VTX_REQUIRE(p->modal.log_poles && p->modal.res_re && p->modal.G > 0 && p->modal.S > 0 && p->modal.S <= 16 &&
                        p->D % p->modal.G == 0 && p->iir_state_in && p->iir_state_out,
                    VTX_ERR_BAD_ARG, "decode_layer: bad modal arguments");
        // tiled kernel: channel groups that are whole tiles of 8 (1, 2, 4, 8 or 16 tiles per block of 16 half-warps)
        const int64_t cpg = p->D / p->modal.G;
        const int64_t tpg = cpg / 8;                    // tiles per group
        const bool tiled = p->K3 == 3 && p->fir_state_dtype == VTX_F32 && cpg % 8 == 0 && (tpg == 1 || tpg == 2 || tpg == 4 || tpg == 8 || tpg == 16);
        const bool cplx = p->modal.theta != nullptr;
        // one system per channel (or per few): real poles, 16 states, four lanes per row
        const bool quad = !cplx && p->modal.S == 16 && p->K3 == 3 && p->fir_state_dtype == VTX_F32 &&
                          reinterpret_cast<uintptr_t>(p->iir_state_in) % 16 == 0 &&
                          reinterpret_cast<uintptr_t>(p->iir_state_out) % 16 == 0 &&
                          reinterpret_cast<uintptr_t>(p->modal.log_poles) % 16 == 0 &&
                          reinterpret_cast<uintptr_t>(p->modal.res_re) % 16 == 0;
        VTX_DISPATCH_IO(p->io_dtype, T, {
            if (tiled) {
                // a block = 16 tiles of one group: 16 / tpg batch elements share one evaluation of the group's poles
                const int gpb = 1;
                const int64_t bpb = 16 / (gpb * tpg);
                const int64_t nblk = (p->modal.G / gpb) * ceil_div<int64_t>(p->B, bpb);
                if (cplx) decode_iir_tile_kernel<T, 8, true><<<(unsigned)nblk, 256, 0, s>>>(*p, (int)tpg, gpb);
                else decode_iir_tile_kernel<T, 8, false><<<(unsigned)nblk, 256, 0, s>>>(*p, (int)tpg, gpb);
            } else if (quad) {
                decode_iir_quad_kernel<T><<<(unsigned)ceil_div<int64_t>(rows * 4, 256), 256, 0, s>>>(*p);
            } else {
                decode_layer_kernel<T, 16, 1><<<(unsigned)ceil_div<int64_t>(rows * 16, 256), 256, 0, s>>>(*p);
            }
        });
    }
    return check_launch("decode_layer");
}
