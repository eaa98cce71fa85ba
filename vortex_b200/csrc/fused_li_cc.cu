// Fused Hyena-LI block for modal systems that are NOT shared by groups of 16 channels (Evo 2 gives every channel
// its own 16 real poles, configs/evo2-7b-8k.yml:11 `hcl_filter_groups: 4096`), any I/O dtype, channel-last in and
// out:  featurizer (3 taps) -> q/k/v selection -> k*v -> modal recurrence -> (+ bias*kv) -> q gate.
// Fuses model.py:233-316 (featurizer parallel_fir + parallel_iir, engine.py:262-353) and the end state of
// engine.py:525-559 without the [B,3D,L] intermediate.
//
// A per-channel filter has no operand that tensor cores could share between channels, so the recurrence itself runs
// on the fp32 pipe:  sigma_s[t] = p_s sigma_s[t-1] + kv[t],  y[t] = q[t] (sum_s R_s sigma_s[t] + bias kv[t]),
// 32 FMA per sample and channel (real poles; issued as 16 packed fma.rn.f32x2).
// Thread = (batch, channel, time segment), lane = channel, so that a warp reads 32 neighbouring channels of a row.
// Segments make the parallelism batch*channels alone does not have; the carry between them takes three launches:
//   A  end state of every segment from a zero start            (reads k, v rows)
//   B  scan over the segments of a channel: start states        (tiny)
//   C  recurrence from the true start state, writes y           (reads q, k, v rows)
// Nothing between the input rows and the output is rounded to the I/O dtype (the reference rounds the featurizer
// output, k*v and the convolution result, engine.py:208,159,230): the result is closer to the fp32 reference.
// A call can continue an earlier one (chunked prefill): state_in is the modal state and fir_state_in the two
// projection rows the earlier call ended with.
#include "common.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace vtx {

VTX_DEFINE_STATUS_READER()

namespace licc {

using umma::f32x2;
using umma::fma2;
using umma::pk2;
using umma::up2;
using umma::add2;
using umma::mul2;

constexpr int NS = 16;         // states per thread (shorter systems are padded with p = R = 0)
constexpr int THREADS = 128;
#ifndef VTX_LICC_TB
#define VTX_LICC_TB 4
#endif
#ifndef VTX_LICC_MINB
#define VTX_LICC_MINB 4
#endif
constexpr int TB = VTX_LICC_TB;   // samples per software-pipeline block

struct Plan {
    int64_t nseg, seg_len;
    int pairs_a, pairs_c;      // staged kernels only: phase A / phase C run two channels per thread
};

// Segments per channel: about four rounds of resident threads over the SMs, segments of at least 64 samples.
static Plan plan(int64_t B, int64_t L, int64_t D, bool have_scratch) {
    Plan pl{1, L, 0, 0};
    if (!have_scratch) return pl;
    const int64_t rows = B * D, want = (int64_t)kNumSMs * 640 * 4;
    int64_t nseg = ceil_div<int64_t>(want, rows);
    if (nseg > L / 64) nseg = L / 64;
    if (nseg < 1) nseg = 1;
    int64_t seg = ceil_div<int64_t>(ceil_div<int64_t>(L, nseg), (int64_t)8) * 8;      // a multiple of both block sizes
    pl.seg_len = seg;
    pl.nseg = ceil_div<int64_t>(L, seg);
    return pl;
}

struct Args {
    const void* u; int64_t sb, sl;
    const void* w3; int64_t w3_dtype;
    const void* b3; int64_t b3_dtype;
    vtx_modal_params m;
    const void* bias; int64_t bias_dtype;
    void* y; int64_t ysb, ysl;
    float* state; const float* state_in;
    const void* fs_in; int64_t fs_dtype;
    int64_t hist_rows;             // rows in front of u that hold the sequence's earlier samples
    float* scratch;
    int64_t B, L, D;
    QkvMap map;
    Plan pl;
};

// scratch[(seg * SS + j) * rows + row]: component j of the state at the START of segment seg (after phase B)
template <bool CPLX> constexpr int comps(int S) { return CPLX ? 2 * S : S; }

template <bool CPLX>
struct Modes {
    float pr[NS], pi[CPLX ? NS : 1], rr[NS], ri[CPLX ? NS : 1];
    __device__ __forceinline__ void load(const vtx_modal_params& m, int64_t g) {
        const int S = (int)m.S;
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            pr[s] = rr[s] = 0.f;
            if constexpr (CPLX) pi[s] = ri[s] = 0.f;
            if (s < S) {
                const float mag = expf(static_cast<const float*>(m.log_poles)[g * S + s]);
                rr[s] = static_cast<const float*>(m.res_re)[g * S + s];
                if constexpr (CPLX) {
                    float sn, cs;
                    sincosf(static_cast<const float*>(m.theta)[g * S + s], &sn, &cs);
                    pr[s] = mag * cs; pi[s] = mag * sn;
                    ri[s] = m.res_im ? static_cast<const float*>(m.res_im)[g * S + s] : 0.f;
                } else {
                    pr[s] = mag;
                }
            }
        }
    }
};

// Real systems keep poles, residues and states as f32x2 pairs: one packed FMA advances two states.
template <bool CPLX> struct Sys;

template <>
struct Sys<false> {
    f32x2 p2[NS / 2], r2[NS / 2], s2[NS / 2];
    __device__ __forceinline__ void init(const Modes<false>& m) {
#pragma unroll
        for (int j = 0; j < NS / 2; ++j) {
            p2[j] = pk2(m.pr[2 * j], m.pr[2 * j + 1]);
            r2[j] = pk2(m.rr[2 * j], m.rr[2 * j + 1]);
            s2[j] = pk2(0.f, 0.f);
        }
    }
    // components j < n of a state vector stored with the given stride
    __device__ __forceinline__ void load(const float* in, int64_t stride, int n) {
#pragma unroll
        for (int j = 0; j < NS / 2; ++j) {
            const float lo = 2 * j < n ? in[(2 * j) * stride] : 0.f;
            const float hi = 2 * j + 1 < n ? in[(2 * j + 1) * stride] : 0.f;
            s2[j] = pk2(lo, hi);
        }
    }
    __device__ __forceinline__ void store(float* out, int64_t stride, int n) const {
#pragma unroll
        for (int j = 0; j < NS / 2; ++j) {
            float lo, hi;
            up2(s2[j], lo, hi);
            if (2 * j < n) out[(2 * j) * stride] = lo;
            if (2 * j + 1 < n) out[(2 * j + 1) * stride] = hi;
        }
    }
    __device__ __forceinline__ void advance(float x) {
        const f32x2 x2 = pk2(x, x);
#pragma unroll
        for (int j = 0; j < NS / 2; ++j) s2[j] = fma2(p2[j], s2[j], x2);
    }
    __device__ __forceinline__ float step(float x) {
        const f32x2 x2 = pk2(x, x);
        f32x2 a0 = pk2(0.f, 0.f), a1 = a0;
#pragma unroll
        for (int j = 0; j < NS / 2; j += 2) {
            s2[j] = fma2(p2[j], s2[j], x2);
            s2[j + 1] = fma2(p2[j + 1], s2[j + 1], x2);
            a0 = fma2(r2[j], s2[j], a0);
            a1 = fma2(r2[j + 1], s2[j + 1], a1);
        }
        float u0, u1, v0, v1;
        up2(a0, u0, u1);
        up2(a1, v0, v1);
        return (u0 + v0) + (u1 + v1);
    }
};

template <>
struct Sys<true> {
    float pr[NS], pi[NS], rr[NS], ri[NS], re[NS], im[NS];
    __device__ __forceinline__ void init(const Modes<true>& m) {
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            pr[s] = m.pr[s]; pi[s] = m.pi[s]; rr[s] = m.rr[s]; ri[s] = m.ri[s];
            re[s] = im[s] = 0.f;
        }
    }
    // components (re, im interleaved) j < n of a state vector stored with the given stride
    __device__ __forceinline__ void load(const float* in, int64_t stride, int n) {
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            re[s] = 2 * s < n ? in[(2 * s) * stride] : 0.f;
            im[s] = 2 * s + 1 < n ? in[(2 * s + 1) * stride] : 0.f;
        }
    }
    __device__ __forceinline__ void store(float* out, int64_t stride, int n) const {
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            if (2 * s < n) out[(2 * s) * stride] = re[s];
            if (2 * s + 1 < n) out[(2 * s + 1) * stride] = im[s];
        }
    }
    __device__ __forceinline__ void advance(float x) {
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            const float nr = fmaf(pr[s], re[s], fmaf(-pi[s], im[s], x));
            const float ni = fmaf(pr[s], im[s], pi[s] * re[s]);
            re[s] = nr; im[s] = ni;
        }
    }
    __device__ __forceinline__ float step(float x) {
        float acc = 0.f;
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            const float nr = fmaf(pr[s], re[s], fmaf(-pi[s], im[s], x));
            const float ni = fmaf(pr[s], im[s], pi[s] * re[s]);
            re[s] = nr; im[s] = ni;
            acc = fmaf(rr[s], nr, fmaf(-ri[s], ni, acc));
        }
        return acc;
    }
};

struct Work {
    int64_t b, d, row, seg, t0, t1;
    bool valid;
};
// Segment index slowest, so that the lanes of a warp sit on neighbouring channels of one segment.
__device__ __forceinline__ Work work_of(const Args& a) {
    Work w;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t rows = a.B * a.D;
    w.valid = i < rows * a.pl.nseg;
    w.row = i % rows;
    w.seg = i / rows;
    w.b = w.row / a.D;
    w.d = w.row % a.D;
    w.t0 = w.seg * a.pl.seg_len;
    w.t1 = w.t0 + a.pl.seg_len < a.L ? w.t0 + a.pl.seg_len : a.L;
    return w;
}

// One packed channel of the featurizer: taps, bias and the two samples before the current one.
template <typename T>
struct Stream {
    float w0, w1, w2, b;   // z[t] = w0 u[t-2] + w1 u[t-1] + w2 u[t] (+ b)
    float u1, u2;          // u[t-1], u[t-2]
    __device__ __forceinline__ void init(const Args& a, int64_t bidx, int64_t c, int64_t t0) {
        const T* col = static_cast<const T*>(a.u) + bidx * a.sb + c;
        w0 = ld_param(a.w3, a.w3_dtype, c * 3 + 0);
        w1 = ld_param(a.w3, a.w3_dtype, c * 3 + 1);
        w2 = ld_param(a.w3, a.w3_dtype, c * 3 + 2);
        b = a.b3 ? ld_param(a.b3, a.b3_dtype, c) : 0.f;
        u1 = hist(a, col, bidx, c, t0 - 1);
        u2 = hist(a, col, bidx, c, t0 - 2);
    }
    // sample at time t < t0: this call's rows, else the rows the previous call ended with, else zero
    __device__ __forceinline__ float hist(const Args& a, const T* col, int64_t bidx, int64_t c, int64_t t) const {
        if (t >= -a.hist_rows) return to_f32<T>(col[t * a.sl]);
        if (!a.fs_in) return 0.f;
        return ld_param(a.fs_in, a.fs_dtype, (bidx * 3 * a.D + c) * 2 + (2 + t));
    }
    __device__ __forceinline__ float feat(float u0) {
        const float z = fmaf(w2, u0, fmaf(w1, u1, fmaf(w0, u2, b)));
        u2 = u1; u1 = u0;
        return z;
    }
};

// Rows a segment will read PF samples from now, asked into L2 once per block of NB samples by 3 * NB lanes of the warp
// (NB rows x 3 pieces: the q, k, v columns of the warp's 32 channels, or the three thirds of their interleaved span).
constexpr int PF = 48;
template <typename T, int NB>
struct Prefetch {
    const T* piece;     // lane < 3 * NB: piece lane % 3 of the row PF + lane / 3 ahead of the block being computed
    int64_t step;       // NB rows
    int left;           // rows until the end of the tensor, counted from that row
    // cq, ck, cv: the thread's columns in the first row of its segment.  All 32 lanes of the warp must be here.
    __device__ __forceinline__ void init(const Args& a, const T* cq, const T* ck, const T* cv, int64_t t0) {
        const int lane = threadIdx.x & 31, j = lane % 3, row = lane / 3;
        const unsigned long long q0 = __shfl_sync(0xffffffffu, (unsigned long long)cq, 0);
        const unsigned long long k0 = __shfl_sync(0xffffffffu, (unsigned long long)ck, 0);
        const unsigned long long v0 = __shfl_sync(0xffffffffu, (unsigned long long)cv, 0);
        const unsigned long long lo = q0 < k0 ? (q0 < v0 ? q0 : v0) : (k0 < v0 ? k0 : v0);
        const bool inter = a.map.layout == VTX_QKV_INTERLEAVED;
        piece = (inter ? reinterpret_cast<const T*>(lo) + 32 * j : reinterpret_cast<const T*>(j == 0 ? q0 : j == 1 ? k0 : v0)) +
                (PF + row) * a.sl;
        step = NB * a.sl;
        const int64_t l = a.L - (t0 + PF + row);
        left = lane < 3 * NB ? (int)(l < 0 ? 0 : l > 0x7fffffff ? 0x7fffffff : l) : 0;
    }
    __device__ __forceinline__ void ask() {
        if (left > 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(piece));
        piece += step;
        left -= NB;
    }
};

template <typename T, bool CPLX>
__device__ __forceinline__ void load_state(Sys<CPLX>& sys, const Args& a, const Work& w) {
    const int SS = comps<CPLX>((int)a.m.S);
    if (w.seg > 0) {
        const int64_t rows = a.B * a.D;
        sys.load(a.scratch + (w.seg * SS) * rows + w.row, rows, SS);
    } else if (a.state_in) {
        sys.load(a.state_in + w.row * SS, 1, SS);
    }
}

// ---- phase A: end state of every segment but the last, from a zero start ------------------------------------------
constexpr int TBA = 8;         // samples per software-pipeline block (every segment but the last is a multiple of it)
template <typename T, bool CPLX>
__global__ void __launch_bounds__(THREADS) licc_segment_state_kernel(Args a) {
    const Work w = work_of(a);
    if (!w.valid || w.seg == a.pl.nseg - 1) return;
    Modes<CPLX> md;
    md.load(a.m, w.d / (a.D / a.m.G));
    Sys<CPLX> sys;
    sys.init(md);
    int64_t cq, ck, cv;
    a.map.get(w.d, cq, ck, cv);
    Stream<T> sk, sv;
    sk.init(a, w.b, ck, w.t0);
    sv.init(a, w.b, cv, w.t0);
    const T* row0 = static_cast<const T*>(a.u) + w.b * a.sb + w.t0 * a.sl;      // first row of the segment
    const bool use_pf = (a.B * a.D) % 32 == 0;       // whole warps on one segment
    Prefetch<T, TBA> pf;
    // interleaved rows hold q between k and v anyway; the other layouts read the k and v columns only
    if (use_pf) pf.init(a, row0 + (a.map.layout == VTX_QKV_INTERLEAVED ? cq : ck), row0 + ck, row0 + cv, w.t0);
    const T* pk = row0 + ck;        // running pointers of the loads, one block ahead of the arithmetic
    const T* pv = row0 + cv;
    const int64_t sl = a.sl;
    T bk[2][TBA], bv[2][TBA];
    auto fetch = [&](int which) {
#pragma unroll
        for (int i = 0; i < TBA; ++i) {
            bk[which][i] = *pk; bv[which][i] = *pv;
            pk += sl; pv += sl;
        }
    };
    auto consume = [&](int which) {
#pragma unroll
        for (int i = 0; i < TBA; ++i) sys.advance(sk.feat(to_f32<T>(bk[which][i])) * sv.feat(to_f32<T>(bv[which][i])));
    };
    int64_t left = (w.t1 - w.t0) / TBA;      // blocks
    fetch(0);
    while (true) {
        if (use_pf) pf.ask();
        if (left > 1) fetch(1);
        consume(0);
        if (--left == 0) break;
        if (use_pf) pf.ask();
        if (left > 1) fetch(0);
        consume(1);
        if (--left == 0) break;
    }
    const int SS = comps<CPLX>((int)a.m.S);
    const int64_t rows = a.B * a.D;
    sys.store(a.scratch + (w.seg * SS) * rows + w.row, rows, SS);
}

// ---- phase B: scratch[seg] <- state at the START of segment seg ----------------------------------------------------
template <bool CPLX>
__global__ void licc_carry_kernel(Args a) {
    const int S = (int)a.m.S, SS = comps<CPLX>(S);
    const int64_t rows = a.B * a.D;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * S) return;
    const int64_t row = i % rows;
    const int s = (int)(i / rows);
    const int64_t d = row % a.D, g = d / (a.D / a.m.G);
    // p^seg_len in polar form
    const float lam = static_cast<const float*>(a.m.log_poles)[g * S + s];
    const float mag = expf(lam * (float)a.pl.seg_len);
    float pr = mag, pi = 0.f;
    if (CPLX) {
        double ang = (double)static_cast<const float*>(a.m.theta)[g * S + s] * (double)a.pl.seg_len;
        ang -= 6.283185307179586 * floor(ang / 6.283185307179586);
        float sn, cs;
        sincosf((float)ang, &sn, &cs);
        pr = mag * cs; pi = mag * sn;
    }
    float cr = 0.f, ci = 0.f;
    if (a.state_in) {
        cr = a.state_in[row * SS + (CPLX ? 2 * s : s)];
        if (CPLX) ci = a.state_in[row * SS + 2 * s + 1];
    }
    // the end states of CB segments are read together (independent loads: the kernel is bound by memory latency),
    // then scanned and overwritten
    constexpr int CB = CPLX ? 8 : 24;       // (real systems: half the registers per segment, three times the loads in flight)
    const int64_t nseg = a.pl.nseg, seg_stride = (int64_t)SS * rows;
    float* e0 = a.scratch + (int64_t)(CPLX ? 2 * s : s) * rows + row;
    for (int64_t sb = 0; sb < nseg; sb += CB) {
        float er[CB], ei[CB];
#pragma unroll
        for (int k = 0; k < CB; ++k) {
            er[k] = ei[k] = 0.f;
            if (sb + k + 1 < nseg) {          // the last segment's end state is not a carry (phase A leaves it unwritten)
                er[k] = e0[(sb + k) * seg_stride];
                if (CPLX) ei[k] = e0[(sb + k) * seg_stride + rows];
            }
        }
#pragma unroll
        for (int k = 0; k < CB; ++k) {
            if (sb + k < nseg) {
                e0[(sb + k) * seg_stride] = cr;
                if (CPLX) e0[(sb + k) * seg_stride + rows] = ci;
                const float nr = pr * cr - pi * ci + er[k];
                const float ni = pr * ci + pi * cr + ei[k];
                cr = nr; ci = ni;
            }
        }
    }
}

// ---- phase C: outputs --------------------------------------------------------------------------------------------
// INTER: the three packed channels of a hidden channel are neighbours in a row (one running pointer, constant
// offsets); streams are then kept by POSITION in the row and q / k picked after the featurizer (flip_x1x2 swaps them).
template <typename T, bool CPLX, bool INTER>
__global__ void __launch_bounds__(THREADS, VTX_LICC_MINB) licc_output_kernel(Args a) {
    const Work w = work_of(a);
    if (!w.valid) return;
    Modes<CPLX> md;
    md.load(a.m, w.d / (a.D / a.m.G));
    Sys<CPLX> sys;
    sys.init(md);
    load_state<T, CPLX>(sys, a, w);
    int64_t cq, ck, cv;
    a.map.get(w.d, cq, ck, cv);
    const bool swap01 = INTER && a.map.flip;      // position 0 holds k, position 1 holds q
    if (swap01) { const int64_t t = cq; cq = ck; ck = t; }
    Stream<T> s0, s1, s2;                         // INTER: by position; else q, k, v
    s0.init(a, w.b, cq, w.t0);
    s1.init(a, w.b, ck, w.t0);
    s2.init(a, w.b, cv, w.t0);
    const float bias = a.bias ? ld_param(a.bias, a.bias_dtype, w.d) : 0.f;
    const T* row0 = static_cast<const T*>(a.u) + w.b * a.sb + w.t0 * a.sl;
    const bool use_pf = (a.B * a.D) % 32 == 0;       // whole warps on one segment
    Prefetch<T, TB> pf;
    if (use_pf) pf.init(a, row0 + cq, row0 + ck, row0 + cv, w.t0);
    const T* p0 = row0 + cq;        // running pointers of the loads, one block ahead of the arithmetic
    const T* p1 = row0 + ck;
    const T* p2 = row0 + cv;
    T* yp = static_cast<T*>(a.y) + w.b * a.ysb + w.t0 * a.ysl + w.d;
    const int64_t sl = a.sl, ysl = a.ysl;

    auto sample = [&](float e0, float e1, float e2) {
        const float z0 = s0.feat(e0), z1 = s1.feat(e1), v = s2.feat(e2);
        const float q = swap01 ? z1 : z0, k = swap01 ? z0 : z1;
        const float x = k * v;
        const float z = fmaf(bias, x, sys.step(x));
        *yp = from_f32<T>(z * q);
        yp += ysl;
    };
    T b0[2][TB], b1[2][TB], b2[2][TB];
    auto fetch = [&](int which) {
#pragma unroll
        for (int i = 0; i < TB; ++i) {
            if (INTER) {
                b0[which][i] = p0[0]; b1[which][i] = p0[1]; b2[which][i] = p0[2];
                p0 += sl;
            } else {
                b0[which][i] = *p0; b1[which][i] = *p1; b2[which][i] = *p2;
                p0 += sl; p1 += sl; p2 += sl;
            }
        }
    };
    auto consume = [&](int which) {
#pragma unroll
        for (int i = 0; i < TB; ++i) sample(to_f32<T>(b0[which][i]), to_f32<T>(b1[which][i]), to_f32<T>(b2[which][i]));
    };
    int64_t left = (w.t1 - w.t0) / TB;       // whole blocks
    const int ragged = (int)((w.t1 - w.t0) - left * TB);
    if (left > 0) {
        fetch(0);
        while (true) {
            if (use_pf) pf.ask();
            if (left > 1) fetch(1);
            consume(0);
            if (--left == 0) break;
            if (use_pf) pf.ask();
            if (left > 1) fetch(0);
            consume(1);
            if (--left == 0) break;
        }
    }
    for (int i = 0; i < ragged; ++i) {        // ragged end of the sequence (p0.. stand on its first row)
        if (INTER) sample(to_f32<T>(p0[0]), to_f32<T>(p0[1]), to_f32<T>(p0[2]));
        else sample(to_f32<T>(*p0), to_f32<T>(*p1), to_f32<T>(*p2));
        p0 += sl; p1 += sl; p2 += sl;
    }

    if (a.state && w.seg == a.pl.nseg - 1) {
        const int SS = comps<CPLX>((int)a.m.S);
        sys.store(a.state + w.row * SS, 1, SS);
    }
}


// ---- phases A and C with rows staged by TMA (16-bit I/O, real poles, interleaved q/k/v, D a multiple of 128) ------
// A CTA owns 128 neighbouring channels of one segment of one sequence.  The segment's rows (768 bytes per row: 128
// channels x q,k,v) stream through a ring of shared-memory stages as two TMA boxes of 64 channels; the four warps read
// their samples from the stage with constant offsets, so the arithmetic never waits on a global load and carries no
// load buffers in registers.  There is no producer warp: the warp that is LAST to finish a stage (an arrival counter
// in shared memory) re-arms the stage's barrier and issues the boxes that refill it, so no warp ever waits for a stage
// to drain.  A warp takes the EVEN or the ODD channels of 64: a channel's three
// 16-bit values (6 bytes) then sit in one aligned 32-bit word and one 16-bit half at the same place for every lane
// (word first for even channels, half first for odd ones), which makes two conflict-free shared loads per sample.
// ROLE names what the word's low half, its high half and the single half hold (flip_x1x2 swaps q and k):
//   0: q k | v     1: k q | v     2: q | k v  (half first)     3: k | q v  (half first)
constexpr int TC = 128;                     // channels per CTA
constexpr int RS = 8;                       // rows per stage (every segment but the last is a multiple of it)
constexpr int NST = 6;                      // stages in flight
constexpr int HALF_ROW = 64 * 3 * 2;        // bytes of a row of one 64-channel box
constexpr int HALF_BYTES = RS * HALF_ROW;
constexpr int STAGE_BYTES = 2 * HALF_BYTES;
constexpr int TTHREADS = 128;
constexpr int MINB_A = 5, MINB_C = 4;      // resident CTAs per SM asked of the compiler: phase A, phase C

template <typename T> __device__ __forceinline__ float lo_f32(uint32_t w);
template <typename T> __device__ __forceinline__ float hi_f32(uint32_t w);
template <> __device__ __forceinline__ float lo_f32<__nv_bfloat16>(uint32_t w) { return __uint_as_float(w << 16); }
template <> __device__ __forceinline__ float hi_f32<__nv_bfloat16>(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
template <> __device__ __forceinline__ float lo_f32<__half>(uint32_t w) { return __half2float(__ushort_as_half((unsigned short)(w & 0xffffu))); }
template <> __device__ __forceinline__ float hi_f32<__half>(uint32_t w) { return __half2float(__ushort_as_half((unsigned short)(w >> 16))); }
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
// arrival at a stage's counter; release / acquire so that the warp that sees the last arrival may overwrite the stage
__device__ __forceinline__ uint32_t arrive_count(uint32_t addr) {
    uint32_t old;
    asm volatile("atom.acq_rel.cta.shared.add.u32 %0, [%1], 1;" : "=r"(old) : "r"(addr) : "memory");
    return old;
}
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
    unsigned short v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}

// Per-thread state of the staged kernels: the modal system as packed pairs, the featurizer of k and v as one packed
// stream, the featurizer of q as a scalar one.  The output of a sample uses the state BEFORE the sample,
//   y[t] = q[t] (sum_s (R_s p_s) sigma_s[t-1] + (sum_s R_s + bias) kv[t]),
// so that its 8 packed FMAs do not wait for the 8 that advance the state.
template <bool OUT>
struct Lane {
    f32x2 p2[NS / 2], c2[NS / 2], s2[NS / 2];      // poles, R p (OUT), states
    f32x2 W0, W1, W2, WB, U1, U2;                  // featurizer of (k, v): taps, bias, the two samples before
    float q0, q1, q2, qb, qu1, qu2;                // featurizer of q (OUT)
    float direct;                                  // sum of residues + skip (OUT)
};

template <typename T, bool OUT, int ROLE>
__device__ __forceinline__ void tma_segment(const CUtensorMap* tmu, const Args& a, Lane<OUT>& ln, int64_t b, int64_t d,
                                            int64_t t0, int64_t t1, int x0, int lane, int par, int half, uint32_t stage0,
                                            uint32_t full0, uint32_t cnt0) {
    // position of q and of k in the channel's three packed values (v is the third)
    constexpr int PQ = (ROLE & 1) ? 1 : 0, PK = 1 - PQ;
    T* yp = OUT ? static_cast<T*>(a.y) + b * a.ysb + t0 * a.ysl + d : nullptr;
    const int64_t ysl = a.ysl;
    // byte offsets of the lane's word and half inside a row of its box
    const uint32_t off_w = 12 * lane + (par ? 8 : 0), off_s = 12 * lane + (par ? 6 : 4);

    // featurizer of one row: k*v and (OUT) q of the sample, from the lane's word and half
    auto front = [&](uint32_t wd, uint32_t hs, float& x, float& q) {
        const float fl = lo_f32<T>(wd), fh = hi_f32<T>(wd), fs = lo_f32<T>(hs);
        // par 0: positions 0, 1 in the word, 2 in the half;  par 1: position 0 in the half, 1, 2 in the word
        const float u_pos0 = (ROLE < 2) ? fl : fs, u_pos1 = (ROLE < 2) ? fh : fl, u_pos2 = (ROLE < 2) ? fs : fh;
        const float uk = PK == 0 ? u_pos0 : u_pos1, uq = PQ == 0 ? u_pos0 : u_pos1;
        const f32x2 u0 = pk2(uk, u_pos2);
        const f32x2 z = fma2(ln.W2, u0, fma2(ln.W1, ln.U1, fma2(ln.W0, ln.U2, ln.WB)));
        ln.U2 = ln.U1; ln.U1 = u0;
        float zk, zv;
        up2(z, zk, zv);
        x = zk * zv;
        if (OUT) {
            q = fmaf(ln.q2, uq, fmaf(ln.q1, ln.qu1, fmaf(ln.q0, ln.qu2, ln.qb)));
            ln.qu2 = ln.qu1; ln.qu1 = uq;
        }
    };
    // the recurrence of one sample; returns the gated output (OUT)
    auto back = [&](float x, float q) -> float {
        const f32x2 x2 = pk2(x, x);
        float y = 0.f;
        if (OUT) {
            f32x2 a0 = mul2(ln.c2[0], ln.s2[0]), a1 = mul2(ln.c2[1], ln.s2[1]);
#pragma unroll
            for (int j = 2; j < NS / 2; j += 2) {
                a0 = fma2(ln.c2[j], ln.s2[j], a0);
                a1 = fma2(ln.c2[j + 1], ln.s2[j + 1], a1);
            }
            float e0, e1;
            up2(add2(a0, a1), e0, e1);
            y = fmaf(ln.direct, x, e0 + e1) * q;
        }
#pragma unroll
        for (int j = 0; j < NS / 2; ++j) ln.s2[j] = fma2(ln.p2[j], ln.s2[j], x2);
        return y;
    };
    // A stage in three sweeps over its rows: every shared load, every featurizer (independent between rows), then the
    // recurrence with the stores.  Written out this way the loads of a row never sit behind the store of the row before.
    auto stage_full = [&](uint32_t base) {
        uint32_t wd[RS], hs[RS];
        float x[RS], q[RS];
#pragma unroll
        for (int r = 0; r < RS; ++r) { wd[r] = lds32(base + r * HALF_ROW + off_w); hs[r] = lds16(base + r * HALF_ROW + off_s); }
#pragma unroll
        for (int r = 0; r < RS; ++r) front(wd[r], hs[r], x[r], q[r]);
#pragma unroll
        for (int r = 0; r < RS; ++r) {
            const float y = back(x[r], q[r]);
            if (OUT) { *yp = from_f32<T>(y); yp += ysl; }
        }
    };
    auto sample = [&](uint32_t row) {
        float x, q = 0.f;
        front(lds32(row + off_w), lds16(row + off_s), x, q);
        const float y = back(x, q);
        if (OUT) { *yp = from_f32<T>(y); yp += ysl; }
    };

    const int nrows = (int)(t1 - t0), nfull = nrows / RS, rem = nrows - nfull * RS;
    const int nstage = nfull + (rem ? 1 : 0);
    for (int k = 0; k < nstage; ++k) {
        const int st = k % NST;
        if (!mbar_wait(full0 + 8 * st, (k / NST) & 1, 61)) return;
        const uint32_t base = stage0 + st * STAGE_BYTES + half * HALF_BYTES;
        if (k < nfull) {
            stage_full(base);
        } else {
            for (int r = 0; r < rem; ++r) sample(base + r * HALF_ROW);
        }
        __syncwarp();
        // the counter only grows: the fourth arrival of round k / NST finds 4 (k / NST) + 3
        if (lane == 0 && arrive_count(cnt0 + 4 * st) == 4u * (uint32_t)(k / NST) + 3u && k + NST < nstage) {
            mbar_expect_tx(full0 + 8 * st, STAGE_BYTES);
            const uint32_t dst = stage0 + st * STAGE_BYTES;
            const int y = (int)(t0 + (int64_t)(k + NST) * RS);
            tma_load_3d(dst, tmu, full0 + 8 * st, x0, y, (int)b);
            tma_load_3d(dst + HALF_BYTES, tmu, full0 + 8 * st, x0 + 3 * 64, y, (int)b);
        }
    }
}

template <typename T, bool OUT, int MINB>
__global__ void __launch_bounds__(TTHREADS, MINB) licc_tma_kernel(const __grid_constant__ CUtensorMap tmu, Args a) {
    __shared__ __align__(128) uint8_t stages[NST * STAGE_BYTES];
    __shared__ __align__(8) uint64_t bars[NST];
    __shared__ uint32_t counts[NST];
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t stage0 = smem_u32(stages), full0 = smem_u32(&bars[0]), cnt0 = smem_u32(&counts[0]);
    // blockIdx = (segment, sequence, channel tile), channel tile fastest: neighbouring CTAs read neighbouring pieces of a row
    const int64_t ntile = a.D / TC;
    const int64_t tile = blockIdx.x % ntile, b = (blockIdx.x / ntile) % a.B, seg = blockIdx.x / (ntile * a.B);
    const int64_t t0 = seg * a.pl.seg_len, t1 = t0 + a.pl.seg_len < a.L ? t0 + a.pl.seg_len : a.L;
    const int half = (warp >> 1) & 1, par = warp & 1;
    const int64_t d = tile * TC + half * 64 + 2 * lane + par, row = b * a.D + d, rows = a.B * a.D;
    const int S = (int)a.m.S;

    // ---- the first boxes, then every global load of the set-up, before anything waits
    const int x0 = (int)(tile * 3 * TC);
    if (tid == 0) {
        for (int s = 0; s < NST; ++s) { mbar_init(full0 + 8 * s, 1); counts[s] = 0; }
        fence_mbar_init();
        const int nstage = (int)((t1 - t0 + RS - 1) / RS);
        for (int k = 0; k < NST && k < nstage; ++k) {
            mbar_expect_tx(full0 + 8 * k, STAGE_BYTES);
            const uint32_t dst = stage0 + k * STAGE_BYTES;
            tma_load_3d(dst, &tmu, full0 + 8 * k, x0, (int)(t0 + (int64_t)k * RS), (int)b);
            tma_load_3d(dst + HALF_BYTES, &tmu, full0 + 8 * k, x0 + 3 * 64, (int)(t0 + (int64_t)k * RS), (int)b);
        }
    }
    float lp[NS], rr[NS], st[NS];
    uint32_t wraw[9], braw[3] = {0, 0, 0}, hraw[6] = {0, 0, 0, 0, 0, 0}, draw = 0;
    const bool slow_hist = t0 < 2 && a.hist_rows < 2;       // the sequence starts here: rows of an earlier call, or zeros
    {
        const int64_t g = d / (a.D / a.m.G);
        const float* lpp = static_cast<const float*>(a.m.log_poles) + g * S;
        const float* rrp = static_cast<const float*>(a.m.res_re) + g * S;
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            lp[s] = s < S ? lpp[s] : 0.f;
            rr[s] = s < S ? rrp[s] : 0.f;
            st[s] = 0.f;
        }
        if (OUT) {
            if (seg > 0) {
#pragma unroll
                for (int s = 0; s < NS; ++s) if (s < S) st[s] = a.scratch[(seg * S + s) * rows + row];
            } else if (a.state_in) {
#pragma unroll
                for (int s = 0; s < NS; ++s) if (s < S) st[s] = a.state_in[row * S + s];
            }
        }
        const bool w_wide = a.w3_dtype == VTX_F32;
#pragma unroll
        for (int i = 0; i < 9; ++i) wraw[i] = ld_raw(a.w3, w_wide, 9 * d + i);
        if (a.b3) {
            const bool b_wide = a.b3_dtype == VTX_F32;
#pragma unroll
            for (int i = 0; i < 3; ++i) braw[i] = ld_raw(a.b3, b_wide, 3 * d + i);
        }
        if (OUT && a.bias) draw = ld_raw(a.bias, a.bias_dtype == VTX_F32, d);
        if (!slow_hist) {
            const unsigned short* up = reinterpret_cast<const unsigned short*>(a.u) + b * a.sb + (t0 - 2) * a.sl + 3 * d;
#pragma unroll
            for (int i = 0; i < 3; ++i) { hraw[i] = up[i]; hraw[3 + i] = up[a.sl + i]; }      // rows t0-2 and t0-1
        }
    }
    __syncthreads();

    // ---- values
    Lane<OUT> ln;
    const int PQ = a.map.flip ? 1 : 0, PK = 1 - PQ;
    float wv[9], bv[3], hv[6];
#pragma unroll
    for (int i = 0; i < 9; ++i) wv[i] = cvt_raw(wraw[i], a.w3_dtype);
#pragma unroll
    for (int i = 0; i < 3; ++i) bv[i] = a.b3 ? cvt_raw(braw[i], a.b3_dtype) : 0.f;
    if (slow_hist) {
        // sample at time t < 0: this call's rows in front of u, else the rows the previous call ended with, else zero
#pragma unroll
        for (int i = 0; i < 6; ++i) {
            const int64_t c = 3 * d + i % 3, t = t0 - 2 + i / 3;
            float v = 0.f;
            if (t >= -a.hist_rows) v = to_f32<T>(static_cast<const T*>(a.u)[b * a.sb + t * a.sl + c]);
            else if (a.fs_in) v = ld_param(a.fs_in, a.fs_dtype, (b * 3 * a.D + c) * 2 + (2 + t));
            hv[i] = v;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 6; ++i) hv[i] = lo_f32<T>(hraw[i]);
    }
    // packed channel pos: taps wv[3 pos + tap], bias bv[pos], history hv[pos] (t0-2), hv[3 + pos] (t0-1)
    ln.W0 = pk2(wv[3 * PK + 0], wv[6]); ln.W1 = pk2(wv[3 * PK + 1], wv[7]); ln.W2 = pk2(wv[3 * PK + 2], wv[8]);
    ln.WB = pk2(bv[PK], bv[2]);
    ln.U2 = pk2(hv[PK], hv[2]); ln.U1 = pk2(hv[3 + PK], hv[5]);
    ln.q0 = wv[3 * PQ + 0]; ln.q1 = wv[3 * PQ + 1]; ln.q2 = wv[3 * PQ + 2]; ln.qb = bv[PQ];
    ln.qu2 = hv[PQ]; ln.qu1 = hv[3 + PQ];
    float rsum = 0.f;
    {
        float pm[NS], cm[NS];
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            pm[s] = s < S ? expf(lp[s]) : 0.f;
            cm[s] = rr[s] * pm[s];
            rsum += rr[s];
        }
#pragma unroll
        for (int j = 0; j < NS / 2; ++j) {
            ln.p2[j] = pk2(pm[2 * j], pm[2 * j + 1]);
            ln.c2[j] = pk2(cm[2 * j], cm[2 * j + 1]);
            ln.s2[j] = pk2(st[2 * j], st[2 * j + 1]);
        }
    }
    ln.direct = rsum + (OUT && a.bias ? cvt_raw(draw, a.bias_dtype) : 0.f);

    switch (par * 2 + PQ) {
        case 0: tma_segment<T, OUT, 0>(&tmu, a, ln, b, d, t0, t1, x0, lane, par, half, stage0, full0, cnt0); break;
        case 1: tma_segment<T, OUT, 1>(&tmu, a, ln, b, d, t0, t1, x0, lane, par, half, stage0, full0, cnt0); break;
        case 2: tma_segment<T, OUT, 2>(&tmu, a, ln, b, d, t0, t1, x0, lane, par, half, stage0, full0, cnt0); break;
        default: tma_segment<T, OUT, 3>(&tmu, a, ln, b, d, t0, t1, x0, lane, par, half, stage0, full0, cnt0); break;
    }
    float* out = OUT ? (a.state && seg == a.pl.nseg - 1 ? a.state + row * S : nullptr) : a.scratch + (seg * S) * rows + row;
    const int64_t stride = OUT ? 1 : rows;
    if (out) {
#pragma unroll
        for (int j = 0; j < NS / 2; ++j) {
            float lo, hi;
            up2(ln.s2[j], lo, hi);
            if (2 * j < S) out[(2 * j) * stride] = lo;
            if (2 * j + 1 < S) out[(2 * j + 1) * stride] = hi;
        }
    }
}

// ---- the same two phases with TWO channels per thread, packed ACROSS the channels ------------------------------
// A lane owns a channel pair (12 bytes of a row: three aligned words); every value of the recurrence is an f32x2 of
// the two channels, so the k*v product is born packed (no broadcast move), the q featurizer is packed too, a sample
// costs three shared loads, six conversions and one 4-byte store per PAIR, and the two outputs leave as one bf16x2.
// Per sample and channel that is 52 issue cycles in C and 27 in A against 67 and 33 of the kernel above, at twice the
// registers (three resident CTAs per SM in C, four in A).  A warp streams its own 64 channels through its own ring of
// stages: no barrier is shared between warps.  Needs D a multiple of 256 and no featurizer bias.
// Measured (B=1, L=131072, D=4096): 1.67 ms with both phases this way, 1.86 ms with phase A only, 1.93 ms with
// neither.  The segment plan picks the form of each phase (both read the same plan and the same scratch).
constexpr int TC2 = 256;                    // channels per CTA
constexpr int NST2 = 3;                     // stages in flight per warp
constexpr int BOX2_BYTES = RS * HALF_ROW;   // one stage of one warp: RS rows of 64 channels
constexpr int MINB2_A = 4, MINB2_C = 3;

template <typename T> __device__ __forceinline__ uint32_t pack_io(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack_io<__nv_bfloat16>(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
template <> __device__ __forceinline__ uint32_t pack_io<__half>(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

template <typename T, bool OUT, bool FLIP, int MINB>
__global__ void __launch_bounds__(TTHREADS, MINB) licc_tma2_kernel(const __grid_constant__ CUtensorMap tmu, Args a) {
    __shared__ __align__(128) uint8_t stages[4 * NST2 * BOX2_BYTES];
    __shared__ __align__(8) uint64_t bars[4 * NST2];
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t stage0 = smem_u32(stages) + warp * NST2 * BOX2_BYTES, full0 = smem_u32(&bars[warp * NST2]);
    const int64_t ntile = a.D / TC2;
    const int64_t tile = blockIdx.x % ntile, b = (blockIdx.x / ntile) % a.B, seg = blockIdx.x / (ntile * a.B);
    const int64_t t0 = seg * a.pl.seg_len, t1 = t0 + a.pl.seg_len < a.L ? t0 + a.pl.seg_len : a.L;
    const int64_t d0 = tile * TC2 + warp * 64 + 2 * lane, row0 = b * a.D + d0, rows = a.B * a.D;
    const int S = (int)a.m.S;
    const int nrows = (int)(t1 - t0), nfull = nrows / RS, rem = nrows - nfull * RS, nstage = nfull + (rem ? 1 : 0);
    const int x0 = (int)(tile * 3 * TC2 + warp * 3 * 64);

    // ---- the warp's first boxes, then every global load of the set-up, before anything waits
    if (lane == 0) {
        for (int k = 0; k < NST2; ++k) mbar_init(full0 + 8 * k, 1);
        fence_mbar_init();
        for (int k = 0; k < NST2 && k < nstage; ++k) {
            mbar_expect_tx(full0 + 8 * k, BOX2_BYTES);
            tma_load_3d(stage0 + k * BOX2_BYTES, &tmu, full0 + 8 * k, x0, (int)(t0 + (int64_t)k * RS), (int)b);
        }
    }
    float lp[2][NS], rr[2][NS], st[2][NS];
    uint32_t wraw[18], hraw[12], draw[2] = {0, 0};
    const bool slow_hist = t0 < 2 && a.hist_rows < 2;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const int64_t g = (d0 + c) / (a.D / a.m.G);
        const float* lpp = static_cast<const float*>(a.m.log_poles) + g * S;
        const float* rrp = static_cast<const float*>(a.m.res_re) + g * S;
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            lp[c][s] = s < S ? lpp[s] : 0.f;
            rr[c][s] = s < S ? rrp[s] : 0.f;
            st[c][s] = 0.f;
        }
        if (OUT) {
            if (seg > 0) {
#pragma unroll
                for (int s = 0; s < NS; ++s) if (s < S) st[c][s] = a.scratch[(seg * S + s) * rows + row0 + c];
            } else if (a.state_in) {
#pragma unroll
                for (int s = 0; s < NS; ++s) if (s < S) st[c][s] = a.state_in[(row0 + c) * S + s];
            }
        }
        if (OUT && a.bias) draw[c] = ld_raw(a.bias, a.bias_dtype == VTX_F32, d0 + c);
    }
    {
        const bool w_wide = a.w3_dtype == VTX_F32;
#pragma unroll
        for (int i = 0; i < 18; ++i) wraw[i] = ld_raw(a.w3, w_wide, 9 * d0 + i);
        if (!slow_hist) {
            const unsigned short* up = reinterpret_cast<const unsigned short*>(a.u) + b * a.sb + (t0 - 2) * a.sl + 3 * d0;
#pragma unroll
            for (int i = 0; i < 6; ++i) { hraw[i] = up[i]; hraw[6 + i] = up[a.sl + i]; }      // rows t0-2 and t0-1
        }
    }
    __syncwarp();

    // ---- values: everything as pairs (channel d0, channel d0 + 1)
    constexpr int PQ = FLIP ? 1 : 0, PK = 1 - PQ;
    float hv[12];
    if (slow_hist) {
#pragma unroll
        for (int i = 0; i < 12; ++i) {
            const int64_t c = 3 * d0 + i % 6, t = t0 - 2 + i / 6;
            float v = 0.f;
            if (t >= -a.hist_rows) v = to_f32<T>(static_cast<const T*>(a.u)[b * a.sb + t * a.sl + c]);
            else if (a.fs_in) v = ld_param(a.fs_in, a.fs_dtype, (b * 3 * a.D + c) * 2 + (2 + t));
            hv[i] = v;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 12; ++i) hv[i] = lo_f32<T>(hraw[i]);
    }
    // packed position pos of channel c: taps wraw[9 c + 3 pos + tap], history hv[3 c + pos] (t0-2), hv[6 + 3 c + pos] (t0-1)
    auto tap2 = [&](int pos, int tap) {
        return pk2(cvt_raw(wraw[3 * pos + tap], a.w3_dtype), cvt_raw(wraw[9 + 3 * pos + tap], a.w3_dtype));
    };
    f32x2 Wk[3], Wv[3], Wq[3];
#pragma unroll
    for (int j = 0; j < 3; ++j) { Wk[j] = tap2(PK, j); Wv[j] = tap2(2, j); Wq[j] = tap2(PQ, j); }
    f32x2 Uk2 = pk2(hv[PK], hv[3 + PK]), Uk1 = pk2(hv[6 + PK], hv[9 + PK]);
    f32x2 Uv2 = pk2(hv[2], hv[5]), Uv1 = pk2(hv[8], hv[11]);
    f32x2 Uq2 = pk2(hv[PQ], hv[3 + PQ]), Uq1 = pk2(hv[6 + PQ], hv[9 + PQ]);
    f32x2 p2[NS], c2[OUT ? NS : 1], s2[NS];
    float rsum0 = 0.f, rsum1 = 0.f;
#pragma unroll
    for (int s = 0; s < NS; ++s) {
        const float pa = s < S ? expf(lp[0][s]) : 0.f, pb = s < S ? expf(lp[1][s]) : 0.f;
        p2[s] = pk2(pa, pb);
        if (OUT) c2[s] = pk2(rr[0][s] * pa, rr[1][s] * pb);
        s2[s] = pk2(st[0][s], st[1][s]);
        rsum0 += rr[0][s]; rsum1 += rr[1][s];
    }
    const f32x2 direct = pk2(rsum0 + (OUT && a.bias ? cvt_raw(draw[0], a.bias_dtype) : 0.f),
                             rsum1 + (OUT && a.bias ? cvt_raw(draw[1], a.bias_dtype) : 0.f));
    uint32_t* yp = OUT ? reinterpret_cast<uint32_t*>(static_cast<T*>(a.y) + b * a.ysb + t0 * a.ysl + d0) : nullptr;
    const int64_t ysl2 = a.ysl / 2;                 // row pitch in 4-byte words (rows are 4-byte aligned: checked by the host)
    const uint32_t off = 12 * lane;

    auto sample = [&](uint32_t rowaddr) {
        const uint32_t w0 = lds32(rowaddr + off), w1 = lds32(rowaddr + off + 4), w2 = lds32(rowaddr + off + 8);
        // channel d0: positions 0, 1 in w0, 2 in the low half of w1; channel d0 + 1: 0 in the high half of w1, 1, 2 in w2
        const f32x2 P0 = pk2(lo_f32<T>(w0), hi_f32<T>(w1)), P1 = pk2(hi_f32<T>(w0), lo_f32<T>(w2)),
                    P2 = pk2(lo_f32<T>(w1), hi_f32<T>(w2));
        const f32x2 uk = PK == 0 ? P0 : P1, uq = PQ == 0 ? P0 : P1;
        const f32x2 zk = fma2(Wk[2], uk, fma2(Wk[1], Uk1, mul2(Wk[0], Uk2)));
        const f32x2 zv = fma2(Wv[2], P2, fma2(Wv[1], Uv1, mul2(Wv[0], Uv2)));
        Uk2 = Uk1; Uk1 = uk; Uv2 = Uv1; Uv1 = P2;
        const f32x2 x2 = mul2(zk, zv);
        if (OUT) {
            const f32x2 zq = fma2(Wq[2], uq, fma2(Wq[1], Uq1, mul2(Wq[0], Uq2)));
            Uq2 = Uq1; Uq1 = uq;
            f32x2 a0 = mul2(c2[0], s2[0]), a1 = mul2(c2[1], s2[1]);
#pragma unroll
            for (int j = 2; j < NS; j += 2) {
                a0 = fma2(c2[j], s2[j], a0);
                a1 = fma2(c2[j + 1], s2[j + 1], a1);
            }
#pragma unroll
            for (int j = 0; j < NS; ++j) s2[j] = fma2(p2[j], s2[j], x2);
            float y0, y1;
            up2(mul2(fma2(direct, x2, add2(a0, a1)), zq), y0, y1);
            *yp = pack_io<T>(y0, y1);
            yp += ysl2;
        } else {
#pragma unroll
            for (int j = 0; j < NS; ++j) s2[j] = fma2(p2[j], s2[j], x2);
        }
    };

    for (int k = 0; k < nstage; ++k) {
        const int sl = k % NST2;
        if (!mbar_wait(full0 + 8 * sl, (k / NST2) & 1, 63)) return;
        const uint32_t base = stage0 + sl * BOX2_BYTES;
        if (k < nfull) {
#pragma unroll
            for (int r = 0; r < RS; ++r) sample(base + r * HALF_ROW);
        } else {
            for (int r = 0; r < rem; ++r) sample(base + r * HALF_ROW);
        }
        __syncwarp();
        if (lane == 0 && k + NST2 < nstage) {
            mbar_expect_tx(full0 + 8 * sl, BOX2_BYTES);
            tma_load_3d(base, &tmu, full0 + 8 * sl, x0, (int)(t0 + (int64_t)(k + NST2) * RS), (int)b);
        }
    }
    float* out = OUT ? (a.state && seg == a.pl.nseg - 1 ? a.state + row0 * S : nullptr) : a.scratch + (seg * S) * rows + row0;
    if (out) {
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            float lo, hi;
            up2(s2[s], lo, hi);
            if (s < S) {
                if (OUT) { out[s] = lo; out[S + s] = hi; }
                else { out[s * rows] = lo; out[s * rows + 1] = hi; }
            }
        }
    }
}

// the staged kernels take bf16 / fp16 rows whose q, k, v are neighbours, 128 channels at a time
static bool tma_path(const vtx_fused_iir_params* p) {
    return (p->io_dtype == VTX_BF16 || p->io_dtype == VTX_F16) && !p->modal.theta && p->layout == VTX_QKV_INTERLEAVED &&
           p->D % TC == 0 && reinterpret_cast<uintptr_t>(p->u) % 16 == 0 && (p->u_stride_l * 2) % 16 == 0 &&
           (p->u_stride_b * 2) % 16 == 0 && p->L < ((int64_t)1 << 31) && p->B < 65536;
}
// ... two channels per thread: 256 channels at a time, no featurizer bias, output rows on 4-byte boundaries
static bool tma2_path(const vtx_fused_iir_params* p) {
    return tma_path(p) && p->D % TC2 == 0 && !p->b3 && reinterpret_cast<uintptr_t>(p->y) % 4 == 0 && p->y_stride_l % 2 == 0 &&
           p->y_stride_b % 2 == 0;
}

// Segments for the staged kernels.  CTAs of a launch take the same time and run in waves of (SMs x resident CTAs), so
// the cost of a plan is counted in waves: phase C over all segments, phase A over all but the last, each CTA paying
// a fixed set-up worth ~30 samples.  One segment means no phase A and no carries at all.  Either phase can run one
// channel per thread (128 channels per CTA) or two (256 per CTA, fewer resident CTAs): per sample a CTA then takes
// (issue cycles per warp x warps per scheduler) = C 67 x 4, A 33 x 5, C pairs 103 x 3, A pairs 53 x 4, i.e. 1, 0.62,
// 1.15 and 0.79 in units of the first.  Pairs move more channels per cycle when their CTAs fill the machine, fewer when
// they leave it half empty (B=16, L=8192, D=4096 as one segment: 256 CTAs on 444 places), so the plan tries both.
static Plan plan_staged(int64_t B, int64_t L, int64_t D, bool have_scratch, bool pairs_ok) {
    Plan best{1, L, 0, 0};
    double best_cost = 0;
    const int64_t max_seg = !have_scratch ? 1 : (L / 64 < 1 ? 1 : (L / 64 > 4096 ? 4096 : L / 64));
    for (int pc = 0; pc <= (pairs_ok ? 1 : 0); ++pc) {
        for (int pa = 0; pa <= (pairs_ok ? 1 : 0); ++pa) {
            const int64_t base_c = B * (D / (pc ? TC2 : TC)), base_a = B * (D / (pa ? TC2 : TC));
            const int64_t slots_c = (int64_t)kNumSMs * (pc ? MINB2_C : MINB_C), slots_a = (int64_t)kNumSMs * (pa ? MINB2_A : MINB_A);
            const double tc = pc ? 1.15 : 1.0, ta = pa ? 0.79 : 0.62;
            for (int64_t n = 1; n <= max_seg; ++n) {
                const int64_t seg = ceil_div<int64_t>(ceil_div<int64_t>(L, n), (int64_t)RS) * RS;
                const int64_t nseg = ceil_div<int64_t>(L, seg);
                if (nseg != n) continue;
                const double cost = (double)ceil_div<int64_t>(base_c * nseg, slots_c) * tc * (double)(seg + 32) +
                                    (nseg > 1 ? (double)ceil_div<int64_t>(base_a * (nseg - 1), slots_a) * ta * (double)(seg + 32) +
                                                    4.0 * (double)nseg        /* carry scan */
                                              : 0.0);
                if (best_cost == 0 || cost < best_cost) { best_cost = cost; best = Plan{nseg, seg, pa, pc}; }
            }
        }
    }
    return best;
}

static bool tma_path(const vtx_fused_iir_params* p);
static bool tma2_path(const vtx_fused_iir_params* p);

int64_t scratch_bytes(const vtx_fused_iir_params* p) {
    const Plan pl = tma_path(p) ? plan_staged(p->B, p->L, p->D, true, tma2_path(p)) : plan(p->B, p->L, p->D, true);
    if (pl.nseg <= 1) return 0;
    return p->B * p->D * pl.nseg * p->modal.S * (p->modal.theta ? 2 : 1) * (int64_t)sizeof(float);
}

int fwd(const vtx_fused_iir_params* p, cudaStream_t stream) {
    VTX_REQUIRE(p->K3 == 3, VTX_ERR_UNSUPPORTED, "fused_iir: needs a 3-tap featurizer (got %lld taps)", (long long)p->K3);
    VTX_REQUIRE(p->modal.S <= NS, VTX_ERR_UNSUPPORTED, "fused_iir: state size %lld > %d", (long long)p->modal.S, NS);
    VTX_REQUIRE(p->D % p->modal.G == 0, VTX_ERR_BAD_ARG, "fused_iir: D not a multiple of the number of modal systems");
    VTX_REQUIRE(p->u_hist_rows == 0 || (p->u_hist_rows >= 2 && !p->fir_state_in), VTX_ERR_BAD_ARG,
                "fused_iir: u_hist_rows must be 0 or >= 2, and excludes fir_state_in");
    VTX_REQUIRE(valid_dtype(p->w3_dtype) && (!p->b3 || valid_dtype(p->b3_dtype)) && (!p->bias || valid_dtype(p->bias_dtype)) &&
                    (!p->fir_state_in || valid_dtype(p->fir_state_dtype)),
                VTX_ERR_BAD_ARG, "fused_iir: bad parameter dtype");
    Args a{};
    a.u = p->u; a.sb = p->u_stride_b; a.sl = p->u_stride_l;
    a.w3 = p->w3; a.w3_dtype = p->w3_dtype; a.b3 = p->b3; a.b3_dtype = p->b3_dtype;
    a.m = p->modal; a.bias = p->bias; a.bias_dtype = p->bias_dtype;
    a.y = p->y; a.ysb = p->y_stride_b; a.ysl = p->y_stride_l;
    a.state = p->state; a.state_in = p->state_in; a.fs_in = p->fir_state_in; a.fs_dtype = p->fir_state_dtype;
    a.hist_rows = p->u_hist_rows;
    a.scratch = static_cast<float*>(p->scratch);
    a.B = p->B; a.L = p->L; a.D = p->D;
    a.map.layout = (int)p->layout; a.map.flip = p->flip_x1x2 != 0; a.map.D = p->D; a.map.hd = p->D;
    if (p->layout == VTX_QKV_COLUMN_SPLIT) {
        VTX_REQUIRE(p->num_heads > 0 && p->D % p->num_heads == 0, VTX_ERR_BAD_ARG, "fused_iir: bad num_heads");
        a.map.hd = p->D / p->num_heads;
    }
    a.pl = tma_path(p) ? plan_staged(p->B, p->L, p->D, p->scratch != nullptr, tma2_path(p))
                       : plan(p->B, p->L, p->D, p->scratch != nullptr);
    const bool cplx = p->modal.theta != nullptr;
    const int64_t n = p->B * p->D * a.pl.nseg;
    VTX_REQUIRE(ceil_div<int64_t>(n, THREADS) < ((int64_t)1 << 31), VTX_ERR_UNSUPPORTED, "fused_iir: problem too large");
    const unsigned blocks = (unsigned)ceil_div<int64_t>(n, THREADS);
    if (tma_path(p)) {
        CUtensorMap tmu;
        if (int rc = make_tmap_3d(&tmu, p->u, p->io_dtype, 3 * p->D, p->L, p->B, p->u_stride_l, p->u_stride_b, 3 * 64, RS, 0,
                                  "fused_iir"))
            return rc;
        const int64_t per_seg = p->B * (p->D / TC);
        VTX_REQUIRE(per_seg * a.pl.nseg < ((int64_t)1 << 31), VTX_ERR_UNSUPPORTED, "fused_iir: problem too large");
        const bool flip = a.map.flip != 0;
        const unsigned ga1 = (unsigned)(per_seg * (a.pl.nseg - 1)), gc1 = (unsigned)(per_seg * a.pl.nseg);
        const unsigned ga2 = (unsigned)(p->B * (p->D / TC2) * (a.pl.nseg - 1)), gc2 = (unsigned)(p->B * (p->D / TC2) * a.pl.nseg);
#define VTX_LICC_STAGED(T)                                                                                       \
    do {                                                                                                         \
        if (a.pl.nseg > 1) {                                                                                     \
            if (a.pl.pairs_a && flip) licc_tma2_kernel<T, false, true, MINB2_A><<<ga2, TTHREADS, 0, stream>>>(tmu, a);       \
            else if (a.pl.pairs_a) licc_tma2_kernel<T, false, false, MINB2_A><<<ga2, TTHREADS, 0, stream>>>(tmu, a);         \
            else licc_tma_kernel<T, false, MINB_A><<<ga1, TTHREADS, 0, stream>>>(tmu, a);                        \
            const int64_t nc = p->B * p->D * p->modal.S;                                                         \
            licc_carry_kernel<false><<<(unsigned)ceil_div<int64_t>(nc, 128), 128, 0, stream>>>(a);               \
        }                                                                                                        \
        if (a.pl.pairs_c && flip) licc_tma2_kernel<T, true, true, MINB2_C><<<gc2, TTHREADS, 0, stream>>>(tmu, a);            \
        else if (a.pl.pairs_c) licc_tma2_kernel<T, true, false, MINB2_C><<<gc2, TTHREADS, 0, stream>>>(tmu, a);              \
        else licc_tma_kernel<T, true, MINB_C><<<gc1, TTHREADS, 0, stream>>>(tmu, a);                             \
    } while (0)
        if (p->io_dtype == VTX_BF16) VTX_LICC_STAGED(__nv_bfloat16);
        else VTX_LICC_STAGED(__half);
#undef VTX_LICC_STAGED
        return check_launch("fused_iir", a.pl.nseg > 1 ? 3 : 1);
    }
    VTX_DISPATCH_IO(p->io_dtype, T, {
        if (a.pl.nseg > 1) {
            const unsigned ablocks = (unsigned)ceil_div<int64_t>(p->B * p->D * (a.pl.nseg - 1), THREADS);
            if (cplx) licc_segment_state_kernel<T, true><<<ablocks, THREADS, 0, stream>>>(a);
            else licc_segment_state_kernel<T, false><<<ablocks, THREADS, 0, stream>>>(a);
            const int64_t nc = p->B * p->D * p->modal.S;
            if (cplx) licc_carry_kernel<true><<<(unsigned)ceil_div<int64_t>(nc, 128), 128, 0, stream>>>(a);
            else licc_carry_kernel<false><<<(unsigned)ceil_div<int64_t>(nc, 128), 128, 0, stream>>>(a);
        }
        const bool inter = p->layout == VTX_QKV_INTERLEAVED;
        if (cplx && inter) licc_output_kernel<T, true, true><<<blocks, THREADS, 0, stream>>>(a);
        else if (cplx) licc_output_kernel<T, true, false><<<blocks, THREADS, 0, stream>>>(a);
        else if (inter) licc_output_kernel<T, false, true><<<blocks, THREADS, 0, stream>>>(a);
        else licc_output_kernel<T, false, false><<<blocks, THREADS, 0, stream>>>(a);
    });
    return check_launch("fused_iir", a.pl.nseg > 1 ? 3 : 1);
}

}  // namespace licc
}  // namespace vtx
