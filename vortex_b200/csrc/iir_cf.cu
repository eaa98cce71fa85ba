// Modal (IIR) long convolution on channel-first tensors, evaluated as the
// recurrence itself:  sigma_s[t] = p_s sigma_s[t-1] + kv[t],
//                     y[t] = q[t] * (sum_s Re(R_s sigma_s[t]) + bias * kv[t]).
// One thread owns one (batch, channel, time segment) and keeps all S <= 16
// states in registers.  When batch*channels alone cannot fill the GPU the
// sequence is cut into segments and the carry is resolved in three phases:
//   A  end state of every segment from a zero start   (reads k, v)
//   B  sequential scan over the segments of a row     (tiny)
//   C  recurrence from the true start state, outputs  (reads q, k, v, writes y)
// With one segment per row only phase C runs.  The state after the last token
// (what the reference extracts with 2*S extra FFTs) is a by-product of C.
#include "common.cuh"

namespace vtx {

constexpr int IS = 16;        // states held per thread (shorter systems are padded with p = R = 0)
constexpr int ITHREADS = 128;

struct IirPlan {
    int64_t nseg, seg_len;
};

__host__ __device__ inline IirPlan iir_plan(int64_t B, int64_t L, int64_t D) {
    IirPlan pl;
    int64_t rows = B * D, nseg = 1;
    const int64_t want = (int64_t)kNumSMs * 1024;
    while (rows * nseg < want && L / (nseg * 2) >= 512) nseg *= 2;
    int64_t seg = (L + nseg - 1) / nseg;
    seg = (seg + 15) / 16 * 16;          // keeps 16-byte vector loads aligned inside a row
    pl.nseg = (L + seg - 1) / seg;
    pl.seg_len = seg;
    return pl;
}

template <bool CPLX>
struct Modes {
    float pr[IS], pi[IS], rr[IS], ri[IS];
    __device__ __forceinline__ void load(const vtx_modal_params& m, int64_t g) {
#pragma unroll
        for (int s = 0; s < IS; ++s) {
            pr[s] = pi[s] = rr[s] = ri[s] = 0.f;
            if (s < m.S) {
                float mag = expf(static_cast<const float*>(m.log_poles)[g * m.S + s]);
                rr[s] = static_cast<const float*>(m.res_re)[g * m.S + s];
                if (CPLX) {
                    float sn, cs;
                    sincosf(static_cast<const float*>(m.theta)[g * m.S + s], &sn, &cs);
                    pr[s] = mag * cs; pi[s] = mag * sn;
                    ri[s] = m.res_im ? static_cast<const float*>(m.res_im)[g * m.S + s] : 0.f;
                } else {
                    pr[s] = mag;
                }
            }
        }
    }
};

template <bool CPLX>
struct State {
    float re[IS], im[IS];
    __device__ __forceinline__ void zero() {
#pragma unroll
        for (int s = 0; s < IS; ++s) re[s] = im[s] = 0.f;
    }
    // sigma <- p*sigma + x ; returns sum_s Re(R sigma)
    __device__ __forceinline__ float step(const Modes<CPLX>& m, float x) {
        float acc = 0.f;
#pragma unroll
        for (int s = 0; s < IS; ++s) {
            if (CPLX) {
                float nr = fmaf(m.pr[s], re[s], fmaf(-m.pi[s], im[s], x));
                float ni = fmaf(m.pr[s], im[s], m.pi[s] * re[s]);
                re[s] = nr; im[s] = ni;
                acc = fmaf(m.rr[s], nr, fmaf(-m.ri[s], ni, acc));
            } else {
                re[s] = fmaf(m.pr[s], re[s], x);
                acc = fmaf(m.rr[s], re[s], acc);
            }
        }
        return acc;
    }
    __device__ __forceinline__ void advance(const Modes<CPLX>& m, float x) {
#pragma unroll
        for (int s = 0; s < IS; ++s) {
            if (CPLX) {
                float nr = fmaf(m.pr[s], re[s], fmaf(-m.pi[s], im[s], x));
                float ni = fmaf(m.pr[s], im[s], m.pi[s] * re[s]);
                re[s] = nr; im[s] = ni;
            } else {
                re[s] = fmaf(m.pr[s], re[s], x);
            }
        }
    }
};

template <typename T> struct Vec { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, bool vec_ok, int64_t n_valid, float (&out)[Vec<T>::N]) {
    constexpr int N = Vec<T>::N;
    if (vec_ok && n_valid >= N) {
        uint4 raw = *reinterpret_cast<const uint4*>(p);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int i = 0; i < N; ++i) out[i] = to_f32<T>(e[i]);
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) out[i] = i < n_valid ? to_f32<T>(p[i]) : 0.f;
    }
}

// phase 0: thread -> (row, segment).  Segment index is the slow one so that the threads of a warp
// sit on neighbouring channels of the same segment.
struct Work {
    int64_t b, d, seg, t0, t1;
    bool valid;
};
__device__ __forceinline__ Work iir_work(const vtx_iir_params& p, const IirPlan& pl) {
    Work w;
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t rows = p.B * p.D;
    w.valid = i < rows * pl.nseg;
    int64_t row = i % rows;
    w.seg = i / rows;
    w.b = row / p.D;
    w.d = row % p.D;
    w.t0 = w.seg * pl.seg_len;
    w.t1 = w.t0 + pl.seg_len < p.L ? w.t0 + pl.seg_len : p.L;
    return w;
}

template <typename T, bool CPLX>
__global__ void __launch_bounds__(ITHREADS) iir_segment_state_kernel(vtx_iir_params p, IirPlan pl) {
    Work w = iir_work(p, pl);
    if (!w.valid || w.seg == pl.nseg - 1) return;   // the last segment's end state is not a carry
    constexpr int N = Vec<T>::N;
    Modes<CPLX> m;
    m.load(p.modal, w.d / (p.D / p.modal.G));
    State<CPLX> st;
    st.zero();
    const int64_t hn = w.d / p.head_dim, hj = w.d % p.head_dim;
    const T* k = static_cast<const T*>(p.k) + w.b * p.k_stride_b + hn * p.k_stride_h + hj * p.k_stride_d;
    const T* v = static_cast<const T*>(p.v) + w.b * p.v_stride_b + hn * p.v_stride_h + hj * p.v_stride_d;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) == 0;
    for (int64_t t = w.t0; t < w.t1; t += N) {
        float kk[N], vv[N];
        load_vec<T>(k + t, vec_ok, w.t1 - t, kk);
        load_vec<T>(v + t, vec_ok, w.t1 - t, vv);
#pragma unroll
        for (int i = 0; i < N; ++i) {
            if (t + i < w.t1) {
                float x = kk[i] * vv[i];
                if (p.round_kv) x = round_io<T>(x);
                st.advance(m, x);
            }
        }
    }
    const int S = (int)p.modal.S;
    float* out = static_cast<float*>(p.scratch) + ((w.b * p.D + w.d) * pl.nseg + w.seg) * S * (CPLX ? 2 : 1);
    for (int s = 0; s < S; ++s) {
        if (CPLX) { out[2 * s] = st.re[s]; out[2 * s + 1] = st.im[s]; }
        else out[s] = st.re[s];
    }
}

// After this kernel scratch[row][seg] holds the state at the START of segment seg.
template <bool CPLX>
__global__ void iir_carry_kernel(vtx_iir_params p, IirPlan pl) {
    const int S = (int)p.modal.S;
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.B * p.D * S) return;
    int s = (int)(i % S);
    int64_t row = i / S;
    int64_t d = row % p.D, g = d / (p.D / p.modal.G);
    // p^seg_len in polar form
    float lam = static_cast<const float*>(p.modal.log_poles)[g * S + s];
    float mag = expf(lam * (float)pl.seg_len), pr = mag, pi = 0.f;
    if (CPLX) {
        double a = (double)static_cast<const float*>(p.modal.theta)[g * S + s] * (double)pl.seg_len;
        a -= 6.283185307179586 * floor(a / 6.283185307179586);
        float sn, cs;
        sincosf((float)a, &sn, &cs);
        pr = mag * cs; pi = mag * sn;
    }
    float* base = static_cast<float*>(p.scratch) + row * pl.nseg * S * (CPLX ? 2 : 1);
    float cr = 0.f, ci = 0.f;
    for (int64_t seg = 0; seg < pl.nseg; ++seg) {
        float* e = base + seg * S * (CPLX ? 2 : 1) + (CPLX ? 2 * s : s);
        float er = e[0], ei = CPLX ? e[1] : 0.f;   // end state of this segment from a zero start
        e[0] = cr;
        if (CPLX) e[1] = ci;
        float nr = pr * cr - pi * ci + er;
        float ni = pr * ci + pi * cr + ei;
        cr = nr; ci = ni;
    }
}

template <typename T, bool CPLX>
__global__ void __launch_bounds__(ITHREADS) iir_output_kernel(vtx_iir_params p, IirPlan pl) {
    Work w = iir_work(p, pl);
    if (!w.valid) return;
    constexpr int N = Vec<T>::N;
    const int S = (int)p.modal.S;
    Modes<CPLX> m;
    m.load(p.modal, w.d / (p.D / p.modal.G));
    State<CPLX> st;
    st.zero();
    if (pl.nseg > 1) {
        const float* in = static_cast<const float*>(p.scratch) +
                          ((w.b * p.D + w.d) * pl.nseg + w.seg) * S * (CPLX ? 2 : 1);
        for (int s = 0; s < S; ++s) {
            if (CPLX) { st.re[s] = in[2 * s]; st.im[s] = in[2 * s + 1]; }
            else st.re[s] = in[s];
        }
    }
    const int64_t hn = w.d / p.head_dim, hj = w.d % p.head_dim;
    const T* q = static_cast<const T*>(p.q) + w.b * p.q_stride_b + hn * p.q_stride_h + hj * p.q_stride_d;
    const T* k = static_cast<const T*>(p.k) + w.b * p.k_stride_b + hn * p.k_stride_h + hj * p.k_stride_d;
    const T* v = static_cast<const T*>(p.v) + w.b * p.v_stride_b + hn * p.v_stride_h + hj * p.v_stride_d;
    T* y = static_cast<T*>(p.y) + w.b * p.y_stride_b + w.d * p.y_stride_d;
    const bool vec_ok =
        ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) == 0;
    const bool vec_st = p.y_stride_l == 1 && (reinterpret_cast<uintptr_t>(y) & 15) == 0;
    const float bias = p.bias ? ld_param(p.bias, p.bias_dtype, w.d) : 0.f;
    for (int64_t t = w.t0; t < w.t1; t += N) {
        float qq[N], kk[N], vv[N];
        load_vec<T>(q + t, vec_ok, w.t1 - t, qq);
        load_vec<T>(k + t, vec_ok, w.t1 - t, kk);
        load_vec<T>(v + t, vec_ok, w.t1 - t, vv);
        alignas(16) T out[N];
#pragma unroll
        for (int i = 0; i < N; ++i) {
            if (t + i < w.t1) {
                float x = kk[i] * vv[i];
                if (p.round_kv) x = round_io<T>(x);
                float conv = round_io<T>(st.step(m, x));
                float z = p.round_kv ? round_io<T>(conv + round_io<T>(bias * x)) : fmaf(bias, x, conv);
                out[i] = from_f32<T>(z * qq[i]);
            }
        }
        if (vec_st && w.t1 - t >= N) {
            *reinterpret_cast<uint4*>(y + t) = *reinterpret_cast<const uint4*>(out);
        } else {
            for (int i = 0; i < N && t + i < w.t1; ++i) y[(t + i) * p.y_stride_l] = out[i];
        }
    }
    if (p.state && w.seg == pl.nseg - 1) {
        float* so = p.state + (w.b * p.D + w.d) * S * (CPLX ? 2 : 1);
        for (int s = 0; s < S; ++s) {
            if (CPLX) { so[2 * s] = st.re[s]; so[2 * s + 1] = st.im[s]; }
            else so[s] = st.re[s];
        }
    }
}

// The reference's legacy recurrent prefill (vortex/model/engine.py:473-504), step for step: complex poles and
// residues given as (re, im) pairs, the state kept in the I/O dtype (the reference builds it from x1*v, so with bf16
// activations every update is rounded to bf16), and the real part updated in place BEFORE the imaginary part reads
// it:   re' = pr re - pi im + x ;  im' = pr im + pi re'   (not a complex product: that is what the reference
// computes, and its cached state continues from it).  Every product, difference and sum is rounded on its own, as
// the reference's separate tensor operations are.  out[t] = sum_s Re(R_s) re_s[t] in the I/O dtype, then the same
// skip term and gate as the FFT branch.  One thread walks one (batch, channel) row: a compatibility path.
// modal.log_poles holds Re(p), modal.theta Im(p), modal.res_re Re(R), all fp32 [G, S].
template <typename T>
__global__ void __launch_bounds__(ITHREADS) iir_recurrence_kernel(vtx_iir_params p) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.B * p.D) return;
    const int64_t b = i / p.D, d = i % p.D, g = d / (p.D / p.modal.G);
    const int S = (int)p.modal.S;
    float pr[IS], pi[IS], rr[IS], re[IS], im[IS];
#pragma unroll
    for (int s = 0; s < IS; ++s) {
        pr[s] = pi[s] = rr[s] = re[s] = im[s] = 0.f;
        if (s < S) {
            pr[s] = static_cast<const float*>(p.modal.log_poles)[g * S + s];
            pi[s] = static_cast<const float*>(p.modal.theta)[g * S + s];
            rr[s] = static_cast<const float*>(p.modal.res_re)[g * S + s];
        }
    }
    const int64_t hn = d / p.head_dim, hj = d % p.head_dim;
    const T* q = static_cast<const T*>(p.q) + b * p.q_stride_b + hn * p.q_stride_h + hj * p.q_stride_d;
    const T* k = static_cast<const T*>(p.k) + b * p.k_stride_b + hn * p.k_stride_h + hj * p.k_stride_d;
    const T* v = static_cast<const T*>(p.v) + b * p.v_stride_b + hn * p.v_stride_h + hj * p.v_stride_d;
    T* y = static_cast<T*>(p.y) + b * p.y_stride_b + d * p.y_stride_d;
    const float bias = p.bias ? ld_param(p.bias, p.bias_dtype, d) : 0.f;
    for (int64_t t = 0; t < p.L; ++t) {
        const float x = round_io<T>(to_f32<T>(k[t]) * to_f32<T>(v[t]));
        float acc = 0.f;
#pragma unroll
        for (int s = 0; s < IS; ++s) {
            const float nr = round_io<T>(__fadd_rn(__fsub_rn(__fmul_rn(pr[s], re[s]), __fmul_rn(pi[s], im[s])), x));
            const float ni = round_io<T>(__fadd_rn(__fmul_rn(pr[s], im[s]), __fmul_rn(pi[s], nr)));
            re[s] = nr; im[s] = ni;
            acc = __fadd_rn(acc, __fmul_rn(rr[s], nr));
        }
        const float conv = round_io<T>(acc);
        const float z = round_io<T>(conv + round_io<T>(bias * x));
        y[t * p.y_stride_l] = from_f32<T>(z * to_f32<T>(q[t]));
    }
    if (p.state) {
        float* so = p.state + (b * p.D + d) * S * 2;
        for (int s = 0; s < S; ++s) { so[2 * s] = re[s]; so[2 * s + 1] = im[s]; }
    }
}

__global__ void modal_filter_kernel(vtx_modal_params m, float* h, int64_t L) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= m.G * L) return;
    int64_t g = i / L, t = i % L;
    const float* lp = static_cast<const float*>(m.log_poles) + g * m.S;
    const float* rr = static_cast<const float*>(m.res_re) + g * m.S;
    float acc = 0.f;
    for (int s = 0; s < m.S; ++s) {
        float mag = expf(lp[s] * (float)t);
        if (m.theta) {
            double a = (double)static_cast<const float*>(m.theta)[g * m.S + s] * (double)t;
            a -= 6.283185307179586 * floor(a / 6.283185307179586);
            float sn, cs;
            sincosf((float)a, &sn, &cs);
            float ri = m.res_im ? static_cast<const float*>(m.res_im)[g * m.S + s] : 0.f;
            acc += mag * (rr[s] * cs - ri * sn);
        } else {
            acc += rr[s] * mag;
        }
    }
    h[i] = acc;
}

static int check_modal(const vtx_modal_params& m, const char* who) {
    VTX_REQUIRE(m.log_poles && m.res_re, VTX_ERR_BAD_ARG, "%s: null poles/residues", who);
    VTX_REQUIRE(m.G > 0 && m.S > 0, VTX_ERR_BAD_ARG, "%s: G and S must be positive", who);
    VTX_REQUIRE(!m.res_im || m.theta, VTX_ERR_BAD_ARG, "%s: complex residues need complex poles", who);
    return VTX_OK;
}

}  // namespace vtx

extern "C" int vtx_modal_filter(const vtx_modal_params* m, float* h, int64_t L, void* stream) {
    using namespace vtx;
    VTX_REQUIRE(m && h && L > 0, VTX_ERR_BAD_ARG, "modal_filter: bad argument");
    if (int rc = check_modal(*m, "modal_filter")) return rc;
    int64_t n = m->G * L;
    modal_filter_kernel<<<(unsigned)ceil_div<int64_t>(n, 256), 256, 0, (cudaStream_t)stream>>>(*m, h, L);
    return check_launch("modal_filter");
}

extern "C" int64_t vtx_iir_scratch_bytes(int64_t B, int64_t L, int64_t D, int64_t S, int64_t complex_poles) {
    if (B <= 0 || L <= 0 || D <= 0 || S <= 0) return 0;
    vtx::IirPlan pl = vtx::iir_plan(B, L, D);
    if (pl.nseg <= 1) return 0;
    return B * D * pl.nseg * S * (complex_poles ? 2 : 1) * (int64_t)sizeof(float);
}

extern "C" int vtx_iir_fwd(const vtx_iir_params* p, void* stream) {
    using namespace vtx;
    VTX_REQUIRE(p && p->q && p->k && p->v && p->y, VTX_ERR_BAD_ARG, "iir: null pointer");
    VTX_REQUIRE(p->B > 0 && p->L > 0 && p->D > 0, VTX_ERR_BAD_ARG, "iir: sizes must be positive");
    VTX_REQUIRE(p->head_dim > 0 && p->D % p->head_dim == 0, VTX_ERR_BAD_ARG, "iir: head_dim must divide D");
    if (int rc = check_modal(p->modal, "iir")) return rc;
    VTX_REQUIRE(p->D % p->modal.G == 0, VTX_ERR_BAD_ARG, "iir: D not a multiple of the number of modal systems");
    VTX_REQUIRE(p->modal.S <= IS, VTX_ERR_UNSUPPORTED, "iir: state size %lld > %d", (long long)p->modal.S, IS);
    const bool cplx = p->modal.theta != nullptr;
    IirPlan pl = iir_plan(p->B, p->L, p->D);
    VTX_REQUIRE(pl.nseg == 1 || p->scratch, VTX_ERR_BAD_ARG, "iir: scratch needed (%lld bytes)",
                (long long)vtx_iir_scratch_bytes(p->B, p->L, p->D, p->modal.S, cplx));
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t n = p->B * p->D * pl.nseg;
    const unsigned blocks = (unsigned)ceil_div<int64_t>(n, ITHREADS);
    VTX_DISPATCH_IO(p->io_dtype, T, {
        if (pl.nseg > 1) {
            if (cplx) iir_segment_state_kernel<T, true><<<blocks, ITHREADS, 0, s>>>(*p, pl);
            else iir_segment_state_kernel<T, false><<<blocks, ITHREADS, 0, s>>>(*p, pl);
            const int64_t nc = p->B * p->D * p->modal.S;
            if (cplx) iir_carry_kernel<true><<<(unsigned)ceil_div<int64_t>(nc, 128), 128, 0, s>>>(*p, pl);
            else iir_carry_kernel<false><<<(unsigned)ceil_div<int64_t>(nc, 128), 128, 0, s>>>(*p, pl);
        }
        if (cplx) iir_output_kernel<T, true><<<blocks, ITHREADS, 0, s>>>(*p, pl);
        else iir_output_kernel<T, false><<<blocks, ITHREADS, 0, s>>>(*p, pl);
    });
    return check_launch("iir", pl.nseg > 1 ? 3 : 1);
}

extern "C" int vtx_iir_recurrence_fwd(const vtx_iir_params* p, void* stream) {
    using namespace vtx;
    VTX_REQUIRE(p && p->q && p->k && p->v && p->y, VTX_ERR_BAD_ARG, "iir(recurrence): null pointer");
    VTX_REQUIRE(p->B > 0 && p->L > 0 && p->D > 0, VTX_ERR_BAD_ARG, "iir(recurrence): sizes must be positive");
    VTX_REQUIRE(p->head_dim > 0 && p->D % p->head_dim == 0, VTX_ERR_BAD_ARG, "iir(recurrence): head_dim must divide D");
    VTX_REQUIRE(p->modal.log_poles && p->modal.theta && p->modal.res_re, VTX_ERR_BAD_ARG,
                "iir(recurrence): Re(p), Im(p) and Re(R) are needed");
    VTX_REQUIRE(p->modal.G > 0 && p->modal.S > 0 && p->D % p->modal.G == 0, VTX_ERR_BAD_ARG,
                "iir(recurrence): D not a multiple of the number of modal systems");
    VTX_REQUIRE(p->modal.S <= IS, VTX_ERR_UNSUPPORTED, "iir(recurrence): state size %lld > %d", (long long)p->modal.S, IS);
    const unsigned blocks = (unsigned)ceil_div<int64_t>(p->B * p->D, ITHREADS);
    VTX_DISPATCH_IO(p->io_dtype, T, { iir_recurrence_kernel<T><<<blocks, ITHREADS, 0, (cudaStream_t)stream>>>(*p); });
    return check_launch("iir(recurrence)");
}

// ---------------------------------------------------------------------------------------------------
// vtx_iir_fwd_noalloc: the same modal long convolution for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc (or torch's allocator) at the point where they need the
// operator: an inference server that handed all free HBM to its KV-cache pool at start-up, a plain C caller
// that has no allocator of its own on the device, or code in the middle of a latency-critical loop where an
// allocation could stall or fail.  vtx_iir_fwd asks such a caller for a scratch buffer (the carries between
// time segments).  This variant brings its own: a fixed array in device global memory that is part of the
// library image, so every GPU that loads the library sets VTX_IIR_STATIC_SCRATCH_BYTES aside until the
// process exits.  Inputs and outputs are still the caller's.
//
// * Sizes whose carries do not fit (vtx_iir_scratch_bytes(...) > VTX_IIR_STATIC_SCRATCH_BYTES) are refused
//   with VTX_ERR_UNSUPPORTED; nothing is launched.
// * The first call on a device looks the array's device address up (cudaGetSymbolAddress with that device
//   current -- the array's name is only a host-side handle, never a pointer a kernel could use) and keeps it
//   per device.  Make that first call outside any stream capture -- and during start-up, before the host
//   commits the rest of the device memory: with CUDA's default lazy module loading the array is reserved on a
//   device when this file's module is first used there (this call, vtx_iir_fwd or vtx_modal_filter), not when
//   the library is loaded.
// * All calls share the one array and it keeps whatever the last call left in it.  Nothing in it has to be
//   zero at the start: every word a call reads was written earlier by the same call, except the carry slot of
//   the last segment, whose value is computed but never used.  Two calls that overlap on the GPU (different
//   streams, or different host threads) race on the array: serialise them.
// * No cudaMalloc / cudaFree / allocating library routine is called on this path.
constexpr size_t kIirStaticScratchBytes = VTX_IIR_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_iir_static_scratch[kIirStaticScratchBytes];

extern "C" int vtx_iir_fwd_noalloc(const vtx_iir_params* p, void* stream) {
    using namespace vtx;
    VTX_REQUIRE(p, VTX_ERR_BAD_ARG, "iir(noalloc): null parameter block");
    VTX_REQUIRE(p->B > 0 && p->L > 0 && p->D > 0 && p->modal.S > 0, VTX_ERR_BAD_ARG, "iir(noalloc): sizes must be positive");
    const int64_t need = vtx_iir_scratch_bytes(p->B, p->L, p->D, p->modal.S, p->modal.theta != nullptr);
    VTX_REQUIRE(need <= (int64_t)kIirStaticScratchBytes, VTX_ERR_UNSUPPORTED,
                "iir(noalloc): this size needs %lld bytes of carries, the built-in scratch holds %lld; "
                "use vtx_iir_fwd with a caller-provided buffer",
                (long long)need, (long long)kIirStaticScratchBytes);
    constexpr int kMaxDevices = 64;
    static void* dev_ptr[kMaxDevices] = {nullptr};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
        return fail(VTX_ERR_LAUNCH, "iir(noalloc): cudaGetDevice: %s", e == cudaSuccess ? "device index out of range" : cudaGetErrorString(e));
    if (!dev_ptr[dev]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_iir_static_scratch);
        if (e != cudaSuccess || !ptr) return fail(VTX_ERR_LAUNCH, "iir(noalloc): cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        dev_ptr[dev] = ptr;
    }
    vtx_iir_params q = *p;
    q.scratch = dev_ptr[dev];
    return vtx_iir_fwd(&q, stream);
}
