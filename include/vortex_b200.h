/*
 * vortex_b200 -- C ABI of the B200 (sm_100a) Hyena convolution kernels.
 *
 * Every entry point takes plain device pointers, 64-bit sizes/strides and a
 * CUDA stream (passed as void*), returns 0 on success or a negative
 * vtx_status, never throws, never exits and never synchronises the device.
 * Unless stated otherwise an entry point allocates nothing: the caller owns
 * every buffer.  All struct fields are 8 bytes wide so that a binding in any
 * language can mirror the structs without padding rules.
 *
 * "Reference" below means Zymrael/vortex; paths are relative to its root.
 *
 * Tensors.  B batch, L sequence length, D hidden channels, C = 3*D packed
 * projection channels, G filter groups (D % G == 0, blocked sharing:
 * group(d) = d / (D/G)), K filter length, S state size.
 * dtype codes: VTX_F32, VTX_BF16, VTX_F16.  "io" tensors (activations,
 * outputs, prefill caches) share one dtype per call; parameters carry their
 * own dtype code; arithmetic is fp32 unless stated otherwise.
 */
#ifndef VORTEX_B200_H
#define VORTEX_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum vtx_status {
    VTX_OK = 0,
    VTX_ERR_BAD_ARG = -1,      /* null pointer, non-positive size, inconsistent shapes */
    VTX_ERR_UNSUPPORTED = -2,  /* legal request this build has no kernel for           */
    VTX_ERR_ALIGNMENT = -3,    /* pointer or stride not aligned as the kernel needs    */
    VTX_ERR_LAUNCH = -4,       /* CUDA reported an error at launch                     */
    VTX_ERR_DEVICE = -5        /* a kernel set its status word (bounded wait ran out)  */
} vtx_status;

enum { VTX_F32 = 0, VTX_BF16 = 1, VTX_F16 = 2 };

/* How q (reference name x2), k (x1) and v are laid out in the 3*D packed
 * channels of the featurizer output (vortex/model/utils.py:26-85,
 * vortex/model/engine.py:150-158):
 *   SPLIT        q = c[d],   k = c[D+d],   v = c[2D+d]
 *   INTERLEAVED  q = c[3d],  k = c[3d+1],  v = c[3d+2]      (config.interleave)
 *   COLUMN_SPLIT per head n = d / hd, j = d % hd:
 *                q = c[3*hd*n + j], k = c[3*hd*n + hd + j], v = c[3*hd*n + 2*hd + j]
 * flip_x1x2 != 0 swaps q and k afterwards (engine.py:157-158). */
enum { VTX_QKV_SPLIT = 0, VTX_QKV_INTERLEAVED = 1, VTX_QKV_COLUMN_SPLIT = 2 };

/* Tap convention of a causal FIR y[t] = sum_j h[j] x[t - lag(j)]:
 *   XCORR lag(j) = K-1-j  (F.conv1d with left padding, engine.py:197-204; K < 128)
 *   CONV  lag(j) = j      (FFT product, engine.py:38-83,174-187;        K >= 128) */
enum { VTX_TAPS_XCORR = 0, VTX_TAPS_CONV = 1 };

/* Bias handling of the FIR paths (engine.py:78,219-223). */
enum { VTX_BIAS_NONE = 0, VTX_BIAS_ADD = 1, VTX_BIAS_GATED = 2 /* + bias[d] * kv */ };

/* Copies the message of the calling thread's last failed vtx_* call into buf. */
size_t vtx_last_error(char* buf, size_t len);
/* ABI version of this header: major * 1000 + minor.  vtx_abi_version() returns the value the library was
 * built with; a binding compares the two (same major, library minor >= the minor it was written for). */
#define VTX_ABI_VERSION 1005
int64_t vtx_abi_version(void);
/* sizeof() of the parameter structs in declaration order (0 = vtx_featurizer_params, ...),
 * -1 past the end; lets a binding verify that its mirror of a struct has the same size. */
int64_t vtx_struct_size(int64_t which);
/* Reads and clears the device status word that kernels set when one of their bounded waits
 * (mbarrier / TMA completion) ran out.  Synchronous (a small device-to-host copy); meant to be
 * called after the stream was synchronised.  Returns VTX_OK or VTX_ERR_DEVICE. */
int vtx_device_status(void);
/* Kernels launched by this library since it was loaded (all entry points, all threads).  A caller that wants the
 * launches of a region reads it before and after.  No counterpart in the reference. */
int64_t vtx_launch_count(void);
/* Diagnostics: how often a kernel polls a global-memory flag written by another block (the hand-over between the
 * time slices of one long-filter walk) before it gives up, sets the status word and carries on with what it has.
 * 0 restores the default (2^21 polls with a short sleep each, far beyond any real wait).  A tiny value makes the
 * give-up path observable: the launch still ends normally, its output is not valid, vtx_device_status() reports
 * VTX_ERR_DEVICE.  Process-wide; applies to launches made after the call.  No counterpart in the reference. */
int vtx_debug_set_flag_poll_limit(int64_t polls);

/* ------------------------------------------------------------------------
 * Featurizer: depthwise causal FIR of length K <= 8 over the packed
 * projection channels, channel-last in, channel-first out.
 * Replaces HyenaInferenceEngine.parallel_fir(gate=False)
 * (vortex/model/engine.py:131-149,188-227,255-260; caller
 * vortex/model/model.py:233-249) and the width-2..4 kernels
 * causal_conv1d_fwd (vortex/ops/conv/csrc/causal_conv1d.cpp:130-136,
 * causal_conv1d_fwd.cu:44-135,208-346).
 *   z[b,c,t] = sum_j w[c,j] * u[b,t-(K-1)+j,c] (+ bias[c]) (* mask[b,t])
 *   state[b,c,:] = u[b, L-min(L,K-1):L, c]   (pre-convolution input)
 * ------------------------------------------------------------------------ */
typedef struct vtx_featurizer_params {
    const void* u;       int64_t u_stride_b, u_stride_l, u_stride_c; /* logical [B,L,C], element strides */
    const void* w;       int64_t w_dtype;      /* [C,K] contiguous                       */
    const void* bias;    int64_t bias_dtype;   /* [C] or NULL                            */
    const void* mask;    int64_t mask_dtype;   /* [B,L] contiguous or NULL               */
    void* z;                                    /* [B,C,L] contiguous, io dtype           */
    void* state;                                /* [B,C,min(L,K-1)] contiguous or NULL    */
    int64_t B, L, C, K;
    int64_t io_dtype;
} vtx_featurizer_params;
int vtx_featurizer_fwd(const vtx_featurizer_params* p, void* stream);

/* ------------------------------------------------------------------------
 * Gate -> grouped causal FIR -> gate, channel-first.  Any K >= 1, fp32 math
 * on CUDA cores (exact-order accumulation, used for fp32 I/O and as the
 * general path).  Replaces HyenaInferenceEngine.parallel_fir(gate=True)
 * (engine.py:150-159,174-232,255-258; caller model.py:271-291) including
 * fftconv_func (engine.py:38-83), and the hyena_ops forward
 * two_pass_fwd_grouped (vortex/ops/hyena_se/fwd.py:17-310, reference math
 * vortex/ops/hyena_se/ref_fwd.py:80-127).
 *   kv = k*v ; y[b,d,t] = q * ( FIR_h[group(d)](kv)[t] (+bias) ) ;
 *   state[b,d,:] = kv[b,d, L-min(L,K-1):L]
 * q, k, v are three independent strided views [B,D,L] (so the same entry
 * point serves the packed [B,3D,L] tensor in any vtx_qkv layout and the
 * (x, B, C) operands of hyena_ops); their time stride must be 1.  Channel d
 * sits at element offset (d / head_dim) * stride_h + (d % head_dim) * stride_d
 * of its batch row (two-level so that the per-head column split is a view).
 * round_kv != 0 rounds kv to the io dtype before the filter, as the
 * reference does when it materialises x1*v (engine.py:159).
 * ------------------------------------------------------------------------ */
typedef struct vtx_gcg_params {
    const void* q;  int64_t q_stride_b, q_stride_h, q_stride_d;
    const void* k;  int64_t k_stride_b, k_stride_h, k_stride_d;
    const void* v;  int64_t v_stride_b, v_stride_h, v_stride_d;
    int64_t head_dim;                           /* channels per head; D when there is one   */
    const void* h;       int64_t h_dtype;      /* [G,K] contiguous                        */
    const void* bias;    int64_t bias_dtype;   /* [D] or NULL                             */
    const void* mask;    int64_t mask_dtype;   /* [B,L] or NULL                           */
    void* y;             int64_t y_stride_b, y_stride_d, y_stride_l; /* [B,D,L] logical   */
    void* state;                                /* [B,D,min(L,K-1)] contiguous or NULL     */
    int64_t B, L, D, G, K;
    int64_t taps;        /* VTX_TAPS_*   */
    int64_t bias_mode;   /* VTX_BIAS_*   */
    int64_t round_kv;
    int64_t io_dtype;
} vtx_gcg_params;
int vtx_gcg_fwd(const vtx_gcg_params* p, void* stream);

/* The same operator on three CHANNEL-LAST operands q, k, v [B,L,D] (channel stride 1) -- the layout of the reference's
 * hyena_ops kernels, (bs, l, g, dg) with d = g*dg (vortex/ops/hyena_se/fwd.py:56-64).  Replaces two_pass_fwd_grouped
 * (fwd.py:17-310, kernels fwd_kernels.py:268-626) and its reference gcg_fwd_ref_corrected (ref_fwd.py:80-127) for
 * bf16 operands and bf16 filters of up to 128 taps shared by a multiple of 16 channels: one launch of the tcgen05
 * blocked-Toeplitz kernel (no featurizer in front), k*v and the filter output rounded to bf16 where the reference
 * materialises them.  bias_mode: VTX_BIAS_NONE or VTX_BIAS_GATED.  state [B,D,min(L,K-1)] (channel-first, as the
 * caches are) or NULL.  Bases and row pitches 16-byte aligned, y rows 32-byte aligned. */
typedef struct vtx_gcg_cl_params {
    const void* q;  int64_t q_stride_b, q_stride_l;
    const void* k;  int64_t k_stride_b, k_stride_l;
    const void* v;  int64_t v_stride_b, v_stride_l;
    const void* h;       int64_t h_dtype;      /* [G,K] contiguous                        */
    const void* bias;    int64_t bias_dtype;   /* [D] or NULL                             */
    void* y;             int64_t y_stride_b, y_stride_l;
    void* state;                                /* or NULL                                 */
    int64_t B, L, D, G, K;
    int64_t taps, bias_mode;
    int64_t io_dtype;
} vtx_gcg_cl_params;
int vtx_gcg_cl_fwd(const vtx_gcg_cl_params* p, void* stream);

/* Backward of the same operator on channel-last tensors [B,L,D] (channel stride 1): replaces two_pass_bwd_grouped
 * (vortex/ops/hyena_se/bwd.py:11-330, kernels bwd_kernels.py:239,468; restated by gcg_two_pass_chunked_bwd,
 * ref_bwd.py:31-115).  With z = Bg * x, y2 = xcorr(h_g, z) (saved by the forward) and y = C * y2:
 *   dC = dy * y2,   dz = h_g run against time over dy * C,   dx = dz * Bg,   dB = dz * x,
 *   dh32[g,k] += sum over batch, time and the group's channels of (dy * C)[t] z[t - (K-1) + k].
 * dx, dB, dC are contiguous [B,L,D] in the I/O dtype; dh32 is an fp32 [G,K] accumulator the caller zeroes (partial
 * sums are added with atomics: the order, hence the last bits, can differ between runs).  K <= 128; any I/O dtype;
 * fp32 accumulation on the CUDA cores. */
typedef struct vtx_gcg_bwd_params {
    const void* dy;  int64_t dy_stride_b, dy_stride_l;
    const void* x;   int64_t x_stride_b, x_stride_l;
    const void* Bg;  int64_t b_stride_b, b_stride_l;
    const void* C;   int64_t c_stride_b, c_stride_l;
    const void* y2;  int64_t y2_stride_b, y2_stride_l;
    const void* h;   int64_t h_dtype;           /* [G,K] contiguous */
    void* dx; void* dB; void* dC;               /* [B,L,D] contiguous */
    float* dh32;                                /* [G,K] fp32, zeroed by the caller */
    int64_t B, L, D, G, K;
    int64_t io_dtype;
} vtx_gcg_bwd_params;
int vtx_gcg_bwd(const vtx_gcg_bwd_params* p, void* stream);

/* ------------------------------------------------------------------------
 * Fused Hyena FIR block on the projection output, channel-last in and out:
 * featurizer (K3 <= 4) -> q/k/v selection -> k*v -> grouped FIR -> q gate,
 * one pass over HBM.  Fuses model.py:233-291 (HyenaCascade.parallel_forward,
 * both parallel_fir calls and interleave) -- the hyena_se_fwd / hyena_mr_fwd
 * entry points the reference imports but never defines
 * (vortex/model/layers.py:18-21).
 *   u [B,L,3D] -> y [B,L,D]; fir_state [B,3D,min(L,K3-1)];
 *   inner_state [B,D,min(L,K-1)]  (both channel-first, as the caches are)
 * bf16 io with groups of 16 channels and K <= 128 runs as a blocked-Toeplitz contraction on tcgen05
 * (persistent CTAs, Toeplitz operand in TMEM); other dtypes / group sizes with K <= 16 run on CUDA cores
 * with TMA-staged rows.
 * The base address and the row pitch of u and y must be 16-byte aligned.
 * Chunked prefill (a long prompt in pieces; the reference forces it token by token, generation.py:94-101):
 * u_hist_rows = H > 0 says that the H rows BEFORE u[b][0] in memory (same row pitch) are the projection rows
 * that precede this chunk in the sequence; the kernels then read them as the halo of the first outputs
 * instead of zeros.  H must be at least K + 1 (K - 1 taps back plus the 2 rows of the featurizer).  The caches
 * written are then always full: fir_state [B,3D,2], inner_state [B,D,K-1].
 * ------------------------------------------------------------------------ */
typedef struct vtx_fused_fir_params {
    const void* u;       int64_t u_stride_b, u_stride_l;   /* channel stride 1 */
    const void* w3;      int64_t w3_dtype;     /* [3D,K3] featurizer taps                 */
    const void* b3;      int64_t b3_dtype;     /* [3D] featurizer bias or NULL            */
    const void* h;       int64_t h_dtype;      /* [G,K]                                   */
    const void* bias;    int64_t bias_dtype;   /* [D] or NULL                             */
    void* y;             int64_t y_stride_b, y_stride_l;   /* channel stride 1 */
    void* fir_state;                            /* or NULL                                 */
    void* inner_state;                          /* or NULL                                 */
    int64_t B, L, D, G, K3, K;
    int64_t layout, num_heads, flip_x1x2;
    int64_t taps, bias_mode;
    int64_t io_dtype;
    int64_t u_hist_rows;                        /* 0, or >= K + 1 valid rows before u[b][0]  */
} vtx_fused_fir_params;
int vtx_fused_fir_fwd(const vtx_fused_fir_params* p, void* stream);

/* ------------------------------------------------------------------------
 * Modal (IIR) long convolution.
 *
 * vtx_modal_filter materialises h[g,t] = sum_s R[g,s] exp(lambda[g,s] t)
 * (HyenaCascade.compute_filter, model.py:390-398) into fp32 [G,L].
 * With im parts given (complex != 0: lambda = log|p|, theta = arg p,
 * R = Rre + i Rim) it evaluates sum_s Re(R p^t) (model.py:842-848).
 * ------------------------------------------------------------------------ */
typedef struct vtx_modal_params {
    const void* log_poles;   /* fp32 [G,S]  lambda = log|p|                      */
    const void* theta;       /* fp32 [G,S]  arg p, or NULL for real poles        */
    const void* res_re;      /* fp32 [G,S]                                       */
    const void* res_im;      /* fp32 [G,S] or NULL                               */
    int64_t G, S;
} vtx_modal_params;
int vtx_modal_filter(const vtx_modal_params* m, float* h, int64_t L, void* stream);

/* Gate -> modal long convolution -> gate, channel-first, evaluated as the
 * modal recurrence itself (sigma_s[t] = p_s sigma_s[t-1] + kv[t];
 * y = q * (sum_s Re(R_s sigma_s) + bias*kv)) instead of a length-2L FFT;
 * the state after the last token falls out of the same pass.
 * Replaces HyenaInferenceEngine.parallel_iir with its FFT branch
 * (engine.py:262-353,404) and prefill_via_modal_fft (engine.py:525-559).
 *   y [B,D,L] (strided: the engine returns it viewed as [B,L,D]);
 *   state fp32 [B,D,S] (real poles) or [B,D,S,2] (complex), or NULL.
 * scratch: fp32, vtx_iir_scratch_bytes(...) bytes, may be NULL when that is 0.
 * ------------------------------------------------------------------------ */
typedef struct vtx_iir_params {
    const void* q;  int64_t q_stride_b, q_stride_h, q_stride_d;   /* as in vtx_gcg_params */
    const void* k;  int64_t k_stride_b, k_stride_h, k_stride_d;
    const void* v;  int64_t v_stride_b, v_stride_h, v_stride_d;
    int64_t head_dim;
    vtx_modal_params modal;                     /* G must divide D                         */
    const void* bias;    int64_t bias_dtype;   /* [D] skip term or NULL                   */
    void* y;             int64_t y_stride_b, y_stride_d, y_stride_l;
    float* state;
    void* scratch;
    int64_t B, L, D;
    int64_t round_kv;
    int64_t io_dtype;
} vtx_iir_params;
int64_t vtx_iir_scratch_bytes(int64_t B, int64_t L, int64_t D, int64_t S, int64_t complex_poles);
int vtx_iir_fwd(const vtx_iir_params* p, void* stream);

/* The legacy recurrent prefill, HyenaInferenceEngine.prefill_via_direct_recurrence (engine.py:473-504; taken by
 * parallel_iir with prefill_style="recurrence", engine.py:314-321): complex poles and residues as (re, im) pairs,
 * the state held in the I/O dtype and updated in the reference's order (real part first, the imaginary part then
 * reads the NEW real part), y = q * (sum_s Re(R_s) Re(sigma_s) + bias * kv).
 *   modal.log_poles = Re(p), modal.theta = Im(p), modal.res_re = Re(R), fp32 [G,S]; modal.res_im is not read.
 *   state fp32 [B,D,S,2] = (re, im) after the last token, or NULL.  scratch is not used.
 * One thread per (batch, channel) row walks the sequence: a compatibility path, not a fast one. */
int vtx_iir_recurrence_fwd(const vtx_iir_params* p, void* stream);

/* Same operator for callers that cannot allocate device memory where they need it (a server that gave all
 * free HBM to its cache pool, a C host without a device allocator, a latency-critical loop).  It has no
 * counterpart in the reference.  p->scratch is ignored: the segment carries live in an array of
 * VTX_IIR_STATIC_SCRATCH_BYTES that is part of the library image (each GPU that loads the library holds it
 * until exit).  Sizes needing more (see vtx_iir_scratch_bytes) return VTX_ERR_UNSUPPORTED.  The first call on
 * a device resolves the array's device address; make it before any stream capture.  With CUDA's default lazy
 * module loading the array's bytes are reserved on a device when the library's long-convolution module is first
 * used there (this first call, or the first vtx_iir_fwd / vtx_modal_filter), not when the library is loaded: make
 * that call during start-up, BEFORE the host hands the rest of the device memory to its own pools, or the
 * reservation itself can fail with an out-of-memory launch error.  All calls share the
 * array and it keeps the last call's contents (nothing needs clearing); calls that overlap on the GPU race.
 * Calls no cudaMalloc, cudaFree or other allocating routine. */
#define VTX_IIR_STATIC_SCRATCH_BYTES (16u << 20)
int vtx_iir_fwd_noalloc(const vtx_iir_params* p, void* stream);

/* Fused Hyena-LI block on the projection output, channel-last in and out: featurizer (3 taps) -> q/k/v
 * selection -> k*v -> modal long convolution -> (+ bias*kv) -> q gate in ONE pass over the rows (no [B,3D,L]
 * intermediate).  Fuses model.py:233-316 (HyenaCascade.parallel_forward for a long-filter layer: featurizer
 * parallel_fir + parallel_iir with its FFT branch, engine.py:262-353, and the end state of
 * prefill_via_modal_fft, engine.py:525-559) -- the hyena_li_fwd entry point the reference imports but never
 * defines (vortex/model/layers.py:18-21).  Two kernels, chosen by shape:
 *   - bf16 I/O, modal systems of up to 16 poles shared by groups of 16 channels (G * 16 == D), no featurizer
 *     bias; a call that continues an earlier one only when L is a multiple of 384 and its history comes as
 *     u_hist_rows (not fir_state_in): a chunked state-space scan whose Toeplitz, state-input and state-update
 *     contractions run on tcgen05 tensor cores;
 *   - everything else (a modal system per channel as in Evo 2, configs/evo2-7b-8k.yml:11, any G dividing D,
 *     fp32 / fp16 / bf16 I/O, featurizer bias, a call that continues an earlier one): the recurrence itself on
 *     the fp32 pipe, time segments with a carry scan.
 *   u [B,L,3D] -> y [B,L,D]; state fp32 [B,D,S] (real poles) or [B,D,S,2] (complex) after the last token, or NULL.
 * Chunked prefill (what generation.py:94-101 does token by token): state_in is the modal state and
 * fir_state_in [B,3D,2] the featurizer cache (the last two projection rows, packed-channel order) that the
 * call on the previous chunk returned; NULL = start of a sequence.
 * ------------------------------------------------------------------------ */
typedef struct vtx_fused_iir_params {
    const void* u;       int64_t u_stride_b, u_stride_l;   /* channel stride 1 */
    const void* w3;      int64_t w3_dtype;     /* [3D,3] featurizer taps                  */
    const void* b3;      int64_t b3_dtype;     /* [3D] featurizer bias or NULL            */
    vtx_modal_params modal;                     /* G modal systems, G divides D            */
    const void* bias;    int64_t bias_dtype;   /* [D] skip term or NULL                   */
    void* y;             int64_t y_stride_b, y_stride_l;   /* channel stride 1 */
    float* state;                               /* or NULL                                 */
    void* scratch;                              /* vtx_fused_iir_scratch_bytes(p) bytes, 16-byte aligned, or NULL:
                                                   lets a sequence be cut into time segments that run on different
                                                   SMs (without it every channel or group is walked by one thread
                                                   or block from the first sample to the last) */
    int64_t B, L, D, K3;
    int64_t layout, num_heads, flip_x1x2;
    int64_t io_dtype;
    const float* state_in;                      /* modal state to start from, layout of state, or NULL (zero) */
    const void* fir_state_in; int64_t fir_state_dtype;   /* [B,3D,2] rows before the first one, or NULL (zero) */
    int64_t u_hist_rows;                        /* 0, or >= 2: that many rows in front of u in memory (same row pitch)
                                                   are the sequence's preceding projection rows and take the place
                                                   of fir_state_in (which must then be NULL), as in vtx_fused_fir_params */
} vtx_fused_iir_params;
/* Scratch the call described by p can use (p->scratch itself is not read); 0 = none needed. */
int64_t vtx_fused_iir_scratch_bytes(const vtx_fused_iir_params* p);
int vtx_fused_iir_fwd(const vtx_fused_iir_params* p, void* stream);

/* Short depthwise causal convolution of the reference's conv extension (its pybind module
 * local_causal_conv1d_cuda, vortex/ops/conv/csrc/causal_conv1d.cpp:473-477):
 *   vtx_causal_conv1d_fwd    replaces causal_conv1d_fwd    (causal_conv1d.cpp:130-236, causal_conv1d_fwd.cu)
 *   vtx_causal_conv1d_update replaces causal_conv1d_update (causal_conv1d.cpp:382-470, causal_conv1d_update.cu)
 * x, out [B,D,L] of the I/O dtype with element strides (time-contiguous or channel-contiguous, as the reference
 * accepts), weight [D,W] contiguous with W in 2..4, optional bias [D], optional SiLU.
 * fwd: seq_idx int32 [B,L] contiguous (packed sequences: a tap counts only if it has the same index as the
 * output sample), initial_states [B,D,W-1] (samples before the first), final_states [B,D,W-1] written when given.
 * update: conv_state [rows,D,state_len] updated in place; cache_seqlens int32 [B] makes it a circular buffer
 * written at cache_seqlens[b] + i (mod state_len); conv_state_indices int32 [B] picks the row of conv_state
 * per batch element (continuous batching).
 * ------------------------------------------------------------------------ */
typedef struct vtx_causal_conv1d_params {
    const void* x;       int64_t x_stride_b, x_stride_d, x_stride_l;
    const void* weight;  int64_t weight_dtype;
    const void* bias;    int64_t bias_dtype;       /* or NULL */
    const int32_t* seq_idx;                         /* or NULL */
    const void* initial_states; int64_t is_stride_b, is_stride_d, is_stride_l;   /* or NULL */
    void* final_states;  int64_t fs_stride_b, fs_stride_d, fs_stride_l;          /* or NULL */
    void* out;           int64_t out_stride_b, out_stride_d, out_stride_l;
    int64_t B, D, L, W;
    int64_t silu;
    int64_t io_dtype;
} vtx_causal_conv1d_params;
int vtx_causal_conv1d_fwd(const vtx_causal_conv1d_params* p, void* stream);

typedef struct vtx_causal_conv1d_update_params {
    const void* x;       int64_t x_stride_b, x_stride_d, x_stride_l;
    void* conv_state;    int64_t cs_stride_b, cs_stride_d, cs_stride_l; int64_t state_len;
    const void* weight;  int64_t weight_dtype;
    const void* bias;    int64_t bias_dtype;       /* or NULL */
    const int32_t* cache_seqlens;                   /* or NULL */
    const int32_t* conv_state_indices;              /* or NULL */
    void* out;           int64_t out_stride_b, out_stride_d, out_stride_l;
    int64_t B, D, L, W;
    int64_t silu;
    int64_t io_dtype;
} vtx_causal_conv1d_update_params;
int vtx_causal_conv1d_update(const vtx_causal_conv1d_update_params* p, void* stream);

/* Conv states of packed sequences (vortex/ops/conv/local_causal_conv1d/causal_conv1d_varlen.py:42-75
 * causal_conv1d_varlen_states): x [total, dim] holds the sequences back to back, cu_seqlens int32 [batch+1] their
 * boundaries; states[b, :, state_len-n:] = the last n = min(state_len, length_b) rows of sequence b, zeros before.
 * states is addressed by element strides (the reference returns memory [batch, state_len, dim] viewed as
 * [batch, dim, state_len]). */
typedef struct vtx_varlen_states_params {
    const void* x;       int64_t x_stride_t, x_stride_c;
    const int32_t* cu_seqlens;
    void* states;        int64_t st_stride_b, st_stride_c, st_stride_l;
    int64_t total, batch, dim, state_len;
    int64_t io_dtype;
} vtx_varlen_states_params;
int vtx_causal_conv1d_varlen_states(const vtx_varlen_states_params* p, void* stream);

/* Hyena-X forward (vortex/ops/hyena_x/triton_indirect_fwd.py:262 hyena_x_bdl_fwd, reference :413-424):
 * o = fir(h[0:D], q) * fir(h[D:2D], k) * fir(h[2D:3D], v), depthwise causal filters of Lh <= 16 taps
 * (cross-correlation order), q, k, v, o [B,D,L] contiguous, h [3D,Lh]. */
typedef struct vtx_hyena_x_params {
    const void* q; const void* k; const void* v;
    const void* h;       int64_t h_dtype;
    void* y;
    int64_t B, D, L, Lh;
    int64_t io_dtype;
} vtx_hyena_x_params;
int vtx_hyena_x_fwd(const vtx_hyena_x_params* p, void* stream);

/* ------------------------------------------------------------------------
 * Decode (one token).
 *
 * vtx_step_fir: HyenaInferenceEngine.step_fir (engine.py:406-449) and the
 * unbuilt launcher step_fir_fwd_cuda (vortex/ops/conv/csrc/step_fir.cu:94-119);
 * for K <= 4 also causal_conv1d_update (causal_conv1d.cpp:382-390).
 *   cache = state_in length c (0 <= c <= K-1), oldest sample first.
 *   flip_filter: taps used are reversed(h)[K-1-c:]  else h[:c+1]
 *   y = tap_last * u + sum_i state[i] * tap[i]  (+ bias | + bias*u)
 *   state_out (fp32, always): c < K-1 ? [state, u] : [state[1:], u]
 * state_in may be any dtype; it must not alias state_out.
 * ------------------------------------------------------------------------ */
typedef struct vtx_step_fir_params {
    const void* u;           /* [B,C] contiguous, io dtype                       */
    const void* state_in;    int64_t state_dtype;  /* [B,C,c] contiguous          */
    const void* w;           int64_t w_dtype;      /* [Gw,K]; C % Gw == 0         */
    const void* bias;        int64_t bias_dtype;   /* [C] or NULL                 */
    void* y;                 /* [B,C] io dtype                                    */
    float* state_out;        /* [B,C,min(c+1,K-1)]                                */
    int64_t B, C, Gw, K, c;
    int64_t flip_filter, bias_mode;
    int64_t io_dtype;
} vtx_step_fir_params;
int vtx_step_fir(const vtx_step_fir_params* p, void* stream);

/* vtx_step_iir: HyenaInferenceEngine.step_iir (engine.py:451-467).
 *   sigma <- p*sigma + k*v ; y = q * (sum_s Re(R sigma) + bias * k*v), fp32 out.
 * state fp32 [B,D,S] (real) / [B,D,S,2] (complex); in and out may alias. */
typedef struct vtx_step_iir_params {
    const void* q; const void* k; const void* v;   /* [B,D] contiguous, io dtype */
    vtx_modal_params modal;                        /* G must divide D             */
    const void* bias;        int64_t bias_dtype;
    const float* state_in;   float* state_out;
    float* y;                                      /* [B,D] fp32                  */
    int64_t B, D;
    int64_t io_dtype;
} vtx_step_iir_params;
int vtx_step_iir(const vtx_step_iir_params* p, void* stream);

/* vtx_decode_layer: the whole HyenaCascade.sequential_forward
 * (model.py:318-375) for one layer in one launch: featurizer step ->
 * q/k/v selection -> inner FIR step (K > 0) or modal step (K == 0) -> gate.
 *   u [B,3D] io dtype -> y [B,D] io dtype; caches as in the step functions
 *   (fir states fp32 out; full caches only: c3 == K3-1, c == K-1). */
typedef struct vtx_decode_layer_params {
    const void* u;
    const void* w3;          int64_t w3_dtype;     /* [3D,K3]                     */
    const void* b3;          int64_t b3_dtype;     /* [3D] or NULL                */
    const void* fir_state_in;   int64_t fir_state_dtype;   /* [B,3D,K3-1]          */
    float* fir_state_out;
    const void* h;           int64_t h_dtype;      /* [G,K] (K > 0)               */
    const void* inner_state_in; int64_t inner_state_dtype; /* [B,D,K-1]            */
    float* inner_state_out;
    vtx_modal_params modal;                        /* K == 0                      */
    const float* iir_state_in;  float* iir_state_out;
    const void* bias;        int64_t bias_dtype;   /* [D] or NULL                 */
    void* y;
    int64_t B, D, G, K3, K;
    int64_t layout, num_heads, flip_x1x2;
    int64_t flip_filter, bias_mode;
    int64_t io_dtype;
} vtx_decode_layer_params;
int vtx_decode_layer(const vtx_decode_layer_params* p, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* VORTEX_B200_H */
