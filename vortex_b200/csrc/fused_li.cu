// Hyena-LI fused block on tcgen05 / TMEM (bf16 I/O, modal filter of up to 16 complex poles per group of 16 channels):
//   featurizer FIR (3 taps) -> q/k/v selection -> k*v -> causal convolution with h[t] = sum_s Re(R_s p_s^t)
//   -> (+ D*kv) -> q gate, in one pass over HBM, channel-last in and out.
//
// The filter is as long as the sequence, so the convolution is evaluated as a chunked state-space scan whose heavy
// parts are dense contractions.  For a chunk of 96 samples of one channel group (sigma = modal state, one complex
// number per pole and channel, sigma[t] = p sigma[t-1] + kv[t]):
//   Y[96 x N]   = T[96 x 96] KV[96 x N]  +  C[96 x 32] S[32 x N]       T[i][j] = h[i-j],  C[i] = R p^(i+1)
//   Inc[32 x N] = Bm[32 x 96] KV[96 x N]                               Bm[.][j] = p^(95-j)
//   S'          = p^96 S + Inc                                          (state at the start of the next chunk)
// with S = [Re sigma; Im sigma].  T and Bm are stacked into ONE 128-row operand, so a single MMA sequence
// yields the chunk's outputs (TMEM lanes 0..95) and its state increment (lanes 96..127).  A CTA owns one group of one
// sequence and walks it front to back; its four "streams" are four CONSECUTIVE chunks, so every MMA is 128 columns
// wide (4 x 16 channels, bf16 head | bf16 remainder of k*v).  The states at the four chunk starts follow from the
// four increments by a short recurrence in registers (one warp owning lanes 96..127), are written back to shared
// memory as bf16 head + remainder, and a second, short MMA sequence adds C S.  All operands that come from fp32 math
// (taps, pole powers, states, k*v) are carried as bf16 head + remainder, which keeps ~16 bits; the gate q crosses
// shared memory as fp16 (11 bits: 2.8e-4, beside the 1.7e-3 of the output's own rounding; saturating at +-65504).
//
// The walk is aligned to the END of the sequence: the first step is padded in front with rows before the sequence start
// (zeros, like the featurizer's own history), so the state after the last step is the state after the last token.
//
// Warp roles (16 warps): 0-7 front end (as in the medium-filter kernel: TMA-staged rows -> featurizer -> k*v and q
// tiles), 8-10 epilogue (TMEM lanes 0..95), 11 state recurrence (lanes 96..127), 12 MMA issue, 13-14 TMA issue.
// All waits are bounded.
#include <cstdlib>

#include "tma.cuh"
#include "umma.cuh"

namespace vtx {

VTX_DEFINE_STATUS_READER()

namespace li {

using namespace umma;

constexpr int NS = 4;                      // consecutive chunks per MMA step
constexpr int CH = 16;                     // channels per group
constexpr int CHUNK = 96;                  // samples per chunk (TMEM lanes 0..95); lanes 96..127 carry the state increment
constexpr int SUPER = NS * CHUNK;          // samples per step of the walk
constexpr int NPOLE = 16;
constexpr int NFE = 8;
constexpr int WROWS = CHUNK / NFE;         // 12 rows of a chunk per front-end warp
constexpr int RB = WROWS / 2;              // register batch
constexpr int HROWS = CHUNK / 2;           // rows per staged box: half a chunk, shared by four front-end warps
constexpr int BOX_ROWS = HROWS + 2 + (NS - 1);         // featurizer halo + stream skew
constexpr int BOX_BYTES = BOX_ROWS * 3 * CH * 2;
constexpr int IN_PLANE = (BOX_ROWS * 32 + 127) / 128 * 128;
constexpr int BOX_STRIDE = 3 * IN_PLANE;
constexpr int IN_STAGES = 4;
constexpr int STAGE_BYTES = NS * BOX_STRIDE;
constexpr int KV_TILE = CHUNK * 128;       // [96 rows][64 channels] bf16, 128-byte swizzle
constexpr int QH_TILE = KV_TILE;          // q as fp16 (11 significant bits: 2.8e-4, against 1.7e-3 of the output's own rounding)
constexpr int S_TILE = 2 * NPOLE * 128;    // [32 state rows][64 channels] bf16, 128-byte swizzle
constexpr int HI_OFF = 0, LO_OFF = KV_TILE, QH_OFF = 2 * KV_TILE, SH_OFF = QH_OFF + QH_TILE, SL_OFF = SH_OFF + S_TILE;
constexpr int SLOT_BYTES = SL_OFF + S_TILE;
constexpr int NPW = CHUNK + 4;             // pole powers p^0 .. p^96 (padded)
constexpr int NSLOT = 3;                   // a slot lives from the front end's stores to the end of its epilogue, i.e.
                                           // across MMA -> state recurrence -> MMA -> epilogue: two front-end periods
constexpr int OFF_SLOTS = IN_STAGES * STAGE_BYTES;
// set-up tables live in the last slot, which the front end does not touch before the operands are expanded
constexpr int OFF_PW = OFF_SLOTS + (NSLOT - 1) * SLOT_BYTES; // float2 [16][NPW]
constexpr int OFF_H = OFF_PW + NPOLE * NPW * 8;              // float [96]: first taps of the filter
constexpr int OFF_RES = OFF_H + CHUNK * 4;                   // float2 [16]: residues
static_assert(OFF_RES + NPOLE * 8 <= OFF_SLOTS + NSLOT * SLOT_BYTES, "set-up tables must fit into a slot");
constexpr int OFF_DIAG = OFF_SLOTS + NSLOT * SLOT_BYTES;     // float [16]: skip parameters
constexpr int OFF_BARS = OFF_DIAG + 64;
constexpr int NBARS = IN_STAGES * 2 + NSLOT * 3 + 2 * 3 + 1;
constexpr int SMEM_BYTES = OFF_BARS + NBARS * 8 + 16 + 1024;
static_assert(OFF_SLOTS % 1024 == 0 && SLOT_BYTES % 1024 == 0 && QH_OFF % 1024 == 0 &&
              SH_OFF % 1024 == 0 && SL_OFF % 1024 == 0, "tiles must be 1024-byte aligned");
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
// TMEM columns: stacked [T; Bm] head and remainder (96 K elements = 48 columns each), [C; 0] head and remainder
// (32 K elements = 16 columns each), two accumulators of 128 columns
constexpr int A_HI = 0, A_LO = 48, C_HI = 96, C_LO = 112, D_COL = 128, TMEM_COLS = 512;
constexpr int W_EP = NFE, W_ST = NFE + 3, W_MMA = NFE + 4, W_TMA = NFE + 5, NTMA = 2, W_ST2 = NFE + 7;   // state warps: warp % 4 == 3
constexpr int THREADS = 32 * 16;

struct Args {
    const void* w3; int64_t w3_dtype;
    const void* bias; int64_t bias_dtype;
    const float* log_poles; const float* theta; const float* res_re; const float* res_im;
    __nv_bfloat16* y; int64_t y_stride_b, y_stride_l;
    float* state; const float* state_in;   // state after the last token (out), state before the first (in, or null)
    int hist;                      // rows in front of u covered by the tensor map (the sequence's earlier samples)
    float* carry; int* flags;      // [walk][slice][32][16] states handed from slice to slice, arrival counters
    int64_t L, D, G, S, B;
    int spp, nslice;               // steps per slice, slices per walk
    int poll_limit;                // polls of a slice's arrival counter before the next slice gives up
    int layout, flip;
    int64_t hd;
};

template <bool INTERLEAVED, bool SWAP>
__global__ void __launch_bounds__(THREADS, 1) fused_li_kernel(const __grid_constant__ CUtensorMap tmap, Args a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t sm_u = smem_u32(sm);
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + OFF_BARS);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + OFF_BARS + NBARS * 8);
    auto in_full = [&](int st) { return smem_u32(&bars[st * 2]); };
    auto in_empty = [&](int st) { return smem_u32(&bars[st * 2 + 1]); };
    const int BB = IN_STAGES * 2;
    auto kv_full = [&](int sl) { return smem_u32(&bars[BB + sl]); };                      // front end -> MMA: k*v and q tiles written
    auto slot_free = [&](int sl) { return smem_u32(&bars[BB + NSLOT + sl]); };            // 3 epilogue warps + MMA commit: slot reusable
    auto s_full = [&](int sl) { return smem_u32(&bars[BB + 2 * NSLOT + sl]); };           // state warps: chunk-start states in shared memory
    const int BD = BB + 3 * NSLOT;
    auto inc_full = [&](int d) { return smem_u32(&bars[BD + d]); };                       // MMA commit: T/Bm part accumulated
    auto d_full = [&](int d) { return smem_u32(&bars[BD + 2 + d]); };                     // MMA commit: C S part accumulated too
    auto d_empty = [&](int d) { return smem_u32(&bars[BD + 4 + d]); };                    // 3 epilogue warps + 2 state warps: accumulator read
    const uint32_t a_ready = smem_u32(&bars[BD + 6]);                                     // operands expanded, set-up tables no longer needed

    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    // blockIdx = (time slice, batch element, group), slices of a walk in increasing block order: a slice starts from the
    // state its predecessor leaves in global memory (a.carry), which an earlier block of the same launch produces
    const int64_t nwalk = a.G * a.B, walk = blockIdx.x % nwalk;
    const int slice = (int)(blockIdx.x / nwalk);
    const int64_t g = walk % a.G, b = walk / a.G;
    const int ntotal = (int)((a.L + SUPER - 1) / SUPER);     // steps of the whole walk
    const int pad = (int)((int64_t)ntotal * SUPER - a.L);    // rows in front of the sequence in the first step
    const int kbase = slice * a.spp;                         // first step of this slice
    const int nsc = ntotal - kbase < a.spp ? ntotal - kbase : a.spp;   // steps of this slice

    // ---------------- setup -------------------------------------------------------------------
    if (tid == 0) {
        for (int st = 0; st < IN_STAGES; ++st) { mbar_init(in_full(st), NTMA); mbar_init(in_empty(st), NFE / 2); }
        for (int sl = 0; sl < NSLOT; ++sl) { mbar_init(kv_full(sl), NFE); mbar_init(slot_free(sl), 4); mbar_init(s_full(sl), 2); }
        for (int d = 0; d < 2; ++d) { mbar_init(inc_full(d), 1); mbar_init(d_full(d), 1); mbar_init(d_empty(d), 5); }
        mbar_init(a_ready, NFE + 5);
        fence_mbar_init();
    }
    if (warp == W_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    float2* pw = reinterpret_cast<float2*>(sm + OFF_PW);         // pw[s * NPW + n] = p_s^n
    float* htab = reinterpret_cast<float*>(sm + OFF_H);
    float2* res = reinterpret_cast<float2*>(sm + OFF_RES);
    {
        const int S = (int)a.S;
        for (int idx = tid; idx < NPOLE * NPW; idx += THREADS) {
            const int s = idx / NPW, n = idx % NPW;
            float2 v = make_float2(0.f, 0.f);
            if (s < S) {
                const float mag = expf(a.log_poles[g * S + s] * (float)n);
                if (a.theta) {
                    double ang = (double)a.theta[g * S + s] * (double)n;
                    ang -= 6.283185307179586 * floor(ang / 6.283185307179586);
                    float sn, cs;
                    sincosf((float)ang, &sn, &cs);
                    v = make_float2(mag * cs, mag * sn);
                } else {
                    v = make_float2(mag, 0.f);
                }
            }
            pw[idx] = v;
        }
        for (int s = tid; s < NPOLE; s += THREADS)
            res[s] = s < S ? make_float2(a.res_re[g * S + s], a.res_im ? a.res_im[g * S + s] : 0.f) : make_float2(0.f, 0.f);
        float* dsk = reinterpret_cast<float*>(sm + OFF_DIAG);
        for (int c = tid; c < CH; c += THREADS) dsk[c] = a.bias ? ld_param(a.bias, a.bias_dtype, g * CH + c) : 0.f;
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    for (int lag = tid; lag < CHUNK; lag += THREADS) {          // h[lag] = sum_s Re(R_s p_s^lag)
        float acc = 0.f;
#pragma unroll
        for (int s = 0; s < NPOLE; ++s) {
            const float2 p = pw[s * NPW + lag], r = res[s];
            acc = fmaf(r.x, p.x, fmaf(-r.y, p.y, acc));
        }
        htab[lag] = acc;
    }
    __syncthreads();

    // p^96 of this lane's pole (used by the state warps), read before the tables' slot is released through a_ready
    const float2 Pst = pw[(lane >> 1) * NPW + CHUNK];
    asm volatile("" ::"f"(Pst.x), "f"(Pst.y));

    if (warp < NFE + 4) {
        // Expand the operands into TMEM: lane i holds row i.  A warp reaches the lanes of its quarter (warp % 4); the
        // three warps of a quarter share the column blocks.  Every value is split into a bf16 head and a bf16 remainder.
        const int i = (warp % 4) * 32 + lane, part = warp / 4;
        const uint32_t lane_base = tmem + ((uint32_t)((warp % 4) * 32) << 16);
        auto split_store = [&](const float (&v)[32], uint32_t col_hi, uint32_t col_lo) {
            uint32_t hi[16], lo[16];
#pragma unroll
            for (int m = 0; m < 16; ++m) {
                hi[m] = pack_bf16(v[2 * m], v[2 * m + 1]);
                lo[m] = pack_bf16(v[2 * m] - bf_lo(hi[m]), v[2 * m + 1] - bf_hi(hi[m]));
            }
            tmem_st16(lane_base + col_hi, hi);
            tmem_st16(lane_base + col_lo, lo);
        };
        {   // stacked [T; Bm]: K elements 32 part .. 32 part + 31
            float v[32];
#pragma unroll
            for (int m = 0; m < 32; ++m) {
                const int j = 32 * part + m;
                if (i < CHUNK) {
                    v[m] = j <= i ? htab[i - j] : 0.f;
                } else {
                    const float2 p = pw[((i - CHUNK) >> 1) * NPW + (CHUNK - 1 - j)];
                    v[m] = ((i - CHUNK) & 1) ? p.y : p.x;
                }
            }
            split_store(v, A_HI + 16 * part, A_LO + 16 * part);
        }
        if (part == 0) {   // [C; 0]: K element 2s = Re(R_s p_s^(i+1)), 2s+1 = -Im(R_s p_s^(i+1))
            float v[32];
#pragma unroll
            for (int m = 0; m < 32; ++m) {
                float x = 0.f;
                if (i < CHUNK) {
                    const float2 p = pw[(m >> 1) * NPW + i + 1], r = res[m >> 1];
                    x = (m & 1) ? -(r.x * p.y + r.y * p.x) : (r.x * p.x - r.y * p.y);
                }
                v[m] = x;
            }
            split_store(v, C_HI, C_LO);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(a_ready);
    }

    // ---------------- roles ---------------------------------------------------------------------
    if (warp < NFE) {
        // ======== front end: warp w owns rows [12w, 12w+12) of each of the four chunks of a step =========
        const int w = warp, p = lane % 8, s = lane / 8;
        f32x2 w3[3][3];     // [q|k|v][tap], each the pair of this lane's two channels
        {
            QkvMap map{a.layout, INTERLEAVED ? 0 : a.flip, a.D, a.hd};
            int64_t pc[2][3];
#pragma unroll
            for (int c = 0; c < 2; ++c) map.get(g * CH + 2 * p + c, pc[c][0], pc[c][1], pc[c][2]);
#pragma unroll
            for (int x = 0; x < 3; ++x)
#pragma unroll
                for (int j = 0; j < 3; ++j)
                    w3[x][j] = pk2(ld_param(a.w3, a.w3_dtype, pc[0][x] * 3 + j), ld_param(a.w3, a.w3_dtype, pc[1][x] * 3 + j));
        }
        const uint32_t kv_chunk = (uint32_t)(s * 2 + p / 4), kv_in = (uint32_t)((p % 4) * 4);   // 16-byte chunk and offset of this lane's bf16 pair in a k*v row
        constexpr int ROWB = INTERLEAVED ? 96 : 32;             // bytes per staged row (per plane in the planar layouts)
        auto box_addr = [&](int k, int hb) {
            const int nh = 2 * k + w / (NFE / 2), stg = nh % IN_STAGES;
            return sm_u + (uint32_t)(stg * STAGE_BYTES + s * BOX_STRIDE + ((w % (NFE / 2)) * WROWS + hb * RB + s) * ROWB +
                                     (INTERLEAVED ? 12 : 4) * p);
        };
        auto fetch = [&](uint32_t addr, uint32_t (&raw)[RB + 2][3]) {
#pragma unroll
            for (int r = 0; r < RB + 2; ++r)
#pragma unroll
                for (int j = 0; j < 3; ++j)
                    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(raw[r][j]) : "r"(addr + (uint32_t)(r * ROWB + (INTERLEAVED ? 4 * j : j * IN_PLANE))));
        };
        auto unpack = [&](const uint32_t (&e)[3], f32x2 (&x)[3]) {
            if (INTERLEAVED) {
                x[0] = pk2(bf_lo(e[0]), bf_hi(e[1]));
                x[1] = pk2(bf_hi(e[0]), bf_lo(e[2]));
                x[2] = pk2(bf_lo(e[1]), bf_hi(e[2]));
            } else {
#pragma unroll
                for (int pl = 0; pl < 3; ++pl) x[pl] = pk2(bf_lo(e[pl]), bf_hi(e[pl]));
            }
        };
        auto compute = [&](int slot, int hb, const uint32_t (&raw)[RB + 2][3]) {
            const uint32_t row0 = (uint32_t)(w * WROWS + hb * RB);
            const uint32_t slot_u = sm_u + OFF_SLOTS + slot * SLOT_BYTES;
            // Tiles are 1024-byte aligned: the swizzle (16-byte chunk index XOR row phase) is an XOR on the address of the
            // lane's element; the row phase is (row & 7) for the 128-byte rows and ((row >> 1) & 3) for the 64-byte rows.
            // row = 12 w + 6 hb + i, and adding 4 (mod 8) or 2 (mod 4) is an XOR: the warp's part of the phase,
            // 4 (w & 1) resp. 2 (w & 1), is folded into the lane's chunk index once, the rest, (6 hb + i) & 7 resp.
            // ((6 hb + i) >> 1) & 3, is a compile-time constant of each store.
            const uint32_t kv_a0 = slot_u + ((kv_chunk ^ (uint32_t)((w & 1) * 4)) << 4) + kv_in + row0 * 128;
            f32x2 x1[3], x2[3];
            unpack(raw[0], x2);
            unpack(raw[1], x1);
#pragma unroll
            for (int i = 0; i < RB; ++i) {
                f32x2 x0[3], z[3];
                unpack(raw[i + 2], x0);
#pragma unroll
                for (int x = 0; x < 3; ++x) {
                    z[x] = fma2(w3[x][0], x2[x], fma2(w3[x][1], x1[x], mul2(w3[x][2], x0[x])));
                    x2[x] = x1[x];
                    x1[x] = x0[x];
                }
                const f32x2 q = SWAP ? z[1] : z[0];
                const f32x2 kv = mul2(SWAP ? z[0] : z[1], z[2]);          // rows before the sequence start are zeros
                float kv0, kv1;
                up2(kv, kv0, kv1);
                const uint32_t hi = pack_bf16(kv0, kv1);
                float r0, r1;
                up2(sub2(kv, pk2(bf_lo(hi), bf_hi(hi))), r0, r1);
                const uint32_t lo = pack_bf16(r0, r1);
                const uint32_t kaddr = (kv_a0 ^ (uint32_t)(((RB * hb + i) & 7) << 4)) + i * 128;
                asm volatile("st.shared.b32 [%0], %1;" ::"r"(kaddr + HI_OFF), "r"(hi));
                asm volatile("st.shared.b32 [%0], %1;" ::"r"(kaddr + LO_OFF), "r"(lo));
                float q0, q1;
                up2(q, q0, q1);
                asm volatile("st.shared.b32 [%0], %1;" ::"r"(kaddr + QH_OFF), "r"(pack_f16(q0, q1)));
            }
        };
        auto stage_of = [&](int k) { return (2 * k + w / (NFE / 2)) % IN_STAGES; };
        auto stage_parity = [&](int k) { return (uint32_t)(((2 * k + w / (NFE / 2)) / IN_STAGES) & 1); };

        // Software pipeline over register batches A (rows 0..RB-1 of the warp's rows) and B (the rest):
        //   fetch B(k) | wait slot | compute A(k) | release stage | wait stage(k+1), fetch A(k+1) | compute B(k) | publish
        uint32_t rawA[RB + 2][3], rawB[RB + 2][3];
        bool ok = mbar_wait(in_full(stage_of(0)), stage_parity(0), 4);
        if (ok) fetch(box_addr(0, 0), rawA);
        for (int k = 0; k < nsc && ok; ++k) {
            const int slot = k % NSLOT;
            fetch(box_addr(k, 1), rawB);
            if (k >= NSLOT && !mbar_wait(slot_free(slot), (uint32_t)(((k - NSLOT) / NSLOT) & 1), 2)) break;
            if (k == NSLOT - 1 && !mbar_wait(a_ready, 0, 14)) break;      // the set-up tables live in the last slot
            compute(slot, 0, rawA);
#pragma unroll
            for (int r = 0; r < RB + 2; ++r) asm volatile("" ::"r"(rawB[r][0]), "r"(rawB[r][1]), "r"(rawB[r][2]));
            __syncwarp();
            if (lane == 0) mbar_arrive(in_empty(stage_of(k)));
            if (k + 1 < nsc) {
                if (!mbar_wait(in_full(stage_of(k + 1)), stage_parity(k + 1), 4)) break;
                fetch(box_addr(k + 1, 0), rawA);
            }
            compute(slot, 1, rawB);
            fence_proxy_async_smem();      // generic-proxy writes -> visible to the tensor core's async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(kv_full(slot));
        }
    } else if (warp < W_EP + 3) {
        // ======== epilogue: thread = output row of a chunk (TMEM lanes 0..95) ==============================
        const int e = warp - W_EP, r = e * 32 + lane;
        // this thread's row of chunk 0 of step 0, relative to the sequence start (negative: padding, not stored)
        const int first0 = r - pad;
        __nv_bfloat16* const yrow0 = a.y + b * a.y_stride_b + (int64_t)first0 * a.y_stride_l + g * CH;
        const int64_t chunk_pitch = (int64_t)CHUNK * a.y_stride_l;
        const float4* dsk = reinterpret_cast<const float4*>(sm + OFF_DIAG);    // skip parameters D[g*16 .. +16), fp32
        bool has_skip = false;
#pragma unroll
        for (int c = 0; c < CH / 4; ++c) {
            const float4 d = dsk[c];
            has_skip = has_skip || d.x != 0.f || d.y != 0.f || d.z != 0.f || d.w != 0.f;
        }
        const int64_t step_pitch = (int64_t)SUPER * a.y_stride_l;
        for (int k = 0; k < nsc; ++k) {
            const int slot = k % NSLOT, dbuf = k % 2;
            if (!mbar_wait(d_full(dbuf), (uint32_t)((k / 2) & 1), 5)) break;
            tc_fence_after();
            __syncwarp();
            const uint32_t taddr = tmem + ((uint32_t)(e * 32) << 16) + D_COL + dbuf * 128;
            const uint8_t* slot_p = sm + OFF_SLOTS + slot * SLOT_BYTES;
            const uint8_t* qh_p = slot_p + QH_OFF + r * 128;
            const int64_t yoff = (int64_t)(kbase + k) * step_pitch;
            // (rolled over the four chunks: the unrolled form of this loop, with the skip term, does not fit the
            // instruction cache next to the other roles' loops)
#pragma unroll 1
            for (int s = 0; s < NS; ++s) {
                uint32_t ah[16], al[16];
                tmem_ld16(taddr + s * 16, ah);
                tmem_ld16(taddr + 64 + s * 16, al);
                tmem_ld_wait(ah, al);
                if (s + 1 == NS) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(d_empty(dbuf));
                }
                f32x2 y[8];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    y[i] = add2(pk2(__uint_as_float(ah[2 * i]), __uint_as_float(ah[2 * i + 1])),
                                pk2(__uint_as_float(al[2 * i]), __uint_as_float(al[2 * i + 1])));
                if (has_skip) {
                    // skip term D[c] * kv[t, c] from this row of the k*v tile (head + remainder)
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
                        const uint32_t off = (uint32_t)(r * 128) + (uint32_t)(((2 * s + hf) ^ (r & 7)) << 4);
                        const uint4 h4 = *reinterpret_cast<const uint4*>(slot_p + HI_OFF + off);
                        const uint4 l4 = *reinterpret_cast<const uint4*>(slot_p + LO_OFF + off);
                        const float4 d0 = dsk[2 * hf], d1 = dsk[2 * hf + 1];
                        f32x2* yy = &y[4 * hf];
                        yy[0] = fma2(pk2(d0.x, d0.y), add2(pk2(bf_lo(h4.x), bf_hi(h4.x)), pk2(bf_lo(l4.x), bf_hi(l4.x))), yy[0]);
                        yy[1] = fma2(pk2(d0.z, d0.w), add2(pk2(bf_lo(h4.y), bf_hi(h4.y)), pk2(bf_lo(l4.y), bf_hi(l4.y))), yy[1]);
                        yy[2] = fma2(pk2(d1.x, d1.y), add2(pk2(bf_lo(h4.z), bf_hi(h4.z)), pk2(bf_lo(l4.z), bf_hi(l4.z))), yy[2]);
                        yy[3] = fma2(pk2(d1.z, d1.w), add2(pk2(bf_lo(h4.w), bf_hi(h4.w)), pk2(bf_lo(l4.w), bf_hi(l4.w))), yy[3]);
                    }
                }
                uint32_t o[8];
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    const uint4 qh4 = *reinterpret_cast<const uint4*>(qh_p + (((2 * s + hf) ^ (r & 7)) << 4));
                    const uint32_t qh[4] = {qh4.x, qh4.y, qh4.z, qh4.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {          // channels 8 hf + 2 j, + 1
                        float o0, o1;
                        up2(mul2(y[4 * hf + j], unpack_f16(qh[j])), o0, o1);
                        o[4 * hf + j] = pack_bf16(o0, o1);
                    }
                }
                if ((kbase + k) * SUPER + s * CHUNK + first0 >= 0)
                    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(yrow0 + yoff + s * chunk_pitch), "r"(o[0]),
                                 "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]));
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(slot_free(slot));
        }
    } else if (warp == W_ST || warp == W_ST2) {
        // ======== state recurrence: lane = row of the state tile (pole lane/2, real or imaginary part); each of the
        // two warps owns eight of the sixteen channels ========================================================
        const int jj = lane, half = warp == W_ST2;
        const float2 P = Pst;                                  // p^96: one chunk ahead
        const float Pa = P.x, Pb = (jj & 1) ? P.y : -P.y;      // new = Pa * own + Pb * partner + increment
        if (warp == W_ST2) {                                   // (the other state warp arrives with the expanding warps)
            __syncwarp();
            if (lane == 0) mbar_arrive(a_ready);
        }
        float S[8];                                            // this component of the state at a chunk start
#pragma unroll
        for (int c = 0; c < 8; ++c) S[c] = 0.f;
        if (slice == 0 && a.state_in && (jj >> 1) < (int)a.S) {
            // a call that continues an earlier one starts from that call's end state (same layout as a.state);
            // the walk then has no padding in front (the host only routes such calls here when L % SUPER == 0)
            const bool cplx = a.theta != nullptr;
            if (cplx || !(jj & 1)) {
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const int64_t d = g * CH + 8 * half + c;
                    const int64_t idx = (b * a.D + d) * a.S + (jj >> 1);
                    S[c] = a.state_in[cplx ? 2 * idx + (jj & 1) : idx];
                }
            }
        }
        if (slice > 0) {
            // wait (bounded) for both state warps of the previous slice, then take its final state over
            const int64_t prev = walk * (a.nslice - 1) + (slice - 1);
            bool have = false;
            for (int it = 0; it < a.poll_limit && !have; ++it) {
                int v;
                asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(a.flags + prev) : "memory");
                have = v >= 2;
                if (!have) __nanosleep(200);
            }
            if (!have) atomicCAS(&g_device_status, 0, 15);
            have = __all_sync(0xffffffffu, have);
            if (have) {
                const float4* src = reinterpret_cast<const float4*>(a.carry + (prev * 32 + jj) * 16 + 8 * half);
                const float4 v0 = src[0], v1 = src[1];
                S[0] = v0.x; S[1] = v0.y; S[2] = v0.z; S[3] = v0.w; S[4] = v1.x; S[5] = v1.y; S[6] = v1.z; S[7] = v1.w;
            }
        }
        for (int k = 0; k < nsc; ++k) {
            const int slot = k % NSLOT, dbuf = k % 2;
            if (!mbar_wait(inc_full(dbuf), (uint32_t)((k / 2) & 1), 12)) break;
            tc_fence_after();
            __syncwarp();
            const uint32_t taddr = tmem + ((uint32_t)CHUNK << 16) + D_COL + dbuf * 128 + 8 * half;
            uint8_t* sh_row = sm + OFF_SLOTS + slot * SLOT_BYTES + SH_OFF + jj * 128;
            uint32_t inc[2][2][8];
            tmem_ld8(taddr, inc[0][0]);
            tmem_ld8(taddr + 64, inc[0][1]);
#pragma unroll
            for (int i = 0; i < NS; ++i) {
                // state at the start of chunk i -> shared memory (head + remainder): 16-byte chunk 2 i + half of the row
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    hi[m] = pack_bf16(S[2 * m], S[2 * m + 1]);
                    lo[m] = pack_bf16(S[2 * m] - bf_lo(hi[m]), S[2 * m + 1] - bf_hi(hi[m]));
                }
                const uint32_t off = (uint32_t)(((2 * i + half) ^ (jj & 7)) << 4);
                *reinterpret_cast<uint4*>(sh_row + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<uint4*>(sh_row + S_TILE + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                uint32_t (&ia)[8] = inc[i & 1][0];
                uint32_t (&ib)[8] = inc[i & 1][1];
                tmem_ld8_wait(ia, ib);
                if (i + 1 < NS) {
                    tmem_ld8(taddr + (i + 1) * 16, inc[(i + 1) & 1][0]);
                    tmem_ld8(taddr + 64 + (i + 1) * 16, inc[(i + 1) & 1][1]);
                }
                // state at the start of the next chunk
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const float partner = __shfl_xor_sync(0xffffffffu, S[c], 1);
                    const float add = __uint_as_float(ia[c]) + __uint_as_float(ib[c]);
                    S[c] = fmaf(Pa, S[c], fmaf(Pb, partner, add));
                }
            }
            tc_fence_before();
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) { mbar_arrive(s_full(slot)); mbar_arrive(d_empty(dbuf)); }
        }
        if (slice + 1 < a.nslice) {
            // hand the state to the next slice
            const int64_t mine = walk * (a.nslice - 1) + slice;
            float4* dst = reinterpret_cast<float4*>(a.carry + (mine * 32 + jj) * 16 + 8 * half);
            dst[0] = make_float4(S[0], S[1], S[2], S[3]);
            dst[1] = make_float4(S[4], S[5], S[6], S[7]);
            __threadfence();
            __syncwarp();
            if (lane == 0) atomicAdd(a.flags + mine, 1);
        } else if (a.state && (jj >> 1) < (int)a.S) {
            // state after the last token: [B, D, S] (real poles) or [B, D, S, 2]
            const bool cplx = a.theta != nullptr;
            if (cplx || !(jj & 1)) {
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const int64_t d = g * CH + 8 * half + c;
                    const int64_t idx = (b * a.D + d) * a.S + (jj >> 1);
                    a.state[cplx ? 2 * idx + (jj & 1) : idx] = S[c];
                }
            }
        }
    } else if (warp == W_MMA) {
        // ======== MMA issue =========================================================================
        if (lane == 0) {
            const uint32_t idesc = instr_desc(128, 2 * NS * CH, 1);
            const uint64_t kv_desc0 = smem_desc(sm_u + OFF_SLOTS + HI_OFF, KV_TILE, 1024, 2);
            const uint64_t s_desc0 = smem_desc(sm_u + OFF_SLOTS + SH_OFF, S_TILE, 1024, 2);
            bool ok = mbar_wait(a_ready, 0, 10);
            for (int k = 0; k < nsc && ok; ++k) {
                const int slot = k % NSLOT, dbuf = k % 2;
                if (!mbar_wait(kv_full(slot), (uint32_t)((k / NSLOT) & 1), 6)) break;
                if (k >= 2 && !mbar_wait(d_empty(dbuf), (uint32_t)(((k - 2) / 2) & 1), 8)) break;
                tc_fence_after();
                const uint32_t d = tmem + D_COL + dbuf * 128;
                // descriptors of the slot's tiles: the start-address field counts 16-byte units
                const uint64_t dk = kv_desc0 + (uint64_t)(slot * (SLOT_BYTES / 16)), ds = s_desc0 + (uint64_t)(slot * (SLOT_BYTES / 16));
                // outputs of the four chunks (lanes 0..95) and their state increments (lanes 96..127)
#pragma unroll
                for (int part = 0; part < 2; ++part)
#pragma unroll
                    for (int jj = 0; jj < CHUNK / 16; ++jj)
                        mma_ts(d, tmem + (part ? A_LO : A_HI) + 8 * jj, dk + (uint64_t)(jj * 128), idesc, (part || jj) ? 1u : 0u);
                mma_commit(inc_full(dbuf));
                // + C S: contribution of everything before each chunk
                if (!mbar_wait(s_full(slot), (uint32_t)((k / NSLOT) & 1), 13)) break;
                tc_fence_after();
#pragma unroll
                for (int part = 0; part < 2; ++part)
#pragma unroll
                    for (int jj = 0; jj < 2; ++jj)
                        mma_ts(d, tmem + (part ? C_LO : C_HI) + 8 * jj, ds + (uint64_t)(jj * 128), idesc, 1u);
                mma_commit(d_full(dbuf));
                mma_commit(slot_free(slot));
            }
        }
    } else if (warp < W_TMA + NTMA) {
        int col[3] = {0, 0, 0};
        if (INTERLEAVED) {
            col[0] = (int)(3 * g * CH);
        } else {
            const int64_t d0 = g * CH;
            if (a.layout == VTX_QKV_COLUMN_SPLIT) {
                int64_t n = d0 / a.hd, j = d0 - n * a.hd;
                col[0] = (int)(n * 3 * a.hd + j); col[1] = col[0] + (int)a.hd; col[2] = col[0] + 2 * (int)a.hd;
            } else {
                col[0] = (int)d0; col[1] = (int)(a.D + d0); col[2] = (int)(2 * a.D + d0);
            }
            if (a.flip) { int t = col[0]; col[0] = col[1]; col[1] = t; }
        }
        const int tw = warp - W_TMA;                 // this warp issues the boxes of streams tw, tw + NTMA, ...
        if (lane == 0) {
            // ======== TMA issue ======================================================================
            tma_prefetch_desc(&tmap);
            for (int nh = 0; nh < 2 * nsc; ++nh) {
                const int stg = nh % IN_STAGES, k = nh / 2, h = nh % 2;
                if (nh >= IN_STAGES && !mbar_wait(in_empty(stg), (uint32_t)(((nh - IN_STAGES) / IN_STAGES) & 1), 9)) break;
                const uint32_t bar = in_full(stg);
                mbar_expect_tx(bar, NS / NTMA * BOX_BYTES);
#pragma unroll
                for (int s = 0; s < NS; ++s) {
                    if (s % NTMA != tw) continue;
                    const uint32_t dst = sm_u + (uint32_t)(stg * STAGE_BYTES + s * BOX_STRIDE);
                    const int row = (NS * (kbase + k) + s) * CHUNK + h * HROWS - 2 - s - pad + a.hist;      // stream s is staged s rows early
                    if (INTERLEAVED) {
                        tma_load_3d(dst, &tmap, bar, col[0], row, (int)b);
                    } else {
#pragma unroll
                        for (int pl = 0; pl < 3; ++pl) tma_load_3d(dst + pl * IN_PLANE, &tmap, bar, col[pl], row, (int)b);
                    }
                }
            }
        }
    }

    // ---------------- teardown -------------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == W_MMA) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
    }
}

// Time slices per walk: with one CTA per SM, B*G walks fill the SMs in whole rounds; cutting every walk into slices
// (handed from block to block through global memory) evens the last round out.
static void plan_slices(int64_t walks, int64_t ntotal, int& nslice, int& spp) {
    int best = 1;
    double best_cost = 1e30;
    for (int nt = 1; nt <= 8; ++nt) {
        if (nt > 1 && ntotal / nt < 16) break;
        const double cost = (double)ceil_div<int64_t>(walks * nt, kNumSMs) / nt + 0.002 * nt;   // + per-CTA set-up
        if (cost < best_cost * 0.98) { best_cost = cost; best = nt; }
    }
    spp = (int)ceil_div<int64_t>(ntotal, best);
    nslice = (int)ceil_div<int64_t>(ntotal, spp);
}

}  // namespace li
}  // namespace vtx

namespace vtx {
namespace licc {   // fused_li_cc.cu: the recurrence on the fp32 pipe (modal systems of any grouping, any I/O dtype)
int64_t scratch_bytes(const vtx_fused_iir_params* p);
int fwd(const vtx_fused_iir_params* p, cudaStream_t stream);
}  // namespace licc

// Shapes the tensor-core kernel takes; every other call runs the recurrence kernel.
static bool li_tc_shape(const vtx_fused_iir_params* p) {
    using namespace li;
    return p->io_dtype == VTX_BF16 && p->D == p->modal.G * CH && p->modal.S <= NPOLE && p->K3 == 3 && !p->b3 &&
           !p->fir_state_in && ((!p->state_in && p->u_hist_rows == 0) || (p->L % SUPER == 0 && (p->u_hist_rows == 0 || p->u_hist_rows >= 2))) &&
           (reinterpret_cast<uintptr_t>(p->y) % 32) == 0 && (p->y_stride_l % 16) == 0 &&
           (p->y_stride_b % 16) == 0 && (reinterpret_cast<uintptr_t>(p->u) % 16) == 0 && (p->u_stride_l % 8) == 0 &&
           (p->u_stride_b % 8) == 0 &&
           (p->layout == VTX_QKV_INTERLEAVED || (p->D % 8) == 0) &&
           (p->layout != VTX_QKV_COLUMN_SPLIT || (p->num_heads > 0 && p->D % p->num_heads == 0 && (p->D / p->num_heads) % CH == 0));
}
}  // namespace vtx

extern "C" int64_t vtx_fused_iir_scratch_bytes(const vtx_fused_iir_params* p) {
    using namespace vtx::li;
    if (!p || p->B <= 0 || p->L <= 0 || p->D <= 0 || p->modal.G <= 0 || p->modal.S <= 0) return 0;
    if (!vtx::li_tc_shape(p)) return vtx::licc::scratch_bytes(p);
    int nslice, spp;
    plan_slices(p->B * (p->D / CH), (p->L + SUPER - 1) / SUPER, nslice, spp);
    return (int64_t)p->B * (p->D / CH) * (nslice - 1) * (32 * 16 * 4 + 4);
}

extern "C" int vtx_fused_iir_fwd(const vtx_fused_iir_params* p, void* stream_) {
    using namespace vtx;
    using namespace vtx::li;
    cudaStream_t stream = (cudaStream_t)stream_;
    VTX_REQUIRE(p && p->u && p->w3 && p->y && p->modal.log_poles && p->modal.res_re, VTX_ERR_BAD_ARG, "fused_iir: null pointer");
    VTX_REQUIRE(p->B > 0 && p->L > 0 && p->D > 0 && p->modal.G > 0 && p->modal.S > 0, VTX_ERR_BAD_ARG, "fused_iir: sizes must be positive");
    VTX_REQUIRE(!p->modal.res_im || p->modal.theta, VTX_ERR_BAD_ARG, "fused_iir: complex residues need complex poles");
    if (!li_tc_shape(p)) return licc::fwd(p, stream);
    VTX_REQUIRE(p->L < ((int64_t)1 << 30) && p->B <= 65535 && p->modal.G * p->B < ((int64_t)1 << 27), VTX_ERR_UNSUPPORTED,
                "fused_iir: problem too large");
    Args a{};
    a.w3 = p->w3; a.w3_dtype = p->w3_dtype; a.bias = p->bias; a.bias_dtype = p->bias_dtype;
    a.log_poles = static_cast<const float*>(p->modal.log_poles); a.theta = static_cast<const float*>(p->modal.theta);
    a.res_re = static_cast<const float*>(p->modal.res_re); a.res_im = static_cast<const float*>(p->modal.res_im);
    a.y = static_cast<__nv_bfloat16*>(p->y); a.y_stride_b = p->y_stride_b; a.y_stride_l = p->y_stride_l;
    a.state = p->state; a.state_in = p->state_in; a.hist = (int)p->u_hist_rows;
    a.L = p->L; a.D = p->D; a.G = p->modal.G; a.S = p->modal.S; a.B = p->B;
    const int64_t walks = p->B * p->modal.G, ntotal = (p->L + SUPER - 1) / SUPER;
    a.nslice = 1; a.spp = (int)ntotal;
    a.poll_limit = flag_poll_limit();
    if (p->scratch) {       // without scratch every walk is one block
        plan_slices(walks, ntotal, a.nslice, a.spp);
        if (a.nslice > 1) {
            VTX_REQUIRE(reinterpret_cast<uintptr_t>(p->scratch) % 16 == 0, VTX_ERR_ALIGNMENT, "fused_iir: scratch must be 16-byte aligned");
            a.carry = static_cast<float*>(p->scratch);
            a.flags = reinterpret_cast<int*>(a.carry + walks * (a.nslice - 1) * 32 * 16);
            cudaError_t e = cudaMemsetAsync(a.flags, 0, (size_t)(walks * (a.nslice - 1)) * sizeof(int), stream);
            if (e != cudaSuccess) return fail(VTX_ERR_LAUNCH, "fused_iir: clearing the slice counters: %s", cudaGetErrorString(e));
        }
    }
    a.layout = (int)p->layout; a.flip = p->flip_x1x2 != 0;
    a.hd = p->D;
    if (p->layout == VTX_QKV_COLUMN_SPLIT) {
        VTX_REQUIRE(p->num_heads > 0 && p->D % p->num_heads == 0, VTX_ERR_BAD_ARG, "fused_iir: bad num_heads");
        a.hd = p->D / p->num_heads;
        VTX_REQUIRE(a.hd % CH == 0, VTX_ERR_UNSUPPORTED, "fused_iir: column split needs head size %% %d == 0", CH);
    }
    VTX_REQUIRE(p->layout == VTX_QKV_INTERLEAVED || (p->D * 2) % 16 == 0, VTX_ERR_ALIGNMENT,
                "fused_iir: D*itemsize must be a multiple of 16 bytes for this q/k/v layout");
    const bool inter = p->layout == VTX_QKV_INTERLEAVED;
    CUtensorMap tmap;
    const __nv_bfloat16* u_first = static_cast<const __nv_bfloat16*>(p->u) - p->u_hist_rows * p->u_stride_l;
    if (int rc = make_tmap_3d(&tmap, u_first, VTX_BF16, 3 * p->D, p->L + p->u_hist_rows, p->B, p->u_stride_l, p->u_stride_b,
                              inter ? 3 * CH : CH, BOX_ROWS, 0, "fused_iir"))
        return rc;
    const int variant = !inter ? 0 : (a.flip ? 2 : 1);
    auto kern = variant == 0 ? fused_li_kernel<false, false> : variant == 1 ? fused_li_kernel<true, false> : fused_li_kernel<true, true>;
    static bool attr_set[64][3] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_set[dev][variant]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return fail(VTX_ERR_LAUNCH, "fused_iir: shared memory opt-in: %s", cudaGetErrorString(e));
        if (dev >= 0 && dev < 64) attr_set[dev][variant] = true;
    }
    kern<<<(unsigned)(walks * a.nslice), THREADS, SMEM_BYTES, stream>>>(tmap, a);
    return check_launch("fused_iir");
}
