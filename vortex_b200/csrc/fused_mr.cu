// Hyena-MR fused block on tcgen05 / TMEM (bf16 I/O, filters of 17..128 taps, one per channel group of 16):
//   featurizer FIR (3 taps) -> q/k/v selection -> k*v -> grouped causal FIR -> (+ D*kv) -> q gate
// in one pass over HBM, channel-last in and out.
//
// The FIR is a blocked-Toeplitz contraction.  For a chunk of 128 output samples of one channel group
//   Y[128 x N] = [T^ | T][128 x 256] * KV[256 x N],   [T^|T][i][j] = h[128 + i - j]  (0 outside 0..K-1)
// where KV holds the previous and the current chunk of k*v.  The Toeplitz matrix depends on the group
// only, so it is expanded ONCE per CTA from the taps straight into tensor memory (A operand in TMEM,
// 128 lanes x 128 columns of packed bf16) and every tcgen05.mma reads only the data tile from shared
// memory.  A CTA owns one group and FOUR independent streams (a stream = one batch element and one
// segment of the time axis), so N = 4 x 16 channels; k*v is split into a bf16 head and a bf16 remainder
// (two MMAs accumulate into the same fp32 TMEM columns), which keeps the product exact to ~16 bits.
// The skip term D[c]*kv is one more K=16 MMA per stream against diag(D) with the same shared-memory
// tile read as a K-major A operand.
//
// Warp roles (14 warps): 0-7 front end (TMA-staged rows -> featurizer -> k*v head/remainder and q into
// the MMA tile), 8-11 epilogue (tcgen05.ld -> q gate -> bf16 -> global), 12 MMA issue, 13 TMA issue.
// A front-end lane owns one channel pair of one stream and walks 16 rows per chunk with the featurizer
// history in registers; the four streams of a warp are staged one row apart in shared memory, which makes
// every shared-memory access of the front end bank-conflict free.  All waits are bounded.
#include <cstdlib>

#include "tma.cuh"
#include "umma.cuh"

namespace vtx {

VTX_DEFINE_STATUS_READER()

int launch_fused_state_bf16(const vtx_fused_fir_params* p, cudaStream_t s);   // fused_fir.cu

namespace mr {

using namespace umma;

constexpr int NS = 4;                      // streams per CTA
constexpr int CH = 16;                     // channels per group
constexpr int CHUNK = 128;                 // output samples per MMA chunk
#ifndef VTX_MR_NFE
#define VTX_MR_NFE 8
#endif
constexpr int NFE = VTX_MR_NFE;                     // front-end warps (two per scheduler: the featurizer chain is latency-bound)
constexpr int WROWS = CHUNK / NFE;         // rows of a chunk owned by one front-end warp
#ifndef VTX_MR_RB
#define VTX_MR_RB 8
#endif
constexpr int RB = VTX_MR_RB;                     // rows a front-end lane fetches into registers at a time
constexpr int HROWS = 64;                  // rows per staged box: half a chunk, shared by two front-end warps
                                           // (the TMA unit retires ~12 boxes per microsecond and SM whatever their
                                           // size, so boxes are made as tall as the shared-memory budget allows)
constexpr int BOX_ROWS = HROWS + 2 + (NS - 1);         // featurizer halo + stream skew
constexpr int BOX_BYTES = BOX_ROWS * 3 * CH * 2;       // 6624
constexpr int IN_PLANE = (BOX_ROWS * 32 + 127) / 128 * 128;   // q | k | v planes of the non-interleaved layouts (TMA wants 128-byte aligned tiles)
constexpr int BOX_STRIDE = 3 * IN_PLANE;               // 6912 >= BOX_BYTES
#ifndef VTX_MR_IN_STAGES
#define VTX_MR_IN_STAGES 4
#endif
constexpr int IN_STAGES = VTX_MR_IN_STAGES;            // ring of half-chunk stages (a stage is handed back as soon as its rows sit
                                                       // in registers); HBM latency under load is ~2 us, so full bandwidth needs
                                                       // ~100 KB in flight per SM: the ring gets all the shared memory that is left
constexpr int STAGE_BYTES = NS * BOX_STRIDE;           // one stage: the four streams' boxes of one half chunk
// k*v tiles: [128 rows (time)][128 B = 64 channels] bf16 with the 128-byte swizzle (16-byte chunk c of row r is
// stored at chunk c ^ (r & 7)); the tensor core fetches such rows whole, whereas the unswizzled form is fetched
// 16 bytes at a time (measured: ~130 instead of ~32 cycles per MMA).  Tiles are 1024-byte aligned.
constexpr int KV_TILE = CHUNK * 128;       // 16384
// q tile: the gate is kept to 24 bits (sign, exponent, 15 mantissa bits: a bf16-rounded gate would by itself cost as
// much accuracy as the rounding of the output).  Upper 16 bits in a tile shaped like a k*v tile (same swizzle, so the
// front end reuses its store address), third byte in a [128 rows][64 B] tile whose 16-byte chunk c of row r sits at
// chunk c ^ ((r >> 1) & 3) (conflict-free for the row-per-lane 16-byte reads of the epilogue).
constexpr int QH_TILE = KV_TILE, QM_TILE = CHUNK * 64;
constexpr int Q_BYTES = QH_TILE + QM_TILE;     // 24576
constexpr int HI_OFF = 0, LO_OFF = KV_TILE, QH_OFF = 2 * KV_TILE;   // (third bytes of q follow at QH_OFF + QH_TILE)
constexpr int SLOT_BYTES = 2 * KV_TILE + Q_BYTES;      // one chunk: k*v head, k*v remainder, q upper halves, q third bytes
constexpr int DIAG_BYTES = 128;            // skip parameters D[16] of the group, fp32
constexpr int TAPS_BYTES = 384 * 2;        // zero-padded taps, bf16
constexpr int SMEM_IN = IN_STAGES * STAGE_BYTES;
constexpr int SMEM_SLOTS = 2 * SLOT_BYTES;
constexpr int OFF_SLOTS = SMEM_IN;
constexpr int OFF_DIAG = OFF_SLOTS + SMEM_SLOTS;
constexpr int OFF_TAPS = OFF_DIAG + DIAG_BYTES;
constexpr int OFF_BARS = OFF_TAPS + TAPS_BYTES;
constexpr int NBARS = IN_STAGES * 2 + 2 * 4 + 1;   // in_full/in_empty per stage; kv_full, slot_free, d_full, d_empty x2; a_ready
constexpr int SMEM_BYTES = OFF_BARS + NBARS * 8 + 16 + 1024;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
static_assert(OFF_SLOTS % 1024 == 0 && SLOT_BYTES % 1024 == 0, "k*v tiles must be 1024-byte aligned");
constexpr int TMEM_COLS = 512;             // A: [0,128); accumulator buffer b at 128 + 128 b: [head part 64 | remainder part 64]
#ifndef VTX_MR_NTMA
#define VTX_MR_NTMA 2
#endif
constexpr int NTMA = VTX_MR_NTMA;          // TMA issue warps: one thread issues a box of 96-byte rows every ~300 cycles only
constexpr int W_EP = NFE, W_MMA = NFE + 4, W_TMA = NFE + 5;   // first epilogue warp (multiple of 4), MMA warp, first TMA warp
constexpr int NWARPS = (NFE + 5 + NTMA + 3) / 4 * 4;    // whole warpgroups (register reallocation is per warpgroup)
constexpr int THREADS = 32 * NWARPS;
static_assert(NS % NTMA == 0 && THREADS <= 1024 && NFE % 8 == 0 && (CHUNK / NFE) % RB == 0, "warp roles");

// L2 prefetch of rows that will be staged later: keeps HBM requests in flight without shared memory
// (full HBM bandwidth needs ~100 KB in flight per SM; the staging ring holds a third of that).
__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

struct Args {
    const void* w3; int64_t w3_dtype;
    const void* h;  int64_t h_dtype;
    const void* bias; int64_t bias_dtype;
    const __nv_bfloat16* u; int64_t u_stride_b, u_stride_l;
    __nv_bfloat16* y; int64_t y_stride_b, y_stride_l;
    int64_t B, L, D, G, K;
    int64_t nseg, seg_len, nstream;        // streams per group = B * nseg
    int layout, flip, taps, has_bias;
    int64_t hd;
    int pf;          // chunks of L2 prefetch distance (0 = off)
    int dbg;         // diagnostic builds only: knock out parts of the kernel to time the rest
    unsigned long long* trace;   // diagnostic builds only
};

#ifdef VTX_MR_KNOCKOUT
#define KO(bit) (a.dbg & (bit))
#else
#define KO(bit) false
#endif

#ifdef VTX_MR_LANE0_WAIT
// One lane polls, the warp learns the outcome through a shuffle (the warp-level barrier inside it orders memory).
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, int code) {
    bool ok = true;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, code);
    return __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
}
#define WARP_WAIT warp_wait
#else
#define WARP_WAIT mbar_wait
#endif
#ifdef VTX_MR_SPIN
#undef WARP_WAIT
#define WARP_WAIT mbar_spin
#define MBAR_WAIT mbar_spin
#else
#define MBAR_WAIT mbar_wait
#endif

// Diagnostic builds only (-DVTX_MR_TRACE): CTA 0 logs (event, clock) pairs per warp into a.trace[warp][256].
#ifdef VTX_MR_TRACE
#define TRACE(code)                                                                              \
    do {                                                                                         \
        if (blockIdx.x == 0 && lane == 0 && a.trace && trace_n < 256)                            \
            a.trace[warp * 256 + trace_n++] = ((unsigned long long)(code) << 48) | (unsigned long long)(clock64() & 0xffffffffffffull); \
    } while (0)
#else
#define TRACE(code) do {} while (0)
#endif

struct Stream {
    int64_t b, ts, te;   // batch, first row, one past the last row this stream stores
    bool active;
};
__device__ __forceinline__ Stream stream_of(const Args& a, int64_t quad, int s) {
    Stream st;
    int64_t id = quad * NS + s;
    st.active = id < a.nstream;
    if (!st.active) id = a.nstream - 1;            // duplicate a real stream; its stores are suppressed
    st.b = id / a.nseg;
    st.ts = (id % a.nseg) * a.seg_len;
    st.te = st.ts + a.seg_len < a.L ? st.ts + a.seg_len : a.L;
    return st;
}

// SWAP: interleaved layout with the q and k roles exchanged (the planar layouts exchange their TMA columns instead).
template <bool INTERLEAVED, bool SWAP>
__global__ void __launch_bounds__(THREADS, 1) fused_mr_kernel(const __grid_constant__ CUtensorMap tmap, Args a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t sm_u = smem_u32(sm);
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + OFF_BARS);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + OFF_BARS + NBARS * 8);
    // barrier indices
    auto in_full = [&](int st) { return smem_u32(&bars[st * 2]); };
    auto in_empty = [&](int st) { return smem_u32(&bars[st * 2 + 1]); };
    const int BB = IN_STAGES * 2;
    auto kv_full = [&](int sl) { return smem_u32(&bars[BB + sl]); };
    // slot_free: the chunk in this slot is no longer needed.  Five arrivals: the four epilogue warps (k*v rows of the skip
    // term and the q tile read) and the MMA warp's commit behind the MMAs of the next chunk that read the k*v tile.
    auto slot_free = [&](int sl) { return smem_u32(&bars[BB + 2 + sl]); };
    auto d_full = [&](int sl) { return smem_u32(&bars[BB + 4 + sl]); };
    auto d_empty = [&](int sl) { return smem_u32(&bars[BB + 6 + sl]); };
    const uint32_t a_ready = smem_u32(&bars[BB + 8]);       // the Toeplitz operand is in TMEM (one arrival per expanding warp)

    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    int trace_n = 0;
    (void)trace_n;
    const int64_t g = blockIdx.x % a.G, quad = blockIdx.x / a.G;
    const int K = (int)a.K;
    const int nchunk = KO(512) ? 0 : (int)(a.seg_len / CHUNK) + 1;     // chunk 0 is the halo chunk (front end only)

    // ---------------- setup -------------------------------------------------------------------
    if (tid == 0) {
        for (int st = 0; st < IN_STAGES; ++st) { mbar_init(in_full(st), NTMA); mbar_init(in_empty(st), NFE / 2); }
        for (int sl = 0; sl < 2; ++sl) {
            mbar_init(kv_full(sl), NFE); mbar_init(slot_free(sl), 5); mbar_init(d_full(sl), 1); mbar_init(d_empty(sl), 4);
        }
        mbar_init(a_ready, NFE + 4);
        fence_mbar_init();
    }
    if (warp == W_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    {   // taps, zero padded: tp[m] = tap at lag (m - 128), lags outside [0, K) are zero
        __nv_bfloat16* tp = reinterpret_cast<__nv_bfloat16*>(sm + OFF_TAPS);
        for (int m = tid; m < 384; m += THREADS) {
            int l = m - 128;
            float v = 0.f;
            if (l >= 0 && l < K) v = ld_param(a.h, a.h_dtype, g * K + (a.taps == VTX_TAPS_CONV ? l : K - 1 - l));
            tp[m] = __float2bfloat16_rn(v);
        }
        float* dsk = reinterpret_cast<float*>(sm + OFF_DIAG);                 // skip parameters of this group, fp32
        for (int c = tid; c < CH; c += THREADS) dsk[c] = a.has_bias ? ld_param(a.bias, a.bias_dtype, g * CH + c) : 0.f;
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp < NFE + 4) {
        // Expand the Toeplitz matrix into TMEM: lane i holds row i.  A warp reaches the TMEM lanes of its quarter
        // (warp % 4); the front-end and epilogue warps of a quarter share its 8 column blocks.  Only the MMA warp
        // waits for the result (a_ready): the TMA warps start fetching at once and the other roles follow as soon as
        // their share is written.
        const int i = (warp % 4) * 32 + lane, part = warp / 4, nparts = (NFE + 4) / 4;
        const uint16_t* tp = reinterpret_cast<const uint16_t*>(sm + OFF_TAPS);
        for (int c0 = 16 * part; c0 < 128; c0 += 16 * nparts) {
            uint32_t v[16];
#pragma unroll
            for (int m = 0; m < 16; ++m) {
                int j = 2 * (c0 + m);                                  // columns j, j+1 of [T^|T]: lag = 128 + i - j
                uint32_t e0 = tp[128 + 128 + i - j], e1 = tp[128 + 127 + i - j];
                v[m] = e1 << 16 | e0;
            }
            tmem_st16(tmem + ((uint32_t)((warp % 4) * 32) << 16) + c0, v);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(a_ready);
    }

    // ---------------- roles ---------------------------------------------------------------------
    if (warp < NFE) {
        // ======== front end: warp w owns rows [16w, 16w+16) of every chunk =========================
        const int w = warp, p = lane % 8, s = lane / 8;
        const Stream st = stream_of(a, quad, s);
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
        const uint32_t qm_in = (uint32_t)(2 * p);                                          // this lane's two third-bytes in the 16-byte chunk s of a q row
        static_assert(WROWS == 2 * RB, "the front end walks a chunk as two register batches");
        constexpr int ROWB = INTERLEAVED ? 96 : 32;             // bytes per staged row (per plane in the planar layouts)
        // shared-memory address of this lane's first word of batch hb of chunk k (the box row of the batch's first
        // sample minus the two featurizer history rows; stream s was staged s rows early)
        auto box_addr = [&](int k, int hb) {
            const int nh = 2 * k + w / (NFE / 2), stg = nh % IN_STAGES;
            return sm_u + (uint32_t)(stg * STAGE_BYTES + s * BOX_STRIDE + ((w % (NFE / 2)) * WROWS + hb * RB + s) * ROWB +
                                     (INTERLEAVED ? 12 : 4) * p);
        };
        // Volatile loads: they are issued where they stand, one batch ahead of the arithmetic that consumes them, so
        // that their latency (and the wait for the stage before them) overlaps the previous batch's arithmetic.
        auto fetch = [&](uint32_t addr, uint32_t (&raw)[RB + 2][3]) {
#pragma unroll
            for (int r = 0; r < RB + 2; ++r) {
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    if (KO(2))
                        raw[r][j] = 0x3f803f80u + r + lane;
                    else
                        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(raw[r][j]) : "r"(addr + (uint32_t)(r * ROWB + (INTERLEAVED ? 4 * j : j * IN_PLANE))));
                }
            }
        };
        // x[0..2] = q | k | v samples of the lane's channel pair (packed positions before any q/k swap)
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
        // featurizer -> k*v head/remainder and q of RB rows, written into the chunk's slot
        auto compute = [&](int slot, int hb, const uint32_t (&raw)[RB + 2][3]) {
            const uint32_t row0 = (uint32_t)(w * WROWS + hb * RB);
            const uint32_t slot_u = sm_u + OFF_SLOTS + slot * SLOT_BYTES;
            // Tiles are 1024-byte aligned, so the swizzle (16-byte chunk index XOR row phase) is one XOR on the address
            // of the lane's element in row 0; row offsets are compile-time immediates of the stores.
            const uint32_t kv_a0 = slot_u + (kv_chunk << 4) + kv_in + row0 * 128;
            const uint32_t qh_a0 = kv_a0 + QH_OFF;
            const uint32_t qm_a0 = slot_u + QH_OFF + QH_TILE + ((uint32_t)s << 4) + qm_in + row0 * 64;
            f32x2 x1[3], x2[3];
            unpack(raw[0], x2);
            unpack(raw[1], x1);
#pragma unroll
            for (int i = 0; i < RB; ++i) {
                if (KO(16)) {
                    asm volatile("st.shared.b32 [%0], %1;" ::"r"(kv_a0 + i * 128), "r"(raw[i + 2][0]));
                    continue;
                }
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
                // row0 is a multiple of 8, so the swizzle phase of row row0 + i is i & 7
                const uint32_t kaddr = kv_a0 ^ (uint32_t)((i & 7) << 4);
                if (KO(1) && hi != 0x12345678u) continue;
                asm volatile("st.shared.b32 [%0], %1;" ::"r"(kaddr + (HI_OFF + i * 128)), "r"(hi));
                asm volatile("st.shared.b32 [%0], %1;" ::"r"(kaddr + (LO_OFF + i * 128)), "r"(lo));
                float q0, q1;
                up2(q, q0, q1);
                const uint32_t qh = __byte_perm(__float_as_uint(q0), __float_as_uint(q1), 0x7632);   // upper halves
                const uint32_t qm = __byte_perm(__float_as_uint(q0), __float_as_uint(q1), 0x5151);   // third bytes
                asm volatile("st.shared.b32 [%0], %1;" ::"r"((qh_a0 ^ (uint32_t)((i & 7) << 4)) + i * 128), "r"(qh));
                asm volatile("st.shared.u16 [%0], %1;" ::"r"((qm_a0 ^ (uint32_t)(((i >> 1) & 3) << 4)) + i * 64), "h"((unsigned short)qm));
            }
        };
        auto stage_of = [&](int k) { return (2 * k + w / (NFE / 2)) % IN_STAGES; };
        auto stage_parity = [&](int k) { return (uint32_t)(((2 * k + w / (NFE / 2)) / IN_STAGES) & 1); };

        // Software pipeline over register batches A (rows 0..RB-1 of the warp's rows) and B (the rest):
        //   fetch B(k) | wait slot | compute A(k) | release stage | wait stage(k+1), fetch A(k+1) | compute B(k) | publish
        uint32_t rawA[RB + 2][3], rawB[RB + 2][3];
        bool ok = KO(128) || WARP_WAIT(in_full(stage_of(0)), stage_parity(0), 4);
        if (ok) fetch(box_addr(0, 0), rawA);
        for (int k = 0; k < nchunk && ok; ++k) {
            const int slot = k % 2;
            TRACE(0);
            fetch(box_addr(k, 1), rawB);
            // slot reuse: the MMAs that read chunk k-2 and the epilogue that read its k*v rows and q tile are done
            if (k >= 2 && !WARP_WAIT(slot_free(slot), (uint32_t)(((k - 2) / 2) & 1), 2)) break;
            TRACE(1);
            compute(slot, 0, rawA);
            // Every row this warp needs from the stage now sits in registers: hand the stage back to the TMA warp (HBM
            // latency under load is ~2 us, so as much of the ring as possible should be in flight).  The empty asm
            // makes the loaded values a dependency of the arrive.
#pragma unroll
            for (int r = 0; r < RB + 2; ++r) asm volatile("" ::"r"(rawB[r][0]), "r"(rawB[r][1]), "r"(rawB[r][2]));
            __syncwarp();
            if (lane == 0 && !KO(128)) mbar_arrive(in_empty(stage_of(k)));
            TRACE(3);
            if (k + 1 < nchunk) {
                if (!KO(128) && !WARP_WAIT(in_full(stage_of(k + 1)), stage_parity(k + 1), 4)) break;
                fetch(box_addr(k + 1, 0), rawA);
            }
            TRACE(2);
            compute(slot, 1, rawB);
            TRACE(4);
            fence_proxy_async_smem();      // generic-proxy writes -> visible to the tensor core's async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(kv_full(slot));
            TRACE(5);
        }
    } else if (warp < W_EP + 4) {
        // ======== epilogue: thread = output row (TMEM lane) ========================================
        const int e = warp - W_EP, r = e * 32 + lane;
        // per stream: pointer to this thread's first output row and the number of rows of the segment from there on
        // (<= 0: nothing to store).  Kept as one pointer and one int per stream to save registers.
        __nv_bfloat16* yrow[NS];
        int nleft[NS];
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            const Stream st = stream_of(a, quad, s);
            yrow[s] = a.y + st.b * a.y_stride_b + (st.ts + r) * a.y_stride_l + g * CH;
            nleft[s] = st.active ? (int)(st.te - st.ts) - r : 0;
        }
        const float4* dsk = reinterpret_cast<const float4*>(sm + OFF_DIAG);    // skip parameters D[g*16 .. +16), fp32
        bool has_skip = false;       // the skip parameter is all zeros at initialisation: then its term is not evaluated
#pragma unroll
        for (int c = 0; c < CH / 4; ++c) {
            const float4 d = dsk[c];
            has_skip = has_skip || d.x != 0.f || d.y != 0.f || d.z != 0.f || d.w != 0.f;
        }
        const int64_t chunk_pitch = (int64_t)CHUNK * a.y_stride_l;
        if (lane == 0) mbar_arrive(slot_free(0));      // chunk 0 (the halo chunk) has no epilogue
        for (int k = 1; k < nchunk; ++k) {
            const int slot = k % 2;
            TRACE(10);
            if (!WARP_WAIT(d_full(slot), (uint32_t)(((k - 1) / 2) & 1), 5)) break;
            TRACE(11);
            tc_fence_after();
            __syncwarp();
            const uint32_t taddr = tmem + ((uint32_t)(e * 32) << 16) + 128 + slot * 128;
            const uint8_t* slot_p = sm + OFF_SLOTS + slot * SLOT_BYTES;
            const uint8_t* qh_p = slot_p + QH_OFF + r * 128;
            const uint8_t* qm_p = qh_p + QH_TILE - r * 64;
            const int64_t yoff = (int64_t)(k - 1) * chunk_pitch;
            // One stream at a time (16 channels: head and remainder accumulators -> gate -> 32 bytes of output), with the
            // accumulators of the next stream already on their way from TMEM: at most two streams' values are live, so
            // nothing spills (a spilled value is reloaded from L2 here: L1 is almost entirely carved out as shared memory).
#ifdef VTX_MR_EP_UNROLLED
            uint32_t acc[2][2][16];
            tmem_ld16(taddr, acc[0][0]);
            tmem_ld16(taddr + 64, acc[0][1]);
#pragma unroll
            for (int s = 0; s < NS; ++s) {
                uint32_t (&ah)[16] = acc[s & 1][0];
                uint32_t (&al)[16] = acc[s & 1][1];
                tmem_ld_wait(ah, al);
                if (s + 1 < NS) {
                    tmem_ld16(taddr + (s + 1) * 16, acc[(s + 1) & 1][0]);
                    tmem_ld16(taddr + 64 + (s + 1) * 16, acc[(s + 1) & 1][1]);
                } else {
#else
            // (rolled over the streams: keeps the instruction-cache footprint of this role small)
#pragma unroll 1
            for (int s = 0; s < NS; ++s) {
                uint32_t ah[16], al[16];
                tmem_ld16(taddr + s * 16, ah);
                tmem_ld16(taddr + 64 + s * 16, al);
                tmem_ld_wait(ah, al);
                if (s + 1 == NS) {
#endif
                    // every accumulator of this chunk has left TMEM: hand the buffer back to the MMA warp
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(d_empty(slot));
                    TRACE(12);
                }
                // this stream's output pointer and row count (selects, not indexed arrays: the loop may be rolled)
                __nv_bfloat16* ys = yrow[0];
                int nl = nleft[0];
#pragma unroll
                for (int t = 1; t < NS; ++t)
                    if (s == t) { ys = yrow[t]; nl = nleft[t]; }
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
                if (KO(32)) continue;
                uint32_t o[8];
                const uint4 qm4 = *reinterpret_cast<const uint4*>(qm_p + ((s ^ ((r >> 1) & 3)) << 4));
                const uint32_t qm[4] = {qm4.x, qm4.y, qm4.z, qm4.w};
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    const uint4 qh4 = *reinterpret_cast<const uint4*>(qh_p + (((2 * s + hf) ^ (r & 7)) << 4));
                    const uint32_t qh[4] = {qh4.x, qh4.y, qh4.z, qh4.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {          // channels 8 hf + 2 j, + 1: third bytes 2 (j % 2), + 1 of word 2 hf + j / 2
                        const uint32_t mw = qm[2 * hf + j / 2];
                        const uint32_t qa = __byte_perm(qh[j], mw, (j % 2) ? 0x1066 : 0x1044);
                        const uint32_t qb = __byte_perm(qh[j], mw, (j % 2) ? 0x3277 : 0x3255);
                        float o0, o1;
                        up2(mul2(y[4 * hf + j], pk2(__uint_as_float(qa), __uint_as_float(qb))), o0, o1);
                        o[4 * hf + j] = pack_bf16(o0, o1);
                    }
                }
                // (no "memory" clobber: nothing in this kernel reads y, and the shared-memory reads of the next stream
                // may then be scheduled above this store)
#ifdef VTX_MR_CHECK
                {   // diagnostic builds: a store outside y is recorded and skipped
                    const int64_t off = (ys + yoff) - a.y;
                    if ((k - 1) * CHUNK < nl && (off < 0 || off + 16 > a.B * a.y_stride_b)) {
                        atomicCAS(&g_device_status, 0, 21);
                        continue;
                    }
                }
#endif
                if ((k - 1) * CHUNK < nl && !(KO(4) && o[0] != 0x12345678u))
                    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ys + yoff), "r"(o[0]),
                                 "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]));
            }
            // every shared-memory read of this chunk is done: its k*v slot and q tile may be rewritten
            __syncwarp();
            if (lane == 0) mbar_arrive(slot_free(slot));
            TRACE(13);
        }
    } else if (warp == W_MMA) {
        // ======== MMA issue =========================================================================
        if (lane == 0) {
            const uint32_t idesc = instr_desc(128, 2 * NS * CH, 1);
            // Chunk k accumulates into D[k%2]:  prev(k) = T^ * kv(k-1)  and  cur(k) = T * kv(k) (+ skip).
            // prev(k+1) is issued right behind cur(k), long before chunk k+1 is staged, so the tile of chunk k
            // is released (slot_free) one whole chunk before the front end needs its slot again.
            // Descriptors are built once; a K step of 16 rows moves the start-address field by 2048 B (128 units).
            // The issue loop is fully unrolled: the issuing thread is on the critical path of every chunk.
            // B operand of one K step: 16 rows x [head tile | remainder tile] = N-major, two 64-channel atoms
            // KV_TILE bytes apart (LBO), 8-row groups 1024 B apart (SBO), 128-byte swizzle.  N = 128 per MMA:
            // narrower MMAs run at a fixed ~70 cycles each at this tile height, so both parts go into one.
            uint64_t kv_desc[2];
#pragma unroll
            for (int sl = 0; sl < 2; ++sl) kv_desc[sl] = smem_desc(sm_u + OFF_SLOTS + sl * SLOT_BYTES + HI_OFF, KV_TILE, 1024, 2);
            auto issue_half = [&](int k, bool cur) {
                const int slot = cur ? k % 2 : (k - 1) % 2;
                const uint32_t d = tmem + 128 + (k % 2) * 128;
                const uint32_t a0 = tmem + (cur ? 64 : 0);
                const uint64_t dk = slot ? kv_desc[1] : kv_desc[0];
                const int nj = KO(64) ? 0 : KO(8) ? 1 : 8;
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) {
                    if (jj >= nj) continue;
                    // the first MMA of a chunk (K step 0 of the previous-chunk part) overwrites the accumulator
                    mma_ts(d, a0 + 8 * jj, dk + (uint64_t)(jj * (16 * 128 / 16)), idesc, (cur || jj > 0) ? 1u : 0u);
                }
            };
            bool ok = MBAR_WAIT(a_ready, 0, 10) && MBAR_WAIT(kv_full(0), 0, 7);          // the Toeplitz operand; the halo chunk
            if (ok && nchunk > 1) {
                tc_fence_after();
                issue_half(1, false);
                mma_commit(slot_free(0));
            }
            for (int k = 1; k < nchunk && ok; ++k) {
                TRACE(20);
                if (!MBAR_WAIT(kv_full(k % 2), (uint32_t)((k / 2) & 1), 6)) break;
                TRACE(21);
                tc_fence_after();
                issue_half(k, true);
                mma_commit(d_full(k % 2));
                TRACE(22);
                if (k + 1 < nchunk) {
                    // D[(k+1)%2] was last read by the epilogue of chunk k-1
                    if (k + 1 >= 3 && !MBAR_WAIT(d_empty((k + 1) % 2), (uint32_t)(((k - 2) / 2) & 1), 8)) break;
                    TRACE(23);
                    tc_fence_after();
                    issue_half(k + 1, false);
                }
                mma_commit(slot_free(k % 2));
                TRACE(24);
            }
        }
    } else if (warp < W_TMA + NTMA) {
        // first packed column of this group's q | k | v data (one contiguous run when interleaved)
        int row_base[NS], bidx[NS];      // first staged row of chunk 0 (the halo chunk) and batch index, per stream
        int col[3] = {0, 0, 0};
#pragma unroll
        for (int s = 0; s < NS; ++s) {
            const Stream st = stream_of(a, quad, s);
            row_base[s] = (int)st.ts - CHUNK - 2 - s;
            bidx[s] = (int)st.b;
        }
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
            for (int nh = 0; nh < 2 * nchunk; ++nh) {
                if (KO(128)) break;
                const int stg = nh % IN_STAGES, k = nh / 2, h = nh % 2;
                if (nh >= IN_STAGES && !MBAR_WAIT(in_empty(stg), (uint32_t)(((nh - IN_STAGES) / IN_STAGES) & 1), 9)) break;
                TRACE(30);
                const uint32_t bar = in_full(stg);
                mbar_expect_tx(bar, NS / NTMA * BOX_BYTES);
#pragma unroll
                for (int s = 0; s < NS; ++s) {
                    if (s % NTMA != tw) continue;
                    const uint32_t dst = sm_u + (uint32_t)(stg * STAGE_BYTES + s * BOX_STRIDE);
                    const int row = row_base[s] + k * CHUNK + h * HROWS;
                    if (INTERLEAVED) {
                        tma_load_3d(dst, &tmap, bar, col[0], row, bidx[s]);
                    } else {
#pragma unroll
                        for (int pl = 0; pl < 3; ++pl)
                            tma_load_3d(dst + pl * IN_PLANE, &tmap, bar, col[pl], row, bidx[s]);
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

}  // namespace mr

int fused_mr_tc_fwd(const vtx_fused_fir_params* p, cudaStream_t stream) {
    using namespace mr;
    VTX_REQUIRE(p->io_dtype == VTX_BF16, VTX_ERR_UNSUPPORTED, "fused_fir: the tensor-core path takes bf16 I/O");
    VTX_REQUIRE(p->K <= CHUNK, VTX_ERR_UNSUPPORTED, "fused_fir: filter length %lld > %d", (long long)p->K, CHUNK);
    VTX_REQUIRE(p->D == p->G * CH, VTX_ERR_UNSUPPORTED, "fused_fir: the tensor-core path needs groups of %d channels", CH);
    VTX_REQUIRE(p->K3 == 3 && !p->b3, VTX_ERR_UNSUPPORTED, "fused_fir: tensor-core path needs a 3-tap featurizer without bias");
    VTX_REQUIRE(p->bias_mode != VTX_BIAS_ADD, VTX_ERR_UNSUPPORTED, "fused_fir: additive bias is not fused on this path");
    VTX_REQUIRE((reinterpret_cast<uintptr_t>(p->y) % 32) == 0 && (p->y_stride_l % 16) == 0 && (p->y_stride_b % 16) == 0,
                VTX_ERR_ALIGNMENT, "fused_fir: y rows must be 32-byte aligned");
    Args a{};
    a.w3 = p->w3; a.w3_dtype = p->w3_dtype; a.h = p->h; a.h_dtype = p->h_dtype;
    a.bias = p->bias; a.bias_dtype = p->bias_dtype; a.has_bias = p->bias_mode == VTX_BIAS_GATED;
    a.u = static_cast<const __nv_bfloat16*>(p->u); a.u_stride_b = p->u_stride_b; a.u_stride_l = p->u_stride_l;
    a.y = static_cast<__nv_bfloat16*>(p->y); a.y_stride_b = p->y_stride_b; a.y_stride_l = p->y_stride_l;
    a.B = p->B; a.L = p->L; a.D = p->D; a.G = p->G; a.K = p->K;
    a.layout = (int)p->layout; a.flip = p->flip_x1x2 != 0; a.taps = (int)p->taps;
    a.hd = p->D;
    a.pf = getenv("VTX_MR_PF") ? atoi(getenv("VTX_MR_PF")) : 0;
    a.dbg = getenv("VTX_MR_DBG") ? atoi(getenv("VTX_MR_DBG")) : 0;
    a.trace = getenv("VTX_MR_TRACE_PTR") ? (unsigned long long*)strtoull(getenv("VTX_MR_TRACE_PTR"), nullptr, 0) : nullptr;
    if (p->layout == VTX_QKV_COLUMN_SPLIT) {
        VTX_REQUIRE(p->num_heads > 0 && p->D % p->num_heads == 0, VTX_ERR_BAD_ARG, "fused_fir: bad num_heads");
        a.hd = p->D / p->num_heads;
        VTX_REQUIRE(a.hd % CH == 0, VTX_ERR_UNSUPPORTED, "fused_fir: column split needs head size %% %d == 0", CH);
    }
    VTX_REQUIRE(p->layout == VTX_QKV_INTERLEAVED || (p->D * 2) % 16 == 0, VTX_ERR_ALIGNMENT,
                "fused_fir: D*itemsize must be a multiple of 16 bytes for this q/k/v layout");
    // segments: enough CTAs (group x stream quads) for ~7 rounds over the SMs, whole chunks each
    const int64_t nchunks_total = ceil_div<int64_t>(p->L, CHUNK);
    int64_t nseg = 1;
    while (p->G * ceil_div<int64_t>(p->B * nseg, NS) < (int64_t)kNumSMs * 6 && nseg * 2 <= nchunks_total &&
           ceil_div<int64_t>(nchunks_total, nseg * 2) >= 8)
        nseg *= 2;
#ifdef VTX_MR_KNOCKOUT
    if (getenv("VTX_MR_NSEG")) nseg = atoi(getenv("VTX_MR_NSEG"));
#endif
    a.seg_len = ceil_div<int64_t>(nchunks_total, nseg) * CHUNK;
    a.nseg = ceil_div<int64_t>(p->L, a.seg_len);
    a.nstream = p->B * a.nseg;
    const int64_t nquad = ceil_div<int64_t>(a.nstream, NS);
    VTX_REQUIRE(p->G * nquad < (int64_t)1 << 31, VTX_ERR_UNSUPPORTED, "fused_fir: too many work items");

    const bool inter = p->layout == VTX_QKV_INTERLEAVED;
    CUtensorMap tmap;
    if (int rc = make_tmap_3d(&tmap, p->u, VTX_BF16, 3 * p->D, p->L, p->B, p->u_stride_l, p->u_stride_b,
                              inter ? 3 * CH : CH, BOX_ROWS, 0, "fused_fir(mr)"))
        return rc;
    const int variant = !inter ? 0 : (a.flip ? 2 : 1);
    auto kern = variant == 0 ? fused_mr_kernel<false, false> : variant == 1 ? fused_mr_kernel<true, false> : fused_mr_kernel<true, true>;
    // the opt-in is a per-device property of the function: remember it per device
    static bool attr_set[64][3] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_set[dev][variant]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return fail(VTX_ERR_LAUNCH, "fused_fir(mr): shared memory opt-in: %s", cudaGetErrorString(e));
        if (dev >= 0 && dev < 64) attr_set[dev][variant] = true;
    }
    kern<<<(unsigned)(p->G * nquad), THREADS, SMEM_BYTES, stream>>>(tmap, a);
    if (int rc = check_launch("fused_fir(mr)")) return rc;
    if (p->fir_state || p->inner_state) return launch_fused_state_bf16(p, stream);
    return VTX_OK;
}

}  // namespace vtx
