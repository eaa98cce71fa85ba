// Hyena-MR / Hyena-SE fused block on tcgen05 / TMEM (bf16 I/O, filters of up to 128 taps, one per group of 16 channels):
//   featurizer FIR (3 taps) -> q/k/v selection -> k*v -> grouped causal FIR -> (+ D*kv) -> q gate
// in one pass over HBM, channel-last in and out; the prefill caches fall out of the same launch.
//
// The FIR is a blocked-Toeplitz contraction.  For a chunk of 128 output samples of one channel group
//   Y[128 x N] = [T^ | T][128 x 256] * KV[256 x N],   [T^|T][i][j] = h[128 + i - j]  (0 outside 0..K-1)
// where KV holds the previous and the current chunk of k*v.  The Toeplitz matrix depends on the group
// only: it is expanded from the taps straight into tensor memory (A operand in TMEM, 128 lanes x 128 columns of
// packed fp16) and every tcgen05.mma reads only the data tile from shared memory.  A work item is one group and
// FOUR independent streams (a stream = one batch element and one segment of the time axis), so N = 4 x 16 channels.
//
// Precision.  The output is rounded to bf16 once (1.7e-3 relative L2 on its own), so nothing else may lose more than
// a few 1e-4: the featurizer runs in fp32, k*v and the gate q cross shared memory as fp16 (11 significant bits,
// 2.8e-4 each; bf16 would cost 1.1e-3 each), bf16 taps are exact in fp16 (8 of its 11 bits) and the accumulation is
// fp32.  fp16 has a narrow range, so k*v is carried scaled by 2^-6 (the featurizer taps of v are scaled when they are
// staged, the Toeplitz operand and the skip parameter by 2^6: powers of two, exact): k*v up to 4e6 and down to 4e-6
// keeps its bits, taps between 1e-6 and 1e3 keep theirs (smaller ones lose bits they contribute nothing with);
// conversions saturate instead of overflowing, q beyond +-65504 is clamped.
//
// One persistent CTA per SM walks through its work items (blockIdx, blockIdx + gridDim, ...: at any time the CTAs of
// the launch read neighbouring groups of the same rows).  Warp roles (16 warps): 0-7 front end (TMA-staged rows ->
// featurizer -> k*v and q as fp16 into the chunk's slot), 8-11 epilogue (tcgen05.ld -> skip -> q gate -> bf16 ->
// global; they also expand the NEXT item's Toeplitz operand into the other half of a TMEM double buffer while the
// current item streams), 12 MMA issue, 13-14 TMA issue, 15 prefill caches (the last two input rows of every sequence,
// and its last K-1 samples of k*v read back from the tiles the front end publishes).  A front-end lane owns one channel pair of one stream and walks 16 rows per chunk in two register
// batches, the next batch fetched before the current one is computed; the four streams of a warp are staged one
// row apart in shared memory so that the lanes of a warp read distinct banks.  All waits are bounded.
#include <cstdint>

#include "tma.cuh"
#include "umma.cuh"

namespace vtx {

VTX_DEFINE_STATUS_READER()

namespace mr {

using namespace umma;

constexpr int NS = 4;                      // streams per CTA
constexpr int CH = 16;                     // channels per group
constexpr int CHUNK = 128;                 // output samples per MMA chunk
#ifndef VTX_MR_NFE
#define VTX_MR_NFE 8
#endif
constexpr int NFE = VTX_MR_NFE;            // front-end warps (two per scheduler: the featurizer chain is latency-bound)
constexpr int WROWS = CHUNK / NFE;         // rows of a chunk owned by one front-end warp
constexpr int RB = 8;                      // rows a front-end lane fetches into registers at a time
constexpr int HROWS = 64;                  // rows per staged box: half a chunk, shared by two front-end warps
                                           // (the TMA unit retires ~12 boxes per microsecond and SM whatever their
                                           // size, so boxes are made as tall as the shared-memory budget allows)
constexpr int BOX_ROWS = HROWS + 2 + (NS - 1);         // featurizer halo + stream skew
constexpr int BOX_BYTES = BOX_ROWS * 3 * CH * 2;       // 6624
constexpr int IN_PLANE = (BOX_ROWS * 32 + 127) / 128 * 128;   // q | k | v planes of the non-interleaved layouts (TMA wants 128-byte aligned tiles)
constexpr float KV_SCALE = 0.015625f, KV_UNSCALE = 64.f;      // k*v crosses shared memory as fp16 scaled by 2^-6

// k*v and q tiles of a chunk: [128 rows (time)][128 B = 64 channels] fp16 with the 128-byte swizzle (16-byte chunk c of
// row r is stored at chunk c ^ (r & 7)); the tensor core fetches such rows whole, whereas the unswizzled form is fetched
// 16 bytes at a time (measured: ~130 instead of ~32 cycles per MMA).  Tiles are 1024-byte aligned.  The same swizzle
// makes the row-per-lane 16-byte reads of the epilogue conflict-free.
constexpr int KV_TILE = CHUNK * 128;       // 16384
constexpr int Q_OFF = KV_TILE;
constexpr int SLOT_BYTES = 2 * KV_TILE;    // one chunk: k*v tile, q tile
constexpr int DIAG_BYTES = 2 * 64;         // skip parameters D[16] of the group (times 2^6), fp32; two buffers (this item, next item)
constexpr int TAPS_BYTES = 2 * 384 * 2;    // zero-padded taps (times 2^6), fp16; two buffers
constexpr int W3S_BYTES = 3 * 3 * CH * 4;  // featurizer taps of a group as fp32 [q|k|v][tap][channel]; two buffers

// Shared-memory plan.  HBM latency under load is ~2 us, so full bandwidth needs ~100 KB in flight per SM: the ring of
// half-chunk stages (a stage is handed back as soon as its rows sit in registers) gets all the memory the two chunk
// slots leave.  The planar q | k | v layouts stage three 128-byte aligned planes per box, the interleaved layout one.
template <bool INTERLEAVED>
struct Lay {
    static constexpr int BOX_STRIDE = INTERLEAVED ? (BOX_BYTES + 127) / 128 * 128 : 3 * IN_PLANE;   // 6656 : 6912
    static constexpr int IN_STAGES = INTERLEAVED ? 6 : 5;
    static constexpr int STAGE_BYTES = NS * BOX_STRIDE;           // the four streams' boxes of one half chunk
    static constexpr int OFF_SLOTS = IN_STAGES * STAGE_BYTES;
    static constexpr int OFF_DIAG = OFF_SLOTS + 2 * SLOT_BYTES;
    static constexpr int OFF_TAPS = OFF_DIAG + DIAG_BYTES;
    static constexpr int OFF_W3S = OFF_TAPS + TAPS_BYTES;
    static constexpr int OFF_BARS = OFF_W3S + 2 * W3S_BYTES;
    static constexpr int NBARS = IN_STAGES * 2 + 2 * 6;   // in_full/in_empty per stage; kv_full, slot_free, d_full, d_empty, a_ready, taps_ready x2
    static constexpr int OFF_TSLOT = OFF_BARS + NBARS * 8;
    static constexpr int SMEM_BYTES = OFF_TSLOT + 48 + 1024;
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
    static_assert(OFF_SLOTS % 1024 == 0, "k*v tiles must be 1024-byte aligned");
    static_assert((BOX_STRIDE / 4) % 32 == 0 && BOX_STRIDE % 128 == 0, "stream boxes start on bank 0 and on a TMA boundary");
};
constexpr int TMEM_COLS = 512;             // Toeplitz operand of item t at 128 (t & 1); accumulator buffer b at 256 + 64 b
constexpr int D_COL = 256;
constexpr int NTMA = 2;                    // TMA issue warps: one thread issues a box of 96-byte rows every ~300 cycles only
constexpr int W_EP = NFE, W_MMA = NFE + 4, W_TMA = NFE + 5, W_STATE = NFE + 5 + NTMA;   // first epilogue warp (multiple of 4), MMA, first TMA, cache warp
constexpr int NWARPS = (W_STATE + 1 + 3) / 4 * 4;       // whole warpgroups
constexpr int THREADS = 32 * NWARPS;
static_assert(NS % NTMA == 0 && THREADS <= 1024 && NFE % 8 == 0 && WROWS == 2 * RB, "warp roles");

struct Args {
    const void* w3; int64_t w3_dtype;
    const void* h;  int64_t h_dtype;
    const void* bias; int64_t bias_dtype;
    const __nv_bfloat16* u; int64_t u_stride_b, u_stride_l;
    __nv_bfloat16* y; int64_t y_stride_b, y_stride_l;
    __nv_bfloat16* fir_state; __nv_bfloat16* inner_state;    // prefill caches, or null
    int64_t B, L, D, G, K;
    int64_t nseg, seg_len, nstream;        // streams per group = B * nseg
    int64_t nquad, nitems;                 // stream quads per group; work items (group x quad) of the call
    int64_t item0, item1;                  // the items of this launch
    int layout, flip, taps, has_bias;
    int64_t hd;
    int hist;        // rows before u[b][0] that hold the sequence's earlier samples (the tensor map starts there)
    int64_t dg;      // channels that share a filter (a multiple of 16): the filter of group g is h[16 g / dg]
};

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

// instruction descriptor: f32 accumulate, A fp16 (K-major, from TMEM), B fp16 (N-major).  Both operands have the same
// format: a descriptor that asked for bf16 x fp16 raised "illegal instruction" on this part.
__device__ __forceinline__ uint32_t instr_desc_f16(int M, int N) {
    return (1u << 4) | (0u << 7) | (0u << 10) | (1u << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// taps and other parameters -> fp16 bits, clamped to the finite range
__device__ __forceinline__ uint16_t f16_bits(float v) {
    return __half_as_ushort(__float2half_rn(fminf(fmaxf(v, -65504.f), 65504.f)));
}

// SWAP: interleaved layout with the q and k roles exchanged (the planar layouts exchange their TMA columns instead).
// FEAT = false: the gate-conv-gate operator on its own, on three channel-last operands q, k, v [B, L, D] that are
// already featurised (the hyena_ops (bs, l, g, dg) convention, vortex/ops/hyena_se/fwd.py:56-64): no featurizer in
// the front end, one tensor map per operand (planes of the planar staging), and the reference's rounding points --
// k*v and the filter output are rounded to bf16 where ref_fwd.py:80-127 materialises them.
template <bool INTERLEAVED, bool SWAP, bool FEAT>
__global__ void __launch_bounds__(THREADS, 1) fused_mr_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ CUtensorMap tmap_k,
                                                              const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ Args a) {
    static_assert(FEAT || (!INTERLEAVED && !SWAP), "the operator-only variant stages three planes");
    using LY = Lay<INTERLEAVED>;
    constexpr int IN_STAGES = LY::IN_STAGES, BOX_STRIDE = LY::BOX_STRIDE, STAGE_BYTES = LY::STAGE_BYTES;
    constexpr int OFF_SLOTS = LY::OFF_SLOTS, OFF_DIAG = LY::OFF_DIAG, OFF_TAPS = LY::OFF_TAPS, OFF_W3S = LY::OFF_W3S;
    extern __shared__ uint8_t smem_raw[];
    // Only the 32-bit shared-memory address of the (1024-byte aligned) buffer stays live; generic pointers are made
    // from it where a role needs one (the front end runs at the register limit).
    const uint32_t sm_u = (smem_u32(smem_raw) + 1023u) & ~1023u;
    auto smp = [&](uint32_t off) { return reinterpret_cast<uint8_t*>(__cvta_shared_to_generic(sm_u + off)); };
    // barrier addresses (32-bit shared-memory addresses: no generic pointer has to stay live in the role loops)
    const uint32_t bar_u = sm_u + LY::OFF_BARS;
    auto in_full = [&](int st) { return bar_u + 16u * (uint32_t)st; };
    auto in_empty = [&](int st) { return bar_u + 16u * (uint32_t)st + 8u; };
    constexpr uint32_t BB = IN_STAGES * 2;
    auto kv_full = [&](int sl) { return bar_u + 8u * (BB + (uint32_t)sl); };
    // slot_free: the chunk in this slot is no longer needed.  Six arrivals: the four epilogue warps (k*v rows of the skip
    // term and the q tile read), the cache warp, and the MMA warp's commit behind the MMAs of the next chunk that read
    // the k*v tile.
    auto slot_free = [&](int sl) { return bar_u + 8u * (BB + 2 + (uint32_t)sl); };
    auto d_full = [&](int sl) { return bar_u + 8u * (BB + 4 + (uint32_t)sl); };
    auto d_empty = [&](int sl) { return bar_u + 8u * (BB + 6 + (uint32_t)sl); };
    auto a_ready = [&](int ab) { return bar_u + 8u * (BB + 8 + (uint32_t)ab); };     // Toeplitz operand expanded (4 epilogue warps)
    auto taps_ready = [&](int ab) { return bar_u + 8u * (BB + 10 + (uint32_t)ab); };  // taps of the next item in shared memory (4 epilogue warps)

    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    // Persistent CTA: work items (item = quad * G + group) as many as the launch has blocks apart: at any time the CTAs
    // of the launch read neighbouring groups of the same rows, which keeps the concurrent reads inside few DRAM
    // pages.  Every item has its own group, hence its own Toeplitz operand: the epilogue warps expand the operand
    // of the NEXT item into the other half of a double buffer while the current item streams, so the roles run
    // through the items without draining.  Per-role running counters give the barrier phases.
    const int ncta = (int)gridDim.x;
    const int nmine = (int)((a.item1 - a.item0 - (int64_t)blockIdx.x + ncta - 1) / ncta);      // items item0 + blockIdx, + ncta, ...
    const int K = (int)a.K;
    const int nchunk = (int)(a.seg_len / CHUNK) + 1;     // chunk 0 of an item is its halo chunk (front end only)
    auto item_group = [&](int t) { return (int)((a.item0 + (int64_t)blockIdx.x + (int64_t)t * ncta) % a.G); };
    auto item_quad = [&](int t) { return (int)((a.item0 + (int64_t)blockIdx.x + (int64_t)t * ncta) / a.G); };

    // ---------------- setup -------------------------------------------------------------------
    if (tid == 0) {
        for (int st = 0; st < IN_STAGES; ++st) { mbar_init(in_full(st), NTMA); mbar_init(in_empty(st), NFE / 2); }
        for (int sl = 0; sl < 2; ++sl) {
            mbar_init(kv_full(sl), NFE); mbar_init(slot_free(sl), 6); mbar_init(d_full(sl), 1); mbar_init(d_empty(sl), 4);
            mbar_init(a_ready(sl), 4); mbar_init(taps_ready(sl), 4);
        }
        fence_mbar_init();
    }
    if (warp == W_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sm_u + LY::OFF_TSLOT), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem;
    asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(tmem) : "r"(sm_u + LY::OFF_TSLOT) : "memory");
    uint32_t cc = 0;          // chunks this role has gone through (halo chunks included): slot = cc & 1
    uint32_t oc = 0;          // output chunks: accumulator buffer = oc & 1

    // ---------------- roles ---------------------------------------------------------------------
    if (warp < NFE) {
        // ======== front end: warp w owns rows [16w, 16w+16) of every chunk =========================
        // (item-agnostic: the rows arrive staged; only the featurizer taps depend on the group)
        const int w = warp, p = lane % 8, s = lane / 8;
        f32x2 w3[3][3];     // [q|k|v][tap], each the pair of this lane's two channels (of the current item's group)
        // featurizer taps of item t: staged in shared memory by the epilogue warps before they expand the item's Toeplitz
        // operand (taps_ready: the front end of a launch's first item starts while that expansion still runs);
        // [feature][tap][channel] fp32, this lane's two channels as one 8-byte load
        auto load_w3 = [&](int t) {
            if (!FEAT) return true;
            if (!mbar_wait(taps_ready(t & 1), (uint32_t)((t >> 1) & 1), 17)) return false;
            const uint32_t base = sm_u + OFF_W3S + (uint32_t)((t & 1) * W3S_BYTES) + 8u * (uint32_t)p;
#pragma unroll
            for (int x = 0; x < 3; ++x)
#pragma unroll
                for (int j = 0; j < 3; ++j)
                    asm volatile("ld.shared.b64 %0, [%1];" : "=l"(w3[x][j]) : "r"(base + (uint32_t)((x * 3 + j) * CH * 4)));
            return true;
        };
        // lane constants folded into two offsets: the lane's first staged word of a half chunk, and its fp16 pair in row
        // 16 w of a k*v tile (16-byte chunk 2 s + p / 4, bytes 4 (p % 4))
        const uint32_t lane_box = (uint32_t)(s * BOX_STRIDE + ((w % (NFE / 2)) * WROWS + s) * (INTERLEAVED ? 96 : 32) + (INTERLEAVED ? 12 : 4) * p);
        const uint32_t lane_kv = (uint32_t)(((s * 2 + p / 4) << 4) + (p % 4) * 4 + w * WROWS * 128);
        const uint32_t half = (uint32_t)(w / (NFE / 2));
        constexpr int ROWB = INTERLEAVED ? 96 : 32;             // bytes per staged row (per plane in the planar layouts)
        // shared-memory address of this lane's first word of batch hb of chunk k (the box row of the batch's first
        // sample minus the two featurizer history rows; stream s was staged s rows early)
        auto box_addr = [&](uint32_t k, int hb) {
            const uint32_t stg = (2 * k + half) % IN_STAGES;
            return sm_u + stg * STAGE_BYTES + lane_box + (uint32_t)(hb * RB * ROWB);
        };
        // Volatile loads: they are issued where they stand, one batch ahead of the arithmetic that consumes them, so
        // that their latency (and the wait for the stage before them) overlaps the previous batch's arithmetic.
        auto fetch = [&](uint32_t addr, uint32_t (&raw)[RB + 2][3]) {
#pragma unroll
            for (int r = 0; r < RB + 2; ++r) {
#pragma unroll
                for (int j = 0; j < 3; ++j)
                    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(raw[r][j]) : "r"(addr + (uint32_t)(r * ROWB + (INTERLEAVED ? 4 * j : j * IN_PLANE))));
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
        // featurizer -> k*v and q of RB rows as fp16, written into the chunk's slot
        auto compute = [&](int slot, int hb, const uint32_t (&raw)[RB + 2][3]) {
            // Tiles are 1024-byte aligned, so the swizzle (16-byte chunk index XOR row phase) is one XOR on the address
            // of the lane's element in row 0; row offsets are compile-time immediates of the stores.
            const uint32_t kv_a0 = sm_u + OFF_SLOTS + slot * SLOT_BYTES + lane_kv + (uint32_t)(hb * RB * 128);
            f32x2 x1[3], x2[3];
            unpack(raw[0], x2);
            unpack(raw[1], x1);
#pragma unroll
            for (int i = 0; i < RB; ++i) {
                f32x2 x0[3], z[3];
                unpack(raw[i + 2], x0);
                float kv0, kv1, q0, q1;
                if (FEAT) {
#pragma unroll
                    for (int x = 0; x < 3; ++x) {
                        z[x] = fma2(w3[x][0], x2[x], fma2(w3[x][1], x1[x], mul2(w3[x][2], x0[x])));
                        x2[x] = x1[x];
                        x1[x] = x0[x];
                    }
                    // (the staged taps of v carry the 2^-6 of the k*v tile; rows before the sequence start are zeros)
                    up2(mul2(SWAP ? z[0] : z[1], z[2]), kv0, kv1);
                    up2(SWAP ? z[1] : z[0], q0, q1);
                } else {
                    // k*v rounded to bf16 as the reference materialises it, then scaled: exact in fp16
                    up2(mul2(x0[1], x0[2]), kv0, kv1);
                    const uint32_t r = pack_bf16(kv0, kv1);
                    kv0 = bf_lo(r) * KV_SCALE; kv1 = bf_hi(r) * KV_SCALE;
                    up2(x0[0], q0, q1);
                }
                // row0 is a multiple of 8, so the swizzle phase of row row0 + i is i & 7
                const uint32_t kaddr = kv_a0 ^ (uint32_t)((i & 7) << 4);
                asm volatile("st.shared.b32 [%0], %1;" ::"r"(kaddr + i * 128), "r"(pack_f16(kv0, kv1)));
                asm volatile("st.shared.b32 [%0], %1;" ::"r"(kaddr + (Q_OFF + i * 128)), "r"(pack_f16(q0, q1)));
            }
        };
        auto stage_of = [&](uint32_t k) { return (int)((2 * k + half) % IN_STAGES); };
        auto stage_parity = [&](uint32_t k) { return ((2 * k + half) / IN_STAGES) & 1u; };

        // Software pipeline over register batches A (rows 0..RB-1 of the warp's rows) and B (the rest):
        //   fetch B(k) | wait slot | compute A(k) | release stage | wait stage(k+1), fetch A(k+1) | compute B(k) | publish
        uint32_t rawA[RB + 2][3], rawB[RB + 2][3];
        uint32_t c_end = (uint32_t)nmine * (uint32_t)nchunk;
        int kin = 0, t = 0;       // chunk within the item, item
        if (!mbar_wait(in_full(stage_of(cc)), stage_parity(cc), 4)) c_end = cc;     // (gave up: nothing to do)
        fetch(box_addr(cc, 0), rawA);
        for (; cc < c_end; ++cc) {
            const int slot = cc & 1;
            if (kin == 0 && !load_w3(t)) break;         // a new item: its group's featurizer taps
            if (++kin == nchunk) { kin = 0; ++t; }
            fetch(box_addr(cc, 1), rawB);
            // slot reuse: the MMAs that read chunk cc-2 and the epilogue that read its k*v rows and q tile are done
            if (cc >= 2 && !mbar_wait(slot_free(slot), ((cc - 2) >> 1) & 1u, 2)) break;
            compute(slot, 0, rawA);
            // Every row this warp needs from the stage now sits in registers: hand the stage back to the TMA warp (HBM
            // latency under load is ~2 us, so as much of the ring as possible should be in flight).  The empty asm
            // makes the loaded values a dependency of the arrive.
#pragma unroll
            for (int r = 0; r < RB + 2; ++r) asm volatile("" ::"r"(rawB[r][0]), "r"(rawB[r][1]), "r"(rawB[r][2]));
            __syncwarp();
            if (lane == 0) mbar_arrive(in_empty(stage_of(cc)));
            if (cc + 1 < c_end) {
                if (!mbar_wait(in_full(stage_of(cc + 1)), stage_parity(cc + 1), 4)) break;
                fetch(box_addr(cc + 1, 0), rawA);
            }
            compute(slot, 1, rawB);
            fence_proxy_async_smem();      // generic-proxy writes -> visible to the tensor core's async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(kv_full(slot));
        }
    } else if (warp < W_EP + 4) {
        // ======== epilogue: thread = output row (TMEM lane) ========================================
        const int e = warp - W_EP, r = e * 32 + lane;
        const int64_t chunk_pitch = (int64_t)CHUNK * a.y_stride_l;
        // Toeplitz operand of item t -> TMEM buffer t & 1: the group's taps (zero padded: tp[m] = tap at lag m - 128,
        // times 2^6) and skip parameters go through shared memory, then lane i writes row i of [T^|T].  Runs while the
        // item before streams; the four epilogue warps meet on a barrier of their own (bounded wait) between the steps.
        auto expand = [&](int t) {
            const int g = item_group(t), ab = t & 1;
            uint16_t* tp = reinterpret_cast<uint16_t*>(smp(OFF_TAPS + ab * 768));
            // every global load of the staging first (raw bits, no dtype branch in between): one memory round trip
            // instead of five, which at the start of a launch is what the front end waits for
            const bool h_wide = a.h_dtype == VTX_F32, w_wide = a.w3_dtype == VTX_F32;
            const int64_t hrow = (int64_t)((unsigned)(g * CH) / (unsigned)a.dg) * K;      // the group's filter row
            uint32_t traw[3], braw = 0, wraw[2] = {0, 0};
#pragma unroll
            for (int i = 0; i < 3; ++i) {
                const int l = r + 128 * i - 128;
                traw[i] = (l >= 0 && l < K) ? ld_raw(a.h, h_wide, hrow + (a.taps == VTX_TAPS_CONV ? l : K - 1 - l)) : 0u;
            }
            if (r < CH && a.has_bias) braw = ld_raw(a.bias, a.bias_dtype == VTX_F32, (int64_t)g * CH + r);
            if (FEAT) {   // featurizer taps of the group's 16 channels (the front end picks them up at the item's first chunk)
                QkvMap map{a.layout, INTERLEAVED ? 0 : a.flip, a.D, a.hd};
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int m = r + 128 * i;
                    if (m < 3 * 3 * CH) {
                        const int c = m % CH, j = (m / CH) % 3, x = m / (3 * CH);
                        int64_t pc[3];
                        map.get((int64_t)g * CH + c, pc[0], pc[1], pc[2]);
                        wraw[i] = ld_raw(a.w3, w_wide, (x == 0 ? pc[0] : x == 1 ? pc[1] : pc[2]) * 3 + j);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 3; ++i) {
                const int l = r + 128 * i - 128;
                tp[r + 128 * i] = f16_bits((l >= 0 && l < K) ? KV_UNSCALE * cvt_raw(traw[i], a.h_dtype) : 0.f);
            }
            if (r < CH) reinterpret_cast<float*>(smp(OFF_DIAG + ab * 64))[r] = a.has_bias ? KV_UNSCALE * cvt_raw(braw, a.bias_dtype) : 0.f;
            if (FEAT) {
                float* w3s = reinterpret_cast<float*>(smp(OFF_W3S + ab * W3S_BYTES));
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int m = r + 128 * i;
                    if (m < 3 * 3 * CH) w3s[m] = cvt_raw(wraw[i], a.w3_dtype) * (m / (3 * CH) == 2 ? KV_SCALE : 1.f);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(taps_ready(ab));
            if (!mbar_wait(taps_ready(ab), (uint32_t)((t >> 1) & 1), 16)) return false;
            const uint16_t* tpr = tp;
            for (int c0 = 0; c0 < 128; c0 += 16) {
                uint32_t v[16];
#pragma unroll
                for (int m = 0; m < 16; ++m) {
                    const int j = 2 * (c0 + m);                            // columns j, j+1 of [T^|T]: lag = 128 + i - j
                    const uint32_t e0 = tpr[128 + 128 + r - j], e1 = tpr[128 + 127 + r - j];
                    v[m] = e1 << 16 | e0;
                }
                tmem_st16(tmem + ((uint32_t)(e * 32) << 16) + ab * 128 + c0, v);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(a_ready(ab));
            return true;
        };
        bool ok = expand(0);
        for (int t = 0; t < nmine && ok; ++t) {
            const int g = item_group(t);
            const float4* dsk = reinterpret_cast<const float4*>(smp(OFF_DIAG + (t & 1) * 64));    // 2^6 D[g*16 .. +16), fp32
            bool has_skip = false;       // the skip parameter is all zeros at initialisation: then its term is not evaluated
#pragma unroll
            for (int c = 0; c < CH / 4; ++c) {
                const float4 d = dsk[c];
                has_skip = has_skip || d.x != 0.f || d.y != 0.f || d.z != 0.f || d.w != 0.f;
            }
            // per stream: pointer to this thread's first output row and the number of rows of the segment from there on
            // (<= 0: nothing to store).  Kept as one pointer and one int per stream to save registers.
            __nv_bfloat16* yrow[NS];
            int nleft[NS];
#pragma unroll
            for (int s = 0; s < NS; ++s) {
                const Stream st = stream_of(a, item_quad(t), s);
                yrow[s] = a.y + st.b * a.y_stride_b + (st.ts + r) * a.y_stride_l + (int64_t)g * CH;
                nleft[s] = st.active ? (int)(st.te - st.ts) - r : 0;
            }
            if (lane == 0) mbar_arrive(slot_free(cc & 1));      // the item's halo chunk has no epilogue
            ++cc;
            for (int k = 1; k < nchunk; ++k, ++cc, ++oc) {
                const int slot = cc & 1, dbuf = oc & 1;
                if (!mbar_wait(d_full(dbuf), (oc >> 1) & 1u, 5)) { ok = false; break; }
                tc_fence_after();
                __syncwarp();
                const uint32_t taddr = tmem + ((uint32_t)(e * 32) << 16) + D_COL + dbuf * 64;
                const uint8_t* kv_p = smp(OFF_SLOTS + slot * SLOT_BYTES) + r * 128;     // this row of the k*v tile; q: + Q_OFF
                const int64_t yoff = (int64_t)(k - 1) * chunk_pitch;
                // One stream at a time (16 channels: accumulators -> skip -> gate -> 32 bytes of output), rolled over the
                // streams: keeps the instruction-cache footprint of this role small and nothing spills (a spilled value
                // is reloaded from L2 here: L1 is almost entirely carved out as shared memory).
#pragma unroll 1
                for (int s = 0; s < NS; ++s) {
                    uint32_t acc[16];
                    tmem_ld16(taddr + s * 16, acc);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    tmem_ld_touch(acc);
                    if (s + 1 == NS) {
                        // every accumulator of this chunk has left TMEM: hand the buffer back to the MMA warp
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(d_empty(dbuf));
                    }
                    // this stream's output pointer and row count (selects, not indexed arrays: the loop is rolled)
                    __nv_bfloat16* ys = yrow[0];
                    int nl = nleft[0];
#pragma unroll
                    for (int tt = 1; tt < NS; ++tt)
                        if (s == tt) { ys = yrow[tt]; nl = nleft[tt]; }
                    uint32_t o[8];
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
                        const uint32_t off = (uint32_t)(((2 * s + hf) ^ (r & 7)) << 4);
                        f32x2 y[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) y[j] = pk2(__uint_as_float(acc[8 * hf + 2 * j]), __uint_as_float(acc[8 * hf + 2 * j + 1]));
                        // rounds a pair to bf16 and back (the operator-only variant materialises what the reference does)
                        auto rnd = [](f32x2 v) {
                            float v0, v1;
                            up2(v, v0, v1);
                            const uint32_t r = pack_bf16(v0, v1);
                            return pk2(bf_lo(r), bf_hi(r));
                        };
                        if (has_skip) {
                            // skip term D[c] * kv[t, c] from this row of the k*v tile (both carry their power of two)
                            const uint4 k4 = *reinterpret_cast<const uint4*>(kv_p + off);
                            const uint32_t kw[4] = {k4.x, k4.y, k4.z, k4.w};
                            const float4 d0 = dsk[2 * hf], d1 = dsk[2 * hf + 1];
                            const f32x2 dd[4] = {pk2(d0.x, d0.y), pk2(d0.z, d0.w), pk2(d1.x, d1.y), pk2(d1.z, d1.w)};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                if (FEAT || a.taps == VTX_TAPS_CONV) y[j] = fma2(dd[j], unpack_f16(kw[j]), y[j]);     // fp32 sum, one rounding
                                else y[j] = add2(rnd(y[j]), rnd(mul2(dd[j], unpack_f16(kw[j]))));     // filter output and skip rounded apart
                            }
                        }
                        if (!FEAT) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) y[j] = rnd(y[j]);
                        }
                        const uint4 q4 = *reinterpret_cast<const uint4*>(kv_p + Q_OFF + off);
                        const uint32_t qw[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            float o0, o1;
                            up2(mul2(y[j], unpack_f16(qw[j])), o0, o1);
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
                    if ((k - 1) * CHUNK < nl)
                        asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ys + yoff), "r"(o[0]),
                                     "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]));
                }
                // every shared-memory read of this chunk is done: its k*v slot and q tile may be rewritten
                __syncwarp();
                if (lane == 0) mbar_arrive(slot_free(slot));
                if (k == 1 && t + 1 < nmine && !expand(t + 1)) { ok = false; break; }
            }
        }
    } else if (warp == W_MMA) {
        // ======== MMA issue =========================================================================
        if (lane == 0) {
            const uint32_t idesc = instr_desc_f16(128, NS * CH);
            // An output chunk accumulates  prev = T^ * kv(chunk before)  and  cur = T * kv(chunk)  into one buffer.
            // The prev half of the NEXT chunk is issued right behind cur, long before that chunk is staged, so a tile
            // is released (slot_free) one whole chunk before the front end needs its slot again.
            // Descriptors are built once; a K step of 16 rows moves the start-address field by 2048 B (128 units).
            // The issue loop is fully unrolled: the issuing thread is on the critical path of every chunk.
            // B operand of one K step: 16 rows x 64 channels, N-major, one 128-byte swizzle atom wide, 8-row groups
            // 1024 B apart (SBO); the leading-dimension offset is not used with a single atom.
            uint64_t kv_desc[2];
#pragma unroll
            for (int sl = 0; sl < 2; ++sl) kv_desc[sl] = smem_desc(sm_u + OFF_SLOTS + sl * SLOT_BYTES, KV_TILE, 1024, 2);
            // one half of a chunk's contraction: T^ (cur == false) or T (cur == true) times the k*v tile in `slot`,
            // accumulated into buffer `dbuf`; the previous-chunk half comes first and overwrites the accumulator
            auto issue_half = [&](int abuf, int slot, int dbuf, bool cur) {
                const uint32_t d = tmem + D_COL + dbuf * 64;
                const uint32_t a0 = tmem + abuf * 128 + (cur ? 64 : 0);
                const uint64_t dk = slot ? kv_desc[1] : kv_desc[0];
#pragma unroll
                for (int jj = 0; jj < 8; ++jj)
                    mma_ts(d, a0 + 8 * jj, dk + (uint64_t)(jj * (16 * 128 / 16)), idesc, (cur || jj > 0) ? 1u : 0u);
            };
            bool ok = true;
            for (int t = 0; t < nmine && ok; ++t) {
                const int ab = t & 1;
                // the item's Toeplitz operand (expanded by the epilogue warps while the item before was streaming)
                if (!mbar_wait(a_ready(ab), (uint32_t)((t >> 1) & 1), 10)) { ok = false; break; }
                // halo chunk of the item: its tile only feeds the previous-chunk half of the first output chunk
                if (!mbar_wait(kv_full(cc & 1), (cc >> 1) & 1u, 7)) { ok = false; break; }
                if (nchunk > 1) {
                    // the accumulator of output chunk oc was last read by the epilogue of output chunk oc - 2
                    if (oc >= 2 && !mbar_wait(d_empty(oc & 1), ((oc - 2) >> 1) & 1u, 8)) { ok = false; break; }
                    tc_fence_after();
                    issue_half(ab, cc & 1, oc & 1, false);
                }
                mma_commit(slot_free(cc & 1));
                ++cc;
                for (int k = 1; k < nchunk; ++k, ++cc, ++oc) {
                    if (!mbar_wait(kv_full(cc & 1), (cc >> 1) & 1u, 6)) { ok = false; break; }
                    tc_fence_after();
                    issue_half(ab, cc & 1, oc & 1, true);
                    mma_commit(d_full(oc & 1));
                    if (k + 1 < nchunk) {
                        // the next output chunk's accumulator was last read by the epilogue of output chunk oc - 1
                        if (oc >= 1 && !mbar_wait(d_empty((oc + 1) & 1), ((oc - 1) >> 1) & 1u, 8)) { ok = false; break; }
                        tc_fence_after();
                        issue_half(ab, cc & 1, (oc + 1) & 1, false);
                    }
                    mma_commit(slot_free(cc & 1));
                }
            }
        }
    } else if (warp < W_TMA + NTMA) {
        const int tw = warp - W_TMA;                 // this warp issues the boxes of streams tw, tw + NTMA, ...
        if (lane == 0) {
            // ======== TMA issue ======================================================================
            tma_prefetch_desc(&tmap);
            if (!FEAT) { tma_prefetch_desc(&tmap_k); tma_prefetch_desc(&tmap_v); }
            uint32_t nh = 2 * cc;                    // staged half chunks so far
            bool ok = true;
            for (int t = 0; t < nmine && ok; ++t) {
                // first packed column of the item's group in q | k | v (one contiguous run when interleaved)
                const int g = item_group(t);
                int col[3] = {0, 0, 0};
                if (INTERLEAVED) {
                    col[0] = 3 * g * CH;
                } else if (!FEAT) {
                    col[0] = col[1] = col[2] = g * CH;          // the same channels of three tensors
                } else {
                    const int64_t d0 = (int64_t)g * CH;
                    if (a.layout == VTX_QKV_COLUMN_SPLIT) {
                        int64_t n = d0 / a.hd, j = d0 - n * a.hd;
                        col[0] = (int)(n * 3 * a.hd + j); col[1] = col[0] + (int)a.hd; col[2] = col[0] + 2 * (int)a.hd;
                    } else {
                        col[0] = (int)d0; col[1] = (int)(a.D + d0); col[2] = (int)(2 * a.D + d0);
                    }
                    if (a.flip) { int tt = col[0]; col[0] = col[1]; col[1] = tt; }
                }
                int row_base[NS], bidx[NS];          // first staged row of the item's halo chunk and batch index, per stream
#pragma unroll
                for (int s = 0; s < NS; ++s) {
                    const Stream st = stream_of(a, item_quad(t), s);
                    row_base[s] = (int)st.ts - CHUNK - 2 - s + a.hist;
                    bidx[s] = (int)st.b;
                }
                for (int hh = 0; hh < 2 * nchunk; ++hh, ++nh) {
                    const int stg = (int)(nh % IN_STAGES), k = hh / 2, h = hh % 2;
                    if (nh >= IN_STAGES && !mbar_wait(in_empty(stg), ((nh - IN_STAGES) / IN_STAGES) & 1u, 9)) { ok = false; break; }
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
                                tma_load_3d(dst + pl * IN_PLANE, FEAT || pl == 0 ? &tmap : pl == 1 ? &tmap_k : &tmap_v, bar, col[pl], row, bidx[s]);
                        }
                    }
                }
            }
        }
    } else if (warp == W_STATE) {
        // ======== prefill caches ======================================================================
        // fir_state[b, c, :] = u[b, L-n3:L, c] (n3 = min(L, 2)): a copy of a few input words, made when the item starts.
        // inner_state[b, d, :] = bf16(kv[b, d, L-ns:L]) (ns = min(L, K-1)): read back from the k*v tiles the front end
        // publishes -- this warp takes part in every chunk's hand-over (it waits for the tile and is one of the
        // arrivals that free its slot) and touches only the chunks that hold the last ns rows of a sequence, the halo
        // chunk included.  With history rows in front of u both caches are always full.  Exactly one stream of a
        // (batch, group) ends its sequence.  lane = row of the tile: the stores of a channel run along time.
        const int64_t L = a.L;
        const int ns = (a.hist > 0 || L >= K - 1) ? K - 1 : (int)L;
        const int n3 = (a.hist > 0 || L >= 2) ? 2 : (int)L;
        bool ok = true;
        for (int t = 0; t < nmine && ok; ++t) {
            const int g = item_group(t);
            int tr1[NS];          // rows [tr1 - ns, tr1), relative to the stream's first row, feed inner_state
            int sb[NS];
#pragma unroll
            for (int s = 0; s < NS; ++s) {
                const Stream st = stream_of(a, item_quad(t), s);
                sb[s] = (int)st.b;
                tr1[s] = (st.active && st.te == L) ? (int)(L - st.ts) : -(1 << 29);
            }
            // the input words of fir_state are requested now (volatile: issued where they stand) and stored at the end
            // of the item, so that the round trip to memory never holds up a slot
            uint16_t fsv[NS][3];
            auto fs_col = [&](int m) {      // m-th of the group's 3 x 16 packed columns times n3 rows -> packed column
                const QkvMap map{a.layout, 0, a.D, a.hd};
                int64_t pc[3];
                map.get((int64_t)g * CH + (m / n3) % CH, pc[0], pc[1], pc[2]);
                return m / n3 < CH ? pc[0] : m / n3 < 2 * CH ? pc[1] : pc[2];
            };
            if (a.fir_state && n3 > 0) {
#pragma unroll
                for (int s = 0; s < NS; ++s) {
                    if (tr1[s] <= 0) continue;
                    const uint16_t* ub = reinterpret_cast<const uint16_t*>(a.u) + (int64_t)sb[s] * a.u_stride_b;
#pragma unroll
                    for (int i = 0; i < 3; ++i) {
                        const int m = lane + 32 * i;
                        fsv[s][i] = 0;
                        if (m < 3 * CH * n3)
                            asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(fsv[s][i]) : "l"(ub + (L - n3 + m % n3) * a.u_stride_l + fs_col(m)));
                    }
                }
            }
            for (int k = 0; k < nchunk; ++k, ++cc) {
                const int slot = cc & 1;
                if (!mbar_wait(kv_full(slot), (cc >> 1) & 1u, 18)) { ok = false; break; }
                const int rel0 = (k - 1) * CHUNK;
                if (a.inner_state) {
#pragma unroll 1
                    for (int s = 0; s < NS; ++s) {
                        int t1 = tr1[0], b1 = sb[0];
#pragma unroll
                        for (int x = 1; x < NS; ++x)
                            if (s == x) { t1 = tr1[x]; b1 = sb[x]; }
                        if (rel0 + CHUNK <= t1 - ns || rel0 >= t1) continue;
                        __nv_bfloat16* dst = a.inner_state + ((int64_t)b1 * a.D + (int64_t)g * CH) * ns;
#pragma unroll 1
                        for (int r = lane; r < CHUNK; r += 32) {
                            const int rel = rel0 + r;
                            if (rel < t1 - ns || rel >= t1) continue;
                            const uint8_t* row = smp(OFF_SLOTS + slot * SLOT_BYTES) + r * 128;
#pragma unroll
                            for (int hf = 0; hf < 2; ++hf) {
                                const uint4 k4 = *reinterpret_cast<const uint4*>(row + (((2 * s + hf) ^ (r & 7)) << 4));
                                const uint32_t kw[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    float v0, v1;
                                    up2(unpack_f16(kw[j]), v0, v1);
                                    __nv_bfloat16* d0 = dst + (int64_t)(8 * hf + 2 * j) * ns + (rel - (t1 - ns));
                                    d0[0] = __float2bfloat16_rn(v0 * KV_UNSCALE);
                                    d0[ns] = __float2bfloat16_rn(v1 * KV_UNSCALE);
                                }
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(slot_free(slot));
                // (stored at the item's last chunk: by then the words requested at its start have long arrived, and
                // this warp never sits on a memory round trip while slots wait for its hand-over)
                if (k == nchunk - 1 && a.fir_state && n3 > 0) {
#pragma unroll
                    for (int s = 0; s < NS; ++s) {
                        if (tr1[s] <= 0) continue;
                        uint16_t* fs = reinterpret_cast<uint16_t*>(a.fir_state) + (int64_t)sb[s] * 3 * a.D * n3;
#pragma unroll
                        for (int i = 0; i < 3; ++i) {
                            const int m = lane + 32 * i;
                            if (m < 3 * CH * n3) fs[fs_col(m) * n3 + m % n3] = fsv[s][i];
                        }
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
        uint32_t tmem;
        asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(tmem) : "r"(sm_u + LY::OFF_TSLOT) : "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
    }
}

}  // namespace mr

namespace mr {

// Time segments: a sequence is cut into nseg segments of whole chunks, a work item is one group x four streams
// (batch element x segment), the items are dealt round-robin to one persistent CTA per SM.  Every item pays one
// halo chunk, and the launch lasts as long as the CTA with the most chunks: pick the segment length that makes
// that CTA's chunk count smallest (ties: fewer items).
static int plan_items(Args& a) {
    const int64_t nchunks_total = ceil_div<int64_t>(a.L, CHUNK);
    int64_t nseg = 1, best_cost = INT64_MAX;
    for (int64_t seg_chunks = nchunks_total; seg_chunks >= 1; --seg_chunks) {
        const int64_t ns_ = ceil_div<int64_t>(nchunks_total, seg_chunks);
        if (ceil_div<int64_t>(nchunks_total, ns_) != seg_chunks) continue;       // same plan as a shorter segment
        const int64_t items = a.G * ceil_div<int64_t>(a.B * ns_, NS);
        const int64_t cost = ceil_div<int64_t>(items, kNumSMs) * (seg_chunks + 1) * 64 + ns_;   // (+ a little per segment)
        if (cost < best_cost) { best_cost = cost; nseg = ns_; }
        if (seg_chunks <= 2 || items > (int64_t)kNumSMs * 64) break;            // shorter segments only add halo chunks
    }
    a.seg_len = ceil_div<int64_t>(nchunks_total, nseg) * CHUNK;
    a.nseg = ceil_div<int64_t>(a.L, a.seg_len);
    a.nstream = a.B * a.nseg;
    a.nquad = ceil_div<int64_t>(a.nstream, NS);
    VTX_REQUIRE(a.G * a.nquad < (int64_t)1 << 31, VTX_ERR_UNSUPPORTED, "fused_fir: too many work items");
    a.nitems = a.G * a.nquad;
    return VTX_OK;
}

// One persistent CTA per SM (the shared-memory footprint allows no more), each walking the items blockIdx,
// blockIdx + gridDim, ...  The CTA count must not exceed what is resident at once: a second round would double the time.
template <typename Kern>
static int launch(Kern kern, int variant, int smem_bytes, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                  const Args& a, cudaStream_t stream) {
    // the opt-in is a per-device property of the function: remember it per device
    static bool attr_set[64][4] = {};
    static int resident[64][4] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const bool known = dev >= 0 && dev < 64;
    if (!known || !attr_set[dev][variant]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        if (e != cudaSuccess) return fail(VTX_ERR_LAUNCH, "fused_fir(mr): shared memory opt-in: %s", cudaGetErrorString(e));
        if (known) attr_set[dev][variant] = true;
    }
    int nres = known ? resident[dev][variant] : 0;
    if (nres == 0) {
        int sms = 0, per_sm = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, THREADS, smem_bytes);
        nres = sms * per_sm;
        if (nres <= 0) return fail(VTX_ERR_LAUNCH, "fused_fir(mr): the kernel does not fit an SM (%d SMs, %d blocks each)", sms, per_sm);
        if (known) resident[dev][variant] = nres;
    }
    // The CTAs of a launch start side by side on neighbouring groups of the same rows: their 96-byte pieces of a row
    // share 128-byte lines and DRAM pages.  Nothing holds them together afterwards, and over a few milliseconds they
    // drift apart; measured on a 1 M-token sequence of 8192 channels, one launch of 66 items per CTA ran at half the
    // speed of the same items in launches of a few milliseconds each.  So a call is cut into launches of about
    // 500 chunks per CTA (250 and 500 measured alike, 1000 a little slower on the short filter, 2000 clearly slower);
    // each starts its CTAs side by side again.
    const int64_t nchunk = a.seg_len / CHUNK + 1;
#ifndef VTX_MR_LAUNCH_CHUNKS
#define VTX_MR_LAUNCH_CHUNKS 500
#endif
    int64_t rounds = VTX_MR_LAUNCH_CHUNKS / nchunk;
    if (rounds < 1) rounds = 1;
    Args b = a;
    long long launches = 0;
    for (int64_t i0 = 0; i0 < a.nitems; i0 += rounds * nres, ++launches) {
        b.item0 = i0;
        b.item1 = i0 + rounds * nres < a.nitems ? i0 + rounds * nres : a.nitems;
        const int64_t n = b.item1 - b.item0, ncta = n < nres ? n : nres;
        kern<<<(unsigned)ncta, THREADS, smem_bytes, stream>>>(tq, tk, tv, b);
    }
    return check_launch("fused_fir(mr)", launches);
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
    a.fir_state = static_cast<__nv_bfloat16*>(p->fir_state); a.inner_state = static_cast<__nv_bfloat16*>(p->inner_state);
    a.B = p->B; a.L = p->L; a.D = p->D; a.G = p->G; a.K = p->K; a.dg = CH;
    a.layout = (int)p->layout; a.flip = p->flip_x1x2 != 0; a.taps = (int)p->taps;
    a.hd = p->D;
    a.hist = (int)p->u_hist_rows;
    if (p->layout == VTX_QKV_COLUMN_SPLIT) {
        VTX_REQUIRE(p->num_heads > 0 && p->D % p->num_heads == 0, VTX_ERR_BAD_ARG, "fused_fir: bad num_heads");
        a.hd = p->D / p->num_heads;
        VTX_REQUIRE(a.hd % CH == 0, VTX_ERR_UNSUPPORTED, "fused_fir: column split needs head size %% %d == 0", CH);
    }
    VTX_REQUIRE(p->layout == VTX_QKV_INTERLEAVED || (p->D * 2) % 16 == 0, VTX_ERR_ALIGNMENT,
                "fused_fir: D*itemsize must be a multiple of 16 bytes for this q/k/v layout");
    if (int rc = plan_items(a)) return rc;
    const bool inter = p->layout == VTX_QKV_INTERLEAVED;
    CUtensorMap tmap;
    // the tensor map starts at the first history row (chunked prefill), else at u
    const __nv_bfloat16* u_first = static_cast<const __nv_bfloat16*>(p->u) - p->u_hist_rows * p->u_stride_l;
    if (int rc = make_tmap_3d(&tmap, u_first, VTX_BF16, 3 * p->D, p->L + p->u_hist_rows, p->B, p->u_stride_l, p->u_stride_b,
                              inter ? 3 * CH : CH, BOX_ROWS, 0, "fused_fir(mr)"))
        return rc;
    if (!inter) return launch(fused_mr_kernel<false, false, true>, 0, Lay<false>::SMEM_BYTES, tmap, tmap, tmap, a, stream);
    if (!a.flip) return launch(fused_mr_kernel<true, false, true>, 1, Lay<true>::SMEM_BYTES, tmap, tmap, tmap, a, stream);
    return launch(fused_mr_kernel<true, true, true>, 2, Lay<true>::SMEM_BYTES, tmap, tmap, tmap, a, stream);
}

}  // namespace vtx

namespace vtx {
// Inner FIR cache of the operator-only call: state[b, d, j] = bf16(k * v)[b, L - ns + j, d], ns = min(L, K - 1).  A copy
// of products of the inputs, so it is made from them directly (the k*v tiles of the main kernel are fp16 and scaled:
// exact for the contraction's purposes, but not bit for bit for products below 2^-11).
__global__ void gcg_cl_state_kernel(const __nv_bfloat16* k, int64_t k_stride_b, int64_t k_stride_l, const __nv_bfloat16* v,
                                    int64_t v_stride_b, int64_t v_stride_l, __nv_bfloat16* state, int64_t B, int64_t L,
                                    int64_t D, int64_t ns) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= B * ns * D) return;
    const int64_t d = i % D, j = (i / D) % ns, b = i / (D * ns), t = L - ns + j;
    const float p = __bfloat162float(k[b * k_stride_b + t * k_stride_l + d]) * __bfloat162float(v[b * v_stride_b + t * v_stride_l + d]);
    state[(b * D + d) * ns + j] = __float2bfloat16_rn(p);
}
}  // namespace vtx

// Gate -> grouped causal FIR -> gate on three channel-last operands (no featurizer): the tensor-core kernel in its
// operator-only form.
extern "C" int vtx_gcg_cl_fwd(const vtx_gcg_cl_params* p, void* stream) {
    using namespace vtx;
    using namespace vtx::mr;
    VTX_REQUIRE(p && p->q && p->k && p->v && p->h && p->y, VTX_ERR_BAD_ARG, "gcg_cl: null pointer");
    VTX_REQUIRE(p->B > 0 && p->L > 0 && p->D > 0 && p->G > 0 && p->K > 0, VTX_ERR_BAD_ARG, "gcg_cl: sizes must be positive");
    VTX_REQUIRE(p->D % p->G == 0, VTX_ERR_BAD_ARG, "gcg_cl: D not a multiple of G");
    VTX_REQUIRE(p->io_dtype == VTX_BF16 && p->h_dtype == VTX_BF16, VTX_ERR_UNSUPPORTED, "gcg_cl: bf16 operands and filters only");
    VTX_REQUIRE(p->K <= CHUNK, VTX_ERR_UNSUPPORTED, "gcg_cl: filter length %lld > %d", (long long)p->K, CHUNK);
    VTX_REQUIRE((p->D / p->G) % CH == 0, VTX_ERR_UNSUPPORTED, "gcg_cl: filters must be shared by multiples of %d channels", CH);
    VTX_REQUIRE(p->bias_mode == VTX_BIAS_NONE || (p->bias_mode == VTX_BIAS_GATED && p->bias), VTX_ERR_UNSUPPORTED,
                "gcg_cl: bias mode must be none or gated");
    VTX_REQUIRE(p->B <= 65535 && p->L < ((int64_t)1 << 30), VTX_ERR_UNSUPPORTED, "gcg_cl: problem too large");
    VTX_REQUIRE((reinterpret_cast<uintptr_t>(p->y) % 32) == 0 && (p->y_stride_l % 16) == 0 && (p->y_stride_b % 16) == 0,
                VTX_ERR_ALIGNMENT, "gcg_cl: y rows must be 32-byte aligned");
    Args a{};
    a.h = p->h; a.h_dtype = p->h_dtype; a.bias = p->bias; a.bias_dtype = p->bias_dtype; a.has_bias = p->bias_mode == VTX_BIAS_GATED;
    a.y = static_cast<__nv_bfloat16*>(p->y); a.y_stride_b = p->y_stride_b; a.y_stride_l = p->y_stride_l;
    a.B = p->B; a.L = p->L; a.D = p->D; a.G = p->D / CH; a.K = p->K; a.dg = p->D / p->G;
    a.layout = VTX_QKV_SPLIT; a.taps = (int)p->taps; a.hd = p->D;
    if (int rc = plan_items(a)) return rc;
    CUtensorMap tm[3];
    const void* ptrs[3] = {p->q, p->k, p->v};
    const int64_t sl[3] = {p->q_stride_l, p->k_stride_l, p->v_stride_l}, sb[3] = {p->q_stride_b, p->k_stride_b, p->v_stride_b};
    for (int i = 0; i < 3; ++i)
        if (int rc = make_tmap_3d(&tm[i], ptrs[i], VTX_BF16, p->D, p->L, p->B, sl[i], sb[i], CH, BOX_ROWS, 0, "gcg_cl")) return rc;
    if (int rc = launch(fused_mr_kernel<false, false, false>, 3, Lay<false>::SMEM_BYTES, tm[0], tm[1], tm[2], a, (cudaStream_t)stream))
        return rc;
    const int64_t ns = p->L < p->K - 1 ? p->L : p->K - 1;
    if (p->state && ns > 0) {
        const int64_t n = p->B * ns * p->D;
        gcg_cl_state_kernel<<<(unsigned)ceil_div<int64_t>(n, 256), 256, 0, (cudaStream_t)stream>>>(
            static_cast<const __nv_bfloat16*>(p->k), p->k_stride_b, p->k_stride_l, static_cast<const __nv_bfloat16*>(p->v),
            p->v_stride_b, p->v_stride_l, static_cast<__nv_bfloat16*>(p->state), p->B, p->L, p->D, ns);
        return check_launch("gcg_cl state");
    }
    return VTX_OK;
}
