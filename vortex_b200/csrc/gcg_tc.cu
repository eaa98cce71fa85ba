// Gate -> grouped causal FIR -> gate on channel-first tensors, on tcgen05 / TMEM: the tensor-core path behind
// vtx_gcg_fwd, i.e. behind the drop-in HyenaInferenceEngine.parallel_fir(gate=True) and the (b, d, l) operands of
// hyena_ops, for bf16 I/O, filters of up to 128 taps shared by blocks of 16 (or a multiple of 16) channels.
//
//   kv = bf16(k * v);  z = bf16(FIR_h(kv) [+ D * kv]);  y = bf16(q * z)       (the reference's own rounding points,
//   vortex/model/engine.py:159,187,208,231: nothing is lost against its bf16 pipeline -- k*v, a bf16 value, is an exact
//   tensor-core operand, the taps are bf16 parameters, the accumulation is fp32)
//
// Same blocked-Toeplitz contraction as the fused projection-output kernel: per chunk of 128 output samples of one
// block of 16 channels  Y[128 x N] = [T^ | T][128 x 256] * KV[256 x N], the Toeplitz operand expanded from the taps
// into tensor memory once per work item.  What differs is the data side: the operands are channel-first, time
// contiguous, so a [16 channels x 64 samples] TMA box (128-byte rows, 128-byte swizzle) IS the K-major B operand of
// the MMA -- nothing is transposed.  A work item is one channel block and four streams (N = 64 columns): four batch
// elements over the same time segment, fetched as ONE box [4 x 16 x 64] per operand and half chunk (mode A, batch of
// three or more), or four (batch element, segment) pairs fetched box by box (mode B).
//
// One persistent CTA per SM, 16 warps: 0-3 front end (k*v of the staged k and v tiles into the chunk's slot, and the
// inner FIR cache from the last K-1 products of a sequence), 4-11 epilogue (thread = output sample, two warps per TMEM
// lane quarter with two streams each: TMEM -> skip -> round -> gate, the result written over the q tile in place and
// stored by TMA in whole 128-byte rows along time; the first four also expand the next item's Toeplitz operand),
// 12 MMA issue, 13 TMA issue for k and v, 14 TMA issue for q.  q
// never passes through the front end: its tiles stay in their ring until their chunk's outputs have left through
// them.  All waits are bounded.
#include <cstdint>

#include "tma.cuh"
#include "umma.cuh"

namespace vtx {

VTX_DEFINE_STATUS_READER()

namespace gtc {

using namespace umma;

constexpr int NS = 4, CH = 16, CHUNK = 128, NCOL = NS * CH;
constexpr int TILE = NCOL * CHUNK * 2;        // 16384: [2 halves of 64 samples][64 rows][128 B], 128-byte swizzle
constexpr int HALF_TILE = TILE / 2;
constexpr int NKV = 3;                        // ring of (k tile, v tile) stages
constexpr int NQ = 5;                         // ring of q tiles (a tile waits for its chunk's epilogue)
constexpr int NSLOT = 2;                      // k*v tiles: the chunk being contracted and the one before
constexpr int OFF_KV_IN = 0;
constexpr int OFF_Q = OFF_KV_IN + NKV * 2 * TILE;
constexpr int OFF_SLOTS = OFF_Q + NQ * TILE;
constexpr int OFF_TAPS = OFF_SLOTS + NSLOT * TILE;
constexpr int TAPS_BYTES = 2 * 384 * 2;       // zero-padded taps, bf16; two buffers (this item, next item)
constexpr int OFF_DIAG = OFF_TAPS + TAPS_BYTES;
constexpr int DIAG_BYTES = 2 * 64;            // skip parameters of the block's 16 channels, fp32; two buffers
constexpr int OFF_BARS = OFF_DIAG + DIAG_BYTES;
constexpr int NBARS = 2 * NKV + 2 * NQ + 2 * NSLOT + 2 * 5;
constexpr int OFF_TSLOT = OFF_BARS + NBARS * 8;
constexpr int SMEM_BYTES = OFF_TSLOT + 16 + 1024;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
static_assert(OFF_Q % 1024 == 0 && OFF_SLOTS % 1024 == 0, "tiles are 1024-byte aligned (swizzle atoms)");
constexpr int TMEM_COLS = 512;                // Toeplitz operand of item t at 128 (t & 1); accumulator buffer b at 256 + 64 b
constexpr int D_COL = 256;
constexpr int NFE = 4, W_EP = 4, NEP = 8, W_MMA = 12, W_TKV = 13, W_TQ = 14;   // NEP epilogue warps: two per TMEM lane quarter
constexpr int THREADS = 16 * 32;

struct Args {
    const void* h;  int64_t h_dtype;
    const void* bias; int64_t bias_dtype;
    __nv_bfloat16* y; int64_t y_stride_b, y_stride_d;
    __nv_bfloat16* state;                  // [B, D, ns] inner FIR cache, or null
    int64_t B, L, D, K, dg;                // dg: channels that share a filter (a multiple of 16)
    int64_t hd;                            // channels per head
    int64_t hdy;                           // "head" size of the output's tensor map (D: y has one channel pitch)
    int64_t nseg, seg_len, nquad, nitems, nblk;   // nblk = D / 16 channel blocks
    int taps, bias_mode, batch_quads;      // batch_quads: mode A
};

struct Stream {
    int64_t b, ts, te;
    bool active;
};
__device__ __forceinline__ Stream stream_of(const Args& a, int64_t quad, int s) {
    Stream st;
    int64_t seg;
    if (a.batch_quads) {                   // quad = (batch quad, segment): streams are four consecutive batch elements
        st.b = (quad / a.nseg) * NS + s;
        seg = quad % a.nseg;
        st.active = st.b < a.B;
    } else {                               // quad = four consecutive (batch element, segment) pairs
        int64_t id = quad * NS + s;
        st.active = id < a.B * a.nseg;
        if (!st.active) id = a.B * a.nseg - 1;
        st.b = id / a.nseg;
        seg = id % a.nseg;
    }
    st.ts = seg * a.seg_len;
    st.te = st.ts + a.seg_len < a.L ? st.ts + a.seg_len : a.L;
    return st;
}

// instruction descriptor: f32 accumulate, A bf16 (from TMEM), B bf16 K-major
__device__ __forceinline__ uint32_t instr_desc_kmajor(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (0u << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// byte offset of (column n, sample t) in a tile
__device__ __forceinline__ uint32_t tile_off(int n, int t) {
    return (uint32_t)((t >> 6) * HALF_TILE + n * 128 + ((((t & 63) >> 3) ^ (n & 7)) << 4) + (t & 7) * 2);
}

__global__ void __launch_bounds__(THREADS, 1)
gcg_tc_kernel(const __grid_constant__ CUtensorMap tmq, const __grid_constant__ CUtensorMap tmk,
              const __grid_constant__ CUtensorMap tmv, const __grid_constant__ CUtensorMap tmy,
              const __grid_constant__ Args a) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t sm_u = (smem_u32(smem_raw) + 1023u) & ~1023u;
    auto smp = [&](uint32_t off) { return reinterpret_cast<uint8_t*>(__cvta_shared_to_generic(sm_u + off)); };
    const uint32_t bar_u = sm_u + OFF_BARS;
    auto kvin_full = [&](int i) { return bar_u + 8u * (uint32_t)i; };
    auto kvin_empty = [&](int i) { return bar_u + 8u * (uint32_t)(NKV + i); };
    auto q_full = [&](int i) { return bar_u + 8u * (uint32_t)(2 * NKV + i); };
    auto q_empty = [&](int i) { return bar_u + 8u * (uint32_t)(2 * NKV + NQ + i); };
    constexpr int BB = 2 * NKV + 2 * NQ;
    auto kv_full = [&](int i) { return bar_u + 8u * (uint32_t)(BB + i); };
    // kv_free: nine arrivals -- the eight epilogue warps (skip term read) and the MMA warp's commit behind the last MMAs
    // that read the tile (the previous-chunk half of the NEXT chunk is issued right behind the chunk's own half)
    auto kv_free = [&](int i) { return bar_u + 8u * (uint32_t)(BB + NSLOT + i); };
    constexpr int BC = BB + 2 * NSLOT;
    auto d_full = [&](int i) { return bar_u + 8u * (uint32_t)(BC + i); };
    auto d_empty = [&](int i) { return bar_u + 8u * (uint32_t)(BC + 2 + i); };
    auto a_ready = [&](int i) { return bar_u + 8u * (uint32_t)(BC + 4 + i); };
    auto taps_ready = [&](int i) { return bar_u + 8u * (uint32_t)(BC + 6 + i); };
    auto y_ready = [&](int i) { return bar_u + 8u * (uint32_t)(BC + 8 + i); };        // a chunk's outputs written (4 epilogue warps)

    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const int ncta = (int)gridDim.x;
    const int nmine = (int)((a.nitems - (int64_t)blockIdx.x + ncta - 1) / ncta);
    const int K = (int)a.K;
    const int nchunk = (int)(a.seg_len / CHUNK) + 1;          // chunk 0 of an item is its halo chunk
    auto item_blk = [&](int t) { return (int)(((int64_t)blockIdx.x + (int64_t)t * ncta) % a.nblk); };
    auto item_quad = [&](int t) { return (int64_t)(((int64_t)blockIdx.x + (int64_t)t * ncta) / a.nblk); };

    if (tid == 0) {
        for (int i = 0; i < NKV; ++i) { mbar_init(kvin_full(i), 1); mbar_init(kvin_empty(i), NFE); }
        for (int i = 0; i < NQ; ++i) { mbar_init(q_full(i), 1); mbar_init(q_empty(i), 1); }
        for (int i = 0; i < NSLOT; ++i) { mbar_init(kv_full(i), NFE); mbar_init(kv_free(i), NEP + 1); }
        for (int i = 0; i < 2; ++i) {
            mbar_init(d_full(i), 1); mbar_init(d_empty(i), NEP); mbar_init(a_ready(i), 4); mbar_init(taps_ready(i), 4); mbar_init(y_ready(i), NEP);
        }
        fence_mbar_init();
    }
    if (warp == W_MMA) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sm_u + OFF_TSLOT), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    uint32_t tmem;
    asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(tmem) : "r"(sm_u + OFF_TSLOT) : "memory");
    uint32_t cc = 0;          // chunks this role has gone through (halo chunks included)
    uint32_t oc = 0;          // output chunks

    if (warp < NFE) {
        // ======== front end: k*v of the staged tiles, 16-byte vector by vector (same place in every tile) ========
        const int ns = a.L < K - 1 ? (int)a.L : K - 1;            // samples the inner FIR cache holds
        bool ok = true;
        for (int t = 0; t < nmine && ok; ++t) {
            const int blk = item_blk(t);
            int tr1[NS], sb[NS];       // rows [tr1 - ns, tr1), relative to the stream's first sample, feed the cache
#pragma unroll
            for (int s = 0; s < NS; ++s) {
                const Stream st = stream_of(a, item_quad(t), s);
                sb[s] = (int)st.b;
                tr1[s] = (a.state && st.active && st.te == a.L) ? (int)(a.L - st.ts) : -(1 << 29);
            }
            for (int k = 0; k < nchunk; ++k, ++cc) {
                const int stage = cc % NKV, slot = cc % NSLOT;
                if (!mbar_wait(kvin_full(stage), (cc / NKV) & 1u, 31)) { ok = false; break; }
                if (cc >= NSLOT && !mbar_wait(kv_free(slot), ((cc - NSLOT) / NSLOT) & 1u, 32)) { ok = false; break; }
                const uint8_t* kt = smp(OFF_KV_IN + stage * 2 * TILE);
                const uint8_t* vt = kt + TILE;
                uint8_t* dst = smp(OFF_SLOTS + slot * TILE);
                const int rel0 = (k - 1) * CHUNK;
                bool tail = false;
#pragma unroll
                for (int s = 0; s < NS; ++s) tail = tail || (rel0 + CHUNK > tr1[s] - ns && rel0 < tr1[s]);
#pragma unroll 1
                for (int i = 0; i < TILE / 16 / (NFE * 32); ++i) {
                    const int vi = tid + i * NFE * 32;
                    const uint4 kk = *reinterpret_cast<const uint4*>(kt + vi * 16);
                    const uint4 vv = *reinterpret_cast<const uint4*>(vt + vi * 16);
                    const uint32_t kw[4] = {kk.x, kk.y, kk.z, kk.w}, vw[4] = {vv.x, vv.y, vv.z, vv.w};
                    uint32_t o[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float p0, p1;
                        up2(mul2(pk2(bf_lo(kw[j]), bf_hi(kw[j])), pk2(bf_lo(vw[j]), bf_hi(vw[j]))), p0, p1);
                        o[j] = pack_bf16(p0, p1);
                    }
                    *reinterpret_cast<uint4*>(dst + vi * 16) = make_uint4(o[0], o[1], o[2], o[3]);
                    if (tail) {
                        // the vector's column and its eight samples: undo the swizzle of its 16-byte position
                        const int n = (vi % 512) / 8, s = n / CH, c = n % CH;
                        const int t0 = (vi / 512) * 64 + (((vi % 8) ^ (n & 7)) << 3);
                        int t1 = tr1[0], b1 = sb[0];
#pragma unroll
                        for (int x = 1; x < NS; ++x)
                            if (s == x) { t1 = tr1[x]; b1 = sb[x]; }
                        uint16_t* st = reinterpret_cast<uint16_t*>(a.state) + ((int64_t)b1 * a.D + (int64_t)blk * CH + c) * ns;
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const int rel = rel0 + t0 + e;
                            if (rel >= t1 - ns && rel < t1) st[rel - (t1 - ns)] = (uint16_t)(e & 1 ? o[e / 2] >> 16 : o[e / 2] & 0xffffu);
                        }
                    }
                }
                fence_proxy_async_smem();      // generic-proxy writes -> visible to the tensor core's async proxy
                __syncwarp();
                if (lane == 0) { mbar_arrive(kv_full(slot)); mbar_arrive(kvin_empty(stage)); }
            }
        }
    } else if (warp < W_EP + NEP) {
        // ======== epilogue: thread = output sample (TMEM lane); warps e and e + 4 share a lane quarter and take two
        // streams each (a single warp per scheduler leaves the latency of its shared-memory reads exposed) ========
        const int e = (warp - W_EP) % 4, r = e * 32 + lane, sh = (warp - W_EP) / 4;
        // Toeplitz operand of item t -> TMEM buffer t & 1 (lane i writes row i of [T^|T]); the block's taps (zero padded:
        // tp[m] = tap at lag m - 128) and skip parameters go through shared memory.  Runs while the item before streams.
        auto expand = [&](int t) {
            const int blk = item_blk(t), ab = t & 1;
            const int64_t fg = ((int64_t)blk * CH) / a.dg;                   // the filter this block uses
            uint16_t* tp = reinterpret_cast<uint16_t*>(smp(OFF_TAPS + ab * 768));
            for (int m = r; m < 384; m += 128) {
                const int l = m - 128;
                float v = 0.f;
                if (l >= 0 && l < K) v = ld_param(a.h, a.h_dtype, fg * K + (a.taps == VTX_TAPS_CONV ? l : K - 1 - l));
                tp[m] = __bfloat16_as_ushort(__float2bfloat16_rn(v));
            }
            if (r < CH) reinterpret_cast<float*>(smp(OFF_DIAG + ab * 64))[r] = a.bias_mode == VTX_BIAS_GATED ? ld_param(a.bias, a.bias_dtype, (int64_t)blk * CH + r) : 0.f;
            __syncwarp();
            if (lane == 0) mbar_arrive(taps_ready(ab));
            if (!mbar_wait(taps_ready(ab), (uint32_t)((t >> 1) & 1), 33)) return false;
            for (int c0 = 0; c0 < 128; c0 += 16) {
                uint32_t v[16];
#pragma unroll
                for (int m = 0; m < 16; ++m) {
                    const int j = 2 * (c0 + m);                            // columns j, j+1 of [T^|T]: lag = 128 + i - j
                    const uint32_t e0 = tp[128 + 128 + r - j], e1 = tp[128 + 127 + r - j];
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
        bool ok = sh == 0 ? expand(0) : true;      // (the first four warps expand the operands)
        int pending = -1;          // q stage whose tile of outputs the TMA unit may still be reading
        for (int t = 0; t < nmine && ok; ++t) {
            const int blk = item_blk(t);
            const float* dsk = reinterpret_cast<const float*>(smp(OFF_DIAG + (t & 1) * 64));
            // The outputs of a chunk replace the q tile in place (same column, same sample), and one thread hands the
            // tile to the TMA unit: boxes of [16 channels x 64 samples] (x 4 batch elements) stored with whole 128-byte
            // rows along time; samples past the end of the sequence are clipped by the tensor map.
            int x0[NS], bi[NS];
            bool act[NS];
#pragma unroll
            for (int s = 0; s < NS; ++s) {
                const Stream st = stream_of(a, item_quad(t), s);
                x0[s] = (int)st.ts; bi[s] = (int)st.b; act[s] = st.active;
            }
            const int64_t d0 = (int64_t)blk * CH;
            if (lane == 0) mbar_arrive(kv_free(cc % NSLOT));       // the item's halo chunk has no epilogue
            ++cc;
            for (int k = 1; k < nchunk; ++k, ++cc, ++oc) {
                const int slot = cc % NSLOT, dbuf = oc & 1, qs = oc % NQ;
                if (!mbar_wait(d_full(dbuf), (oc >> 1) & 1u, 34)) { ok = false; break; }
                if (!mbar_wait(q_full(qs), (oc / NQ) & 1u, 35)) { ok = false; break; }
                tc_fence_after();
                __syncwarp();
                const uint32_t taddr = tmem + ((uint32_t)(e * 32) << 16) + D_COL + dbuf * 64;
                // this thread's sample in column n of a tile: base + n * 128 + xo[n & 7]
                const uint32_t rbase = (uint32_t)((r >> 6) * HALF_TILE + (r & 7) * 2);
                const uint32_t q_u = sm_u + OFF_Q + qs * TILE + rbase, kv_u = sm_u + OFF_SLOTS + slot * TILE + rbase;
                uint32_t xo[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) xo[i] = (uint32_t)(((((r & 63) >> 3) ^ i)) << 4);
                auto lds16 = [&](uint32_t addr) {
                    unsigned short v;
                    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
                    return (uint32_t)v;
                };
                // (rolled over the streams: the unrolled form did not fit the instruction cache next to the other roles)
#pragma unroll 1
                for (int s = 2 * sh; s < 2 * sh + 2; ++s) {
                    uint32_t acc[16];
                    tmem_ld16(taddr + s * 16, acc);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    tmem_ld_touch(acc);
                    if (s == 2 * sh + 1) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(d_empty(dbuf));
                    }
#pragma unroll
                    for (int c = 0; c < CH; c += 2) {
                        // (16 s + c) & 7 == c & 7: the swizzle term of a column does not depend on the stream
                        const uint32_t o0 = (uint32_t)((s * CH + c) * 128) + xo[c & 7], o1 = (uint32_t)((s * CH + c + 1) * 128) + xo[(c + 1) & 7];
                        f32x2 z = pk2(__uint_as_float(acc[c]), __uint_as_float(acc[c + 1]));
                        if (a.bias_mode == VTX_BIAS_GATED) {
                            const f32x2 kvv = pk2(__uint_as_float(lds16(kv_u + o0) << 16), __uint_as_float(lds16(kv_u + o1) << 16));
                            const f32x2 dd = *reinterpret_cast<const f32x2*>(dsk + c);
                            if (a.taps == VTX_TAPS_CONV) {
                                z = fma2(dd, kvv, z);                       // fp32 sum, one rounding (engine.py:78,187)
                            } else {
                                float z0, z1, b0, b1;
                                up2(z, z0, z1);
                                up2(mul2(dd, kvv), b0, b1);
                                const uint32_t zr = pack_bf16(z0, z1), br = pack_bf16(b0, b1);
                                z = add2(pk2(bf_lo(zr), bf_hi(zr)), pk2(bf_lo(br), bf_hi(br)));
                            }
                        }
                        float z0, z1;
                        up2(z, z0, z1);
                        const uint32_t zr = pack_bf16(z0, z1);                 // the filter output in the I/O dtype
                        const f32x2 qv = pk2(__uint_as_float(lds16(q_u + o0) << 16), __uint_as_float(lds16(q_u + o1) << 16));
                        float y0, y1;
                        up2(mul2(qv, pk2(bf_lo(zr), bf_hi(zr))), y0, y1);
                        const uint32_t yr = pack_bf16(y0, y1);
                        asm volatile("st.shared.u16 [%0], %1;" ::"r"(q_u + o0), "h"((unsigned short)(yr & 0xffffu)) : "memory");
                        asm volatile("st.shared.u16 [%0], %1;" ::"r"(q_u + o1), "h"((unsigned short)(yr >> 16)) : "memory");
                    }
                }
                // k*v has been read: the slot may go; the tile of outputs goes to the TMA unit once all four warps wrote it
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) { mbar_arrive(kv_free(slot)); mbar_arrive(y_ready(oc & 1)); }
                if (warp == W_EP && lane == 0 && mbar_wait(y_ready(oc & 1), (oc >> 1) & 1u, 42)) {
                    const uint32_t src = sm_u + OFF_Q + qs * TILE;
                    const int row = (int)(d0 % a.hdy), head = (int)(d0 / a.hdy);
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
                        if (a.batch_quads) {
                            const int x = x0[0] + (k - 1) * CHUNK + hf * 64;
                            if (x < a.L) tma_store_4d(&tmy, src + hf * HALF_TILE, x, row, head, bi[0]);
                        } else {
#pragma unroll
                            for (int s = 0; s < NS; ++s) {
                                const int x = x0[s] + (k - 1) * CHUNK + hf * 64;
                                if (act[s] && x < a.L) tma_store_4d(&tmy, src + hf * HALF_TILE + s * CH * 128, x, row, head, bi[s]);
                            }
                        }
                    }
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    // the tile before this one has been read by now (one group may stay in flight): its stage is free
                    asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    if (pending >= 0) mbar_arrive(q_empty(pending));
                    pending = qs;
                }
                if (sh == 0 && k == 1 && t + 1 < nmine && !expand(t + 1)) { ok = false; break; }
            }
        }
        if (warp == W_EP && lane == 0) {
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            if (pending >= 0) mbar_arrive(q_empty(pending));
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");        // the last stores have landed before the CTA ends
        }
    } else if (warp == W_MMA) {
        // ======== MMA issue =========================================================================
        if (lane == 0) {
            const uint32_t idesc = instr_desc_kmajor(128, NCOL);
            // B operand of one K step: 64 columns x 16 samples, K-major: rows of 128 bytes (64 samples) with the
            // 128-byte swizzle, 8-row groups 1024 B apart (SBO); a K step moves the start address by 32 bytes inside
            // the row, the second half of the chunk sits HALF_TILE further on.
            uint64_t kv_desc[NSLOT];
#pragma unroll
            for (int sl = 0; sl < NSLOT; ++sl) kv_desc[sl] = smem_desc(sm_u + OFF_SLOTS + sl * TILE, 16, 1024, 2);
            auto issue_half = [&](int abuf, int slot, int dbuf, bool cur) {
                const uint32_t d = tmem + D_COL + dbuf * 64;
                const uint32_t a0 = tmem + abuf * 128 + (cur ? 64 : 0);
                const uint64_t dk = slot ? kv_desc[1] : kv_desc[0];
#pragma unroll
                for (int jj = 0; jj < 8; ++jj)
                    mma_ts(d, a0 + 8 * jj, dk + (uint64_t)(((jj / 4) * HALF_TILE + (jj % 4) * 32) >> 4), idesc, (cur || jj > 0) ? 1u : 0u);
            };
            bool ok = true;
            for (int t = 0; t < nmine && ok; ++t) {
                const int ab = t & 1;
                if (!mbar_wait(a_ready(ab), (uint32_t)((t >> 1) & 1), 36)) { ok = false; break; }
                if (!mbar_wait(kv_full(cc % NSLOT), (cc / NSLOT) & 1u, 37)) { ok = false; break; }
                if (nchunk > 1) {
                    if (oc >= 2 && !mbar_wait(d_empty(oc & 1), ((oc - 2) >> 1) & 1u, 38)) { ok = false; break; }
                    tc_fence_after();
                    issue_half(ab, cc % NSLOT, oc & 1, false);
                }
                mma_commit(kv_free(cc % NSLOT));
                ++cc;
                for (int k = 1; k < nchunk; ++k, ++cc, ++oc) {
                    if (!mbar_wait(kv_full(cc % NSLOT), (cc / NSLOT) & 1u, 39)) { ok = false; break; }
                    tc_fence_after();
                    issue_half(ab, cc % NSLOT, oc & 1, true);
                    mma_commit(d_full(oc & 1));
                    if (k + 1 < nchunk) {
                        if (oc >= 1 && !mbar_wait(d_empty((oc + 1) & 1), ((oc - 1) >> 1) & 1u, 40)) { ok = false; break; }
                        tc_fence_after();
                        issue_half(ab, cc % NSLOT, (oc + 1) & 1, false);
                    }
                    mma_commit(kv_free(cc % NSLOT));
                }
            }
        }
    } else if (warp == W_TKV || warp == W_TQ) {
        // ======== TMA issue: one warp for the k and v tiles of every chunk, one for the q tiles of the output chunks ====
        if (lane == 0) {
            const bool isq = warp == W_TQ;
            tma_prefetch_desc(isq ? &tmq : &tmk);
            if (!isq) tma_prefetch_desc(&tmv);
            uint32_t n = 0;
            bool ok = true;
            for (int t = 0; t < nmine && ok; ++t) {
                const int64_t d0 = (int64_t)item_blk(t) * CH;
                const int row = (int)(d0 % a.hd), head = (int)(d0 / a.hd);
                int t0[NS], bi[NS];
#pragma unroll
                for (int s = 0; s < NS; ++s) {
                    const Stream st = stream_of(a, item_quad(t), s);
                    t0[s] = (int)st.ts - CHUNK;
                    bi[s] = (int)st.b;
                }
                for (int k = isq ? 1 : 0; k < nchunk; ++k, ++n) {
                    const int ring = isq ? NQ : NKV, stg = (int)(n % ring);
                    const uint32_t full = isq ? q_full(stg) : kvin_full(stg), empty = isq ? q_empty(stg) : kvin_empty(stg);
                    if (n >= (uint32_t)ring && !mbar_wait(empty, ((n - ring) / ring) & 1u, 41)) { ok = false; break; }
                    mbar_expect_tx(full, isq ? TILE : 2 * TILE);
                    const uint32_t base = sm_u + (isq ? OFF_Q + stg * TILE : OFF_KV_IN + stg * 2 * TILE);
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
                        if (a.batch_quads) {
                            const int x = t0[0] + k * CHUNK + hf * 64;
                            if (isq) {
                                tma_load_4d(base + hf * HALF_TILE, &tmq, full, x, row, head, bi[0]);
                            } else {
                                tma_load_4d(base + hf * HALF_TILE, &tmk, full, x, row, head, bi[0]);
                                tma_load_4d(base + TILE + hf * HALF_TILE, &tmv, full, x, row, head, bi[0]);
                            }
                        } else {
#pragma unroll
                            for (int s = 0; s < NS; ++s) {
                                const int x = t0[s] + k * CHUNK + hf * 64;
                                const uint32_t o = (uint32_t)(hf * HALF_TILE + s * CH * 128);
                                if (isq) {
                                    tma_load_4d(base + o, &tmq, full, x, row, head, bi[s]);
                                } else {
                                    tma_load_4d(base + o, &tmk, full, x, row, head, bi[s]);
                                    tma_load_4d(base + TILE + o, &tmv, full, x, row, head, bi[s]);
                                }
                            }
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == W_MMA) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
    }
}

}  // namespace gtc

// Shapes the tensor-core path takes; everything else stays on the general kernel.
bool gcg_tc_shape(const vtx_gcg_params* p) {
    using namespace gtc;
    if (p->io_dtype != VTX_BF16 || p->h_dtype != VTX_BF16 || p->K > CHUNK || p->K < 1 || !p->round_kv || p->mask ||
        p->bias_mode == VTX_BIAS_ADD)
        return false;
    if (p->D % CH || p->G <= 0 || p->D % p->G || (p->D / p->G) % CH || p->head_dim % CH) return false;
    if (p->y_stride_l != 1 || p->L % 8 || reinterpret_cast<uintptr_t>(p->y) % 16 || p->y_stride_d <= 0 || p->y_stride_d % 8 ||
        (p->B > 1 && (p->y_stride_b <= 0 || p->y_stride_b % 8)))
        return false;
    const void* ptrs[3] = {p->q, p->k, p->v};
    const int64_t sd[3] = {p->q_stride_d, p->k_stride_d, p->v_stride_d}, sh[3] = {p->q_stride_h, p->k_stride_h, p->v_stride_h},
                  sb[3] = {p->q_stride_b, p->k_stride_b, p->v_stride_b};
    const int64_t heads = p->D / p->head_dim;
    for (int i = 0; i < 3; ++i) {
        if (reinterpret_cast<uintptr_t>(ptrs[i]) % 16 || sd[i] <= 0 || sd[i] % 8) return false;
        if (heads > 1 && (sh[i] <= 0 || sh[i] % 8)) return false;
        if (p->B > 1 && (sb[i] <= 0 || sb[i] % 8)) return false;
    }
    return p->L < ((int64_t)1 << 30) && p->B < 65536;
}

int gcg_tc_fwd(const vtx_gcg_params* p, cudaStream_t stream) {
    using namespace gtc;
    Args a{};
    a.h = p->h; a.h_dtype = p->h_dtype; a.bias = p->bias; a.bias_dtype = p->bias_dtype;
    a.y = static_cast<__nv_bfloat16*>(p->y); a.y_stride_b = p->y_stride_b; a.y_stride_d = p->y_stride_d;
    a.state = (p->state && p->K > 1) ? static_cast<__nv_bfloat16*>(p->state) : nullptr;
    a.B = p->B; a.L = p->L; a.D = p->D; a.K = p->K; a.dg = p->D / p->G; a.hd = p->head_dim;
    a.taps = (int)p->taps; a.bias_mode = (int)p->bias_mode;
    a.nblk = p->D / CH;
    a.batch_quads = p->B >= 3;
    // time segments: as in the fused kernel, the launch lasts as long as the CTA with the most chunks
    const int64_t nchunks_total = ceil_div<int64_t>(p->L, CHUNK);
    int64_t nseg = 1, best_cost = INT64_MAX;
    for (int64_t seg_chunks = nchunks_total; seg_chunks >= 1; --seg_chunks) {
        const int64_t ns_ = ceil_div<int64_t>(nchunks_total, seg_chunks);
        if (ceil_div<int64_t>(nchunks_total, ns_) != seg_chunks) continue;
        const int64_t quads = a.batch_quads ? ceil_div<int64_t>(p->B, NS) * ns_ : ceil_div<int64_t>(p->B * ns_, NS);
        const int64_t items = a.nblk * quads;
        const int64_t cost = ceil_div<int64_t>(items, kNumSMs) * (seg_chunks + 1) * 64 + ns_;
        if (cost < best_cost) { best_cost = cost; nseg = ns_; }
        if (seg_chunks <= 2 || items > (int64_t)kNumSMs * 64) break;
    }
    a.seg_len = ceil_div<int64_t>(nchunks_total, nseg) * CHUNK;
    a.nseg = ceil_div<int64_t>(p->L, a.seg_len);
    a.nquad = a.batch_quads ? ceil_div<int64_t>(p->B, NS) * a.nseg : ceil_div<int64_t>(p->B * a.nseg, NS);
    a.nitems = a.nblk * a.nquad;
    VTX_REQUIRE(a.nitems < (int64_t)1 << 31, VTX_ERR_UNSUPPORTED, "gcg: too many work items");

    CUtensorMap tm[3];
    const void* ptrs[3] = {p->q, p->k, p->v};
    const int64_t sd[3] = {p->q_stride_d, p->k_stride_d, p->v_stride_d}, sh[3] = {p->q_stride_h, p->k_stride_h, p->v_stride_h},
                  sb[3] = {p->q_stride_b, p->k_stride_b, p->v_stride_b};
    for (int i = 0; i < 3; ++i)
        if (int rc = make_tmap_bhdl(&tm[i], ptrs[i], VTX_BF16, p->L, p->head_dim, p->D / p->head_dim, p->B, sd[i], sh[i], sb[i],
                                    64, CH, a.batch_quads ? NS : 1, "gcg(tensor cores)"))
            return rc;
    CUtensorMap tmy;
    if (int rc = make_tmap_bhdl(&tmy, p->y, VTX_BF16, p->L, p->D, 1, p->B, p->y_stride_d, p->y_stride_d * p->D, p->y_stride_b,
                                64, CH, a.batch_quads ? NS : 1, "gcg(tensor cores, y)"))
        return rc;
    a.hdy = p->D;
    static bool attr_set[64] = {};
    static int resident[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    const bool known = dev >= 0 && dev < 64;
    if (!known || !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(gcg_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return fail(VTX_ERR_LAUNCH, "gcg(tensor cores): shared memory opt-in: %s", cudaGetErrorString(e));
        if (known) attr_set[dev] = true;
    }
    int nres = known ? resident[dev] : 0;
    if (nres == 0) {
        int sms = 0, per_sm = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gcg_tc_kernel, THREADS, SMEM_BYTES);
        nres = sms * per_sm;
        if (nres <= 0) return fail(VTX_ERR_LAUNCH, "gcg(tensor cores): the kernel does not fit an SM");
        if (known) resident[dev] = nres;
    }
    const int64_t ncta = a.nitems < nres ? a.nitems : nres;
    gcg_tc_kernel<<<(unsigned)ncta, THREADS, SMEM_BYTES, stream>>>(tm[0], tm[1], tm[2], tmy, a);
    return check_launch("gcg(tensor cores)");
}

}  // namespace vtx
