// TMA (cp.async.bulk.tensor) and mbarrier helpers, plus host-side tensor-map
// encoding through the driver entry point (no link-time dependency on libcuda).
// No cluster multicast anywhere: every CTA fetches its own tiles.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace vtx {

// Device status word (one per translation unit that includes this header): a
// kernel whose bounded wait ran out stores a code here and returns;
// vtx_device_status() reads and clears the words of all units.
static __device__ int g_device_status;

struct StatusReader {
    int (*take)();
    StatusReader* next;
};
void register_status_reader(StatusReader* r);
#define VTX_DEFINE_STATUS_READER()                                              \
    namespace {                                                                 \
    int tu_take_status() {                                                      \
        int v = 0;                                                              \
        if (cudaMemcpyFromSymbol(&v, ::vtx::g_device_status, sizeof(int)) != cudaSuccess) return -1; \
        if (v) { int z = 0; cudaMemcpyToSymbol(::vtx::g_device_status, &z, sizeof(int)); }           \
        return v;                                                               \
    }                                                                           \
    struct Registrar {                                                          \
        ::vtx::StatusReader r{tu_take_status, nullptr};                         \
        Registrar() { ::vtx::register_status_reader(&r); }                      \
    } g_registrar;                                                              \
    }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded spin without suspending (for single issuing threads that sit on the critical path).
__device__ __forceinline__ bool mbar_spin(uint32_t bar, uint32_t parity, int code) {
    for (int it = 0; it < (1 << 26); ++it)
        if (mbar_test_wait(bar, parity)) return true;
    atomicCAS(&g_device_status, 0, code);
    return false;
}
// Bounded wait: gives up after ~2^22 polls (each poll may itself block for a
// hardware-defined interval), records `code` in the status word and returns false.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int code) {
    for (int it = 0; it < (1 << 22); ++it)
        if (mbar_try_wait(bar, parity)) return true;
    atomicCAS(&g_device_status, 0, code);
    return false;
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z, int w) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}
// shared -> global tile store (bulk async group of the issuing thread); out-of-range elements are not written
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int x, int y, int z, int w) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(map), "r"(src), "r"(x), "r"(y), "r"(z), "r"(w)
                 : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(map), "r"(src), "r"(x), "r"(y), "r"(z)
                 : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- host: tensor map over a [batch, rows, cols] tensor, cols contiguous -------------------------
// Element strides; box = [1, box_rows, box_cols].  Out-of-range box elements read as zero.
int make_tmap_3d(CUtensorMap* out, const void* base, int64_t dtype, int64_t cols, int64_t rows, int64_t batch,
                 int64_t row_stride, int64_t batch_stride, int box_cols, int box_rows, int swizzle_bytes,
                 const char* who);

// Tensor map over a channel-first operand [batch, head, channel-in-head, time], time contiguous, the other three
// dimensions by element strides; box = [box_batch, 1, box_rows, box_cols] with the 128-byte swizzle (box_cols * element
// size must be 128 bytes).  Out-of-range box elements read as zero.
int make_tmap_bhdl(CUtensorMap* out, const void* base, int64_t dtype, int64_t L, int64_t head_dim, int64_t heads,
                   int64_t batch, int64_t stride_d, int64_t stride_h, int64_t stride_b, int box_cols, int box_rows,
                   int box_batch, const char* who);

}  // namespace vtx
