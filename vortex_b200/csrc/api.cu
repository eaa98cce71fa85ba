// Error plumbing and ABI version of the vortex_b200 C ABI.
#include <atomic>
#include <cstring>

#include "common.cuh"
#include "tma.cuh"

namespace vtx {

static thread_local char g_last_error[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
    return code;
}

static std::atomic<long long> g_launches{0};
int check_launch(const char* what, long long launches) {
    g_launches.fetch_add(launches, std::memory_order_relaxed);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(VTX_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
    return VTX_OK;
}

static int g_flag_poll_limit = 1 << 21;
int flag_poll_limit() { return g_flag_poll_limit; }

static StatusReader* g_readers = nullptr;
void register_status_reader(StatusReader* r) {
    r->next = g_readers;
    g_readers = r;
}

// ---- tensor-map encoding through the driver entry point ------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

int make_tmap_3d(CUtensorMap* out, const void* base, int64_t dtype, int64_t cols, int64_t rows, int64_t batch,
                 int64_t row_stride, int64_t batch_stride, int box_cols, int box_rows, int swizzle_bytes,
                 const char* who) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(VTX_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled entry point unavailable", who);
    const int64_t es = dtype_size(dtype);
    if (reinterpret_cast<uintptr_t>(base) % 16 || (row_stride * es) % 16 || (batch_stride * es) % 16)
        return fail(VTX_ERR_ALIGNMENT, "%s: base address and row/batch pitch must be multiples of 16 bytes", who);
    if ((box_cols * es) % 16) return fail(VTX_ERR_ALIGNMENT, "%s: box width must be a multiple of 16 bytes", who);
    CUtensorMapDataType dt = dtype == VTX_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                             : dtype == VTX_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
    cuuint64_t strides[2] = {(cuuint64_t)(row_stride * es), (cuuint64_t)(batch_stride * es)};
    if (batch == 1) strides[1] = strides[0] * (cuuint64_t)rows;   // any legal value: never used to step
    cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUtensorMapSwizzle sw = swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                            : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                            : swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                                  : CU_TENSOR_MAP_SWIZZLE_NONE;
    // 256-byte L2 promotion: the row pieces of neighbouring CTAs are neighbours in memory (measured on the fused FIR
    // kernel against none / 64 / 128 bytes: 1 % faster than 128, 2 % faster than 64)
    CUresult r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(VTX_ERR_BAD_ARG, "%s: cuTensorMapEncodeTiled failed with CUresult %d", who, (int)r);
    return VTX_OK;
}

int make_tmap_bhdl(CUtensorMap* out, const void* base, int64_t dtype, int64_t L, int64_t head_dim, int64_t heads,
                   int64_t batch, int64_t stride_d, int64_t stride_h, int64_t stride_b, int box_cols, int box_rows,
                   int box_batch, const char* who) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(VTX_ERR_LAUNCH, "%s: cuTensorMapEncodeTiled entry point unavailable", who);
    const int64_t es = dtype_size(dtype);
    if (heads <= 1) { heads = 1; stride_h = stride_d * head_dim; }      // never stepped: any legal pitch
    if (batch <= 1) { batch = 1; stride_b = stride_h * heads; }
    if (reinterpret_cast<uintptr_t>(base) % 16 || (stride_d * es) % 16 || (stride_h * es) % 16 || (stride_b * es) % 16 ||
        stride_d <= 0 || stride_h <= 0 || stride_b <= 0)
        return fail(VTX_ERR_ALIGNMENT, "%s: base address and channel / head / batch pitch must be positive multiples of 16 bytes", who);
    if (box_cols * es != 128) return fail(VTX_ERR_ALIGNMENT, "%s: a swizzled box row is 128 bytes", who);
    CUtensorMapDataType dt = dtype == VTX_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                             : dtype == VTX_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    cuuint64_t dims[4] = {(cuuint64_t)L, (cuuint64_t)head_dim, (cuuint64_t)heads, (cuuint64_t)batch};
    cuuint64_t strides[3] = {(cuuint64_t)(stride_d * es), (cuuint64_t)(stride_h * es), (cuuint64_t)(stride_b * es)};
    cuuint32_t box[4] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1, (cuuint32_t)box_batch};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(out, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(VTX_ERR_BAD_ARG, "%s: cuTensorMapEncodeTiled failed with CUresult %d", who, (int)r);
    return VTX_OK;
}

}  // namespace vtx

extern "C" int vtx_device_status(void) {
    int worst = 0;
    for (vtx::StatusReader* r = vtx::g_readers; r; r = r->next) {
        int v = r->take();
        if (v && !worst) worst = v;
    }
    if (worst) vtx::fail(VTX_ERR_DEVICE, "a kernel gave up a bounded wait (code %d)", worst);
    return worst ? VTX_ERR_DEVICE : VTX_OK;
}

extern "C" int64_t vtx_launch_count(void) { return (int64_t)vtx::g_launches.load(std::memory_order_relaxed); }

extern "C" int vtx_debug_set_flag_poll_limit(int64_t polls) {
    if (polls < 0 || polls > (1 << 30)) return vtx::fail(VTX_ERR_BAD_ARG, "flag poll limit out of range");
    vtx::g_flag_poll_limit = polls == 0 ? 1 << 21 : (int)polls;
    return VTX_OK;
}

extern "C" size_t vtx_last_error(char* buf, size_t len) {
    size_t n = strlen(vtx::g_last_error);
    if (buf && len) {
        size_t m = n < len - 1 ? n : len - 1;
        memcpy(buf, vtx::g_last_error, m);
        buf[m] = 0;
    }
    return n;
}

extern "C" int64_t vtx_abi_version(void) { return VTX_ABI_VERSION; }

extern "C" int64_t vtx_struct_size(int64_t which) {
    switch (which) {
        case 0: return sizeof(vtx_featurizer_params);
        case 1: return sizeof(vtx_gcg_params);
        case 2: return sizeof(vtx_fused_fir_params);
        case 3: return sizeof(vtx_modal_params);
        case 4: return sizeof(vtx_iir_params);
        case 5: return sizeof(vtx_step_fir_params);
        case 6: return sizeof(vtx_step_iir_params);
        case 7: return sizeof(vtx_decode_layer_params);
        case 8: return sizeof(vtx_fused_iir_params);
        case 9: return sizeof(vtx_hyena_x_params);
        case 10: return sizeof(vtx_causal_conv1d_params);
        case 11: return sizeof(vtx_causal_conv1d_update_params);
        case 12: return sizeof(vtx_varlen_states_params);
        case 13: return sizeof(vtx_gcg_cl_params);
        case 14: return sizeof(vtx_gcg_bwd_params);
        default: return -1;
    }
}
