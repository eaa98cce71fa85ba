// Hyena-MR fused block (placeholder translation unit until the tcgen05 kernel lands).
#include "common.cuh"

namespace vtx {
int fused_mr_tc_fwd(const vtx_fused_fir_params* p, cudaStream_t) {
    return fail(VTX_ERR_UNSUPPORTED, "fused_fir: filter length %lld has no fused kernel", (long long)p->K);
}
}  // namespace vtx
