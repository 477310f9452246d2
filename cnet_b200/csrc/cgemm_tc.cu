// tcgen05 3xTF32 complex GEMM (placeholder until the tensor-core tiles land: reports every
// shape as unsupported so the dispatch uses the fp32 SIMT tiles).
#include "common.cuh"

namespace cnb {
bool cgemm_tc_shape_ok(int, int, int) { return false; }
int cgemm_tc_nt(cnb_ctx*, const float*, const float*, const float*, const float*, int, const float*, const float*,
                float*, float*, int, int, int, int, cudaStream_t) {
    return set_error(CNB_ERR_UNSUPPORTED, "tensor-core GEMM not built");
}
void cgemm_tc_release(cnb_ctx*) {}
}  // namespace cnb
