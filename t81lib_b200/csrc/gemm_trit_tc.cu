// Prefill-shaped TRIT-mode kernel on the 5th-generation tensor cores (placeholder
// until the tcgen05 pipeline lands: reports "not eligible" so the dispatcher uses
// the general kernel).
#include "common.cuh"

namespace t81b200 {

bool gemm_trit_tc_eligible(int, int, int, int64_t, int64_t, int64_t) { return false; }
size_t gemm_trit_tc_workspace(int, int, int, int64_t, int64_t, int64_t) { return 0; }
int gemm_trit_tc_launch(const uint8_t *, const float *, const void *, int, int, int64_t, const float *, void *, int,
                        int64_t, int64_t, int64_t, int64_t, float, float, void *, size_t, cudaStream_t) {
    return fail(T81B200_EINVAL, "tensor-core kernel not built");
}

}  // namespace t81b200
