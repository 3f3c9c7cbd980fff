// Tensor-core (tcgen05 / TMEM) nearest-centroid assignment for bf16 points.
#include "common.cuh"

namespace hira {

bool assign_tc_supported(int dtype, int n, int k, int dim) {
    (void)dtype; (void)n; (void)k; (void)dim;
    return false;
}

int launch_assign_tc(const void*, long long, const void*, const float*, int, int, int, int, int32_t*, float*,
                     cudaStream_t) {
    set_error("tensor-core assignment is not available for this shape");
    return HIRA_ERR_ARG;
}

}  // namespace hira
