// Log-sum-exp merge of the softmax partials of one query head, by one thread block.
#pragma once
#include <math_constants.h>

namespace hira {

// part_o / part_ml point at the head's row of part 0; part s lies s * {o,ml}_part_stride floats on.
//   out = sum_s e^{m_s-M} o_s / sum_s e^{m_s-M} l_s      (o_s unnormalised), or with normalised o_s
//   (sequence shards) o_s first scaled back by l_s.
// The partials are read past L1 (ld.global.cg): they may have been written by another GPU.
__device__ __forceinline__ void merge_row(const float* part_o, const float* part_ml, long long o_part_stride,
                                          long long ml_part_stride, int n_parts, int vdim, int normalised,
                                          float* __restrict__ out, float* __restrict__ out_ml) {
    float M = -CUDART_INF_F;
    for (int s = 0; s < n_parts; ++s) M = fmaxf(M, __ldcg(part_ml + s * ml_part_stride));
    float L = 0.f;
    for (int s = 0; s < n_parts; ++s) {
        const float ms = __ldcg(part_ml + s * ml_part_stride);
        const float ls = __ldcg(part_ml + s * ml_part_stride + 1);
        if (ms > -CUDART_INF_F) L += ls * __expf(ms - M);
    }
    for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
        float o = 0.f;
        for (int s = 0; s < n_parts; ++s) {
            const float ms = __ldcg(part_ml + s * ml_part_stride);
            if (ms > -CUDART_INF_F) {
                float w = __expf(ms - M);
                if (normalised) w *= __ldcg(part_ml + s * ml_part_stride + 1);
                o += w * __ldcg(part_o + s * o_part_stride + d);
            }
        }
        out[d] = L > 0.f ? o / L : 0.f;
    }
    if (out_ml && threadIdx.x == 0) {
        out_ml[0] = M;
        out_ml[1] = L;
    }
}

}  // namespace hira
