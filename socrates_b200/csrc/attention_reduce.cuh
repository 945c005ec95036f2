// Merge of the key partitions of split attention, shared by the SIMT and the
// tensor-core attention kernels.
#pragma once

#include <math.h>

#include "common.cuh"

namespace sb {

// out[n,h,:] = sum_p e^{m_p - M} o_p / sum_p e^{m_p - M} l_p,  M = max_p m_p.
// Partitions with l == 0 hold no key and are skipped (their o is not even read).
template <typename T>
__global__ void attn_reduce_kernel(T* __restrict__ out, const float* __restrict__ part_o,
                                   const float* __restrict__ part_ml, int Hq, int D, int NP) {
    sb::pdl_launch_dependents();     // the next kernel may begin its prologue
    sb::pdl_wait();                  // everything before this kernel is complete and visible
    const int h = blockIdx.x, n = blockIdx.y;
    const size_t base = ((size_t)n * Hq + h) * NP;
    float M = -INFINITY;
    for (int p = 0; p < NP; ++p)
        if (part_ml[(base + p) * 2 + 1] > 0.f) M = fmaxf(M, part_ml[(base + p) * 2]);
    float L = 0.f;
    for (int p = 0; p < NP; ++p) {
        const float l = part_ml[(base + p) * 2 + 1];
        if (l > 0.f) L += expf(part_ml[(base + p) * 2] - M) * l;
    }
    const float inv = 1.0f / L;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float o = 0.f;
        for (int p = 0; p < NP; ++p) {
            const float l = part_ml[(base + p) * 2 + 1];
            if (l > 0.f) o += expf(part_ml[(base + p) * 2] - M) * part_o[(base + p) * D + d];
        }
        out[((size_t)n * Hq + h) * D + d] = from_float<T>(o * inv);
    }
}


}  // namespace sb
