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
    const float2* ml = reinterpret_cast<const float2*>(part_ml) + base;     // (max, sum) per partition
    // Loads go out eight at a time and none depends on another's value, so a merge costs one or
    // two round trips to L2 however many partitions there are; terms are added in the order p = 0, 1, ...
    float M = -INFINITY;
    for (int p0 = 0; p0 < NP; p0 += 8) {
        float2 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (p0 + j < NP) v[j] = ml[p0 + j];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (p0 + j < NP && v[j].y > 0.f) M = fmaxf(M, v[j].x);
    }
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float L = 0.f, o = 0.f;
        for (int p0 = 0; p0 < NP; p0 += 8) {
            float2 v[8];
            float x[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                v[j] = make_float2(0.f, 0.f);
                if (p0 + j < NP) v[j] = ml[p0 + j];                          // in L1 after the first pass
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                x[j] = 0.f;
                if (v[j].y > 0.f) x[j] = part_o[(base + p0 + j) * D + d];    // an empty partition's o is never read
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (v[j].y > 0.f) {
                    const float w = expf(v[j].x - M);
                    L += w * v[j].y;
                    o += w * x[j];
                }
        }
        out[((size_t)n * Hq + h) * D + d] = from_float<T>(o * (1.0f / L));
    }
}

}  // namespace sb
