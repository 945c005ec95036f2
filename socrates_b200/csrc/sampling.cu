// Sampling over float32 logits: greedy argmax and temperature (Gumbel-max) with a
// counter-based generator, one block per row.  The generator is a function of
// (seed, counter, vocabulary index) alone, so a request's draws do not depend on
// what else is in the batch.
#include "common.cuh"

namespace {

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
    x ^= x >> 16;
    x *= 0x7FEB352Du;
    x ^= x >> 15;
    x *= 0x846CA68Bu;
    x ^= x >> 16;
    return x;
}

// Uniform in (0,1) with 23 random bits, centred in its cell: (k + 0.5) / 2^23 is
// exact in float32 and never 0 or 1.
__device__ __forceinline__ float uniform_for(uint32_t key, uint32_t index) {
    const uint32_t x = mix32((index + 0x165667B1u) ^ key);
    return ((float)(x >> 9) + 0.5f) * (1.0f / 8388608.0f);
}

__device__ __forceinline__ bool better(float v, int i, float best, int best_i) {
    return v > best || (v == best && i < best_i);
}

// temperature[m] == 0: argmax, ties to the lowest index.
// temperature[m] > 0 : argmax_i (logit_i / T - log(-log u_i)).
// grid (M, C): block c of row m scans one slice of the vocabulary and leaves its best
// (score, index) in `scratch`; the block of a row that finishes last (a counter in
// `scratch`) merges the C candidates and writes out[m].  The merge is an argmax over
// exact values with the index as tie-break, so its order does not matter.
//   scratch: int32 [M, 2*C + 1]; the counters (last entry of each row) are zero before
//   the first call and are reset by the merging block.
__global__ void sample_kernel(int* __restrict__ out, const float* __restrict__ logits,
                              const float* __restrict__ temperature, const uint32_t* __restrict__ seeds,
                              const uint32_t* __restrict__ counters, int V, int* __restrict__ scratch) {
    sb::pdl_launch_dependents();     // the next kernel may begin its prologue
    sb::pdl_wait();                  // everything before this kernel is complete and visible
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ int s_last;
    const int m = blockIdx.x, C = gridDim.y;
    const float* row = logits + (size_t)m * V;
    const float T = temperature ? temperature[m] : 0.f;
    uint32_t key = 0;
    if (T > 0.f) {
        key = mix32(seeds[m] ^ 0x9E3779B9u);
        key = mix32(key ^ mix32(counters[m] + 0x85EBCA6Bu));
    }
    const float inv_t = T > 0.f ? 1.0f / T : 1.0f;
    const int per = (V + C - 1) / C;
    const int begin = blockIdx.y * per, end = min(V, begin + per);
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        float v = row[i];
        if (T > 0.f) {
            const float u = uniform_for(key, (uint32_t)i);
            v = v * inv_t - logf(-logf(u));
        }
        if (better(v, i, best, best_i)) { best = v; best_i = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
    __syncthreads();
    int* mine = scratch + (size_t)m * (2 * C + 1);
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        best = lane < nw ? s_val[lane] : -INFINITY;
        best_i = lane < nw ? s_idx[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
        }
        if (lane == 0) {
            mine[2 * blockIdx.y] = __float_as_int(best);
            mine[2 * blockIdx.y + 1] = best_i;
            __threadfence();
            s_last = atomicAdd(&mine[2 * C], 1) == C - 1;
        }
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (warp == 0) {
        best = -INFINITY;
        best_i = 0x7fffffff;
        for (int c = lane; c < C; c += 32) {
            const float v = __int_as_float(((volatile int*)mine)[2 * c]);
            const int i = ((volatile int*)mine)[2 * c + 1];
            if (better(v, i, best, best_i)) { best = v; best_i = i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
        }
        if (lane == 0) {
            // A row of NaNs or -inf leaves best_i untouched; report index 0 rather than garbage.
            out[m] = best_i == 0x7fffffff ? 0 : best_i;
            mine[2 * C] = 0;
        }
    }
}

}  // namespace

// How many slices a row of V logits is cut into (so callers can size `scratch`).
extern "C" int sb_sample_slices(int V) {
    int c = (V + 8191) / 8192;
    return c < 1 ? 1 : (c > 32 ? 32 : c);
}

// scratch: int32, at least M * (2 * sb_sample_slices(V) + 1) entries, zero before the first use.
extern "C" int sb_sample(int* out, const float* logits, const float* temperature, const uint32_t* seeds,
                         const uint32_t* counters, int M, int V, int* scratch, cudaStream_t stream) {
    SB_REQUIRE(M >= 0 && V > 0, "sample: bad sizes M=%d V=%d", M, V);
    SB_REQUIRE(temperature == nullptr || (seeds != nullptr && counters != nullptr),
               "sample: temperature sampling needs seeds and counters");
    SB_REQUIRE(scratch != nullptr, "sample: scratch is required");
    SB_REQUIRE(M <= 65535 * 32, "sample: too many rows");
    if (M == 0) return 0;
    dim3 grid(M, sb_sample_slices(V));
    sb::launch(sample_kernel, dim3(grid), dim3(512), 0, stream, out, logits, temperature, seeds, counters, V, scratch);
    SB_LAUNCH_CHECK();
}
