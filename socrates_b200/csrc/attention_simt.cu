// Paged causal attention on the CUDA cores, any mix of queries.
//
// Every token of the step is a query of its own: token n of cache row r at position
// p sees the keys of row r at positions lo..p, lo = max(0, p - window + 1) (window 0
// means all keys), read from the row's pages.  The step's own keys are already in the
// pages (the KV-write kernel runs first), so prompt portions and decode tokens need
// no distinction here.  One block serves all G query heads of one KV head for one
// token and one partition of the keys; partitions are merged by the reduce kernel.
//
// Scores, softmax and the weighted sum are float32 with expf; slots outside lo..p are
// never read, so whatever a page's previous owner left there cannot reach the result.
// This is the attention of the true 32-bit path and, in bfloat16, of head sizes the
// tensor-core kernel is not built for.
#include <math.h>

#include "common.cuh"
#include "attention_reduce.cuh"

using namespace sb;

namespace {

constexpr int THREADS = 128;
constexpr int CHUNK = 128;    // keys per pass of the online softmax
constexpr int GMAX = 8;       // query heads per pass

template <typename T>
__global__ void __launch_bounds__(THREADS)
attn_tokens_kernel(T* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                   const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                   const int* __restrict__ block_table, int table_width,
                   const int* __restrict__ token_rows, const int* __restrict__ positions, int Hq,
                   int Hkv, int D, int BS, int window, float scale, int NP) {
    sb::pdl_launch_dependents();     // the next kernel may begin its prologue
    sb::pdl_wait();                  // everything before this kernel is complete and visible
    __shared__ float qs[GMAX][256];
    __shared__ float sc[GMAX][CHUNK];
    __shared__ float s_m[GMAX], s_l[GMAX], s_alpha[GMAX];

    const int kh = blockIdx.x, n = blockIdx.y, part = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = Hq / Hkv;
    const int row = token_rows[n];
    const int pos = positions[n];
    const int hi = pos + 1;
    const int lo = (window > 0 && hi > window) ? hi - window : 0;
    const int first_pg = lo / BS, last_pg = (hi - 1) / BS;
    const int npg = last_pg - first_pg + 1;
    const int ppp = (npg + NP - 1) / NP;
    const int pg_begin = first_pg + part * ppp;
    const int pg_end = min(pg_begin + ppp, last_pg + 1);
    const int k_begin = max(lo, pg_begin * BS);
    const int k_end = min(hi, pg_end * BS);
    const int* table = block_table + (size_t)row * table_width;
    constexpr int VEC = Vec16<T>::N;

    for (int g0 = 0; g0 < G; g0 += GMAX) {
        const int gn = min(GMAX, G - g0);
        const int h0 = kh * G + g0;
        if (k_begin >= k_end) {
            // An empty partition: the reduce kernel skips it by l == 0.
            if (NP > 1 && tid < gn) {
                float* ml = part_ml + (((size_t)n * Hq + h0 + tid) * NP + part) * 2;
                ml[0] = -INFINITY;
                ml[1] = 0.f;
            }
            continue;
        }
        __syncthreads();
        for (int i = tid; i < gn * D; i += THREADS) {
            const int g = i / D, d = i - g * D;
            qs[g][d] = to_float(q[((size_t)n * Hq + h0 + g) * D + d]) * scale;
        }
        if (tid < GMAX) { s_m[tid] = -INFINITY; s_l[tid] = 0.f; s_alpha[tid] = 0.f; }
        float acc[GMAX][2];
#pragma unroll
        for (int g = 0; g < GMAX; ++g) acc[g][0] = acc[g][1] = 0.f;
        __syncthreads();

        for (int c0 = k_begin; c0 < k_end; c0 += CHUNK) {
            const int nvalid = min(CHUNK, k_end - c0);
            // ---- scores: one key per thread
            {
                float dot[GMAX];
#pragma unroll
                for (int g = 0; g < GMAX; ++g) dot[g] = 0.f;
                if (tid < nvalid) {
                    const int key = c0 + tid;
                    const int page = table[key / BS];
                    const T* kp = k_pool + (((size_t)page * Hkv + kh) * BS + (key % BS)) * D;
                    for (int d = 0; d < D; d += VEC) {
                        Vec16<T> kv;
                        kv.load(kp + d);
#pragma unroll
                        for (int e = 0; e < VEC; ++e) {
                            const float kf = kv.get(e);
#pragma unroll
                            for (int g = 0; g < GMAX; ++g)
                                if (g < gn) dot[g] = fmaf(qs[g][d + e], kf, dot[g]);
                        }
                    }
                }
#pragma unroll
                for (int g = 0; g < GMAX; ++g)
                    if (g < gn) sc[g][tid] = tid < nvalid ? dot[g] : -INFINITY;
            }
            __syncthreads();
            // ---- online softmax: one warp per head
            for (int g = warp; g < gn; g += THREADS / 32) {
                float mx = -INFINITY;
                for (int t = lane; t < nvalid; t += 32) mx = fmaxf(mx, sc[g][t]);
                mx = warp_max(mx);
                const float m_old = s_m[g];
                const float m_new = fmaxf(m_old, mx);
                float sum = 0.f;
                for (int t = lane; t < nvalid; t += 32) {
                    const float p = expf(sc[g][t] - m_new);
                    sc[g][t] = p;
                    sum += p;
                }
                sum = warp_sum(sum);
                if (lane == 0) {
                    const float alpha = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
                    s_alpha[g] = alpha;
                    s_l[g] = s_l[g] * alpha + sum;
                    s_m[g] = m_new;
                }
            }
            __syncthreads();
            // ---- weighted sum of values: thread t owns dims t and t + 128
#pragma unroll
            for (int g = 0; g < GMAX; ++g)
                if (g < gn) { acc[g][0] *= s_alpha[g]; acc[g][1] *= s_alpha[g]; }
            const int d0 = tid, d1 = tid + THREADS;
            for (int t = 0; t < nvalid; ++t) {
                const int key = c0 + t;
                const int page = table[key / BS];
                const T* vp = v_pool + (((size_t)page * Hkv + kh) * BS + (key % BS)) * D;
                const float v0 = d0 < D ? to_float(vp[d0]) : 0.f;
                const float v1 = d1 < D ? to_float(vp[d1]) : 0.f;
#pragma unroll
                for (int g = 0; g < GMAX; ++g)
                    if (g < gn) {
                        const float p = sc[g][t];
                        acc[g][0] = fmaf(p, v0, acc[g][0]);
                        acc[g][1] = fmaf(p, v1, acc[g][1]);
                    }
            }
            __syncthreads();
        }
        // ---- write
#pragma unroll
        for (int g = 0; g < GMAX; ++g) {
            if (g >= gn) continue;
            const int h = h0 + g;
            if (NP == 1) {
                const float inv = 1.0f / s_l[g];
                T* o = out + ((size_t)n * Hq + h) * D;
                if (tid < D) o[tid] = from_float<T>(acc[g][0] * inv);
                if (tid + THREADS < D) o[tid + THREADS] = from_float<T>(acc[g][1] * inv);
            } else {
                float* o = part_o + (((size_t)n * Hq + h) * NP + part) * D;
                if (tid < D) o[tid] = acc[g][0];
                if (tid + THREADS < D) o[tid + THREADS] = acc[g][1];
                if (tid == 0) {
                    float* ml = part_ml + (((size_t)n * Hq + h) * NP + part) * 2;
                    ml[0] = s_m[g];
                    ml[1] = s_l[g];
                }
            }
        }
    }
}

template <typename T>
void launch(void* out, float* part_o, float* part_ml, const void* q, const void* k_pool,
            const void* v_pool, const int* block_table, int table_width, const int* token_rows,
            const int* positions, int N, int Hq, int Hkv, int D, int BS, int window, float scale, int NP,
            cudaStream_t stream) {
    dim3 grid(Hkv, N, NP);
    sb::launch(attn_tokens_kernel<T>, dim3(grid), dim3(THREADS), 0, stream, 
        (T*)out, part_o, part_ml, (const T*)q, (const T*)k_pool, (const T*)v_pool, block_table,
        table_width, token_rows, positions, Hq, Hkv, D, BS, window, scale, NP);
    if (NP > 1) {
        dim3 rgrid(Hq, N);
        sb::launch(attn_reduce_kernel<T>, dim3(rgrid), dim3(128), 0, stream, (T*)out, part_o, part_ml, Hq, D, NP);
    }
}

}  // namespace

// part_o: float32 [N, Hq, NP, D]; part_ml: float32 [N, Hq, NP, 2]; both unused when NP == 1.
extern "C" int sb_attention_simt(void* out, float* part_o, float* part_ml, const void* q,
                                 const void* k_pool, const void* v_pool, const int* block_table,
                                 int table_width, const int* token_rows, const int* positions, int N,
                                 int Hq, int Hkv, int D, int page_size, int window, float scale,
                                 int num_partitions, int dtype, cudaStream_t stream) {
    SB_REQUIRE(N >= 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0,
               "attention: %d query heads are no multiple of %d KV heads", Hq, Hkv);
    SB_REQUIRE(D >= 16 && D <= 256 && D % 16 == 0,
               "attention: head_dim %d must be a multiple of 16 between 16 and 256", D);
    SB_REQUIRE(page_size > 0 && table_width > 0, "attention: bad page_size %d or table width %d",
               page_size, table_width);
    SB_REQUIRE(window >= 0, "attention: window %d is negative", window);
    SB_REQUIRE(num_partitions >= 1 && num_partitions <= 65535, "attention: %d partitions", num_partitions);
    SB_REQUIRE(num_partitions == 1 || (part_o != nullptr && part_ml != nullptr),
               "attention: split over %d partitions needs scratch buffers", num_partitions);
    SB_REQUIRE(N <= 65535, "attention: %d tokens exceed one launch", N);
    if (N == 0) return 0;
    if (dtype == SB_F32)
        launch<float>(out, part_o, part_ml, q, k_pool, v_pool, block_table, table_width, token_rows,
                      positions, N, Hq, Hkv, D, page_size, window, scale, num_partitions, stream);
    else if (dtype == SB_BF16)
        launch<__nv_bfloat16>(out, part_o, part_ml, q, k_pool, v_pool, block_table, table_width,
                              token_rows, positions, N, Hq, Hkv, D, page_size, window, scale,
                              num_partitions, stream);
    else
        SB_REQUIRE(false, "attention: unknown dtype %d", dtype);
    SB_LAUNCH_CHECK();
}
