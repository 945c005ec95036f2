// Memory-bound kernels of the step: embedding gather, residual add + RMSNorm,
// QK-norm + rotation + paged KV write, SiLU*mul.  All arithmetic is float32;
// only loads and stores see the model dtype.
#include "common.cuh"

using namespace sb;

// ----------------------------------------------------------------------------------------
// Embedding gather: residual[n, :] = float(table[ids[n], :]).
// The residual stream is float32 in both dtypes of the engine.
// A negative id -1 - j stands for feedback[j]: a token that an earlier kernel on the stream
// wrote (the previous step's sample), so that a step can be launched before the host has read
// the tokens it continues from.
template <typename T>
__global__ void embed_kernel(float* __restrict__ out, const T* __restrict__ table,
                             const int* __restrict__ ids, int d, int V, const int* __restrict__ feedback) {
    sb::pdl_launch_dependents();     // the next kernel may begin its prologue
    sb::pdl_wait();                  // everything before this kernel is complete and visible
    const int n = blockIdx.x;
    int id = ids[n];
    if (id < 0 && feedback != nullptr) id = feedback[-1 - id];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);   // ids are validated on the host; stay in bounds regardless
    const T* src = table + (size_t)id * d;
    float* dst = out + (size_t)n * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = to_float(src[i]);
}

// d a multiple of 8 (bfloat16) or 4 (float32): 16-byte loads, one thread per vector.
template <typename T>
__global__ void embed_vec_kernel(float* __restrict__ out, const T* __restrict__ table,
                                 const int* __restrict__ ids, int d, int V, const int* __restrict__ feedback) {
    sb::pdl_launch_dependents();     // the next kernel may begin its prologue
    sb::pdl_wait();                  // everything before this kernel is complete and visible
    constexpr int VEC = Vec16<T>::N;
    const int n = blockIdx.x;
    int id = ids[n];
    if (id < 0 && feedback != nullptr) id = feedback[-1 - id];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    const T* src = table + (size_t)id * d;
    float* dst = out + (size_t)n * d;
    for (int i = threadIdx.x * VEC; i < d; i += blockDim.x * VEC) {
        Vec16<T> v;
        v.load(src + i);
#pragma unroll
        for (int e = 0; e < VEC; e += 4)
            *reinterpret_cast<float4*>(dst + i + e) = make_float4(v.get(e), v.get(e + 1), v.get(e + 2), v.get(e + 3));
    }
}

// feedback: null, or int32 tokens that ids -1 - j refer to (see above).
extern "C" int sb_embed(float* out, const void* table, const int* ids, int N, int d, int V,
                        int dtype, const int* feedback, cudaStream_t stream) {
    SB_REQUIRE(N >= 0 && d > 0 && V > 0, "embed: bad sizes N=%d d=%d V=%d", N, d, V);
    if (N == 0) return 0;
    const bool aligned = (reinterpret_cast<uintptr_t>(table) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
    if (dtype == SB_F32) {
        if (aligned && d % 4 == 0) sb::launch(embed_vec_kernel<float>, dim3(N), dim3(256), 0, stream, out, (const float*)table, ids, d, V, feedback);
        else sb::launch(embed_kernel<float>, dim3(N), dim3(256), 0, stream, out, (const float*)table, ids, d, V, feedback);
    } else if (dtype == SB_BF16) {
        if (aligned && d % 8 == 0)
            sb::launch(embed_vec_kernel<__nv_bfloat16>, dim3(N), dim3(256), 0, stream, out, (const __nv_bfloat16*)table, ids, d, V, feedback);
        else
            sb::launch(embed_kernel<__nv_bfloat16>, dim3(N), dim3(256), 0, stream, out, (const __nv_bfloat16*)table, ids, d, V, feedback);
    } else {
        SB_REQUIRE(false, "embed: unknown dtype %d", dtype);
    }
    SB_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// Residual add + RMSNorm.
//   v = residual[r] + sum_{s<S} delta[s][r]      (fixed order: s = 0, 1, ...)
//   residual[r] = v                               (when write_residual)
//   out[m] = v / sqrt(mean(v^2) + eps) * gain     (in T)
// `row_index` (may be null) selects rows r = row_index[m]; then nothing is written
// back to the residual (the rows may repeat).  The S partial sums are the split-K
// outputs of the GEMM before it, so their reduction costs no pass of its own.
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const float* __restrict__ delta,
                                   int S, size_t delta_stride, const float* __restrict__ gain,
                                   T* __restrict__ out, const int* __restrict__ row_index, int d,
                                   float eps, int write_residual) {
    sb::pdl_launch_dependents();     // the next kernel may begin its prologue
    sb::pdl_wait();                  // everything before this kernel is complete and visible
    extern __shared__ float row[];          // d floats
    __shared__ float scratch[33];
    const int m = blockIdx.x;
    const int r = row_index ? row_index[m] : m;
    float* res = residual + (size_t)r * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float v = res[i];
        for (int s = 0; s < S; ++s) v += delta[s * delta_stride + (size_t)r * d + i];
        row[i] = v;
        if (write_residual) res[i] = v;
        ss += v * v;
    }
    const float total = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(total / (float)d + eps);
    T* o = out + (size_t)m * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = from_float<T>(row[i] * rinv * gain[i]);
}

// The same with 16-byte accesses (d a multiple of 4, 16-byte aligned rows): each thread
// owns whole float4 columns, the S partial sums of a column are loaded back to back
// (independent loads) and added in the fixed order s = 0, 1, ...
// DEPTH partial sums' loads are in flight at once: 16 for the few rows of a decode step (one round
// trip for the 13 or 14 parts of its narrow projections; about a hundred registers, so at most
// 640 threads a block), 2 for many rows, where the rows themselves keep memory busy.
template <typename T, int DEPTH>
__global__ void __launch_bounds__(DEPTH > 8 ? 640 : 768) add_rmsnorm_vec_kernel(float* __restrict__ residual, const float* __restrict__ delta,
                                       int S, size_t delta_stride, const float* __restrict__ gain,
                                       T* __restrict__ out, const int* __restrict__ row_index, int d,
                                       float eps, int write_residual) {
    sb::pdl_launch_dependents();     // the next kernel may begin its prologue
    extern __shared__ float row[];          // d floats
    __shared__ float scratch[33];
    const int m = blockIdx.x;
    const int d4 = d / 4;
    // The gain is a weight (nobody writes it): a thread's first column of it is fetched before
    // the wait on the preceding kernel instead of after the reduction.
    const float4* gain4 = reinterpret_cast<const float4*>(gain);
    const float4 g_first = threadIdx.x < d4 ? __ldg(gain4 + threadIdx.x) : make_float4(0.f, 0.f, 0.f, 0.f);
    sb::pdl_wait();                  // everything before this kernel is complete and visible
    const int r = row_index ? row_index[m] : m;
    float4* res4 = reinterpret_cast<float4*>(residual + (size_t)r * d);
    const float4* del4 = reinterpret_cast<const float4*>(delta + (size_t)r * d);
    const size_t stride4 = delta_stride / 4;
    float4* row4 = reinterpret_cast<float4*>(row);
    float ss = 0.f;
    if constexpr (DEPTH <= 2) {
        // Many rows: a thread owns several columns.  The residual and the first partial sum of up
        // to three of them are loaded before any is used, so that a row costs one round trip to
        // memory, not one per column; the sums keep the order s = 0, 1, ...
        constexpr int CM = 3;
        for (int i0 = threadIdx.x; i0 < d4; i0 += CM * blockDim.x) {
            float4 v[CM], p0[CM];
#pragma unroll
            for (int c = 0; c < CM; ++c) {
                const int i = i0 + c * blockDim.x;
                if (i < d4) {
                    v[c] = res4[i];
                    if (S > 0) p0[c] = __ldg(del4 + i);
                }
            }
#pragma unroll
            for (int c = 0; c < CM; ++c) {
                const int i = i0 + c * blockDim.x;
                if (i < d4) {
                    float4 u = v[c];
                    if (S > 0) { u.x += p0[c].x; u.y += p0[c].y; u.z += p0[c].z; u.w += p0[c].w; }
                    for (int s = 1; s < S; ++s) {
                        const float4 p = __ldg(del4 + (size_t)s * stride4 + i);
                        u.x += p.x; u.y += p.y; u.z += p.z; u.w += p.w;
                    }
                    row4[i] = u;
                    if (write_residual) res4[i] = u;
                    ss += u.x * u.x + u.y * u.y + u.z * u.z + u.w * u.w;
                }
            }
        }
    } else
    for (int i = threadIdx.x; i < d4; i += blockDim.x) {
        float4 v = res4[i];
        // DEPTH loads in flight, added in the order s = 0, 1, ...
        for (int s0 = 0; s0 < S; s0 += DEPTH) {
            float4 p[DEPTH];
#pragma unroll
            for (int j = 0; j < DEPTH; ++j)
                if (s0 + j < S) p[j] = __ldg(del4 + (size_t)(s0 + j) * stride4 + i);
#pragma unroll
            for (int j = 0; j < DEPTH; ++j)
                if (s0 + j < S) { v.x += p[j].x; v.y += p[j].y; v.z += p[j].z; v.w += p[j].w; }
        }
        row4[i] = v;
        if (write_residual) res4[i] = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    const float total = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(total / (float)d + eps);
    T* o = out + (size_t)m * d;
    for (int i = threadIdx.x; i < d4; i += blockDim.x) {
        const float4 v = row4[i], g = i == (int)threadIdx.x ? g_first : __ldg(gain4 + i);
        const float a = v.x * rinv * g.x, b = v.y * rinv * g.y, c = v.z * rinv * g.z, e = v.w * rinv * g.w;
        if constexpr (sizeof(T) == 2) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, e);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&lo);
            pk.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(o + 4 * i) = pk;
        } else {
            *reinterpret_cast<float4*>(o + 4 * i) = make_float4(a, b, c, e);
        }
    }
}

// the output pointer type of a norm kernel instantiation (its first template argument)
template <typename T, int DEPTH = 0> T* sb_out_type();

extern "C" int sb_add_rmsnorm(float* residual, const float* delta, int S, long long delta_stride,
                              const float* gain, void* out, const int* row_index, int M, int d,
                              float eps, int dtype, cudaStream_t stream) {
    SB_REQUIRE(M >= 0 && d > 0 && S >= 0, "add_rmsnorm: bad sizes M=%d d=%d S=%d", M, d, S);
    SB_REQUIRE(S == 0 || delta != nullptr, "add_rmsnorm: S=%d partial sums but no buffer", S);
    if (M == 0) return 0;
    const size_t smem = (size_t)d * sizeof(float);
    SB_REQUIRE(smem <= 200 * 1024, "add_rmsnorm: width %d does not fit one block's shared memory", d);
    const int write_residual = row_index == nullptr && S > 0;
    const bool vec = d % 4 == 0 && delta_stride % 4 == 0 &&
                     ((reinterpret_cast<uintptr_t>(residual) | reinterpret_cast<uintptr_t>(delta) |
                       reinterpret_cast<uintptr_t>(gain) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    // vector kernel: one float4 column per thread where the row allows it (few rows are the
    // decode regime, where the S partial sums of a column should all be in flight at once)
    int threads = d >= 2048 ? 512 : 256;
    if (vec) {
        threads = ((d / 4 + 31) / 32) * 32;
        if (threads > (M <= 64 ? 640 : 768)) threads = M <= 64 ? 640 : 768;
        if (M > 512 && threads > 256) threads = 256;
    }
#define SB_NORM_LAUNCH(KERNEL, ...)                                                                      \
    do {                                                                                                  \
        if (smem > 48 * 1024)                                                                             \
            cudaFuncSetAttribute(KERNEL<__VA_ARGS__>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
        sb::launch(KERNEL<__VA_ARGS__>, dim3(M), dim3(threads), smem, stream, residual, delta, S, (size_t)delta_stride, gain, \
                   (decltype(sb_out_type<__VA_ARGS__>()))out, row_index, d, eps, write_residual);        \
    } while (0)
    if (dtype == SB_F32) {
        if (vec && M <= 64) SB_NORM_LAUNCH(add_rmsnorm_vec_kernel, float, 16);
        else if (vec) SB_NORM_LAUNCH(add_rmsnorm_vec_kernel, float, 2);
        else SB_NORM_LAUNCH(add_rmsnorm_kernel, float);
    } else if (dtype == SB_BF16) {
        if (vec && M <= 64) SB_NORM_LAUNCH(add_rmsnorm_vec_kernel, __nv_bfloat16, 16);
        else if (vec) SB_NORM_LAUNCH(add_rmsnorm_vec_kernel, __nv_bfloat16, 2);
        else SB_NORM_LAUNCH(add_rmsnorm_kernel, __nv_bfloat16);
    } else {
        SB_REQUIRE(false, "add_rmsnorm: unknown dtype %d", dtype);
    }
#undef SB_NORM_LAUNCH
    SB_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// Per-head QK-RMSNorm, rotation and paged KV write, one warp per (token, head).
//   heads 0..Hq-1        : q  -> norm(q_gain) -> rotate -> q_out[n, h, :]
//   heads Hq..Hq+Hkv-1   : k  -> norm(k_gain) -> rotate -> k_pool[page, kh, off, :]
//   heads Hq+Hkv..       : v  ->                           v_pool[page, kh, off, :]
// page = block_table[row, pos / BS], off = pos % BS.  A null gain means no norm.
// Rotation: angle_j = float(pos) * inv_freq[j], j < R/2; dim j pairs with j + R/2;
// dims >= R pass through.  cosf/sinf are the accurate library functions.
// The input is either qkv in the model dtype, or (parts != null) S float32 partial sums
// of a split-K product, added here in the order s = 0, 1, ...
template <typename T>
__global__ void qk_norm_rope_kvwrite_kernel(
    const T* __restrict__ qkv, const float* __restrict__ parts, int S, size_t part_stride,
    T* __restrict__ q_out, T* __restrict__ k_pool, T* __restrict__ v_pool,
    const float* __restrict__ q_gain, const float* __restrict__ k_gain,
    const float* __restrict__ inv_freq, int R, const int* __restrict__ positions,
    const int* __restrict__ token_rows, const int* __restrict__ block_table, int table_width,
    int BS, float eps, int Hq, int Hkv, int D, int write_kv) {
    sb::pdl_launch_dependents();     // the next kernel may begin its prologue
    sb::pdl_wait();                  // everything before this kernel is complete and visible
    __shared__ float buf[4][256];
    const int n = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * 4 + warp;
    const int n_heads = Hq + 2 * Hkv;
    if (head >= n_heads) return;
    const bool is_q = head < Hq;
    const bool is_k = !is_q && head < Hq + Hkv;
    const bool is_v = !is_q && !is_k;
    if (!is_q && !write_kv) return;

    const size_t base = ((size_t)n * n_heads + head) * D;
    float* y = buf[warp];
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) {
        float v;
        if (parts != nullptr) {
            v = 0.f;
            for (int s = 0; s < S; ++s) v += parts[s * part_stride + base + i];
        } else {
            v = to_float(qkv[base + i]);
        }
        y[i] = v;
        ss += v * v;
    }
    const int pos = positions[n];
    const float* gain = is_q ? q_gain : (is_k ? k_gain : nullptr);
    if (gain != nullptr) {
        ss = warp_sum(ss);
        const float rinv = 1.0f / sqrtf(ss / (float)D + eps);
        for (int i = lane; i < D; i += 32) y[i] = y[i] * rinv * gain[i];
    }
    __syncwarp();

    T* dst;
    if (is_q) {
        dst = q_out + ((size_t)n * Hq + head) * D;
    } else {
        const int kh = is_k ? head - Hq : head - Hq - Hkv;
        const int row = token_rows[n];
        const int page = block_table[(size_t)row * table_width + pos / BS];
        T* pool = is_k ? k_pool : v_pool;
        dst = pool + (((size_t)page * Hkv + kh) * BS + (pos % BS)) * D;
    }
    const int half = R >> 1;
    for (int i = lane; i < D; i += 32) {
        float o = y[i];
        if (!is_v && i < R) {
            const int j = i < half ? i : i - half;
            const float ang = (float)pos * inv_freq[j];
            const float c = cosf(ang), s = sinf(ang);
            o = i < half ? y[i] * c - y[i + half] * s : y[i] * c + y[i - half] * s;
        }
        dst[i] = from_float<T>(o);
    }
}

// VPL consecutive elements of T as one aligned vector.
template <typename T, int VPL> struct alignas(sizeof(T) * VPL) Pack { T v[VPL]; };

// The same for the few tokens of a decode step and head_dim = 32 * VPL with all dims rotating
// (R == D) or none (R == 0): lane l owns elements l*VPL .. l*VPL+VPL-1, loads and stores them as one vector, and
// finds its rotation partner (dim +- D/2) in lane l ^ 16.  A block serves `heads_per_block`
// heads of one token; its first D/2 threads compute the token's cosines and sines once
// into shared memory, so the trigonometry is not repeated for every head.
template <typename T, int VPL>
__global__ void qk_norm_rope_kvwrite_fast_kernel(
    const T* __restrict__ qkv, const float* __restrict__ parts, int S, size_t part_stride,
    T* __restrict__ q_out, T* __restrict__ k_pool, T* __restrict__ v_pool,
    const float* __restrict__ q_gain, const float* __restrict__ k_gain,
    const float* __restrict__ inv_freq, int R, const int* __restrict__ positions,
    const int* __restrict__ token_rows, const int* __restrict__ block_table, int table_width,
    int BS, float eps, int Hq, int Hkv, int write_kv, int heads_per_block) {
    sb::pdl_launch_dependents();     // the next kernel may begin its prologue
    constexpr int D = 32 * VPL;
    __shared__ float cs[D / 2], sn[D / 2];
    const int n = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_heads = Hq + 2 * Hkv;
    const int pos = positions[n];
    if (R == D) {
        for (int j = threadIdx.x; j < D / 2; j += blockDim.x) {
            const float ang = (float)pos * inv_freq[j];
            cs[j] = cosf(ang);
            sn[j] = sinf(ang);
        }
    }
    // positions, rows and the block table are older than the preceding kernel (a host copy),
    // inv_freq and the gains are weights: the trigonometry above, the page of this token's key
    // and value, and this lane's gains are all there before that kernel has finished.
    // (in the few blocks of a decode step every round trip after the wait counts; prompt portions
    // go through qk_norm_rope_kvwrite_rows_kernel, where the rows themselves hide the latency)
    size_t kv_slot = 0;
    float gq[VPL], gk[VPL];
    if (write_kv) {
        const int page = block_table[(size_t)token_rows[n] * table_width + pos / BS];
        kv_slot = ((size_t)page * Hkv * BS + (pos % BS)) * D;            // + kh * BS * D per KV head
    }
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
        gq[i] = q_gain != nullptr ? q_gain[lane * VPL + i] : 1.f;
        gk[i] = k_gain != nullptr ? k_gain[lane * VPL + i] : 1.f;
    }
    sb::pdl_wait();                  // everything before this kernel is complete and visible
    __syncthreads();
    const int head_end = min(n_heads, (int)(blockIdx.y + 1) * heads_per_block);
    const int nwarps = blockDim.x >> 5;
    constexpr int U = 1;             // heads whose loads a warp has in flight at once (4 was measured slower)
    for (int head0 = blockIdx.y * heads_per_block + warp; head0 < head_end; head0 += U * nwarps) {
        float y[U][VPL];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int head = head0 + u * nwarps;
            if (head >= head_end || (head >= Hq && !write_kv)) continue;
            const size_t base = ((size_t)n * n_heads + head) * D + lane * VPL;
            if (parts != nullptr) {
#pragma unroll
                for (int i = 0; i < VPL; ++i) y[u][i] = 0.f;
                // eight partial sums' loads in flight at a time; added in the order s = 0, 1, ...
                for (int s0 = 0; s0 < S; s0 += 8) {
                    Pack<float, VPL> p[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (s0 + j < S)
                            p[j] = *reinterpret_cast<const Pack<float, VPL>*>(parts + (s0 + j) * part_stride + base);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (s0 + j < S) {
#pragma unroll
                            for (int i = 0; i < VPL; ++i) y[u][i] += p[j].v[i];
                        }
                }
            } else {
                const Pack<T, VPL> p = *reinterpret_cast<const Pack<T, VPL>*>(qkv + base);
#pragma unroll
                for (int i = 0; i < VPL; ++i) y[u][i] = to_float(p.v[i]);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int head = head0 + u * nwarps;
            if (head >= head_end) continue;
            const bool is_q = head < Hq;
            const bool is_k = !is_q && head < Hq + Hkv;
            const bool is_v = !is_q && !is_k;
            if (!is_q && !write_kv) continue;
            const float* gain = is_q ? q_gain : (is_k ? k_gain : nullptr);
            if (gain != nullptr) {
                float ss = 0.f;
#pragma unroll
                for (int i = 0; i < VPL; ++i) ss += y[u][i] * y[u][i];
                ss = warp_sum(ss);
                const float rinv = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
                for (int i = 0; i < VPL; ++i)
                    y[u][i] = y[u][i] * rinv * (is_q ? gq[i] : gk[i]);
            }
            Pack<T, VPL> o;
            if (!is_v && R == D) {
#pragma unroll
                for (int i = 0; i < VPL; ++i) {
                    const float partner = __shfl_xor_sync(0xffffffffu, y[u][i], 16);
                    const float c = cs[(lane & 15) * VPL + i], s = sn[(lane & 15) * VPL + i];
                    o.v[i] = from_float<T>(lane < 16 ? y[u][i] * c - partner * s : y[u][i] * c + partner * s);
                }
            } else {
#pragma unroll
                for (int i = 0; i < VPL; ++i) o.v[i] = from_float<T>(y[u][i]);
            }
            T* dst;
            if (is_q) {
                dst = q_out + ((size_t)n * Hq + head) * D;
            } else {
                const int kh = is_k ? head - Hq : head - Hq - Hkv;
                T* pool = is_k ? k_pool : v_pool;
                dst = pool + kv_slot + (size_t)kh * BS * D;
            }
            *reinterpret_cast<Pack<T, VPL>*>(dst + lane * VPL) = o;
        }
    }
}

// The same for many tokens (prompt portions), where the kernel is bound by its instruction
// count, not by latency: half a warp per head (lane l of the half owns VPL = D/16 consecutive
// elements, its rotation partner is lane l ^ 8), so a warp serves two heads with the
// instructions of one.  Every shuffle is executed by all lanes whatever their heads are (the
// two halves may hold heads of different kinds); loads and stores are predicated instead.
template <typename T, int VPL>
__global__ void qk_norm_rope_kvwrite_rows_kernel(
    const T* __restrict__ qkv, const float* __restrict__ parts, int S, size_t part_stride,
    T* __restrict__ q_out, T* __restrict__ k_pool, T* __restrict__ v_pool,
    const float* __restrict__ q_gain, const float* __restrict__ k_gain,
    const float* __restrict__ inv_freq, int R, const int* __restrict__ positions,
    const int* __restrict__ token_rows, const int* __restrict__ block_table, int table_width,
    int BS, float eps, int Hq, int Hkv, int write_kv, int heads_per_block) {
    sb::pdl_launch_dependents();     // the next kernel may begin its prologue
    constexpr int D = 16 * VPL;
    __shared__ float cs[D / 2], sn[D / 2];
    const int n = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane >> 4, l = lane & 15;           // which of the warp's two heads, lane within it
    const int n_heads = Hq + 2 * Hkv;
    const int pos = positions[n];
    if (R == D) {
        for (int j = threadIdx.x; j < D / 2; j += blockDim.x) {
            const float ang = (float)pos * inv_freq[j];
            cs[j] = cosf(ang);
            sn[j] = sinf(ang);
        }
    }
    sb::pdl_wait();                  // everything before this kernel is complete and visible
    __syncthreads();
    size_t kv_slot = 0;
    if (write_kv) {
        const int page = block_table[(size_t)token_rows[n] * table_width + pos / BS];
        kv_slot = ((size_t)page * Hkv * BS + (pos % BS)) * D;            // + kh * BS * D per KV head
    }
    const int head_end = min(n_heads, (int)(blockIdx.y + 1) * heads_per_block);
    const int nwarps = blockDim.x >> 5;
    for (int head0 = blockIdx.y * heads_per_block + 2 * warp; head0 < head_end; head0 += 2 * nwarps) {
        const int head = head0 + sub;
        const bool is_q = head < Hq;
        const bool is_k = !is_q && head < Hq + Hkv;
        const bool is_v = !is_q && !is_k;
        const bool live = head < head_end && (is_q || write_kv);
        float y[VPL];
#pragma unroll
        for (int i = 0; i < VPL; ++i) y[i] = 0.f;
        if (live) {
            const size_t base = ((size_t)n * n_heads + head) * D + l * VPL;
            if (parts != nullptr) {
                for (int s = 0; s < S; ++s) {               // added in the order s = 0, 1, ...
                    const Pack<float, VPL> p = *reinterpret_cast<const Pack<float, VPL>*>(parts + s * part_stride + base);
#pragma unroll
                    for (int i = 0; i < VPL; ++i) y[i] += p.v[i];
                }
            } else {
                const Pack<T, VPL> p = *reinterpret_cast<const Pack<T, VPL>*>(qkv + base);
#pragma unroll
                for (int i = 0; i < VPL; ++i) y[i] = to_float(p.v[i]);
            }
        }
        const float* gain = is_q ? q_gain : (is_k ? k_gain : nullptr);
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) ss += y[i] * y[i];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);      // over the head's 16 lanes
        if (live && gain != nullptr) {
            const float rinv = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
            for (int i = 0; i < VPL; ++i) y[i] = y[i] * rinv * gain[l * VPL + i];
        }
        Pack<T, VPL> o;
        const bool rotate = !is_v && R == D;
#pragma unroll
        for (int i = 0; i < VPL; ++i) {
            const float partner = __shfl_xor_sync(0xffffffffu, y[i], 8);
            const float c = cs[(l & 7) * VPL + i], s = sn[(l & 7) * VPL + i];
            const float r = l < 8 ? y[i] * c - partner * s : y[i] * c + partner * s;
            o.v[i] = from_float<T>(rotate ? r : y[i]);
        }
        if (!live) continue;
        T* dst;
        if (is_q) {
            dst = q_out + ((size_t)n * Hq + head) * D;
        } else {
            const int kh = is_k ? head - Hq : head - Hq - Hkv;
            dst = (is_k ? k_pool : v_pool) + kv_slot + (size_t)kh * BS * D;
        }
        *reinterpret_cast<Pack<T, VPL>*>(dst + l * VPL) = o;
    }
}

template <typename T>
static void qk_launch(const void* qkv, const float* parts, int S, size_t part_stride, void* q_out, void* k_pool,
                      void* v_pool, const float* q_gain, const float* k_gain, const float* inv_freq,
                      int rotary_dim, const int* positions, const int* token_rows, const int* block_table,
                      int table_width, int page_size, float eps, int Hq, int Hkv, int D, int N, int write_kv,
                      cudaStream_t stream) {
    const bool fast = (rotary_dim == D || rotary_dim == 0) && (D == 64 || D == 128 || D == 256);
    const int n_heads = Hq + 2 * Hkv;
    // Heads per block: 4 (a head per warp) while that still fills the GPU, more for long batches.
    int hpb = 4;
    if (fast) {
        const long long blocks_wanted = 148LL * 8;
        hpb = (int)(((long long)N * n_heads + blocks_wanted - 1) / blocks_wanted);
        hpb = ((hpb + 3) / 4) * 4;
        if (hpb < 4) hpb = 4;
        if (hpb > n_heads) hpb = ((n_heads + 3) / 4) * 4;
    }
    dim3 grid(N, (n_heads + hpb - 1) / hpb);
#define SB_QK_ARGS (const T*)qkv, parts, S, part_stride, (T*)q_out, (T*)k_pool, (T*)v_pool, q_gain, k_gain, \
                   inv_freq, rotary_dim, positions, token_rows, block_table, table_width, page_size, eps, Hq, Hkv
    // (Four heads' loads in flight per warp, U = 4, were measured slower for prompt portions:
    // 35.5 against 29.0 us for 2,048 tokens of the 4B shape.)
    // Many tokens (hpb > 4): the kernel with half a warp per head (a prompt of 2,048 tokens through the 36
    // layers of the 4B shape: 20.5 -> 19.9 ms).
#define SB_QK_FAST(VPL_) \
    if (hpb > 4) sb::launch(qk_norm_rope_kvwrite_rows_kernel<T, 2 * VPL_>, dim3(grid), dim3(128), 0, stream, SB_QK_ARGS, write_kv, hpb); \
    else sb::launch(qk_norm_rope_kvwrite_fast_kernel<T, VPL_>, dim3(grid), dim3(128), 0, stream, SB_QK_ARGS, write_kv, hpb);
    if (fast && D == 64) { SB_QK_FAST(2) }
    else if (fast && D == 128) { SB_QK_FAST(4) }
    else if (fast) { SB_QK_FAST(8) }
#undef SB_QK_FAST
    else sb::launch(qk_norm_rope_kvwrite_kernel<T>, dim3(grid), dim3(128), 0, stream, SB_QK_ARGS, D, write_kv);
#undef SB_QK_ARGS
}

// qkv: [N, (Hq+2Hkv)*D] in the model dtype, or null when `parts` (float32
// [S, N, (Hq+2Hkv)*D], `part_stride` floats apart) holds split-K partial sums instead.
extern "C" int sb_qk_norm_rope_kvwrite(const void* qkv, const float* parts, int S, long long part_stride,
                                       void* q_out, void* k_pool, void* v_pool,
                                       const float* q_gain, const float* k_gain,
                                       const float* inv_freq, int rotary_dim, const int* positions,
                                       const int* token_rows, const int* block_table, int table_width,
                                       int page_size, float eps, int Hq, int Hkv, int D, int N,
                                       int write_kv, int dtype, cudaStream_t stream) {
    SB_REQUIRE(N >= 0 && Hq > 0 && Hkv > 0, "qk_norm_rope: bad sizes N=%d Hq=%d Hkv=%d", N, Hq, Hkv);
    SB_REQUIRE(D > 0 && D <= 256, "qk_norm_rope: head_dim %d is outside 1..256", D);
    SB_REQUIRE(rotary_dim >= 0 && rotary_dim <= D && rotary_dim % 2 == 0,
               "qk_norm_rope: rotary_dim %d must be even and at most head_dim %d", rotary_dim, D);
    SB_REQUIRE(page_size > 0 && table_width > 0, "qk_norm_rope: bad page_size %d or table width %d",
               page_size, table_width);
    SB_REQUIRE((qkv != nullptr) != (parts != nullptr), "qk_norm_rope: give qkv or partial sums, not both");
    SB_REQUIRE(parts == nullptr || S >= 1, "qk_norm_rope: %d partial sums", S);
    if (N == 0) return 0;
    if (dtype == SB_F32)
        qk_launch<float>(qkv, parts, S, (size_t)part_stride, q_out, k_pool, v_pool, q_gain, k_gain, inv_freq,
                         rotary_dim, positions, token_rows, block_table, table_width, page_size, eps, Hq, Hkv, D, N,
                         write_kv, stream);
    else if (dtype == SB_BF16)
        qk_launch<__nv_bfloat16>(qkv, parts, S, (size_t)part_stride, q_out, k_pool, v_pool, q_gain, k_gain,
                                 inv_freq, rotary_dim, positions, token_rows, block_table, table_width, page_size,
                                 eps, Hq, Hkv, D, N, write_kv, stream);
    else
        SB_REQUIRE(false, "qk_norm_rope: unknown dtype %d", dtype);
    SB_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// SiLU*mul: out[n, f] = up * gate * sigmoid(gate).  Two layouts of the input row of 2F:
// concatenated (gate = in[n, f], up = in[n, F + f]) or interleaved (gate = in[n, 2f],
// up = in[n, 2f + 1]; the layout of a product with interleaved gate/up weight rows).
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ in, size_t total, int F,
                                int interleaved) {
    sb::pdl_launch_dependents();     // the next kernel may begin its prologue
    sb::pdl_wait();                  // everything before this kernel is complete and visible
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / F;
        const int f = (int)(i - n * F);
        const float g = to_float(in[n * 2 * F + (interleaved ? 2 * f : f)]);
        const float u = to_float(in[n * 2 * F + (interleaved ? 2 * f + 1 : F + f)]);
        out[i] = from_float<T>(u * (g / (1.0f + expf(-g))));
    }
}

// F a multiple of the 16-byte vector width: one vector of gate and one of up per thread.
template <typename T>
__global__ void silu_mul_vec_kernel(T* __restrict__ out, const T* __restrict__ in, size_t total_vec, int F,
                                    int interleaved) {
    sb::pdl_launch_dependents();     // the next kernel may begin its prologue
    sb::pdl_wait();                  // everything before this kernel is complete and visible
    constexpr int VEC = Vec16<T>::N;
    const int fv = F / VEC;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_vec;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / fv;
        const int f = (int)(i - n * fv) * VEC;
        Vec16<T> g, u;
        float r[VEC];
        if (interleaved) {          // two consecutive vectors hold VEC (gate, up) pairs
            g.load(in + n * 2 * F + 2 * f);
            u.load(in + n * 2 * F + 2 * f + VEC);
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                const float gv = e < VEC / 2 ? g.get(2 * e) : u.get(2 * e - VEC);
                const float uv = e < VEC / 2 ? g.get(2 * e + 1) : u.get(2 * e + 1 - VEC);
                r[e] = uv * (gv / (1.0f + expf(-gv)));
            }
        } else {
            g.load(in + n * 2 * F + f);
            u.load(in + n * 2 * F + F + f);
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                const float gv = g.get(e);
                r[e] = u.get(e) * (gv / (1.0f + expf(-gv)));
            }
        }
        T* o = out + n * F + f;
        if constexpr (sizeof(T) == 2) {
            uint32_t pk[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                __nv_bfloat162 v = __floats2bfloat162_rn(r[2 * e], r[2 * e + 1]);
                pk[e] = *reinterpret_cast<uint32_t*>(&v);
            }
            *reinterpret_cast<uint4*>(o) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        } else {
            *reinterpret_cast<float4*>(o) = make_float4(r[0], r[1], r[2], r[3]);
        }
    }
}

extern "C" int sb_silu_mul(void* out, const void* gate_up, int N, int F, int interleaved, int dtype,
                           cudaStream_t stream) {
    SB_REQUIRE(N >= 0 && F > 0, "silu_mul: bad sizes N=%d F=%d", N, F);
    if (N == 0) return 0;
    const size_t total = (size_t)N * F;
    const bool aligned = ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(gate_up)) & 15) == 0;
    const int vec = dtype == SB_F32 ? 4 : 8;
    if (aligned && F % vec == 0) {
        const size_t total_vec = total / vec;
        size_t blocks = (total_vec + 255) / 256;
        if (blocks > 148 * 32) blocks = 148 * 32;
        if (dtype == SB_F32)
            sb::launch(silu_mul_vec_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, (float*)out, (const float*)gate_up, total_vec, F, interleaved);
        else if (dtype == SB_BF16)
            sb::launch(silu_mul_vec_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, stream, 
                (__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up, total_vec, F, interleaved);
        else
            SB_REQUIRE(false, "silu_mul: unknown dtype %d", dtype);
        SB_LAUNCH_CHECK();
    }
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == SB_F32)
        sb::launch(silu_mul_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, (float*)out, (const float*)gate_up, total, F, interleaved);
    else if (dtype == SB_BF16)
        sb::launch(silu_mul_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(256), 0, stream, 
            (__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up, total, F, interleaved);
    else
        SB_REQUIRE(false, "silu_mul: unknown dtype %d", dtype);
    SB_LAUNCH_CHECK();
}
