// Memory-bound kernels of the step: embedding gather, residual add + RMSNorm,
// QK-norm + rotation + paged KV write, SiLU*mul.  All arithmetic is float32;
// only loads and stores see the model dtype.
#include "common.cuh"

using namespace sb;

// ----------------------------------------------------------------------------------------
// Embedding gather: residual[n, :] = float(table[ids[n], :]).
// The residual stream is float32 in both dtypes of the engine.
template <typename T>
__global__ void embed_kernel(float* __restrict__ out, const T* __restrict__ table,
                             const int* __restrict__ ids, int d, int V) {
    const int n = blockIdx.x;
    int id = ids[n];
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);   // ids are validated on the host; stay in bounds regardless
    const T* src = table + (size_t)id * d;
    float* dst = out + (size_t)n * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = to_float(src[i]);
}

extern "C" int sb_embed(float* out, const void* table, const int* ids, int N, int d, int V,
                        int dtype, cudaStream_t stream) {
    SB_REQUIRE(N >= 0 && d > 0 && V > 0, "embed: bad sizes N=%d d=%d V=%d", N, d, V);
    if (N == 0) return 0;
    if (dtype == SB_F32)
        embed_kernel<float><<<N, 256, 0, stream>>>(out, (const float*)table, ids, d, V);
    else if (dtype == SB_BF16)
        embed_kernel<__nv_bfloat16><<<N, 256, 0, stream>>>(out, (const __nv_bfloat16*)table, ids, d, V);
    else
        SB_REQUIRE(false, "embed: unknown dtype %d", dtype);
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

extern "C" int sb_add_rmsnorm(float* residual, const float* delta, int S, long long delta_stride,
                              const float* gain, void* out, const int* row_index, int M, int d,
                              float eps, int dtype, cudaStream_t stream) {
    SB_REQUIRE(M >= 0 && d > 0 && S >= 0, "add_rmsnorm: bad sizes M=%d d=%d S=%d", M, d, S);
    SB_REQUIRE(S == 0 || delta != nullptr, "add_rmsnorm: S=%d partial sums but no buffer", S);
    if (M == 0) return 0;
    const size_t smem = (size_t)d * sizeof(float);
    SB_REQUIRE(smem <= 200 * 1024, "add_rmsnorm: width %d does not fit one block's shared memory", d);
    const int write_residual = row_index == nullptr && S > 0;
    const int threads = d >= 2048 ? 512 : 256;
    if (dtype == SB_F32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        add_rmsnorm_kernel<float><<<M, threads, smem, stream>>>(
            residual, delta, S, (size_t)delta_stride, gain, (float*)out, row_index, d, eps, write_residual);
    } else if (dtype == SB_BF16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_rmsnorm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        add_rmsnorm_kernel<__nv_bfloat16><<<M, threads, smem, stream>>>(
            residual, delta, S, (size_t)delta_stride, gain, (__nv_bfloat16*)out, row_index, d, eps, write_residual);
    } else {
        SB_REQUIRE(false, "add_rmsnorm: unknown dtype %d", dtype);
    }
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
template <typename T>
__global__ void qk_norm_rope_kvwrite_kernel(
    const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_pool, T* __restrict__ v_pool,
    const float* __restrict__ q_gain, const float* __restrict__ k_gain,
    const float* __restrict__ inv_freq, int R, const int* __restrict__ positions,
    const int* __restrict__ token_rows, const int* __restrict__ block_table, int table_width,
    int BS, float eps, int Hq, int Hkv, int D, int write_kv) {
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

    const T* src = qkv + ((size_t)n * n_heads + head) * D;
    float* y = buf[warp];
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) {
        const float v = to_float(src[i]);
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

extern "C" int sb_qk_norm_rope_kvwrite(const void* qkv, void* q_out, void* k_pool, void* v_pool,
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
    if (N == 0) return 0;
    dim3 grid(N, (Hq + 2 * Hkv + 3) / 4);
    if (dtype == SB_F32)
        qk_norm_rope_kvwrite_kernel<float><<<grid, 128, 0, stream>>>(
            (const float*)qkv, (float*)q_out, (float*)k_pool, (float*)v_pool, q_gain, k_gain, inv_freq,
            rotary_dim, positions, token_rows, block_table, table_width, page_size, eps, Hq, Hkv, D, write_kv);
    else if (dtype == SB_BF16)
        qk_norm_rope_kvwrite_kernel<__nv_bfloat16><<<grid, 128, 0, stream>>>(
            (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool,
            (__nv_bfloat16*)v_pool, q_gain, k_gain, inv_freq, rotary_dim, positions, token_rows,
            block_table, table_width, page_size, eps, Hq, Hkv, D, write_kv);
    else
        SB_REQUIRE(false, "qk_norm_rope: unknown dtype %d", dtype);
    SB_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// SiLU*mul: out[n, f] = up * gate * sigmoid(gate), gate = in[n, f], up = in[n, F + f].
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ in, size_t total, int F) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t n = i / F;
        const int f = (int)(i - n * F);
        const float g = to_float(in[n * 2 * F + f]);
        const float u = to_float(in[n * 2 * F + F + f]);
        out[i] = from_float<T>(u * (g / (1.0f + expf(-g))));
    }
}

extern "C" int sb_silu_mul(void* out, const void* gate_up, int N, int F, int dtype, cudaStream_t stream) {
    SB_REQUIRE(N >= 0 && F > 0, "silu_mul: bad sizes N=%d F=%d", N, F);
    if (N == 0) return 0;
    const size_t total = (size_t)N * F;
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == SB_F32)
        silu_mul_kernel<float><<<(int)blocks, 256, 0, stream>>>((float*)out, (const float*)gate_up, total, F);
    else if (dtype == SB_BF16)
        silu_mul_kernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>(
            (__nv_bfloat16*)out, (const __nv_bfloat16*)gate_up, total, F);
    else
        SB_REQUIRE(false, "silu_mul: unknown dtype %d", dtype);
    SB_LAUNCH_CHECK();
}
