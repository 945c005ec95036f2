// C[M,N] = A[M,K] * W[N,K]^T on the CUDA cores, float32 FMA accumulation.
//
// This is the matrix product of the true 32-bit path (no tensor-core kind, no TF32)
// and the fallback of the bfloat16 path for shapes the tensor-core kernel refuses.
// Any M, N, K; A, W and C each float32 or bfloat16.  With splits > 1 the K range is
// cut into `splits` parts and part z writes float32 partial sums to C + z*M*N.
#include "common.cuh"

using namespace sb;

namespace {

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(TC* __restrict__ C, const TA* __restrict__ A, const TW* __restrict__ W, int M, int N,
                 int K, int k_per_split) {
    sb::pdl_launch_dependents();     // the next kernel may begin its prologue
    sb::pdl_wait();                  // everything before this kernel is complete and visible
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int k_begin = blockIdx.z * k_per_split;
    const int k_end = min(K, k_begin + k_per_split);
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = k_begin; k0 < k_end; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256;
            const int r = idx >> 4, c = idx & 15;
            const int k = k0 + c;
            const int m = m0 + r, n = n0 + r;
            As[c][r] = (m < M && k < k_end) ? to_float(A[(size_t)m * K + k]) : 0.f;
            Ws[c][r] = (n < N && k < k_end) ? to_float(W[(size_t)n * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
    TC* Cz = C + (size_t)blockIdx.z * M * N;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) Cz[(size_t)m * N + n] = from_float<TC>(acc[i][j]);
        }
    }
}

template <typename TA, typename TW, typename TC>
void launch(void* C, const void* A, const void* W, int M, int N, int K, int splits, cudaStream_t stream) {
    const int k_per_split = ((K + splits - 1) / splits + BK - 1) / BK * BK;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, splits);
    sb::launch(gemm_simt_kernel<TA, TW, TC>, dim3(grid), dim3(256), 0, stream, (TC*)C, (const TA*)A, (const TW*)W, M, N, K,
                                                           k_per_split);
}

}  // namespace

extern "C" int sb_gemm_simt(void* C, const void* A, const void* W, int M, int N, int K, int a_dtype,
                            int w_dtype, int c_dtype, int splits, cudaStream_t stream) {
    SB_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_simt: bad sizes M=%d N=%d K=%d", M, N, K);
    SB_REQUIRE(splits >= 1 && splits <= 64, "gemm_simt: splits=%d is outside 1..64", splits);
    SB_REQUIRE(splits == 1 || c_dtype == SB_F32, "gemm_simt: partial sums of a split product are float32");
    SB_REQUIRE((M + BM - 1) / BM <= 65535, "gemm_simt: M=%d is too large", M);
    if (M == 0) return 0;
    const int key = a_dtype * 4 + w_dtype * 2 + c_dtype;
    typedef __nv_bfloat16 bf;
    switch (key) {
        case 0: launch<float, float, float>(C, A, W, M, N, K, splits, stream); break;
        case 1: launch<float, float, bf>(C, A, W, M, N, K, splits, stream); break;
        case 2: launch<float, bf, float>(C, A, W, M, N, K, splits, stream); break;
        case 3: launch<float, bf, bf>(C, A, W, M, N, K, splits, stream); break;
        case 4: launch<bf, float, float>(C, A, W, M, N, K, splits, stream); break;
        case 5: launch<bf, float, bf>(C, A, W, M, N, K, splits, stream); break;
        case 6: launch<bf, bf, float>(C, A, W, M, N, K, splits, stream); break;
        case 7: launch<bf, bf, bf>(C, A, W, M, N, K, splits, stream); break;
        default: SB_REQUIRE(false, "gemm_simt: unknown dtypes %d %d %d", a_dtype, w_dtype, c_dtype);
    }
    SB_LAUNCH_CHECK();
}
