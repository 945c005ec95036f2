// C[M,N] = A[M,K] * W[N,K]^T in bfloat16 on the 5th-generation tensor cores:
// tcgen05.mma with the accumulator in tensor memory, operands brought to shared
// memory by TMA (128-byte swizzle, K-major), a ring of stages between one producer
// thread and one MMA thread, and a tcgen05.ld epilogue by four warps.
//
// The kernel of this file computes one tile per block and serves two regimes:
//   * few rows (decode, M <= 64): operands are swapped so that 128 rows of the WEIGHT
//     matrix fill the lanes and the batch is the N operand (BN = 16, 32 or 64).  The
//     kernel is then a weight stream at HBM rate; K is cut into `splits` parts so that
//     narrow matrices still cover every SM, and part z writes float32 partial sums to
//     C + z*M*N, which the consuming kernel adds up in a fixed order;
//   * many rows with a K split or a narrow N: the activations fill the 128 accumulator
//     lanes and the weights are the N operand (tile 128 x BN).
// Many rows without a split go to the persistent kernels of gemm_tcgen05_rows.cu.
//
// No multicast: every block loads its own tiles.  Every wait on
// an mbarrier is bounded; if one gives up, the block records a code in *status, waits
// (again bounded) for its own copies in flight, frees its tensor memory and returns.
#include <cuda.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tma_maps.cuh"

namespace sb {
namespace {
constexpr int kMapBoxCols = 64;     // 128 bytes of bfloat16: one swizzle row
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

struct MapKey {
    const void* ptr;
    int rows, cols, box_rows;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = reinterpret_cast<size_t>(k.ptr);
        h ^= (size_t)k.rows * 0x9E3779B97F4A7C15ull + (size_t)k.cols * 0xC2B2AE3D27D4EB4Full + k.box_rows;
        return h;
    }
};

// Tensor map of a row-major bfloat16 matrix [rows, cols] with boxes of {64 cols, box_rows}
// and 128-byte swizzle.  Maps are pure functions of their arguments, so they are cached.
}  // namespace

bool get_map(CUtensorMap* out, const void* ptr, int rows, int cols, int box_rows) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    MapKey key{ptr, rows, cols, box_rows};
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = cache.find(key);
        if (it != cache.end()) { *out = it->second; return true; }
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)kMapBoxCols, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    std::lock_guard<std::mutex> lock(mu);
    if (cache.size() > 8192) cache.clear();
    cache[key] = *out;
    return true;
}

}  // namespace sb

#include "tcgen05_gemm.cuh"

namespace sb {
// The kernels for many rows (gemm_tcgen05_rows.cu).  0, a cudaError_t or SB_ERR_ARG.
int gemm_tcgen05_many_rows(const void* A, const void* W, void* C, int M, int N, int K, int c_dtype, int* status,
                           int variant, int epi, cudaStream_t stream);
// The pair kernel in equal shares of K blocks (gemm_tcgen05_rows.cu): float32 [parts, M, N].
int gemm_tcgen05_shares_parts(int M, int N, int K);
int gemm_tcgen05_shares(const void* A, const void* W, float* C, int M, int N, int K, int* status, cudaStream_t stream);
}  // namespace sb

namespace {

// ----------------------------------------------------------------------------- the kernel
// tma_a: the operand whose rows become accumulator lanes, [rows_a, K], box {64, 128}.
// tma_b: the operand whose rows become accumulator columns, [rows_b, K], box {64, BN}.
// SWAP = false: lanes are rows of C (m), columns are columns of C (n).
// SWAP = true : lanes are columns of C (n), columns are rows of C (m).
//
// A thread issues a tcgen05.mma about every 80 ns however narrow the tile, which for the narrow
// tiles of weight streaming is longer than the tile's loads take.  With SWAP, `issuers` (1 to
// kMaxIssuers) threads therefore share the issuing, each into an accumulator of its own, and the
// epilogue adds the accumulators.  A ring stage always belongs to the same thread (stage s to
// thread s mod issuers): a thread that met only some of a stage's uses could not tell, from the
// parity it waits for, a stage that has been refilled from one that has not been filled yet.
constexpr int kMaxIssuers = 3;
constexpr int kDefaultIssuers = 2;      // measured: 2.58 ms a decode step against 2.62 (one) and 2.59 (three)
template <int BN, bool SWAP> constexpr int acc_cols() {
    constexpr int want = (SWAP ? kMaxIssuers : 1) * BN;
    return want <= 32 ? 32 : want <= 64 ? 64 : want <= 128 ? 128 : want <= 256 ? 256 : 512;
}

template <int BN, int STAGES, bool SWAP, typename TC, int EPI = 0>
__global__ void __launch_bounds__(128, 2)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    TC* __restrict__ C, int M, int N, int K, int kb_per_split, int* __restrict__ status,
                    const uint8_t* __restrict__ next_w, long long next_bytes, int issuers) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[STAGES];
    __shared__ __align__(8) uint64_t empty_bar[STAGES];
    __shared__ __align__(8) uint64_t accum_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int a0 = blockIdx.x * BM, b0 = blockIdx.y * BN;
    const int kb_total = (K + BK - 1) / BK;
    const int kb_begin = blockIdx.z * kb_per_split;
    const int kb_end = min(kb_total, kb_begin + kb_per_split);
    const int kb_count = kb_end - kb_begin;
    if (!SWAP) issuers = 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        mbar_init(smem_u32(&accum_bar), issuers);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(acc_cols<BN, SWAP>()) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_d = tmem_base_slot;

    sb::pdl_launch_dependents();          // the next kernel may begin its prologue
    if (warp == 0 && lane == 0) {
        // ---------------- producer: TMA loads into the ring.
        // (both tensor maps are fetched now: the activations' map is first used right after the
        // wait on the previous kernel, where its fetch would be on the step's critical path)
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tma_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tma_b) : "memory");
        // The weight operand (tma_a when SWAP, else tma_b) is written by no kernel, so its
        // tiles of the first ring-full of stages are fetched BEFORE the wait on the previous
        // kernel; the activation tiles of those stages follow after it.
        const int ahead = min(kb_count, STAGES);
        for (int i = 0; i < ahead; ++i) {
            const uint32_t bar = smem_u32(&full_bar[i]);
            const uint32_t sa = tiles + i * stage_bytes<BN>();
            const uint32_t sb_ = sa + BM * BK * 2;
            mbar_arrive_expect_tx(bar, stage_bytes<BN>());
            if (SWAP) tma_load_2d(sa, &tma_a, bar, (kb_begin + i) * BK, a0);
            else tma_load_2d(sb_, &tma_b, bar, (kb_begin + i) * BK, b0);
        }
        sb::pdl_wait();
        for (int i = 0; i < ahead; ++i) {
            const uint32_t bar = smem_u32(&full_bar[i]);
            const uint32_t sa = tiles + i * stage_bytes<BN>();
            const uint32_t sb_ = sa + BM * BK * 2;
            if (SWAP) tma_load_2d(sb_, &tma_b, bar, (kb_begin + i) * BK, b0);
            else tma_load_2d(sa, &tma_a, bar, (kb_begin + i) * BK, a0);
        }
        int issued = ahead;
        for (int i = ahead; i < kb_count; ++i) {
            const int s = i % STAGES;
            if (!mbar_wait(smem_u32(&empty_bar[s]), ((i / STAGES) - 1) & 1)) {
                atomicExch(status, 1);
                atomicExch(&abort_flag, 1);
                break;
            }
            if (*((volatile int*)&abort_flag)) break;
            const uint32_t bar = smem_u32(&full_bar[s]);
            const uint32_t sa = tiles + s * stage_bytes<BN>();
            const uint32_t sb_ = sa + BM * BK * 2;
            mbar_arrive_expect_tx(bar, stage_bytes<BN>());
            tma_load_2d(sa, &tma_a, bar, (kb_begin + i) * BK, a0);
            tma_load_2d(sb_, &tma_b, bar, (kb_begin + i) * BK, b0);
            issued = i + 1;
        }
        if (*((volatile int*)&abort_flag)) {
            // Wait (bounded) for the copies this thread issued, so none lands after exit.
            for (int i = max(0, issued - STAGES); i < issued; ++i)
                mbar_wait(smem_u32(&full_bar[i % STAGES]), (i / STAGES) & 1);
        } else if (next_bytes > 0) {
            // All of this block's own loads are on their way: ask for this block's share of
            // the weights that the next product streams to be brought into L2, so that memory
            // keeps streaming through this kernel's epilogue and the next kernel's start.
            const long long nblk = (long long)gridDim.x * gridDim.y * gridDim.z;
            const long long blk = ((long long)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
            const long long chunks = (next_bytes + kL2Chunk - 1) / kL2Chunk;
            for (long long c = blk; c < chunks; c += nblk) {
                const long long off = c * kL2Chunk, left = next_bytes - off;
                l2_prefetch(next_w + off, (uint32_t)(left < kL2Chunk ? left : kL2Chunk));
            }
        }
    } else if (warp >= 1 && warp <= issuers && lane == 0) {
        // ---------------- MMA issuer q of `issuers`: the K blocks of its stages into accumulator q
        constexpr uint32_t idesc = make_idesc(BN);
        const int q = warp - 1;
        const uint32_t acc = tmem_d + q * BN;
        bool ok = true, first = true;
        // s, owner and parity follow i % STAGES, s % issuers and (i / STAGES) & 1 without dividing
        int s = -1, owner = -1;
        uint32_t parity = 0;
        for (int i = 0; i < kb_count && ok; ++i) {
            if (++owner == issuers) owner = 0;
            if (++s == STAGES) { s = 0; owner = 0; parity ^= (i > 0); }
            if (owner != q) continue;
            if (!mbar_wait(smem_u32(&full_bar[s]), parity)) {
                atomicExch(status, 2);
                atomicExch(&abort_flag, 1);
                ok = false;
                break;
            }
            tcgen05_fence_after();
            const uint32_t sa = tiles + s * stage_bytes<BN>();
            const uint32_t sb = sa + BM * BK * 2;
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
                const uint64_t da = make_smem_desc(sa + k * UMMA_K * 2);
                const uint64_t db = make_smem_desc(sb + k * UMMA_K * 2);
                tcgen05_mma_bf16(acc, da, db, idesc, (!first || k > 0) ? 1u : 0u);
            }
            first = false;
            tcgen05_commit(smem_u32(&empty_bar[s]));   // frees the stage when these MMAs have read it
        }
        tcgen05_commit(smem_u32(&accum_bar));          // arrives when every MMA of this thread has completed
    }
    __syncwarp();

    // ---------------- epilogue: all four warps, warp w owns lanes 32w .. 32w+31
    sb::pdl_wait();                       // C may still be read by an earlier kernel until now
    bool good = mbar_wait(smem_u32(&accum_bar), 0);
    if (!good) atomicExch(status, 3);
    if (*((volatile int*)&abort_flag)) good = false;
    good = __all_sync(0xffffffffu, good);      // tcgen05.ld below needs the whole warp
    tcgen05_fence_after();
    if (good && kb_count > 0) {
        TC* Cz = C + (size_t)blockIdx.z * M * N;
        const int lane_row = warp * 32 + lane;
#pragma unroll
        for (int c0 = 0; c0 < BN; c0 += 16) {
            uint32_t r[16];
            const uint32_t at = tmem_d + (static_cast<uint32_t>(warp * 32) << 16) + c0;
            tmem_ld16(at, r);
            if constexpr (SWAP) {
                // the accumulators of the other issuing threads count where those had a K block
                // (all are read, so that the loads overlap; what an unused one holds is dropped)
                const int used = min(issuers, kb_count);
                uint32_t r1[16], r2[16];
                tmem_ld16(at + BN, r1);
                tmem_ld16(at + 2 * BN, r2);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float v1 = used > 1 ? __uint_as_float(r1[j]) : 0.0f;
                    const float v2 = used > 2 ? __uint_as_float(r2[j]) : 0.0f;
                    r[j] = __float_as_uint(__uint_as_float(r[j]) + v1 + v2);
                }
            } else {
                tmem_ld_wait();
            }
            if (SWAP && EPI == 1) {
                // weight rows interleave gate and up: lane pairs (even = gate_f, odd = up_f);
                // the even lane writes C[m, f] = up * silu(gate), C has N/2 columns
                const int n = a0 + lane_row;
                const int F = N >> 1;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float v = __uint_as_float(r[j]);
                    const float up = __shfl_xor_sync(0xffffffffu, v, 1);
                    const int m = b0 + c0 + j;
                    if ((lane & 1) == 0 && n + 1 < N && m < M)
                        store_out<TC>(C + (size_t)m * F + (n >> 1), up * (v / (1.0f + expf(-v))));
                }
            } else if (SWAP) {
                const int n = a0 + lane_row;
                if (n < N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = b0 + c0 + j;
                        if (m < M) store_out<TC>(Cz + (size_t)m * N + n, __uint_as_float(r[j]));
                    }
                }
            } else {
                const int m = a0 + lane_row;
                if (m < M) {
                    TC* row = Cz + (size_t)m * N + b0 + c0;
                    if (b0 + c0 + 16 <= N && ((reinterpret_cast<uintptr_t>(row) & 15) == 0)) {
                        if constexpr (sizeof(TC) == 2) {
                            uint32_t packed[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * j]),
                                                                         __uint_as_float(r[2 * j + 1]));
                                packed[j] = *reinterpret_cast<uint32_t*>(&v);
                            }
                            uint4* dst = reinterpret_cast<uint4*>(row);
                            dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                            dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                        } else {
                            uint4* dst = reinterpret_cast<uint4*>(row);
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                dst[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (b0 + c0 + j < N) store_out<TC>(row + j, __uint_as_float(r[j]));
                    }
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(acc_cols<BN, SWAP>())
                     : "memory");
    }
}

// ----------------------------------------------------------------------------- host side
using sb::get_map;

// The weights of the product that follows the one being launched (set by sb_gemm_tcgen05 for
// the duration of one dispatch; the weight-streaming kernel passes them on).
struct NextWeights { const uint8_t* ptr = nullptr; long long bytes = 0; };
thread_local NextWeights g_next;

// How many threads issue the MMAs of a weight-streaming block (SOCRATES_GEMM_ISSUERS, 1 to 3).
int issuing_threads() {
    static const int n = [] {
        const char* e = getenv("SOCRATES_GEMM_ISSUERS");
        const int v = e ? atoi(e) : kDefaultIssuers;
        return v < 1 ? 1 : (v > kMaxIssuers ? kMaxIssuers : v);
    }();
    return n;
}

template <int BN, int STAGES, bool SWAP, typename TC, int EPI = 0>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, void* C, int M, int N, int K, dim3 grid, int kb_per_split,
           int* status, cudaStream_t stream) {
    auto kernel = gemm_tcgen05_kernel<BN, STAGES, SWAP, TC, EPI>;
    constexpr int smem = STAGES * stage_bytes<BN>() + 1024;
    static sb::OncePerDevice once_per_device;
    bool& configured = once_per_device.flag();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) { sb_set_error("gemm_tcgen05: %s", cudaGetErrorString(e)); return (int)e; }
        configured = true;
    }
    const NextWeights next = SWAP ? g_next : NextWeights{};
    sb::launch(kernel, dim3(grid), dim3(128), smem, stream, ma, mb, (TC*)C, M, N, K, kb_per_split, status,
               next.ptr, next.bytes, issuing_threads());
    return 0;
}

template <typename TC>
int dispatch(const void* A, const void* W, void* C, int M, int N, int K, int splits, int* status,
             cudaStream_t stream, int* splits_out, int variant, int epi) {
    const int kb_total = (K + BK - 1) / BK;
    if (splits > kb_total) splits = kb_total;
    const int kb_per_split = (kb_total + splits - 1) / splits;
    splits = (kb_total + kb_per_split - 1) / kb_per_split;      // no empty part
    *splits_out = splits;
    CUtensorMap ma, mb;
    if (M <= 64 && epi != 0 && splits != 1) {
        sb_set_error("gemm_tcgen05: the fused SiLU*mul epilogue cannot follow a K split");
        return SB_ERR_ARG;
    }
    if (M <= 64) {
        const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
        if (!get_map(&ma, W, N, K, BM) || !get_map(&mb, A, M, K, bn)) {
            sb_set_error("gemm_tcgen05: cuTensorMapEncodeTiled failed (M=%d N=%d K=%d)", M, N, K);
            return SB_ERR_ARG;
        }
        dim3 grid((N + BM - 1) / BM, 1, splits);
        // Weight streaming.  The ring leaves room for two blocks on an SM (and for the next kernel's
        // blocks to start their prologue beside it).  Rings of 3 to 5 stages and one that fills an
        // SM's shared memory from a single block were measured slower in the decode graph of the
        // 4B shape (2.78 to 3.05 against 2.75 ms a step).
        if (epi == 1) {
            if (bn == 16) return launch<16, 6, true, TC, 1>(ma, mb, C, M, N, K, grid, kb_per_split, status, stream);
            if (bn == 32) return launch<32, 5, true, TC, 1>(ma, mb, C, M, N, K, grid, kb_per_split, status, stream);
            return launch<64, 4, true, TC, 1>(ma, mb, C, M, N, K, grid, kb_per_split, status, stream);
        }
        if (bn == 16) return launch<16, 6, true, TC>(ma, mb, C, M, N, K, grid, kb_per_split, status, stream);
        if (bn == 32) return launch<32, 5, true, TC>(ma, mb, C, M, N, K, grid, kb_per_split, status, stream);
        return launch<64, 4, true, TC>(ma, mb, C, M, N, K, grid, kb_per_split, status, stream);
    }
    if (splits == 1 && N >= 128 && variant != 4)      // the persistent kernels (gemm_tcgen05_rows.cu)
        return sb::gemm_tcgen05_many_rows(A, W, C, M, N, K, sizeof(TC) == 2 ? SB_BF16 : SB_F32, status, variant, epi, stream);
    if (epi != 0) {
        sb_set_error("gemm_tcgen05: the fused SiLU*mul epilogue needs N >= 128 and no K split");
        return SB_ERR_ARG;
    }
    // variant 4: the one-tile-per-block kernel also for many rows
    const int bn = N >= 256 ? 256 : (N > 64 ? 128 : 64);
    if (!get_map(&ma, A, M, K, BM) || !get_map(&mb, W, N, K, bn)) {
        sb_set_error("gemm_tcgen05: cuTensorMapEncodeTiled failed (M=%d N=%d K=%d)", M, N, K);
        return SB_ERR_ARG;
    }
    dim3 grid((M + BM - 1) / BM, (N + bn - 1) / bn, splits);
    if (bn == 256) return launch<256, 4, false, TC>(ma, mb, C, M, N, K, grid, kb_per_split, status, stream);
    if (bn == 128) return launch<128, 3, false, TC>(ma, mb, C, M, N, K, grid, kb_per_split, status, stream);
    return launch<64, 4, false, TC>(ma, mb, C, M, N, K, grid, kb_per_split, status, stream);
}

}  // namespace

// A [M,K] and W [N,K] bfloat16, row-major, 16-byte aligned, K a multiple of 8.
// C: c_dtype [M,N] when the effective split count is 1, else float32 [splits, M, N].
// *splits_io: wanted number of K parts in, number actually written out (never more).
// status: device int the kernel writes a non-zero code to if a bounded wait gave up.
// variant: 0 = the kernels chosen by shape; 4 = one tile per block also for many rows
//          (the default there is the persistent kernel); 128, 160, 256 = that tile width
//          in the persistent kernel instead of the one it would choose; 1128, 1160, 1192,
//          1256 = the pair kernel (two SMs per tile, cta_group::2) with tiles 256 x (variant - 1000);
//          2000 = the pair kernel dealing equal shares of K blocks, float32 partial sums
//          [parts, M, N] with *splits_io == sb_gemm_tcgen05_shares_parts(M, N, K).
// epilogue: 0 = C[M,N]; 1 = W interleaves gate and up rows and C is [M, N/2] = up * silu(gate)
//          (no K split; for many rows N >= 128).
// next_weights / next_bytes: null / 0, or a 16-byte aligned range that the product after this
//          one streams; the weight-streaming kernel (M <= 64) asks for it in L2 once its own
//          loads are issued.  A hint: other kernels ignore it.
extern "C" int sb_gemm_tcgen05(void* C, const void* A, const void* W, int M, int N, int K, int c_dtype,
                               int* splits_io, int* status, int variant, int epilogue,
                               const void* next_weights, long long next_bytes, cudaStream_t stream) {
    SB_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tcgen05: bad sizes M=%d N=%d K=%d", M, N, K);
    SB_REQUIRE(K % 8 == 0, "gemm_tcgen05: K=%d must be a multiple of 8 (16-byte rows for TMA)", K);
    SB_REQUIRE((reinterpret_cast<uintptr_t>(A) & 15) == 0 && (reinterpret_cast<uintptr_t>(W) & 15) == 0,
               "gemm_tcgen05: operands must be 16-byte aligned");
    SB_REQUIRE(status != nullptr && splits_io != nullptr, "gemm_tcgen05: status and splits are required");
    int splits = *splits_io;
    SB_REQUIRE(splits >= 1 && splits <= 64, "gemm_tcgen05: splits=%d is outside 1..64", splits);
    SB_REQUIRE(splits == 1 || c_dtype == SB_F32, "gemm_tcgen05: partial sums of a split product are float32");
    SB_REQUIRE(epilogue == 0 || (epilogue == 1 && N % 2 == 0), "gemm_tcgen05: bad epilogue %d for N=%d", epilogue, N);
    SB_REQUIRE((M + 127) / 128 <= 65535 && (N + 63) / 64 <= 65535, "gemm_tcgen05: matrix too large");
    SB_REQUIRE(next_bytes >= 0 && (reinterpret_cast<uintptr_t>(next_weights) & 15) == 0,
               "gemm_tcgen05: the next-weights hint must be 16-byte aligned");
    if (variant == 2000) {
        // many rows as float32 partial sums from the pair kernel in equal shares of K blocks
        const int parts = sb::gemm_tcgen05_shares_parts(M, N, K);
        SB_REQUIRE(parts > 0 && c_dtype == SB_F32 && epilogue == 0 && splits == parts,
                   "gemm_tcgen05: equal shares need float32 output of %d parts (asked: %d) for M=%d N=%d K=%d",
                   parts, splits, M, N, K);
        const int rc = sb::gemm_tcgen05_shares(A, W, static_cast<float*>(C), M, N, K, status, stream);
        if (rc != 0) return rc;
        SB_LAUNCH_CHECK();
    }
    g_next.ptr = static_cast<const uint8_t*>(next_weights);
    g_next.bytes = next_weights != nullptr ? (next_bytes & ~15LL) : 0;
    int rc;
    if (c_dtype == SB_F32)
        rc = dispatch<float>(A, W, C, M, N, K, splits, status, stream, splits_io, variant, epilogue);
    else if (c_dtype == SB_BF16)
        rc = dispatch<__nv_bfloat16>(A, W, C, M, N, K, splits, status, stream, splits_io, variant, epilogue);
    else
        SB_REQUIRE(false, "gemm_tcgen05: unknown output dtype %d", c_dtype);
    g_next = NextWeights{};
    if (rc != 0) return rc;
    SB_LAUNCH_CHECK();
}

// How many float32 parts variant 2000 (the pair kernel in equal shares of K blocks) writes for this
// shape; 0 if it does not serve it (few rows, a narrow N, more than four pieces to a tile).
extern "C" int sb_gemm_tcgen05_shares_parts(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0 || K % 8) return 0;
    return sb::gemm_tcgen05_shares_parts(M, N, K);
}

// How many K parts sb_gemm_tcgen05 will actually write for a wanted count (host only).
extern "C" int sb_gemm_tcgen05_splits(int K, int splits) {
    const int kb_total = (K + BK - 1) / BK;
    if (splits > kb_total) splits = kb_total;
    if (splits < 1) splits = 1;
    const int per = (kb_total + splits - 1) / splits;
    return (kb_total + per - 1) / per;
}
