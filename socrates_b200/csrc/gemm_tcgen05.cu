// C[M,N] = A[M,K] * W[N,K]^T in bfloat16 on the 5th-generation tensor cores:
// tcgen05.mma with the accumulator in tensor memory, operands brought to shared
// memory by TMA (128-byte swizzle, K-major), a ring of stages between one producer
// thread and one MMA thread, and a tcgen05.ld epilogue by four warps.
//
// One kernel serves both regimes of the engine:
//   * many rows (prompt portions): the activations fill the 128 accumulator lanes and
//     the weights are the N operand (tile 128 x BN, BN up to 256);
//   * few rows (decode, M <= 64): operands are swapped so that 128 rows of the WEIGHT
//     matrix fill the lanes and the batch is the N operand (BN = 16, 32 or 64).  The
//     kernel is then a weight stream at HBM rate; K is cut into `splits` parts so that
//     narrow matrices still cover every SM, and part z writes float32 partial sums to
//     C + z*M*N, which the consuming kernel adds up in a fixed order.
//
// No cluster launch and no multicast: every block loads its own tiles.  Every wait on
// an mbarrier is bounded; if one gives up, the block records a code in *status, waits
// (again bounded) for its own copies in flight, frees its tensor memory and returns.
#include <cuda.h>
#include <stdint.h>
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

namespace {

constexpr int BM = 128;          // accumulator lanes
constexpr int BK = 64;           // K elements per stage: one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;   // a wait gives up after two seconds

// ----------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: false if the phase did not complete within WAIT_LIMIT_NS.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (int i = 0; i < 4096; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer_ns();
    for (;;) {
        for (int i = 0; i < 1024; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_timer_ns() - t0 > WAIT_LIMIT_NS) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of
// 128 bytes, 8-row groups 1024 bytes apart (stride byte offset 64 in 16-byte units),
// leading byte offset 1 (unused with swizzle), descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr) {
    const uint32_t lo = ((addr & 0x3FFFFu) >> 4) | (1u << 16);
    const uint32_t hi = 64u | (1u << 14) | (2u << 29);
    return (static_cast<uint64_t>(hi) << 32) | lo;
}

// Instruction descriptor: D float32, A and B bfloat16, both K-major, M = 128, N = BN.
__host__ __device__ constexpr uint32_t make_idesc(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(bn >> 3) << 17) |
           (static_cast<uint32_t>(BM >> 4) << 24);
}

template <int BN> constexpr int tmem_cols() { return BN < 32 ? 32 : BN; }
template <int BN> constexpr int stage_bytes() { return BM * BK * 2 + BN * BK * 2; }

template <typename TC> __device__ __forceinline__ void store_out(TC* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) {
    *p = __float2bfloat16_rn(v);
}

constexpr long long kL2Chunk = 16384;                       // bytes per L2 prefetch instruction
__device__ __forceinline__ void l2_prefetch(const void* p, uint32_t bytes) {
    const uint8_t* a = static_cast<const uint8_t*>(p);
    for (uint32_t o = 0; o < bytes; o += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(a + o));
}

// ----------------------------------------------------------------------------- the kernel
// tma_a: the operand whose rows become accumulator lanes, [rows_a, K], box {64, 128}.
// tma_b: the operand whose rows become accumulator columns, [rows_b, K], box {64, BN}.
// SWAP = false: lanes are rows of C (m), columns are columns of C (n).
// SWAP = true : lanes are columns of C (n), columns are rows of C (m).
template <int BN, int STAGES, bool SWAP, typename TC, int EPI = 0>
__global__ void __launch_bounds__(128)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    TC* __restrict__ C, int M, int N, int K, int kb_per_split, int* __restrict__ status,
                    const uint8_t* __restrict__ next_w, long long next_bytes) {
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

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        mbar_init(smem_u32(&accum_bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(tmem_cols<BN>()) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_d = tmem_base_slot;

    sb::pdl_launch_dependents();          // the next kernel may begin its prologue
    if (warp == 0 && lane == 0) {
        // ---------------- producer: TMA loads into the ring.
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
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer
        constexpr uint32_t idesc = make_idesc(BN);
        bool ok = true;
        for (int i = 0; i < kb_count && ok; ++i) {
            const int s = i % STAGES;
            if (!mbar_wait(smem_u32(&full_bar[s]), (i / STAGES) & 1)) {
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
                tcgen05_mma_bf16(tmem_d, da, db, idesc, (i > 0 || k > 0) ? 1u : 0u);
            }
            tcgen05_commit(smem_u32(&empty_bar[s]));   // frees the stage when these MMAs have read it
        }
        tcgen05_commit(smem_u32(&accum_bar));          // arrives when every MMA above has completed
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
            tmem_ld16(tmem_d + (static_cast<uint32_t>(warp * 32) << 16) + c0, r);
            tmem_ld_wait();
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(tmem_cols<BN>())
                     : "memory");
    }
}

// One thread's row of a finished accumulator tile, BN columns from tensor memory at `taddr`,
// to row m of C (columns b0 ..).  Called by whole warps: the loads are warp-wide.
//   EPI = 0: C[m, n] = acc
//   EPI = 1: columns interleave gate and up; C[m, f] = up * silu(gate), C has N/2 columns.
template <int BN, typename TC, int EPI>
__device__ __forceinline__ void drain_tile(uint32_t taddr, TC* __restrict__ C, int M, int N, int m, int b0) {
#pragma unroll 2
    for (int c0 = 0; c0 < BN; c0 += 16) {
        uint32_t r[16];
        tmem_ld16(taddr + c0, r);
        tmem_ld_wait();
        if (m >= M) continue;
        if (EPI == 1) {
            // columns come in (gate, up) pairs: 16 accumulator columns -> 8 outputs
            const int f0 = (b0 + c0) >> 1, F = N >> 1;
            TC* row = C + (size_t)m * F + f0;
            float o[8];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float g = __uint_as_float(r[2 * q]), u = __uint_as_float(r[2 * q + 1]);
                o[q] = u * (g / (1.0f + expf(-g)));
            }
            if (f0 + 8 <= F && ((reinterpret_cast<uintptr_t>(row) & 15) == 0) && sizeof(TC) == 2) {
                uint32_t pk[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    __nv_bfloat162 v = __floats2bfloat162_rn(o[2 * q], o[2 * q + 1]);
                    pk[q] = *reinterpret_cast<uint32_t*>(&v);
                }
                *reinterpret_cast<uint4*>(row) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            } else {
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    if (f0 + q < F) store_out<TC>(row + q, o[q]);
            }
        } else {
            TC* row = C + (size_t)m * N + b0 + c0;
            if (b0 + c0 + 16 <= N && ((reinterpret_cast<uintptr_t>(row) & 15) == 0)) {
                if constexpr (sizeof(TC) == 2) {
                    uint32_t packed[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * q]),
                                                                 __uint_as_float(r[2 * q + 1]));
                        packed[q] = *reinterpret_cast<uint32_t*>(&v);
                    }
                    uint4* dst = reinterpret_cast<uint4*>(row);
                    dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                } else {
                    uint4* dst = reinterpret_cast<uint4*>(row);
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        dst[q] = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
                }
            } else {
#pragma unroll
                for (int q = 0; q < 16; ++q)
                    if (b0 + c0 + q < N) store_out<TC>(row + q, __uint_as_float(r[q]));
            }
        }
    }
}

// ----------------------------------------------------------------------------- persistent kernel
// Many rows (prompt portions): one block per SM walks over output tiles of 128 x BN.
// Six warps: warp 0 lane 0 feeds the shared-memory ring by TMA, warp 1 lane 0 issues the
// MMAs, warps 2-5 read finished accumulators out of tensor memory and store C.  There are
// two accumulators (TMEM columns 0.. and 256..), so the epilogue of tile i runs beside the
// main loop of tile i+1.  Tiles are walked with the row index fastest: blocks running at
// the same time share the weight panel, which stays in L2.
//   EPI = 0: C[m, n] = acc
//   EPI = 1: the weight rows interleave gate and up (row 2f = gate_f, row 2f+1 = up_f);
//            C[m, f] = up * silu(gate), C has N/2 columns (SiLU*mul fused into the product).
constexpr int ACC_STRIDE = 256;          // TMEM columns between the two accumulators

template <int BN, int STAGES, typename TC, int EPI>
__global__ void __launch_bounds__(192)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                               TC* __restrict__ C, int M, int N, int K, int tiles_m, int tiles_n,
                               int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[STAGES];
    __shared__ __align__(8) uint64_t empty_bar[STAGES];
    __shared__ __align__(8) uint64_t acc_full[2];
    __shared__ __align__(8) uint64_t acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int kb_total = (K + BK - 1) / BK;
    const int n_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&acc_full[a]), 1);
            mbar_init(smem_u32(&acc_empty[a]), 4);      // one arrival per epilogue warp
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_d = tmem_base_slot;
    sb::pdl_launch_dependents();

    if (warp == 0 && lane == 0) {
        // ---------------- producer
        // The weight tiles (tma_b) of the first ring-full are fetched before the wait on the
        // previous kernel, the activation tiles after it.
        uint32_t it = 0;                                   // k-blocks issued so far, over all tiles
        bool waited = false;
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
            const int a0 = (t % tiles_m) * BM, b0 = (t / tiles_m) * BN;
            if (!waited) {
                const int ahead = min(kb_total, STAGES);
                for (int i = 0; i < ahead; ++i) {
                    const uint32_t bar = smem_u32(&full_bar[i]);
                    mbar_arrive_expect_tx(bar, stage_bytes<BN>());
                    tma_load_2d(tiles + i * stage_bytes<BN>() + BM * BK * 2, &tma_b, bar, i * BK, b0);
                }
                sb::pdl_wait();
                for (int i = 0; i < ahead; ++i)
                    tma_load_2d(tiles + i * stage_bytes<BN>(), &tma_a, smem_u32(&full_bar[i]), i * BK, a0);
                waited = true;
                it = ahead;
                for (int i = ahead; i < kb_total && ok; ++i, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(smem_u32(&empty_bar[s]), ((it / STAGES) - 1) & 1)) { ok = false; break; }
                    const uint32_t bar = smem_u32(&full_bar[s]);
                    mbar_arrive_expect_tx(bar, stage_bytes<BN>());
                    tma_load_2d(tiles + s * stage_bytes<BN>(), &tma_a, bar, i * BK, a0);
                    tma_load_2d(tiles + s * stage_bytes<BN>() + BM * BK * 2, &tma_b, bar, i * BK, b0);
                }
                continue;
            }
            for (int i = 0; i < kb_total && ok; ++i, ++it) {
                const int s = it % STAGES;
                if (it >= STAGES && !mbar_wait(smem_u32(&empty_bar[s]), ((it / STAGES) - 1) & 1)) { ok = false; break; }
                if (*((volatile int*)&abort_flag)) { ok = false; break; }
                const uint32_t bar = smem_u32(&full_bar[s]);
                mbar_arrive_expect_tx(bar, stage_bytes<BN>());
                tma_load_2d(tiles + s * stage_bytes<BN>(), &tma_a, bar, i * BK, a0);
                tma_load_2d(tiles + s * stage_bytes<BN>() + BM * BK * 2, &tma_b, bar, i * BK, b0);
            }
        }
        if (!ok) {
            atomicExch(status, 1);
            atomicExch(&abort_flag, 1);
            // Wait (bounded) for the copies in flight, so that none lands after exit.
            for (uint32_t i = it > STAGES ? it - STAGES : 0; i < it; ++i)
                mbar_wait(smem_u32(&full_bar[i % STAGES]), (i / STAGES) & 1);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issuer
        constexpr uint32_t idesc = make_idesc(BN);
        uint32_t it = 0;
        int j = 0;                                         // tiles done by this block
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++j) {
            const int acc = j & 1;
            // the epilogue must have drained this accumulator (first use of each passes at once)
            if (j >= 2 && !mbar_wait(smem_u32(&acc_empty[acc]), ((j >> 1) - 1) & 1)) { ok = false; break; }
            tcgen05_fence_after();
            const uint32_t d = tmem_d + acc * ACC_STRIDE;
            for (int i = 0; i < kb_total; ++i, ++it) {
                const int s = it % STAGES;
                if (!mbar_wait(smem_u32(&full_bar[s]), (it / STAGES) & 1)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t sa = tiles + s * stage_bytes<BN>();
                const uint32_t sb_ = sa + BM * BK * 2;
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    tcgen05_mma_bf16(d, make_smem_desc(sa + k * UMMA_K * 2), make_smem_desc(sb_ + k * UMMA_K * 2),
                                     idesc, (i > 0 || k > 0) ? 1u : 0u);
                tcgen05_commit(smem_u32(&empty_bar[s]));
            }
            if (!ok) break;
            tcgen05_commit(smem_u32(&acc_full[acc]));
        }
        if (!ok) {
            atomicExch(status, 2);
            atomicExch(&abort_flag, 1);
        }
    } else if (warp >= 2) {
        // ---------------- epilogue: warp w owns TMEM lanes 32*(w%4) .. +31
        sb::pdl_wait();                                    // C may still be read by an earlier kernel until now
        const int quarter = warp & 3;
        int j = 0;
        for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++j) {
            const int acc = j & 1;
            bool good = mbar_wait(smem_u32(&acc_full[acc]), (j >> 1) & 1);
            if (*((volatile int*)&abort_flag)) good = false;
            good = __all_sync(0xffffffffu, good);
            if (!good) {
                if (lane == 0) { atomicExch(status, 3); atomicExch(&abort_flag, 1); }
                break;
            }
            tcgen05_fence_after();
            const int a0 = (t % tiles_m) * BM, b0 = (t / tiles_m) * BN;
            const int m = a0 + quarter * 32 + lane;
            const uint32_t taddr = tmem_d + acc * ACC_STRIDE + (static_cast<uint32_t>(quarter * 32) << 16);
            drain_tile<BN, TC, EPI>(taddr, C, M, N, m, b0);
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&acc_empty[acc])) : "memory");
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(512) : "memory");
    }
}

// ----------------------------------------------------------------------------- pair kernel
// Many rows, two SMs per tile: a cluster of two blocks owns output tiles of 256 x BN.  Block r
// of the pair brings rows 128r .. 128r+127 of the A tile and rows (BN/2)r .. of the B tile
// into ITS shared memory; one thread of block 0 issues tcgen05.mma.cta_group::2 (M = 256),
// which reads both blocks' shared memory and writes rows 128r .. of the accumulator into
// block r's tensor memory.  Per output element the pair moves (256 + BN) / (256 * BN) operand
// elements from L2 to shared memory against (128 + BN) / (128 * BN) of a single block: a third
// less at BN = 256, which is what bounds the single-block kernel on narrow projections.
//   * full_bar[s] lives in block 0; both blocks' TMA copies complete on it (cta_group::2 form
//     of the copy, barrier address mapped into block 0), block 0's producer arms it with the
//     bytes of both.
//   * empty_bar[s] and acc_full[a] exist in both blocks and are signalled by one multicast
//     tcgen05.commit; acc_empty[a] lives in block 0 and collects the 8 epilogue warps of both.
//   * Nothing here waits without a limit except the cluster barriers at start and end, which
//     every thread reaches: each role leaves its loop on the first wait that gives up.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The copy of a block of a pair; `bar` is a shared::cluster address (either block's barrier).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"(mask) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                                      uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Bounded wait with cluster scope, for a phase that threads of the other block complete.  (The
// phases that copies and tcgen05.commit complete are waited for with the plain form: the
// cluster-scope acquire in the issuing thread's inner loop cost a fifth of the throughput.)
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity) {
    for (int i = 0; i < 4096; ++i)
        if (mbar_try_wait_cluster(bar, parity)) return true;
    const unsigned long long t0 = global_timer_ns();
    for (;;) {
        for (int i = 0; i < 1024; ++i)
            if (mbar_try_wait_cluster(bar, parity)) return true;
        if (global_timer_ns() - t0 > WAIT_LIMIT_NS) return false;
    }
}

// Instruction descriptor of the pair's product: M = 256, N = BN.
__host__ __device__ constexpr uint32_t make_idesc_pair(int bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(bn >> 3) << 17) |
           (static_cast<uint32_t>(256 >> 4) << 24);
}
template <int BN> constexpr int pair_stage_bytes() { return BM * BK * 2 + (BN / 2) * BK * 2; }

template <int BN, int STAGES, typename TC, int EPI>
__global__ void __launch_bounds__(192)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                         TC* __restrict__ C, int M, int N, int K, int tiles_m, int tiles_n,
                         int* __restrict__ status) {
    constexpr int ACC_COLS = BN <= 128 ? 128 : 256;       // TMEM columns between the two accumulators
    constexpr int SB = pair_stage_bytes<BN>();
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[STAGES];
    __shared__ __align__(8) uint64_t empty_bar[STAGES];
    __shared__ __align__(8) uint64_t acc_full[2];
    __shared__ __align__(8) uint64_t acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const uint32_t tiles = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int kb_total = (K + BK - 1) / BK;
    const int n_tiles = tiles_m * tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&acc_full[a]), 1);
            mbar_init(smem_u32(&acc_empty[a]), 8);      // four epilogue warps in each block of the pair
        }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // executed by one warp of EACH block of the pair
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(2 * ACC_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();                                    // both blocks' barriers exist from here on
    tcgen05_fence_after();
    const uint32_t tmem_d = tmem_base_slot;
    // The product addresses the accumulator by ONE tensor-memory address for both blocks.
    uint32_t peer_base;
    asm volatile("ld.shared::cluster.u32 %0, [%1];"
                 : "=r"(peer_base) : "r"(map_to_cta(smem_u32(&tmem_base_slot), rank ^ 1u)) : "memory");
    const bool bases_agree = peer_base == tmem_d;
    if (!bases_agree && threadIdx.x == 0) atomicExch(status, 4);
    sb::pdl_launch_dependents();

    if (!bases_agree) {
        // nothing is computed; fall through to the common exit
    } else if (warp == 0 && lane == 0) {
        // ---------------- producer (in both blocks): this block's halves of the A and B tiles
        // The weights are written by no kernel: the B tiles of the first ring-full are
        // fetched before the wait on the previous kernel, the A tiles after it.
        uint32_t it = 0;
        bool waited = false, ok = true;
        for (int t = pair; t < n_tiles && ok; t += n_pairs) {
            const int a0 = (t % tiles_m) * 256 + (int)rank * BM;
            const int b0 = (t / tiles_m) * BN + (int)rank * (BN / 2);
            int i = 0;
            if (!waited) {
                const int ahead = min(kb_total, STAGES);
                for (int q = 0; q < ahead; ++q) {
                    if (rank == 0) mbar_arrive_expect_tx(smem_u32(&full_bar[q]), 2 * SB);
                    tma_load_2d_pair(tiles + q * SB + BM * BK * 2, &tma_b, map_to_cta(smem_u32(&full_bar[q]), 0),
                                     q * BK, b0);
                }
                sb::pdl_wait();
                waited = true;
                for (int q = 0; q < ahead; ++q)
                    tma_load_2d_pair(tiles + q * SB, &tma_a, map_to_cta(smem_u32(&full_bar[q]), 0), q * BK, a0);
                i = ahead;
                it = ahead;
            }
            for (; i < kb_total && ok; ++i, ++it) {
                const int s = it % STAGES;
                if (it >= STAGES && !mbar_wait(smem_u32(&empty_bar[s]), ((it / STAGES) - 1) & 1)) { ok = false; break; }
                if (*((volatile int*)&abort_flag)) { ok = false; break; }
                const uint32_t bar0 = map_to_cta(smem_u32(&full_bar[s]), 0);
                if (rank == 0) mbar_arrive_expect_tx(smem_u32(&full_bar[s]), 2 * SB);
                tma_load_2d_pair(tiles + s * SB, &tma_a, bar0, i * BK, a0);
                tma_load_2d_pair(tiles + s * SB + BM * BK * 2, &tma_b, bar0, i * BK, b0);
            }
        }
        if (!ok) {
            atomicExch(status, 1);
            atomicExch(&abort_flag, 1);
            // Copies in flight must not land after exit: block 0 waits (bounded) on the barriers
            // they complete on; block 1, whose copies complete on block 0's barriers, lets a
            // millisecond pass (a copy takes microseconds).
            if (rank == 0) {
                for (uint32_t q = it > STAGES ? it - STAGES : 0; q < it; ++q)
                    mbar_wait(smem_u32(&full_bar[q % STAGES]), (q / STAGES) & 1);
            } else {
                const unsigned long long t0 = global_timer_ns();
                while (global_timer_ns() - t0 < 1000000ull) {}
            }
        }
    } else if (warp == 1 && lane == 0 && rank == 0) {
        // ---------------- MMA issuer: one thread of block 0 for the pair
        constexpr uint32_t idesc = make_idesc_pair(BN);
        uint32_t it = 0;
        int j = 0;
        bool ok = true;
        for (int t = pair; t < n_tiles && ok; t += n_pairs, ++j) {
            const int acc = j & 1;
            if (j >= 2 && !mbar_wait_cluster(smem_u32(&acc_empty[acc]), ((j >> 1) - 1) & 1)) { ok = false; break; }
            tcgen05_fence_after();
            const uint32_t d = tmem_d + acc * ACC_COLS;
            for (int i = 0; i < kb_total; ++i, ++it) {
                const int s = it % STAGES;
                if (!mbar_wait(smem_u32(&full_bar[s]), (it / STAGES) & 1)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t sa = tiles + s * SB;
                const uint32_t sb_ = sa + BM * BK * 2;
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    tcgen05_mma_bf16_pair(d, make_smem_desc(sa + k * UMMA_K * 2), make_smem_desc(sb_ + k * UMMA_K * 2),
                                          idesc, (i > 0 || k > 0) ? 1u : 0u);
                tcgen05_commit_pair(smem_u32(&empty_bar[s]));        // frees the stage in both blocks
            }
            if (!ok) break;
            tcgen05_commit_pair(smem_u32(&acc_full[acc]));           // both blocks' epilogues may read
        }
        if (!ok) {
            atomicExch(status, 2);
            atomicExch(&abort_flag, 1);
        }
    } else if (warp >= 2) {
        // ---------------- epilogue (in both blocks): warp w owns TMEM lanes 32*(w%4) .. +31
        sb::pdl_wait();                                    // C may still be read by an earlier kernel until now
        const int quarter = warp & 3;
        int j = 0;
        for (int t = pair; t < n_tiles; t += n_pairs, ++j) {
            const int acc = j & 1;
            bool good = mbar_wait(smem_u32(&acc_full[acc]), (j >> 1) & 1);
            if (*((volatile int*)&abort_flag)) good = false;
            good = __all_sync(0xffffffffu, good);
            if (!good) {
                if (lane == 0) { atomicExch(status, 3); atomicExch(&abort_flag, 1); }
                break;
            }
            tcgen05_fence_after();
            const int a0 = (t % tiles_m) * 256 + (int)rank * BM, b0 = (t / tiles_m) * BN;
            const int m = a0 + quarter * 32 + lane;
            const uint32_t taddr = tmem_d + acc * ACC_COLS + (static_cast<uint32_t>(quarter * 32) << 16);
            drain_tile<BN, TC, EPI>(taddr, C, M, N, m, b0);
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(map_to_cta(smem_u32(&acc_empty[acc]), 0));
        }
    }
    // Neither block may leave while the other can still read its shared memory or signal its
    // barriers: both meet here after their last tile (or after giving up).
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(2 * ACC_COLS)
                     : "memory");
    }
}

// ----------------------------------------------------------------------------- host side
using sb::get_map;

// The weights of the product that follows the one being launched (set by sb_gemm_tcgen05 for
// the duration of one dispatch; the weight-streaming kernel passes them on).
struct NextWeights { const uint8_t* ptr = nullptr; long long bytes = 0; };
thread_local NextWeights g_next;

template <int BN, int STAGES, bool SWAP, typename TC, int EPI = 0>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, void* C, int M, int N, int K, dim3 grid, int kb_per_split,
           int* status, cudaStream_t stream) {
    auto kernel = gemm_tcgen05_kernel<BN, STAGES, SWAP, TC, EPI>;
    constexpr int smem = STAGES * stage_bytes<BN>() + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) { sb_set_error("gemm_tcgen05: %s", cudaGetErrorString(e)); return (int)e; }
        configured = true;
    }
    const NextWeights next = SWAP ? g_next : NextWeights{};
    sb::launch(kernel, dim3(grid), dim3(128), smem, stream, ma, mb, (TC*)C, M, N, K, kb_per_split, status,
               next.ptr, next.bytes);
    return 0;
}

template <int BN, int STAGES, typename TC, int EPI>
int launch_persistent(const CUtensorMap& ma, const CUtensorMap& mb, void* C, int M, int N, int K, int* status,
                      cudaStream_t stream) {
    auto kernel = gemm_tcgen05_persistent_kernel<BN, STAGES, TC, EPI>;
    constexpr int smem = STAGES * stage_bytes<BN>() + 1024;
    static bool configured = false;
    static int num_sms = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) { sb_set_error("gemm_tcgen05: %s", cudaGetErrorString(e)); return (int)e; }
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
        configured = true;
    }
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
    const int blocks = min(tiles_m * tiles_n, num_sms);
    sb::launch(kernel, dim3(blocks), dim3(192), smem, stream, ma, mb, (TC*)C, M, N, K, tiles_m, tiles_n, status);
    return 0;
}

template <int BN, int STAGES, typename TC, int EPI>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, void* C, int M, int N, int K, int* status,
                cudaStream_t stream) {
    auto kernel = gemm_tcgen05_pair_kernel<BN, STAGES, TC, EPI>;
    constexpr int smem = STAGES * pair_stage_bytes<BN>() + 1024;
    static bool configured = false;
    static int max_pairs = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) { sb_set_error("gemm_tcgen05: %s", cudaGetErrorString(e)); return (int)e; }
        // how many pairs the GPU holds at once: the grid of the persistent kernel
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2, 1, 1);
        cfg.blockDim = dim3(192, 1, 1);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        e = cudaOccupancyMaxActiveClusters(&max_pairs, kernel, &cfg);
        if (e != cudaSuccess || max_pairs < 1) {
            sb_set_error("gemm_tcgen05: no pair of blocks fits on this GPU (%s)", cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : SB_ERR_ARG;
        }
        configured = true;
    }
    const int tiles_m = (M + 255) / 256, tiles_n = (N + BN - 1) / BN;
    const int pairs = min(tiles_m * tiles_n, max_pairs);
    sb::launch_cluster(kernel, dim3(2 * pairs), dim3(192), smem, stream, 2u, ma, mb, (TC*)C, M, N, K, tiles_m,
                       tiles_n, status);
    return 0;
}

// Tile widths of the pair kernel and their ring depths.
#define SB_PAIR_WIDTHS(X) X(256) X(192) X(160) X(128)
constexpr int pair_stages(int bn) {
    const int s = (222 * 1024) / (BM * BK * 2 + (bn / 2) * BK * 2);
    return s > 8 ? 8 : s;
}

// Tile widths of the persistent kernel, and the ring depth that fits in shared memory for each.
#define SB_PERSISTENT_WIDTHS(X) X(256) X(160) X(128)
constexpr int persistent_stages(int bn) {
    const int s = (222 * 1024) / (BM * BK * 2 + bn * BK * 2);
    return s > 6 ? 6 : s;
}

// Tile width for many rows.  Blocks take tiles in a fixed stride, so the time is the number
// of waves times the time of one tile: choose the width for which that is least.  Narrower
// tiles re-read more of A per flop, so they have to win by a margin that grows as they shrink.
static int pick_bn(int M, int N, int num_sms) {
    const int tiles_m = (M + BM - 1) / BM;
    int best = 256;
    double best_cost = -1.0;
#define SB_CONSIDER(bn) { \
        const long tiles = (long)tiles_m * ((N + bn - 1) / bn); \
        const double cost = (double)((tiles + num_sms - 1) / num_sms) * bn * (1.0 + 0.15 * (256 - bn) / 128.0); \
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; } }
    SB_PERSISTENT_WIDTHS(SB_CONSIDER)
#undef SB_CONSIDER
    return best;
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
        // Weight streaming.  Two ring depths: the shallow one leaves room for two blocks on
        // an SM (and for the next kernel's blocks to start their prologue beside it), the
        // deep one fills an SM's shared memory from a single block.  Measured back to back
        // in a graph the shallow ring is faster for every projection of the 4B shape
        // (qkv 7.6 vs 10.3 us, gate_up 19.1 vs 33.7 us), so it is the default; variant 2
        // selects the deep one.
        const bool deep = variant == 2;
        if (epi == 1) {
            if (bn == 16) return launch<16, 6, true, TC, 1>(ma, mb, C, M, N, K, grid, kb_per_split, status, stream);
            if (bn == 32) return launch<32, 5, true, TC, 1>(ma, mb, C, M, N, K, grid, kb_per_split, status, stream);
            return launch<64, 4, true, TC, 1>(ma, mb, C, M, N, K, grid, kb_per_split, status, stream);
        }
        if (bn == 16) return deep ? launch<16, 12, true, TC>(ma, mb, C, M, N, K, grid, kb_per_split, status, stream)
                                  : launch<16, 6, true, TC>(ma, mb, C, M, N, K, grid, kb_per_split, status, stream);
        if (bn == 32) return deep ? launch<32, 10, true, TC>(ma, mb, C, M, N, K, grid, kb_per_split, status, stream)
                                  : launch<32, 5, true, TC>(ma, mb, C, M, N, K, grid, kb_per_split, status, stream);
        return deep ? launch<64, 8, true, TC>(ma, mb, C, M, N, K, grid, kb_per_split, status, stream)
                    : launch<64, 4, true, TC>(ma, mb, C, M, N, K, grid, kb_per_split, status, stream);
    }
    // The pair kernel is chosen for 4,096 rows and more (measured on the 4B shape: at 8,192 rows
    // the narrow projections gain a fifth and the wide ones 0 to 2 %; at 2,048 rows the wide ones
    // lose 3 %, because both kernels are then bound by how the tiles divide among the SMs), or
    // forced with variant 1000 + width.
    const bool many_waves = M >= 4096 && (long)((M + 255) / 256) * ((N + 255) / 256) >= 4L * 74;
    if (splits == 1 && N >= 128 && ((variant >= 1128 && variant <= 1256) || (variant == 0 && M > 256 && many_waves))) {
        const int bn = variant == 0 ? 256 : variant - 1000;
        if (!get_map(&ma, A, M, K, BM) || !get_map(&mb, W, N, K, bn / 2)) {
            sb_set_error("gemm_tcgen05: cuTensorMapEncodeTiled failed (M=%d N=%d K=%d)", M, N, K);
            return SB_ERR_ARG;
        }
#define SB_TRY(BN_) \
        if (bn == BN_) return epi == 1 ? launch_pair<BN_, pair_stages(BN_), TC, 1>(ma, mb, C, M, N, K, status, stream) \
                                       : launch_pair<BN_, pair_stages(BN_), TC, 0>(ma, mb, C, M, N, K, status, stream);
        SB_PAIR_WIDTHS(SB_TRY)
#undef SB_TRY
        sb_set_error("gemm_tcgen05: no pair kernel of width %d", bn);
        return SB_ERR_ARG;
    }
    if (splits == 1 && N >= 128 && variant != 4) {
        // the persistent kernel: one block per SM, epilogue beside the next tile's main loop
        int dev = 0, num_sms = 148;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
        const int bn = (variant >= 128 && variant <= 256 && variant % 16 == 0) ? variant : pick_bn(M, N, num_sms);
        if (!get_map(&ma, A, M, K, BM) || !get_map(&mb, W, N, K, bn)) {
            sb_set_error("gemm_tcgen05: cuTensorMapEncodeTiled failed (M=%d N=%d K=%d)", M, N, K);
            return SB_ERR_ARG;
        }
#define SB_TRY(BN_) \
        if (bn == BN_) return epi == 1 ? launch_persistent<BN_, persistent_stages(BN_), TC, 1>(ma, mb, C, M, N, K, status, stream) \
                                       : launch_persistent<BN_, persistent_stages(BN_), TC, 0>(ma, mb, C, M, N, K, status, stream);
        SB_PERSISTENT_WIDTHS(SB_TRY)
#undef SB_TRY
        sb_set_error("gemm_tcgen05: no persistent kernel of width %d", bn);
        return SB_ERR_ARG;
    }
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
// variant: 0 or 1 = shallow ring of the weight-streaming kernel (two blocks per SM),
//          2 = deep ring (one block per SM); 4 = one tile per block also for many rows
//          (the default there is the persistent kernel); 128, 144, ..., 256 = that tile width
//          in the persistent kernel instead of the one it would choose; 1128, 1160, 1192,
//          1256 = the pair kernel (two SMs per tile, cta_group::2) with tiles 256 x (variant - 1000).
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

// How many K parts sb_gemm_tcgen05 will actually write for a wanted count (host only).
extern "C" int sb_gemm_tcgen05_splits(int K, int splits) {
    const int kb_total = (K + BK - 1) / BK;
    if (splits > kb_total) splits = kb_total;
    if (splits < 1) splits = 1;
    const int per = (kb_total + splits - 1) / splits;
    return (kb_total + per - 1) / per;
}
