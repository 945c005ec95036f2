// Helpers shared by the tcgen05 matrix-product kernels: PTX wrappers with bounded waits,
// shared-memory and instruction descriptors, and the epilogue that drains one accumulator row.
#pragma once

#include <cuda.h>
#include <stdint.h>

#include "common.cuh"

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

// Staging of float32 output through shared memory.  A thread holds one ROW of the accumulator, so
// stores straight from registers put the 32 lanes of a store instruction on 32 different rows of C:
// 32 half-filled sectors per instruction, measured at 9 us for a 2,048 x 2,560 float32 output (15 us
// for the pair kernel's wider tiles) where a bfloat16 output of the same shape costs 1.7.  Staged,
// a warp writes 32 x 32 blocks: each lane puts its row's 32 values into a shared-memory block of its
// warp (row pitch 36 floats: conflict-free float4 accesses by quarter warp), and the block is read
// back so that eight lanes write 128 contiguous bytes of one row (four rows an instruction).
constexpr int kStagePitch = 36;                                       // floats per staged row
constexpr int kStageBytesPerWarp = 32 * kStagePitch * 4;              // 4,608
constexpr int kStageBytes = 4 * kStageBytesPerWarp;                   // four epilogue warps

// The rows m_base .. m_base + 31 of a finished accumulator tile (BN columns at `taddr`, this warp's
// lanes) to float32 C, columns b0 ..; `stage` is this warp's staging block.  Called by whole warps.
//   ADD > 0: a second accumulator ADD columns further on is added to the first.
template <int BN, int ADD = 0>
__device__ __forceinline__ void drain_tile_f32_staged(uint32_t taddr, float* __restrict__ C, int M, int N,
                                                      int m_base, int lane, int b0, float* stage) {
    static_assert(BN % 32 == 0, "staged epilogue works on blocks of 32 columns");
    const bool vec_ok = N % 4 == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld16(taddr + c0, *reinterpret_cast<uint32_t(*)[16]>(&r[0]));
        tmem_ld16(taddr + c0 + 16, *reinterpret_cast<uint32_t(*)[16]>(&r[16]));
        if constexpr (ADD > 0) {
            uint32_t r2[32];
            tmem_ld16(taddr + ADD + c0, *reinterpret_cast<uint32_t(*)[16]>(&r2[0]));
            tmem_ld16(taddr + ADD + c0 + 16, *reinterpret_cast<uint32_t(*)[16]>(&r2[16]));
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 32; ++q) r[q] = __float_as_uint(__uint_as_float(r[q]) + __uint_as_float(r2[q]));
        } else {
            tmem_ld_wait();
        }
        if (b0 + c0 >= N) continue;                                   // warp-uniform
        float4* mine = reinterpret_cast<float4*>(stage + lane * kStagePitch);
#pragma unroll
        for (int q = 0; q < 8; ++q)
            mine[q] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                  __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
        __syncwarp();
        const int col = b0 + c0 + 4 * (lane & 7);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int row = 4 * j + (lane >> 3);
            const int m = m_base + row;
            const float4 v = *reinterpret_cast<const float4*>(stage + row * kStagePitch + 4 * (lane & 7));
            if (m >= M) continue;
            float* dst = C + (size_t)m * N + col;
            if (vec_ok && col + 4 <= N) {
                *reinterpret_cast<float4*>(dst) = v;
            } else {
                if (col < N) dst[0] = v.x;
                if (col + 1 < N) dst[1] = v.y;
                if (col + 2 < N) dst[2] = v.z;
                if (col + 3 < N) dst[3] = v.w;
            }
        }
        __syncwarp();                                                 // the block is free for the next 32 columns
    }
}

// One thread's row of a finished accumulator tile, BN columns from tensor memory at `taddr`,
// to row m of C (columns b0 ..).  Called by whole warps: the loads are warp-wide.
//   EPI = 0: C[m, n] = acc
//   EPI = 1: columns interleave gate and up; C[m, f] = up * silu(gate), C has N/2 columns.
//   ADD > 0: a second accumulator ADD columns further on is added to the first.
template <int BN, typename TC, int EPI, int ADD = 0>
__device__ __forceinline__ void drain_tile(uint32_t taddr, TC* __restrict__ C, int M, int N, int m, int b0) {
#pragma unroll 2
    for (int c0 = 0; c0 < BN; c0 += 16) {
        uint32_t r[16];
        tmem_ld16(taddr + c0, r);
        if constexpr (ADD > 0) {
            uint32_t r2[16];
            tmem_ld16(taddr + ADD + c0, r2);
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 16; ++q) r[q] = __float_as_uint(__uint_as_float(r[q]) + __uint_as_float(r2[q]));
        } else {
            tmem_ld_wait();
        }
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

}  // namespace
