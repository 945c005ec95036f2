// The tcgen05 matrix-product kernels for many rows (prompt portions): a persistent kernel
// with one block per SM and a pair kernel in which two SMs share a tile of 256 rows
// (cta_group::2).  Operands and conventions as in gemm_tcgen05.cu, which dispatches here.
#include <cuda.h>
#include <stdint.h>

#include "common.cuh"
#include "tma_maps.cuh"
#include "tcgen05_gemm.cuh"

namespace {

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
//
// ISSUERS = 2 (tile widths below 256, where one thread's rate of about one product every 80 ns,
// not the tensor core, sets the pace): a seventh warp issues too.  Each of the two threads issues
// half of every K block's products into an accumulator of its own (columns BN.. beside the
// first), and the epilogue adds the two.  Where four such accumulators do not fit into the 512
// columns, a tile's main loop waits for the epilogue of the tile before it.
constexpr int ACC_STRIDE = 256;          // TMEM columns between the two accumulators

template <int BN, int ISSUERS> constexpr int acc_buffers() { return 2 * ISSUERS * BN <= 512 ? 2 : 1; }

template <int BN, int STAGES, typename TC, int EPI, int ISSUERS>
__global__ void __launch_bounds__(160 + 32 * ISSUERS, 1)
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
            mbar_init(smem_u32(&empty_bar[s]), ISSUERS);   // one commit per issuing thread
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&acc_full[a]), ISSUERS);
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
    } else if ((warp == 1 || warp == 6) && lane == 0) {
        // ---------------- MMA issuer q (warp 1, and warp 6 when there are two)
        constexpr uint32_t idesc = make_idesc(BN);
        constexpr int NACC = acc_buffers<BN, ISSUERS>();
        constexpr int KPER = (BK / UMMA_K) / ISSUERS;      // products of a K block per issuing thread
        const int q = warp == 1 ? 0 : 1;
        uint32_t it = 0;
        int j = 0;                                         // tiles done by this block
        bool ok = true;
        for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, ++j) {
            const int acc = j % NACC;
            // the epilogue must have drained this accumulator (first use of each passes at once)
            if (j >= NACC && !mbar_wait(smem_u32(&acc_empty[acc]), ((j / NACC) - 1) & 1)) { ok = false; break; }
            tcgen05_fence_after();
            const uint32_t d = tmem_d + acc * ACC_STRIDE + q * BN;
            for (int i = 0; i < kb_total; ++i, ++it) {
                const int s = it % STAGES;
                if (!mbar_wait(smem_u32(&full_bar[s]), (it / STAGES) & 1)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t sa = tiles + s * stage_bytes<BN>();
                const uint32_t sb_ = sa + BM * BK * 2;
#pragma unroll
                for (int k = q * KPER; k < (q + 1) * KPER; ++k)
                    tcgen05_mma_bf16(d, make_smem_desc(sa + k * UMMA_K * 2), make_smem_desc(sb_ + k * UMMA_K * 2),
                                     idesc, (i > 0 || k > q * KPER) ? 1u : 0u);
                tcgen05_commit(smem_u32(&empty_bar[s]));
            }
            if (!ok) break;
            tcgen05_commit(smem_u32(&acc_full[acc]));
        }
        if (!ok) {
            atomicExch(status, 2);
            atomicExch(&abort_flag, 1);
        }
    } else if (warp >= 2 && warp < 6) {
        // ---------------- epilogue: warp w owns TMEM lanes 32*(w%4) .. +31
        sb::pdl_wait();                                    // C may still be read by an earlier kernel until now
        constexpr int NACC = acc_buffers<BN, ISSUERS>();
        const int quarter = warp & 3;
        int j = 0;
        for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, ++j) {
            const int acc = j % NACC;
            bool good = mbar_wait(smem_u32(&acc_full[acc]), (j / NACC) & 1);
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
            if constexpr (sizeof(TC) == 4 && EPI == 0 && BN % 32 == 0) {
                float* stage = reinterpret_cast<float*>(smem_raw + (tiles - smem_u32(smem_raw)) +
                                                        STAGES * stage_bytes<BN>() + quarter * kStageBytesPerWarp);
                drain_tile_f32_staged<BN, (ISSUERS == 2 ? BN : 0)>(taddr, reinterpret_cast<float*>(C), M, N,
                                                                    a0 + quarter * 32, lane, b0, stage);
            } else {
                drain_tile<BN, TC, EPI, (ISSUERS == 2 ? BN : 0)>(taddr, C, M, N, m, b0);
            }
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
__global__ void __launch_bounds__(192, 1)
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
            if constexpr (sizeof(TC) == 4 && EPI == 0 && BN % 32 == 0) {
                float* stage = reinterpret_cast<float*>(smem_raw + (tiles - smem_u32(smem_raw)) + STAGES * SB +
                                                        quarter * kStageBytesPerWarp);
                drain_tile_f32_staged<BN>(taddr, reinterpret_cast<float*>(C), M, N, a0 + quarter * 32, lane, b0, stage);
            } else {
                drain_tile<BN, TC, EPI>(taddr, C, M, N, m, b0);
            }
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

// ----------------------------------------------------------------------------- pair kernel, equal shares
// The pair kernel with the work dealt in equal shares of (tile, K block) units instead of whole
// tiles: pair p takes units [total * p / pairs, total * (p + 1) / pairs) of the tiles' K blocks
// laid end to end (tiles in the order of the pair kernel, row index fastest).  Where a share
// ends inside a tile, the tile's K range is finished by the next pair.  Nothing is handed over
// between pairs: the output is float32 partial sums [parts, M, N], as the products with few
// rows write them, and the consumer (the norm that folds a branch into the residual) adds the
// parts in their fixed order.  A piece of a tile that starts at K block 0 writes part 0; a piece
// that starts later writes part (its pair - the pair that owns the tile's first unit); the piece
// that ends a tile also writes zeros to the parts the tile did not use.
// Why: at 2,048 rows a narrow projection has 80 tiles of 256 x 256 for 74 pairs: whole tiles take
// two waves of which the second is 8 % full; equal shares take 1.08 waves' worth of time.
struct Piece {
    int tile, kb0, kb1, part;
    bool ends_tile;
};
struct PieceWalk {
    long long u, u_end, total;
    int kb_total, pair, n_pairs;
    __device__ PieceWalk(int pair_, int n_pairs_, int n_tiles, int kb_total_)
        : total((long long)n_tiles * kb_total_), kb_total(kb_total_), pair(pair_), n_pairs(n_pairs_) {
        u = total * pair / n_pairs;
        u_end = total * (pair + 1) / n_pairs;
    }
    // the next piece of this pair's share; false when the share is done
    __device__ bool next(Piece& pc) {
        if (u >= u_end) return false;
        pc.tile = (int)(u / kb_total);
        pc.kb0 = (int)(u - (long long)pc.tile * kb_total);
        const long long left = u_end - u;
        pc.kb1 = (int)min((long long)kb_total, pc.kb0 + left);
        pc.ends_tile = pc.kb1 == kb_total;
        if (pc.kb0 == 0) {
            pc.part = 0;
        } else {
            // the pair that owns unit x is ((x + 1) * pairs - 1) / total
            const long long first = (long long)pc.tile * kb_total;
            pc.part = pair - (int)(((first + 1) * n_pairs - 1) / total);
        }
        u += pc.kb1 - pc.kb0;
        return true;
    }
};

template <int STAGES>
__global__ void __launch_bounds__(192, 1)
gemm_tcgen05_pair_shares_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                                float* __restrict__ C, int M, int N, int K, int tiles_m, int tiles_n, int parts,
                                int* __restrict__ status) {
    constexpr int BN = 256;
    constexpr int ACC_COLS = 256;
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
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(2 * ACC_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();                                    // both blocks' barriers exist from here on
    tcgen05_fence_after();
    const uint32_t tmem_d = tmem_base_slot;
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
        uint32_t it = 0;
        bool waited = false, ok = true;
        PieceWalk walk(pair, n_pairs, n_tiles, kb_total);
        Piece pc;
        while (ok && walk.next(pc)) {
            const int a0 = (pc.tile % tiles_m) * 256 + (int)rank * BM;
            const int b0 = (pc.tile / tiles_m) * BN + (int)rank * (BN / 2);
            int i = pc.kb0;
            if (!waited) {
                // weights first (nobody writes them), the activations after the wait on the previous kernel
                const int ahead = min(pc.kb1 - pc.kb0, STAGES);
                for (int q = 0; q < ahead; ++q) {
                    if (rank == 0) mbar_arrive_expect_tx(smem_u32(&full_bar[q]), 2 * SB);
                    tma_load_2d_pair(tiles + q * SB + BM * BK * 2, &tma_b, map_to_cta(smem_u32(&full_bar[q]), 0),
                                     (pc.kb0 + q) * BK, b0);
                }
                sb::pdl_wait();
                waited = true;
                for (int q = 0; q < ahead; ++q)
                    tma_load_2d_pair(tiles + q * SB, &tma_a, map_to_cta(smem_u32(&full_bar[q]), 0), (pc.kb0 + q) * BK, a0);
                i = pc.kb0 + ahead;
                it = ahead;
            }
            for (; i < pc.kb1 && ok; ++i, ++it) {
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
        PieceWalk walk(pair, n_pairs, n_tiles, kb_total);
        Piece pc;
        for (; ok && walk.next(pc); ++j) {
            const int acc = j & 1;
            if (j >= 2 && !mbar_wait_cluster(smem_u32(&acc_empty[acc]), ((j >> 1) - 1) & 1)) { ok = false; break; }
            tcgen05_fence_after();
            const uint32_t d = tmem_d + acc * ACC_COLS;
            for (int i = pc.kb0; i < pc.kb1; ++i, ++it) {
                const int s = it % STAGES;
                if (!mbar_wait(smem_u32(&full_bar[s]), (it / STAGES) & 1)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t sa = tiles + s * SB;
                const uint32_t sb_ = sa + BM * BK * 2;
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    tcgen05_mma_bf16_pair(d, make_smem_desc(sa + k * UMMA_K * 2), make_smem_desc(sb_ + k * UMMA_K * 2),
                                          idesc, (i > pc.kb0 || k > 0) ? 1u : 0u);
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
        const size_t part_stride = (size_t)M * N;
        int j = 0;
        PieceWalk walk(pair, n_pairs, n_tiles, kb_total);
        Piece pc;
        for (; walk.next(pc); ++j) {
            const int acc = j & 1;
            bool good = mbar_wait(smem_u32(&acc_full[acc]), (j >> 1) & 1);
            if (*((volatile int*)&abort_flag)) good = false;
            good = __all_sync(0xffffffffu, good);
            if (!good) {
                if (lane == 0) { atomicExch(status, 3); atomicExch(&abort_flag, 1); }
                break;
            }
            tcgen05_fence_after();
            const int a0 = (pc.tile % tiles_m) * 256 + (int)rank * BM, b0 = (pc.tile / tiles_m) * BN;
            const int m = a0 + quarter * 32 + lane;
            const uint32_t taddr = tmem_d + acc * ACC_COLS + (static_cast<uint32_t>(quarter * 32) << 16);
            float* stage = reinterpret_cast<float*>(smem_raw + (tiles - smem_u32(smem_raw)) + STAGES * SB +
                                                    quarter * kStageBytesPerWarp);
            drain_tile_f32_staged<BN>(taddr, C + (size_t)pc.part * part_stride, M, N, a0 + quarter * 32, lane, b0, stage);
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_remote(map_to_cta(smem_u32(&acc_empty[acc]), 0));
            if (pc.ends_tile && m < M) {
                // the parts this tile did not use count as zero
                for (int z = pc.part + 1; z < parts; ++z) {
                    float* row = C + (size_t)z * part_stride + (size_t)m * N + b0;
                    const int cols = min(BN, N - b0);
                    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0 && cols % 4 == 0) {
                        for (int c = 0; c < cols; c += 4) *reinterpret_cast<float4*>(row + c) = make_float4(0.f, 0.f, 0.f, 0.f);
                    } else {
                        for (int c = 0; c < cols; ++c) row[c] = 0.f;
                    }
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(2 * ACC_COLS)
                     : "memory");
    }
}

using sb::get_map;

template <int BN, int STAGES, typename TC, int EPI, int ISSUERS>
int launch_persistent(const CUtensorMap& ma, const CUtensorMap& mb, void* C, int M, int N, int K, int* status,
                      cudaStream_t stream) {
    auto kernel = gemm_tcgen05_persistent_kernel<BN, STAGES, TC, EPI, ISSUERS>;
    constexpr int smem = STAGES * stage_bytes<BN>() + 1024 + kStageBytes;
    static sb::OncePerDevice once_per_device;
    bool& configured = once_per_device.flag();
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
    sb::launch(kernel, dim3(blocks), dim3(160 + 32 * ISSUERS), smem, stream, ma, mb, (TC*)C, M, N, K, tiles_m, tiles_n,
               status);
    return 0;
}

template <int BN, int STAGES, typename TC, int EPI>
int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, void* C, int M, int N, int K, int* status,
                cudaStream_t stream) {
    auto kernel = gemm_tcgen05_pair_kernel<BN, STAGES, TC, EPI>;
    constexpr int smem = STAGES * pair_stage_bytes<BN>() + 1024 + kStageBytes;
    static sb::OncePerDevice once_per_device;
    bool& configured = once_per_device.flag();
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
    sb::launch_cluster(kernel, dim3(2 * pairs), dim3(192), smem, stream, dim3(2, 1, 1), ma, mb, (TC*)C, M, N, K, tiles_m,
                       tiles_n, status);
    return 0;
}

// Tile widths of the pair kernel and their ring depths.
#define SB_PAIR_WIDTHS(X) X(256) X(192) X(160) X(128)
constexpr int pair_stages(int bn) {
    const int s = (222 * 1024 - kStageBytes) / (BM * BK * 2 + (bn / 2) * BK * 2);
    return s > 8 ? 8 : s;
}

// Tile widths of the persistent kernel, and the ring depth that fits in shared memory for each.
#define SB_PERSISTENT_WIDTHS(X) X(256) X(160) X(128)
constexpr int persistent_stages(int bn) {
    const int s = (222 * 1024 - kStageBytes) / (BM * BK * 2 + bn * BK * 2);
    return s > 6 ? 6 : s;
}

// Tile width for many rows.  Blocks take tiles in a fixed stride, so the time is the number
// of waves times the time of one tile: choose the width for which that is least.  A tile's time
// per K block was measured at 2,048 x 2,560 x 9,728 (clocks: 659 at width 128, 697 at 160, 780 at
// 256): narrow tiles save far less than their width, because the 128 rows of A are fetched for
// each of them and shared memory, not the tensor core, sets the pace.
static int pick_bn(int M, int N, int num_sms) {
    const int tiles_m = (M + BM - 1) / BM;
    int best = 256;
    double best_cost = -1.0;
#define SB_CONSIDER(bn) { \
        const long tiles = (long)tiles_m * ((N + bn - 1) / bn); \
        const double cost = (double)((tiles + num_sms - 1) / num_sms) * (540.0 + 0.94 * bn); \
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = bn; } }
    SB_PERSISTENT_WIDTHS(SB_CONSIDER)
#undef SB_CONSIDER
    return best;
}

// Two issuing threads: at width 128 always (four accumulators fit, the epilogue still overlaps
// the next tile), at 160 only without the SiLU*mul epilogue (one tile at a time there: with the
// heavier epilogue exposed, gate/up lost 4 %; o and down gain 1 to 10 %).
constexpr int row_issuers(int bn, int epi) { return bn == 128 || (bn == 160 && epi == 0) ? 2 : 1; }

template <typename TC>
int many_rows(const void* A, const void* W, void* C, int M, int N, int K, int* status, int variant, int epi,
              cudaStream_t stream) {
    CUtensorMap ma, mb;
    // The pair kernel is chosen for 4,096 rows and more (measured on the 4B shape: at 8,192 rows
    // the narrow projections gain a fifth and the wide ones 0 to 2 %; at 2,048 rows the wide ones
    // lose 3 %, because both kernels are then bound by how the tiles divide among the SMs), or
    // forced with variant 1000 + width.
    const bool many_waves = M >= 4096 && (long)((M + 255) / 256) * ((N + 255) / 256) >= 4L * 74;
    if ((variant >= 1128 && variant <= 1256) || (variant == 0 && M > 256 && many_waves)) {
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
    {
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
        if (bn == BN_) return epi == 1 ? launch_persistent<BN_, persistent_stages(BN_), TC, 1, row_issuers(BN_, 1)>(ma, mb, C, M, N, K, status, stream) \
                                       : launch_persistent<BN_, persistent_stages(BN_), TC, 0, row_issuers(BN_, 0)>(ma, mb, C, M, N, K, status, stream);
        SB_PERSISTENT_WIDTHS(SB_TRY)
#undef SB_TRY
        sb_set_error("gemm_tcgen05: no persistent kernel of width %d", bn);
        return SB_ERR_ARG;
    }
}


// How many pairs of blocks the GPU holds at once for the equal-shares kernel (0 if none fits).
int shares_pairs() {
    static sb::OncePerDevice once_per_device;
    static int max_pairs = 0;
    bool& configured = once_per_device.flag();
    if (!configured) {
        auto kernel = gemm_tcgen05_pair_shares_kernel<pair_stages(256)>;
        constexpr int smem = pair_stages(256) * pair_stage_bytes<256>() + 1024 + kStageBytes;
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return 0;
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
        if (cudaOccupancyMaxActiveClusters(&max_pairs, kernel, &cfg) != cudaSuccess) max_pairs = 0;
        configured = true;
    }
    return max_pairs;
}

// Parts that the equal-shares kernel writes for this shape with `pairs` pairs: a tile of kb_total
// K blocks is cut by at most ceil((kb_total - 1) / smallest share) share ends.
int shares_parts(int M, int N, int K, int pairs) {
    const long long n_tiles = (long long)((M + 255) / 256) * ((N + 255) / 256);
    const int kb_total = (K + BK - 1) / BK;
    if (pairs < 1 || n_tiles < 1) return 0;
    const long long smallest = n_tiles * kb_total / pairs;
    if (smallest < 1) return 0;
    return (int)((kb_total - 1 + smallest - 1) / smallest) + 1;
}

}  // namespace

namespace sb {
// The pair kernel in equal shares of K blocks: float32 partial sums C [parts, M, N] with
// parts = gemm_tcgen05_shares_parts(M, N, K) (0: this shape is not served).
int gemm_tcgen05_shares_parts(int M, int N, int K) {
    if (M <= 256 || N < 256 || K < BK) return 0;
    const long long n_tiles = (long long)((M + 255) / 256) * ((N + 255) / 256);
    const int pairs = (int)min((long long)shares_pairs(), n_tiles * ((K + BK - 1) / BK));
    const int parts = shares_parts(M, N, K, pairs);
    return parts >= 1 && parts <= 4 ? parts : 0;
}

int gemm_tcgen05_shares(const void* A, const void* W, float* C, int M, int N, int K, int* status,
                        cudaStream_t stream) {
    const int parts = gemm_tcgen05_shares_parts(M, N, K);
    if (parts == 0) {
        sb_set_error("gemm_tcgen05: the equal-shares kernel does not serve M=%d N=%d K=%d", M, N, K);
        return SB_ERR_ARG;
    }
    CUtensorMap ma, mb;
    if (!get_map(&ma, A, M, K, BM) || !get_map(&mb, W, N, K, 128)) {
        sb_set_error("gemm_tcgen05: cuTensorMapEncodeTiled failed (M=%d N=%d K=%d)", M, N, K);
        return SB_ERR_ARG;
    }
    const int tiles_m = (M + 255) / 256, tiles_n = (N + 255) / 256;
    const long long units = (long long)tiles_m * tiles_n * ((K + BK - 1) / BK);
    const int pairs = (int)min((long long)shares_pairs(), units);
    auto kernel = gemm_tcgen05_pair_shares_kernel<pair_stages(256)>;
    constexpr int smem = pair_stages(256) * pair_stage_bytes<256>() + 1024 + kStageBytes;
    sb::launch_cluster(kernel, dim3(2 * pairs), dim3(192), smem, stream, dim3(2, 1, 1), ma, mb, C, M, N, K, tiles_m,
                       tiles_n, parts, status);
    return 0;
}
}  // namespace sb

namespace sb {
// Products with many rows (prompt portions), no K split, N >= 128: the persistent kernel or,
// from 4,096 rows, the pair kernel.  `variant` as in sb_gemm_tcgen05.
int gemm_tcgen05_many_rows(const void* A, const void* W, void* C, int M, int N, int K, int c_dtype, int* status,
                           int variant, int epi, cudaStream_t stream) {
    return c_dtype == SB_BF16 ? many_rows<__nv_bfloat16>(A, W, C, M, N, K, status, variant, epi, stream)
                              : many_rows<float>(A, W, C, M, N, K, status, variant, epi, stream);
}
}  // namespace sb
