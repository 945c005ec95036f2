// Paged causal GQA attention of prompt portions on the 5th-generation tensor cores.
//
// One block per (query tile, KV head).  A query tile is 128 accumulator rows: floor(128/G)
// consecutive tokens of ONE request times the G query heads of the KV head; row r is
// TMEM lane r and belongs to thread r for the softmax.  Keys and values come from the
// pages in tiles of 64 keys, one TMA box per (page, 64-dim panel) into 128-byte swizzled
// shared memory, double buffered.  Per key tile:
//   S = Q K^T          tcgen05.mma kind::f16, A and B from shared memory (K-major), S in TMEM
//   softmax            thread r reads row r of S (tcgen05.ld), masks by position, keeps the
//                      running maximum and sum in float32 (exp2f), and writes the weights
//                      back to TMEM as TWO bfloat16 terms, p = hi + lo (tcgen05.st)
//   O += P V           tcgen05.mma with A = P from TMEM (hi, then lo on top) and B = V from
//                      shared memory, MN-major (keys are the K dimension); O stays in TMEM.
// The weights of tile i are written over the scores of tile i (same TMEM columns), there
// are two such S/P buffers.  Three more warps only issue work: one the score products, one the
// P.V products (a thread issues a product about every 80 ns whatever its size, so the two
// chains have a thread each), one the TMA copies (one box per lane).  QK(i+1) goes out before
// the softmax warps have finished tile i and PV(i) as soon as they have, so the tensor core
// works on tile i+1's scores and tile i-1's product during tile i's softmax.
// O is rescaled lazily: the exponent's reference maximum of a row only moves when the row
// maximum grows by more than 2^8, and then the row of O in TMEM is multiplied once.
// Tiles whose keys every row of the block may see skip the position masks.
// Tiles are found on the device from the step's request offsets, and queries read their
// request's earlier portions from the pages, exactly as the mma.sync tile kernel does.
//
// Whole pages are copied, so a tile's buffer may hold slots outside the keys [lo, hi) a
// block may see (slots past the row's length, before its window, or of the null page).
// Their scores are replaced (not multiplied) by -inf and their V rows are zeroed in
// shared memory before the product, so whatever a previous owner left there cannot reach
// the result.
//
// head_dim 64 or 128, any group size up to 128 (128 / G whole tokens a tile, the rows left over idle),
// page sizes 16, 32 or 64.  Every wait on
// an mbarrier is bounded; a give-up sets *status, and the block still frees its TMEM.
#include <cuda.h>
#include <math.h>
#include <stdint.h>

#include "common.cuh"
#include "tma_maps.cuh"

using namespace sb;
typedef __nv_bfloat16 bf16;

namespace {

constexpr int ROWS = 128;            // accumulator rows = threads
constexpr int KTILE = 64;            // keys per tile
constexpr float LOG2E = 1.4426950408889634f;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

// TMEM columns of one block (256 allocated).  S/P buffer b occupies 64 columns at 64*b:
// first the float32 scores of a tile, then (written over them by the softmax) the weights:
// the high bfloat16 terms in its columns 0..31 (two keys per column), the low terms in 32..63.
constexpr int COL_SP = 0;
constexpr int COL_O = 128;           // D columns: the output accumulator, float32
constexpr float RESCALE_LOG2 = 8.0f; // a row's reference maximum moves when its maximum grew by 2^8

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
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d), "l"(da), "l"(db), "r"(idesc), "r"(acc)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a, uint64_t db, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d), "r"(a), "l"(db), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory descriptors, 128-byte swizzle, descriptor version 1.
//   K-major operand (rows of 128 bytes, the contraction dim contiguous): 8-row groups 1024 B apart.
//   MN-major operand (the contraction dim runs over rows): `lbo16` = distance (in 16 B) between
//   blocks of 64 elements of the non-contracted dim, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
    const uint32_t lo = ((addr & 0x3FFFFu) >> 4) | (1u << 16);
    const uint32_t hi = 64u | (1u << 14) | (2u << 29);
    return (static_cast<uint64_t>(hi) << 32) | lo;
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr, uint32_t lbo16) {
    const uint32_t lo = ((addr & 0x3FFFFu) >> 4) | (lbo16 << 16);
    const uint32_t hi = 64u | (1u << 14) | (2u << 29);
    return (static_cast<uint64_t>(hi) << 32) | lo;
}
// Instruction descriptor: D float32, A and B bfloat16, A K-major, M = 128.
__host__ __device__ constexpr uint32_t make_idesc(int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) |
           (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(ROWS >> 4) << 24);
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int D> constexpr int q_bytes() { return ROWS * D * 2; }
template <int D> constexpr int kv_bytes() { return KTILE * D * 2; }          // one of K or V, one buffer
template <int D> constexpr int smem_bytes() { return q_bytes<D>() + 4 * kv_bytes<D>() + 1024; }

// ----------------------------------------------------------------------------- the kernel
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// four softmax warps, the warp that issues the score products, the copy-issuing warp, the warp
// that issues the P.V products
constexpr int THREADS = ROWS + 96;

template <int D>
__global__ void __launch_bounds__(THREADS)
attn_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap tma_k, const __grid_constant__ CUtensorMap tma_v,
                            bf16* __restrict__ out, const bf16* __restrict__ q,
                            const int* __restrict__ block_table, int table_width,
                            const int* __restrict__ seq_starts, const int* __restrict__ seq_rows,
                            const int* __restrict__ seq_first_pos, int R, int Hq, int Hkv, int BS, int window,
                            float scale_log2, int* __restrict__ status) {
    constexpr int PANELS = D / 64;                         // 64-dim panels of 128-byte rows
    constexpr int PANEL_Q = ROWS * 128;                    // bytes of one Q panel
    constexpr int PANEL_KV = KTILE * 128;                  // bytes of one K or V panel
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t k_full[2], v_full[2];
    __shared__ __align__(8) uint64_t s_full[2], p_ready[2], v_free[2], pv_full;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5;
    const bool issuer = warp == 4;                          // S = Q K^T
    const bool copier = warp == 5;
    const bool pv_issuer = warp == 6;                       // O += P V
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t q_s = base;
    const uint32_t k_s = q_s + q_bytes<D>();               // 2 buffers
    const uint32_t v_s = k_s + 2 * kv_bytes<D>();          // 2 buffers
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    int* stab = reinterpret_cast<int*>(gen_base + q_bytes<D>() + 4 * kv_bytes<D>());

    const int G = Hq / Hkv;
    const int bs_log2 = 31 - __clz(BS);
    const int TQ = ROWS / G;
    const int kh = blockIdx.x % Hkv;          // the KV heads of a query tile are neighbours in launch order

    if (tid == 0) {
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&k_full[b]), 1);
            mbar_init(smem_u32(&v_full[b]), 1);
            mbar_init(smem_u32(&s_full[b]), 1);
            mbar_init(smem_u32(&p_ready[b]), ROWS);
            mbar_init(smem_u32(&v_free[b]), 1);
        }
        mbar_init(smem_u32(&pv_full), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (issuer) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_slot)), "r"(256) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    sb::pdl_launch_dependents();
    sb::pdl_wait();                                        // q and the pages are written by earlier kernels

    // ---- which request, which tile.  Blocks are handed out in launch order and later tiles of
    // a prompt have more keys, so the order is reversed: the longest tiles (of every KV head) start
    // first and the short ones fill the tail.  With the KV head as the slow index instead, the
    // longest tiles of the last heads started when half of the SMs had nothing else left: 93 us
    // against 66 for one prompt of 2,048 tokens.
    int tile = gridDim.x / Hkv - 1 - blockIdx.x / Hkv, r = 0, t0 = 0, n_tok = 0;
    for (; r < R; ++r) {
        const int a = seq_starts[r], len = seq_starts[r + 1] - a;
        const int tiles = (len + TQ - 1) / TQ;
        if (tile < tiles) {
            t0 = a + tile * TQ;
            n_tok = min(TQ, len - tile * TQ);
            break;
        }
        tile -= tiles;
    }
    const bool active = r < R;
    int first_pos = 0, lo = 0, hi = 0, tile_begin = 0, n_tiles = 0, table_base = 0, table_count = 0;
    if (active) {
        first_pos = seq_first_pos[r] + tile * TQ;
        hi = first_pos + n_tok;
        lo = (window > 0 && first_pos + 1 > window) ? first_pos + 1 - window : 0;
        tile_begin = lo / KTILE;
        n_tiles = (hi + KTILE - 1) / KTILE - tile_begin;
        table_base = lo >> bs_log2;
        table_count = ((hi - 1) >> bs_log2) - table_base + 1;
        const int* table = block_table + (size_t)seq_rows[r] * table_width;
        for (int i = tid; i < table_count; i += THREADS) stab[i] = table[table_base + i];
        if (tid < ROWS) {
            // ---- Q: thread r copies row r (token r / G, head r % G) into the swizzled panels
            const int tok = tid / G, g = tid - tok * G;
            const bool valid = tok < n_tok;
            const uint4* src =
                reinterpret_cast<const uint4*>(q + ((size_t)(t0 + (valid ? tok : 0)) * Hq + kh * G + g) * D);
#pragma unroll
            for (int c = 0; c < D / 8; ++c) {
                const uint4 v = valid ? __ldg(src + c) : make_uint4(0, 0, 0, 0);
                const int panel = c >> 3, cc = c & 7;
                uint8_t* dst = gen_base + panel * PANEL_Q + tid * 128 + ((cc ^ (tid & 7)) << 4);
                *reinterpret_cast<uint4*>(dst) = v;
            }
        }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // Q is read by the tensor core (async proxy)
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_slot;
    // rows of this block see every key of a tile when it ends at or before the first query's
    // position and starts at or after the last query's window start
    const int last_qlo = (window > 0 && hi > window) ? hi - window : 0;

    if (copier) {
        // =============================================================== the copy-issuing warp
        // Tile t's keys go to K buffer t&1 once QK(t-2) has read it, its values to V buffer t&1
        // once PV(t-2) has.  Each lane issues one box (page, panel); lane 0 arms the barrier.
        if (active) {
            const int lane = tid & 31;
            const int pages = KTILE >> bs_log2;
            const int n_ops = pages * PANELS;               // at most 8
            bool ok = true;
            for (int t = 0; t < n_tiles && ok; ++t) {
                const int b = t & 1;
                const int pg = lane / PANELS, p = lane - pg * PANELS;
                int y = 0;
                if (lane < n_ops) {
                    const int logical = (((tile_begin + t) * KTILE) >> bs_log2) + pg - table_base;
                    const int phys = (logical >= 0 && logical < table_count) ? stab[logical] : 0;
                    y = (phys * Hkv + kh) * BS;
                }
                const uint32_t off = b * kv_bytes<D>() + p * PANEL_KV + pg * BS * 128;
                // ---- keys
                if (t >= 2) {
                    bool got = mbar_wait(smem_u32(&s_full[b]), ((t - 2) >> 1) & 1);
                    got = __all_sync(0xffffffffu, got);
                    if (!got) { ok = false; if (lane == 0) { atomicExch(status, 17); atomicExch(&abort_flag, 1); } break; }
                }
                if (lane == 0) mbar_arrive_expect_tx(smem_u32(&k_full[b]), kv_bytes<D>());
                __syncwarp();
                if (lane < n_ops) tma_load_2d(k_s + off, &tma_k, smem_u32(&k_full[b]), p * 64, y);
                // ---- values
                // (a barrier of its own per buffer: pv_full advances every tile and this warp runs
                // two tiles ahead, so a parity wait on it could fall two phases behind)
                if (t >= 2) {
                    bool got = mbar_wait(smem_u32(&v_free[b]), ((t - 2) >> 1) & 1);
                    got = __all_sync(0xffffffffu, got);
                    if (!got) { ok = false; if (lane == 0) { atomicExch(status, 18); atomicExch(&abort_flag, 1); } break; }
                }
                if (lane == 0) mbar_arrive_expect_tx(smem_u32(&v_full[b]), kv_bytes<D>());
                __syncwarp();
                if (lane < n_ops) tma_load_2d(v_s + off, &tma_v, smem_u32(&v_full[b]), p * 64, y);
            }
        }
    } else if (issuer) {
        // =============================================================== the warp that issues Q K^T
        // One thread issues a tcgen05.mma about every 80 ns whatever its size (measured), and a
        // key tile needs 8 products for the scores and 8 for P.V: issued by one thread they, not
        // the tensor core, set the pace.  So scores and P.V have an issuing thread each; they
        // write different accumulators and meet only through barriers.
        if (active && (tid & 31) == 0) {
            constexpr uint32_t idesc_qk = make_idesc(KTILE, false);
            const uint64_t dq = desc_kmajor(q_s), dk = desc_kmajor(k_s);
            for (int i = 0; i < n_tiles; ++i) {
                const int b = i & 1;
                if (!mbar_wait(smem_u32(&k_full[b]), (i >> 1) & 1)) { atomicExch(status, 11); atomicExch(&abort_flag, 1); break; }
                // S[b] still holds P(i-2), the A operand of PV(i-2).  The tensor core orders
                // products by their accumulators only, not by an operand read from tensor memory,
                // so PV(i-2) must have COMPLETED before its weights are overwritten.  v_free[b]
                // completes once per product on buffer b, and the next one cannot come before the
                // scores issued here: the wait is never two phases behind.
                if (i >= 2 && !mbar_wait(smem_u32(&v_free[b]), ((i - 2) >> 1) & 1)) {
                    atomicExch(status, 13); atomicExch(&abort_flag, 1); break;
                }
                if (*((volatile int*)&abort_flag)) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    // the start address sits in the low bits of a descriptor in units of 16 bytes
                    const uint32_t pq = ((kk >> 2) * PANEL_Q + (kk & 3) * 32) >> 4;
                    const uint32_t pk = (b * kv_bytes<D>() + (kk >> 2) * PANEL_KV + (kk & 3) * 32) >> 4;
                    mma_ss(tmem + COL_SP + 64 * b, dq + pq, dk + pk, idesc_qk, kk > 0 ? 1u : 0u);
                }
                tc_commit(smem_u32(&s_full[b]));
            }
        }
    } else if (pv_issuer) {
        // =============================================================== the warp that issues P V
        if (active && (tid & 31) == 0) {
            constexpr uint32_t idesc_pv = make_idesc(D, true);
            const uint64_t dv = desc_mnmajor(v_s, PANEL_KV >> 4);
            for (int i = 0; i < n_tiles; ++i) {
                const int b = i & 1;
                // the softmax warps have written P(i) (and zeroed unseen V rows); V(i) has landed
                if (!mbar_wait(smem_u32(&p_ready[b]), (i >> 1) & 1)) { atomicExch(status, 16); atomicExch(&abort_flag, 1); break; }
                if (!mbar_wait(smem_u32(&v_full[b]), (i >> 1) & 1)) { atomicExch(status, 14); atomicExch(&abort_flag, 1); break; }
                if (*((volatile int*)&abort_flag)) break;
                tc_fence_after();
                const uint32_t pbase = tmem + COL_SP + 64 * b;
#pragma unroll
                for (int j = 0; j < KTILE / 16; ++j)
                    mma_ts(tmem + COL_O, pbase + j * 8, dv + ((b * kv_bytes<D>() + j * 2048) >> 4), idesc_pv,
                           (i > 0 || j > 0) ? 1u : 0u);
#pragma unroll
                for (int j = 0; j < KTILE / 16; ++j)
                    mma_ts(tmem + COL_O, pbase + 32 + j * 8, dv + ((b * kv_bytes<D>() + j * 2048) >> 4), idesc_pv, 1u);
                tc_commit(smem_u32(&pv_full));
                tc_commit(smem_u32(&v_free[b]));            // V buffer b and S/P buffer b may be reused
            }
        }
    } else if (active) {
        // =============================================================== the softmax warps
        float m_ref = -INFINITY, l_run = 0.f;
        const int tok = tid / G, g = tid - tok * G;
        const int qpos = tok < n_tok ? first_pos + tok : -1;   // rows past the tile see no key
        const int qlo = (window > 0 && qpos + 1 > window) ? qpos + 1 - window : 0;
        const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
        bool ok = true;
        for (int i = 0; i < n_tiles; ++i) {
            const int b = i & 1;
            const int tile_start = (tile_begin + i) * KTILE;
            bool got = mbar_wait(smem_u32(&s_full[b]), (i >> 1) & 1);
            if (*((volatile int*)&abort_flag)) got = false;
            got = __all_sync(0xffffffffu, got);
            if (!got) { ok = false; if ((tid & 31) == 0) { atomicExch(status, 12); atomicExch(&abort_flag, 1); } break; }
            tc_fence_after();

            float s[64];
            {
                uint32_t raw[32];
                tmem_ld32(lane_base + COL_SP + 64 * b, raw);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) s[j] = __uint_as_float(raw[j]);
                tmem_ld32(lane_base + COL_SP + 64 * b + 32, raw);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) s[32 + j] = __uint_as_float(raw[j]);
            }
            // position masks only where some row of the block cannot see some key of the tile;
            // rows past the tile (qpos = -1) are masked by the same test
            const bool masked = tile_start + KTILE - 1 > first_pos || tile_start < last_qlo || n_tok < TQ;
            if (masked) {
#pragma unroll
                for (int j = 0; j < 64; ++j) {
                    const int kpos = tile_start + j;
                    s[j] = (kpos <= qpos && kpos >= qlo) ? s[j] : -INFINITY;
                }
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < 64; j += 4) {
                mx4[0] = fmaxf(mx4[0], s[j]);
                mx4[1] = fmaxf(mx4[1], s[j + 1]);
                mx4[2] = fmaxf(mx4[2], s[j + 2]);
                mx4[3] = fmaxf(mx4[3], s[j + 3]);
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            // lazy rescale: move the reference maximum only when the row maximum outgrew it
            const bool grow = mx > -INFINITY && (m_ref == -INFINITY || (mx - m_ref) * scale_log2 > RESCALE_LOG2);
            if (__any_sync(0xffffffffu, grow)) {
                float alpha = 1.0f;
                if (grow) {
                    alpha = m_ref == -INFINITY ? 0.f : exp2f((m_ref - mx) * scale_log2);
                    m_ref = mx;
                    l_run *= alpha;
                }
                if (i > 0) {
                    // O of the tiles before this one is complete once PV(i-1) is
                    bool done = mbar_wait(smem_u32(&pv_full), (i - 1) & 1);
                    done = __all_sync(0xffffffffu, done);
                    if (!done) { ok = false; if ((tid & 31) == 0) { atomicExch(status, 13); atomicExch(&abort_flag, 1); } break; }
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < D; c += 32) {
                        uint32_t ov[32];
                        tmem_ld32(lane_base + COL_O + c, ov);
                        tmem_ld_wait();
                        uint32_t w0[16], w1[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            w0[j] = __float_as_uint(__uint_as_float(ov[j]) * alpha);
                            w1[j] = __float_as_uint(__uint_as_float(ov[16 + j]) * alpha);
                        }
                        tmem_st16(lane_base + COL_O + c, w0);
                        tmem_st16(lane_base + COL_O + c + 16, w1);
                    }
                }
            }
            // p = 2^((s - m) * scale) as one multiply-add and one ex2; masked scores are -inf -> 0
            const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref * scale_log2;
            float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < KTILE; c += 32) {
                uint32_t ph[16], pl[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const float p0 = ex2_approx(fmaf(s[c + 2 * j], scale_log2, neg_m));
                    const float p1 = ex2_approx(fmaf(s[c + 2 * j + 1], scale_log2, neg_m));
                    l4[j & 3] += p0 + p1;
                    const uint32_t h = pack_bf16(p0, p1);
                    ph[j] = h;
                    pl[j] = pack_bf16(p0 - __uint_as_float(h << 16), p1 - __uint_as_float(h & 0xffff0000u));
                }
                // over the scores of this very row: all 64 were read into registers above
                tmem_st16(lane_base + COL_SP + 64 * b + (c >> 1), ph);
                tmem_st16(lane_base + COL_SP + 64 * b + 32 + (c >> 1), pl);
            }
            l_run += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            tmem_st_wait();
            // slots of this tile outside [lo, hi): zero their V rows (thread j < 64 owns key j)
            if (tile_start < lo || tile_start + KTILE > hi) {
                bool landed = mbar_wait(smem_u32(&v_full[b]), (i >> 1) & 1);
                landed = __all_sync(0xffffffffu, landed);
                if (!landed) { ok = false; if ((tid & 31) == 0) { atomicExch(status, 14); atomicExch(&abort_flag, 1); } break; }
                if (tid < KTILE) {
                    const int kpos = tile_start + tid;
                    if (kpos < lo || kpos >= hi) {
#pragma unroll
                        for (int p = 0; p < PANELS; ++p) {
                            uint4* row = reinterpret_cast<uint4*>(gen_base + q_bytes<D>() + 2 * kv_bytes<D>() +
                                                                  b * kv_bytes<D>() + p * PANEL_KV + tid * 128);
#pragma unroll
                            for (int c = 0; c < 8; ++c) row[c] = make_uint4(0, 0, 0, 0);
                        }
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            // Follow the product barrier phase by phase.  A parity wait can only tell the
            // current phase from the one before it: a warp that skipped phases and then waited
            // for a later one while the barrier was still two behind would return at once (a
            // fast warp read O before the last product this way).  PV(i-1) was issued when
            // every warp had finished tile i-1, so by now this returns without stalling.
            if (i > 0) {
                bool done = mbar_wait(smem_u32(&pv_full), (i - 1) & 1);
                done = __all_sync(0xffffffffu, done);
                if (!done) { ok = false; if ((tid & 31) == 0) { atomicExch(status, 13); atomicExch(&abort_flag, 1); } break; }
            }
            tc_fence_before();
            mbar_arrive(smem_u32(&p_ready[b]));             // this row's weights are in TMEM
        }
        // ---- write row `tid`
        if (ok && n_tiles > 0) {
            bool done = mbar_wait(smem_u32(&pv_full), (n_tiles - 1) & 1);
            if (*((volatile int*)&abort_flag)) done = false;
            done = __all_sync(0xffffffffu, done);
            if (!done) {
                if ((tid & 31) == 0) atomicExch(status, 15);
            } else {
                tc_fence_after();
                const float inv = 1.0f / l_run;
                uint4* dst = reinterpret_cast<uint4*>(out + ((size_t)(t0 + (tok < n_tok ? tok : 0)) * Hq + kh * G + g) * D);
#pragma unroll
                for (int c = 0; c < D; c += 32) {
                    uint32_t ov[32];
                    tmem_ld32(lane_base + COL_O + c, ov);
                    tmem_ld_wait();
                    if (tok < n_tok) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float* f = reinterpret_cast<const float*>(ov) + 8 * j;
                            dst[c / 8 + j] = make_uint4(pack_bf16(f[0] * inv, f[1] * inv), pack_bf16(f[2] * inv, f[3] * inv),
                                                        pack_bf16(f[4] * inv, f[5] * inv), pack_bf16(f[6] * inv, f[7] * inv));
                        }
                    }
                }
            }
        }
    }
    if (tid == 0 && *((volatile int*)&abort_flag)) {
        // a wait gave up: let copies in flight land (bounded) before the block exits
        for (int b = 0; b < 2; ++b) {
            mbar_wait(smem_u32(&k_full[b]), 0);
            mbar_wait(smem_u32(&v_full[b]), 0);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (issuer) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256) : "memory");
    }
}

template <int D>
int launch(const CUtensorMap& mk, const CUtensorMap& mv, void* out, const void* q, const int* block_table,
           int table_width, const int* seq_starts, const int* seq_rows, const int* seq_first_pos, int R, int N,
           int Hq, int Hkv, int BS, int window, float scale, int* status, cudaStream_t stream) {
    auto kernel = attn_prefill_tcgen05_kernel<D>;
    static sb::OncePerDevice once_per_device;
    bool& configured = once_per_device.flag();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             smem_bytes<D>() + 4096 * 4);
        if (e != cudaSuccess) { sb_set_error("attention_tcgen05: %s", cudaGetErrorString(e)); return (int)e; }
        configured = true;
    }
    const int TQ = ROWS / (Hq / Hkv);
    dim3 grid((N / TQ + R) * Hkv);                           // an upper bound of the number of tiles, times heads
    sb::launch(kernel, grid, dim3(THREADS), smem_bytes<D>() + table_width * 4, stream, mk, mv, (bf16*)out,
               (const bf16*)q, block_table, table_width, seq_starts, seq_rows, seq_first_pos, R, Hq, Hkv, BS, window,
               scale * LOG2E, status);
    return 0;
}

}  // namespace

// 1 if the tcgen05 tile kernel takes this shape (bfloat16 only), else 0.
extern "C" int sb_attention_tcgen05_supports(int Hq, int Hkv, int D, int page_size) {
    if (Hq <= 0 || Hkv <= 0 || Hq % Hkv) return 0;
    if (!(D == 64 || D == 128)) return 0;
    if (!(page_size == 16 || page_size == 32 || page_size == 64)) return 0;
    return Hq / Hkv <= ROWS;       // a group that does not divide 128 leaves the last rows of a tile unused
}

// Arguments as sb_attention_prefill_mma, plus `num_pages` (pages of the pools, the null
// page included) and the status word of the bounded waits.
extern "C" int sb_attention_prefill_tcgen05(void* out, const void* q, const void* k_pool, const void* v_pool,
                                            int num_pages, const int* block_table, int table_width,
                                            const int* seq_starts, const int* seq_rows,
                                            const int* seq_first_pos, int R, int N, int Hq, int Hkv, int D,
                                            int page_size, int window, float scale, int* status,
                                            cudaStream_t stream) {
    SB_REQUIRE(sb_attention_tcgen05_supports(Hq, Hkv, D, page_size),
               "attention_tcgen05: Hq=%d Hkv=%d head_dim=%d page_size=%d is not supported", Hq, Hkv, D, page_size);
    SB_REQUIRE(R > 0 && N > 0 && window >= 0 && table_width > 0 && table_width <= 4096 && num_pages > 0,
               "attention_tcgen05: bad sizes R=%d N=%d table_width=%d", R, N, table_width);
    SB_REQUIRE(status != nullptr, "attention_tcgen05: status is required");
    SB_REQUIRE((long long)num_pages * Hkv * page_size < (1ll << 31), "attention_tcgen05: pool too large");
    CUtensorMap mk, mv;
    const int rows = num_pages * Hkv * page_size;
    if (!sb::get_map(&mk, k_pool, rows, D, page_size) || !sb::get_map(&mv, v_pool, rows, D, page_size)) {
        sb_set_error("attention_tcgen05: cuTensorMapEncodeTiled failed");
        return SB_ERR_ARG;
    }
    int rc;
    if (D == 64)
        rc = launch<64>(mk, mv, out, q, block_table, table_width, seq_starts, seq_rows, seq_first_pos, R, N, Hq, Hkv,
                        page_size, window, scale, status, stream);
    else
        rc = launch<128>(mk, mv, out, q, block_table, table_width, seq_starts, seq_rows, seq_first_pos, R, N, Hq,
                         Hkv, page_size, window, scale, status, stream);
    if (rc != 0) return rc;
    SB_LAUNCH_CHECK();
}
