// Paged causal GQA attention in bfloat16 on the tensor cores (mma.sync m16n8k16,
// float32 accumulation), flash style: keys and values come from the pages in tiles of
// 64 keys through cp.async into swizzled shared memory, scores never leave registers,
// softmax is online in float32 with exp2f.
//
// Two kernels share the tile code:
//   * attn_prefill_kernel: one block per (query tile, KV head).  A query tile is up to
//     64/G consecutive tokens of ONE request with all G query heads of the KV head:
//     64 accumulator rows, 16 per warp.  Tiles are found on the device from the step's
//     request offsets, so the launch shape depends only on the token count.  Queries
//     see the row's pages from the window's start up to their own position, earlier
//     portions included.
//   * attn_decode_kernel: one block per (KV head, token, key partition) for steps in
//     which every request brings one token.  The products are transposed there: a warp's 16
//     keys are the accumulator rows and the G query heads the 8 (or 16) columns.  Each warp
//     takes a quarter of every key tile and the warps are merged at the end; 2 to 4 partitions
//     are merged through the cluster's shared memory, more by the reduce kernel.
//
// Keys outside [lo, hi) are never read from the pool (their shared-memory rows are
// zero-filled by cp.async and their scores are masked), so whatever a page's previous
// owner left in a slot cannot reach the result.  Head sizes 16, 32, 64, 128; group
// sizes that divide 64 (prefill) or are at most 16 (decode); anything else is refused
// and runs on the SIMT kernel.
#include <math.h>
#include <stdlib.h>

#include "attention_reduce.cuh"
#include "common.cuh"

using namespace sb;
typedef __nv_bfloat16 bf16;

extern "C" int sb_attention_decode_mma_kernels(int num_partitions);

namespace {

constexpr int THREADS = 128;
constexpr int KT = 64;              // keys per tile
constexpr float LOG2E = 1.4426950408889634f;

// ----------------------------------------------------------------------------- primitives
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Element offset of 16-byte chunk `chunk` of row `row` in a [rows][D] bfloat16 tile
// whose chunks are XOR-swizzled so that ldmatrix reads eight rows without bank conflicts.
template <int D> __device__ __forceinline__ int tile_off(int row, int chunk) {
    constexpr int CH = D / 8;
    int x;
    if (CH >= 8) x = row & 7;
    else if (CH == 4) x = (row >> 1) & 3;
    else x = (row >> 2) & 1;
    return row * D + ((chunk ^ x) << 3);
}

// Bring keys [tile_start, tile_start + KTILE) of one KV head into shared memory.  Rows of
// keys outside [lo, hi) are zero-filled and never read from the pool.  `table` maps the
// logical page (pos >> bs_log2) - table_base to the physical page; it is a shared-memory
// copy of the block-table segment the block needs, so that no copy waits on a global
// table read.  A thread always copies the same 16-byte column of the rows it serves, so
// its address arithmetic per row is a shift, a mask and a table read.
template <int D, int KTILE = KT, int NTHR = THREADS>
__device__ __forceinline__ void load_kv_tile(bf16* ks, bf16* vs, const bf16* __restrict__ k_pool,
                                             const bf16* __restrict__ v_pool, const int* table, int table_base,
                                             int bs_log2, int Hkv, int kh, int tile_start, int lo, int hi) {
    constexpr int CH = D / 8;                       // 16-byte columns of a row
    constexpr int ROWS = NTHR / CH;                 // rows served per pass
    static_assert(NTHR % CH == 0, "threads must tile the columns");
    const int c = threadIdx.x % CH;
    const int r0 = threadIdx.x / CH;
    const int bs_mask = (1 << bs_log2) - 1;
#pragma unroll
    for (int key = r0; key < KTILE; key += ROWS) {
        const int pos = tile_start + key;
        const bool valid = pos >= lo && pos < hi;
        size_t src = 0;
        if (valid) {
            const int page = table[(pos >> bs_log2) - table_base];
            src = ((((size_t)page * Hkv + kh) << bs_log2) + (pos & bs_mask)) * D + c * 8;
        }
        const int off = tile_off<D>(key, c);
        cp_async16(smem_u32(ks + off), k_pool + src, valid ? 16 : 0);
        cp_async16(smem_u32(vs + off), v_pool + src, valid ? 16 : 0);
    }
}

// Quarter `part` (0..3) of load_kv_tile's copies: the decode kernel issues a tile's copies in
// four doses between the phases of the tile before it.  Sixteen cp.async per thread in one
// burst, from every warp of the SM at the same moment after the block's barrier, queue up in
// the load/store unit: a warp then sat 1,500 clocks of a 3,400-clock tile in that burst.
template <int D, int KTILE, int NTHR>
__device__ __forceinline__ void load_kv_tile_part(int part, bf16* ks, bf16* vs, const bf16* __restrict__ k_pool,
                                                  const bf16* __restrict__ v_pool, const int* table, int table_base,
                                                  int bs_log2, int Hkv, int kh, int tile_start, int lo, int hi) {
    constexpr int CH = D / 8;
    constexpr int ROWS = NTHR / CH;
    constexpr int IT = KTILE / ROWS;                // copies of one thread per tile and pool
    static_assert(NTHR % CH == 0 && KTILE % ROWS == 0, "threads must tile the tile");
    const int c = threadIdx.x % CH;
    const int r0 = threadIdx.x / CH;
    const int bs_mask = (1 << bs_log2) - 1;
#pragma unroll
    for (int it = 0; it < IT; ++it) {
        if (it * 4 / IT != part) continue;          // dose `part` holds the copies it with it*4/IT == part
        const int key = r0 + it * ROWS;
        const int pos = tile_start + key;
        const bool valid = pos >= lo && pos < hi;
        size_t src = 0;
        if (valid) {
            const int page = table[(pos >> bs_log2) - table_base];
            src = ((((size_t)page * Hkv + kh) << bs_log2) + (pos & bs_mask)) * D + c * 8;
        }
        const int off = tile_off<D>(key, c);
        cp_async16(smem_u32(ks + off), k_pool + src, valid ? 16 : 0);
        cp_async16(smem_u32(vs + off), v_pool + src, valid ? 16 : 0);
    }
}

// State of the two accumulator rows a thread owns (rows lane/4 and lane/4 + 8 of the
// warp's 16): running maximum (raw scores), this thread's share of the running sum, and
// the output accumulators.
template <int D> struct RowState {
    float m[2], l[2];
    float o[D / 8][4];
    __device__ __forceinline__ void init() {
        m[0] = m[1] = -INFINITY;
        l[0] = l[1] = 0.f;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    }
};

// One warp: scores of its 16 rows against NK keys of the tile starting at key `kb`,
// masked by per-row [qlo, qpos] and the block's [klo, khi), then online softmax and PV.
//   qf: Q fragments of the warp's rows, D/16 k-steps.
template <int D, int NK>
__device__ __forceinline__ void warp_tile(RowState<D>& st, const uint32_t (&qf)[D / 16][4], const bf16* ks,
                                          const bf16* vs, int kb, int tile_start, const int (&qpos)[2],
                                          const int (&qlo)[2], int klo, int khi, float scale_log2, bool masked) {
    const int lane = threadIdx.x & 31;
    float s[NK / 8][4];
#pragma unroll
    for (int i = 0; i < NK / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;

    // ---- S = Q K^T
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
        for (int nb2 = 0; nb2 < NK / 16; ++nb2) {
            const int j = lane >> 3;
            const int key = kb + nb2 * 16 + (j >> 1) * 8 + (lane & 7);
            uint32_t r[4];
            ldmatrix_x4(r, smem_u32(ks + tile_off<D>(key, kk * 2 + (j & 1))));
            mma_bf16(s[2 * nb2], qf[kk], r[0], r[1]);
            mma_bf16(s[2 * nb2 + 1], qf[kk], r[2], r[3]);
        }
    }
    // ---- mask (only where some key of these NK may be invisible to some row) and row maxima
    float mx[2] = {-INFINITY, -INFINITY};
    if (masked) {
#pragma unroll
        for (int nb = 0; nb < NK / 8; ++nb) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kpos = tile_start + kb + nb * 8 + 2 * (lane & 3) + (e & 1);
                const int r = e >> 1;
                const bool keep = kpos <= qpos[r] && kpos >= qlo[r] && kpos >= klo && kpos < khi;
                s[nb][e] = keep ? s[nb][e] : -INFINITY;
            }
        }
    }
#pragma unroll
    for (int nb = 0; nb < NK / 8; ++nb) {
        mx[0] = fmaxf(mx[0], fmaxf(s[nb][0], s[nb][1]));
        mx[1] = fmaxf(mx[1], fmaxf(s[nb][2], s[nb][3]));
    }
    // The exponent's reference st.m[r] of a row moves only when the row maximum outgrew it by
    // more than 2^8 (weights then stay below 2^8, far inside float32 and bfloat16 range), so
    // most tiles rescale nothing.
    float neg_m[2];
    bool any_grow = false;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const bool grow = mx[r] > -INFINITY && (st.m[r] == -INFINITY || (mx[r] - st.m[r]) * scale_log2 > 8.0f);
        if (grow) {
            const float alpha = st.m[r] == -INFINITY ? 0.f : exp2f((st.m[r] - mx[r]) * scale_log2);
            st.m[r] = mx[r];
            st.l[r] *= alpha;
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
                st.o[i][2 * r] *= alpha;
                st.o[i][2 * r + 1] *= alpha;
            }
        }
        any_grow |= grow;
        neg_m[r] = st.m[r] == -INFINITY ? 0.f : -st.m[r] * scale_log2;
    }
    (void)any_grow;
    // ---- P = 2^(S*scale - m*scale) in float32 (one multiply-add, one ex2; masked scores
    // are -inf and give 0).  For the product with V each weight is split into two bfloat16
    // terms, p = hi + lo (16 bits of mantissa together), so that the softmax weights are not
    // cut to 8 bits before they are used.
    uint32_t pk_hi[NK / 8][2], pk_lo[NK / 8][2];
#pragma unroll
    for (int nb = 0; nb < NK / 8; ++nb) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const float p0 = ex2_approx(fmaf(s[nb][2 * r], scale_log2, neg_m[r]));
            const float p1 = ex2_approx(fmaf(s[nb][2 * r + 1], scale_log2, neg_m[r]));
            st.l[r] += p0 + p1;
            const uint32_t hi = pack_bf16(p0, p1);
            pk_hi[nb][r] = hi;
            pk_lo[nb][r] = pack_bf16(p0 - __uint_as_float(hi << 16), p1 - __uint_as_float(hi & 0xffff0000u));
        }
    }
    // ---- O += P V
#pragma unroll
    for (int k16 = 0; k16 < NK / 16; ++k16) {
        const uint32_t pa[4] = {pk_hi[2 * k16][0], pk_hi[2 * k16][1], pk_hi[2 * k16 + 1][0], pk_hi[2 * k16 + 1][1]};
        const uint32_t pb[4] = {pk_lo[2 * k16][0], pk_lo[2 * k16][1], pk_lo[2 * k16 + 1][0], pk_lo[2 * k16 + 1][1]};
#pragma unroll
        for (int nb2 = 0; nb2 < D / 16; ++nb2) {
            const int j = lane >> 3;
            const int key = kb + k16 * 16 + (j & 1) * 8 + (lane & 7);
            uint32_t r[4];
            ldmatrix_x4_trans(r, smem_u32(vs + tile_off<D>(key, nb2 * 2 + (j >> 1))));
            mma_bf16(st.o[2 * nb2], pa, r[0], r[1]);
            mma_bf16(st.o[2 * nb2 + 1], pa, r[2], r[3]);
            mma_bf16(st.o[2 * nb2], pb, r[0], r[1]);
            mma_bf16(st.o[2 * nb2 + 1], pb, r[2], r[3]);
        }
    }
}

// ---- the decode step's tile: one token, so only the G query heads of the KV head are rows.
// With the query rows on the 16 accumulator rows of an m16n8k16 product at least half of them
// (three quarters at G = 4) would be padding, and the products, not memory, bounded the kernel
// (64 clocks per product and warp measured).  Here the products are transposed: the KEYS are
// the 16 accumulator rows and the query heads the 8 columns (NBQ = 1, G <= 8) or 16 (NBQ = 2):
//   S^T = K Q^T      A = 16 keys x 16 dims from the key tile, B = Q^T (the query fragments)
//   O^T += V^T P^T   A = 16 dims x 16 keys (ldmatrix.trans of the value tile), B = P^T
// which halves the products per key at G <= 8.  A thread owns two query heads (columns
// 2*(lane%4), +1 of each column block): maxima and sums run down the columns (over the lanes
// with the same lane%4), and P^T becomes a B operand through movmatrix.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

// m[c], l[c]: reference maximum and this thread's share of the sum of column c = 2*nb + e;
// o[mb][nb][4]: O^T, dims 16*mb + lane/4 (+8 for [2], [3]) by the thread's two columns.
template <int D, int NBQ> struct ColState {
    float m[2 * NBQ], l[2 * NBQ];
    float o[D / 16][NBQ][4];
    __device__ __forceinline__ void init() {
#pragma unroll
        for (int c = 0; c < 2 * NBQ; ++c) { m[c] = -INFINITY; l[c] = 0.f; }
#pragma unroll
        for (int i = 0; i < D / 16; ++i)
#pragma unroll
            for (int nb = 0; nb < NBQ; ++nb) o[i][nb][0] = o[i][nb][1] = o[i][nb][2] = o[i][nb][3] = 0.f;
    }
};

// One warp: its 16 keys (kb .. kb+15 of the tile at tile_start) against the token's query heads.
//   qf: the query fragments as loaded for an A operand (rows 0-7 and 8-15, two 8-dim chunks).
//   Keys outside [klo, khi) or beyond qpos are masked when `masked`.
//   between(p), p = 0..3: called between the phases (the caller issues a later tile's copies there).
template <int D, int NBQ, typename Between>
__device__ __forceinline__ void warp_tile_decode(ColState<D, NBQ>& st, const uint32_t (&qf)[D / 16][4],
                                                 const bf16* ks, const bf16* vs, int kb, int tile_start, int qpos,
                                                 int klo, int khi, float scale_log2, bool masked, Between between) {
    const int lane = threadIdx.x & 31;
    const int j = lane >> 3;
    // ---- S^T = K Q^T.  The D/16 products of a column block would be one chain through their
    // accumulator; they go to CH accumulators in turn (four chains a quarter as long), added at the end.
    constexpr int CH = D / 16 >= 4 ? 4 : D / 16;
    float sp[CH][NBQ][4];
#pragma unroll
    for (int c = 0; c < CH; ++c)
#pragma unroll
        for (int nb = 0; nb < NBQ; ++nb) sp[c][nb][0] = sp[c][nb][1] = sp[c][nb][2] = sp[c][nb][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4];
        ldmatrix_x4(a, smem_u32(ks + tile_off<D>(kb + (j & 1) * 8 + (lane & 7), kk * 2 + (j >> 1))));
        mma_bf16(sp[kk % CH][0], a, qf[kk][0], qf[kk][2]);
        if constexpr (NBQ == 2) mma_bf16(sp[kk % CH][1], a, qf[kk][1], qf[kk][3]);
        if (kk == D / 32) between(0);
    }
    between(1);
    float s[NBQ][4];
#pragma unroll
    for (int nb = 0; nb < NBQ; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float v = sp[0][nb][e];
#pragma unroll
            for (int c = 1; c < CH; ++c) v += sp[c][nb][e];
            s[nb][e] = v;
        }
    // ---- mask: the thread's keys are rows lane/4 and lane/4 + 8
    if (masked) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int kpos = tile_start + kb + (lane >> 2) + 8 * h;
            const bool keep = kpos <= qpos && kpos >= klo && kpos < khi;
#pragma unroll
            for (int nb = 0; nb < NBQ; ++nb) {
                s[nb][2 * h] = keep ? s[nb][2 * h] : -INFINITY;
                s[nb][2 * h + 1] = keep ? s[nb][2 * h + 1] : -INFINITY;
            }
        }
    }
    // ---- column maxima over the warp's 16 keys, lazy move of the reference (as in warp_tile)
    float neg_m[2 * NBQ];
#pragma unroll
    for (int nb = 0; nb < NBQ; ++nb) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int c = 2 * nb + e;
            float mx = fmaxf(s[nb][e], s[nb][e + 2]);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const bool grow = mx > -INFINITY && (st.m[c] == -INFINITY || (mx - st.m[c]) * scale_log2 > 8.0f);
            if (grow) {
                const float alpha = st.m[c] == -INFINITY ? 0.f : exp2f((st.m[c] - mx) * scale_log2);
                st.m[c] = mx;
                st.l[c] *= alpha;
#pragma unroll
                for (int i = 0; i < D / 16; ++i) {
                    st.o[i][nb][e] *= alpha;
                    st.o[i][nb][e + 2] *= alpha;
                }
            }
            neg_m[c] = st.m[c] == -INFINITY ? 0.f : -st.m[c] * scale_log2;
        }
    }
    between(2);
    // ---- P^T = 2^(S^T*scale - m*scale), split into two bfloat16 terms, transposed into B operands
    uint32_t bhi[NBQ][2], blo[NBQ][2];
#pragma unroll
    for (int nb = 0; nb < NBQ; ++nb) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {                       // keys lane/4 (h = 0) and lane/4 + 8 (h = 1)
            const float p0 = ex2_approx(fmaf(s[nb][2 * h], scale_log2, neg_m[2 * nb]));
            const float p1 = ex2_approx(fmaf(s[nb][2 * h + 1], scale_log2, neg_m[2 * nb + 1]));
            st.l[2 * nb] += p0;
            st.l[2 * nb + 1] += p1;
            const uint32_t hi = pack_bf16(p0, p1);
            const uint32_t lo = pack_bf16(p0 - __uint_as_float(hi << 16), p1 - __uint_as_float(hi & 0xffff0000u));
            bhi[nb][h] = movmatrix_trans(hi);
            blo[nb][h] = movmatrix_trans(lo);
        }
    }
    // ---- O^T += V^T P^T
#pragma unroll
    for (int mb = 0; mb < D / 16; ++mb) {
        uint32_t a[4];
        ldmatrix_x4_trans(a, smem_u32(vs + tile_off<D>(kb + (j >> 1) * 8 + (lane & 7), mb * 2 + (j & 1))));
#pragma unroll
        for (int nb = 0; nb < NBQ; ++nb) {
            mma_bf16(st.o[mb][nb], a, bhi[nb][0], bhi[nb][1]);
            mma_bf16(st.o[mb][nb], a, blo[nb][0], blo[nb][1]);
        }
        if (mb == D / 32) between(3);
    }
}

// ----------------------------------------------------------------------------- prefill
// grid (max_tiles, Hkv).  seq_starts [R+1], seq_rows [R], seq_first_pos [R].
template <int D>
__global__ void __launch_bounds__(THREADS)
attn_prefill_kernel(bf16* __restrict__ out, const bf16* __restrict__ q, const bf16* __restrict__ k_pool,
                    const bf16* __restrict__ v_pool, const int* __restrict__ block_table, int table_width,
                    const int* __restrict__ seq_starts, const int* __restrict__ seq_rows,
                    const int* __restrict__ seq_first_pos, int R, int Hq, int Hkv, int BS, int window,
                    float scale_log2) {
    sb::pdl_launch_dependents();     // the next kernel may begin its prologue
    sb::pdl_wait();                  // everything before this kernel is complete and visible
    extern __shared__ __align__(128) uint8_t smem[];
    bf16* qs = reinterpret_cast<bf16*>(smem);               // [64][D]
    bf16* kbuf = qs + 64 * D;                               // 2 x [64][D]
    bf16* vbuf = kbuf + 2 * KT * D;                         // 2 x [64][D]
    int* stab = reinterpret_cast<int*>(vbuf + 2 * KT * D);  // the pages of keys [lo, hi): up to table_width

    const int G = Hq / Hkv;
    const int bs_log2 = 31 - __clz(BS);                     // the page size is a power of two
    const int TQ = 64 / G;                                  // tokens per tile
    const int kh = blockIdx.y;
    // ---- which request, which tile (reversed: later tiles of a prompt have more keys and
    // should start first)
    int tile = gridDim.x - 1 - blockIdx.x, r = 0, t0 = 0, n_tok = 0;
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
    if (r >= R) return;
    const int first_pos = seq_first_pos[r] + tile * TQ;
    const int* table = block_table + (size_t)seq_rows[r] * table_width;
    const int hi = first_pos + n_tok;                       // keys [lo, hi) are needed by this tile
    const int lo = (window > 0 && first_pos + 1 > window) ? first_pos + 1 - window : 0;
    const int tile_begin = lo / KT, tile_end = (hi + KT - 1) / KT;
    const int last_qlo = (window > 0 && hi > window) ? hi - window : 0;
    const int table_base = lo / BS;
    for (int i = threadIdx.x; i <= (hi - 1) / BS - table_base; i += THREADS) stab[i] = table[table_base + i];
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // ---- Q tile: row = token * G + head
    constexpr int CH = D / 8;
    for (int idx = threadIdx.x; idx < 64 * CH; idx += THREADS) {
        const int row = idx / CH, c = idx - row * CH;
        const int tok = row / G, g = row - tok * G;
        const bool valid = tok < n_tok;
        const bf16* src = q + ((size_t)(t0 + (valid ? tok : 0)) * Hq + kh * G + g) * D + c * 8;
        cp_async16(smem_u32(qs + tile_off<D>(row, c)), src, valid ? 16 : 0);
    }
    load_kv_tile<D>(kbuf, vbuf, k_pool, v_pool, stab, table_base, bs_log2, Hkv, kh, tile_begin * KT, lo, hi);
    cp_async_commit();

    int qpos[2], qlo[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int row = warp * 16 + (lane >> 2) + i * 8;
        const int tok = row / G;
        qpos[i] = tok < n_tok ? first_pos + tok : -1;       // rows past the tile see no key
        qlo[i] = (window > 0 && qpos[i] + 1 > window) ? qpos[i] + 1 - window : 0;
    }
    RowState<D> st;
    st.init();
    uint32_t qf[D / 16][4];

    const int n_tiles = tile_end - tile_begin;
    for (int i = 0; i < n_tiles; ++i) {
        const int buf = i & 1;
        if (i + 1 < n_tiles) {
            load_kv_tile<D>(kbuf + (buf ^ 1) * KT * D, vbuf + (buf ^ 1) * KT * D, k_pool, v_pool, stab, table_base,
                            bs_log2, Hkv, kh, (tile_begin + i + 1) * KT, lo, hi);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (i == 0) {
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk)
                ldmatrix_x4(qf[kk], smem_u32(qs + tile_off<D>(warp * 16 + (lane & 15), kk * 2 + (lane >> 4))));
        }
        // every row of the block sees every key of a tile that ends at or before the first query
        // and starts at or after the last query's window start; other tiles need the masks
        const int ts = (tile_begin + i) * KT;
        const bool masked = ts + KT - 1 > first_pos || ts < last_qlo || n_tok < TQ;
        warp_tile<D, KT>(st, qf, kbuf + buf * KT * D, vbuf + buf * KT * D, 0, ts, qpos, qlo, lo, hi, scale_log2,
                         masked);
        __syncthreads();
    }
    // ---- write
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        float l = st.l[i];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int row = warp * 16 + (lane >> 2) + i * 8;
        const int tok = row / G, g = row - tok * G;
        if (tok >= n_tok) continue;
        const float inv = 1.0f / l;
        bf16* dst = out + ((size_t)(t0 + tok) * Hq + kh * G + g) * D + 2 * (lane & 3);
#pragma unroll
        for (int nb = 0; nb < D / 8; ++nb)
            *reinterpret_cast<uint32_t*>(dst + nb * 8) = pack_bf16(st.o[nb][2 * i] * inv, st.o[nb][2 * i + 1] * inv);
    }
}

// ----------------------------------------------------------------------------- decode
// grid (Hkv, N, NP); every token is one query at position positions[n] of row token_rows[n].
// NW warps; a key tile holds 16 keys per warp; S stages of tiles are kept in flight.
// CLUSTER: the NP blocks of a (token, KV head) are one thread-block cluster and merge their
// partial results through distributed shared memory: no scratch in global memory, no reduce
// kernel.  Every block of the cluster reaches both cluster barriers (an empty partition too).
template <int D, int NW, int S, bool CLUSTER = false, int NBQ = 1>
__global__ void __launch_bounds__(32 * NW)
attn_decode_kernel(bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                   const bf16* __restrict__ q, const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool,
                   const int* __restrict__ block_table, int table_width, const int* __restrict__ token_rows,
                   const int* __restrict__ positions, int Hq, int Hkv, int BS, int window, float scale_log2,
                   int NP) {
    sb::pdl_launch_dependents();     // the next kernel may begin its prologue
    // What is read before pdl_wait() below was complete before the preceding kernel began:
    // the block table, rows and positions (copied from the host at the start of the step)
    // and keys and values below the newest position (written by earlier steps).  The query
    // and the newest key and value come from the preceding kernel and are read after it.
    constexpr int KTD = 16 * NW;                            // keys per tile
    constexpr int NTHR = 32 * NW;
    extern __shared__ __align__(128) uint8_t smem[];
    bf16* qs = reinterpret_cast<bf16*>(smem);               // [16][D]
    bf16* kbuf = qs + 16 * D;                               // S x [KTD][D]
    bf16* vbuf = kbuf + S * KTD * D;                        // S x [KTD][D]
    int* stab = reinterpret_cast<int*>(vbuf + S * KTD * D); // the pages of this partition: up to table_width
    __shared__ float w_m[NW][16], w_l[NW][16];
    __shared__ float c_ml[16][2];                           // CLUSTER: this partition's (max, sum) per row

    const int G = Hq / Hkv;
    const int bs_log2 = 31 - __clz(BS);                     // the page size is a power of two
    const int kh = blockIdx.x, n = blockIdx.y, part = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = positions[n];
    const int* table = block_table + (size_t)token_rows[n] * table_width;
    const int hi = pos + 1;
    const int lo = (window > 0 && hi > window) ? hi - window : 0;
    const int first_pg = lo / BS, last_pg = (hi - 1) / BS;
    const int ppp = (last_pg - first_pg + 1 + NP - 1) / NP;
    const int pg_begin = first_pg + part * ppp;
    const int pg_end = min(pg_begin + ppp, last_pg + 1);
    const int k_begin = max(lo, pg_begin * BS);
    const int k_end = min(hi, pg_end * BS);
    const int h0 = kh * G;

    const bool empty = k_begin >= k_end;                    // an empty partition (only when NP > 1)
    if (empty && CLUSTER) {
        sb::pdl_wait();
        if (threadIdx.x < 16) { c_ml[threadIdx.x][0] = -INFINITY; c_ml[threadIdx.x][1] = 0.f; }
    } else if (empty) {
        sb::pdl_wait();
        if (threadIdx.x < G) {
            float* ml = part_ml + (((size_t)n * Hq + h0 + threadIdx.x) * NP + part) * 2;
            ml[0] = -INFINITY;
            ml[1] = 0.f;
        }
        return;                                             // the reduce kernel follows
    }
    if (!empty) {
    const int tile_begin = k_begin / KTD, tile_end = (k_end + KTD - 1) / KTD;
    const int n_tiles = tile_end - tile_begin;
    for (int i = threadIdx.x; i < pg_end - pg_begin; i += NTHR) stab[i] = table[pg_begin + i];
    __syncthreads();
    // Tiles that end below the newest key are fetched now, the others after the wait.
    int s_first_late = 0;
#pragma unroll
    for (int s = 0; s < S - 1; ++s) {
        if (s == s_first_late && s < n_tiles && (tile_begin + s + 1) * KTD <= pos) {
            load_kv_tile<D, KTD, NTHR>(kbuf + s * KTD * D, vbuf + s * KTD * D, k_pool, v_pool, stab, pg_begin,
                                       bs_log2, Hkv, kh, (tile_begin + s) * KTD, k_begin, k_end);
            cp_async_commit();
            s_first_late = s + 1;
        }
    }
    sb::pdl_wait();                  // everything before this kernel is complete and visible
    constexpr int CH = D / 8;
    for (int idx = threadIdx.x; idx < 16 * CH; idx += NTHR) {
        const int row = idx / CH, c = idx - row * CH;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (row < G) v = *reinterpret_cast<const uint4*>(q + ((size_t)n * Hq + h0 + row) * D + c * 8);
        *reinterpret_cast<uint4*>(qs + tile_off<D>(row, c)) = v;
    }
#pragma unroll
    for (int s = 0; s < S - 1; ++s) {
        if (s >= s_first_late) {
            if (s < n_tiles)
                load_kv_tile<D, KTD, NTHR>(kbuf + s * KTD * D, vbuf + s * KTD * D, k_pool, v_pool, stab, pg_begin,
                                           bs_log2, Hkv, kh, (tile_begin + s) * KTD, k_begin, k_end);
            cp_async_commit();
        }
    }

    ColState<D, NBQ> st;
    st.init();
    uint32_t qf[D / 16][4];
    for (int i = 0; i < n_tiles; ++i) {
        cp_async_wait<S - 2>();                             // tile i has landed (this thread's share)
        __syncthreads();                                    // ... and everybody's; slot (i-1)%S is free
        const int nxt = i + S - 1;
        if (i == 0) {
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk)
                ldmatrix_x4(qf[kk], smem_u32(qs + tile_off<D>(lane & 15, kk * 2 + (lane >> 4))));
        }
        // warp w takes keys 16w .. 16w+15 of the tile
        const int buf = i % S;
        const int ts = (tile_begin + i) * KTD;
        const bool masked = ts < k_begin || ts + KTD > k_end;       // only the partition's edge tiles
        // tile nxt's copies go out in four doses between the phases of tile i (slot (i-1)%S is free)
        auto between = [&](int part) {
            if (nxt < n_tiles)
                load_kv_tile_part<D, KTD, NTHR>(part, kbuf + (nxt % S) * KTD * D, vbuf + (nxt % S) * KTD * D, k_pool,
                                                v_pool, stab, pg_begin, bs_log2, Hkv, kh, (tile_begin + nxt) * KTD,
                                                k_begin, k_end);
        };
        warp_tile_decode<D, NBQ>(st, qf, kbuf + buf * KTD * D, vbuf + buf * KTD * D, warp * 16, ts, pos, k_begin,
                                 k_end, scale_log2, masked, between);
        cp_async_commit();
    }
    cp_async_wait<0>();
    __syncthreads();
    // ---- merge the warps: each writes its query heads' (m, l, O) to shared memory
    float* wo = reinterpret_cast<float*>(kbuf);             // [NW][16][D] floats: fits in the K and V buffers
#pragma unroll
    for (int nb = 0; nb < NBQ; ++nb) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int c = 2 * nb + e;
            float l = st.l[c];
            l += __shfl_xor_sync(0xffffffffu, l, 4);
            l += __shfl_xor_sync(0xffffffffu, l, 8);
            l += __shfl_xor_sync(0xffffffffu, l, 16);
            const int row = 8 * nb + 2 * (lane & 3) + e;    // the query head of this column
            if (lane < 4) { w_m[warp][row] = st.m[c]; w_l[warp][row] = l; }
#pragma unroll
            for (int mb = 0; mb < D / 16; ++mb) {
                float* dst = wo + ((size_t)(warp * 16 + row)) * D + mb * 16 + (lane >> 2);
                dst[0] = st.o[mb][nb][e];
                dst[8] = st.o[mb][nb][e + 2];
            }
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < G * D; idx += NTHR) {
        const int row = idx / D, d = idx - row * D;
        // every warp's (max, sum, value) first, so that the loads are in flight together; a warp
        // without a visible key (sum 0) has weight 0 whatever its other numbers are
        float wm[NW], wl[NW], wv[NW];
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            wm[w] = w_m[w][row];
            wl[w] = w_l[w][row];
            wv[w] = wo[((size_t)(w * 16 + row)) * D + d];
        }
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) M = wl[w] > 0.f ? fmaxf(M, wm[w]) : M;
        float L = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) {
            const float f = wl[w] > 0.f ? ex2_approx((wm[w] - M) * scale_log2) : 0.f;
            L += f * wl[w];
            o += wl[w] > 0.f ? f * wv[w] : 0.f;
        }
        const int h = h0 + row;
        if (NP == 1) {
            out[((size_t)n * Hq + h) * D + d] = __float2bfloat16_rn(o / L);
        } else if (CLUSTER) {
            wo[(size_t)NW * 16 * D + idx] = o;              // behind the warps' rows: [G][D] of this partition
            if (d == 0) {
                c_ml[row][0] = M * scale_log2 / LOG2E;      // natural exponents, as in the reduce kernel
                c_ml[row][1] = L;
            }
        } else {
            part_o[(((size_t)n * Hq + h) * NP + part) * D + d] = o;
            if (d == 0) {
                float* ml = part_ml + (((size_t)n * Hq + h) * NP + part) * 2;
                ml[0] = M * scale_log2 / LOG2E;             // natural exponents, as the reduce kernel expects
                ml[1] = L;
            }
        }
    }
    }   // !empty
    if constexpr (CLUSTER) {
        // ---- merge over the cluster: block r writes the outputs idx = r, r + NP, ... of the G x D
        //      out[h,:] = sum_p e^{m_p - M} o_p / sum_p e^{m_p - M} l_p over partitions with l > 0
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        const float* co = reinterpret_cast<const float*>(kbuf) + (size_t)NW * 16 * D;
        const uint32_t co_addr = static_cast<uint32_t>(__cvta_generic_to_shared(co));
        const uint32_t ml_addr = static_cast<uint32_t>(__cvta_generic_to_shared(&c_ml[0][0]));
        for (int idx = part * NTHR + threadIdx.x; idx < G * D; idx += NP * NTHR) {
            const int row = idx / D;
            // every partition's (max, sum) and value first (NP <= 4: all loads in flight at once; an
            // empty partition's value is whatever its shared memory holds and is not used), then the sum
            float pm[4], pl[4], pv[4];
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                pm[p] = -INFINITY; pl[p] = 0.f; pv[p] = 0.f;
                if (p < NP) {
                    uint32_t a, b;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(ml_addr + row * 8), "r"(p));
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(b) : "r"(co_addr + idx * 4), "r"(p));
                    asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(pm[p]), "=f"(pl[p]) : "r"(a) : "memory");
                    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(pv[p]) : "r"(b) : "memory");
                }
            }
            float M = -INFINITY;
#pragma unroll
            for (int p = 0; p < 4; ++p)
                if (pl[p] > 0.f) M = fmaxf(M, pm[p]);
            float L = 0.f, o = 0.f;
#pragma unroll
            for (int p = 0; p < 4; ++p)
                if (pl[p] > 0.f) {
                    const float f = expf(pm[p] - M);
                    L += f * pl[p];
                    o += f * pv[p];
                }
            out[((size_t)n * Hq + h0 + row) * D + (idx - row * D)] = __float2bfloat16_rn(o / L);
        }
        // nobody leaves while another block may still read its shared memory
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        return;
    }
}

template <int D> constexpr int prefill_smem() { return (64 * D + 4 * KT * D) * 2; }
template <int D, int NW, int S> constexpr int decode_smem() { return (16 * D + 2 * S * 16 * NW * D) * 2; }
constexpr int kMaxTableWidth = 4096;                         // entries of the staged block-table segment

template <int D>
int launch_prefill(void* out, const void* q, const void* k_pool, const void* v_pool, const int* block_table,
                   int table_width, const int* seq_starts, const int* seq_rows, const int* seq_first_pos, int R,
                   int N, int Hq, int Hkv, int BS, int window, float scale, cudaStream_t stream) {
    auto kernel = attn_prefill_kernel<D>;
    static sb::OncePerDevice once_per_device;
    bool& configured = once_per_device.flag();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             prefill_smem<D>() + kMaxTableWidth * 4);
        if (e != cudaSuccess) { sb_set_error("attention_mma: %s", cudaGetErrorString(e)); return (int)e; }
        configured = true;
    }
    const int TQ = 64 / (Hq / Hkv);
    dim3 grid(N / TQ + R, Hkv);                              // an upper bound of the number of tiles
    sb::launch(kernel, grid, dim3(THREADS), prefill_smem<D>() + table_width * 4, stream,
        (bf16*)out, (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, block_table, table_width, seq_starts,
        seq_rows, seq_first_pos, R, Hq, Hkv, BS, window, scale * LOG2E);
    return 0;
}

// The partitions are merged through the cluster when there are 2 to 4 of them;
// SOCRATES_CLUSTER_MERGE=0 keeps the reduce kernel.  Measured
// in the decode graph of the 4B shape: 4 partitions (batch 8) 2.69 against 2.74 ms a step, 2 (batch
// 16) 3.25 against 3.31; clusters of 8 (batch 2 to 4) are slower than 9 partitions with the reduce
// kernel (2.64 against 2.54 ms at batch 4): eight blocks have to find room at the same time.
inline bool cluster_merge_enabled() {
    static const bool on = [] { const char* e = getenv("SOCRATES_CLUSTER_MERGE"); return !(e && e[0] == '0'); }();
    return on;
}

template <int D, int NW, int S, int NBQ>
int launch_decode_v(void* out, float* part_o, float* part_ml, const void* q, const void* k_pool, const void* v_pool,
                    const int* block_table, int table_width, const int* token_rows, const int* positions, int N,
                    int Hq, int Hkv, int BS, int window, float scale, int NP, cudaStream_t stream) {
    constexpr int smem = decode_smem<D, NW, S>();
    const bool cluster = NP >= 2 && sb_attention_decode_mma_kernels(NP) == 1;
    static sb::OncePerDevice once_per_device;
    bool& configured = once_per_device.flag();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<D, NW, S, false, NBQ>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem + kMaxTableWidth * 4);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_decode_kernel<D, NW, S, true, NBQ>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, smem + kMaxTableWidth * 4);
        if (e != cudaSuccess) { sb_set_error("attention_mma: %s", cudaGetErrorString(e)); return (int)e; }
        configured = true;
    }
    dim3 grid(Hkv, N, NP);
    if (cluster) {
        sb::launch_cluster(attn_decode_kernel<D, NW, S, true, NBQ>, dim3(grid), dim3(32 * NW), smem + table_width * 4, stream,
            dim3(1, 1, NP), (bf16*)out, part_o, part_ml, (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool,
            block_table, table_width, token_rows, positions, Hq, Hkv, BS, window, scale * LOG2E, NP);
        return 0;
    }
    sb::launch(attn_decode_kernel<D, NW, S, false, NBQ>, dim3(grid), dim3(32 * NW), smem + table_width * 4, stream, 
        (bf16*)out, part_o, part_ml, (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, block_table,
        table_width, token_rows, positions, Hq, Hkv, BS, window, scale * LOG2E, NP);
    if (NP > 1) {
        dim3 rgrid(Hq, N);
        sb::launch(attn_reduce_kernel<bf16>, dim3(rgrid), dim3(128), 0, stream, (bf16*)out, part_o, part_ml, Hq, D, NP);
    }
    return 0;
}

// Shapes of the decode kernel: (warps, stages).  Variant 0 is the default; variant 1 holds one
// stage less, so that three blocks fit an SM.  (Two warps with rings of 4 or 6 stages and four
// warps with 4 stages were measured slower at every batch size and are gone.)
constexpr int kDecodeVariants = 2;
constexpr int kVariantWarps[kDecodeVariants] = {4, 4};
constexpr int kVariantStages[kDecodeVariants] = {3, 2};

template <int D>
int launch_decode(void* out, float* part_o, float* part_ml, const void* q, const void* k_pool, const void* v_pool,
                  const int* block_table, int table_width, const int* token_rows, const int* positions, int N,
                  int Hq, int Hkv, int BS, int window, float scale, int NP, cudaStream_t stream, int variant = 0) {
#define SB_DEC(NW, S, NBQ) launch_decode_v<D, NW, S, NBQ>(out, part_o, part_ml, q, k_pool, v_pool, block_table, \
                                                          table_width, token_rows, positions, N, Hq, Hkv, BS, window, \
                                                          scale, NP, stream)
    // query heads of a KV head: one block of 8 columns, or two
    if (Hq / Hkv <= 8) return variant == 1 ? SB_DEC(4, 2, 1) : SB_DEC(4, 3, 1);
    return variant == 1 ? SB_DEC(4, 2, 2) : SB_DEC(4, 3, 2);
#undef SB_DEC
}

}  // namespace

// 1 if the tensor-core kernels take this shape (bfloat16 only), else 0.
extern "C" int sb_attention_mma_supports(int Hq, int Hkv, int D, int page_size, int decode) {
    if (Hq <= 0 || Hkv <= 0 || Hq % Hkv) return 0;
    if (!(D == 16 || D == 32 || D == 64 || D == 128)) return 0;
    if (page_size <= 0 || (page_size & (page_size - 1))) return 0;     // a power of two
    const int G = Hq / Hkv;
    return decode ? (G <= 16) : (64 % G == 0);
}

// Prompt portions and mixed steps: requests r = 0..R-1 bring tokens
// seq_starts[r] .. seq_starts[r+1]-1 at positions seq_first_pos[r]... of cache row seq_rows[r].
extern "C" int sb_attention_prefill_mma(void* out, const void* q, const void* k_pool, const void* v_pool,
                                        const int* block_table, int table_width, const int* seq_starts,
                                        const int* seq_rows, const int* seq_first_pos, int R, int N, int Hq,
                                        int Hkv, int D, int page_size, int window, float scale,
                                        cudaStream_t stream) {
    SB_REQUIRE(sb_attention_mma_supports(Hq, Hkv, D, page_size, 0),
               "attention_mma (prefill): Hq=%d Hkv=%d head_dim=%d is not supported", Hq, Hkv, D);
    SB_REQUIRE(R > 0 && N > 0 && window >= 0 && table_width > 0, "attention_mma: bad sizes R=%d N=%d", R, N);
    SB_REQUIRE(table_width <= kMaxTableWidth, "attention_mma: block table of %d pages per row exceeds %d",
               table_width, kMaxTableWidth);
    int rc;
    switch (D) {
        case 16: rc = launch_prefill<16>(out, q, k_pool, v_pool, block_table, table_width, seq_starts, seq_rows, seq_first_pos, R, N, Hq, Hkv, page_size, window, scale, stream); break;
        case 32: rc = launch_prefill<32>(out, q, k_pool, v_pool, block_table, table_width, seq_starts, seq_rows, seq_first_pos, R, N, Hq, Hkv, page_size, window, scale, stream); break;
        case 64: rc = launch_prefill<64>(out, q, k_pool, v_pool, block_table, table_width, seq_starts, seq_rows, seq_first_pos, R, N, Hq, Hkv, page_size, window, scale, stream); break;
        default: rc = launch_prefill<128>(out, q, k_pool, v_pool, block_table, table_width, seq_starts, seq_rows, seq_first_pos, R, N, Hq, Hkv, page_size, window, scale, stream); break;
    }
    if (rc != 0) return rc;
    SB_LAUNCH_CHECK();
}

// How many kernels sb_attention_decode_mma launches for this many partitions (1, or 2 when a
// reduce kernel follows): what callers that count launches add.
extern "C" int sb_attention_decode_mma_kernels(int num_partitions) {
    if (num_partitions <= 1) return 1;
    return (num_partitions <= 4 && cluster_merge_enabled()) ? 1 : 2;
}

// Blocks of the decode kernel that fit one SM at a time (shared memory is the limit):
// what the caller sizes the number of key partitions with.
extern "C" int sb_attention_decode_mma_blocks_per_sm(int D, int variant) {
    if (variant < 0 || variant >= kDecodeVariants) variant = 0;
    const int smem = (16 * D + 2 * kVariantStages[variant] * 16 * kVariantWarps[variant] * D) * 2 + 1024 + 2048;
    int b = (227 * 1024) / smem;
    return b < 1 ? 1 : (b > 16 ? 16 : b);
}

// Steps in which every request brings one token.  Scratch as for sb_attention_simt.
// `variant` selects (warps, stages) of the kernel; 0 is the default.
// The block table, rows, positions, and keys and values below each token's position must be
// complete before the kernel that precedes this one on the stream started; the query and
// the newest key and value may come from that kernel.
extern "C" int sb_attention_decode_mma(void* out, float* part_o, float* part_ml, const void* q,
                                       const void* k_pool, const void* v_pool, const int* block_table,
                                       int table_width, const int* token_rows, const int* positions, int N,
                                       int Hq, int Hkv, int D, int page_size, int window, float scale,
                                       int num_partitions, int variant, cudaStream_t stream) {
    SB_REQUIRE(sb_attention_mma_supports(Hq, Hkv, D, page_size, 1),
               "attention_mma (decode): Hq=%d Hkv=%d head_dim=%d is not supported", Hq, Hkv, D);
    SB_REQUIRE(N > 0 && N <= 65535 && window >= 0 && table_width > 0, "attention_mma: bad sizes N=%d", N);
    SB_REQUIRE(table_width <= kMaxTableWidth, "attention_mma: block table of %d pages per row exceeds %d",
               table_width, kMaxTableWidth);
    SB_REQUIRE(num_partitions >= 1 && num_partitions <= 65535, "attention_mma: %d partitions", num_partitions);
    SB_REQUIRE(num_partitions == 1 || (part_o != nullptr && part_ml != nullptr),
               "attention_mma: split over %d partitions needs scratch buffers", num_partitions);
    int rc;
    switch (D) {
        case 16: rc = launch_decode<16>(out, part_o, part_ml, q, k_pool, v_pool, block_table, table_width, token_rows, positions, N, Hq, Hkv, page_size, window, scale, num_partitions, stream, variant); break;
        case 32: rc = launch_decode<32>(out, part_o, part_ml, q, k_pool, v_pool, block_table, table_width, token_rows, positions, N, Hq, Hkv, page_size, window, scale, num_partitions, stream, variant); break;
        case 64: rc = launch_decode<64>(out, part_o, part_ml, q, k_pool, v_pool, block_table, table_width, token_rows, positions, N, Hq, Hkv, page_size, window, scale, num_partitions, stream, variant); break;
        default: rc = launch_decode<128>(out, part_o, part_ml, q, k_pool, v_pool, block_table, table_width, token_rows, positions, N, Hq, Hkv, page_size, window, scale, num_partitions, stream, variant); break;
    }
    if (rc != 0) return rc;
    SB_LAUNCH_CHECK();
}

// ----------------------------------------------------------------------------------------
// The variant that allocates nothing (see no_alloc.h): scratch for the key partitions
// lives in this file-scope device array.  In host code the name below is only a handle
// for cudaGetSymbolAddress, never a pointer a kernel may be given.
#include "no_alloc.h"

static __device__ __align__(256) float g_noalloc_scratch[SB_NOALLOC_MAX_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};   // device address of the array, per device
}  // namespace

extern "C" int sb_attention_decode_mma_noalloc(void* out, const void* q, const void* k_pool, const void* v_pool,
                                               const int* block_table, int table_width, const int* token_rows,
                                               const int* positions, int tokens, int query_heads, int kv_heads,
                                               int head_dim, int page_size, int window, float scale,
                                               int num_partitions, cudaStream_t stream) {
    SB_REQUIRE(sb_attention_mma_supports(query_heads, kv_heads, head_dim, page_size, 1),
               "attention (no-alloc): Hq=%d Hkv=%d head_dim=%d is not supported", query_heads, kv_heads, head_dim);
    SB_REQUIRE(tokens > 0 && tokens <= 65535 && window >= 0 && table_width > 0 && table_width <= kMaxTableWidth,
               "attention (no-alloc): bad sizes tokens=%d table_width=%d", tokens, table_width);
    SB_REQUIRE(num_partitions >= 1 && num_partitions <= 65535, "attention (no-alloc): %d partitions",
               num_partitions);
    const long long slots = (long long)tokens * query_heads * num_partitions;
    const long long need = slots * (head_dim + 2);
    SB_REQUIRE(need <= (long long)SB_NOALLOC_MAX_FLOATS,
               "attention (no-alloc): tokens*heads*partitions*(head_dim+2) = %lld floats exceed the built-in "
               "scratch of %d floats; use fewer partitions or the entry point that takes scratch buffers",
               need, SB_NOALLOC_MAX_FLOATS);
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) { sb_set_error("attention (no-alloc): %s", cudaGetErrorString(e)); return (int)e; }
    SB_REQUIRE(device >= 0 && device < kMaxDevices, "attention (no-alloc): device %d is not supported", device);
    if (g_noalloc_ptr[device] == nullptr) {
        // Once per device, with that device current: the array's address on THIS device.
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr) {
            sb_set_error("attention (no-alloc): cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : SB_ERR_ARG;
        }
        g_noalloc_ptr[device] = p;
    }
    float* part_o = g_noalloc_ptr[device];                     // [tokens, heads, partitions, head_dim]
    float* part_ml = part_o + slots * head_dim;                // [tokens, heads, partitions, 2]
    int rc;
    switch (head_dim) {
        case 16: rc = launch_decode<16>(out, part_o, part_ml, q, k_pool, v_pool, block_table, table_width, token_rows, positions, tokens, query_heads, kv_heads, page_size, window, scale, num_partitions, stream); break;
        case 32: rc = launch_decode<32>(out, part_o, part_ml, q, k_pool, v_pool, block_table, table_width, token_rows, positions, tokens, query_heads, kv_heads, page_size, window, scale, num_partitions, stream); break;
        case 64: rc = launch_decode<64>(out, part_o, part_ml, q, k_pool, v_pool, block_table, table_width, token_rows, positions, tokens, query_heads, kv_heads, page_size, window, scale, num_partitions, stream); break;
        default: rc = launch_decode<128>(out, part_o, part_ml, q, k_pool, v_pool, block_table, table_width, token_rows, positions, tokens, query_heads, kv_heads, page_size, window, scale, num_partitions, stream); break;
    }
    if (rc != 0) return rc;
    SB_LAUNCH_CHECK();
}
