// Tile code shared by the mma.sync attention kernels (bfloat16, m16n8k16, float32
// accumulation): copies of key and value tiles into swizzled shared memory, the warp's
// score / softmax / P.V step with the queries on the accumulator rows (prompt portions)
// and with the keys on the rows (decode tokens).  Included by attention_mma.cu and
// attention_decode.cu; everything sits in an anonymous namespace of the including file.
#pragma once

#include <math.h>

#include "common.cuh"

using namespace sb;
typedef __nv_bfloat16 bf16;

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


}  // namespace
