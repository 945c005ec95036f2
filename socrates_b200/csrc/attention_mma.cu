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

#include "attention_mma.cuh"

extern "C" int sb_attention_decode_mma_kernels(int num_partitions);

namespace {

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
