// Paged GQA attention of decode steps (every request brings one token), bfloat16, as ONE
// persistent kernel: warps pull work items and stream keys and values at their own pace.
//
// A work item is (token, KV head, chunk): the keys [c*CK, (c+1)*CK) of the token's row that the
// token may see, CK a fixed number of keys (a multiple of 16).  Where a chunk begins and ends
// depends on nothing but the key positions, so the numbers a request gets do not depend on how
// many other requests share the step or on how many SMs the GPU has (the reference splits its
// rows at fixed multiples of its partition size too, model/kernels/csrc/paged_attention.cu:80-96).
//
// One WARP owns an item: it copies the chunk in 16-key subtiles through a cp.async ring of its own
// (S stages), runs the transposed products of attention_mma.cuh on each (keys on the accumulator
// rows, the G query heads of the KV head on the columns) and keeps (max, sum, O) of the chunk in
// registers.  No barrier joins the warps of a block, and nothing is merged between warps: a warp
// whose chunk is the whole row writes the output itself; otherwise it writes the chunk's
// (max, sum, O) to scratch and counts itself in, and the warp that finds every chunk of its
// (token, KV head) counted merges them in chunk order and clears the counter for the next launch.
// The copy ring runs on across items: while the last subtiles of one item are computed the first
// of the next are already in flight, so a warp pays the latency of memory once, not once an item.
//
// Before it waits for the kernel that precedes it on the stream (programmatic dependent launch) a
// warp reads only what older kernels left: the block table, rows and positions (a host copy at the
// start of the step) and keys and values below the token's own position.  The query and the newest
// key and value come from the preceding kernel and are read after the wait.
//
// Keys outside a chunk's visible range are never read from the pool (their rows are zero-filled and
// their scores masked), so whatever a page's previous owner left in a slot cannot reach the result.
#include <math.h>
#include <stdlib.h>

#include "attention_mma.cuh"

namespace {

constexpr int kMaxTokens = 1024;                 // decode tokens of one launch (prefix sums in shared memory)

// Where a warp stands in its sequence of items: one cursor for the copies (ahead), one for the products.
struct Cursor {
    int item;                // index of the item, or -1 when the warp has no more
    int n, kh;               // token, KV head
    int c_rel, nc;           // this chunk among the token's chunks, and how many there are
    int pos;                 // the token's position (the newest key)
    int k_begin, k_end;      // visible keys of the chunk
    int sub, nsub;           // current 16-key subtile, and how many the chunk has
    int key0;                // first key slot of the current subtile (a multiple of 16)
    const int* table;        // the row's block table
    long long src;           // element offset of the subtile's first key row in the pools (one page: BS >= 16)
};

__device__ __forceinline__ void cursor_seek_subtile(Cursor& c, int bs_log2, int Hkv, int D) {
    c.key0 = (c.k_begin & ~15) + 16 * c.sub;
    const int page = c.table[c.key0 >> bs_log2];
    c.src = ((((long long)page * Hkv + c.kh) << bs_log2) + (c.key0 & ((1 << bs_log2) - 1))) * D;
}

// Item `item` of the launch: chunk g = item / Hkv of all tokens' chunks in token order, head item % Hkv.
__device__ __forceinline__ void cursor_load(Cursor& c, int item, int n_items, const int* prefix, int N, int Hkv,
                                            int CK, int window, const int* __restrict__ positions,
                                            const int* __restrict__ token_rows,
                                            const int* __restrict__ block_table, int table_width, int bs_log2,
                                            int D) {
    if (item >= n_items) { c.item = -1; return; }
    c.item = item;
    const int g = item / Hkv;
    c.kh = item - g * Hkv;
    int lo_n = 0, hi_n = N - 1;                  // the last n with prefix[n] <= g
    while (lo_n < hi_n) {
        const int mid = (lo_n + hi_n + 1) >> 1;
        if (prefix[mid] <= g) lo_n = mid; else hi_n = mid - 1;
    }
    c.n = lo_n;
    c.pos = positions[c.n];
    const int hi = c.pos + 1;
    const int lo = (window > 0 && hi > window) ? hi - window : 0;
    const int first = lo / CK;
    c.nc = (hi - 1) / CK - first + 1;
    c.c_rel = g - prefix[c.n];
    const int chunk = first + c.c_rel;
    c.k_begin = max(lo, chunk * CK);
    c.k_end = min(hi, (chunk + 1) * CK);
    c.sub = 0;
    c.nsub = ((c.k_end + 15) >> 4) - (c.k_begin >> 4);
    c.table = block_table + (size_t)token_rows[c.n] * table_width;
    cursor_seek_subtile(c, bs_log2, Hkv, D);
}

// Dose `part` (0..3) of the copies of the cursor's subtile into one ring stage: a lane always
// copies the same 16-byte column of the rows it serves.
template <int D>
__device__ __forceinline__ void copy_subtile_part(int part, bf16* ks, bf16* vs, const bf16* __restrict__ k_pool,
                                                  const bf16* __restrict__ v_pool, const Cursor& c, int lane) {
    constexpr int CH = D / 8;                    // 16-byte columns of a row
    constexpr int ROWS = 32 / CH;                // rows served per pass
    constexpr int IT = 16 / ROWS;                // passes per subtile
    const int col = lane % CH, r0 = lane / CH;
#pragma unroll
    for (int it = 0; it < IT; ++it) {
        if (it * 4 / IT != part) continue;
        const int row = r0 + it * ROWS;
        const int kpos = c.key0 + row;
        const bool valid = kpos >= c.k_begin && kpos < c.k_end;
        const long long src = valid ? c.src + (long long)row * D + col * 8 : 0;
        const int off = tile_off<D>(row, col);
        cp_async16(smem_u32(ks + off), k_pool + src, valid ? 16 : 0);
        cp_async16(smem_u32(vs + off), v_pool + src, valid ? 16 : 0);
    }
}

// Merge of the nc chunks of G heads by one warp: out[g,:] = sum_c 2^(m_c - M) o_c / sum_c 2^(m_c - M) l_c,
// M = max_c m_c, terms added in chunk order.  Every chunk 0..nc-1 holds at least one visible key, so
// every slot was written by this launch.  A lane owns four consecutive dims (D/4 lanes work); the
// loads of two heads x four chunks go out together, so the merge costs a few round trips to L2
// however many chunks there are.
template <int D>
__device__ __forceinline__ void merge_chunks(bf16* __restrict__ out, const float* __restrict__ part_o,
                                             const float* __restrict__ part_ml, size_t slot0, int NCmax,
                                             size_t out0, int G, int nc, int lane) {
    constexpr int HB = 2, CB = 4;                // heads and chunks whose loads are in flight together
    const float2* ml = reinterpret_cast<const float2*>(part_ml);
    const bool active = lane * 4 < D;
    for (int g0 = 0; g0 < G; g0 += HB) {
        float M[HB];
#pragma unroll
        for (int u = 0; u < HB; ++u) {
            M[u] = -INFINITY;
            if (g0 + u < G)
                for (int c = lane; c < nc; c += 32) M[u] = fmaxf(M[u], __ldcg(ml + slot0 + (size_t)(g0 + u) * NCmax + c).x);
        }
#pragma unroll
        for (int u = 0; u < HB; ++u)
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) M[u] = fmaxf(M[u], __shfl_xor_sync(0xffffffffu, M[u], d));
        float4 acc[HB];
        float L[HB];
#pragma unroll
        for (int u = 0; u < HB; ++u) { acc[u] = make_float4(0.f, 0.f, 0.f, 0.f); L[u] = 0.f; }
        for (int c0 = 0; c0 < nc; c0 += CB) {
            float2 v[HB][CB];
            float4 x[HB][CB];
#pragma unroll
            for (int u = 0; u < HB; ++u)
#pragma unroll
                for (int t = 0; t < CB; ++t) {
                    const bool on = g0 + u < G && c0 + t < nc;
                    const size_t slot = slot0 + (size_t)(g0 + u) * NCmax + c0 + t;
                    v[u][t] = on ? __ldcg(ml + slot) : make_float2(-INFINITY, 0.f);
                    x[u][t] = (on && active) ? __ldcg(reinterpret_cast<const float4*>(part_o + slot * D) + lane)
                                             : make_float4(0.f, 0.f, 0.f, 0.f);
                }
#pragma unroll
            for (int u = 0; u < HB; ++u)
#pragma unroll
                for (int t = 0; t < CB; ++t) {
                    const float w = v[u][t].y > 0.f ? ex2_approx(v[u][t].x - M[u]) : 0.f;
                    L[u] += w * v[u][t].y;
                    acc[u].x += w * x[u][t].x;
                    acc[u].y += w * x[u][t].y;
                    acc[u].z += w * x[u][t].z;
                    acc[u].w += w * x[u][t].w;
                }
        }
#pragma unroll
        for (int u = 0; u < HB; ++u) {
            if (g0 + u >= G || !active) continue;
            const float inv = 1.0f / L[u];
            uint2 packed;
            packed.x = pack_bf16(acc[u].x * inv, acc[u].y * inv);
            packed.y = pack_bf16(acc[u].z * inv, acc[u].w * inv);
            *reinterpret_cast<uint2*>(out + out0 + (size_t)(g0 + u) * D + lane * 4) = packed;
        }
    }
}

template <int D, int NW, int S, int NBQ>
__global__ void __launch_bounds__(32 * NW, (NW * S * 2 * 16 * D * 2 + 8192) * 2 <= 227 * 1024 ? (NW <= 4 && (NW * S * 2 * 16 * D * 2 + 8192) * 3 <= 227 * 1024 ? 3 : 2) : 1)
attn_decode_stream_kernel(bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                          int* __restrict__ counters, const bf16* __restrict__ q, const bf16* __restrict__ k_pool,
                          const bf16* __restrict__ v_pool, const int* __restrict__ block_table, int table_width,
                          const int* __restrict__ token_rows, const int* __restrict__ positions, int N, int Hq,
                          int Hkv, int BS, int window, float scale_log2, int CK, int NCmax) {
    sb::pdl_launch_dependents();                 // the next kernel may begin its prologue
    constexpr int STAGE = 16 * D;                // elements of one stage of K (and of V)
    extern __shared__ __align__(128) uint8_t smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    bf16* ring = reinterpret_cast<bf16*>(smem) + (size_t)warp * S * 2 * STAGE;      // [S][K | V]
    int* prefix = reinterpret_cast<int*>(reinterpret_cast<bf16*>(smem) + (size_t)NW * S * 2 * STAGE);   // [N + 1]

    // ---- chunks per token and their running sum (positions are older than the preceding kernel)
    for (int n = threadIdx.x; n < N; n += 32 * NW) {
        const int hi = positions[n] + 1;
        const int lo = (window > 0 && hi > window) ? hi - window : 0;
        prefix[n + 1] = (hi - 1) / CK - lo / CK + 1;
    }
    __syncthreads();
    if (warp == 0) {
        int carry = 0;
        for (int base = 0; base < N; base += 32) {
            int v = base + lane < N ? prefix[base + lane + 1] : 0;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int u = __shfl_up_sync(0xffffffffu, v, d);
                if (lane >= d) v += u;
            }
            if (base + lane < N) prefix[base + lane + 1] = carry + v;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
        if (lane == 0) prefix[0] = 0;
    }
    __syncthreads();                             // the only barriers of the kernel
    const int n_items = prefix[N] * Hkv;
    const int worker = blockIdx.x * NW + warp, workers = gridDim.x * NW;
    if (worker >= n_items) return;

    const int G = Hq / Hkv;
    const int bs_log2 = 31 - __clz(BS);
    Cursor prod, cons;
    cursor_load(prod, worker, n_items, prefix, N, Hkv, CK, window, positions, token_rows, block_table, table_width,
                bs_log2, D);
    cons = prod;

    auto advance = [&](Cursor& c) {
        if (c.item < 0) return;
        if (++c.sub < c.nsub) cursor_seek_subtile(c, bs_log2, Hkv, D);
        else cursor_load(c, c.item + workers, n_items, prefix, N, Hkv, CK, window, positions, token_rows,
                         block_table, table_width, bs_log2, D);
    };

    // ---- fill the ring.  A subtile that holds its token's newest key is written by the preceding
    // kernel: it is copied only after the wait.
    bool waited = false;
#pragma unroll
    for (int s = 0; s < S - 1; ++s) {
        if (prod.item >= 0) {
            if (!waited && prod.key0 + 16 > prod.pos) { sb::pdl_wait(); waited = true; }
#pragma unroll
            for (int p = 0; p < 4; ++p)
                copy_subtile_part<D>(p, ring + (s * 2) * STAGE, ring + (s * 2 + 1) * STAGE, k_pool, v_pool, prod, lane);
        }
        cp_async_commit();
        advance(prod);
    }
    if (!waited) sb::pdl_wait();                 // everything before this kernel is complete and visible

    ColState<D, NBQ> st;
    uint32_t qf[D / 16][4];
    for (int j = 0; cons.item >= 0; ++j) {
        if (cons.sub == 0) {
            // ---- a new item: its query heads straight from global memory in the B-operand layout
            // (head lane/4 (+8), dims 16kk + 2*(lane%4) (+8)); heads past the group are zero
            st.init();
            const int h0 = cons.kh * G;
            const int hA = lane >> 2, hB = 8 + (lane >> 2);
            const bf16* qa = q + ((size_t)cons.n * Hq + h0 + hA) * D + 2 * (lane & 3);
            const bf16* qb = q + ((size_t)cons.n * Hq + h0 + hB) * D + 2 * (lane & 3);
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                qf[kk][0] = hA < G ? *reinterpret_cast<const uint32_t*>(qa + 16 * kk) : 0u;
                qf[kk][2] = hA < G ? *reinterpret_cast<const uint32_t*>(qa + 16 * kk + 8) : 0u;
                qf[kk][1] = (NBQ == 2 && hB < G) ? *reinterpret_cast<const uint32_t*>(qb + 16 * kk) : 0u;
                qf[kk][3] = (NBQ == 2 && hB < G) ? *reinterpret_cast<const uint32_t*>(qb + 16 * kk + 8) : 0u;
            }
        }
        cp_async_wait<S - 2>();                  // this lane's share of subtile j has landed
        __syncwarp();                            // ... and every lane's
        const int slot = j % S, fill = (j + S - 1) % S;      // `fill` was read by the products of subtile j - 1
        auto between = [&](int p) {
            if (prod.item >= 0)
                copy_subtile_part<D>(p, ring + (fill * 2) * STAGE, ring + (fill * 2 + 1) * STAGE, k_pool, v_pool,
                                     prod, lane);
        };
        const bool masked = cons.key0 < cons.k_begin || cons.key0 + 16 > cons.k_end;
        warp_tile_decode<D, NBQ>(st, qf, ring + (slot * 2) * STAGE, ring + (slot * 2 + 1) * STAGE, 0, cons.key0,
                                 cons.pos, cons.k_begin, cons.k_end, scale_log2, masked, between);
        cp_async_commit();
        advance(prod);

        if (cons.sub == cons.nsub - 1) {
            // ---- the chunk is done: (max, sum, O) of the group's heads are in this warp's registers
            const int h0 = cons.kh * G;
            const size_t slot0 = ((size_t)cons.n * Hq + h0) * NCmax + cons.c_rel;    // + head * NCmax
#pragma unroll
            for (int nb = 0; nb < NBQ; ++nb) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int c = 2 * nb + e;
                    float l = st.l[c];
                    l += __shfl_xor_sync(0xffffffffu, l, 4);
                    l += __shfl_xor_sync(0xffffffffu, l, 8);
                    l += __shfl_xor_sync(0xffffffffu, l, 16);
                    const int head = 8 * nb + 2 * (lane & 3) + e;
                    if (head >= G) continue;
                    if (cons.nc == 1) {
                        const float inv = 1.0f / l;
                        bf16* dst = out + ((size_t)cons.n * Hq + h0 + head) * D + (lane >> 2);
#pragma unroll
                        for (int mb = 0; mb < D / 16; ++mb) {
                            dst[mb * 16] = __float2bfloat16_rn(st.o[mb][nb][e] * inv);
                            dst[mb * 16 + 8] = __float2bfloat16_rn(st.o[mb][nb][e + 2] * inv);
                        }
                    } else {
                        float* dst = part_o + (slot0 + (size_t)head * NCmax) * D + (lane >> 2);
#pragma unroll
                        for (int mb = 0; mb < D / 16; ++mb) {
                            dst[mb * 16] = st.o[mb][nb][e];
                            dst[mb * 16 + 8] = st.o[mb][nb][e + 2];
                        }
                        if (lane < 4) {
                            float* ml = part_ml + (slot0 + (size_t)head * NCmax) * 2;
                            ml[0] = st.m[c] * scale_log2;     // exponent of the reference maximum, base 2
                            ml[1] = l;
                        }
                    }
                }
            }
            if (cons.nc > 1) {
                // count this chunk in; whoever completes the count merges (in chunk order, whoever it is)
                __threadfence();
                __syncwarp();
                int before = 0;
                if (lane == 0) before = atomicAdd(counters + cons.n * Hkv + cons.kh, 1);
                before = __shfl_sync(0xffffffffu, before, 0);
                if (before == cons.nc - 1) {
                    __threadfence();
                    merge_chunks<D>(out, part_o, part_ml, ((size_t)cons.n * Hq + h0) * NCmax, NCmax,
                                    ((size_t)cons.n * Hq + h0) * D, G, cons.nc, lane);
                    if (lane == 0) counters[cons.n * Hkv + cons.kh] = 0;     // ready for the next launch
                }
            }
        }
        advance(cons);
    }
    cp_async_wait<0>();
}

// Variants of the kernel: (warps a block, ring stages); shared memory decides how many blocks fit an SM.
//   0: (13, 2), one block an SM   1: (4, 2), three   2: (4, 3), two   3: (6, 2), two   4: (10, 2), one
constexpr int kVariants = 5;

template <int D, int NW, int S, int NBQ>
int launch_v(void* out, float* part_o, float* part_ml, int* counters, const void* q, const void* k_pool,
             const void* v_pool, const int* block_table, int table_width, const int* token_rows,
             const int* positions, int N, int Hq, int Hkv, int BS, int window, float scale, int CK, int NCmax,
             cudaStream_t stream) {
    auto kernel = attn_decode_stream_kernel<D, NW, S, NBQ>;
    constexpr int ring = NW * S * 2 * 16 * D * 2;
    const int smem = ring + (kMaxTokens + 1) * 4;
    static sb::OncePerDevice once_per_device;
    static int blocks_per_sm = 0, num_sms = 0;
    bool& configured = once_per_device.flag();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks_per_sm, kernel, 32 * NW, smem);
        int dev = 0;
        if (e == cudaSuccess) e = cudaGetDevice(&dev);
        if (e == cudaSuccess) e = cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess || blocks_per_sm < 1) {
            sb_set_error("attention_decode: %s", cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : SB_ERR_ARG;
        }
        configured = true;
    }
    // no more blocks than could ever have an item (the host does not know the rows' lengths)
    const long long most_items = (long long)N * Hkv * NCmax;
    const long long blocks = min((long long)num_sms * blocks_per_sm, (most_items + NW - 1) / NW);
    sb::launch(kernel, dim3((unsigned)blocks), dim3(32 * NW), smem, stream, (bf16*)out, part_o, part_ml, counters,
               (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, block_table, table_width, token_rows,
               positions, N, Hq, Hkv, BS, window, scale * LOG2E, CK, NCmax);
    return 0;
}

template <int D>
int launch(int variant, void* out, float* part_o, float* part_ml, int* counters, const void* q, const void* k_pool,
           const void* v_pool, const int* block_table, int table_width, const int* token_rows, const int* positions,
           int N, int Hq, int Hkv, int BS, int window, float scale, int CK, int NCmax, cudaStream_t stream) {
#define SB_DEC(NW, S, NBQ) launch_v<D, NW, S, NBQ>(out, part_o, part_ml, counters, q, k_pool, v_pool, block_table, \
                                                   table_width, token_rows, positions, N, Hq, Hkv, BS, window, scale, \
                                                   CK, NCmax, stream)
    const bool wide = Hq / Hkv > 8;              // query heads of a KV head: one block of 8 columns, or two
    switch (variant) {
        case 1: return wide ? SB_DEC(4, 2, 2) : SB_DEC(4, 2, 1);
        case 2: return wide ? SB_DEC(4, 3, 2) : SB_DEC(4, 3, 1);
        case 3: return wide ? SB_DEC(6, 2, 2) : SB_DEC(6, 2, 1);
        case 4: return wide ? SB_DEC(10, 2, 2) : SB_DEC(10, 2, 1);
        default: return wide ? SB_DEC(13, 2, 2) : SB_DEC(13, 2, 1);
    }
#undef SB_DEC
}

}  // namespace

// 1 if the streaming decode kernel takes this shape (bfloat16 only), else 0.
extern "C" int sb_attention_decode_stream_supports(int Hq, int Hkv, int D, int page_size) {
    if (Hq <= 0 || Hkv <= 0 || Hq % Hkv || Hq / Hkv > 16) return 0;
    if (!(D == 16 || D == 32 || D == 64 || D == 128)) return 0;
    return page_size >= 16 && (page_size & (page_size - 1)) == 0;    // a 16-key subtile lies in one page
}

// Decode attention over `chunk_keys`-key chunks (a multiple of 16).  Scratch: part_o
// [N, Hq, max_chunks, D] and part_ml [N, Hq, max_chunks, 2] float32, counters [N * Hkv] int32 that
// are ZERO at the first call (the kernel leaves them zero); max_chunks bounds the chunks any
// token's visible keys may span.  What must be older than the preceding kernel: see the file header.
extern "C" int sb_attention_decode_stream(void* out, float* part_o, float* part_ml, int* counters, const void* q,
                                          const void* k_pool, const void* v_pool, const int* block_table,
                                          int table_width, const int* token_rows, const int* positions, int N,
                                          int Hq, int Hkv, int D, int page_size, int window, float scale,
                                          int chunk_keys, int max_chunks, int variant, cudaStream_t stream) {
    SB_REQUIRE(sb_attention_decode_stream_supports(Hq, Hkv, D, page_size),
               "attention_decode: Hq=%d Hkv=%d head_dim=%d page_size=%d is not supported", Hq, Hkv, D, page_size);
    SB_REQUIRE(N > 0 && N <= kMaxTokens && window >= 0 && table_width > 0,
               "attention_decode: bad sizes N=%d (at most %d tokens a launch)", N, kMaxTokens);
    SB_REQUIRE(chunk_keys >= 16 && chunk_keys % 16 == 0 && max_chunks >= 1,
               "attention_decode: chunks of %d keys (a multiple of 16), at most %d of them", chunk_keys, max_chunks);
    SB_REQUIRE(max_chunks == 1 || (part_o != nullptr && part_ml != nullptr && counters != nullptr),
               "attention_decode: rows of up to %d chunks need scratch buffers", max_chunks);
    if (variant < 0 || variant >= kVariants) variant = 0;
    int rc;
    switch (D) {
        case 16: rc = launch<16>(variant, out, part_o, part_ml, counters, q, k_pool, v_pool, block_table, table_width, token_rows, positions, N, Hq, Hkv, page_size, window, scale, chunk_keys, max_chunks, stream); break;
        case 32: rc = launch<32>(variant, out, part_o, part_ml, counters, q, k_pool, v_pool, block_table, table_width, token_rows, positions, N, Hq, Hkv, page_size, window, scale, chunk_keys, max_chunks, stream); break;
        case 64: rc = launch<64>(variant, out, part_o, part_ml, counters, q, k_pool, v_pool, block_table, table_width, token_rows, positions, N, Hq, Hkv, page_size, window, scale, chunk_keys, max_chunks, stream); break;
        default: rc = launch<128>(variant, out, part_o, part_ml, counters, q, k_pool, v_pool, block_table, table_width, token_rows, positions, N, Hq, Hkv, page_size, window, scale, chunk_keys, max_chunks, stream); break;
    }
    if (rc != 0) return rc;
    SB_LAUNCH_CHECK();
}
