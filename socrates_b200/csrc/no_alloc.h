/* Decode attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference: there the split-key decode
 * kernel always takes its scratch from the framework's caching allocator
 * (model/kernels/csrc/paged_attention.cu:331-336).
 *
 * Who needs it.  Some users of this library run where cudaMalloc (or any allocating
 * call, torch's included) is not an option at the moment of the call: code that drives
 * the kernels from a plain C or C++ host program without a tensor library, a real-time
 * loop that must not enter the driver's allocator, or a process whose memory budget was
 * handed out completely at start-up.  The regular entry point,
 * sb_attention_decode_mma, asks such a caller for two float32 scratch buffers whenever
 * the keys are cut into more than one partition.  This variant brings its own: a
 * file-scope `static __device__` array inside the library.
 *
 * What it costs.  The array holds SB_NOALLOC_MAX_FLOATS floats (8 MiB).  Every GPU on
 * which the library is loaded keeps it until the process exits, whether or not this
 * entry point is ever called.
 *
 * Limits.  tokens * query_heads * partitions * (head_dim + 2) must not exceed
 * SB_NOALLOC_MAX_FLOATS; a larger call is refused with SB_ERR_ARG and a message in
 * sb_last_error(), nothing is launched.  Inputs and the output are still the caller's.
 *
 * First call.  The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current) and configures the kernel; make
 * that first call before any stream capture begins on that device.  The address is kept
 * in a plain per-device table without a lock: two host threads that both make a device's
 * first call look the same address up twice and store the same value, which is harmless.
 *
 * Sharing.  All calls on a device use the same array, and it keeps whatever the last
 * call left in it.  Nothing in it has to start at zero: every partition slot that is
 * read was written by the same call (empty partitions are marked as such).  Two calls
 * whose kernels may overlap on the GPU (different streams, or different host threads
 * without ordering) race on the array; order them on one stream.
 *
 * Arguments are those of sb_attention_decode_mma without the two scratch pointers:
 *   out, q          bfloat16 [tokens, query_heads * head_dim]
 *   k_pool, v_pool  bfloat16 [pages, kv_heads, page_size, head_dim]
 *   block_table     int32 [rows, table_width]
 *   token_rows      int32 [tokens]   cache row of each token
 *   positions       int32 [tokens]   position of each token; it sees keys 0..position
 *                                    (or the last `window` of them when window > 0)
 * Returns 0, SB_ERR_ARG, or a cudaError_t.
 */
#pragma once

#include <cuda_runtime.h>

#define SB_NOALLOC_MAX_FLOATS (2 * 1024 * 1024)

#ifdef __cplusplus
extern "C" {
#endif

int sb_attention_decode_mma_noalloc(void* out, const void* q, const void* k_pool, const void* v_pool,
                                    const int* block_table, int table_width, const int* token_rows,
                                    const int* positions, int tokens, int query_heads, int kv_heads,
                                    int head_dim, int page_size, int window, float scale,
                                    int num_partitions, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
