/* Decode attention for callers that cannot allocate device memory.
 *
 * This entry point has no counterpart in the reference (andrei-borcea/liyab); it
 * exists for users of this library who reach it only through its C symbols and
 * have no allocator to hand it scratch from: an FFI binding or a plugin host that
 * gave the whole device to a pool of its own, or a latency-critical loop in which
 * cudaMalloc (which synchronises the device) must never run.  It is
 * lb_decode_attention (api.h) with the scratch memory of the key split taken from
 * an array that is part of the library itself.
 *
 * What to know before calling it:
 *  - It allocates nothing: no cudaMalloc, cudaFree or any allocating library call.
 *    The scratch is a file-scope device array of LB_NOALLOC_SCRATCH_FLOATS floats
 *    plus LB_NOALLOC_COUNTER_INTS ints (about 4.02 MiB); every GPU that loads the
 *    library holds that much until the process exits.
 *  - Limits: n_seq * n_head * n_splits * (head_dim + 2) <= LB_NOALLOC_SCRATCH_FLOATS
 *    and n_seq * n_kv_head <= LB_NOALLOC_COUNTER_INTS; anything larger is refused
 *    with LB_ERR_INVALID_ARGUMENT (1) and a message (lb_last_error) that names the
 *    limit.  A call with n_splits = 1 uses no scratch, so neither limit applies to it.
 *    Shapes that lb_decode_attention_supports refuses are refused here too.
 *  - The first call on each device looks up the array's device address (once per
 *    device, with that device current).  Make that first call before any stream
 *    capture begins.
 *  - All calls share the one array, and it keeps whatever the last call left in
 *    it.  The entry point clears the counters that must start at zero on `stream`
 *    before it launches.  Two calls whose work overlaps on the GPU (different
 *    streams, no ordering between them) race on the scratch and give wrong results:
 *    order them, or use lb_decode_attention with scratch of your own.
 *
 * Arguments are those of lb_decode_attention without `partial` and `counters`.
 */
#pragma once

#include <stdint.h>

#define LB_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define LB_NOALLOC_COUNTER_INTS 4096

#ifdef __cplusplus
extern "C" {
#endif

int lb_decode_attention_noalloc(const void* q, int64_t q_stride, const void* cache, const int32_t* positions,
                                const int32_t* block_table, int table_stride, void* out, int64_t out_stride, int n_seq,
                                int n_head, int n_kv_head, int head_dim, int page_size, float scale, int window,
                                int n_splits, void* stream);

#ifdef __cplusplus
}
#endif
