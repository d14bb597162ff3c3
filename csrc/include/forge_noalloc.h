/* Allocation-free decode attention (C interface).  No counterpart in the reference.
 *
 * For callers that cannot obtain device memory at the point where they need the kernel: host callbacks and
 * plug-ins that run inside another component's fixed memory plan, latency-critical loops that must stay away
 * from the allocator, processes whose pool is sized once and then frozen.  The split-context scratch that the
 * regular entry point (forge_decode_attention) takes from its caller is, here, a 16 MiB array built into the
 * library's device image; the caller passes inputs and outputs only.
 *
 *   - Limit: B * nq * max_chunks * 130 <= forge_decode_attention_noalloc_capacity_floats() (4 Mi floats).
 *     Beyond it the call returns FORGE_NOALLOC_TOO_LARGE (-20) and launches nothing.
 *   - Every GPU that loads the library holds the 16 MiB until the process exits.
 *   - The first call on a device resolves the array's device address (cudaGetSymbolAddress); make that call
 *     before any stream capture begins.
 *   - Calls on one device share the array: keep them ordered (same stream); overlapping calls race.
 *   - Nothing is allocated or freed on any path.
 *   - `stream` must belong to the device that is current at the call (the array's address and the kernels'
 *     shared-memory limit are resolved for the current device).
 *   - A context length that the block table or the slices cannot describe (greater than table_width * block_size
 *     or max_chunks * chunk) is clamped and reported through `status` (the bad-index bit, value 4); nothing is read out of range.
 *
 * Tensors (all device pointers, bf16 unless noted):
 *   q [B, nq, 128]; k_cache, v_cache [num_blocks, nkv, block_size, 128]; block_tables int32 [B, table_width];
 *   context_lens int32 [B]; out [B, nq * 128]; status: optional device word that collects error bits.
 *   chunk: tokens per context slice, a multiple of min(block_size, 64); max_chunks * chunk >= longest context.
 * Returns 0 on success, a negative code otherwise (see forge_decode_attention_noalloc_strerror).
 */
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

int forge_decode_attention_noalloc(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                                   const int* context_lens, void* out, int B, int nq, int nkv, int head_dim, int block_size,
                                   int table_width, int num_blocks, int chunk, int max_chunks, float scale, unsigned* status,
                                   cudaStream_t stream);
size_t forge_decode_attention_noalloc_capacity_floats(void);
const char* forge_decode_attention_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
