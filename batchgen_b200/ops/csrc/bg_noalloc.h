// Allocation-free entry point of the kernel library.
//
// This entry point has no counterpart in the reference engine.  It exists for callers that are not
// allowed to allocate device memory at the time they need attention computed: code running between
// the begin and end of a CUDA stream capture, real-time or interrupt-style serving loops that must
// not take the allocator lock, and embedders whose memory budget was fixed at start-up and who cannot
// accept a cudaMalloc (an implicit device synchronisation, and a possible failure) on the request path.
//
// bg_mla_decode_split_noalloc computes exactly what the split-KV path of bg_mla_attention + bg_mla_merge
// computes (paged absorbed multi-head latent attention for one query token per sequence, with the KV
// range of every sequence cut into `num_splits` parts that are merged afterwards), but the split
// partials, the work list and the merge list live in one file-scope device array of the library
// instead of buffers the caller has to provide.
//
//   * Limit: batch * (heads / heads_per_group) * num_splits <= BG_NOALLOC_MAX_WORK (256).  Larger
//     problems are refused with BG_NOALLOC_E_TOO_LARGE and nothing is launched.
//   * Cost: the array is about 16.9 MB and is held by every GPU that loads the library, until the
//     process exits.
//   * The first call on a device resolves the array's device address (cudaGetSymbolAddress) and sets the
//     shared-memory attribute of both column variants of the kernel on that device.  Make that first call
//     before any stream capture begins on that device.
//   * Every call shares the one array, which keeps the contents of the previous call.  Each call first
//     resets the (max, sum) pair of every partial it owns to "empty", and the kernels overwrite every
//     other word they later read.  Two calls whose kernels can overlap on the GPU (different streams
//     without an ordering between them) race on it: serialise them.
//   * Pass a non-null `status` when the result must be trusted: a CTA whose bounded wait ran out writes
//     no partial (the merge then leaves it out) and raises *status; with a null `status` nothing tells
//     the caller that the output misses part of the KV range.
//   * The call itself calls no cudaMalloc / cudaFree and no allocating library routine.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BG_NOALLOC_MAX_WORK 256
#define BG_NOALLOC_E_TOO_LARGE (-20)
#define BG_NOALLOC_E_BAD_SHAPE (-21)
#define BG_NOALLOC_E_SETUP (-22)

// q_abs: [B*H, 512] bf16 contiguous.  q_pe: [B*H, 64] bf16, row stride `qpe_stride` elements.
// cache: [cache_rows, 576] bf16 (64-token pages).  block_table: [B, bt_stride] int32.  seqlens: [B] int32.
// out: [B*H, 512] bf16.  status (may be null): device int raised when a bounded wait expires.
// Returns 0 when all three kernels were launched on `stream`.
int bg_mla_decode_split_noalloc(const void* q_abs, const void* q_pe, long long qpe_stride, int B, int H,
                                const void* cache, long long cache_rows, const int* block_table, int bt_stride,
                                const int* seqlens, void* out, int num_splits, float scale, int* status,
                                cudaStream_t stream);

// Text for a return code of the call above.
const char* bg_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
