// Sparse MLA attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference engine.  It exists for hosts that drive the
// library from a context where cudaMalloc is off limits: a real-time or safety-partitioned process whose
// memory is fixed at start-up, a plug-in that runs inside another framework's memory pool and may not
// touch the driver allocator, or a latency-critical loop in which the implicit synchronisation of
// cudaMalloc/cudaFree is unacceptable.  Such callers own their input and output buffers, but they cannot
// provide the intermediate buffers the attention kernels need (the per-chunk partial outputs and softmax
// statistics), and they cannot let the library create them on demand.
//
// glmb_sparse_mla_attention_noalloc computes the same result as glmb_sparse_mla_partial followed by
// glmb_attn_local_merge on one GPU, but keeps the intermediates in a fixed array that is part of the
// library image (file scope, `static __device__`), so no allocation happens at any time:
//
//   * neither this function nor anything it calls uses cudaMalloc, cudaFree or an allocating library routine;
//   * the array is GLMB_NOALLOC_SCRATCH_BYTES large on EVERY GPU that loads the library, from load to exit;
//   * problem sizes whose intermediates would not fit are refused (see the limits below);
//   * the first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device
//     current).  Make that first call outside of any stream capture; later calls only launch kernels;
//   * all calls on a device share the one array, which keeps whatever the last call left in it.  Nothing in
//     it needs to start at zero (every element that is read has been written by the same call), but two calls
//     whose kernels overlap on the GPU -- different streams, or different host threads -- would overwrite each
//     other's intermediates: issue calls for one device on one stream, or order them yourself.
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Limits of the built-in scratch array.
#define GLMB_NOALLOC_MAX_ROWS 2      // query rows per call
#define GLMB_NOALLOC_MAX_HEADS 64    // heads
#define GLMB_NOALLOC_MAX_LATENT 512  // kv_lora_rank
#define GLMB_NOALLOC_MAX_TOPK 2048   // selected keys per row
#define GLMB_NOALLOC_CHUNK 64        // keys per partial (must equal glmb_attn_chunk())
#define GLMB_NOALLOC_SCRATCH_FLOATS \
    ((GLMB_NOALLOC_MAX_ROWS) * (GLMB_NOALLOC_MAX_TOPK / GLMB_NOALLOC_CHUNK) * (GLMB_NOALLOC_MAX_HEADS) * (GLMB_NOALLOC_MAX_LATENT + 2))
#define GLMB_NOALLOC_SCRATCH_BYTES (4ull * GLMB_NOALLOC_SCRATCH_FLOATS)  // about 8.4 MB per GPU

#define GLMB_NOALLOC_MAX_ROPE 256     // rope width (q_full and the cache rows are latent + rope wide)

// Return codes.  The entry point's own refusals are negative, so they cannot be mistaken for a cudaError_t (all positive).
#define GLMB_NOALLOC_OK 0
#define GLMB_NOALLOC_TOO_LARGE (-1)   // rows, heads, latent width, rope width or top_k beyond the limits above
#define GLMB_NOALLOC_BAD_SHAPE (-2)   // a size the attention kernels do not support: a count below 1, rd below 0, a latent other than
                                      // 64, 128 or 512, latent + rope not a multiple of 16
#define GLMB_NOALLOC_NO_SYMBOL (-3)   // the scratch array's address could not be resolved on this device
// Any positive value is the cudaError_t of a failed launch.

// q_full     [rows, H, L + rd] bf16   absorbed queries (q_c | q_rope)
// kv_cache   [lanes, layers, local_cap, L + rd] bf16
// sel_local  [rows, top_k] int32      cache rows to attend, ascending
// sel_counts [rows, 2] int32          element 1 of each pair = number of valid entries of sel_local
// row_lane   [rows] int32             lane (chat) of each query row
// o_lat      [rows, H, L] bf16        output: normalized attention over the latent; zeros for an empty row
// status     device uint32 or NULL    receives GLMB_STATUS_* bits (clamped index, non-finite score)
// All pointers are device pointers on the current device; the work is enqueued on `stream`.
int glmb_sparse_mla_attention_noalloc(const void* q_full, const void* kv_cache, const int* sel_local, const int* sel_counts,
                                      const int* row_lane, int rows, int H, int L, int rd, int layer, int layers, int local_cap,
                                      int top_k, float scale, void* o_lat, uint32_t* status, void* stream);

// A one-line description of a return code of the function above.
const char* glmb_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
