// Allocation-free variant of the single-GPU sparse MLA attention (see no_alloc_attention.h for who needs it
// and for the rules of use).  The intermediates of the two-kernel attention (per-chunk partial outputs and
// softmax statistics) live in a file-scope device array instead of caller- or library-allocated memory.
#include "no_alloc_attention.h"

#include <cuda_runtime.h>
#include <mutex>

// The existing entry points of this library that do the work (attention.cu).  They only launch kernels.
extern "C" int glmb_attn_chunk(void);
extern "C" int glmb_sparse_mla_partial(const void* q_full, const void* kv_cache, const int* sel_local, const int* sel_counts,
                                       const int* row_lane, int rows, int H, int L, int rd, int layer, int layers, int local_cap,
                                       int top_k, int max_chunks, float scale, float* part_o, float* part_ml, const void* comm,
                                       int wait_sig, uint32_t* status, void* stream);
extern "C" int glmb_attn_local_merge(const float* part_o, const float* part_ml, const int* sel_counts, int rows, int H, int L,
                                     int top_k, int max_chunks, void* o_lat, int heads_local, int64_t xpart_offset,
                                     const void* comm, int sig, void* stream);

// The scratch itself.  In host code this name is only a stand-in for the device object: its device address
// is obtained once per device with cudaGetSymbolAddress and that pointer is what the kernels receive.
static __device__ __align__(256) float g_noalloc_scratch[GLMB_NOALLOC_SCRATCH_FLOATS];

#define NOALLOC_MAX_DEVICES 64
static float* g_scratch_ptr[NOALLOC_MAX_DEVICES];
static std::mutex g_scratch_mutex;

// Device address of the scratch array on the current device (resolved on the first call for that device).
static float* scratch_for_current_device(int* error) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) { *error = GLMB_NOALLOC_NO_SYMBOL; return nullptr; }
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_ptr[dev]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || !ptr) { *error = GLMB_NOALLOC_NO_SYMBOL; return nullptr; }
        g_scratch_ptr[dev] = static_cast<float*>(ptr);
    }
    return g_scratch_ptr[dev];
}

extern "C" __attribute__((visibility("default")))
int glmb_sparse_mla_attention_noalloc(const void* q_full, const void* kv_cache, const int* sel_local, const int* sel_counts,
                                      const int* row_lane, int rows, int H, int L, int rd, int layer, int layers, int local_cap,
                                      int top_k, float scale, void* o_lat, uint32_t* status, void* stream) {
    if (rows < 1 || H < 1 || L < 1 || top_k < 1 || rd < 0 || layers < 1 || layer < 0 || layer >= layers || local_cap < 1)
        return GLMB_NOALLOC_BAD_SHAPE;
    if (rows > GLMB_NOALLOC_MAX_ROWS || H > GLMB_NOALLOC_MAX_HEADS || L > GLMB_NOALLOC_MAX_LATENT || top_k > GLMB_NOALLOC_MAX_TOPK ||
        rd > GLMB_NOALLOC_MAX_ROPE)
        return GLMB_NOALLOC_TOO_LARGE;
    if ((L != 64 && L != 128 && L != 512) || ((L + rd) & 15)) return GLMB_NOALLOC_BAD_SHAPE;
    if (glmb_attn_chunk() != GLMB_NOALLOC_CHUNK) return GLMB_NOALLOC_BAD_SHAPE;
    const int max_chunks = (top_k + GLMB_NOALLOC_CHUNK - 1) / GLMB_NOALLOC_CHUNK;
    // layout inside the scratch: partial outputs [rows, max_chunks, H, L], then statistics [rows, max_chunks, H, 2]
    const size_t part_o_floats = (size_t)rows * max_chunks * H * L;
    const size_t part_ml_floats = (size_t)rows * max_chunks * H * 2;
    if (part_o_floats + part_ml_floats > (size_t)GLMB_NOALLOC_SCRATCH_FLOATS) return GLMB_NOALLOC_TOO_LARGE;
    int error = 0;
    float* scratch = scratch_for_current_device(&error);
    if (!scratch) return error;
    float* part_o = scratch;
    float* part_ml = scratch + part_o_floats;
    int code = glmb_sparse_mla_partial(q_full, kv_cache, sel_local, sel_counts, row_lane, rows, H, L, rd, layer, layers, local_cap,
                                       top_k, max_chunks, scale, part_o, part_ml, nullptr, -1, status, stream);
    // the inner entry points answer 1 (a shape they do not take) or 2 (a tile that does not fit shared memory) before they launch
    // anything; both are refusals of the shape, not CUDA errors.  Larger values are the cudaError_t of a launch.
    if (code == 1 || code == 2) return GLMB_NOALLOC_BAD_SHAPE;
    if (code != 0) return code;
    code = glmb_attn_local_merge(part_o, part_ml, sel_counts, rows, H, L, top_k, max_chunks, o_lat, H, 0, nullptr, 0, stream);
    return (code == 1 || code == 2) ? GLMB_NOALLOC_BAD_SHAPE : code;
}

extern "C" __attribute__((visibility("default")))
const char* glmb_noalloc_strerror(int code) {
    switch (code) {
        case GLMB_NOALLOC_OK: return "ok";
        case GLMB_NOALLOC_TOO_LARGE:
            return "problem exceeds the built-in scratch: at most 2 rows, 64 heads, latent 512, rope 256, top_k 2048 per call";
        case GLMB_NOALLOC_BAD_SHAPE:
            return "unsupported shape: counts must be positive, rope width non-negative, latent 64, 128 or 512 and latent + rope width a multiple of 16";
        case GLMB_NOALLOC_NO_SYMBOL: return "the scratch array could not be resolved on the current device";
        default: return code > 0 ? "CUDA error (the value is the cudaError_t of the failed call)" : "unknown code";
    }
}
