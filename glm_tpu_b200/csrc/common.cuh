// Shared device helpers for every kernel of the engine (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#define GLMB_API extern "C" __attribute__((visibility("default")))

typedef __nv_bfloat16 bf16;

// Bits of the device status word. A kernel never traps: it records the condition here, finishes
// with defined (if meaningless) outputs, and the host reads the word after the step.
enum : uint32_t {
    GLMB_STATUS_WAIT_TIMEOUT = 1u,   // a bounded wait on a peer flag or an mbarrier ran out
    GLMB_STATUS_BAD_INDEX = 2u,      // an index was outside its table and was clamped
    GLMB_STATUS_NONFINITE = 4u,      // a score or logit was NaN or infinite
    GLMB_STATUS_BAD_SHAPE = 8u,      // a launch was refused because a size exceeds a compiled limit
};

#define GLMB_MAX_WORLD 8
#define GLMB_MAX_ROWS 8  // rows (lanes) handled by the skinny decode kernels in one pass

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// The two bf16 halves of a packed 32-bit word, widened to fp32 (exact).
__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// 16-byte streaming load of weights: read-only path, no L1 allocation (weights are read once per step).
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// 16-byte load of a small, hot operand (activations): cached in L1.
__device__ __forceinline__ uint4 ld_hot16(const void* p) { return *reinterpret_cast<const uint4*>(p); }

// Two e4m3 bytes (low 16 bits of v) widened to fp32 (exact).
__device__ __forceinline__ float2 e4m3x2_to_float2(uint32_t v) {
    __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(v & 0xffffu), __NV_E4M3);
    return __half22float2(*reinterpret_cast<__half2*>(&h));
}

// bf16(f32(e4m3) * scale) widened back to fp32: the weight-decode contract.
__device__ __forceinline__ float2 decode_e4m3x2(uint32_t v, float scale) {
    float2 f = e4m3x2_to_float2(v);
    uint32_t p = pack_bf16(f.x * scale, f.y * scale);
    return make_float2(bf16_lo(p), bf16_hi(p));
}

__device__ __forceinline__ float sigmoidf_precise(float x) { return 1.0f / (1.0f + expf(-x)); }

// Monotone map of fp32 to uint32: integer order == total fp32 order (-0 < +0; NaNs at the extremes).
__device__ __forceinline__ uint32_t orderable_u32(float x) {
    uint32_t b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// A sampling candidate packed so that an unsigned 64-bit maximum picks the highest logit and, among equal
// logits, the lowest token id (-0 is folded into +0 first).
__device__ __forceinline__ unsigned long long candidate_key(float value, int id) {
    return ((unsigned long long)orderable_u32(value + 0.0f) << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)id);
}
__device__ __forceinline__ int candidate_id(unsigned long long key) { return (int)(0xFFFFFFFFu - (uint32_t)(key & 0xFFFFFFFFull)); }

__device__ __forceinline__ void raise_status(uint32_t* status, uint32_t bits) {
    if (status) atomicOr(status, bits);
}

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// ---- programmatic dependent launch ----------------------------------------------------------------------
// Every kernel starts with GLMB_PDL_PROLOGUE: it lets the NEXT kernel of the stream start launching right away
// (its CTAs become resident as this grid's CTAs retire) and then waits until the PREVIOUS kernel has completed and
// its memory is visible.  With ~1500 small kernels per decode step this hides most of the launch latency.
// Nothing may be read or written before the wait.  Without the launch attribute both instructions are no-ops.
#define GLMB_PDL_PROLOGUE()                                      \
    do {                                                         \
        asm volatile("griddepcontrol.launch_dependents;");       \
        asm volatile("griddepcontrol.wait;" ::: "memory");       \
    } while (0)

// 1: launch with the programmatic-serialization attribute (default); 0: plain stream order.
extern int g_glmb_pdl_enabled;

template <typename... KArgs, typename... Args>
static inline cudaError_t glmb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                      Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = g_glmb_pdl_enabled ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#define GLMB_LAUNCH(kernel, grid, block, smem, stream, ...) (void)glmb_launch(kernel, dim3(grid), dim3(block), smem, stream, __VA_ARGS__)

// A once-per-device latch for settings that belong to a device, not to the process (cudaFuncSetAttribute: the opt-in to large
// dynamic shared memory has to be repeated on every GPU a process drives).  `pending()` names the current device if the setting
// has not been made there yet, SET if it has; `mark(d)` records it.  Two threads racing on a device both make the (idempotent)
// setting.
struct DeviceOnce {
    static constexpr int SET = -2, UNKNOWN = -1, MAX_DEVICES = 64;
    std::atomic<bool> made[MAX_DEVICES] = {};
    int pending() {
        int dev = UNKNOWN;
        if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return UNKNOWN;  // make the setting every time
        return made[dev].load(std::memory_order_acquire) ? SET : dev;
    }
    void mark(int dev) {
        if (dev >= 0 && dev < MAX_DEVICES) made[dev].store(true, std::memory_order_release);
    }
};
