// Kernel tails: a small grid-wide step that follows a kernel, run by the LAST CTA of that kernel to finish instead of by a launch of
// its own.  Every CTA, after its stores, fences and bumps a counter; the CTA that sees the final count re-reads what the grid wrote
// (past the L1) and does the step.  Two tails exist, both a few microseconds of work for one CTA and both on the critical path of
// every decode layer:
//   TAIL_ADD_RMSNORM  residual <- bf16(update + residual); x <- RMSNorm(residual) * weight, where `update` is the bf16 output of the
//                     kernel itself (an all-reduced projection); rows <= 2, blockDim.x == 256
//   TAIL_ROUTER_TOPK  top-k of the router logits the kernel just produced (fp32 output), one warp per row; E <= 256
//   TAIL_QKV_A_POST   the LoRA norms, RoPE and cache-row write that consume the fused q_a | kv_a | index projection the kernel just
//                     produced (fp32 output); rows <= 2; its arguments are a QkvPostArgs block in device memory
// The arithmetic is that of add_rmsnorm_kernel / router_topk256_kernel (the same device functions), so the bits are the same; the
// counter is left at zero, so a captured graph replays the kernel unchanged.
#pragma once

#include "common.cuh"
#include "norm_rope_core.cuh"

enum { TAIL_NONE = 0, TAIL_ADD_RMSNORM = 1, TAIL_ROUTER_TOPK = 2, TAIL_QKV_A_POST = 3 };

struct KernelTail {
    int kind;
    int rows;
    unsigned int* counter;   // one zeroed word per call site
    // TAIL_ADD_RMSNORM
    const bf16* update;      // [rows, H] the host kernel's output
    bf16* residual;          // [rows, H]
    const bf16* weight;      // [H]
    bf16* x_out;             // [rows, H]
    int H;
    float eps;
    // TAIL_ROUTER_TOPK
    const float* logits;     // [rows, logits_stride] the host kernel's output
    const float* bias;       // [E]
    int* ids;                // [rows, top_k]
    float* wts;              // [rows, top_k]
    int64_t logits_stride;
    int E;
    int top_k;
    // TAIL_QKV_A_POST
    const QkvPostArgs* qkv;  // device memory; proj = the host kernel's output
};

// Router choice of one row by one warp (E <= 256): sigmoid scores, the correction bias enters the choice only, ties to the lowest
// expert id, fp32 weights normalised over the chosen scores.  FRESH: the logits were written by other CTAs of the same launch.
template <bool FRESH>
__device__ __forceinline__ void router_topk256_row(const float* lg, const float* bias, int E, int top_k, int* ids, float* weights, int lane) {
    float lv[8], bv[8], sc[8];
    uint32_t key[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = lane + 32 * i;
        lv[i] = e < E ? (FRESH ? __ldcg(lg + e) : lg[e]) : 0.f;
        bv[i] = e < E ? bias[e] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        sc[i] = sigmoidf_precise(lv[i]);
        key[i] = orderable_u32(__fadd_rn(sc[i], bv[i]));
    }
    uint32_t taken = 0;
    float picked_sum = 0.f, my_score = 0.f;
    for (int s = 0; s < top_k; ++s) {
        uint32_t best_key = 0;
        int best_e = 0x7fffffff;
        float best_score = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = lane + 32 * i;
            if (e < E && !((taken >> i) & 1u) && (best_e == 0x7fffffff || key[i] > best_key)) {
                best_key = key[i]; best_e = e; best_score = sc[i];
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const uint32_t k2 = __shfl_xor_sync(0xffffffffu, best_key, o);
            const int e2 = __shfl_xor_sync(0xffffffffu, best_e, o);
            const float s2 = __shfl_xor_sync(0xffffffffu, best_score, o);
            const bool theirs = e2 != 0x7fffffff && (best_e == 0x7fffffff || k2 > best_key || (k2 == best_key && e2 < best_e));
            if (theirs) { best_key = k2; best_e = e2; best_score = s2; }
        }
        if (best_e != 0x7fffffff && (best_e & 31) == lane) taken |= 1u << (best_e >> 5);
        if (lane == s) my_score = best_score;
        picked_sum += best_score;
        if (lane == 0) ids[s] = best_e == 0x7fffffff ? 0 : best_e;
    }
    if (lane < top_k) weights[lane] = my_score / (picked_sum + 1e-20f);
}

// Every thread of the CTA (256 threads) calls it once, after the CTA's last store.  `scratch`: >= 40 floats of shared memory.
__device__ __forceinline__ void run_kernel_tail(const KernelTail& t, float* scratch) {
    if (t.kind == TAIL_NONE) return;
    __shared__ int s_last;
    __shared__ float s_qkv_scratch[3][40];
    __shared__ float s_qkv_key[256];
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned total = gridDim.x * gridDim.y * gridDim.z;
        s_last = atomicAdd(t.counter, 1u) == total - 1 ? 1 : 0;
    }
    __syncthreads();
    if (!s_last) return;
    if (threadIdx.x == 0) *t.counter = 0u;
    __threadfence();
    if (t.kind == TAIL_ADD_RMSNORM) {
        for (int r = 0; r < t.rows; ++r)
            add_rmsnorm_row<true>(t.update + (int64_t)r * t.H, t.residual + (int64_t)r * t.H, t.weight, t.x_out + (int64_t)r * t.H, t.H, t.eps,
                                  scratch);
    } else if (t.kind == TAIL_QKV_A_POST) {
        const QkvPostArgs a = *t.qkv;
        for (int r = 0; r < t.rows; ++r) {
            qkv_a_post_row(a, r, s_qkv_scratch, s_qkv_key);
            __syncthreads();
        }
    } else if (t.kind == TAIL_ROUTER_TOPK) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        if (warp < t.rows)
            router_topk256_row<true>(t.logits + (int64_t)warp * t.logits_stride, t.bias, t.E, t.top_k, t.ids + (int64_t)warp * t.top_k,
                                     t.wts + (int64_t)warp * t.top_k, lane);
    }
}

static inline KernelTail no_tail() {
    KernelTail t;
    memset(&t, 0, sizeof(t));
    return t;
}
