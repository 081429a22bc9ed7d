// The router's choice of one row by one warp, shared by the stand-alone kernels (misc.cu).
#pragma once

#include "common.cuh"

// Router choice of one row by one warp (E <= 256): sigmoid scores, the correction bias enters the choice only, ties to the lowest
// expert id, fp32 weights normalised over the chosen scores.  FRESH: read the logits past the L1 (they were written by other CTAs of a launch still in flight).
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
