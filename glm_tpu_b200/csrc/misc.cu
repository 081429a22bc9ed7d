// Router top-k, greedy sampling, step bookkeeping, load-time weight decode and random initialisation.
//
//   router_topk       sigmoid scores, correction bias in the choice only, top-k with ties to the lowest expert
//                     id, fp32 normalized weights         (reference `glm_tpu/layers/moe/router.py:20-99`)
//   argmax_rows       per-row maximum of the bf16 logits of this rank's vocabulary slice, ties to the lowest
//                     id; the candidate is pushed to every peer (reference `layers/sampler.py:58-99`)
//   step_finalize     picks the best candidate over the ranks, writes the token, advances the lane position
//   fp8_to_bf16       bf16(f32(e4m3) * scale_inv[n/bn][k/bk]) for a whole table at load time
//                     (reference `layers/fp8.py:113-126`, `models/glm_moe_dsa/weights.py:112-181`)
//   fill_random_*     counter-based random initialisation of weights directly in device memory
#include "common.cuh"
#include "peer.cuh"
#include "router_core.cuh"

// ---------------------------------------------------------------------------------------------------
// One warp per row.  E <= 1024.
__global__ void __launch_bounds__(128)
router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int rows, int E, int top_k,
                   int* __restrict__ ids, float* __restrict__ weights) {
    GLMB_PDL_PROLOGUE();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + warp;
    if (r >= rows) return;
    const float* lg = logits + (int64_t)r * E;
    const int per = (E + 31) / 32;  // <= 32
    uint32_t taken = 0;             // bit i: this lane's i-th expert (e = lane + 32*i) is already chosen
    float picked_sum = 0.f;
    float my_score = 0.f;           // lane s (< top_k) keeps the unbiased score of slot s
    for (int s = 0; s < top_k; ++s) {
        uint32_t best_key = 0;
        int best_e = 0x7fffffff;
        float best_score = 0.f;
        for (int i = 0; i < per; ++i) {
            const int e = lane + 32 * i;
            if (e < E && !((taken >> i) & 1u)) {
                const float sc = sigmoidf_precise(lg[e]);
                const uint32_t key = orderable_u32(__fadd_rn(sc, bias[e]));
                if (best_e == 0x7fffffff || key > best_key) { best_key = key; best_e = e; best_score = sc; }
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
        if (lane == 0) ids[(int64_t)r * top_k + s] = best_e == 0x7fffffff ? 0 : best_e;
    }
    if (lane < top_k) weights[(int64_t)r * top_k + lane] = my_score / (picked_sum + 1e-20f);
}

// Same selection for E <= 256: every lane loads its (up to 8) logits once and keeps score and key in registers (router_core.cuh).
__global__ void __launch_bounds__(128)
router_topk256_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int rows, int E, int top_k,
                      int* __restrict__ ids, float* __restrict__ weights) {
    GLMB_PDL_PROLOGUE();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + warp;
    if (r >= rows) return;
    router_topk256_row<false>(logits + (int64_t)r * E, bias, E, top_k, ids + (int64_t)r * top_k, weights + (int64_t)r * top_k, lane);
}

// ---------------------------------------------------------------------------------------------------
// cand [world][rows][2] (fp32 value, int32 global id) lives in the staging buffer when world > 1.
__global__ void __launch_bounds__(1024)
argmax_rows_kernel(const bf16* __restrict__ logits, int64_t stride, int V, int vocab_base, float* __restrict__ cand,
                   int64_t cand_offset, PeerComm comm, int sig, uint32_t* status) {
    GLMB_PDL_PROLOGUE();
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    const int r = blockIdx.x, rows = gridDim.x;
    const bf16* lg = logits + (int64_t)r * stride;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    bool bad = false;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = __bfloat162float(lg[i]);
        if (!isfinite(v)) bad = true;
        if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    }
    if (bad) raise_status(status, GLMB_STATUS_NONFINITE);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v2 = __shfl_xor_sync(0xffffffffu, best, o);
        const int i2 = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (v2 > best || (v2 == best && i2 < best_i)) { best = v2; best_i = i2; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? s_val[lane] : -INFINITY;
        best_i = lane < nw ? s_idx[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float v2 = __shfl_xor_sync(0xffffffffu, best, o);
            const int i2 = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (v2 > best || (v2 == best && i2 < best_i)) { best = v2; best_i = i2; }
        }
        if (lane == 0) {
            const int gid = best_i == 0x7fffffff ? vocab_base : vocab_base + best_i;
            const unsigned long long key = candidate_key(best, gid);
            const int64_t at = (int64_t)comm.rank * rows + r;
            reinterpret_cast<unsigned long long*>(cand)[at] = key;
            for (int p = 0; p < comm.world; ++p)
                if (p != comm.rank) reinterpret_cast<unsigned long long*>(comm.data[p] + cand_offset)[at] = key;
        }
    }
    grid_signal_peers(comm, sig);
}

// One CTA.  tokens / positions are the device-resident lane state that the next step reads.
// n_sets candidate keys per row, cand[set][row] (one set per rank), are compared.  When `local_best` is given
// (the lm_head kernel reduced this rank's vocabulary slice into it with atomicMax) this kernel first publishes
// local_best[r] as this rank's candidate -- locally and into every peer's candidate table -- clears it for the
// next step, signals and waits for the peers; otherwise the candidates were already exchanged by argmax_rows
// (or by a library all-gather) and it only waits.  advance bit 0: write the token into tokens[r]; bit 1:
// increment positions[r].  Inactive rows are left untouched and report -1.
__global__ void step_finalize_kernel(unsigned long long* __restrict__ cand, int64_t cand_offset,
                                     unsigned long long* __restrict__ local_best, int n_sets, int rows,
                                     const int* __restrict__ row_active, int* __restrict__ tokens, int* __restrict__ positions,
                                     int* __restrict__ out_tokens, int* __restrict__ step_counter, int ring, int advance,
                                     PeerComm comm, int sig) {
    GLMB_PDL_PROLOGUE();
    const int r = threadIdx.x;
    if (local_best) {
        if (r < rows) {
            const unsigned long long key = local_best[r];
            local_best[r] = 0ull;
            const int64_t at = (int64_t)comm.rank * rows + r;
            cand[at] = key;
            for (int p = 0; p < comm.world; ++p)
                if (p != comm.rank) reinterpret_cast<unsigned long long*>(comm.data[p] + cand_offset)[at] = key;
        }
        grid_signal_peers(comm, sig);
        __syncthreads();
    }
    cta_wait_signal(comm, sig);
    const int step = step_counter ? *step_counter : 0;
    if (r < rows) {
        unsigned long long best = 0ull;
        for (int p = 0; p < n_sets; ++p) {
            unsigned long long key;
            if (comm.world > 1) asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(key) : "l"(cand + (int64_t)p * rows + r) : "memory");
            else key = cand[(int64_t)p * rows + r];
            best = key > best ? key : best;
        }
        int best_id = best ? candidate_id(best) : 0;
        const bool active = row_active ? row_active[r] != 0 : true;
        out_tokens[(int64_t)(step % ring) * rows + r] = active ? best_id : -1;
        if (active && (advance & 1)) tokens[r] = best_id;
        if (active && (advance & 2)) positions[r] += 1;
    }
    __syncthreads();
    if (threadIdx.x == 0 && step_counter) *step_counter = step + 1;
}

// ---------------------------------------------------------------------------------------------------
__global__ void fp8_to_bf16_kernel(const uint8_t* __restrict__ bits, const float* __restrict__ scale, int64_t N, int64_t K,
                                   int bn, int bk, bf16* __restrict__ out, uint32_t* status) {
    GLMB_PDL_PROLOGUE();
    const int64_t total = N * K;
    const int64_t kb = (K + bk - 1) / bk;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / K, k = i % K;
        const uint8_t b = bits[i];
        if ((b & 0x7f) == 0x7f) raise_status(status, GLMB_STATUS_NONFINITE);  // e4m3fn NaN codes are refused
        const float s = scale[(n / bn) * kb + k / bk];
        const float2 f = e4m3x2_to_float2((uint32_t)b);
        out[i] = __float2bfloat16_rn(f.x * s);
    }
}

__device__ __forceinline__ uint32_t mix32(uint64_t x) {
    x ^= x >> 33; x *= 0xff51afd7ed558ccdULL; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ULL; x ^= x >> 33;
    return (uint32_t)x;
}
// Approximately normal deviate from 32 random bits (sum of four bytes, variance-normalized).
__device__ __forceinline__ float approx_normal(uint32_t h) {
    const float s = (float)(h & 255u) + (float)((h >> 8) & 255u) + (float)((h >> 16) & 255u) + (float)(h >> 24);
    return (s - 510.0f) * (1.0f / 147.8f);
}

// e4m3 codes whose decoded values are ~N(0, 112^2) clipped to +-448 (4 sigma fills the e4m3 range).
__global__ void fill_random_fp8_kernel(uint8_t* __restrict__ out, int64_t n, uint64_t seed) {
    GLMB_PDL_PROLOGUE();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const float z = approx_normal(mix32(seed * 0x9e3779b97f4a7c15ULL + (uint64_t)i));
        out[i] = (uint8_t)__nv_cvt_float_to_fp8(z * 112.0f, __NV_SATFINITE, __NV_E4M3);
    }
}
__global__ void fill_random_bf16_kernel(bf16* __restrict__ out, int64_t n, uint64_t seed, float mean, float std) {
    GLMB_PDL_PROLOGUE();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = __float2bfloat16_rn(mean + std * approx_normal(mix32(seed * 0x9e3779b97f4a7c15ULL + (uint64_t)i)));
}
__global__ void fill_uniform_f32_kernel(float* __restrict__ out, int64_t n, uint64_t seed, float lo, float hi) {
    GLMB_PDL_PROLOGUE();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = lo + (hi - lo) * ((float)mix32(seed * 0x9e3779b97f4a7c15ULL + (uint64_t)i) * (1.0f / 4294967296.0f));
}

// ===================================================================================================
GLMB_API int glmb_router_topk(const float* logits, const float* bias, int rows, int E, int top_k, int* ids, float* weights,
                              void* stream) {
    if (E > 1024 || top_k > 32 || top_k > E) return 1;
    if (E <= 256)
        GLMB_LAUNCH(router_topk256_kernel, ceil_div(rows, 4), 128, 0, (cudaStream_t)stream, logits, bias, rows, E, top_k, ids, weights);
    else
        GLMB_LAUNCH(router_topk_kernel, ceil_div(rows, 4), 128, 0, (cudaStream_t)stream, logits, bias, rows, E, top_k, ids, weights);
    return (int)cudaGetLastError();
}

GLMB_API int glmb_argmax_rows(const void* logits, int64_t stride, int rows, int V, int vocab_base, float* cand, int64_t cand_offset,
                              const PeerComm* comm, int sig, uint32_t* status, void* stream) {
    PeerComm c;
    if (comm) c = *comm; else { memset(&c, 0, sizeof(c)); c.world = 1; }
    GLMB_LAUNCH(argmax_rows_kernel, rows, 1024, 0, (cudaStream_t)stream, (const bf16*)logits, stride, V, vocab_base, cand, cand_offset, c, sig,
                                                                status);
    return (int)cudaGetLastError();
}

GLMB_API int glmb_step_finalize(void* cand, int64_t cand_offset, void* local_best, int n_sets, int rows, const int* row_active,
                                int* tokens, int* positions, int* out_tokens, int* step_counter, int ring, int advance,
                                const PeerComm* comm, int sig, void* stream) {
    if (rows > 32 || n_sets < 1 || ring < 1) return 1;
    PeerComm c;
    if (comm) c = *comm; else { memset(&c, 0, sizeof(c)); c.world = 1; }
    GLMB_LAUNCH(step_finalize_kernel, 1, 32, 0, (cudaStream_t)stream, (unsigned long long*)cand, cand_offset, (unsigned long long*)local_best,
                                                             n_sets, rows, row_active, tokens, positions, out_tokens, step_counter,
                                                             ring, advance, c, sig);
    return (int)cudaGetLastError();
}

GLMB_API int glmb_fp8_to_bf16(const void* bits, const float* scale, int64_t N, int64_t K, int bn, int bk, void* out,
                              uint32_t* status, void* stream) {
    const int64_t total = N * K;
    const int grid = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    GLMB_LAUNCH(fp8_to_bf16_kernel, grid, 256, 0, (cudaStream_t)stream, (const uint8_t*)bits, scale, N, K, bn, bk, (bf16*)out, status);
    return (int)cudaGetLastError();
}

GLMB_API int glmb_fill_random_fp8(void* out, int64_t n, uint64_t seed, void* stream) {
    GLMB_LAUNCH(fill_random_fp8_kernel, 148 * 8, 256, 0, (cudaStream_t)stream, (uint8_t*)out, n, seed);
    return (int)cudaGetLastError();
}
GLMB_API int glmb_fill_random_bf16(void* out, int64_t n, uint64_t seed, float mean, float std, void* stream) {
    GLMB_LAUNCH(fill_random_bf16_kernel, 148 * 8, 256, 0, (cudaStream_t)stream, (bf16*)out, n, seed, mean, std);
    return (int)cudaGetLastError();
}
GLMB_API int glmb_fill_uniform_f32(float* out, int64_t n, uint64_t seed, float lo, float hi, void* stream) {
    GLMB_LAUNCH(fill_uniform_f32_kernel, 148 * 8, 256, 0, (cudaStream_t)stream, out, n, seed, lo, hi);
    return (int)cudaGetLastError();
}
