// DSA lightning indexer: owner-local scoring of the index cache and the exact top-k selection.
//
//   indexer_score   score[pos] = sum_h w_h * relu(q_h . key[pos] * scale)  in fp32 over this rank's stripe
//                   of the index cache; every score is stored at its GLOBAL position in this rank's score
//                   row and in every peer's (the all-gather of the scores is fused into the store), then
//                   the last CTA signals.
//   topk_select     exact selection of the top_k best positions of score[0..ctx) under the total order
//                   (descending score, ties to the lowest position, +0 > -0): 4-pass radix select on the
//                   order-preserving key, then an ordered compaction.  Output is ascending in position:
//                   the global list (-1 padded) and the list of this rank's own cache rows among them.
//
// Replaces reference `glm_tpu/layers/attention/dsa_indexer.py:129-150,352-393` (scoring) and `:35-126`
// (two-stage top-k with its candidate exchange and fallback), `layers/attention/kv_cache.py:223-260,297-352`
// (canonicalize + owner subset).
#include "common.cuh"
#include "peer.cuh"

// One thread per cached key.  The key (D bf16) lives in registers as packed words; the query heads are
// read from shared memory as broadcast float4.
template <int D>
__global__ void __launch_bounds__(256)
indexer_score_kernel(const float* __restrict__ q_idx, const float* __restrict__ head_w, const bf16* __restrict__ index_cache,
                     const int* __restrict__ row_pos, const int* __restrict__ row_lane, int IH, int index_slot, int full_layers,
                     int local_cap, int stripe, int world, int rank, int capacity, int64_t score_stride, float scale,
                     float* __restrict__ scores, int64_t scores_offset, PeerComm comm, int sig, uint32_t* status) {
    GLMB_PDL_PROLOGUE();
    extern __shared__ float sq[];  // IH * D query, then IH weights
    float* sw = sq + IH * D;
    const int r = blockIdx.y;
    for (int i = threadIdx.x; i < IH * D; i += blockDim.x) sq[i] = q_idx[(int64_t)r * IH * D + i];
    for (int i = threadIdx.x; i < IH; i += blockDim.x) sw[i] = head_w[(int64_t)r * IH + i];
    __syncthreads();
    const int pos = min(max(row_pos[r], 0), capacity - 1);
    const int ctx = pos + 1;
    const int page = stripe * world;
    // number of positions < ctx stored on this rank
    const int rest = ctx % page;
    const int owned = (ctx / page) * stripe + min(max(rest - rank * stripe, 0), stripe);
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j < owned) {
        const bf16* key = index_cache + (((int64_t)row_lane[r] * full_layers + index_slot) * local_cap + j) * D;
        uint32_t kw[D / 2];
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            const uint4 v = *reinterpret_cast<const uint4*>(key + i * 8);
            kw[4 * i] = v.x; kw[4 * i + 1] = v.y; kw[4 * i + 2] = v.z; kw[4 * i + 3] = v.w;
        }
        float score = 0.f;
        for (int h = 0; h < IH; ++h) {
            const float4* qh = reinterpret_cast<const float4*>(sq + h * D);
            float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;  // four chains: the dot is latency-, not throughput-bound
#pragma unroll
            for (int i = 0; i < D / 4; ++i) {
                const float4 qv = qh[i];
                d0 = fmaf(qv.x, bf16_lo(kw[2 * i]), d0);
                d1 = fmaf(qv.y, bf16_hi(kw[2 * i]), d1);
                d2 = fmaf(qv.z, bf16_lo(kw[2 * i + 1]), d2);
                d3 = fmaf(qv.w, bf16_hi(kw[2 * i + 1]), d3);
            }
            const float dot = (d0 + d1) + (d2 + d3);
            score = fmaf(sw[h], fmaxf(__fmul_rn(dot, scale), 0.f), score);
        }
        if (!isfinite(score)) raise_status(status, GLMB_STATUS_NONFINITE);
        const int g = (j / stripe) * page + rank * stripe + j % stripe;
        const int64_t at = (int64_t)r * score_stride + g;
        scores[at] = score;
        for (int p = 0; p < comm.world; ++p)
            if (p != comm.rank) reinterpret_cast<float*>(comm.data[p] + scores_offset)[at] = score;
    }
    grid_signal_peers(comm, sig);
}

// ---------------------------------------------------------------------------------------------------
#define TK_THREADS 1024

// Exclusive block scan of one uint32 per thread; returns the exclusive prefix, *total receives the sum.
__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t* warp_totals, uint32_t* total) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    __syncthreads();
    if (lane == 31) warp_totals[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        uint32_t w = warp_totals[lane];
        uint32_t winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t t = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += t;
        }
        warp_totals[lane] = winc - w;
        if (lane == 31) warp_totals[32] = winc;
    }
    __syncthreads();
    *total = warp_totals[32];
    return warp_totals[warp] + inc - v;
}

__global__ void __launch_bounds__(TK_THREADS)
topk_select_kernel(const float* __restrict__ scores, const int* __restrict__ row_pos, int capacity, int64_t score_stride, int top_k, int stripe,
                   int world, int rank, int* __restrict__ sel_global, int* __restrict__ sel_local, int* __restrict__ sel_counts,
                   PeerComm comm, int sig) {
    GLMB_PDL_PROLOGUE();
    __shared__ uint32_t hist[256];
    __shared__ uint32_t warp_totals[33];
    __shared__ uint32_t s_bucket, s_need;
    cta_wait_signal(comm, sig);
    const int r = blockIdx.x;
    const int n = min(max(row_pos[r], 0), capacity - 1) + 1;
    const float* sc = scores + (int64_t)r * score_stride;
    int* out_g = sel_global + (int64_t)r * top_k;
    int* out_l = sel_local + (int64_t)r * top_k;
    const int page = stripe * world;
    const int ipt = (n + TK_THREADS - 1) / TK_THREADS;
    const int begin = min(n, (int)threadIdx.x * ipt), end = min(n, begin + ipt);

    uint32_t thresh = 0, need = 0;
    const bool take_all = n <= top_k;
    if (!take_all) {
        uint32_t prefix = 0, mask = 0;
        need = top_k;
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            if (threadIdx.x < 256) hist[threadIdx.x] = 0;
            __syncthreads();
            for (int i = threadIdx.x; i < n; i += TK_THREADS) {
                const uint32_t key = orderable_u32(sc[i]);
                if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (threadIdx.x < 32) {
                // lane l owns bins 255-8l .. 248-8l (descending); find the bin where the running count reaches `need`
                const int lane = threadIdx.x;
                uint32_t local[8], sum = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) { local[i] = hist[255 - (lane * 8 + i)]; sum += local[i]; }
                uint32_t inc = sum;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
                    if (lane >= o) inc += t;
                }
                const uint32_t before = inc - sum;
                if (before < need && inc >= need) {
                    uint32_t cum = before;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        if (cum < need && cum + local[i] >= need) { s_bucket = 255 - (lane * 8 + i); s_need = need - cum; }
                        cum += local[i];
                    }
                }
            }
            __syncthreads();
            prefix |= s_bucket << shift;
            mask |= 255u << shift;
            need = s_need;
            __syncthreads();
        }
        thresh = prefix;
    }
    // ordered compaction: each thread owns a contiguous run of positions
    uint32_t eq_mine = 0;
    if (!take_all)
        for (int i = begin; i < end; ++i) eq_mine += orderable_u32(sc[i]) == thresh;
    uint32_t eq_total;
    uint32_t eq_before = block_exclusive_scan(eq_mine, warp_totals, &eq_total);
    uint32_t sel_mine = 0, own_mine = 0;
    for (int i = begin; i < end; ++i) {
        bool sel = true;
        if (!take_all) {
            const uint32_t key = orderable_u32(sc[i]);
            sel = key > thresh;
            if (key == thresh) { sel = eq_before < need; ++eq_before; }
        }
        if (sel) { ++sel_mine; own_mine += ((i / stripe) % world) == rank; }
    }
    eq_before -= eq_mine;  // restore for the second sweep
    uint32_t packed_total;
    const uint32_t packed_before = block_exclusive_scan(sel_mine | (own_mine << 16), warp_totals, &packed_total);
    uint32_t at_g = packed_before & 0xffffu, at_l = packed_before >> 16;
    for (int i = begin; i < end; ++i) {
        bool sel = true;
        if (!take_all) {
            const uint32_t key = orderable_u32(sc[i]);
            sel = key > thresh;
            if (key == thresh) { sel = eq_before < need; ++eq_before; }
        }
        if (sel) {
            if (at_g < (uint32_t)top_k) out_g[at_g] = i;
            ++at_g;
            if (((i / stripe) % world) == rank) {
                if (at_l < (uint32_t)top_k) out_l[at_l] = (i / page) * stripe + i % stripe;
                ++at_l;
            }
        }
    }
    const int total_sel = packed_total & 0xffffu, total_own = packed_total >> 16;
    for (int i = total_sel + threadIdx.x; i < top_k; i += TK_THREADS) out_g[i] = -1;
    for (int i = total_own + threadIdx.x; i < top_k; i += TK_THREADS) out_l[i] = -1;
    if (threadIdx.x == 0) { sel_counts[2 * r] = total_sel; sel_counts[2 * r + 1] = total_own; }
}

// ===================================================================================================
// scores must be the staging address comm->data[rank] + scores_offset when world > 1.
GLMB_API int glmb_indexer_score(const float* q_idx, const float* head_w, const void* index_cache, const int* row_pos,
                                const int* row_lane, int rows, int IH, int D, int index_slot, int full_layers, int local_cap,
                                int stripe, int world, int rank, int capacity, int max_ctx, int64_t score_stride, float scale,
                                float* scores, int64_t scores_offset, const PeerComm* comm, int sig, uint32_t* status, void* stream) {
    PeerComm c;
    if (comm) c = *comm; else { memset(&c, 0, sizeof(c)); c.world = 1; }
    // grid.x covers the largest number of rows any rank can own for a context of max_ctx positions
    const int page = stripe * world;
    const int owned_max = (max_ctx / page) * stripe + min(max_ctx % page, stripe);
    dim3 grid(ceil_div(owned_max > 0 ? owned_max : 1, 256), rows);
    const size_t smem = (size_t)(IH * D + IH) * sizeof(float);
    cudaStream_t st = (cudaStream_t)stream;
#define CALL(DD)                                                                                                          \
    GLMB_LAUNCH(indexer_score_kernel<DD>, grid, 256, smem, st, q_idx, head_w, (const bf16*)index_cache, row_pos, row_lane, IH, index_slot, \
                                                      full_layers, local_cap, stripe, world, rank, capacity, score_stride, scale, scores,  \
                                                      scores_offset, c, sig, status)
    if (D == 128) { CALL(128); } else if (D == 64) { CALL(64); } else if (D == 32) { CALL(32); } else return 1;
#undef CALL
    return (int)cudaGetLastError();
}

// top_k <= 65535 (the scan packs two 16-bit counters).
GLMB_API int glmb_topk_select(const float* scores, const int* row_pos, int rows, int capacity, int64_t score_stride, int top_k, int stripe, int world,
                              int rank, int* sel_global, int* sel_local, int* sel_counts, const PeerComm* comm, int sig,
                              void* stream) {
    if (top_k > 65535) return 1;
    PeerComm c;
    if (comm) c = *comm; else { memset(&c, 0, sizeof(c)); c.world = 1; }
    GLMB_LAUNCH(topk_select_kernel, rows, TK_THREADS, 0, (cudaStream_t)stream, scores, row_pos, capacity, score_stride, top_k, stripe, world, rank,
                                                                      sel_global, sel_local, sel_counts, c, sig);
    return (int)cudaGetLastError();
}
