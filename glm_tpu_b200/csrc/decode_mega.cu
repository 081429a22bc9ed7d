// The decode step as ONE persistent, cooperatively launched kernel per stretch of layers.
//
// A decode step of the per-kernel path is ~17 dependent launches per layer; on 8 GPUs every one of them is a few
// microseconds of launch, ramp-up and drain around well under a microsecond of memory traffic, so the step runs at a
// fifth of its HBM bound.  Here the whole layer sequence runs inside one grid that stays resident (two 256-thread
// CTAs per SM): a *phase* is what used to be a kernel, the CTAs share each phase's work items with a grid-stride
// loop, and a device-side grid barrier replaces the kernel boundary.  Small dependent steps that every consumer can
// recompute from a few kilobytes (add + RMSNorm of the 12 KB hidden row, the q_a LoRA norm, the router's top-k) are
// folded into the prologue of their consumers, which deletes their phases altogether.
//
// Phases of layer l (each ends with a grid barrier):
//    1 QKV_A    [add + RMSNorm prologue]  q_a | kv_a | indexer key | indexer head weights projection  -> proj_a (fp32)
//    2 Q_B      [q_a norm prologue; CTA r: LoRA norms, RoPE, cache-row and index-key write of row r]  q_b (+ indexer wq_b) -> q_proj (fp32)
//    3 ABSORB   rounded / rotated queries of this GPU's heads, q_nope @ W_k  -> q_full
//         (a layer with its own indexer ends its stretch here: the tcgen05 indexer and the cluster top-k run as kernels of
//          their own, then the next stretch starts at phase 4)
//    4 ATTN     16 heads x 64 gathered keys per tile (mma.sync), chunk-local softmax  -> partials
//    5 MERGE    log-sum-exp merge of a row's chunks per head  -> o_lat
//    6 VPROJ    per-head value projection  -> attn_v
//    7 OPROJ    output projection of this GPU's heads + all-reduce over the GPUs (peer memory)  -> attn_out
//    8 MLP_A    [add + RMSNorm prologue]  dense: gate/up + SwiGLU;  sparse: router logits, shared-expert gate/up + SwiGLU
//    9 MLP_B    dense: down + all-reduce -> update;  sparse: [router top-k prologue] routed FP8 gate/up + SwiGLU, shared down
//   10 MOE_DOWN routed FP8 down projections, route weights
//   11 COMBINE  route sums + shared expert, all-reduce over the GPUs, x 2.5 + shared  -> update
// and of the head (layer index == number of layers):  1 [final norm prologue] lm_head with the greedy reduction,
// 2 candidate exchange, token store, lane advance.
//
// The arithmetic of every phase is the per-kernel path's (the same inner functions, `*_core.cuh`); with `compat_ksplit`
// even the split of K over warps is the same, and the two paths then agree bit for bit, which is how the tests pin this
// kernel.  The default split balances the 2,368 resident warps instead.
//
// Waits: the grid barrier and the peer waits inside the all-reduces spin under an iteration limit; a wait that runs out
// raises GLMB_STATUS_WAIT_TIMEOUT, sets the barrier's abort word so that every later barrier falls through at once, and
// the kernel finishes with meaningless outputs (the host reads the status word and poisons the engine).
//
// Cache layouts: the kernel attends over keys of this GPU's own cache (one GPU, or a replica of the latent cache per
// GPU); position-striped caches keep the per-kernel path.
//
// Replaces the launch sequence of reference `glm_tpu/models/glm_moe_dsa/model.py:86-135`, `decoder_layer.py:656-740`.
#include "common.cuh"

#include <string.h>
#include "attention_core.cuh"
#include "gemv_core.cuh"
#include "moe_mma_core.cuh"
#include "norm_rope_core.cuh"
#include "peer.cuh"

#define MG_THREADS 256
#ifndef MG_CALL
#define MG_CALL __noinline__  // phases and their shared pieces are functions of their own (code size, register allocation per phase)
#endif
#ifndef MG_CTAS_PER_SM
#define MG_CTAS_PER_SM 2  // resident CTAs per SM the kernel is compiled and launched for
#endif
#define MG_WARPS 8
#define MG_MAX_TOPK 32
#define MG_BIG_BYTES (100 * 1024)
#define MG_MERGE_MAX_CHUNKS 128
#define MG_MM_ROWS 16

enum { MG_QKV_A = 1, MG_Q_B, MG_ABSORB, MG_ATTN, MG_MERGE, MG_VPROJ, MG_OPROJ, MG_MLP_A, MG_MLP_B, MG_MOE_DOWN, MG_COMBINE };
enum { MG_HEAD_LOGITS = 1, MG_HEAD_FINALIZE = 2 };

// The words of the grid barrier, each on a cache line of its own: the arrival counter takes one atomic per CTA, the
// generation word is polled by every waiting CTA, and the two must not queue behind each other at one L2 line.
struct MegaBarrier {
    unsigned int arrive;
    unsigned int pad0[31];
    unsigned int gen;
    unsigned int pad1[31];
    unsigned int abort;
    unsigned int pad2[31];
    unsigned int flags[1024];  // variant 2 of the barrier: one arrival word per CTA
};

// One per layer, in device memory (pointers first: no padding).
struct MegaLayer {
    const bf16* input_norm;
    const bf16* post_norm;
    const bf16* w_qkv_a;
    const bf16* q_a_norm;
    const bf16* kv_a_norm;
    const bf16* w_q_b;
    const bf16* kv_b;
    const bf16* w_o;
    const float* k_norm_w;
    const float* k_norm_b;
    const bf16* dense_gate;
    const bf16* dense_up;
    const bf16* dense_down;
    const bf16* router_w;
    const float* router_bias;
    const uint8_t* exp_gate;
    const uint8_t* exp_up;
    const uint8_t* exp_down;
    const float* exp_gate_scale;
    const float* exp_up_scale;
    const float* exp_down_scale;
    const bf16* shared_gate;
    const bf16* shared_up;
    const bf16* shared_down;
    int full;        // the layer has its own indexer
    int dense;       // dense MLP (else mixture of experts)
    int index_slot;  // slot of the layer in the index cache (full layers)
    int n_qkv_a;     // rows of w_qkv_a
    int n_q_b;       // rows of w_q_b
    int pad_;
};

struct MegaArgs {
    const MegaLayer* layers;
    // tables
    const bf16* embed;
    const bf16* final_norm;
    const bf16* lm_head;
    const bf16* rope_table;
    const float* inv_freq;
    // lane state
    int* tokens;
    int* positions;
    const int* active;
    const int* lane_ids;
    int* out_tokens;
    int* step_counter;
    // caches
    bf16* kv_cache;
    bf16* index_cache;
    // workspace
    bf16* residual_a;
    bf16* residual_b;
    bf16* x;
    bf16* update;
    bf16* attn_out;
    float* proj_a;
    bf16* q_resid;
    float* head_w;
    bf16* kv_new;
    bf16* idx_key_new;
    float* q_proj;
    bf16* q_full;
    const int* sel_local;
    const int* sel_counts;
    float* part_o;
    float* part_ml;
    bf16* o_lat;
    bf16* attn_v;
    float* router_logits;
    int* topk_ids;
    float* topk_w;
    bf16* act_shared;
    bf16* dense_act;
    float* partial;
    bf16* act;
    bf16* dw;
    unsigned long long* local_best;
    unsigned long long* cand;
    MegaBarrier* bar;
    uint32_t* status;
    unsigned long long* timeline;  // optional: [0] = entries written, then (code, globaltimer ns) pairs; code = layer << 8 | phase
    int64_t proj_stride, q_stride, act_shared_stride, dense_act_stride, cand_offset, timeline_cap, prefetch_cap;
    // geometry and layout
    int rows, H, Q, L, rd, nope, vdim, D, IH;
    int heads_local, head_base, heads_total, E, top_k, I, experts_local, expert_base, shared_cols, dense_cols;
    int vocab, vocab_local, vocab_base, num_layers, n_full_layers, index_top_k, max_chunks;
    int local_cap, stripe, cache_world, cache_rank, capacity, ring, compat_ksplit;
    uint32_t bar_limit;
    float eps, key_eps, head_scale, softmax_scale, routed_scale;
    int layer0, phase0, layer1, phase1;  // the stretch to run: (layer, phase) pairs, both ends inclusive
    PeerComm comm;
};

struct MgSmall {
    MegaArgs args;    // the kernel's argument block, copied once: phase functions read it here, not through a generic pointer
    MegaLayer layer;  // the pointer-table entry of the layer in progress
    float red[MG_WARPS][2][GLMB_MAX_ROWS];
    float sh[GLMB_AR_SLICE];
    float scratch[3][40];
    float s_key[256];
    unsigned long long best[MG_WARPS][GLMB_MAX_ROWS];
    int ids[GLMB_MAX_ROWS][MG_MAX_TOPK];
    float wts[GLMB_MAX_ROWS][MG_MAX_TOPK];
    int loc[GLMB_MAX_ROWS * MG_MAX_TOPK];
    float w_s[MG_MERGE_MAX_CHUNKS];
    float red_s[8];
    int n_loc;
    int big_bytes;                 // size of the big region behind this block (a launch-time choice)
    int stamping;                  // this thread block's first thread writes per-phase time stamps (measurements)
    unsigned long long stamp_at;   // next free entry of the stamp buffer
};

// (code, %globaltimer) into the stamp buffer; CTA 0's first thread only.  code = layer << 8 | phase (bit 7: before the
// phase's grid barrier; bits 16..: a step inside the phase).
__device__ __forceinline__ void mg_stamp(MgSmall& sm, unsigned long long code) {
    if (!sm.stamping || threadIdx.x != 0) return;
    const MegaArgs& a = sm.args;
    if ((int64_t)sm.stamp_at < a.timeline_cap) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
        a.timeline[1 + 2 * sm.stamp_at] = code;
        a.timeline[2 + 2 * sm.stamp_at] = now;
    }
    ++sm.stamp_at;
}

// ---------------------------------------------------------------------------------------------------
// Grid barrier over all CTAs of the (cooperative) launch.  `epoch` is each thread's copy of the generation the
// grid has completed; it starts from the value every CTA reads at kernel entry (no barrier is in flight then).
__device__ __forceinline__ unsigned int mg_ld_relaxed(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// VARIANT 1: one atomic per CTA on the arrival counter, the last arriver publishes the generation, the others poll it
// with relaxed loads (a fence on either side orders the data).  VARIANT 2: every CTA stores its own arrival word, CTA 0
// gathers them (one word per thread) and publishes.  VARIANT 0: counter and generation on neighbouring words, acquire
// polling (the first form, kept for the measurement in `glmb_mega_barrier_bench`).
template <int VARIANT>
__device__ __forceinline__ void mg_grid_barrier_v(MegaBarrier* b, unsigned int& epoch, uint32_t limit, uint32_t* status) {
    const unsigned int target = epoch + 1;
    if (VARIANT == 2) {
        const bool live = __syncthreads_or(mg_ld_relaxed(&b->abort) != 0u) == 0;  // the same answer in every thread of the CTA
        if (threadIdx.x == 0 && live) {
            __threadfence();
            asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(&b->flags[blockIdx.x]), "r"(target) : "memory");
        }
        if (blockIdx.x == 0 && live) {
            bool ok = true;
            for (unsigned int c = threadIdx.x; c < gridDim.x; c += blockDim.x) {
                bool seen = false;
                for (uint32_t i = 0; i < limit; ++i) {
                    if ((int)(mg_ld_relaxed(&b->flags[c]) - target) >= 0) { seen = true; break; }
                    if (i > 4096) { if (mg_ld_relaxed(&b->abort)) break; __nanosleep(64); }
                }
                ok = ok && seen;
            }
            if (!ok) { atomicExch(&b->abort, 1u); raise_status(status, GLMB_STATUS_WAIT_TIMEOUT); }
            __syncthreads();
            if (threadIdx.x == 0) {
                __threadfence();
                asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(&b->gen), "r"(target) : "memory");
            }
        } else if (threadIdx.x == 0 && live) {
            bool ok = false;
            for (uint32_t i = 0; i < limit; ++i) {
                if ((int)(mg_ld_relaxed(&b->gen) - target) >= 0) { ok = true; break; }
                if (i > 4096) { if (mg_ld_relaxed(&b->abort)) break; __nanosleep(64); }
            }
            if (!ok) { atomicExch(&b->abort, 1u); raise_status(status, GLMB_STATUS_WAIT_TIMEOUT); }
        }
        if (threadIdx.x == 0) __threadfence();
        epoch += 1;
        __syncthreads();
        return;
    }
    __syncthreads();
    if (threadIdx.x == 0 && mg_ld_relaxed(&b->abort) == 0u) {
        unsigned int* gen = VARIANT == 0 ? &b->pad0[0] : &b->gen;
        __threadfence();
        if (atomicAdd(&b->arrive, 1u) == gridDim.x - 1) {
            b->arrive = 0;  // nobody arrives at the next barrier before the release below
            __threadfence();
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(gen), "r"(target) : "memory");
        } else {
            bool ok = false;
            for (uint32_t i = 0; i < limit; ++i) {
                unsigned int g;
                if (VARIANT == 0) asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(g) : "l"(gen) : "memory");
                else g = mg_ld_relaxed(gen);
                if ((int)(g - target) >= 0) { ok = true; break; }
                if (i > 4096) {
                    if (mg_ld_relaxed(&b->abort)) break;
                    __nanosleep(64);
                }
            }
            if (!ok) {
                atomicExch(&b->abort, 1u);
                raise_status(status, GLMB_STATUS_WAIT_TIMEOUT);
            }
        }
        __threadfence();
    }
    epoch += 1;
    __syncthreads();
}

#ifndef MG_BARRIER_VARIANT
#define MG_BARRIER_VARIANT 1
#endif
__device__ __forceinline__ void mg_grid_barrier(MegaBarrier* b, unsigned int& epoch, uint32_t limit, uint32_t* status) {
    mg_grid_barrier_v<MG_BARRIER_VARIANT>(b, epoch, limit, status);
}

// ---------------------------------------------------------------------------------------------------
// How many warps split K for one unit of output.  compat: the rule of the stand-alone skinny kernels (gemv.cu), so that
// both paths add the same partial sums.  Otherwise: the split that minimises rounds x span over the resident warps.
__device__ __forceinline__ int mg_pick_ks(int units, int K, bool compat, int max_rounds_words /* 0: no limit */, int words_per_team) {
    if (compat) {
        int ks = 1;
        while (ks < MG_WARPS && units * ks < 148 * 4 * MG_WARPS && K % (ks * 2 * 256) == 0 && K / (ks * 2) >= 512) ks *= 2;
        return ks;
    }
    int best = 1;
    long best_cost = -1;
    for (int ks = 1; ks <= MG_WARPS; ks *= 2) {
        if (ks > 1 && (K % (ks * 256))) break;
        const int teams = (int)gridDim.x * (MG_WARPS / ks);
        const int rounds = (units + teams - 1) / teams;
        if (max_rounds_words && rounds * (MG_WARPS / ks) * words_per_team > max_rounds_words && ks < MG_WARPS) continue;
        const long cost = (long)rounds * (K / ks + 256);  // 256: the fixed cost of a round (reduction, epilogue)
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = ks; }
    }
    return best;
}

// warp_dot_bf16 (gemv_core.cuh) with U steps of loads issued before their arithmetic: the same products added in the same
// order, but 2 * U 16-byte loads in flight per lane, which the 16 resident warps of an SM need to keep HBM busy.
template <int R, int U>
__device__ __forceinline__ void mg_warp_dot(const bf16* const (&xr)[R], const bf16* const (&wp)[2], int kbeg, int kend, int lane,
                                            float (&acc)[2][R]) {
    int k = kbeg + lane * 8;
    for (; k + (U - 1) * 256 < kend; k += U * 256) {
        uint4 wv[U][2];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int j = 0; j < 2; ++j) wv[u][j] = ld_stream16(wp[j] + k + u * 256);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            float wf[2][8];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint4 v = wv[u][j];
                wf[j][0] = bf16_lo(v.x); wf[j][1] = bf16_hi(v.x); wf[j][2] = bf16_lo(v.y); wf[j][3] = bf16_hi(v.y);
                wf[j][4] = bf16_lo(v.z); wf[j][5] = bf16_hi(v.z); wf[j][6] = bf16_lo(v.w); wf[j][7] = bf16_hi(v.w);
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint4 v = ld_hot16(xr[r] + k + u * 256);
                const float xf[8] = {bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y),
                                     bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w)};
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[j][r] = fmaf(wf[j][i], xf[i], acc[j][r]);
            }
        }
    }
    if (k < kend) {  // the tail, one step at a time, in the same order
        const int done = k - (kbeg + lane * 8);
        warp_dot_bf16<R, 2>(xr, wp, kbeg + done, kend, lane, acc);
    }
}

// Ask the L2 for `bytes` at p (capped): every CTA requests its slice, one thread issues, nothing waits for it.
__device__ __forceinline__ void mg_prefetch_l2(const void* p, size_t bytes, size_t cap) {
    if (threadIdx.x != 0 || p == nullptr) return;
    if (bytes > cap) bytes = cap;
    const size_t per = ((bytes + gridDim.x - 1) / gridDim.x + 127) & ~(size_t)127;
    const size_t off = per * blockIdx.x;
    if (off >= bytes) return;
    const size_t n = (per < bytes - off ? per : bytes - off) & ~(size_t)15;
    if (n) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<const char*>(p) + off), "r"((uint32_t)n) : "memory");
}

// Shared-memory scratch of the balanced projections: what is left of the big region after `used_bytes`.
__device__ __forceinline__ float* mg_scratch(unsigned char* big, size_t used_bytes, int* floats) {
    const size_t at = (used_bytes + 15) & ~(size_t)15;
    const MgSmall* sm = reinterpret_cast<const MgSmall*>(big - ((sizeof(MgSmall) + 15) & ~(size_t)15));
    *floats = (int)(((size_t)sm->big_bytes - at) / sizeof(float));
    return reinterpret_cast<float*>(big + at);
}

// fp32 store of a pass of the balanced projection: out[r][first + i] = vals[i][r]
template <int R>
__device__ __forceinline__ void mg_store_f32(float* out, int64_t stride, int rows, int p0, int cnt, const float* vals) {
    for (int t = threadIdx.x; t < cnt * R; t += MG_THREADS) {
        const int i = t / R, r = t % R;
        if (r < rows) out[(int64_t)r * stride + p0 + i] = vals[t];
    }
}

struct MgUnit {
    const bf16* x;   // activation row 0
    int64_t xs;      // activation row stride
    const bf16* w0;  // the unit's two weight rows
    const bf16* w1;
};

// Units of two weight rows over the whole grid: a team of `ks` warps of one CTA owns a unit, splits K, and its first
// lane hands the R x 2 sums to `epi(unit, acc)`.
template <int R, typename Get, typename Epi>
__device__ __forceinline__ void mg_gemv(int units, int K, int ks, int rows, MgSmall& sm, Get get, Epi epi) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tpc = MG_WARPS / ks, team = warp / ks, kpart = warp % ks;
    const int total_teams = gridDim.x * tpc;
    const int rounds = (units + total_teams - 1) / total_teams;
    const int kspan = K / ks;
    for (int it = 0; it < rounds; ++it) {
        const int u = (it * (int)gridDim.x + (int)blockIdx.x) * tpc + team;
        float acc[2][R];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int r = 0; r < R; ++r) acc[j][r] = 0.f;
        if (u < units) {
            const MgUnit m = get(u);
            const bf16* xr[R];
#pragma unroll
            for (int r = 0; r < R; ++r) xr[r] = m.x + (int64_t)(r < rows ? r : 0) * m.xs;
            const bf16* wp[2] = {m.w0, m.w1};
            mg_warp_dot<R, (R <= 2 ? 8 : (R <= 4 ? 4 : 2))>(xr, wp, kpart * kspan, (kpart + 1) * kspan, lane, acc);
            warp_reduce_all<R, 2>(acc);
        }
        if (ks > 1) {
            __syncthreads();
            if (lane == 0) {
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int r = 0; r < R; ++r) sm.red[warp][j][r] = acc[j][r];
            }
            __syncthreads();
            if (kpart == 0 && lane == 0) {
                for (int p = 1; p < ks; ++p)
#pragma unroll
                    for (int j = 0; j < 2; ++j)
#pragma unroll
                        for (int r = 0; r < R; ++r) acc[j][r] += sm.red[warp + p][j][r];
            }
        }
        if (kpart == 0 && lane == 0 && u < units) epi(u, it, team, acc);
    }
}

// ---------------------------------------------------------------------------------------------------
// Balanced form of the projections: the weight rows are dealt to the CTAs in contiguous blocks (a CTA's share is one
// contiguous piece of memory), `kw` warps split K for the same rows and the remaining warps take other rows of the block.
// A warp walks its rows G at a time with G x U independent 16-byte loads in flight per lane and the activation vector of
// a K step reused for the G rows; partial sums meet in shared memory once per pass, so a phase is one or two memory
// round trips and one pair of CTA barriers, however the rows divide among the CTAs.  The activations are in shared
// memory (two resident CTAs leave the SM almost no L1).  The pass is ONE function shared by every projection of the
// step, so its code stays in the instruction cache from phase to phase.

// Row v of a weight table: plain tables are base0 + v * stride; a gate / up pair interleaves two tables (row 2u is gate
// row u, row 2u + 1 is up row u), so that the two halves of a SwiGLU unit land in the same CTA.
struct MgRowMap {
    const bf16* base0;
    const bf16* base1;
    int64_t stride;
    int pair;
    __device__ __forceinline__ const bf16* row(int v) const {
        return pair ? ((v & 1) ? base1 : base0) + (int64_t)(v >> 1) * stride : base0 + (int64_t)v * stride;
    }
};

template <int R, int G, int U>
__device__ __forceinline__ void mg_block_pass_impl(const bf16* x, int64_t xs, int rows, const MgRowMap& m, int n_first, int n_cnt, int K,
                                                   int kw, float* red) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rg = MG_WARPS / kw, grp = warp / kw, kpart = warp % kw;
    const int span = K / kw, kbeg = kpart * span, kend = kbeg + span;
    const bf16* xr[R];
#pragma unroll
    for (int r = 0; r < R; ++r) xr[r] = x + (int64_t)(r < rows ? r : 0) * xs;
    for (int i0 = grp * G; i0 < n_cnt; i0 += rg * G) {
        const bf16* wp[G];
#pragma unroll
        for (int g = 0; g < G; ++g) wp[g] = m.row(n_first + min(i0 + g, n_cnt - 1));
        float acc[G][R];
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int r = 0; r < R; ++r) acc[g][r] = 0.f;
        int k = kbeg + lane * 8;
        for (; k + (U - 1) * 256 < kend; k += U * 256) {
            uint4 wv[U][G];
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int g = 0; g < G; ++g) wv[u][g] = ld_stream16(wp[g] + k + u * 256);
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    float xf[8];
                    unpack8(ld_hot16(xr[r] + k + u * 256), xf);
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        float wf[8];
                        unpack8(wv[u][g], wf);
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[g][r] = fmaf(wf[i], xf[i], acc[g][r]);
                    }
                }
        }
        if (U > 1)
            for (; k < kend; k += 256) {
                uint4 wv[G];
#pragma unroll
                for (int g = 0; g < G; ++g) wv[g] = ld_stream16(wp[g] + k);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    float xf[8];
                    unpack8(ld_hot16(xr[r] + k), xf);
#pragma unroll
                    for (int g = 0; g < G; ++g) {
                        float wf[8];
                        unpack8(wv[g], wf);
#pragma unroll
                        for (int i = 0; i < 8; ++i) acc[g][r] = fmaf(wf[i], xf[i], acc[g][r]);
                    }
                }
            }
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float v = warp_sum(acc[g][r]);
                if (lane == 0 && i0 + g < n_cnt) red[((i0 + g) * kw + kpart) * R + r] = v;
            }
    }
}

// One pass: rows n_first .. n_first + n_cnt - 1 of the table against the activation rows x (shared memory); partial sums
// of the kw K-splitters into red[i][kpart][r], then summed in split order into vals[i * R + r].  Ends with a CTA barrier.
template <int R>
__device__ MG_CALL void mg_block_pass(const bf16* x, int64_t xs, int rows, MgRowMap m, int n_first, int n_cnt, int K, int kw, float* red,
                                           float* vals) {
    constexpr int G1 = R <= 2 ? 12 : (R <= 4 ? 8 : 4), G3 = R <= 4 ? 4 : 2;
    if ((K / kw + 255) / 256 == 1) mg_block_pass_impl<R, G1, 1>(x, xs, rows, m, n_first, n_cnt, K, kw, red);
    else mg_block_pass_impl<R, G3, 3>(x, xs, rows, m, n_first, n_cnt, K, kw, red);
    __syncthreads();
    for (int t = threadIdx.x; t < n_cnt * R; t += MG_THREADS) {
        const int i = t / R, r = t % R;
        float sum = 0.f;
        for (int kp = 0; kp < kw; ++kp) sum += red[(i * kw + kp) * R + r];
        vals[t] = sum;
    }
    __syncthreads();
}

// NV weight rows (K bf16 values each) against the step's activation rows x.  The rows of a CTA come in multiples of
// `align`.  `scratch` is shared memory of `scratch_floats` floats.  After every pass all threads call
// post(first_row, count, vals) with vals[i * R + r] = x_r . w_(first_row + i), fp32.
template <int R, typename Post>
__device__ __forceinline__ void mg_gemv_blocks(int NV, int align, int K, int rows, const bf16* x, int64_t xs, const MgRowMap& m, float* scratch,
                                               int scratch_floats, Post post) {
    int rpc = (NV + (int)gridDim.x - 1) / (int)gridDim.x;
    rpc = (rpc + align - 1) / align * align;
    const int n_begin = (int)blockIdx.x * rpc, n_end = min(NV, n_begin + rpc);
    int kw = MG_WARPS;
    while (kw > 1 && (K / kw < 256 || K % (kw * 8))) kw >>= 1;
    int P = scratch_floats / ((kw + 1) * R);
    P = P / align * align;
    if (P > 256) P = 256;
    float* red = scratch;
    float* vals = scratch + (size_t)P * kw * R;
    for (int p0 = n_begin; p0 < n_end; p0 += P) {
        const int cnt = min(P, n_end - p0);
        mg_block_pass<R>(x, xs, rows, m, p0, cnt, K, kw, red, vals);
        post(p0, cnt, vals);
        __syncthreads();
    }
}

// Activation rows from global memory into shared memory (16-byte pieces); returns the bytes used.  Ends with a CTA barrier.
__device__ __forceinline__ size_t mg_stage_rows(bf16* dst, const bf16* src, int64_t src_stride, int rows, int K) {
    const int vec = K >> 3;
    for (int i = threadIdx.x; i < rows * vec; i += MG_THREADS) {
        const int r = i / vec, v = i % vec;
        reinterpret_cast<uint4*>(dst)[i] = *reinterpret_cast<const uint4*>(src + (int64_t)r * src_stride + v * 8);
    }
    __syncthreads();
    return (size_t)rows * K * 2;
}

// The balanced form of mg_gemv_allreduce: every CTA's block of output columns is summed over the GPUs in one exchange.
template <int R>
__device__ __forceinline__ void mg_blocks_allreduce(const bf16* x, int64_t xs, const bf16* w, int64_t ws, int N, int K, int rows, bf16* out,
                                                    int64_t os, int channel, const MegaArgs& a, MgSmall& sm, unsigned char* big) {
    const int rpc = (N + (int)gridDim.x - 1) / (int)gridDim.x;
    const int n_begin = (int)blockIdx.x * rpc, n_cnt = min(N, n_begin + rpc) - n_begin;
    if (rpc * R > GLMB_AR_SLICE) {
        if (threadIdx.x == 0 && blockIdx.x == 0) raise_status(a.status, GLMB_STATUS_BAD_SHAPE);
        return;
    }
    if (n_cnt <= 0) return;  // the same CTAs on every GPU
    // the activations go to shared memory when they fit beside the scratch; rows wider than that are read in place
    const bf16* xs_ptr = x;
    int64_t x_stride = xs;
    size_t used = 0;
    if ((size_t)rows * K * 2 + 8192 <= (size_t)sm.big_bytes) {
        used = mg_stage_rows(reinterpret_cast<bf16*>(big), x, xs, rows, K);
        xs_ptr = reinterpret_cast<const bf16*>(big);
        x_stride = K;
    }
    int nf;
    float* scratch = mg_scratch(big, used, &nf);
    const MgRowMap m{w, w, ws, 0};
    mg_gemv_blocks<R>(N, 1, K, rows, xs_ptr, x_stride, m, scratch, nf, [&](int p0, int cnt, const float* vals) {
        for (int t = threadIdx.x; t < cnt * R; t += MG_THREADS) sm.sh[(p0 - n_begin) * R + t] = vals[t];
    });
    cta_allreduce_f32_slot(a.comm, channel, blockIdx.x, sm.sh, n_cnt * R);
    for (int t = threadIdx.x; t < n_cnt * R; t += MG_THREADS) {
        const int i = t / R, r = t % R;
        if (r < rows) out[(int64_t)r * os + n_begin + i] = __float2bfloat16_rn(sm.sh[t]);
    }
    __syncthreads();
}

// out[r][n] = bf16(sum over the GPUs of x_r . w_n) for a K-split projection: the sums of every round are parked in shared
// memory, one all-reduce per CTA (slot = CTA index) adds the GPUs' partials in rank order, then the owners store.
template <int R>
__device__ __forceinline__ void mg_gemv_allreduce(const bf16* x, int64_t xs, const bf16* w, int64_t ws, int N, int K, int rows, bf16* out,
                                                  int64_t os, int channel, const MegaArgs& a, MgSmall& sm) {
    const int units = (N + 1) / 2;
    const int ks = mg_pick_ks(units, K, true, GLMB_AR_SLICE, 2 * R);
    const int tpc = MG_WARPS / ks;
    const int total_teams = gridDim.x * tpc;
    const int rounds = (units + total_teams - 1) / total_teams;
    const int per_round = tpc * 2 * R;
    if (rounds * per_round > GLMB_AR_SLICE) {  // does not happen for the supported shapes: refuse instead of overrunning
        if (threadIdx.x == 0 && blockIdx.x == 0) raise_status(a.status, GLMB_STATUS_BAD_SHAPE);
        return;
    }
    mg_gemv<R>(units, K, ks, rows, sm,
               [&](int u) {
                   const int n0 = u * 2;
                   return MgUnit{x, xs, w + (int64_t)n0 * ws, w + (int64_t)min(n0 + 1, N - 1) * ws};
               },
               [&](int, int it, int team, float (&acc)[2][R]) {
#pragma unroll
                   for (int j = 0; j < 2; ++j)
#pragma unroll
                       for (int r = 0; r < R; ++r) sm.sh[it * per_round + (team * 2 + j) * R + r] = acc[j][r];
               });
    // a CTA whose every unit is past the end has nothing to exchange (the same CTAs on every rank)
    const int first_unit = (int)blockIdx.x * tpc;
    if (first_unit >= units) return;
    __syncthreads();
    cta_allreduce_f32_slot(a.comm, channel, blockIdx.x, sm.sh, rounds * per_round);
    for (int i = threadIdx.x; i < rounds * per_round; i += MG_THREADS) {
        const int it = i / per_round, rest = i % per_round;
        const int team = rest / (2 * R), j = (rest / R) & 1, r = rest % R;
        const int n = ((it * (int)gridDim.x + (int)blockIdx.x) * tpc + team) * 2 + j;
        if (n < N && r < rows) out[(int64_t)r * os + n] = __float2bfloat16_rn(sm.sh[i]);
    }
    __syncthreads();
}

// ---------------------------------------------------------------------------------------------------
// add + RMSNorm of one row with the stand-alone kernel's thread mapping and reduction tree (add_rmsnorm_kernel), by the whole
// CTA.  x_out: shared memory; res_out / x_glob (may be null): global copies.
__device__ MG_CALL void mg_addnorm_block(const bf16* update, const bf16* residual, const bf16* weight, bf16* x_out,
                                                 bf16* res_out, bf16* x_glob, int H, float eps, float* scratch) {
    const int nvec = H >> 3;
    uint4 rv[RN_VECS], uv[RN_VECS], wv[RN_VECS];
#pragma unroll
    for (int i = 0; i < RN_VECS; ++i) {
        const int v = threadIdx.x + i * 256;
        if (v < nvec) {
            rv[i] = *reinterpret_cast<const uint4*>(residual + v * 8);
            uv[i] = update ? *reinterpret_cast<const uint4*>(update + v * 8) : make_uint4(0, 0, 0, 0);
            wv[i] = *reinterpret_cast<const uint4*>(weight + v * 8);
        }
    }
    float s[RN_VECS][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < RN_VECS; ++i) {
        const int v = threadIdx.x + i * 256;
        if (v < nvec) {
            float r8[8], u8[8];
            unpack8(rv[i], r8);
            unpack8(uv[i], u8);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                s[i][e] = update ? __fadd_rn(u8[e], r8[e]) : r8[e];
                ss = fmaf(s[i][e], s[i][e], ss);
            }
        }
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / (float)H + eps);
#pragma unroll
    for (int i = 0; i < RN_VECS; ++i) {
        const int v = threadIdx.x + i * 256;
        if (v < nvec) {
            float w8[8];
            unpack8(wv[i], w8);
            uint4 o, rr;
            uint32_t* op = reinterpret_cast<uint32_t*>(&o);
            uint32_t* rp = reinterpret_cast<uint32_t*>(&rr);
#pragma unroll
            for (int e = 0; e < 8; e += 2) {
                op[e >> 1] = pack_bf16(bf16_round(s[i][e] * inv) * w8[e], bf16_round(s[i][e + 1] * inv) * w8[e + 1]);
                rp[e >> 1] = pack_bf16(s[i][e], s[i][e + 1]);
            }
            *reinterpret_cast<uint4*>(x_out + v * 8) = o;
            if (x_glob) *reinterpret_cast<uint4*>(x_glob + v * 8) = o;
            if (res_out) *reinterpret_cast<uint4*>(res_out + v * 8) = rr;
        }
    }
}

// The same row by ONE warp, which plays the eight warps of the CTA version one after the other (same per-thread order,
// same warp sums, same final tree), so that the rows of a step are normalised side by side, one per warp.
__device__ MG_CALL void mg_addnorm_warp(const bf16* update, const bf16* residual, const bf16* weight, bf16* x_out, bf16* res_out,
                                                bf16* x_glob, int H, float eps) {
    const int lane = threadIdx.x & 31, nvec = H >> 3;
    float mine = 0.f;
    for (int vw = 0; vw < 8; ++vw) {
        const int t = vw * 32 + lane;
        uint4 rv[RN_VECS], uv[RN_VECS];
#pragma unroll
        for (int i = 0; i < RN_VECS; ++i) {
            const int v = t + i * 256;
            if (v < nvec) {
                rv[i] = *reinterpret_cast<const uint4*>(residual + v * 8);
                uv[i] = update ? *reinterpret_cast<const uint4*>(update + v * 8) : make_uint4(0, 0, 0, 0);
            }
        }
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < RN_VECS; ++i) {
            const int v = t + i * 256;
            if (v < nvec) {
                float r8[8], u8[8];
                unpack8(rv[i], r8);
                unpack8(uv[i], u8);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float s = update ? __fadd_rn(u8[e], r8[e]) : r8[e];
                    ss = fmaf(s, s, ss);
                }
            }
        }
        ss = warp_sum(ss);
        if (lane == vw) mine = ss;
    }
    const float total = warp_sum(lane < 8 ? mine : 0.f);
    const float inv = 1.0f / sqrtf(total / (float)H + eps);
    for (int vw = 0; vw < 8; ++vw) {
        const int t = vw * 32 + lane;
#pragma unroll
        for (int i = 0; i < RN_VECS; ++i) {
            const int v = t + i * 256;
            if (v < nvec) {
                const uint4 rv = *reinterpret_cast<const uint4*>(residual + v * 8);
                const uint4 uv = update ? *reinterpret_cast<const uint4*>(update + v * 8) : make_uint4(0, 0, 0, 0);
                const uint4 wv = *reinterpret_cast<const uint4*>(weight + v * 8);
                float r8[8], u8[8], w8[8];
                unpack8(rv, r8);
                unpack8(uv, u8);
                unpack8(wv, w8);
                uint4 o, rr;
                uint32_t* op = reinterpret_cast<uint32_t*>(&o);
                uint32_t* rp = reinterpret_cast<uint32_t*>(&rr);
#pragma unroll
                for (int e = 0; e < 8; e += 2) {
                    const float s0 = update ? __fadd_rn(u8[e], r8[e]) : r8[e];
                    const float s1 = update ? __fadd_rn(u8[e + 1], r8[e + 1]) : r8[e + 1];
                    op[e >> 1] = pack_bf16(bf16_round(s0 * inv) * w8[e], bf16_round(s1 * inv) * w8[e + 1]);
                    rp[e >> 1] = pack_bf16(s0, s1);
                }
                *reinterpret_cast<uint4*>(x_out + v * 8) = o;
                if (x_glob) *reinterpret_cast<uint4*>(x_glob + v * 8) = o;
                if (res_out) *reinterpret_cast<uint4*>(res_out + v * 8) = rr;
            }
        }
    }
}

// x_s[r] = RMSNorm(update[r] + residual_in[r]) for every row of the step, in every CTA; CTA 0 also stores the new residual
// (and the normalised rows when x_glob is given).  layer0 rows come straight from the embedding table.
__device__ __forceinline__ void mg_norm_rows(const MegaArgs& a, const bf16* update, const bf16* res_in, bool from_embedding,
                                             const bf16* weight, bf16* x_s, bf16* res_out, bf16* x_glob, MgSmall& sm) {
    const int H = a.H, rows = a.rows, warp = threadIdx.x >> 5;
    const bool writer = blockIdx.x == 0;
    auto source = [&](int r) -> const bf16* {
        if (!from_embedding) return res_in + (int64_t)r * H;
        int t = a.tokens[r];
        if (t < 0 || t >= a.vocab) {
            if (writer && (threadIdx.x & 31) == 0) raise_status(a.status, GLMB_STATUS_BAD_INDEX);
            t = min(max(t, 0), a.vocab - 1);
        }
        return a.embed + (int64_t)t * H;
    };
    if (rows == 1) {
        mg_addnorm_block(update, source(0), weight, x_s, writer ? res_out : nullptr, writer ? x_glob : nullptr, H, a.eps, sm.scratch[0]);
    } else if (warp < rows) {
        const int r = warp;
        mg_addnorm_warp(update ? update + (int64_t)r * H : nullptr, source(r), weight, x_s + (int64_t)r * H,
                        writer && res_out ? res_out + (int64_t)r * H : nullptr, writer && x_glob ? x_glob + (int64_t)r * H : nullptr, H, a.eps);
    }
    __syncthreads();
}

// q_resid row (the q_a LoRA RMSNorm) with the thread mapping and reduction tree of qkv_a_post_row: by the CTA ...
__device__ MG_CALL void mg_qnorm_block(const float* p, int Q, const bf16* q_norm_w, float eps, bf16* dst, float (*scratch)[40]) {
    const int tid = threadIdx.x;
    float4 qv[2];
    uint2 qw[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int i = tid * 4 + k * 1024;
        qv[k] = i < Q ? *reinterpret_cast<const float4*>(p + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        qw[k] = i < Q ? *reinterpret_cast<const uint2*>(q_norm_w + i) : make_uint2(0, 0);
    }
    float ss = 0.f, z0 = 0.f, z1 = 0.f;
    float qr[2][4];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        qr[k][0] = bf16_round(qv[k].x); qr[k][1] = bf16_round(qv[k].y); qr[k][2] = bf16_round(qv[k].z); qr[k][3] = bf16_round(qv[k].w);
#pragma unroll
        for (int e = 0; e < 4; ++e) ss = fmaf(qr[k][e], qr[k][e], ss);
    }
    block_sum3(ss, z0, z1, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)Q + eps);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int i = tid * 4 + k * 1024;
        if (i < Q) {
            uint2 o;
            o.x = pack_bf16(bf16_round(qr[k][0] * inv) * bf16_lo(qw[k].x), bf16_round(qr[k][1] * inv) * bf16_hi(qw[k].x));
            o.y = pack_bf16(bf16_round(qr[k][2] * inv) * bf16_lo(qw[k].y), bf16_round(qr[k][3] * inv) * bf16_hi(qw[k].y));
            *reinterpret_cast<uint2*>(dst + i) = o;
        }
    }
}

// ... and by one warp playing the eight warps in turn.
__device__ MG_CALL void mg_qnorm_warp(const float* p, int Q, const bf16* q_norm_w, float eps, bf16* dst) {
    const int lane = threadIdx.x & 31;
    float mine = 0.f;
    for (int vw = 0; vw < 8; ++vw) {
        const int t = vw * 32 + lane;
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int i = t * 4 + k * 1024;
            const float4 v = i < Q ? *reinterpret_cast<const float4*>(p + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            const float q0 = bf16_round(v.x), q1 = bf16_round(v.y), q2 = bf16_round(v.z), q3 = bf16_round(v.w);
            ss = fmaf(q0, q0, ss); ss = fmaf(q1, q1, ss); ss = fmaf(q2, q2, ss); ss = fmaf(q3, q3, ss);
        }
        ss = warp_sum(ss);
        if (lane == vw) mine = ss;
    }
    const float total = warp_sum(lane < 8 ? mine : 0.f);
    const float inv = 1.0f / sqrtf(total / (float)Q + eps);
    for (int vw = 0; vw < 8; ++vw) {
        const int t = vw * 32 + lane;
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int i = t * 4 + k * 1024;
            if (i < Q) {
                const float4 v = *reinterpret_cast<const float4*>(p + i);
                const uint2 w = *reinterpret_cast<const uint2*>(q_norm_w + i);
                uint2 o;
                o.x = pack_bf16(bf16_round(bf16_round(v.x) * inv) * bf16_lo(w.x), bf16_round(bf16_round(v.y) * inv) * bf16_hi(w.x));
                o.y = pack_bf16(bf16_round(bf16_round(v.z) * inv) * bf16_lo(w.y), bf16_round(bf16_round(v.w) * inv) * bf16_hi(w.y));
                *reinterpret_cast<uint2*>(dst + i) = o;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// Router choice of one row by one warp (the selection of router_topk256_kernel / router_topk_kernel, misc.cu).
__device__ MG_CALL void mg_router_topk_warp(const float* lg, const float* bias, int E, int top_k, int* ids, float* weights) {
    const int lane = threadIdx.x & 31;
    if (E <= 256) {
        // router_topk256_kernel: every lane loads its (up to 8) logits once and keeps score and key in registers
        float lv[8], bv[8], sc[8];
        uint32_t key[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = lane + 32 * i;
            lv[i] = e < E ? lg[e] : 0.f;
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
        return;
    }
    const int per = (E + 31) / 32;  // <= 32
    uint32_t taken = 0;
    float picked_sum = 0.f, my_score = 0.f;
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
        if (lane == 0) ids[s] = best_e == 0x7fffffff ? 0 : best_e;
    }
    if (lane < top_k) weights[lane] = my_score / (picked_sum + 1e-20f);
}

// The routes (row * top_k + slot, ascending) whose expert lives on this GPU.
__device__ __forceinline__ void mg_local_routes(const int* ids, int n, int expert_base, int experts_local, MgSmall& sm) {
    if (threadIdx.x == 0) {
        int c = 0;
        for (int p = 0; p < n; ++p) {
            const int e = ids[p] - expert_base;
            if (e >= 0 && e < experts_local) sm.loc[c++] = p;
        }
        sm.n_loc = c;
    }
    __syncthreads();
}

// ---------------------------------------------------------------------------------------------------
template <int R, bool COMPAT>
__device__ MG_CALL void mg_qkv_a(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr bool compat = COMPAT;
    (void)rows; (void)H; (void)warp; (void)lane; (void)compat; (void)layer; (void)big;
        bf16* x_s = reinterpret_cast<bf16*>(big);
        mg_norm_rows(a, layer == 0 ? nullptr : a.update, a.residual_a, layer == 0, lw.input_norm, x_s, a.residual_b, nullptr, sm);
        const int N = lw.n_qkv_a, units = (N + 1) / 2;
        if (!compat) {
            int nf;
            float* scratch = mg_scratch(big, (size_t)rows * H * 2, &nf);
            mg_gemv_blocks<R>(N, 1, H, rows, x_s, H, MgRowMap{lw.w_qkv_a, lw.w_qkv_a, H, 0}, scratch, nf,
                              [&](int p0, int cnt, const float* vals) { mg_store_f32<R>(a.proj_a, a.proj_stride, rows, p0, cnt, vals); });
            return;
        }
        const int ks = mg_pick_ks(units, H, compat, 0, 0);
        mg_gemv<R>(units, H, ks, rows, sm,
                   [&](int u) {
                       const int n0 = u * 2;
                       return MgUnit{x_s, H, lw.w_qkv_a + (int64_t)n0 * H, lw.w_qkv_a + (int64_t)min(n0 + 1, N - 1) * H};
                   },
                   [&](int u, int, int, float (&acc)[2][R]) {
#pragma unroll
                       for (int j = 0; j < 2; ++j)
#pragma unroll
                           for (int r = 0; r < R; ++r)
                               if (u * 2 + j < N && r < rows) a.proj_a[(int64_t)r * a.proj_stride + u * 2 + j] = acc[j][r];
                   });
}

template <int R, bool COMPAT>
__device__ MG_CALL void mg_q_b(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr bool compat = COMPAT;
    (void)rows; (void)H; (void)warp; (void)lane; (void)compat; (void)layer; (void)big;
        bf16* q_s = reinterpret_cast<bf16*>(big);  // [rows][Q]
        const int Q = a.Q;
        if (rows == 1) {
            mg_qnorm_block(a.proj_a, Q, lw.q_a_norm, a.eps, q_s, sm.scratch);
        } else if (warp < rows) {
            mg_qnorm_warp(a.proj_a + (int64_t)warp * a.proj_stride, Q, lw.q_a_norm, a.eps, q_s + (int64_t)warp * Q);
        }
        __syncthreads();
        if ((int)blockIdx.x < rows) {
            QkvPostArgs p;
            p.proj = a.proj_a; p.proj_stride = a.proj_stride;
            p.q_norm_w = lw.q_a_norm; p.kv_norm_w = lw.kv_a_norm; p.rope_table = a.rope_table; p.inv_freq = a.inv_freq;
            p.k_norm_w = lw.k_norm_w; p.k_norm_b = lw.k_norm_b;
            p.row_pos = a.positions; p.row_lane = a.lane_ids; p.row_active = a.active;
            p.q_resid = a.q_resid; p.kv_new = a.kv_new; p.kv_cache = a.kv_cache; p.index_cache = a.index_cache;
            p.head_w = a.head_w; p.idx_key_new = a.idx_key_new;
            p.Q = Q; p.L = a.L; p.rd = a.rd; p.D = a.D; p.IH = a.IH;
            p.has_indexer = lw.full;
            p.layer = layer; p.layers = a.num_layers; p.index_slot = lw.index_slot; p.full_layers = a.n_full_layers; p.local_cap = a.local_cap;
            p.stripe = a.stripe; p.world = a.cache_world; p.rank = a.cache_rank; p.capacity = a.capacity;
            p.eps = a.eps; p.key_eps = a.key_eps; p.head_scale = a.head_scale;
            p.status = a.status;
            qkv_a_post_row(p, blockIdx.x, sm.scratch, sm.s_key);
            __syncthreads();
        }
        const int N = lw.n_q_b, units = (N + 1) / 2;
        if (!compat) {
            int nf;
            float* scratch = mg_scratch(big, (size_t)rows * Q * 2, &nf);
            mg_gemv_blocks<R>(N, 1, Q, rows, q_s, Q, MgRowMap{lw.w_q_b, lw.w_q_b, Q, 0}, scratch, nf,
                              [&](int p0, int cnt, const float* vals) { mg_store_f32<R>(a.q_proj, a.q_stride, rows, p0, cnt, vals); });
            return;
        }
        const int ks = mg_pick_ks(units, Q, compat, 0, 0);
        mg_gemv<R>(units, Q, ks, rows, sm,
                   [&](int u) {
                       const int n0 = u * 2;
                       return MgUnit{q_s, Q, lw.w_q_b + (int64_t)n0 * Q, lw.w_q_b + (int64_t)min(n0 + 1, N - 1) * Q};
                   },
                   [&](int u, int, int, float (&acc)[2][R]) {
#pragma unroll
                       for (int j = 0; j < 2; ++j)
#pragma unroll
                           for (int r = 0; r < R; ++r)
                               if (u * 2 + j < N && r < rows) a.q_proj[(int64_t)r * a.q_stride + u * 2 + j] = acc[j][r];
                   });
}

template <int R, bool COMPAT>
__device__ MG_CALL void mg_absorb(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr bool compat = COMPAT;
    (void)rows; (void)H; (void)warp; (void)lane; (void)compat; (void)layer; (void)big;
        float(*red)[R][QA_COLS] = reinterpret_cast<float(*)[R][QA_COLS]>(big);
        float(*qs)[QA_MAX_NOPE] = reinterpret_cast<float(*)[QA_MAX_NOPE]>(big + sizeof(float) * 8 * R * QA_COLS);
        PeerComm single;
        single.world = 1; single.rank = 0; single.wait_limit = 0; single.protocol = 0; single.status = a.status; single.seq = nullptr;
        QAbsorbSource src;
        src.q_proj = a.q_proj; src.q_stride = a.q_stride; src.rope_table = a.rope_table; src.row_pos = a.positions; src.capacity = a.capacity;
        const int col_blocks = (a.L + QA_COLS - 1) / QA_COLS;
        const int items = a.heads_local * col_blocks;
        for (int item = blockIdx.x; item < items; item += gridDim.x) {
            __syncthreads();
            q_absorb_tile<R>(nullptr, rows, lw.kv_b, a.heads_local, a.head_base, a.heads_total, a.nope, a.vdim, a.L, a.rd, a.q_full, 0, single,
                             src, item / col_blocks, item % col_blocks, red, qs);
        }
}

template <int R, bool COMPAT>
__device__ MG_CALL void mg_attn(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr bool compat = COMPAT;
    (void)rows; (void)H; (void)warp; (void)lane; (void)compat; (void)layer; (void)big;
        const int nhz = (a.heads_total + AT_HEADS - 1) / AT_HEADS;
        const int items = rows * nhz * a.max_chunks;
        for (int item = blockIdx.x; item < items; item += gridDim.x) {
            const int chunk = item % a.max_chunks, hz = (item / a.max_chunks) % nhz, r = item / (a.max_chunks * nhz);
            if (chunk * AT_CHUNK >= min(max(a.sel_counts[2 * r + 1], 0), a.index_top_k)) continue;
            __syncthreads();
#define MG_TILE(TPW, PVW)                                                                                                              \
    sparse_mla_partial_tile<TPW, PVW>(a.q_full, a.kv_cache, a.sel_local, a.sel_counts, a.lane_ids, a.heads_total, a.rd, layer, a.num_layers, \
                                      a.local_cap, a.index_top_k, a.max_chunks, a.softmax_scale, a.part_o, a.part_ml, a.status, r, chunk,   \
                                      hz * AT_HEADS, big)
            if (a.L == 512) MG_TILE(8, 8);
            else if (a.L == 128) MG_TILE(2, 8);
            else MG_TILE(2, 4);
#undef MG_TILE
        }
}

template <int R, bool COMPAT>
__device__ MG_CALL void mg_merge(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr bool compat = COMPAT;
    (void)rows; (void)H; (void)warp; (void)lane; (void)compat; (void)layer; (void)big;
        // attn_local_merge_kernel (attention.cu), single-GPU form: o_lat[r][h] = bf16(sum_c o_c w_c / l)
        const int Hh = a.heads_total, L = a.L;
        const int items = Hh * rows;
        for (int item = blockIdx.x; item < items; item += gridDim.x) {
            const int h = item % Hh, r = item / Hh;
            __syncthreads();
            const int count = min(max(a.sel_counts[2 * r + 1], 0), a.index_top_k);
            const int chunks = min((count + AT_CHUNK - 1) / AT_CHUNK, MG_MERGE_MAX_CHUNKS);
            const int64_t base = (int64_t)r * a.max_chunks * Hh + h;
            float my_m = -INFINITY, my_l = 0.f;
            if ((int)threadIdx.x < chunks) {
                const float2 ml = *reinterpret_cast<const float2*>(a.part_ml + (base + (int64_t)threadIdx.x * Hh) * 2);
                my_m = ml.x; my_l = ml.y;
            }
            float M = my_m;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
            if (lane == 0 && warp < 4) sm.red_s[warp] = M;
            __syncthreads();
            M = fmaxf(fmaxf(sm.red_s[0], sm.red_s[1]), fmaxf(sm.red_s[2], sm.red_s[3]));
            const float my_w = (int)threadIdx.x < chunks ? expf(my_m - M) : 0.f;
            if (threadIdx.x < MG_MERGE_MAX_CHUNKS) sm.w_s[threadIdx.x] = my_w;
            float l = my_l * my_w;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
            if (lane == 0 && warp < 4) sm.red_s[4 + warp] = l;
            __syncthreads();
            l = (sm.red_s[4] + sm.red_s[5]) + (sm.red_s[6] + sm.red_s[7]);
            for (int j = threadIdx.x * 4; j < L; j += MG_THREADS * 4) {
                float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int c0 = 0; c0 < chunks; c0 += 8) {
                    float4 v[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        v[u] = c0 + u < chunks ? *reinterpret_cast<const float4*>(a.part_o + (base + (int64_t)(c0 + u) * Hh) * L + j)
                                               : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const float wgt = c0 + u < chunks ? sm.w_s[c0 + u] : 0.f;
                        o.x = fmaf(v[u].x, wgt, o.x); o.y = fmaf(v[u].y, wgt, o.y);
                        o.z = fmaf(v[u].z, wgt, o.z); o.w = fmaf(v[u].w, wgt, o.w);
                    }
                }
                uint2 packed;
                if (chunks > 0) { o.x /= l; o.y /= l; o.z /= l; o.w /= l; }
                packed.x = pack_bf16(o.x, o.y);
                packed.y = pack_bf16(o.z, o.w);
                *reinterpret_cast<uint2*>(a.o_lat + ((int64_t)r * Hh + h) * L + j) = packed;
            }
        }
}

template <int R, bool COMPAT>
__device__ MG_CALL void mg_vproj(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr bool compat = COMPAT;
    (void)rows; (void)H; (void)warp; (void)lane; (void)compat; (void)layer; (void)big;
        const int hl = a.heads_local, vd = a.vdim, L = a.L, per_head = (vd + 1) / 2;
        const int units = hl * per_head;
        const int ks = mg_pick_ks(per_head * hl, L, compat, 0, 0);
        const int64_t head_rows = (int64_t)(a.nope + vd) * L;
        mg_gemv<R>(units, L, ks, rows, sm,
                   [&](int u) {
                       const int h = u / per_head, n0 = (u % per_head) * 2;
                       const bf16* wv = lw.kv_b + h * head_rows + (int64_t)a.nope * L;
                       return MgUnit{a.o_lat + (int64_t)h * L, (int64_t)hl * L, wv + (int64_t)n0 * L, wv + (int64_t)min(n0 + 1, vd - 1) * L};
                   },
                   [&](int u, int, int, float (&acc)[2][R]) {
                       const int h = u / per_head, n0 = (u % per_head) * 2;
#pragma unroll
                       for (int j = 0; j < 2; ++j)
#pragma unroll
                           for (int r = 0; r < R; ++r)
                               if (n0 + j < vd && r < rows) a.attn_v[(int64_t)r * hl * vd + h * vd + n0 + j] = __float2bfloat16_rn(acc[j][r]);
                   });
}

template <int R, bool COMPAT>
__device__ MG_CALL void mg_oproj(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr bool compat = COMPAT;
    (void)rows; (void)H; (void)warp; (void)lane; (void)compat; (void)layer; (void)big;
        const int K = a.heads_local * a.vdim;
        if (!compat) {
            mg_blocks_allreduce<R>(a.attn_v, K, lw.w_o, K, H, K, rows, a.attn_out, H, 0, a, sm, big);
            return;
        }
        mg_gemv_allreduce<R>(a.attn_v, K, lw.w_o, K, H, K, rows, a.attn_out, H, 0, a, sm);
}

template <int R, bool COMPAT>
__device__ MG_CALL void mg_mlp_a(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr bool compat = COMPAT;
    (void)rows; (void)H; (void)warp; (void)lane; (void)compat; (void)layer; (void)big;
        bf16* x_s = reinterpret_cast<bf16*>(big);
        mg_norm_rows(a, a.attn_out, a.residual_b, false, lw.post_norm, x_s, a.residual_a, lw.dense ? nullptr : a.x, sm);
        int nf;
        float* scratch = mg_scratch(big, (size_t)rows * H * 2, &nf);
        auto swiglu = [&](const bf16* wg, const bf16* wu, int N, bf16* act, int64_t as) {
            if (!compat) {  // gate row u and up row u are the virtual rows 2u and 2u + 1: a pair never straddles two CTAs
                mg_gemv_blocks<R>(2 * N, 2, H, rows, x_s, H, MgRowMap{wg, wu, H, 1}, scratch, nf,
                                  [&](int p0, int cnt, const float* vals) {
                                      for (int t = threadIdx.x; t < (cnt / 2) * R; t += MG_THREADS) {
                                          const int i = t / R, r = t % R;
                                          if (r < rows) {
                                              const float g = bf16_round(vals[(2 * i) * R + r]), v = bf16_round(vals[(2 * i + 1) * R + r]);
                                              act[(int64_t)r * as + (p0 >> 1) + i] = __float2bfloat16_rn(g * sigmoidf_precise(g) * v);
                                          }
                                      }
                                  });
                return;
            }
            const int ks = mg_pick_ks(N, H, compat, 0, 0);
            mg_gemv<R>(N, H, ks, rows, sm,
                       [&](int u) { return MgUnit{x_s, H, wg + (int64_t)u * H, wu + (int64_t)u * H}; },
                       [&](int u, int, int, float (&acc)[2][R]) {
#pragma unroll
                           for (int r = 0; r < R; ++r)
                               if (r < rows) {
                                   const float g = bf16_round(acc[0][r]), v = bf16_round(acc[1][r]);
                                   act[(int64_t)r * as + u] = __float2bfloat16_rn(g * sigmoidf_precise(g) * v);
                               }
                       });
        };
        if (lw.dense) {
            swiglu(lw.dense_gate, lw.dense_up, a.dense_cols, a.dense_act, a.dense_act_stride);
        } else {
            const int E = a.E, units = (E + 1) / 2;
            if (!compat) {
                mg_gemv_blocks<R>(E, 1, H, rows, x_s, H, MgRowMap{lw.router_w, lw.router_w, H, 0}, scratch, nf,
                                  [&](int p0, int cnt, const float* vals) { mg_store_f32<R>(a.router_logits, E, rows, p0, cnt, vals); });
                swiglu(lw.shared_gate, lw.shared_up, a.shared_cols, a.act_shared, a.act_shared_stride);
                return;
            }
            const int ks = mg_pick_ks(units, H, compat, 0, 0);
            mg_gemv<R>(units, H, ks, rows, sm,
                       [&](int u) {
                           const int n0 = u * 2;
                           return MgUnit{x_s, H, lw.router_w + (int64_t)n0 * H, lw.router_w + (int64_t)min(n0 + 1, E - 1) * H};
                       },
                       [&](int u, int, int, float (&acc)[2][R]) {
#pragma unroll
                           for (int j = 0; j < 2; ++j)
#pragma unroll
                               for (int r = 0; r < R; ++r)
                                   if (u * 2 + j < E && r < rows) a.router_logits[(int64_t)r * E + u * 2 + j] = acc[j][r];
                       });
            __syncthreads();
            swiglu(lw.shared_gate, lw.shared_up, a.shared_cols, a.act_shared, a.act_shared_stride);
        }
}

template <int R, bool COMPAT>
__device__ MG_CALL void mg_mlp_b(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr bool compat = COMPAT;
    (void)rows; (void)H; (void)warp; (void)lane; (void)compat; (void)layer; (void)big;
        if (lw.dense) {
            if (!compat) {
                mg_blocks_allreduce<R>(a.dense_act, a.dense_act_stride, lw.dense_down, a.dense_cols, H, a.dense_cols, rows, a.update, H, 1, a, sm, big);
                return;
            }
            mg_gemv_allreduce<R>(a.dense_act, a.dense_act_stride, lw.dense_down, a.dense_cols, H, a.dense_cols, rows, a.update, H, 1, a, sm);
            return;
        }
        // router choice of every row (one warp per row), the same in every CTA
        if (warp < rows) mg_router_topk_warp(a.router_logits + (int64_t)warp * a.E, lw.router_bias, a.E, a.top_k, sm.ids[warp], sm.wts[warp]);
        __syncthreads();
        const int tk = a.top_k, routes = rows * tk;
        if (blockIdx.x == 0)
            for (int i = threadIdx.x; i < routes; i += MG_THREADS) {
                a.topk_ids[i] = sm.ids[i / tk][i % tk];
                a.topk_w[i] = sm.wts[i / tk][i % tk];
            }
        if (threadIdx.x == 0) {
            int c = 0;
            for (int p = 0; p < routes; ++p) {
                const int e = sm.ids[p / tk][p % tk] - a.expert_base;
                if (e >= 0 && e < a.experts_local) sm.loc[c++] = p;
            }
            sm.n_loc = c;
        }
        __syncthreads();
        mg_stamp(sm, ((unsigned long long)layer << 8) | MG_MLP_B | (1ull << 16));  // router choice done
        if (a.prefetch_cap > 0)  // the down projections of the chosen experts are next: ask the L2 for them now
            for (int i = 0; i < sm.n_loc; ++i) {
                const int p = sm.loc[i];
                mg_prefetch_l2(lw.exp_down + (int64_t)(sm.ids[p / tk][p % tk] - a.expert_base) * H * a.I, (size_t)H * a.I, (size_t)a.prefetch_cap);
            }
        // routed gate/up of this GPU's routes: one item = (route, 16 output rows), moe_gateup_fp8_mma_kernel<1>
        {
            bf16* x_sm = reinterpret_cast<bf16*>(big);  // the normalised rows, staged once (two resident CTAs leave almost no L1)
            const size_t x_bytes = (mg_stage_rows(x_sm, a.x, H, rows, H) + 15) & ~(size_t)15;
            float(*red)[2][MG_MM_ROWS][8] = reinterpret_cast<float(*)[2][MG_MM_ROWS][8]>(big + x_bytes);
            const int I = a.I, blocks = (I + MG_MM_ROWS - 1) / MG_MM_ROWS;
            const int items = sm.n_loc * blocks;
            const int g = lane >> 2, t = lane & 3;
            const int kb = (H + 127) >> 7, chunks = H >> 6;
            for (int item = blockIdx.x; item < items; item += gridDim.x) {
                const int p = sm.loc[item / blocks], n0 = (item % blocks) * MG_MM_ROWS;
                const int e = sm.ids[p / tk][p % tk] - a.expert_base;
                const int route = g == 0 ? p : -1;
                const bf16* xr = x_sm + (int64_t)(route >= 0 ? route / tk : 0) * H;
                const uint8_t* wg_lo = lw.exp_gate + ((int64_t)e * I + n0 + g) * H;
                const uint8_t* wu_lo = lw.exp_up + ((int64_t)e * I + n0 + g) * H;
                const int64_t hi_off = (int64_t)8 * H;
                const int64_t sofs = ((int64_t)e * ((I + 127) >> 7) + (n0 >> 7)) * kb;
                float acc_g[4] = {0.f, 0.f, 0.f, 0.f}, acc_u[4] = {0.f, 0.f, 0.f, 0.f};
                // this warp's chunks in ascending order, three at a time with their twelve weight loads in flight together
                constexpr int UC = 3;
                for (int c0 = warp; c0 < chunks; c0 += MG_WARPS * UC) {
                    uint4 g_lo[UC], g_hi[UC], u_lo[UC], u_hi[UC], x0[UC], x1[UC];
                    float s_g[UC], s_u[UC];
#pragma unroll
                    for (int u = 0; u < UC; ++u) {
                        const int c = c0 + u * MG_WARPS;
                        if (c < chunks) {
                            const int k = (c << 6) + t * 16;
                            g_lo[u] = ld_stream16(wg_lo + k); g_hi[u] = ld_stream16(wg_lo + hi_off + k);
                            u_lo[u] = ld_stream16(wu_lo + k); u_hi[u] = ld_stream16(wu_lo + hi_off + k);
                            x0[u] = x1[u] = make_uint4(0, 0, 0, 0);
                            if (route >= 0) { x0[u] = ld_hot16(xr + k); x1[u] = ld_hot16(xr + k + 8); }
                            s_g[u] = lw.exp_gate_scale[sofs + (c >> 1)]; s_u[u] = lw.exp_up_scale[sofs + (c >> 1)];
                        }
                    }
#pragma unroll
                    for (int u = 0; u < UC; ++u)
                        if (c0 + u * MG_WARPS < chunks) {
                            chunk_mma(acc_g, g_lo[u], g_hi[u], s_g[u], x0[u], x1[u]);
                            chunk_mma(acc_u, u_lo[u], u_hi[u], s_u[u], x0[u], x1[u]);
                        }
                }
                __syncthreads();
                red[warp][0][g][2 * t] = acc_g[0]; red[warp][0][g][2 * t + 1] = acc_g[1];
                red[warp][0][g + 8][2 * t] = acc_g[2]; red[warp][0][g + 8][2 * t + 1] = acc_g[3];
                red[warp][1][g][2 * t] = acc_u[0]; red[warp][1][g][2 * t + 1] = acc_u[1];
                red[warp][1][g + 8][2 * t] = acc_u[2]; red[warp][1][g + 8][2 * t + 1] = acc_u[3];
                __syncthreads();
                if (threadIdx.x < MG_MM_ROWS) {
                    const int n = threadIdx.x;
                    if (n0 + n < I) {
                        float gs = 0.f, us = 0.f;
#pragma unroll
                        for (int w = 0; w < MG_WARPS; ++w) { gs += red[w][0][n][0]; us += red[w][1][n][0]; }
                        const float gv = bf16_round(gs), uv = bf16_round(us);
                        a.act[(int64_t)p * I + n0 + n] = __float2bfloat16_rn(gv * sigmoidf_precise(gv) * uv);
                    }
                }
            }
            __syncthreads();
        }
        mg_stamp(sm, ((unsigned long long)layer << 8) | MG_MLP_B | (2ull << 16));  // routed gate / up done
        // this GPU's K-slice of the shared expert's down projection (fp32 partial)
        {
            const int K = a.shared_cols, units = (H + 1) / 2;
            if (!compat) {
                __syncthreads();
                const size_t used = mg_stage_rows(reinterpret_cast<bf16*>(big), a.act_shared, a.act_shared_stride, rows, K);
                int nf;
                float* scratch = mg_scratch(big, used, &nf);
                mg_gemv_blocks<R>(H, 1, K, rows, reinterpret_cast<const bf16*>(big), K, MgRowMap{lw.shared_down, lw.shared_down, K, 0}, scratch, nf,
                                  [&](int p0, int cnt, const float* vals) { mg_store_f32<R>(a.partial, H, rows, p0, cnt, vals); });
                return;
            }
            const int ks = mg_pick_ks(units, K, compat, 0, 0);
            mg_gemv<R>(units, K, ks, rows, sm,
                       [&](int u) {
                           const int n0 = u * 2;
                           return MgUnit{a.act_shared, a.act_shared_stride, lw.shared_down + (int64_t)n0 * K,
                                         lw.shared_down + (int64_t)min(n0 + 1, H - 1) * K};
                       },
                       [&](int u, int, int, float (&acc)[2][R]) {
#pragma unroll
                           for (int j = 0; j < 2; ++j)
#pragma unroll
                               for (int r = 0; r < R; ++r)
                                   if (u * 2 + j < H && r < rows) a.partial[(int64_t)r * H + u * 2 + j] = acc[j][r];
                       });
        }
}

template <int R, bool COMPAT>
__device__ MG_CALL void mg_moe_down(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr bool compat = COMPAT;
    (void)rows; (void)H; (void)warp; (void)lane; (void)compat; (void)layer; (void)big;
        if (lw.dense) return;
        const int tk = a.top_k, I = a.I;
        mg_local_routes(a.topk_ids, rows * tk, a.expert_base, a.experts_local, sm);
        float(*red)[MG_MM_ROWS][8] = reinterpret_cast<float(*)[MG_MM_ROWS][8]>(big);
        bf16* act_sm = reinterpret_cast<bf16*>(big + sizeof(float) * MG_WARPS * MG_MM_ROWS * 8);
        const bool staged = sizeof(float) * MG_WARPS * MG_MM_ROWS * 8 + (size_t)sm.n_loc * I * 2 <= (size_t)sm.big_bytes;
        if (staged) {
            const int vec = I >> 3;
            for (int i = threadIdx.x; i < sm.n_loc * vec; i += MG_THREADS)
                reinterpret_cast<uint4*>(act_sm)[i] = *reinterpret_cast<const uint4*>(a.act + (int64_t)sm.loc[i / vec] * I + (i % vec) * 8);
            __syncthreads();
        }
        const int blocks = (H + MG_MM_ROWS - 1) / MG_MM_ROWS;
        const int items = sm.n_loc * blocks;
        const int g = lane >> 2, t = lane & 3;
        const int kb = (I + 127) >> 7, chunks = I >> 6;
        for (int item = blockIdx.x; item < items; item += gridDim.x) {
            const int p = sm.loc[item / blocks], n0 = (item % blocks) * MG_MM_ROWS;
            const int e = a.topk_ids[p] - a.expert_base;
            const int route = g == 0 ? p : -1;
            const bf16* xr = staged ? act_sm + (int64_t)(item / blocks) * I : a.act + (int64_t)(route >= 0 ? route : 0) * I;
            const uint8_t* w_lo = lw.exp_down + ((int64_t)e * H + n0 + g) * I;
            const int64_t hi_off = (int64_t)8 * I;
            const int64_t sofs = ((int64_t)e * ((H + 127) >> 7) + (n0 >> 7)) * kb;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            constexpr int UC = 4;  // this warp's chunks in ascending order, four at a time with their loads in flight together
            for (int c0 = warp; c0 < chunks; c0 += MG_WARPS * UC) {
                uint4 lo[UC], hi[UC], x0[UC], x1[UC];
                float sc[UC];
#pragma unroll
                for (int u = 0; u < UC; ++u) {
                    const int c = c0 + u * MG_WARPS;
                    if (c < chunks) {
                        const int k = (c << 6) + t * 16;
                        lo[u] = ld_stream16(w_lo + k); hi[u] = ld_stream16(w_lo + hi_off + k);
                        x0[u] = x1[u] = make_uint4(0, 0, 0, 0);
                        if (route >= 0) { x0[u] = ld_hot16(xr + k); x1[u] = ld_hot16(xr + k + 8); }
                        sc[u] = lw.exp_down_scale[sofs + (c >> 1)];
                    }
                }
#pragma unroll
                for (int u = 0; u < UC; ++u)
                    if (c0 + u * MG_WARPS < chunks) chunk_mma(acc, lo[u], hi[u], sc[u], x0[u], x1[u]);
            }
            __syncthreads();
            red[warp][g][2 * t] = acc[0]; red[warp][g][2 * t + 1] = acc[1];
            red[warp][g + 8][2 * t] = acc[2]; red[warp][g + 8][2 * t + 1] = acc[3];
            __syncthreads();
            if (threadIdx.x < MG_MM_ROWS) {
                const int n = threadIdx.x;
                if (n0 + n < H) {
                    float s = 0.f;
#pragma unroll
                    for (int w = 0; w < MG_WARPS; ++w) s += red[w][n][0];
                    a.dw[(int64_t)p * H + n0 + n] = __float2bfloat16_rn(bf16_round(s) * bf16_round(a.topk_w[p]));
                }
            }
        }
}

template <int R, bool COMPAT>
__device__ MG_CALL void mg_combine(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr bool compat = COMPAT;
    (void)rows; (void)H; (void)warp; (void)lane; (void)compat; (void)layer; (void)big;
        if (lw.dense) return;
        // moe_combine_kernel (gemv.cu) over column slices: CTA-slice s owns `cols` columns of every row
        const int tk = a.top_k;
        int cols = ((H + (int)gridDim.x - 1) / (int)gridDim.x + 3) & ~3;
        const int cap = (GLMB_AR_SLICE / (2 * rows)) & ~3;
        if (cols > cap) cols = cap;
        const int slices = (H + cols - 1) / cols;
        for (int s = blockIdx.x; s < slices; s += gridDim.x) {
            if (s >= GLMB_AR_MAX_CTAS) {
                if (threadIdx.x == 0) raise_status(a.status, GLMB_STATUS_BAD_SHAPE);
                break;
            }
            const int n0 = s * cols, per = rows * cols;
            __syncthreads();
            for (int i = threadIdx.x; i < per; i += MG_THREADS) {
                const int r = i / cols, n = n0 + i % cols;
                float routed = 0.f, shared = 0.f;
                if (n < H) {
                    shared = a.partial[(int64_t)r * H + n];
                    for (int q = 0; q < tk; ++q) {
                        const int p = r * tk + q;
                        const int e = a.topk_ids[p] - a.expert_base;
                        if (e >= 0 && e < a.experts_local) routed += __bfloat162float(a.dw[(int64_t)p * H + n]);
                    }
                }
                sm.sh[i] = shared;
                sm.sh[per + i] = routed;
            }
            __syncthreads();
            cta_allreduce_f32_slot(a.comm, 1, s, sm.sh, 2 * per);
            for (int i = threadIdx.x; i < per; i += MG_THREADS) {
                const int r = i / cols, n = n0 + i % cols;
                if (n >= H) continue;
                const float v = bf16_round(bf16_round(sm.sh[per + i]) * a.routed_scale) + bf16_round(sm.sh[i]);
                a.update[(int64_t)r * H + n] = __float2bfloat16_rn(v);
            }
        }
}

template <int R, bool COMPAT>
__device__ __forceinline__ void mg_phase(const MegaArgs& a, const MegaLayer& lw, int layer, int phase, MgSmall& sm, unsigned char* big) {
    switch (phase) {
    case MG_QKV_A: mg_qkv_a<R, COMPAT>(a, lw, layer, sm, big); break;
    case MG_Q_B: mg_q_b<R, COMPAT>(a, lw, layer, sm, big); break;
    case MG_ABSORB: mg_absorb<R, COMPAT>(a, lw, layer, sm, big); break;
    case MG_ATTN: mg_attn<R, COMPAT>(a, lw, layer, sm, big); break;
    case MG_MERGE: mg_merge<R, COMPAT>(a, lw, layer, sm, big); break;
    case MG_VPROJ: mg_vproj<R, COMPAT>(a, lw, layer, sm, big); break;
    case MG_OPROJ: mg_oproj<R, COMPAT>(a, lw, layer, sm, big); break;
    case MG_MLP_A: mg_mlp_a<R, COMPAT>(a, lw, layer, sm, big); break;
    case MG_MLP_B: mg_mlp_b<R, COMPAT>(a, lw, layer, sm, big); break;
    case MG_MOE_DOWN: mg_moe_down<R, COMPAT>(a, lw, layer, sm, big); break;
    case MG_COMBINE: mg_combine<R, COMPAT>(a, lw, layer, sm, big); break;
    default: break;
    }
}

template <int R, bool COMPAT>
__device__ MG_CALL void mg_head_phase(const MegaArgs& a, int phase, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (phase == MG_HEAD_LOGITS) {
        bf16* x_s = reinterpret_cast<bf16*>(big);
        mg_norm_rows(a, a.num_layers == 0 ? nullptr : a.update, a.residual_a, a.num_layers == 0, a.final_norm, x_s, nullptr, nullptr, sm);
        const int N = a.vocab_local, units = (N + 1) / 2;
        const int ks = mg_pick_ks(units, H, COMPAT, 0, 0);
        if (!COMPAT) {
            int nf;
            float* scratch = mg_scratch(big, (size_t)rows * H * 2, &nf);
            unsigned long long mine = 0ull;  // thread r keeps the best candidate of row r over this CTA's vocabulary block
            mg_gemv_blocks<R>(N, 1, H, rows, x_s, H, MgRowMap{a.lm_head, a.lm_head, H, 0}, scratch, nf,
                              [&](int p0, int cnt, const float* vals) {
                                  const int r = threadIdx.x;
                                  if (r < rows && r < R)
                                      for (int i = 0; i < cnt; ++i) {
                                          const float v = bf16_round(vals[i * R + r]);
                                          if (!isfinite(v)) raise_status(a.status, GLMB_STATUS_NONFINITE);
                                          const unsigned long long k2 = candidate_key(v, a.vocab_base + p0 + i);
                                          mine = k2 > mine ? k2 : mine;
                                      }
                              });
            if ((int)threadIdx.x < rows && (int)threadIdx.x < R && mine) atomicMax(a.local_best + threadIdx.x, mine);
            return;
        }
        unsigned long long run[R];
#pragma unroll
        for (int r = 0; r < R; ++r) run[r] = 0ull;
        mg_gemv<R>(units, H, ks, rows, sm,
                   [&](int u) {
                       const int n0 = u * 2;
                       return MgUnit{x_s, H, a.lm_head + (int64_t)n0 * H, a.lm_head + (int64_t)min(n0 + 1, N - 1) * H};
                   },
                   [&](int u, int, int, float (&acc)[2][R]) {
#pragma unroll
                       for (int r = 0; r < R; ++r)
#pragma unroll
                           for (int j = 0; j < 2; ++j)
                               if (u * 2 + j < N) {
                                   const float v = bf16_round(acc[j][r]);
                                   if (!isfinite(v)) raise_status(a.status, GLMB_STATUS_NONFINITE);
                                   const unsigned long long k2 = candidate_key(v, a.vocab_base + u * 2 + j);
                                   run[r] = k2 > run[r] ? k2 : run[r];
                               }
                   });
        __syncthreads();
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < R; ++r) sm.best[warp][r] = run[r];
        }
        __syncthreads();
        if ((int)threadIdx.x < rows && (int)threadIdx.x < R) {
            unsigned long long key = 0ull;
#pragma unroll
            for (int w2 = 0; w2 < MG_WARPS; ++w2) key = sm.best[w2][threadIdx.x] > key ? sm.best[w2][threadIdx.x] : key;
            if (key) atomicMax(a.local_best + threadIdx.x, key);
        }
        return;
    }
    // MG_HEAD_FINALIZE: step_finalize_kernel (misc.cu) with the candidates of the lm_head phase; one CTA
    if (blockIdx.x != 0) return;
    const PeerComm& c = a.comm;
    const int r = threadIdx.x;
    if (r < rows) {
        const unsigned long long key = a.local_best[r];
        a.local_best[r] = 0ull;
        const int64_t at = (int64_t)c.rank * rows + r;
        a.cand[at] = key;
        for (int p = 0; p < c.world; ++p)
            if (p != c.rank) reinterpret_cast<unsigned long long*>(c.data[p] + a.cand_offset)[at] = key;
    }
    if (c.world > 1) {
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) {
            const uint32_t e = c.seq[GLMB_SEQ_SIG_BASE + 3] + 1;  // signal 3: the sampler's exchange
            c.seq[GLMB_SEQ_SIG_BASE + 3] = e;
            for (int p = 0; p < c.world; ++p) st_release_sys(c.flags[p] + GLMB_FLAG_SIG_BASE + 3 * GLMB_MAX_WORLD + c.rank, e);
        }
        __syncthreads();
        cta_wait_signal(c, 3);
    }
    __syncthreads();
    const int step = a.step_counter ? *a.step_counter : 0;
    if (r < rows) {
        unsigned long long best = 0ull;
        for (int p = 0; p < c.world; ++p) {
            unsigned long long key;
            if (c.world > 1) asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(key) : "l"(a.cand + (int64_t)p * rows + r) : "memory");
            else key = a.cand[(int64_t)p * rows + r];
            best = key > best ? key : best;
        }
        const int best_id = best ? candidate_id(best) : 0;
        const bool active = a.active ? a.active[r] != 0 : true;
        a.out_tokens[(int64_t)(step % a.ring) * rows + r] = active ? best_id : -1;
        if (active) { a.tokens[r] = best_id; a.positions[r] += 1; }
    }
    __syncthreads();
    if (threadIdx.x == 0 && a.step_counter) *a.step_counter = step + 1;
}

// Weights that later phases will stream are requested into the L2 a few phases ahead (they do not depend on the activations),
// so that the dependent chain of small phases finds them there instead of waiting for HBM each time.  Requests are capped
// (prefetch_cap bytes per table) so that large tables on few GPUs do not sweep the L2.
__device__ __forceinline__ void mg_prefetch_ahead(const MegaArgs& a, const MegaLayer& lw, int layer, int phase) {
    if (a.prefetch_cap <= 0) return;
    const size_t cap = (size_t)a.prefetch_cap, H = a.H;
    switch (phase) {
    case MG_QKV_A:
        mg_prefetch_l2(lw.w_q_b, (size_t)lw.n_q_b * a.Q * 2, cap);
        mg_prefetch_l2(lw.kv_b, (size_t)a.heads_local * (a.nope + a.vdim) * a.L * 2, cap);
        break;
    case MG_Q_B:
        mg_prefetch_l2(lw.w_o, H * a.heads_local * a.vdim * 2, cap);
        break;
    case MG_ABSORB:
        if (lw.dense) {
            mg_prefetch_l2(lw.dense_gate, (size_t)a.dense_cols * H * 2, cap);
            mg_prefetch_l2(lw.dense_up, (size_t)a.dense_cols * H * 2, cap);
        } else {
            mg_prefetch_l2(lw.router_w, (size_t)a.E * H * 2, cap);
            mg_prefetch_l2(lw.shared_gate, (size_t)a.shared_cols * H * 2, cap);
            mg_prefetch_l2(lw.shared_up, (size_t)a.shared_cols * H * 2, cap);
        }
        break;
    case MG_ATTN:
        if (lw.dense) mg_prefetch_l2(lw.dense_down, H * a.dense_cols * 2, cap);
        else mg_prefetch_l2(lw.shared_down, H * a.shared_cols * 2, cap);
        break;
    case MG_MLP_A:
        if (layer + 1 < a.num_layers) mg_prefetch_l2(a.layers[layer + 1].w_qkv_a, (size_t)a.layers[layer + 1].n_qkv_a * H * 2, cap);
        else mg_prefetch_l2(a.lm_head, (size_t)a.vocab_local * H * 2, cap);
        break;
    default:
        break;
    }
}

template <int R, bool COMPAT>
__global__ void __launch_bounds__(MG_THREADS, MG_CTAS_PER_SM) decode_mega_kernel(const MegaArgs* __restrict__ gargs, int layer0, int phase0, int layer1,
                                                                    int phase1) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    MgSmall& sm = *reinterpret_cast<MgSmall*>(smem_raw);
    unsigned char* big = smem_raw + ((sizeof(MgSmall) + 15) & ~(size_t)15);
    {
        // the argument block lives in device memory (no per-thread copy of a by-value parameter); the stretch comes as scalars
        const uint32_t* src = reinterpret_cast<const uint32_t*>(gargs);
        uint32_t* dst = reinterpret_cast<uint32_t*>(&sm.args);
        for (int i = threadIdx.x; i < (int)(sizeof(MegaArgs) / 4); i += MG_THREADS) dst[i] = src[i];
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        sm.args.layer0 = layer0; sm.args.phase0 = phase0; sm.args.layer1 = layer1; sm.args.phase1 = phase1;
        sm.big_bytes = MG_BIG_BYTES;
    }
    __syncthreads();
    const MegaArgs& a = sm.args;
    unsigned int epoch = mg_ld_relaxed(&a.bar->gen);
    // per-phase stamps (measurements only): CTA 0's first thread owns the buffer; stretches of a stream run one after the other
    if (threadIdx.x == 0) {
        sm.stamping = a.timeline != nullptr && blockIdx.x == 0;
        sm.stamp_at = sm.stamping ? *reinterpret_cast<volatile unsigned long long*>(a.timeline) : 0ull;
    }
    __syncthreads();
    mg_stamp(sm, 0ull);  // code 0: the stretch begins
    for (int layer = a.layer0; layer <= a.layer1; ++layer) {
        const bool head = layer >= a.num_layers;
        if (!head) {
            __syncthreads();
            const uint32_t* src = reinterpret_cast<const uint32_t*>(a.layers + layer);
            uint32_t* dst = reinterpret_cast<uint32_t*>(&sm.layer);
            for (int i = threadIdx.x; i < (int)(sizeof(MegaLayer) / 4); i += MG_THREADS) dst[i] = src[i];
            __syncthreads();
        }
        const MegaLayer& lw = sm.layer;
        const int first = layer == a.layer0 ? a.phase0 : 1;
        const int last = layer == a.layer1 ? a.phase1 : (head ? MG_HEAD_FINALIZE : MG_COMBINE);
        for (int phase = first; phase <= last; ++phase) {
            if (head) {
                mg_head_phase<R, COMPAT>(a, phase, sm, big);
            } else {
                if (lw.dense && (phase == MG_MOE_DOWN || phase == MG_COMBINE)) continue;  // no work and no barrier
                mg_prefetch_ahead(a, lw, layer, phase);
                mg_phase<R, COMPAT>(a, lw, layer, phase, sm, big);
                if (a.compat_ksplit == 2) {  // measurement: the same phase once more, with its code and operands warm
                    __syncthreads();
                    mg_stamp(sm, (((unsigned long long)layer << 8) | (unsigned long long)phase) | 0x80ull | (7ull << 16));
                    mg_grid_barrier(a.bar, epoch, a.bar_limit, a.status);
                    mg_stamp(sm, (((unsigned long long)layer << 8) | (unsigned long long)phase) | (8ull << 16));
                    mg_phase<R, COMPAT>(a, lw, layer, phase, sm, big);
                }
            }
            const unsigned long long code = ((unsigned long long)layer << 8) | (unsigned long long)phase;
            if (!(layer == a.layer1 && phase == last)) {
                __syncthreads();
                mg_stamp(sm, code | 0x80ull);  // this CTA's work of the phase is done
                mg_grid_barrier(a.bar, epoch, a.bar_limit, a.status);
            }
            mg_stamp(sm, code);
        }
    }
    if (threadIdx.x == 0 && sm.stamping) *reinterpret_cast<volatile unsigned long long*>(a.timeline) = sm.stamp_at;
}

// ---------------------------------------------------------------------------------------------------
// The same phases as kernels of their own (`decode_path = "phases"`): a kernel boundary with programmatic dependent launch
// takes the place of the grid barrier.  A phase then has the occupancy, the L1 and the instruction footprint of a small kernel,
// which the persistent form gives up (two 100 KB CTAs per SM leave no L1, every phase starts on cold code), and the chain is
// still 11 launches per layer instead of 17.  Before it waits for its predecessor, a projection kernel asks the L2 for its own
// block of weight rows: the fetch overlaps the tail of the previous kernel.
__device__ __forceinline__ void mg_prefetch_rows(const bf16* base, int N, int align, size_t row_bytes) {
    if (threadIdx.x != 0 || base == nullptr) return;
    int rpc = (N + (int)gridDim.x - 1) / (int)gridDim.x;
    rpc = (rpc + align - 1) / align * align;
    const int n_begin = (int)blockIdx.x * rpc, n_cnt = min(N, n_begin + rpc) - n_begin;
    if (n_cnt <= 0) return;
    const size_t bytes = ((size_t)n_cnt * row_bytes) & ~(size_t)15;
    const char* p = reinterpret_cast<const char*>(base) + (size_t)n_begin * row_bytes;
    if (bytes && !((uintptr_t)p & 15)) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"((uint32_t)bytes) : "memory");
}

__device__ __forceinline__ void mg_prefetch_own(const MegaArgs& a, const MegaLayer& lw, int layer, int phase) {
    const size_t H2 = (size_t)a.H * 2;
    if (layer >= a.num_layers) {
        if (phase == MG_HEAD_LOGITS) mg_prefetch_rows(a.lm_head, a.vocab_local, 1, H2);
        return;
    }
    switch (phase) {
    case MG_QKV_A: mg_prefetch_rows(lw.w_qkv_a, lw.n_qkv_a, 1, H2); break;
    case MG_Q_B: mg_prefetch_rows(lw.w_q_b, lw.n_q_b, 1, (size_t)a.Q * 2); break;
    case MG_OPROJ: mg_prefetch_rows(lw.w_o, a.H, 1, (size_t)a.heads_local * a.vdim * 2); break;
    case MG_MLP_A:
        if (lw.dense) {
            mg_prefetch_rows(lw.dense_gate, a.dense_cols, 1, H2);
            mg_prefetch_rows(lw.dense_up, a.dense_cols, 1, H2);
        } else {
            mg_prefetch_rows(lw.router_w, a.E, 1, H2);
            mg_prefetch_rows(lw.shared_gate, a.shared_cols, 1, H2);
            mg_prefetch_rows(lw.shared_up, a.shared_cols, 1, H2);
        }
        break;
    case MG_MLP_B:
        if (lw.dense) mg_prefetch_rows(lw.dense_down, a.H, 1, (size_t)a.dense_cols * 2);
        else mg_prefetch_rows(lw.shared_down, a.H, 1, (size_t)a.shared_cols * 2);
        break;
    default: break;
    }
}

// PHASE: 1..11 a layer's phases, 12 / 13 the head's two (a kernel per phase: its own registers, occupancy and code).
// Resident CTAs per SM a phase kernel is compiled for: the streaming phases want many small CTAs (every byte of the table
// requested at once), which bounds their registers; the tile phases keep the registers they need.
template <int R, int PHASE>
struct MgPhaseBlocks {
    static constexpr bool streaming = PHASE == MG_QKV_A || PHASE == MG_Q_B || PHASE == MG_VPROJ || PHASE == MG_OPROJ || PHASE == MG_MLP_A ||
                                      PHASE == MG_MLP_B || PHASE == MG_COMBINE + MG_HEAD_LOGITS;
    static constexpr int value = !streaming ? 2 : (R <= 2 ? 4 : (R <= 4 ? 3 : 2));
};

template <int R, bool COMPAT, int PHASE>
__global__ void __launch_bounds__(MG_THREADS, (MgPhaseBlocks<R, PHASE>::value)) mega_phase_kernel(const __grid_constant__ MegaArgs args, const __grid_constant__ MegaLayer lwp,
                                                                int layer, int big_bytes) {
    constexpr int phase = PHASE > MG_COMBINE ? PHASE - MG_COMBINE : PHASE;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    MgSmall& sm = *reinterpret_cast<MgSmall*>(smem_raw);
    unsigned char* big = smem_raw + ((sizeof(MgSmall) + 15) & ~(size_t)15);
    asm volatile("griddepcontrol.launch_dependents;");
    mg_prefetch_own(args, lwp, layer, phase);  // weights only: nothing the previous kernel writes
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (threadIdx.x == 0) { sm.big_bytes = big_bytes; sm.stamping = 0; }
    __syncthreads();
    if (PHASE > MG_COMBINE) mg_head_phase<R, COMPAT>(args, phase, sm, big);
    else mg_phase<R, COMPAT>(args, lwp, layer, phase, sm, big);
}

// ===================================================================================================
GLMB_API size_t glmb_mega_args_sizeof(void) { return sizeof(MegaArgs); }
GLMB_API size_t glmb_mega_layer_sizeof(void) { return sizeof(MegaLayer); }
GLMB_API size_t glmb_mega_barrier_sizeof(void) { return sizeof(MegaBarrier); }
static size_t mega_smem_bytes(void) { return ((sizeof(MgSmall) + 15) & ~(size_t)15) + MG_BIG_BYTES; }

static int g_mega_cooperative = 1;
// 1 (default): cooperative launch (the driver checks that every CTA of the grid is resident); 0: an ordinary launch of the
// same grid, for drivers that refuse to capture a cooperative launch in a CUDA graph.
GLMB_API void glmb_set_mega_cooperative(int enabled) { g_mega_cooperative = enabled ? 1 : 0; }

template <int R, bool COMPAT>
static int mega_grid_for(int* grid) {
    static int cached[GLMB_MAX_WORLD * 2] = {0};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= GLMB_MAX_WORLD * 2) return 1;
    if (!cached[dev]) {
        if ((e = cudaFuncSetAttribute(decode_mega_kernel<R, COMPAT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mega_smem_bytes())) != cudaSuccess)
            return (int)e;
        int per_sm = 0, sms = 0;
        if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_mega_kernel<R, COMPAT>, MG_THREADS, mega_smem_bytes())) != cudaSuccess)
            return (int)e;
        if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
        if (per_sm < 1) return 2;
        cached[dev] = sms * (per_sm > MG_CTAS_PER_SM ? MG_CTAS_PER_SM : per_sm);
    }
    *grid = cached[dev];
    return 0;
}

template <int R, bool COMPAT>
static int mega_launch(const MegaArgs* device_args, int layer0, int phase0, int layer1, int phase1, cudaStream_t stream) {
    int grid = 0;
    const int rc = mega_grid_for<R, COMPAT>(&grid);
    if (rc) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(MG_THREADS);
    cfg.dynamicSmemBytes = mega_smem_bytes();
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = g_mega_cooperative ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, decode_mega_kernel<R, COMPAT>, device_args, layer0, phase0, layer1, phase1);
}

// Number of CTAs a stretch is launched with on the current device (the same on every GPU of a box), 0 on error.
GLMB_API int glmb_mega_grid(int rows) {
    int grid = 0, rc;
    if (rows <= 1) rc = mega_grid_for<1, false>(&grid);
    else if (rows <= 2) rc = mega_grid_for<2, false>(&grid);
    else if (rows <= 4) rc = mega_grid_for<4, false>(&grid);
    else rc = mega_grid_for<8, false>(&grid);
    return rc ? 0 : grid;
}

// Shapes the persistent kernel takes; everything else keeps the per-kernel path.  Returns 0 when supported, else a
// code naming the first limit that failed.
GLMB_API int glmb_mega_supported(const MegaArgs* a) {
    if (a->rows < 1 || a->rows > GLMB_MAX_ROWS) return 1;
    if ((a->H & 63) || a->H > 256 * 8 * RN_VECS || (size_t)GLMB_MAX_ROWS * a->H * 2 > MG_BIG_BYTES) return 2;
    if (a->Q > 2048 || (a->Q & 7) || a->L > 1024 || (a->L & 3) || (a->rd & 1) || a->rd > 512 || a->IH > 256 || a->D > 256 || ((a->L + a->rd) & 15)) return 3;
    if (a->L != 512 && a->L != 128 && a->L != 64) return 4;
    if (sparse_mla_tile_smem(a->L + a->rd) > MG_BIG_BYTES) return 5;
    if (a->nope > QA_MAX_NOPE || (a->nope & 1) || (a->q_stride & 1) || (a->proj_stride & 3)) return 6;
    if (a->E > 1024 || a->top_k > MG_MAX_TOPK || a->top_k > a->E) return 7;
    if ((a->I & 63) || (a->shared_cols & 7) || (a->dense_cols & 7) || (a->act_shared_stride & 7) || (a->dense_act_stride & 7)) return 8;
    if (a->max_chunks > MG_MERGE_MAX_CHUNKS || a->max_chunks < 1) return 9;
    if (((a->heads_local * a->vdim) & 7) || (a->vdim & 1)) return 10;
    if (a->cache_world != 1) return 11;
    if (a->heads_total != a->heads_local || a->head_base != 0) return 12;
    return 0;
}

// Run the stretch (layer0, phase0) .. (layer1, phase1) (both ends inclusive; layer == num_layers is the head).  `args` is the host
// copy of the argument block (checked here), `device_args` the same bytes in device memory, which is what the kernel reads.
GLMB_API int glmb_mega_decode(const MegaArgs* args, const void* device_args, int layer0, int phase0, int layer1, int phase1, void* stream) {
    if (glmb_mega_supported(args) || !device_args) return 1;
    if (layer0 < 0 || layer1 > args->num_layers || layer0 > layer1 || phase0 < 1 || phase1 < 1) return 1;
    const MegaArgs* d = reinterpret_cast<const MegaArgs*>(device_args);
    cudaStream_t st = (cudaStream_t)stream;
    const int rows = args->rows;
#define MG_GO(RR, CC) return mega_launch<RR, CC>(d, layer0, phase0, layer1, phase1, st)
    if (args->compat_ksplit == 1) {
        if (rows <= 1) MG_GO(1, true);
        if (rows <= 2) MG_GO(2, true);
        if (rows <= 4) MG_GO(4, true);
        MG_GO(8, true);
    }
    if (rows <= 1) MG_GO(1, false);
    if (rows <= 2) MG_GO(2, false);
    if (rows <= 4) MG_GO(4, false);
    MG_GO(8, false);
#undef MG_GO
}

// ---------------------------------------------------------------------------------------------------
// One phase as a kernel of its own.  Grid and shared memory follow from the shapes alone, so every GPU of a box launches the
// same grid (the exchanges inside the all-reduce phases pair CTA j of every rank).
static size_t phase_big_bytes(const MegaArgs& a, const MegaLayer& lw, int layer, int phase, int Rt) {
    const size_t xH = (size_t)a.rows * a.H * 2, scratch = 16384;
    if (layer >= a.num_layers) return phase == MG_HEAD_LOGITS ? xH + scratch : 16;
    auto staged = [&](size_t K) { const size_t x = (size_t)a.rows * K * 2; return (x <= 65536 ? x : 0) + scratch + 8192; };
    switch (phase) {
    case MG_QKV_A: case MG_MLP_A: return xH + scratch;
    case MG_Q_B: return (size_t)a.rows * a.Q * 2 + scratch;
    case MG_ABSORB: return sizeof(float) * (8 * (size_t)Rt * QA_COLS + (size_t)Rt * QA_MAX_NOPE);
    case MG_ATTN: return sparse_mla_tile_smem(a.L + a.rd);
    case MG_OPROJ: return staged((size_t)a.heads_local * a.vdim);
    case MG_MLP_B: {
        if (lw.dense) return staged(a.dense_cols);
        const size_t gate_up = xH + 16 + sizeof(float) * MG_WARPS * 2 * MG_MM_ROWS * 8;
        const size_t shared_down = (size_t)a.rows * a.shared_cols * 2 + scratch;
        return gate_up > shared_down ? gate_up : shared_down;
    }
    case MG_MOE_DOWN: {
        const int routes = a.rows * a.top_k < 16 ? a.rows * a.top_k : 16;
        return sizeof(float) * MG_WARPS * MG_MM_ROWS * 8 + (size_t)routes * a.I * 2;
    }
    default: return 16;
    }
}

static int host_pick_ks(int units, int K) {
    int ks = 1;
    while (ks < MG_WARPS && units * ks < 148 * 4 * MG_WARPS && K % (ks * 2 * 256) == 0 && K / (ks * 2) >= 512) ks *= 2;
    return ks;
}
// CTAs that give every unit of a projection its team of warps in one round (units: pairs of rows, or gate / up pairs)
static int one_round(int units, int K) { return (units + MG_WARPS / host_pick_ks(units, K) - 1) / (MG_WARPS / host_pick_ks(units, K)); }

static int phase_grid(const MegaArgs& a, const MegaLayer& lw, int layer, int phase, int sms, int per_sm) {
    per_sm = per_sm < 1 ? 1 : (per_sm > 4 ? 4 : per_sm);
    const int wide = sms * per_sm;
    auto at_most = [&](int items) { return items < 1 ? 1 : (items < wide ? items : wide); };
    auto capped = [&](int ctas) { return ctas < 1 ? 1 : (ctas > GLMB_AR_MAX_CTAS ? GLMB_AR_MAX_CTAS : ctas); };
    const int H = a.H;
    if (layer >= a.num_layers) return phase == MG_HEAD_LOGITS ? (a.compat_ksplit == 1 ? sms * 8 : wide) : 1;
    if (a.compat_ksplit == 1) {
        switch (phase) {
        case MG_QKV_A: return capped(one_round((lw.n_qkv_a + 1) / 2, H));
        case MG_Q_B: { const int g = one_round((lw.n_q_b + 1) / 2, a.Q); return g < a.rows ? a.rows : g; }
        case MG_OPROJ: return capped(one_round((H + 1) / 2, a.heads_local * a.vdim));
        case MG_MLP_A: {
            if (lw.dense) return capped(one_round(a.dense_cols, H));
            const int r = one_round((a.E + 1) / 2, H), sg = one_round(a.shared_cols, H);
            return capped(r > sg ? r : sg);
        }
        case MG_MLP_B:
            if (lw.dense) return capped(one_round((H + 1) / 2, a.dense_cols));
            break;
        default: break;
        }
    }
    switch (phase) {
    case MG_ABSORB: return at_most(a.heads_local * ((a.L + QA_COLS - 1) / QA_COLS));
    case MG_ATTN: return at_most(a.rows * ((a.heads_total + AT_HEADS - 1) / AT_HEADS) * a.max_chunks);
    case MG_MERGE: return at_most(a.heads_total * a.rows);
    case MG_VPROJ: return at_most((a.heads_local * ((a.vdim + 1) / 2) + MG_WARPS - 1) / MG_WARPS);
    case MG_COMBINE: return at_most(sms * 2);
    case MG_MOE_DOWN: return lw.dense ? 1 : wide;
    default: return wide;
    }
}

template <int R, bool COMPAT, int PHASE>
static int mega_phase_launch_one(const MegaArgs& a, const MegaLayer& lw, int layer, cudaStream_t stream) {
    constexpr int phase = PHASE > MG_COMBINE ? PHASE - MG_COMBINE : PHASE;
    static int sm_count[GLMB_MAX_WORLD * 2] = {0};
    static size_t occ_smem[GLMB_MAX_WORLD * 2] = {0};  // the occupancy answer is cached per shared-memory size
    static int occ[GLMB_MAX_WORLD * 2] = {0};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= GLMB_MAX_WORLD * 2) return 1;
    if (!sm_count[dev]) {
        if ((e = cudaFuncSetAttribute(mega_phase_kernel<R, COMPAT, PHASE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)) != cudaSuccess)
            return (int)e;
        int sms = 0;
        if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
        sm_count[dev] = sms;
    }
    const size_t big = (phase_big_bytes(a, lw, layer, phase, R) + 15) & ~(size_t)15;
    const size_t smem = ((sizeof(MgSmall) + 15) & ~(size_t)15) + big;
    if (smem > 200 * 1024) return 2;
    if (occ_smem[dev] != smem) {
        int n = 0;
        if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, mega_phase_kernel<R, COMPAT, PHASE>, MG_THREADS, smem)) != cudaSuccess) return (int)e;
        occ[dev] = n;
        occ_smem[dev] = smem;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(phase_grid(a, lw, layer, phase, sm_count[dev], occ[dev]));
    cfg.blockDim = dim3(MG_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = g_glmb_pdl_enabled ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, mega_phase_kernel<R, COMPAT, PHASE>, a, lw, layer, (int)big);
}

template <int R, bool COMPAT>
static int mega_phase_launch(const MegaArgs& a, const MegaLayer& lw, int layer, int phase, cudaStream_t stream) {
    const int id = layer >= a.num_layers ? MG_COMBINE + phase : phase;
    switch (id) {
#define MG_P(N) case N: return mega_phase_launch_one<R, COMPAT, N>(a, lw, layer, stream)
        MG_P(1); MG_P(2); MG_P(3); MG_P(4); MG_P(5); MG_P(6); MG_P(7); MG_P(8); MG_P(9); MG_P(10); MG_P(11); MG_P(12); MG_P(13);
#undef MG_P
    default: return 1;
    }
}

// Launch phase `phase` of `layer` (layer == num_layers: the head) as a kernel of its own.  `entry`: the layer's pointer-table
// entry (host copy; ignored for the head).
GLMB_API int glmb_mega_phase(const MegaArgs* args, const MegaLayer* entry, int layer, int phase, void* stream) {
    if (glmb_mega_supported(args)) return 1;
    if (layer < 0 || layer > args->num_layers || phase < 1 || phase > MG_COMBINE) return 1;
    MegaLayer none;
    memset(&none, 0, sizeof(none));
    const MegaLayer& lw = layer < args->num_layers && entry ? *entry : none;
    if (layer < args->num_layers && !entry) return 1;
    cudaStream_t st = (cudaStream_t)stream;
    const int rows = args->rows;
#define MG_GO(RR, CC) return mega_phase_launch<RR, CC>(*args, lw, layer, phase, st)
    if (args->compat_ksplit == 1) {
        if (rows <= 1) MG_GO(1, true);
        if (rows <= 2) MG_GO(2, true);
        if (rows <= 4) MG_GO(4, true);
        MG_GO(8, true);
    }
    if (rows <= 1) MG_GO(1, false);
    if (rows <= 2) MG_GO(2, false);
    if (rows <= 4) MG_GO(4, false);
    MG_GO(8, false);
#undef MG_GO
}

// The exchange a phase performs between the GPUs, for the collective-plan check: out = {kind (0 none, 1 all-reduce, 2 signal),
// channel or signal, CTAs that exchange, floats per CTA}.  `persistent_grid` > 0: the phase runs inside the persistent kernel of
// that many CTAs; 0: as a kernel of its own (its grid follows from the shapes; needs a CUDA device for the occupancy query).
GLMB_API int glmb_mega_phase_exchange(const MegaArgs* a, const MegaLayer* entry, int layer, int phase, int persistent_grid, int* out) {
    out[0] = out[1] = out[2] = out[3] = 0;
    if (layer >= a->num_layers) {
        if (phase == MG_HEAD_FINALIZE) { out[0] = 2; out[1] = 3; }
        return 0;
    }
    if (!entry) return 1;
    const bool dense = entry->dense != 0;
    const int Rt = a->rows <= 1 ? 1 : (a->rows <= 2 ? 2 : (a->rows <= 4 ? 4 : 8));
    const bool ar_gemv = phase == MG_OPROJ || (phase == MG_MLP_B && dense);
    if (!ar_gemv && !(phase == MG_COMBINE && !dense)) return 0;
    int grid = persistent_grid;
    if (grid <= 0) {
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 2;
        grid = phase_grid(*a, *entry, layer, phase, sms, 4);
    }
    out[0] = 1;
    out[1] = phase == MG_OPROJ ? 0 : 1;
    if (ar_gemv) {
        const int K = phase == MG_OPROJ ? a->heads_local * a->vdim : a->dense_cols, units = (a->H + 1) / 2;
        if (a->compat_ksplit == 1) {
            const int tpc = MG_WARPS / host_pick_ks(units, K), teams = grid * tpc, rounds = (units + teams - 1) / teams;
            out[2] = (units + tpc - 1) / tpc < grid ? (units + tpc - 1) / tpc : grid;
            out[3] = rounds * tpc * 2 * Rt;
        } else {
            const int rpc = (a->H + grid - 1) / grid;
            out[2] = (a->H + rpc - 1) / rpc;
            out[3] = rpc * Rt;
        }
    } else {
        int cols = ((a->H + grid - 1) / grid + 3) & ~3;
        const int cap = (GLMB_AR_SLICE / (2 * a->rows)) & ~3;
        if (cols > cap) cols = cap;
        out[2] = (a->H + cols - 1) / cols;
        out[3] = 2 * a->rows * cols;
    }
    return 0;
}

// Byte offsets of a few members, so that the binding can check that it lays the structure out as the compiler does.
GLMB_API void glmb_mega_args_offsets(size_t* out) {
    out[0] = offsetof(MegaArgs, proj_stride);
    out[1] = offsetof(MegaArgs, rows);
    out[2] = offsetof(MegaArgs, eps);
    out[3] = offsetof(MegaArgs, comm);
    out[5] = offsetof(MegaArgs, timeline_cap);
    out[4] = offsetof(MegaLayer, full);
}

// ---------------------------------------------------------------------------------------------------
// Cost of the grid barrier by itself: `iters` barriers back to back on the grid of the decode kernel; CTA 0 reports the
// nanoseconds of the device's global timer.  variant: see mg_grid_barrier_v.
template <int VARIANT>
__global__ void __launch_bounds__(MG_THREADS, 2) mega_barrier_bench_kernel(MegaBarrier* bar, int iters, uint32_t limit, uint32_t* status,
                                                                             unsigned long long* ns) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    (void)smem_raw;
    unsigned int epoch = mg_ld_relaxed(VARIANT == 0 ? &bar->pad0[0] : &bar->gen);
    unsigned long long t0 = 0, t1 = 0;
    mg_grid_barrier_v<VARIANT>(bar, epoch, limit, status);
    if (blockIdx.x == 0 && threadIdx.x == 0) asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    for (int i = 0; i < iters; ++i) mg_grid_barrier_v<VARIANT>(bar, epoch, limit, status);
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
        *ns = t1 - t0;
    }
}

GLMB_API int glmb_mega_barrier_bench(void* bar, int iters, int variant, uint32_t limit, uint32_t* status, unsigned long long* ns, void* stream) {
    int grid = 0;
    const int rc = mega_grid_for<1, false>(&grid);
    if (rc) return rc;
    void (*kernel)(MegaBarrier*, int, uint32_t, uint32_t*, unsigned long long*) =
        variant == 0 ? mega_barrier_bench_kernel<0> : (variant == 2 ? mega_barrier_bench_kernel<2> : mega_barrier_bench_kernel<1>);
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mega_smem_bytes());
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(MG_THREADS);
    cfg.dynamicSmemBytes = mega_smem_bytes();
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, kernel, (MegaBarrier*)bar, iters, limit, status, ns);
}
