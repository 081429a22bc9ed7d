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
#include "attention_core.cuh"
#include "gemv_core.cuh"
#include "moe_mma_core.cuh"
#include "norm_rope_core.cuh"
#include "peer.cuh"

#define MG_THREADS 256
#define MG_WARPS 8
#define MG_MAX_TOPK 32
#define MG_BIG_BYTES (100 * 1024)
#define MG_MERGE_MAX_CHUNKS 128
#define MG_MM_ROWS 16

enum { MG_QKV_A = 1, MG_Q_B, MG_ABSORB, MG_ATTN, MG_MERGE, MG_VPROJ, MG_OPROJ, MG_MLP_A, MG_MLP_B, MG_MOE_DOWN, MG_COMBINE };
enum { MG_HEAD_LOGITS = 1, MG_HEAD_FINALIZE = 2 };

struct MegaBarrier {
    unsigned int arrive;
    unsigned int gen;
    unsigned int abort;
    unsigned int pad;
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
    int64_t proj_stride, q_stride, act_shared_stride, dense_act_stride, cand_offset;
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
    int pad_[3];
};

// ---------------------------------------------------------------------------------------------------
// Grid barrier over all CTAs of the (cooperative) launch.  `epoch` is each thread's copy of the generation the
// grid has completed; it starts from the value every CTA reads at kernel entry (no barrier is in flight then).
__device__ __forceinline__ void mg_grid_barrier(MegaBarrier* b, unsigned int& epoch, uint32_t limit, uint32_t* status) {
    __syncthreads();
    if (threadIdx.x == 0 && *reinterpret_cast<volatile unsigned int*>(&b->abort) == 0u) {
        const unsigned int target = epoch + 1;
        __threadfence();
        if (atomicAdd(&b->arrive, 1u) == gridDim.x - 1) {
            b->arrive = 0;  // nobody arrives at the next barrier before the release below
            __threadfence();
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(&b->gen), "r"(target) : "memory");
        } else {
            bool ok = false;
            for (uint32_t i = 0; i < limit; ++i) {
                unsigned int g;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(g) : "l"(&b->gen) : "memory");
                if ((int)(g - target) >= 0) { ok = true; break; }
                if (i > 4096) {
                    if (*reinterpret_cast<volatile unsigned int*>(&b->abort)) break;
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
            warp_dot_bf16<R, 2>(xr, wp, kpart * kspan, (kpart + 1) * kspan, lane, acc);
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

// out[r][n] = bf16(sum over the GPUs of x_r . w_n) for a K-split projection: the sums of every round are parked in shared
// memory, one all-reduce per CTA (slot = CTA index) adds the GPUs' partials in rank order, then the owners store.
template <int R>
__device__ __forceinline__ void mg_gemv_allreduce(const bf16* x, int64_t xs, const bf16* w, int64_t ws, int N, int K, int rows, bf16* out,
                                                  int64_t os, int channel, const MegaArgs& a, MgSmall& sm) {
    const int units = (N + 1) / 2;
    const int ks = mg_pick_ks(units, K, a.compat_ksplit != 0, GLMB_AR_SLICE, 2 * R);
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
__device__ __forceinline__ void mg_addnorm_block(const bf16* update, const bf16* residual, const bf16* weight, bf16* x_out,
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
__device__ __forceinline__ void mg_addnorm_warp(const bf16* update, const bf16* residual, const bf16* weight, bf16* x_out, bf16* res_out,
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
__device__ __noinline__ void mg_norm_rows(const MegaArgs& a, const bf16* update, const bf16* res_in, bool from_embedding,
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
__device__ __forceinline__ void mg_qnorm_block(const float* p, int Q, const bf16* q_norm_w, float eps, bf16* dst, float (*scratch)[40]) {
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
__device__ __forceinline__ void mg_qnorm_warp(const float* p, int Q, const bf16* q_norm_w, float eps, bf16* dst) {
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
__device__ __forceinline__ void mg_router_topk_warp(const float* lg, const float* bias, int E, int top_k, int* ids, float* weights) {
    const int lane = threadIdx.x & 31;
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
template <int R>
__device__ __noinline__ void mg_qkv_a(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool compat = a.compat_ksplit != 0;
    (void)rows; (void)H; (void)warp; (void)lane; (void)compat; (void)layer; (void)big;
        bf16* x_s = reinterpret_cast<bf16*>(big);
        mg_norm_rows(a, layer == 0 ? nullptr : a.update, a.residual_a, layer == 0, lw.input_norm, x_s, a.residual_b, nullptr, sm);
        const int N = lw.n_qkv_a, units = (N + 1) / 2;
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

template <int R>
__device__ __noinline__ void mg_q_b(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool compat = a.compat_ksplit != 0;
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

template <int R>
__device__ __noinline__ void mg_absorb(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool compat = a.compat_ksplit != 0;
    (void)rows; (void)H; (void)warp; (void)lane; (void)compat; (void)layer; (void)big;
        float(*red)[R][QA_COLS] = reinterpret_cast<float(*)[R][QA_COLS]>(big);
        float(*qs)[QA_MAX_NOPE] = reinterpret_cast<float(*)[QA_MAX_NOPE]>(big + sizeof(float) * 8 * R * QA_COLS);
        PeerComm single;
        single.world = 1; single.rank = 0; single.wait_limit = 0; single.pad_ = 0; single.status = a.status; single.seq = nullptr;
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

template <int R>
__device__ __noinline__ void mg_attn(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool compat = a.compat_ksplit != 0;
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

template <int R>
__device__ __noinline__ void mg_merge(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool compat = a.compat_ksplit != 0;
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

template <int R>
__device__ __noinline__ void mg_vproj(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool compat = a.compat_ksplit != 0;
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

template <int R>
__device__ __noinline__ void mg_oproj(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool compat = a.compat_ksplit != 0;
    (void)rows; (void)H; (void)warp; (void)lane; (void)compat; (void)layer; (void)big;
        const int K = a.heads_local * a.vdim;
        mg_gemv_allreduce<R>(a.attn_v, K, lw.w_o, K, H, K, rows, a.attn_out, H, 0, a, sm);
}

template <int R>
__device__ __noinline__ void mg_mlp_a(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool compat = a.compat_ksplit != 0;
    (void)rows; (void)H; (void)warp; (void)lane; (void)compat; (void)layer; (void)big;
        bf16* x_s = reinterpret_cast<bf16*>(big);
        mg_norm_rows(a, a.attn_out, a.residual_b, false, lw.post_norm, x_s, a.residual_a, lw.dense ? nullptr : a.x, sm);
        auto swiglu = [&](const bf16* wg, const bf16* wu, int N, bf16* act, int64_t as) {
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

template <int R>
__device__ __noinline__ void mg_mlp_b(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool compat = a.compat_ksplit != 0;
    (void)rows; (void)H; (void)warp; (void)lane; (void)compat; (void)layer; (void)big;
        if (lw.dense) {
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
        // routed gate/up of this GPU's routes: one item = (route, 16 output rows), moe_gateup_fp8_mma_kernel<1>
        {
            float(*red)[2][MG_MM_ROWS][8] = reinterpret_cast<float(*)[2][MG_MM_ROWS][8]>(big);
            const int I = a.I, blocks = (I + MG_MM_ROWS - 1) / MG_MM_ROWS;
            const int items = sm.n_loc * blocks;
            const int g = lane >> 2, t = lane & 3;
            const int kb = (H + 127) >> 7, chunks = H >> 6;
            for (int item = blockIdx.x; item < items; item += gridDim.x) {
                const int p = sm.loc[item / blocks], n0 = (item % blocks) * MG_MM_ROWS;
                const int e = sm.ids[p / tk][p % tk] - a.expert_base;
                const int route = g == 0 ? p : -1;
                const bf16* xr = a.x + (int64_t)(route >= 0 ? route / tk : 0) * H;
                const uint8_t* wg_lo = lw.exp_gate + ((int64_t)e * I + n0 + g) * H;
                const uint8_t* wu_lo = lw.exp_up + ((int64_t)e * I + n0 + g) * H;
                const int64_t hi_off = (int64_t)8 * H;
                const int64_t sofs = ((int64_t)e * ((I + 127) >> 7) + (n0 >> 7)) * kb;
                float acc_g[4] = {0.f, 0.f, 0.f, 0.f}, acc_u[4] = {0.f, 0.f, 0.f, 0.f};
                for (int c = warp; c < chunks; c += MG_WARPS) {
                    const int k = (c << 6) + t * 16;
                    const uint4 g_lo = ld_stream16(wg_lo + k), g_hi = ld_stream16(wg_lo + hi_off + k);
                    const uint4 u_lo = ld_stream16(wu_lo + k), u_hi = ld_stream16(wu_lo + hi_off + k);
                    uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0;
                    if (route >= 0) { x0 = ld_hot16(xr + k); x1 = ld_hot16(xr + k + 8); }
                    const float s_g = lw.exp_gate_scale[sofs + (c >> 1)], s_u = lw.exp_up_scale[sofs + (c >> 1)];
                    chunk_mma(acc_g, g_lo, g_hi, s_g, x0, x1);
                    chunk_mma(acc_u, u_lo, u_hi, s_u, x0, x1);
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
        // this GPU's K-slice of the shared expert's down projection (fp32 partial)
        {
            const int K = a.shared_cols, units = (H + 1) / 2;
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

template <int R>
__device__ __noinline__ void mg_moe_down(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool compat = a.compat_ksplit != 0;
    (void)rows; (void)H; (void)warp; (void)lane; (void)compat; (void)layer; (void)big;
        if (lw.dense) return;
        const int tk = a.top_k, I = a.I;
        mg_local_routes(a.topk_ids, rows * tk, a.expert_base, a.experts_local, sm);
        float(*red)[MG_MM_ROWS][8] = reinterpret_cast<float(*)[MG_MM_ROWS][8]>(big);
        const int blocks = (H + MG_MM_ROWS - 1) / MG_MM_ROWS;
        const int items = sm.n_loc * blocks;
        const int g = lane >> 2, t = lane & 3;
        const int kb = (I + 127) >> 7, chunks = I >> 6;
        for (int item = blockIdx.x; item < items; item += gridDim.x) {
            const int p = sm.loc[item / blocks], n0 = (item % blocks) * MG_MM_ROWS;
            const int e = a.topk_ids[p] - a.expert_base;
            const int route = g == 0 ? p : -1;
            const bf16* xr = a.act + (int64_t)(route >= 0 ? route : 0) * I;
            const uint8_t* w_lo = lw.exp_down + ((int64_t)e * H + n0 + g) * I;
            const int64_t hi_off = (int64_t)8 * I;
            const int64_t sofs = ((int64_t)e * ((H + 127) >> 7) + (n0 >> 7)) * kb;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (int c = warp; c < chunks; c += MG_WARPS) {
                const int k = (c << 6) + t * 16;
                const uint4 lo = ld_stream16(w_lo + k), hi = ld_stream16(w_lo + hi_off + k);
                uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0;
                if (route >= 0) { x0 = ld_hot16(xr + k); x1 = ld_hot16(xr + k + 8); }
                chunk_mma(acc, lo, hi, lw.exp_down_scale[sofs + (c >> 1)], x0, x1);
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

template <int R>
__device__ __noinline__ void mg_combine(const MegaArgs& a, const MegaLayer& lw, int layer, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool compat = a.compat_ksplit != 0;
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

template <int R>
__device__ __forceinline__ void mg_phase(const MegaArgs& a, const MegaLayer& lw, int layer, int phase, MgSmall& sm, unsigned char* big) {
    switch (phase) {
    case MG_QKV_A: mg_qkv_a<R>(a, lw, layer, sm, big); break;
    case MG_Q_B: mg_q_b<R>(a, lw, layer, sm, big); break;
    case MG_ABSORB: mg_absorb<R>(a, lw, layer, sm, big); break;
    case MG_ATTN: mg_attn<R>(a, lw, layer, sm, big); break;
    case MG_MERGE: mg_merge<R>(a, lw, layer, sm, big); break;
    case MG_VPROJ: mg_vproj<R>(a, lw, layer, sm, big); break;
    case MG_OPROJ: mg_oproj<R>(a, lw, layer, sm, big); break;
    case MG_MLP_A: mg_mlp_a<R>(a, lw, layer, sm, big); break;
    case MG_MLP_B: mg_mlp_b<R>(a, lw, layer, sm, big); break;
    case MG_MOE_DOWN: mg_moe_down<R>(a, lw, layer, sm, big); break;
    case MG_COMBINE: mg_combine<R>(a, lw, layer, sm, big); break;
    default: break;
    }
}

template <int R>
__device__ __noinline__ void mg_head_phase(const MegaArgs& a, int phase, MgSmall& sm, unsigned char* big) {
    const int rows = a.rows, H = a.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (phase == MG_HEAD_LOGITS) {
        bf16* x_s = reinterpret_cast<bf16*>(big);
        mg_norm_rows(a, a.num_layers == 0 ? nullptr : a.update, a.residual_a, a.num_layers == 0, a.final_norm, x_s, nullptr, nullptr, sm);
        const int N = a.vocab_local, units = (N + 1) / 2;
        const int ks = mg_pick_ks(units, H, a.compat_ksplit != 0, 0, 0);
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

template <int R>
__global__ void __launch_bounds__(MG_THREADS, 2) decode_mega_kernel(const __grid_constant__ MegaArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    MgSmall& sm = *reinterpret_cast<MgSmall*>(smem_raw);
    unsigned char* big = smem_raw + ((sizeof(MgSmall) + 15) & ~(size_t)15);
    unsigned int epoch = *reinterpret_cast<volatile unsigned int*>(&a.bar->gen);
    for (int layer = a.layer0; layer <= a.layer1; ++layer) {
        const bool head = layer >= a.num_layers;
        const int first = layer == a.layer0 ? a.phase0 : 1;
        const int last = layer == a.layer1 ? a.phase1 : (head ? MG_HEAD_FINALIZE : MG_COMBINE);
        for (int phase = first; phase <= last; ++phase) {
            if (head) {
                mg_head_phase<R>(a, phase, sm, big);
            } else {
                const MegaLayer& lw = a.layers[layer];
                if (lw.dense && (phase == MG_MOE_DOWN || phase == MG_COMBINE)) continue;  // no work and no barrier
                mg_phase<R>(a, lw, layer, phase, sm, big);
            }
            if (!(layer == a.layer1 && phase == last)) mg_grid_barrier(a.bar, epoch, a.bar_limit, a.status);
        }
    }
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

template <int R>
static int mega_grid_for(int* grid) {
    static int cached[GLMB_MAX_WORLD * 2] = {0};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= GLMB_MAX_WORLD * 2) return 1;
    if (!cached[dev]) {
        if ((e = cudaFuncSetAttribute(decode_mega_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mega_smem_bytes())) != cudaSuccess)
            return (int)e;
        int per_sm = 0, sms = 0;
        if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_mega_kernel<R>, MG_THREADS, mega_smem_bytes())) != cudaSuccess)
            return (int)e;
        if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
        if (per_sm < 1) return 2;
        cached[dev] = sms * (per_sm > 2 ? 2 : per_sm);
    }
    *grid = cached[dev];
    return 0;
}

template <int R>
static int mega_launch(const MegaArgs& a, cudaStream_t stream) {
    int grid = 0;
    const int rc = mega_grid_for<R>(&grid);
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
    return (int)cudaLaunchKernelEx(&cfg, decode_mega_kernel<R>, a);
}

// Number of CTAs a stretch is launched with on the current device (the same on every GPU of a box), 0 on error.
GLMB_API int glmb_mega_grid(int rows) {
    int grid = 0, rc;
    if (rows <= 1) rc = mega_grid_for<1>(&grid);
    else if (rows <= 2) rc = mega_grid_for<2>(&grid);
    else if (rows <= 4) rc = mega_grid_for<4>(&grid);
    else rc = mega_grid_for<8>(&grid);
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

// Run the stretch (layer0, phase0) .. (layer1, phase1) of `args` (both ends inclusive; layer == num_layers is the head).
GLMB_API int glmb_mega_decode(const MegaArgs* args, int layer0, int phase0, int layer1, int phase1, void* stream) {
    if (glmb_mega_supported(args)) return 1;
    if (layer0 < 0 || layer1 > args->num_layers || layer0 > layer1 || phase0 < 1 || phase1 < 1) return 1;
    MegaArgs a = *args;
    a.layer0 = layer0; a.phase0 = phase0; a.layer1 = layer1; a.phase1 = phase1;
    cudaStream_t st = (cudaStream_t)stream;
    if (a.rows <= 1) return mega_launch<1>(a, st);
    if (a.rows <= 2) return mega_launch<2>(a, st);
    if (a.rows <= 4) return mega_launch<4>(a, st);
    return mega_launch<8>(a, st);
}

// Byte offsets of a few members, so that the binding can check that it lays the structure out as the compiler does.
GLMB_API void glmb_mega_args_offsets(size_t* out) {
    out[0] = offsetof(MegaArgs, proj_stride);
    out[1] = offsetof(MegaArgs, rows);
    out[2] = offsetof(MegaArgs, eps);
    out[3] = offsetof(MegaArgs, comm);
    out[4] = offsetof(MegaLayer, full);
}
