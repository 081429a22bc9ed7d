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

#include <cooperative_groups.h>

// Each thread scores IX_KPT adjacent cached keys.  The keys (D bf16 each) live in registers as packed words; the
// query heads are read from shared memory as broadcast float4, HG heads at a time.  A broadcast float4 read
// still returns 512 bytes to the warp, so the shared-memory return path, not the FMA pipe, is the limit: every
// query value fetched is therefore used for IX_KPT keys, and each key element is unpacked once per group of heads.
// Per key and head the dot product is four chains combined as (d0+d1)+(d2+d3).
#define IX_KPT 2
#define IX_THREADS 128
template <int D, int HG>
__global__ void __launch_bounds__(IX_THREADS)
indexer_score_kernel(const float* __restrict__ q_idx, const float* __restrict__ head_w, const bf16* __restrict__ index_cache,
                     const int* __restrict__ row_pos, const int* __restrict__ row_lane, int IH, int index_slot, int full_layers,
                     int local_cap, int stripe, int world, int rank, int capacity, int64_t score_stride, float scale,
                     float* __restrict__ scores, int64_t scores_offset, PeerComm comm, int sig, uint32_t* status) {
    GLMB_PDL_PROLOGUE();
    extern __shared__ float sq[];  // IH * D query, then IH weights
    float* sw = sq + IH * D;
    const int r = blockIdx.y;
    {
        // the query (IH * D fp32, D % 4 == 0) in batches of eight independent 16-byte loads per thread
        const float4* src = reinterpret_cast<const float4*>(q_idx + (int64_t)r * IH * D);
        float4* dst = reinterpret_cast<float4*>(sq);
        const int nvec = IH * D / 4;
        for (int base = 0; base < nvec; base += IX_THREADS * 8) {
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = base + u * IX_THREADS + threadIdx.x;
                v[u] = i < nvec ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = base + u * IX_THREADS + threadIdx.x;
                if (i < nvec) dst[i] = v[u];
            }
        }
    }
    for (int i = threadIdx.x; i < IH; i += blockDim.x) sw[i] = head_w[(int64_t)r * IH + i];
    const int pos = min(max(row_pos[r], 0), capacity - 1);
    const int ctx = pos + 1;
    const int page = stripe * world;
    // number of positions < ctx stored on this rank
    const int rest = ctx % page;
    const int owned = (ctx / page) * stripe + min(max(rest - rank * stripe, 0), stripe);
    const int j0 = (blockIdx.x * blockDim.x + threadIdx.x) * IX_KPT;
    uint32_t kw[IX_KPT][D / 2];
    if (j0 < owned) {
        const bf16* key = index_cache + (((int64_t)row_lane[r] * full_layers + index_slot) * local_cap + j0) * D;
#pragma unroll
        for (int k = 0; k < IX_KPT; ++k)
#pragma unroll
            for (int i = 0; i < D / 8; ++i) {
                // a key past the owned range is read as its own neighbour and its score dropped
                const uint4 v = *reinterpret_cast<const uint4*>(key + (j0 + k < owned ? k : 0) * D + i * 8);
                kw[k][4 * i] = v.x; kw[k][4 * i + 1] = v.y; kw[k][4 * i + 2] = v.z; kw[k][4 * i + 3] = v.w;
            }
    }
    __syncthreads();
    if (j0 < owned) {
        float score[IX_KPT];
#pragma unroll
        for (int k = 0; k < IX_KPT; ++k) score[k] = 0.f;
        for (int h0 = 0; h0 < IH; h0 += HG) {
            float acc[IX_KPT][HG][4];
#pragma unroll
            for (int k = 0; k < IX_KPT; ++k)
#pragma unroll
                for (int h = 0; h < HG; ++h) acc[k][h][0] = acc[k][h][1] = acc[k][h][2] = acc[k][h][3] = 0.f;
            // The unpacking constants come from an opaque move so that the compiler re-unpacks the keys in every
            // group of heads instead of hoisting 2 * D fp32 values out of the loop (which spills).
            uint32_t lo_shift, hi_mask;
            asm volatile("mov.u32 %0, 16; mov.u32 %1, 0xffff0000;" : "=r"(lo_shift), "=r"(hi_mask));
#pragma unroll
            for (int i = 0; i < D / 4; ++i) {
                float kv[IX_KPT][4];
#pragma unroll
                for (int k = 0; k < IX_KPT; ++k) {
                    kv[k][0] = __uint_as_float(kw[k][2 * i] << lo_shift); kv[k][1] = __uint_as_float(kw[k][2 * i] & hi_mask);
                    kv[k][2] = __uint_as_float(kw[k][2 * i + 1] << lo_shift); kv[k][3] = __uint_as_float(kw[k][2 * i + 1] & hi_mask);
                }
#pragma unroll
                for (int h = 0; h < HG; ++h) {
                    const float4 qv = reinterpret_cast<const float4*>(sq + (h0 + h) * D)[i];
#pragma unroll
                    for (int k = 0; k < IX_KPT; ++k) {
                        acc[k][h][0] = fmaf(qv.x, kv[k][0], acc[k][h][0]);
                        acc[k][h][1] = fmaf(qv.y, kv[k][1], acc[k][h][1]);
                        acc[k][h][2] = fmaf(qv.z, kv[k][2], acc[k][h][2]);
                        acc[k][h][3] = fmaf(qv.w, kv[k][3], acc[k][h][3]);
                    }
                }
            }
#pragma unroll
            for (int h = 0; h < HG; ++h)
#pragma unroll
                for (int k = 0; k < IX_KPT; ++k) {
                    const float dot = (acc[k][h][0] + acc[k][h][1]) + (acc[k][h][2] + acc[k][h][3]);
                    score[k] = fmaf(sw[h0 + h], fmaxf(__fmul_rn(dot, scale), 0.f), score[k]);
                }
        }
#pragma unroll
        for (int k = 0; k < IX_KPT; ++k) {
            const int j = j0 + k;
            if (j >= owned) break;
            if (!isfinite(score[k])) raise_status(status, GLMB_STATUS_NONFINITE);
            const int g = (j / stripe) * page + rank * stripe + j % stripe;
            const int64_t at = (int64_t)r * score_stride + g;
            scores[at] = score[k];
            for (int p = 0; p < comm.world; ++p)
                if (p != comm.rank) reinterpret_cast<float*>(comm.data[p] + scores_offset)[at] = score[k];
        }
    }
    grid_signal_peers(comm, sig);
}

// ---------------------------------------------------------------------------------------------------
#define TK_THREADS 1024
#define TK_SMEM_LIMIT (200 * 1024)  // score rows up to 51,200 positions are selected out of shared memory

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

// SMEM: the order-preserving keys of the whole score row are staged in shared memory once (capacity * 4 bytes)
// and every pass runs over shared memory; otherwise every pass re-reads the scores through L2.
// POW2: stripe and world are powers of two, so the owner / local-row arithmetic is shifts and masks (an integer
// division by a run-time value costs more than the rest of the per-position work).
template <bool SMEM, bool POW2>
__global__ void __launch_bounds__(TK_THREADS)
topk_select_kernel(const float* __restrict__ scores, const int* __restrict__ row_pos, int capacity, int64_t score_stride, int top_k, int stripe,
                   int world, int rank, int* __restrict__ sel_global, int* __restrict__ sel_local, int* __restrict__ sel_counts,
                   PeerComm comm, int sig) {
    GLMB_PDL_PROLOGUE();
    extern __shared__ uint32_t keys_s[];
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
    const int stripe_sh = 31 - __clz(stripe), page_sh = 31 - __clz(page);
    auto owner_is_me = [&](int i) -> bool { return (POW2 ? ((i >> stripe_sh) & (world - 1)) : ((i / stripe) % world)) == rank; };
    auto local_row = [&](int i) -> int {
        return POW2 ? (((i >> page_sh) << stripe_sh) | (i & (stripe - 1))) : ((i / page) * stripe + i % stripe);
    };
    const int ipt = (n + TK_THREADS - 1) / TK_THREADS;
    const int begin = min(n, (int)threadIdx.x * ipt), end = min(n, begin + ipt);
    const int lane = threadIdx.x & 31;
    if (SMEM) {
        for (int base = 0; base < n; base += TK_THREADS * 8) {  // eight independent loads per thread per round trip
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = base + u * TK_THREADS + threadIdx.x;
                v[u] = i < n ? __ldcg(sc + i) : 0.f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = base + u * TK_THREADS + threadIdx.x;
                if (i < n) keys_s[i] = orderable_u32(v[u]);
            }
        }
        __syncthreads();
    }
    auto key_at = [&](int i) -> uint32_t { return SMEM ? keys_s[i] : orderable_u32(sc[i]); };

    uint32_t thresh = 0, need = 0;
    const bool take_all = n <= top_k;
    if (!take_all) {
        uint32_t prefix = 0, mask = 0;
        need = top_k;
        const int n_up = ipt * TK_THREADS;  // whole warps walk the row together (the ballots need every lane)
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            if (threadIdx.x < 256) hist[threadIdx.x] = 0;
            __syncthreads();
            for (int i = threadIdx.x; i < n_up; i += TK_THREADS) {
                const uint32_t key = i < n ? key_at(i) : 0u;
                const bool in = i < n && (key & mask) == prefix;
                const uint32_t bin = (key >> shift) & 255u;
                const unsigned active = __ballot_sync(0xffffffffu, in);
                if (in) {
                    // scores cluster in a few bins: one atomic per distinct bin per warp instead of one per key
                    const unsigned same = __match_any_sync(active, bin);
                    if (lane == __ffs(same) - 1) atomicAdd(&hist[bin], (uint32_t)__popc(same));
                }
            }
            __syncthreads();
            if (threadIdx.x < 32) {
                // lane l owns bins 255-8l .. 248-8l (descending); find the bin where the running count reaches `need`
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
        for (int i = begin; i < end; ++i) eq_mine += key_at(i) == thresh;
    uint32_t eq_total;
    uint32_t eq_before = block_exclusive_scan(eq_mine, warp_totals, &eq_total);
    uint32_t sel_mine = 0, own_mine = 0;
    for (int i = begin; i < end; ++i) {
        bool sel = true;
        if (!take_all) {
            const uint32_t key = key_at(i);
            sel = key > thresh;
            if (key == thresh) { sel = eq_before < need; ++eq_before; }
        }
        if (sel) { ++sel_mine; own_mine += owner_is_me(i); }
    }
    eq_before -= eq_mine;  // restore for the second sweep
    uint32_t packed_total;
    const uint32_t packed_before = block_exclusive_scan(sel_mine | (own_mine << 16), warp_totals, &packed_total);
    uint32_t at_g = packed_before & 0xffffu, at_l = packed_before >> 16;
    for (int i = begin; i < end; ++i) {
        bool sel = true;
        if (!take_all) {
            const uint32_t key = key_at(i);
            sel = key > thresh;
            if (key == thresh) { sel = eq_before < need; ++eq_before; }
        }
        if (sel) {
            if (at_g < (uint32_t)top_k) out_g[at_g] = i;
            ++at_g;
            if (owner_is_me(i)) {
                if (at_l < (uint32_t)top_k) out_l[at_l] = local_row(i);
                ++at_l;
            }
        }
    }
    const int total_sel = packed_total & 0xffffu, total_own = packed_total >> 16;
    for (int i = total_sel + threadIdx.x; i < top_k; i += TK_THREADS) out_g[i] = -1;
    for (int i = total_own + threadIdx.x; i < top_k; i += TK_THREADS) out_l[i] = -1;
    if (threadIdx.x == 0) { sel_counts[2 * r] = total_sel; sel_counts[2 * r + 1] = total_own; }
}

// ---------------------------------------------------------------------------------------------------
// The same exact selection spread over a thread-block cluster of 8 CTAs (8 SMs) per query row: each CTA stages one
// eighth of the score row in its shared memory; the per-pass histograms are combined by reading the other CTAs'
// histograms through distributed shared memory after a cluster barrier (one barrier per radix pass, one histogram
// per pass so none is reused); the ordered compaction exchanges per-CTA counts the same way.  Every CTA derives the
// same threshold from the same totals.  The single-CTA kernel above is instruction-bound on one SM (~45 us at 30,000
// positions); this one divides the per-position work by eight.
#define TKC_CTAS 8
template <bool POW2>
__global__ void __cluster_dims__(TKC_CTAS, 1, 1) __launch_bounds__(TK_THREADS)
topk_select_cluster_kernel(const float* __restrict__ scores, const int* __restrict__ row_pos, int capacity, int64_t score_stride, int top_k,
                           int stripe, int world, int rank, int* __restrict__ sel_global, int* __restrict__ sel_local,
                           int* __restrict__ sel_counts, PeerComm comm, int sig) {
    GLMB_PDL_PROLOGUE();
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    extern __shared__ uint32_t keys_s[];
    __shared__ uint32_t hist[4][256];
    __shared__ uint32_t tot[256];
    __shared__ uint32_t warp_totals[33];
    __shared__ uint32_t cnt[4];  // published to the cluster: [0] ties at the threshold, [1] selected, [2] selected and owned
    __shared__ uint32_t s_bucket, s_need;
    cta_wait_signal(comm, sig);
    const int r = blockIdx.y;
    const unsigned crank = cluster.block_rank();
    const int n = min(max(row_pos[r], 0), capacity - 1) + 1;
    const float* sc = scores + (int64_t)r * score_stride;
    int* out_g = sel_global + (int64_t)r * top_k;
    int* out_l = sel_local + (int64_t)r * top_k;
    const int page = stripe * world;
    const int stripe_sh = 31 - __clz(stripe), page_sh = 31 - __clz(page);
    auto owner_is_me = [&](int i) -> bool { return (POW2 ? ((i >> stripe_sh) & (world - 1)) : ((i / stripe) % world)) == rank; };
    auto local_row = [&](int i) -> int {
        return POW2 ? (((i >> page_sh) << stripe_sh) | (i & (stripe - 1))) : ((i / page) * stripe + i % stripe);
    };
    auto owned_before = [&](int x) -> int {  // owned positions below x
        const int rest = x % page;
        return (x / page) * stripe + min(max(rest - rank * stripe, 0), stripe);
    };
    const int seg = (n + TKC_CTAS - 1) / TKC_CTAS;
    const int lo = min(n, (int)crank * seg), hi = min(n, lo + seg);
    const int len = hi - lo;
    const int lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < 4 * 256; i += TK_THREADS) (&hist[0][0])[i] = 0;
    for (int base = 0; base < len; base += TK_THREADS * 8) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = base + u * TK_THREADS + threadIdx.x;
            v[u] = i < len ? __ldcg(sc + lo + i) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int i = base + u * TK_THREADS + threadIdx.x;
            if (i < len) keys_s[i] = orderable_u32(v[u]);
        }
    }
    __syncthreads();

    uint32_t thresh = 0, need = 0;
    const bool take_all = n <= top_k;
    if (!take_all) {
        uint32_t prefix = 0, mask = 0;
        need = top_k;
        const int len_up = ((len + TK_THREADS - 1) / TK_THREADS) * TK_THREADS;
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            for (int i = threadIdx.x; i < len_up; i += TK_THREADS) {
                const uint32_t key = i < len ? keys_s[i] : 0u;
                const bool in = i < len && (key & mask) == prefix;
                const uint32_t bin = (key >> shift) & 255u;
                const unsigned active = __ballot_sync(0xffffffffu, in);
                if (in) {
                    const unsigned same = __match_any_sync(active, bin);
                    if (lane == __ffs(same) - 1) atomicAdd(&hist[pass][bin], (uint32_t)__popc(same));
                }
            }
            cluster.sync();  // every CTA's histogram of this pass is complete
            if (threadIdx.x < 256) {
                uint32_t sum = 0;
#pragma unroll
                for (unsigned c = 0; c < TKC_CTAS; ++c) sum += cluster.map_shared_rank(&hist[pass][0], c)[threadIdx.x];
                tot[threadIdx.x] = sum;
            }
            __syncthreads();
            if (threadIdx.x < 32) {
                uint32_t local[8], sum = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i) { local[i] = tot[255 - (lane * 8 + i)]; sum += local[i]; }
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
    // ordered compaction: each thread owns a contiguous run of this CTA's segment
    const int ipt = (len + TK_THREADS - 1) / TK_THREADS;
    const int begin = min(len, (int)threadIdx.x * ipt), end = min(len, begin + ipt);
    uint32_t eq_mine = 0;
    if (!take_all)
        for (int i = begin; i < end; ++i) eq_mine += keys_s[i] == thresh;
    uint32_t eq_total;
    uint32_t eq_before = block_exclusive_scan(eq_mine, warp_totals, &eq_total);
    if (threadIdx.x == 0) cnt[0] = eq_total;
    cluster.sync();
    for (unsigned c = 0; c < crank; ++c) eq_before += cluster.map_shared_rank(&cnt[0], c)[0];  // ties in lower segments come first
    uint32_t sel_mine = 0, own_mine = 0;
    {
        uint32_t eq_run = eq_before;
        for (int i = begin; i < end; ++i) {
            bool sel = true;
            if (!take_all) {
                const uint32_t key = keys_s[i];
                sel = key > thresh;
                if (key == thresh) { sel = eq_run < need; ++eq_run; }
            }
            if (sel) { ++sel_mine; own_mine += owner_is_me(lo + i); }
        }
    }
    uint32_t packed_total;
    const uint32_t packed_before = block_exclusive_scan(sel_mine | (own_mine << 16), warp_totals, &packed_total);
    if (threadIdx.x == 0) { cnt[1] = packed_total & 0xffffu; cnt[2] = packed_total >> 16; }
    cluster.sync();
    uint32_t at_g = packed_before & 0xffffu, at_l = packed_before >> 16, total_sel = 0, total_own = 0;
    for (unsigned c = 0; c < TKC_CTAS; ++c) {
        const uint32_t* peer_cnt = cluster.map_shared_rank(&cnt[0], c);
        const uint32_t s = peer_cnt[1], o = peer_cnt[2];
        if (c < crank) { at_g += s; at_l += o; }
        total_sel += s; total_own += o;
    }
    for (int i = begin; i < end; ++i) {
        bool sel = true;
        if (!take_all) {
            const uint32_t key = keys_s[i];
            sel = key > thresh;
            if (key == thresh) { sel = eq_before < need; ++eq_before; }
        }
        if (sel) {
            const int g = lo + i;
            if (at_g < (uint32_t)top_k) out_g[at_g] = g;
            ++at_g;
            if (owner_is_me(g)) {
                if (at_l < (uint32_t)top_k) out_l[at_l] = local_row(g);
                ++at_l;
            }
        }
    }
    for (int i = (int)total_sel + (int)crank * TK_THREADS + (int)threadIdx.x; i < top_k; i += TKC_CTAS * TK_THREADS) out_g[i] = -1;
    for (int i = (int)total_own + (int)crank * TK_THREADS + (int)threadIdx.x; i < top_k; i += TKC_CTAS * TK_THREADS) out_l[i] = -1;
    if (crank == 0 && threadIdx.x == 0) { sel_counts[2 * r] = (int)total_sel; sel_counts[2 * r + 1] = (int)total_own; }
    (void)owned_before;
    cluster.sync();  // nobody leaves while a peer may still read its shared memory
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
    dim3 grid(ceil_div(owned_max > 0 ? owned_max : 1, IX_THREADS * IX_KPT), rows);
    const size_t smem = (size_t)(IH * D + IH) * sizeof(float);
    cudaStream_t st = (cudaStream_t)stream;
#define CALL(DD, HH)                                                                                                      \
    GLMB_LAUNCH((indexer_score_kernel<DD, HH>), grid, IX_THREADS, smem, st, q_idx, head_w, (const bf16*)index_cache, row_pos, row_lane, IH, index_slot, \
                                                      full_layers, local_cap, stripe, world, rank, capacity, score_stride, scale, scores,  \
                                                      scores_offset, c, sig, status)
#define CALL_D(DD) do { if (IH % 8 == 0) { CALL(DD, 8); } else if (IH % 4 == 0) { CALL(DD, 4); } else if (IH % 2 == 0) { CALL(DD, 2); } else { CALL(DD, 1); } } while (0)
    if (D == 128) CALL_D(128); else if (D == 64) CALL_D(64); else if (D == 32) CALL_D(32); else return 1;
#undef CALL_D
#undef CALL
    return (int)cudaGetLastError();
}

#define TKC_MAX_ROWS 48
static int g_topk_cluster = 1;
// 1 (default): the 8-CTA cluster kernel for up to TKC_MAX_ROWS rows; 0: always the single-CTA kernel.
GLMB_API void glmb_set_topk_cluster(int enabled) { g_topk_cluster = enabled ? 1 : 0; }

// top_k <= 65535 (the scan packs two 16-bit counters).
GLMB_API int glmb_topk_select(const float* scores, const int* row_pos, int rows, int capacity, int64_t score_stride, int top_k, int stripe, int world,
                              int rank, int* sel_global, int* sel_local, int* sel_counts, const PeerComm* comm, int sig,
                              void* stream) {
    if (top_k > 65535) return 1;
    PeerComm c;
    if (comm) c = *comm; else { memset(&c, 0, sizeof(c)); c.world = 1; }
    const bool pow2 = stripe > 0 && world > 0 && !(stripe & (stripe - 1)) && !(world & (world - 1));
    const size_t seg_bytes = (size_t)ceil_div(capacity, TKC_CTAS) * sizeof(uint32_t);
    // A cluster per row wins on latency while the rows fit the GPU in about one wave (decode: 21 vs 44 us per row); a prefill chunk
    // has thousands of rows, and there the single-CTA kernel does the same work with a third of the CTA-time (1.4 vs 4.2 ms for 4,096
    // rows of 30k scores).
    if (g_topk_cluster && rows <= TKC_MAX_ROWS && seg_bytes <= TK_SMEM_LIMIT) {
        // 8-CTA cluster per row (distributed shared memory): contexts up to 8 x 51,200 positions
        static DeviceOnce cluster_attr_set;
        const int cluster_attr_set_dev = cluster_attr_set.pending();
        if (cluster_attr_set_dev != DeviceOnce::SET) {
            cudaError_t e = cudaFuncSetAttribute(topk_select_cluster_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, TK_SMEM_LIMIT);
            if (e == cudaSuccess)
                e = cudaFuncSetAttribute(topk_select_cluster_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, TK_SMEM_LIMIT);
            if (e != cudaSuccess) return (int)e;
            cluster_attr_set.mark(cluster_attr_set_dev);
        }
        dim3 grid(TKC_CTAS, rows);
        if (pow2)
            GLMB_LAUNCH(topk_select_cluster_kernel<true>, grid, TK_THREADS, seg_bytes, (cudaStream_t)stream, scores, row_pos, capacity, score_stride,
                        top_k, stripe, world, rank, sel_global, sel_local, sel_counts, c, sig);
        else
            GLMB_LAUNCH(topk_select_cluster_kernel<false>, grid, TK_THREADS, seg_bytes, (cudaStream_t)stream, scores, row_pos, capacity, score_stride,
                        top_k, stripe, world, rank, sel_global, sel_local, sel_counts, c, sig);
        return (int)cudaGetLastError();
    }
    const size_t smem = (size_t)capacity * sizeof(uint32_t);
#define TK_LAUNCH(S, P, BYTES)                                                                                              \
    GLMB_LAUNCH((topk_select_kernel<S, P>), rows, TK_THREADS, BYTES, (cudaStream_t)stream, scores, row_pos, capacity, score_stride, top_k, \
                stripe, world, rank, sel_global, sel_local, sel_counts, c, sig)
    if (smem <= TK_SMEM_LIMIT) {
        static DeviceOnce attr_set;
        const int attr_set_dev = attr_set.pending();
        if (attr_set_dev != DeviceOnce::SET) {
            cudaError_t e = cudaFuncSetAttribute(topk_select_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, TK_SMEM_LIMIT);
            if (e == cudaSuccess)
                e = cudaFuncSetAttribute(topk_select_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, TK_SMEM_LIMIT);
            if (e != cudaSuccess) return (int)e;
            attr_set.mark(attr_set_dev);
        }
        if (pow2) { TK_LAUNCH(true, true, smem); } else { TK_LAUNCH(true, false, smem); }
    } else {
        if (pow2) { TK_LAUNCH(false, true, 0); } else { TK_LAUNCH(false, false, 0); }
    }
#undef TK_LAUNCH
    return (int)cudaGetLastError();
}
