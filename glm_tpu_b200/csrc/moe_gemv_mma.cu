// Routed-expert projections of the decode step with the multiply-accumulate on warp-level tensor-core instructions.
//
// The FP8 expert GEMVs are bound by instruction issue, not by HBM: decoding a weight (e4m3 -> fp32, block scale, round to
// bf16) and then unpacking it and issuing an fp32 FMA costs ~5 instructions per weight.  Here the decoded bf16 pairs go
// straight into mma.sync m16n8k16 (bf16 x bf16 -> fp32): the unpack and the FMA disappear (~3 instructions per weight),
// and the 8 columns of the instruction carry up to 8 activation rows (routes of the same expert) at no extra cost.
//
//   A (16 x 16)  weights: 16 output rows n, 16 of the k values this thread group owns
//   B (16 x 8)   activations: the same 16 k values of up to 8 routes
//   C (16 x 8)   fp32
//
// The k index inside an instruction is a permutation of the true k (both operands use the same one): lane (g, t) loads 16
// consecutive FP8 bytes of weight rows g and g + 8 at byte offset 16 t of a 64-byte chunk, and feeds bytes 4j .. 4j+3 of
// them to the j-th of four instructions, so every weight load is a full 16-byte vector and nothing is shuffled.
// A CTA covers 16 output rows; its 8 warps split K (chunks of 64 round-robin) and combine through shared memory.
//
// Same numerical contract and interfaces as `moe_gateup_fp8_kernel` / `moe_down_fp8_kernel` (`gemv.cu`), which remain for
// shapes these kernels do not take.  Replaces reference `glm_tpu/kernels/fp8_grouped_matmul/kernel.py:51-191` (decode).
#include "common.cuh"
#include "moe_mma_core.cuh"
#include "peer.cuh"

#define MM_WARPS 8
#define MM_THREADS (32 * MM_WARPS)
#define MM_ROWS 16  // output rows per CTA

// act[p][n] = bf16( silu(bf16(x_p . wg[e][n])) * bf16(x_p . wu[e][n]) ) for the routes p of tile t.  H % 64 == 0, I % 16 == 0.
// MM_DEPTH: chunks of a warp whose loads are in flight together (4 for grids of up to two CTAs per SM, where DRAM latency is the
// bound; 1 for large grids, where the registers of a deep pipeline would cost resident CTAs).
template <int RT, int MM_DEPTH>
__global__ void __launch_bounds__(MM_THREADS)
moe_gateup_fp8_mma_kernel(const bf16* __restrict__ x, int64_t xs, int top_k, const int* __restrict__ tile_expert,
                          const int* __restrict__ tile_routes, const int* __restrict__ n_tiles, const uint8_t* __restrict__ wg,
                          const uint8_t* __restrict__ wu, const float* __restrict__ sg, const float* __restrict__ su, int expert_base,
                          int experts_local, int I, int H, bf16* __restrict__ act) {
    GLMB_PDL_PROLOGUE();
    __shared__ float red[MM_WARPS][2][MM_ROWS][8];
    const int tile = blockIdx.y;
    if (n_tiles && tile >= *n_tiles) return;
    const int e = tile_expert[tile] - expert_base;
    if (e < 0 || e >= experts_local) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * MM_ROWS;
    // activation row of this lane's column g
    const int route = g < RT ? (tile_routes ? tile_routes[tile * RT + g] : (g == 0 ? tile : -1)) : -1;
    const bf16* xr = x + (int64_t)(route >= 0 ? route / top_k : 0) * xs;
    const int kb = (H + 127) >> 7;
    const uint8_t* wg_lo = wg + ((int64_t)e * I + n0 + g) * H;
    const uint8_t* wu_lo = wu + ((int64_t)e * I + n0 + g) * H;
    const int64_t hi_off = (int64_t)8 * H;
    const int64_t sofs = ((int64_t)e * ((I + 127) >> 7) + (n0 >> 7)) * kb;
    float acc_g[4] = {0.f, 0.f, 0.f, 0.f}, acc_u[4] = {0.f, 0.f, 0.f, 0.f};
    const int chunks = H >> 6;
    // MM_DEPTH chunks of every warp are in flight at once (all their loads are issued before the first multiply): with one CTA per
    // 16 output rows a grid is a few hundred CTAs, and a warp that waited for one chunk at a time would spend its life in DRAM
    // latency.  The chunks still enter the accumulators in ascending order, so the sums are the same bits at any depth.
    for (int c0 = warp; c0 < chunks; c0 += MM_WARPS * MM_DEPTH) {
        uint4 g_lo[MM_DEPTH], g_hi[MM_DEPTH], u_lo[MM_DEPTH], u_hi[MM_DEPTH], x0[MM_DEPTH], x1[MM_DEPTH];
        float s_g[MM_DEPTH], s_u[MM_DEPTH];
#pragma unroll
        for (int u = 0; u < MM_DEPTH; ++u) {
            const int c = c0 + u * MM_WARPS;
            x0[u] = make_uint4(0, 0, 0, 0); x1[u] = x0[u];
            if (c < chunks) {
                const int k = (c << 6) + t * 16;
                g_lo[u] = ld_stream16(wg_lo + k); g_hi[u] = ld_stream16(wg_lo + hi_off + k);
                u_lo[u] = ld_stream16(wu_lo + k); u_hi[u] = ld_stream16(wu_lo + hi_off + k);
                if (route >= 0) { x0[u] = ld_hot16(xr + k); x1[u] = ld_hot16(xr + k + 8); }
                s_g[u] = sg[sofs + (c >> 1)]; s_u[u] = su[sofs + (c >> 1)];
            }
        }
#pragma unroll
        for (int u = 0; u < MM_DEPTH; ++u) {
            if (c0 + u * MM_WARPS < chunks) {
                chunk_mma(acc_g, g_lo[u], g_hi[u], s_g[u], x0[u], x1[u]);
                chunk_mma(acc_u, u_lo[u], u_hi[u], s_u[u], x0[u], x1[u]);
            }
        }
    }
    // C fragment: (row g, routes 2t, 2t+1), (row g + 8, routes 2t, 2t+1)
    red[warp][0][g][2 * t] = acc_g[0]; red[warp][0][g][2 * t + 1] = acc_g[1];
    red[warp][0][g + 8][2 * t] = acc_g[2]; red[warp][0][g + 8][2 * t + 1] = acc_g[3];
    red[warp][1][g][2 * t] = acc_u[0]; red[warp][1][g][2 * t + 1] = acc_u[1];
    red[warp][1][g + 8][2 * t] = acc_u[2]; red[warp][1][g + 8][2 * t + 1] = acc_u[3];
    __syncthreads();
    if (threadIdx.x < MM_ROWS * RT) {
        const int n = threadIdx.x % MM_ROWS, col = threadIdx.x / MM_ROWS;
        const int p = tile_routes ? tile_routes[tile * RT + col] : (col == 0 ? tile : -1);
        if (p >= 0 && n0 + n < I) {
            float gs = 0.f, us = 0.f;
#pragma unroll
            for (int w = 0; w < MM_WARPS; ++w) { gs += red[w][0][n][col]; us += red[w][1][n][col]; }
            const float gv = bf16_round(gs), uv = bf16_round(us);
            act[(int64_t)p * I + n0 + n] = __float2bfloat16_rn(gv * sigmoidf_precise(gv) * uv);
        }
    }
}

// dw[p][n] = bf16( bf16(act[p] . wd[e][n]) * bf16(route_weight[p]) ).  I % 64 == 0, H % 16 == 0.
template <int RT, int MM_DEPTH>
__global__ void __launch_bounds__(MM_THREADS)
moe_down_fp8_mma_kernel(const bf16* __restrict__ act, const float* __restrict__ route_weight, const int* __restrict__ tile_expert,
                        const int* __restrict__ tile_routes, const int* __restrict__ n_tiles, const uint8_t* __restrict__ wd,
                        const float* __restrict__ sd, int expert_base, int experts_local, int I, int H, bf16* __restrict__ dw) {
    GLMB_PDL_PROLOGUE();
    __shared__ float red[MM_WARPS][MM_ROWS][8];
    const int tile = blockIdx.y;
    if (n_tiles && tile >= *n_tiles) return;
    const int e = tile_expert[tile] - expert_base;
    if (e < 0 || e >= experts_local) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * MM_ROWS;
    const int route = g < RT ? (tile_routes ? tile_routes[tile * RT + g] : (g == 0 ? tile : -1)) : -1;
    const bf16* xr = act + (int64_t)(route >= 0 ? route : 0) * I;
    const int kb = (I + 127) >> 7;
    const uint8_t* w_lo = wd + ((int64_t)e * H + n0 + g) * I;
    const int64_t hi_off = (int64_t)8 * I;
    const int64_t sofs = ((int64_t)e * ((H + 127) >> 7) + (n0 >> 7)) * kb;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const int chunks = I >> 6;
    for (int c0 = warp; c0 < chunks; c0 += MM_WARPS * MM_DEPTH) {  // MM_DEPTH chunks in flight, entered in ascending order
        uint4 lo[MM_DEPTH], hi[MM_DEPTH], x0[MM_DEPTH], x1[MM_DEPTH];
        float sc[MM_DEPTH];
#pragma unroll
        for (int u = 0; u < MM_DEPTH; ++u) {
            const int c = c0 + u * MM_WARPS;
            x0[u] = make_uint4(0, 0, 0, 0); x1[u] = x0[u];
            if (c < chunks) {
                const int k = (c << 6) + t * 16;
                lo[u] = ld_stream16(w_lo + k); hi[u] = ld_stream16(w_lo + hi_off + k);
                if (route >= 0) { x0[u] = ld_hot16(xr + k); x1[u] = ld_hot16(xr + k + 8); }
                sc[u] = sd[sofs + (c >> 1)];
            }
        }
#pragma unroll
        for (int u = 0; u < MM_DEPTH; ++u)
            if (c0 + u * MM_WARPS < chunks) chunk_mma(acc, lo[u], hi[u], sc[u], x0[u], x1[u]);
    }
    red[warp][g][2 * t] = acc[0]; red[warp][g][2 * t + 1] = acc[1];
    red[warp][g + 8][2 * t] = acc[2]; red[warp][g + 8][2 * t + 1] = acc[3];
    __syncthreads();
    if (threadIdx.x < MM_ROWS * RT) {
        const int n = threadIdx.x % MM_ROWS, col = threadIdx.x / MM_ROWS;
        const int p = tile_routes ? tile_routes[tile * RT + col] : (col == 0 ? tile : -1);
        if (p >= 0 && n0 + n < H) {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < MM_WARPS; ++w) s += red[w][n][col];
            dw[(int64_t)p * H + n0 + n] = __float2bfloat16_rn(bf16_round(s) * bf16_round(route_weight[p]));
        }
    }
}

// The same projection for a SHORT K (experts sliced by intermediate column: I is a few hundred) and tiles of several routes (prefill
// chunks of few rows): with K split over the warps a CTA would stream 16 x I bytes and spend its life starting and ending, so here a
// warp walks the whole K of its own 16 output rows (up to four 64-wide chunks in flight) and a CTA covers 16 * MM_WARPS rows; nothing
// crosses warps.  Same slices and roundings as `moe_down_fp8_mma_kernel`; the fp32 sum over K runs in one accumulator.
template <int RT>
__global__ void __launch_bounds__(MM_THREADS)
moe_down_fp8_mma_shortk_kernel(const bf16* __restrict__ act, const float* __restrict__ route_weight, const int* __restrict__ tile_expert,
                               const int* __restrict__ tile_routes, const int* __restrict__ n_tiles, const uint8_t* __restrict__ wd,
                               const float* __restrict__ sd, int expert_base, int experts_local, int I, int H, bf16* __restrict__ dw) {
    GLMB_PDL_PROLOGUE();
    const int tile = blockIdx.y;
    if (n_tiles && tile >= *n_tiles) return;
    const int e = tile_expert[tile] - expert_base;
    if (e < 0 || e >= experts_local) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int n0 = (blockIdx.x * MM_WARPS + warp) * MM_ROWS;
    if (n0 >= H) return;
    const int route = g < RT ? tile_routes[tile * RT + g] : -1;
    const bf16* xr = act + (int64_t)(route >= 0 ? route : 0) * I;
    const int kb = (I + 127) >> 7;
    const uint8_t* w_lo = wd + ((int64_t)e * H + n0 + g) * I;
    const int64_t hi_off = (int64_t)8 * I;
    const int64_t sofs = ((int64_t)e * ((H + 127) >> 7) + (n0 >> 7)) * kb;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const int chunks = I >> 6;
    for (int c0 = 0; c0 < chunks; c0 += 4) {
        uint4 lo[4], hi[4], x0[4], x1[4];
        float sc[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int c = c0 + u;
            x0[u] = make_uint4(0, 0, 0, 0); x1[u] = x0[u];
            if (c < chunks) {
                const int k = (c << 6) + t * 16;
                lo[u] = ld_stream16(w_lo + k); hi[u] = ld_stream16(w_lo + hi_off + k);
                if (route >= 0) { x0[u] = ld_hot16(xr + k); x1[u] = ld_hot16(xr + k + 8); }
                sc[u] = sd[sofs + (c >> 1)];
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (c0 + u < chunks) chunk_mma(acc, lo[u], hi[u], sc[u], x0[u], x1[u]);
    }
    // C fragment: (row g, routes 2t, 2t+1), (row g + 8, routes 2t, 2t+1)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int col = 2 * t + j;
        const int p = col < RT ? tile_routes[tile * RT + col] : -1;
        if (p >= 0) {
            const float rw = bf16_round(route_weight[p]);
            dw[(int64_t)p * H + n0 + g] = __float2bfloat16_rn(bf16_round(acc[j]) * rw);
            dw[(int64_t)p * H + n0 + g + 8] = __float2bfloat16_rn(bf16_round(acc[2 + j]) * rw);
        }
    }
}

// Experts sliced by intermediate column (every GPU holds I columns of EVERY expert): the down projection of all routes of a
// row, the route sum, the shared expert's partial and the all-reduce over the GPUs in one kernel.  A route's whole K (= this GPU's
// I columns, a few hundred) fits one warp, so warp w takes route w of the row and nothing is reduced across warps but the route
// sum itself.  A CTA owns 16 output columns of up to GLMB_MAX_ROWS rows: the same slices, the same route order and the same
// roundings as `moe_down_fp8_mma_kernel` followed by `moe_combine_kernel` (gemv.cu) in one launch instead of two (the fp32 sum
// over K runs inside one warp's accumulator instead of across eight warps, so a value may land on the neighbouring bf16).
//   dw[p][n] = bf16( bf16(act[p] . wd[e_p][n]) * bf16(route_weight[p]) );  routed = sum_p dw[p][n] (fp32, route order)
//   out[r][n] = bf16( bf16(bf16(allreduce(routed)) * scale) + bf16(allreduce(shared_partial[r][n])) )
// I % 64 == 0, H % 16 == 0, top_k <= MM_WARPS.
__global__ void __launch_bounds__(MM_THREADS)
moe_down_combine_kernel(const bf16* __restrict__ act, const float* __restrict__ route_weight, const int* __restrict__ topk_ids,
                        const uint8_t* __restrict__ wd, const float* __restrict__ sd, int experts, int I, int H, int rows_total, int top_k,
                        const float* __restrict__ shared_partial, float scale, bf16* __restrict__ out, PeerComm comm, int channel) {
    GLMB_PDL_PROLOGUE();
    __shared__ float red[GLMB_MAX_ROWS][MM_WARPS][MM_ROWS];
    __shared__ float sh[2 * GLMB_MAX_ROWS * MM_ROWS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * MM_ROWS;
    const int r0 = blockIdx.y * GLMB_MAX_ROWS;
    const int rows = min(GLMB_MAX_ROWS, rows_total - r0);
    const int kb = (I + 127) >> 7, chunks = I >> 6;
    const int64_t hi_off = (int64_t)8 * I;
    for (int r = 0; r < rows; ++r) {
        float lo_sum = 0.f, hi_sum = 0.f;
        if (warp < top_k) {
            const int p = (r0 + r) * top_k + warp;
            const int e = topk_ids[p];
            if (e >= 0 && e < experts) {
                const bf16* xr = act + (int64_t)p * I;
                const uint8_t* w_lo = wd + ((int64_t)e * H + n0 + g) * I;
                const int64_t sofs = ((int64_t)e * ((H + 127) >> 7) + (n0 >> 7)) * kb;
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
                for (int c = 0; c < chunks; ++c) {
                    const int k = (c << 6) + t * 16;
                    const uint4 lo = ld_stream16(w_lo + k), hi = ld_stream16(w_lo + hi_off + k);
                    uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0;
                    if (g == 0) { x0 = ld_hot16(xr + k); x1 = ld_hot16(xr + k + 8); }  // the route is column 0 of the B operand
                    chunk_mma(acc, lo, hi, sd[sofs + (c >> 1)], x0, x1);
                }
                // column 0 of the C fragment: lanes with t == 0 hold (row g) in acc[0] and (row g + 8) in acc[2]
                const float wgt = bf16_round(route_weight[p]);
                lo_sum = bf16_round(bf16_round(acc[0]) * wgt);
                hi_sum = bf16_round(bf16_round(acc[2]) * wgt);
            }
        }
        if (t == 0) { red[r][warp][g] = lo_sum; red[r][warp][g + 8] = hi_sum; }
    }
    __syncthreads();
    const int per = rows * MM_ROWS;
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
        const int r = i / MM_ROWS, c = i % MM_ROWS;
        float routed = 0.f;
#pragma unroll
        for (int w = 0; w < MM_WARPS; ++w) routed += red[r][w][c];
        sh[i] = shared_partial ? shared_partial[(int64_t)(r0 + r) * H + n0 + c] : 0.f;
        sh[per + i] = routed;
    }
    __syncthreads();
    cta_allreduce_f32(comm, channel, sh, 2 * per);
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
        const int r = i / MM_ROWS, c = i % MM_ROWS;
        out[(int64_t)(r0 + r) * H + n0 + c] = __float2bfloat16_rn(bf16_round(bf16_round(sh[per + i]) * scale) + bf16_round(sh[i]));
    }
}

GLMB_API int glmb_moe_down_combine(const void* act, const float* route_weight, const int* topk_ids, const void* wd, const float* sd,
                                   int experts, int I, int H, int rows, int top_k, const float* shared_partial, float scale, void* out,
                                   const PeerComm* comm, int channel, void* stream) {
    if (rows < 1 || top_k < 1 || top_k > MM_WARPS || (I & 63) || (H & 15)) return 1;
    PeerComm c;
    if (comm) c = *comm;
    else { memset(&c, 0, sizeof(c)); c.world = 1; }
    const dim3 grid(H / MM_ROWS, ceil_div(rows, GLMB_MAX_ROWS));
    if (c.world > 1 && (int)(grid.x * grid.y) > GLMB_AR_MAX_CTAS) return 2;
    GLMB_LAUNCH(moe_down_combine_kernel, grid, MM_THREADS, 0, (cudaStream_t)stream, (const bf16*)act, route_weight, topk_ids, (const uint8_t*)wd,
                sd, experts, I, H, rows, top_k, shared_partial, scale, (bf16*)out, c, channel);
    return (int)cudaGetLastError();
}

// How many CTAs of a (rows x tiles) grid are expected to do work: a tile whose expert lives on another GPU returns at once, and
// with E experts of which this GPU holds `experts_local` a route is local with probability experts_local / E.  The model tells the
// library E once (0: every tile is local); the estimate only selects the pipeline depth, never the result.
static int g_moe_experts_total = 0;
GLMB_API void glmb_set_moe_experts_total(int experts) { g_moe_experts_total = experts > 0 ? experts : 0; }
static long live_ctas(unsigned per_tile, int tiles, int experts_local) {
    long live_tiles = tiles;
    if (g_moe_experts_total > experts_local && experts_local > 0)
        live_tiles = max(1L, ((long)tiles * experts_local * 2 + g_moe_experts_total - 1) / g_moe_experts_total);  // twice the mean: the busy GPU
    return (long)per_tile * live_tiles;
}

// ===================================================================================================
// Launchers used by glmb_moe_gateup_fp8 / glmb_moe_down_fp8 (gemv.cu) when the shape fits.  rt in {1, 8}.
int glmb_launch_moe_gateup_mma(const void* x, int64_t xs, int top_k, const int* tile_expert, const int* tile_routes, const int* n_tiles,
                               int tiles, int rt, const void* wg, const void* wu, const float* sg, const float* su, int expert_base,
                               int experts_local, int I, int H, void* act, cudaStream_t stream) {
    dim3 grid(ceil_div(I, MM_ROWS), tiles);
    const long live = live_ctas(grid.x, tiles, experts_local);
#define CALL(RT_, D_)                                                                                                                      \
    GLMB_LAUNCH((moe_gateup_fp8_mma_kernel<RT_, D_>), grid, MM_THREADS, 0, stream, (const bf16*)x, xs, top_k, tile_expert, tile_routes, n_tiles, \
                (const uint8_t*)wg, (const uint8_t*)wu, sg, su, expert_base, experts_local, I, H, (bf16*)act)
    if (rt == 1) { if (live <= 2 * 148) CALL(1, 4); else if (live <= 4 * 148) CALL(1, 2); else CALL(1, 1); }
    else CALL(8, 1);
#undef CALL
    return (int)cudaGetLastError();
}

int glmb_launch_moe_down_mma(const void* act, const float* route_weight, const int* tile_expert, const int* tile_routes, const int* n_tiles,
                             int tiles, int rt, const void* wd, const float* sd, int expert_base, int experts_local, int I, int H, void* dw,
                             cudaStream_t stream) {
    dim3 grid(ceil_div(H, MM_ROWS), tiles);
    const long live = live_ctas(grid.x, tiles, experts_local);
#define CALL(RT_, D_)                                                                                                                        \
    GLMB_LAUNCH((moe_down_fp8_mma_kernel<RT_, D_>), grid, MM_THREADS, 0, stream, (const bf16*)act, route_weight, tile_expert, tile_routes, n_tiles, \
                (const uint8_t*)wd, sd, expert_base, experts_local, I, H, (bf16*)dw)
    if (rt == 1) { if (live <= 2 * 148) CALL(1, 4); else if (live <= 4 * 148) CALL(1, 2); else CALL(1, 1); }
    else if (tile_routes && I <= 512) {  // a short K: one warp per 16 output rows
        GLMB_LAUNCH(moe_down_fp8_mma_shortk_kernel<8>, dim3(ceil_div(H, MM_ROWS * MM_WARPS), tiles), MM_THREADS, 0, stream, (const bf16*)act,
                    route_weight, tile_expert, tile_routes, n_tiles, (const uint8_t*)wd, sd, expert_base, experts_local, I, H, (bf16*)dw);
    } else CALL(8, 1);
#undef CALL
    return (int)cudaGetLastError();
}
