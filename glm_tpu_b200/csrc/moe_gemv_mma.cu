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

#define MM_WARPS 8
#define MM_THREADS (32 * MM_WARPS)
#define MM_ROWS 16  // output rows per CTA

// act[p][n] = bf16( silu(bf16(x_p . wg[e][n])) * bf16(x_p . wu[e][n]) ) for the routes p of tile t.  H % 64 == 0, I % 16 == 0.
template <int RT>
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
    for (int c = warp; c < chunks; c += MM_WARPS) {
        const int k = (c << 6) + t * 16;
        const uint4 g_lo = ld_stream16(wg_lo + k), g_hi = ld_stream16(wg_lo + hi_off + k);
        const uint4 u_lo = ld_stream16(wu_lo + k), u_hi = ld_stream16(wu_lo + hi_off + k);
        uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0;
        if (route >= 0) { x0 = ld_hot16(xr + k); x1 = ld_hot16(xr + k + 8); }
        const float s_g = sg[sofs + (c >> 1)], s_u = su[sofs + (c >> 1)];
        chunk_mma(acc_g, g_lo, g_hi, s_g, x0, x1);
        chunk_mma(acc_u, u_lo, u_hi, s_u, x0, x1);
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
template <int RT>
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
    for (int c = warp; c < chunks; c += MM_WARPS) {
        const int k = (c << 6) + t * 16;
        const uint4 lo = ld_stream16(w_lo + k), hi = ld_stream16(w_lo + hi_off + k);
        uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0;
        if (route >= 0) { x0 = ld_hot16(xr + k); x1 = ld_hot16(xr + k + 8); }
        chunk_mma(acc, lo, hi, sd[sofs + (c >> 1)], x0, x1);
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

// ===================================================================================================
// Launchers used by glmb_moe_gateup_fp8 / glmb_moe_down_fp8 (gemv.cu) when the shape fits.  rt in {1, 8}.
int glmb_launch_moe_gateup_mma(const void* x, int64_t xs, int top_k, const int* tile_expert, const int* tile_routes, const int* n_tiles,
                               int tiles, int rt, const void* wg, const void* wu, const float* sg, const float* su, int expert_base,
                               int experts_local, int I, int H, void* act, cudaStream_t stream) {
    dim3 grid(ceil_div(I, MM_ROWS), tiles);
    if (rt == 1)
        GLMB_LAUNCH(moe_gateup_fp8_mma_kernel<1>, grid, MM_THREADS, 0, stream, (const bf16*)x, xs, top_k, tile_expert, tile_routes, n_tiles,
                    (const uint8_t*)wg, (const uint8_t*)wu, sg, su, expert_base, experts_local, I, H, (bf16*)act);
    else
        GLMB_LAUNCH(moe_gateup_fp8_mma_kernel<8>, grid, MM_THREADS, 0, stream, (const bf16*)x, xs, top_k, tile_expert, tile_routes, n_tiles,
                    (const uint8_t*)wg, (const uint8_t*)wu, sg, su, expert_base, experts_local, I, H, (bf16*)act);
    return (int)cudaGetLastError();
}

int glmb_launch_moe_down_mma(const void* act, const float* route_weight, const int* tile_expert, const int* tile_routes, const int* n_tiles,
                             int tiles, int rt, const void* wd, const float* sd, int expert_base, int experts_local, int I, int H, void* dw,
                             cudaStream_t stream) {
    dim3 grid(ceil_div(H, MM_ROWS), tiles);
    if (rt == 1)
        GLMB_LAUNCH(moe_down_fp8_mma_kernel<1>, grid, MM_THREADS, 0, stream, (const bf16*)act, route_weight, tile_expert, tile_routes, n_tiles,
                    (const uint8_t*)wd, sd, expert_base, experts_local, I, H, (bf16*)dw);
    else
        GLMB_LAUNCH(moe_down_fp8_mma_kernel<8>, grid, MM_THREADS, 0, stream, (const bf16*)act, route_weight, tile_expert, tile_routes, n_tiles,
                    (const uint8_t*)wd, sd, expert_base, experts_local, I, H, (bf16*)dw);
    return (int)cudaGetLastError();
}
