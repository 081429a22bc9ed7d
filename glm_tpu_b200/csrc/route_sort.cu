// Expert sort of a prefill chunk's routes in ONE launch: stable counting sort of the routes whose expert lives on this GPU,
// cut into tiles of 128 routes for the grouped expert GEMM, or into tiles of 8 routes for the tensor-core GEMV kernels that serve
// chunks with only a few routes per expert (moe_gemv_mma.cu).
//
//   perm[sorted position]  = route id (row * top_k + slot), -1 past this GPU's routes
//   n_tiles[0]             = number of tiles
//   tiles of 128:  tiles[t] = (first sorted row, end row of the expert, local expert, 0), zeros past the last tile
//   tiles of 8:    tiles[t] = GLOBAL expert id of tile t (-1 past the last tile); tile_routes[8 t + c] = route id of slot c, or -1
//
// One CTA of 1,024 threads: a shared-memory histogram, a scan over <= 256 experts, then the routes in rounds of 1,024 in
// route order: the rank of a route among the routes of its expert = routes of earlier rounds (running count) + routes of
// earlier warps in this round (per-warp counts) + earlier lanes of its warp (__match_any_sync), so the order inside an expert
// is the route order (stable, the same permutation as a stable argsort).  Replaces ~40 library launches (argsort, bincount,
// cumsum, searchsorted, gathers) per MoE layer and chunk, which cost more host time than the expert GEMMs cost GPU time once
// the experts are spread over 8 GPUs.
//
// Reference counterpart: the stable group-by-expert of `glm_tpu/layers/moe/routed_experts.py:27-127`.
#include "common.cuh"

#define RS_THREADS 1024
#define RS_WARPS (RS_THREADS / 32)
#define RS_MAX_EXPERTS 256

template <int TILE>
__global__ void __launch_bounds__(RS_THREADS)
route_sort_kernel(const int* __restrict__ topk_ids, int P, int ebase, int el, int max_tiles, int* __restrict__ tiles, int* __restrict__ n_tiles,
                  int* __restrict__ perm, int* __restrict__ tile_routes) {
    GLMB_PDL_PROLOGUE();
    __shared__ int count[RS_MAX_EXPERTS + 1], start[RS_MAX_EXPERTS + 1], running[RS_MAX_EXPERTS], tile_start[RS_MAX_EXPERTS + 1];
    __shared__ unsigned char warp_count[RS_WARPS][RS_MAX_EXPERTS];  // routes of one expert in one warp of one round: <= 32
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    for (int k = threadIdx.x; k <= el; k += RS_THREADS) count[k] = 0;
    for (int k = threadIdx.x; k < el; k += RS_THREADS) running[k] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < P; i += RS_THREADS) {
        const int e = topk_ids[i] - ebase;
        if (e >= 0 && e < el) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {  // <= 256 experts: a serial scan costs less than a microsecond
        int rows = 0, t = 0;
        for (int e = 0; e < el; ++e) {
            start[e] = rows; tile_start[e] = t;
            rows += count[e]; t += (count[e] + TILE - 1) / TILE;
        }
        start[el] = rows; tile_start[el] = t;
        n_tiles[0] = t;
    }
    __syncthreads();
    const int n_local = start[el], total_tiles = tile_start[el];

    for (int base = 0; base < P; base += RS_THREADS) {
        for (int j = threadIdx.x; j < RS_WARPS * RS_MAX_EXPERTS; j += RS_THREADS) (&warp_count[0][0])[j] = 0;
        __syncthreads();
        const int i = base + threadIdx.x;
        int e = -1;
        if (i < P) { e = topk_ids[i] - ebase; if (e < 0 || e >= el) e = -1; }
        const unsigned active = __ballot_sync(0xffffffffu, e >= 0);
        int rank = 0;
        if (e >= 0) {
            const unsigned same = __match_any_sync(active, e);
            rank = __popc(same & ((1u << lane) - 1u));
            if (rank == 0) warp_count[warp][e] = (unsigned char)__popc(same);
        }
        __syncthreads();
        if (e >= 0) {
            int before = running[e];
            for (int w = 0; w < warp; ++w) before += warp_count[w][e];
            perm[start[e] + before + rank] = i;
        }
        __syncthreads();
        for (int k = threadIdx.x; k < el; k += RS_THREADS) {
            int add = 0;
            for (int w = 0; w < RS_WARPS; ++w) add += warp_count[w][k];
            running[k] += add;
        }
        __syncthreads();
    }
    for (int i = n_local + threadIdx.x; i < P; i += RS_THREADS) perm[i] = -1;
    if (TILE == 128) {
        for (int e = threadIdx.x; e < el; e += RS_THREADS) {
            const int c = count[e], first = start[e];
            for (int j = 0, t = tile_start[e]; j * 128 < c; ++j, ++t)
                if (t < max_tiles) reinterpret_cast<int4*>(tiles)[t] = make_int4(first + j * 128, first + c, e, 0);
        }
        for (int t = total_tiles + threadIdx.x; t < max_tiles; t += RS_THREADS) reinterpret_cast<int4*>(tiles)[t] = make_int4(0, 0, 0, 0);
    } else {
        // perm was written by this CTA and every round ended with a barrier: its entries are visible here
        for (int e = threadIdx.x; e < el; e += RS_THREADS) {
            const int c = count[e], first = start[e];
            for (int j = 0, t = tile_start[e]; j * TILE < c; ++j, ++t) {
                if (t >= max_tiles) break;
                tiles[t] = e + ebase;
                for (int k = 0; k < TILE; ++k) tile_routes[t * TILE + k] = j * TILE + k < c ? perm[first + j * TILE + k] : -1;
            }
        }
        for (int t = total_tiles + threadIdx.x; t < max_tiles; t += RS_THREADS) tiles[t] = -1;
    }
}

// topk_ids: [P] global expert ids of the routes (row-major [rows, top_k]); this GPU holds experts [ebase, ebase + el).
// tiles: [max_tiles, 4] int32 with max_tiles >= P / 128 + el; n_tiles: [1]; perm: [P].  All 16-byte aligned device buffers.
GLMB_API int glmb_route_sort128(const int* topk_ids, int P, int ebase, int el, int max_tiles, int* tiles, int* n_tiles, int* perm, void* stream) {
    if (P < 1 || el < 1 || el > RS_MAX_EXPERTS || max_tiles < P / 128 + el || (reinterpret_cast<uintptr_t>(tiles) & 15)) return 1;
    GLMB_LAUNCH(route_sort_kernel<128>, 1, RS_THREADS, 0, (cudaStream_t)stream, topk_ids, P, ebase, el, max_tiles, tiles, n_tiles, perm,
                (int*)nullptr);
    return (int)cudaGetLastError();
}

// The same sort cut into tiles of 8 routes.  tile_expert: [max_tiles] with max_tiles >= P / 8 + el (global expert ids);
// tile_routes: [max_tiles, 8]; n_tiles: [1]; perm: [P] (scratch: the sorted order).
GLMB_API int glmb_route_sort8(const int* topk_ids, int P, int ebase, int el, int max_tiles, int* tile_expert, int* tile_routes, int* n_tiles,
                              int* perm, void* stream) {
    if (P < 1 || el < 1 || el > RS_MAX_EXPERTS || max_tiles < P / 8 + el) return 1;
    GLMB_LAUNCH(route_sort_kernel<8>, 1, RS_THREADS, 0, (cudaStream_t)stream, topk_ids, P, ebase, el, max_tiles, tile_expert, n_tiles, perm,
                tile_routes);
    return (int)cudaGetLastError();
}
