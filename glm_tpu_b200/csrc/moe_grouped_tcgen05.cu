// Routed experts for many rows (prefill): grouped GEMM over expert-sorted routes with the FP8 weights decoded
// inside the kernel, on the 5th-generation tensor cores.
//
//   C[sorted route, n] = sum_k A[sorted route, k] * bf16(f32(e4m3 W[e][n][k]) * scale[e][n / 128][k / 128])
//
// One CTA computes a 128-route x 256-column tile of one expert.  Per 64-wide k step:
//
//   warp 0        TMA: the activation tile (bf16, 128-byte swizzle) and two 128-row FP8 weight tiles (raw bytes)
//   warps 2-9     decode: each thread reads 16 FP8 codes from shared memory, applies the block scale in fp32,
//                 rounds to bf16 (the weight-decode contract) and writes the result into a second shared-memory
//                 tile in the 128-byte-swizzled K-major layout the tensor core expects; a proxy fence publishes it
//   warp 1        one lane issues tcgen05.mma (bf16 x bf16 -> fp32, M 128, N 256) into 256 TMEM columns
//   warps 2-5     epilogue (after the k loop): tcgen05.ld, then
//                   gate/up mode  columns 0-127 are gate, 128-255 up of the same 128 outputs:
//                                 act = bf16( silu(bf16 gate) * bf16 up ), stored in sorted order
//                   down mode     dw[route] = bf16( bf16(acc) * bf16(route weight) ), scattered to the route's slot
//
// The FP8 bytes cross HBM once and are never materialised as bf16 in global memory.  Every mbarrier wait is
// bounded; on a timeout the kernel raises GLMB_STATUS_WAIT_TIMEOUT, skips its stores and still frees its TMEM.
//
// Replaces reference `glm_tpu/kernels/fp8_grouped_matmul/panel_kernel.py:31-153` + `layers/moe/routed_experts.py:27-127`
// (prefill: stable group-by-expert, M32 panels, three FP8 panel matmuls, bf16 SiLU, bf16 route weighting).
#include "common.cuh"
#include "tcgen05.cuh"

#define MG_BM 128
#define MG_BN 256
#define MG_BK 64
#define MG_STAGES 4
#define MG_BSTAGES 2
#define MG_CONV_WARPS 8
#define MG_THREADS (64 + 32 * MG_CONV_WARPS)
#define MG_A_BYTES (MG_BM * MG_BK * 2)
#define MG_W8_BYTES (MG_BN * MG_BK)
#define MG_STAGE_BYTES (MG_A_BYTES + MG_W8_BYTES)
#define MG_B_BYTES (MG_BN * MG_BK * 2)
#define MG_SMEM_BYTES (MG_STAGES * MG_STAGE_BYTES + MG_BSTAGES * MG_B_BYTES + 1024 + 256)
#define MG_TMEM_COLS 256

struct MoeGroupedArgs {
    const TcTile* tiles;      // [max_tiles] 128-route tiles of the expert-sorted route list (row0, row_end, local expert)
    const int* n_tiles;       // [1] on the device
    const float* scale0;      // block scales of the first weight [experts, ceil(N/128), ceil(K/128)]
    const float* scale1;      // ... of the second weight (gate/up mode: up; down mode: the same tensor as scale0)
    const int* perm;          // [sorted routes] -> route id (row * top_k + slot), -1 for none   (down mode)
    const float* route_weight;  // [routes] fp32                                                  (down mode)
    void* out;                // gate/up: act_sorted [sorted routes, N] bf16;  down: dw [routes, N] bf16
    int N, K, mode;           // mode 0: gate/up (N = expert FFN width), 1: down (N = hidden size)
    uint32_t* status;
};

__device__ __forceinline__ uint32_t decode_pair(uint32_t two_codes, float scale) {
    const float2 f = e4m3x2_to_float2(two_codes);
    return pack_bf16(f.x * scale, f.y * scale);
}

__global__ void __launch_bounds__(MG_THREADS, 1)
moe_grouped_fp8w_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w0,
                        const __grid_constant__ CUtensorMap map_w1, MoeGroupedArgs a) {
    GLMB_PDL_PROLOGUE();
    const int t = blockIdx.y;
    if (t >= *a.n_tiles) return;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* bring = ring + MG_STAGES * MG_STAGE_BYTES;  // decoded weight tiles (1024-byte aligned: 32 KB stages)
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(bring + MG_BSTAGES * MG_B_BYTES);
    uint64_t* empty_bar = full_bar + MG_STAGES;     // 8 decode warps + the MMA commit
    uint64_t* b_full = empty_bar + MG_STAGES;       // 8 decode warps
    uint64_t* b_empty = b_full + MG_BSTAGES;        // MMA commit
    uint64_t* acc_bar = b_empty + MG_BSTAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
    volatile uint32_t* fail_slot = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = a.tiles[t].row0, row_end = a.tiles[t].row_end, expert = a.tiles[t].expert;
    const int nb = blockIdx.x;
    const int kblocks = (a.K + MG_BK - 1) / MG_BK;
    const int n_scale_rows = (a.N + 127) >> 7, n_scale_cols = (a.K + 127) >> 7;
    // first output column of the tile, and the weight rows / scale rows its two 128-row halves come from
    const int n0 = a.mode == 0 ? nb * 128 : nb * MG_BN;
    const int w_row0 = expert * a.N + n0;
    const int w_row1 = a.mode == 0 ? w_row0 : w_row0 + 128;
    const int srow0 = n0 >> 7;
    const int srow1 = a.mode == 0 ? srow0 : min(srow0 + 1, n_scale_rows - 1);
    const float* sc0 = a.scale0 + ((int64_t)expert * n_scale_rows + srow0) * n_scale_cols;
    const float* sc1 = a.scale1 + ((int64_t)expert * n_scale_rows + srow1) * n_scale_cols;

    if (threadIdx.x == 0) {
        for (int s = 0; s < MG_STAGES; ++s) { mbar_init(full_bar + s, 1); mbar_init(empty_bar + s, MG_CONV_WARPS + 1); }
        for (int j = 0; j < MG_BSTAGES; ++j) { mbar_init(b_full + j, MG_CONV_WARPS); mbar_init(b_empty + j, 1); }
        mbar_init(acc_bar, 1);
        *fail_slot = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(MG_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < kblocks; ++kb) {
                const int s = kb % MG_STAGES, lap = kb / MG_STAGES;
                if (lap > 0 && !mbar_wait(empty_bar + s, (lap - 1) & 1)) { *fail_slot = 1; break; }
                unsigned char* a_dst = ring + s * MG_STAGE_BYTES;
                unsigned char* w_dst = a_dst + MG_A_BYTES;
                mbar_expect_tx(full_bar + s, MG_STAGE_BYTES);
                tma_load_2d(a_dst, &map_a, full_bar + s, kb * MG_BK, row0);
                tma_load_2d(w_dst, &map_w0, full_bar + s, kb * MG_BK, w_row0);
                tma_load_2d(w_dst + 128 * MG_BK, &map_w1, full_bar + s, kb * MG_BK, w_row1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(MG_BM, MG_BN);
            for (int kb = 0; kb < kblocks; ++kb) {
                const int s = kb % MG_STAGES, lap = kb / MG_STAGES;
                const int j = kb % MG_BSTAGES, blap = kb / MG_BSTAGES;
                if (!mbar_wait(full_bar + s, lap & 1) || !mbar_wait(b_full + j, blap & 1)) { *fail_slot = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_u32(ring + s * MG_STAGE_BYTES);
                const uint32_t b_addr = smem_u32(bring + j * MG_B_BYTES);
#pragma unroll
                for (int k = 0; k < MG_BK / 16; ++k)
                    umma_bf16(tmem_base, umma_desc_sw128(a_addr + k * 32), umma_desc_sw128(b_addr + k * 32), idesc,
                              (kb > 0 || k > 0) ? 1u : 0u);
                umma_commit(empty_bar + s);  // the activation tile of this stage has been read
                umma_commit(b_empty + j);    // and so has the decoded weight tile
            }
            umma_commit(acc_bar);
        }
    } else {
        // ---- decode: FP8 tile (row-major, 64 bytes per row) -> bf16 tile (K-major, 128-byte swizzle) ----------
        const int ct = threadIdx.x - 64;  // 0 .. 255
        bool ok = true;
        float next_lo = sc0[0], next_hi = sc1[0];
        for (int kb = 0; kb < kblocks && ok; ++kb) {
            const int s = kb % MG_STAGES, lap = kb / MG_STAGES;
            const int j = kb % MG_BSTAGES, blap = kb / MG_BSTAGES;
            // the block scales of the NEXT k step are requested now, a whole step before their first use: a load issued
            // after the waits below would add its L2 latency to every step of the warps that bound this kernel
            const float scale_lo = next_lo, scale_hi = next_hi;
            const int kblk = min(((kb + 1) * MG_BK) >> 7, n_scale_cols - 1);
            next_lo = sc0[kblk]; next_hi = sc1[kblk];
            if (!mbar_wait(full_bar + s, lap & 1) || (blap > 0 && !mbar_wait(b_empty + j, (blap - 1) & 1))) { *fail_slot = 1; ok = false; break; }
            const unsigned char* w8 = ring + s * MG_STAGE_BYTES + MG_A_BYTES;
            unsigned char* bt = bring + j * MG_B_BYTES;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int q = ct + 256 * i;            // 16-byte piece of the FP8 tile: eight lanes cover two whole rows
                const int row = q >> 2, c = q & 3;     // rows 0-127 (i < 2): first weight, 128-255: second weight
                const uint4 w = *reinterpret_cast<const uint4*>(w8 + row * MG_BK + c * 16);
                const float scale = i < 2 ? scale_lo : scale_hi;
                uint4 o0, o1;
                o0.x = decode_pair(w.x & 0xffffu, scale); o0.y = decode_pair(w.x >> 16, scale);
                o0.z = decode_pair(w.y & 0xffffu, scale); o0.w = decode_pair(w.y >> 16, scale);
                o1.x = decode_pair(w.z & 0xffffu, scale); o1.y = decode_pair(w.z >> 16, scale);
                o1.z = decode_pair(w.w & 0xffffu, scale); o1.w = decode_pair(w.w >> 16, scale);
                unsigned char* line = bt + (row >> 3) * 1024 + (row & 7) * 128;
                *reinterpret_cast<uint4*>(line + (((2 * c) ^ (row & 7)) << 4)) = o0;
                *reinterpret_cast<uint4*>(line + (((2 * c + 1) ^ (row & 7)) << 4)) = o1;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy stores -> visible to the tensor core
            __syncwarp();
            if (lane == 0) { mbar_arrive(b_full + j); mbar_arrive(empty_bar + s); }
        }
        // ---- epilogue (warps 2-5) ----------------------------------------------------------------------------
        if (warp < 6) {
            const int quarter = warp & 3;
            const bool done = mbar_wait(acc_bar, 0);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (!done || !ok || *fail_slot) {
                if (lane == 0) raise_status(a.status, GLMB_STATUS_WAIT_TIMEOUT);
            } else {
                const int row = row0 + quarter * 32 + lane;
                const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
                if (a.mode == 0) {
                    bf16* dst_row = reinterpret_cast<bf16*>(a.out) + (int64_t)row * a.N;
#pragma unroll 1
                    for (int cb = 0; cb < 4; ++cb) {
                        uint32_t g[32], u[32];
                        tmem_ld32(lane_addr + cb * 32, g);
                        tmem_ld32(lane_addr + 128 + cb * 32, u);
                        const int col = n0 + cb * 32;
                        if (row < row_end && col < a.N) {
#pragma unroll
                            for (int e = 0; e < 32; e += 8) {
                                if (col + e >= a.N) break;
                                uint32_t o[4];
#pragma unroll
                                for (int p = 0; p < 4; ++p) {
                                    const float g0 = bf16_round(__uint_as_float(g[e + 2 * p])), g1 = bf16_round(__uint_as_float(g[e + 2 * p + 1]));
                                    const float u0 = bf16_round(__uint_as_float(u[e + 2 * p])), u1 = bf16_round(__uint_as_float(u[e + 2 * p + 1]));
                                    o[p] = pack_bf16(g0 * sigmoidf_precise(g0) * u0, g1 * sigmoidf_precise(g1) * u1);
                                }
                                *reinterpret_cast<uint4*>(dst_row + col + e) = make_uint4(o[0], o[1], o[2], o[3]);
                            }
                        }
                    }
                } else {
                    const int route = row < row_end ? a.perm[row] : -1;
                    const float wgt = route >= 0 ? bf16_round(a.route_weight[route]) : 0.f;
                    bf16* dst_row = reinterpret_cast<bf16*>(a.out) + (int64_t)(route >= 0 ? route : 0) * a.N;
#pragma unroll 1
                    for (int cb = 0; cb < MG_BN / 32; ++cb) {
                        uint32_t v[32];
                        tmem_ld32(lane_addr + cb * 32, v);
                        const int col = n0 + cb * 32;
                        if (route >= 0 && col < a.N) {
#pragma unroll
                            for (int e = 0; e < 32; e += 8) {
                                if (col + e >= a.N) break;
                                uint32_t o[4];
#pragma unroll
                                for (int p = 0; p < 4; ++p)
                                    o[p] = pack_bf16(bf16_round(__uint_as_float(v[e + 2 * p])) * wgt, bf16_round(__uint_as_float(v[e + 2 * p + 1])) * wgt);
                                *reinterpret_cast<uint4*>(dst_row + col + e) = make_uint4(o[0], o[1], o[2], o[3]);
                            }
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(MG_TMEM_COLS) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------
// dst[i] = src[idx[i]] (rows of `width` bf16, width % 8 == 0); idx < 0 -> a row of zeros.  Expert-sorted copy of the
// activations, so that one TMA box covers 128 routes of one expert.
__global__ void __launch_bounds__(256)
gather_rows_kernel(const bf16* __restrict__ src, int64_t src_stride, const int* __restrict__ idx, int divisor, bf16* __restrict__ dst,
                   int width) {
    GLMB_PDL_PROLOGUE();
    const int i = blockIdx.x;
    const int from = idx[i];
    const uint4* s = reinterpret_cast<const uint4*>(src + (int64_t)(from >= 0 ? from / divisor : 0) * src_stride);
    uint4* d = reinterpret_cast<uint4*>(dst + (int64_t)i * width);
    for (int v = threadIdx.x; v < width / 8; v += blockDim.x) d[v] = from >= 0 ? s[v] : make_uint4(0, 0, 0, 0);
}

// ===================================================================================================
// a_sorted [sorted_rows, K] bf16 (expert-sorted routes), w0/w1 [experts, N, K] FP8 bytes with block scales s0/s1,
// tiles/n_tiles on the device (max_tiles entries).  mode 0: out = act_sorted [sorted_rows, N] (w0 gate, w1 up);
// mode 1: out = dw [routes, N] scattered through perm, scaled by route_weight (w1/s1 ignored, the kernel uses w0/s0).
GLMB_API int glmb_moe_grouped_fp8w(const void* a_sorted, int sorted_rows, const void* w0, const void* w1, const float* s0,
                                   const float* s1, int experts, int N, int K, const void* tiles, const int* n_tiles, int max_tiles,
                                   int mode, const int* perm, const float* route_weight, void* out, uint32_t* status, void* stream) {
    if (sorted_rows < 1 || experts < 1 || max_tiles < 1 || N < 8 || (N & 7) || K < 16 || (K & 15) || mode < 0 || mode > 1) return 1;
    if (mode == 1 && (!perm || !route_weight)) return 1;
    if ((reinterpret_cast<uintptr_t>(a_sorted) & 15) || (reinterpret_cast<uintptr_t>(w0) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return 1;
    if (mode == 0 && (!w1 || !s1 || (reinterpret_cast<uintptr_t>(w1) & 15))) return 1;
    CUtensorMap map_a, map_w0, map_w1;
    if (make_map(&map_a, a_sorted, (uint64_t)sorted_rows, (uint64_t)K, (uint64_t)K, MG_BM)) return 3;
    if (make_map_u8(&map_w0, w0, (uint64_t)experts * N, (uint64_t)K, (uint64_t)K, 128)) return 3;
    if (make_map_u8(&map_w1, mode == 0 ? w1 : w0, (uint64_t)experts * N, (uint64_t)K, (uint64_t)K, 128)) return 3;
    static DeviceOnce attr_set;
    const int attr_set_dev = attr_set.pending();
    if (attr_set_dev != DeviceOnce::SET) {
        cudaError_t e = cudaFuncSetAttribute(moe_grouped_fp8w_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MG_SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        attr_set.mark(attr_set_dev);
    }
    MoeGroupedArgs args;
    args.tiles = (const TcTile*)tiles;
    args.n_tiles = n_tiles;
    args.scale0 = s0;
    args.scale1 = mode == 0 ? s1 : s0;
    args.perm = perm;
    args.route_weight = route_weight;
    args.out = out;
    args.N = N; args.K = K; args.mode = mode;
    args.status = status;
    dim3 grid(mode == 0 ? ceil_div(N, 128) : ceil_div(N, MG_BN), max_tiles);
    GLMB_LAUNCH(moe_grouped_fp8w_kernel, grid, MG_THREADS, MG_SMEM_BYTES, (cudaStream_t)stream, map_a, map_w0, map_w1, args);
    return (int)cudaGetLastError();
}

// dst [n, width] = src[idx[i] / divisor] (idx < 0: zeros).  width % 8 == 0, rows 16-byte aligned.
GLMB_API int glmb_gather_rows(const void* src, int64_t src_stride, const int* idx, int divisor, void* dst, int n, int width,
                              void* stream) {
    if (n < 1 || (width & 7) || divisor < 1 || (src_stride & 7)) return 1;
    GLMB_LAUNCH(gather_rows_kernel, n, 256, 0, (cudaStream_t)stream, (const bf16*)src, src_stride, idx, divisor, (bf16*)dst, width);
    return (int)cudaGetLastError();
}
