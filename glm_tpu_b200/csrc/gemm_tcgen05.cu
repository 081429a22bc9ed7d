// Dense and grouped bf16 GEMM on the 5th-generation tensor cores:  C[rows, N] = A[rows, K] . B[N, K]^T.
//
// One CTA computes a 128 x 128 output tile.  Operands are staged by TMA (cp.async.bulk.tensor, 128-byte swizzle,
// no multicast) through a 4-stage ring of shared-memory buffers guarded by full/empty mbarriers; one elected
// thread issues tcgen05.mma (kind::f16, bf16 inputs, fp32 accumulate) into a 128-lane x 128-column TMEM
// accumulator; four epilogue warps read it back with tcgen05.ld, round to bf16 (or keep fp32) and store.
//
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocation, MMA issue (one elected lane), TMEM release
//   warps 2-5   epilogue: warp w owns TMEM lanes 32*(w%4) .. +31
//
// Grouped mode (routed experts in prefill): `tiles` lists (first row, end row, expert) per 128-row tile of the
// expert-sorted activation buffer; the weight tile of expert e starts at row e*N of B viewed as [E*N, K]; rows
// past `end row` are computed but not stored.
//
// Every mbarrier wait is bounded: when the limit runs out the kernel raises GLMB_STATUS_WAIT_TIMEOUT, stops
// issuing work, and still releases its TMEM before it returns.
//
// Replaces reference `glm_tpu/kernels/fp8_grouped_matmul/panel_kernel.py:31-153` (prefill expert panels, after the
// load-time style decode of the FP8 tables to bf16) and the prefill projections of `layers/linear.py:89-128`.
#include "common.cuh"
#include "peer.cuh"
#include "tcgen05.cuh"

#define TC_BM 128
#define TC_BN 128
#define TC_BK 64
#define TC_STAGES 4
#define TC_UMMA_K 16
#define TC_THREADS 192
#define TC_TMEM_COLS 128
#define TC_STAGE_BYTES ((TC_BM + TC_BN) * TC_BK * 2)
#define TC_SMEM_BYTES (TC_STAGES * TC_STAGE_BYTES + 1024 + 256)



// tiles == nullptr: dense GEMM, tile t covers rows 128 t .. of `rows` rows.  out_f32: store fp32 instead of bf16.
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, void* __restrict__ c,
                         int64_t ldc, int rows, int N, int K, const TcTile* __restrict__ tiles, const int* __restrict__ n_tiles,
                         int out_f32, uint32_t* status) {
    GLMB_PDL_PROLOGUE();
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte alignment of the operand ring is required by the 128-byte swizzle
    unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(ring + TC_STAGES * TC_STAGE_BYTES);
    uint64_t* empty_bar = full_bar + TC_STAGES;
    uint64_t* acc_bar = empty_bar + TC_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
    uint32_t* fail_slot = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.y;
    if (n_tiles && t >= *n_tiles) return;
    int row0, row_end, expert;
    if (tiles) { row0 = tiles[t].row0; row_end = tiles[t].row_end; expert = tiles[t].expert; }
    else { row0 = t * TC_BM; row_end = rows; expert = 0; }
    const int n0 = blockIdx.x * TC_BN;
    const int kblocks = (K + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) { mbar_init(full_bar + s, 1); mbar_init(empty_bar + s, 1); }
        mbar_init(acc_bar, 1);
        *fail_slot = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < kblocks; ++kb) {
                const int s = kb % TC_STAGES;
                if (kb >= TC_STAGES && !mbar_wait(empty_bar + s, ((kb / TC_STAGES) - 1) & 1)) { *fail_slot = 1; break; }
                unsigned char* a_dst = ring + s * TC_STAGE_BYTES;
                unsigned char* b_dst = a_dst + TC_BM * TC_BK * 2;
                mbar_expect_tx(full_bar + s, TC_STAGE_BYTES);
                tma_load_2d(a_dst, &map_a, full_bar + s, kb * TC_BK, row0);
                tma_load_2d(b_dst, &map_b, full_bar + s, kb * TC_BK, expert * N + n0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(TC_BM, TC_BN);
            bool ok = true;
            for (int kb = 0; kb < kblocks && ok; ++kb) {
                const int s = kb % TC_STAGES;
                if (!mbar_wait(full_bar + s, (kb / TC_STAGES) & 1)) { *fail_slot = 1; ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_u32(ring + s * TC_STAGE_BYTES);
                const uint32_t b_addr = a_addr + TC_BM * TC_BK * 2;
#pragma unroll
                for (int k = 0; k < TC_BK / TC_UMMA_K; ++k) {
                    const uint64_t da = umma_desc_sw128(a_addr + k * TC_UMMA_K * 2);
                    const uint64_t db = umma_desc_sw128(b_addr + k * TC_UMMA_K * 2);
                    umma_bf16(tmem_base, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(empty_bar + s);  // the stage may be refilled once these MMAs have read it
            }
            umma_commit(acc_bar);            // accumulator complete (or abandoned): release the epilogue
        }
    } else {
        // epilogue
        const int quarter = warp & 3;
        const bool ok = mbar_wait(acc_bar, 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (!ok || *reinterpret_cast<volatile uint32_t*>(fail_slot)) {
            if (lane == 0) raise_status(status, GLMB_STATUS_WAIT_TIMEOUT);
        } else {
            const int row = row0 + quarter * 32 + lane;
#pragma unroll
            for (int cb = 0; cb < TC_BN / 32; ++cb) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + cb * 32, v);
                const int col = n0 + cb * 32;
                if (row < row_end && col < N) {
                    if (out_f32) {
                        float* dst = reinterpret_cast<float*>(c) + (int64_t)row * ldc + col;
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            if (col + i < N)
                                *reinterpret_cast<float4*>(dst + i) = make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]),
                                                                                  __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
                    } else {
                        bf16* dst = reinterpret_cast<bf16*>(c) + (int64_t)row * ldc + col;
#pragma unroll
                        for (int i = 0; i < 32; i += 8)
                            if (col + i < N) {
                                uint4 o;
                                o.x = pack_bf16(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                                o.y = pack_bf16(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
                                o.z = pack_bf16(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
                                o.w = pack_bf16(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
                                *reinterpret_cast<uint4*>(dst + i) = o;
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TC_TMEM_COLS) : "memory");
    }
}

// ===================================================================================================
// Persistent variant for large problems: one CTA per SM walks 128 x 256 output tiles.  The TMEM holds two
// 256-column accumulators, so the epilogue warps drain tile i while the MMA warp already fills tile i + 1; the
// operand ring (4 stages of 48 KB) keeps running across tile boundaries.  Tiles are visited in groups of eight
// row-tiles by all column-tiles so that CTAs running at the same time share operand tiles in L2.
#define T2_BN 256
#define T2_STAGES 4
#define T2_STAGE_BYTES ((TC_BM + T2_BN) * TC_BK * 2)
#define T2_EPI_STRIDE 36   // floats per row of a 32 x 32 fp32 epilogue staging tile (16-byte aligned rows)
#define T2_EPI_HSTRIDE 40  // bf16 per row of the 32 x 32 bf16 result tile behind it
#define T2_EPI_WARP_BYTES (32 * T2_EPI_STRIDE * 4 + 32 * T2_EPI_HSTRIDE * 2)
#define T2_SMEM_BYTES (T2_STAGES * T2_STAGE_BYTES + 1024 + 256 + 4 * T2_EPI_WARP_BYTES)
#define T2_TMEM_COLS 512
#define T2_GROUP_M 8

// Fused all-reduce of K-split partial products over NVLink peer memory (enabled != 0; dense mode, bf16 output).
// Every rank runs the same GEMM on its K-slice.  The 32-column block cb of tile t belongs to rank (t + cb) % world: the
// other ranks store their fp32 partial block into the owner's staging (slot (owned-block index, source rank)) and raise
// a flag per block; the owner waits for the world - 1 flags, adds the partials to its own accumulator in rank order,
// rounds to bf16 and stores the block into every rank's output buffer (the same offset in every staging buffer).  So
// every CTA of every rank pushes, reduces and broadcasts the same amount.  The last CTA to finish signals `sig` to all
// ranks; the consumer waits for that signal from every rank before it reads.  world must divide 8.
struct GemmAllReduce {
    int enabled;
    int sig;
    int64_t part_offset;  // byte offset of the partial-tile slots inside every staging buffer
    int64_t out_offset;   // byte offset of the bf16 output [rows, N] inside every staging buffer
    PeerComm comm;
};
#define T2_TILE_FLOATS (TC_BM * T2_BN)
#define T2_BLOCK_FLOATS (TC_BM * 32)  // one 32-column block of a tile

__device__ __forceinline__ void t2_tile(int t, int m_tiles, int n_blocks, int& m, int& n) {
    const int group = T2_GROUP_M * n_blocks;
    const int first_m = (t / group) * T2_GROUP_M;
    const int gm = min(m_tiles - first_m, T2_GROUP_M);
    m = first_m + (t % group) % gm;
    n = (t % group) / gm;
}

__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_bf16_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                    void* __restrict__ c, int64_t ldc, int rows, int N, int K, const TcTile* __restrict__ tiles,
                                    const int* __restrict__ n_tiles, int max_tiles, int out_f32, uint32_t* status, GemmAllReduce ar) {
    GLMB_PDL_PROLOGUE();
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(ring + T2_STAGES * T2_STAGE_BYTES);
    uint64_t* empty_bar = full_bar + T2_STAGES;
    uint64_t* acc_full = empty_bar + T2_STAGES;   // [2] MMA -> epilogue
    uint64_t* acc_empty = acc_full + 2;           // [2] epilogue (4 warps) -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile uint32_t* fail_slot = tmem_slot + 1;
    unsigned char* epi_stage = ring + T2_STAGES * T2_STAGE_BYTES + 256;  // per epilogue warp: fp32 tile, then bf16 tile

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // every CTA reads the round number before any CTA can finish, and the last CTA to finish advances it
    const uint32_t ar_epoch = ar.enabled ? ar.comm.seq[GLMB_SEQ_GEMM] + 1 : 0;
    const int m_tiles = tiles ? min(max(*n_tiles, 0), max_tiles) : (rows + TC_BM - 1) / TC_BM;
    const int n_blocks = (N + T2_BN - 1) / T2_BN;
    const int total = m_tiles * n_blocks;
    const int kblocks = (K + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < T2_STAGES; ++s) { mbar_init(full_bar + s, 1); mbar_init(empty_bar + s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(acc_full + a, 1); mbar_init(acc_empty + a, 4); }
        *fail_slot = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(T2_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t g = 0;  // k-blocks issued so far, across tiles
            for (int t = blockIdx.x; t < total && !*fail_slot; t += gridDim.x) {
                int m, n;
                t2_tile(t, m_tiles, n_blocks, m, n);
                const int row0 = tiles ? tiles[m].row0 : m * TC_BM;
                const int b_row = (tiles ? tiles[m].expert : 0) * N + n * T2_BN;
                for (int kb = 0; kb < kblocks; ++kb, ++g) {
                    const uint32_t s = g % T2_STAGES, lap = g / T2_STAGES;
                    if (lap > 0 && !mbar_wait(empty_bar + s, (lap - 1) & 1)) { *fail_slot = 1; break; }
                    unsigned char* a_dst = ring + s * T2_STAGE_BYTES;
                    unsigned char* b_dst = a_dst + TC_BM * TC_BK * 2;
                    mbar_expect_tx(full_bar + s, T2_STAGE_BYTES);
                    tma_load_2d(a_dst, &map_a, full_bar + s, kb * TC_BK, row0);
                    tma_load_2d(b_dst, &map_b, full_bar + s, kb * TC_BK, b_row);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(TC_BM, T2_BN);
            uint32_t g = 0, i = 0;
            for (int t = blockIdx.x; t < total && !*fail_slot; t += gridDim.x, ++i) {
                const uint32_t acc = i & 1, use = i >> 1;
                if (use > 0 && !mbar_wait(acc_empty + acc, (use - 1) & 1)) { *fail_slot = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + acc * T2_BN;
                bool ok = true;
                for (int kb = 0; kb < kblocks; ++kb, ++g) {
                    const uint32_t s = g % T2_STAGES, lap = g / T2_STAGES;
                    if (!mbar_wait(full_bar + s, lap & 1)) { *fail_slot = 1; ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_addr = smem_u32(ring + s * T2_STAGE_BYTES);
                    const uint32_t b_addr = a_addr + TC_BM * TC_BK * 2;
#pragma unroll
                    for (int k = 0; k < TC_BK / TC_UMMA_K; ++k)
                        umma_bf16(tmem_d, umma_desc_sw128(a_addr + k * TC_UMMA_K * 2), umma_desc_sw128(b_addr + k * TC_UMMA_K * 2), idesc,
                                  (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(empty_bar + s);
                }
                umma_commit(acc_full + acc);  // complete, or abandoned after a timeout: either way release the epilogue
                if (!ok) break;
            }
        }
    } else {
        const int quarter = warp & 3;
        uint32_t i = 0;
        for (int t = blockIdx.x; t < total; t += gridDim.x, ++i) {
            const uint32_t acc = i & 1, use = i >> 1;
            const bool ok = mbar_wait(acc_full + acc, use & 1);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (!ok || *fail_slot) {
                if (lane == 0) { *fail_slot = 1; raise_status(status, GLMB_STATUS_WAIT_TIMEOUT); }
                break;
            }
            int m, n;
            t2_tile(t, m_tiles, n_blocks, m, n);
            const int row0 = tiles ? tiles[m].row0 : m * TC_BM;
            const int row_end = tiles ? tiles[m].row_end : rows;
            const int row = row0 + quarter * 32 + lane;
            const int n0 = n * T2_BN;
            if (ar.enabled) {
                // Ownership is per 32-column block of a tile: block cb of tile t belongs to rank (t + cb) % world, so every CTA
                // of every rank pushes 7/8 of its tile, reduces 1/8 of it and broadcasts that eighth: the reduce work is spread
                // over all SMs of all GPUs instead of sitting on the one CTA that owned a whole tile.
                const PeerComm& pc = ar.comm;
                const int per_tile = (T2_BN / 32) / pc.world;  // owned blocks per tile (world divides 8)
                const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * T2_BN;
                // Row-per-thread accumulator fragments go through a per-warp shared-memory tile so that every store
                // instruction writes whole 128-byte lines (8 lanes x 16 bytes per row, 4 rows): NVLink and HBM both
                // want full lines, and a 16-byte store per lane at a 1 KB stride wastes most of each packet.
                float* stage = reinterpret_cast<float*>(epi_stage + (warp - 2) * T2_EPI_WARP_BYTES);
                bf16* tile_h = reinterpret_cast<bf16*>(stage) + 32 * T2_EPI_STRIDE * 2;
                const int sub_row = lane >> 3, sub_col = (lane & 7) * 4;
                const int out_col = (lane & 3) * 8;
                // ---- push the blocks other ranks own: slot (owned-block index, source rank), 128 rows x 32 fp32 each
#pragma unroll 1
                for (int cb = 0; cb < T2_BN / 32; ++cb) {
                    const int owner = (t + cb) % pc.world;
                    if (owner == pc.rank) continue;
                    uint32_t v[32];
                    tmem_ld32(lane_addr + cb * 32, v);
                    __syncwarp();
#pragma unroll
                    for (int e = 0; e < 32; e += 4)
                        *reinterpret_cast<uint4*>(stage + lane * T2_EPI_STRIDE + e) = make_uint4(v[e], v[e + 1], v[e + 2], v[e + 3]);
                    __syncwarp();
                    const int64_t idx = (int64_t)t * per_tile + cb / pc.world;
                    float* dst = reinterpret_cast<float*>(pc.data[owner] + ar.part_offset) + (idx * pc.world + pc.rank) * T2_BLOCK_FLOATS +
                                 (quarter * 32) * 32;
#pragma unroll
                    for (int r4 = 0; r4 < 32; r4 += 4) {
                        const int r = r4 + sub_row;
                        *reinterpret_cast<uint4*>(dst + r * 32 + sub_col) = *reinterpret_cast<const uint4*>(stage + r * T2_EPI_STRIDE + sub_col);
                    }
                }
                __threadfence_system();
                asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps: the whole tile's pushes are out
                if (warp == 2 && lane < T2_BN / 32) {
                    const int cb = lane, owner = (t + cb) % pc.world;
                    if (owner != pc.rank)
                        st_release_sys(pc.flags[owner] + GLMB_FLAG_GEMM_BASE + ((size_t)t * (T2_BN / 32) + cb) * GLMB_MAX_WORLD + pc.rank, ar_epoch);
                }
                // ---- reduce and broadcast the blocks this rank owns
#pragma unroll 1
                for (int cb = 0; cb < T2_BN / 32; ++cb) {
                    if ((t + cb) % pc.world != pc.rank) continue;
                    if (warp == 2 && lane < pc.world && lane != pc.rank) {
                        if (!wait_flag_reached(pc.flags[pc.rank] + GLMB_FLAG_GEMM_BASE + ((size_t)t * (T2_BN / 32) + cb) * GLMB_MAX_WORLD + lane,
                                               ar_epoch, pc.wait_limit))
                            raise_status(status, GLMB_STATUS_WAIT_TIMEOUT);
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    uint32_t v[32];
                    tmem_ld32(lane_addr + cb * 32, v);
                    __syncwarp();
#pragma unroll
                    for (int e = 0; e < 32; e += 4)
                        *reinterpret_cast<uint4*>(stage + lane * T2_EPI_STRIDE + e) = make_uint4(v[e], v[e + 1], v[e + 2], v[e + 3]);
                    __syncwarp();
                    const int64_t idx = (int64_t)t * per_tile + cb / pc.world;
                    const float* inbox = reinterpret_cast<const float*>(pc.data[pc.rank] + ar.part_offset) + idx * pc.world * T2_BLOCK_FLOATS +
                                         (quarter * 32) * 32;
                    float4 sum[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) sum[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int p = 0; p < pc.world; ++p) {  // rank order: the same sum on every run
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int r = i * 4 + sub_row;
                            float4 x;
                            if (p == pc.rank) {
                                x = *reinterpret_cast<const float4*>(stage + r * T2_EPI_STRIDE + sub_col);
                            } else {
                                const uint4 u = ld_sys_u4(inbox + (int64_t)p * T2_BLOCK_FLOATS + r * 32 + sub_col);
                                x = make_float4(__uint_as_float(u.x), __uint_as_float(u.y), __uint_as_float(u.z), __uint_as_float(u.w));
                            }
                            sum[i].x += x.x; sum[i].y += x.y; sum[i].z += x.z; sum[i].w += x.w;
                        }
                    }
                    __syncwarp();
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int r = i * 4 + sub_row;
                        *reinterpret_cast<uint2*>(tile_h + r * T2_EPI_HSTRIDE + sub_col) =
                            make_uint2(pack_bf16(sum[i].x, sum[i].y), pack_bf16(sum[i].z, sum[i].w));
                    }
                    __syncwarp();
                    const int col = n0 + cb * 32 + out_col;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int r = i * 8 + (lane >> 2);
                        const int grow = row0 + quarter * 32 + r;
                        if (grow < rows && col < N) {
                            const uint4 o = *reinterpret_cast<const uint4*>(tile_h + r * T2_EPI_HSTRIDE + out_col);
                            const int64_t at = (int64_t)grow * N + col;
                            for (int p = 0; p < pc.world; ++p)
                                *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(pc.data[p] + ar.out_offset) + at) = o;
                        }
                    }
                }
            } else
#pragma unroll 2
            for (int cb = 0; cb < T2_BN / 32; ++cb) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * T2_BN + cb * 32, v);
                const int col = n0 + cb * 32;
                if (row < row_end && col < N) {

                    if (out_f32) {
                        float* dst = reinterpret_cast<float*>(c) + (int64_t)row * ldc + col;
#pragma unroll
                        for (int e = 0; e < 32; e += 4)
                            if (col + e < N)
                                *reinterpret_cast<float4*>(dst + e) = make_float4(__uint_as_float(v[e]), __uint_as_float(v[e + 1]),
                                                                                  __uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
                    } else {
                        bf16* dst = reinterpret_cast<bf16*>(c) + (int64_t)row * ldc + col;
#pragma unroll
                        for (int e = 0; e < 32; e += 8)
                            if (col + e < N) {
                                uint4 o;
                                o.x = pack_bf16(__uint_as_float(v[e]), __uint_as_float(v[e + 1]));
                                o.y = pack_bf16(__uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
                                o.z = pack_bf16(__uint_as_float(v[e + 4]), __uint_as_float(v[e + 5]));
                                o.w = pack_bf16(__uint_as_float(v[e + 6]), __uint_as_float(v[e + 7]));
                                *reinterpret_cast<uint4*>(dst + e) = o;
                            }
                    }
                }
            }
            // this warp's quarter of the accumulator has been read: hand it back to the MMA warp
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty + acc);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(T2_TMEM_COLS) : "memory");
    }
    if (ar.enabled) {
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) {
            const PeerComm& pc = ar.comm;
            uint32_t* done = pc.seq + GLMB_SEQ_DONE_BASE + ar.sig;
            if (atomicAdd(done, 1u) == gridDim.x - 1) {
                __threadfence_system();
                atomicExch(done, 0u);
                pc.seq[GLMB_SEQ_GEMM] = ar_epoch;
                const uint32_t e = pc.seq[GLMB_SEQ_SIG_BASE + ar.sig] + 1;
                pc.seq[GLMB_SEQ_SIG_BASE + ar.sig] = e;
                for (int p = 0; p < pc.world; ++p)
                    st_release_sys(pc.flags[p] + GLMB_FLAG_SIG_BASE + ar.sig * GLMB_MAX_WORLD + pc.rank, e);
            }
        }
    }
}

// ===================================================================================================
static int g_gemm_variant = 0;

static GemmAllReduce no_allreduce() {
    GemmAllReduce ar;
    memset(&ar, 0, sizeof(ar));
    return ar;
}

// a [rows, K] bf16 (lda), b [experts * N, K] bf16 (ldb), c [rows, N] bf16 or fp32 (ldc).  K % 8 == 0; a, b 16-byte
// aligned with lda, ldb multiples of 8.  tiles / n_tiles: device arrays for grouped mode (max_tiles entries) or NULL.
GLMB_API int glmb_gemm_bf16_tcgen05(const void* a, int64_t lda, const void* b, int64_t ldb, void* c, int64_t ldc, int rows, int N,
                                    int K, int experts, const void* tiles, const int* n_tiles, int max_tiles, int out_f32,
                                    uint32_t* status, void* stream) {
    if (rows < 1 || N < 8 || (N & 7) || K < 8 || (K & 7) || (lda & 7) || (ldb & 7) || (ldc & (out_f32 ? 3 : 7)) || experts < 1) return 1;
    if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) || (reinterpret_cast<uintptr_t>(c) & 15)) return 1;
    CUtensorMap map_a, map_b;
    const int m_tiles = tiles ? max_tiles : ceil_div(rows, TC_BM);
    static int sm_count = 0;
    if (!sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count < 1) sm_count = 148;
    }
    // Problems of at least 64 tiles of 128 x 256 run the persistent kernel (measured faster from there on); smaller ones keep 128 x 128 tiles,
    // which give twice as many CTAs to spread over the SMs.
    const int total2 = m_tiles * ceil_div(N, T2_BN);
    const bool persistent = g_gemm_variant == 2 || (g_gemm_variant == 0 && total2 >= 64);
    if (make_map(&map_a, a, (uint64_t)rows, (uint64_t)K, (uint64_t)lda)) return 3;
    if (make_map(&map_b, b, (uint64_t)experts * N, (uint64_t)K, (uint64_t)ldb, persistent ? T2_BN : TC_BN)) return 3;
    static DeviceOnce attr_set;
    const int attr_set_dev = attr_set.pending();
    if (attr_set_dev != DeviceOnce::SET) {
        cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(gemm_bf16_tcgen05_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T2_SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        attr_set.mark(attr_set_dev);
    }
    if (persistent) {
        GLMB_LAUNCH(gemm_bf16_tcgen05_persistent_kernel, dim3(total2 < sm_count ? total2 : sm_count), TC_THREADS, T2_SMEM_BYTES,
                    (cudaStream_t)stream, map_a, map_b, c, ldc, rows, N, K, (const TcTile*)tiles, n_tiles, max_tiles, out_f32, status, no_allreduce());
        return (int)cudaGetLastError();
    }
    dim3 grid(ceil_div(N, TC_BN), m_tiles);
    GLMB_LAUNCH(gemm_bf16_tcgen05_kernel, grid, TC_THREADS, TC_SMEM_BYTES, (cudaStream_t)stream, map_a, map_b, c, ldc, rows, N, K,
                (const TcTile*)tiles, n_tiles, out_f32, status);
    return (int)cudaGetLastError();
}

// 0: choose by problem size; 1: always 128 x 128 tiles, one per CTA; 2: always the persistent 128 x 256 kernel.
GLMB_API void glmb_set_gemm_variant(int variant) { g_gemm_variant = variant; }

// out[rows, N] (bf16, at comm->data[p] + out_offset on EVERY rank p) = sum over ranks of a_r[rows, K_r] . b_r[N, K_r]^T.
// One kernel: tcgen05 tiles, partial tiles pushed to the tile owner over NVLink, rank-ordered fp32 sum, bf16 result
// pushed to all ranks, then signal `sig`.  The caller launches glmb_wait_signal(sig) before reading the output.
// part_offset must leave room for tiles * 128 x 256 fp32 (tiles = ceil(rows/128) * ceil(N/256)): see glmb_gemm_allreduce_part_bytes.
GLMB_API int glmb_gemm_bf16_tcgen05_allreduce(const void* a, int64_t lda, const void* b, int64_t ldb, int rows, int N, int K,
                                              const PeerComm* comm, int64_t part_offset, int64_t out_offset, int sig, uint32_t* status,
                                              void* stream) {
    if (!comm || comm->world < 2 || rows < 1 || N < 8 || (N & 7) || K < 8 || (K & 7) || (lda & 7) || (ldb & 7)) return 1;
    if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) || (part_offset & 15) || (out_offset & 15)) return 1;
    const int total = ceil_div(rows, TC_BM) * ceil_div(N, T2_BN);
    if (total * (T2_BN / 32) > GLMB_GEMM_MAX_TILES || sig < 0 || sig >= GLMB_SIGNALS || (T2_BN / 32) % comm->world) return 2;
    CUtensorMap map_a, map_b;
    if (make_map(&map_a, a, (uint64_t)rows, (uint64_t)K, (uint64_t)lda)) return 3;
    if (make_map(&map_b, b, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, T2_BN)) return 3;
    static DeviceOnce attr_set;
    const int attr_set_dev = attr_set.pending();
    if (attr_set_dev != DeviceOnce::SET) {
        cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tcgen05_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T2_SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        attr_set.mark(attr_set_dev);
    }
    int dev = 0, sm_count = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sm_count < 1) sm_count = 148;
    GemmAllReduce ar;
    ar.enabled = 1;
    ar.sig = sig;
    ar.part_offset = part_offset;
    ar.out_offset = out_offset;
    ar.comm = *comm;
    void* c = comm->data[comm->rank] + out_offset;
    GLMB_LAUNCH(gemm_bf16_tcgen05_persistent_kernel, dim3(total < sm_count ? total : sm_count), TC_THREADS, T2_SMEM_BYTES, (cudaStream_t)stream,
                map_a, map_b, c, (int64_t)N, rows, N, K, (const TcTile*)nullptr, (const int*)nullptr, 0, 0, status, ar);
    return (int)cudaGetLastError();
}

// Bytes of partial-tile slots glmb_gemm_bf16_tcgen05_allreduce needs at part_offset.
GLMB_API int64_t glmb_gemm_allreduce_part_bytes(int rows, int N, int world) {
    (void)world;  // every rank owns 8 / world blocks of every tile and receives world - 1 (+ its own unused) copies of each
    const int64_t total = (int64_t)ceil_div(rows, TC_BM) * ceil_div(N, T2_BN);
    return total * (int64_t)T2_TILE_FLOATS * 4;
}
