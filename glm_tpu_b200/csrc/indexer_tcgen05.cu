// DSA lightning-indexer scoring on the 5th-generation tensor cores (index head width 128, 32 index heads).
//
//   score[key] = sum_h w_h * relu( (q_h . key) * scale )          q fp32, key bf16, everything accumulated in fp32
//
// The contraction is a GEMM with the KEYS as the 128-row M operand, so after tcgen05.ld every thread owns one key and
// all of its 32 head dot products: the relu / weight / sum over heads is thread-local.  The fp32 query is split exactly
// into three bf16 pieces (q = hi + mid + lo to 2^-24), giving a 96-row N operand [piece][head]; bf16 x bf16 products are
// exact in fp32, so the three partial dots add up to the fp32-accurate q . key.
//
//   all threads   split the query row into pieces and write them to shared memory in the 128-byte-swizzled K-major layout
//   thread 0      TMA: 128 keys x 128 features (two 64-wide boxes) straight from the index cache, issued first
//   warp 1        one lane issues 8 tcgen05.mma (M 128, N 96, K 16) into 96 TMEM columns
//   warps 2-5     tcgen05.ld (lane = key), per-head relu and weighting, store the score at its global position in this
//                 rank's score row and in every peer's (fused all-gather), then the last CTA signals
//
// One CTA per (128 owned keys, query row); ~57 KB of shared memory, so several CTAs share an SM.  Waits are bounded.
//
// Replaces reference `glm_tpu/layers/attention/dsa_indexer.py:129-150,352-393`; same contract as `indexer_score_kernel`
// (`indexer.cu`), which remains the path for other head shapes.
#include "common.cuh"
#include "peer.cuh"
#include "tcgen05.cuh"
#include "indexer_query.cuh"

#define IT_KEYS 128
#define IT_D 128
#define IT_IH 32
#define IT_N (3 * IT_IH)
#define IT_THREADS 192
#define IT_A_BYTES (IT_KEYS * IT_D * 2)      // two 16 KB boxes
#define IT_B_BYTES (2 * IT_N * 64 * 2)       // two K-halves of the 96-row query tile
#define IT_SMEM_BYTES (IT_A_BYTES + IT_B_BYTES + 1024 + 128 + IT_IH * 4)
#define IT_TMEM_COLS 128

// When q_raw is set, the query comes straight from the q_b projection (fp32, before RoPE) and the kernel rotates its first
// rd features itself (fp32 cos/sin of position * inv_freq, interleaved pairs: the arithmetic of q_post).
struct IndexerRawQuery {
    const float* q_raw;  // [rows, q_stride], index head h at q_offset + h * 128
    int64_t q_stride, q_offset;
    const float* inv_freq;  // [rd / 2]
    int rd;
};

__global__ void __launch_bounds__(IT_THREADS)
indexer_score_tc_kernel(const __grid_constant__ CUtensorMap map_keys, const float* __restrict__ q_idx, const float* __restrict__ head_w,
                        const int* __restrict__ row_pos, const int* __restrict__ row_lane, int index_slot, int full_layers, int local_cap,
                        int stripe, int world, int rank, int capacity, int64_t score_stride, float scale, float* __restrict__ scores,
                        int64_t scores_offset, PeerComm comm, int sig, uint32_t* status, IndexerRawQuery raw) {
    GLMB_PDL_PROLOGUE();
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* a_s = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* b_s = a_s + IT_A_BYTES;  // 1024-byte aligned: [k-half][96 rows][64 bf16], swizzled
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(b_s + IT_B_BYTES);
    uint64_t* acc_bar = full_bar + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
    float* w_s = reinterpret_cast<float*>(b_s + IT_B_BYTES + 128);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.y;
    const int pos = min(max(row_pos[r], 0), capacity - 1);
    const int ctx = pos + 1;
    const int page = stripe * world;
    const int rest = ctx % page;
    const int owned = (ctx / page) * stripe + min(max(rest - rank * stripe, 0), stripe);  // positions < ctx stored on this rank
    const int j0 = blockIdx.x * IT_KEYS;
    const bool live = j0 < owned;  // uniform per CTA; a CTA past the owned range only takes part in the signal

    if (live) {
        if (threadIdx.x == 0) {
            mbar_init(full_bar, 1);
            mbar_init(acc_bar, 1);
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            // the key tile is requested first, so that it lands while the query pieces are being built
            const int cache_row = (row_lane[r] * full_layers + index_slot) * local_cap + j0;
            mbar_expect_tx(full_bar, IT_A_BYTES);
            tma_load_2d(a_s, &map_keys, full_bar, 0, cache_row);
            tma_load_2d(a_s + IT_KEYS * 128, &map_keys, full_bar, 64, cache_row);
        }
        if (warp == 1) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(IT_TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
        // query row -> three exact bf16 pieces, rows [piece * 32 + head] of the N operand
        IndexerQuerySource src;
        src.q = raw.q_raw ? raw.q_raw : q_idx;
        src.q_stride = raw.q_raw ? raw.q_stride : (int64_t)IT_IH * IT_D;
        src.q_offset = raw.q_raw ? raw.q_offset : 0;
        src.inv_freq = raw.q_raw ? raw.inv_freq : nullptr;
        src.rd = raw.q_raw ? raw.rd : 0;
        for (int i = threadIdx.x; i < IT_IH * IT_D / 8; i += IT_THREADS) {  // one 8-feature chunk of one head per step
            const int h = i / (IT_D / 8), c8 = i % (IT_D / 8);             // c8: 16-byte chunk index along K (0..15)
            uint4 piece[3];
            indexer_query_pieces(src, r, h, c8, IT_D, pos, piece);
            const int khalf = c8 >> 3, chunk = c8 & 7;
#pragma unroll
            for (int p = 0; p < 3; ++p) {
                const int n = p * IT_IH + h;
                unsigned char* line = b_s + khalf * (IT_N * 128) + (n >> 3) * 1024 + (n & 7) * 128;
                *reinterpret_cast<uint4*>(line + ((chunk ^ (n & 7)) << 4)) = piece[p];
            }
        }
        if (threadIdx.x < IT_IH) w_s[threadIdx.x] = head_w[(int64_t)r * IT_IH + threadIdx.x];
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_base = *tmem_slot;

        if (warp == 1) {
            if (lane == 0) {
                constexpr uint32_t idesc = umma_idesc_bf16(IT_KEYS, IT_N);
                if (mbar_wait(full_bar, 0)) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (int kh = 0; kh < 2; ++kh)
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma_bf16(tmem_base, umma_desc_sw128(smem_u32(a_s + kh * (IT_KEYS * 128)) + k * 32),
                                      umma_desc_sw128(smem_u32(b_s + kh * (IT_N * 128)) + k * 32), idesc, (kh > 0 || k > 0) ? 1u : 0u);
                } else {
                    raise_status(status, GLMB_STATUS_WAIT_TIMEOUT);
                }
                umma_commit(acc_bar);
            }
        } else {
            const int quarter = warp & 3;
            const bool ok = mbar_wait(acc_bar, 0);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (!ok) {
                if (lane == 0) raise_status(status, GLMB_STATUS_WAIT_TIMEOUT);
            } else {
                uint32_t c0[32], c1[32], c2[32];
                const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
                tmem_ld32(lane_addr, c0);
                tmem_ld32(lane_addr + 32, c1);
                tmem_ld32(lane_addr + 64, c2);
                const int j = j0 + quarter * 32 + lane;  // this thread's key (row of the local cache slice)
                if (j < owned) {
                    float score = 0.f;
#pragma unroll
                    for (int h = 0; h < IT_IH; ++h) {
                        const float dot = (__uint_as_float(c0[h]) + __uint_as_float(c1[h])) + __uint_as_float(c2[h]);
                        score = fmaf(w_s[h], fmaxf(__fmul_rn(dot, scale), 0.f), score);
                    }
                    if (!isfinite(score)) raise_status(status, GLMB_STATUS_NONFINITE);
                    const int g = (j / stripe) * page + rank * stripe + j % stripe;
                    const int64_t at = (int64_t)r * score_stride + g;
                    scores[at] = score;
                    for (int p = 0; p < comm.world; ++p)
                        if (p != comm.rank) reinterpret_cast<float*>(comm.data[p] + scores_offset)[at] = score;
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (warp == 1) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(IT_TMEM_COLS) : "memory");
        }
    }
    grid_signal_peers(comm, sig);
}

// Same contract as glmb_indexer_score for D == 128 and IH == 32.  cache_rows: rows of the whole index cache viewed as
// [lanes * full_layers * local_cap, 128] bf16 (the TMA tensor map covers it; a tile is addressed by its first row).
static int indexer_tc_launch(const float* q_idx, const IndexerRawQuery& raw, const float* head_w, const void* index_cache, int64_t cache_rows,
                             const int* row_pos, const int* row_lane, int rows, int IH, int D, int index_slot, int full_layers, int local_cap,
                             int stripe, int world, int rank, int capacity, int max_ctx, int64_t score_stride, float scale, float* scores,
                             int64_t scores_offset, const PeerComm* comm, int sig, uint32_t* status, void* stream);

GLMB_API int glmb_indexer_score_tc(const float* q_idx, const float* head_w, const void* index_cache, int64_t cache_rows, const int* row_pos,
                                   const int* row_lane, int rows, int IH, int D, int index_slot, int full_layers, int local_cap, int stripe,
                                   int world, int rank, int capacity, int max_ctx, int64_t score_stride, float scale, float* scores,
                                   int64_t scores_offset, const PeerComm* comm, int sig, uint32_t* status, void* stream) {
    if (!q_idx || (reinterpret_cast<uintptr_t>(q_idx) & 15)) return 1;
    IndexerRawQuery raw;
    memset(&raw, 0, sizeof(raw));
    return indexer_tc_launch(q_idx, raw, head_w, index_cache, cache_rows, row_pos, row_lane, rows, IH, D, index_slot, full_layers, local_cap, stripe,
                             world, rank, capacity, max_ctx, score_stride, scale, scores, scores_offset, comm, sig, status, stream);
}

// The same with the query taken from the raw q_b projection (fp32 [rows, q_stride], index heads at q_offset) and rotated in-kernel.
GLMB_API int glmb_indexer_score_tc_raw(const float* q_raw, int64_t q_stride, int64_t q_offset, const float* inv_freq, int rd, const float* head_w,
                                       const void* index_cache, int64_t cache_rows, const int* row_pos, const int* row_lane, int rows, int IH,
                                       int D, int index_slot, int full_layers, int local_cap, int stripe, int world, int rank, int capacity,
                                       int max_ctx, int64_t score_stride, float scale, float* scores, int64_t scores_offset,
                                       const PeerComm* comm, int sig, uint32_t* status, void* stream) {
    if (!q_raw || !inv_freq || (rd & 1) || rd > D || (q_stride & 3) || (q_offset & 3) || (reinterpret_cast<uintptr_t>(q_raw) & 15)) return 1;
    IndexerRawQuery raw;
    raw.q_raw = q_raw; raw.q_stride = q_stride; raw.q_offset = q_offset; raw.inv_freq = inv_freq; raw.rd = rd;
    return indexer_tc_launch(nullptr, raw, head_w, index_cache, cache_rows, row_pos, row_lane, rows, IH, D, index_slot, full_layers, local_cap,
                             stripe, world, rank, capacity, max_ctx, score_stride, scale, scores, scores_offset, comm, sig, status, stream);
}

static int indexer_tc_launch(const float* q_idx, const IndexerRawQuery& raw, const float* head_w, const void* index_cache, int64_t cache_rows,
                             const int* row_pos, const int* row_lane, int rows, int IH, int D, int index_slot, int full_layers, int local_cap,
                             int stripe, int world, int rank, int capacity, int max_ctx, int64_t score_stride, float scale, float* scores,
                             int64_t scores_offset, const PeerComm* comm, int sig, uint32_t* status, void* stream) {
    if (IH != IT_IH || D != IT_D || rows < 1 || cache_rows < 1 || (reinterpret_cast<uintptr_t>(index_cache) & 15)) return 1;
    PeerComm c;
    if (comm) c = *comm; else { memset(&c, 0, sizeof(c)); c.world = 1; }
    CUtensorMap map_keys;
    if (make_map(&map_keys, index_cache, (uint64_t)cache_rows, (uint64_t)IT_D, (uint64_t)IT_D, IT_KEYS)) return 3;
    static DeviceOnce attr_set;
    const int attr_set_dev = attr_set.pending();
    if (attr_set_dev != DeviceOnce::SET) {
        cudaError_t e = cudaFuncSetAttribute(indexer_score_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, IT_SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        attr_set.mark(attr_set_dev);
    }
    const int page = stripe * world;
    const int owned_max = (max_ctx / page) * stripe + min(max_ctx % page, stripe);
    dim3 grid(ceil_div(owned_max > 0 ? owned_max : 1, IT_KEYS), rows);
    GLMB_LAUNCH(indexer_score_tc_kernel, grid, IT_THREADS, IT_SMEM_BYTES, (cudaStream_t)stream, map_keys, q_idx, head_w, row_pos, row_lane,
                index_slot, full_layers, local_cap, stripe, world, rank, capacity, score_stride, scale, scores, scores_offset, c, sig, status, raw);
    return (int)cudaGetLastError();
}
