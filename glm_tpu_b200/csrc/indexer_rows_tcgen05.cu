// DSA lightning-indexer scoring for MANY query rows of one chat (prefill chunks) on the 5th-generation tensor cores.
//
//   score[row][key] = sum_h w[row][h] * relu( (q[row][h] . key) * scale )      q fp32, key bf16, accumulated in fp32
//
// The one-row kernel (`indexer_tcgen05.cu`) spends a whole CTA on (128 keys, one row) and rebuilds the query pieces in each
// of them: right for decode, wasteful when thousands of rows score the same keys.  Here
//
//   1. `indexer_split_rows_kernel` builds the N operand of every row ONCE: the fp32 query (rotated here when it comes
//      straight from the q_b projection) split exactly into three bf16 pieces, [row][piece * 32 + head][128] in global memory;
//   2. `indexer_score_rows_kernel`: one CTA keeps 4 key tiles (512 keys x 128 features, 128 KB) resident in shared memory and
//      walks up to 128 rows: a 3-stage TMA ring streams each row's 24 KB of pieces and its 32 head weights, one lane issues
//      8 tcgen05.mma (M 128 keys, N 96, K 16) per (row, key tile) into a ring of four 96-column TMEM accumulators (four
//      issuing threads, one per accumulator: one thread cannot issue as fast as these small MMAs retire), and two
//      groups of four epilogue warps (thread = key), taking the accumulators alternately, apply relu, the head weights and the
//      sum over heads and store the scores.
//
// Per (row, key tile) the SM reads 6 KB of L2 instead of 56 KB, no CTA is launched per row, and the tensor pipe sees back-to-
// back MMAs.  Rows above a key tile in the causal triangle (context <= first key) are skipped by every role alike.
// All rows of a call belong to one chat (one cache lane): the caller guarantees it.  Waits are bounded.
//
// Replaces reference `glm_tpu/layers/attention/dsa_indexer.py:129-150,352-393` for prefill chunks.
#include "common.cuh"
#include "peer.cuh"
#include "tcgen05.cuh"
#include "indexer_query.cuh"

#define IR_KEYS 128
#define IR_D 128
#define IR_IH 32
#define IR_N (3 * IR_IH)
#define IR_TILES 4
#define IR_QSTAGES 3
#define IR_BUFS 4                                  // TMEM accumulators: accumulator b belongs to issuing thread b and to epilogue group b & 1
#define IR_ROWS 128
#define IR_ISSUERS 4                               // one lane of each of four warps issues the MMAs of every fourth accumulator
#define IR_THREADS 416                             // TMA warp, MMA warp, two epilogue groups of 4 warps, three more MMA warps
#define IR_A_BYTES (IR_KEYS * IR_D * 2)            // one key tile: two 16 KB boxes
#define IR_Q_BYTES (IR_N * IR_D * 2)               // one row's pieces: two 12 KB boxes
#define IR_W_BYTES (IR_IH * 4)
#define IR_STAGE_BYTES (IR_Q_BYTES + 1024)         // pieces, then the head weights (padding keeps every stage 1024-byte aligned)
#define IR_TMEM_COLS 512
static_assert(IR_BUFS == IR_ISSUERS && IR_BUFS % 2 == 0 && IR_BUFS * IR_N <= IR_TMEM_COLS, "one accumulator per issuing thread, alternating between the two epilogue groups");
#define IR_SMEM_BYTES (1024 + IR_TILES * IR_A_BYTES + IR_QSTAGES * IR_STAGE_BYTES + 256 + IR_ROWS * 4)

// positions < ctx of a position-striped cache that this rank stores
__device__ __forceinline__ int ir_owned(int pos, int capacity, int stripe, int world, int rank) {
    const int ctx = min(max(pos, 0), capacity - 1) + 1;
    const int page = stripe * world;
    const int rest = ctx % page;
    return (ctx / page) * stripe + min(max(rest - rank * stripe, 0), stripe);
}

__global__ void __launch_bounds__(256)
indexer_split_rows_kernel(IndexerQuerySource src, const int* __restrict__ row_pos, int capacity, __nv_bfloat16* __restrict__ pieces) {
    GLMB_PDL_PROLOGUE();
    const int r = blockIdx.x;
    const int pos = min(max(row_pos[r], 0), capacity - 1);
    for (int i = threadIdx.x; i < IR_IH * IR_D / 8; i += blockDim.x) {  // one 8-feature chunk of one head per step
        const int h = i / (IR_D / 8), c8 = i % (IR_D / 8);
        uint4 piece[3];
        indexer_query_pieces(src, r, h, c8, IR_D, pos, piece);
#pragma unroll
        for (int p = 0; p < 3; ++p)
            *reinterpret_cast<uint4*>(pieces + ((int64_t)r * IR_N + p * IR_IH + h) * IR_D + c8 * 8) = piece[p];
    }
}

__device__ __forceinline__ void ir_bulk_load(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(smem_dst)), "l"(src),
                 "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// tcgen05.ld of 32 columns without the wait: the caller issues several and waits once
__device__ __forceinline__ void ir_tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}

__global__ void __launch_bounds__(IR_THREADS, 1)
indexer_score_rows_kernel(const __grid_constant__ CUtensorMap map_keys, const __grid_constant__ CUtensorMap map_q, const float* __restrict__ head_w,
                          const int* __restrict__ row_pos, int cache_row_base, int rows, int stripe, int world, int rank, int capacity,
                          int64_t score_stride, float scale, float* __restrict__ scores, int64_t scores_offset, PeerComm comm, int sig,
                          uint32_t* status) {
    GLMB_PDL_PROLOGUE();
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* a_s = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_s = a_s + IR_TILES * IR_A_BYTES;
    uint64_t* a_bar = reinterpret_cast<uint64_t*>(q_s + IR_QSTAGES * IR_STAGE_BYTES);
    uint64_t* q_full = a_bar + 1;
    uint64_t* q_empty = q_full + IR_QSTAGES;
    uint64_t* t_full = q_empty + IR_QSTAGES;
    uint64_t* t_empty = t_full + IR_BUFS;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(t_empty + IR_BUFS);
    volatile uint32_t* fail_slot = tmem_slot + 1;
    int* owned_max_slot = reinterpret_cast<int*>(tmem_slot + 2);
    int* owned_s = reinterpret_cast<int*>(reinterpret_cast<unsigned char*>(a_bar) + 256);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j0 = blockIdx.x * (IR_TILES * IR_KEYS);  // first key (row of this rank's cache slice) of the CTA
    const int r0 = blockIdx.y * IR_ROWS;
    const int n_rows = min(IR_ROWS, rows - r0);
    const int page = stripe * world;

    if (threadIdx.x == 0) {
        mbar_init(a_bar, 1);
        for (int s = 0; s < IR_QSTAGES; ++s) { mbar_init(q_full + s, 1); mbar_init(q_empty + s, IR_ISSUERS + 8); }  // the MMA issuers' commits + 8 epilogue warps
        for (int b = 0; b < IR_BUFS; ++b) { mbar_init(t_full + b, 1); mbar_init(t_empty + b, 4); }
        *fail_slot = 0;
        *owned_max_slot = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_rows; i += IR_THREADS) {
        const int own = ir_owned(row_pos[r0 + i], capacity, stripe, world, rank);
        owned_s[i] = own;
        atomicMax(owned_max_slot, own);
    }
    __syncthreads();
    const int owned_max = *owned_max_slot;
    const bool live = owned_max > j0;  // uniform per CTA; a CTA above the causal triangle only takes part in the signal

    if (live) {
        const int cta_tiles = min(IR_TILES, (owned_max - j0 + IR_KEYS - 1) / IR_KEYS);
        if (warp == 1) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(IR_TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_base = *tmem_slot;

        if (warp == 0) {
            // ---- producer: the key tiles once, then one stage per live row -----------------------------------------
            if (lane == 0) {
                mbar_expect_tx(a_bar, (uint32_t)cta_tiles * IR_A_BYTES);
                for (int t = 0; t < cta_tiles; ++t) {
                    tma_load_2d(a_s + t * IR_A_BYTES, &map_keys, a_bar, 0, cache_row_base + j0 + t * IR_KEYS);
                    tma_load_2d(a_s + t * IR_A_BYTES + IR_KEYS * 128, &map_keys, a_bar, 64, cache_row_base + j0 + t * IR_KEYS);
                }
                int li = 0;
                for (int i = 0; i < n_rows; ++i) {
                    if (owned_s[i] <= j0) continue;
                    const int s = li % IR_QSTAGES, lap = li / IR_QSTAGES;
                    if (*fail_slot || (lap > 0 && !mbar_wait(q_empty + s, (lap - 1) & 1))) { *fail_slot = 1; break; }
                    unsigned char* dst = q_s + s * IR_STAGE_BYTES;
                    mbar_expect_tx(q_full + s, IR_Q_BYTES + IR_W_BYTES);
                    tma_load_2d(dst, &map_q, q_full + s, 0, (r0 + i) * IR_N);
                    tma_load_2d(dst + IR_N * 128, &map_q, q_full + s, 64, (r0 + i) * IR_N);
                    ir_bulk_load(dst + IR_Q_BYTES, head_w + (int64_t)(r0 + i) * IR_IH, IR_W_BYTES, q_full + s);
                    ++li;
                }
            }
        } else if (warp == 1 || warp >= 10) {
            // ---- MMA issuers: an N = 96 instruction keeps the tensor core busy for ~50 cycles, less than one thread needs to wait for
            //      a free accumulator, build the descriptors and issue; four threads take the accumulators in turn ------------------------------------------------------------------------------------------
            if (lane == 0) {
                constexpr uint32_t idesc = umma_idesc_bf16(IR_KEYS, IR_N);
                const int issuer = warp == 1 ? 0 : warp - 9;
                bool ok = mbar_wait(a_bar, 0);
                int li = 0, n = 0;
                for (int i = 0; i < n_rows && ok; ++i) {
                    const int own = owned_s[i];
                    if (own <= j0) continue;
                    const int s = li % IR_QSTAGES, lap = li / IR_QSTAGES;
                    if (*fail_slot || !mbar_wait(q_full + s, lap & 1)) { ok = false; break; }
                    const uint32_t b_addr = smem_u32(q_s + s * IR_STAGE_BYTES);
                    const int tiles = min(IR_TILES, (own - j0 + IR_KEYS - 1) / IR_KEYS);
                    for (int t = 0; t < tiles; ++t, ++n) {
                        // IR_BUFS == IR_ISSUERS: accumulator b is filled by thread b alone and drained by epilogue group b & 1 alone,
                        // each in increasing n.  A parity wait can only tell the current phase of an mbarrier from the previous one,
                        // so no two threads that may drift apart by a lap of the ring may share one of these barriers.
                        if (n % IR_ISSUERS != issuer) continue;
                        const int b = n % IR_BUFS, blap = n / IR_BUFS;
                        if (blap > 0 && !mbar_wait(t_empty + b, (blap - 1) & 1)) { ok = false; break; }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t a_addr = smem_u32(a_s + t * IR_A_BYTES);
#pragma unroll
                        for (int kh = 0; kh < 2; ++kh)
#pragma unroll
                            for (int k = 0; k < 4; ++k)
                                umma_bf16(tmem_base + b * IR_N, umma_desc_sw128(a_addr + kh * (IR_KEYS * 128) + k * 32),
                                          umma_desc_sw128(b_addr + kh * (IR_N * 128) + k * 32), idesc, (kh > 0 || k > 0) ? 1u : 0u);
                        umma_commit(t_full + b);
                    }
                    if (!ok) break;
                    umma_commit(q_empty + s);  // this thread's MMAs on the row's pieces have retired (at once, if it issued none)
                    ++li;
                }
                if (!ok) { *fail_slot = 1; raise_status(status, GLMB_STATUS_WAIT_TIMEOUT); }
            }
        } else {
            // ---- epilogue: thread = key ------------------------------------------------------------------------------
            const int quarter = warp & 3, group = (warp - 2) >> 2;  // a warp reads the TMEM lanes of its quarter; group g takes accumulators n = g (mod 2)
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
            bool ok = true;
            int li = 0, n = 0;
            for (int i = 0; i < n_rows && ok; ++i) {
                const int own = owned_s[i];
                if (own <= j0) continue;
                const int s = li % IR_QSTAGES, lap = li / IR_QSTAGES;
                if (*fail_slot || !mbar_wait(q_full + s, lap & 1)) { ok = false; break; }  // the head weights of this row have landed
                const float4* w4 = reinterpret_cast<const float4*>(q_s + s * IR_STAGE_BYTES + IR_Q_BYTES);
                const int tiles = min(IR_TILES, (own - j0 + IR_KEYS - 1) / IR_KEYS);
                const int r = r0 + i;
                for (int t = 0; t < tiles; ++t, ++n) {
                    if ((n & 1) != group) continue;
                    const int b = n % IR_BUFS, blap = n / IR_BUFS;
                    if (!mbar_wait(t_full + b, blap & 1)) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    uint32_t c0[32], c1[32], c2[32];
                    ir_tmem_ld32_issue(lane_addr + b * IR_N, c0);  // three loads in flight, one wait
                    ir_tmem_ld32_issue(lane_addr + b * IR_N + 32, c1);
                    ir_tmem_ld32_issue(lane_addr + b * IR_N + 64, c2);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(t_empty + b);  // the accumulator is in registers: the tensor core may overwrite it
                    const int j = j0 + t * IR_KEYS + quarter * 32 + lane;  // this thread's key (row of the local cache slice)
                    if (j < own) {
                        float score = 0.f;
#pragma unroll
                        for (int h4 = 0; h4 < IR_IH / 4; ++h4) {
                            const float4 w = w4[h4];
                            const float wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int h = h4 * 4 + e;
                                const float dot = (__uint_as_float(c0[h]) + __uint_as_float(c1[h])) + __uint_as_float(c2[h]);
                                score = fmaf(wv[e], fmaxf(__fmul_rn(dot, scale), 0.f), score);
                            }
                        }
                        if (!isfinite(score)) raise_status(status, GLMB_STATUS_NONFINITE);
                        const int g = (j / stripe) * page + rank * stripe + j % stripe;
                        const int64_t at = (int64_t)r * score_stride + g;
                        scores[at] = score;
                        for (int p = 0; p < comm.world; ++p)
                            if (p != comm.rank) reinterpret_cast<float*>(comm.data[p] + scores_offset)[at] = score;
                    }
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) mbar_arrive(q_empty + s);  // this warp has read the row's head weights
                ++li;
            }
            if (!ok) { *fail_slot = 1; if (lane == 0) raise_status(status, GLMB_STATUS_WAIT_TIMEOUT); }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (warp == 1) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(IR_TMEM_COLS) : "memory");
        }
    }
    grid_signal_peers(comm, sig);
}

GLMB_API int64_t glmb_indexer_rows_scratch_bytes(int rows) { return (int64_t)rows * IR_N * IR_D * 2; }

// Scores of `rows` query rows of ONE chat (cache lane `lane`) against this rank's slice of the index cache; the contract of
// glmb_indexer_score for D == 128 and IH == 32.  q: fp32 [rows, q_stride] with the index heads at q_offset; inv_freq != null
// means q is the raw q_b projection and the first rd features of every head are rotated here.  pieces: scratch of
// glmb_indexer_rows_scratch_bytes(rows) bytes, 16-byte aligned.
GLMB_API int glmb_indexer_score_tc_rows(const float* q, int64_t q_stride, int64_t q_offset, const float* inv_freq, int rd, const float* head_w,
                                        const void* index_cache, int64_t cache_rows, const int* row_pos, int lane, int rows, int IH, int D,
                                        int index_slot, int full_layers, int local_cap, int stripe, int world, int rank, int capacity,
                                        int max_ctx, int64_t score_stride, float scale, float* scores, int64_t scores_offset, void* pieces,
                                        const PeerComm* comm, int sig, uint32_t* status, void* stream) {
    if (IH != IR_IH || D != IR_D || rows < 1 || cache_rows < 1 || !q || !pieces || (rd & 1) || rd > D || (q_stride & 3) || (q_offset & 3)) return 1;
    if ((reinterpret_cast<uintptr_t>(index_cache) & 15) || (reinterpret_cast<uintptr_t>(pieces) & 15) || (reinterpret_cast<uintptr_t>(q) & 15) ||
        (reinterpret_cast<uintptr_t>(head_w) & 15))
        return 1;
    PeerComm c;
    if (comm) c = *comm; else { memset(&c, 0, sizeof(c)); c.world = 1; }
    CUtensorMap map_keys, map_q;
    if (make_map(&map_keys, index_cache, (uint64_t)cache_rows, (uint64_t)IR_D, (uint64_t)IR_D, IR_KEYS)) return 3;
    if (make_map(&map_q, pieces, (uint64_t)rows * IR_N, (uint64_t)IR_D, (uint64_t)IR_D, IR_N)) return 3;
    static DeviceOnce attr_set;
    const int attr_set_dev = attr_set.pending();
    if (attr_set_dev != DeviceOnce::SET) {
        cudaError_t e = cudaFuncSetAttribute(indexer_score_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, IR_SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        attr_set.mark(attr_set_dev);
    }
    IndexerQuerySource src;
    src.q = q; src.q_stride = q_stride; src.q_offset = q_offset; src.inv_freq = inv_freq; src.rd = rd;
    GLMB_LAUNCH(indexer_split_rows_kernel, dim3(rows), 256, 0, (cudaStream_t)stream, src, row_pos, capacity, reinterpret_cast<__nv_bfloat16*>(pieces));
    const int page = stripe * world;
    const int owned_max = (max_ctx / page) * stripe + min(max_ctx % page, stripe);
    dim3 grid(ceil_div(owned_max > 0 ? owned_max : 1, IR_TILES * IR_KEYS), ceil_div(rows, IR_ROWS));
    const int cache_row_base = (lane * full_layers + index_slot) * local_cap;
    GLMB_LAUNCH(indexer_score_rows_kernel, grid, IR_THREADS, IR_SMEM_BYTES, (cudaStream_t)stream, map_keys, map_q, head_w, row_pos, cache_row_base,
                rows, stripe, world, rank, capacity, score_stride, scale, scores, scores_offset, c, sig, status);
    return (int)cudaGetLastError();
}
