// DeepSeek-sparse absorbed-MLA attention over the position-striped cache.
//
// Each GPU holds 1/world of the cached rows.  For a query row the selection kernel has already listed
// which of the top-k positions live on this GPU (ascending).  Attention runs owner-locally:
//
//   sparse_mla_partial   one CTA per (chunk of AT_CHUNK owned selected rows, query row): gathers the rows
//                        into shared memory, computes the fp32 scores of ALL heads against them, the
//                        chunk-local softmax statistics and the unnormalized bf16-P . latent product
//   attn_local_merge     merges a row's chunks per head (log-sum-exp algebra).  With one GPU it normalizes
//                        and stores bf16.  With several it pushes (o, m, l) of head h straight into the
//                        buffer of the GPU that owns head h (tensor-parallel by heads) and signals.
//   attn_final_merge     the head owner waits for the signal, merges the `world` partials in rank order,
//                        normalizes and stores bf16.
//
// The 2.6 MB selected-row all-reduce of the reference (`glm_tpu/layers/attention/mla.py:484-485`) becomes an
// exchange of heads x (latent + 2) fp32 per row.  Numerics restate `kernels/sparse_mla/kernel.py:128-183`
// (fp32 scores, bf16 P before P.V, one final normalisation, empty row -> zeros) and the owner-local
// partial/LSE-merge of `kernels/sparse_mla/partial_kernel.py:45-78`, `layers/attention/mla.py:288-376`.
#include "common.cuh"
#include "peer.cuh"

#define AT_CHUNK 32
#define AT_THREADS 256
#define AT_HEAD_TILE 16

// part_o  [rows, max_chunks, H, L] fp32 (unnormalized, relative to the chunk max)
// part_ml [rows, max_chunks, H, 2] fp32 (max, sum)
__global__ void __launch_bounds__(AT_THREADS)
sparse_mla_partial_kernel(const bf16* __restrict__ q_full, const bf16* __restrict__ kv_cache, const int* __restrict__ sel_local,
                          const int* __restrict__ sel_counts, const int* __restrict__ row_lane, int H, int L, int rd, int layer,
                          int layers, int local_cap, int top_k, int max_chunks, float scale, float* __restrict__ part_o,
                          float* __restrict__ part_ml, PeerComm comm, int wait_sig, uint32_t* status) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int W = L + rd;
    const int WP = W + 8;  // padded row (bf16 elements): keeps 16-byte alignment, staggers banks
    bf16* kv_s = reinterpret_cast<bf16*>(smem_raw);                        // [AT_CHUNK][WP]
    float* p_s = reinterpret_cast<float*>(kv_s + AT_CHUNK * WP);           // [H][AT_CHUNK]
    float* ml_s = p_s + H * AT_CHUNK;                                      // [H][2]
    if (wait_sig >= 0) cta_wait_signal(comm, wait_sig);
    const int r = blockIdx.y, chunk = blockIdx.x;
    const int count = min(max(sel_counts[2 * r + 1], 0), top_k);
    const int start = chunk * AT_CHUNK;
    if (start >= count) return;
    const int cnt = min(AT_CHUNK, count - start);
    const bf16* cache = kv_cache + ((int64_t)row_lane[r] * layers + layer) * (int64_t)local_cap * W;
    // gather
    const int vec_per_row = W / 8;
    for (int i = threadIdx.x; i < cnt * vec_per_row; i += AT_THREADS) {
        const int c = i / vec_per_row, v = i % vec_per_row;
        int row = sel_local[(int64_t)r * top_k + start + c];
        if (row < 0 || row >= local_cap) { raise_status(status, GLMB_STATUS_BAD_INDEX); row = min(max(row, 0), local_cap - 1); }
        *reinterpret_cast<uint4*>(kv_s + c * WP + v * 8) = *reinterpret_cast<const uint4*>(cache + (int64_t)row * W + v * 8);
    }
    __syncthreads();
    // scores
    const bf16* q = q_full + (int64_t)r * H * W;
    for (int idx = threadIdx.x; idx < H * AT_CHUNK; idx += AT_THREADS) {
        const int h = idx / AT_CHUNK, c = idx % AT_CHUNK;
        float s = -INFINITY;
        if (c < cnt) {
            float dot = 0.f;
            const bf16* qh = q + (int64_t)h * W;
            const bf16* kr = kv_s + c * WP;
            for (int v = 0; v < vec_per_row; ++v) {
                const uint4 a = ld_hot16(qh + v * 8);
                const uint4 b = *reinterpret_cast<const uint4*>(kr + v * 8);
                dot = fmaf(bf16_lo(a.x), bf16_lo(b.x), dot); dot = fmaf(bf16_hi(a.x), bf16_hi(b.x), dot);
                dot = fmaf(bf16_lo(a.y), bf16_lo(b.y), dot); dot = fmaf(bf16_hi(a.y), bf16_hi(b.y), dot);
                dot = fmaf(bf16_lo(a.z), bf16_lo(b.z), dot); dot = fmaf(bf16_hi(a.z), bf16_hi(b.z), dot);
                dot = fmaf(bf16_lo(a.w), bf16_lo(b.w), dot); dot = fmaf(bf16_hi(a.w), bf16_hi(b.w), dot);
            }
            s = __fmul_rn(dot, scale);
            if (!isfinite(s)) raise_status(status, GLMB_STATUS_NONFINITE);
        }
        p_s[idx] = s;
    }
    __syncthreads();
    // chunk-local softmax statistics: one warp per head (AT_CHUNK == 32 == warp width)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int h = warp; h < H; h += AT_THREADS / 32) {
        const float s = p_s[h * AT_CHUNK + lane];
        const float m = warp_max(s);
        const float p = lane < cnt ? expf(s - m) : 0.f;
        const float l = warp_sum(p);
        p_s[h * AT_CHUNK + lane] = bf16_round(p);
        if (lane == 0) { ml_s[2 * h] = m; ml_s[2 * h + 1] = l; }
    }
    __syncthreads();
    // P . latent
    const int64_t obase = ((int64_t)r * max_chunks + chunk) * H;
    for (int h0 = 0; h0 < H; h0 += AT_HEAD_TILE) {
        const int hn = min(AT_HEAD_TILE, H - h0);
        for (int j2 = threadIdx.x; j2 < L / 2; j2 += AT_THREADS) {
            float acc[AT_HEAD_TILE][2];
#pragma unroll
            for (int i = 0; i < AT_HEAD_TILE; ++i) acc[i][0] = acc[i][1] = 0.f;
            for (int c = 0; c < cnt; ++c) {
                const uint32_t kvv = *reinterpret_cast<const uint32_t*>(kv_s + c * WP + 2 * j2);
                const float v0 = bf16_lo(kvv), v1 = bf16_hi(kvv);
#pragma unroll
                for (int i = 0; i < AT_HEAD_TILE; ++i) {
                    if (i < hn) {
                        const float p = p_s[(h0 + i) * AT_CHUNK + c];
                        acc[i][0] = fmaf(p, v0, acc[i][0]);
                        acc[i][1] = fmaf(p, v1, acc[i][1]);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < AT_HEAD_TILE; ++i)
                if (i < hn) *reinterpret_cast<float2*>(part_o + (obase + h0 + i) * L + 2 * j2) = make_float2(acc[i][0], acc[i][1]);
        }
    }
    for (int i = threadIdx.x; i < 2 * H; i += AT_THREADS) part_ml[obase * 2 + i] = ml_s[i];
}

// grid (H, rows).  world == 1: o_lat[r][h] = bf16(o / l).  world > 1: push (o[L], m, l) to head owner.
__global__ void __launch_bounds__(128)
attn_local_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const int* __restrict__ sel_counts,
                        int H, int L, int top_k, int max_chunks, bf16* __restrict__ o_lat, int heads_local,
                        int64_t xpart_offset, PeerComm comm, int sig) {
    const int h = blockIdx.x, r = blockIdx.y;
    const int count = min(max(sel_counts[2 * r + 1], 0), top_k);
    const int chunks = (count + AT_CHUNK - 1) / AT_CHUNK;
    float M = -INFINITY;
    for (int c = 0; c < chunks; ++c) M = fmaxf(M, part_ml[(((int64_t)r * max_chunks + c) * H + h) * 2]);
    float l = 0.f;
    for (int c = 0; c < chunks; ++c) {
        const float* ml = part_ml + (((int64_t)r * max_chunks + c) * H + h) * 2;
        l += ml[1] * expf(ml[0] - M);
    }
    const int rows = gridDim.y;
    for (int j = threadIdx.x; j < L; j += blockDim.x) {
        float o = 0.f;
        for (int c = 0; c < chunks; ++c) {
            const int64_t at = ((int64_t)r * max_chunks + c) * H + h;
            o = fmaf(part_o[at * L + j], expf(part_ml[at * 2] - M), o);
        }
        if (comm.world == 1) {
            o_lat[((int64_t)r * H + h) * L + j] = __float2bfloat16_rn(chunks > 0 ? o / l : 0.f);
        } else {
            const int dst = h / heads_local, hl = h % heads_local;
            float* box = reinterpret_cast<float*>(comm.data[dst] + xpart_offset) +
                         (((int64_t)comm.rank * rows + r) * heads_local + hl) * (L + 2);
            box[j] = o;
            if (j == 0) { box[L] = chunks > 0 ? M : -INFINITY; box[L + 1] = chunks > 0 ? l : 0.f; }
        }
    }
    grid_signal_peers(comm, sig);
}

// grid (heads_local, rows): merge the `world` partials of this rank's heads in rank order.
__global__ void __launch_bounds__(128)
attn_final_merge_kernel(int L, int heads_local, int64_t xpart_offset, bf16* __restrict__ o_lat, PeerComm comm, int sig) {
    cta_wait_signal(comm, sig);
    const int hl = blockIdx.x, r = blockIdx.y, rows = gridDim.y;
    const float* base = reinterpret_cast<const float*>(comm.data[comm.rank] + xpart_offset);
    float M = -INFINITY;
    for (int p = 0; p < comm.world; ++p) M = fmaxf(M, ld_sys_f32(base + (((int64_t)p * rows + r) * heads_local + hl) * (L + 2) + L));
    float l = 0.f;
    float wgt[GLMB_MAX_WORLD];
    for (int p = 0; p < comm.world; ++p) {
        const float* box = base + (((int64_t)p * rows + r) * heads_local + hl) * (L + 2);
        const float m = ld_sys_f32(box + L);
        wgt[p] = (m == -INFINITY) ? 0.f : expf(m - M);
        l += ld_sys_f32(box + L + 1) * wgt[p];
    }
    for (int j = threadIdx.x; j < L; j += blockDim.x) {
        float o = 0.f;
        for (int p = 0; p < comm.world; ++p)
            o = fmaf(ld_sys_f32(base + (((int64_t)p * rows + r) * heads_local + hl) * (L + 2) + j), wgt[p], o);
        o_lat[((int64_t)r * heads_local + hl) * L + j] = __float2bfloat16_rn(l > 0.f ? o / l : 0.f);
    }
}

// ===================================================================================================
GLMB_API int glmb_attn_chunk(void) { return AT_CHUNK; }

GLMB_API int glmb_sparse_mla_partial(const void* q_full, const void* kv_cache, const int* sel_local, const int* sel_counts,
                                     const int* row_lane, int rows, int H, int L, int rd, int layer, int layers, int local_cap,
                                     int top_k, int max_chunks, float scale, float* part_o, float* part_ml, const PeerComm* comm,
                                     int wait_sig, uint32_t* status, void* stream) {
    if (((L + rd) & 7) || (L & 1)) return 1;
    PeerComm c;
    if (comm) c = *comm; else { memset(&c, 0, sizeof(c)); c.world = 1; }
    const size_t smem = (size_t)AT_CHUNK * (L + rd + 8) * 2 + (size_t)H * AT_CHUNK * 4 + (size_t)H * 2 * 4;
    static bool attr_set = false;
    if (!attr_set) {
        cudaFuncSetAttribute(sparse_mla_partial_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
        attr_set = true;
    }
    if (smem > 100 * 1024) return 2;
    dim3 grid(max_chunks, rows);
    sparse_mla_partial_kernel<<<grid, AT_THREADS, smem, (cudaStream_t)stream>>>(
        (const bf16*)q_full, (const bf16*)kv_cache, sel_local, sel_counts, row_lane, H, L, rd, layer, layers, local_cap, top_k,
        max_chunks, scale, part_o, part_ml, c, wait_sig, status);
    return (int)cudaGetLastError();
}

GLMB_API int glmb_attn_local_merge(const float* part_o, const float* part_ml, const int* sel_counts, int rows, int H, int L,
                                   int top_k, int max_chunks, void* o_lat, int heads_local, int64_t xpart_offset,
                                   const PeerComm* comm, int sig, void* stream) {
    PeerComm c;
    if (comm) c = *comm; else { memset(&c, 0, sizeof(c)); c.world = 1; }
    dim3 grid(H, rows);
    attn_local_merge_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(part_o, part_ml, sel_counts, H, L, top_k, max_chunks,
                                                                    (bf16*)o_lat, heads_local, xpart_offset, c, sig);
    return (int)cudaGetLastError();
}

GLMB_API int glmb_attn_final_merge(int rows, int L, int heads_local, int64_t xpart_offset, void* o_lat, const PeerComm* comm,
                                   int sig, void* stream) {
    if (!comm || comm->world < 2) return 1;
    dim3 grid(heads_local, rows);
    attn_final_merge_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(L, heads_local, xpart_offset, (bf16*)o_lat, *comm, sig);
    return (int)cudaGetLastError();
}
