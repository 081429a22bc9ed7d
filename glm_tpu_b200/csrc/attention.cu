// DeepSeek-sparse absorbed-MLA attention over the position-striped cache.
//
// Each GPU holds 1/world of the cached rows.  For a query row the selection kernel has already listed
// which of the top-k positions live on this GPU (ascending).  Attention runs owner-locally:
//
//   sparse_mla_partial   one CTA per (chunk of 64 owned selected rows, query row, block of 16 heads): gathers
//                        the rows and the absorbed queries into shared memory, computes S = Q K^T on the
//                        tensor cores (bf16 in, fp32 out), the chunk-local softmax statistics in fp32, rounds
//                        P to bf16 and computes the unnormalized P . latent product on the tensor cores
//   attn_local_merge     merges a row's chunks per head (log-sum-exp algebra).  With one GPU it normalizes
//                        and stores bf16.  With several it pushes (o, m, l) of head h straight into the
//                        buffer of the GPU that owns head h (tensor-parallel by heads) and signals.
//   attn_final_merge     the head owner waits for the signal, merges the `world` partials in rank order,
//                        normalizes and stores bf16.
//
// The per-row problem is 64 heads x <=2048 gathered keys x 576: far too small and too irregular (every query
// row has its own key set) to fill a 128-row tcgen05 tile, and it is bound by the gather latency, so the
// contraction uses warp-level mma.sync m16n8k16 with ldmatrix-fed fragments; the large dense and grouped
// GEMMs of the model are the tcgen05 kernels.
//
// The 2.6 MB selected-row all-reduce of the reference (`glm_tpu/layers/attention/mla.py:484-485`) becomes an
// exchange of heads x (latent + 2) fp32 per row.  Numerics restate `kernels/sparse_mla/kernel.py:128-183`
// (fp32 scores, bf16 P before P.V, one final normalisation, empty row -> zeros) and the owner-local
// partial/LSE-merge of `kernels/sparse_mla/partial_kernel.py:45-78`, `layers/attention/mla.py:288-376`.
#include "common.cuh"
#include "attention_core.cuh"
#include "gemv_core.cuh"
#include "peer.cuh"

// One CTA: one tile of attention_core.cuh (16 heads x 64 gathered keys).
template <int TPW, int PVW>
__global__ void __launch_bounds__(AT_THREADS)
sparse_mla_partial_kernel(const bf16* __restrict__ q_full, const bf16* __restrict__ kv_cache, const int* __restrict__ sel_local,
                          const int* __restrict__ sel_counts, const int* __restrict__ row_lane, int H, int rd, int layer,
                          int layers, int local_cap, int top_k, int max_chunks, float scale, float* __restrict__ part_o,
                          float* __restrict__ part_ml, PeerComm comm, int wait_sig, uint32_t* status) {
    GLMB_PDL_PROLOGUE();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    if (wait_sig >= 0) cta_wait_signal(comm, wait_sig);
    sparse_mla_partial_tile<TPW, PVW>(q_full, kv_cache, sel_local, sel_counts, row_lane, H, rd, layer, layers, local_cap, top_k, max_chunks,
                                      scale, part_o, part_ml, status, blockIdx.y, blockIdx.x, blockIdx.z * AT_HEADS, smem_raw);
}

// ---------------------------------------------------------------------------------------------------
// Many query rows (prefill) on one GPU's cache: one CTA per (query row, block of 16 heads) walks ALL of the row's
// selected keys in chunks of 64 with a running (max, sum) per head and rescaled accumulators, normalizes at the
// end and stores bf16 directly.  Nothing is written per chunk, so the [rows, chunks, heads, latent] fp32 partials
// of the split kernels (the bulk of their memory traffic when there are thousands of rows) and the merge kernel
// disappear.  Decode keeps the split kernels: with 1-8 rows the chunks are the parallelism.
template <int TPW, int PVW>
__global__ void __launch_bounds__(AT_THREADS)
sparse_mla_rows_kernel(const bf16* __restrict__ q_full, const bf16* __restrict__ kv_cache, const int* __restrict__ sel_local,
                       const int* __restrict__ sel_counts, const int* __restrict__ row_lane, int H, int rd, int layer, int layers,
                       int local_cap, int top_k, float scale, bf16* __restrict__ o_lat, uint32_t* status) {
    GLMB_PDL_PROLOGUE();
    constexpr int L = 8 * TPW * PVW;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int W = L + rd;
    const int WP = W + 8;
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);
    bf16* kv_s = q_s + AT_HEADS * WP;
    bf16* p_s = kv_s + AT_CHUNK * WP;
    float* max_s = reinterpret_cast<float*>(p_s + AT_HEADS * AT_PSTRIDE);
    float* sum_s = max_s + AT_WARPS * AT_HEADS;
    __shared__ int row_s[AT_CHUNK];
    const int r = blockIdx.x, h_base = blockIdx.y * AT_HEADS;
    const int count = min(max(sel_counts[2 * r + 1], 0), top_k);
    const bf16* cache = kv_cache + ((int64_t)row_lane[r] * layers + layer) * (int64_t)local_cap * W;
    const int vec_per_row = W / 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3, mi = lane >> 3, mr = lane & 7;
    const int h0 = h_base + g, h1 = h0 + 8;

    const bf16* q = q_full + (int64_t)r * H * W;
    for (int i = threadIdx.x; i < AT_HEADS * vec_per_row; i += AT_THREADS) {
        const int h = i / vec_per_row, v = i % vec_per_row;
        bf16* dst = q_s + h * WP + v * 8;
        if (h_base + h < H) cp_async16(dst, q + (int64_t)(h_base + h) * W + v * 8);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o_acc[TPW][4];
#pragma unroll
    for (int j = 0; j < TPW; ++j) o_acc[j][0] = o_acc[j][1] = o_acc[j][2] = o_acc[j][3] = 0.f;

    for (int start = 0; start < count; start += AT_CHUNK) {
        const int cnt = min(AT_CHUNK, count - start);
        if (threadIdx.x < AT_CHUNK) {
            int row = -1;
            if ((int)threadIdx.x < cnt) {
                row = sel_local[(int64_t)r * top_k + start + threadIdx.x];
                if (row < 0 || row >= local_cap) { raise_status(status, GLMB_STATUS_BAD_INDEX); row = min(max(row, 0), local_cap - 1); }
            }
            row_s[threadIdx.x] = row;
        }
        __syncthreads();  // also: every warp has finished reading kv_s / p_s of the previous chunk
        // a warp per key row, lanes across its 16-byte pieces: no division by the (runtime) row width in the copy loop
        for (int c = warp; c < AT_CHUNK; c += AT_WARPS) {
            const int row = row_s[c];
            bf16* dst = kv_s + c * WP;
            const bf16* src = cache + (int64_t)max(row, 0) * W;
            for (int v = lane; v < vec_per_row; v += 32) {
                if (row >= 0) cp_async16(dst + v * 8, src + v * 8);
                else *reinterpret_cast<uint4*>(dst + v * 8) = make_uint4(0, 0, 0, 0);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();

        float s_acc[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const bf16* a_base = q_s + (mr + 8 * (mi & 1)) * WP + 8 * (mi >> 1);
            const bf16* b_base = kv_s + (warp * 8 + mr) * WP + 8 * (mi & 1);
            for (int k0 = 0; k0 < W; k0 += 16) {
                uint32_t a[4], b[2];
                ldmatrix_x4(a, a_base + k0);
                ldmatrix_x2(b, b_base + k0);
                mma_bf16_16816(s_acc, a, b[0], b[1]);
            }
        }
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int c = warp * 8 + 2 * t + (e & 1);
            float s = __fmul_rn(s_acc[e], scale);
            if (c >= cnt) s = -INFINITY;
            else if (!isfinite(s)) raise_status(status, GLMB_STATUS_NONFINITE);
            s_acc[e] = s;
            mx[e >> 1] = fmaxf(mx[e >> 1], s);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
        }
        if (t == 0) { max_s[warp * AT_HEADS + g] = mx[0]; max_s[warp * AT_HEADS + g + 8] = mx[1]; }
        __syncthreads();
        float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int w2 = 0; w2 < AT_WARPS; ++w2) {
            m_new[0] = fmaxf(m_new[0], max_s[w2 * AT_HEADS + g]);
            m_new[1] = fmaxf(m_new[1], max_s[w2 * AT_HEADS + g + 8]);
        }
        float ls[2] = {0.f, 0.f};
        {
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                p[e] = s_acc[e] == -INFINITY ? 0.f : expf(s_acc[e] - m_new[e >> 1]);
                ls[e >> 1] += p[e];
            }
            const int c = warp * 8 + 2 * t;
            *reinterpret_cast<uint32_t*>(p_s + g * AT_PSTRIDE + c) = pack_bf16(p[0], p[1]);
            *reinterpret_cast<uint32_t*>(p_s + (g + 8) * AT_PSTRIDE + c) = pack_bf16(p[2], p[3]);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            ls[i] += __shfl_xor_sync(0xffffffffu, ls[i], 1);
            ls[i] += __shfl_xor_sync(0xffffffffu, ls[i], 2);
        }
        if (t == 0) { sum_s[warp * AT_HEADS + g] = ls[0]; sum_s[warp * AT_HEADS + g + 8] = ls[1]; }
        __syncthreads();
        // running statistics (every thread keeps the pair of its heads g and g + 8) and accumulator rescale
        float alpha[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            float chunk_sum = 0.f;
#pragma unroll
            for (int w2 = 0; w2 < AT_WARPS; ++w2) chunk_sum += sum_s[w2 * AT_HEADS + g + 8 * i];
            alpha[i] = m_run[i] == -INFINITY ? 0.f : expf(m_run[i] - m_new[i]);
            l_run[i] = l_run[i] * alpha[i] + chunk_sum;
            m_run[i] = m_new[i];
        }
        if (warp < PVW) {
#pragma unroll
            for (int j = 0; j < TPW; ++j) { o_acc[j][0] *= alpha[0]; o_acc[j][1] *= alpha[0]; o_acc[j][2] *= alpha[1]; o_acc[j][3] *= alpha[1]; }
            const bf16* pa_base = p_s + (mr + 8 * (mi & 1)) * AT_PSTRIDE + 8 * (mi >> 1);
            const bf16* vb_base = kv_s + (mr + 8 * (mi & 1)) * WP + warp * (8 * TPW) + 8 * (mi >> 1);
#pragma unroll
            for (int kk = 0; kk < AT_CHUNK; kk += 16) {
                uint32_t a[4];
                ldmatrix_x4(a, pa_base + kk);
#pragma unroll
                for (int jn = 0; jn < TPW; jn += 2) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, vb_base + kk * WP + jn * 8);
                    mma_bf16_16816(o_acc[jn], a, b[0], b[1]);
                    mma_bf16_16816(o_acc[jn + 1], a, b[2], b[3]);
                }
            }
        }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");  // an empty row never waited for its query copies
    if (warp < PVW) {
        // an empty row (no selected key) gives zeros
#pragma unroll
        for (int jn = 0; jn < TPW; ++jn) {
            const int col = warp * (8 * TPW) + jn * 8 + 2 * t;
            if (h0 < H)
                *reinterpret_cast<uint32_t*>(o_lat + ((int64_t)r * H + h0) * L + col) =
                    count > 0 ? pack_bf16(o_acc[jn][0] / l_run[0], o_acc[jn][1] / l_run[0]) : 0u;
            if (h1 < H)
                *reinterpret_cast<uint32_t*>(o_lat + ((int64_t)r * H + h1) * L + col) =
                    count > 0 ? pack_bf16(o_acc[jn][2] / l_run[1], o_acc[jn][3] / l_run[1]) : 0u;
        }
    }
}

// grid (H, rows).  world == 1: o_lat[r][h] = bf16(o / l).  world > 1: push (o[L], m, l) to head owner.
// The chunk statistics are fetched by one thread per chunk and the partial rows by float4 loads issued eight
// chunks at a time, so the kernel costs a few memory round trips however many chunks a row has.
#define AM_MAX_CHUNKS 128
__global__ void __launch_bounds__(128)
attn_local_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const int* __restrict__ sel_counts,
                        int H, int L, int top_k, int max_chunks, bf16* __restrict__ o_lat, int heads_local,
                        int64_t xpart_offset, PeerComm comm, int sig) {
    GLMB_PDL_PROLOGUE();
    __shared__ float w_s[AM_MAX_CHUNKS];
    __shared__ float red_s[8];
    const int h = blockIdx.x, r = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int count = min(max(sel_counts[2 * r + 1], 0), top_k);
    const int chunks = min((count + AT_CHUNK - 1) / AT_CHUNK, AM_MAX_CHUNKS);
    const int64_t base = (int64_t)r * max_chunks * H + h;  // chunk c of this (row, head) is at base + c * H
    // every thread owns at most one chunk's statistics (chunks <= 128 == blockDim.x)
    float my_m = -INFINITY, my_l = 0.f;
    if ((int)threadIdx.x < chunks) {
        const float2 ml = *reinterpret_cast<const float2*>(part_ml + (base + (int64_t)threadIdx.x * H) * 2);
        my_m = ml.x; my_l = ml.y;
    }
    float M = my_m;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    if (lane == 0) red_s[warp] = M;
    __syncthreads();
    M = fmaxf(fmaxf(red_s[0], red_s[1]), fmaxf(red_s[2], red_s[3]));
    const float my_w = (int)threadIdx.x < chunks ? expf(my_m - M) : 0.f;
    w_s[threadIdx.x] = my_w;
    float l = my_l * my_w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) red_s[4 + warp] = l;
    __syncthreads();
    l = (red_s[4] + red_s[5]) + (red_s[6] + red_s[7]);
    const int rows = gridDim.y;
    for (int j = threadIdx.x * 4; j < L; j += blockDim.x * 4) {
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int c0 = 0; c0 < chunks; c0 += 8) {
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                v[u] = c0 + u < chunks ? *reinterpret_cast<const float4*>(part_o + (base + (int64_t)(c0 + u) * H) * L + j)
                                       : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float wgt = c0 + u < chunks ? w_s[c0 + u] : 0.f;
                o.x = fmaf(v[u].x, wgt, o.x); o.y = fmaf(v[u].y, wgt, o.y);
                o.z = fmaf(v[u].z, wgt, o.z); o.w = fmaf(v[u].w, wgt, o.w);
            }
        }
        if (comm.world == 1) {
            uint2 packed;
            if (chunks > 0) { o.x /= l; o.y /= l; o.z /= l; o.w /= l; }  // the contract divides (no reciprocal)
            packed.x = pack_bf16(o.x, o.y);
            packed.y = pack_bf16(o.z, o.w);
            *reinterpret_cast<uint2*>(o_lat + ((int64_t)r * H + h) * L + j) = packed;
        } else {
            const int dst = h / heads_local, hl = h % heads_local;
            float* box = reinterpret_cast<float*>(comm.data[dst] + xpart_offset) +
                         (((int64_t)comm.rank * rows + r) * heads_local + hl) * (L + 2);
            box[j] = o.x; box[j + 1] = o.y; box[j + 2] = o.z; box[j + 3] = o.w;  // L + 2 floats per box: 8-byte aligned only
            if (j == 0) { box[L] = chunks > 0 ? M : -INFINITY; box[L + 1] = chunks > 0 ? l : 0.f; }
        }
    }
    grid_signal_peers(comm, sig);
}

// grid (heads_local, rows): merge the `world` partials of this rank's heads in rank order.
__global__ void __launch_bounds__(128)
attn_final_merge_kernel(int L, int heads_local, int64_t xpart_offset, bf16* __restrict__ o_lat, PeerComm comm, int sig) {
    GLMB_PDL_PROLOGUE();
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

template <int TPW, int PVW>
static int launch_partial(const void* q_full, const void* kv_cache, const int* sel_local, const int* sel_counts, const int* row_lane,
                          int rows, int H, int rd, int layer, int layers, int local_cap, int top_k, int max_chunks, float scale,
                          float* part_o, float* part_ml, const PeerComm& c, int wait_sig, uint32_t* status, cudaStream_t stream) {
    const int W = 8 * TPW * PVW + rd;
    const size_t smem = sparse_mla_tile_smem(W);
    if (smem > 200 * 1024) return 2;
    static DeviceOnce attr_set;
    const int attr_set_dev = attr_set.pending();
    if (attr_set_dev != DeviceOnce::SET) {
        cudaError_t e = cudaFuncSetAttribute(sparse_mla_partial_kernel<TPW, PVW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
        attr_set.mark(attr_set_dev);
    }
    dim3 grid(max_chunks, rows, (H + AT_HEADS - 1) / AT_HEADS);
    GLMB_LAUNCH((sparse_mla_partial_kernel<TPW, PVW>), grid, AT_THREADS, smem, stream, (const bf16*)q_full, (const bf16*)kv_cache, sel_local,
                                                                           sel_counts, row_lane, H, rd, layer, layers, local_cap,
                                                                           top_k, max_chunks, scale, part_o, part_ml, c, wait_sig,
                                                                           status);
    return (int)cudaGetLastError();
}

// L in {64, 128, 512}; (L + rd) % 16 == 0.
GLMB_API int glmb_sparse_mla_partial(const void* q_full, const void* kv_cache, const int* sel_local, const int* sel_counts,
                                     const int* row_lane, int rows, int H, int L, int rd, int layer, int layers, int local_cap,
                                     int top_k, int max_chunks, float scale, float* part_o, float* part_ml, const PeerComm* comm,
                                     int wait_sig, uint32_t* status, void* stream) {
    if ((L + rd) & 15) return 1;
    PeerComm c;
    if (comm) c = *comm; else { memset(&c, 0, sizeof(c)); c.world = 1; }
    cudaStream_t st = (cudaStream_t)stream;
#define ARGS q_full, kv_cache, sel_local, sel_counts, row_lane, rows, H, rd, layer, layers, local_cap, top_k, max_chunks, scale, part_o, \
             part_ml, c, wait_sig, status, st
    if (L == 512) return launch_partial<8, 8>(ARGS);
    if (L == 128) return launch_partial<2, 8>(ARGS);
    if (L == 64) return launch_partial<2, 4>(ARGS);
#undef ARGS
    return 1;
}

template <int TPW, int PVW>
static int launch_rows(const void* q_full, const void* kv_cache, const int* sel_local, const int* sel_counts, const int* row_lane, int rows,
                       int H, int rd, int layer, int layers, int local_cap, int top_k, float scale, void* o_lat, uint32_t* status,
                       cudaStream_t stream) {
    const int W = 8 * TPW * PVW + rd;
    const size_t smem = (size_t)(AT_HEADS + AT_CHUNK) * (W + 8) * 2 + (size_t)AT_HEADS * AT_PSTRIDE * 2 + 2 * AT_WARPS * AT_HEADS * 4;
    if (smem > 200 * 1024) return 2;
    static DeviceOnce attr_set;
    const int attr_set_dev = attr_set.pending();
    if (attr_set_dev != DeviceOnce::SET) {
        cudaError_t e = cudaFuncSetAttribute(sparse_mla_rows_kernel<TPW, PVW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
        attr_set.mark(attr_set_dev);
    }
    dim3 grid(rows, (H + AT_HEADS - 1) / AT_HEADS);
    GLMB_LAUNCH((sparse_mla_rows_kernel<TPW, PVW>), grid, AT_THREADS, smem, stream, (const bf16*)q_full, (const bf16*)kv_cache, sel_local, sel_counts,
                row_lane, H, rd, layer, layers, local_cap, top_k, scale, (bf16*)o_lat, status);
    return (int)cudaGetLastError();
}

// o_lat[rows, H, L] (bf16, normalized) for any number of rows: every selected key of a row lives in this GPU's cache
// (single GPU, or a replicated cache).  L in {64, 128, 512}; (L + rd) % 16 == 0.
GLMB_API int glmb_sparse_mla_rows(const void* q_full, const void* kv_cache, const int* sel_local, const int* sel_counts, const int* row_lane,
                                  int rows, int H, int L, int rd, int layer, int layers, int local_cap, int top_k, float scale, void* o_lat,
                                  uint32_t* status, void* stream) {
    if (((L + rd) & 15) || rows < 1) return 1;
    cudaStream_t st = (cudaStream_t)stream;
#define ARGS q_full, kv_cache, sel_local, sel_counts, row_lane, rows, H, rd, layer, layers, local_cap, top_k, scale, o_lat, status, st
    if (L == 512) return launch_rows<8, 8>(ARGS);
    if (L == 128) return launch_rows<2, 8>(ARGS);
    if (L == 64) return launch_rows<2, 4>(ARGS);
#undef ARGS
    return 1;
}

GLMB_API int glmb_attn_local_merge(const float* part_o, const float* part_ml, const int* sel_counts, int rows, int H, int L,
                                   int top_k, int max_chunks, void* o_lat, int heads_local, int64_t xpart_offset,
                                   const PeerComm* comm, int sig, void* stream) {
    if ((L & 3) || max_chunks > AM_MAX_CHUNKS) return 1;
    PeerComm c;
    if (comm) c = *comm; else { memset(&c, 0, sizeof(c)); c.world = 1; }
    dim3 grid(H, rows);
    GLMB_LAUNCH(attn_local_merge_kernel, grid, 128, 0, (cudaStream_t)stream, part_o, part_ml, sel_counts, H, L, top_k, max_chunks,
                                                                    (bf16*)o_lat, heads_local, xpart_offset, c, sig);
    return (int)cudaGetLastError();
}

// Decode with every key local: the merge of a (row, head)'s chunk partials AND that head's value projection in one launch.
//   o_lat[r][h] = bf16(sum_c w_c o_c / l)   exactly as attn_local_merge_kernel (same thread-to-column map, same order over chunks)
//   attn_v[r][h * N + n] = bf16(o_lat[r][h] . w_v[h][n])   exactly as skinny_bf16_kernel with one K part (same lane-to-k map, xor tree)
// grid (H, rows, N / cols): a (row, head) is merged redundantly by the N / cols CTAs that share its value projection (64 KB of
// L2-resident partials each) so that the 256 KB of a head's value table are streamed by several SMs instead of 1 (8 when a GPU holds 8
// heads of one row; fewer slices when rows x heads alone fill the machine, where the repeated merges would only cost); every chunk row a thread
// needs is requested before the first is used, and the CTA's slice of the value table is asked into L2 before the wait for the
// attention kernel.  One launch and ~3 memory round trips where merge + projection took two launches and ~8.
#define MV_THREADS 256
#define MV_MIN_COLS 32
#define MV_BATCH 16
__global__ void __launch_bounds__(MV_THREADS)
attn_merge_vproj_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const int* __restrict__ sel_counts, int H, int L,
                        int top_k, int max_chunks, const bf16* __restrict__ w_v, int64_t w_head_stride, int N, int cols,
                        bf16* __restrict__ o_lat, bf16* __restrict__ attn_v) {
    asm volatile("griddepcontrol.launch_dependents;");
    const int h = blockIdx.x, r = blockIdx.y, n_base = blockIdx.z * cols;
    const int n_here = min(cols, N - n_base);
    const bf16* w_head = w_v + (int64_t)h * w_head_stride;
    if (threadIdx.x == 0) {
        const char* p = reinterpret_cast<const char*>(w_head + (int64_t)n_base * L);
        const uint32_t bytes = (uint32_t)(((int64_t)n_here * L * 2) & ~(int64_t)15);
        if (bytes && !((uintptr_t)p & 15)) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float w_s[AM_MAX_CHUNKS];
    __shared__ float red_s[8];
    __shared__ __align__(16) bf16 o_s[512];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int count = min(max(sel_counts[2 * r + 1], 0), top_k);
    const int chunks = min((count + AT_CHUNK - 1) / AT_CHUNK, AM_MAX_CHUNKS);
    const int64_t base = (int64_t)r * max_chunks * H + h;
    // ---- merge: the first 128 threads are the 128 threads of attn_local_merge_kernel
    float my_m = -INFINITY, my_l = 0.f;
    if ((int)threadIdx.x < chunks) {
        const float2 ml = *reinterpret_cast<const float2*>(part_ml + (base + (int64_t)threadIdx.x * H) * 2);
        my_m = ml.x; my_l = ml.y;
    }
    float M = my_m;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    if (lane == 0 && warp < 4) red_s[warp] = M;
    __syncthreads();
    M = fmaxf(fmaxf(red_s[0], red_s[1]), fmaxf(red_s[2], red_s[3]));
    const float my_w = (int)threadIdx.x < chunks ? expf(my_m - M) : 0.f;
    if (threadIdx.x < AM_MAX_CHUNKS) w_s[threadIdx.x] = my_w;
    float l = my_l * my_w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0 && warp < 4) red_s[4 + warp] = l;
    __syncthreads();
    l = (red_s[4] + red_s[5]) + (red_s[6] + red_s[7]);
    if (threadIdx.x < 128) {
        for (int j = threadIdx.x * 4; j < L; j += 128 * 4) {
            float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int c0 = 0; c0 < chunks; c0 += MV_BATCH) {
                float4 v[MV_BATCH];
#pragma unroll
                for (int u = 0; u < MV_BATCH; ++u)
                    v[u] = c0 + u < chunks ? *reinterpret_cast<const float4*>(part_o + (base + (int64_t)(c0 + u) * H) * L + j)
                                           : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int u = 0; u < MV_BATCH; ++u) {
                    const float wgt = c0 + u < chunks ? w_s[c0 + u] : 0.f;
                    o.x = fmaf(v[u].x, wgt, o.x); o.y = fmaf(v[u].y, wgt, o.y);
                    o.z = fmaf(v[u].z, wgt, o.z); o.w = fmaf(v[u].w, wgt, o.w);
                }
            }
            if (chunks > 0) { o.x /= l; o.y /= l; o.z /= l; o.w /= l; }  // the contract divides (no reciprocal)
            uint2 packed;
            packed.x = pack_bf16(o.x, o.y);
            packed.y = pack_bf16(o.z, o.w);
            *reinterpret_cast<uint2*>(o_s + j) = packed;
            if (o_lat && blockIdx.z == 0) *reinterpret_cast<uint2*>(o_lat + ((int64_t)r * H + h) * L + j) = packed;
        }
    }
    __syncthreads();
    // ---- value projection of this CTA's columns: a warp per pair of output columns over the whole K = L
    const bf16* const xr[1] = {o_s};
    for (int pair = warp; pair * 2 < n_here; pair += MV_THREADS / 32) {
        const int n0 = n_base + pair * 2;
        const bf16* const wp[2] = {w_head + (int64_t)n0 * L, w_head + (int64_t)min(n0 + 1, N - 1) * L};
        float acc[2][1] = {{0.f}, {0.f}};
        warp_dot_bf16<1, 2>(xr, wp, 0, L, lane, acc);
        warp_reduce_all<1, 2>(acc);
        if (lane == 0) {
            bf16* dst = attn_v + ((int64_t)r * H + h) * N + n0;
            dst[0] = __float2bfloat16_rn(acc[0][0]);
            if (n0 + 1 < N) dst[1] = __float2bfloat16_rn(acc[1][0]);
        }
    }
}

// w_v: the value rows of head 0 ([N, L] bf16, rows L apart); the next head's start w_head_stride elements later.
GLMB_API int glmb_attn_merge_vproj(const float* part_o, const float* part_ml, const int* sel_counts, int rows, int H, int L, int top_k,
                                   int max_chunks, const void* w_v, int64_t w_head_stride, int N, void* o_lat, void* attn_v, void* stream) {
    if ((L & 7) || L > 512 || max_chunks > AM_MAX_CHUNKS || N < 1 || rows < 1 || H < 1 || (w_head_stride & 7)) return 1;
    // slices of the value columns per (row, head): enough CTAs for two per SM, never narrower than MV_MIN_COLS columns
    int slices = 1;
    while (slices * 2 * MV_MIN_COLS <= N && (long)H * rows * slices < 2 * 148) slices *= 2;
    const int cols = ((N + slices - 1) / slices + 1) & ~1;
    dim3 grid(H, rows, (N + cols - 1) / cols);
    GLMB_LAUNCH(attn_merge_vproj_kernel, grid, MV_THREADS, 0, (cudaStream_t)stream, part_o, part_ml, sel_counts, H, L, top_k, max_chunks,
                (const bf16*)w_v, w_head_stride, N, cols, (bf16*)o_lat, (bf16*)attn_v);
    return (int)cudaGetLastError();
}

GLMB_API int glmb_attn_final_merge(int rows, int L, int heads_local, int64_t xpart_offset, void* o_lat, const PeerComm* comm,
                                   int sig, void* stream) {
    if (!comm || comm->world < 2) return 1;
    dim3 grid(heads_local, rows);
    GLMB_LAUNCH(attn_final_merge_kernel, grid, 128, 0, (cudaStream_t)stream, L, heads_local, xpart_offset, (bf16*)o_lat, *comm, sig);
    return (int)cudaGetLastError();
}
