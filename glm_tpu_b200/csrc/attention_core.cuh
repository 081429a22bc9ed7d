// The absorbed-MLA attention tile of the decode step (16 heads x 64 gathered keys on mma.sync), shared by the stand-alone
// kernels (attention.cu) and the persistent decode kernel (decode_mega.cu).
#pragma once

#include "common.cuh"

#define AT_CHUNK 64
#define AT_THREADS 256
#define AT_WARPS 8
#define AT_HEADS 16   // heads per CTA (one m16 tile)
#define AT_PSTRIDE 72 // bf16 elements per P row (64 + 8 padding)

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_ptr) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], const void* smem_ptr) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_ptr) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Dynamic shared memory one tile needs for a row of W = L + rd bf16 values.
static inline size_t sparse_mla_tile_smem(int W) {
    return (size_t)(AT_HEADS + AT_CHUNK) * (W + 8) * 2 + (size_t)AT_HEADS * AT_PSTRIDE * 2 + 2 * AT_WARPS * AT_HEADS * 4 + AT_CHUNK * 4;
}

// One tile: query row r, chunk `chunk` of its selected keys, heads h_base .. h_base + 15; every thread of a 256-thread
// CTA calls it with the same arguments.  smem_raw: sparse_mla_tile_smem(W) bytes, 16-byte aligned.
// part_o  [rows, max_chunks, H, L] fp32 (unnormalized, relative to the chunk max)
// part_ml [rows, max_chunks, H, 2] fp32 (max, sum)
// Scores: warp w owns keys 8w..8w+7.  P.V: PVW warps each own TPW 8-column tiles of the latent (L == 8 * TPW * PVW).
template <int TPW, int PVW>
__device__ __forceinline__ void sparse_mla_partial_tile(const bf16* __restrict__ q_full, const bf16* __restrict__ kv_cache,
                                                        const int* __restrict__ sel_local, const int* __restrict__ sel_counts,
                                                        const int* __restrict__ row_lane, int H, int rd, int layer, int layers,
                                                        int local_cap, int top_k, int max_chunks, float scale,
                                                        float* __restrict__ part_o, float* __restrict__ part_ml, uint32_t* status,
                                                        int r, int chunk, int h_base, unsigned char* smem_raw) {
    constexpr int L = 8 * TPW * PVW;
    const int W = L + rd;
    const int WP = W + 8;  // padded row (bf16 elements): 16-byte aligned, staggers the banks for ldmatrix
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);               // [AT_HEADS][WP]
    bf16* kv_s = q_s + AT_HEADS * WP;                            // [AT_CHUNK][WP]
    bf16* p_s = kv_s + AT_CHUNK * WP;                            // [AT_HEADS][AT_PSTRIDE]
    float* max_s = reinterpret_cast<float*>(p_s + AT_HEADS * AT_PSTRIDE);  // [AT_WARPS][AT_HEADS]
    float* sum_s = max_s + AT_WARPS * AT_HEADS;                  // [AT_WARPS][AT_HEADS]
    const int count = min(max(sel_counts[2 * r + 1], 0), top_k);
    const int start = chunk * AT_CHUNK;
    if (start >= count) return;
    const int cnt = min(AT_CHUNK, count - start);
    const bf16* cache = kv_cache + ((int64_t)row_lane[r] * layers + layer) * (int64_t)local_cap * W;
    const int vec_per_row = W / 8;
    // Gather the selected rows (zero-fill the tail of a short chunk) and this CTA's heads of the query.  The row
    // numbers are fetched first, then every 16-byte piece is an asynchronous copy (L2 -> shared memory, no
    // registers, all in flight at once): the gather costs about one memory round trip.
    int* row_s = reinterpret_cast<int*>(sum_s + AT_WARPS * AT_HEADS);                              // [AT_CHUNK]
    if (threadIdx.x < AT_CHUNK) {
        int row = -1;
        if ((int)threadIdx.x < cnt) {
            row = sel_local[(int64_t)r * top_k + start + threadIdx.x];
            if (row < 0 || row >= local_cap) { raise_status(status, GLMB_STATUS_BAD_INDEX); row = min(max(row, 0), local_cap - 1); }
        }
        row_s[threadIdx.x] = row;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < AT_CHUNK * vec_per_row; i += AT_THREADS) {
        const int c = i / vec_per_row, v = i % vec_per_row;
        const int row = row_s[c];
        bf16* dst = kv_s + c * WP + v * 8;
        if (row >= 0) cp_async16(dst, cache + (int64_t)row * W + v * 8);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    const bf16* q = q_full + (int64_t)r * H * W;
    for (int i = threadIdx.x; i < AT_HEADS * vec_per_row; i += AT_THREADS) {
        const int h = i / vec_per_row, v = i % vec_per_row;
        bf16* dst = q_s + h * WP + v * 8;
        if (h_base + h < H) cp_async16(dst, q + (int64_t)(h_base + h) * W + v * 8);  // .cg: read at L2, where peers' pushes land
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3, mi = lane >> 3, mr = lane & 7;

    // ---- S = Q K^T: 16 heads x 8 keys per warp ------------------------------------------------------
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
    // s_acc[e]: head g (e < 2) or g + 8 (e >= 2), key 8*warp + 2t + (e & 1)
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
    float m[2] = {-INFINITY, -INFINITY}, ls[2] = {0.f, 0.f};
#pragma unroll
    for (int w2 = 0; w2 < AT_WARPS; ++w2) {
        m[0] = fmaxf(m[0], max_s[w2 * AT_HEADS + g]);
        m[1] = fmaxf(m[1], max_s[w2 * AT_HEADS + g + 8]);
    }
    {
        float p[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            p[e] = s_acc[e] == -INFINITY ? 0.f : expf(s_acc[e] - m[e >> 1]);
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

    // ---- O = P V: 16 heads x (8 * TPW) latent columns per warp ---------------------------------------
    const int64_t obase = ((int64_t)r * max_chunks + chunk) * H;
    const int h0 = h_base + g, h1 = h0 + 8;
    if (warp < PVW) {
        float o_acc[TPW][4];
#pragma unroll
        for (int j = 0; j < TPW; ++j) o_acc[j][0] = o_acc[j][1] = o_acc[j][2] = o_acc[j][3] = 0.f;
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
#pragma unroll
        for (int jn = 0; jn < TPW; ++jn) {
            const int col = warp * (8 * TPW) + jn * 8 + 2 * t;
            if (h0 < H) *reinterpret_cast<float2*>(part_o + (obase + h0) * L + col) = make_float2(o_acc[jn][0], o_acc[jn][1]);
            if (h1 < H) *reinterpret_cast<float2*>(part_o + (obase + h1) * L + col) = make_float2(o_acc[jn][2], o_acc[jn][3]);
        }
    }
    if (warp == 0 && t == 0) {
        float l0 = 0.f, l1 = 0.f;
#pragma unroll
        for (int w2 = 0; w2 < AT_WARPS; ++w2) { l0 += sum_s[w2 * AT_HEADS + g]; l1 += sum_s[w2 * AT_HEADS + g + 8]; }
        if (h0 < H) { part_ml[(obase + h0) * 2] = m[0]; part_ml[(obase + h0) * 2 + 1] = l0; }
        if (h1 < H) { part_ml[(obase + h1) * 2] = m[1]; part_ml[(obase + h1) * 2 + 1] = l1; }
    }
}

