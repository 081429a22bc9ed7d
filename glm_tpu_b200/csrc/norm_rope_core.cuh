// Row-level pieces of the normalisation / RoPE / query-preparation kernels, shared by the stand-alone kernels
// (norm_rope.cu) and the persistent decode kernel (decode_mega.cu).
#pragma once

#include "common.cuh"
#include "peer.cuh"

__device__ __forceinline__ float block_sum(float v, float* scratch) {
    // scratch: >= 33 floats of shared memory; every thread of the block must call
    v = warp_sum(v);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < (int)((blockDim.x + 31) >> 5) ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}


#define RN_VECS 4
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}

// ---------------------------------------------------------------------------------------------------
struct QkvPostArgs {
    const float* proj;      // [rows, proj_stride]: q_a (Q) | kv_a (L + rd) | idx_k (D) | idx_w (IH)
    int64_t proj_stride;
    const bf16* q_norm_w;   // [Q]
    const bf16* kv_norm_w;  // [L]
    const bf16* rope_table; // [capacity, rd]  cos | sin
    const float* inv_freq;  // [rd/2] fp32, indexer RoPE
    const float* k_norm_w;  // [D] fp32 (indexer key LayerNorm)
    const float* k_norm_b;  // [D]
    const int* row_pos;     // [rows]
    const int* row_lane;    // [rows]
    const int* row_active;  // [rows] or nullptr
    bf16* q_resid;          // [rows, Q]
    bf16* kv_new;           // [rows, L + rd] this step's rows (also attended by peers in prefill tests); may be nullptr
    bf16* kv_cache;         // [lanes, layers, local_cap, L + rd]
    bf16* index_cache;      // [lanes, full_layers, local_cap, D]
    float* head_w;          // [rows, IH]
    bf16* idx_key_new;      // [rows, D] may be nullptr
    int Q, L, rd, D, IH;
    int has_indexer;
    int layer, layers, index_slot, full_layers, local_cap;
    int stripe, world, rank, capacity;
    float eps, key_eps, head_scale;  // head_scale = IH**-0.5 rounded to fp32 by the host
    uint32_t* status;
};


// residual <- bf16(update + residual);  out <- bf16(bf16(residual * rsqrt(mean(residual^2) + eps)) * weight)   for one row.
// Every thread of a 256-thread CTA calls it; every thread owns up to RN_VECS 8-element vectors, all loaded before any arithmetic
// so the row costs one memory round trip.  FRESH: `update` was written earlier by other CTAs of the SAME launch (a kernel tail):
// read it past the L1.
template <bool FRESH>
__device__ __forceinline__ void add_rmsnorm_row(const bf16* update, bf16* residual, const bf16* weight, bf16* out, int H, float eps,
                                                float* scratch) {
    const int nvec = H >> 3;
    uint4 rv[RN_VECS], uv[RN_VECS], wv[RN_VECS];
#pragma unroll
    for (int i = 0; i < RN_VECS; ++i) {
        const int v = threadIdx.x + i * 256;
        if (v < nvec) {
            rv[i] = *reinterpret_cast<const uint4*>(residual + v * 8);
            if (!update) uv[i] = make_uint4(0, 0, 0, 0);
            else if (FRESH) uv[i] = __ldcg(reinterpret_cast<const uint4*>(update + v * 8));
            else uv[i] = *reinterpret_cast<const uint4*>(update + v * 8);
            wv[i] = *reinterpret_cast<const uint4*>(weight + v * 8);
        }
    }
    float s[RN_VECS][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < RN_VECS; ++i) {
        const int v = threadIdx.x + i * 256;
        if (v < nvec) {
            float r8[8], u8[8];
            unpack8(rv[i], r8);
            unpack8(uv[i], u8);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                s[i][e] = update ? __fadd_rn(u8[e], r8[e]) : r8[e];
                ss = fmaf(s[i][e], s[i][e], ss);
            }
        }
    }
    const float total = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(total / (float)H + eps);
#pragma unroll
    for (int i = 0; i < RN_VECS; ++i) {
        const int v = threadIdx.x + i * 256;
        if (v < nvec) {
            float w8[8];
            unpack8(wv[i], w8);
            uint4 o, rr;
            uint32_t* op = reinterpret_cast<uint32_t*>(&o);
            uint32_t* rp = reinterpret_cast<uint32_t*>(&rr);
#pragma unroll
            for (int e = 0; e < 8; e += 2) {
                op[e >> 1] = pack_bf16(bf16_round(s[i][e] * inv) * w8[e], bf16_round(s[i][e + 1] * inv) * w8[e + 1]);
                rp[e >> 1] = pack_bf16(s[i][e], s[i][e + 1]);
            }
            *reinterpret_cast<uint4*>(out + v * 8) = o;
            *reinterpret_cast<uint4*>(residual + v * 8) = rr;
        }
    }
}

// Three block sums with the reduction tree of block_sum (so each is bit-identical to a separate call), one barrier set.
__device__ __forceinline__ void block_sum3(float& a, float& b, float& c, float (*scratch)[40]) {
    a = warp_sum(a); b = warp_sum(b); c = warp_sum(c);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) { scratch[0][warp] = a; scratch[1][warp] = b; scratch[2][warp] = c; }
    __syncthreads();
    if (warp < 3) {
        float t = lane < (int)((blockDim.x + 31) >> 5) ? scratch[warp][lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[warp][32] = t;
    }
    __syncthreads();
    a = scratch[0][32]; b = scratch[1][32]; c = scratch[2][32];
}

// The q_a / kv_a post-processing of one row for Q <= 2048 and L <= 1024 (every supported geometry): all of the
// row's inputs are fetched before the first reduction, the three independent sums share one reduction, and the latent
// is stored four values at a time.  One memory round trip and two reductions.
// Every thread of a 256-thread CTA calls it for row r; scratch and s_key are shared memory.
__device__ __forceinline__ void qkv_a_post_row(const QkvPostArgs& a, int r, float (*scratch)[40], float* s_key) {
    const int tid = threadIdx.x;
    const float* p = a.proj + (int64_t)r * a.proj_stride;
    int pos = a.row_pos[r];
    const int lane_id = a.row_lane[r];
    const bool active = a.row_active ? a.row_active[r] != 0 : true;
    // A position outside the context is reported and the row is computed at a clamped position (no address leaves the
    // tables), but it is NOT stored: bad metadata leaves the caches as they were and the host poisons the engine.
    const bool bad_pos = pos < 0 || pos >= a.capacity;
    if (bad_pos) {
        if (tid == 0) raise_status(a.status, GLMB_STATUS_BAD_INDEX);
        pos = min(max(pos, 0), a.capacity - 1);
    }
    const int page = a.stripe * a.world;
    const bool owner = ((pos / a.stripe) % a.world) == a.rank;
    const int local_row = (pos / page) * a.stripe + pos % a.stripe;
    const int W = a.L + a.rd, half = a.rd / 2;
    bf16* cache_row = a.kv_cache + (((int64_t)lane_id * a.layers + a.layer) * a.local_cap + local_row) * W;
    const bool write_cache = owner && active && !bad_pos;
    const float* c = p + a.Q;
    const float* kx = c + W;

    // ---- every input of the row, before any arithmetic
    float4 qv[2];
    uint2 qw[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int i = tid * 4 + k * 1024;
        qv[k] = i < a.Q ? *reinterpret_cast<const float4*>(p + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        qw[k] = i < a.Q ? *reinterpret_cast<const uint2*>(a.q_norm_w + i) : make_uint2(0, 0);
    }
    const int li = tid * 4;
    const float4 cv = li < a.L ? *reinterpret_cast<const float4*>(c + li) : make_float4(0.f, 0.f, 0.f, 0.f);
    const uint2 cw = li < a.L ? *reinterpret_cast<const uint2*>(a.kv_norm_w + li) : make_uint2(0, 0);
    float r_even = 0.f, r_odd = 0.f, r_cs = 0.f, r_sn = 0.f;
    if (tid < half) {
        r_even = c[a.L + 2 * tid]; r_odd = c[a.L + 2 * tid + 1];
        r_cs = __bfloat162float(a.rope_table[(int64_t)pos * a.rd + tid]);
        r_sn = __bfloat162float(a.rope_table[(int64_t)pos * a.rd + half + tid]);
    }
    float key_v = 0.f, key_w = 0.f, key_b = 0.f, key_f = 0.f, hw_v = 0.f;
    if (a.has_indexer) {
        if (tid < a.D) { key_v = kx[tid]; key_w = a.k_norm_w[tid]; key_b = a.k_norm_b[tid]; }
        if (tid < a.rd) key_f = a.inv_freq[tid >> 1];
        if (tid < a.IH) hw_v = kx[a.D + tid];
    }

    // ---- sums of squares of q_a and of the latent (bf16-rounded inputs), and the indexer key's sum, in one reduction
    float ss = 0.f, ss_kv = 0.f, ksum = key_v;
    float qr[2][4];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        qr[k][0] = bf16_round(qv[k].x); qr[k][1] = bf16_round(qv[k].y); qr[k][2] = bf16_round(qv[k].z); qr[k][3] = bf16_round(qv[k].w);
#pragma unroll
        for (int e = 0; e < 4; ++e) ss = fmaf(qr[k][e], qr[k][e], ss);
    }
    const float cr[4] = {bf16_round(cv.x), bf16_round(cv.y), bf16_round(cv.z), bf16_round(cv.w)};
#pragma unroll
    for (int e = 0; e < 4; ++e) ss_kv = fmaf(cr[e], cr[e], ss_kv);
    block_sum3(ss, ss_kv, ksum, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)a.Q + a.eps);
    const float inv_kv = 1.0f / sqrtf(ss_kv / (float)a.L + a.eps);

    // ---- q_a RMSNorm -> q_resid
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int i = tid * 4 + k * 1024;
        if (i < a.Q) {
            uint2 o;
            o.x = pack_bf16(bf16_round(qr[k][0] * inv) * bf16_lo(qw[k].x), bf16_round(qr[k][1] * inv) * bf16_hi(qw[k].x));
            o.y = pack_bf16(bf16_round(qr[k][2] * inv) * bf16_lo(qw[k].y), bf16_round(qr[k][3] * inv) * bf16_hi(qw[k].y));
            *reinterpret_cast<uint2*>(a.q_resid + (int64_t)r * a.Q + i) = o;
        }
    }
    // ---- kv_a latent RMSNorm -> cache row (and this step's row)
    if (li < a.L) {
        uint2 o;
        o.x = pack_bf16(bf16_round(cr[0] * inv_kv) * bf16_lo(cw.x), bf16_round(cr[1] * inv_kv) * bf16_hi(cw.x));
        o.y = pack_bf16(bf16_round(cr[2] * inv_kv) * bf16_lo(cw.y), bf16_round(cr[3] * inv_kv) * bf16_hi(cw.y));
        if (write_cache) *reinterpret_cast<uint2*>(cache_row + li) = o;
        if (a.kv_new) *reinterpret_cast<uint2*>(a.kv_new + (int64_t)r * W + li) = o;
    }
    // ---- RoPE of the key part: interleaved pairs, bf16 table, fp32 products, one rounding
    if (tid < half) {
        const float even = bf16_round(r_even), odd = bf16_round(r_odd);
        const uint32_t o = pack_bf16(__fsub_rn(__fmul_rn(even, r_cs), __fmul_rn(odd, r_sn)), __fadd_rn(__fmul_rn(odd, r_cs), __fmul_rn(even, r_sn)));
        if (write_cache) *reinterpret_cast<uint32_t*>(cache_row + a.L + 2 * tid) = o;
        if (a.kv_new) *reinterpret_cast<uint32_t*>(a.kv_new + (int64_t)r * W + a.L + 2 * tid) = o;
    }
    if (!a.has_indexer) return;
    // ---- indexer key: affine LayerNorm (fp32), RoPE on the first rd features (fp32 cos/sin), bf16 store
    const float mean = ksum / (float)a.D;
    const float d = tid < a.D ? key_v - mean : 0.f;
    const float var = block_sum(d * d, scratch[0]) / (float)a.D;
    const float rstd = 1.0f / sqrtf(var + a.key_eps);
    if (tid < a.D) s_key[tid] = __fadd_rn(__fmul_rn(__fmul_rn(d, rstd), key_w), key_b);
    __syncthreads();
    bf16* idx_row = a.index_cache + (((int64_t)lane_id * a.full_layers + a.index_slot) * a.local_cap + local_row) * a.D;
    if (tid < a.D) {
        float o = s_key[tid];
        if (tid < a.rd) {
            const int j = tid >> 1;
            const float angle = __fmul_rn((float)pos, key_f);
            const float cs = cosf(angle), sn = sinf(angle);
            const float even = s_key[2 * j], odd = s_key[2 * j + 1];
            o = (tid & 1) ? __fadd_rn(__fmul_rn(odd, cs), __fmul_rn(even, sn)) : __fsub_rn(__fmul_rn(even, cs), __fmul_rn(odd, sn));
        }
        const bf16 ob = __float2bfloat16_rn(o);
        if (write_cache) idx_row[tid] = ob;
        if (a.idx_key_new) a.idx_key_new[(int64_t)r * a.D + tid] = ob;
    }
    if (tid < a.IH) a.head_w[(int64_t)r * a.IH + tid] = __fmul_rn(hw_v, a.head_scale);
}


// ---------------------------------------------------------------------------------------------------
#define QA_COLS 128
#define QA_BATCH 12     // weight rows in flight per thread
#define QA_MAX_NOPE 256 // widest no-position part of a query head the kernel stages
// When q_proj is set the kernel takes the raw q_b projection (fp32 [rows, q_stride], head h at h * (nope + rd)) instead of
// the rounded q_nope, and also rotates the rope part of its head into q_full: the separate q_post launch is not needed.
struct QAbsorbSource {
    const float* q_proj;
    int64_t q_stride;
    const bf16* rope_table;  // [capacity, rd] cos | sin
    const int* row_pos;
    int capacity;
};


// One (head h, block `by` of QA_COLS latent columns) tile; every thread of a 256-thread CTA calls it.  red and qs are
// shared memory.  The caller signals the peers (grid_signal_peers) once all of its tiles are done.
template <int R>
__device__ __forceinline__ void q_absorb_tile(const bf16* __restrict__ q_nope, int rows, const bf16* __restrict__ kv_b, int heads_local,
                                              int head_base, int heads_total, int nope, int vdim, int L, int rd, bf16* __restrict__ q_full,
                                              int64_t q_full_offset, const PeerComm& comm, const QAbsorbSource& src, int h, int by,
                                              float (*red)[R][QA_COLS], float (*qs)[QA_MAX_NOPE]) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c0 = by * QA_COLS + lane * 4;
    const int per = (nope + 7) / 8;
    const int d0 = warp * per, d1 = min(nope, d0 + per);
    for (int i = threadIdx.x; i < R * nope; i += blockDim.x) {
        const int r = i / nope, d = i % nope;
        qs[r][d] = src.q_proj ? bf16_round(src.q_proj[(int64_t)(r < rows ? r : 0) * src.q_stride + h * (nope + rd) + d])
                              : __bfloat162float(q_nope[((int64_t)(r < rows ? r : 0) * heads_local + h) * nope + d]);
    }
    float acc[R][4];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;
    const bf16* wk = kv_b + (int64_t)h * (nope + vdim) * L;
    // this warp's slice of the weight in two batches of independent loads, issued before the query is needed
    uint2 wv[QA_BATCH];
    if (c0 < L) {
#pragma unroll
        for (int u = 0; u < QA_BATCH; ++u)
            wv[u] = d0 + u < d1 ? *reinterpret_cast<const uint2*>(wk + (int64_t)(d0 + u) * L + c0) : make_uint2(0, 0);
    }
    __syncthreads();
    if (c0 < L) {
        for (int db = d0; db < d1; db += QA_BATCH) {
            uint2 nx[QA_BATCH];
#pragma unroll
            for (int u = 0; u < QA_BATCH; ++u)
                nx[u] = db + QA_BATCH + u < d1 ? *reinterpret_cast<const uint2*>(wk + (int64_t)(db + QA_BATCH + u) * L + c0) : make_uint2(0, 0);
#pragma unroll
            for (int u = 0; u < QA_BATCH; ++u) {
                if (db + u >= d1) break;
                const float w0 = bf16_lo(wv[u].x), w1 = bf16_hi(wv[u].x), w2 = bf16_lo(wv[u].y), w3 = bf16_hi(wv[u].y);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float qv = qs[r][db + u];
                    acc[r][0] = fmaf(qv, w0, acc[r][0]); acc[r][1] = fmaf(qv, w1, acc[r][1]);
                    acc[r][2] = fmaf(qv, w2, acc[r][2]); acc[r][3] = fmaf(qv, w3, acc[r][3]);
                }
            }
#pragma unroll
            for (int u = 0; u < QA_BATCH; ++u) wv[u] = nx[u];
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int i = 0; i < 4; ++i) red[warp][r][lane * 4 + i] = acc[r][i];
    __syncthreads();
    const int W = L + rd;
    for (int i = threadIdx.x; i < R * QA_COLS; i += blockDim.x) {
        const int r = i / QA_COLS, cc = i % QA_COLS, c = by * QA_COLS + cc;
        if (r >= rows || c >= L) continue;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) s += red[w][r][cc];
        const bf16 o = __float2bfloat16_rn(s);
        const int64_t at = ((int64_t)r * heads_total + head_base + h) * W + c;
        q_full[at] = o;
        for (int p = 0; p < comm.world; ++p)
            if (p != comm.rank) reinterpret_cast<bf16*>(comm.data[p] + q_full_offset)[at] = o;
    }
    if (src.q_proj && by == 0) {
        // rope part of this head: interleaved pairs, bf16 table, fp32 products, one rounding (as q_post does)
        const int half = rd / 2;
        for (int i = threadIdx.x; i < rows * half; i += blockDim.x) {
            const int r = i / half, j = i % half;
            const int pos = min(max(src.row_pos[r], 0), src.capacity - 1);
            const float* q = src.q_proj + (int64_t)r * src.q_stride + h * (nope + rd) + nope;
            const float even = bf16_round(q[2 * j]), odd = bf16_round(q[2 * j + 1]);
            const float cs = __bfloat162float(src.rope_table[(int64_t)pos * rd + j]);
            const float sn = __bfloat162float(src.rope_table[(int64_t)pos * rd + half + j]);
            bf16* dst = q_full + ((int64_t)r * heads_total + head_base + h) * W + L;
            dst[2 * j] = __float2bfloat16_rn(__fsub_rn(__fmul_rn(even, cs), __fmul_rn(odd, sn)));
            dst[2 * j + 1] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(odd, cs), __fmul_rn(even, sn)));
        }
        __syncthreads();
    }
    if (comm.world > 1 && by == 0) {
        // the rope part was written locally (above, or by q_post in an earlier kernel); forward it to the peers
        for (int i = threadIdx.x; i < rows * rd; i += blockDim.x) {
            const int r = i / rd, j = i % rd;
            const int64_t at = ((int64_t)r * heads_total + head_base + h) * W + L + j;
            const bf16 o = q_full[at];
            for (int p = 0; p < comm.world; ++p)
                if (p != comm.rank) reinterpret_cast<bf16*>(comm.data[p] + q_full_offset)[at] = o;
        }
    }
}

