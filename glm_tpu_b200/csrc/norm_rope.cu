// Normalisation, RoPE, cache-row write and query preparation kernels.
//
//   embed_rows          residual[r] = embedding[token[r]]
//   add_rmsnorm         s = f32(update) + f32(residual); residual = bf16(s); x = bf16(bf16(s*rsqrt(ms+eps)) * w)
//   qkv_a_post          q_a/kv_a LoRA RMSNorms, RoPE of the key part, cache-row write into the owner's
//                       stripe, indexer key LayerNorm + RoPE + index-cache write, indexer head weights
//   q_post              RoPE of every head's query rope part, bf16 rounding of the nope part, indexer
//                       query RoPE (fp32)
//   q_absorb            q_c[h] = bf16(q_nope[h] @ W_k[h]) for <= 8 rows, written (and pushed to the
//                       peers: fused all-gather) into the all-heads query buffer
//
// Rounding rules restate reference `glm_tpu/layers/norm.py:55-122,226-248`, `layers/rope.py:94-99,145-199`,
// `layers/attention/mla.py:379-403,441-475`, `layers/attention/dsa_indexer.py:808-843`.
#include "common.cuh"
#include "norm_rope_core.cuh"
#include "peer.cuh"

// ---------------------------------------------------------------------------------------------------
__global__ void embed_rows_kernel(const int* __restrict__ tokens, const bf16* __restrict__ table, int vocab, int H,
                                  bf16* __restrict__ residual, uint32_t* status) {
    GLMB_PDL_PROLOGUE();
    const int r = blockIdx.x;
    int t = tokens[r];
    if (t < 0 || t >= vocab) {
        if (threadIdx.x == 0) raise_status(status, GLMB_STATUS_BAD_INDEX);
        t = min(max(t, 0), vocab - 1);
    }
    const uint4* src = reinterpret_cast<const uint4*>(table + (int64_t)t * H);
    uint4* dst = reinterpret_cast<uint4*>(residual + (int64_t)r * H);
    for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

// ---------------------------------------------------------------------------------------------------
// One CTA per row (see add_rmsnorm_row in norm_rope_core.cuh).  H % 8 == 0 and H <= 256 * 8 * RN_VECS.
__global__ void __launch_bounds__(256)
add_rmsnorm_kernel(const bf16* __restrict__ update, bf16* __restrict__ residual, const bf16* __restrict__ weight,
                   bf16* __restrict__ out, int H, float eps) {
    GLMB_PDL_PROLOGUE();
    __shared__ float scratch[40];
    const int64_t base = (int64_t)blockIdx.x * H;
    add_rmsnorm_row<false>(update ? update + base : nullptr, residual + base, weight, out + base, H, eps, scratch);
}

// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) qkv_a_post_generic_kernel(QkvPostArgs a) {
    GLMB_PDL_PROLOGUE();
    __shared__ float scratch[40];
    __shared__ float s_key[256];
    const int r = blockIdx.x;
    const float* p = a.proj + (int64_t)r * a.proj_stride;
    int pos = a.row_pos[r];
    const int lane_id = a.row_lane[r];
    const bool active = a.row_active ? a.row_active[r] != 0 : true;
    // A position outside the context is reported and the row is computed at a clamped position (no address leaves the
    // tables), but it is NOT stored: bad metadata leaves the caches as they were and the host poisons the engine.
    const bool bad_pos = pos < 0 || pos >= a.capacity;
    if (bad_pos) {
        if (threadIdx.x == 0) raise_status(a.status, GLMB_STATUS_BAD_INDEX);
        pos = min(max(pos, 0), a.capacity - 1);
    }
    const int page = a.stripe * a.world;
    const bool owner = ((pos / a.stripe) % a.world) == a.rank;
    const int local_row = (pos / page) * a.stripe + pos % a.stripe;
    const int W = a.L + a.rd;
    bf16* cache_row = a.kv_cache + (((int64_t)lane_id * a.layers + a.layer) * a.local_cap + local_row) * W;
    const bool write_cache = owner && active && !bad_pos;

    // q_a RMSNorm
    // (both sums of squares are accumulated in one sweep of float4 loads and reduced together)
    const float* c = p + a.Q;
    float ss = 0.f, ss_kv = 0.f;
    for (int i = threadIdx.x * 4; i < a.Q; i += blockDim.x * 4) {
        const float4 v4 = *reinterpret_cast<const float4*>(p + i);
        const float v0 = bf16_round(v4.x), v1 = bf16_round(v4.y), v2 = bf16_round(v4.z), v3 = bf16_round(v4.w);
        ss = fmaf(v0, v0, ss); ss = fmaf(v1, v1, ss); ss = fmaf(v2, v2, ss); ss = fmaf(v3, v3, ss);
    }
    for (int i = threadIdx.x * 4; i < a.L; i += blockDim.x * 4) {
        const float4 v4 = *reinterpret_cast<const float4*>(c + i);
        const float v0 = bf16_round(v4.x), v1 = bf16_round(v4.y), v2 = bf16_round(v4.z), v3 = bf16_round(v4.w);
        ss_kv = fmaf(v0, v0, ss_kv); ss_kv = fmaf(v1, v1, ss_kv); ss_kv = fmaf(v2, v2, ss_kv); ss_kv = fmaf(v3, v3, ss_kv);
    }
    float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)a.Q + a.eps);
    const float inv_kv = 1.0f / sqrtf(block_sum(ss_kv, scratch) / (float)a.L + a.eps);
    for (int i = threadIdx.x * 4; i < a.Q; i += blockDim.x * 4) {
        const float4 v4 = *reinterpret_cast<const float4*>(p + i);
        const uint2 w2 = *reinterpret_cast<const uint2*>(a.q_norm_w + i);
        uint2 o;
        o.x = pack_bf16(bf16_round(bf16_round(v4.x) * inv) * bf16_lo(w2.x), bf16_round(bf16_round(v4.y) * inv) * bf16_hi(w2.x));
        o.y = pack_bf16(bf16_round(bf16_round(v4.z) * inv) * bf16_lo(w2.y), bf16_round(bf16_round(v4.w) * inv) * bf16_hi(w2.y));
        *reinterpret_cast<uint2*>(a.q_resid + (int64_t)r * a.Q + i) = o;
    }
    // kv_a latent RMSNorm
    inv = inv_kv;
    for (int i = threadIdx.x; i < a.L; i += blockDim.x) {
        const float y = bf16_round(bf16_round(c[i]) * inv);
        const bf16 o = __float2bfloat16_rn(y * __bfloat162float(a.kv_norm_w[i]));
        if (write_cache) cache_row[i] = o;
        if (a.kv_new) a.kv_new[(int64_t)r * W + i] = o;
    }
    // RoPE of the key part: interleaved pairs, bf16 table, fp32 products, one rounding
    const int half = a.rd / 2;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        const float even = bf16_round(c[a.L + 2 * j]), odd = bf16_round(c[a.L + 2 * j + 1]);
        const float cs = __bfloat162float(a.rope_table[(int64_t)pos * a.rd + j]);
        const float sn = __bfloat162float(a.rope_table[(int64_t)pos * a.rd + half + j]);
        const bf16 oe = __float2bfloat16_rn(__fsub_rn(__fmul_rn(even, cs), __fmul_rn(odd, sn)));
        const bf16 oo = __float2bfloat16_rn(__fadd_rn(__fmul_rn(odd, cs), __fmul_rn(even, sn)));
        if (write_cache) { cache_row[a.L + 2 * j] = oe; cache_row[a.L + 2 * j + 1] = oo; }
        if (a.kv_new) { a.kv_new[(int64_t)r * W + a.L + 2 * j] = oe; a.kv_new[(int64_t)r * W + a.L + 2 * j + 1] = oo; }
    }
    if (!a.has_indexer) return;
    // Indexer key: affine LayerNorm (fp32), RoPE on the first rd features (fp32 cos/sin), bf16 store
    const float* kx = c + W;
    float v = threadIdx.x < a.D ? kx[threadIdx.x] : 0.f;
    const float mean = block_sum(v, scratch) / (float)a.D;
    const float d = threadIdx.x < a.D ? v - mean : 0.f;
    const float var = block_sum(d * d, scratch) / (float)a.D;
    const float rstd = 1.0f / sqrtf(var + a.key_eps);
    if (threadIdx.x < a.D) s_key[threadIdx.x] = __fadd_rn(__fmul_rn(__fmul_rn(d, rstd), a.k_norm_w[threadIdx.x]), a.k_norm_b[threadIdx.x]);
    __syncthreads();
    bf16* idx_row = a.index_cache + (((int64_t)lane_id * a.full_layers + a.index_slot) * a.local_cap + local_row) * a.D;
    if (threadIdx.x < a.D) {
        const int i = threadIdx.x;
        float o = s_key[i];
        if (i < a.rd) {
            const int j = i >> 1;
            const float angle = __fmul_rn((float)pos, a.inv_freq[j]);
            const float cs = cosf(angle), sn = sinf(angle);
            const float even = s_key[2 * j], odd = s_key[2 * j + 1];
            o = (i & 1) ? __fadd_rn(__fmul_rn(odd, cs), __fmul_rn(even, sn)) : __fsub_rn(__fmul_rn(even, cs), __fmul_rn(odd, sn));
        }
        const bf16 ob = __float2bfloat16_rn(o);
        if (write_cache) idx_row[i] = ob;
        if (a.idx_key_new) a.idx_key_new[(int64_t)r * a.D + i] = ob;
    }
    // Indexer head weights
    const float* hw = kx + a.D;
    const float hscale = a.head_scale;
    for (int h = threadIdx.x; h < a.IH; h += blockDim.x) a.head_w[(int64_t)r * a.IH + h] = __fmul_rn(hw[h], hscale);
}

// ---------------------------------------------------------------------------------------------------
// The same computation as qkv_a_post_generic_kernel for Q <= 2048 and L <= 1024 (every supported geometry): all of the
// row's inputs are fetched before the first reduction, the three independent sums share one reduction, and the latent
// is stored four values at a time.  One memory round trip and two reductions instead of four and four.
__global__ void __launch_bounds__(256) qkv_a_post_kernel(QkvPostArgs a) {
    GLMB_PDL_PROLOGUE();
    __shared__ float scratch[3][40];
    __shared__ float s_key[256];
    qkv_a_post_row(a, blockIdx.x, scratch, s_key);
}

// ---------------------------------------------------------------------------------------------------
struct QPostArgs {
    const float* q;          // [rows, q_stride]: heads_local * (nope + rd)  |  IH * D (indexer, when has_indexer)
    int64_t q_stride;
    const bf16* rope_table;  // [capacity, rd]
    const float* inv_freq;   // [rd/2]
    const int* row_pos;
    bf16* q_nope;            // [rows, heads_local, nope] bf16-rounded
    bf16* q_full;            // [rows, heads_total, L + rd]; the rope part of this rank's heads is written here
    float* q_idx;            // [rows, IH, D] fp32 with RoPE applied
    int heads_local, head_base, heads_total, nope, rd, L, IH, D, has_indexer, capacity;
};

__global__ void __launch_bounds__(256) q_post_kernel(QPostArgs a) {
    GLMB_PDL_PROLOGUE();
    const int r = blockIdx.x;
    const float* q = a.q + (int64_t)r * a.q_stride;
    const int pos = min(max(a.row_pos[r], 0), a.capacity - 1);
    const int qk = a.nope + a.rd, half = a.rd / 2, W = a.L + a.rd;
    // blockIdx.y spreads one row's work over several CTAs: each thread touches a few elements only
    const int tid = blockIdx.y * blockDim.x + threadIdx.x, nth = gridDim.y * blockDim.x;
    const int np2 = a.nope >> 1;
    for (int i = tid; i < a.heads_local * np2; i += nth) {
        const int h = i / np2, d = (i % np2) * 2;
        const float2 v = *reinterpret_cast<const float2*>(q + h * qk + d);
        *reinterpret_cast<uint32_t*>(a.q_nope + ((int64_t)r * a.heads_local + h) * a.nope + d) = pack_bf16(v.x, v.y);
    }
    for (int i = tid; i < a.heads_local * half; i += nth) {
        const int h = i / half, j = i % half;
        const float even = bf16_round(q[h * qk + a.nope + 2 * j]), odd = bf16_round(q[h * qk + a.nope + 2 * j + 1]);
        const float cs = __bfloat162float(a.rope_table[(int64_t)pos * a.rd + j]);
        const float sn = __bfloat162float(a.rope_table[(int64_t)pos * a.rd + half + j]);
        bf16* dst = a.q_full + ((int64_t)r * a.heads_total + a.head_base + h) * W + a.L;
        dst[2 * j] = __float2bfloat16_rn(__fsub_rn(__fmul_rn(even, cs), __fmul_rn(odd, sn)));
        dst[2 * j + 1] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(odd, cs), __fmul_rn(even, sn)));
    }
    if (!a.has_indexer) return;
    const float* qi = q + a.heads_local * qk;
    for (int i = tid; i < a.IH * a.D; i += nth) {
        const int h = i / a.D, d = i % a.D;
        float o = qi[i];
        if (d < a.rd) {
            const int j = d >> 1;
            const float angle = __fmul_rn((float)pos, a.inv_freq[j]);
            const float cs = cosf(angle), sn = sinf(angle);
            const float even = qi[h * a.D + 2 * j], odd = qi[h * a.D + 2 * j + 1];
            o = (d & 1) ? __fadd_rn(__fmul_rn(odd, cs), __fmul_rn(even, sn)) : __fsub_rn(__fmul_rn(even, cs), __fmul_rn(odd, sn));
        }
        a.q_idx[(int64_t)r * a.IH * a.D + i] = o;
    }
}

// ---------------------------------------------------------------------------------------------------
// q_c[r][h][c] = bf16( sum_d q_nope[r][h][d] * W_k[h][d][c] ),  W_k[h] = kv_b rows h*(nope+v) .. +nope, [nope, L].
// grid (heads_local, ceil(L/128)); 8 warps split d, a lane owns 4 columns.  The result row (and, from the
// blockIdx.y == 0 CTA, the rope part) is also stored into every peer's query buffer: the all-gather of
// the queries over heads is fused here, and the last CTA signals GLMB_SIG_Q.
template <int R>
__global__ void __launch_bounds__(256)
q_absorb_kernel(const bf16* __restrict__ q_nope, int rows, const bf16* __restrict__ kv_b, int heads_local, int head_base,
                int heads_total, int nope, int vdim, int L, int rd, bf16* __restrict__ q_full, int64_t q_full_offset,
                PeerComm comm, int sig, QAbsorbSource src) {
    GLMB_PDL_PROLOGUE();
    __shared__ float red[8][R][QA_COLS];
    __shared__ float qs[R][QA_MAX_NOPE];
    q_absorb_tile<R>(q_nope, rows, kv_b, heads_local, head_base, heads_total, nope, vdim, L, rd, q_full, q_full_offset, comm, src,
                     blockIdx.x, blockIdx.y, red, qs);
    grid_signal_peers(comm, sig);
}

// ===================================================================================================
GLMB_API int glmb_embed_rows(const int* tokens, const void* table, int rows, int vocab, int H, void* residual, uint32_t* status,
                             void* stream) {
    if (H & 7) return 1;
    GLMB_LAUNCH(embed_rows_kernel, rows, 256, 0, (cudaStream_t)stream, tokens, (const bf16*)table, vocab, H, (bf16*)residual, status);
    return (int)cudaGetLastError();
}

GLMB_API int glmb_add_rmsnorm(const void* update, void* residual, const void* weight, void* out, int rows, int H, float eps,
                              void* stream) {
    if ((H & 7) || H > 256 * 8 * RN_VECS) return 1;
    GLMB_LAUNCH(add_rmsnorm_kernel, rows, 256, 0, (cudaStream_t)stream, (const bf16*)update, (bf16*)residual, (const bf16*)weight,
                                                                  (bf16*)out, H, eps);
    return (int)cudaGetLastError();
}

static int g_qkv_fast = 1;
// The generic kernel serves geometries beyond the limits of the single-round-trip kernel (q_lora_rank > 2048, kv_lora_rank > 1024,
// rope > 512, more than 256 index heads); the switch lets the tests run both on a geometry both take.
GLMB_API void glmb_set_qkv_fast(int enabled) { g_qkv_fast = enabled ? 1 : 0; }

GLMB_API int glmb_qkv_a_post(const QkvPostArgs* args, int rows, void* stream) {
    if (args->D > 256 || (args->rd & 1) || (args->Q & 3) || (args->L & 3) || (args->proj_stride & 3)) return 1;
    const int W = args->L + args->rd;
    if (g_qkv_fast && args->Q <= 2048 && args->L <= 1024 && args->rd <= 512 && args->IH <= 256 && !(W & 3))
        GLMB_LAUNCH(qkv_a_post_kernel, rows, 256, 0, (cudaStream_t)stream, *args);
    else
        GLMB_LAUNCH(qkv_a_post_generic_kernel, rows, 256, 0, (cudaStream_t)stream, *args);
    return (int)cudaGetLastError();
}

GLMB_API int glmb_q_post(const QPostArgs* args, int rows, void* stream) {
    if ((args->nope & 1) || (args->q_stride & 1)) return 1;
    const int work = args->heads_local * (args->nope / 2 + args->rd / 2) + (args->has_indexer ? args->IH * args->D : 0);
    dim3 grid(rows, rows <= 16 ? max(1, min(32, ceil_div(work, 512))) : 1);
    GLMB_LAUNCH(q_post_kernel, grid, 256, 0, (cudaStream_t)stream, *args);
    return (int)cudaGetLastError();
}

static int launch_q_absorb(const void* q_nope, int rows, const void* kv_b, int heads_local, int head_base, int heads_total, int nope, int vdim,
                           int L, int rd, void* q_full, int64_t q_full_offset, const PeerComm& c, int sig, const QAbsorbSource& src, void* stream) {
    dim3 grid(heads_local, ceil_div(L, QA_COLS));
#define CALL(RR)                                                                                                              \
    GLMB_LAUNCH(q_absorb_kernel<RR>, grid, 256, 0, (cudaStream_t)stream, (const bf16*)q_nope, rows, (const bf16*)kv_b, heads_local, head_base, \
                                                                heads_total, nope, vdim, L, rd, (bf16*)q_full, q_full_offset, c, sig, src)
    if (rows <= 1) { CALL(1); } else if (rows <= 2) { CALL(2); } else if (rows <= 4) { CALL(4); } else { CALL(8); }
#undef CALL
    return (int)cudaGetLastError();
}

// q_full must be the staging-buffer address `comm->data[rank] + q_full_offset` when world > 1.
GLMB_API int glmb_q_absorb(const void* q_nope, int rows, const void* kv_b, int heads_local, int head_base, int heads_total,
                           int nope, int vdim, int L, int rd, void* q_full, int64_t q_full_offset, const PeerComm* comm, int sig,
                           void* stream) {
    if (rows < 1 || rows > GLMB_MAX_ROWS || (L & 3) || nope > QA_MAX_NOPE) return 1;
    PeerComm c;
    if (comm) c = *comm; else { memset(&c, 0, sizeof(c)); c.world = 1; }
    QAbsorbSource src;
    memset(&src, 0, sizeof(src));
    return launch_q_absorb(q_nope, rows, kv_b, heads_local, head_base, heads_total, nope, vdim, L, rd, q_full, q_full_offset, c, sig, src, stream);
}

// The same with the q_post work folded in: q_proj is the fp32 output of the q_b projection ([rows, q_stride]); the kernel
// rounds the no-position parts itself and writes the rotated rope parts of its heads into q_full.
GLMB_API int glmb_q_absorb_from_proj(const float* q_proj, int64_t q_stride, const void* rope_table, const int* row_pos, int capacity,
                                     int rows, const void* kv_b, int heads_local, int head_base, int heads_total, int nope, int vdim,
                                     int L, int rd, void* q_full, int64_t q_full_offset, const PeerComm* comm, int sig, void* stream) {
    if (rows < 1 || rows > GLMB_MAX_ROWS || (L & 3) || nope > QA_MAX_NOPE || (rd & 1) || !q_proj || !rope_table || !row_pos) return 1;
    PeerComm c;
    if (comm) c = *comm; else { memset(&c, 0, sizeof(c)); c.world = 1; }
    QAbsorbSource src;
    src.q_proj = q_proj; src.q_stride = q_stride; src.rope_table = (const bf16*)rope_table; src.row_pos = row_pos; src.capacity = capacity;
    return launch_q_absorb(nullptr, rows, kv_b, heads_local, head_base, heads_total, nope, vdim, L, rd, q_full, q_full_offset, c, sig, src, stream);
}
