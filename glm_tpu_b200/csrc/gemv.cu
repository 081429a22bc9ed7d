// Skinny (1..8 row) weight-streaming projections for decode.
//
// With 1-8 live rows every projection of the decode step is bound by streaming the weight matrix from
// HBM once, so these kernels are organised around 16-byte streaming loads (L1 no-allocate), one warp per
// output feature (two when that shares the activation registers), fp32 accumulation and a fused epilogue:
// fp32/bf16 store, SwiGLU of a gate/up pair, or an in-kernel all-reduce over peer memory for K-split
// (tensor-parallel) projections.  FP8 weights are decoded with the contract formula
// bf16(f32(e4m3) * scale_inv[n/128][k/128]) on the fly; the product with the bf16 activation is exact in
// fp32.
//
// Replaces: reference `glm_tpu/layers/linear.py:89-128` (+ psum), `layers/mlp.py:55-68`,
// `kernels/fp8_grouped_matmul/kernel.py:125-299` (decode routed projection, t=1 and t=2).
#include "common.cuh"
#include "gemv_core.cuh"
#include "peer.cuh"

#define SK_WARPS 8
#define SK_THREADS (SK_WARPS * 32)

// With programmatic dependent launch a kernel's CTAs become resident while its predecessor still runs and then wait for it.
// The weights do not depend on the predecessor, so before waiting a CTA asks the L2 for the rows it is about to stream: the HBM
// fetch overlaps the predecessor's tail instead of starting after it.  Tables larger than SK_PREFETCH_LIMIT are left alone (they
// would only sweep the L2).
#define SK_PREFETCH_LIMIT ((int64_t)48 << 20)
__device__ __forceinline__ void sk_prefetch_rows(const void* first_row, int rows, int64_t row_stride_elems, int K, int elem_bytes) {
    if (threadIdx.x != 0 || rows <= 0) return;
    const char* p = reinterpret_cast<const char*>(first_row);
    if (row_stride_elems == K) {
        const uint32_t bytes = (uint32_t)(((int64_t)rows * K * elem_bytes) & ~(int64_t)15);
        if (bytes && !((uintptr_t)p & 15)) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
        return;
    }
    for (int r = 0; r < rows; ++r) {
        const char* q = p + (int64_t)r * row_stride_elems * elem_bytes;
        const uint32_t bytes = (uint32_t)(((int64_t)K * elem_bytes) & ~(int64_t)15);
        if (bytes && !((uintptr_t)q & 15)) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(q), "r"(bytes) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------
// out[r][n] = sum_k x[r][k] * w[n][k]          (bf16 weights)
enum { SK_OUT_F32 = 0, SK_OUT_BF16 = 1, SK_OUT_ALLREDUCE_BF16 = 2, SK_OUT_ARGMAX = 3 };

// ks (1, 2, 4 or 8) warps of a CTA split K for the same pair of output rows and add their partial sums through
// shared memory: small-N projections then still fill the machine.  A CTA produces 16 / ks output rows.
template <int R>
__global__ void __launch_bounds__(SK_THREADS)
skinny_bf16_kernel(const bf16* __restrict__ x, int64_t xs, int rows, const bf16* __restrict__ w, int64_t ws, int N, int K,
                   void* __restrict__ out, int64_t os, int mode, int ks, int64_t xb, int64_t wb, int64_t ob, PeerComm comm,
                   int channel) {
    asm volatile("griddepcontrol.launch_dependents;");
    if ((int64_t)N * K * 2 * gridDim.y <= SK_PREFETCH_LIMIT) {
        const int first = blockIdx.x * (SK_WARPS / ks) * 2;
        sk_prefetch_rows(w + (int64_t)blockIdx.y * wb + (int64_t)first * ws, min((SK_WARPS / ks) * 2, N - first), ws, K, 2);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float red[SK_WARPS][2][R];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = warp / ks, kpart = warp % ks, groups = SK_WARPS / ks;
    const int n0 = (blockIdx.x * groups + group) * 2;
    // blockIdx.y selects one problem of a batch (per-head projections): element offsets xb / wb / ob.
    x += (int64_t)blockIdx.y * xb;
    w += (int64_t)blockIdx.y * wb;
    out = mode == SK_OUT_F32 ? (void*)(reinterpret_cast<float*>(out) + (int64_t)blockIdx.y * ob)
                             : (void*)(reinterpret_cast<bf16*>(out) + (int64_t)blockIdx.y * ob);
    const bf16* xr[R];
#pragma unroll
    for (int r = 0; r < R; ++r) xr[r] = x + (int64_t)(r < rows ? r : 0) * xs;
    float acc[2][R];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int r = 0; r < R; ++r) acc[j][r] = 0.f;
    if (n0 < N) {
        const bf16* wp[2] = {w + (int64_t)n0 * ws, w + (int64_t)min(n0 + 1, N - 1) * ws};
        const int kspan = K / ks;
        warp_dot_bf16<R, 2>(xr, wp, kpart * kspan, (kpart + 1) * kspan, lane, acc);
        warp_reduce_all<R, 2>(acc);
    }
    if (ks > 1) {
        if (lane == 0) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int r = 0; r < R; ++r) red[warp][j][r] = acc[j][r];
        }
        __syncthreads();
        if (kpart == 0 && lane == 0) {
            for (int p = 1; p < ks; ++p)
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int r = 0; r < R; ++r) acc[j][r] += red[warp + p][j][r];
        }
    }
    const bool writer = lane == 0 && kpart == 0;
    if (mode == SK_OUT_ALLREDUCE_BF16) {
        __shared__ float sh[SK_WARPS * 2 * R];
        if (writer) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int r = 0; r < R; ++r) sh[(group * 2 + j) * R + r] = acc[j][r];
        }
        __syncthreads();
        cta_allreduce_f32(comm, channel, sh, groups * 2 * R);
        if (writer) {
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int r = 0; r < R; ++r)
                    if (n0 + j < N && r < rows)
                        reinterpret_cast<bf16*>(out)[(int64_t)r * os + n0 + j] = __float2bfloat16_rn(sh[(group * 2 + j) * R + r]);
        }
        return;
    }
    if (mode == SK_OUT_ARGMAX) {
        // out: unsigned long long best[rows]; `channel` carries the id of output column 0 (vocabulary offset).
        __shared__ unsigned long long best_s[SK_WARPS][R];
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < R; ++r) {
                unsigned long long key = 0ull;
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    if (kpart == 0 && n0 + j < N) {
                        const float v = bf16_round(acc[j][r]);
                        if (!isfinite(v)) raise_status(comm.status, GLMB_STATUS_NONFINITE);
                        const unsigned long long k2 = candidate_key(v, channel + n0 + j);
                        key = k2 > key ? k2 : key;
                    }
                best_s[warp][r] = key;
            }
        }
        __syncthreads();
        if ((int)threadIdx.x < rows && (int)threadIdx.x < R) {
            unsigned long long key = 0ull;
#pragma unroll
            for (int w2 = 0; w2 < SK_WARPS; ++w2) key = best_s[w2][threadIdx.x] > key ? best_s[w2][threadIdx.x] : key;
            if (key) atomicMax(reinterpret_cast<unsigned long long*>(out) + threadIdx.x, key);
        }
        return;
    }
    if (writer && n0 < N) {
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int r = 0; r < R; ++r)
                if (n0 + j < N && r < rows) {
                    if (mode == SK_OUT_F32) reinterpret_cast<float*>(out)[(int64_t)r * os + n0 + j] = acc[j][r];
                    else reinterpret_cast<bf16*>(out)[(int64_t)r * os + n0 + j] = __float2bfloat16_rn(acc[j][r]);
                }
    }
}

// act[r][n] = bf16( silu(bf16(x.w_gate[n])) * bf16(x.w_up[n]) )       (bf16 weights; dense MLP / shared expert)
template <int R>
__global__ void __launch_bounds__(SK_THREADS)
skinny_bf16_swiglu_kernel(const bf16* __restrict__ x, int64_t xs, int rows, const bf16* __restrict__ wg,
                          const bf16* __restrict__ wu, int64_t ws, int N, int K, bf16* __restrict__ act, int64_t as, int ks) {
    asm volatile("griddepcontrol.launch_dependents;");
    if ((int64_t)N * K * 4 <= SK_PREFETCH_LIMIT) {
        const int first = blockIdx.x * (SK_WARPS / ks), cnt = min(SK_WARPS / ks, N - first);
        sk_prefetch_rows(wg + (int64_t)first * ws, cnt, ws, K, 2);
        sk_prefetch_rows(wu + (int64_t)first * ws, cnt, ws, K, 2);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float red[SK_WARPS][2][R];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = warp / ks, kpart = warp % ks;
    const int n = blockIdx.x * (SK_WARPS / ks) + group;
    const bool valid = n < N;
    const bf16* xr[R];
#pragma unroll
    for (int r = 0; r < R; ++r) xr[r] = x + (int64_t)(r < rows ? r : 0) * xs;
    float acc[2][R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[0][r] = acc[1][r] = 0.f;
    if (valid) {
        const bf16* wp[2] = {wg + (int64_t)n * ws, wu + (int64_t)n * ws};
        const int kspan = K / ks;
        warp_dot_bf16<R, 2>(xr, wp, kpart * kspan, (kpart + 1) * kspan, lane, acc);
        warp_reduce_all<R, 2>(acc);
    }
    if (ks > 1) {
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < R; ++r) { red[warp][0][r] = acc[0][r]; red[warp][1][r] = acc[1][r]; }
        }
        __syncthreads();
        if (kpart == 0 && lane == 0)
            for (int p = 1; p < ks; ++p)
#pragma unroll
                for (int r = 0; r < R; ++r) { acc[0][r] += red[warp + p][0][r]; acc[1][r] += red[warp + p][1][r]; }
    }
    if (lane == 0 && kpart == 0 && valid) {
#pragma unroll
        for (int r = 0; r < R; ++r)
            if (r < rows) {
                const float g = bf16_round(acc[0][r]), u = bf16_round(acc[1][r]);
                act[(int64_t)r * as + n] = __float2bfloat16_rn(g * sigmoidf_precise(g) * u);
            }
    }
}

// ---------------------------------------------------------------------------------------------------
// Routed experts (FP8), organised as tiles: tile t = up to RT routes of ONE expert.
//   tile_expert[t]  global expert id (< 0: empty tile)
//   tile_routes[t*RT + i]  route index p = token_row * top_k + slot, or -1
// When tile_routes == nullptr every tile is the single route t and its expert is tile_expert[t] (decode).
// A tile whose expert is not stored on this rank is skipped: expert-parallel ownership is resolved here.
template <int RT>
__global__ void __launch_bounds__(SK_THREADS)
moe_gateup_fp8_kernel(const bf16* __restrict__ x, int64_t xs, int top_k, const int* __restrict__ tile_expert,
                      const int* __restrict__ tile_routes, const int* __restrict__ n_tiles, const uint8_t* __restrict__ wg,
                      const uint8_t* __restrict__ wu, const float* __restrict__ sg, const float* __restrict__ su,
                      int expert_base, int experts_local, int I, int H, bf16* __restrict__ act) {
    GLMB_PDL_PROLOGUE();
    const int t = blockIdx.y;
    if (n_tiles && t >= *n_tiles) return;
    const int e = tile_expert[t] - expert_base;
    if (e < 0 || e >= experts_local) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * SK_WARPS + warp;
    if (n >= I) return;
    int route[RT];
    const bf16* xr[RT];
#pragma unroll
    for (int i = 0; i < RT; ++i) {
        route[i] = tile_routes ? tile_routes[t * RT + i] : (i == 0 ? t : -1);
        xr[i] = x + (int64_t)(route[i] >= 0 ? route[i] / top_k : 0) * xs;
    }
    const int kb = (H + 127) >> 7;
    const int64_t wofs = ((int64_t)e * I + n) * H;
    const int64_t sofs = ((int64_t)e * ((I + 127) >> 7) + (n >> 7)) * kb;
    const uint8_t* wp[2] = {wg + wofs, wu + wofs};
    const float* sp[2] = {sg + sofs, su + sofs};
    float acc[2][RT];
#pragma unroll
    for (int i = 0; i < RT; ++i) acc[0][i] = acc[1][i] = 0.f;
    warp_dot_fp8<RT, 2>(xr, wp, sp, H, lane, acc);
    warp_reduce_all<RT, 2>(acc);
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < RT; ++i)
            if (route[i] >= 0) {
                const float g = bf16_round(acc[0][i]), u = bf16_round(acc[1][i]);
                act[(int64_t)route[i] * I + n] = __float2bfloat16_rn(g * sigmoidf_precise(g) * u);
            }
    }
}

// dw[p][n] = bf16( bf16(act[p] . w_down[e][n]) * bf16(route_weight[p]) )
template <int RT>
__global__ void __launch_bounds__(SK_THREADS)
moe_down_fp8_kernel(const bf16* __restrict__ act, const float* __restrict__ route_weight, const int* __restrict__ tile_expert,
                    const int* __restrict__ tile_routes, const int* __restrict__ n_tiles, const uint8_t* __restrict__ wd,
                    const float* __restrict__ sd, int expert_base, int experts_local, int I, int H, bf16* __restrict__ dw) {
    GLMB_PDL_PROLOGUE();
    const int t = blockIdx.y;
    if (n_tiles && t >= *n_tiles) return;
    const int e = tile_expert[t] - expert_base;
    if (e < 0 || e >= experts_local) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = (blockIdx.x * SK_WARPS + warp) * 2;
    if (n0 >= H) return;
    int route[RT];
    const bf16* xr[RT];
#pragma unroll
    for (int i = 0; i < RT; ++i) {
        route[i] = tile_routes ? tile_routes[t * RT + i] : (i == 0 ? t : -1);
        xr[i] = act + (int64_t)(route[i] >= 0 ? route[i] : 0) * I;
    }
    const int kb = (I + 127) >> 7;
    const int n1 = min(n0 + 1, H - 1);
    const uint8_t* wp[2] = {wd + ((int64_t)e * H + n0) * I, wd + ((int64_t)e * H + n1) * I};
    const float* sp[2] = {sd + ((int64_t)e * ((H + 127) >> 7) + (n0 >> 7)) * kb, sd + ((int64_t)e * ((H + 127) >> 7) + (n1 >> 7)) * kb};
    float acc[2][RT];
#pragma unroll
    for (int i = 0; i < RT; ++i) acc[0][i] = acc[1][i] = 0.f;
    warp_dot_fp8<RT, 2>(xr, wp, sp, I, lane, acc);
    warp_reduce_all<RT, 2>(acc);
    if (lane == 0) {
#pragma unroll
        for (int i = 0; i < RT; ++i)
            if (route[i] >= 0) {
                const float wgt = bf16_round(route_weight[route[i]]);
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    if (n0 + j < H) dw[(int64_t)route[i] * H + n0 + j] = __float2bfloat16_rn(bf16_round(acc[j][i]) * wgt);
            }
    }
}

// ---------------------------------------------------------------------------------------------------
// MoE combine: for row r, column n
//   routed = sum over the row's routes owned by this rank, in slot order, of dw[p][n]      (fp32)
//   shared = this rank's K-slice of the shared-expert down projection                       (fp32, given)
//   both are summed over the ranks in-kernel (peer-memory all-reduce), then
//   out = bf16( bf16( bf16(routed) * scale ) + bf16(shared) )
// plain != 0: out = bf16(sum over ranks of shared_partial)   -- dense MLP / any K-split partial.
// routed_partial != nullptr: only write the local fp32 route sums there (the caller reduces them with a
//   library collective: the NCCL baseline and prefill); no exchange, no output.
// blockIdx.y selects a chunk of GLMB_MAX_ROWS rows.
#define CB_COLS 16
__global__ void __launch_bounds__(128)
moe_combine_kernel(const bf16* __restrict__ dw, const int* __restrict__ topk_ids, const float* __restrict__ shared_partial,
                   int rows_total, int top_k, int H, int expert_base, int experts_local, float scale, int plain,
                   bf16* __restrict__ out, float* __restrict__ routed_partial, PeerComm comm, int channel) {
    GLMB_PDL_PROLOGUE();
    __shared__ float sh[2 * GLMB_MAX_ROWS * CB_COLS];
    const int n0 = blockIdx.x * CB_COLS;
    const int r0 = blockIdx.y * GLMB_MAX_ROWS;
    const int rows = min(GLMB_MAX_ROWS, rows_total - r0);
    const int per = rows * CB_COLS;
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
        const int r = r0 + i / CB_COLS, n = n0 + i % CB_COLS;
        float routed = 0.f, shared = 0.f;
        if (n < H) {
            shared = shared_partial ? shared_partial[(int64_t)r * H + n] : 0.f;
            if (!plain) {
                for (int s = 0; s < top_k; ++s) {
                    const int p = r * top_k + s;
                    const int e = topk_ids[p] - expert_base;
                    if (e >= 0 && e < experts_local) routed += __bfloat162float(dw[(int64_t)p * H + n]);
                }
            }
            if (routed_partial) routed_partial[(int64_t)r * H + n] = routed;
        }
        sh[i] = shared;
        sh[per + i] = routed;
    }
    if (routed_partial) return;
    __syncthreads();
    cta_allreduce_f32(comm, channel, sh, plain ? per : 2 * per);
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
        const int r = r0 + i / CB_COLS, n = n0 + i % CB_COLS;
        if (n >= H) continue;
        float v;
        if (plain) v = sh[i];
        else v = bf16_round(bf16_round(sh[per + i]) * scale) + bf16_round(sh[i]);
        out[(int64_t)r * H + n] = __float2bfloat16_rn(v);
    }
}

// Many rows, several GPUs, library all-reduce: what follows the all-reduce of the routed and the shared partial sums of a prefill
// chunk, in one launch:  out = bf16( bf16(bf16(routed) * scale) + bf16(shared) )  -- the last line of moe_combine_kernel.
__global__ void __launch_bounds__(256)
moe_finish_kernel(const float* __restrict__ routed, const float* __restrict__ shared, int64_t n, float scale, bf16* __restrict__ out) {
    GLMB_PDL_PROLOGUE();
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 3 < n) {
        const float4 r = *reinterpret_cast<const float4*>(routed + i), s = *reinterpret_cast<const float4*>(shared + i);
        uint2 packed;
        packed.x = pack_bf16(bf16_round(bf16_round(r.x) * scale) + bf16_round(s.x), bf16_round(bf16_round(r.y) * scale) + bf16_round(s.y));
        packed.y = pack_bf16(bf16_round(bf16_round(r.z) * scale) + bf16_round(s.z), bf16_round(bf16_round(r.w) * scale) + bf16_round(s.w));
        *reinterpret_cast<uint2*>(out + i) = packed;
    } else {
        for (int64_t j = i; j < n; ++j) out[j] = __float2bfloat16_rn(bf16_round(bf16_round(routed[j]) * scale) + bf16_round(shared[j]));
    }
}

GLMB_API int glmb_moe_finish(const float* routed, const float* shared, int64_t n, float scale, void* out, void* stream) {
    if (n < 1 || (reinterpret_cast<uintptr_t>(routed) & 15) || (reinterpret_cast<uintptr_t>(shared) & 15) || (reinterpret_cast<uintptr_t>(out) & 7)) return 1;
    GLMB_LAUNCH(moe_finish_kernel, (unsigned)((n / 4 + 255) / 256 + 1), 256, 0, (cudaStream_t)stream, routed, shared, n, scale, (bf16*)out);
    return (int)cudaGetLastError();
}

// ===================================================================================================
// Host launchers
#define DISPATCH_R(rows, CALL)                                \
    do {                                                      \
        if ((rows) <= 1) { CALL(1); }                         \
        else if ((rows) <= 2) { CALL(2); }                    \
        else if ((rows) <= 4) { CALL(4); }                    \
        else { CALL(8); }                                     \
    } while (0)

// How many warps share one unit of output (a row pair or a gate/up pair) so that about four CTAs land on every SM.
static int pick_ksplit(int units, int K) {
    int ks = 1;
    while (ks < SK_WARPS && units * ks < 148 * 4 * SK_WARPS && K % (ks * 2 * 256) == 0 && K / (ks * 2) >= 512) ks *= 2;
    return ks;
}

static PeerComm single_comm() {
    PeerComm c;
    memset(&c, 0, sizeof(c));
    c.world = 1;
    return c;
}

// x [rows<=8, K] bf16, w [N, K] bf16 -> out [rows, N] (fp32, bf16, or all-reduced bf16).  K % 8 == 0.
// batch > 1 runs `batch` independent problems whose x / w / out start xb / wb / ob elements apart.
GLMB_API int glmb_skinny_bf16(const void* x, int64_t xs, int rows, const void* w, int64_t ws, int N, int K, void* out, int64_t os,
                              int mode, int batch, int64_t xb, int64_t wb, int64_t ob, const PeerComm* comm, int channel,
                              void* stream) {
    if (rows < 1 || rows > GLMB_MAX_ROWS || (K & 7) || (xs & 7) || (ws & 7) || (xb & 7) || (wb & 7) || batch < 1) return 1;
    int ks = pick_ksplit(ceil_div(N, 2) * batch, K);
    PeerComm c = comm ? *comm : single_comm();
    // A CTA that all-reduces waits for the same CTA of every peer before it retires.  CTAs beyond the first wave would start only
    // after such a wait and then wait again: keep the grid within one wave (three CTAs per SM fit whatever the row count).
    if (mode == SK_OUT_ALLREDUCE_BF16 && c.world > 1)
        while (ks > 1 && ceil_div(N, (SK_WARPS / ks) * 2) * batch > 148 * 3) ks >>= 1;
    const dim3 grid(ceil_div(N, (SK_WARPS / ks) * 2), batch);
    if (mode == SK_OUT_ALLREDUCE_BF16 && c.world > 1 && (int)(grid.x * grid.y) > GLMB_AR_MAX_CTAS) return 2;
    if (mode == SK_OUT_ALLREDUCE_BF16 && c.world == 1) mode = SK_OUT_BF16;
#define CALL(RR)                                                                                                   \
    GLMB_LAUNCH(skinny_bf16_kernel<RR>, grid, SK_THREADS, 0, (cudaStream_t)stream, (const bf16*)x, xs, rows, (const bf16*)w, ws, N, K, \
                                                                          out, os, mode, ks, xb, wb, ob, c, channel)
    DISPATCH_R(rows, CALL);
#undef CALL
    return (int)cudaGetLastError();
}

GLMB_API int glmb_skinny_bf16_swiglu(const void* x, int64_t xs, int rows, const void* wg, const void* wu, int64_t ws, int N, int K,
                                     void* act, int64_t as, void* stream) {
    if (rows < 1 || rows > GLMB_MAX_ROWS || (K & 7) || (xs & 7) || (ws & 7)) return 1;
    const int ks = pick_ksplit(N, K);
    const int grid = ceil_div(N, SK_WARPS / ks);
#define CALL(RR)                                                                                                          \
    GLMB_LAUNCH(skinny_bf16_swiglu_kernel<RR>, grid, SK_THREADS, 0, (cudaStream_t)stream, (const bf16*)x, xs, rows, (const bf16*)wg, \
                                                                                 (const bf16*)wu, ws, N, K, (bf16*)act, as, ks)
    DISPATCH_R(rows, CALL);
#undef CALL
    return (int)cudaGetLastError();
}

// Tensor-core variants (moe_gemv_mma.cu), used when the shapes are whole 64-wide k chunks and 16-row panels.
int glmb_launch_moe_gateup_mma(const void* x, int64_t xs, int top_k, const int* tile_expert, const int* tile_routes, const int* n_tiles,
                               int tiles, int rt, const void* wg, const void* wu, const float* sg, const float* su, int expert_base,
                               int experts_local, int I, int H, void* act, cudaStream_t stream);
int glmb_launch_moe_down_mma(const void* act, const float* route_weight, const int* tile_expert, const int* tile_routes, const int* n_tiles,
                             int tiles, int rt, const void* wd, const float* sd, int expert_base, int experts_local, int I, int H, void* dw,
                             cudaStream_t stream);
static int g_moe_mma = 1;
// The fp32-FMA kernels below serve the shapes the mma.sync kernels refuse (hidden size not a multiple of 64, intermediate not a
// multiple of 16, unaligned rows: fixtures).  The switch exists so that the tests can run BOTH families on shapes both take
// (tests/test_gpu_ops.py::test_routed_experts); nothing in the product turns it off.
GLMB_API void glmb_set_moe_mma(int enabled) { g_moe_mma = enabled ? 1 : 0; }

// Routed gate/up for `tiles` tiles of `rt` routes (rt in {1, 8}).  H % 16 == 0.
GLMB_API int glmb_moe_gateup_fp8(const void* x, int64_t xs, int top_k, const int* tile_expert, const int* tile_routes,
                                 const int* n_tiles, int tiles, int rt, const void* wg, const void* wu, const float* sg,
                                 const float* su, int expert_base, int experts_local, int I, int H, void* act, void* stream) {
    if ((H & 15) || tiles < 1) return 1;
    if (g_moe_mma && (rt == 1 || rt == 8) && !(H & 63) && !(I & 15) && !(xs & 7))
        return glmb_launch_moe_gateup_mma(x, xs, top_k, tile_expert, tile_routes, n_tiles, tiles, rt, wg, wu, sg, su, expert_base,
                                          experts_local, I, H, act, (cudaStream_t)stream);
    dim3 grid(ceil_div(I, SK_WARPS), tiles);
    if (rt == 1)
        GLMB_LAUNCH(moe_gateup_fp8_kernel<1>, grid, SK_THREADS, 0, (cudaStream_t)stream, 
            (const bf16*)x, xs, top_k, tile_expert, tile_routes, n_tiles, (const uint8_t*)wg, (const uint8_t*)wu, sg, su,
            expert_base, experts_local, I, H, (bf16*)act);
    else if (rt == 8)
        GLMB_LAUNCH(moe_gateup_fp8_kernel<8>, grid, SK_THREADS, 0, (cudaStream_t)stream, 
            (const bf16*)x, xs, top_k, tile_expert, tile_routes, n_tiles, (const uint8_t*)wg, (const uint8_t*)wu, sg, su,
            expert_base, experts_local, I, H, (bf16*)act);
    else
        return 1;
    return (int)cudaGetLastError();
}

GLMB_API int glmb_moe_down_fp8(const void* act, const float* route_weight, const int* tile_expert, const int* tile_routes,
                               const int* n_tiles, int tiles, int rt, const void* wd, const float* sd, int expert_base,
                               int experts_local, int I, int H, void* dw, void* stream) {
    if ((I & 15) || tiles < 1) return 1;
    if (g_moe_mma && (rt == 1 || rt == 8) && !(I & 63) && !(H & 15))
        return glmb_launch_moe_down_mma(act, route_weight, tile_expert, tile_routes, n_tiles, tiles, rt, wd, sd, expert_base, experts_local,
                                        I, H, dw, (cudaStream_t)stream);
    dim3 grid(ceil_div(H, SK_WARPS * 2), tiles);
    if (rt == 1)
        GLMB_LAUNCH(moe_down_fp8_kernel<1>, grid, SK_THREADS, 0, (cudaStream_t)stream, (const bf16*)act, route_weight, tile_expert, tile_routes,
                                                                             n_tiles, (const uint8_t*)wd, sd, expert_base,
                                                                             experts_local, I, H, (bf16*)dw);
    else if (rt == 8)
        GLMB_LAUNCH(moe_down_fp8_kernel<8>, grid, SK_THREADS, 0, (cudaStream_t)stream, (const bf16*)act, route_weight, tile_expert, tile_routes,
                                                                             n_tiles, (const uint8_t*)wd, sd, expert_base,
                                                                             experts_local, I, H, (bf16*)dw);
    else
        return 1;
    return (int)cudaGetLastError();
}

// Any number of rows when the exchange is off (world == 1 or routed_partial given); with the in-kernel
// all-reduce the grid must fit the per-CTA flag table.
GLMB_API int glmb_moe_combine(const void* dw, const int* topk_ids, const float* shared_partial, int rows, int top_k, int H,
                              int expert_base, int experts_local, float scale, int plain, void* out, float* routed_partial,
                              const PeerComm* comm, int channel, void* stream) {
    if (rows < 1) return 1;
    dim3 grid(ceil_div(H, CB_COLS), ceil_div(rows, GLMB_MAX_ROWS));
    PeerComm c = comm ? *comm : single_comm();
    if (c.world > 1 && !routed_partial && (int)(grid.x * grid.y) > GLMB_AR_MAX_CTAS) return 2;
    GLMB_LAUNCH(moe_combine_kernel, grid, 128, 0, (cudaStream_t)stream, (const bf16*)dw, topk_ids, shared_partial, rows, top_k, H, expert_base,
                                                               experts_local, scale, plain, (bf16*)out, routed_partial, c, channel);
    return (int)cudaGetLastError();
}
