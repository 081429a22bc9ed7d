// Per-warp inner loops of the weight-streaming (1..8 row) projections, shared by the stand-alone skinny kernels
// (gemv.cu) and the persistent decode kernel (decode_mega.cu).  A warp owns NPW weight rows over a K range: every
// lane streams 16-byte pieces (L1 no-allocate), multiplies them with the R activation rows in fp32 and the warp
// reduces with the xor tree of warp_sum, so every caller gets the same bits for the same (rows, K range).
#pragma once

#include "common.cuh"

// ---------------------------------------------------------------------------------------------------
// Per-warp dot products.  acc[j][r] accumulates this lane's share of  sum_k w_j[k] * x_r[k].
template <int R, int NPW>
__device__ __forceinline__ void warp_dot_bf16(const bf16* const (&xr)[R], const bf16* const (&wp)[NPW], int kbeg, int kend,
                                              int lane, float (&acc)[NPW][R]) {
#pragma unroll (R * NPW <= 4 ? 4 : 2)
    for (int k = kbeg + lane * 8; k < kend; k += 256) {
        float wf[NPW][8];
#pragma unroll
        for (int j = 0; j < NPW; ++j) {
            const uint4 v = ld_stream16(wp[j] + k);
            wf[j][0] = bf16_lo(v.x); wf[j][1] = bf16_hi(v.x); wf[j][2] = bf16_lo(v.y); wf[j][3] = bf16_hi(v.y);
            wf[j][4] = bf16_lo(v.z); wf[j][5] = bf16_hi(v.z); wf[j][6] = bf16_lo(v.w); wf[j][7] = bf16_hi(v.w);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint4 v = ld_hot16(xr[r] + k);
            const float xf[8] = {bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y),
                                 bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w)};
#pragma unroll
            for (int j = 0; j < NPW; ++j)
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[j][r] = fmaf(wf[j][i], xf[i], acc[j][r]);
        }
    }
}

// FP8 (e4m3 + 128x128 fp32 block scales).  sp[j] points at the scale row of weight row j (K/128 entries).
template <int R, int NPW>
__device__ __forceinline__ void warp_dot_fp8(const bf16* const (&xr)[R], const uint8_t* const (&wp)[NPW],
                                             const float* const (&sp)[NPW], int K, int lane, float (&acc)[NPW][R]) {
#pragma unroll (R * NPW <= 2 ? 4 : 2)
    for (int k = lane * 16; k < K; k += 512) {
        float wf[NPW][16];
#pragma unroll
        for (int j = 0; j < NPW; ++j) {
            const uint4 v = ld_stream16(wp[j] + k);
            const float s = __ldg(sp[j] + (k >> 7));
            const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float2 a = decode_e4m3x2(words[q], s);
                const float2 b = decode_e4m3x2(words[q] >> 16, s);
                wf[j][4 * q + 0] = a.x; wf[j][4 * q + 1] = a.y; wf[j][4 * q + 2] = b.x; wf[j][4 * q + 3] = b.y;
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint4 v0 = ld_hot16(xr[r] + k);
            const uint4 v1 = ld_hot16(xr[r] + k + 8);
            const float xf[16] = {bf16_lo(v0.x), bf16_hi(v0.x), bf16_lo(v0.y), bf16_hi(v0.y), bf16_lo(v0.z), bf16_hi(v0.z),
                                  bf16_lo(v0.w), bf16_hi(v0.w), bf16_lo(v1.x), bf16_hi(v1.x), bf16_lo(v1.y), bf16_hi(v1.y),
                                  bf16_lo(v1.z), bf16_hi(v1.z), bf16_lo(v1.w), bf16_hi(v1.w)};
#pragma unroll
            for (int j = 0; j < NPW; ++j)
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[j][r] = fmaf(wf[j][i], xf[i], acc[j][r]);
        }
    }
}

template <int R, int NPW>
__device__ __forceinline__ void warp_reduce_all(float (&acc)[NPW][R]) {
#pragma unroll
    for (int j = 0; j < NPW; ++j)
#pragma unroll
        for (int r = 0; r < R; ++r) acc[j][r] = warp_sum(acc[j][r]);
}

