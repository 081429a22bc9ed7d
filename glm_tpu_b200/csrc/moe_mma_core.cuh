// Tensor-core inner step of the FP8 routed-expert projections of the decode step, shared by the stand-alone kernels
// (moe_gemv_mma.cu) and the persistent decode kernel (decode_mega.cu): decoded e4m3 pairs go straight into
// mma.sync m16n8k16 (see moe_gemv_mma.cu for the operand layout).
#pragma once

#include "common.cuh"

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t dec2(uint32_t two_codes, float scale) {
    const float2 f = e4m3x2_to_float2(two_codes);
    return pack_bf16(f.x * scale, f.y * scale);
}

// One 64-wide k chunk of one 16-row weight panel against the activation fragment xv (16 k values of route g).
__device__ __forceinline__ void chunk_mma(float (&acc)[4], const uint4& w_lo, const uint4& w_hi, float scale, const uint4& x0, const uint4& x1) {
    const uint32_t wl[4] = {w_lo.x, w_lo.y, w_lo.z, w_lo.w}, wh[4] = {w_hi.x, w_hi.y, w_hi.z, w_hi.w};
    const uint32_t xw[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
    for (int j = 0; j < 4; ++j)
        mma_16816(acc, dec2(wl[j] & 0xffffu, scale), dec2(wh[j] & 0xffffu, scale), dec2(wl[j] >> 16, scale), dec2(wh[j] >> 16, scale),
                  xw[2 * j], xw[2 * j + 1]);
}

