// SwiGLU on whole rows for the prefill path: act = bf16( g * sigmoid(g) * u ) with g, u the bf16 outputs of the gate and up
// GEMMs, computed in fp32 and rounded once (the activation contract; the decode GEMVs and the grouped expert GEMM apply the
// same expression in their epilogues).  One launch instead of six elementwise library launches per layer and chunk.
//
// Reference counterpart: `glm_tpu/layers/mlp.py:21-51`.
#include "common.cuh"

__global__ void __launch_bounds__(256)
swiglu_rows_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up, uint4* __restrict__ act, int64_t n8) {
    GLMB_PDL_PROLOGUE();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
        const uint4 g = gate[i], u = up[i];
        const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
        uint32_t o[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const float g0 = __uint_as_float(gw[p] << 16), g1 = __uint_as_float(gw[p] & 0xffff0000u);
            const float u0 = __uint_as_float(uw[p] << 16), u1 = __uint_as_float(uw[p] & 0xffff0000u);
            o[p] = pack_bf16(g0 * sigmoidf_precise(g0) * u0, g1 * sigmoidf_precise(g1) * u1);
        }
        act[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// gate, up, act: contiguous bf16 arrays of n elements (n % 8 == 0), 16-byte aligned; act may alias gate.
GLMB_API int glmb_swiglu_rows(const void* gate, const void* up, void* act, int64_t n, void* stream) {
    if (n < 8 || (n & 7) || ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(act)) & 15)) return 1;
    const int64_t n8 = n / 8;
    const int64_t blocks = (n8 + 255) / 256;
    const int grid = blocks < 148 * 8 ? (int)blocks : 148 * 8;
    GLMB_LAUNCH(swiglu_rows_kernel, grid, 256, 0, (cudaStream_t)stream, (const uint4*)gate, (const uint4*)up, (uint4*)act, n8);
    return (int)cudaGetLastError();
}
