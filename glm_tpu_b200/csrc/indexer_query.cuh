// The N operand of the tcgen05 indexers: an fp32 index query split exactly into three bf16 pieces.
//
// q = hi + mid + lo with hi = bf16(q), mid = bf16(q - hi), lo = bf16(q - hi - mid): the residuals are exact in fp32, so the
// three pieces reproduce q to 2^-24 of its magnitude, and because bf16 x bf16 products are exact in fp32 the three partial dot
// products against bf16 keys add up to the fp32-accurate q . key.  When the query comes straight from the q_b projection, the
// first rd features of every head are rotated here first (interleaved pairs, fp32 angle = position * inv_freq: the arithmetic
// of the q_post kernel, so both routes give the same bits).
#pragma once

#include "common.cuh"

struct IndexerQuerySource {
    const float* q;         // [rows, q_stride] fp32, index head h at q_offset + h * D
    int64_t q_stride, q_offset;
    const float* inv_freq;  // [rd / 2]: rotate here; null: the query is already rotated
    int rd;
};

// Eight consecutive features (chunk c8 of head h, D features per head) of row r at position pos -> three packed bf16 octets.
__device__ __forceinline__ void indexer_query_pieces(const IndexerQuerySource& src, int r, int h, int c8, int D, int pos, uint4 (&piece)[3]) {
    const float* q = src.q + (int64_t)r * src.q_stride + src.q_offset + h * D + c8 * 8;
    const float4 x0 = *reinterpret_cast<const float4*>(q);
    const float4 x1 = *reinterpret_cast<const float4*>(q + 4);
    float v[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
    if (src.inv_freq && c8 * 8 < src.rd) {
#pragma unroll
        for (int pr = 0; pr < 4; ++pr) {
            const int d = c8 * 8 + 2 * pr;
            if (d < src.rd) {
                const float angle = __fmul_rn((float)pos, src.inv_freq[d >> 1]);
                const float cs = cosf(angle), sn = sinf(angle);
                const float even = v[2 * pr], odd = v[2 * pr + 1];
                v[2 * pr] = __fsub_rn(__fmul_rn(even, cs), __fmul_rn(odd, sn));
                v[2 * pr + 1] = __fadd_rn(__fmul_rn(odd, cs), __fmul_rn(even, sn));
            }
        }
    }
    float hi[8], mid[8], lo[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        hi[e] = bf16_round(v[e]);
        const float r1 = v[e] - hi[e];
        mid[e] = bf16_round(r1);
        lo[e] = bf16_round(r1 - mid[e]);
    }
    piece[0] = make_uint4(pack_bf16(hi[0], hi[1]), pack_bf16(hi[2], hi[3]), pack_bf16(hi[4], hi[5]), pack_bf16(hi[6], hi[7]));
    piece[1] = make_uint4(pack_bf16(mid[0], mid[1]), pack_bf16(mid[2], mid[3]), pack_bf16(mid[4], mid[5]), pack_bf16(mid[6], mid[7]));
    piece[2] = make_uint4(pack_bf16(lo[0], lo[1]), pack_bf16(lo[2], lo[3]), pack_bf16(lo[4], lo[5]), pack_bf16(lo[6], lo[7]));
}
