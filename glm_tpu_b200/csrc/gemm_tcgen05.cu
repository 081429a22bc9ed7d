// Dense and grouped bf16 GEMM on the 5th-generation tensor cores:  C[rows, N] = A[rows, K] . B[N, K]^T.
//
// One CTA computes a 128 x 128 output tile.  Operands are staged by TMA (cp.async.bulk.tensor, 128-byte swizzle,
// no multicast) through a 4-stage ring of shared-memory buffers guarded by full/empty mbarriers; one elected
// thread issues tcgen05.mma (kind::f16, bf16 inputs, fp32 accumulate) into a 128-lane x 128-column TMEM
// accumulator; four epilogue warps read it back with tcgen05.ld, round to bf16 (or keep fp32) and store.
//
//   warp 0      TMA producer (one elected lane)
//   warp 1      TMEM allocation, MMA issue (one elected lane), TMEM release
//   warps 2-5   epilogue: warp w owns TMEM lanes 32*(w%4) .. +31
//
// Grouped mode (routed experts in prefill): `tiles` lists (first row, end row, expert) per 128-row tile of the
// expert-sorted activation buffer; the weight tile of expert e starts at row e*N of B viewed as [E*N, K]; rows
// past `end row` are computed but not stored.
//
// Every mbarrier wait is bounded: when the limit runs out the kernel raises GLMB_STATUS_WAIT_TIMEOUT, stops
// issuing work, and still releases its TMEM before it returns.
//
// Replaces reference `glm_tpu/kernels/fp8_grouped_matmul/panel_kernel.py:31-153` (prefill expert panels, after the
// load-time style decode of the FP8 tables to bf16) and the prefill projections of `layers/linear.py:89-128`.
#include "common.cuh"

#include <cuda.h>
#include <mutex>

#define TC_BM 128
#define TC_BN 128
#define TC_BK 64
#define TC_STAGES 4
#define TC_UMMA_K 16
#define TC_THREADS 192
#define TC_TMEM_COLS 128
#define TC_STAGE_BYTES ((TC_BM + TC_BN) * TC_BK * 2)
#define TC_SMEM_BYTES (TC_STAGES * TC_STAGE_BYTES + 1024 + 256)
#define TC_WAIT_LIMIT 4000000u

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded parity wait.  Returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < TC_WAIT_LIMIT; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// K-major operand tile, 128-byte swizzle: rows are 128 bytes, 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16: D fp32, A and B bf16, both K-major, M = 128, N = 128.
__device__ __forceinline__ constexpr uint32_t umma_idesc_bf16_128x128() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TC_BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct TcTile { int row0, row_end, expert, pad; };

// tiles == nullptr: dense GEMM, tile t covers rows 128 t .. of `rows` rows.  out_f32: store fp32 instead of bf16.
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, void* __restrict__ c,
                         int64_t ldc, int rows, int N, int K, const TcTile* __restrict__ tiles, const int* __restrict__ n_tiles,
                         int out_f32, uint32_t* status) {
    GLMB_PDL_PROLOGUE();
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte alignment of the operand ring is required by the 128-byte swizzle
    unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(ring + TC_STAGES * TC_STAGE_BYTES);
    uint64_t* empty_bar = full_bar + TC_STAGES;
    uint64_t* acc_bar = empty_bar + TC_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
    uint32_t* fail_slot = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.y;
    if (n_tiles && t >= *n_tiles) return;
    int row0, row_end, expert;
    if (tiles) { row0 = tiles[t].row0; row_end = tiles[t].row_end; expert = tiles[t].expert; }
    else { row0 = t * TC_BM; row_end = rows; expert = 0; }
    const int n0 = blockIdx.x * TC_BN;
    const int kblocks = (K + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; ++s) { mbar_init(full_bar + s, 1); mbar_init(empty_bar + s, 1); }
        mbar_init(acc_bar, 1);
        *fail_slot = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < kblocks; ++kb) {
                const int s = kb % TC_STAGES;
                if (kb >= TC_STAGES && !mbar_wait(empty_bar + s, ((kb / TC_STAGES) - 1) & 1)) { *fail_slot = 1; break; }
                unsigned char* a_dst = ring + s * TC_STAGE_BYTES;
                unsigned char* b_dst = a_dst + TC_BM * TC_BK * 2;
                mbar_expect_tx(full_bar + s, TC_STAGE_BYTES);
                tma_load_2d(a_dst, &map_a, full_bar + s, kb * TC_BK, row0);
                tma_load_2d(b_dst, &map_b, full_bar + s, kb * TC_BK, expert * N + n0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_bf16_128x128();
            bool ok = true;
            for (int kb = 0; kb < kblocks && ok; ++kb) {
                const int s = kb % TC_STAGES;
                if (!mbar_wait(full_bar + s, (kb / TC_STAGES) & 1)) { *fail_slot = 1; ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a_addr = smem_u32(ring + s * TC_STAGE_BYTES);
                const uint32_t b_addr = a_addr + TC_BM * TC_BK * 2;
#pragma unroll
                for (int k = 0; k < TC_BK / TC_UMMA_K; ++k) {
                    const uint64_t da = umma_desc_sw128(a_addr + k * TC_UMMA_K * 2);
                    const uint64_t db = umma_desc_sw128(b_addr + k * TC_UMMA_K * 2);
                    umma_bf16(tmem_base, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(empty_bar + s);  // the stage may be refilled once these MMAs have read it
            }
            umma_commit(acc_bar);            // accumulator complete (or abandoned): release the epilogue
        }
    } else {
        // epilogue
        const int quarter = warp & 3;
        const bool ok = mbar_wait(acc_bar, 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (!ok || *reinterpret_cast<volatile uint32_t*>(fail_slot)) {
            if (lane == 0) raise_status(status, GLMB_STATUS_WAIT_TIMEOUT);
        } else {
            const int row = row0 + quarter * 32 + lane;
#pragma unroll
            for (int cb = 0; cb < TC_BN / 32; ++cb) {
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + cb * 32, v);
                const int col = n0 + cb * 32;
                if (row < row_end && col < N) {
                    if (out_f32) {
                        float* dst = reinterpret_cast<float*>(c) + (int64_t)row * ldc + col;
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            if (col + i < N)
                                *reinterpret_cast<float4*>(dst + i) = make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]),
                                                                                  __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
                    } else {
                        bf16* dst = reinterpret_cast<bf16*>(c) + (int64_t)row * ldc + col;
#pragma unroll
                        for (int i = 0; i < 32; i += 8)
                            if (col + i < N) {
                                uint4 o;
                                o.x = pack_bf16(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                                o.y = pack_bf16(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
                                o.z = pack_bf16(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
                                o.w = pack_bf16(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
                                *reinterpret_cast<uint4*>(dst + i) = o;
                            }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TC_TMEM_COLS) : "memory");
    }
}

// ===================================================================================================
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// [rows, K] bf16 row-major (leading dimension ld elements), box 128 rows x 64 columns, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint64_t ld) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return 1;
    const cuuint64_t dims[2] = {K, rows};
    const cuuint64_t strides[1] = {ld * 2};
    const cuuint32_t box[2] = {TC_BK, TC_BM};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 2;
}

// a [rows, K] bf16 (lda), b [experts * N, K] bf16 (ldb), c [rows, N] bf16 or fp32 (ldc).  K % 8 == 0; a, b 16-byte
// aligned with lda, ldb multiples of 8.  tiles / n_tiles: device arrays for grouped mode (max_tiles entries) or NULL.
GLMB_API int glmb_gemm_bf16_tcgen05(const void* a, int64_t lda, const void* b, int64_t ldb, void* c, int64_t ldc, int rows, int N,
                                    int K, int experts, const void* tiles, const int* n_tiles, int max_tiles, int out_f32,
                                    uint32_t* status, void* stream) {
    if (rows < 1 || N < 8 || (N & 7) || K < 8 || (K & 7) || (lda & 7) || (ldb & 7) || (ldc & (out_f32 ? 3 : 7)) || experts < 1) return 1;
    if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) || (reinterpret_cast<uintptr_t>(c) & 15)) return 1;
    CUtensorMap map_a, map_b;
    if (make_map(&map_a, a, (uint64_t)rows, (uint64_t)K, (uint64_t)lda)) return 3;
    if (make_map(&map_b, b, (uint64_t)experts * N, (uint64_t)K, (uint64_t)ldb)) return 3;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    const int tile_rows = tiles ? max_tiles : ceil_div(rows, TC_BM);
    dim3 grid(ceil_div(N, TC_BN), tile_rows);
    GLMB_LAUNCH(gemm_bf16_tcgen05_kernel, grid, TC_THREADS, TC_SMEM_BYTES, (cudaStream_t)stream, map_a, map_b, c, ldc, rows, N, K,
                (const TcTile*)tiles, n_tiles, out_f32, status);
    return (int)cudaGetLastError();
}
