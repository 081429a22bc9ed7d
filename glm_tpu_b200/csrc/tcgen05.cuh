// Building blocks of the tcgen05 kernels: bounded mbarrier waits, TMA tile loads (never multicast), shared-memory
// matrix descriptors for the 128-byte swizzle, tcgen05.mma / commit / ld wrappers, and the host-side tensor-map
// encoder (resolved through the runtime's driver entry point, so nothing links against libcuda).
#pragma once

#include <mutex>
#include <unordered_map>

#include "common.cuh"

#include <cuda.h>
#include <mutex>

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

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Instruction descriptor, kind::f16: D fp32, A and B bf16, both K-major, tile m x n.
__device__ __forceinline__ constexpr uint32_t umma_idesc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---- host side -------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_tiled() {
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

// A tensor map is a pure function of (element type, base, extents, leading dimension, box): the same workspaces and weight tables
// come back on every layer and every chunk, so the encoded maps are kept (per translation unit, under a mutex) instead of asking
// the driver again for each GEMM call.  The table is emptied when it has grown to 8,192 entries.
struct TensorMapKey {
    int kind;
    const void* base;
    uint64_t rows, K, ld;
    uint32_t box_rows;
    bool operator==(const TensorMapKey& o) const {
        return kind == o.kind && base == o.base && rows == o.rows && K == o.K && ld == o.ld && box_rows == o.box_rows;
    }
};
struct TensorMapKeyHash {
    size_t operator()(const TensorMapKey& k) const {
        size_t h = std::hash<const void*>()(k.base);
        for (uint64_t v : {(uint64_t)k.kind, k.rows, k.K, k.ld, (uint64_t)k.box_rows}) h = h * 1099511628211ull ^ std::hash<uint64_t>()(v);
        return h;
    }
};
template <typename Encode>
static inline int cached_map(CUtensorMap* map, const TensorMapKey& key, Encode encode) {
    static std::mutex mutex;
    static std::unordered_map<TensorMapKey, CUtensorMap, TensorMapKeyHash> table;
    std::lock_guard<std::mutex> lock(mutex);
    auto hit = table.find(key);
    if (hit != table.end()) { *map = hit->second; return 0; }
    const int code = encode(map);
    if (code == 0) {
        if (table.size() >= 8192) table.clear();
        table.emplace(key, *map);
    }
    return code;
}

// [rows, K] bf16 row-major (leading dimension ld elements), box `box_rows` rows x 64 columns, 128-byte swizzle.
static inline int make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint64_t ld, uint32_t box_rows = 128) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return 1;
    return cached_map(map, TensorMapKey{0, base, rows, K, ld, box_rows}, [&](CUtensorMap* out) {
        const cuuint64_t dims[2] = {K, rows};
        const cuuint64_t strides[1] = {ld * 2};
        const cuuint32_t box[2] = {64, box_rows};
        const cuuint32_t elem[2] = {1, 1};
        CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        return r == CUDA_SUCCESS ? 0 : 2;
    });
}


// [rows, K] bytes row-major (leading dimension ld bytes), box `box_rows` rows x 64 bytes, no swizzle: FP8 weight tiles
// that CUDA threads (not the tensor core) read back from shared memory.
static inline int make_map_u8(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint64_t ld, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return 1;
    return cached_map(map, TensorMapKey{1, base, rows, K, ld, box_rows}, [&](CUtensorMap* out) {
        const cuuint64_t dims[2] = {K, rows};
        const cuuint64_t strides[1] = {ld};
        const cuuint32_t box[2] = {64, box_rows};
        const cuuint32_t elem[2] = {1, 1};
        CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        return r == CUDA_SUCCESS ? 0 : 2;
    });
}
