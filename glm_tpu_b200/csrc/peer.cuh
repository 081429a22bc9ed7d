// In-kernel collectives over NVLink peer memory (plain P2P stores and loads; no multimem, no TMA multicast).
//
// Every rank owns a *staging* buffer and a *flag* buffer that all peers have mapped (CUDA IPC).  A rank
// only ever WRITES into a peer's staging/flags (push model: NVLink writes are posted) and only READS its
// own.  The protocol is "data stores, system fence, flag store (release)"; the reader spins on its own
// flag with acquire loads under an iteration limit, then reads the data with system-coherent loads.
//
// Flags carry sequence numbers kept in device memory (`seq`), so a captured CUDA graph can be replayed
// any number of times.  All ranks run the same launch sequence, hence agree on every sequence number.
//
// Two primitives:
//   * cta_allreduce_f32: CTA j of every rank sums its slice with CTA j of all peers (per-CTA flags, no
//     grid-wide sync).  Used as the epilogue of K-split GEMVs and of the MoE combine.
//   * grid_signal_peers / cta_wait_signal: a producer kernel pushes data to all peers, its last CTA
//     signals; the consumer kernel (later in each rank's stream) waits in its prologue.  Used for the
//     query all-gather, the indexer-score all-gather, the attention partial exchange and the sampler.
//
// Buffer reuse is safe because consecutive users of the same all-reduce channel are always separated by
// an all-reduce on the other channel, and consecutive rounds of a signal are separated by an all-reduce:
// a rank can only get one exchange ahead of its slowest peer.
//
// A wait that runs out sets GLMB_STATUS_WAIT_TIMEOUT in the status word and the kernel continues with
// whatever data is there; the host reads the status after the step and poisons the engine.
#pragma once

#include "common.cuh"

#define GLMB_AR_CHANNELS 2
#define GLMB_AR_MAX_CTAS 1024
#define GLMB_AR_SLICE 256  // fp32 values one CTA may reduce
#define GLMB_SIGNALS 16

// Offsets (in uint32 words) inside the flag buffer and the local sequence buffer.
#define GLMB_FLAG_AR_WORDS (GLMB_AR_CHANNELS * GLMB_AR_MAX_CTAS * GLMB_MAX_WORLD)
#define GLMB_FLAG_SIG_BASE GLMB_FLAG_AR_WORDS
#define GLMB_GEMM_MAX_TILES 16384  // 32-column blocks of the output tiles of one GEMM with a fused all-reduce: one flag per (block, source rank)
#define GLMB_FLAG_GEMM_BASE (GLMB_FLAG_SIG_BASE + GLMB_SIGNALS * GLMB_MAX_WORLD)
#define GLMB_FLAG_WORDS (GLMB_FLAG_GEMM_BASE + GLMB_GEMM_MAX_TILES * GLMB_MAX_WORLD)
#define GLMB_SEQ_AR_WORDS (GLMB_AR_CHANNELS * GLMB_AR_MAX_CTAS)
#define GLMB_SEQ_SIG_BASE GLMB_SEQ_AR_WORDS
#define GLMB_SEQ_DONE_BASE (GLMB_SEQ_SIG_BASE + GLMB_SIGNALS)
#define GLMB_SEQ_GEMM (GLMB_SEQ_DONE_BASE + GLMB_SIGNALS)  // number of fused GEMM all-reduces completed
#define GLMB_SEQ_WORDS (GLMB_SEQ_GEMM + 1)
// Bytes at the start of the staging buffer reserved for the all-reduce channels: one (value, sequence number) pair per fp32 value.
#define GLMB_AR_BYTES ((size_t)GLMB_AR_CHANNELS * GLMB_AR_MAX_CTAS * GLMB_MAX_WORLD * GLMB_AR_SLICE * 8)
// How a CTA's all-reduce hands its values to the peers (PeerComm::protocol).
#define GLMB_AR_FENCE_FLAG 0  // values, system fence, one flag per (CTA, source rank) with release; the reader acquires the flag
#define GLMB_AR_PAIRS 1       // every value travels as an 8-byte (value, sequence number) pair: no fence, no separate flag

struct PeerComm {
    int world;
    int rank;
    uint32_t wait_limit;            // iteration limit of every spin
    uint32_t protocol;              // GLMB_AR_FENCE_FLAG or GLMB_AR_PAIRS: the same on every rank
    uint32_t* status;               // local status word
    uint32_t* seq;                  // local sequence numbers [GLMB_SEQ_WORDS]
    char* data[GLMB_MAX_WORLD];     // data[p]: rank p's staging buffer as mapped here
    uint32_t* flags[GLMB_MAX_WORLD];  // flags[p]: rank p's flag buffer as mapped here
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float ld_sys_f32(const float* p) {
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_sys_u4(const void* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

__device__ __forceinline__ void st_sys_u2(void* p, uint32_t a, uint32_t b) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ uint2 ld_sys_u2(const void* p) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

// Spin until *p has reached `expect` (sequence numbers only grow).  Returns false when the limit ran out.
__device__ __forceinline__ bool wait_flag_reached(const uint32_t* p, uint32_t expect, uint32_t limit) {
    for (uint32_t i = 0; i < limit; ++i) {
        if ((int32_t)(ld_acquire_sys(p) - expect) >= 0) return true;
        if (i > 128) __nanosleep(64);
    }
    return false;
}

// Sum `count` fp32 values held in shared memory `sh` over all ranks, in rank order (bitwise identical on
// every rank).  Every thread of the CTA must call it; count <= GLMB_AR_SLICE; blockDim.x >= world.
// `cta` (< GLMB_AR_MAX_CTAS) names the exchange slot: the same number on every rank for the same slice.
__device__ __forceinline__ void cta_allreduce_f32_slot(const PeerComm& c, int channel, int cta, float* sh, int count) {
    if (c.world == 1) return;
    __shared__ uint32_t s_epoch;
    const int slot = channel * GLMB_AR_MAX_CTAS + cta;
    if (threadIdx.x == 0) s_epoch = c.seq[slot] + 1;
    __syncthreads();
    const uint32_t e = s_epoch;
    const size_t mine = ((size_t)slot * GLMB_MAX_WORLD + c.rank) * GLMB_AR_SLICE;
    if (c.protocol == GLMB_AR_PAIRS) {
        // An aligned 8-byte store lands whole, so the sequence number beside a value says that the value is this round's: the
        // sender neither fences nor raises a flag, and the reader polls the very words it is going to add.  One NVLink crossing
        // instead of the fence's round trip plus the flag's crossing.
        for (int i = threadIdx.x; i < count; i += blockDim.x) {
            const uint32_t bits = __float_as_uint(sh[i]);
            for (int p = 0; p < c.world; ++p)
                if (p != c.rank) st_sys_u2(reinterpret_cast<uint2*>(c.data[p]) + mine + i, bits, e);
        }
        const uint2* inbox = reinterpret_cast<const uint2*>(c.data[c.rank]) + (size_t)slot * GLMB_MAX_WORLD * GLMB_AR_SLICE;
        bool late = false;
        for (int i = threadIdx.x; i < count; i += blockDim.x) {
            // fully unrolled over the largest world so that the arrived values stay in registers
            float vals[GLMB_MAX_WORLD];
            uint32_t pending = ((1u << c.world) - 1u) & ~(1u << c.rank);
            for (uint32_t it = 0; pending && it < c.wait_limit; ++it) {
#pragma unroll
                for (int p = 0; p < GLMB_MAX_WORLD; ++p) {
                    if (pending >> p & 1u) {
                        const uint2 v = ld_sys_u2(inbox + (size_t)p * GLMB_AR_SLICE + i);
                        if (v.y == e) { vals[p] = __uint_as_float(v.x); pending &= ~(1u << p); }
                    }
                }
                if (it > 128) __nanosleep(64);
            }
            if (pending) late = true;
            float sum = 0.f;
#pragma unroll
            for (int p = 0; p < GLMB_MAX_WORLD; ++p)
                if (p < c.world) sum += (p == c.rank) ? sh[i] : ((pending >> p & 1u) ? 0.f : vals[p]);
            sh[i] = sum;
        }
        if (late) raise_status(c.status, GLMB_STATUS_WAIT_TIMEOUT);
        if (threadIdx.x == 0) c.seq[slot] = e;
        __syncthreads();
        return;
    }
    for (int p = 0; p < c.world; ++p) {
        if (p == c.rank) continue;
        float* dst = reinterpret_cast<float*>(c.data[p]) + mine;
        for (int i = threadIdx.x; i < count; i += blockDim.x) dst[i] = sh[i];
    }
    __threadfence_system();
    __syncthreads();
    if ((int)threadIdx.x < c.world && (int)threadIdx.x != c.rank) {
        const int p = threadIdx.x;
        st_release_sys(c.flags[p] + (size_t)slot * GLMB_MAX_WORLD + c.rank, e);
        if (!wait_flag_reached(c.flags[c.rank] + (size_t)slot * GLMB_MAX_WORLD + p, e, c.wait_limit))
            raise_status(c.status, GLMB_STATUS_WAIT_TIMEOUT);
    }
    __syncthreads();
    const float* inbox = reinterpret_cast<const float*>(c.data[c.rank]) + (size_t)slot * GLMB_MAX_WORLD * GLMB_AR_SLICE;
    for (int i = threadIdx.x; i < count; i += blockDim.x) {
        float sum = 0.f;
        for (int p = 0; p < c.world; ++p) sum += (p == c.rank) ? sh[i] : ld_sys_f32(inbox + (size_t)p * GLMB_AR_SLICE + i);
        sh[i] = sum;
    }
    if (threadIdx.x == 0) c.seq[slot] = e;
    __syncthreads();
}

// The slot is this CTA's index in its grid.
__device__ __forceinline__ void cta_allreduce_f32(const PeerComm& c, int channel, float* sh, int count) {
    cta_allreduce_f32_slot(c, channel, blockIdx.x + blockIdx.y * gridDim.x, sh, count);
}

// Producer side of a signal: call once per CTA after the CTA's pushes.  The last CTA of the grid bumps the
// signal's sequence number and writes it into every rank's flag (its own included).
__device__ __forceinline__ void grid_signal_peers(const PeerComm& c, int sig) {
    if (c.world == 1) return;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned total = gridDim.x * gridDim.y * gridDim.z;
        uint32_t* done = c.seq + GLMB_SEQ_DONE_BASE + sig;
        if (atomicAdd(done, 1u) == total - 1) {
            __threadfence_system();
            atomicExch(done, 0u);
            const uint32_t e = c.seq[GLMB_SEQ_SIG_BASE + sig] + 1;
            c.seq[GLMB_SEQ_SIG_BASE + sig] = e;
            for (int p = 0; p < c.world; ++p)
                st_release_sys(c.flags[p] + GLMB_FLAG_SIG_BASE + sig * GLMB_MAX_WORLD + c.rank, e);
        }
    }
}

// Consumer side: the producer kernel of this rank ran earlier in the stream, so seq[sig] already holds the
// round's number; wait until every rank's flag has reached it.  Every thread of the CTA must call it.
__device__ __forceinline__ void cta_wait_signal(const PeerComm& c, int sig) {
    if (c.world == 1) return;
    if ((int)threadIdx.x < c.world) {
        const uint32_t e = c.seq[GLMB_SEQ_SIG_BASE + sig];
        if (!wait_flag_reached(c.flags[c.rank] + GLMB_FLAG_SIG_BASE + sig * GLMB_MAX_WORLD + threadIdx.x, e, c.wait_limit))
            raise_status(c.status, GLMB_STATUS_WAIT_TIMEOUT);
    }
    __syncthreads();
}
