// Peer-buffer registry: the B200 replacement of the reference's device mesh (`glm_tpu/distributed/mesh.py`).
//
// Every rank (one process per GPU) allocates a staging buffer, a flag buffer, a sequence buffer and a status
// word with cudaMalloc, exports the first two as CUDA IPC handles, and maps its peers' handles.  The table
// of mapped pointers (PeerComm) is passed by value to every kernel that communicates.  NVLink peer access
// is enabled lazily by cudaIpcOpenMemHandle.  No multicast object is created: the kernels use plain peer
// stores and loads only.
//
// The handle exchange itself (64 opaque bytes per buffer per rank) is done by the Python side over the
// process group's store; this file only allocates, exports, maps and unmaps.
#include "common.cuh"
#include "peer.cuh"

#include <string.h>

struct PeerRegistry {
    int world, rank;
    size_t data_bytes;
    char* data;
    uint32_t* flags;
    uint32_t* seq;
    uint32_t* status;
    void* peer_data[GLMB_MAX_WORLD];
    void* peer_flags[GLMB_MAX_WORLD];
    bool mapped[GLMB_MAX_WORLD];
};

GLMB_API size_t glmb_peer_ar_bytes(void) { return GLMB_AR_BYTES; }
GLMB_API size_t glmb_peer_comm_sizeof(void) { return sizeof(PeerComm); }
GLMB_API int glmb_peer_signals(void) { return GLMB_SIGNALS; }

// data_bytes: total staging size (the first glmb_peer_ar_bytes() are reserved for the all-reduce channels).
GLMB_API int glmb_peer_create(int world, int rank, size_t data_bytes, PeerRegistry** out) {
    if (world < 1 || world > GLMB_MAX_WORLD || rank < 0 || rank >= world || data_bytes < GLMB_AR_BYTES) return 1;
    PeerRegistry* r = new PeerRegistry();
    memset(r, 0, sizeof(*r));
    r->world = world;
    r->rank = rank;
    r->data_bytes = data_bytes;
    cudaError_t e;
    if ((e = cudaMalloc(&r->data, data_bytes)) != cudaSuccess) { delete r; return (int)e; }
    if ((e = cudaMalloc(&r->flags, GLMB_FLAG_WORDS * sizeof(uint32_t))) != cudaSuccess) { cudaFree(r->data); delete r; return (int)e; }
    if ((e = cudaMalloc(&r->seq, (GLMB_SEQ_WORDS + 1) * sizeof(uint32_t))) != cudaSuccess) {
        cudaFree(r->data); cudaFree(r->flags); delete r; return (int)e;
    }
    r->status = r->seq + GLMB_SEQ_WORDS;
    cudaMemset(r->data, 0, data_bytes);
    cudaMemset(r->flags, 0, GLMB_FLAG_WORDS * sizeof(uint32_t));
    cudaMemset(r->seq, 0, (GLMB_SEQ_WORDS + 1) * sizeof(uint32_t));
    cudaDeviceSynchronize();
    r->peer_data[rank] = r->data;
    r->peer_flags[rank] = r->flags;
    *out = r;
    return 0;
}

// handles: 128 bytes = data handle (64) followed by flag handle (64).
GLMB_API int glmb_peer_export(PeerRegistry* r, unsigned char* handles) {
    cudaIpcMemHandle_t h;
    cudaError_t e;
    if ((e = cudaIpcGetMemHandle(&h, r->data)) != cudaSuccess) return (int)e;
    memcpy(handles, &h, sizeof(h));
    if ((e = cudaIpcGetMemHandle(&h, r->flags)) != cudaSuccess) return (int)e;
    memcpy(handles + 64, &h, sizeof(h));
    return 0;
}

GLMB_API int glmb_peer_import(PeerRegistry* r, int peer, const unsigned char* handles) {
    if (peer < 0 || peer >= r->world || peer == r->rank || r->mapped[peer]) return 1;
    cudaIpcMemHandle_t h;
    cudaError_t e;
    memcpy(&h, handles, sizeof(h));
    if ((e = cudaIpcOpenMemHandle(&r->peer_data[peer], h, cudaIpcMemLazyEnablePeerAccess)) != cudaSuccess) return (int)e;
    memcpy(&h, handles + 64, sizeof(h));
    if ((e = cudaIpcOpenMemHandle(&r->peer_flags[peer], h, cudaIpcMemLazyEnablePeerAccess)) != cudaSuccess) {
        cudaIpcCloseMemHandle(r->peer_data[peer]);
        return (int)e;
    }
    r->mapped[peer] = true;
    return 0;
}

// Which protocol the all-reduces of communicators handed out from now on use (GLMB_AR_*); every rank must choose the same.
static int g_ar_protocol = GLMB_AR_PAIRS;
GLMB_API void glmb_set_ar_protocol(int protocol) { g_ar_protocol = protocol == GLMB_AR_FENCE_FLAG ? GLMB_AR_FENCE_FLAG : GLMB_AR_PAIRS; }
GLMB_API int glmb_get_ar_protocol(void) { return g_ar_protocol; }

GLMB_API int glmb_peer_comm(PeerRegistry* r, uint32_t wait_limit, PeerComm* out) {
    memset(out, 0, sizeof(*out));
    out->world = r->world;
    out->rank = r->rank;
    out->wait_limit = wait_limit;
    out->protocol = (uint32_t)g_ar_protocol;
    out->status = r->status;
    out->seq = r->seq;
    for (int p = 0; p < r->world; ++p) {
        if (p != r->rank && !r->mapped[p]) return 1;
        out->data[p] = (char*)r->peer_data[p];
        out->flags[p] = (uint32_t*)r->peer_flags[p];
    }
    return 0;
}

GLMB_API void* glmb_peer_data(PeerRegistry* r) { return r->data; }
GLMB_API void* glmb_peer_status_ptr(PeerRegistry* r) { return r->status; }

// Read (and optionally clear) the status word.  Synchronizes the given stream first.
GLMB_API int glmb_peer_read_status(PeerRegistry* r, int clear, void* stream, uint32_t* value) {
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return (int)e;
    if ((e = cudaMemcpy(value, r->status, sizeof(uint32_t), cudaMemcpyDeviceToHost)) != cudaSuccess) return (int)e;
    if (clear && *value) cudaMemset(r->status, 0, sizeof(uint32_t));
    return 0;
}

GLMB_API int glmb_peer_destroy(PeerRegistry* r) {
    if (!r) return 0;
    cudaDeviceSynchronize();
    for (int p = 0; p < r->world; ++p)
        if (r->mapped[p]) { cudaIpcCloseMemHandle(r->peer_data[p]); cudaIpcCloseMemHandle(r->peer_flags[p]); }
    cudaFree(r->data);
    cudaFree(r->flags);
    cudaFree(r->seq);
    delete r;
    return 0;
}

// ---------------------------------------------------------------------------------------------------
// Self-test kernels for the wait primitive: a wait on a flag that nothing sets must give up after the
// iteration limit, set the status word and return (the context stays usable).
__global__ void wait_probe_kernel(PeerComm c, int sig, uint32_t bump) {
    GLMB_PDL_PROLOGUE();
    if (threadIdx.x == 0 && bump) c.seq[GLMB_SEQ_SIG_BASE + sig] += bump;  // expect a round nobody signalled
    __syncthreads();
    // force the wait path even with one rank
    if ((int)threadIdx.x < c.world) {
        const uint32_t e = c.seq[GLMB_SEQ_SIG_BASE + sig];
        if (!wait_flag_reached(c.flags[c.rank] + GLMB_FLAG_SIG_BASE + sig * GLMB_MAX_WORLD + threadIdx.x, e, c.wait_limit))
            raise_status(c.status, GLMB_STATUS_WAIT_TIMEOUT);
    }
    __syncthreads();
    if (threadIdx.x == 0 && bump) {
        // put the books back so later rounds stay aligned
        c.seq[GLMB_SEQ_SIG_BASE + sig] -= bump;
    }
}

GLMB_API int glmb_peer_wait_probe(const PeerComm* comm, int sig, uint32_t bump, void* stream) {
    GLMB_LAUNCH(wait_probe_kernel, 1, 32, 0, (cudaStream_t)stream, *comm, sig, bump);
    return (int)cudaGetLastError();
}

// Consumer side of a signal as a kernel of its own: later kernels of the stream start after every rank's round of
// `sig` has arrived (used after a GEMM with a fused all-reduce, whose consumers are ordinary kernels).
__global__ void wait_signal_kernel(PeerComm c, int sig) {
    GLMB_PDL_PROLOGUE();
    cta_wait_signal(c, sig);
}

GLMB_API int glmb_wait_signal(const PeerComm* comm, int sig, void* stream) {
    if (!comm || sig < 0 || sig >= GLMB_SIGNALS) return 1;
    GLMB_LAUNCH(wait_signal_kernel, 1, 32, 0, (cudaStream_t)stream, *comm, sig);
    return (int)cudaGetLastError();
}

// All-reduce self-test: every rank contributes `count` floats; result (identical on all ranks) in `out`.
__global__ void allreduce_probe_kernel(const float* in, float* out, int count, PeerComm c, int channel) {
    GLMB_PDL_PROLOGUE();
    __shared__ float sh[GLMB_AR_SLICE];
    const int base = blockIdx.x * GLMB_AR_SLICE;
    const int n = min(GLMB_AR_SLICE, count - base);
    for (int i = threadIdx.x; i < n; i += blockDim.x) sh[i] = in[base + i];
    __syncthreads();
    cta_allreduce_f32(c, channel, sh, n);
    for (int i = threadIdx.x; i < n; i += blockDim.x) out[base + i] = sh[i];
}

GLMB_API int glmb_peer_allreduce_probe(const float* in, float* out, int count, const PeerComm* comm, int channel, void* stream) {
    const int grid = ceil_div(count, GLMB_AR_SLICE);
    if (grid > GLMB_AR_MAX_CTAS) return 1;
    GLMB_LAUNCH(allreduce_probe_kernel, grid, 128, 0, (cudaStream_t)stream, in, out, count, *comm, channel);
    return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------
// Library-wide launch mode (see GLMB_PDL_PROLOGUE in common.cuh).
int g_glmb_pdl_enabled = 1;
GLMB_API void glmb_set_pdl(int enabled) { g_glmb_pdl_enabled = enabled ? 1 : 0; }
GLMB_API int glmb_get_pdl(void) { return g_glmb_pdl_enabled; }
