// Multi-GPU output exchange without a library collective: buffers that every rank of a node can address
// (CUDA IPC), the decode GEMV storing its band of y into all of them (see gemv.cu: GemvParams::ypeer), and a
// flag barrier that tells each rank when every band has landed.
//
// One process per GPU.  Each rank allocates one exchange buffer (gllmk_shared_alloc), publishes its 64-byte
// handle through the host framework's process group, and opens the other ranks' handles (gllmk_shared_open).
// The first GLLMK_PEER_FLAG_BYTES of every buffer are its flag words: flags[src] = last sequence number rank
// `src` signalled.  Plain peer stores and loads only: no multicast object, no cluster-multicast load.
#include "common.cuh"

namespace gllmk {

struct PeerBarrierParams {
    uint32_t *mine;                      // this rank's flag words
    uint32_t *peer[GLLMK_MAX_PEERS];     // the other ranks' flag words (peer-mapped)
    int npeer, rank;
    uint32_t seq;
    uint32_t spins;                      // probes before the wait gives up
    int *status;
};

// thread q talks to the q-th other rank (rank numbers skip this rank)
__global__ void peer_barrier_kernel(const __grid_constant__ PeerBarrierParams p) {
    // Launched with programmatic stream serialization: it may become resident while the product in front of it is
    // still running and lets the kernel behind it do the same; it orders itself after the product here.
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    const int q = threadIdx.x;
    // seq == 0: the sequence number lives in this rank's flag area (word 16) and advances by one per barrier,
    // so that a captured graph can be replayed
    __shared__ uint32_t seq_s;
    if (q == 0) {
        uint32_t sq = p.seq;
        if (sq == 0) {
            sq = p.mine[16] + 1;
            if (sq == 0) sq = 1;
            p.mine[16] = sq;
        }
        seq_s = sq;
    }
    __syncthreads();
    const uint32_t seq = seq_s;
    if (q >= p.npeer) return;
    const int src = q < p.rank ? q : q + 1;
    // everything this GPU wrote before this kernel (its GEMV's stores into the peers' buffers) is ordered
    // before the flag at system scope
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(p.peer[q] + p.rank), "r"(seq) : "memory");
    // bounded wait for the same sequence number from that rank (it can be at most one barrier ahead)
    const uint32_t *flag = p.mine + src;
    bool seen = false;
    for (uint32_t it = 0; it < p.spins && !seen; it++) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(flag) : "memory");
        seen = (int32_t)(v - seq) >= 0;
        if (!seen && it > 64) __nanosleep(200);
    }
    if (!seen) atomicExch(p.status, 31);  // the host reads it with gllmk_ctx_status; the kernel just returns
}

// End of a chain of exchange products (gllmk_gemv_exchange): thread q waits until the q-th other rank has
// completed as many of them as this rank.  Inside a chain the next product's staging kernel does this wait itself.
__global__ void exchange_wait_kernel(const uint32_t *flags, int nranks, int rank, uint32_t spins, int *status) {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    const int q = threadIdx.x;
    if (q >= nranks - 1) return;
    const int src = q < rank ? q : q + 1;
    const uint32_t want = *reinterpret_cast<const volatile uint32_t *>(flags + XF_EPOCH);
    bool seen = false;
    for (uint32_t it = 0; it < spins && !seen; it++) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(flags + XF_FLAGS + src) : "memory");
        seen = (int32_t)(v - want) >= 0;
        if (!seen && it > 64) __nanosleep(100);
    }
    if (!seen) atomicExch(status, 32);
}

int32_t peer_barrier_launch(Ctx *c, uint32_t *mine, uint32_t *const *peers, int n_peers, int rank, uint32_t seq, cudaStream_t s) {
    PeerBarrierParams p{};
    p.mine = mine;
    for (int q = 0; q < n_peers; q++) p.peer[q] = peers[q];
    p.npeer = n_peers;
    p.rank = rank;
    p.seq = seq;
    p.spins = (uint32_t)c->peer_wait_spins;
    p.status = c->status_dev;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = c->gemv_pdl != 0 ? 1 : 0;
    GK_CUDA(c, cudaLaunchKernelEx(&cfg, peer_barrier_kernel, p));
    return GLLMK_STATUS_OK;
}

}  // namespace gllmk

using namespace gllmk;

extern "C" int32_t gllmk_shared_alloc(gllmk_ctx ctx, size_t bytes, void **dev_ptr, uint8_t *handle) {
    if (!ctx || !dev_ptr || !handle || bytes == 0) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    static_assert(sizeof(cudaIpcMemHandle_t) == GLLMK_IPC_HANDLE_BYTES, "handle size");
    int prev = -1;
    cudaGetDevice(&prev);
    GK_CUDA(c, cudaSetDevice(c->device));
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);  // flag words start at zero
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        if (p) cudaFree(p);
        if (prev >= 0) cudaSetDevice(prev);
        return cuda_fail(c, e, "gllmk_shared_alloc");
    }
    memcpy(handle, &h, sizeof(h));
    *dev_ptr = p;
    if (prev >= 0) cudaSetDevice(prev);
    return GLLMK_STATUS_OK;
}

extern "C" int32_t gllmk_shared_open(gllmk_ctx ctx, const uint8_t *handle, void **peer_ptr) {
    if (!ctx || !handle || !peer_ptr) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    int prev = -1;
    cudaGetDevice(&prev);
    GK_CUDA(c, cudaSetDevice(c->device));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void *p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (prev >= 0) cudaSetDevice(prev);
    if (e != cudaSuccess) return cuda_fail(c, e, "cudaIpcOpenMemHandle");
    *peer_ptr = p;
    return GLLMK_STATUS_OK;
}

extern "C" int32_t gllmk_shared_close(gllmk_ctx ctx, void *peer_ptr) {
    if (!ctx) return GLLMK_STATUS_INVALID_ARG;
    if (!peer_ptr) return GLLMK_STATUS_OK;
    Ctx *c = static_cast<Ctx *>(ctx);
    GK_CUDA(c, cudaIpcCloseMemHandle(peer_ptr));
    return GLLMK_STATUS_OK;
}

extern "C" int32_t gllmk_shared_free(gllmk_ctx ctx, void *dev_ptr) {
    if (!ctx) return GLLMK_STATUS_INVALID_ARG;
    if (!dev_ptr) return GLLMK_STATUS_OK;
    Ctx *c = static_cast<Ctx *>(ctx);
    GK_CUDA(c, cudaDeviceSynchronize());
    GK_CUDA(c, cudaFree(dev_ptr));
    return GLLMK_STATUS_OK;
}

extern "C" int32_t gllmk_peer_barrier(gllmk_ctx ctx, void *flags_local, void *const *flags_peers, int32_t n_peers, int32_t rank,
                                      uint32_t seq, void *stream) {
    if (!ctx || !flags_local || (n_peers > 0 && !flags_peers)) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    if (n_peers < 0 || n_peers > GLLMK_MAX_PEERS || rank < 0 || rank > n_peers)
        return fail(c, GLLMK_STATUS_INVALID_ARG, "peer_barrier: %d peers / rank %d out of range", n_peers, rank);
    for (int q = 0; q < n_peers; q++)
        if (!flags_peers[q]) return fail(c, GLLMK_STATUS_INVALID_ARG, "peer_barrier: null peer pointer");
    if (n_peers == 0) return GLLMK_STATUS_OK;
    return peer_barrier_launch(c, static_cast<uint32_t *>(flags_local), reinterpret_cast<uint32_t *const *>(flags_peers), n_peers, rank,
                               seq, static_cast<cudaStream_t>(stream));
}

extern "C" int32_t gllmk_gemv_exchange(gllmk_ctx ctx, gllmk_weight wh, const float *x_dev, const float *x_up_dev, int64_t x_stride_t,
                                       int64_t x_stride_k, int32_t m, float *y_local, int64_t y_stride_t, int64_t y_stride_r,
                                       void *const *y_peers, void *flags_local, void *const *flags_peers, int32_t n_peers, int32_t rank,
                                       void *stream) {
    if (!ctx || !wh || !x_dev || !y_local || !flags_local || (n_peers > 0 && (!y_peers || !flags_peers))) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    const Weight *w = static_cast<const Weight *>(wh);
    if (m < 1 || m > GLLMK_GEMV_MAX_M) return fail(c, GLLMK_STATUS_INVALID_ARG, "gemv_exchange: m=%d outside 1..%d", m, GLLMK_GEMV_MAX_M);
    if (n_peers < 0 || n_peers > GLLMK_MAX_PEERS || rank < 0 || rank > n_peers)
        return fail(c, GLLMK_STATUS_INVALID_ARG, "gemv_exchange: %d peers / rank %d out of range", n_peers, rank);
    Exchange x{};
    x.flags_local = static_cast<uint32_t *>(flags_local);
    x.n_peers = n_peers;
    x.rank = rank;
    for (int q = 0; q < n_peers; q++) {
        if (!y_peers[q] || !flags_peers[q]) return fail(c, GLLMK_STATUS_INVALID_ARG, "gemv_exchange: null peer pointer");
        x.flags_peer[q] = static_cast<uint32_t *>(flags_peers[q]);
    }
    if (w->device != c->device) return fail(c, GLLMK_STATUS_INVALID_ARG, "weight lives on another device");
    DeviceGuard g(c->device);
    return gemv_launch(c, w, x_dev, x_stride_t, x_stride_k, m, y_local, y_stride_t, y_stride_r, nullptr, 0,
                       static_cast<cudaStream_t>(stream), y_peers, n_peers, x_up_dev, &x);
}

extern "C" int32_t gllmk_exchange_wait(gllmk_ctx ctx, void *flags_local, int32_t n_peers, int32_t rank, void *stream) {
    if (!ctx || !flags_local) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    if (n_peers < 0 || n_peers > GLLMK_MAX_PEERS || rank < 0 || rank > n_peers)
        return fail(c, GLLMK_STATUS_INVALID_ARG, "exchange_wait: %d peers / rank %d out of range", n_peers, rank);
    if (n_peers == 0) return GLLMK_STATUS_OK;
    DeviceGuard g(c->device);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = c->gemv_pdl != 0 ? 1 : 0;
    GK_CUDA(c, cudaLaunchKernelEx(&cfg, exchange_wait_kernel, static_cast<const uint32_t *>(flags_local), n_peers + 1, (int)rank,
                                  (uint32_t)c->peer_wait_spins, c->status_dev));
    return GLLMK_STATUS_OK;
}
