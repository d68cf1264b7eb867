// extern "C" boundary of libgllmk.so (declared in include/gllmk.h).  Argument validation happens
// here, before any launch; nothing below throws.
#include <cuda_bf16.h>

#include <vector>

#include "common.cuh"

namespace gllmk {

int32_t fail(Ctx *c, int32_t code, const char *fmt, ...) {
    if (c) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        c->err = buf;
    }
    return code;
}

int32_t cuda_fail(Ctx *c, cudaError_t e, const char *what) {
    const int32_t code = (e == cudaErrorMemoryAllocation) ? GLLMK_STATUS_OUT_OF_MEMORY : GLLMK_STATUS_RUNTIME_ERROR;
    (void)cudaGetLastError();  // clear the sticky-free error state
    return fail(c, code, "CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
}

static int32_t grow(Ctx *c, void **p, size_t *have, size_t want, bool pinned) {
    if (*have >= want) return GLLMK_STATUS_OK;
    // every buffer is used stream-ordered on streams the caller may still have work on
    GK_CUDA(c, cudaDeviceSynchronize());
    if (*p) {
        if (pinned) cudaFreeHost(*p);
        else cudaFree(*p);
        *p = nullptr;
        *have = 0;
    }
    const size_t sz = (want + (1u << 20) - 1) & ~((size_t)(1u << 20) - 1);
    if (pinned) GK_CUDA(c, cudaMallocHost(p, sz));
    else GK_CUDA(c, cudaMalloc(p, sz));
    *have = sz;
    return GLLMK_STATUS_OK;
}
int32_t ensure_ws(Ctx *c, size_t bytes) { return grow(c, &c->ws, &c->ws_bytes, bytes, false); }
int32_t ensure_red(Ctx *c, size_t bytes) { return grow(c, &c->red, &c->red_bytes, bytes, false); }
int32_t ensure_act(Ctx *c, size_t bytes) { return grow(c, &c->act, &c->act_bytes, bytes, false); }
int32_t ensure_cnt(Ctx *c, size_t bytes) {
    if (c->cnt_bytes >= bytes) return GLLMK_STATUS_OK;
    int32_t rc = grow(c, &c->cnt, &c->cnt_bytes, bytes, false);
    if (rc) return rc;
    GK_CUDA(c, cudaMemset(c->cnt, 0, c->cnt_bytes));  // arrival counters start at zero and reset themselves
    return GLLMK_STATUS_OK;
}
int32_t ensure_pin(Ctx *c, size_t bytes) { return grow(c, &c->pin, &c->pin_bytes, bytes, true); }
int32_t ensure_dev_io(Ctx *c, size_t bytes) { return grow(c, &c->dev_io, &c->dev_io_bytes, bytes, false); }

// QuantType::block_size / block_bytes: read from the format descriptor table (quant_format.cuh)
static int block_size_of(int qt, int mx) { return quant_format(qt, mx).block_size; }
static int block_bytes_of(int qt, int mx) { return quant_format(qt, mx).block_bytes; }

// Creates the handle and its device buffers for an n x k matrix of type qt (no data yet).
static int32_t weight_alloc(Ctx *c, int32_t qt, int64_t n, int64_t k, int32_t mx_block, float global, Weight **out) {
    if (qt != GLLMK_QUANT_Q4K && qt != GLLMK_QUANT_Q8_0 && qt != GLLMK_QUANT_MXFP4 && qt != GLLMK_QUANT_NVFP4 && !raw_format(qt))
        return fail(c, GLLMK_STATUS_UNSUPPORTED, "unknown quant type %d", qt);
    if (qt == GLLMK_QUANT_MXFP4 && mx_block != 32)
        return fail(c, GLLMK_STATUS_UNSUPPORTED, "MXFP4 weights need block_size 32 (got %d)", mx_block);
    if (n <= 0 || k <= 0) return fail(c, GLLMK_STATUS_INVALID_ARG, "n and k must be positive");
    const int bs = block_size_of(qt, mx_block);
    const int64_t kmul = bs;
    if (k % kmul) return fail(c, GLLMK_STATUS_INVALID_ARG, "k=%lld is not a multiple of %lld", (long long)k, (long long)kmul);
    if (n > (int64_t)1 << 30 || k > (int64_t)1 << 30) return fail(c, GLLMK_STATUS_INVALID_ARG, "matrix too large");
    Weight *w = new (std::nothrow) Weight();
    if (!w) return fail(c, GLLMK_STATUS_OUT_OF_MEMORY, "host allocation failed");
    w->qt = qt;
    w->mx_block = (qt == GLLMK_QUANT_MXFP4) ? mx_block : 0;
    w->n = n;
    w->k = k;
    w->k_pad = k;
    w->nb = k / bs;
    w->global_scale = global;
    w->device = c->device;
    w->ref_bytes = (uint64_t)n * (uint64_t)w->nb * (uint64_t)block_bytes_of(qt, mx_block);
    if (raw_format(qt)) {
        // reference blocks as they are; 16 spare bytes let the GEMV's 16-byte loads run past the last row
        w->n_pad = n;
        w->qs_bytes = (size_t)n * w->nb * raw_dev_block_bytes(qt) + 16;
        w->aux_bytes = 0;
    } else if (qt == GLLMK_QUANT_Q4K) {
        w->n_pad = (n + 127) / 128 * 128;
        w->qs_bytes = (size_t)(w->n_pad / 16) * w->nb * Q4K_CHUNK;
        w->aux_bytes = 0;
    } else if (qt == GLLMK_QUANT_Q8_0) {
        w->n_pad = (n + 127) / 128 * 128;
        w->nb8 = (w->nb + 7) / 8;
        w->qs_bytes = (size_t)(w->n_pad / 16) * w->nb8 * Q80_CHUNK;
        w->aux_bytes = 0;
    } else {
        // FP4 planes are tiled in 256-element k-steps: k is padded with zero codes and zero scale bytes
        w->n_pad = (n + 127) / 128 * 128;
        w->k_pad = (k + 255) / 256 * 256;
        w->qs_bytes = (size_t)w->n_pad * (w->k_pad / 2);
        w->aux_bytes = (size_t)w->n_pad * (w->k_pad / (qt == GLLMK_QUANT_NVFP4 ? 16 : 32));
    }
    cudaError_t e = cudaMalloc(&w->qs, w->qs_bytes);
    if (e == cudaSuccess && w->aux_bytes) e = cudaMalloc(&w->aux, w->aux_bytes);
    if (e != cudaSuccess) {
        if (w->qs) cudaFree(w->qs);
        delete w;
        return cuda_fail(c, e, "cudaMalloc(weight)");
    }
    *out = w;
    return GLLMK_STATUS_OK;
}

static void weight_destroy(Weight *w) {
    if (!w) return;
    DeviceGuard g(w->device);
    if (w->qs) cudaFree(w->qs);
    if (w->aux) cudaFree(w->aux);
    delete w;
}

// blocks/scales: host or device according to on_device.  Synchronous: returns once repacked.
static int32_t weight_fill(Ctx *c, Weight *w, const void *blocks, const void *scales, bool on_device) {
    const size_t raw = (w->qt == GLLMK_QUANT_MXFP4 && scales) ? (size_t)w->n * (w->k / 2) : (size_t)w->ref_bytes;
    const size_t sraw = (w->qt == GLLMK_QUANT_MXFP4 && scales) ? (size_t)w->n * (w->k / 32) : 0;
    const void *bdev = blocks, *sdev = scales;
    void *stage = nullptr;
    if (!on_device) {
        const size_t off = (raw + 255) & ~(size_t)255;
        GK_CUDA(c, cudaMalloc(&stage, off + sraw + 256));
        cudaError_t e = cudaMemcpyAsync(stage, blocks, raw, cudaMemcpyHostToDevice, c->stream);
        if (e == cudaSuccess && sraw)
            e = cudaMemcpyAsync(static_cast<char *>(stage) + off, scales, sraw, cudaMemcpyHostToDevice, c->stream);
        if (e != cudaSuccess) { cudaFree(stage); return cuda_fail(c, e, "cudaMemcpyAsync(weight blocks)"); }
        bdev = stage;
        sdev = sraw ? static_cast<char *>(stage) + off : nullptr;
    } else {
        if (((uintptr_t)blocks & 15) != 0) return fail(c, GLLMK_STATUS_INVALID_ARG, "device block pointer must be 16-byte aligned");
        // The caller's kernels that produce the blocks run on streams this library does not know: the repack (on the
        // context's own non-blocking stream) must not start before they have finished.  Load-time call: wait for the device.
        GK_CUDA(c, cudaDeviceSynchronize());
    }
    int32_t rc = repack_upload(c, w, bdev, sdev, c->stream);
    cudaError_t e = cudaStreamSynchronize(c->stream);
    if (stage) cudaFree(stage);
    if (rc) return rc;
    if (e != cudaSuccess) return cuda_fail(c, e, "repack");
    return GLLMK_STATUS_OK;
}

}  // namespace gllmk

using namespace gllmk;

extern "C" {

const char *gllmk_version(void) { return "gllmk 0.1.0 (sm_100a)"; }

int32_t gllmk_hw_info(char *buf, size_t len) {
    if (!buf || len == 0) return GLLMK_STATUS_INVALID_ARG;
    int ndev = 0;
    cudaDeviceProp prop;
    int n;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0 || cudaGetDeviceProperties(&prop, 0) != cudaSuccess) {
        (void)cudaGetLastError();
        n = snprintf(buf, len, "no CUDA device");
    } else {
        n = snprintf(buf, len, "%s sm_%d%d, %d SMs, %.1f GiB, L2 %d MiB, %d device(s)", prop.name, prop.major, prop.minor,
                     prop.multiProcessorCount, (double)prop.totalGlobalMem / (1 << 30), prop.l2CacheSize >> 20, ndev);
    }
    if (n < 0) return GLLMK_STATUS_RUNTIME_ERROR;
    return (int32_t)((size_t)n < len ? (size_t)n : len - 1);
}

int32_t gllmk_quant_format_descriptor_for_type(int32_t quant_type, int32_t mx_block, gllmk_quant_format_descriptor *out) {
    if (!out) return GLLMK_STATUS_INVALID_ARG;
    const gllmk_quant_format_descriptor d = quant_format(quant_type, mx_block);
    if (d.quant_type == 0) return GLLMK_STATUS_UNSUPPORTED;
    if (quant_type == GLLMK_QUANT_MXFP4 && (mx_block <= 0 || (mx_block & 1))) return GLLMK_STATUS_INVALID_ARG;
    *out = d;
    return GLLMK_STATUS_OK;
}

int32_t gllmk_quant_format_registry(int32_t *quant_types, int32_t cap) {
    static const int32_t ids[] = {GLLMK_QUANT_Q4_0, GLLMK_QUANT_Q5_0, GLLMK_QUANT_Q8_0, GLLMK_QUANT_Q4K, GLLMK_QUANT_Q5_K,
                                  GLLMK_QUANT_Q6_K, GLLMK_QUANT_Q8_K, GLLMK_QUANT_MXFP4, GLLMK_QUANT_NVFP4};
    const int32_t n = (int32_t)(sizeof(ids) / sizeof(ids[0]));
    for (int32_t i = 0; quant_types && i < n && i < cap; i++) quant_types[i] = ids[i];
    return n;
}

int32_t gllmk_quant_block_size(int32_t qt, int32_t mx_block) { return block_size_of(qt, mx_block); }
int32_t gllmk_quant_block_bytes(int32_t qt, int32_t mx_block) { return block_bytes_of(qt, mx_block); }

int32_t gllmk_ctx_create(int32_t device, gllmk_ctx *out) {
    if (!out) return GLLMK_STATUS_INVALID_ARG;
    *out = nullptr;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
        (void)cudaGetLastError();
        return GLLMK_STATUS_RUNTIME_ERROR;  // no CPU fallback
    }
    if (device < 0 || device >= ndev) return GLLMK_STATUS_INVALID_ARG;
    DeviceGuard g(device);
    if (!g.ok) return GLLMK_STATUS_RUNTIME_ERROR;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return GLLMK_STATUS_RUNTIME_ERROR;
    if (prop.major != 10) return GLLMK_STATUS_UNSUPPORTED;  // kernels are sm_100a only
    Ctx *c = new (std::nothrow) Ctx();
    if (!c) return GLLMK_STATUS_OUT_OF_MEMORY;
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaMalloc(reinterpret_cast<void **>(&c->status_dev), 16384) != cudaSuccess ||
        cudaMemset(c->status_dev, 0, 16384) != cudaSuccess) {
        (void)cudaGetLastError();
        if (c->stream) cudaStreamDestroy(c->stream);
        delete c;
        return GLLMK_STATUS_RUNTIME_ERROR;
    }
    *out = c;
    return GLLMK_STATUS_OK;
}

void gllmk_ctx_free(gllmk_ctx ctx) {
    if (!ctx) return;
    Ctx *c = static_cast<Ctx *>(ctx);
    DeviceGuard g(c->device);
    cudaDeviceSynchronize();
    if (c->ws) cudaFree(c->ws);
    if (c->red) cudaFree(c->red);
    if (c->act) cudaFree(c->act);
    if (c->cnt) cudaFree(c->cnt);
    if (c->status_dev) cudaFree(c->status_dev);
    if (c->dev_io) cudaFree(c->dev_io);
    if (c->pin) cudaFreeHost(c->pin);
    if (c->batch_exec) cudaGraphExecDestroy(c->batch_exec);
    for (cudaEvent_t e : c->events) cudaEventDestroy(e);
    if (c->copy_stream) cudaStreamDestroy(c->copy_stream);
    if (c->stream) cudaStreamDestroy(c->stream);
    delete c;
}

const char *gllmk_last_error(gllmk_ctx ctx) {
    if (!ctx) return "";
    return static_cast<Ctx *>(ctx)->err.c_str();
}

int32_t gllmk_ctx_status(gllmk_ctx ctx, int32_t *device_status) {
    if (!ctx || !device_status) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    DeviceGuard g(c->device);
    GK_CUDA(c, cudaDeviceSynchronize());
    int v = 0;
    GK_CUDA(c, cudaMemcpy(&v, c->status_dev, sizeof(int), cudaMemcpyDeviceToHost));
    *device_status = v;
    if (v) {
        GK_CUDA(c, cudaMemset(c->status_dev, 0, sizeof(int)));
        // A kernel that gave up left without arriving at its row tiles' counters: the "zero between launches"
        // rule of the split-k arrival counters (decode GEMV and FP4 decode GEMV share them) no longer holds.
        if (c->cnt) GK_CUDA(c, cudaMemset(c->cnt, 0, c->cnt_bytes));
        return fail(c, GLLMK_STATUS_RUNTIME_ERROR, "a kernel gave up a bounded wait (status word %d)", v);
    }
    return GLLMK_STATUS_OK;
}

int32_t gllmk_ctx_set(gllmk_ctx ctx, const char *key, int64_t value) {
    if (!ctx || !key) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    if (!strcmp(key, "gemv_ctas_per_sm")) c->gemv_ctas_per_sm = value;
    else if (!strcmp(key, "gemv_pdl")) c->gemv_pdl = value;
    else if (!strcmp(key, "gemv_fp4_int")) c->gemv_fp4_int = value;
    else if (!strcmp(key, "gemm_fp4_pair")) c->gemm_fp4_pair = value;
    else if (!strcmp(key, "gemm_i8_pair")) c->gemm_i8_pair = value;
    else if (!strcmp(key, "gemv_fuse")) c->gemv_fuse = value;
    else if (!strcmp(key, "gemm_tail_split")) c->gemm_tail_split = value;
    else if (!strcmp(key, "gemm_raw_slots")) c->gemm_raw_slots = value;
    else if (!strcmp(key, "gemm_row_tiles")) c->gemm_row_tiles = value;
    else if (!strcmp(key, "raw_gemv_mma")) c->raw_gemv_mma = value;
    else if (!strcmp(key, "gemm_pdl")) c->gemm_pdl = value;
    else if (!strcmp(key, "host_batch_graph")) c->host_batch_graph = value;
    else if (!strcmp(key, "peer_wait_spins")) {
        if (value < 1 || value > ((int64_t)1 << 30)) return fail(c, GLLMK_STATUS_INVALID_ARG, "peer_wait_spins outside 1..2^30");
        c->peer_wait_spins = value;
    } else if (!strcmp(key, "inject_give_up")) {
        // Host-side fault injection for tests of the failure path: leaves the context exactly as a kernel that gave
        // up a bounded wait would (status word = value, arrival counters non-zero) without making any kernel wait.
        if (value < 1 || value > 255) return fail(c, GLLMK_STATUS_INVALID_ARG, "inject_give_up takes a status code 1..255");
        DeviceGuard g(c->device);
        GK_CUDA(c, cudaDeviceSynchronize());
        const int v = (int)value;
        GK_CUDA(c, cudaMemcpy(c->status_dev, &v, sizeof(int), cudaMemcpyHostToDevice));
        if (c->cnt) GK_CUDA(c, cudaMemset(c->cnt, 1, c->cnt_bytes));
    }
    else return fail(c, GLLMK_STATUS_INVALID_ARG, "unknown key %s", key);
    return GLLMK_STATUS_OK;
}

int32_t gllmk_weight_upload(gllmk_ctx ctx, int32_t quant_type, int64_t n, int64_t k, int32_t mx_block,
                            const void *blocks, const void *scales, float global_scale, int32_t src_on_device,
                            gllmk_weight *out) {
    if (!ctx || !blocks || !out) return GLLMK_STATUS_INVALID_ARG;
    *out = nullptr;
    Ctx *c = static_cast<Ctx *>(ctx);
    if (scales && quant_type != GLLMK_QUANT_MXFP4)
        return fail(c, GLLMK_STATUS_INVALID_ARG, "scales must be NULL unless the type is MXFP4 (split form)");
    DeviceGuard g(c->device);
    Weight *w = nullptr;
    int32_t rc = weight_alloc(c, quant_type, n, k, mx_block, global_scale, &w);
    if (rc) return rc;
    rc = weight_fill(c, w, blocks, scales, src_on_device != 0);
    if (rc) { weight_destroy(w); return rc; }
    *out = w;
    return GLLMK_STATUS_OK;
}

void gllmk_weight_free(gllmk_weight w) { weight_destroy(static_cast<Weight *>(w)); }

int32_t gllmk_weight_info(gllmk_weight wh, int32_t *quant_type, int64_t *n, int64_t *k, uint64_t *ref_bytes,
                          uint64_t *dev_bytes) {
    if (!wh) return GLLMK_STATUS_INVALID_ARG;
    const Weight *w = static_cast<const Weight *>(wh);
    if (quant_type) *quant_type = w->qt;
    if (n) *n = w->n;
    if (k) *k = w->k;
    if (ref_bytes) *ref_bytes = w->ref_bytes;
    if (dev_bytes) *dev_bytes = (uint64_t)w->qs_bytes + (uint64_t)w->aux_bytes;
    return GLLMK_STATUS_OK;
}

int32_t gllmk_weight_unpack(gllmk_ctx ctx, gllmk_weight wh, void *blocks, void *scales, int32_t dst_on_device) {
    if (!ctx || !wh || !blocks) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    const Weight *w = static_cast<const Weight *>(wh);
    if (w->qt == GLLMK_QUANT_INT8) return fail(c, GLLMK_STATUS_UNSUPPORTED, "unpack: not a block-quantized weight");
    if (w->qt == GLLMK_QUANT_MXFP4 && !scales)
        return fail(c, GLLMK_STATUS_INVALID_ARG, "MXFP4 unpack writes the split form and needs a scales buffer");
    DeviceGuard g(c->device);
    const bool split = w->qt == GLLMK_QUANT_MXFP4;
    const size_t raw = split ? (size_t)w->n * (w->k / 2) : (size_t)w->ref_bytes;
    const size_t sraw = split ? (size_t)w->n * (w->k / 32) : 0;
    if (dst_on_device) {
        int32_t rc = repack_unpack(c, w, blocks, scales, c->stream);
        if (rc) return rc;
        GK_CUDA(c, cudaStreamSynchronize(c->stream));
        return GLLMK_STATUS_OK;
    }
    void *stage = nullptr;
    const size_t off = (raw + 255) & ~(size_t)255;
    GK_CUDA(c, cudaMalloc(&stage, off + sraw + 256));
    int32_t rc = repack_unpack(c, w, stage, static_cast<char *>(stage) + off, c->stream);
    cudaError_t e = cudaSuccess;
    if (!rc) {
        e = cudaMemcpyAsync(blocks, stage, raw, cudaMemcpyDeviceToHost, c->stream);
        if (e == cudaSuccess && sraw)
            e = cudaMemcpyAsync(scales, static_cast<char *>(stage) + off, sraw, cudaMemcpyDeviceToHost, c->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    }
    cudaFree(stage);
    if (rc) return rc;
    if (e != cudaSuccess) return cuda_fail(c, e, "unpack copy");
    return GLLMK_STATUS_OK;
}

int32_t gllmk_dequant(gllmk_ctx ctx, gllmk_weight wh, float *out_dev, void *stream) {
    if (!ctx || !wh || !out_dev) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    if (((uintptr_t)out_dev & 15) != 0) return fail(c, GLLMK_STATUS_INVALID_ARG, "out_dev must be 16-byte aligned");
    if (static_cast<const Weight *>(wh)->qt == GLLMK_QUANT_INT8)
        return fail(c, GLLMK_STATUS_UNSUPPORTED, "dequant: not a block-quantized weight");
    DeviceGuard g(c->device);
    return dequant_matrix(c, static_cast<const Weight *>(wh), out_dev, static_cast<cudaStream_t>(stream));
}

int32_t gllmk_embedding_gather(gllmk_ctx ctx, gllmk_weight wh, const int32_t *ids_dev, int64_t count, float *out_dev, void *stream) {
    if (!ctx || !wh || !ids_dev || !out_dev) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    const Weight *w = static_cast<const Weight *>(wh);
    if (count < 0) return fail(c, GLLMK_STATUS_INVALID_ARG, "embedding_gather: negative count");
    if (((uintptr_t)out_dev & 15) != 0) return fail(c, GLLMK_STATUS_INVALID_ARG, "out_dev must be 16-byte aligned");
    if (w->qt == GLLMK_QUANT_INT8) return fail(c, GLLMK_STATUS_UNSUPPORTED, "embedding_gather: not a block-quantized weight");
    if (w->device != c->device) return fail(c, GLLMK_STATUS_INVALID_ARG, "weight lives on another device");
    DeviceGuard g(c->device);
    return dequant_matrix(c, w, out_dev, static_cast<cudaStream_t>(stream), ids_dev, count);
}

int32_t gllmk_gemv(gllmk_ctx ctx, gllmk_weight wh, const float *x_dev, int64_t x_stride_t, int64_t x_stride_k,
                   int32_t m, float *y_dev, int64_t y_stride_t, int64_t y_stride_r, const float *row_scales,
                   int64_t n_row_scales, void *stream) {
    if (!ctx || !wh || !x_dev || !y_dev) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    const Weight *w = static_cast<const Weight *>(wh);
    if (m < 1 || m > GLLMK_GEMV_MAX_M)
        return fail(c, GLLMK_STATUS_INVALID_ARG, "gemv: m=%d outside 1..%d", m, GLLMK_GEMV_MAX_M);
    if (row_scales && n_row_scales != 1 && n_row_scales != w->n)
        return fail(c, GLLMK_STATUS_INVALID_ARG, "gemv: n_row_scales=%lld must be 1 or n=%lld", (long long)n_row_scales, (long long)w->n);
    if (w->device != c->device) return fail(c, GLLMK_STATUS_INVALID_ARG, "weight lives on another device");
    DeviceGuard g(c->device);
    return gemv_launch(c, w, x_dev, x_stride_t, x_stride_k, m, y_dev, y_stride_t, y_stride_r, row_scales, n_row_scales,
                       static_cast<cudaStream_t>(stream));
}

int32_t gllmk_ffn_decode(gllmk_ctx ctx, gllmk_weight w_gate_up, gllmk_weight w_down, const float *x_dev, int32_t m, float *h_dev,
                         float *y_dev, void *stream) {
    if (!ctx || !w_gate_up || !w_down || !x_dev || !h_dev || !y_dev) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    const Weight *wg = static_cast<const Weight *>(w_gate_up), *wd = static_cast<const Weight *>(w_down);
    if (m < 1 || m > GLLMK_GEMV_MAX_M) return fail(c, GLLMK_STATUS_INVALID_ARG, "ffn_decode: m=%d outside 1..%d", m, GLLMK_GEMV_MAX_M);
    if (wg->n % 2 || wg->n / 2 != wd->k || wd->n != wg->k)
        return fail(c, GLLMK_STATUS_INVALID_ARG, "ffn_decode: shapes do not chain: gate||up [%lld, %lld], down [%lld, %lld]",
                    (long long)wg->n, (long long)wg->k, (long long)wd->n, (long long)wd->k);
    if (wg->device != c->device || wd->device != c->device) return fail(c, GLLMK_STATUS_INVALID_ARG, "weight lives on another device");
    DeviceGuard g(c->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t f = wd->k;
    // h = [gate | up] = W_gate_up x : [m, 2f]
    int32_t rc = gemv_launch(c, wg, x_dev, wg->k, 1, m, h_dev, 2 * f, 1, nullptr, 0, s);
    if (rc) return rc;
    // y = W_down (silu(gate) * up): the activation staging of the second product applies SwiGLU while it reads h
    return gemv_launch(c, wd, h_dev, 2 * f, 1, m, y_dev, wd->n, 1, nullptr, 0, s, nullptr, 0, h_dev + f);
}

int32_t gllmk_ffn_prefill(gllmk_ctx ctx, gllmk_weight w_gate_up, gllmk_weight w_down, const void *x_dev, int32_t x_dtype, int64_t ldx,
                          int32_t m, void *h_dev, void *y_dev, int32_t y_dtype, int64_t ldy, void *stream) {
    if (!ctx || !w_gate_up || !w_down || !x_dev || !h_dev || !y_dev) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    const Weight *wg = static_cast<const Weight *>(w_gate_up), *wd = static_cast<const Weight *>(w_down);
    if (m < 1) return fail(c, GLLMK_STATUS_INVALID_ARG, "ffn_prefill: m must be positive");
    if ((x_dtype != GLLMK_DTYPE_F32 && x_dtype != GLLMK_DTYPE_BF16) || (y_dtype != GLLMK_DTYPE_F32 && y_dtype != GLLMK_DTYPE_BF16))
        return fail(c, GLLMK_STATUS_UNSUPPORTED, "ffn_prefill: dtype must be f32 or bf16");
    if (wg->n % 2 || wg->n / 2 != wd->k || wd->n != wg->k)
        return fail(c, GLLMK_STATUS_INVALID_ARG, "ffn_prefill: shapes do not chain: gate||up [%lld, %lld], down [%lld, %lld]", (long long)wg->n,
                    (long long)wg->k, (long long)wd->n, (long long)wd->k);
    // (a GGUF file may mix formats inside a block: Q4_K gate / up with a Q6_K down projection is common)
    const auto has_tc_gemm = [](const Weight *w) {
        return w->qt != GLLMK_QUANT_INT8 && (!raw_format(w->qt) || w->qt == GLLMK_QUANT_Q6_K || w->qt == GLLMK_QUANT_Q5_K ||
                                             ((w->qt == GLLMK_QUANT_Q4_0 || w->qt == GLLMK_QUANT_Q5_0) && w->k % 256 == 0));
    };
    if (!has_tc_gemm(wg) || !has_tc_gemm(wd))
        return fail(c, GLLMK_STATUS_UNSUPPORTED, "ffn_prefill: weight type has no tensor-core prefill kernel");
    const int64_t f = wd->k;
    if (f % 8) return fail(c, GLLMK_STATUS_INVALID_ARG, "ffn_prefill: the intermediate width must be a multiple of 8");
    if (ldx < wg->k || ldy < wd->n) return fail(c, GLLMK_STATUS_INVALID_ARG, "ffn_prefill: leading dimension smaller than the row");
    if (wg->device != c->device || wd->device != c->device) return fail(c, GLLMK_STATUS_INVALID_ARG, "weight lives on another device");
    DeviceGuard g(c->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // h = [gate | up] = W_gate_up x, kept in bf16: [m, 2f]
    int32_t rc = gemm_launch(c, wg, x_dev, x_dtype == GLLMK_DTYPE_BF16, ldx, m, h_dev, 1, 2 * f, s);
    if (rc) return rc;
    // y = W_down (silu(gate) * up): SwiGLU is applied by the second product's activation staging while it reads h
    return gemm_launch(c, wd, h_dev, 1, 2 * f, m, y_dev, y_dtype == GLLMK_DTYPE_BF16, ldy, s,
                       static_cast<const __nv_bfloat16 *>(h_dev) + f);
}

int32_t gllmk_gemv_allgather(gllmk_ctx ctx, gllmk_weight wh, const float *x_dev, int64_t x_stride_t, int64_t x_stride_k, int32_t m,
                             float *y_local, int64_t y_stride_t, int64_t y_stride_r, void *const *y_peers, int32_t n_peers,
                             void *stream) {
    if (!ctx || !wh || !x_dev || !y_local || (n_peers > 0 && !y_peers)) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    const Weight *w = static_cast<const Weight *>(wh);
    if (m < 1 || m > GLLMK_GEMV_MAX_M)
        return fail(c, GLLMK_STATUS_INVALID_ARG, "gemv_allgather: m=%d outside 1..%d", m, GLLMK_GEMV_MAX_M);
    if (n_peers < 0 || n_peers > GLLMK_MAX_PEERS)
        return fail(c, GLLMK_STATUS_INVALID_ARG, "gemv_allgather: %d peers (at most %d)", n_peers, GLLMK_MAX_PEERS);
    for (int q = 0; q < n_peers; q++)
        if (!y_peers[q]) return fail(c, GLLMK_STATUS_INVALID_ARG, "gemv_allgather: null peer pointer");
    if (w->device != c->device) return fail(c, GLLMK_STATUS_INVALID_ARG, "weight lives on another device");
    DeviceGuard g(c->device);
    return gemv_launch(c, w, x_dev, x_stride_t, x_stride_k, m, y_local, y_stride_t, y_stride_r, nullptr, 0,
                       static_cast<cudaStream_t>(stream), y_peers, n_peers);
}

int32_t gllmk_gemm(gllmk_ctx ctx, gllmk_weight wh, const void *a_dev, int32_t a_dtype, int64_t lda, int32_t m, void *y_dev,
                   int32_t y_dtype, int64_t ldy, void *stream) {
    if (!ctx || !wh || !a_dev || !y_dev) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    const Weight *w = static_cast<const Weight *>(wh);
    if (m < 1) return fail(c, GLLMK_STATUS_INVALID_ARG, "gemm: m must be positive");
    if ((a_dtype != GLLMK_DTYPE_F32 && a_dtype != GLLMK_DTYPE_BF16) || (y_dtype != GLLMK_DTYPE_F32 && y_dtype != GLLMK_DTYPE_BF16))
        return fail(c, GLLMK_STATUS_UNSUPPORTED, "gemm: dtype must be f32 or bf16");
    if (lda < w->k || ldy < w->n) return fail(c, GLLMK_STATUS_INVALID_ARG, "gemm: leading dimension smaller than the row");
    if (w->device != c->device) return fail(c, GLLMK_STATUS_INVALID_ARG, "weight lives on another device");
    DeviceGuard g(c->device);
    // Q6_K, Q5_K and (when a row's blocks come in whole 16-byte aligned groups of eight: k a multiple of 256) Q4_0 / Q5_0 have
    // a place in the fused-dequant tensor-core GEMM.  On W[8192, 28672] it takes ~100 us up to 128 tokens; Q6_K's batch GEMV
    // needs 100 us up to 8 tokens and 135 us up to 16, the dp2a kernel of the other three 150 - 170 us for 2 tokens and
    // 590 us for 16
    if ((w->qt == GLLMK_QUANT_Q6_K && m > 8) || (w->qt == GLLMK_QUANT_Q5_K && m >= 2) ||
        ((w->qt == GLLMK_QUANT_Q4_0 || w->qt == GLLMK_QUANT_Q5_0) && w->k % 256 == 0 && m >= 2))
        return gemm_launch(c, w, a_dev, a_dtype == GLLMK_DTYPE_BF16, lda, m, y_dev, y_dtype == GLLMK_DTYPE_BF16, ldy,
                           static_cast<cudaStream_t>(stream));
    if (raw_format(w->qt)) {
        // no tensor-core prefill kernel for these formats: the streaming GEMV takes any number of tokens
        if (a_dtype != GLLMK_DTYPE_F32 || y_dtype != GLLMK_DTYPE_F32)
            return fail(c, GLLMK_STATUS_UNSUPPORTED, "gemm: quant type %d takes f32 activations and outputs only", w->qt);
        return gemv_launch(c, w, static_cast<const float *>(a_dev), lda, 1, m, static_cast<float *>(y_dev), ldy, 1, nullptr, 0,
                           static_cast<cudaStream_t>(stream));
    }
    // A few dozen tokens are still bound by the weight stream, which the decode kernel reads at several times
    // the rate the tensor-core pipeline reaches with a nearly empty N: run them as passes of up to 16 tokens.
    if (m <= GLLMK_GEMM_GEMV_MAX_M && a_dtype == GLLMK_DTYPE_F32 && y_dtype == GLLMK_DTYPE_F32) {
        for (int t0 = 0; t0 < m; t0 += GLLMK_GEMV_MAX_M) {
            const int mm = m - t0 < GLLMK_GEMV_MAX_M ? m - t0 : GLLMK_GEMV_MAX_M;
            const int32_t rc = gemv_launch(c, w, static_cast<const float *>(a_dev) + (int64_t)t0 * lda, lda, 1, mm,
                                           static_cast<float *>(y_dev) + (int64_t)t0 * ldy, ldy, 1, nullptr, 0,
                                           static_cast<cudaStream_t>(stream));
            if (rc) return rc;
        }
        return GLLMK_STATUS_OK;
    }
    return gemm_launch(c, w, a_dev, a_dtype == GLLMK_DTYPE_BF16, lda, m, y_dev, y_dtype == GLLMK_DTYPE_BF16, ldy,
                       static_cast<cudaStream_t>(stream));
}

int32_t gllmk_gemm_grouped(gllmk_ctx ctx, int32_t n_groups, const gllmk_weight *weights, const void *a_dev, int32_t a_dtype,
                           int64_t lda, const int64_t *row_offsets, void *y_dev, int32_t y_dtype, int64_t ldy, void *stream) {
    if (!ctx || !weights || !a_dev || !y_dev || !row_offsets) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    if (n_groups < 1 || n_groups > 4096) return fail(c, GLLMK_STATUS_INVALID_ARG, "gemm_grouped: n_groups=%d", n_groups);
    if ((a_dtype != GLLMK_DTYPE_F32 && a_dtype != GLLMK_DTYPE_BF16) || (y_dtype != GLLMK_DTYPE_F32 && y_dtype != GLLMK_DTYPE_BF16))
        return fail(c, GLLMK_STATUS_UNSUPPORTED, "gemm_grouped: dtype must be f32 or bf16");
    const Weight *w0 = static_cast<const Weight *>(weights[0]);
    if (!w0) return GLLMK_STATUS_INVALID_ARG;
    std::vector<const Weight *> ws((size_t)n_groups);
    for (int g = 0; g < n_groups; g++) {
        const Weight *w = static_cast<const Weight *>(weights[g]);
        if (!w) return GLLMK_STATUS_INVALID_ARG;
        if (w->qt != w0->qt || w->n != w0->n || w->k != w0->k || w->mx_block != w0->mx_block)
            return fail(c, GLLMK_STATUS_INVALID_ARG, "gemm_grouped: weight %d differs in type or shape from weight 0", g);
        if (w->device != c->device) return fail(c, GLLMK_STATUS_INVALID_ARG, "weight lives on another device");
        if (row_offsets[g + 1] < row_offsets[g] || row_offsets[g] < 0 || row_offsets[g + 1] > 0x7fffffff)
            return fail(c, GLLMK_STATUS_INVALID_ARG, "gemm_grouped: row_offsets must be non-decreasing and fit 31 bits");
        ws[(size_t)g] = w;
    }
    if (lda < w0->k || ldy < w0->n) return fail(c, GLLMK_STATUS_INVALID_ARG, "gemm_grouped: leading dimension smaller than the row");
    DeviceGuard g(c->device);
    return gemm_grouped_launch(c, ws.data(), n_groups, a_dev, a_dtype == GLLMK_DTYPE_BF16, lda, row_offsets, y_dev,
                               y_dtype == GLLMK_DTYPE_BF16, ldy, static_cast<cudaStream_t>(stream));
}

// ---- W8A8 integer path ----
static int32_t int8_weight_create(Ctx *c, int64_t n, int64_t k, const int8_t *b, int layout, bool on_device, Weight **out) {
    if (n <= 0 || k <= 0 || n > (int64_t)1 << 30 || k > (int64_t)1 << 30) return fail(c, GLLMK_STATUS_INVALID_ARG, "int8 weight: bad shape");
    if (layout != 0 && layout != 1) return fail(c, GLLMK_STATUS_INVALID_ARG, "int8 weight: layout must be 0 ([k, n]) or 1 ([n, k])");
    Weight *w = new (std::nothrow) Weight();
    if (!w) return fail(c, GLLMK_STATUS_OUT_OF_MEMORY, "host allocation failed");
    w->qt = GLLMK_QUANT_INT8;
    w->n = n;
    w->k = k;
    w->n_pad = (n + 127) / 128 * 128;
    w->k_pad = (k + 127) / 128 * 128;
    w->device = c->device;
    w->ref_bytes = (uint64_t)n * (uint64_t)k;
    w->qs_bytes = (size_t)w->n_pad * (size_t)w->k_pad;
    w->aux_bytes = (size_t)n * sizeof(int32_t);  // column sums of B (zero-point correction of the f32 activation path)
    cudaError_t e = cudaMalloc(&w->qs, w->qs_bytes);
    if (e == cudaSuccess) e = cudaMalloc(&w->aux, w->aux_bytes);
    if (e != cudaSuccess) {
        if (w->qs) cudaFree(w->qs);
        delete w;
        return cuda_fail(c, e, "cudaMalloc(int8 weight)");
    }
    const int8_t *bdev = b;
    void *stage = nullptr;
    if (!on_device) {
        e = cudaMalloc(&stage, (size_t)n * (size_t)k);
        if (e == cudaSuccess) e = cudaMemcpyAsync(stage, b, (size_t)n * (size_t)k, cudaMemcpyHostToDevice, c->stream);
        if (e != cudaSuccess) {
            if (stage) cudaFree(stage);
            weight_destroy(w);
            return cuda_fail(c, e, "upload(int8 weight)");
        }
        bdev = static_cast<const int8_t *>(stage);
    } else {
        (void)cudaDeviceSynchronize();  // the kernels that produced b ran on the caller's streams (see weight_fill)
    }
    int32_t rc = i8_weight_fill(c, w, bdev, layout, c->stream);
    e = cudaStreamSynchronize(c->stream);
    if (stage) cudaFree(stage);
    if (!rc && e != cudaSuccess) rc = cuda_fail(c, e, "repack(int8 weight)");
    if (rc) {
        weight_destroy(w);
        return rc;
    }
    *out = w;
    return GLLMK_STATUS_OK;
}

int32_t gllmk_int8_weight_upload(gllmk_ctx ctx, int64_t n, int64_t k, const int8_t *b, int32_t layout, int32_t src_on_device,
                                 gllmk_weight *out) {
    if (!ctx || !b || !out) return GLLMK_STATUS_INVALID_ARG;
    *out = nullptr;
    Ctx *c = static_cast<Ctx *>(ctx);
    DeviceGuard g(c->device);
    Weight *w = nullptr;
    const int32_t rc = int8_weight_create(c, n, k, b, layout, src_on_device != 0, &w);
    if (!rc) *out = w;
    return rc;
}

int32_t gllmk_gemm_int8(gllmk_ctx ctx, gllmk_weight wh, const uint8_t *a_dev, int64_t lda, int32_t m, int32_t *c_dev, int64_t ldc,
                        void *stream) {
    if (!ctx || !wh || !a_dev || !c_dev) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    const Weight *w = static_cast<const Weight *>(wh);
    if (w->qt != GLLMK_QUANT_INT8) return fail(c, GLLMK_STATUS_INVALID_ARG, "gemm_int8: the weight was not uploaded with gllmk_int8_weight_upload");
    if (m < 1) return fail(c, GLLMK_STATUS_INVALID_ARG, "gemm_int8: m must be positive");
    if (lda < w->k || ldc < w->n) return fail(c, GLLMK_STATUS_INVALID_ARG, "gemm_int8: leading dimension smaller than the row");
    if (w->device != c->device) return fail(c, GLLMK_STATUS_INVALID_ARG, "weight lives on another device");
    DeviceGuard g(c->device);
    return gemm_i8_launch(c, w, a_dev, lda, m, c_dev, ldc, static_cast<cudaStream_t>(stream));
}

int32_t gllmk_dequantize_i32_f32(gllmk_ctx ctx, const int32_t *c_dev, float *out_dev, int64_t m, int64_t n, float scale_a, float scale_b,
                                 const float *bias_dev, int32_t activation, void *stream) {
    if (!ctx || !c_dev || !out_dev) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    if (m < 0 || n < 0) return fail(c, GLLMK_STATUS_INVALID_ARG, "dequantize: negative shape");
    if (activation < 0 || activation > 4) return fail(c, GLLMK_STATUS_UNSUPPORTED, "dequantize: activation %d", activation);
    DeviceGuard g(c->device);
    return dequant_i32_launch(c, c_dev, out_dev, m, n, n, n, scale_a, scale_b, bias_dev, activation, static_cast<cudaStream_t>(stream));
}

int32_t gllmk_quantize_act_int8(gllmk_ctx ctx, const float *x_dev, int64_t rows, int64_t k, int64_t ldx, void *q_dev, int64_t ldq,
                                int32_t as_unsigned, float *scale_dev, void *stream) {
    if (!ctx || !x_dev || !q_dev || !scale_dev) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    if (rows < 1 || k < 1 || ldx < k || ldq < k) return fail(c, GLLMK_STATUS_INVALID_ARG, "quantize_act_int8: bad shape");
    DeviceGuard g(c->device);
    return act_quant_i8_launch(c, x_dev, rows, k, ldx, static_cast<uint8_t *>(q_dev), ldq, as_unsigned ? 128 : 0, scale_dev,
                               static_cast<cudaStream_t>(stream));
}

int32_t gllmk_w8a8_linear_f32(gllmk_ctx ctx, gllmk_weight wh, const float *x_dev, int64_t ldx, int32_t m, float *y_dev, int64_t ldy,
                              float scale_b, const float *bias_dev, int32_t activation, void *stream) {
    if (!ctx || !wh || !x_dev || !y_dev) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    const Weight *w = static_cast<const Weight *>(wh);
    if (w->qt != GLLMK_QUANT_INT8) return fail(c, GLLMK_STATUS_INVALID_ARG, "w8a8_linear: the weight was not uploaded with gllmk_int8_weight_upload");
    if (m < 1 || ldx < w->k || ldy < w->n) return fail(c, GLLMK_STATUS_INVALID_ARG, "w8a8_linear: bad shape");
    if (activation < 0 || activation > 4) return fail(c, GLLMK_STATUS_UNSUPPORTED, "w8a8_linear: activation %d", activation);
    if (w->device != c->device) return fail(c, GLLMK_STATUS_INVALID_ARG, "weight lives on another device");
    DeviceGuard g(c->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // context scratch: [scale f32, amax u32 | pad to 256] [u8 activations m x k] [s32 products m x n]
    const size_t ab = ((size_t)m * (size_t)w->k + 255) & ~(size_t)255, cb = (size_t)m * (size_t)w->n * sizeof(int32_t);
    // (the context's device I/O buffer: the integer GEMM stages its tile images in the activation workspace itself)
    int32_t rc = ensure_dev_io(c, 256 + ab + cb);
    if (rc) return rc;
    char *base = static_cast<char *>(c->dev_io);
    float *scale = reinterpret_cast<float *>(base);
    uint8_t *q = reinterpret_cast<uint8_t *>(base + 256);
    int32_t *ci = reinterpret_cast<int32_t *>(base + 256 + ab);
    rc = act_quant_i8_launch(c, x_dev, m, w->k, ldx, q, w->k, 128, scale, s);
    if (!rc) rc = gemm_i8_launch(c, w, q, w->k, m, ci, w->n, s);
    if (!rc) rc = dequant_i32_launch(c, ci, y_dev, m, w->n, w->n, ldy, 0.0f, scale_b, bias_dev, activation, s, scale,
                                     static_cast<const int32_t *>(w->aux));
    return rc;
}

int32_t gllmk_gemm_int8_host(gllmk_ctx ctx, const uint8_t *a, const int8_t *b_kn, int32_t *c_out, size_t m, size_t n, size_t k) {
    if (!ctx || !a || !b_kn || !c_out) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    if (m == 0 || n == 0) return GLLMK_STATUS_OK;
    if (k == 0) {
        memset(c_out, 0, m * n * sizeof(int32_t));
        return GLLMK_STATUS_OK;
    }
    if (m > 0x7fffffffu) return fail(c, GLLMK_STATUS_INVALID_ARG, "gemm_int8: m too large");
    DeviceGuard g(c->device);
    Weight *w = nullptr;
    int32_t rc = int8_weight_create(c, (int64_t)n, (int64_t)k, b_kn, 0, false, &w);
    if (rc) return rc;
    const size_t ab = m * k, cb = m * n * sizeof(int32_t), co = (ab + 255) & ~(size_t)255;
    rc = ensure_dev_io(c, co + cb);
    if (!rc) {
        char *dev = static_cast<char *>(c->dev_io);
        cudaError_t e = cudaMemcpyAsync(dev, a, ab, cudaMemcpyHostToDevice, c->stream);
        if (e == cudaSuccess) {
            rc = gemm_i8_launch(c, w, reinterpret_cast<const uint8_t *>(dev), (int64_t)k, (int)m, reinterpret_cast<int32_t *>(dev + co),
                                (int64_t)n, c->stream);
            if (!rc) e = cudaMemcpyAsync(c_out, dev + co, cb, cudaMemcpyDeviceToHost, c->stream);
        }
        if (!rc && e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
        if (!rc && e != cudaSuccess) rc = cuda_fail(c, e, "gemm_int8_host");
    }
    weight_destroy(w);
    return rc;
}

int32_t gllmk_gemm_fp4(gllmk_ctx ctx, gllmk_weight wh, gllmk_weight xh, void *y_dev, int32_t y_dtype, int64_t ldy, void *stream) {
    if (!ctx || !wh || !xh || !y_dev) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    const Weight *w = static_cast<const Weight *>(wh), *x = static_cast<const Weight *>(xh);
    if (y_dtype != GLLMK_DTYPE_F32 && y_dtype != GLLMK_DTYPE_BF16) return fail(c, GLLMK_STATUS_UNSUPPORTED, "gemm_fp4: y dtype");
    if (ldy < w->n) return fail(c, GLLMK_STATUS_INVALID_ARG, "gemm_fp4: ldy smaller than n");
    if (w->device != c->device || x->device != c->device) return fail(c, GLLMK_STATUS_INVALID_ARG, "operand lives on another device");
    DeviceGuard g(c->device);
    return gemm_fp4_launch(c, w, x, y_dev, y_dtype == GLLMK_DTYPE_BF16, ldy, static_cast<cudaStream_t>(stream));
}

int32_t gllmk_probe_fp4_mma(gllmk_ctx ctx, int32_t cta_pair, int32_t with_scale_copies, int32_t nvfp4, int32_t ksteps, float *tflops) {
    if (!ctx || !tflops) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    if (ksteps < 1 || ksteps > (1 << 20)) return fail(c, GLLMK_STATUS_INVALID_ARG, "probe_fp4_mma: ksteps outside 1..2^20");
    DeviceGuard g(c->device);
    if (with_scale_copies < 0 || with_scale_copies > 2) return fail(c, GLLMK_STATUS_INVALID_ARG, "probe_fp4_mma: scale-factor mode outside 0..2");
    return probe_fp4_mma(c, cta_pair != 0, with_scale_copies, nvfp4 != 0, ksteps, tflops);
}

// Shared body of the host-pointer matmuls: weight rows n_w, tokens m_t, reduction k.
//   ref_layout: input [k, m_t], output [n_w, m_t]; else input [m_t, k], output [m_t, n_w].
static int32_t matmul_host_impl(Ctx *c, const Weight *w, const float *x_host, int m_t, float *y_host, bool ref_layout,
                                const float *scales_host, size_t n_scales) {
    const int64_t n_w = w->n, k = w->k;
    const size_t xb = (size_t)m_t * k * sizeof(float), yb = (size_t)m_t * n_w * sizeof(float);
    const size_t sb = (n_scales == 1 || (int64_t)n_scales == n_w) ? n_scales * sizeof(float) : 0;
    const size_t xo = 0, yo = (xb + 255) & ~(size_t)255, so = yo + ((yb + 255) & ~(size_t)255);
    int32_t rc = ensure_pin(c, so + sb + 256);
    if (!rc) rc = ensure_dev_io(c, so + sb + 256);
    if (rc) return rc;
    char *pin = static_cast<char *>(c->pin), *dev = static_cast<char *>(c->dev_io);
    // Page-locked caller buffers (cudaMallocHost / cudaHostRegister) are used as they are: no staging copy on the
    // host.  Anything else goes through the context's own pinned buffer.
    const auto pinned_alias = [](const void *h) -> const void * {
        cudaPointerAttributes at;
        if (cudaPointerGetAttributes(&at, h) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        return at.type == cudaMemoryTypeHost ? at.devicePointer : nullptr;
    };
    const void *x_alias = pinned_alias(x_host);
    const bool y_pinned = pinned_alias(y_host) != nullptr;
    const char *x_src = reinterpret_cast<const char *>(x_host);  // host address copies are issued from
    if (!x_alias) {
        memcpy(pin + xo, x_host, xb);
        x_src = pin + xo;
        x_alias = pin + xo;  // cudaMallocHost memory: same address on the device
    }
    if (sb) memcpy(pin + so, scales_host, sb);
    // Small activation blocks are read by the staging kernel straight from page-locked host memory (mapped into
    // the device's address space): one copy call and its latency less per product.  Larger ones go through HBM.
    const bool zero_copy_x = xb <= (size_t)256 * 1024;
    if (!zero_copy_x) GK_CUDA(c, cudaMemcpyAsync(dev + xo, x_src, xb, cudaMemcpyHostToDevice, c->stream));
    if (sb) GK_CUDA(c, cudaMemcpyAsync(dev + so, pin + so, sb, cudaMemcpyHostToDevice, c->stream));
    const float *xd = reinterpret_cast<const float *>(zero_copy_x ? static_cast<const char *>(x_alias) : dev + xo);
    float *yd = reinterpret_cast<float *>(dev + yo);
    const float *sd = sb ? reinterpret_cast<const float *>(dev + so) : nullptr;
    if (!ref_layout && !sb && m_t > GLLMK_GEMM_GEMV_MAX_M && !raw_format(w->qt)) {
        // prefill-sized batch: one tensor-core GEMM
        rc = gemm_launch(c, w, xd, 0, k, m_t, yd, 0, n_w, c->stream);
        if (rc) return rc;
    } else
    for (int t0 = 0; t0 < m_t; t0 += GLLMK_GEMV_MAX_M) {
        const int mt = (m_t - t0 < GLLMK_GEMV_MAX_M) ? m_t - t0 : GLLMK_GEMV_MAX_M;
        if (ref_layout)
            rc = gemv_launch(c, w, xd + t0, 1, m_t, mt, yd + t0, 1, m_t, sd, (int64_t)n_scales, c->stream);
        else
            rc = gemv_launch(c, w, xd + (size_t)t0 * k, k, 1, mt, yd + (size_t)t0 * n_w, n_w, 1, sd, (int64_t)n_scales,
                             c->stream);
        if (rc) return rc;
    }
    GK_CUDA(c, cudaMemcpyAsync(y_pinned ? static_cast<void *>(y_host) : static_cast<void *>(pin + yo), dev + yo, yb, cudaMemcpyDeviceToHost,
                               c->stream));
    GK_CUDA(c, cudaStreamSynchronize(c->stream));
    if (!y_pinned) memcpy(y_host, pin + yo, yb);
    return GLLMK_STATUS_OK;
}

// Several products with host activations / outputs, enqueued back to back and awaited ONCE: what a decode step is (a
// handful of products whose host-side inputs are all known when the step starts).  The products run on the context's
// stream; every x goes up and every y comes back on a second stream, so the copies of product i + 1 and i - 1 run beside
// product i.  An argument list seen twice in a row is captured as a CUDA graph (same pointers, same shapes, same scratch
// buffers) and replayed from then on: one launch instead of ~3 per product.
struct BatchItem {
    const Weight *w;
    int m;
    size_t xo, yo, xb, yb;
    const char *x_src;  // page-locked source of the upload (the caller's buffer or the staging area)
    void *y_dst;        // page-locked destination of the download
    bool x_staged, y_staged;
};

static int32_t batch_enqueue(Ctx *c, const std::vector<BatchItem> &items, bool ref_layout) {
    char *dev = static_cast<char *>(c->dev_io);
    const size_t count = items.size();
    while (c->events.size() < 2 * count + 2) {
        cudaEvent_t e;
        GK_CUDA(c, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        c->events.push_back(e);
    }
    cudaEvent_t *ev_x = c->events.data() + 2, *ev_y = ev_x + count;
    GK_CUDA(c, cudaEventRecord(c->events[0], c->stream));
    GK_CUDA(c, cudaStreamWaitEvent(c->copy_stream, c->events[0], 0));
    for (size_t i = 0; i < count; i++) {
        GK_CUDA(c, cudaMemcpyAsync(dev + items[i].xo, items[i].x_src, items[i].xb, cudaMemcpyHostToDevice, c->copy_stream));
        GK_CUDA(c, cudaEventRecord(ev_x[i], c->copy_stream));
    }
    for (size_t i = 0; i < count; i++) {
        const BatchItem &it = items[i];
        const Weight *w = it.w;
        const int m_t = it.m;
        const int64_t n_w = w->n, k = w->k;
        const float *xd = reinterpret_cast<const float *>(dev + it.xo);
        float *yd = reinterpret_cast<float *>(dev + it.yo);
        // The upload of product i + 1 is awaited BEFORE product i is enqueued (all uploads were issued up front and take
        // a few us each): the staging kernel of product i + 1 then depends on nothing but the GEMV in front of it, which
        // keeps the programmatic (early) launch between the two.
        if (i == 0) GK_CUDA(c, cudaStreamWaitEvent(c->stream, ev_x[0], 0));
        if (i + 1 < count) GK_CUDA(c, cudaStreamWaitEvent(c->stream, ev_x[i + 1], 0));
        int32_t rc = 0;
        if (!ref_layout && m_t > GLLMK_GEMM_GEMV_MAX_M && !raw_format(w->qt)) {
            rc = gemm_launch(c, w, xd, 0, k, m_t, yd, 0, n_w, c->stream);
            if (rc) return rc;
        } else {
            for (int t0 = 0; t0 < m_t; t0 += GLLMK_GEMV_MAX_M) {
                const int mt = (m_t - t0 < GLLMK_GEMV_MAX_M) ? m_t - t0 : GLLMK_GEMV_MAX_M;
                if (ref_layout) rc = gemv_launch(c, w, xd + t0, 1, m_t, mt, yd + t0, 1, m_t, nullptr, 0, c->stream);
                else rc = gemv_launch(c, w, xd + (size_t)t0 * k, k, 1, mt, yd + (size_t)t0 * n_w, n_w, 1, nullptr, 0, c->stream);
                if (rc) return rc;
            }
        }
        GK_CUDA(c, cudaEventRecord(ev_y[i], c->stream));
        GK_CUDA(c, cudaStreamWaitEvent(c->copy_stream, ev_y[i], 0));
        GK_CUDA(c, cudaMemcpyAsync(it.y_dst, dev + it.yo, it.yb, cudaMemcpyDeviceToHost, c->copy_stream));
    }
    GK_CUDA(c, cudaEventRecord(c->events[1], c->copy_stream));
    GK_CUDA(c, cudaStreamWaitEvent(c->stream, c->events[1], 0));
    return GLLMK_STATUS_OK;
}

static int32_t matmul_host_batch_impl(Ctx *c, int count, const gllmk_weight *ws, const float *const *xs, const int32_t *ms,
                                      float *const *ys, bool ref_layout) {
    const auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    size_t total = 256;
    for (int i = 0; i < count; i++) {
        const Weight *w = static_cast<const Weight *>(ws[i]);
        total += up((size_t)ms[i] * w->k * sizeof(float)) + up((size_t)ms[i] * w->n * sizeof(float));
    }
    int32_t rc = ensure_pin(c, total);
    if (!rc) rc = ensure_dev_io(c, total);
    if (rc) return rc;
    if (!c->copy_stream) GK_CUDA(c, cudaStreamCreateWithFlags(&c->copy_stream, cudaStreamNonBlocking));
    char *pin = static_cast<char *>(c->pin);
    const auto page_locked = [](const void *h) {
        cudaPointerAttributes at;
        if (cudaPointerGetAttributes(&at, h) != cudaSuccess) {
            (void)cudaGetLastError();
            return false;
        }
        return at.type == cudaMemoryTypeHost;
    };
    // what a captured graph depends on: the argument list and every scratch buffer a launch may take its pointers from
    const auto make_key = [&]() {
        std::vector<uint64_t> key;
        key.reserve(8 + 6 * (size_t)count);
        for (const void *q : {static_cast<const void *>(c->pin), static_cast<const void *>(c->dev_io), static_cast<const void *>(c->ws),
                              static_cast<const void *>(c->red), static_cast<const void *>(c->cnt), static_cast<const void *>(c->act)})
            key.push_back((uint64_t)(uintptr_t)q);
        key.push_back((uint64_t)count);
        key.push_back(ref_layout ? 1u : 0u);
        for (int i = 0; i < count; i++) {
            const Weight *w = static_cast<const Weight *>(ws[i]);
            key.push_back((uint64_t)(uintptr_t)ws[i]);
            key.push_back((uint64_t)(uintptr_t)w->qs);
            key.push_back(((uint64_t)w->n << 32) ^ (uint64_t)w->k ^ ((uint64_t)w->qt << 60));
            key.push_back((uint64_t)(uintptr_t)xs[i]);
            key.push_back((uint64_t)(uintptr_t)ys[i]);
            key.push_back((uint64_t)(uint32_t)ms[i]);
        }
        return key;
    };
    const bool replay = c->host_batch_graph && c->batch_exec && make_key() == c->batch_key;
    std::vector<BatchItem> items((size_t)count);
    size_t off = 0;
    for (int i = 0; i < count; i++) {
        BatchItem &it = items[(size_t)i];
        it.w = static_cast<const Weight *>(ws[i]);
        it.m = ms[i];
        it.xb = (size_t)it.m * it.w->k * sizeof(float);
        it.yb = (size_t)it.m * it.w->n * sizeof(float);
        it.xo = off;
        it.yo = off + up(it.xb);
        off = it.yo + up(it.yb);
        // which host buffers are page-locked was found out when the list was captured (same pointers since)
        it.x_staged = replay ? (c->batch_staged[(size_t)i] & 1) != 0 : !page_locked(xs[i]);
        it.y_staged = replay ? (c->batch_staged[(size_t)i] & 2) != 0 : !page_locked(ys[i]);
        it.x_src = it.x_staged ? pin + it.xo : reinterpret_cast<const char *>(xs[i]);
        it.y_dst = it.y_staged ? static_cast<void *>(pin + it.yo) : static_cast<void *>(ys[i]);
        if (it.x_staged) memcpy(pin + it.xo, xs[i], it.xb);
    }
    const auto finish = [&]() -> int32_t {
        GK_CUDA(c, cudaStreamSynchronize(c->stream));
        for (int i = 0; i < count; i++)
            if (items[(size_t)i].y_staged) memcpy(ys[i], pin + items[(size_t)i].yo, items[(size_t)i].yb);
        return GLLMK_STATUS_OK;
    };
    if (replay) {
        GK_CUDA(c, cudaGraphLaunch(c->batch_exec, c->stream));
        return finish();
    }
    rc = batch_enqueue(c, items, ref_layout);
    if (rc) return rc;
    rc = finish();
    if (rc || !c->host_batch_graph) return rc;
    // The scratch buffers have their final sizes now.  Second sighting of this list in a row: capture it for next time.
    std::vector<uint64_t> key = make_key();
    if (key != c->batch_candidate) {
        c->batch_candidate.swap(key);
        return GLLMK_STATUS_OK;
    }
    if (c->batch_exec) {
        cudaGraphExecDestroy(c->batch_exec);
        c->batch_exec = nullptr;
        c->batch_key.clear();
    }
    if (cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeRelaxed) != cudaSuccess) {
        (void)cudaGetLastError();
        return GLLMK_STATUS_OK;  // no graph: the next call enqueues again
    }
    const int32_t crc = batch_enqueue(c, items, ref_layout);
    cudaGraph_t graph = nullptr;
    const cudaError_t ce = cudaStreamEndCapture(c->stream, &graph);
    if (crc == GLLMK_STATUS_OK && ce == cudaSuccess && graph && make_key() == key &&
        cudaGraphInstantiate(&c->batch_exec, graph, 0) == cudaSuccess) {
        c->batch_key.swap(key);
        c->batch_staged.assign((size_t)count, 0);
        for (int i = 0; i < count; i++)
            c->batch_staged[(size_t)i] = (uint8_t)((items[(size_t)i].x_staged ? 1 : 0) | (items[(size_t)i].y_staged ? 2 : 0));
    } else {
        (void)cudaGetLastError();
        c->batch_exec = nullptr;
        c->err.clear();
    }
    if (graph) cudaGraphDestroy(graph);
    return GLLMK_STATUS_OK;
}

int32_t gllmk_matmul_host_batch(gllmk_ctx ctx, int32_t count, const gllmk_weight *weights, const float *const *x_host, const int32_t *m,
                                float *const *y_host, int32_t ref_layout) {
    if (!ctx || !weights || !x_host || !m || !y_host) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    if (count < 0 || count > 4096) return fail(c, GLLMK_STATUS_INVALID_ARG, "matmul_host_batch: count=%d", count);
    for (int i = 0; i < count; i++) {
        if (!weights[i] || !x_host[i] || !y_host[i]) return fail(c, GLLMK_STATUS_INVALID_ARG, "matmul_host_batch: null pointer in product %d", i);
        if (m[i] < 1) return fail(c, GLLMK_STATUS_INVALID_ARG, "matmul_host_batch: m must be positive");
        const Weight *w = static_cast<const Weight *>(weights[i]);
        if (w->qt == GLLMK_QUANT_INT8) return fail(c, GLLMK_STATUS_UNSUPPORTED, "matmul_host_batch: not a block-quantized weight");
        if (w->device != c->device) return fail(c, GLLMK_STATUS_INVALID_ARG, "weight lives on another device");
    }
    if (count == 0) return GLLMK_STATUS_OK;
    DeviceGuard g(c->device);
    return matmul_host_batch_impl(c, count, weights, x_host, m, y_host, ref_layout != 0);
}

int32_t gllmk_matmul_host(gllmk_ctx ctx, gllmk_weight wh, const float *x_host, int32_t m, float *y_host,
                          int32_t ref_layout) {
    if (!ctx || !wh || !x_host || !y_host) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    if (m < 1) return fail(c, GLLMK_STATUS_INVALID_ARG, "m must be positive");
    const Weight *w = static_cast<const Weight *>(wh);
    if (w->device != c->device) return fail(c, GLLMK_STATUS_INVALID_ARG, "weight lives on another device");
    DeviceGuard g(c->device);
    return matmul_host_impl(c, w, x_host, m, y_host, ref_layout != 0, nullptr, 0);
}

static int32_t family_matmul(gllmk_ctx ctx, const uint8_t *wb, const float *input, float *output, int32_t qt,
                             bool kquant, size_t m, size_t n, size_t k) {
    if (!ctx || !wb || !input || !output) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    // kquant_matmul takes the 256-element K-quants, classic_matmul the 32-element formats (src/cpu_kernels/mod.rs:3226-3394)
    const bool ok = kquant ? (qt == GLLMK_QUANT_Q4K || qt == GLLMK_QUANT_Q6_K || qt == GLLMK_QUANT_Q5_K || qt == GLLMK_QUANT_Q8_K)
                           : (qt == GLLMK_QUANT_Q8_0 || qt == GLLMK_QUANT_Q4_0 || qt == GLLMK_QUANT_Q5_0);
    if (!ok)
        return fail(c, GLLMK_STATUS_UNSUPPORTED, "quant type %d is not handled by this entry point", qt);
    if (m == 0 || n == 0) return GLLMK_STATUS_OK;
    if (n > 0x7fffffffu) return fail(c, GLLMK_STATUS_INVALID_ARG, "n too large");
    DeviceGuard g(c->device);
    Weight *w = nullptr;
    int32_t rc = weight_alloc(c, qt, (int64_t)m, (int64_t)k, 0, 1.0f, &w);
    if (rc) return rc;
    rc = weight_fill(c, w, wb, nullptr, false);
    if (!rc) rc = matmul_host_impl(c, w, input, (int)n, output, true, nullptr, 0);
    weight_destroy(w);
    return rc;
}

int32_t gllmk_kquant_matmul_f32(gllmk_ctx ctx, const uint8_t *weight_blocks, const float *input, float *output,
                                int32_t quant_type, size_t m, size_t n, size_t k) {
    return family_matmul(ctx, weight_blocks, input, output, quant_type, true, m, n, k);
}
int32_t gllmk_classic_matmul_f32(gllmk_ctx ctx, const uint8_t *weight_blocks, const float *input, float *output,
                                 int32_t quant_type, size_t m, size_t n, size_t k) {
    return family_matmul(ctx, weight_blocks, input, output, quant_type, false, m, n, k);
}

// gemm_q4 / gemm_q8 share everything but the block format (Q4_K / Q8_K rows of k / 256 blocks).
static int32_t gemm_kq_host(gllmk_ctx ctx, int32_t qt, const char *what, const void *weight, const float *input, float *output,
                            const float *scales, size_t n_scales, size_t m, size_t n, size_t k) {
    if (!ctx || !weight || !input || !output) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    if (n_scales && !scales) return GLLMK_STATUS_INVALID_ARG;
    if (k % 256) return fail(c, GLLMK_STATUS_INVALID_ARG, "%s: k %% 256 != 0", what);
    if (m == 0 || n == 0) return GLLMK_STATUS_OK;
    if (m > 0x7fffffffu) return fail(c, GLLMK_STATUS_INVALID_ARG, "m too large");
    DeviceGuard g(c->device);
    Weight *w = nullptr;
    int32_t rc = weight_alloc(c, qt, (int64_t)n, (int64_t)k, 0, 1.0f, &w);
    if (rc) return rc;
    rc = weight_fill(c, w, weight, nullptr, false);
    if (!rc) rc = matmul_host_impl(c, w, input, (int)m, output, false, scales, n_scales);
    weight_destroy(w);
    return rc;
}

int32_t gllmk_gemm_q4_f32(gllmk_ctx ctx, const uint8_t *weight, const float *input, float *output, const float *scales,
                          size_t n_scales, size_t m, size_t n, size_t k) {
    return gemm_kq_host(ctx, GLLMK_QUANT_Q4K, "gemm_q4", weight, input, output, scales, n_scales, m, n, k);
}
int32_t gllmk_gemm_q8_f32(gllmk_ctx ctx, const int8_t *weight, const float *input, float *output, const float *scales,
                          size_t n_scales, size_t m, size_t n, size_t k) {
    return gemm_kq_host(ctx, GLLMK_QUANT_Q8_K, "gemm_q8", weight, input, output, scales, n_scales, m, n, k);
}
int32_t gllmk_gemv_q4_f32(gllmk_ctx ctx, const uint8_t *weight, const float *input, float scale, size_t n, float *out) {
    if (!out) return GLLMK_STATUS_INVALID_ARG;
    return gemm_kq_host(ctx, GLLMK_QUANT_Q4K, "gemv_q4", weight, input, out, &scale, 1, 1, 1, n);
}
int32_t gllmk_gemv_q8_f32(gllmk_ctx ctx, const int8_t *weight, const float *input, float scale, size_t n, float *out) {
    if (!out) return GLLMK_STATUS_INVALID_ARG;
    return gemm_kq_host(ctx, GLLMK_QUANT_Q8_K, "gemv_q8", weight, input, out, &scale, 1, 1, 1, n);
}

static int32_t dequant_host(gllmk_ctx ctx, int32_t qt, const uint8_t *blocks, const uint8_t *scales, float global,
                            float *out, size_t nblocks, size_t bs) {
    if (!ctx || !blocks || !out) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    if (nblocks == 0) return GLLMK_STATUS_OK;
    DeviceGuard g(c->device);
    const size_t bbytes = (qt == GLLMK_QUANT_MXFP4) ? bs / 2 : (size_t)block_bytes_of(qt, 0);
    const size_t raw = nblocks * bbytes, sraw = (qt == GLLMK_QUANT_MXFP4) ? nblocks : 0, ob = nblocks * bs * sizeof(float);
    const size_t so = (raw + 255) & ~(size_t)255, oo = so + ((sraw + 255) & ~(size_t)255);
    int32_t rc = ensure_dev_io(c, oo + ob + 256);
    if (rc) return rc;
    char *dev = static_cast<char *>(c->dev_io);
    GK_CUDA(c, cudaMemcpyAsync(dev, blocks, raw, cudaMemcpyHostToDevice, c->stream));
    if (sraw) GK_CUDA(c, cudaMemcpyAsync(dev + so, scales, sraw, cudaMemcpyHostToDevice, c->stream));
    rc = dequant_raw(c, qt, reinterpret_cast<uint8_t *>(dev), reinterpret_cast<uint8_t *>(dev + so), global,
                     reinterpret_cast<float *>(dev + oo), nblocks, bs, c->stream);
    if (rc) return rc;
    GK_CUDA(c, cudaMemcpyAsync(out, dev + oo, ob, cudaMemcpyDeviceToHost, c->stream));
    GK_CUDA(c, cudaStreamSynchronize(c->stream));
    return GLLMK_STATUS_OK;
}

int32_t gllmk_dequant_q4_k(gllmk_ctx ctx, const uint8_t *blocks, float *out, size_t nblocks) {
    return dequant_host(ctx, GLLMK_QUANT_Q4K, blocks, nullptr, 1.0f, out, nblocks, 256);
}
int32_t gllmk_dequant_q8_0(gllmk_ctx ctx, const uint8_t *blocks, float *out, size_t nblocks) {
    return dequant_host(ctx, GLLMK_QUANT_Q8_0, blocks, nullptr, 1.0f, out, nblocks, 32);
}
int32_t gllmk_dequant_gguf(gllmk_ctx ctx, int32_t quant_type, const uint8_t *blocks, float *out, size_t nblocks) {
    if (!ctx) return GLLMK_STATUS_INVALID_ARG;
    if (quant_type != GLLMK_QUANT_Q4K && quant_type != GLLMK_QUANT_Q8_0 && !raw_format(quant_type))
        return fail(static_cast<Ctx *>(ctx), GLLMK_STATUS_UNSUPPORTED, "dequant_gguf: quant type %d", quant_type);
    return dequant_host(ctx, quant_type, blocks, nullptr, 1.0f, out, nblocks, (size_t)block_size_of(quant_type, 0));
}
int32_t gllmk_dequant_mxfp4(gllmk_ctx ctx, const uint8_t *blocks, const uint8_t *scales, float *out, size_t num_blocks,
                            size_t block_size) {
    if (!ctx || !scales) return GLLMK_STATUS_INVALID_ARG;
    if (block_size == 0 || (block_size & 1))
        return fail(static_cast<Ctx *>(ctx), GLLMK_STATUS_INVALID_ARG, "mxfp4 block_size must be even and non-zero");
    return dequant_host(ctx, GLLMK_QUANT_MXFP4, blocks, scales, 1.0f, out, num_blocks, block_size);
}
int32_t gllmk_dequant_nvfp4(gllmk_ctx ctx, const uint8_t *blocks, float global_scale, float *out, size_t nblocks) {
    return dequant_host(ctx, GLLMK_QUANT_NVFP4, blocks, nullptr, global_scale, out, nblocks, 64);
}

int32_t gllmk_quantize(gllmk_ctx ctx, int32_t quant_type, const float *x_dev, int64_t rows, int64_t k, int32_t mx_block,
                       void *blocks_dev, void *scales_dev, float *global_scale, void *stream) {
    if (!ctx || !x_dev || !blocks_dev) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    if (rows <= 0 || k <= 0) return fail(c, GLLMK_STATUS_INVALID_ARG, "rows and k must be positive");
    const int bs = block_size_of(quant_type, mx_block);
    if (bs <= 0) return fail(c, GLLMK_STATUS_UNSUPPORTED, "unknown quant type %d", quant_type);
    if (k % bs) return fail(c, GLLMK_STATUS_INVALID_ARG, "k=%lld is not a multiple of the block size %d", (long long)k, bs);
    if (quant_type == GLLMK_QUANT_MXFP4 && !scales_dev) return GLLMK_STATUS_INVALID_ARG;
    if (quant_type == GLLMK_QUANT_NVFP4 && !global_scale) return GLLMK_STATUS_INVALID_ARG;
    DeviceGuard g(c->device);
    return quantize_launch(c, quant_type, x_dev, rows, k, mx_block, blocks_dev, scales_dev, global_scale,
                           static_cast<cudaStream_t>(stream));
}

}  // extern "C"
