// Mixture-of-experts plumbing around the grouped expert GEMM, with the reference's data conventions
// (scalar-ops/src/moe.rs:59-157): the top-k selection writes expert indices as u32 bit patterns stored in f32
// slots followed by the renormalised weights; the recombination adds weight * expert row in k order.
// Between the two, the (token, k) slots are grouped per expert (what gllmk_gemm_grouped takes) and the
// activation rows gathered in that order.
#include <cuda_bf16.h>

#include "common.cuh"

namespace gllmk {

constexpr int MOE_MAX_TOPK = 16;
constexpr int MOE_MAX_EXPERTS = 1024;
// small device scratch inside the context's status allocation (16 KB): ints [256, 256 + 1024) expert counts,
// ints [1280, 1280 + 1025) row offsets
constexpr int MOE_CNT_OFF = 256, MOE_OFF_OFF = 1280;

// scalar_topk, one thread per token: insertion of each expert's probability into a descending list with a
// strict '>' (the earlier expert wins a tie, NaN never enters), then weights = value * (1 / sum) (0 if sum <= 0).
__global__ void moe_topk_kernel(const float *__restrict__ probs, float *__restrict__ out, int64_t seq, int ne, int top_k) {
    const int64_t s = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= seq) return;
    uint32_t ti[MOE_MAX_TOPK];
    float tv[MOE_MAX_TOPK];
    for (int i = 0; i < top_k; i++) { ti[i] = 0u; tv[i] = __int_as_float(0xFF800000); }
    const float *row = probs + s * ne;
    for (int e = 0; e < ne; e++) {
        const float v = row[e];
        int pos = top_k;
        for (int ki = 0; ki < top_k; ki++)
            if (v > tv[ki]) { pos = ki; break; }
        if (pos < top_k) {
            for (int ki = top_k - 1; ki > pos; ki--) { ti[ki] = ti[ki - 1]; tv[ki] = tv[ki - 1]; }
            ti[pos] = (uint32_t)e;
            tv[pos] = v;
        }
    }
    float sum = 0.0f;
    for (int ki = 0; ki < top_k; ki++) sum = __fadd_rn(sum, tv[ki]);
    const float inv = sum > 0.0f ? __fdiv_rn(1.0f, sum) : 0.0f;
    for (int ki = 0; ki < top_k; ki++) {
        out[s * top_k + ki] = __uint_as_float(ti[ki]);
        out[seq * top_k + s * top_k + ki] = __fmul_rn(tv[ki], inv);
    }
}

// One warp per expert walks the index section 32 slots at a time.  place == 0: counts[e] = slots of expert e.
// place != 0: the g-th slot of expert e (in slot order: stable) becomes grouped row offs[e] + g:
// perm[row] = slot, inv[slot] = row.  Slots whose index is >= ne belong to no expert (the reference skips them,
// scalar-ops/src/moe_dispatch_packed.rs:113-116): inv[slot] = -1, written by the warp of expert 0.
__global__ void moe_route_kernel(const float *__restrict__ idx, int64_t slots, int ne, int *counts, const int *offs, int *perm,
                                 int *inv, int place) {
    const int e = blockIdx.x, lane = threadIdx.x;
    int base = place ? offs[e] : 0, n = 0;
    for (int64_t s0 = 0; s0 < slots; s0 += 32) {
        const int64_t s = s0 + lane;
        const uint32_t id = s < slots ? __float_as_uint(idx[s]) : 0xFFFFFFFFu;
        const bool mine = s < slots && id == (uint32_t)e;
        const uint32_t mask = __ballot_sync(0xffffffffu, mine);
        if (place) {
            if (mine) {
                const int row = base + n + __popc(mask & ((1u << lane) - 1u));
                perm[row] = (int)s;
                inv[s] = row;
            } else if (e == 0 && s < slots && id >= (uint32_t)ne) {
                inv[s] = -1;
            }
        }
        n += __popc(mask);
    }
    if (!place && lane == 0) counts[e] = n;
}

template <typename T>
__global__ void moe_gather_kernel(const T *__restrict__ x, int64_t ldx, const int *__restrict__ perm, int top_k, int64_t k,
                                  T *__restrict__ out, int64_t ldo) {
    const int64_t g = blockIdx.x;
    const T *src = x + (int64_t)(perm[g] / top_k) * ldx;
    T *dst = out + g * ldo;
    for (int64_t c = (int64_t)blockIdx.y * blockDim.x + threadIdx.x; c < k; c += (int64_t)gridDim.y * blockDim.x) dst[c] = src[c];
}

// scalar_weighted_sum: out[s, d] = ((0 + w_0 * r_0[d]) + w_1 * r_1[d]) + ... with a separate multiply and add per
// term.  inv == nullptr: expert_outputs is the reference's [expert][seq][hidden] buffer; else it holds the grouped
// rows and inv[s * top_k + ki] names the row (negative: the slot has no expert and adds nothing).
__global__ void moe_wsum_kernel(const float *__restrict__ eo, const float *__restrict__ idx, const float *__restrict__ wts,
                                const int *__restrict__ inv, float *__restrict__ out, int64_t seq, int64_t hidden, int64_t ld,
                                int top_k, int ne) {
    const int64_t s = blockIdx.x;
    for (int64_t d = (int64_t)blockIdx.y * blockDim.x + threadIdx.x; d < hidden; d += (int64_t)gridDim.y * blockDim.x) {
        float acc = 0.0f;
        for (int ki = 0; ki < top_k; ki++) {
            const float w = wts[s * top_k + ki];
            const float *row;
            if (inv) {
                const int r = inv[s * top_k + ki];
                if (r < 0) continue;
                row = eo + (int64_t)r * ld;
            } else {
                const uint32_t e = __float_as_uint(idx[s * top_k + ki]);
                if (e >= (uint32_t)ne) continue;
                row = eo + ((int64_t)e * seq + s) * ld;
            }
            acc = __fadd_rn(acc, __fmul_rn(w, row[d]));
        }
        out[s * hidden + d] = acc;
    }
}

}  // namespace gllmk

using namespace gllmk;

extern "C" int32_t gllmk_moe_topk(gllmk_ctx ctx, const float *gate_probs_dev, float *out_dev, int64_t seq_len, int32_t num_experts,
                                  int32_t top_k, void *stream) {
    if (!ctx || !gate_probs_dev || !out_dev) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    if (seq_len < 0 || num_experts < 1) return fail(c, GLLMK_STATUS_INVALID_ARG, "moe_topk: bad shape");
    if (top_k < 1 || top_k > MOE_MAX_TOPK) return fail(c, GLLMK_STATUS_UNSUPPORTED, "moe_topk: top_k=%d outside 1..%d", top_k, MOE_MAX_TOPK);
    if (seq_len == 0) return GLLMK_STATUS_OK;
    DeviceGuard g(c->device);
    moe_topk_kernel<<<(unsigned)((seq_len + 127) / 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(gate_probs_dev, out_dev, seq_len,
                                                                                                     num_experts, top_k);
    GK_CUDA(c, cudaGetLastError());
    return GLLMK_STATUS_OK;
}

extern "C" int32_t gllmk_moe_route(gllmk_ctx ctx, const float *indices_dev, int64_t seq_len, int32_t num_experts, int32_t top_k,
                                   int64_t *row_offsets_host, int32_t *perm_dev, int32_t *inv_dev, void *stream) {
    if (!ctx || !indices_dev || !row_offsets_host || !perm_dev || !inv_dev) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    if (num_experts < 1 || num_experts > MOE_MAX_EXPERTS)
        return fail(c, GLLMK_STATUS_UNSUPPORTED, "moe_route: num_experts=%d outside 1..%d", num_experts, MOE_MAX_EXPERTS);
    const int64_t slots = seq_len * (int64_t)top_k;
    if (seq_len < 0 || top_k < 1 || slots > 0x7fffffff) return fail(c, GLLMK_STATUS_INVALID_ARG, "moe_route: bad shape");
    DeviceGuard g(c->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int *counts = c->status_dev + MOE_CNT_OFF, *offs = c->status_dev + MOE_OFF_OFF;
    moe_route_kernel<<<num_experts, 32, 0, s>>>(indices_dev, slots, num_experts, counts, nullptr, nullptr, nullptr, 0);
    GK_CUDA(c, cudaGetLastError());
    int host_counts[MOE_MAX_EXPERTS], host_offs[MOE_MAX_EXPERTS + 1];
    GK_CUDA(c, cudaMemcpyAsync(host_counts, counts, sizeof(int) * num_experts, cudaMemcpyDeviceToHost, s));
    GK_CUDA(c, cudaStreamSynchronize(s));
    host_offs[0] = 0;
    for (int e = 0; e < num_experts; e++) host_offs[e + 1] = host_offs[e] + host_counts[e];
    for (int e = 0; e <= num_experts; e++) row_offsets_host[e] = host_offs[e];
    GK_CUDA(c, cudaMemcpyAsync(offs, host_offs, sizeof(int) * (num_experts + 1), cudaMemcpyHostToDevice, s));
    moe_route_kernel<<<num_experts, 32, 0, s>>>(indices_dev, slots, num_experts, counts, offs, perm_dev, inv_dev, 1);
    GK_CUDA(c, cudaGetLastError());
    GK_CUDA(c, cudaStreamSynchronize(s));  // host_offs lives on this stack frame
    return GLLMK_STATUS_OK;
}

extern "C" int32_t gllmk_moe_gather(gllmk_ctx ctx, const void *x_dev, int32_t dtype, int64_t ldx, const int32_t *perm_dev, int64_t rows,
                                    int32_t top_k, int64_t k, void *out_dev, int64_t ldo, void *stream) {
    if (!ctx || !x_dev || !perm_dev || !out_dev) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    if (dtype != GLLMK_DTYPE_F32 && dtype != GLLMK_DTYPE_BF16) return fail(c, GLLMK_STATUS_UNSUPPORTED, "moe_gather: dtype");
    if (rows < 0 || rows > 0x7fffffff || top_k < 1 || k < 1 || ldx < k || ldo < k) return fail(c, GLLMK_STATUS_INVALID_ARG, "moe_gather: bad shape");
    if (rows == 0) return GLLMK_STATUS_OK;
    DeviceGuard g(c->device);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    dim3 grid((unsigned)rows, (unsigned)((k + 1023) / 1024 > 8 ? 8 : (k + 1023) / 1024));
    if (dtype == GLLMK_DTYPE_F32)
        moe_gather_kernel<float><<<grid, 256, 0, s>>>(static_cast<const float *>(x_dev), ldx, perm_dev, top_k, k, static_cast<float *>(out_dev), ldo);
    else
        moe_gather_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16 *>(x_dev), ldx, perm_dev, top_k, k,
                                                              static_cast<__nv_bfloat16 *>(out_dev), ldo);
    GK_CUDA(c, cudaGetLastError());
    return GLLMK_STATUS_OK;
}

extern "C" int32_t gllmk_moe_weighted_sum(gllmk_ctx ctx, const float *expert_outputs_dev, int64_t ld, const float *indices_dev,
                                          const float *weights_dev, const int32_t *inv_dev, float *out_dev, int64_t seq_len,
                                          int64_t hidden, int32_t top_k, int32_t num_experts, void *stream) {
    if (!ctx || !expert_outputs_dev || !indices_dev || !weights_dev || !out_dev) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    if (seq_len < 0 || seq_len > 0x7fffffff || hidden < 1 || ld < hidden || top_k < 1 || num_experts < 1)
        return fail(c, GLLMK_STATUS_INVALID_ARG, "moe_weighted_sum: bad shape");
    if (seq_len == 0) return GLLMK_STATUS_OK;
    DeviceGuard g(c->device);
    dim3 grid((unsigned)seq_len, (unsigned)((hidden + 1023) / 1024 > 16 ? 16 : (hidden + 1023) / 1024));
    moe_wsum_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(expert_outputs_dev, indices_dev, weights_dev, inv_dev, out_dev,
                                                                        seq_len, hidden, ld, top_k, num_experts);
    GK_CUDA(c, cudaGetLastError());
    return GLLMK_STATUS_OK;
}
