// Prefill path: fused dequantize + GEMM on tcgen05 tensor cores with the accumulator in TMEM.
//
//   Y[t, r] = sum_k W[r, k] * X[t, k]        t < M tokens (M > 16), r < N weight rows
//
// Weight-only formats (Q4_K, Q8_0, MXFP4, NVFP4 weights with bf16/f32 activations), gemm_wq_kernel:
//   UMMA operand A = 128 weight rows x 64 k, dequantized to fp16 by four producer warps straight into the
//   128-byte-swizzled K-major shared-memory layout the tensor core reads (one thread = one weight row);
//   operand B = up to 256 tokens x 64 k of activations (f32 or bf16 in memory, fp16 in shared memory:
//   kind::f16 takes one 16-bit format for both operands; mixing f16 and bf16 is an illegal instruction);
//   D = 128 lanes (weight rows) x up to 256 columns (tokens) of f32 in tensor memory.
//   Putting the weights on the M side means a CTA dequantizes its weight tile once for all of its tokens
//   and the epilogue's warp-wide stores (lane = consecutive r) are coalesced in Y's row-major layout.
//   One elected thread issues tcgen05.mma (kind::f16); tcgen05.commit releases the shared-memory stage.
//   Staging: weights fp16, activations fp16/bf16, accumulate f32 (parity bar 1e-2; measured ~1e-3).
// No cluster-multicast load is used anywhere (the same kernel serves the multi-GPU configuration).
#include <cuda_bf16.h>

#include "common.cuh"
#include "tc05.cuh"

namespace gllmk {

constexpr int GEMM_BM = 128;     // weight rows per CTA (UMMA M)
constexpr int GEMM_BN = 256;     // tokens per CTA (UMMA N, <= 256)
constexpr int GEMM_BK = 64;      // k per stage: 64 bf16 = one 128-byte swizzle row
constexpr int GEMM_STAGES = 4;
constexpr int GEMM_A_BYTES = GEMM_BM * 128, GEMM_B_BYTES = GEMM_BN * 128;
constexpr int GEMM_STAGE_BYTES = GEMM_A_BYTES + GEMM_B_BYTES;
constexpr int GEMM_THREADS = 160;  // warps 0-3: producers, then epilogue; warp 4: MMA issue + TMEM
constexpr size_t GEMM_SMEM = (size_t)GEMM_STAGES * GEMM_STAGE_BYTES + 1024;

struct GemmParams {
    const uint8_t *qs;   // weight plane (format-specific, see common.cuh)
    const uint8_t *aux;  // FP4 scale-factor plane
    int qt;
    int64_t n, k, nb;    // nb: blocks per row (Q4_K 256-blocks, Q8_0 groups of 8 blocks)
    float global_scale;
    const void *a;       // activations [m, k] row-major, leading dimension lda (elements)
    int a_bf16;          // 1: bf16, 0: f32
    int64_t lda;
    int m;
    void *y;             // [m, n] row-major, leading dimension ldy
    int y_bf16;
    int64_t ldy;
    int *status;
};

// weights are staged in fp16 (11 significant bits; |w| of these formats is far inside its range)
__device__ __forceinline__ uint32_t pack_w(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&v);
}
// activations are staged in fp16 too, saturating at +-65504
__device__ __forceinline__ uint32_t pack_x(float a, float b) {
    uint32_t r;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;\n" : "=r"(r) : "f"(b), "f"(a));
    return r;
}
__device__ __forceinline__ size_t fp4_sf_offset(int64_t row, int64_t s, int64_t s_per_row) {
    const size_t atom = (size_t)(row >> 7) * (size_t)(s_per_row >> 2) + (size_t)(s >> 2);
    return atom * 512 + (size_t)(row & 31) * 16 + (size_t)((row & 127) >> 5) * 4 + (size_t)(s & 3);
}

// Decodes 64 consecutive k (stage ks) of weight row `row` to fp16: out[c] = 16-byte chunk c (8 values).
// Values are d*sc*q - dmin*m etc. evaluated in f32 and rounded once to fp16.
__device__ __forceinline__ void dequant_row64(const GemmParams &p, int64_t row, int ks, uint4 (&out)[8]) {
    const int64_t T = row >> 4;
    const int rr = (int)(row & 15), g = rr & 7, h = rr >> 3;
    if (p.qt == GLLMK_QUANT_Q4K) {
        const int64_t b = ks >> 2;
        const int pg = ks & 3;
        const uint8_t *chunk = p.qs + q4k_chunk_index(T, b, p.nb) * Q4K_CHUNK;
        const uint4 hd = *reinterpret_cast<const uint4 *>(chunk + 2048 + rr * 16);
        const uint32_t dd = *reinterpret_cast<const uint32_t *>(chunk + 2304 + (g * 2 + h) * 4);
        const float d = __half2float(__ushort_as_half((unsigned short)(dd & 0xFFFFu)));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(dd >> 16)));
        const uint32_t scw = pg < 2 ? hd.x : hd.y, mnw = pg < 2 ? hd.z : hd.w;
        const int sh = 16 * (pg & 1);
        const float d1 = d * (float)((scw >> sh) & 0xFFu), m1 = dmin * (float)((mnw >> sh) & 0xFFu);
        const float d2 = d * (float)((scw >> (sh + 8)) & 0xFFu), m2 = dmin * (float)((mnw >> (sh + 8)) & 0xFFu);
#pragma unroll
        for (int t = 0; t < 4; t++) {
            const uint2 w = *reinterpret_cast<const uint2 *>(chunk + (pg * 32 + 4 * g + t) * 16 + h * 8);
            uint32_t lo[4], hi[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t word = j < 2 ? w.x : w.y;
                const int s0 = 16 * (j & 1);
                lo[j] = pack_w(fmaf(d1, (float)((word >> s0) & 15u), -m1), fmaf(d1, (float)((word >> (s0 + 8)) & 15u), -m1));
                hi[j] = pack_w(fmaf(d2, (float)((word >> (s0 + 4)) & 15u), -m2), fmaf(d2, (float)((word >> (s0 + 12)) & 15u), -m2));
            }
            out[t] = make_uint4(lo[0], lo[1], lo[2], lo[3]);      // elements 8t .. 8t+7 (low nibbles, sub-block 2pg)
            out[4 + t] = make_uint4(hi[0], hi[1], hi[2], hi[3]);  // elements 32+8t .. (high nibbles, sub-block 2pg+1)
        }
    } else if (p.qt == GLLMK_QUANT_Q8_0) {
        const int64_t b8 = ks >> 2;
        const int bb0 = (2 * ks) & 7;
        const uint8_t *chunk = p.qs + q4k_chunk_index(T, b8, p.nb) * Q80_CHUNK;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int bb = bb0 + j;
            const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(chunk + 4096 + (rr * 8 + bb) * 2)));
#pragma unroll
            for (int t = 0; t < 4; t++) {
                const uint2 w = *reinterpret_cast<const uint2 *>(chunk + (bb * 32 + 4 * g + t) * 16 + h * 8);
                uint32_t o[4];
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const uint32_t word = q < 2 ? w.x : w.y;
                    const int s0 = 16 * (q & 1);
                    o[q] = pack_w(d * (float)(int8_t)((word >> s0) & 0xFFu), d * (float)(int8_t)((word >> (s0 + 8)) & 0xFFu));
                }
                out[4 * j + t] = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
    } else {
        const bool nv = p.qt == GLLMK_QUANT_NVFP4;
        const uint4 *src = reinterpret_cast<const uint4 *>(p.qs + (size_t)row * (p.k >> 1) + 32 * ks);
        const uint4 raw[2] = {src[0], src[1]};
#pragma unroll
        for (int c = 0; c < 8; c++) {
            const uint4 r4 = raw[c >> 2];
            const uint32_t word = (c & 3) == 0 ? r4.x : ((c & 3) == 1 ? r4.y : ((c & 3) == 2 ? r4.z : r4.w));
            float s;
            if (nv) s = p.global_scale * e4m3_to_f32(p.aux[fp4_sf_offset(row, 4 * ks + (c >> 1), p.k >> 4)]);
            else s = e8m0_to_f32(p.aux[fp4_sf_offset(row, 2 * ks + (c >> 2), p.k >> 5)]);
            uint32_t o[4];
#pragma unroll
            for (int q = 0; q < 4; q++)
                o[q] = pack_w(e2m1_to_f32((word >> (8 * q)) & 15u) * s, e2m1_to_f32((word >> (8 * q + 4)) & 15u) * s);
            out[c] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

// Loads 64 k of one activation row (token) as bf16 chunks; rows >= m give zeros.
__device__ __forceinline__ void load_act_row64(const GemmParams &p, int64_t tok, int ks, uint4 (&out)[8]) {
    if (tok >= p.m) {
#pragma unroll
        for (int c = 0; c < 8; c++) out[c] = make_uint4(0, 0, 0, 0);
        return;
    }
    if (p.a_bf16) {
        const uint4 *src = reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(p.a) + tok * p.lda + (int64_t)ks * 64);
#pragma unroll
        for (int c = 0; c < 8; c++) {
            // bf16 -> fp16 (exact inside fp16's range): kind::f16 wants both operands in one 16-bit format
            const uint4 v = __ldg(src + c);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            uint32_t o[4];
#pragma unroll
            for (int q = 0; q < 4; q++) o[q] = pack_x(__uint_as_float(w[q] << 16), __uint_as_float(w[q] & 0xFFFF0000u));
            out[c] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    } else {
        const float4 *src = reinterpret_cast<const float4 *>(static_cast<const float *>(p.a) + tok * p.lda + (int64_t)ks * 64);
#pragma unroll
        for (int c = 0; c < 8; c++) {
            const float4 a = __ldg(src + 2 * c), b = __ldg(src + 2 * c + 1);
            out[c] = make_uint4(pack_x(a.x, a.y), pack_x(a.z, a.w), pack_x(b.x, b.y), pack_x(b.z, b.w));
        }
    }
}

__device__ __forceinline__ void store_row_sw128(uint8_t *tile, int row, const uint4 (&v)[8]) {
#pragma unroll
    for (int c = 0; c < 8; c++) *reinterpret_cast<uint4 *>(tile + tc::sw128_offset(row, c)) = v[c];
}

// grid: (weight-row tiles of 128, token tiles of 256).  ntok = MMA N of this launch (multiple of 16, <= 256).
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_wq_kernel(const __grid_constant__ GemmParams p, const int ntok) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * GEMM_STAGES + 1];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    uint8_t *smem = smem_raw + ((1024u - (tc::smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t smem_s = tc::smem_u32(smem);
    const uint32_t full = tc::smem_u32(&bars[0]), empty = tc::smem_u32(&bars[GEMM_STAGES]),
                   accum = tc::smem_u32(&bars[2 * GEMM_STAGES]);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row0 = (int64_t)blockIdx.x * GEMM_BM, tok0 = (int64_t)blockIdx.y * GEMM_BN;
    const int nks = (int)(p.k / GEMM_BK);
    volatile int *abort_flag = &abort_s;

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < GEMM_STAGES; s++) {
            tc::mbar_init(full + 8 * s, 128);
            tc::mbar_init(empty + 8 * s, 1);
        }
        tc::mbar_init(accum, 1);
        tc::mbar_init_fence();
    }
    if (warp == 4) tc::tmem_alloc(tc::smem_u32(&tmem_base_s), 256);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_d = tmem_base_s;

    if (warp < 4) {
        // ---------------- producers: one weight row and up to two token rows per thread ----------------
        const int r = threadIdx.x;
        for (int ks = 0; ks < nks; ks++) {
            const int s = ks % GEMM_STAGES;
            if (ks >= GEMM_STAGES && !tc::mbar_wait(empty + 8 * s, (uint32_t)((ks / GEMM_STAGES - 1) & 1), abort_flag)) {
                abort_s = 1;
                atomicExch(p.status, 11);
                break;
            }
            uint8_t *at = smem + s * GEMM_STAGE_BYTES, *bt = at + GEMM_A_BYTES;
            uint4 v[8];
            dequant_row64(p, row0 + r, ks, v);
            store_row_sw128(at, r, v);
#pragma unroll 1
            for (int half = 0; half < 2; half++) {
                const int tr = r + 128 * half;
                if (tr < ntok) {
                    load_act_row64(p, tok0 + tr, ks, v);
                    store_row_sw128(bt, tr, v);
                }
            }
            tc::fence_proxy_async();
            tc::mbar_arrive(full + 8 * s);
        }
    } else if (lane == 0) {
        // ---------------- MMA issue: one thread ----------------
        const uint32_t idesc = tc::idesc_f16(GEMM_BM, ntok, 0, 0);  // fp16 x fp16 -> f32
        for (int ks = 0; ks < nks; ks++) {
            const int s = ks % GEMM_STAGES;
            if (!tc::mbar_wait(full + 8 * s, (uint32_t)((ks / GEMM_STAGES) & 1), abort_flag)) {
                abort_s = 1;
                atomicExch(p.status, 12);
                break;
            }
            tc::fence_after_sync();
            const uint64_t ad = tc::smem_desc_sw128(smem_s + s * GEMM_STAGE_BYTES);
            const uint64_t bd = tc::smem_desc_sw128(smem_s + s * GEMM_STAGE_BYTES + GEMM_A_BYTES);
#pragma unroll
            for (int k4 = 0; k4 < 4; k4++) tc::mma_f16(tmem_d, ad + 2 * k4, bd + 2 * k4, idesc, (uint32_t)((ks | k4) != 0));
            tc::mma_commit(empty + 8 * s);  // frees the stage when these MMAs have read it
        }
        tc::mma_commit(accum);
    }
    __syncwarp();

    if (warp < 4) {
        // ---------------- epilogue: warp w owns TMEM lanes 32w .. 32w+31 = weight rows ----------------
        bool ok = !abort_s && tc::mbar_wait(accum, 0u, abort_flag);
        if (!ok && !abort_s) {
            abort_s = 1;
            atomicExch(p.status, 13);
        }
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc::fence_after_sync();
            const int64_t row = row0 + threadIdx.x;
            for (int c = 0; c < ntok; c += 32) {
                uint32_t v[32];
                tc::tmem_ld32(tmem_d + ((uint32_t)(32 * warp) << 16) + (uint32_t)c, v);
                tc::tmem_ld_wait();
                if (row < p.n) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int64_t tok = tok0 + c + j;
                        if (tok < p.m && c + j < ntok) {
                            if (p.y_bf16) static_cast<__nv_bfloat16 *>(p.y)[tok * p.ldy + row] = __float2bfloat16_rn(__uint_as_float(v[j]));
                            else static_cast<float *>(p.y)[tok * p.ldy + row] = __uint_as_float(v[j]);
                        }
                    }
                }
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 4) tc::tmem_dealloc(tmem_d, 256);
}

// ---------------------------------------------------------------------------------------------
int32_t gemm_launch(Ctx *c, const Weight *w, const void *a, int a_bf16, int64_t lda, int m, void *y, int y_bf16, int64_t ldy,
                    cudaStream_t s) {
    if (w->k % GEMM_BK) return fail(c, GLLMK_STATUS_INVALID_ARG, "gemm: k=%lld is not a multiple of %d", (long long)w->k, GEMM_BK);
    const int align = a_bf16 ? 8 : 4;
    if (((uintptr_t)a & 15) || (lda % align)) return fail(c, GLLMK_STATUS_INVALID_ARG, "gemm: activations must be 16-byte aligned rows");
    static bool attr_set = false;
    if (!attr_set) {
        GK_CUDA(c, cudaFuncSetAttribute(gemm_wq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM_SMEM));
        attr_set = true;
    }
    GemmParams p{};
    p.qs = static_cast<const uint8_t *>(w->qs);
    p.aux = static_cast<const uint8_t *>(w->aux);
    p.qt = w->qt;
    p.n = w->n;
    p.k = w->k;
    p.nb = (w->qt == GLLMK_QUANT_Q8_0) ? w->nb8 : w->nb;
    p.global_scale = w->global_scale;
    p.a = a;
    p.a_bf16 = a_bf16;
    p.lda = lda;
    p.m = m;
    p.y = y;
    p.y_bf16 = y_bf16;
    p.ldy = ldy;
    p.status = c->status_dev;
    const int mtiles = (m + GEMM_BN - 1) / GEMM_BN;
    // MMA N: the whole 256-token tile, or the remainder rounded up to a multiple of 32 when m is small
    const int ntok = (m >= GEMM_BN) ? GEMM_BN : ((m + 31) / 32) * 32;
    dim3 grid((unsigned)(w->n_pad / GEMM_BM), (unsigned)mtiles);
    gemm_wq_kernel<<<grid, GEMM_THREADS, GEMM_SMEM, s>>>(p, ntok);
    GK_CUDA(c, cudaGetLastError());
    return GLLMK_STATUS_OK;
}

}  // namespace gllmk
