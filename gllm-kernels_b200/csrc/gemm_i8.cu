// W8A8 integer GEMM: C (s32) = A (u8 activations) x W (s8 weights), exact, on tcgen05 (kind::i8) with the
// accumulator in tensor memory; plus the dequantize epilogue of the reference as a separate element-wise pass.
//
//   C[t, r] = sum_k A[t, k] * W[r, k]          t < M tokens, r < N weight rows        (all integers, no rounding)
//
// Counterpart: avx512_int8::gemm_int8 / dequantize_i32_to_f32 (src/macros/matmul_x86_int8.rs:307-440), whose B
// operand is [K, N] row-major s8 (and a packed copy of it).  Here the weight is repacked once into 16 KB tile
// images (128 rows x 128 k, 128-byte swizzle, order [row tile][k-step]) and the u8 activations are turned into
// the same kind of images per call, so every operand stage is a plain bulk copy; one thread issues four
// tcgen05.mma of K = 32 per stage into a 128 x N s32 accumulator; eight warps store it (transposed through
// shared memory, 16 bytes per lane).  Weights on the M side as in the other prefill kernels.
#include "common.cuh"
#include "tc05.cuh"

namespace gllmk {

constexpr int I8_BM = 128, I8_BN = 256, I8_TILE = 16384;
constexpr int I8_MAX_STAGES = 4;
// a stage = MT weight tiles + up to two activation tiles; MT = 2 (two accumulators share one activation stage)
// needs a third fewer bytes from L2 per MAC, which is what bounds this kernel
template <int MT>
__host__ __device__ constexpr int i8_stage_bytes() { return MT * I8_TILE + 2 * I8_TILE; }
template <int MT>
__host__ __device__ constexpr int i8_stages() { return MT == 2 ? 3 : 4; }
constexpr int I8_EPI_WARPS = 8;
constexpr int I8_THREADS = 64 + 32 * I8_EPI_WARPS;     // warp 0: copies, warp 1: MMA + TMEM, then the epilogue warps
template <int MT>
__host__ __device__ constexpr size_t i8_smem() { return (size_t)i8_stages<MT>() * i8_stage_bytes<MT>() + 1024; }

struct I8Params {
    const uint8_t *w;   // weight tile images
    const uint8_t *xt;  // activation tile images [token tile of 128][k-step][16384]
    int64_t n;
    int row_tiles;
    int nks;            // k-steps of 128
    int m;
    int32_t *c;         // [m, n] row-major, leading dimension ldc
    int64_t ldc;
    int vec;
    int *status;
};

__device__ __forceinline__ void i8_bulk(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}

// ---- repack: s8 weights [K, N] (layout 0, the reference's B) or [N, K] (layout 1) -> tile images; thread = 16 k of a row
__global__ void __launch_bounds__(256) repack_i8_kernel(const int8_t *__restrict__ b, uint8_t *__restrict__ out, int64_t n, int64_t k,
                                                        int64_t k_pad, int layout, size_t total) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // (k chunk, padded row): rows fastest for layout 0
    if (idx >= total) return;
    const int64_t n_pad = (n + 127) / 128 * 128;
    const int64_t row = (int64_t)(idx % (size_t)n_pad), kc = (int64_t)(idx / (size_t)n_pad);
    uint32_t v[4] = {0, 0, 0, 0};
    if (row < n) {
        for (int i = 0; i < 16; i++) {
            const int64_t kk = kc * 16 + i;
            if (kk < k) {
                const uint8_t by = (uint8_t)(layout == 0 ? b[kk * n + row] : b[row * k + kk]);
                v[i >> 2] |= (uint32_t)by << (8 * (i & 3));
            }
        }
    }
    const size_t tile = (size_t)(row >> 7) * (size_t)(k_pad >> 7) + (size_t)(kc >> 3);
    *reinterpret_cast<uint4 *>(out + tile * I8_TILE + tc::sw128_offset((int)(row & 127), (int)(kc & 7))) = make_uint4(v[0], v[1], v[2], v[3]);
}

// ---- u8 activations [m, k] (leading dimension lda, any alignment) -> tile images; grid (k-steps, token tiles of 128)
__global__ void __launch_bounds__(256) stage_act_u8_kernel(const uint8_t *__restrict__ a, int64_t lda, int m, int64_t k,
                                                           uint8_t *__restrict__ xt) {
    const int ks = blockIdx.x, tile = blockIdx.y;
    uint8_t *dst = xt + ((size_t)tile * gridDim.x + ks) * I8_TILE;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int item = threadIdx.x + 256 * i, row = item >> 3, chunk = item & 7;
        const int64_t tok = (int64_t)tile * 128 + row, k0 = (int64_t)ks * 128 + chunk * 16;
        uint32_t v[4] = {0, 0, 0, 0};
        if (tok < m) {
            const uint8_t *src = a + tok * lda + k0;
            for (int j = 0; j < 16; j++)
                if (k0 + j < k) v[j >> 2] |= (uint32_t)src[j] << (8 * (j & 3));
        }
        *reinterpret_cast<uint4 *>(dst + tc::sw128_offset(row, chunk)) = make_uint4(v[0], v[1], v[2], v[3]);
    }
}

// grid (groups of MT weight-row tiles, token tiles of 256); ntok = MMA N (multiple of 32, <= 256)
template <int MT>
__global__ void __launch_bounds__(I8_THREADS, 1) gemm_i8_kernel(const __grid_constant__ I8Params p, const int ntok) {
    constexpr int I8_STAGES = i8_stages<MT>(), I8_STAGE_BYTES = i8_stage_bytes<MT>();
    constexpr uint32_t TMEM_COLS = MT == 2 ? 512 : 256;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * I8_MAX_STAGES + 1];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    const uint32_t smem_s = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t full = tc::smem_u32(&bars[0]), empty = tc::smem_u32(&bars[I8_MAX_STAGES]), accum = tc::smem_u32(&bars[2 * I8_MAX_STAGES]);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile0 = (int)blockIdx.x * MT;
    const int mt = min(MT, p.row_tiles - tile0);  // row tiles this CTA really has
    const int64_t tok0 = (int64_t)blockIdx.y * I8_BN;
    volatile int *abort_flag = &abort_s;

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < I8_STAGES; s++) {
            tc::mbar_init(full + 8 * s, 1);
            tc::mbar_init(empty + 8 * s, 1);
        }
        tc::mbar_init(accum, 1);
        tc::mbar_init_fence();
    }
    if (warp == 1) tc::tmem_alloc(tc::smem_u32(&tmem_base_s), TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = tmem_base_s;

    if (warp == 0 && lane == 0) {
        // ---------------- copies: one weight tile and one or two activation tiles per k-step ----------------
        const int halves = (ntok + 127) / 128;
        const uint32_t bbytes = (uint32_t)ntok * 128u;
        const uint32_t hb[2] = {ntok > 128 ? (uint32_t)I8_TILE : bbytes, bbytes - (uint32_t)I8_TILE};
        for (int ks = 0; ks < p.nks; ks++) {
            const int s = ks % I8_STAGES;
            if (ks >= I8_STAGES && !tc::mbar_wait(empty + 8 * s, (uint32_t)((ks / I8_STAGES - 1) & 1), abort_flag)) {
                abort_s = 1;
                atomicExch(p.status, 41);
                break;
            }
            const uint32_t st = smem_s + s * I8_STAGE_BYTES;
            tc::mbar_expect_tx(full + 8 * s, (uint32_t)(mt * I8_TILE) + bbytes);
            for (int i = 0; i < mt; i++)
                i8_bulk(st + i * I8_TILE, p.w + ((size_t)(tile0 + i) * p.nks + ks) * I8_TILE, I8_TILE, full + 8 * s);
            for (int h = 0; h < halves; h++)
                i8_bulk(st + MT * I8_TILE + h * I8_TILE, p.xt + ((size_t)((tok0 >> 7) + h) * p.nks + ks) * I8_TILE, hb[h], full + 8 * s);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- MMA issue: weights signed (operand A), activations unsigned (operand B) ----------------
        const uint32_t idesc = tc::idesc_i8(I8_BM, ntok, 1, 0);
        bool ok = true;
        for (int ks = 0; ks < p.nks; ks++) {
            const int s = ks % I8_STAGES;
            if (!tc::mbar_wait(full + 8 * s, (uint32_t)((ks / I8_STAGES) & 1), abort_flag)) {
                abort_s = 1;
                atomicExch(p.status, 42);
                ok = false;
                break;
            }
            tc::fence_after_sync();
            const uint32_t st = smem_s + s * I8_STAGE_BYTES;
            const uint64_t bd = tc::smem_desc_sw128(st + MT * I8_TILE);
            for (int i = 0; i < mt; i++) {
                const uint64_t ad = tc::smem_desc_sw128(st + i * I8_TILE);
#pragma unroll
                for (int j = 0; j < 4; j++) tc::mma_i8(tmem + 256u * (uint32_t)i, ad + 2 * j, bd + 2 * j, idesc, (uint32_t)((ks | j) != 0));
            }
            tc::mma_commit(empty + 8 * s);
        }
        if (ok) tc::mma_commit(accum);
    }
    __syncwarp();

    if (warp >= 2) {
        // ---------------- epilogue: warp w reads TMEM lane quadrant w % 4 = weight rows ----------------
        const int quad = warp & 3;
        bool ok = !abort_s && tc::mbar_wait(accum, 0u, abort_flag);
        if (!ok && !abort_s) {
            abort_s = 1;
            atomicExch(p.status, 43);
        }
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc::fence_after_sync();
            // all MMAs have completed, so the stages are free: each warp stages its blocks in 4 KB of stage 0
            uint8_t *stage = smem_raw + (smem_s - tc::smem_u32(smem_raw)) + (warp - 2) * 4096;
            for (int i = 0; i < mt; i++) {
                const int64_t row0 = (int64_t)(tile0 + i) * I8_BM;
                for (int c = 32 * ((warp - 2) >> 2); c < ntok; c += 32 * (I8_EPI_WARPS / 4)) {
                    uint32_t v[32];
                    tc::tmem_ld32(tmem + ((uint32_t)(32 * quad) << 16) + 256u * (uint32_t)i + (uint32_t)c, v);
                    tc::tmem_ld_wait();
                    float o[32];  // the s32 bit patterns travel through the 32-bit store helper unchanged
#pragma unroll
                    for (int j = 0; j < 32; j++) o[j] = __uint_as_float(v[j]);
                    tc::store_block_32x32<false>(p.c, p.ldc, row0 + 32 * quad, tok0 + c, p.n, p.m, o, stage, lane, p.vec);
                }
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem, TMEM_COLS);
}

// dequantize_i32_to_f32 (src/macros/matmul_x86_int8.rs:414-456, scalar tail semantics): (c as f32) * scale_a * scale_b
// (+ bias[j]), then the activation of src/macros/gemm_epilogue.rs:131-152
// scale_a_dev != nullptr: the activation scale is read from device memory (written by the activation quantizer of the
// same stream).  colsum != nullptr: the activations were stored as q + 128 (unsigned), so 128 * sum_k B[k, j] is
// taken off the integer result first — exact, the s32 range holds both terms for k < 66000.
__global__ void __launch_bounds__(256) dequant_i32_kernel(const int32_t *__restrict__ c, float *__restrict__ out, int64_t n, int64_t ldc,
                                                          int64_t ldo, float scale_a, float scale_b, const float *__restrict__ bias,
                                                          int act, size_t total, const float *__restrict__ scale_a_dev,
                                                          const int32_t *__restrict__ colsum) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int64_t i = (int64_t)(idx / (size_t)n), j = (int64_t)(idx % (size_t)n);
    if (scale_a_dev) scale_a = *scale_a_dev;
    int32_t ci = c[i * ldc + j];
    if (colsum) ci -= 128 * colsum[j];
    float v = __fmul_rn(__fmul_rn((float)ci, scale_a), scale_b);
    if (bias) v = __fadd_rn(v, bias[j]);
    if (act == 1) v = v < 0.0f ? 0.0f : v;
    else if (act == 2) v = v / (1.0f + expf(-v));
    else if (act == 3 || act == 4) {
        const float inner = 0.7978845608f * (v + 0.044715f * v * v * v);
        v = 0.5f * v * (1.0f + tanhf(inner));
    }
    out[i * ldo + j] = v;
}

// ---------------------------------------------------------------------------------------------
// one warp per weight row j: colsum[j] = sum_k B[k, j]
__global__ void __launch_bounds__(256) i8_colsum_kernel(const int8_t *__restrict__ b, int64_t n, int64_t k, int layout, int32_t *__restrict__ colsum) {
    const int64_t j = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (j >= n) return;
    int32_t acc = 0;
    for (int64_t kk = lane; kk < k; kk += 32) acc += layout == 0 ? (int32_t)b[kk * n + j] : (int32_t)b[j * k + kk];
#pragma unroll
    for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) colsum[j] = acc;
}

int32_t i8_weight_fill(Ctx *c, Weight *w, const int8_t *b_dev, int layout, cudaStream_t s) {
    const size_t total = (size_t)w->n_pad * (size_t)(w->k_pad / 16);
    repack_i8_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(b_dev, static_cast<uint8_t *>(w->qs), w->n, w->k, w->k_pad, layout, total);
    GK_CUDA(c, cudaGetLastError());
    if (w->aux) {  // per-column sums of B: the zero-point correction of the f32 -> u8 activation path
        i8_colsum_kernel<<<(unsigned)((w->n * 32 + 255) / 256), 256, 0, s>>>(b_dev, w->n, w->k, layout, static_cast<int32_t *>(w->aux));
        GK_CUDA(c, cudaGetLastError());
    }
    return GLLMK_STATUS_OK;
}

// quantize_from_fp32 / QuantFormat::Int8PerTensor (src/compiler/quant_convert.rs:17-20,165-177): scale = max|x| / 127,
// q = (x / scale).round().clamp(-128, 127) as i8 (round half away from zero; NaN, i.e. 0 / 0 for an all-zero tensor, -> 0).
__global__ void __launch_bounds__(256) act_amax_kernel(const float *__restrict__ x, int64_t rows, int64_t k, int64_t ld, uint32_t *amax_bits) {
    float a = 0.0f;
    const int64_t total = rows * k;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const float v = fabsf(x[(i / k) * ld + i % k]);
        if (v > a) a = v;  // f32::max semantics: a NaN operand is ignored
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    if ((threadIdx.x & 31) == 0) atomicMax(amax_bits, __float_as_uint(a));  // non-negative floats order like their bits
}
__global__ void __launch_bounds__(256) act_quant_i8_kernel(const float *__restrict__ x, int64_t rows, int64_t k, int64_t ld, uint8_t *__restrict__ q,
                                                           int64_t ldq, int offset, const uint32_t *amax_bits, float *scale_out) {
    const float scale = __fdiv_rn(__uint_as_float(*amax_bits), 127.0f);
    const int64_t total = rows * k;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / k, cidx = i % k;
        float v = roundf(__fdiv_rn(x[r * ld + cidx], scale));
        if (v != v) v = 0.0f;
        v = fminf(fmaxf(v, -128.0f), 127.0f);
        q[r * ldq + cidx] = (uint8_t)((int)v + offset);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
}

int32_t act_quant_i8_launch(Ctx *c, const float *x, int64_t rows, int64_t k, int64_t ld, uint8_t *q, int64_t ldq, int offset,
                            float *scale_dev, cudaStream_t s) {
    // the running maximum lives next to the caller's scale word: [scale f32][amax bits u32]
    uint32_t *amax = reinterpret_cast<uint32_t *>(scale_dev) + 1;
    GK_CUDA(c, cudaMemsetAsync(amax, 0, sizeof(uint32_t), s));
    const int64_t total = rows * k;
    const unsigned grid = (unsigned)((total + 1023) / 1024 > 1184 ? 1184 : (total + 1023) / 1024);
    act_amax_kernel<<<grid, 256, 0, s>>>(x, rows, k, ld, amax);
    act_quant_i8_kernel<<<grid, 256, 0, s>>>(x, rows, k, ld, q, ldq, offset, amax, scale_dev);
    GK_CUDA(c, cudaGetLastError());
    return GLLMK_STATUS_OK;
}

template <int MT>
static int32_t i8_launch_mt(Ctx *c, const I8Params &p, dim3 grid, int ntok, cudaStream_t s) {
    static bool attr_set[64] = {};  // function attributes are per device
    const int dev_slot = c->device & 63;
    if (!attr_set[dev_slot]) {
        GK_CUDA(c, cudaFuncSetAttribute(gemm_i8_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)i8_smem<MT>()));
        attr_set[dev_slot] = true;
    }
    gemm_i8_kernel<MT><<<grid, I8_THREADS, i8_smem<MT>(), s>>>(p, ntok);
    GK_CUDA(c, cudaGetLastError());
    return GLLMK_STATUS_OK;
}

int32_t gemm_i8_launch(Ctx *c, const Weight *w, const uint8_t *a, int64_t lda, int m, int32_t *out, int64_t ldc, cudaStream_t s) {
    const int ntok = m > 128 ? I8_BN : (m + 31) / 32 * 32;
    const int mtiles = (m + I8_BN - 1) / I8_BN;
    const int atiles = ntok > 128 ? 2 * mtiles : 1;
    I8Params p{};
    p.w = static_cast<const uint8_t *>(w->qs);
    p.n = w->n;
    p.row_tiles = (int)(w->n_pad / I8_BM);
    p.nks = (int)(w->k_pad / 128);
    p.m = m;
    p.c = out;
    p.ldc = ldc;
    p.vec = (((uintptr_t)out & 15) == 0 && (ldc * 4) % 16 == 0) ? 1 : 0;
    p.status = c->status_dev;
    int32_t rc = ensure_act(c, (size_t)atiles * p.nks * I8_TILE);
    if (rc) return rc;
    p.xt = static_cast<const uint8_t *>(c->act);
    stage_act_u8_kernel<<<dim3((unsigned)p.nks, (unsigned)atiles), 256, 0, s>>>(a, lda, m, w->k, static_cast<uint8_t *>(c->act));
    GK_CUDA(c, cudaGetLastError());
    // two row tiles per CTA when the estimated time (waves x (k-steps per CTA x relative step cost + a fixed
    // prologue / epilogue worth ~8 steps)) is lower
    const auto waves = [&](int ctas) { return (double)((ctas + c->sm_count - 1) / c->sm_count); };
    const int pairs = (p.row_tiles + 1) / 2;
    const double t1 = waves(mtiles * p.row_tiles) * (p.nks + 8.0), t2 = waves(mtiles * pairs) * (2.0 * p.nks * 0.75 + 8.0);
    if (ntok > 128 && t2 < t1) return i8_launch_mt<2>(c, p, dim3((unsigned)pairs, (unsigned)mtiles), ntok, s);
    return i8_launch_mt<1>(c, p, dim3((unsigned)p.row_tiles, (unsigned)mtiles), ntok, s);
}

int32_t dequant_i32_launch(Ctx *c, const int32_t *ci, float *out, int64_t m, int64_t n, int64_t ldc, int64_t ldo, float scale_a,
                           float scale_b, const float *bias, int act, cudaStream_t s, const float *scale_a_dev, const int32_t *colsum) {
    const size_t total = (size_t)m * (size_t)n;
    if (total == 0) return GLLMK_STATUS_OK;
    dequant_i32_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(ci, out, n, ldc, ldo, scale_a, scale_b, bias, act, total, scale_a_dev,
                                                                      colsum);
    GK_CUDA(c, cudaGetLastError());
    return GLLMK_STATUS_OK;
}

}  // namespace gllmk
