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

// ---------------------------------------------------------------------------------------------
// m > 128: CTA pairs (tcgen05 cta_group::2, MMA M = 256), persistent, two accumulators.
//
// The kernel above runs at what an SM can take in from L2: 64 KB per k-step for two 128 x 256 tiles.  As a pair, each
// CTA brings in its own 128 weight rows and HALF of the 256-token activation tile (the tensor core reads the other half
// from the partner's shared memory): 32 KB per k-step and tile.  One 256-column accumulator per tile leaves room for a
// second one, so the eight epilogue warps store tile i while the MMA thread fills the accumulator of tile i + 1, and the
// grid is the resident pairs with tiles dealt round robin.  Structure and hand-shakes are those of gemm_fp4_pair_kernel
// (gemm_fp4.cu) without the scale-factor path: the partner's copy thread cannot signal the leader's barrier with a plain
// bulk copy, so a relay thread forwards "my stage has landed"; stages go back to both CTAs with one commit per barrier.
// ---------------------------------------------------------------------------------------------
constexpr int I8P_STAGES = 6, I8P_STAGE_BYTES = 2 * I8_TILE, I8P_EPI_WARPS = 8;
constexpr int I8P_THREADS = 64 + 32 * I8P_EPI_WARPS;
constexpr size_t I8P_SMEM = (size_t)I8P_STAGES * I8P_STAGE_BYTES + (size_t)I8P_EPI_WARPS * 4096 + 1024;

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(I8P_THREADS, 1)
gemm_i8_pair_kernel(const __grid_constant__ I8Params p, const int tok_tiles, const int x_tiles) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[3 * I8P_STAGES + 4];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    const uint32_t smem_s = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t full = tc::smem_u32(&bars[0]), empty = tc::smem_u32(&bars[I8P_STAGES]), full2 = tc::smem_u32(&bars[2 * I8P_STAGES]);
    const uint32_t accum_full = tc::smem_u32(&bars[3 * I8P_STAGES]), accum_empty = accum_full + 16;  // two each
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = tc::cluster_ctarank();
    const int pair = (int)(blockIdx.x >> 1), npairs = (int)(gridDim.x >> 1);
    const int row_pairs = (p.row_tiles + 1) >> 1;
    const int ntiles = row_pairs * tok_tiles;
    volatile int *abort_flag = &abort_s;

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < I8P_STAGES; s++) {
            tc::mbar_init(full + 8 * s, 1);
            tc::mbar_init(empty + 8 * s, 1);
            tc::mbar_init(full2 + 8 * s, 1);
        }
        for (int a = 0; a < 2; a++) {
            tc::mbar_init(accum_full + 8 * a, 1);
            tc::mbar_init(accum_empty + 8 * a, 2 * I8P_EPI_WARPS);  // the epilogue warps of both CTAs (used in the leader only)
        }
        tc::mbar_init_fence();
    }
    if (warp == 1) tc::tmem_alloc_pair(tc::smem_u32(&tmem_base_s), 512);
    tc::fence_before_sync();
    __syncthreads();
    tc::cluster_arrive();  // both CTAs' barriers exist before either CTA arrives on the other's
    tc::cluster_wait();
    tc::fence_after_sync();
    const uint32_t tmem = tmem_base_s;

    if (warp == 0 && lane == 0) {
        // ---------------- copies: own weight rows, own half of the activation tile ----------------
        uint32_t g = 0;
        for (int t = pair; t < ntiles && !*abort_flag; t += npairs) {
            const int rp = t / tok_tiles, tt = t % tok_tiles;
            const int my_row_tile = 2 * rp + (int)rank, my_x_tile = 2 * tt + (int)rank;
            const bool a_ok = my_row_tile < p.row_tiles, b_ok = my_x_tile < x_tiles;
            // rows / tokens that do not exist are not copied: what the stage holds there only reaches accumulator rows /
            // columns that are never stored
            const uint32_t tx = (a_ok ? (uint32_t)I8_TILE : 0u) + (b_ok ? (uint32_t)I8_TILE : 0u);
            for (int ks = 0; ks < p.nks; ks++, g++) {
                const uint32_t s = g % I8P_STAGES;
                if (g >= (uint32_t)I8P_STAGES && !tc::mbar_wait_cluster(empty + 8 * s, (g / I8P_STAGES - 1) & 1u, abort_flag)) {
                    abort_s = 1;
                    atomicExch(p.status, 44);
                    break;
                }
                const uint32_t st = smem_s + s * I8P_STAGE_BYTES;
                tc::mbar_expect_tx(full + 8 * s, tx);
                if (a_ok) i8_bulk(st, p.w + ((size_t)my_row_tile * p.nks + ks) * I8_TILE, I8_TILE, full + 8 * s);
                if (b_ok) i8_bulk(st + I8_TILE, p.xt + ((size_t)my_x_tile * p.nks + ks) * I8_TILE, I8_TILE, full + 8 * s);
            }
        }
    } else if (warp == 1 && lane == 0 && rank != 0) {
        // ---------------- partner CTA: tell the leader when this CTA's stage has landed ----------------
        uint32_t g = 0;
        bool ok = true;
        for (int t = pair; t < ntiles && ok && !*abort_flag; t += npairs)
            for (int ks = 0; ks < p.nks; ks++, g++) {
                const uint32_t s = g % I8P_STAGES;
                if (!tc::mbar_wait(full + 8 * s, (g / I8P_STAGES) & 1u, abort_flag)) {
                    abort_s = 1;
                    atomicExch(p.status, 45);
                    ok = false;
                    break;
                }
                // the stage's bytes are in place before this arrive is issued (the barrier phase was observed)
                tc::mbar_arrive_cluster_relaxed(tc::map_to_cta(full2 + 8 * s, 0));
            }
    } else if (warp == 1 && lane == 0) {
        // ---------------- leader CTA: MMA issue for the pair, accumulator (tile & 1) ----------------
        const uint32_t idesc = tc::idesc_i8(256, I8_BN, 1, 0);  // weights signed (operand A), activations unsigned (operand B)
        uint32_t g = 0, it = 0;
        for (int t = pair; t < ntiles && !*abort_flag; t += npairs, it++) {
            const uint32_t acc = it & 1u;
            // the tile before last used this accumulator: all sixteen epilogue warps of the pair have read it out
            if (it >= 2 && !tc::mbar_wait_cluster(accum_empty + 8 * acc, ((it >> 1) - 1) & 1u, abort_flag)) {
                abort_s = 1;
                atomicExch(p.status, 46);
                break;
            }
            tc::fence_after_sync();
            const uint32_t td = tmem + 256u * acc;
            bool ok = true;
            for (int ks = 0; ks < p.nks; ks++, g++) {
                const uint32_t s = g % I8P_STAGES, ph = (g / I8P_STAGES) & 1u;
                if (!tc::mbar_wait(full + 8 * s, ph, abort_flag) || !tc::mbar_wait_cluster(full2 + 8 * s, ph, abort_flag)) {
                    abort_s = 1;
                    atomicExch(p.status, 42);
                    ok = false;
                    break;
                }
                tc::fence_after_sync();
                const uint32_t st = smem_s + s * I8P_STAGE_BYTES;
                const uint64_t ad = tc::smem_desc_sw128(st), bd = tc::smem_desc_sw128(st + I8_TILE);
#pragma unroll
                for (int j = 0; j < 4; j++) tc::mma_i8_pair(td, ad + 2 * j, bd + 2 * j, idesc, (uint32_t)((ks | j) != 0));
                // once these MMAs have completed, stage s is free in BOTH CTAs
                tc::mma_commit_pair(empty + 8 * s);
                tc::mma_commit_pair(tc::map_to_cta(empty + 8 * s, 1));
            }
            if (!ok) break;
            tc::mma_commit_pair(accum_full + 8 * acc);
            tc::mma_commit_pair(tc::map_to_cta(accum_full + 8 * acc, 1));
        }
    }
    __syncwarp();

    if (warp >= 2) {
        // ---------------- epilogue: this CTA's 128 rows x 256 tokens of accumulator (tile & 1) ----------------
        // warp w reads TMEM lane quadrant w % 4; the two warps of a quadrant take 128 token columns each
        const int quad = warp & 3, half = (warp - 2) >> 2;
        uint8_t *stage = smem_raw + (smem_s - tc::smem_u32(smem_raw)) + (size_t)I8P_STAGES * I8P_STAGE_BYTES + (size_t)(warp - 2) * 4096;
        const uint32_t accum_empty_leader = tc::map_to_cta(accum_empty, 0);
        uint32_t it = 0;
        for (int t = pair; t < ntiles; t += npairs, it++) {
            const uint32_t acc = it & 1u;
            bool ok = !abort_s && tc::mbar_wait_cluster(accum_full + 8 * acc, (it >> 1) & 1u, abort_flag);
            if (!ok && !abort_s) {
                abort_s = 1;
                atomicExch(p.status, 43);
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc::fence_after_sync();
            const int rp = t / tok_tiles, tt = t % tok_tiles;
            const int64_t row0 = (int64_t)(2 * rp + (int)rank) * I8_BM + 32 * quad, tok0 = (int64_t)tt * I8_BN + 128 * half;
            const uint32_t tbase = tmem + ((uint32_t)(32 * quad) << 16) + 256u * acc + (uint32_t)(128 * half);
#pragma unroll 1
            for (int c = 0; c < 128; c += 32) {
                uint32_t v[32];
                tc::tmem_ld32(tbase + (uint32_t)c, v);
                tc::tmem_ld_wait();
                if (row0 < p.n && tok0 + c < p.m) {
                    float o[32];  // the s32 bit patterns travel through the 32-bit store helper unchanged
#pragma unroll
                    for (int j = 0; j < 32; j++) o[j] = __uint_as_float(v[j]);
                    tc::store_block_32x32<false>(p.c, p.ldc, row0, tok0 + c, p.n, p.m, o, stage, lane, p.vec);
                }
            }
            // this warp's reads of the accumulator are complete (wait::ld): the leader may reuse it for the tile after next
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive_cluster_relaxed(accum_empty_leader + 8 * acc);
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    // neither CTA may leave (or give TMEM back) while the pair's MMAs can still read its shared memory
    tc::cluster_arrive();
    tc::cluster_wait();
    if (warp == 1) tc::tmem_dealloc_pair(tmem, 512);
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
    // estimated times in k-steps of a 128 x 256 tile (waves x (k-steps per CTA x relative step cost + a fixed prologue /
    // epilogue worth ~8 steps)): one row tile per CTA, two row tiles per CTA (a third fewer bytes per MAC), CTA pairs
    // (half the bytes per MAC of one tile per CTA; measured 0.82 of the two-tile form on W[11008, 4096] x 2048, 1.06 x 512)
    const auto waves = [&](int ctas) { return (double)((ctas + c->sm_count - 1) / c->sm_count); };
    const int pairs = (p.row_tiles + 1) / 2;
    const double t1 = waves(mtiles * p.row_tiles) * (p.nks + 8.0), t2 = waves(mtiles * pairs) * (2.0 * p.nks * 0.75 + 8.0);
    const int half_sms = c->sm_count / 2 > 0 ? c->sm_count / 2 : 1;
    const double tp = (double)((mtiles * pairs + half_sms - 1) / half_sms) * (p.nks * 0.6 + 8.0);
    if (m > 128 && (c->gemm_i8_pair == 2 || (c->gemm_i8_pair == 1 && tp < 0.9 * (t1 < t2 ? t1 : t2)))) {
        const void *fn = (const void *)gemm_i8_pair_kernel;
        static int pairs_resident[64] = {};  // per device: CTA pairs resident at once (0 = not yet asked)
        const int dev_slot = c->device & 63;
        if (!pairs_resident[dev_slot]) {
            GK_CUDA(c, cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)I8P_SMEM));
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)c->sm_count & ~1u);
            cfg.blockDim = dim3((unsigned)I8P_THREADS);
            cfg.dynamicSmemBytes = I8P_SMEM;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = 2;
            at[0].val.clusterDim.y = 1;
            at[0].val.clusterDim.z = 1;
            cfg.attrs = at;
            cfg.numAttrs = 1;
            int nclusters = 0;
            if (cudaOccupancyMaxActiveClusters(&nclusters, fn, &cfg) != cudaSuccess || nclusters < 1) {
                (void)cudaGetLastError();
                nclusters = c->sm_count / 2;
            }
            pairs_resident[dev_slot] = nclusters < c->sm_count / 2 ? nclusters : c->sm_count / 2;
        }
        const int ntiles = ((p.row_tiles + 1) / 2) * mtiles;
        const int npairs = ntiles < pairs_resident[dev_slot] ? ntiles : pairs_resident[dev_slot];
        gemm_i8_pair_kernel<<<dim3(2u * (unsigned)npairs), I8P_THREADS, I8P_SMEM, s>>>(p, mtiles, atiles);
        GK_CUDA(c, cudaGetLastError());
        return GLLMK_STATUS_OK;
    }
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
