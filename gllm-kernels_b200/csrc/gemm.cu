// Prefill path: fused dequantize + GEMM on tcgen05 tensor cores with the accumulator in TMEM.
//
//   Y[t, r] = sum_k W[r, k] * X[t, k]        t < M tokens (M > 16), r < N weight rows
//
// Weight-only formats (Q4_K, Q8_0, MXFP4, NVFP4 weights with bf16/f32 activations), gemm_wq_kernel.
// A CTA owns MT (1 or 2) tiles of 128 weight rows (UMMA M, one TMEM accumulator each) x up to 256 tokens
// (UMMA N) and walks K in steps of 64 (64 fp16 = one 128-byte swizzle row).  With MT = 2 one activation tile
// feeds two MMAs, which halves the shared-memory fill traffic per flop (the L2 -> SM path, not the tensor
// core, is what bounds a 128 x 256 tile):
//   * the RAW quantized weights of its 128 rows arrive as one bulk copy per 256 k ("super-chunk": the same
//     contiguous byte range the decode GEMV streams) into a shared-memory ring, mbarrier-tracked;
//   * four dequant warps turn a quarter of a super-chunk (64 k) into fp16 with packed half2 arithmetic and
//     store it as the 128-byte-swizzled K-major operand A tile the tensor core reads;
//   * the activations were converted once per call to fp16 tile images (stage_act_kernel), so operand B
//     of a k-step is one or two bulk copies of 16 KB;
//   * one elected thread issues tcgen05.mma (kind::f16, f32 accumulate in TMEM); tcgen05.commit hands the
//     A and B stages back; after the last k-step the dequant warps read the accumulator (tcgen05.ld:
//     lane = weight row, so the warp-wide stores are coalesced in Y's row-major layout).
// kind::f16 takes one 16-bit format for both operands (mixing f16 and bf16 is an illegal instruction), so
// weights and activations are both staged in fp16: 11 significant bits, accumulate f32 (parity bar 1e-2).
// No cluster-multicast load is used anywhere (the same kernel serves the multi-GPU configuration).
#include <cuda_bf16.h>

#include "common.cuh"
#include "tc05.cuh"

namespace gllmk {

constexpr int WQ_BM = 128;         // weight rows per CTA (UMMA M)
constexpr int WQ_BN = 256;         // tokens per CTA (UMMA N, <= 256)
constexpr int WQ_TILE = 16384;     // one operand tile: 128 rows x 128 bytes
constexpr int WQ_SA = 4;           // operand A (dequantized weight tiles) ring: one slot per dequant group
constexpr int WQ_MAX_SB = 12;      // operand B (activation) stages, at most
constexpr int WQ_MAX_R = 8;        // raw super-chunk ring, at most
constexpr int WQ_DW = 16;          // dequant warps
constexpr int WQ_CTRL = 4;         // warp 0: raw copies, warp 1: activation copies, warps 2 and 3: MMA issue (row tile 0 / row tile 1), warp 2: TMEM
constexpr int WQ_THREADS = 32 * (WQ_CTRL + WQ_DW);  // then the dequant / epilogue warps
constexpr int WQ_SMEM_LIMIT = 232448 - 1024 - 1024;  // ring space: 227 KB less the static variables' share and the alignment slack

enum { FMT_Q4K = 0, FMT_Q80 = 1, FMT_NVFP4 = 2, FMT_MXFP4 = 3, FMT_Q6K = 4, FMT_Q5K = 5, FMT_Q40 = 6, FMT_Q50 = 7 };
// Q6_K and Q5_K stay on the device as the reference stores them, row after row of blocks (these kernels' other formats
// are repacked into tile images): a raw super-chunk is then one block of each of a tile's 128 rows.
constexpr int Q6K_SLOT = 224;        // a Q6_K block (210 bytes) on the device: reference layout in a 16-byte aligned slot
constexpr int Q6K_ROW_STRIDE = 240;  // and in shared memory, so that eight rows' 16-byte words fall on different banks
constexpr int Q5K_SLOT = 176;        // a Q5_K block: 11 x 16 bytes, an odd count, so its own size is a conflict-free stride
constexpr int Q40_SLOT = 144;        // eight Q4_0 blocks (18 bytes, 32 elements each) = 256 elements of a row whose k is a multiple of 256
constexpr int Q50_SLOT = 176;        // eight Q5_0 blocks (22 bytes)
constexpr bool wq_row_major(int fmt) { return fmt >= FMT_Q6K; }
constexpr int wq_slot(int fmt) { return fmt == FMT_Q6K ? Q6K_SLOT : (fmt == FMT_Q40 ? Q40_SLOT : (fmt == FMT_Q5K ? Q5K_SLOT : Q50_SLOT)); }
constexpr int wq_row_stride(int fmt) { return fmt == FMT_Q6K ? Q6K_ROW_STRIDE : wq_slot(fmt); }
__host__ __device__ constexpr int wq_raw_bytes(int fmt) {
    return fmt == FMT_Q4K ? 8 * Q4K_CHUNK : (fmt == FMT_Q80 ? 8 * Q80_CHUNK : (fmt == FMT_NVFP4 ? WQ_TILE + 2048 : (fmt == FMT_MXFP4 ? WQ_TILE + 1024 : 128 * wq_row_stride(fmt))));
}

constexpr int WQ_MAX_GROUPS = 32;      // weights (experts) per launch
constexpr int WQ_MAX_TOK_TILES = 64;   // token tiles per launch
constexpr int WQ_MAX_IMG_TILES = 128;  // 128-row activation images per launch

// One launch serves up to WQ_MAX_GROUPS weights of the same shape and format, each with its own rows of the
// activation matrix (a mixture-of-experts layer; a plain GEMM is one group).  blockIdx.x walks the token tiles.
struct GemmGroups {
    const uint8_t *qs[WQ_MAX_GROUPS];   // weight plane (format-specific, see common.cuh)
    const uint8_t *aux[WQ_MAX_GROUPS];  // FP4 scale-factor plane
    float gs[WQ_MAX_GROUPS];            // NVFP4 per-tensor scale
    int tile_group[WQ_MAX_TOK_TILES];   // which weight
    int tile_tok0[WQ_MAX_TOK_TILES];    // first row of a / y
    int tile_cnt[WQ_MAX_TOK_TILES];     // rows (<= ntok)
    int tile_img[WQ_MAX_TOK_TILES];     // first activation image of the tile
};
struct ImgTiles {
    int tok0[WQ_MAX_IMG_TILES];  // first row of a in the image
    int cnt[WQ_MAX_IMG_TILES];   // rows present (the rest of the 128 are zero)
};

struct GemmParams {
    int64_t n;
    int nsc;             // super-chunks (256 k) per row
    const uint8_t *xt;   // fp16 activation tile images [image][k-step of 64][16384]
    void *y;             // [tokens, n] row-major, leading dimension ldy
    int y_bf16;
    int64_t ldy;
    int vec;             // Y allows 16-byte stores
    int ntok;            // MMA N of this launch (multiple of 32, <= 256)
    int row_tiles;       // 128-row tiles of the weight matrix
    int sb, r;           // ring depths: B stages, raw super-chunks
    int *status;
    // Tail split (split_s > 1; the grid is then one-dimensional): units [0, split_f) are whole tiles, in the order
    // tile = token tile + ntt * row group; every later tile is cut along k into split_s units whose f32 partial
    // accumulators meet in `partial`, added up in unit order by whichever unit of the tile finishes last.
    int split_f, split_s, ntt;
    float *partial;      // [tail tile][split][row tile of the CTA][token][128 rows]
    int *tail_cnt;       // [tail tile] arrivals, zero between launches
};

// ---- activations -> fp16 tile images ------------------------------------------------------------
// grid (k-steps, images of 128 rows); rows past an image's count and k >= k_valid are zero
// a_up != nullptr: the activation is silu(a) * a_up (SwiGLU of the two halves of a gate || up product, same dtype and
// leading dimension), evaluated in f32 as scalar_swiglu does (scalar-ops/src/activations.rs:57-66) before the fp16 rounding
__device__ __forceinline__ float swiglu_f32(float g, float u) { return (g / (1.0f + expf(-g))) * u; }
__global__ void __launch_bounds__(256) stage_act_kernel(const void *__restrict__ a, int a_bf16, int64_t lda, int64_t k_valid,
                                                        uint8_t *__restrict__ xt, const __grid_constant__ ImgTiles imgs,
                                                        const void *__restrict__ a_up) {
    // The GEMM behind this launch may start now (programmatic dependent launch): its CTAs take the SMs this grid leaves,
    // allocate tensor memory and stream raw weights; the one thread that reads these tile images orders itself after
    // this grid with griddepcontrol.wait.
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const int ks = blockIdx.x, tile = blockIdx.y;
    const int64_t img_tok0 = imgs.tok0[tile];
    const int img_cnt = imgs.cnt[tile];
    uint8_t *dst = xt + ((size_t)tile * gridDim.x + ks) * WQ_TILE;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int item = threadIdx.x + 256 * i, row = item >> 3, chunk = item & 7;
        const int64_t tok = img_tok0 + row, k0 = (int64_t)ks * 64 + chunk * 8;
        uint4 o = make_uint4(0, 0, 0, 0);
        if (row < img_cnt && k0 < k_valid) {
            if (a_bf16) {
                // bf16 -> fp16 through f32, saturating at +-65504
                const uint4 v = __ldg(reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(a) + tok * lda + k0));
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
                uint32_t r[4];
                if (a_up) {
                    const uint4 vu = __ldg(reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(a_up) + tok * lda + k0));
                    const uint32_t wu[4] = {vu.x, vu.y, vu.z, vu.w};
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const float lo = swiglu_f32(__uint_as_float(w[q] << 16), __uint_as_float(wu[q] << 16));
                        const float hi = swiglu_f32(__uint_as_float(w[q] & 0xFFFF0000u), __uint_as_float(wu[q] & 0xFFFF0000u));
                        asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;\n" : "=r"(r[q]) : "f"(hi), "f"(lo));
                    }
                } else {
#pragma unroll
                    for (int q = 0; q < 4; q++)
                        asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;\n" : "=r"(r[q]) : "f"(__uint_as_float(w[q] & 0xFFFF0000u)), "f"(__uint_as_float(w[q] << 16)));
                }
                o = make_uint4(r[0], r[1], r[2], r[3]);
            } else {
                const float4 *src = reinterpret_cast<const float4 *>(static_cast<const float *>(a) + tok * lda + k0);
                float4 x0 = __ldg(src), x1 = __ldg(src + 1);
                if (a_up) {
                    const float4 *su = reinterpret_cast<const float4 *>(static_cast<const float *>(a_up) + tok * lda + k0);
                    const float4 u0 = __ldg(su), u1 = __ldg(su + 1);
                    x0 = make_float4(swiglu_f32(x0.x, u0.x), swiglu_f32(x0.y, u0.y), swiglu_f32(x0.z, u0.z), swiglu_f32(x0.w, u0.w));
                    x1 = make_float4(swiglu_f32(x1.x, u1.x), swiglu_f32(x1.y, u1.y), swiglu_f32(x1.z, u1.z), swiglu_f32(x1.w, u1.w));
                }
                uint32_t r[4];
                asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;\n" : "=r"(r[0]) : "f"(x0.y), "f"(x0.x));
                asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;\n" : "=r"(r[1]) : "f"(x0.w), "f"(x0.z));
                asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;\n" : "=r"(r[2]) : "f"(x1.y), "f"(x1.x));
                asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;\n" : "=r"(r[3]) : "f"(x1.w), "f"(x1.z));
                o = make_uint4(r[0], r[1], r[2], r[3]);
            }
        }
        *reinterpret_cast<uint4 *>(dst + tc::sw128_offset(row, chunk)) = o;
    }
}

// ---- packed dequant arithmetic --------------------------------------------------------------------
__device__ __forceinline__ __half2 u32_as_h2(uint32_t v) { return *reinterpret_cast<__half2 *>(&v); }
__device__ __forceinline__ uint32_t h2_as_u32(__half2 v) { return *reinterpret_cast<uint32_t *>(&v); }
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}

// Four unsigned bytes (each < 256) -> their values as two half2, exactly: the byte becomes the low mantissa
// bits of 1024.0 (0x6400) and 1024 is subtracted again.
__device__ __forceinline__ void bytes_to_h2(uint32_t b, float bias, __half2 &lo, __half2 &hi) {
    const __half2 off = __float2half2_rn(bias);
    lo = __hsub2(u32_as_h2(__byte_perm(b, 0x64646464u, 0x5140)), off);
    hi = __hsub2(u32_as_h2(__byte_perm(b, 0x64646464u, 0x5342)), off);
}
// Q4_K: one 32-bit word = 4 low-nibble elements (sub-block 2p) and 4 high-nibble elements (sub-block 2p+1);
// e = (d*sc, -dmin*m) of the sub-block: value = q * d*sc - dmin*m, one fp16 rounding after the product
__device__ __forceinline__ void q4k_word(uint32_t w, __half2 e_lo, __half2 e_hi, uint32_t &lo01, uint32_t &lo23, uint32_t &hi01,
                                         uint32_t &hi23) {
    __half2 a, b;
    bytes_to_h2(w & 0x0F0F0F0Fu, 1024.0f, a, b);
    lo01 = h2_as_u32(__hfma2(a, __low2half2(e_lo), __high2half2(e_lo)));
    lo23 = h2_as_u32(__hfma2(b, __low2half2(e_lo), __high2half2(e_lo)));
    bytes_to_h2((w >> 4) & 0x0F0F0F0Fu, 1024.0f, a, b);
    hi01 = h2_as_u32(__hfma2(a, __low2half2(e_hi), __high2half2(e_hi)));
    hi23 = h2_as_u32(__hfma2(b, __low2half2(e_hi), __high2half2(e_hi)));
}
// Q8_0: four int8 of one word times the block scale
__device__ __forceinline__ void q80_word(uint32_t w, __half2 d2, uint32_t &o01, uint32_t &o23) {
    __half2 a, b;
    bytes_to_h2(w ^ 0x80808080u, 1152.0f, a, b);  // (q + 128) + 1024 - 1152 = q
    o01 = h2_as_u32(__hmul2(a, d2));
    o23 = h2_as_u32(__hmul2(b, d2));
}
// FP4: eight E2M1 codes of one word -> fp16 (hardware conversion, exact), times the scale
__device__ __forceinline__ uint4 fp4_word(uint32_t w, __half2 s2) {
    uint32_t o0, o1, o2, o3;
    asm("{\n.reg .b8 a, b, c, d;\nmov.b32 {a, b, c, d}, %4;\n"
        "cvt.rn.f16x2.e2m1x2 %0, a;\ncvt.rn.f16x2.e2m1x2 %1, b;\ncvt.rn.f16x2.e2m1x2 %2, c;\ncvt.rn.f16x2.e2m1x2 %3, d;\n}\n"
        : "=r"(o0), "=r"(o1), "=r"(o2), "=r"(o3)
        : "r"(w));
    return make_uint4(h2_as_u32(__hmul2(u32_as_h2(o0), s2)), h2_as_u32(__hmul2(u32_as_h2(o1), s2)),
                      h2_as_u32(__hmul2(u32_as_h2(o2), s2)), h2_as_u32(__hmul2(u32_as_h2(o3), s2)));
}
__device__ __forceinline__ __half2 scale_h2(float s) {
    uint32_t r;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %1;\n" : "=r"(r) : "f"(s));
    return u32_as_h2(r);
}

// ---- dequant of one k-step (64 k) of a 128-row weight tile into an operand A tile --------------------
// The sixteen dequant warps form four groups of four; a group turns out a whole A tile (128 rows x 64 k) on
// its own and the groups work on four consecutive tiles at once, so the latency of one tile's chain (wait,
// shared-memory loads, shuffles, half2 arithmetic, stores, proxy fence, arrive) is overlapped four ways.
// wg = warp inside the group (0..3), lane = 4*g + t.  `raw` is the super-chunk in shared memory, p = k-step
// inside it (0..3), `at` the A tile.
//
// Q4_K / Q8_0: warp wg handles the 16-row chunks wg and wg + 4; its lane reads the uint4 the device layout
// keeps for it (rows g and g + 8, bytes 8t..8t+7 of the 32-byte group) and produces, for both rows, the
// 16-byte fp16 groups t (low nibbles / even block) and 4 + t (high nibbles / odd block).
// Which of a chunk's row pairs (g, g + 8) a lane works on.  With g = lane / 4 the eight lanes that a 16-byte shared-memory
// access handles together (lanes 8i .. 8i+7) would write rows g and g + 1 of the swizzled A tile, whose four 16-byte
// groups (t ^ g) fall on the same four bank groups: a two-way conflict on every store.  Pairing rows q and q ^ 5 in such
// an octet puts its eight stores on eight different bank groups and keeps its eight loads of the raw chunk (16-byte
// slots 4g + t) on eight different ones as well.
__device__ __forceinline__ int wq_row_of_lane(int lane) {
    const int q = lane >> 3;
    return (lane & 4) ? (q ^ 5) : q;
}

// Q4_K / Q8_0: the eight 16-byte groups a lane has made (o[4 * ci + 2 * h + {0, 1}] = groups t and 4 + t of row
// 16 * (wg + 4 * ci) + 8 * h + g) go to the swizzled A tile
__device__ __forceinline__ void store_kq(uint8_t *at, int wg, int lane, const uint4 (&o)[8]) {
    const int g = wq_row_of_lane(lane), t = lane & 3;
#pragma unroll
    for (int ci = 0; ci < 2; ci++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            uint8_t *rowp = at + (16 * (wg + 4 * ci) + 8 * h + g) * 128;  // (row & 7) == g
            *reinterpret_cast<uint4 *>(rowp + ((t ^ g) << 4)) = o[4 * ci + 2 * h];
            *reinterpret_cast<uint4 *>(rowp + (((4 + t) ^ g) << 4)) = o[4 * ci + 2 * h + 1];
        }
}

template <int FMT>
struct Dequant;

template <>
struct Dequant<FMT_Q4K> {
    float global;
    __device__ __forceinline__ void compute(const uint8_t *raw, int p, int wg, int lane, uint4 (&o)[8]) {
        const int g = wq_row_of_lane(lane), t = lane & 3, vl = 4 * g + t;
        // (d*sc, -dmin*m) of sub-blocks 2p and 2p+1: lane t works them out for (chunk, row) pair t of the four
        // pairs its quad shares; everyone fetches all four pairs with shuffles
        __half2 mine_lo, mine_hi;
        {
            const uint8_t *chunk = raw + (wg + 4 * (t >> 1)) * Q4K_CHUNK;
            const int h = t & 1, rr = g + 8 * h;
            const uint32_t dd = *reinterpret_cast<const uint32_t *>(chunk + 2304 + (g * 2 + h) * 4);
            const float d = __half2float(__ushort_as_half((unsigned short)(dd & 0xFFFFu)));
            const float dmin = __half2float(__ushort_as_half((unsigned short)(dd >> 16)));
            const uint32_t sc = *reinterpret_cast<const unsigned short *>(chunk + 2048 + rr * 16 + 2 * p);
            const uint32_t mn = *reinterpret_cast<const unsigned short *>(chunk + 2048 + rr * 16 + 8 + 2 * p);
            mine_lo = __floats2half2_rn(d * (float)(sc & 0xFFu), -(dmin * (float)(mn & 0xFFu)));
            mine_hi = __floats2half2_rn(d * (float)(sc >> 8), -(dmin * (float)(mn >> 8)));
        }
#pragma unroll
        for (int ci = 0; ci < 2; ci++) {
            const int c = wg + 4 * ci;
            const uint4 q = *reinterpret_cast<const uint4 *>(raw + c * Q4K_CHUNK + (p * 32 + vl) * 16);
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int src = (lane & ~3) | (2 * ci + h);
                const __half2 e_lo = u32_as_h2(__shfl_sync(0xffffffffu, h2_as_u32(mine_lo), src));
                const __half2 e_hi = u32_as_h2(__shfl_sync(0xffffffffu, h2_as_u32(mine_hi), src));
                uint4 &lo = o[4 * ci + 2 * h], &hi = o[4 * ci + 2 * h + 1];
                q4k_word(h ? q.z : q.x, e_lo, e_hi, lo.x, lo.y, hi.x, hi.y);
                q4k_word(h ? q.w : q.y, e_lo, e_hi, lo.z, lo.w, hi.z, hi.w);
            }
        }
    }
    __device__ __forceinline__ void store(uint8_t *at, int wg, int lane, const uint4 (&o)[8]) { store_kq(at, wg, lane, o); }
};

template <>
struct Dequant<FMT_Q80> {
    float global;
    __device__ __forceinline__ void compute(const uint8_t *raw, int p, int wg, int lane, uint4 (&o)[8]) {
        const int g = wq_row_of_lane(lane), t = lane & 3, vl = 4 * g + t;
#pragma unroll
        for (int ci = 0; ci < 2; ci++) {
            const int c = wg + 4 * ci;
            const uint8_t *chunk = raw + c * Q80_CHUNK;
            const uint4 q0 = *reinterpret_cast<const uint4 *>(chunk + ((2 * p) * 32 + vl) * 16);
            const uint4 q1 = *reinterpret_cast<const uint4 *>(chunk + ((2 * p + 1) * 32 + vl) * 16);
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int rr = g + 8 * h;
                const __half2 dd = u32_as_h2(*reinterpret_cast<const uint32_t *>(chunk + 4096 + (rr * 8 + 2 * p) * 2));
                uint4 &lo = o[4 * ci + 2 * h], &hi = o[4 * ci + 2 * h + 1];
                q80_word(h ? q0.z : q0.x, __low2half2(dd), lo.x, lo.y);
                q80_word(h ? q0.w : q0.y, __low2half2(dd), lo.z, lo.w);
                q80_word(h ? q1.z : q1.x, __high2half2(dd), hi.x, hi.y);
                q80_word(h ? q1.w : q1.y, __high2half2(dd), hi.z, hi.w);
            }
        }
    }
    __device__ __forceinline__ void store(uint8_t *at, int wg, int lane, const uint4 (&o)[8]) { store_kq(at, wg, lane, o); }
};

// FP4: the raw super-chunk is the row tile's swizzled data image (16 KB) followed by its scale atoms (512 B
// each: [row % 32][row / 32][4 scales]).  Thread = weight row 32 * wg + lane.
template <int FMT>
struct DequantFp4 {
    float global;
    __device__ __forceinline__ void compute(const uint8_t *raw, int p, int wg, int lane, uint4 (&o)[8]) {
        const int r = 32 * wg + lane;
        const uint4 v0 = *reinterpret_cast<const uint4 *>(raw + tc::sw128_offset(r, 2 * p));
        const uint4 v1 = *reinterpret_cast<const uint4 *>(raw + tc::sw128_offset(r, 2 * p + 1));
        const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        __half2 s[4];
        if (FMT == FMT_NVFP4) {
            const uint32_t sf = *reinterpret_cast<const uint32_t *>(raw + WQ_TILE + p * 512 + lane * 16 + wg * 4);
#pragma unroll
            for (int j = 0; j < 4; j++) s[j] = scale_h2(global * e4m3_to_f32((sf >> (8 * j)) & 0xFFu));
        } else {
            const uint32_t sf = *reinterpret_cast<const unsigned short *>(raw + WQ_TILE + (p >> 1) * 512 + lane * 16 + wg * 4 + 2 * (p & 1));
            s[0] = s[1] = scale_h2(e8m0_to_f32(sf & 0xFFu));
            s[2] = s[3] = scale_h2(e8m0_to_f32(sf >> 8));
        }
#pragma unroll
        for (int c = 0; c < 8; c++) o[c] = fp4_word(w[c], s[c >> 1]);
    }
    __device__ __forceinline__ void store(uint8_t *at, int wg, int lane, const uint4 (&o)[8]) {
        const int r = 32 * wg + lane;
        uint8_t *rowp = at + r * 128;
#pragma unroll
        for (int c = 0; c < 8; c++) *reinterpret_cast<uint4 *>(rowp + ((c ^ (r & 7)) << 4)) = o[c];
    }
};
template <>
struct Dequant<FMT_NVFP4> : DequantFp4<FMT_NVFP4> {};
template <>
struct Dequant<FMT_MXFP4> : DequantFp4<FMT_MXFP4> {};

// Q6_K (k_quant.rs:441-472): the raw super-chunk is one reference-layout block (ql[128] @0, qh[64] @128, scales[16] i8 @192,
// d f16 @208) of each of the tile's 128 rows, Q6K_ROW_STRIDE bytes apart.  Thread = weight row 32 * wg + lane.  k-step p of
// the block (64 elements) is half hh = p / 2, runs j0 = 2 (p % 2) and j0 + 1 of that half: run j takes the nibble p % 2 of
// ql[hh * 64 + (j % 2) * 32 + l] and bits 2j, 2j + 1 of qh[hh * 32 + l], l = 0 .. 31; scale sc[hh * 8 + l / 16 + 2 j].
// A word of four 6-bit values becomes the s8 word 4 (q - 32) (bit 5 flipped, two places up), that the fp16 pairs
// 4 (q - 32) exactly (the byte in the mantissa of 1024, as for Q8_0), times d * sc / 4 rounded to fp16.
// 16 bytes global -> shared without passing registers; and "this thread's copies so far" as one arrival at an mbarrier
__device__ __forceinline__ void cp_async16_s(uint32_t dst_smem, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t q6k_word(uint32_t lo4, uint32_t hi2_at_4) {
    return ((((lo4 & 0x0F0F0F0Fu) | (hi2_at_4 & 0x30303030u)) ^ 0x20202020u) << 2) & 0xFCFCFCFCu;
}
template <>
struct Dequant<FMT_Q6K> {
    float global;
    __device__ __forceinline__ void compute(const uint8_t *raw, int p, int wg, int lane, uint4 (&o)[8]) {
        const uint8_t *b = raw + (32 * wg + lane) * Q6K_ROW_STRIDE;
        const int hh = p >> 1, nib = 4 * (p & 1);  // low or high nibbles; qh bits 4 (p % 2) .. + 3
        const uint4 S = *reinterpret_cast<const uint4 *>(b + 192);
        // the four scale bytes this step uses: index hh * 8 + 4 (p % 2) + (half + 2 r), half, r = 0, 1
        const uint32_t sw = (p & 1) ? (hh ? S.w : S.y) : (hh ? S.z : S.x);
        const float d = 0.25f * __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(b + 208)));
#pragma unroll
        for (int half = 0; half < 2; half++) {  // l = 16 half .. 16 half + 15: one 16-byte word of each field
            const uint4 A = *reinterpret_cast<const uint4 *>(b + hh * 64 + 16 * half);        // run j0
            const uint4 B = *reinterpret_cast<const uint4 *>(b + hh * 64 + 32 + 16 * half);   // run j0 + 1
            const uint4 H = *reinterpret_cast<const uint4 *>(b + 128 + hh * 32 + 16 * half);
            const uint32_t aw[4] = {A.x, A.y, A.z, A.w}, bw[4] = {B.x, B.y, B.z, B.w}, hw[4] = {H.x, H.y, H.z, H.w};
#pragma unroll
            for (int r = 0; r < 2; r++) {  // run j0 + r
                const __half2 sc2 = scale_h2(d * (float)(int8_t)((sw >> (8 * (half + 2 * r))) & 0xFF));
#pragma unroll
                for (int c = 0; c < 2; c++) {  // eight elements: words 2c, 2c + 1 of the 16
                    uint32_t q[2];
#pragma unroll
                    for (int i = 0; i < 2; i++) {
                        const uint32_t lo = (r ? bw[2 * c + i] : aw[2 * c + i]) >> nib;
                        const uint32_t hi = nib ? (r ? hw[2 * c + i] >> 2 : hw[2 * c + i]) : (r ? hw[2 * c + i] << 2 : hw[2 * c + i] << 4);
                        q[i] = q6k_word(lo, hi);
                    }
                    uint4 &out = o[4 * r + 2 * half + c];  // k = 32 r + 16 half + 8 c .. + 7 of the step
                    q80_word(q[0], sc2, out.x, out.y);
                    q80_word(q[1], sc2, out.z, out.w);
                }
            }
        }
    }
    __device__ __forceinline__ void store(uint8_t *at, int wg, int lane, const uint4 (&o)[8]) {
        const int r = 32 * wg + lane;
        uint8_t *rowp = at + r * 128;
#pragma unroll
        for (int c = 0; c < 8; c++) *reinterpret_cast<uint4 *>(rowp + ((c ^ (r & 7)) << 4)) = o[c];
    }
};

// Q5_K (k_quant.rs:381-436): d f16 @0, dmin f16 @2, scales[12] @4, qh[32] @16, qs[128] @48.  Thread = weight row.  k-step p
// is the 64-element group p: its first 32 elements are the low nibbles of qs[32 p + l] with bit 2p of qh[l] on top
// (sub-block 2p), the next 32 the high nibbles with bit 2p + 1 (sub-block 2p + 1); value = q * d*sc - dmin*m as for Q4_K.
template <>
struct Dequant<FMT_Q5K> {
    float global;
    __device__ __forceinline__ void compute(const uint8_t *raw, int p, int wg, int lane, uint4 (&o)[8]) {
        const uint8_t *b = raw + (32 * wg + lane) * Q5K_SLOT;
        const uint4 hd = *reinterpret_cast<const uint4 *>(b);  // d, dmin and the twelve scale bytes
        const float d = __half2float(__ushort_as_half((unsigned short)(hd.x & 0xFFFFu)));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(hd.x >> 16)));
        __half2 e[2];  // (d*sc, -dmin*m) of sub-blocks 2p and 2p + 1 (get_scale_min_k4, k_quant.rs:388-397, without a branch)
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int j = 2 * p + i, sh = 8 * (j & 3);
            const uint32_t a = (hd.y >> sh) & 0xFFu, bb = (hd.z >> sh) & 0xFFu, c = (hd.w >> sh) & 0xFFu;
            const uint32_t sc = j < 4 ? (a & 63u) : ((c & 0xFu) | ((a >> 6) << 4)), mn = j < 4 ? (bb & 63u) : ((c >> 4) | ((bb >> 6) << 4));
            e[i] = __floats2half2_rn(d * (float)sc, -(dmin * (float)mn));
        }
#pragma unroll
        for (int half = 0; half < 2; half++) {  // l = 16 half .. 16 half + 15
            const uint4 Q = *reinterpret_cast<const uint4 *>(b + 48 + 32 * p + 16 * half);
            const uint4 H = *reinterpret_cast<const uint4 *>(b + 16 + 16 * half);
            const uint32_t qw[4] = {Q.x, Q.y, Q.z, Q.w}, hw[4] = {H.x, H.y, H.z, H.w};
#pragma unroll
            for (int i = 0; i < 2; i++)      // sub-block 2p + i: nibble i, qh bit 2p + i
#pragma unroll
                for (int c = 0; c < 2; c++) {  // eight elements: words 2c, 2c + 1
                    uint4 &out = o[4 * i + 2 * half + c];  // k = 32 i + 16 half + 8 c .. + 7 of the step
                    uint32_t r[4];
#pragma unroll
                    for (int w = 0; w < 2; w++) {
                        const uint32_t q = ((qw[2 * c + w] >> (4 * i)) & 0x0F0F0F0Fu) | (((hw[2 * c + w] >> (2 * p + i)) & 0x01010101u) << 4);
                        __half2 lo, hi;
                        bytes_to_h2(q, 1024.0f, lo, hi);
                        r[2 * w] = h2_as_u32(__hfma2(lo, __low2half2(e[i]), __high2half2(e[i])));
                        r[2 * w + 1] = h2_as_u32(__hfma2(hi, __low2half2(e[i]), __high2half2(e[i])));
                    }
                    out = make_uint4(r[0], r[1], r[2], r[3]);
                }
        }
    }
    __device__ __forceinline__ void store(uint8_t *at, int wg, int lane, const uint4 (&o)[8]) {
        const int r = 32 * wg + lane;
        uint8_t *rowp = at + r * 128;
#pragma unroll
        for (int c = 0; c < 8; c++) *reinterpret_cast<uint4 *>(rowp + ((c ^ (r & 7)) << 4)) = o[c];
    }
};

// Q4_0 / Q5_0 (classic.rs:15-29, 484-504): blocks of 32 elements, 18 / 22 bytes: d f16, (Q5_0: qh u32 = the fifth bits,)
// qs[16]: byte j holds elements j (low nibble) and j + 16 (high).  Thread = weight row; k-step p is blocks 2p and 2p + 1 of
// the row's eight.  A block starts on a 2-byte boundary only: an even block's fields are read as aligned words from the
// block start and shifted down 16 bits; an odd block's qs (and qh) are word-aligned themselves.
__device__ __forceinline__ uint32_t spread4_bits(uint32_t v) { return ((v & 0xFu) * 0x00204081u) & 0x01010101u; }  // bits 0..3 -> bit 0 of bytes 0..3
template <int FMT>
struct DequantClassic {
    float global;
    static constexpr int BB = FMT == FMT_Q40 ? 18 : 22, QS = FMT == FMT_Q40 ? 2 : 6, BIAS = FMT == FMT_Q40 ? 8 : 16;
    __device__ __forceinline__ void compute(const uint8_t *raw, int p, int wg, int lane, uint4 (&o)[8]) {
        const uint8_t *row = raw + (32 * wg + lane) * wq_slot(FMT);
#pragma unroll
        for (int i = 0; i < 2; i++) {  // block 2p + i; its parity is i
            const uint8_t *b = row + (2 * p + i) * BB;
            uint32_t qs[4], qh = 0, dbits;
            if (i == 0) {  // block start word-aligned: words from the start, fields 16 bits further on
                const uint32_t *w = reinterpret_cast<const uint32_t *>(b);
                constexpr int NW = (BB + 2 + 3) / 4;
                uint32_t v[NW];
#pragma unroll
                for (int j = 0; j < NW; j++) v[j] = w[j];
                dbits = v[0] & 0xFFFFu;
                if (FMT == FMT_Q50) qh = __funnelshift_r(v[0], v[1], 16);
#pragma unroll
                for (int j = 0; j < 4; j++) qs[j] = __funnelshift_r(v[QS / 4 + j], v[QS / 4 + j + 1], 16);
            } else {  // block start = 2 mod 4: d is a half-word, everything after it word-aligned
                dbits = *reinterpret_cast<const unsigned short *>(b);
                if (FMT == FMT_Q50) qh = *reinterpret_cast<const uint32_t *>(b + 2);
#pragma unroll
                for (int j = 0; j < 4; j++) qs[j] = *reinterpret_cast<const uint32_t *>(b + QS + 4 * j);
            }
            const __half2 d2 = __half2half2(__ushort_as_half((unsigned short)dbits));
#pragma unroll
            for (int hi = 0; hi < 2; hi++)      // low nibbles = elements 0 .. 15, high = 16 .. 31
#pragma unroll
                for (int c = 0; c < 2; c++) {  // eight elements: words 2c, 2c + 1
                    uint32_t r[4];
#pragma unroll
                    for (int w = 0; w < 2; w++) {
                        uint32_t q = (qs[2 * c + w] >> (4 * hi)) & 0x0F0F0F0Fu;
                        if (FMT == FMT_Q50) q |= spread4_bits(qh >> (16 * hi + 4 * (2 * c + w))) << 4;
                        __half2 lo2, hi2;
                        bytes_to_h2(q, 1024.0f + (float)BIAS, lo2, hi2);  // q - 8 (q - 16), exact
                        r[2 * w] = h2_as_u32(__hmul2(lo2, d2));
                        r[2 * w + 1] = h2_as_u32(__hmul2(hi2, d2));
                    }
                    o[4 * i + 2 * hi + c] = make_uint4(r[0], r[1], r[2], r[3]);  // k = 32 i + 16 hi + 8 c .. + 7 of the step
                }
        }
    }
    __device__ __forceinline__ void store(uint8_t *at, int wg, int lane, const uint4 (&o)[8]) {
        const int r = 32 * wg + lane;
        uint8_t *rowp = at + r * 128;
#pragma unroll
        for (int c = 0; c < 8; c++) *reinterpret_cast<uint4 *>(rowp + ((c ^ (r & 7)) << 4)) = o[c];
    }
};
template <>
struct Dequant<FMT_Q40> : DequantClassic<FMT_Q40> {};
template <>
struct Dequant<FMT_Q50> : DequantClassic<FMT_Q50> {};

// ---- the kernel -----------------------------------------------------------------------------------
// grid: (token tiles, groups of MT weight-row tiles): CTAs that share weight tiles run side by side, so the
// second reader finds the raw bytes in L2.
// Sequence numbers: raw super-chunk q = j * mt + i (k-block j, row tile i of the CTA), A tile a = ks * mt + i
// (k-step ks); B stage = ks.  Each ring slot is sequence % depth with the usual phase parity.
#ifdef GLLMK_WQ_PROF
// Development aid (not built by default): cycles each warp of gemm_wq_kernel spends in its phases.
__device__ unsigned long long g_wq_prof[1024 * 20 * 8];
#define WQP_DECL unsigned long long wqp_t = 0, wqp_a[7] = {0, 0, 0, 0, 0, 0, 0}, wqp_start = clock64()
#define WQP_T0() wqp_t = clock64()
#define WQP_ACC(i) do { const unsigned long long n_ = clock64(); wqp_a[i] += n_ - wqp_t; wqp_t = n_; } while (0)
#define WQP_OUT() do { if (lane == 0 && blockIdx.y * gridDim.x + blockIdx.x < 1024) { unsigned long long *o_ = g_wq_prof + ((blockIdx.y * gridDim.x + blockIdx.x) * 20 + warp) * 8; \
    for (int i_ = 0; i_ < 7; i_++) o_[i_] = wqp_a[i_]; o_[7] = clock64() - wqp_start; } } while (0)
#else
#define WQP_DECL
#define WQP_T0()
#define WQP_ACC(i)
#define WQP_OUT()
#endif

template <int FMT, int MT>
__global__ void __launch_bounds__(WQ_THREADS, 1) gemm_wq_kernel(const __grid_constant__ GemmParams p, const __grid_constant__ GemmGroups G) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * WQ_SA + 2 * WQ_MAX_SB + 2 * WQ_MAX_R + 1];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    constexpr int RAW = wq_raw_bytes(FMT);
    constexpr uint32_t TMEM_COLS = MT == 2 ? 512 : 256;
    const uint32_t smem_s = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (smem_s - tc::smem_u32(smem_raw));
    const int bstage = p.ntok * 128;
    const uint32_t a_off = 0, b_off = (uint32_t)(WQ_SA * WQ_TILE), raw_off = b_off + (uint32_t)(p.sb * bstage);
    const uint32_t fullA = tc::smem_u32(&bars[0]), emptyA = fullA + 8 * WQ_SA, fullB = emptyA + 8 * WQ_SA,
                   emptyB = fullB + 8 * WQ_MAX_SB, rawfull = emptyB + 8 * WQ_MAX_SB, rawempty = rawfull + 8 * WQ_MAX_R,
                   accum = rawempty + 8 * WQ_MAX_R;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // which tile, and which part of its k range
    int bx = blockIdx.x, by = blockIdx.y, jb0 = 0, njb = p.nsc, split = 0, nsplit = 1, tail_tile = 0;
    if (p.split_s > 1) {
        const int u = (int)blockIdx.x;
        int t = u;
        if (u >= p.split_f) {
            tail_tile = (u - p.split_f) / p.split_s;
            split = (u - p.split_f) % p.split_s;
            nsplit = p.split_s;
            t = p.split_f + tail_tile;
            jb0 = (int)((int64_t)p.nsc * split / nsplit);
            njb = (int)((int64_t)p.nsc * (split + 1) / nsplit) - jb0;
        }
        bx = t % p.ntt;
        by = t / p.ntt;
    }
    const int tile0 = by * MT;
    const int mt = min(MT, p.row_tiles - tile0);  // row tiles this CTA really has
    const int grp_id = G.tile_group[bx];
    const int64_t tok0 = G.tile_tok0[bx], tok_end = tok0 + G.tile_cnt[bx];
    const int nks = 4 * njb, nks_row = 4 * p.nsc;  // k-steps of this unit / of a whole row
    volatile int *abort_flag = &abort_s;

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < WQ_SA; s++) {
            tc::mbar_init(fullA + 8 * s, WQ_DW / 4);  // one arrival per warp of the slot's dequant group
            tc::mbar_init(emptyA + 8 * s, 1);
        }
        for (int s = 0; s < WQ_MAX_SB; s++) {
            tc::mbar_init(fullB + 8 * s, 1);
            tc::mbar_init(emptyB + 8 * s, (uint32_t)mt);  // one commit per MMA issuer
        }
        for (int s = 0; s < WQ_MAX_R; s++) {
            tc::mbar_init(rawfull + 8 * s, wq_row_major(FMT) ? 32 : 1);  // row-major formats: one arrival per lane of the copy warp
            tc::mbar_init(rawempty + 8 * s, WQ_DW / mt);  // the warps that read a super-chunk
        }
        tc::mbar_init(accum, (uint32_t)mt);
        tc::mbar_init_fence();
    }
    if (warp == 2) tc::tmem_alloc(tc::smem_u32(&tmem_base_s), TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_d = tmem_base_s;
    WQP_DECL;

    if (warp == 0 && wq_row_major(FMT)) {
        constexpr int SLOT = wq_slot(FMT), RSTRIDE = wq_row_stride(FMT), CPR = SLOT / 16;  // 16-byte chunks per row piece
        // ---------------- raw weight blocks: one block of each of the tile's 128 rows per super-chunk ----------------
        // The blocks of a tile lie a whole row apart in memory, so a super-chunk is 128 pieces of 224 / 176 / 144 bytes.  As 128
        // bulk copies they paced the kernel (a copy engine request per piece: ~1.8 k cycles per tile step); the whole warp
        // copies them with 16-byte cp.async instead — 64 per lane — and every lane's copies arrive at the slot's barrier
        // when they have landed (cp.async.mbarrier.arrive.noinc).
        int slot = 0, round = 0;
        bool ok = true;
        for (int jl = 0; jl < njb && ok; jl++) {
            const int jb = jb0 + jl;
            for (int ti = 0; ti < mt && ok; ti++) {
                if (lane == 0 && round > 0 && !tc::mbar_wait(rawempty + 8 * slot, (uint32_t)((round - 1) & 1), abort_flag)) {
                    abort_s = 1;
                    atomicExch(p.status, 10);
                    ok = false;
                }
                ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
                if (!ok) break;
                const uint32_t dst = smem_s + raw_off + (uint32_t)(slot * RAW);
                const int64_t trow0 = (int64_t)(tile0 + ti) * WQ_BM;
                const int rmax = (int)(p.n - 1 - trow0 < WQ_BM - 1 ? p.n - 1 - trow0 : WQ_BM - 1);  // rows past the matrix repeat the last one; not stored
                // half a warp per row piece: lane % 16 = 16-byte chunk (the lanes past the piece's CPR chunks idle), rows 2 j +
                // lane / 16 — constant strides, so an iteration is the copy and two additions
                const size_t row_bytes = (size_t)p.nsc * SLOT;
                const int hrow = lane >> 4, ch = lane & 15;
                const uint8_t *tile_src = G.qs[grp_id] + ((size_t)trow0 * p.nsc + jb) * SLOT + 16 * ch;
                if (ch < CPR) {
                    if (rmax == WQ_BM - 1) {
                        const uint8_t *src = tile_src + (size_t)hrow * row_bytes;
                        uint32_t d = dst + (uint32_t)(hrow * RSTRIDE + 16 * ch);
#pragma unroll 8
                        for (int j = 0; j < WQ_BM / 2; j++, src += 2 * row_bytes, d += 2 * RSTRIDE) cp_async16_s(d, src);
                    } else {
                        for (int r = hrow; r < WQ_BM; r += 2)
                            cp_async16_s(dst + (uint32_t)(r * RSTRIDE + 16 * ch), tile_src + (size_t)(r < rmax ? r : rmax) * row_bytes);
                    }
                }
                cp_async_arrive(rawfull + 8 * slot);
                if (++slot == p.r) slot = 0, round++;
            }
        }
    } else if (warp == 0) {
        // ---------------- raw weight super-chunks: one thread, bulk copies ----------------
        if (lane == 0) {
            int slot = 0, round = 0;
            for (int jl = 0; jl < njb; jl++) {
                const int jb = jb0 + jl;
                for (int ti = 0; ti < mt; ti++) {
                    WQP_T0();
                    if (round > 0 && !tc::mbar_wait(rawempty + 8 * slot, (uint32_t)((round - 1) & 1), abort_flag)) {
                        abort_s = 1;
                        atomicExch(p.status, 10);
                        jl = njb;
                        break;
                    }
                    WQP_ACC(0);
                    const int tile = tile0 + ti;
                    const uint32_t dst = smem_s + raw_off + (uint32_t)(slot * RAW);
                    tc::mbar_expect_tx(rawfull + 8 * slot, RAW);
                    if (FMT == FMT_Q4K || FMT == FMT_Q80) {
                        // the eight 16-row chunks of a 128-row tile for k-block jb are contiguous
                        bulk_g2s(dst, G.qs[grp_id] + ((size_t)tile * p.nsc + jb) * RAW, RAW, rawfull + 8 * slot);
                    } else {
                        constexpr int SFB = RAW - WQ_TILE;
                        bulk_g2s(dst, G.qs[grp_id] + ((size_t)tile * p.nsc + jb) * WQ_TILE, WQ_TILE, rawfull + 8 * slot);
                        bulk_g2s(dst + WQ_TILE, G.aux[grp_id] + ((size_t)tile * p.nsc + jb) * SFB, SFB, rawfull + 8 * slot);
                    }
                    if (++slot == p.r) slot = 0, round++;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- activation tiles: one thread, bulk copies ----------------
        if (lane == 0) {
            // a tile of more than 128 tokens is two activation images: a whole one and the first ntok - 128 rows
            const int halves = (p.ntok + 127) / 128, img0 = G.tile_img[bx];
            const uint32_t hbytes[2] = {(uint32_t)(p.ntok > 128 ? WQ_TILE : bstage), (uint32_t)(bstage - WQ_TILE)};
            int slot = 0, round = 0;
            asm volatile("griddepcontrol.wait;\n" ::: "memory");  // the staging kernel's tile images are complete from here on
            for (int ks = 0; ks < nks; ks++) {
                WQP_T0();
                if (round > 0 && !tc::mbar_wait(emptyB + 8 * slot, (uint32_t)((round - 1) & 1), abort_flag)) {
                    abort_s = 1;
                    atomicExch(p.status, 11);
                    break;
                }
                WQP_ACC(0);
                const uint32_t dst = smem_s + b_off + (uint32_t)(slot * bstage);
                tc::mbar_expect_tx(fullB + 8 * slot, (uint32_t)bstage);
                for (int h = 0; h < halves; h++)
                    bulk_g2s(dst + h * WQ_TILE, p.xt + ((size_t)(img0 + h) * nks_row + 4 * jb0 + ks) * WQ_TILE, hbytes[h], fullB + 8 * slot);
                if (++slot == p.sb) slot = 0, round++;
            }
        }
    } else if (warp < WQ_CTRL) {
        // ---------------- MMA issue: one thread per row tile ----------------
        // Every step of this role (barrier probe, fence, MMA, commit) has a long issue latency, ~0.9 k cycles per A tile
        // in all, against 0.25 - 0.5 k cycles of tensor-pipe time: with two row tiles, two threads in two warps — each with
        // its own accumulator and its own A slots (tile a = 2 * ks + i lives in slot a % 4) — keep the pipe fed.
        const int i = warp - 2;
        if (lane == 0 && i < mt) {
            const uint32_t idesc = tc::idesc_f16(WQ_BM, p.ntok, 0, 0);  // fp16 x fp16 -> f32
            bool ok = true;
            int sb = 0, bround = 0;
            for (int ks = 0; ks < nks && ok; ks++) {
                WQP_T0();
                const uint64_t bd = tc::smem_desc_sw128(smem_s + b_off + (uint32_t)(sb * bstage));
                const int a = ks * mt + i, sa = a % WQ_SA;
                // probes that do not suspend the thread: its reaction time is on the critical path of every tile
                ok = tc::mbar_spin(fullB + 8 * sb, (uint32_t)(bround & 1), abort_flag) &&
                     tc::mbar_spin(fullA + 8 * sa, (uint32_t)((a / WQ_SA) & 1), abort_flag);
                WQP_ACC(0);
                if (!ok) {
                    abort_s = 1;
                    atomicExch(p.status, 12);
                    break;
                }
                tc::fence_after_sync();
                const uint64_t ad = tc::smem_desc_sw128(smem_s + a_off + sa * WQ_TILE);
#pragma unroll
                for (int k4 = 0; k4 < 4; k4++)
                    tc::mma_f16(tmem_d + 256u * (uint32_t)i, ad + 2 * k4, bd + 2 * k4, idesc, (uint32_t)((ks | k4) != 0));
                tc::mma_commit(emptyA + 8 * sa);  // the A tile is free when these MMAs have read it
                tc::mma_commit(emptyB + 8 * sb);  // the stage, when both issuers' MMAs have
                if (++sb == p.sb) sb = 0, bround++;
            }
            if (ok) tc::mma_commit(accum);
        }
    } else {
        // ---------------- dequant warps, then epilogue ----------------
        const int dw = warp - WQ_CTRL, grp = dw >> 2, wg = dw & 3;
        Dequant<FMT> dq;
        dq.global = G.gs[grp_id];
        bool ok = true;
        // group grp makes the A tiles a = grp, grp + 4, ... (slot grp of the A ring); a = ks * mt + i.
        // mt == 1: the group always has quarter grp of every super-chunk; mt == 2: row tile i = grp % 2 and
        // the quarters grp / 2 and grp / 2 + 2.
        const int na = nks * mt;
        const int qstep = (MT == 2 && mt == 2) ? 2 : 1;  // raw sequence numbers between this group's super-chunks
        int rslot = (MT == 2 && mt == 2) ? (grp & 1) : 0, rround = 0;
        if (rslot >= p.r) rslot -= p.r, rround++;
        // A tile = conversion into registers, then stores.  The group's first warp does the waiting — for this tile's A
        // slot and for the raw super-chunk of the NEXT tile — between the two, so that the MMAs still reading the slot run
        // under the conversion; the other three warps sleep on a hardware barrier.  The probes do not suspend the
        // thread (a suspended thread wakes up late, and the group's reaction time is on the critical path).
        if (wg == 0 && grp < na && !tc::mbar_spin(rawfull + 8 * rslot, (uint32_t)(rround & 1), abort_flag)) abort_s = 1;
        tc::named_bar_sync(1 + grp, 128);
        ok = !*abort_flag;
        for (int a = grp, it = 0; a < na && ok; a += 4, it++) {
            const int ks = (MT == 2 && mt == 2) ? (a >> 1) : a;
            const int pp = ks & 3;
            uint4 o[8];
            WQP_T0();
            dq.compute(smem + raw_off + rslot * RAW, pp, wg, lane, o);
            // the values are needed in registers HERE: without this the compiler moves the arithmetic below the waits
#pragma unroll
            for (int i = 0; i < 8; i++) asm volatile("" ::"r"(o[i].x), "r"(o[i].y), "r"(o[i].z), "r"(o[i].w));
            // last quarter this warp reads of the super-chunk: hand the slot back and move to the next one
            const bool last = !(MT == 2 && mt == 2) || pp >= 2;
            if (last) {
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(rawempty + 8 * rslot);
                rslot += qstep;
                if (rslot >= p.r) rslot -= p.r, rround++;
            }
            WQP_ACC(0);
            if (wg == 0) {
                bool ready = (it == 0 || tc::mbar_spin(emptyA + 8 * grp, (uint32_t)((it - 1) & 1), abort_flag));
                WQP_ACC(1);
                ready = ready && (a + 4 >= na || !last || tc::mbar_spin(rawfull + 8 * rslot, (uint32_t)(rround & 1), abort_flag));
                if (!ready) abort_s = 1;
                WQP_ACC(2);
            }
            tc::named_bar_sync(1 + grp, 128);
            WQP_ACC(3);
            ok = !*abort_flag;
            if (!ok) break;
            dq.store(smem + a_off + grp * WQ_TILE, wg, lane, o);
            WQP_ACC(4);
            tc::fence_proxy_async();  // every writer makes its own stores visible to the tensor core's proxy
            WQP_ACC(5);
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(fullA + 8 * grp);
            WQP_ACC(6);
        }
        if (!ok && !abort_s) {
            abort_s = 1;
            atomicExch(p.status, 13);
        }
        ok = ok && !abort_s && tc::mbar_wait(accum, 0u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            // warp w may read TMEM lanes 32 * (w % 4) .. + 31 = weight rows; the four warps of a quadrant take
            // every fourth group of 32 token columns
            tc::fence_after_sync();
            const int quad = warp & 3;
            // all MMAs have completed, so the rings are free: each warp stages its blocks in 4 KB of the A ring
            uint8_t *stage = smem + a_off + dw * 4096;
            if (nsplit == 1) {
                for (int i = 0; i < mt; i++) {
                    const int64_t row_base = (int64_t)(tile0 + i) * WQ_BM + 32 * quad;
                    for (int c = 32 * (dw >> 2); c < p.ntok; c += 32 * (WQ_DW / 4)) {
                        uint32_t v[32];
                        tc::tmem_ld32(tmem_d + ((uint32_t)(32 * quad) << 16) + 256u * (uint32_t)i + (uint32_t)c, v);
                        tc::tmem_ld_wait();
                        float o[32];
#pragma unroll
                        for (int jj = 0; jj < 32; jj++) o[jj] = __uint_as_float(v[jj]);
                        if (p.y_bf16) tc::store_block_32x32<true>(p.y, p.ldy, row_base, tok0 + c, p.n, tok_end, o, stage, lane, p.vec);
                        else tc::store_block_32x32<false>(p.y, p.ldy, row_base, tok0 + c, p.n, tok_end, o, stage, lane, p.vec);
                    }
                }
            } else {
                // A unit of a split tile: the accumulator goes to this unit's partial area ([row tile][token][128 rows]
                // f32), and the unit that arrives last at the tile's counter adds the partials in unit order — the
                // result does not depend on which one that is — and stores y.
                const size_t unit_floats = (size_t)MT * p.ntok * WQ_BM;
                float *tile_part = p.partial + (size_t)tail_tile * nsplit * unit_floats, *mine = tile_part + (size_t)split * unit_floats;
                for (int i = 0; i < mt; i++)
                    for (int c = 32 * (dw >> 2); c < p.ntok; c += 32 * (WQ_DW / 4)) {
                        uint32_t v[32];
                        tc::tmem_ld32(tmem_d + ((uint32_t)(32 * quad) << 16) + 256u * (uint32_t)i + (uint32_t)c, v);
                        tc::tmem_ld_wait();
                        float *dst = mine + ((size_t)i * p.ntok + c) * WQ_BM + 32 * quad + lane;
#pragma unroll
                        for (int jj = 0; jj < 32; jj++) __stcg(dst + (size_t)jj * WQ_BM, __uint_as_float(v[jj]));  // lanes: 32 consecutive rows
                    }
                __threadfence();
                tc::named_bar_sync(6, 32 * WQ_DW);  // every dequant / epilogue warp has written and fenced
                __shared__ int last_s;
                if (dw == 0 && lane == 0) {
                    const int old = atomicAdd(p.tail_cnt + tail_tile, 1);
                    last_s = (old == nsplit - 1);
                    if (last_s) p.tail_cnt[tail_tile] = 0;  // ready for the next launch
                    __threadfence();
                }
                tc::named_bar_sync(6, 32 * WQ_DW);
                if (last_s) {
                    for (int i = 0; i < mt; i++) {
                        const int64_t row_base = (int64_t)(tile0 + i) * WQ_BM + 32 * quad;
                        for (int c = 32 * (dw >> 2); c < p.ntok; c += 32 * (WQ_DW / 4)) {
                            float o[32];
#pragma unroll
                            for (int jj = 0; jj < 32; jj++) o[jj] = 0.0f;
                            for (int sp = 0; sp < nsplit; sp++) {
                                const float *src = tile_part + (size_t)sp * unit_floats + ((size_t)i * p.ntok + c) * WQ_BM + 32 * quad + lane;
#pragma unroll
                                for (int jj = 0; jj < 32; jj++) o[jj] += __ldcg(src + (size_t)jj * WQ_BM);
                            }
                            if (p.y_bf16) tc::store_block_32x32<true>(p.y, p.ldy, row_base, tok0 + c, p.n, tok_end, o, stage, lane, p.vec);
                            else tc::store_block_32x32<false>(p.y, p.ldy, row_base, tok0 + c, p.n, tok_end, o, stage, lane, p.vec);
                        }
                    }
                }
            }
        } else if (!abort_s) {
            abort_s = 1;
            atomicExch(p.status, 14);
        }
    }
    WQP_OUT();
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 2) tc::tmem_dealloc(tmem_d, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
template <int FMT, int MT>
static int32_t launch_wq(Ctx *c, const GemmParams &p, const GemmGroups &G, dim3 grid, size_t smem, cudaStream_t s) {
    static bool attr_set[64] = {};  // function attributes are per device
    const int dev_slot = c->device & 63;
    if (!attr_set[dev_slot]) {
        GK_CUDA(c, cudaFuncSetAttribute(gemm_wq_kernel<FMT, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, WQ_SMEM_LIMIT + 1024));
        attr_set[dev_slot] = true;
    }
    // launched programmatically behind the staging kernel (which everything earlier in the stream precedes)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(WQ_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = c->gemm_pdl ? 1 : 0;
    GK_CUDA(c, cudaLaunchKernelEx(&cfg, gemm_wq_kernel<FMT, MT>, p, G));
    return GLLMK_STATUS_OK;
}
template <int FMT>
static int32_t launch_wq_mt(Ctx *c, const GemmParams &p, const GemmGroups &G, int mt, dim3 grid, size_t smem, cudaStream_t s) {
    return mt == 2 ? launch_wq<FMT, 2>(c, p, G, grid, smem, s) : launch_wq<FMT, 1>(c, p, G, grid, smem, s);
}

// One launch: groups [g0, g1) with their token ranges cut into tiles of `ntok` tokens.
static int32_t gemm_groups_chunk(Ctx *c, const Weight *const *ws, int ng, const void *a, int a_bf16, int64_t lda,
                                 const int64_t *tok_begin, const int64_t *tok_count, int ntok, void *y, int y_bf16, int64_t ldy,
                                 cudaStream_t s, const void *a_up) {
    const Weight *w = ws[0];
    const int fmt = w->qt == GLLMK_QUANT_Q4K ? FMT_Q4K : (w->qt == GLLMK_QUANT_Q8_0 ? FMT_Q80 : (w->qt == GLLMK_QUANT_NVFP4 ? FMT_NVFP4 : (w->qt == GLLMK_QUANT_Q6_K ? FMT_Q6K : (w->qt == GLLMK_QUANT_Q5_K ? FMT_Q5K : (w->qt == GLLMK_QUANT_Q4_0 ? FMT_Q40 : (w->qt == GLLMK_QUANT_Q5_0 ? FMT_Q50 : FMT_MXFP4))))));
    const int raw = wq_raw_bytes(fmt);
    GemmParams p{};
    GemmGroups G{};
    ImgTiles imgs{};
    p.n = w->n;
    p.nsc = (int)((w->k + 255) / 256);
    p.y = y;
    p.y_bf16 = y_bf16;
    p.ldy = ldy;
    p.vec = (((uintptr_t)y & 15) == 0 && (ldy * (y_bf16 ? 2 : 4)) % 16 == 0) ? 1 : 0;
    p.status = c->status_dev;
    p.ntok = ntok;
    const int halves = (ntok + 127) / 128;
    int ntiles = 0, nimg = 0;
    for (int g = 0; g < ng; g++) {
        G.qs[g] = static_cast<const uint8_t *>(ws[g]->qs);
        G.aux[g] = static_cast<const uint8_t *>(ws[g]->aux);
        G.gs[g] = ws[g]->global_scale;
        for (int64_t t0 = 0; t0 < tok_count[g]; t0 += ntok) {
            const int cnt = (int)(tok_count[g] - t0 < ntok ? tok_count[g] - t0 : ntok);
            G.tile_group[ntiles] = g;
            G.tile_tok0[ntiles] = (int)(tok_begin[g] + t0);
            G.tile_cnt[ntiles] = cnt;
            G.tile_img[ntiles] = nimg;
            for (int h = 0; h < halves; h++) {
                imgs.tok0[nimg] = (int)(tok_begin[g] + t0 + 128 * h);
                imgs.cnt[nimg] = cnt - 128 * h < 0 ? 0 : (cnt - 128 * h > 128 ? 128 : cnt - 128 * h);
                nimg++;
            }
            ntiles++;
        }
    }
    if (ntiles == 0) return GLLMK_STATUS_OK;
    const int row_tiles = (int)((w->n_pad + WQ_BM - 1) / WQ_BM);  // (Q6_K rows are not padded on the device)
    const int bstage = ntok * 128;
    // Row tiles per CTA and how the last wave is cut along k, chosen together.  Two row tiles share one activation stage
    // (less shared-memory fill traffic per flop, two issuing threads, fixed costs paid once) but halve the CTA count; a
    // last — or only — wave that fills a fraction of the SMs is cut along k into units (tail split, below).  Estimated
    // time, in k-steps of a single tile: whole waves + the tail, times (k-steps per CTA x relative step cost + a fixed
    // prologue / epilogue worth ~16 steps).
    const int sms = c->sm_count;
    const auto estimate = [&](int m_t, int *split) -> double {
        const double step = m_t == 2 ? 2.0 * (ntok > 128 ? 0.68 : 0.62) : 1.0;  // measured: a pair step costs 1.36 / 1.24 single steps
        const int tiles = ntiles * ((row_tiles + m_t - 1) / m_t), full = tiles / sms, tail = tiles - full * sms;
        double tail_t = tail > 0 ? 1.0 : 0.0;
        *split = 1;
        if (tail > 0 && c->gemm_tail_split != 1)
            for (int sp = 2; sp <= 8 && p.nsc / sp >= 4; sp++) {
                const double t = (double)((tail * sp + sms - 1) / sms) / sp + 0.05 * sp;  // + fill / drain and the partial traffic
                if (t < tail_t) tail_t = t, *split = sp;
            }
        return (full + tail_t) * (4.0 * p.nsc * step + 16.0);
    };
    int mt = 1;
    if (row_tiles % 2 == 0) {
        int s1, s2;
        if (estimate(2, &s2) < estimate(1, &s1)) mt = 2;
        if (c->gemm_row_tiles == 1 || c->gemm_row_tiles == 2) mt = (int)c->gemm_row_tiles;
    }
    // Shared-memory plan: four A tiles; three B stages (activation tiles come from L2: ~1 us of latency against
    // 0.2 - 0.5 us per k-step); everything else goes to the raw ring, because the weight stream comes from HBM and
    // with few tokens a k-step is short: two super-chunks in flight per SM cap the stream at ~15 GB/s per SM.
    p.sb = 3;
    p.r = (WQ_SMEM_LIMIT - WQ_SA * WQ_TILE - p.sb * bstage) / raw;
    if (p.r < mt + 1) {  // big raw super-chunks (Q8_0) with a 256-token tile
        p.sb = 2;
        p.r = (WQ_SMEM_LIMIT - WQ_SA * WQ_TILE - p.sb * bstage) / raw;
        if (p.r < mt + 1) mt = 1;
    }
    if (p.r > WQ_MAX_R) p.r = WQ_MAX_R;
    if (c->gemm_raw_slots >= mt + 1 && c->gemm_raw_slots < p.r) p.r = (int)c->gemm_raw_slots;
    if (p.r < mt + 1) return fail(c, GLLMK_STATUS_RUNTIME_ERROR, "gemm: shared-memory plan does not fit");
    // what the raw ring cannot use goes back to B stages
    const int more_sb = (WQ_SMEM_LIMIT - WQ_SA * WQ_TILE - p.r * raw) / bstage;
    p.sb = more_sb > WQ_MAX_SB ? WQ_MAX_SB : more_sb;
    const size_t smem = 1024 + (size_t)WQ_SA * WQ_TILE + (size_t)p.sb * bstage + (size_t)p.r * raw;
    p.row_tiles = row_tiles;
    // activations -> fp16 tile images in the context's scratch
    const int nks = 4 * p.nsc;
    int32_t rc = ensure_act(c, (size_t)nimg * nks * WQ_TILE);
    if (rc) return rc;
    p.xt = static_cast<const uint8_t *>(c->act);
    stage_act_kernel<<<dim3((unsigned)nks, (unsigned)nimg), 256, 0, s>>>(a, a_bf16, lda, w->k, static_cast<uint8_t *>(c->act), imgs, a_up);
    GK_CUDA(c, cudaGetLastError());
    dim3 grid((unsigned)ntiles, (unsigned)((row_tiles + mt - 1) / mt));
    // Tail split: the last, partly filled wave of tiles — the only one, when there are fewer tiles than SMs — is cut along
    // k so that its work spreads over all SMs (224 tiles on 148 SMs: 148 whole tiles, then 76 tiles in thirds = 228 units
    // in two short waves — 1.67 tile times instead of 2; 64 two-tile CTAs: 128 half units).  Only when a unit keeps at
    // least four k-blocks.
    p.split_s = 1;
    if (c->gemm_tail_split != 1) {
        const int tiles = (int)(grid.x * grid.y);
        const int full = tiles / sms * sms, tail = tiles - full;
        int best_s = 1;
        estimate(mt, &best_s);
        if (c->gemm_tail_split > 1 && p.nsc / (int)c->gemm_tail_split >= 1) best_s = (int)c->gemm_tail_split;
        if (tail > 0 && best_s > 1) {
            const size_t unit_floats = (size_t)mt * ntok * WQ_BM;
            rc = ensure_red(c, (size_t)tail * best_s * unit_floats * sizeof(float));
            if (!rc) rc = ensure_cnt(c, (size_t)(tail + 1) * sizeof(int));
            if (rc) return rc;
            p.split_s = best_s;
            p.split_f = full;
            p.ntt = (int)grid.x;
            p.partial = static_cast<float *>(c->red);
            p.tail_cnt = static_cast<int *>(c->cnt);
            grid = dim3((unsigned)(full + tail * best_s), 1u);
        }
    }
    switch (fmt) {
        case FMT_Q4K: return launch_wq_mt<FMT_Q4K>(c, p, G, mt, grid, smem, s);
        case FMT_Q80: return launch_wq_mt<FMT_Q80>(c, p, G, mt, grid, smem, s);
        case FMT_NVFP4: return launch_wq_mt<FMT_NVFP4>(c, p, G, mt, grid, smem, s);
        case FMT_Q6K: return launch_wq_mt<FMT_Q6K>(c, p, G, mt, grid, smem, s);
        case FMT_Q5K: return launch_wq_mt<FMT_Q5K>(c, p, G, mt, grid, smem, s);
        case FMT_Q40: return launch_wq_mt<FMT_Q40>(c, p, G, mt, grid, smem, s);
        case FMT_Q50: return launch_wq_mt<FMT_Q50>(c, p, G, mt, grid, smem, s);
        default: return launch_wq_mt<FMT_MXFP4>(c, p, G, mt, grid, smem, s);
    }
}

// Groups g use rows [row_offsets[g], row_offsets[g + 1]) of a and y with weight ws[g] (all of one shape and type).
int32_t gemm_grouped_launch(Ctx *c, const Weight *const *ws, int n_groups, const void *a, int a_bf16, int64_t lda,
                            const int64_t *row_offsets, void *y, int y_bf16, int64_t ldy, cudaStream_t s, const void *a_up) {
    const int align = a_bf16 ? 8 : 4;
    const bool row_major_ok = ws[0]->qt == GLLMK_QUANT_Q6_K || ws[0]->qt == GLLMK_QUANT_Q5_K ||
                              ((ws[0]->qt == GLLMK_QUANT_Q4_0 || ws[0]->qt == GLLMK_QUANT_Q5_0) && ws[0]->k % 256 == 0);
    if ((ws[0]->qt < GLLMK_QUANT_Q4K || ws[0]->qt > GLLMK_QUANT_NVFP4) && !row_major_ok)
        return fail(c, GLLMK_STATUS_UNSUPPORTED, "gemm: weight type %d is not block-quantized (use gllmk_gemm_int8)", ws[0]->qt);
    if (((uintptr_t)a & 15) || (lda % align)) return fail(c, GLLMK_STATUS_INVALID_ARG, "gemm: activations must be 16-byte aligned rows");
    if (ws[0]->k % 8) return fail(c, GLLMK_STATUS_INVALID_ARG, "gemm: k=%lld is not a multiple of 8", (long long)ws[0]->k);
    // MMA N: 256-token tiles, or the largest group rounded up to a multiple of 32 when no group has more
    int64_t most = 0;
    for (int g = 0; g < n_groups; g++) most = most > row_offsets[g + 1] - row_offsets[g] ? most : row_offsets[g + 1] - row_offsets[g];
    if (most <= 0) return GLLMK_STATUS_OK;
    const int ntok = most >= WQ_BN ? WQ_BN : (int)((most + 31) / 32 * 32);
    const int halves = (ntok + 127) / 128;
    // launches of at most WQ_MAX_GROUPS groups, WQ_MAX_TOK_TILES token tiles, WQ_MAX_IMG_TILES images
    const Weight *cw[WQ_MAX_GROUPS];
    int64_t cb[WQ_MAX_GROUPS], cc[WQ_MAX_GROUPS];
    int ng = 0, tiles = 0;
    const auto flush = [&]() -> int32_t {
        if (ng == 0) return GLLMK_STATUS_OK;
        const int32_t rc = gemm_groups_chunk(c, cw, ng, a, a_bf16, lda, cb, cc, ntok, y, y_bf16, ldy, s, a_up);
        ng = 0;
        tiles = 0;
        return rc;
    };
    const int tile_cap = WQ_MAX_IMG_TILES / halves < WQ_MAX_TOK_TILES ? WQ_MAX_IMG_TILES / halves : WQ_MAX_TOK_TILES;
    for (int g = 0; g < n_groups; g++) {
        int64_t begin = row_offsets[g], left = row_offsets[g + 1] - row_offsets[g];
        while (left > 0) {
            if (ng == WQ_MAX_GROUPS || tiles == tile_cap) {
                const int32_t rc = flush();
                if (rc) return rc;
            }
            const int64_t room = (int64_t)(tile_cap - tiles) * ntok;
            const int64_t take = left < room ? left : room;
            cw[ng] = ws[g];
            cb[ng] = begin;
            cc[ng] = take;
            ng++;
            tiles += (int)((take + ntok - 1) / ntok);
            begin += take;
            left -= take;
        }
    }
    return flush();
}

int32_t gemm_launch(Ctx *c, const Weight *w, const void *a, int a_bf16, int64_t lda, int m, void *y, int y_bf16, int64_t ldy,
                    cudaStream_t s, const void *a_up) {
    const int64_t offs[2] = {0, m};
    return gemm_grouped_launch(c, &w, 1, a, a_bf16, lda, offs, y, y_bf16, ldy, s, a_up);
}

}  // namespace gllmk

#ifdef GLLMK_WQ_PROF
extern "C" __attribute__((visibility("default"))) int gllmk_debug_wq_prof(unsigned long long *out) {
    return (int)cudaMemcpyFromSymbol(out, gllmk::g_wq_prof, sizeof(gllmk::g_wq_prof));
}
#endif
