// Internal declarations shared by the translation units of libgllmk.so.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/gllmk.h"
#include "quant_format.cuh"

namespace gllmk {

constexpr int Q4K_CHUNK = 2368;
constexpr int Q80_CHUNK = 4352;
// chunk order of the Q4_K plane: [tile group TG = T / 8][k-block b][tile in group T % 8]
__host__ __device__ inline size_t q4k_chunk_index(int64_t T, int64_t b, int64_t nb) {
    return ((size_t)(T >> 3) * (size_t)nb + (size_t)b) * 8 + (size_t)(T & 7);
}

// ---- device layouts -------------------------------------------------------------------------
//
// Q4_K (256 el / 144 B), rows padded to a multiple of 128, T = row / 16, b = k-block.  One plane of
// 2368-byte chunks in the order [T / 8][b][T % 8]: the eight 16-row tiles a CTA works on side by side
// sit next to each other for one k-block ("super-chunk"), and a CTA's whole stream is one contiguous
// byte range.  Inside a chunk, with lane = 4*g + t of a warp:
//   [0, 2048)    uint4 [p = 0..3][lane] = {W(g,p,2t), W(g,p,2t+1), W(g+8,p,2t), W(g+8,p,2t+1)}, W(r,p,i) the
//                i-th 32-bit word of the 32-byte group p of row 16T+r's qs: masking a word with
//                0x0F0F0F0F (after a shift by 4 for the odd sub-block) IS an A-fragment register of
//                mma.m16n8k32.u8 for sub-block 2p (2p+1), k-slot 4t+j <-> element 8t+j of the sub-block
//   [2048, 2304) uint4 [row 0..15] = bytes {sc_0..sc_7, m_0..m_7}: the 6-bit scales and mins unpacked to
//                bytes (re-packed bit-exactly on the way out)
//   [2304, 2368) uint32 [g][h]: d | dmin << 16 (f16 bits) of row 16T + g + 8h
//
// Q8_0 (32 el / 34 B), rows padded to 128, blocks padded to groups of 8 (nb8 per row).  One plane of
// 4352-byte chunks in the order [T / 8][b8][T % 8]:
//   [0, 4096)    uint4 [block 0..7][lane] = {row g bytes 8t..8t+7, row g+8 bytes 8t..8t+7}: the four words
//                are the A-fragment registers a0, a2, a1, a3 of mma.m16n8k32.s8 for that block
//   [4096, 4352) half  [row 0..15][block 0..7]  f16 scale bits (0 for padding blocks)
//
// MXFP4 (block 32) and NVFP4 (block 64 = 4 x 16), rows padded to 128, k padded to 256 (k_pad):
//   data: uint8 [n_pad / 128][k_pad / 256][16384]   nibbles as in the reference (low nibble = even element), in
//                                                tiles of 128 rows x 128 bytes (256 elements) stored as the
//                                                128-byte-swizzled shared-memory image the tensor core reads:
//                                                byte j of row r at r*128 + (((j/16) ^ (r%8)) * 16) + j%16;
//                                                one bulk copy of 16 KB brings a tile in ready to use
//   sf   : uint8 [n_pad / 128][k_pad / (4*sfb)][512] one scale byte per sfb = 32 (MXFP4, E8M0) or 16 (NVFP4,
//                                                UE4M3) elements, in 128-row x 4-scale atoms:
//                                                offset = (r % 32) * 16 + ((r % 128) / 32) * 4 + (s % 4)
//                                                (the tile order tcgen05 block-scaled MMA takes its
//                                                scale factors in)
struct Weight {
    int32_t qt = 0;
    int32_t mx_block = 0;
    int64_t n = 0, k = 0;
    int64_t n_pad = 0;
    int64_t k_pad = 0;  // FP4 planes: k rounded up to 256
    int64_t nb = 0;   // blocks per row
    int64_t nb8 = 0;  // Q8_0: groups of 8 blocks per row
    float global_scale = 1.0f;
    int device = 0;
    void *qs = nullptr;   // Q4_K / Q8_0 quant plane, FP4 data plane
    void *aux = nullptr;  // Q4_K headers, Q8_0 scales, FP4 scale-factor plane
    size_t qs_bytes = 0, aux_bytes = 0;
    uint64_t ref_bytes = 0;
};

struct Ctx {
    int device = 0;
    int sm_count = 0;
    std::string err;
    // activation staging workspace (global scratch written by the staging kernel, read by the GEMV)
    void *ws = nullptr;
    size_t ws_bytes = 0;
    int64_t ws_k = -1;  // K the workspace is currently laid out (and zero-padded) for
    // prefill: activations converted to fp16 shared-memory tile images
    void *act = nullptr;
    size_t act_bytes = 0;
    // split-k partial sums; per-tile arrival counters (zeroed at allocation, self-resetting); status word
    void *red = nullptr;
    size_t red_bytes = 0;
    void *cnt = nullptr;
    size_t cnt_bytes = 0;
    int *status_dev = nullptr;
    // pinned host staging + device staging for the host-pointer entry points
    void *pin = nullptr;
    size_t pin_bytes = 0;
    void *dev_io = nullptr;
    size_t dev_io_bytes = 0;
    cudaStream_t stream = nullptr;  // the context's own stream for host-pointer entry points
    // gllmk_matmul_host_batch: a second stream for the host <-> device copies (they run beside the products), events
    // for the hand-overs, and the instantiated graph of the last argument list that was seen twice
    cudaStream_t copy_stream = nullptr;
    std::vector<cudaEvent_t> events;
    std::vector<uint64_t> batch_key, batch_candidate;
    std::vector<uint8_t> batch_staged;  // of the captured list: per product, bit 0 = x goes through the staging area, bit 1 = y
    cudaGraphExec_t batch_exec = nullptr;
    int64_t host_batch_graph = 1;  // 0: never replay a graph in gllmk_matmul_host_batch
    int64_t gemv_pdl = 1;
    int64_t gemv_fp4_int = 0;  // 1: FP4 decode on the integer-decode GEMV kernel instead of the tensor-core one
    int64_t gemv_ctas_per_sm = 0;  // 0 = what the occupancy calculator allows
    int64_t gemm_tail_split = 0;  // prefill GEMM: 0 = cut the last partial wave of tiles along k when that pays, 1 = never, n = into n
    int64_t gemv_fuse = 0;      // decode GEMV, small shares convert their activation slices inside the GEMV (no staging launch):
                                // 0 never (default: the staging launch overlaps the weight stream and measured faster on one
                                // and two GPUs), 1 exchange products only, 2 every product
    int64_t gemm_fp4_pair = 1;  // FP4 x FP4 GEMM with m > 128 on CTA pairs (cta_group::2, persistent): 0 off, 1 one 256-token
                                // accumulator (fastest measured), 2 two 192-token accumulators, 3 two 128-token accumulators
    int64_t gemm_i8_pair = 1;   // W8A8 GEMM with m > 128 on CTA pairs (cta_group::2, persistent, two accumulators): 0 never,
                                // 1 when the estimate favours it, 2 always
    int64_t gemm_raw_slots = 0;  // weight-only GEMM: raw super-chunk ring depth (0 = chosen by the shared-memory plan)
    int64_t gemm_pdl = 1;        // weight-only GEMM launched programmatically behind its activation staging kernel
    int64_t raw_gemv_mma = 1;    // Q6_K products of 2 tokens and more on the tensor-core kernel (0 = dp2a kernel, 2 = also a single token)
    int64_t gemm_row_tiles = 0;  // weight-only GEMM: row tiles per CTA (0 = estimated, 1, 2)
    int64_t peer_wait_spins = (int64_t)1 << 22;  // probes of another rank's flag before a wait gives up (status 31 / 32)
};

int32_t fail(Ctx *c, int32_t code, const char *fmt, ...);
int32_t cuda_fail(Ctx *c, cudaError_t e, const char *what);
int32_t ensure_ws(Ctx *c, size_t bytes);
int32_t ensure_red(Ctx *c, size_t bytes);
int32_t ensure_act(Ctx *c, size_t bytes);
int32_t ensure_cnt(Ctx *c, size_t bytes);
int32_t ensure_pin(Ctx *c, size_t bytes);
int32_t ensure_dev_io(Ctx *c, size_t bytes);

// Makes the context's device current for the duration of an entry point and restores the caller's.
struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; (void)cudaGetLastError(); return; }
        if (prev != dev && cudaSetDevice(dev) != cudaSuccess) { ok = false; (void)cudaGetLastError(); }
    }
    ~DeviceGuard() {
        if (ok && prev >= 0) cudaSetDevice(prev);
    }
};

#define GK_CUDA(c, call)                                             \
    do {                                                             \
        cudaError_t e__ = (call);                                    \
        if (e__ != cudaSuccess) return cuda_fail((c), e__, #call);   \
    } while (0)

// ---- repack.cu ----
int32_t repack_upload(Ctx *c, Weight *w, const void *blocks_dev, const void *scales_dev, cudaStream_t s);
int32_t repack_unpack(Ctx *c, const Weight *w, void *blocks_dev, void *scales_dev, cudaStream_t s);
int32_t dequant_matrix(Ctx *c, const Weight *w, float *out_dev, cudaStream_t s, const int32_t *ids = nullptr, int64_t count = 0);
int32_t dequant_raw(Ctx *c, int32_t qt, const uint8_t *blocks_dev, const uint8_t *scales_dev, float global,
                    float *out_dev, size_t nblocks, size_t block_size, cudaStream_t s);
// ---- gemv.cu ----
// Flag words of a row-sharded decode product that signals its own completion (gllmk_gemv_exchange): the first
// GLLMK_PEER_FLAG_BYTES of every rank's exchange buffer, viewed as uint32_t[64].
//   [0, 8)   gllmk_peer_barrier: last sequence number signalled by each source rank      [16] its replay counter
//   [32, 40) exchange products:  epoch (= products completed) last signalled by each source rank
//   [48]     this rank's own epoch, advanced by the last block of each exchange product
constexpr int XF_FLAGS = 32, XF_EPOCH = 48;
struct Exchange {
    uint32_t *flags_local = nullptr;               // this rank's flag words; nullptr: no signalling
    uint32_t *flags_peer[GLLMK_MAX_PEERS] = {};    // the other ranks' flag words (peer-mapped), rank order
    int n_peers = 0, rank = 0;
};
int32_t gemv_launch(Ctx *c, const Weight *w, const float *x, int64_t xst, int64_t xsk, int m, float *y, int64_t yst,
                    int64_t ysr, const float *row_scales, int64_t n_row_scales, cudaStream_t s, void *const *y_peers = nullptr,
                    int n_peers = 0, const float *x_up = nullptr, const Exchange *xch = nullptr);
size_t gemv_ws_bytes(const Weight *w, int m);
// ---- gemm.cu ----
// a_up != nullptr: the activation matrix is silu(a) * a_up (same dtype / leading dimension), applied while staging
int32_t gemm_launch(Ctx *c, const Weight *w, const void *a, int a_bf16, int64_t lda, int m, void *y, int y_bf16, int64_t ldy,
                    cudaStream_t s, const void *a_up = nullptr);
int32_t gemm_grouped_launch(Ctx *c, const Weight *const *ws, int n_groups, const void *a, int a_bf16, int64_t lda,
                            const int64_t *row_offsets, void *y, int y_bf16, int64_t ldy, cudaStream_t s, const void *a_up = nullptr);
// ---- gemm_fp4.cu ----
int32_t gemm_fp4_launch(Ctx *c, const Weight *w, const Weight *x, void *y, int y_bf16, int64_t ldy, cudaStream_t s);
int32_t probe_fp4_mma(Ctx *c, int pair, int with_cp, int nv, int ksteps, float *tflops);
// ---- gemv_fp4.cu ----
int32_t gemv_fp4_launch(Ctx *c, const Weight *w, const float *x, int64_t xst, int64_t xsk, int m, float *y, int64_t yst, int64_t ysr,
                        cudaStream_t s);
// ---- gemm_i8.cu ----
int32_t i8_weight_fill(Ctx *c, Weight *w, const int8_t *b_dev, int layout, cudaStream_t s);
int32_t gemm_i8_launch(Ctx *c, const Weight *w, const uint8_t *a, int64_t lda, int m, int32_t *out, int64_t ldc, cudaStream_t s);
int32_t dequant_i32_launch(Ctx *c, const int32_t *ci, float *out, int64_t m, int64_t n, int64_t ldc, int64_t ldo, float scale_a,
                           float scale_b, const float *bias, int act, cudaStream_t s, const float *scale_a_dev = nullptr,
                           const int32_t *colsum = nullptr);
// f32 activations -> per-tensor int8 (stored as q + offset); scale_dev: two words of device memory, [0] receives the scale
int32_t act_quant_i8_launch(Ctx *c, const float *x, int64_t rows, int64_t k, int64_t ld, uint8_t *q, int64_t ldq, int offset,
                            float *scale_dev, cudaStream_t s);
// ---- gguf_raw.cu: Q6_K, Q5_K, Q8_K, Q4_0, Q5_0 kept as reference blocks (w->qs = n rows of nb block slots + 16 spare bytes) ----
bool raw_format(int32_t qt);
int raw_dev_block_bytes(int32_t qt);  // Q6_K: 224-byte slots; the others: the reference block size
int32_t raw_fill(Ctx *c, const Weight *w, const void *blocks_dev, cudaStream_t s);
int32_t raw_unfill(Ctx *c, const Weight *w, void *blocks_dev, cudaStream_t s);
int32_t raw_dequant(Ctx *c, int32_t qt, const uint8_t *w, int64_t n, int64_t nb, const int32_t *ids, size_t rows, float *out,
                    cudaStream_t s, bool dev_layout);
int32_t raw_gemv_launch(Ctx *c, const Weight *w, const float *x, int64_t xst, int64_t xsk, int m, float *y, int64_t yst,
                        int64_t ysr, const float *row_scales, int64_t n_row_scales, cudaStream_t s);
// ---- quantize.cu ----
int32_t quantize_launch(Ctx *c, int32_t qt, const float *x, int64_t rows, int64_t k, int mx_block, void *blocks,
                        void *scales, float *global_scale, cudaStream_t s);

// ---- FP4 plane addressing ----
// byte offset of byte `j` of row `row` in the tiled, swizzled data plane (k elements per row)
__host__ __device__ inline size_t fp4_data_offset(int64_t row, int64_t j, int64_t k) {
    const size_t tile = (size_t)(row >> 7) * (size_t)(k >> 8) + (size_t)(j >> 7);
    const int r = (int)(row & 127), c = (int)((j >> 4) & 7);
    return tile * 16384 + (size_t)r * 128 + (size_t)(((c ^ (r & 7)) << 4) + (int)(j & 15));
}
// byte offset of scale `s` of row `row` in the scale-factor plane (s_per_row scales per row)
__host__ __device__ inline size_t fp4_sf_offset(int64_t row, int64_t s, int64_t s_per_row) {
    const size_t atom = (size_t)(row >> 7) * (size_t)(s_per_row >> 2) + (size_t)(s >> 2);
    return atom * 512 + (size_t)(row & 31) * 16 + (size_t)((row & 127) >> 5) * 4 + (size_t)(s & 3);
}

// ---- small device helpers ----
__device__ __forceinline__ float e8m0_to_f32(uint32_t b) {
    // decode_e8m0_scale, src/quant_mxfp4.rs:43-54
    if (b == 255u) return __int_as_float(0x7FC00000);
    if (b == 0u) return __int_as_float(0x00400000);
    return __int_as_float((int)(b << 23));
}
__device__ __forceinline__ float e4m3_to_f32(uint32_t b) {
    // e4m3_to_f32, src/compiler/codegen/vm/numerical_sim.rs:2811-2835
    const uint32_t e = (b >> 3) & 0xFu, m = b & 7u;
    float a;
    if (e == 0u) a = (float)m * (1.0f / 512.0f);
    else if (e == 15u && m == 7u) return __int_as_float(0x7FC00000);
    else a = __int_as_float((int)(((e + 120u) << 23) | (m << 20)));
    return (b & 0x80u) ? -a : a;
}
__device__ __forceinline__ float e2m1_to_f32(uint32_t code) {
    // E2M1_LUT_F32, src/quant_mxfp4.rs:33-35: {0,.5,1,1.5,2,3,4,6} with the sign in bit 3
    const uint32_t mag = code & 7u;
    const uint32_t e = mag >> 1, m = mag & 1u;
    uint32_t bits = (e == 0u) ? (m ? 0x3F000000u : 0u) : (((e + 126u) << 23) | (m << 22));
    return __int_as_float((int)(bits | ((code & 8u) << 28)));
}

}  // namespace gllmk
