// Internal declarations shared by the translation units of libgllmk.so.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>

#include "../../include/gllmk.h"

namespace gllmk {

// ---- device layouts -------------------------------------------------------------------------
//
// Q4_K (256 el / 144 B), rows padded to a multiple of 16, T = row / 16, b = k-block:
//   qs  : uint4 [T][b][j = 0..3][lane = 0..31]   (2048 B per (T, b), one warp-wide 512 B run per j)
//         lane = 4*g + t holds, for row 16T + g + 8*(j >> 1), the 16 bytes qs[16*(2t + (j & 1)) ..]
//         i.e. thread t of quad g owns sub-block pair (2t, 2t+1) of rows g and g+8 — the
//         m16n8k16 A-fragment ownership, so unpacked nibbles land in fragment registers.
//   hdr : uint4 [T][b][16 rows]                  (d, dmin, scales[12] exactly as in the block)
//
// Q8_0 (32 el / 34 B), rows padded to 16, blocks padded to a multiple of 8 (nb8 groups):
//   qs  : uint4 [T][b][lane]                     lane = 4g+t: {row g bytes 8t..8t+7, row g+8 bytes 8t..8t+7}
//   d   : half  [T][b8][16 rows][8 blocks]       (f16 scale bits, 0 for padding)
//
// MXFP4 (block 32) and NVFP4 (block 64 = 4 x 16), rows padded to 128, k % 256 == 0:
//   data: uint8 [n_pad][k / 2]                   nibbles as in the reference (low nibble = even element),
//                                                a plain 2-D byte matrix a TMA tensor map can tile
//   sf   : uint8 [n_pad / 128][k / (4*sfb)][512] one scale byte per sfb = 32 (MXFP4, E8M0) or 16 (NVFP4,
//                                                UE4M3) elements, in 128-row x 4-scale atoms:
//                                                offset = (r % 32) * 16 + ((r % 128) / 32) * 4 + (s % 4)
//                                                (the tile order tcgen05 block-scaled MMA takes its
//                                                scale factors in)
struct Weight {
    int32_t qt = 0;
    int32_t mx_block = 0;
    int64_t n = 0, k = 0;
    int64_t n_pad = 0;
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
    // pinned host staging + device staging for the host-pointer entry points
    void *pin = nullptr;
    size_t pin_bytes = 0;
    void *dev_io = nullptr;
    size_t dev_io_bytes = 0;
    cudaStream_t stream = nullptr;  // the context's own stream for host-pointer entry points
    int64_t gemv_ksplit = 0;
    int64_t gemv_pdl = 1;
};

int32_t fail(Ctx *c, int32_t code, const char *fmt, ...);
int32_t cuda_fail(Ctx *c, cudaError_t e, const char *what);
int32_t ensure_ws(Ctx *c, size_t bytes);
int32_t ensure_pin(Ctx *c, size_t bytes);
int32_t ensure_dev_io(Ctx *c, size_t bytes);

#define GK_CUDA(c, call)                                             \
    do {                                                             \
        cudaError_t e__ = (call);                                    \
        if (e__ != cudaSuccess) return cuda_fail((c), e__, #call);   \
    } while (0)

// ---- repack.cu ----
int32_t repack_upload(Ctx *c, Weight *w, const void *blocks_dev, const void *scales_dev, cudaStream_t s);
int32_t repack_unpack(Ctx *c, const Weight *w, void *blocks_dev, void *scales_dev, cudaStream_t s);
int32_t dequant_matrix(Ctx *c, const Weight *w, float *out_dev, cudaStream_t s);
int32_t dequant_raw(Ctx *c, int32_t qt, const uint8_t *blocks_dev, const uint8_t *scales_dev, float global,
                    float *out_dev, size_t nblocks, size_t block_size, cudaStream_t s);
// ---- gemv.cu ----
int32_t gemv_launch(Ctx *c, const Weight *w, const float *x, int64_t xst, int64_t xsk, int m, float *y, int64_t yst,
                    int64_t ysr, const float *row_scales, int64_t n_row_scales, cudaStream_t s);
size_t gemv_ws_bytes(const Weight *w, int m);
// ---- quantize.cu ----
int32_t quantize_launch(Ctx *c, int32_t qt, const float *x, int64_t rows, int64_t k, int mx_block, void *blocks,
                        void *scales, float *global_scale, cudaStream_t s);

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
