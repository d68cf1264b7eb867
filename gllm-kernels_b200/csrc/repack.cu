// Weight repacker (reference block formats -> tiled device layouts, and back) and the
// bit-exact decode kernels.  Layouts are described in common.cuh.
#include "common.cuh"

namespace gllmk {

// The repack kernels move a Q4_K block's header (d, dmin, the 12 scale bytes) as its first 16-byte word and the
// block as nine such words, Q8_0's scale as the two bytes in front of its data, the FP4 scale bytes in front of
// theirs: what the format descriptors must say for those loads to be right.
static_assert(FD_Q4K.scale_offset == 0 && FD_Q4K.scale_min_offset == 2 && FD_Q4K.sub_scales_offset == 4 && FD_Q4K.data_offset == 16 &&
                  FD_Q4K.block_bytes == 144 && FD_Q4K.sub_scales_bits == 6 && FD_Q4K.data_low_first == 1,
              "Q4_K block layout");
static_assert(FD_Q8_0.scale_offset == 0 && FD_Q8_0.data_offset == 2 && FD_Q8_0.block_bytes == 34 && FD_Q8_0.data_signed == 1, "Q8_0 block layout");
static_assert(FD_MXFP4.scale_offset == 0 && FD_MXFP4.data_offset == 1 && FD_MXFP4.block_bytes == 17, "MXFP4 inline block layout");
static_assert(FD_NVFP4.sub_scales_offset == 0 && FD_NVFP4.sub_scales_count == 4 && FD_NVFP4.data_offset == 4 && FD_NVFP4.block_bytes == 36,
              "NVFP4 block layout");

static inline unsigned grid_for(size_t n, unsigned block) { return (unsigned)((n + block - 1) / block); }

// ================================ Q4_K =====================================================
// chunk (T, b) = 2368 bytes, layout in common.cuh.
__device__ __forceinline__ void q4k_fields(const uint8_t *s, uint32_t *sc, uint32_t *mn) {
    // get_scale_min_k4, src/macros/quant_primitive/k_quant.rs:13-23
#pragma unroll
    for (int j = 0; j < 8; j++) {
        if (j < 4) { sc[j] = s[j] & 63u; mn[j] = s[j + 4] & 63u; }
        else {
            sc[j] = (s[j + 4] & 0xFu) | ((uint32_t)(s[j - 4] >> 6) << 4);
            mn[j] = (uint32_t)(s[j + 4] >> 4) | ((uint32_t)(s[j] >> 6) << 4);
        }
    }
}
// thread = one uint4 of the nibble area: (T, b, p, lane)
__global__ void repack_q4k_qs(const uint8_t *__restrict__ src, uint8_t *__restrict__ chunks, int64_t n, int64_t nb,
                              size_t total) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int lane = (int)(idx & 31), pgrp = (int)((idx >> 5) & 3);
    const size_t tb = idx >> 7;  // T*nb + b
    const int64_t T = (int64_t)(tb / (size_t)nb), b = (int64_t)(tb % (size_t)nb);
    const int g = lane >> 2, t = lane & 3;
    uint32_t v[4] = {0, 0, 0, 0};
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int64_t row = 16 * T + g + 8 * h;
        if (row < n) {
            const uint2 w = *reinterpret_cast<const uint2 *>(src + ((size_t)row * nb + b) * FD_Q4K.block_bytes + FD_Q4K.data_offset + 32 * pgrp + 8 * t);
            v[2 * h] = w.x;
            v[2 * h + 1] = w.y;
        }
    }
    reinterpret_cast<uint4 *>(chunks + q4k_chunk_index(T, b, nb) * Q4K_CHUNK)[pgrp * 32 + lane] =
        make_uint4(v[0], v[1], v[2], v[3]);
}
__global__ void repack_q4k_hdr(const uint8_t *__restrict__ src, uint8_t *__restrict__ chunks, int64_t n, int64_t nb,
                               size_t total) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // (T*nb + b)*16 + rr
    if (idx >= total) return;
    const int rr = (int)(idx & 15);
    const size_t tb = idx >> 4;
    const int64_t T = (int64_t)(tb / (size_t)nb), b = (int64_t)(tb % (size_t)nb);
    const int64_t row = 16 * T + rr;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < n) v = reinterpret_cast<const uint4 *>(src + ((size_t)row * nb + b) * FD_Q4K.block_bytes)[0];
    uint8_t s[12];
    *reinterpret_cast<uint32_t *>(s) = v.y;
    *reinterpret_cast<uint32_t *>(s + 4) = v.z;
    *reinterpret_cast<uint32_t *>(s + 8) = v.w;
    uint32_t sc[8], mn[8];
    q4k_fields(s, sc, mn);
    uint8_t *chunk = chunks + q4k_chunk_index(T, b, nb) * Q4K_CHUNK;
    reinterpret_cast<uint4 *>(chunk + 2048)[rr] =
        make_uint4(sc[0] | (sc[1] << 8) | (sc[2] << 16) | (sc[3] << 24), sc[4] | (sc[5] << 8) | (sc[6] << 16) | (sc[7] << 24),
                   mn[0] | (mn[1] << 8) | (mn[2] << 16) | (mn[3] << 24), mn[4] | (mn[5] << 8) | (mn[6] << 16) | (mn[7] << 24));
    reinterpret_cast<uint32_t *>(chunk + 2304)[(rr & 7) * 2 + (rr >> 3)] = v.x;
}
// reads back 32-bit word `wi` (0..31) of the nibble bytes of (row, b)
__device__ __forceinline__ uint32_t q4k_word(const uint8_t *chunk, int rr, int wi) {
    const int pgrp = wi >> 3, i = wi & 7, t = i >> 1, lane = 4 * (rr & 7) + t;
    const uint4 q = reinterpret_cast<const uint4 *>(chunk)[pgrp * 32 + lane];
    const int sel = 2 * (rr >> 3) + (i & 1);
    return sel == 0 ? q.x : (sel == 1 ? q.y : (sel == 2 ? q.z : q.w));
}
__global__ void unpack_q4k(const uint8_t *__restrict__ chunks, uint8_t *__restrict__ dst, int64_t n, int64_t nb,
                           size_t total) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // (row*nb + b)*9 + u9
    if (idx >= total) return;
    const int u9 = (int)(idx % 9);
    const size_t rb = idx / 9;
    const int64_t row = (int64_t)(rb / (size_t)nb), b = (int64_t)(rb % (size_t)nb);
    const int64_t T = row >> 4;
    const int rr = (int)(row & 15);
    const uint8_t *chunk = chunks + q4k_chunk_index(T, b, nb) * Q4K_CHUNK;
    uint4 v;
    if (u9 == 0) {
        const uint4 h = reinterpret_cast<const uint4 *>(chunk + 2048)[rr];
        uint32_t sc[8], mn[8];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            sc[j] = (h.x >> (8 * j)) & 0xFF; sc[j + 4] = (h.y >> (8 * j)) & 0xFF;
            mn[j] = (h.z >> (8 * j)) & 0xFF; mn[j + 4] = (h.w >> (8 * j)) & 0xFF;
        }
        uint8_t s[12];
#pragma unroll
        for (int j = 0; j < 4; j++) {  // inverse of get_scale_min_k4
            s[j] = (uint8_t)(sc[j] | ((sc[j + 4] >> 4) << 6));
            s[j + 4] = (uint8_t)(mn[j] | ((mn[j + 4] >> 4) << 6));
            s[j + 8] = (uint8_t)((sc[j + 4] & 15) | ((mn[j + 4] & 15) << 4));
        }
        v.x = reinterpret_cast<const uint32_t *>(chunk + 2304)[(rr & 7) * 2 + (rr >> 3)];
        v.y = *reinterpret_cast<uint32_t *>(s);
        v.z = *reinterpret_cast<uint32_t *>(s + 4);
        v.w = *reinterpret_cast<uint32_t *>(s + 8);
    } else {
        const int w0 = 4 * (u9 - 1);
        v = make_uint4(q4k_word(chunk, rr, w0), q4k_word(chunk, rr, w0 + 1), q4k_word(chunk, rr, w0 + 2),
                       q4k_word(chunk, rr, w0 + 3));
    }
    reinterpret_cast<uint4 *>(dst + rb * FD_Q4K.block_bytes)[u9] = v;
    (void)n;
}
// out[row][256b + ...] following k_quant.rs:7-56; thread = one 32-bit word of qs (4 low + 4 high outputs)
// `ids` (optional): output row r decodes weight row ids[r] (embedding gather); rows outside [0, n) decode to zeros
__global__ void dequant_q4k(const uint8_t *__restrict__ chunks, float *__restrict__ out, int64_t n, int64_t nb,
                            size_t total, const int32_t *__restrict__ ids) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // (row*nb + b)*32 + w, w = word 0..31 of qs
    if (idx >= total) return;
    const int wq = (int)(idx & 31);
    const size_t rb = idx >> 5;
    int64_t row = (int64_t)(rb / (size_t)nb);
    const int64_t b = (int64_t)(rb % (size_t)nb);
    if (ids) {
        row = ids[row];
        if (row < 0 || row >= n) {
            float *z = out + rb * 256 + 64 * (wq >> 3) + 4 * (wq & 7);
            *reinterpret_cast<float4 *>(z) = make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4 *>(z + 32) = make_float4(0.f, 0.f, 0.f, 0.f);
            return;
        }
    }
    const int64_t T = row >> 4;
    const int rr = (int)(row & 15);
    const uint8_t *chunk = chunks + q4k_chunk_index(T, b, nb) * Q4K_CHUNK;
    const uint32_t w = q4k_word(chunk, rr, wq);
    const int group = wq >> 3;  // 32 bytes per group = sub-block pair (2*group, 2*group + 1)
    const uint4 h = reinterpret_cast<const uint4 *>(chunk + 2048)[rr];
    const uint32_t scw = group < 2 ? h.x : h.y, mnw = group < 2 ? h.z : h.w;
    const int sh = 16 * (group & 1);
    const uint32_t dd = reinterpret_cast<const uint32_t *>(chunk + 2304)[(rr & 7) * 2 + (rr >> 3)];
    const float d = __half2float(__ushort_as_half((unsigned short)(dd & 0xFFFF)));
    const float dmin = __half2float(__ushort_as_half((unsigned short)(dd >> 16)));
    const float d1 = __fmul_rn(d, (float)((scw >> sh) & 0xFF)), nm1 = __fmul_rn(dmin, (float)((mnw >> sh) & 0xFF));
    const float d2 = __fmul_rn(d, (float)((scw >> (sh + 8)) & 0xFF)), nm2 = __fmul_rn(dmin, (float)((mnw >> (sh + 8)) & 0xFF));
    const int l = 4 * (wq & 7);
    float4 lo, hi;
    lo.x = __fsub_rn(__fmul_rn(d1, (float)(w & 15u)), nm1);
    lo.y = __fsub_rn(__fmul_rn(d1, (float)((w >> 8) & 15u)), nm1);
    lo.z = __fsub_rn(__fmul_rn(d1, (float)((w >> 16) & 15u)), nm1);
    lo.w = __fsub_rn(__fmul_rn(d1, (float)((w >> 24) & 15u)), nm1);
    hi.x = __fsub_rn(__fmul_rn(d2, (float)((w >> 4) & 15u)), nm2);
    hi.y = __fsub_rn(__fmul_rn(d2, (float)((w >> 12) & 15u)), nm2);
    hi.z = __fsub_rn(__fmul_rn(d2, (float)((w >> 20) & 15u)), nm2);
    hi.w = __fsub_rn(__fmul_rn(d2, (float)((w >> 28) & 15u)), nm2);
    float *o = out + rb * 256 + 64 * group + l;
    *reinterpret_cast<float4 *>(o) = lo;
    *reinterpret_cast<float4 *>(o + 32) = hi;
    (void)n;
}

// ================================ Q8_0 =====================================================
// chunk (T, b8) = 4352 bytes: 8 blocks x 512 bytes of int8 in fragment order + 16 rows x 8 f16 scales.
// thread = one uint4 of the int8 area: (T, b8, bb, lane)
__global__ void repack_q80_qs(const uint8_t *__restrict__ src, uint8_t *__restrict__ chunks, int64_t n, int64_t nb,
                              int64_t nb8, size_t total) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // ((T*nb8 + b8)*8 + bb)*32 + lane
    if (idx >= total) return;
    const int lane = (int)(idx & 31), bb = (int)((idx >> 5) & 7);
    const size_t tb = idx >> 8;
    const int64_t T = (int64_t)(tb / (size_t)nb8), b8 = (int64_t)(tb % (size_t)nb8);
    const int64_t b = 8 * b8 + bb;
    const int g = lane >> 2, t = lane & 3;
    uint32_t v[4] = {0, 0, 0, 0};
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const int64_t row = 16 * T + g + 8 * h;
        if (row < n && b < nb) {
            const unsigned short *p =
                reinterpret_cast<const unsigned short *>(src + ((size_t)row * nb + b) * FD_Q8_0.block_bytes + FD_Q8_0.data_offset + 8 * t);
            v[2 * h] = (uint32_t)p[0] | ((uint32_t)p[1] << 16);
            v[2 * h + 1] = (uint32_t)p[2] | ((uint32_t)p[3] << 16);
        }
    }
    reinterpret_cast<uint4 *>(chunks + q4k_chunk_index(T, b8, nb8) * Q80_CHUNK)[bb * 32 + lane] =
        make_uint4(v[0], v[1], v[2], v[3]);
}
__global__ void repack_q80_d(const uint8_t *__restrict__ src, uint8_t *__restrict__ chunks, int64_t n, int64_t nb,
                             int64_t nb8, size_t total) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // ((T*nb8 + b8)*16 + rr)*8 + bb
    if (idx >= total) return;
    const int bb = (int)(idx & 7), rr = (int)((idx >> 3) & 15);
    const size_t tb = idx >> 7;
    const int64_t T = (int64_t)(tb / (size_t)nb8), b8 = (int64_t)(tb % (size_t)nb8);
    const int64_t row = 16 * T + rr, b = 8 * b8 + bb;
    unsigned short v = 0;
    if (row < n && b < nb) v = *reinterpret_cast<const unsigned short *>(src + ((size_t)row * nb + b) * FD_Q8_0.block_bytes + FD_Q8_0.scale_offset);
    reinterpret_cast<unsigned short *>(chunks + q4k_chunk_index(T, b8, nb8) * Q80_CHUNK + 4096)[rr * 8 + bb] = v;
}
__global__ void unpack_q80(const uint8_t *__restrict__ chunks, uint8_t *__restrict__ dst, int64_t n, int64_t nb,
                           int64_t nb8, size_t total) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // (row*nb + b)*4 + t
    if (idx >= total) return;
    const int t = (int)(idx & 3);
    const size_t rb = idx >> 2;
    const int64_t row = (int64_t)(rb / (size_t)nb), b = (int64_t)(rb % (size_t)nb);
    const int64_t T = row >> 4;
    const int rr = (int)(row & 15), g = rr & 7, h = rr >> 3;
    const uint8_t *chunk = chunks + q4k_chunk_index(T, b >> 3, nb8) * Q80_CHUNK;
    const uint4 q = reinterpret_cast<const uint4 *>(chunk)[(b & 7) * 32 + 4 * g + t];
    const uint32_t w0 = h ? q.z : q.x, w1 = h ? q.w : q.y;
    unsigned short *p = reinterpret_cast<unsigned short *>(dst + rb * FD_Q8_0.block_bytes + FD_Q8_0.data_offset + 8 * t);
    p[0] = (unsigned short)(w0 & 0xFFFF); p[1] = (unsigned short)(w0 >> 16);
    p[2] = (unsigned short)(w1 & 0xFFFF); p[3] = (unsigned short)(w1 >> 16);
    if (t == 0)
        *reinterpret_cast<unsigned short *>(dst + rb * FD_Q8_0.block_bytes + FD_Q8_0.scale_offset) =
            reinterpret_cast<const unsigned short *>(chunk + 4096)[rr * 8 + (b & 7)];
    (void)n;
}
// classic.rs:860-868: out = d * q; thread = 8 elements
__global__ void dequant_q80(const uint8_t *__restrict__ chunks, float *__restrict__ out, int64_t n, int64_t nb,
                            int64_t nb8, size_t total, const int32_t *__restrict__ ids) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // (row*nb + b)*4 + t
    if (idx >= total) return;
    const int t = (int)(idx & 3);
    const size_t rb = idx >> 2;
    int64_t row = (int64_t)(rb / (size_t)nb);
    const int64_t b = (int64_t)(rb % (size_t)nb);
    if (ids) {
        row = ids[row];
        if (row < 0 || row >= n) {
            float *z = out + rb * 32 + 8 * t;
            *reinterpret_cast<float4 *>(z) = make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4 *>(z + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
            return;
        }
    }
    const int64_t T = row >> 4;
    const int rr = (int)(row & 15), g = rr & 7, h = rr >> 3;
    const uint8_t *chunk = chunks + q4k_chunk_index(T, b >> 3, nb8) * Q80_CHUNK;
    const uint4 q = reinterpret_cast<const uint4 *>(chunk)[(b & 7) * 32 + 4 * g + t];
    const uint32_t w0 = h ? q.z : q.x, w1 = h ? q.w : q.y;
    const float dv = __half2float(__ushort_as_half(reinterpret_cast<const unsigned short *>(chunk + 4096)[rr * 8 + (b & 7)]));
    float4 a, c;
    a.x = __fmul_rn(dv, (float)(int8_t)(w0 & 0xFF)); a.y = __fmul_rn(dv, (float)(int8_t)((w0 >> 8) & 0xFF));
    a.z = __fmul_rn(dv, (float)(int8_t)((w0 >> 16) & 0xFF)); a.w = __fmul_rn(dv, (float)(int8_t)(w0 >> 24));
    c.x = __fmul_rn(dv, (float)(int8_t)(w1 & 0xFF)); c.y = __fmul_rn(dv, (float)(int8_t)((w1 >> 8) & 0xFF));
    c.z = __fmul_rn(dv, (float)(int8_t)((w1 >> 16) & 0xFF)); c.w = __fmul_rn(dv, (float)(int8_t)(w1 >> 24));
    float *o = out + rb * 32 + 8 * t;
    *reinterpret_cast<float4 *>(o) = a;
    *reinterpret_cast<float4 *>(o + 4) = c;
    (void)n;
}

// ================================ MXFP4 / NVFP4 ============================================
__device__ __forceinline__ size_t sf_offset(int64_t row, int64_t s, int64_t s_per_row) { return fp4_sf_offset(row, s, s_per_row); }
// mode 0: MXFP4 split (blocks [n][k/2], scales [n][k/32]); mode 1: MXFP4 inline 17-byte blocks;
// mode 2: NVFP4 36-byte blocks.  Thread = 4 data bytes (8 elements).
__global__ void repack_fp4_data(const uint8_t *__restrict__ blocks, uint32_t *__restrict__ data, int64_t n,
                                int64_t k, int64_t k_pad, int mode, size_t total) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // row_pad * (k_pad/8) + w
    if (idx >= total) return;
    const int64_t wpr = k_pad >> 3;
    const int64_t row = (int64_t)(idx / (size_t)wpr), w = (int64_t)(idx % (size_t)wpr);
    uint32_t v = 0;
    if (row < n && w < (k >> 3)) {
        const uint8_t *p;
        if (mode == 0) p = blocks + (size_t)row * (k >> 1) + 4 * w;
        else if (mode == 1) p = blocks + ((size_t)row * (k >> 5) + (w >> 2)) * FD_MXFP4.block_bytes + FD_MXFP4.data_offset + 4 * (w & 3);
        else p = blocks + ((size_t)row * (k >> 6) + (w >> 3)) * FD_NVFP4.block_bytes + FD_NVFP4.data_offset + 4 * (w & 7);
        v = (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
    }
    data[fp4_data_offset(row, 4 * w, k_pad) >> 2] = v;
}
__global__ void repack_fp4_sf(const uint8_t *__restrict__ blocks, const uint8_t *__restrict__ scales,
                              uint8_t *__restrict__ sf, int64_t n, int64_t k, int64_t k_pad, int mode, size_t total) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // row_pad * padded s_per_row + s
    if (idx >= total) return;
    const int64_t spr = (mode == 2) ? (k >> 4) : (k >> 5), spr_pad = (mode == 2) ? (k_pad >> 4) : (k_pad >> 5);
    const int64_t row = (int64_t)(idx / (size_t)spr_pad), s = (int64_t)(idx % (size_t)spr_pad);
    uint8_t v = 0;
    if (row < n && s < spr) {
        if (mode == 0) v = scales[(size_t)row * spr + s];
        else if (mode == 1) v = blocks[((size_t)row * spr + s) * FD_MXFP4.block_bytes + FD_MXFP4.scale_offset];
        else v = blocks[((size_t)row * (k >> 6) + (s >> 2)) * FD_NVFP4.block_bytes + FD_NVFP4.sub_scales_offset + (s & 3)];
    }
    sf[sf_offset(row, s, spr_pad)] = v;
}
__global__ void unpack_fp4(const uint8_t *__restrict__ data, const uint8_t *__restrict__ sf, uint8_t *__restrict__ blocks,
                           uint8_t *__restrict__ scales, int64_t n, int64_t k, int64_t k_pad, int nv, size_t total) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // row * (k/2) + byte
    if (idx >= total) return;
    const int64_t bpr = k >> 1;
    const int64_t row = (int64_t)(idx / (size_t)bpr), by = (int64_t)(idx % (size_t)bpr);
    const uint8_t v = data[fp4_data_offset(row, by, k_pad)];
    if (!nv) {
        blocks[idx] = v;
        if ((by & 15) == 0) scales[(size_t)row * (k >> 5) + (by >> 4)] = sf[sf_offset(row, by >> 4, k_pad >> 5)];
    } else {
        uint8_t *blk = blocks + ((size_t)row * (k >> 6) + (by >> 5)) * FD_NVFP4.block_bytes;
        blk[4 + (by & 31)] = v;
        if ((by & 7) == 0) blk[(by & 31) >> 3] = sf[sf_offset(row, by >> 3, k_pad >> 4)];
    }
    (void)n;
}
// thread = 4 data bytes -> 8 f32.  MXFP4: LUT[code] * e8m0 (quant_mxfp4.rs:95-108);
// NVFP4: (global * e4m3(sub)) * LUT[code] (quant.rs:77-86).
__global__ void dequant_fp4(const uint32_t *__restrict__ data, const uint8_t *__restrict__ sf, float *__restrict__ out,
                            int64_t n, int64_t k, int64_t k_pad, int nv, float global, size_t total,
                            const int32_t *__restrict__ ids) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // row * (k/8) + w
    if (idx >= total) return;
    const int64_t wpr = k >> 3;
    const int64_t orow = (int64_t)(idx / (size_t)wpr), w = (int64_t)(idx % (size_t)wpr);
    int64_t row = orow;
    if (ids) {
        row = ids[orow];
        if (row < 0 || row >= n) {
            float *z = out + (size_t)orow * k + 8 * w;
            *reinterpret_cast<float4 *>(z) = make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4 *>(z + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
            return;
        }
    }
    const uint32_t v = data[fp4_data_offset(row, 4 * w, k_pad) >> 2];
    float s;
    if (!nv) s = e8m0_to_f32(sf[sf_offset(row, w >> 2, k_pad >> 5)]);
    else s = __fmul_rn(global, e4m3_to_f32(sf[sf_offset(row, w >> 1, k_pad >> 4)]));
    float r[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float c = e2m1_to_f32((v >> (4 * i)) & 15u);
        r[i] = nv ? __fmul_rn(s, c) : __fmul_rn(c, s);
    }
    float *o = out + (size_t)orow * k + 8 * w;
    *reinterpret_cast<float4 *>(o) = make_float4(r[0], r[1], r[2], r[3]);
    *reinterpret_cast<float4 *>(o + 4) = make_float4(r[4], r[5], r[6], r[7]);
    (void)n;
}

// ================================ raw-block decode (host-pointer drop-ins) ===================
__global__ void dequant_raw_kernel(int qt, const uint8_t *__restrict__ blocks, const uint8_t *__restrict__ scales,
                                   float global, float *__restrict__ out, size_t bs, size_t total) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // output element
    if (idx >= total) return;
    const size_t blk = idx / bs;
    const int e = (int)(idx % bs);
    float r;
    if (qt == GLLMK_QUANT_Q4K) {
        const uint8_t *b = blocks + blk * FD_Q4K.block_bytes;
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(b)));
        const float dmin = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(b + FD_Q4K.scale_min_offset)));
        const uint8_t *s = b + FD_Q4K.sub_scales_offset;
        const int mini = e >> 5, l = e & 31, g = mini >> 1;
        const uint8_t byte = b[FD_Q4K.data_offset + 32 * g + l];
        const float q = (float)((mini & 1) ? (byte >> 4) : (byte & 15));
        float sc, m;
        if (mini < 4) { sc = (float)(s[mini] & 63); m = (float)(s[mini + 4] & 63); }
        else {
            sc = (float)((s[mini + 4] & 0xF) | ((s[mini - 4] >> 6) << 4));
            m = (float)((s[mini + 4] >> 4) | ((s[mini] >> 6) << 4));
        }
        r = __fsub_rn(__fmul_rn(__fmul_rn(d, sc), q), __fmul_rn(dmin, m));
    } else if (qt == GLLMK_QUANT_Q8_0) {
        const uint8_t *b = blocks + blk * FD_Q8_0.block_bytes;
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(b)));
        r = __fmul_rn(d, (float)(int8_t)b[FD_Q8_0.data_offset + e]);
    } else if (qt == GLLMK_QUANT_MXFP4) {
        const uint8_t byte = blocks[blk * (bs / 2) + (e >> 1)];
        r = __fmul_rn(e2m1_to_f32((e & 1) ? (byte >> 4) : (byte & 15)), e8m0_to_f32(scales[blk]));
    } else {
        const uint8_t *b = blocks + blk * FD_NVFP4.block_bytes;
        const uint8_t byte = b[FD_NVFP4.data_offset + (e >> 1)];
        const float s = __fmul_rn(global, e4m3_to_f32(b[e >> 4]));
        r = __fmul_rn(s, e2m1_to_f32((e & 1) ? (byte >> 4) : (byte & 15)));
    }
    out[idx] = r;
}

// ================================ host side ================================================
int32_t repack_upload(Ctx *c, Weight *w, const void *blocks, const void *scales, cudaStream_t s) {
    const uint8_t *src = static_cast<const uint8_t *>(blocks);
    if (raw_format(w->qt)) return raw_fill(c, w, src, s);  // stored as the reference stores it
    if (w->qt == GLLMK_QUANT_Q4K) {
        // n_pad is a multiple of 128: tiles beyond n are written as zero chunks
        const size_t tq = (size_t)(w->n_pad / 16) * w->nb * 128, th = (size_t)(w->n_pad / 16) * w->nb * 16;
        repack_q4k_qs<<<grid_for(tq, 256), 256, 0, s>>>(src, (uint8_t *)w->qs, w->n, w->nb, tq);
        repack_q4k_hdr<<<grid_for(th, 256), 256, 0, s>>>(src, (uint8_t *)w->qs, w->n, w->nb, th);
    } else if (w->qt == GLLMK_QUANT_Q8_0) {
        const size_t tq = (size_t)(w->n_pad / 16) * w->nb8 * 256, td = (size_t)(w->n_pad / 16) * w->nb8 * 128;
        repack_q80_qs<<<grid_for(tq, 256), 256, 0, s>>>(src, (uint8_t *)w->qs, w->n, w->nb, w->nb8, tq);
        repack_q80_d<<<grid_for(td, 256), 256, 0, s>>>(src, (uint8_t *)w->qs, w->n, w->nb, w->nb8, td);
    } else {
        const int mode = (w->qt == GLLMK_QUANT_NVFP4) ? 2 : (scales ? 0 : 1);
        const int64_t spr = (mode == 2) ? (w->k_pad >> 4) : (w->k_pad >> 5);
        const size_t td = (size_t)w->n_pad * (w->k_pad >> 3), ts = (size_t)w->n_pad * spr;
        repack_fp4_data<<<grid_for(td, 256), 256, 0, s>>>(src, (uint32_t *)w->qs, w->n, w->k, w->k_pad, mode, td);
        repack_fp4_sf<<<grid_for(ts, 256), 256, 0, s>>>(src, (const uint8_t *)scales, (uint8_t *)w->aux, w->n, w->k,
                                                        w->k_pad, mode, ts);
    }
    GK_CUDA(c, cudaGetLastError());
    return GLLMK_STATUS_OK;
}

int32_t repack_unpack(Ctx *c, const Weight *w, void *blocks, void *scales, cudaStream_t s) {
    uint8_t *dst = static_cast<uint8_t *>(blocks);
    if (raw_format(w->qt)) return raw_unfill(c, w, dst, s);
    if (w->qt == GLLMK_QUANT_Q4K) {
        const size_t t = (size_t)w->n * w->nb * 9;
        unpack_q4k<<<grid_for(t, 256), 256, 0, s>>>((const uint8_t *)w->qs, dst, w->n, w->nb, t);
    } else if (w->qt == GLLMK_QUANT_Q8_0) {
        const size_t t = (size_t)w->n * w->nb * 4;
        unpack_q80<<<grid_for(t, 256), 256, 0, s>>>((const uint8_t *)w->qs, dst, w->n, w->nb, w->nb8, t);
    } else {
        const size_t t = (size_t)w->n * (w->k >> 1);
        unpack_fp4<<<grid_for(t, 256), 256, 0, s>>>((const uint8_t *)w->qs, (const uint8_t *)w->aux, dst,
                                                    (uint8_t *)scales, w->n, w->k, w->k_pad, w->qt == GLLMK_QUANT_NVFP4, t);
    }
    GK_CUDA(c, cudaGetLastError());
    return GLLMK_STATUS_OK;
}

int32_t dequant_matrix(Ctx *c, const Weight *w, float *out, cudaStream_t s, const int32_t *ids, int64_t count) {
    const size_t rows = ids ? (size_t)count : (size_t)w->n;  // with ids: out [count, k], row r = weight row ids[r]
    if (rows == 0) return GLLMK_STATUS_OK;
    if (raw_format(w->qt)) return raw_dequant(c, w->qt, static_cast<const uint8_t *>(w->qs), w->n, w->nb, ids, rows, out, s, true);
    if (w->qt == GLLMK_QUANT_Q4K) {
        const size_t t = rows * w->nb * 32;
        dequant_q4k<<<grid_for(t, 256), 256, 0, s>>>((const uint8_t *)w->qs, out, w->n, w->nb, t, ids);
    } else if (w->qt == GLLMK_QUANT_Q8_0) {
        const size_t t = rows * w->nb * 4;
        dequant_q80<<<grid_for(t, 256), 256, 0, s>>>((const uint8_t *)w->qs, out, w->n, w->nb, w->nb8, t, ids);
    } else {
        const size_t t = rows * (w->k >> 3);
        dequant_fp4<<<grid_for(t, 256), 256, 0, s>>>((const uint32_t *)w->qs, (const uint8_t *)w->aux, out, w->n, w->k,
                                                     w->k_pad, w->qt == GLLMK_QUANT_NVFP4, w->global_scale, t, ids);
    }
    GK_CUDA(c, cudaGetLastError());
    return GLLMK_STATUS_OK;
}

int32_t dequant_raw(Ctx *c, int32_t qt, const uint8_t *blocks, const uint8_t *scales, float global, float *out,
                    size_t nblocks, size_t block_size, cudaStream_t s) {
    const size_t total = nblocks * block_size;
    if (total == 0) return GLLMK_STATUS_OK;
    if (raw_format(qt)) return raw_dequant(c, qt, blocks, (int64_t)nblocks, 1, nullptr, nblocks, out, s, false);
    dequant_raw_kernel<<<grid_for(total, 256), 256, 0, s>>>(qt, blocks, scales, global, out, block_size, total);
    GK_CUDA(c, cudaGetLastError());
    return GLLMK_STATUS_OK;
}

}  // namespace gllmk
