// The other GGUF block formats of the reference's CPU quant path — Q6_K, Q5_K, Q8_K (256 elements per block) and
// Q4_0, Q5_0 (32 elements per block) — kept on the device as the reference stores them, row after row of blocks
// (Q6_K blocks, 210 bytes, sit in 224-byte slots so that every block starts on a 16-byte boundary).
//
// Decode: one rule per format (an "item" = the elements one data byte, or byte group, yields) with the reference's
// operation order (separately rounded products, no fused multiply-add): matrix decode, embedding gather and the
// host drop-ins are bit-exact.
//
// GEMV: a warp owns two weight rows, streams them through two shared-memory stages with cp.async and accumulates
// integer dot products (dp2a) against s16 fixed-point activations (16 bits per 32-element group, error ~1.5e-5
// of the group maximum, far inside the 2e-3 bar of the decode path).
//
// Reference: src/macros/quant_primitive/k_quant.rs:92-101 (Q8_K), :381-436 (Q5_K), :441-472 (Q6_K);
//            src/macros/quant_primitive/classic.rs:15-29 (Q4_0), :484-504 (Q5_0); block structs src/quant.rs:132-157, 254-275.
#include "common.cuh"

namespace gllmk {

namespace {

__device__ __forceinline__ float f16_at(const uint8_t *p) {
    return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8))));
}

// get_scale_min_k4 of the K-quants (k_quant.rs:388-397): sub-block j's 6-bit scale and min
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t *s, float &sc, float &m) {
    if (j < 4) {
        sc = (float)(s[j] & 63);
        m = (float)(s[j + 4] & 63);
    } else {
        sc = (float)((s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4));
        m = (float)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

// Per format: BS elements and BB bytes per block, ITEMS work items per block, EPI elements per item.
// item(b, it, v, e): decodes item `it` of the block at b into values v[] of elements e[] (indices in the block).
template <int QT>
struct Fmt;

template <>
struct Fmt<GLLMK_QUANT_Q6_K> {  // ql[128] @0, qh[64] @128, scales[16] i8 @192, d f16 @208
    static constexpr int BS = FD_Q6K.block_size, BB = FD_Q6K.block_bytes, DB = 224, ITEMS = 64, EPI = 4;  // DB: bytes per block slot on the device
    static __device__ __forceinline__ void item(const uint8_t *b, int it, float *v, int *e) {
        const int g = it >> 5, l = it & 31, is = l >> 4;
        const uint8_t la = b[FD_Q6K.data_offset + g * 64 + l], lb = b[FD_Q6K.data_offset + g * 64 + l + 32], h = b[FD_Q6K.data_high_offset + g * 32 + l];
        const int8_t *sc = reinterpret_cast<const int8_t *>(b + FD_Q6K.sub_scales_offset + g * 8);
        const float d = f16_at(b + FD_Q6K.scale_offset);
        const int q1 = (int)((la & 0xF) | (((h >> 0) & 3) << 4)) - FD_Q6K.static_bias;
        const int q2 = (int)((lb & 0xF) | (((h >> 2) & 3) << 4)) - FD_Q6K.static_bias;
        const int q3 = (int)((la >> 4) | (((h >> 4) & 3) << 4)) - FD_Q6K.static_bias;
        const int q4 = (int)((lb >> 4) | (((h >> 6) & 3) << 4)) - FD_Q6K.static_bias;
        v[0] = __fmul_rn(__fmul_rn(d, (float)sc[is]), (float)q1);
        v[1] = __fmul_rn(__fmul_rn(d, (float)sc[is + 2]), (float)q2);
        v[2] = __fmul_rn(__fmul_rn(d, (float)sc[is + 4]), (float)q3);
        v[3] = __fmul_rn(__fmul_rn(d, (float)sc[is + 6]), (float)q4);
        e[0] = g * 128 + l;
        e[1] = e[0] + 32;
        e[2] = e[0] + 64;
        e[3] = e[0] + 96;
    }
};

template <>
struct Fmt<GLLMK_QUANT_Q5_K> {  // d @0, dmin @2, scales[12] @4, qh[32] @16, qs[128] @48
    static constexpr int BS = FD_Q5K.block_size, BB = FD_Q5K.block_bytes, DB = 176, ITEMS = 128, EPI = 2;
    static __device__ __forceinline__ void item(const uint8_t *b, int it, float *v, int *e) {
        const int g = it >> 5, l = it & 31;
        const float d = f16_at(b + FD_Q5K.scale_offset), mn = f16_at(b + FD_Q5K.scale_min_offset);
        float sc1, m1, sc2, m2;
        scale_min_k4(2 * g, b + FD_Q5K.sub_scales_offset, sc1, m1);
        scale_min_k4(2 * g + 1, b + FD_Q5K.sub_scales_offset, sc2, m2);
        const uint8_t q = b[FD_Q5K.data_offset + g * 32 + l], h = b[FD_Q5K.data_high_offset + l];
        const int v1 = (q & 0xF) + (((h >> (2 * g)) & 1) ? 16 : 0);
        const int v2 = (q >> 4) + (((h >> (2 * g + 1)) & 1) ? 16 : 0);
        v[0] = __fsub_rn(__fmul_rn(__fmul_rn(d, sc1), (float)v1), __fmul_rn(mn, m1));
        v[1] = __fsub_rn(__fmul_rn(__fmul_rn(d, sc2), (float)v2), __fmul_rn(mn, m2));
        e[0] = g * 64 + l;
        e[1] = e[0] + 32;
    }
};

template <>
struct Fmt<GLLMK_QUANT_Q8_K> {  // d f32 @0, qs[256] i8 @4, bsums[16] i16 @260 (not used by decode)
    static constexpr int BS = FD_Q8K.block_size, BB = FD_Q8K.block_bytes, DB = 292, ITEMS = 64, EPI = 4;
    static __device__ __forceinline__ void item(const uint8_t *b, int it, float *v, int *e) {
        const float d = __uint_as_float((uint32_t)b[0] | ((uint32_t)b[1] << 8) | ((uint32_t)b[2] << 16) | ((uint32_t)b[3] << 24));
#pragma unroll
        for (int j = 0; j < 4; j++) {
            // lanes take neighbouring bytes: element it + 64 j
            e[j] = it + 64 * j;
            v[j] = __fmul_rn(d, (float)(int8_t)b[FD_Q8K.data_offset + e[j]]);
        }
    }
};

template <>
struct Fmt<GLLMK_QUANT_Q4_0> {  // d @0, qs[16] @2: byte j -> elements j (low nibble) and j + 16 (high nibble)
    static constexpr int BS = FD_Q4_0.block_size, BB = FD_Q4_0.block_bytes, DB = 18, ITEMS = 16, EPI = 2;
    static __device__ __forceinline__ void item(const uint8_t *b, int it, float *v, int *e) {
        const float d = f16_at(b);
        const uint8_t q = b[FD_Q4_0.data_offset + it];
        v[0] = __fmul_rn(d, __fsub_rn((float)(q & 0xF), (float)FD_Q4_0.static_bias));
        v[1] = __fmul_rn(d, __fsub_rn((float)(q >> 4), (float)FD_Q4_0.static_bias));
        e[0] = it;
        e[1] = it + 16;
    }
};

template <>
struct Fmt<GLLMK_QUANT_Q5_0> {  // d @0, qh[4] @2 (bit j = fifth bit of element j), qs[16] @6
    static constexpr int BS = FD_Q5_0.block_size, BB = FD_Q5_0.block_bytes, DB = 22, ITEMS = 16, EPI = 2;
    static __device__ __forceinline__ void item(const uint8_t *b, int it, float *v, int *e) {
        const float d = f16_at(b);
        const uint32_t qh = (uint32_t)b[2] | ((uint32_t)b[3] << 8) | ((uint32_t)b[4] << 16) | ((uint32_t)b[5] << 24);
        const uint8_t q = b[FD_Q5_0.data_offset + it];
        const uint32_t lo = (q & 0xF) | (((qh >> it) & 1u) << 4), hi = (q >> 4) | (((qh >> (it + 16)) & 1u) << 4);
        v[0] = __fmul_rn(d, __fsub_rn((float)lo, (float)FD_Q5_0.static_bias));
        v[1] = __fmul_rn(d, __fsub_rn((float)hi, (float)FD_Q5_0.static_bias));
        e[0] = it;
        e[1] = it + 16;
    }
};

// ---- matrix decode / embedding gather: out[r, :] = decode(row ids ? ids[r] : r); rows outside [0, n) -> zeros ----
template <int QT>
__global__ void __launch_bounds__(256) raw_dequant_kernel(const uint8_t *__restrict__ w, int64_t n, int64_t nb,
                                                          const int32_t *__restrict__ ids, float *__restrict__ out,
                                                          size_t total, int stride) {
    using F = Fmt<QT>;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;  // (out row, block, item)
    if (idx >= total) return;
    const int it = (int)(idx % F::ITEMS);
    const size_t rb = idx / F::ITEMS;
    const int64_t blk = (int64_t)(rb % (size_t)nb), orow = (int64_t)(rb / (size_t)nb);
    float *o = out + ((size_t)orow * nb + blk) * F::BS;
    float v[F::EPI];
    int e[F::EPI];
    int64_t row = orow;
    if (ids) row = ids[orow];
    if (row < 0 || row >= n) {
        F::item(w, it, v, e);  // element indices only (block 0 of the matrix always exists)
#pragma unroll
        for (int j = 0; j < F::EPI; j++) o[e[j]] = 0.0f;
        return;
    }
    F::item(w + ((size_t)row * nb + blk) * (size_t)stride, it, v, e);
#pragma unroll
    for (int j = 0; j < F::EPI; j++) o[e[j]] = v[j];
}

// ---- streaming GEMV on integer dot products ------------------------------------------------------
// The activations are quantized once per call to s16 with one f32 scale per 32 elements (act_quant_kernel); a weight
// "unit" is a few 32-bit words of four s8 (or u8 below 128) weight values each, assembled from the block's bit
// fields with word-wide logic, with the f32 factor (and, for Q5_K, the min term) of the sub-block each word lies
// in.  Two dp2a (s16 x s8) per word and token, then acc += x_scale * (w_scale * dot + w_min * sum(x)).
constexpr int RG_WARPS = 8;
constexpr int RG_CHUNK = 2048;  // block bytes staged per warp and pass (two stages of this size per warp)

// x [m tokens, k] (any strides) -> xq s16 [m, k] and xs f32 [m, k / 32] with x ~= xs * xq: 16-bit fixed point per
// 32-element group (relative error ~1.5e-5 of the group's largest value).  One warp per 32 elements.
__global__ void __launch_bounds__(256) act_quant_kernel(const float *__restrict__ x, int64_t xst, int64_t xsk, int m, int64_t k,
                                                        int16_t *__restrict__ xq, float *__restrict__ xs) {
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int64_t per_tok = k >> 5;
    if (warp >= per_tok * m) return;
    const int64_t t = warp / per_tok, b = warp % per_tok;
    const float v = x[(size_t)t * xst + (size_t)(b * 32 + lane) * xsk];
    float a = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
    const float sc = a * (1.0f / 32767.0f);
    const float q = a > 0.0f ? fminf(fmaxf(rintf(v / sc), -32767.0f), 32767.0f) : 0.0f;
    xq[(size_t)t * k + b * 32 + lane] = (int16_t)(int)q;
    if (lane == 0) xs[(size_t)t * per_tok + b] = sc;
}

// f16 field at a 2-byte aligned address
__device__ __forceinline__ float f16_even(const uint8_t *p) {
    return __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(p)));
}
// 32-bit word at a 2-byte aligned shared-memory address (block sizes and field offsets are all even)
// 16 bytes global -> shared without passing registers (both addresses 16-byte aligned)
__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    const unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(gmem) : "memory");
}
template <bool A4>
__device__ __forceinline__ uint32_t ld32(const uint8_t *p) {
    if (A4) return *reinterpret_cast<const uint32_t *>(p);
    const unsigned short *h = reinterpret_cast<const unsigned short *>(p);
    return (uint32_t)h[0] | ((uint32_t)h[1] << 16);
}
// bits 0..3 of v -> bit 0 of bytes 0..3
__device__ __forceinline__ uint32_t spread4(uint32_t v) { return ((v & 0xFu) * 0x00204081u) & 0x01010101u; }

// Per format: UNITS per block, NW words per unit (NP = NW / 2 pairs), MIN = has a min term.
// unit(b, u, q, ko, ws, wm): words q[] (four values each, as s8); words 2i and 2i + 1 are neighbours in k and lie
// in one scale group: pair i starts at element ko[i] of the block (a multiple of 8) and has the weight factor
// ws[i] and the min term wm[i].
template <int QT>
struct Dp;

// 6-bit fields -> s8 4 (q - 32): bit 5 flipped (q - 32 in 6-bit two's complement), two places up
__device__ __forceinline__ uint32_t q6_word(uint32_t lo4, uint32_t hi2_at_4) {
    return ((((lo4 & 0x0F0F0F0Fu) | (hi2_at_4 & 0x30303030u)) ^ 0x20202020u) << 2) & 0xFCFCFCFCu;
}

template <>
struct Dp<GLLMK_QUANT_Q6_K> {
    static constexpr int UNITS = 8, NW = 8;
    static constexpr bool MIN = false;
    static __device__ __forceinline__ void unit(const uint8_t *b, int u, uint32_t *q, int *ko, float *ws, float *) {
        const int g = u >> 2, p = u & 3, is = p >> 1;  // bytes 8p .. 8p + 7 of the half-block's ql / qh runs
        const uint2 A = *reinterpret_cast<const uint2 *>(b + FD_Q6K.data_offset + g * 64 + 8 * p);
        const uint2 B = *reinterpret_cast<const uint2 *>(b + FD_Q6K.data_offset + g * 64 + 32 + 8 * p);
        const uint2 H = *reinterpret_cast<const uint2 *>(b + FD_Q6K.data_high_offset + g * 32 + 8 * p);
        q[0] = q6_word(A.x, H.x << 4);
        q[1] = q6_word(A.y, H.y << 4);
        q[2] = q6_word(B.x, H.x << 2);
        q[3] = q6_word(B.y, H.y << 2);
        q[4] = q6_word(A.x >> 4, H.x);
        q[5] = q6_word(A.y >> 4, H.y);
        q[6] = q6_word(B.x >> 4, H.x >> 2);
        q[7] = q6_word(B.y >> 4, H.y >> 2);
        // the eight scale bytes of this half in one load; run j uses byte is + 2 j
        const uint2 S = *reinterpret_cast<const uint2 *>(b + FD_Q6K.sub_scales_offset + g * 8);
        const uint32_t s01 = S.x >> (8 * is), s23 = S.y >> (8 * is);
        const float d = 0.25f * f16_even(b + FD_Q6K.scale_offset);
        ws[0] = d * (float)(int8_t)(s01 & 0xFF);
        ws[1] = d * (float)(int8_t)((s01 >> 16) & 0xFF);
        ws[2] = d * (float)(int8_t)(s23 & 0xFF);
        ws[3] = d * (float)(int8_t)((s23 >> 16) & 0xFF);
#pragma unroll
        for (int j = 0; j < 4; j++) ko[j] = g * 128 + 32 * j + 8 * p;
    }
};

template <>
struct Dp<GLLMK_QUANT_Q5_K> {
    static constexpr int UNITS = 8, NW = 8;
    static constexpr bool MIN = true;
    static __device__ __forceinline__ void unit(const uint8_t *b, int u, uint32_t *q, int *ko, float *ws, float *wm) {
        const int g = u >> 1, p = u & 1;  // bytes 16p .. 16p + 15 of the 32-byte group g: two sub-blocks, two pairs each
        const uint4 A = *reinterpret_cast<const uint4 *>(b + FD_Q5K.data_offset + g * 32 + 16 * p);
        const uint4 H = *reinterpret_cast<const uint4 *>(b + FD_Q5K.data_high_offset + 16 * p);
        const uint32_t aw[4] = {A.x, A.y, A.z, A.w}, hw[4] = {H.x, H.y, H.z, H.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            q[i] = (aw[i] & 0x0F0F0F0Fu) | (((hw[i] >> (2 * g)) & 0x01010101u) << 4);
            q[4 + i] = ((aw[i] >> 4) & 0x0F0F0F0Fu) | (((hw[i] >> (2 * g + 1)) & 0x01010101u) << 4);
        }
        // d and dmin in one word; the twelve scale bytes as three words.  Sub-blocks 2g and 2g + 1 (get_scale_min_k4,
        // k_quant.rs:388-397) without a branch: both forms from bytes jj = j & 3 of the words, chosen by j < 4.
        static_assert(FD_Q5K.scale_offset == 0 && FD_Q5K.scale_min_offset == 2 && FD_Q5K.sub_scales_offset == 4 && FD_Q5K.data_high_offset == 16,
                      "Q5_K header is the block's first 16 bytes");
        const uint4 hd = *reinterpret_cast<const uint4 *>(b);
        const uint32_t dm = hd.x, w0 = hd.y, w1 = hd.z, w2 = hd.w;
        const float d = __half2float(__ushort_as_half((unsigned short)(dm & 0xFFFF)));
        const float mn = __half2float(__ushort_as_half((unsigned short)(dm >> 16)));
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const int j = 2 * g + i, sh = 8 * (j & 3);
            const uint32_t a = (w0 >> sh) & 0xFF, bb = (w1 >> sh) & 0xFF, c = (w2 >> sh) & 0xFF;
            const uint32_t s_lo = a & 63, m_lo = bb & 63;
            const uint32_t s_hi = (c & 0xF) | ((a >> 6) << 4), m_hi = (c >> 4) | ((bb >> 6) << 4);
            ws[2 * i] = ws[2 * i + 1] = d * (float)(j < 4 ? s_lo : s_hi);
            wm[2 * i] = wm[2 * i + 1] = -(mn * (float)(j < 4 ? m_lo : m_hi));
        }
        ko[0] = g * 64 + 16 * p;
        ko[1] = ko[0] + 8;
        ko[2] = ko[0] + 32;
        ko[3] = ko[0] + 40;
    }
};

template <>
struct Dp<GLLMK_QUANT_Q8_K> {
    static constexpr int UNITS = 16, NW = 4;
    static constexpr bool MIN = false;
    static __device__ __forceinline__ void unit(const uint8_t *b, int u, uint32_t *q, int *ko, float *ws, float *) {
        ws[0] = ws[1] = __uint_as_float(ld32<true>(b + FD_Q8K.scale_offset));
        ko[0] = 8 * u;
        ko[1] = 128 + 8 * u;
        q[0] = ld32<true>(b + FD_Q8K.data_offset + 8 * u);
        q[1] = ld32<true>(b + FD_Q8K.data_offset + 4 + 8 * u);
        q[2] = ld32<true>(b + FD_Q8K.data_offset + 128 + 8 * u);
        q[3] = ld32<true>(b + FD_Q8K.data_offset + 132 + 8 * u);
    }
};

template <>
struct Dp<GLLMK_QUANT_Q4_0> {
    static constexpr int UNITS = 2, NW = 4;
    static constexpr bool MIN = false;
    static __device__ __forceinline__ void unit(const uint8_t *b, int u, uint32_t *q, int *ko, float *ws, float *) {
        const uint32_t W0 = ld32<false>(b + FD_Q4_0.data_offset + 8 * u), W1 = ld32<false>(b + FD_Q4_0.data_offset + 4 + 8 * u);
        // a nibble with bit 3 flipped is q - 8 in 4-bit two's complement; in the high half of a byte it is the s8 16 (q - 8)
        q[0] = ((W0 ^ 0x08080808u) << 4) & 0xF0F0F0F0u;
        q[1] = ((W1 ^ 0x08080808u) << 4) & 0xF0F0F0F0u;
        q[2] = (W0 ^ 0x80808080u) & 0xF0F0F0F0u;
        q[3] = (W1 ^ 0x80808080u) & 0xF0F0F0F0u;
        ko[0] = 8 * u;
        ko[1] = 16 + 8 * u;
        ws[0] = ws[1] = 0.0625f * f16_even(b + FD_Q4_0.scale_offset);
    }
};

template <>
struct Dp<GLLMK_QUANT_Q5_0> {
    static constexpr int UNITS = 2, NW = 4;
    static constexpr bool MIN = false;
    static __device__ __forceinline__ void unit(const uint8_t *b, int u, uint32_t *q, int *ko, float *ws, float *) {
        const uint32_t W0 = ld32<false>(b + FD_Q5_0.data_offset + 8 * u), W1 = ld32<false>(b + FD_Q5_0.data_offset + 4 + 8 * u),
                       qh = ld32<false>(b + FD_Q5_0.data_high_offset);
        // a 5-bit value with bit 4 flipped is q - 16 in 5-bit two's complement; three places up it is the s8 8 (q - 16)
        q[0] = ((((W0 & 0x0F0F0F0Fu) | (spread4(qh >> (8 * u)) << 4)) ^ 0x10101010u) << 3) & 0xF8F8F8F8u;
        q[1] = ((((W1 & 0x0F0F0F0Fu) | (spread4(qh >> (8 * u + 4)) << 4)) ^ 0x10101010u) << 3) & 0xF8F8F8F8u;
        q[2] = (((((W0 >> 4) & 0x0F0F0F0Fu) | (spread4(qh >> (16 + 8 * u)) << 4)) ^ 0x10101010u) << 3) & 0xF8F8F8F8u;
        q[3] = (((((W1 >> 4) & 0x0F0F0F0Fu) | (spread4(qh >> (20 + 8 * u)) << 4)) ^ 0x10101010u) << 3) & 0xF8F8F8F8u;
        ko[0] = 8 * u;
        ko[1] = 16 + 8 * u;
        ws[0] = ws[1] = 0.125f * f16_even(b);
    }
};

struct RawGemvParams {
    const uint8_t *w;
    const int16_t *xq;  // [m, k]
    const float *xs;    // [m, k / 32]
    float *y;
    const float *row_scales;
    int64_t n, nb, k, yst, ysr, n_row_scales;
    int m;
};

constexpr int RG_ROWS = 2;  // rows per warp: their words meet the same activations, loaded once

template <int QT, int MT>
__global__ void __launch_bounds__(RG_WARPS * 32) raw_gemv_kernel(const RawGemvParams p) {
    using F = Fmt<QT>;
    using D = Dp<QT>;
    constexpr int R = RG_ROWS, CH = RG_CHUNK / R;
    constexpr int LPB = D::UNITS < 32 ? 32 / D::UNITS : 1;   // blocks one warp pass over the units covers
    constexpr int CB = (CH / F::DB) / LPB * LPB;             // whole blocks per row and pass, no idle lanes inside a pass
    __shared__ __align__(16) uint8_t buf[RG_WARPS][2][R][CH + 32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k32 = (int)(p.k >> 5);
    const int64_t groups = (p.n + R - 1) / R;
    for (int64_t grp = (int64_t)blockIdx.x * RG_WARPS + warp; grp < groups; grp += (int64_t)gridDim.x * RG_WARPS) {
        const uint8_t *rowp[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int64_t row = grp * R + r < p.n ? grp * R + r : p.n - 1;  // a surplus row repeats the last one; not stored
            rowp[r] = p.w + (size_t)row * p.nb * F::DB;
        }
        for (int t0 = 0; t0 < p.m; t0 += MT) {
            float acc[R][MT];
            const int16_t *xq[MT];
            const float *xs[MT];
#pragma unroll
            for (int t = 0; t < MT; t++) {
                const int tok = t0 + t < p.m ? t0 + t : p.m - 1;  // surplus slots repeat the last token; not stored
                xq[t] = p.xq + (size_t)tok * p.k;
                xs[t] = p.xs + (size_t)tok * k32;
#pragma unroll
                for (int r = 0; r < R; r++) acc[r][t] = 0.0f;
            }
            // two shared-memory stages per warp: the copies of pass i + 1 (cp.async, 16 bytes each) run while pass i
            // is computed.  Copies start at the aligned address below the pass: up to 15 bytes before it and after the
            // row are copied and ignored (the weight buffer starts 256-byte aligned and ends with 16 spare bytes).
            const auto issue = [&](int b0, int st) {
                const int nblk = (int)p.nb - b0 < CB ? (int)p.nb - b0 : CB;
#pragma unroll
                for (int r = 0; r < R; r++) {
                    const uint8_t *src = rowp[r] + (size_t)b0 * F::DB;
                    const uintptr_t a0 = reinterpret_cast<uintptr_t>(src) & ~(uintptr_t)15;
                    const int n16 = ((int)(reinterpret_cast<uintptr_t>(src) - a0) + nblk * F::DB + 15) >> 4;
                    for (int i = lane; i < n16; i += 32) cp_async16(buf[warp][st][r] + 16 * i, reinterpret_cast<const uint8_t *>(a0) + 16 * i);
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
            };
            __syncwarp();
            issue(0, 0);
            int st = 0;
            for (int b0 = 0; b0 < (int)p.nb; b0 += CB, st ^= 1) {
                const int nblk = (int)p.nb - b0 < CB ? (int)p.nb - b0 : CB;
                if (b0 + CB < (int)p.nb) {
                    issue(b0 + CB, st ^ 1);
                    asm volatile("cp.async.wait_group 1;" ::: "memory");
                } else {
                    asm volatile("cp.async.wait_group 0;" ::: "memory");
                }
                __syncwarp();
                const uint8_t *sb[R];
#pragma unroll
                for (int r = 0; r < R; r++)
                    sb[r] = buf[warp][st][r] + (int)(reinterpret_cast<uintptr_t>(rowp[r] + (size_t)b0 * F::DB) & 15);
                for (int u = lane; u < nblk * D::UNITS; u += 32) {
                    const int blk = u / D::UNITS;
                    uint32_t q[R][D::NW];
                    int ko[D::NW / 2];
                    float ws[R][D::NW / 2], wm[R][D::NW / 2];
#pragma unroll
                    for (int r = 0; r < R; r++) D::unit(sb[r] + blk * F::DB, u % D::UNITS, q[r], ko, ws[r], wm[r]);
                    const int kb = (b0 + blk) * F::BS;
#pragma unroll
                    for (int j = 0; j < D::NW / 2; j++) {
                        const int kk = kb + ko[j];
#pragma unroll
                        for (int t = 0; t < MT; t++) {
                            const int4 xw = __ldg(reinterpret_cast<const int4 *>(xq[t] + kk));  // eight s16 activations
                            const float s = __ldg(xs[t] + (kk >> 5));
                            float sx = 0.0f;
                            if (D::MIN)
                                sx = (float)__dp2a_hi(xw.w, 0x01010101, __dp2a_lo(xw.z, 0x01010101,
                                            __dp2a_hi(xw.y, 0x01010101, __dp2a_lo(xw.x, 0x01010101, 0))));
#pragma unroll
                            for (int r = 0; r < R; r++) {
                                // s16 x s8 products: a word's elements 0, 1 against one register, 2, 3 against the next
                                const int q0 = (int)q[r][2 * j], q1 = (int)q[r][2 * j + 1];
                                const float dot =
                                    (float)__dp2a_hi(xw.w, q1, __dp2a_lo(xw.z, q1, __dp2a_hi(xw.y, q0, __dp2a_lo(xw.x, q0, 0))));
                                if (D::MIN) acc[r][t] = fmaf(s, fmaf(ws[r][j], dot, wm[r][j] * sx), acc[r][t]);
                                else acc[r][t] = fmaf(s * ws[r][j], dot, acc[r][t]);
                            }
                        }
                    }
                }
                __syncwarp();  // every lane is done with this stage before the next pass's copies overwrite it
            }
#pragma unroll
            for (int r = 0; r < R; r++)
#pragma unroll
                for (int t = 0; t < MT; t++) {
                    float a = acc[r][t];
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
                    const int64_t row = grp * R + r;
                    if (lane == 0 && t0 + t < p.m && row < p.n) {
                        if (p.n_row_scales == 1) a *= p.row_scales[0];
                        else if (p.n_row_scales > 1) a *= p.row_scales[row];
                        p.y[(size_t)(t0 + t) * p.yst + (size_t)row * p.ysr] = a;
                    }
                }
        }
    }
}

// Q6_K: reference blocks (210 bytes) <-> device slots (224 bytes); one thread per 2 bytes
// ---- Q6_K, 2 tokens and more: the same integer dot products on the tensor core (mma.sync m16n8k16, s8) -------------
// A CTA owns 16 weight rows (the MMA M) and its eight warps split the row's blocks between them; a warp stages one block
// of each of the 16 rows and the same 256 activations of its tokens per pass (cp.async, two or three stages: operand B
// fetched from L2 by every lane as it was needed left the warps waiting for loads most of the time) and issues, per
// 16-element scale group, one MMA per digit of
// the s16 activations (x = 256 * hi + lo, hi signed, lo unsigned: exact) and group of 8 tokens (the MMA N).  Fragment
// layout of m16n8k16: lane (g = lane / 4, t = lane % 4) supplies rows g and g + 8 at k = 4t .. 4t + 3 — one assembled word
// of four s8 values each, the same words the dp2a kernel builds — and token g at the same k; it receives rows g, g + 8
// x tokens 2t, 2t + 1, which it scales by (d * sc of the row's group) x (the token's activation scale) and accumulates
// in f32.  The dp2a kernel spends its time per TOKEN; this one per group of eight.
constexpr int QM_ROWS = 16;
constexpr int QM_ROW_STRIDE = 240;  // a block slot (224 bytes) padded so that eight rows' words fall on different banks
constexpr int QM_TOK_STRIDE = 544;  // a token's 256 s16 activations (512 bytes) padded likewise (8-byte loads, half a warp at a time)
constexpr int qm_stages(int tg) { return tg == 1 ? 3 : 2; }
constexpr int qm_stage_bytes(int tg) { return QM_ROWS * QM_ROW_STRIDE + 8 * tg * QM_TOK_STRIDE; }
constexpr size_t qm_smem_bytes(int tg) { return (size_t)RG_WARPS * qm_stages(tg) * qm_stage_bytes(tg); }

// c = a x b (no accumulator input to keep zeroed: the C operand is one zero register four times)
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0, bool b_unsigned) {
    if (b_unsigned)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.u8.s32 {%0, %1, %2, %3}, {%4, %5}, {%6}, {%7, %7, %7, %7};\n"
                     : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                     : "r"(a0), "r"(a1), "r"(b0), "r"(0));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5}, {%6}, {%7, %7, %7, %7};\n"
                     : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                     : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}

template <int TG>  // groups of 8 tokens per pass over the weights
__global__ void __launch_bounds__(RG_WARPS * 32) q6k_gemv_mma_kernel(const RawGemvParams p) {
    constexpr int DB = Fmt<GLLMK_QUANT_Q6_K>::DB, CPR = DB / 16, NCP = QM_ROWS * CPR / 32;  // 14 chunks of 16 bytes per row and block: 7 per lane
    constexpr int QM_STAGES = qm_stages(TG), QM_STAGE_BYTES = qm_stage_bytes(TG), ACT_OFF = QM_ROWS * QM_ROW_STRIDE;
    extern __shared__ __align__(16) uint8_t qm_smem[];
    __shared__ float red[RG_WARPS][QM_ROWS][8 * TG];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int64_t row0 = (int64_t)blockIdx.x * QM_ROWS;
    const int nb = (int)p.nb, k32 = (int)(p.k >> 5);
    const int b_lo = (int)((int64_t)nb * warp / RG_WARPS), b_hi = (int)((int64_t)nb * (warp + 1) / RG_WARPS);
    uint8_t *stages = qm_smem + (size_t)warp * QM_STAGES * QM_STAGE_BYTES;
    // this lane's chunks of a pass: chunk i = lane + 32 j -> row i / 14 (a surplus row repeats the last one; not stored)
    int soff[NCP];
    const uint8_t *gsrc[NCP];
#pragma unroll
    for (int j = 0; j < NCP; j++) {
        const int i = lane + 32 * j, r = i / CPR, ch = i % CPR;
        const int64_t row = row0 + r < p.n ? row0 + r : p.n - 1;
        soff[j] = r * QM_ROW_STRIDE + 16 * ch;
        gsrc[j] = p.w + (size_t)row * nb * DB + 16 * ch;
    }
    for (int t0 = 0; t0 < p.m; t0 += 8 * TG) {
        float acc[TG][4];
        const float *xsa[TG], *xsb[TG];  // the tokens this lane receives (accumulator columns): t0 + 8 tg + 2t, + 1
        // a pass's activations: 32 chunks of 16 bytes per token, lane = chunk; token tk of the pass = t0 + tk (a surplus
        // column repeats the last token; not stored).  The lane SUPPLIES token 8 tg + g (operand B).
        const auto issue = [&](int b, int st) {
            uint8_t *dst = stages + st * QM_STAGE_BYTES;
#pragma unroll
            for (int j = 0; j < NCP; j++) cp_async16(dst + soff[j], gsrc[j] + (size_t)b * DB);
#pragma unroll
            for (int tk = 0; tk < 8 * TG; tk++) {
                const int tok = t0 + tk < p.m ? t0 + tk : p.m - 1;
                cp_async16(dst + ACT_OFF + tk * QM_TOK_STRIDE + 16 * lane, p.xq + (size_t)tok * p.k + (size_t)b * 256 + 8 * lane);
            }
        };
#pragma unroll
        for (int tg = 0; tg < TG; tg++) {
            const int ta = t0 + 8 * tg + 2 * t;
            xsa[tg] = p.xs + (size_t)(ta < p.m ? ta : p.m - 1) * k32;
            xsb[tg] = p.xs + (size_t)(ta + 1 < p.m ? ta + 1 : p.m - 1) * k32;
#pragma unroll
            for (int i = 0; i < 4; i++) acc[tg][i] = 0.0f;
        }
        __syncwarp();
#pragma unroll
        for (int i = 0; i < QM_STAGES - 1; i++) {
            if (b_lo + i < b_hi) issue(b_lo + i, i);
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
        int st = 0;
        for (int b = b_lo; b < b_hi; b++) {
            // the block's activation scales (eight 32-element groups per token): two 16-byte loads per column, early
            float4 xs4[TG][2][2];
#pragma unroll
            for (int tg = 0; tg < TG; tg++) {
                xs4[tg][0][0] = __ldg(reinterpret_cast<const float4 *>(xsa[tg] + 8 * b));
                xs4[tg][0][1] = __ldg(reinterpret_cast<const float4 *>(xsa[tg] + 8 * b + 4));
                xs4[tg][1][0] = __ldg(reinterpret_cast<const float4 *>(xsb[tg] + 8 * b));
                xs4[tg][1][1] = __ldg(reinterpret_cast<const float4 *>(xsb[tg] + 8 * b + 4));
            }
            if (b + QM_STAGES - 1 < b_hi) issue(b + QM_STAGES - 1, st == 0 ? QM_STAGES - 1 : st - 1);
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group %0;" ::"n"(QM_STAGES - 1) : "memory");
            __syncwarp();
            const uint8_t *r0 = stages + st * QM_STAGE_BYTES + g * QM_ROW_STRIDE, *r8 = r0 + 8 * QM_ROW_STRIDE;
            const uint8_t *xact = stages + st * QM_STAGE_BYTES + ACT_OFF + g * QM_TOK_STRIDE + 8 * t;  // token g, elements 4t .. 4t + 3 of a group
            const uint4 S0 = *reinterpret_cast<const uint4 *>(r0 + FD_Q6K.sub_scales_offset);
            const uint4 S8 = *reinterpret_cast<const uint4 *>(r8 + FD_Q6K.sub_scales_offset);
            const uint32_t s0w[4] = {S0.x, S0.y, S0.z, S0.w}, s8w[4] = {S8.x, S8.y, S8.z, S8.w};
            const float d0 = 0.25f * f16_even(r0 + FD_Q6K.scale_offset), d8 = 0.25f * f16_even(r8 + FD_Q6K.scale_offset);
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {  // half of the block (128 elements)
#pragma unroll
                for (int is = 0; is < 2; is++) {  // which 16 of every 32-element run
                    int2 xw[4][TG];  // operand B of the four runs: four s16 activations each
#pragma unroll
                    for (int j = 0; j < 4; j++)
#pragma unroll
                        for (int tg = 0; tg < TG; tg++)
                            xw[j][tg] = *reinterpret_cast<const int2 *>(xact + 8 * tg * QM_TOK_STRIDE + 2 * (hh * 128 + 32 * j + 16 * is));
                    const int lo_off = FD_Q6K.data_offset + hh * 64 + 16 * is + 4 * t, hi_off = FD_Q6K.data_high_offset + hh * 32 + 16 * is + 4 * t;
                    const uint32_t A0 = *reinterpret_cast<const uint32_t *>(r0 + lo_off), B0 = *reinterpret_cast<const uint32_t *>(r0 + lo_off + 32),
                                   H0 = *reinterpret_cast<const uint32_t *>(r0 + hi_off);
                    const uint32_t A8 = *reinterpret_cast<const uint32_t *>(r8 + lo_off), B8 = *reinterpret_cast<const uint32_t *>(r8 + lo_off + 32),
                                   H8 = *reinterpret_cast<const uint32_t *>(r8 + hi_off);
                    const uint32_t q0[4] = {q6_word(A0, H0 << 4), q6_word(B0, H0 << 2), q6_word(A0 >> 4, H0), q6_word(B0 >> 4, H0 >> 2)};
                    const uint32_t q8[4] = {q6_word(A8, H8 << 4), q6_word(B8, H8 << 2), q6_word(A8 >> 4, H8), q6_word(B8 >> 4, H8 >> 2)};
#pragma unroll
                    for (int j = 0; j < 4; j++) {  // run j of the half: elements hh * 128 + 32 j + 16 is + (0 .. 15), scale byte hh * 8 + is + 2 j
                        const int sb = hh * 8 + is + 2 * j;
                        const float ws0 = d0 * (float)(int8_t)((s0w[sb >> 2] >> (8 * (sb & 3))) & 0xFF);
                        const float ws8 = d8 * (float)(int8_t)((s8w[sb >> 2] >> (8 * (sb & 3))) & 0xFF);
#pragma unroll
                        for (int tg = 0; tg < TG; tg++) {
                            const uint32_t xlo = __byte_perm((uint32_t)xw[j][tg].x, (uint32_t)xw[j][tg].y, 0x6420),
                                           xhi = __byte_perm((uint32_t)xw[j][tg].x, (uint32_t)xw[j][tg].y, 0x7531);
                            int chi[4], clo[4];
                            mma_s8(chi, q0[j], q8[j], xhi, false);
                            mma_s8(clo, q0[j], q8[j], xlo, true);
                            const float4 va = xs4[tg][0][hh], vb = xs4[tg][1][hh];
                            const float xa = j == 0 ? va.x : (j == 1 ? va.y : (j == 2 ? va.z : va.w));
                            const float xb = j == 0 ? vb.x : (j == 1 ? vb.y : (j == 2 ? vb.z : vb.w));
                            acc[tg][0] = fmaf((float)(chi[0] * 256 + clo[0]), ws0 * xa, acc[tg][0]);
                            acc[tg][1] = fmaf((float)(chi[1] * 256 + clo[1]), ws0 * xb, acc[tg][1]);
                            acc[tg][2] = fmaf((float)(chi[2] * 256 + clo[2]), ws8 * xa, acc[tg][2]);
                            acc[tg][3] = fmaf((float)(chi[3] * 256 + clo[3]), ws8 * xb, acc[tg][3]);
                        }
                    }
                }
            }
            __syncwarp();  // every lane is done with this stage before a later pass's copies overwrite it
            st = st + 1 == QM_STAGES ? 0 : st + 1;
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        // the eight warps' partial sums meet in shared memory
#pragma unroll
        for (int tg = 0; tg < TG; tg++) {
            red[warp][g][8 * tg + 2 * t] = acc[tg][0];
            red[warp][g][8 * tg + 2 * t + 1] = acc[tg][1];
            red[warp][g + 8][8 * tg + 2 * t] = acc[tg][2];
            red[warp][g + 8][8 * tg + 2 * t + 1] = acc[tg][3];
        }
        __syncthreads();
        for (int i = threadIdx.x; i < QM_ROWS * 8 * TG; i += RG_WARPS * 32) {
            const int r = i / (8 * TG), tk = i % (8 * TG);
            const int64_t row = row0 + r;
            if (row < p.n && t0 + tk < p.m) {
                float a = 0.0f;
#pragma unroll
                for (int w = 0; w < RG_WARPS; w++) a += red[w][r][tk];
                if (p.n_row_scales == 1) a *= p.row_scales[0];
                else if (p.n_row_scales > 1) a *= p.row_scales[row];
                p.y[(size_t)(t0 + tk) * p.yst + (size_t)row * p.ysr] = a;
            }
        }
        __syncthreads();
    }
}

__global__ void q6k_pad_kernel(const unsigned short *__restrict__ src, unsigned short *__restrict__ dst, size_t total, int to_device) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t blk = idx / 105, o = idx % 105;
    if (to_device) dst[blk * 112 + o] = src[blk * 105 + o];
    else dst[blk * 105 + o] = src[blk * 112 + o];
}

inline unsigned grid_1d(size_t total, int block) { return (unsigned)((total + block - 1) / block); }

template <int QT>
int32_t dequant_t(Ctx *c, const uint8_t *w, int64_t n, int64_t nb, const int32_t *ids, size_t rows, float *out, cudaStream_t s,
                  bool dev_layout) {
    const size_t total = rows * (size_t)nb * Fmt<QT>::ITEMS;
    if (total == 0) return GLLMK_STATUS_OK;
    if (total > (size_t)0x7fffffff * 256) return fail(c, GLLMK_STATUS_INVALID_ARG, "decode: matrix too large for one launch");
    raw_dequant_kernel<QT><<<grid_1d(total, 256), 256, 0, s>>>(w, n, nb, ids, out, total, dev_layout ? Fmt<QT>::DB : Fmt<QT>::BB);
    GK_CUDA(c, cudaGetLastError());
    return GLLMK_STATUS_OK;
}

template <int TG>
int32_t q6k_mma_launch(Ctx *c, const RawGemvParams &p, cudaStream_t s) {
    static bool attr_set[64] = {};  // function attributes are per device
    if (!attr_set[c->device & 63]) {
        GK_CUDA(c, cudaFuncSetAttribute(q6k_gemv_mma_kernel<TG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)qm_smem_bytes(TG)));
        attr_set[c->device & 63] = true;
    }
    q6k_gemv_mma_kernel<TG><<<(unsigned)((p.n + QM_ROWS - 1) / QM_ROWS), RG_WARPS * 32, qm_smem_bytes(TG), s>>>(p);
    GK_CUDA(c, cudaGetLastError());
    return GLLMK_STATUS_OK;
}

template <int QT>
int32_t gemv_t(Ctx *c, const RawGemvParams &p, cudaStream_t s) {
    if (QT == GLLMK_QUANT_Q6_K && c->raw_gemv_mma && (p.m >= 2 || c->raw_gemv_mma == 2) && p.n <= (int64_t)0x7fffffff * QM_ROWS)
        return p.m <= 8 ? q6k_mma_launch<1>(c, p, s) : q6k_mma_launch<2>(c, p, s);
    // 16 rows per CTA and pass; enough CTAs to fill every SM several times over, never more than the rows need
    int64_t ctas = (p.n + RG_WARPS * RG_ROWS - 1) / (RG_WARPS * RG_ROWS);
    const int64_t cap = (int64_t)c->sm_count * 6;
    if (ctas > cap) ctas = cap;
    if (p.m == 1) raw_gemv_kernel<QT, 1><<<(unsigned)ctas, RG_WARPS * 32, 0, s>>>(p);
    else if (p.m <= 4) raw_gemv_kernel<QT, 4><<<(unsigned)ctas, RG_WARPS * 32, 0, s>>>(p);
    else raw_gemv_kernel<QT, 8><<<(unsigned)ctas, RG_WARPS * 32, 0, s>>>(p);
    GK_CUDA(c, cudaGetLastError());
    return GLLMK_STATUS_OK;
}

}  // namespace

bool raw_format(int32_t qt) {
    return qt == GLLMK_QUANT_Q6_K || qt == GLLMK_QUANT_Q5_K || qt == GLLMK_QUANT_Q8_K || qt == GLLMK_QUANT_Q4_0 ||
           qt == GLLMK_QUANT_Q5_0;
}

int raw_dev_block_bytes(int32_t qt) {
    switch (qt) {
        case GLLMK_QUANT_Q6_K: return Fmt<GLLMK_QUANT_Q6_K>::DB;
        case GLLMK_QUANT_Q5_K: return Fmt<GLLMK_QUANT_Q5_K>::DB;
        case GLLMK_QUANT_Q8_K: return Fmt<GLLMK_QUANT_Q8_K>::DB;
        case GLLMK_QUANT_Q4_0: return Fmt<GLLMK_QUANT_Q4_0>::DB;
        case GLLMK_QUANT_Q5_0: return Fmt<GLLMK_QUANT_Q5_0>::DB;
    }
    return 0;
}

// reference-layout blocks (device memory) -> the weight's device buffer, and back
int32_t raw_fill(Ctx *c, const Weight *w, const void *blocks, cudaStream_t s) {
    GK_CUDA(c, cudaMemsetAsync(w->qs, 0, w->qs_bytes, s));
    if (w->qt == GLLMK_QUANT_Q6_K) {
        const size_t total = (size_t)w->n * w->nb * 105;
        q6k_pad_kernel<<<grid_1d(total, 256), 256, 0, s>>>(static_cast<const unsigned short *>(blocks),
                                                           static_cast<unsigned short *>(w->qs), total, 1);
        GK_CUDA(c, cudaGetLastError());
    } else {
        GK_CUDA(c, cudaMemcpyAsync(w->qs, blocks, w->ref_bytes, cudaMemcpyDeviceToDevice, s));
    }
    return GLLMK_STATUS_OK;
}
int32_t raw_unfill(Ctx *c, const Weight *w, void *blocks, cudaStream_t s) {
    if (w->qt == GLLMK_QUANT_Q6_K) {
        const size_t total = (size_t)w->n * w->nb * 105;
        q6k_pad_kernel<<<grid_1d(total, 256), 256, 0, s>>>(static_cast<const unsigned short *>(w->qs),
                                                           static_cast<unsigned short *>(blocks), total, 0);
        GK_CUDA(c, cudaGetLastError());
    } else {
        GK_CUDA(c, cudaMemcpyAsync(blocks, w->qs, w->ref_bytes, cudaMemcpyDeviceToDevice, s));
    }
    return GLLMK_STATUS_OK;
}

// dev_layout: blocks at the device stride (a weight's buffer); otherwise consecutive reference blocks
int32_t raw_dequant(Ctx *c, int32_t qt, const uint8_t *w, int64_t n, int64_t nb, const int32_t *ids, size_t rows, float *out,
                    cudaStream_t s, bool dev_layout) {
    switch (qt) {
        case GLLMK_QUANT_Q6_K: return dequant_t<GLLMK_QUANT_Q6_K>(c, w, n, nb, ids, rows, out, s, dev_layout);
        case GLLMK_QUANT_Q5_K: return dequant_t<GLLMK_QUANT_Q5_K>(c, w, n, nb, ids, rows, out, s, dev_layout);
        case GLLMK_QUANT_Q8_K: return dequant_t<GLLMK_QUANT_Q8_K>(c, w, n, nb, ids, rows, out, s, dev_layout);
        case GLLMK_QUANT_Q4_0: return dequant_t<GLLMK_QUANT_Q4_0>(c, w, n, nb, ids, rows, out, s, dev_layout);
        case GLLMK_QUANT_Q5_0: return dequant_t<GLLMK_QUANT_Q5_0>(c, w, n, nb, ids, rows, out, s, dev_layout);
    }
    return fail(c, GLLMK_STATUS_UNSUPPORTED, "decode: quant type %d", qt);
}

int32_t raw_gemv_launch(Ctx *c, const Weight *w, const float *x, int64_t xst, int64_t xsk, int m, float *y, int64_t yst,
                        int64_t ysr, const float *row_scales, int64_t n_row_scales, cudaStream_t s) {
    // activations -> s16 + one f32 scale per 32 elements, in the context's activation scratch
    const size_t qb = (2 * (size_t)m * w->k + 255) & ~(size_t)255;
    int32_t rc = ensure_act(c, qb + (size_t)m * (w->k / 32) * sizeof(float));
    if (rc) return rc;
    int16_t *xq = static_cast<int16_t *>(c->act);
    float *xs = reinterpret_cast<float *>(static_cast<char *>(c->act) + qb);
    const size_t qthreads = (size_t)m * (w->k / 32) * 32;
    act_quant_kernel<<<grid_1d(qthreads, 256), 256, 0, s>>>(x, xst, xsk, m, w->k, xq, xs);
    GK_CUDA(c, cudaGetLastError());
    RawGemvParams p{};
    p.w = static_cast<const uint8_t *>(w->qs);
    p.xq = xq;
    p.xs = xs;
    p.k = w->k;
    p.y = y;
    p.row_scales = row_scales;
    p.n_row_scales = row_scales ? n_row_scales : 0;
    p.n = w->n;
    p.nb = w->nb;
    p.yst = yst;
    p.ysr = ysr;
    p.m = m;
    switch (w->qt) {
        case GLLMK_QUANT_Q6_K: return gemv_t<GLLMK_QUANT_Q6_K>(c, p, s);
        case GLLMK_QUANT_Q5_K: return gemv_t<GLLMK_QUANT_Q5_K>(c, p, s);
        case GLLMK_QUANT_Q8_K: return gemv_t<GLLMK_QUANT_Q8_K>(c, p, s);
        case GLLMK_QUANT_Q4_0: return gemv_t<GLLMK_QUANT_Q4_0>(c, p, s);
        case GLLMK_QUANT_Q5_0: return gemv_t<GLLMK_QUANT_Q5_0>(c, p, s);
    }
    return fail(c, GLLMK_STATUS_UNSUPPORTED, "gemv: quant type %d", w->qt);
}

}  // namespace gllmk
