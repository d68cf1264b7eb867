/*
 * CPU oracle for the quantized-matmul hot path of gllm-kernels.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the reference's
 * scalar CPU algorithms (the reference is Rust and cannot be compiled where this is
 * built).  It is the checker the CUDA path is compared against and the CPU baseline
 * that the benchmark times; the product library never links, loads or calls it.
 *
 * Every function names the reference source it follows (paths inside gllm-kernels).
 * Build with -ffp-contract=off and without -ffast-math: Rust never fuses a*b+c and
 * the reference accumulates strictly in order.
 *
 * Parity status: Q4_K, Q8_0, MXFP4, E8M0, E2M1 and E4M3 decoders are pinned by the
 * reference's own known-answer tests (see tests/test_oracle_known_answers.py).
 * NVFP4 decoded VALUES are "parity unpinned": the reference has layout tests only,
 * no test fixes a decoded value; the decode follows the formula documented in
 * src/quant.rs:77-86,357-371.  The quantizers at the end are this project's own
 * (the reference ships none for these formats).
 */
#include <math.h>
#include <pthread.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------
 * IEEE binary16 <-> binary32.  The reference uses the `half` crate (half = "2.3.1",
 * Cargo.toml:10): f16::to_f32 is exact, f16::from_f32 rounds to nearest even.  Same bit-level
 * behaviour as the reference's own helper, scalar-ops/src/quant_matmul.rs:415-435.
 * ---------------------------------------------------------------------------------------- */
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

API float gko_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        /* subnormal: normalise */
        int e = -1;
        do { e++; man <<= 1; } while ((man & 0x400u) == 0);
        man &= 0x3FFu;
        return bits_f32(sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13));
    }
    if (exp == 31) return bits_f32(sign | 0x7F800000u | (man << 13));
    return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

API uint16_t gko_f32_to_f16(float f) {
    uint32_t x = f32_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((ax > 0x7F800000u) ? (0x200u | ((ax >> 13) & 0x3FFu)) : 0));
    }
    if (ax >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds to >= 65520 -> inf */
    if (ax < 0x33000001u) return (uint16_t)sign;              /* < 2^-25 (or == 2^-25 tie to 0) */
    int exp = (int)(ax >> 23) - 127;
    uint32_t man = (ax & 0x7FFFFFu) | 0x800000u;
    int shift;
    uint32_t base;
    if (exp < -14) { shift = 13 + (-14 - exp); base = 0; }
    else { shift = 13; base = (uint32_t)(exp + 15) << 10; man &= 0x7FFFFFu; }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    return (uint16_t)(sign | (base + q)); /* carry into the exponent is the right result */
}

/* ------------------------------------------------------------------------------------------
 * Format metadata: src/quant.rs:375-456 (block_size / block_bytes) for the four formats of
 * the path.  Type ids are this boundary's own (the reference enum carries no discriminants).
 * ---------------------------------------------------------------------------------------- */
enum { GKO_Q4K = 1, GKO_Q8_0 = 2, GKO_MXFP4 = 3, GKO_NVFP4 = 4,
       GKO_Q6K = 6, GKO_Q5K = 7, GKO_Q4_0 = 8, GKO_Q5_0 = 9, GKO_Q8K = 10 };

API int gko_block_size(int qt, int mx_block) {
    switch (qt) {
        case GKO_Q4K: return 256;   /* QK_K, src/quant.rs:90 */
        case GKO_Q8_0: return 32;
        case GKO_MXFP4: return mx_block;
        case GKO_NVFP4: return 64;  /* QK_NVFP4, src/quant.rs:92 */
        case GKO_Q6K: case GKO_Q5K: case GKO_Q8K: return 256;
        case GKO_Q4_0: case GKO_Q5_0: return 32;
    }
    return 0;
}
API int gko_block_bytes(int qt, int mx_block) {
    switch (qt) {
        case GKO_Q4K: return 144;
        case GKO_Q8_0: return 34;
        case GKO_MXFP4: return 1 + mx_block / 2; /* src/quant.rs:427 */
        case GKO_NVFP4: return 36;
        case GKO_Q6K: return 210;   /* BlockQ6K, src/quant.rs:143-148 */
        case GKO_Q5K: return 176;   /* BlockQ5K, src/quant.rs:132-138 */
        case GKO_Q4_0: return 18;   /* BlockQ4_0, src/quant.rs:254-257 */
        case GKO_Q5_0: return 22;   /* BlockQ5_0, src/quant.rs:271-275 */
        case GKO_Q8K: return 292;   /* BlockQ8K, src/quant.rs:153-157 */
    }
    return 0;
}

/* ------------------------------------------------------------------------------------------
 * Q4_K.  src/macros/quant_primitive/k_quant.rs:7-56 (decode), :502-547 (dot).
 * Block: d f16 @0, dmin f16 @2, scales[12] @4, qs[128] @16 (src/quant.rs:122-127).
 * ---------------------------------------------------------------------------------------- */
static inline void get_scale_min_k4(int j, const uint8_t *s, float *sc, float *m) {
    if (j < 4) {
        *sc = (float)(s[j] & 63);
        *m = (float)(s[j + 4] & 63);
    } else {
        *sc = (float)((s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4));
        *m = (float)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

API void gko_q4k_scales(const uint8_t *block, uint8_t *sc_out, uint8_t *m_out) {
    for (int j = 0; j < 8; j++) {
        float sc, m;
        get_scale_min_k4(j, block + 4, &sc, &m);
        sc_out[j] = (uint8_t)sc;
        m_out[j] = (uint8_t)m;
    }
}

API void gko_dequant_q4_k(const uint8_t *block, float *out) {
    uint16_t dh, mh;
    memcpy(&dh, block, 2);
    memcpy(&mh, block + 2, 2);
    const float d = gko_f16_to_f32(dh), dmin = gko_f16_to_f32(mh);
    const uint8_t *scales = block + 4, *qs = block + 16;
    int is = 0;
    for (int group = 0; group < 4; group++) {
        const int q_off = group * 32, out_off = group * 64;
        float sc1, m1, sc2, m2;
        get_scale_min_k4(is, scales, &sc1, &m1);
        const float d1 = d * sc1, neg_m1 = dmin * m1;
        get_scale_min_k4(is + 1, scales, &sc2, &m2);
        const float d2 = d * sc2, neg_m2 = dmin * m2;
        for (int l = 0; l < 32; l++) out[out_off + l] = d1 * (float)(qs[q_off + l] & 0xF) - neg_m1;
        for (int l = 0; l < 32; l++) out[out_off + 32 + l] = d2 * (float)(qs[q_off + l] >> 4) - neg_m2;
        is += 2;
    }
}

static float dot_q4_k(const uint8_t *block, const float *x) {
    uint16_t dh, mh;
    memcpy(&dh, block, 2);
    memcpy(&mh, block + 2, 2);
    const float d = gko_f16_to_f32(dh), dmin = gko_f16_to_f32(mh);
    const uint8_t *scales = block + 4, *qs = block + 16;
    float sum = 0.0f;
    int is = 0;
    for (int group = 0; group < 4; group++) {
        const int q_off = group * 32, out_off = group * 64;
        float sc1, m1, sc2, m2;
        get_scale_min_k4(is, scales, &sc1, &m1);
        const float d1 = d * sc1, neg_m1 = dmin * m1;
        get_scale_min_k4(is + 1, scales, &sc2, &m2);
        const float d2 = d * sc2, neg_m2 = dmin * m2;
        for (int l = 0; l < 32; l++) sum += (d1 * (float)(qs[q_off + l] & 0xF) - neg_m1) * x[out_off + l];
        for (int l = 0; l < 32; l++) sum += (d2 * (float)(qs[q_off + l] >> 4) - neg_m2) * x[out_off + 32 + l];
        is += 2;
    }
    return sum;
}
API float gko_dot_q4_k(const uint8_t *block, const float *x) { return dot_q4_k(block, x); }

/* Element-indexed decode, the form used by q4k_decode_step_native
 * (src/asm/x86_64/quant_gemv.rs:2315-2358): d*sc*q - dmin*m. */
API float gko_q4k_element(const uint8_t *block, int e) {
    uint16_t dh, mh;
    memcpy(&dh, block, 2);
    memcpy(&mh, block + 2, 2);
    const float d = gko_f16_to_f32(dh), dmin = gko_f16_to_f32(mh);
    const int mini = e / 32, l = e % 32, g = mini / 2, hi = mini % 2;
    const uint8_t b = block[16 + 32 * g + l];
    const float q = (float)(hi ? (b >> 4) : (b & 0xF));
    float sc, m;
    get_scale_min_k4(mini, block + 4, &sc, &m);
    return d * sc * q - dmin * m;
}

/* ------------------------------------------------------------------------------------------
 * Q8_0.  src/macros/quant_primitive/classic.rs:860-881 (scalar decode and dot).
 * Block: d f16 @0, qs i8[32] @2 (src/quant.rs:290-293).
 * ---------------------------------------------------------------------------------------- */
API void gko_dequant_q8_0(const uint8_t *block, float *out) {
    uint16_t dh;
    memcpy(&dh, block, 2);
    const float d = gko_f16_to_f32(dh);
    const int8_t *qs = (const int8_t *)(block + 2);
    for (int i = 0; i < 32; i++) out[i] = d * (float)qs[i];
}

static float dot_q8_0(const uint8_t *block, const float *x) {
    uint16_t dh;
    memcpy(&dh, block, 2);
    const float d = gko_f16_to_f32(dh);
    const int8_t *qs = (const int8_t *)(block + 2);
    float sum = 0.0f;
    for (int i = 0; i < 32; i++) sum += d * (float)qs[i] * x[i];
    return sum;
}
API float gko_dot_q8_0(const uint8_t *block, const float *x) { return dot_q8_0(block, x); }

/* ------------------------------------------------------------------------------------------
 * MXFP4.  src/quant_mxfp4.rs:33-35 (E2M1 table), :43-54 (E8M0), :72-109 (scalar dequant).
 * ---------------------------------------------------------------------------------------- */
static const float E2M1_LUT_F32[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                       -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};

API float gko_e2m1(int code) { return E2M1_LUT_F32[code & 15]; }

API float gko_decode_e8m0_scale(uint8_t byte) {
    if (byte == 255) return NAN;
    if (byte == 0) return bits_f32(0x00400000u);
    return bits_f32((uint32_t)byte << 23);
}

API void gko_dequant_mxfp4(const uint8_t *blocks, const uint8_t *scales, float *out,
                           size_t num_blocks, size_t block_size) {
    const size_t bpb = block_size / 2;
    for (size_t blk = 0; blk < num_blocks; blk++) {
        const float scale = gko_decode_e8m0_scale(scales[blk]);
        const uint8_t *qs = blocks + blk * bpb;
        float *o = out + blk * block_size;
        for (size_t i = 0; i < bpb; i++) {
            const uint8_t byte = qs[i];
            o[2 * i] = E2M1_LUT_F32[byte & 0x0F] * scale;
            o[2 * i + 1] = E2M1_LUT_F32[(byte >> 4) & 0x0F] * scale;
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * OCP FP8 E4M3.  src/compiler/codegen/vm/numerical_sim.rs:2751-2808 (encode), :2811-2835
 * (decode).  Restated with the reference's own quirks: the subnormal branch rounds with
 * f32::round (half away from zero) and clamps the mantissa to 7.
 * ---------------------------------------------------------------------------------------- */
API float gko_e4m3_to_f32(uint8_t b) {
    const int sign = (b >> 7) & 1, e = (b >> 3) & 0xF, m = b & 7;
    float a;
    if (e == 0) a = (m == 0) ? 0.0f : (float)m * (1.0f / 512.0f);
    else if (e == 15 && m == 7) return NAN;
    else a = (1.0f + (float)m / 8.0f) * ldexpf(1.0f, e - 7);
    return sign ? -a : a;
}

API uint8_t gko_f32_to_e4m3(float v) {
    if (isnan(v)) return 0x7F;
    const uint32_t bits = f32_bits(v);
    const uint32_t sign = (bits >> 31) & 1u;
    float a = bits_f32(bits & 0x7FFFFFFFu);
    if (a > 448.0f) a = 448.0f;
    const uint32_t ab = f32_bits(a);
    const int e = (int)(ab >> 23);
    const uint32_t m23 = ab & 0x7FFFFFu;
    if (a == 0.0f) return (uint8_t)(sign << 7);
    int e4 = (e - 127) + 7;
    int m3;
    if (e4 <= 0) {
        e4 = 0;
        m3 = (int)roundf(a * 512.0f);
    } else {
        const int top3 = (int)(m23 >> 20);
        const uint32_t rem = m23 & 0xFFFFFu, half = 0x80000u;
        int m = top3;
        if (rem > half || (rem == half && (top3 & 1) == 1)) {
            m += 1;
            if (m > 7) { m = 0; e4 += 1; }
        }
        if (e4 > 15) { e4 = 15; m3 = 7; }
        else m3 = m;
    }
    if (e4 < 0) e4 = 0;
    if (e4 > 15) e4 = 15;
    if (m3 < 0) m3 = 0;
    if (m3 > 7) m3 = 7;
    return (uint8_t)((sign << 7) | ((uint32_t)e4 << 3) | (uint32_t)m3);
}

/* ------------------------------------------------------------------------------------------
 * NVFP4.  Block 64 elements / 36 bytes: d[4] UE4M3 @0 (one per 16), qs[32] @4
 * (src/quant.rs:366-371).  value = global * e4m3(d[e/16]) * E2M1[nibble]  (src/quant.rs:77-86);
 * low nibble = even element, as for MXFP4.  Evaluation order (global*sub)*code is this
 * project's choice: PARITY UNPINNED, no reference test fixes an NVFP4 value.
 * ---------------------------------------------------------------------------------------- */
API void gko_dequant_nvfp4(const uint8_t *blocks, float global_scale, float *out, size_t num_blocks) {
    for (size_t blk = 0; blk < num_blocks; blk++) {
        const uint8_t *b = blocks + blk * 36;
        float *o = out + blk * 64;
        for (int sub = 0; sub < 4; sub++) {
            const float s = global_scale * gko_e4m3_to_f32(b[sub]);
            for (int i = 0; i < 8; i++) {
                const uint8_t byte = b[4 + sub * 8 + i];
                o[sub * 16 + 2 * i] = s * E2M1_LUT_F32[byte & 0xF];
                o[sub * 16 + 2 * i + 1] = s * E2M1_LUT_F32[byte >> 4];
            }
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * The other GGUF formats of the reference's CPU quant path.  Each decode / dot keeps the
 * reference's operation order (products left to right, no fused multiply-add).
 *
 * Q6_K  decode src/macros/quant_primitive/k_quant.rs:441-472, dot :723-755.
 *       Block: ql[128] @0, qh[64] @128, scales[16] (i8) @192, d f16 @208 (src/quant.rs:143-148).
 * Q5_K  decode k_quant.rs:381-436, dot :669-721.
 *       Block: d @0, dmin @2, scales[12] @4, qh[32] @16, qs[128] @48 (src/quant.rs:132-138).
 * Q8_K  decode k_quant.rs:92-101, dot :549-561.  Block: d f32 @0, qs[256] i8 @4, bsums @260.
 * Q4_0  decode/dot src/macros/quant_primitive/classic.rs:15-48.  Block: d @0, qs[16] @2.
 * Q5_0  decode/dot classic.rs:484-526.  Block: d @0, qh[4] @2, qs[16] @6.
 * ---------------------------------------------------------------------------------------- */
static inline float rd_f16(const uint8_t *p) {
    uint16_t h;
    memcpy(&h, p, 2);
    return gko_f16_to_f32(h);
}

API void gko_dequant_q6_k(const uint8_t *b, float *out) {
    const uint8_t *ql = b, *qh = b + 128;
    const int8_t *sc = (const int8_t *)(b + 192);
    const float d = rd_f16(b + 208);
    for (int g = 0; g < 2; g++) {
        const int qlo = g * 64, qho = g * 32, so = g * 8, oo = g * 128;
        for (int l = 0; l < 32; l++) {
            const int is = l / 16;
            const int q1 = (int)(int8_t)((ql[qlo + l] & 0xF) | (((qh[qho + l] >> 0) & 3) << 4)) - 32;
            const int q2 = (int)(int8_t)((ql[qlo + l + 32] & 0xF) | (((qh[qho + l] >> 2) & 3) << 4)) - 32;
            const int q3 = (int)(int8_t)((ql[qlo + l] >> 4) | (((qh[qho + l] >> 4) & 3) << 4)) - 32;
            const int q4 = (int)(int8_t)((ql[qlo + l + 32] >> 4) | (((qh[qho + l] >> 6) & 3) << 4)) - 32;
            out[oo + l] = d * (float)sc[so + is] * (float)q1;
            out[oo + l + 32] = d * (float)sc[so + is + 2] * (float)q2;
            out[oo + l + 64] = d * (float)sc[so + is + 4] * (float)q3;
            out[oo + l + 96] = d * (float)sc[so + is + 6] * (float)q4;
        }
    }
}
static float dot_q6_k(const uint8_t *b, const float *x) {
    const uint8_t *ql = b, *qh = b + 128;
    const int8_t *sc = (const int8_t *)(b + 192);
    const float d = rd_f16(b + 208);
    float sum = 0.0f;
    for (int g = 0; g < 2; g++) {
        const int qlo = g * 64, qho = g * 32, so = g * 8, oo = g * 128;
        for (int l = 0; l < 32; l++) {
            const int is = l / 16;
            const int q1 = (int)(int8_t)((ql[qlo + l] & 0xF) | (((qh[qho + l] >> 0) & 3) << 4)) - 32;
            const int q2 = (int)(int8_t)((ql[qlo + l + 32] & 0xF) | (((qh[qho + l] >> 2) & 3) << 4)) - 32;
            const int q3 = (int)(int8_t)((ql[qlo + l] >> 4) | (((qh[qho + l] >> 4) & 3) << 4)) - 32;
            const int q4 = (int)(int8_t)((ql[qlo + l + 32] >> 4) | (((qh[qho + l] >> 6) & 3) << 4)) - 32;
            sum += d * (float)sc[so + is] * (float)q1 * x[oo + l];
            sum += d * (float)sc[so + is + 2] * (float)q2 * x[oo + l + 32];
            sum += d * (float)sc[so + is + 4] * (float)q3 * x[oo + l + 64];
            sum += d * (float)sc[so + is + 6] * (float)q4 * x[oo + l + 96];
        }
    }
    return sum;
}

API void gko_dequant_q5_k(const uint8_t *b, float *out) {
    const float d = rd_f16(b), min = rd_f16(b + 2);
    const uint8_t *scales = b + 4, *qh = b + 16, *ql = b + 48;
    int is = 0;
    uint8_t u1 = 1, u2 = 2;
    for (int g = 0; g < 4; g++) {
        float sc1, m1, sc2, m2;
        get_scale_min_k4(is, scales, &sc1, &m1);
        get_scale_min_k4(is + 1, scales, &sc2, &m2);
        const float d1 = d * sc1, nm1 = min * m1, d2 = d * sc2, nm2 = min * m2;
        for (int l = 0; l < 32; l++) {
            const int v = (ql[g * 32 + l] & 0xF) + ((qh[l] & u1) ? 16 : 0);
            out[g * 64 + l] = d1 * (float)v - nm1;
        }
        for (int l = 0; l < 32; l++) {
            const int v = (ql[g * 32 + l] >> 4) + ((qh[l] & u2) ? 16 : 0);
            out[g * 64 + 32 + l] = d2 * (float)v - nm2;
        }
        is += 2;
        u1 <<= 2;
        u2 <<= 2;
    }
}
static float dot_q5_k(const uint8_t *b, const float *x) {
    const float d = rd_f16(b), min = rd_f16(b + 2);
    const uint8_t *scales = b + 4, *qh = b + 16, *ql = b + 48;
    int is = 0;
    uint8_t u1 = 1, u2 = 2;
    float sum = 0.0f;
    for (int g = 0; g < 4; g++) {
        float sc1, m1, sc2, m2;
        get_scale_min_k4(is, scales, &sc1, &m1);
        get_scale_min_k4(is + 1, scales, &sc2, &m2);
        const float d1 = d * sc1, nm1 = min * m1, d2 = d * sc2, nm2 = min * m2;
        for (int l = 0; l < 32; l++) {
            const int v = (ql[g * 32 + l] & 0xF) + ((qh[l] & u1) ? 16 : 0);
            sum += (d1 * (float)v - nm1) * x[g * 64 + l];
        }
        for (int l = 0; l < 32; l++) {
            const int v = (ql[g * 32 + l] >> 4) + ((qh[l] & u2) ? 16 : 0);
            sum += (d2 * (float)v - nm2) * x[g * 64 + 32 + l];
        }
        is += 2;
        u1 <<= 2;
        u2 <<= 2;
    }
    return sum;
}

API void gko_dequant_q8_k(const uint8_t *b, float *out) {
    float d;
    memcpy(&d, b, 4);
    const int8_t *qs = (const int8_t *)(b + 4);
    for (int i = 0; i < 256; i++) out[i] = d * (float)qs[i];
}
static float dot_q8_k(const uint8_t *b, const float *x) {
    float d;
    memcpy(&d, b, 4);
    const int8_t *qs = (const int8_t *)(b + 4);
    float sum = 0.0f;
    for (int i = 0; i < 256; i++) sum += (d * (float)qs[i]) * x[i];
    return sum;
}

API void gko_dequant_q4_0(const uint8_t *b, float *out) {
    const float d = rd_f16(b);
    for (int j = 0; j < 16; j++) {
        const float lo = (float)(b[2 + j] & 0x0F), hi = (float)(b[2 + j] >> 4);
        out[j] = d * (lo - 8.0f);
        out[j + 16] = d * (hi - 8.0f);
    }
}
static float dot_q4_0(const uint8_t *b, const float *x) {
    const float d = rd_f16(b);
    float sum = 0.0f;
    for (int j = 0; j < 16; j++) {
        const float lo = (float)(b[2 + j] & 0x0F), hi = (float)(b[2 + j] >> 4);
        sum += d * (lo - 8.0f) * x[j];
        sum += d * (hi - 8.0f) * x[j + 16];
    }
    return sum;
}

API void gko_dequant_q5_0(const uint8_t *b, float *out) {
    const float d = rd_f16(b);
    const uint32_t qh = (uint32_t)b[2] | ((uint32_t)b[3] << 8) | ((uint32_t)b[4] << 16) | ((uint32_t)b[5] << 24);
    for (int j = 0; j < 16; j++) {
        const uint32_t lo = b[6 + j] & 0x0F, hi = b[6 + j] >> 4;
        const uint32_t bl = ((qh >> j) & 1) << 4, bh = ((qh >> (j + 16)) & 1) << 4;
        out[j] = d * ((float)(lo | bl) - 16.0f);
        out[j + 16] = d * ((float)(hi | bh) - 16.0f);
    }
}
static float dot_q5_0(const uint8_t *b, const float *x) {
    const float d = rd_f16(b);
    const uint32_t qh = (uint32_t)b[2] | ((uint32_t)b[3] << 8) | ((uint32_t)b[4] << 16) | ((uint32_t)b[5] << 24);
    float sum = 0.0f;
    for (int j = 0; j < 16; j++) {
        const uint32_t lo = b[6 + j] & 0x0F, hi = b[6 + j] >> 4;
        const uint32_t bl = ((qh >> j) & 1) << 4, bh = ((qh >> (j + 16)) & 1) << 4;
        sum += d * ((float)(lo | bl) - 16.0f) * x[j];
        sum += d * ((float)(hi | bh) - 16.0f) * x[j + 16];
    }
    return sum;
}

/* one block of any GGUF format handled above -> block_size floats; 0 on success */
API int gko_dequant_block(int qt, const uint8_t *b, float *out) {
    switch (qt) {
        case GKO_Q4K: gko_dequant_q4_k(b, out); return 0;
        case GKO_Q8_0: gko_dequant_q8_0(b, out); return 0;
        case GKO_Q6K: gko_dequant_q6_k(b, out); return 0;
        case GKO_Q5K: gko_dequant_q5_k(b, out); return 0;
        case GKO_Q8K: gko_dequant_q8_k(b, out); return 0;
        case GKO_Q4_0: gko_dequant_q4_0(b, out); return 0;
        case GKO_Q5_0: gko_dequant_q5_0(b, out); return 0;
    }
    return -5;
}

/* ------------------------------------------------------------------------------------------
 * Matmul drivers.
 *
 * quant_matmul_inner, src/cpu_kernels/mod.rs:443-486: weight rows = m, batch columns = n,
 * input [k, n] row-major, output [m, n] row-major, per (row, col) the block dots are added in
 * increasing block order.  kquant_matmul (Q4_K) and classic_matmul (Q8_0) both land here
 * (src/cpu_kernels/mod.rs:3226-3394).
 * ---------------------------------------------------------------------------------------- */
typedef float (*dot_fn)(const uint8_t *, const float *);

static void matmul_inner_rows(const uint8_t *w, const float *xt, float *out, size_t m, size_t n, size_t k,
                              size_t bb, size_t bs, dot_fn dot, size_t row0, size_t row1) {
    const size_t bpr = k / bs;
    for (size_t j = 0; j < n; j++) {
        const float *in_row = xt + j * k;
        for (size_t i = row0; i < row1; i++) {
            float sum = 0.0f;
            for (size_t b = 0; b < bpr; b++) sum += dot(w + (i * bpr + b) * bb, in_row + b * bs);
            out[i * n + j] = sum;
        }
    }
    (void)m;
}

struct mm_job {
    const uint8_t *w; const float *xt; float *out; size_t m, n, k, bb, bs; dot_fn dot; size_t r0, r1;
};
static void *mm_worker(void *p) {
    struct mm_job *j = (struct mm_job *)p;
    matmul_inner_rows(j->w, j->xt, j->out, j->m, j->n, j->k, j->bb, j->bs, j->dot, j->r0, j->r1);
    return NULL;
}

static int quant_matmul(const uint8_t *w, const float *input, float *out, int qt, size_t m, size_t n,
                        size_t k, int threads) {
    size_t bb, bs;
    dot_fn dot;
    if (qt == GKO_Q4K) { bb = 144; bs = 256; dot = dot_q4_k; }
    else if (qt == GKO_Q8_0) { bb = 34; bs = 32; dot = dot_q8_0; }
    else if (qt == GKO_Q6K) { bb = 210; bs = 256; dot = dot_q6_k; }
    else if (qt == GKO_Q5K) { bb = 176; bs = 256; dot = dot_q5_k; }
    else if (qt == GKO_Q8K) { bb = 292; bs = 256; dot = dot_q8_k; }
    else if (qt == GKO_Q4_0) { bb = 18; bs = 32; dot = dot_q4_0; }
    else if (qt == GKO_Q5_0) { bb = 22; bs = 32; dot = dot_q5_0; }
    else return -5;
    if (k % bs) return -1;
    float *xt = (float *)malloc(sizeof(float) * k * n);
    if (!xt) return -2;
    for (size_t p = 0; p < k; p++)
        for (size_t j = 0; j < n; j++) xt[j * k + p] = input[p * n + j];
    if (threads <= 1) {
        matmul_inner_rows(w, xt, out, m, n, k, bb, bs, dot, 0, m);
    } else {
        /* Row-parallel courtesy variant: the reference quant path is single-threaded. */
        if (threads > 256) threads = 256;
        pthread_t tid[256];
        struct mm_job jobs[256];
        for (int c = 0; c < threads; c++) {
            struct mm_job j = {w, xt, out, m, n, k, bb, bs, dot, m * (size_t)c / (size_t)threads,
                               m * (size_t)(c + 1) / (size_t)threads};
            jobs[c] = j;
            pthread_create(&tid[c], NULL, mm_worker, &jobs[c]);
        }
        for (int c = 0; c < threads; c++) pthread_join(tid[c], NULL);
    }
    free(xt);
    return 0;
}

/* Kernels::kquant_matmul / classic_matmul, f32 element type. */
API int gko_quant_matmul(const uint8_t *w, const float *input, float *out, int qt, size_t m, size_t n,
                         size_t k) {
    return quant_matmul(w, input, out, qt, m, n, k, 1);
}
API int gko_quant_matmul_mt(const uint8_t *w, const float *input, float *out, int qt, size_t m, size_t n,
                            size_t k, int threads) {
    return quant_matmul(w, input, out, qt, m, n, k, threads);
}

/* Kernels::gemm_q4, src/cpu_kernels/mod.rs:2934-2981: m = batch rows, n = output features,
 * input [m,k], output [m,n], weight row j = k/256 Q4_K blocks; result times scales[j]
 * (n_scales == n), scales[0] (n_scales == 1) or 1. */
API int gko_gemm_q4(const uint8_t *w, const float *input, float *out, const float *scales, size_t n_scales,
                    size_t m, size_t n, size_t k) {
    if (k % 256) return -1;
    const size_t bpr = k / 256;
    for (size_t i = 0; i < m; i++) {
        const float *in_row = input + i * k;
        for (size_t j = 0; j < n; j++) {
            float sum = 0.0f;
            for (size_t b = 0; b < bpr; b++) sum += dot_q4_k(w + (j * bpr + b) * 144, in_row + b * 256);
            const float s = (n_scales == n) ? scales[j] : (n_scales == 1 ? scales[0] : 1.0f);
            out[i * n + j] = sum * s;
        }
    }
    return 0;
}

/* Kernels::gemv_q4, src/cpu_kernels/mod.rs:2888-2909: one weight row of n elements. */
API float gko_gemv_q4(const uint8_t *w, const float *input, float scale, size_t n) {
    float sum = 0.0f;
    for (size_t b = 0; b < n / 256; b++) sum += dot_q4_k(w + b * 144, input + b * 256);
    return sum * scale;
}

/* Kernels::gemm_q8 / gemv_q8, src/cpu_kernels/mod.rs:2983-3031, 2910-2932: the same two loops over Q8_K blocks. */
API int gko_gemm_q8(const uint8_t *w, const float *input, float *out, const float *scales, size_t n_scales,
                    size_t m, size_t n, size_t k) {
    if (k % 256) return -1;
    const size_t bpr = k / 256;
    for (size_t i = 0; i < m; i++) {
        const float *in_row = input + i * k;
        for (size_t j = 0; j < n; j++) {
            float sum = 0.0f;
            for (size_t b = 0; b < bpr; b++) sum += dot_q8_k(w + (j * bpr + b) * 292, in_row + b * 256);
            const float s = (n_scales == n) ? scales[j] : (n_scales == 1 ? scales[0] : 1.0f);
            out[i * n + j] = sum * s;
        }
    }
    return 0;
}
API float gko_gemv_q8(const uint8_t *w, const float *input, float scale, size_t n) {
    float sum = 0.0f;
    for (size_t b = 0; b < n / 256; b++) sum += dot_q8_k(w + b * 292, input + b * 256);
    return sum * scale;
}

/* quantize_from_fp32, QuantFormat::Int8PerTensor (src/compiler/quant_convert.rs:17-20,165-177): scale = max|x| / 127,
 * q = (x / scale).round().clamp(-128, 127) as i8 — Rust's round() is half away from zero and `as i8` turns NaN
 * (an all-zero input: 0 / 0) into 0.  Returns the scale. */
API float gko_quantize_int8_per_tensor(const float *x, int8_t *q, size_t count) {
    float max_abs = 0.0f;
    for (size_t i = 0; i < count; i++) {
        const float a = fabsf(x[i]);
        if (a > max_abs) max_abs = a;  /* f32::max ignores NaN operands */
    }
    const float scale = max_abs / 127.0f;
    for (size_t i = 0; i < count; i++) {
        float v = roundf(x[i] / scale);
        if (v != v) v = 0.0f;
        if (v < -128.0f) v = -128.0f;
        if (v > 127.0f) v = 127.0f;
        q[i] = (int8_t)v;
    }
    return scale;
}

/* scalar_gemm loop order, scalar-ops/src/blas.rs:116-135: for i, for j, acc = sum_p a[i,p]*b[p,j].
 * Here b is the dequantised weight held row-major as [n, k] (b[p,j] = wd[j*k+p]) so the
 * accumulation over p is the same sequence of products. */
API void gko_gemm_f32_nt(const float *a, const float *wd, float *c, size_t m, size_t n, size_t k) {
    for (size_t i = 0; i < m; i++)
        for (size_t j = 0; j < n; j++) {
            float acc = 0.0f;
            const float *ar = a + i * k, *wr = wd + j * k;
            for (size_t p = 0; p < k; p++) acc += ar[p] * wr[p];
            c[i * n + j] = acc;
        }
}

/* f64-accumulated truth of the same product, for error reporting. */
API void gko_gemm_f64_nt(const float *a, const float *wd, double *c, size_t m, size_t n, size_t k) {
    for (size_t i = 0; i < m; i++)
        for (size_t j = 0; j < n; j++) {
            double acc = 0.0;
            const float *ar = a + i * k, *wr = wd + j * k;
            for (size_t p = 0; p < k; p++) acc += (double)ar[p] * (double)wr[p];
            c[i * n + j] = acc;
        }
}

/* ---- mixture-of-experts conventions --------------------------------------------------------- */

/* scalar_topk, scalar-ops/src/moe.rs:59-115.  output: indices [seq*top_k] (u32 bit patterns in f32 slots), then
 * weights [seq*top_k].  Insertion with a strict '>' into a list that starts at -inf / index 0; weights are
 * value * (1 / sum), inv_sum = 0 when sum <= 0. */
API void gko_scalar_topk(const float *gate_probs, float *output, size_t seq_len, size_t num_experts, size_t top_k) {
    float *idx_base = output, *wt_base = output + seq_len * top_k;
    for (size_t s = 0; s < seq_len; s++) {
        const float *row = gate_probs + s * num_experts;
        uint32_t ti[64];
        float tv[64];
        for (size_t i = 0; i < top_k; i++) { ti[i] = 0; tv[i] = -INFINITY; }
        for (size_t e = 0; e < num_experts; e++) {
            const float val = row[e];
            size_t pos = top_k;
            for (size_t ki = 0; ki < top_k; ki++)
                if (val > tv[ki]) { pos = ki; break; }
            if (pos < top_k) {
                for (size_t ki = top_k - 1; ki > pos; ki--) { ti[ki] = ti[ki - 1]; tv[ki] = tv[ki - 1]; }
                ti[pos] = (uint32_t)e;
                tv[pos] = val;
            }
        }
        float sum = 0.0f;
        for (size_t ki = 0; ki < top_k; ki++) sum += tv[ki];
        const float inv_sum = sum > 0.0f ? 1.0f / sum : 0.0f;
        for (size_t ki = 0; ki < top_k; ki++) {
            memcpy(idx_base + s * top_k + ki, &ti[ki], 4);
            wt_base[s * top_k + ki] = tv[ki] * inv_sum;
        }
    }
}

/* scalar_weighted_sum, scalar-ops/src/moe.rs:127-157: output zeroed, then for s, for ki: output[s, :] += w * row,
 * row = expert_outputs[expert][s].  rows == NULL: the reference's [expert][seq][hidden] buffer.  rows != NULL: the
 * same sum over a buffer of grouped rows, rows[s*top_k+ki] naming the row (negative = skipped) — the layout
 * gllmk_gemm_grouped writes. */
API void gko_scalar_weighted_sum(const float *expert_outputs, const float *indices, const float *weights, const int64_t *rows,
                                 float *output, size_t seq_len, size_t hidden, size_t top_k) {
    for (size_t i = 0; i < seq_len * hidden; i++) output[i] = 0.0f;
    for (size_t s = 0; s < seq_len; s++)
        for (size_t ki = 0; ki < top_k; ki++) {
            const float w = weights[s * top_k + ki];
            const float *row;
            if (rows) {
                if (rows[s * top_k + ki] < 0) continue;
                row = expert_outputs + (size_t)rows[s * top_k + ki] * hidden;
            } else {
                uint32_t e;
                memcpy(&e, indices + s * top_k + ki, 4);
                row = expert_outputs + ((size_t)e * seq_len + s) * hidden;
            }
            for (size_t d = 0; d < hidden; d++) output[s * hidden + d] += w * row[d];
        }
}

/* Full-matrix decode to f32 [n, k] with the per-format block decoders above.
 * MXFP4 uses the split form (blocks + scales) of src/quant_mxfp4.rs:72; NVFP4 needs `global`. */
API int gko_dequant_matrix(int qt, const uint8_t *blocks, const uint8_t *scales, float global, size_t n,
                           size_t k, int mx_block, float *out) {
    if (qt == GKO_Q4K) {
        if (k % 256) return -1;
        for (size_t b = 0; b < n * (k / 256); b++) gko_dequant_q4_k(blocks + b * 144, out + b * 256);
    } else if (qt == GKO_Q8_0) {
        if (k % 32) return -1;
        for (size_t b = 0; b < n * (k / 32); b++) gko_dequant_q8_0(blocks + b * 34, out + b * 32);
    } else if (qt == GKO_MXFP4) {
        if (mx_block <= 0 || (mx_block & 1) || k % (size_t)mx_block) return -1;
        gko_dequant_mxfp4(blocks, scales, out, n * (k / (size_t)mx_block), (size_t)mx_block);
    } else if (qt == GKO_NVFP4) {
        if (k % 64) return -1;
        gko_dequant_nvfp4(blocks, global, out, n * (k / 64));
    } else if (qt == GKO_Q6K || qt == GKO_Q5K || qt == GKO_Q8K || qt == GKO_Q4_0 || qt == GKO_Q5_0) {
        const size_t bs = (size_t)gko_block_size(qt, 0), bb = (size_t)gko_block_bytes(qt, 0);
        if (k % bs) return -1;
        for (size_t b = 0; b < n * (k / bs); b++) gko_dequant_block(qt, blocks + b * bb, out + b * bs);
    } else return -5;
    return 0;
}

/* ------------------------------------------------------------------------------------------
 * bench_quant kernels, scalar-ops/src/quant_matmul.rs:16-29, 36-53, 114-134, 142-171, 188-219.
 * Simplified formats (per-row / per-column f32 scale, nibble-8, "f32 d + i8 body" blocks).
 * ---------------------------------------------------------------------------------------- */
API float gko_scalar_gemv_q8(const int8_t *w, const float *x, float scale, size_t n) {
    float acc = 0.0f;
    for (size_t i = 0; i < n; i++) acc += (float)w[i] * x[i];
    return acc * scale;
}
API float gko_scalar_gemv_q4(const uint8_t *w, const float *x, float scale, size_t n) {
    float acc = 0.0f;
    for (size_t i = 0; i < n / 2; i++) {
        const uint8_t byte = w[i];
        const int8_t lo = (int8_t)(byte & 0x0F) - 8, hi = (int8_t)(byte >> 4) - 8;
        acc += (float)lo * x[2 * i];
        acc += (float)hi * x[2 * i + 1];
    }
    return acc * scale;
}
/* The row loop benches/bench_quant.rs:84-96 times: one scalar_gemv_q4 call per output row. */
API void gko_bench_gemv_q4_rows(const uint8_t *w, const float *x, const float *scales, float *out, size_t n, size_t k) {
    for (size_t j = 0; j < n; j++) out[j] = gko_scalar_gemv_q4(w + j * (k / 2), x, scales[j], k);
}
/* benches/bench_quant.rs:40-58: one scalar_gemv_q8 call per output row. */
API void gko_bench_gemv_q8_rows(const int8_t *w, const float *x, const float *scales, float *out, size_t n, size_t k) {
    for (size_t j = 0; j < n; j++) out[j] = gko_scalar_gemv_q8(w + j * k, x, scales[j], k);
}
API void gko_scalar_gemm_q8(const int8_t *w, const float *x, float *out, const float *scales, size_t m,
                            size_t n, size_t k) {
    for (size_t i = 0; i < m; i++)
        for (size_t j = 0; j < n; j++) {
            float acc = 0.0f;
            for (size_t p = 0; p < k; p++) acc += (float)w[p * n + j] * x[i * k + p];
            out[i * n + j] = acc * scales[j];
        }
}
API void gko_scalar_gemm_q4(const uint8_t *w, const float *x, float *out, const float *scales, size_t m,
                            size_t n, size_t k) {
    for (size_t i = 0; i < m; i++)
        for (size_t j = 0; j < n; j++) {
            float acc = 0.0f;
            for (size_t p = 0; p < k; p++) {
                const uint8_t byte = w[p * (n / 2) + j / 2];
                const int8_t q = (j % 2 == 0) ? (int8_t)(byte & 0x0F) - 8 : (int8_t)(byte >> 4) - 8;
                acc += (float)q * x[i * k + p];
            }
            out[i * n + j] = acc * scales[j];
        }
}
API void gko_scalar_kquant_matmul(const uint8_t *w, const float *x, float *out, size_t block_bytes,
                                  size_t block_size, size_t m, size_t n, size_t k) {
    const size_t bpr = k / block_size, row_bytes = bpr * block_bytes;
    for (size_t i = 0; i < m; i++)
        for (size_t j = 0; j < n; j++) {
            float acc = 0.0f;
            const uint8_t *row = w + j * row_bytes;
            for (size_t b = 0; b < bpr; b++) {
                const uint8_t *blk = row + b * block_bytes;
                float d;
                memcpy(&d, blk, 4);
                for (size_t e = 0; e < block_size; e++)
                    acc += (float)(int8_t)blk[4 + e] * d * x[i * k + b * block_size + e];
            }
            out[i * n + j] = acc;
        }
}

/* ------------------------------------------------------------------------------------------
 * Quantizers.  The reference has no f32 -> Q4_K / Q8_0 / MXFP4 / NVFP4 encoder (its only
 * quantizer is per-tensor amax/127, src/compiler/quant_convert.rs:17-31,165-205).  These are
 * this project's own deterministic inverses of the decoders above; parity is defined on the
 * packed bytes they produce, which feed both the oracle and the CUDA path.
 * ---------------------------------------------------------------------------------------- */
static inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

API void gko_quantize_q4_k(const float *x, uint8_t *out, size_t num_blocks) {
    for (size_t blk = 0; blk < num_blocks; blk++) {
        const float *xb = x + blk * 256;
        uint8_t *b = out + blk * 144;
        float s[8], o[8], smax = 0.0f, omax = 0.0f;
        for (int j = 0; j < 8; j++) {
            float lo = 0.0f, hi = 0.0f;
            for (int l = 0; l < 32; l++) {
                const float v = xb[j * 32 + l];
                if (v < lo) lo = v;
                if (v > hi) hi = v;
            }
            s[j] = (hi - lo) / 15.0f;
            o[j] = -lo;
            if (s[j] > smax) smax = s[j];
            if (o[j] > omax) omax = o[j];
        }
        const uint16_t dh = gko_f32_to_f16(smax / 63.0f), mh = gko_f32_to_f16(omax / 63.0f);
        const float d = gko_f16_to_f32(dh), dmin = gko_f16_to_f32(mh);
        int sc[8], mn[8];
        for (int j = 0; j < 8; j++) {
            sc[j] = (d > 0.0f) ? clampi((int)rintf(s[j] / d), 0, 63) : 0;
            mn[j] = (dmin > 0.0f) ? clampi((int)rintf(o[j] / dmin), 0, 63) : 0;
        }
        memcpy(b, &dh, 2);
        memcpy(b + 2, &mh, 2);
        uint8_t *sb = b + 4;
        for (int j = 0; j < 4; j++) {
            sb[j] = (uint8_t)(sc[j] | ((sc[j + 4] >> 4) << 6));
            sb[j + 4] = (uint8_t)(mn[j] | ((mn[j + 4] >> 4) << 6));
            sb[j + 8] = (uint8_t)((sc[j + 4] & 15) | ((mn[j + 4] & 15) << 4));
        }
        uint8_t q[256];
        for (int j = 0; j < 8; j++) {
            const float ds = d * (float)sc[j], off = dmin * (float)mn[j];
            for (int l = 0; l < 32; l++)
                q[j * 32 + l] = (ds > 0.0f) ? (uint8_t)clampi((int)rintf((xb[j * 32 + l] + off) / ds), 0, 15) : 0;
        }
        for (int g = 0; g < 4; g++)
            for (int l = 0; l < 32; l++) b[16 + 32 * g + l] = (uint8_t)(q[64 * g + l] | (q[64 * g + 32 + l] << 4));
    }
}

API void gko_quantize_q8_0(const float *x, uint8_t *out, size_t num_blocks) {
    for (size_t blk = 0; blk < num_blocks; blk++) {
        const float *xb = x + blk * 32;
        uint8_t *b = out + blk * 34;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) { const float a = fabsf(xb[i]); if (a > amax) amax = a; }
        const uint16_t dh = gko_f32_to_f16(amax / 127.0f);
        const float d = gko_f16_to_f32(dh);
        memcpy(b, &dh, 2);
        for (int i = 0; i < 32; i++) {
            int q = (d > 0.0f) ? (int)roundf(xb[i] / d) : 0; /* round half away, quant_convert.rs:170-176 */
            b[2 + i] = (uint8_t)(int8_t)clampi(q, -127, 127);
        }
    }
}

static const float E2M1_MAG[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

/* nearest E2M1 code to v (sign from v); ties go to the code with an even low bit. */
static inline uint8_t nearest_e2m1(float v) {
    const float a = fabsf(v);
    int best = 0;
    float bd = a;
    for (int c = 1; c < 8; c++) {
        const float dist = fabsf(a - E2M1_MAG[c]);
        if (dist < bd || (dist == bd && (c & 1) == 0)) { bd = dist; best = c; }
    }
    if (best == 0) return 0;
    return (uint8_t)(best | ((v < 0.0f) ? 8 : 0));
}

/* MXFP4, split form: blocks (block_size/2 bytes per block) and one E8M0 byte per block. */
API void gko_quantize_mxfp4(const float *x, uint8_t *blocks, uint8_t *scales, size_t num_blocks,
                            size_t block_size) {
    for (size_t blk = 0; blk < num_blocks; blk++) {
        const float *xb = x + blk * block_size;
        float amax = 0.0f;
        for (size_t i = 0; i < block_size; i++) { const float a = fabsf(xb[i]); if (a > amax) amax = a; }
        int byte = 127;
        if (amax > 0.0f) {
            int e = (int)ceilf(log2f(amax / 6.0f));
            while (ldexpf(6.0f, e) < amax) e++;           /* guard against log2f rounding */
            while (e > -200 && ldexpf(6.0f, e - 1) >= amax) e--;
            byte = clampi(e + 127, 1, 254);
        }
        scales[blk] = (uint8_t)byte;
        const float inv = ldexpf(1.0f, 127 - byte);
        for (size_t i = 0; i < block_size / 2; i++) {
            const uint8_t lo = nearest_e2m1(xb[2 * i] * inv), hi = nearest_e2m1(xb[2 * i + 1] * inv);
            blocks[blk * (block_size / 2) + i] = (uint8_t)(lo | (hi << 4));
        }
    }
}

/* NVFP4: global = amax_tensor / (6*448) chosen by the caller (gko_nvfp4_global); per 16 a UE4M3
 * scale from gko_f32_to_e4m3(amax_sub / (6*global)). `row_len` elements form one contiguous run of
 * 64-element blocks. */
API float gko_nvfp4_global(const float *x, size_t count) {
    float amax = 0.0f;
    for (size_t i = 0; i < count; i++) { const float a = fabsf(x[i]); if (a > amax) amax = a; }
    return amax > 0.0f ? amax / (6.0f * 448.0f) : 1.0f;
}
API void gko_quantize_nvfp4(const float *x, float global, uint8_t *out, size_t num_blocks) {
    for (size_t blk = 0; blk < num_blocks; blk++) {
        const float *xb = x + blk * 64;
        uint8_t *b = out + blk * 36;
        for (int sub = 0; sub < 4; sub++) {
            float amax = 0.0f;
            for (int i = 0; i < 16; i++) { const float a = fabsf(xb[sub * 16 + i]); if (a > amax) amax = a; }
            const uint8_t sb = (uint8_t)(gko_f32_to_e4m3(amax / (6.0f * global)) & 0x7F);
            b[sub] = sb;
            const float s = global * gko_e4m3_to_f32(sb);
            for (int i = 0; i < 8; i++) {
                uint8_t lo = 0, hi = 0;
                if (s > 0.0f) {
                    lo = nearest_e2m1(xb[sub * 16 + 2 * i] / s);
                    hi = nearest_e2m1(xb[sub * 16 + 2 * i + 1] / s);
                }
                b[4 + sub * 8 + i] = (uint8_t)(lo | (hi << 4));
            }
        }
    }
}

/* GGUF inline MXFP4 (17-byte blocks, scale first; src/quant.rs:66-76,427) <-> split form. */
API void gko_mxfp4_split(const uint8_t *inline_blocks, uint8_t *blocks, uint8_t *scales, size_t num_blocks,
                         size_t block_size) {
    const size_t bpb = block_size / 2;
    for (size_t i = 0; i < num_blocks; i++) {
        scales[i] = inline_blocks[i * (bpb + 1)];
        memcpy(blocks + i * bpb, inline_blocks + i * (bpb + 1) + 1, bpb);
    }
}
