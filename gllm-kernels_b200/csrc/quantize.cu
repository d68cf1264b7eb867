// On-device quantizers f32 -> Q4_K / Q8_0 / MXFP4 / NVFP4 blocks in the reference's byte formats.
// The reference ships no encoder for these formats; the rules below are this library's own and
// are the exact inverse conventions of the decoders (k_quant.rs:7-56, classic.rs:860-868,
// quant_mxfp4.rs:72-109, quant.rs:77-86).  All arithmetic is plain IEEE f32 (the library is
// compiled with -fmad=false) so a CPU implementation of the same rules produces identical bytes.
#include "common.cuh"

namespace gllmk {

__device__ __forceinline__ int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

// nearest E2M1 code; ties go to the code with an even low bit; zero keeps code 0 (+0)
__device__ __forceinline__ uint32_t nearest_e2m1(float v) {
    const float mags[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    const float a = fabsf(v);
    int best = 0;
    float bd = a;
#pragma unroll
    for (int c = 1; c < 8; c++) {
        const float dist = fabsf(a - mags[c]);
        if (dist < bd || (dist == bd && (c & 1) == 0)) { bd = dist; best = c; }
    }
    if (best == 0) return 0u;
    return (uint32_t)best | ((v < 0.0f) ? 8u : 0u);
}

// f32_to_e4m3, src/compiler/codegen/vm/numerical_sim.rs:2751-2808, for v >= 0
__device__ __forceinline__ uint32_t f32_to_ue4m3(float v) {
    if (v != v) return 0x7Fu;
    float a = fabsf(v);
    if (a > 448.0f) a = 448.0f;
    if (a == 0.0f) return 0u;
    const uint32_t ab = (uint32_t)__float_as_int(a);
    int e4 = (int)(ab >> 23) - 127 + 7;
    const uint32_t m23 = ab & 0x7FFFFFu;
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
    e4 = clampi(e4, 0, 15);
    m3 = clampi(m3, 0, 7);
    return ((uint32_t)e4 << 3) | (uint32_t)m3;
}

// ---- Q4_K: one warp per 256-block, lane l handles elements l, 32+l, ... (one per sub-block) ----
__global__ void __launch_bounds__(256) quantize_q4k_kernel(const float *__restrict__ x, uint8_t *__restrict__ out,
                                                            size_t nblocks) {
    const size_t blk = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (blk >= nblocks) return;
    const float *xb = x + blk * 256;
    uint8_t *b = out + blk * 144;
    float v[8], s[8], o[8];
    float smax = 0.0f, omax = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        v[j] = xb[j * 32 + lane];
        float lo = fminf(v[j], 0.0f), hi = fmaxf(v[j], 0.0f);
#pragma unroll
        for (int d = 16; d; d >>= 1) {
            lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, d));
            hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, d));
        }
        s[j] = (hi - lo) / 15.0f;
        o[j] = -lo;
        smax = fmaxf(smax, s[j]);
        omax = fmaxf(omax, o[j]);
    }
    const __half dh = __float2half_rn(smax / 63.0f), mh = __float2half_rn(omax / 63.0f);
    const float d = __half2float(dh), dmin = __half2float(mh);
    int sc[8], mn[8];
    uint32_t q[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        sc[j] = (d > 0.0f) ? clampi((int)rintf(s[j] / d), 0, 63) : 0;
        mn[j] = (dmin > 0.0f) ? clampi((int)rintf(o[j] / dmin), 0, 63) : 0;
        const float ds = d * (float)sc[j], off = dmin * (float)mn[j];
        q[j] = (ds > 0.0f) ? (uint32_t)clampi((int)rintf((v[j] + off) / ds), 0, 15) : 0u;
    }
    if (lane == 0) {
        *reinterpret_cast<unsigned short *>(b) = __half_as_ushort(dh);
        *reinterpret_cast<unsigned short *>(b + 2) = __half_as_ushort(mh);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            b[4 + j] = (uint8_t)(sc[j] | ((sc[j + 4] >> 4) << 6));
            b[8 + j] = (uint8_t)(mn[j] | ((mn[j + 4] >> 4) << 6));
            b[12 + j] = (uint8_t)((sc[j + 4] & 15) | ((mn[j + 4] & 15) << 4));
        }
    }
#pragma unroll
    for (int g = 0; g < 4; g++) b[16 + 32 * g + lane] = (uint8_t)(q[2 * g] | (q[2 * g + 1] << 4));
}

// ---- Q8_0: one warp per 32-block ----
__global__ void __launch_bounds__(256) quantize_q80_kernel(const float *__restrict__ x, uint8_t *__restrict__ out,
                                                            size_t nblocks) {
    const size_t blk = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (blk >= nblocks) return;
    const float v = x[blk * 32 + lane];
    float amax = fabsf(v);
#pragma unroll
    for (int d = 16; d; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    const __half dh = __float2half_rn(amax / 127.0f);
    const float d = __half2float(dh);
    const int q = (d > 0.0f) ? clampi((int)roundf(v / d), -127, 127) : 0;
    uint8_t *b = out + blk * 34;
    if (lane == 0) *reinterpret_cast<unsigned short *>(b) = __half_as_ushort(dh);
    b[2 + lane] = (uint8_t)(int8_t)q;
}

// ---- MXFP4 (block 32): one warp per block, split output (16 nibble bytes + 1 E8M0 byte) ----
__global__ void __launch_bounds__(256) quantize_mxfp4_kernel(const float *__restrict__ x, uint8_t *__restrict__ blocks,
                                                              uint8_t *__restrict__ scales, size_t nblocks) {
    const size_t blk = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (blk >= nblocks) return;
    const float v = x[blk * 32 + lane];
    float amax = fabsf(v);
#pragma unroll
    for (int d = 16; d; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    int byte = 127;
    if (amax > 0.0f) {
        int p;
        const float f = frexpf(amax, &p);  // smallest e with 6 * 2^e >= amax
        const int e = (f <= 0.75f) ? p - 3 : p - 2;
        byte = clampi(e + 127, 1, 254);
    }
    const float inv = ldexpf(1.0f, 127 - byte);
    const uint32_t code = nearest_e2m1(v * inv);
    const uint32_t hi = __shfl_down_sync(0xffffffffu, code, 1);
    if ((lane & 1) == 0) blocks[blk * 16 + (lane >> 1)] = (uint8_t)(code | (hi << 4));
    if (lane == 0) scales[blk] = (uint8_t)byte;
}

// ---- NVFP4 (block 64 = 4 x 16): one warp per block, lane handles elements 2*lane, 2*lane+1 ----
__global__ void __launch_bounds__(256) quantize_nvfp4_kernel(const float *__restrict__ x, uint8_t *__restrict__ out,
                                                              const float *__restrict__ global_ptr, size_t nblocks) {
    const size_t blk = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (blk >= nblocks) return;
    const float global = *global_ptr;
    const float2 v = *reinterpret_cast<const float2 *>(x + blk * 64 + 2 * lane);
    float amax = fmaxf(fabsf(v.x), fabsf(v.y));
#pragma unroll
    for (int d = 4; d; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));  // 8 lanes = 16 el
    const uint32_t sb = f32_to_ue4m3(amax / (6.0f * global)) & 0x7Fu;
    const float s = global * e4m3_to_f32(sb);
    uint32_t lo = 0, hi = 0;
    if (s > 0.0f) {
        lo = nearest_e2m1(v.x / s);
        hi = nearest_e2m1(v.y / s);
    }
    uint8_t *b = out + blk * 36;
    if ((lane & 7) == 0) b[lane >> 3] = (uint8_t)sb;
    b[4 + lane] = (uint8_t)(lo | (hi << 4));
}

// amax over a tensor -> global = amax / (6 * 448), 1 when all zero.  Two small passes.
__global__ void __launch_bounds__(256) amax_partial_kernel(const float *__restrict__ x, size_t count,
                                                            float *__restrict__ partial) {
    __shared__ float red[8];
    float a = 0.0f;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < count; i += (size_t)gridDim.x * 256)
        a = fmaxf(a, fabsf(x[i]));
#pragma unroll
    for (int d = 16; d; d >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, d));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = a;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < 8; i++) a = fmaxf(a, red[i]);
        partial[blockIdx.x] = a;
    }
}
__global__ void amax_final_kernel(const float *__restrict__ partial, int n, float *__restrict__ global_out) {
    float a = 0.0f;
    for (int i = threadIdx.x; i < n; i += 32) a = fmaxf(a, partial[i]);
#pragma unroll
    for (int d = 16; d; d >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, d));
    if (threadIdx.x == 0) *global_out = (a > 0.0f) ? a / (6.0f * 448.0f) : 1.0f;
}

int32_t quantize_launch(Ctx *c, int32_t qt, const float *x, int64_t rows, int64_t k, int mx_block, void *blocks,
                        void *scales, float *global_scale, cudaStream_t s) {
    const size_t count = (size_t)rows * (size_t)k;
    if (qt == GLLMK_QUANT_Q4K) {
        const size_t nb = count / 256;
        quantize_q4k_kernel<<<(unsigned)((nb + 7) / 8), 256, 0, s>>>(x, (uint8_t *)blocks, nb);
    } else if (qt == GLLMK_QUANT_Q8_0) {
        const size_t nb = count / 32;
        quantize_q80_kernel<<<(unsigned)((nb + 7) / 8), 256, 0, s>>>(x, (uint8_t *)blocks, nb);
    } else if (qt == GLLMK_QUANT_MXFP4) {
        if (mx_block != 32) return fail(c, GLLMK_STATUS_UNSUPPORTED, "quantize: MXFP4 block_size %d (only 32)", mx_block);
        const size_t nb = count / 32;
        quantize_mxfp4_kernel<<<(unsigned)((nb + 7) / 8), 256, 0, s>>>(x, (uint8_t *)blocks, (uint8_t *)scales, nb);
    } else if (qt == GLLMK_QUANT_NVFP4) {
        // scratch behind the status word (16 KiB block owned by the context): global scale + partial maxima
        float *gdev = reinterpret_cast<float *>(c->status_dev) + 64;
        float *partial = gdev + 64;
        if (*global_scale > 0.0f) {
            GK_CUDA(c, cudaMemcpyAsync(gdev, global_scale, sizeof(float), cudaMemcpyHostToDevice, s));
        } else {
            const int nblk = (int)((count + 256 * 64 - 1) / (256 * 64) < 1024 ? (count + 256 * 64 - 1) / (256 * 64) : 1024);
            amax_partial_kernel<<<nblk, 256, 0, s>>>(x, count, partial);
            amax_final_kernel<<<1, 32, 0, s>>>(partial, nblk, gdev);
        }
        const size_t nb = count / 64;
        quantize_nvfp4_kernel<<<(unsigned)((nb + 7) / 8), 256, 0, s>>>(x, (uint8_t *)blocks, gdev, nb);
        if (!(*global_scale > 0.0f)) {
            GK_CUDA(c, cudaMemcpyAsync(global_scale, gdev, sizeof(float), cudaMemcpyDeviceToHost, s));
            GK_CUDA(c, cudaStreamSynchronize(s));
        }
    } else {
        return fail(c, GLLMK_STATUS_UNSUPPORTED, "quantize: unknown quant type %d", qt);
    }
    GK_CUDA(c, cudaGetLastError());
    return GLLMK_STATUS_OK;
}

}  // namespace gllmk
