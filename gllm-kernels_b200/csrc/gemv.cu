// Decode path: fused dequantize + GEMV for M <= 16 tokens over the tiled Q4_K / Q8_0 layouts.
//
// The kernels are HBM-bound by design: each warp streams its 16-row tile of packed weights with
// 128-bit coalesced loads (512 contiguous bytes per warp instruction), unpacks nibbles / bytes to
// exact fp16 integers with one logic op + one half2 op per pair, and feeds them as the A operand
// of mma.sync.m16n8k16 (f32 accumulate).  The activations are the B operand: each token is split
// into an fp16 "hi" and a 2^11-scaled fp16 "lo" column (22 significant bits together) after a
// per-token power-of-two normalisation, so products are exact and all rounding happens in the
// f32 accumulators.  Using the tensor pipe for an M=1 product wastes MMA columns on purpose: what
// it buys is issue slots — a scalar-FMA formulation needs ~3 issue slots per nibble, more than the
// ~2.8 per nibble an SM has at full HBM rate.
//
// Q4_K algebra per 256-block and row (reference: k_quant.rs:502-547, sum of (d*sc*q - dmin*m)*x):
//     y += d * sum_sub sc_sub * (q . x)_sub  -  dmin * sum_sub m_sub * (sum x)_sub
// sc*q <= 945 and m <= 63 are exact in fp16; the per-sub-block sums of x are precomputed by the
// staging kernel and enter through one extra MMA per block.
#include "common.cuh"

namespace gllmk {

// ---------------------------------------------------------------------------------------------
// Activation staging: x (f32, strided) -> workspace
//   xs  : half [cols_pad][K]     column 2t = hi(token t), 2t+1 = lo(token t); for Q4_K each aligned
//                                quad of k is stored in order (0,2,1,3) to match the nibble unpack
//   ss  : half [cols_pad][K/32]  hi/lo split of the per-32 sums of the normalised token (Q4_K only)
//   tsc : float[16]              2^e per token, undoes the normalisation
// ---------------------------------------------------------------------------------------------
struct StageParams {
    const float *x;
    int64_t xst, xsk;
    int m;
    int64_t K;
    __half *xs;
    __half *ss;
    float *tsc;
    int perm;  // 1: Q4_K quad permutation + sums
};

__global__ void __launch_bounds__(256) stage_x_kernel(StageParams p) {
    __shared__ float red[8];
    // Let the dependent GEMV grid start streaming weights now; it waits (griddepcontrol.wait) for
    // this grid to finish before it touches the workspace.
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const int tok = blockIdx.y;
    const float *xr = p.x + (int64_t)tok * p.xst;
    // per-token amax (every CTA of the token recomputes it; K*4 bytes from L2)
    float amax = 0.0f;
    for (int64_t k = threadIdx.x; k < p.K; k += 256) amax = fmaxf(amax, fabsf(xr[k * p.xsk]));
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int i = 1; i < 8; i++) amax = fmaxf(amax, red[i]);
    int e = 0;
    if (amax > 0.0f && amax < __int_as_float(0x7F800000)) {
        (void)frexpf(amax, &e);  // amax = f * 2^e, f in [0.5, 1)
        e = max(-126, min(126, e));
    }
    const float inv = ldexpf(1.0f, -e);
    if (blockIdx.x == 0 && threadIdx.x == 0) p.tsc[tok] = ldexpf(1.0f, e);
    // NaN anywhere in the token must reach every output like in the reference (fmaxf drops NaNs,
    // but the converted values themselves carry it into the MMA).
    const int64_t k0 = ((int64_t)blockIdx.x * 256 + threadIdx.x) * 4;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    const bool live = k0 < p.K;
    if (live) {
#pragma unroll
        for (int i = 0; i < 4; i++) v[i] = xr[(k0 + i) * p.xsk] * inv;
    }
    __half hi[4], lo[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        hi[i] = __float2half_rn(v[i]);
        lo[i] = __float2half_rn((v[i] - __half2float(hi[i])) * 2048.0f);
    }
    if (live) {
        __half *ph = p.xs + (int64_t)(2 * tok) * p.K + k0;
        __half *pl = p.xs + (int64_t)(2 * tok + 1) * p.K + k0;
        if (p.perm) {
            *reinterpret_cast<uint2 *>(ph) = make_uint2(
                (uint32_t)__half_as_ushort(hi[0]) | ((uint32_t)__half_as_ushort(hi[2]) << 16),
                (uint32_t)__half_as_ushort(hi[1]) | ((uint32_t)__half_as_ushort(hi[3]) << 16));
            *reinterpret_cast<uint2 *>(pl) = make_uint2(
                (uint32_t)__half_as_ushort(lo[0]) | ((uint32_t)__half_as_ushort(lo[2]) << 16),
                (uint32_t)__half_as_ushort(lo[1]) | ((uint32_t)__half_as_ushort(lo[3]) << 16));
        } else {
            *reinterpret_cast<uint2 *>(ph) = make_uint2(
                (uint32_t)__half_as_ushort(hi[0]) | ((uint32_t)__half_as_ushort(hi[1]) << 16),
                (uint32_t)__half_as_ushort(hi[2]) | ((uint32_t)__half_as_ushort(hi[3]) << 16));
            *reinterpret_cast<uint2 *>(pl) = make_uint2(
                (uint32_t)__half_as_ushort(lo[0]) | ((uint32_t)__half_as_ushort(lo[1]) << 16),
                (uint32_t)__half_as_ushort(lo[2]) | ((uint32_t)__half_as_ushort(lo[3]) << 16));
        }
    }
    if (p.perm) {
        float s = (v[0] + v[1]) + (v[2] + v[3]);
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        if (live && (threadIdx.x & 7) == 0) {
            const __half sh = __float2half_rn(s);
            const __half sl = __float2half_rn((s - __half2float(sh)) * 2048.0f);
            p.ss[(int64_t)(2 * tok) * (p.K >> 5) + (k0 >> 5)] = sh;
            p.ss[(int64_t)(2 * tok + 1) * (p.K >> 5) + (k0 >> 5)] = sl;
        }
    }
}

// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }
__device__ __forceinline__ uint4 ldg_stream(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
// (w & mask) | 0x64006400: two fp16 values 1024 + field
__device__ __forceinline__ uint32_t magic_and(uint32_t w, uint32_t mask) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;\n" : "=r"(r) : "r"(w), "r"(mask), "r"(0x64006400u));
    return r;
}

struct GemvParams {
    const uint4 *qs;
    const uint4 *aux;     // Q4_K headers / Q8_0 scales (as uint4 = 8 halves)
    const __half *xs;
    const __half *ss;
    const float *tsc;
    float *y;
    int64_t yst, ysr;
    const float *row_scales;
    int64_t n_row_scales;
    int64_t n, K;
    int ntiles;  // 16-row tiles
    int nb;      // Q4_K: 256-blocks per row;  Q8_0: 32-blocks per row
    int nb8;     // Q8_0: groups of 8 blocks
    int m;
    int ksplit;  // warps per row tile: 1, 2, 4, 8
};

// Per-row Q4_K scale constants for the sub-block pair (2t, 2t+1) owned by this thread.
struct Q4KRow {
    __half2 mul_lo, add_lo, mul_hi, add_hi;  // fma constants turning 1024+q / 1024+16q into sc*q
    uint32_t mm;                             // half2 {m_2t, m_2t+1}
    float d, dmin;
};
__device__ __forceinline__ Q4KRow q4k_row(const uint4 h, const int t) {
    Q4KRow r;
    const int sh = (t & 1) * 16;
    const uint32_t A0 = (h.y >> sh) & 0xFFFFu, A1 = (h.z >> sh) & 0xFFFFu, A2 = (h.w >> sh) & 0xFFFFu;
    uint32_t scp, mp;  // [sub 2t | sub 2t+1 << 8]
    if (t < 2) {
        scp = A0 & 0x3F3Fu;
        mp = A1 & 0x3F3Fu;
    } else {
        scp = (A2 & 0x0F0Fu) | ((A0 >> 2) & 0x3030u);
        mp = ((A2 >> 4) & 0x0F0Fu) | ((A1 >> 2) & 0x3030u);
    }
    const __half2 k1024 = __float2half2_rn(1024.0f);
    const __half2 sca = __hsub2(u32_as_h2(__byte_perm(scp, 0x64u, 0x4040)), k1024);
    const __half2 scb = __hsub2(u32_as_h2(__byte_perm(scp, 0x64u, 0x4141)), k1024);
    r.mm = h2_as_u32(__hsub2(u32_as_h2(__byte_perm(mp, 0x64u, 0x4140)), k1024));
    r.mul_lo = sca;
    r.add_lo = __hmul2(sca, __float2half2_rn(-1024.0f));
    r.mul_hi = __hmul2(scb, __float2half2_rn(0.0625f));
    r.add_hi = __hmul2(scb, __float2half2_rn(-64.0f));
    r.d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xFFFFu)));
    r.dmin = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
    return r;
}

template <int NT>
__global__ void __launch_bounds__(256) gemv_q4k_kernel(const GemvParams p) {
    __shared__ float red[8][NT * 4][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int S = p.ksplit;
    const int tile = blockIdx.x * (8 / S) + warp / S;
    const int split = warp % S;
    float tot[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) tot[nt][0] = tot[nt][1] = tot[nt][2] = tot[nt][3] = 0.f;

    // Everything up to here is independent of the staging kernel's output.
    asm volatile("griddepcontrol.wait;\n" ::: "memory");

    if (tile < p.ntiles) {
        const int b0 = (int)((int64_t)p.nb * split / S), b1 = (int)((int64_t)p.nb * (split + 1) / S);
        const uint4 *qp = p.qs + ((size_t)tile * p.nb + b0) * 128 + lane;
        const uint4 *hp = p.aux + ((size_t)tile * p.nb + b0) * 16 + g;
        const int ncols = 2 * p.m;
        uint4 q[4], h[2];
        if (b0 < b1) {
#pragma unroll
            for (int j = 0; j < 4; j++) q[j] = ldg_stream(qp + 32 * j);
            h[0] = __ldg(hp);
            h[1] = __ldg(hp + 8);
        }
        for (int b = b0; b < b1; b++) {
            uint4 qn[4], hn[2];
            if (b + 1 < b1) {
#pragma unroll
                for (int j = 0; j < 4; j++) qn[j] = ldg_stream(qp + 128 + 32 * j);
                hn[0] = __ldg(hp + 16);
                hn[1] = __ldg(hp + 24);
            }
            const Q4KRow r0 = q4k_row(h[0], t), r1 = q4k_row(h[1], t);
            float cq[NT][4], cm[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                cq[nt][0] = cq[nt][1] = cq[nt][2] = cq[nt][3] = 0.f;
                cm[nt][0] = cm[nt][1] = cm[nt][2] = cm[nt][3] = 0.f;
            }
            // mins: one MMA per n-tile, A = {m_2t, m_2t+1} in k-slots (2t, 2t+1), upper k half zero
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int col = nt * 8 + g;
                uint32_t sb = 0;
                if (col < ncols)
                    sb = __ldg(reinterpret_cast<const uint32_t *>(p.ss + (size_t)col * (p.K >> 5) + 8 * b + 2 * t));
                mma16816(cm[nt], r0.mm, r1.mm, 0u, 0u, sb, 0u);
            }
#pragma unroll
            for (int jj = 0; jj < 2; jj++) {
                const uint32_t w0[4] = {q[jj].x, q[jj].y, q[jj].z, q[jj].w};              // row g
                const uint32_t w1[4] = {q[2 + jj].x, q[2 + jj].y, q[2 + jj].z, q[2 + jj].w};  // row g + 8
                uint32_t alo[4][4], ahi[4][4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint32_t s0 = w0[i] >> 8, s1 = w1[i] >> 8;
                    alo[i][0] = h2_as_u32(__hfma2(u32_as_h2(magic_and(w0[i], 0x000F000Fu)), r0.mul_lo, r0.add_lo));
                    alo[i][1] = h2_as_u32(__hfma2(u32_as_h2(magic_and(w1[i], 0x000F000Fu)), r1.mul_lo, r1.add_lo));
                    alo[i][2] = h2_as_u32(__hfma2(u32_as_h2(magic_and(s0, 0x000F000Fu)), r0.mul_lo, r0.add_lo));
                    alo[i][3] = h2_as_u32(__hfma2(u32_as_h2(magic_and(s1, 0x000F000Fu)), r1.mul_lo, r1.add_lo));
                    ahi[i][0] = h2_as_u32(__hfma2(u32_as_h2(magic_and(w0[i], 0x00F000F0u)), r0.mul_hi, r0.add_hi));
                    ahi[i][1] = h2_as_u32(__hfma2(u32_as_h2(magic_and(w1[i], 0x00F000F0u)), r1.mul_hi, r1.add_hi));
                    ahi[i][2] = h2_as_u32(__hfma2(u32_as_h2(magic_and(s0, 0x00F000F0u)), r0.mul_hi, r0.add_hi));
                    ahi[i][3] = h2_as_u32(__hfma2(u32_as_h2(magic_and(s1, 0x00F000F0u)), r1.mul_hi, r1.add_hi));
                }
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const int col = nt * 8 + g;
                    uint4 xl[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
                    uint4 xh[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
                    if (col < ncols) {
                        const uint4 *xp = reinterpret_cast<const uint4 *>(p.xs + (size_t)col * p.K +
                                                                          (size_t)256 * b + 64 * t + 16 * jj);
                        xl[0] = __ldg(xp);
                        xl[1] = __ldg(xp + 1);
                        xh[0] = __ldg(xp + 4);
                        xh[1] = __ldg(xp + 5);
                    }
                    mma16816(cq[nt], alo[0][0], alo[0][1], alo[0][2], alo[0][3], xl[0].x, xl[0].y);
                    mma16816(cq[nt], alo[1][0], alo[1][1], alo[1][2], alo[1][3], xl[0].z, xl[0].w);
                    mma16816(cq[nt], alo[2][0], alo[2][1], alo[2][2], alo[2][3], xl[1].x, xl[1].y);
                    mma16816(cq[nt], alo[3][0], alo[3][1], alo[3][2], alo[3][3], xl[1].z, xl[1].w);
                    mma16816(cq[nt], ahi[0][0], ahi[0][1], ahi[0][2], ahi[0][3], xh[0].x, xh[0].y);
                    mma16816(cq[nt], ahi[1][0], ahi[1][1], ahi[1][2], ahi[1][3], xh[0].z, xh[0].w);
                    mma16816(cq[nt], ahi[2][0], ahi[2][1], ahi[2][2], ahi[2][3], xh[1].x, xh[1].y);
                    mma16816(cq[nt], ahi[3][0], ahi[3][1], ahi[3][2], ahi[3][3], xh[1].z, xh[1].w);
                }
            }
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                tot[nt][0] = fmaf(r0.d, cq[nt][0], tot[nt][0]);
                tot[nt][1] = fmaf(r0.d, cq[nt][1], tot[nt][1]);
                tot[nt][2] = fmaf(r1.d, cq[nt][2], tot[nt][2]);
                tot[nt][3] = fmaf(r1.d, cq[nt][3], tot[nt][3]);
                tot[nt][0] = fmaf(-r0.dmin, cm[nt][0], tot[nt][0]);
                tot[nt][1] = fmaf(-r0.dmin, cm[nt][1], tot[nt][1]);
                tot[nt][2] = fmaf(-r1.dmin, cm[nt][2], tot[nt][2]);
                tot[nt][3] = fmaf(-r1.dmin, cm[nt][3], tot[nt][3]);
            }
#pragma unroll
            for (int j = 0; j < 4; j++) q[j] = qn[j];
            h[0] = hn[0];
            h[1] = hn[1];
            qp += 128;
            hp += 16;
        }
    }
    // reduce the k-splits of a tile (fixed order -> deterministic), then write
    if (S > 1) {
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) red[warp][nt * 4 + i][lane] = tot[nt][i];
        __syncthreads();
        if (split == 0) {
            for (int s = 1; s < S; s++)
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
#pragma unroll
                    for (int i = 0; i < 4; i++) tot[nt][i] += red[warp + s][nt * 4 + i][lane];
        }
    }
    if (split == 0 && tile < p.ntiles) {
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const int tok = nt * 4 + t;
            if (tok < p.m) {
                const float ts = p.tsc[tok];
#pragma unroll
                for (int hrow = 0; hrow < 2; hrow++) {
                    const int64_t row = (int64_t)tile * 16 + g + 8 * hrow;
                    if (row < p.n) {
                        float v = fmaf(tot[nt][2 * hrow + 1], 1.0f / 2048.0f, tot[nt][2 * hrow]) * ts;
                        if (p.n_row_scales == 1) v *= p.row_scales[0];
                        else if (p.n_row_scales > 1) v *= p.row_scales[row];
                        p.y[(int64_t)tok * p.yst + row * p.ysr] = v;
                    }
                }
            }
        }
    }
}

// Q8_0: per 32-block and row  y += d * (q . x)   (classic.rs:870-881)
template <int NT>
__global__ void __launch_bounds__(256) gemv_q80_kernel(const GemvParams p) {
    __shared__ float red[8][NT * 4][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int S = p.ksplit;
    const int tile = blockIdx.x * (8 / S) + warp / S;
    const int split = warp % S;
    float tot[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) tot[nt][0] = tot[nt][1] = tot[nt][2] = tot[nt][3] = 0.f;

    asm volatile("griddepcontrol.wait;\n" ::: "memory");

    if (tile < p.ntiles) {
        const int g0 = (int)((int64_t)p.nb8 * split / S), g1 = (int)((int64_t)p.nb8 * (split + 1) / S);
        const int ncols = 2 * p.m;
        const __half2 k1152 = __float2half2_rn(1152.0f);
        for (int g8 = g0; g8 < g1; g8++) {
            const uint4 *dp = p.aux + ((size_t)tile * p.nb8 + g8) * 16;
            const uint4 dg0 = __ldg(dp + g), dg1 = __ldg(dp + g + 8);
            const uint32_t dw0[4] = {dg0.x, dg0.y, dg0.z, dg0.w}, dw1[4] = {dg1.x, dg1.y, dg1.z, dg1.w};
            const int nblk = min(8, p.nb - 8 * g8);
            const uint4 *qp = p.qs + ((size_t)tile * p.nb + 8 * g8) * 32 + lane;
            uint4 q[8];
#pragma unroll
            for (int bb = 0; bb < 8; bb++)
                if (bb < nblk) q[bb] = ldg_stream(qp + 32 * bb);
#pragma unroll
            for (int bb = 0; bb < 8; bb++) {
                if (bb < nblk) {
                    const int b = 8 * g8 + bb;
                    const uint32_t u0 = q[bb].x ^ 0x80808080u, u1 = q[bb].y ^ 0x80808080u;
                    const uint32_t u2 = q[bb].z ^ 0x80808080u, u3 = q[bb].w ^ 0x80808080u;
                    // MMA 1: bytes 0..3 of each row's 8; MMA 2: bytes 4..7
                    const uint32_t a0 = h2_as_u32(__hsub2(u32_as_h2(__byte_perm(u0, 0x64646464u, 0x4140)), k1152));
                    const uint32_t a2 = h2_as_u32(__hsub2(u32_as_h2(__byte_perm(u0, 0x64646464u, 0x4342)), k1152));
                    const uint32_t a1 = h2_as_u32(__hsub2(u32_as_h2(__byte_perm(u2, 0x64646464u, 0x4140)), k1152));
                    const uint32_t a3 = h2_as_u32(__hsub2(u32_as_h2(__byte_perm(u2, 0x64646464u, 0x4342)), k1152));
                    const uint32_t c0 = h2_as_u32(__hsub2(u32_as_h2(__byte_perm(u1, 0x64646464u, 0x4140)), k1152));
                    const uint32_t c2 = h2_as_u32(__hsub2(u32_as_h2(__byte_perm(u1, 0x64646464u, 0x4342)), k1152));
                    const uint32_t c1 = h2_as_u32(__hsub2(u32_as_h2(__byte_perm(u3, 0x64646464u, 0x4140)), k1152));
                    const uint32_t c3 = h2_as_u32(__hsub2(u32_as_h2(__byte_perm(u3, 0x64646464u, 0x4342)), k1152));
                    const uint32_t dsel0 = dw0[bb >> 1], dsel1 = dw1[bb >> 1];
                    const float d0 = __half2float(
                        __ushort_as_half((unsigned short)((bb & 1) ? (dsel0 >> 16) : (dsel0 & 0xFFFFu))));
                    const float d1 = __half2float(
                        __ushort_as_half((unsigned short)((bb & 1) ? (dsel1 >> 16) : (dsel1 & 0xFFFFu))));
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        const int col = nt * 8 + g;
                        uint4 xv = make_uint4(0, 0, 0, 0);
                        if (col < ncols)
                            xv = __ldg(reinterpret_cast<const uint4 *>(p.xs + (size_t)col * p.K + (size_t)32 * b + 8 * t));
                        float c[4] = {0.f, 0.f, 0.f, 0.f};
                        mma16816(c, a0, a1, a2, a3, xv.x, xv.y);
                        mma16816(c, c0, c1, c2, c3, xv.z, xv.w);
                        tot[nt][0] = fmaf(d0, c[0], tot[nt][0]);
                        tot[nt][1] = fmaf(d0, c[1], tot[nt][1]);
                        tot[nt][2] = fmaf(d1, c[2], tot[nt][2]);
                        tot[nt][3] = fmaf(d1, c[3], tot[nt][3]);
                    }
                }
            }
        }
    }
    if (S > 1) {
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) red[warp][nt * 4 + i][lane] = tot[nt][i];
        __syncthreads();
        if (split == 0) {
            for (int s = 1; s < S; s++)
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
#pragma unroll
                    for (int i = 0; i < 4; i++) tot[nt][i] += red[warp + s][nt * 4 + i][lane];
        }
    }
    if (split == 0 && tile < p.ntiles) {
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const int tok = nt * 4 + t;
            if (tok < p.m) {
                const float ts = p.tsc[tok];
#pragma unroll
                for (int hrow = 0; hrow < 2; hrow++) {
                    const int64_t row = (int64_t)tile * 16 + g + 8 * hrow;
                    if (row < p.n) {
                        float v = fmaf(tot[nt][2 * hrow + 1], 1.0f / 2048.0f, tot[nt][2 * hrow]) * ts;
                        if (p.n_row_scales == 1) v *= p.row_scales[0];
                        else if (p.n_row_scales > 1) v *= p.row_scales[row];
                        p.y[(int64_t)tok * p.yst + row * p.ysr] = v;
                    }
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// workspace: xs [32][K] half | ss [32][K/32] half | tsc [16] float
size_t gemv_ws_bytes(const Weight *w, int m) {
    (void)m;
    const size_t K = (size_t)w->k;
    return align_up(32 * K * 2, 256) + align_up(32 * (K / 32) * 2, 256) + 256;
}

template <typename Kern>
static cudaError_t launch_pdl(Kern kern, dim3 grid, dim3 block, cudaStream_t s, bool pdl, const GemvParams &p) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

int32_t gemv_launch(Ctx *c, const Weight *w, const float *x, int64_t xst, int64_t xsk, int m, float *y, int64_t yst,
                    int64_t ysr, const float *row_scales, int64_t n_row_scales, cudaStream_t s) {
    if (w->qt != GLLMK_QUANT_Q4K && w->qt != GLLMK_QUANT_Q8_0)
        return fail(c, GLLMK_STATUS_UNSUPPORTED, "gemv: quant type %d has no decode kernel", w->qt);
    int32_t rc = ensure_ws(c, gemv_ws_bytes(w, m));
    if (rc) return rc;
    const size_t K = (size_t)w->k;
    char *base = static_cast<char *>(c->ws);
    __half *xs = reinterpret_cast<__half *>(base);
    __half *ss = reinterpret_cast<__half *>(base + align_up(32 * K * 2, 256));
    float *tsc = reinterpret_cast<float *>(base + align_up(32 * K * 2, 256) + align_up(32 * (K / 32) * 2, 256));

    StageParams sp{x, xst, xsk, m, (int64_t)K, xs, ss, tsc, w->qt == GLLMK_QUANT_Q4K ? 1 : 0};
    dim3 sgrid((unsigned)((K + 1023) / 1024), (unsigned)m);
    stage_x_kernel<<<sgrid, 256, 0, s>>>(sp);
    GK_CUDA(c, cudaGetLastError());

    GemvParams p{};
    p.qs = static_cast<const uint4 *>(w->qs);
    p.aux = static_cast<const uint4 *>(w->aux);
    p.xs = xs;
    p.ss = ss;
    p.tsc = tsc;
    p.y = y;
    p.yst = yst;
    p.ysr = ysr;
    p.row_scales = row_scales;
    p.n_row_scales = row_scales ? n_row_scales : 0;
    p.n = w->n;
    p.K = w->k;
    p.ntiles = (int)(w->n_pad / 16);
    p.nb = (int)w->nb;
    p.nb8 = (int)w->nb8;
    p.m = m;
    const int units = (w->qt == GLLMK_QUANT_Q4K) ? p.nb : p.nb8;  // what a k-split divides
    int S = (int)c->gemv_ksplit;
    if (S != 1 && S != 2 && S != 4 && S != 8) {
        S = 1;
        while (S < 8 && (int64_t)p.ntiles * S < 4096) S *= 2;
    }
    while (S > 1 && S > units) S /= 2;
    p.ksplit = S;
    const unsigned grid = (unsigned)((p.ntiles + (8 / S) - 1) / (8 / S));
    const int NT = (2 * m + 7) / 8;
    const bool pdl = c->gemv_pdl != 0;
    cudaError_t e;
    if (w->qt == GLLMK_QUANT_Q4K) {
        switch (NT) {
            case 1: e = launch_pdl(gemv_q4k_kernel<1>, grid, 256, s, pdl, p); break;
            case 2: e = launch_pdl(gemv_q4k_kernel<2>, grid, 256, s, pdl, p); break;
            case 3: e = launch_pdl(gemv_q4k_kernel<3>, grid, 256, s, pdl, p); break;
            default: e = launch_pdl(gemv_q4k_kernel<4>, grid, 256, s, pdl, p); break;
        }
    } else {
        switch (NT) {
            case 1: e = launch_pdl(gemv_q80_kernel<1>, grid, 256, s, pdl, p); break;
            case 2: e = launch_pdl(gemv_q80_kernel<2>, grid, 256, s, pdl, p); break;
            case 3: e = launch_pdl(gemv_q80_kernel<3>, grid, 256, s, pdl, p); break;
            default: e = launch_pdl(gemv_q80_kernel<4>, grid, 256, s, pdl, p); break;
        }
    }
    GK_CUDA(c, e);
    return GLLMK_STATUS_OK;
}

}  // namespace gllmk
