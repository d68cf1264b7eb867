// Decode path: fused dequantize + GEMV for M <= 16 tokens over the tiled Q4_K / Q8_0 layouts.
//
// The kernels are HBM-bound by design and built around the instruction budget that leaves: at full
// HBM rate an SM has fewer than three issue slots per weight nibble.  So
//   * the packed integers are never converted: a 32-bit word of Q4_K nibbles masked with 0x0F0F0F0F (a
//     Q8_0 word as it is) IS an A-fragment register of mma.sync.m16n8k32 (u8/s8 x s8 -> s32);
//   * activations are the B operand as two int8 "digit" columns per token: per 256-element block
//     x = amax/127 * (d1 + d2/254) with |d1|, |d2| <= 127 (error <= amax * 1.6e-5), written once per
//     call by a small staging kernel, so every product is an exact integer;
//   * Q4_K's 6-bit sub-block scales multiply the s32 sub-block sums (one IMAD each) and only the per-block
//     totals are converted to f32 and multiplied by d, dmin and the activation scale.
// Weights stream through shared memory with bulk copies (cp.async.bulk + mbarrier), one 18.9 KB / 34.8 KB
// "super-chunk" (8 row tiles x one k-block) per stage, so the copy engine, not the warps, keeps HBM busy.
//
// Q4_K algebra per 256-block and row (reference: k_quant.rs:502-547, sum of (d*sc*q - dmin*m)*x):
//     y += d * sum_sub sc_sub * (q . x)_sub  -  dmin * sum_sub m_sub * (sum x)_sub
// Q8_0 per 32-block and row (classic.rs:870-881):  y += d * (q . x)
#include "common.cuh"

namespace gllmk {

constexpr int FMT_Q4K = 0, FMT_Q80 = 1, FMT_MXFP4 = 2, FMT_NVFP4 = 3;

// ---------------------------------------------------------------------------------------------
// Activation image: one slice per 256 elements of k, the exact bytes a CTA copies into shared memory.
//   [col < 2m][288 B] : int8 digits, column 2*tok = d1, 2*tok+1 = d2, natural k order (256 B used; the
//                       288-byte pitch makes the B-fragment reads bank-conflict free)
//   [col < 2m][16 B]  : per 32-element sub-block sums of the column's digits, S = 64*hi + lo:
//                       bytes 0..7 = hi (s8), bytes 8..15 = lo (0..63)
//   [tok < m] f32     : amax/127 of the token's block (NaN if the block holds a non-finite value),
//                       padded to 16 bytes
// ---------------------------------------------------------------------------------------------
__host__ __device__ inline uint32_t slice_bytes(int m) { return (uint32_t)(2 * m) * 304u + 16u * (uint32_t)((m + 3) / 4); }

struct StageParams {
    const float *x;
    const float *x_up;  // not null: the activation is silu(x[k]) * x_up[k] (SwiGLU of a gate || up product's halves)
    int64_t xst, xsk;
    int m;
    int64_t K;
    uint8_t *img;
    // exchange products: before x is read, wait (bounded) until every other rank has completed as many exchange
    // products as this rank has (its bands of the previous product have then landed in this rank's buffers)
    const uint32_t *xflags;  // this rank's flag words, or nullptr
    int nranks, rank;
    uint32_t spins;
    int *status;
};

__global__ void __launch_bounds__(256) stage_x_kernel(StageParams p) {
    __shared__ float wmax[8];
    __shared__ int wbad[8];
    // Let the dependent GEMV grid start streaming weights now; it waits (griddepcontrol.wait) for
    // this grid to finish before it touches the image.  This grid is itself launched early: it may
    // only read x and overwrite the image once everything before it in the stream has completed.
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    if (p.xflags) {
        // Everything before this grid in the stream is complete, so this rank's own epoch is final: thread q waits
        // for the q-th other rank to reach it.  A rank that never arrives costs `spins` probes, then status 32.
        if ((int)threadIdx.x < p.nranks - 1) {
            const int src = (int)threadIdx.x < p.rank ? (int)threadIdx.x : (int)threadIdx.x + 1;
            const uint32_t want = *reinterpret_cast<const volatile uint32_t *>(p.xflags + XF_EPOCH);  // L2, never a stale L1 line
            bool seen = false;
            for (uint32_t it = 0; it < p.spins && !seen; it++) {
                uint32_t v;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p.xflags + XF_FLAGS + src) : "memory");
                seen = (int32_t)(v - want) >= 0;
                if (!seen && it > 64) __nanosleep(100);
            }
            if (!seen) atomicExch(p.status, 32);
        }
        __syncthreads();
    }
    const int tok = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t k0 = ((int64_t)blockIdx.x * 256 + threadIdx.x) * 4;
    const float *xr = p.x + (int64_t)tok * p.xst;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (k0 < p.K) {
#pragma unroll
        for (int i = 0; i < 4; i++) v[i] = xr[(k0 + i) * p.xsk];
        if (p.x_up) {
            // swiglu (scalar-ops/src/activations.rs:57-66): out = g / (1 + exp(-g)) * u, in f32
            const float *ur = p.x_up + (int64_t)tok * p.xst;
#pragma unroll
            for (int i = 0; i < 4; i++) v[i] = (v[i] / (1.0f + expf(-v[i]))) * ur[(k0 + i) * p.xsk];
        }
    }
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    const float inf = __int_as_float(0x7F800000);
    int bad = !(fabsf(v[0]) < inf) || !(fabsf(v[1]) < inf) || !(fabsf(v[2]) < inf) || !(fabsf(v[3]) < inf);
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    bad = __any_sync(0xffffffffu, bad);
    if (lane == 0) { wmax[warp] = amax; wbad[warp] = bad; }
    __syncthreads();
    amax = fmaxf(wmax[warp & ~1], wmax[warp | 1]);  // a 256-block is two warps
    bad = wbad[warp & ~1] | wbad[warp | 1];
    // tiny blocks are pre-scaled by 2^64 so that 127/amax stays finite
    const float pre = amax < 1e-20f ? 18446744073709551616.0f : 1.0f;
    const float inv = (amax > 0.0f && !bad) ? 127.0f / (amax * pre) : 0.0f;
    int d1[4], d2[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float s = (v[i] * pre) * inv;
        const float r1 = fminf(fmaxf(rintf(s), -127.0f), 127.0f);
        const float r2 = fminf(fmaxf(rintf((s - r1) * 254.0f), -127.0f), 127.0f);
        d1[i] = (int)r1;
        d2[i] = (int)r2;
    }
    const bool inr = k0 < (((p.K + 255) >> 8) << 8);  // inside the last (zero-padded) slice
    uint8_t *slice = p.img + (k0 >> 8) * (int64_t)slice_bytes(p.m);
    const int kk = (int)(k0 & 255), sub = kk >> 5;
    const uint32_t w1 = (uint32_t)(d1[0] & 0xFF) | ((uint32_t)(d1[1] & 0xFF) << 8) | ((uint32_t)(d1[2] & 0xFF) << 16) |
                        ((uint32_t)(d1[3] & 0xFF) << 24);
    const uint32_t w2 = (uint32_t)(d2[0] & 0xFF) | ((uint32_t)(d2[1] & 0xFF) << 8) | ((uint32_t)(d2[2] & 0xFF) << 16) |
                        ((uint32_t)(d2[3] & 0xFF) << 24);
    // k beyond K inside the last slice is written as zero digits (v = 0 above)
    if (inr) {
        *reinterpret_cast<uint32_t *>(slice + (2 * tok) * 288 + kk) = w1;
        *reinterpret_cast<uint32_t *>(slice + (2 * tok + 1) * 288 + kk) = w2;
    }
    int s1 = d1[0] + d1[1] + d1[2] + d1[3], s2 = d2[0] + d2[1] + d2[2] + d2[3];
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    if (inr && (lane & 7) == 0) {
        uint8_t *sp = slice + (2 * p.m) * 288;
        sp[(2 * tok) * 16 + sub] = (uint8_t)(int8_t)(s1 >> 6);
        sp[(2 * tok) * 16 + 8 + sub] = (uint8_t)(s1 & 63);
        sp[(2 * tok + 1) * 16 + sub] = (uint8_t)(int8_t)(s2 >> 6);
        sp[(2 * tok + 1) * 16 + 8 + sub] = (uint8_t)(s2 & 63);
    }
    if (inr && (threadIdx.x & 63) == 0)
        reinterpret_cast<float *>(slice + (2 * p.m) * 304)[tok] = bad ? __int_as_float(0x7FC00000) : amax / 127.0f;
}

// ---------------------------------------------------------------------------------------------
// PTX helpers: integer tensor-core MMA, shared-memory loads, mbarrier + bulk copy (every wait bounded)
// ---------------------------------------------------------------------------------------------
template <bool A_SIGNED>
__device__ __forceinline__ void imma16832(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    if (A_SIGNED)
        asm volatile(
            "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
            : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
    else
        asm volatile(
            "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
            : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Slow path, out of line: bounded spin (a copy lands in microseconds, the bound is on the order of a
// second); false if the barrier never flipped.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity) {
    for (uint32_t it = 0; it < (1u << 22); it++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity);
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ uint32_t byte_of(uint32_t w, int i) { return __byte_perm(w, 0u, 0x4440u + (uint32_t)i); }

struct GemvParams {
    const uint8_t *chunks;  // weight plane (Q4K_CHUNK / Q80_CHUNK byte chunks, 8 per super-chunk; FP4: 16 KB tile images)
    const uint8_t *sf;      // FP4 scale-factor plane (1 KB / 2 KB of atoms per super-chunk)
    float wscale;           // FP4: per-tensor scale x 1/2 (the int8 codes are twice the E2M1 values)
    const uint8_t *img;     // activation image
    float *y;
    int64_t yst, ysr;
    float *ypeer[GLLMK_MAX_PEERS];  // the same element positions in other GPUs' buffers (peer-mapped), npeer of them
    int npeer;
    // exchange products: the CTA that finishes last advances this rank's epoch and
    // signals it to every rank
    uint32_t *xflags;                        // this rank's flag words, or nullptr
    uint32_t *xflags_peer[GLLMK_MAX_PEERS];
    int xrank;
    int ntiles;                              // row tiles of the launch (counters[ntiles] counts the CTAs that have finished)
    // fused staging (small shares): every CTA converts the activation slices of ITS k-steps itself, straight into shared
    // memory, instead of copying them from an image a staging kernel wrote — one launch less per product
    const float *x, *x_up;
    int64_t xst, xsk, K;
    int fuse_slices;                         // slices a CTA keeps (0: the image path)
    int xnranks;                             // exchange products: ranks to wait for before x is read
    uint32_t spins;
    const float *row_scales;
    int64_t n_row_scales;
    int64_t n;
    int nk;            // k-steps per row: Q4_K blocks of 256 / Q8_0 groups of 8 blocks
    int m;
    int64_t nsuper;    // tile groups * nk
    int per_cta;       // super-chunks per CTA: the first `rem` CTAs own per_cta + 1, the others per_cta
    int rem;
    int maxslot;       // partial-sum slots per tile
    float *partial;    // [tiles][maxslot][16 tokens][16 rows]
    int *counters;     // [tiles] arrivals, zero between launches
    int *status;       // device status word
};

// Fused staging pays when a CTA's share is a handful of k-steps (small matrices, row shards of a few thousand
// rows): the staging kernel's launch and the hand-over between the two grids then cost more than converting
// fuse_slices x m slices of 256 activations in every CTA.
constexpr int GEMV_FUSE_MAX_WORK = 10;  // slices x tokens a CTA converts itself at most
constexpr int GEMV_STAGES = 3;  // pipeline depth (stages of one super-chunk + its activation slice)
constexpr int GEMV_WARPS = 8;
constexpr int GEMV_ZERO = 512;  // zero region read by the lanes of unused MMA columns
template <int FMT>
__host__ __device__ constexpr int chunk_bytes() { return FMT == FMT_Q4K ? Q4K_CHUNK : (FMT == FMT_Q80 ? Q80_CHUNK : 2048); }
// FP4: a super-chunk is one tile image (128 rows x 256 k, 16 KB = 8 x 2048) plus its scale atoms
template <int FMT>
__host__ __device__ constexpr int sf_bytes() { return FMT == FMT_MXFP4 ? 1024 : (FMT == FMT_NVFP4 ? 2048 : 0); }
// shared memory: [GEMV_STAGES][8 chunks + slice] | zero [512] | full[GEMV_STAGES], empty[GEMV_STAGES]
template <int FMT>
static inline size_t gemv_smem_bytes(int m) {
    return (size_t)GEMV_STAGES * (GEMV_WARPS * chunk_bytes<FMT>() + sf_bytes<FMT>() + slice_bytes(m)) + GEMV_ZERO + 2 * GEMV_STAGES * 8;
}

template <int FMT>
static inline size_t gemv_smem_bytes_fused(int m, int nslices) {
    return (size_t)GEMV_STAGES * (GEMV_WARPS * chunk_bytes<FMT>() + sf_bytes<FMT>()) + (size_t)nslices * slice_bytes(m) + GEMV_ZERO +
           2 * GEMV_STAGES * 8;
}

// One value of an activation slice turned into its two digits by the whole CTA (thread = element of the 256-block,
// warp = 32-element sub-block), in the layout of the image above: the arithmetic of stage_x_kernel, element for element.
__device__ __forceinline__ void stage_value_in_cta(float v, int m, int tok, uint8_t *slice, float (*wmax)[8], int (*wbad)[8], int &par) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float amax = fabsf(v);
    const float inf = __int_as_float(0x7F800000);
    int bad = !(fabsf(v) < inf);
#pragma unroll
    for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    bad = __any_sync(0xffffffffu, bad);
    if (lane == 0) { wmax[par][warp] = amax; wbad[par][warp] = bad; }
    __syncthreads();  // the other parity's slots are rewritten only after the next barrier: one barrier per value
    amax = 0.f;
    bad = 0;
#pragma unroll
    for (int w = 0; w < 8; w++) { amax = fmaxf(amax, wmax[par][w]); bad |= wbad[par][w]; }
    par ^= 1;
    const float pre = amax < 1e-20f ? 18446744073709551616.0f : 1.0f;
    const float inv = (amax > 0.0f && !bad) ? 127.0f / (amax * pre) : 0.0f;
    const float sc = (v * pre) * inv;
    const float r1 = fminf(fmaxf(rintf(sc), -127.0f), 127.0f);
    const float r2 = fminf(fmaxf(rintf((sc - r1) * 254.0f), -127.0f), 127.0f);
    const int d1 = (int)r1, d2 = (int)r2;
    slice[(2 * tok) * 288 + tid] = (uint8_t)(int8_t)d1;
    slice[(2 * tok + 1) * 288 + tid] = (uint8_t)(int8_t)d2;
    int s1 = d1, s2 = d2;
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
        s2 += __shfl_xor_sync(0xffffffffu, s2, o);
    }
    if (lane == 0) {
        uint8_t *sp = slice + (2 * m) * 288;
        sp[(2 * tok) * 16 + warp] = (uint8_t)(int8_t)(s1 >> 6);
        sp[(2 * tok) * 16 + 8 + warp] = (uint8_t)(s1 & 63);
        sp[(2 * tok + 1) * 16 + warp] = (uint8_t)(int8_t)(s2 >> 6);
        sp[(2 * tok + 1) * 16 + 8 + warp] = (uint8_t)(s2 & 63);
    }
    if (tid == 0) reinterpret_cast<float *>(slice + (2 * m) * 304)[tok] = bad ? __int_as_float(0x7FC00000) : amax / 127.0f;
}

// ---- one 16-row x 256-k chunk of Q4_K -------------------------------------------------------
// ch: this warp's chunk in shared memory; xb[nt]: this lane's digit column (or the zero region);
// sb[nt]: its sub-block sums; xs[nt]: activation scale of the lane's token.  tot[nt][h]: row g + 8h.
template <int NT>
__device__ __forceinline__ void q4k_chunk(uint32_t ch, int lane, const uint32_t (&xb)[NT], const uint32_t (&sb)[NT],
                                          const float (&xs)[NT], float (&tot)[NT][2]) {
    const int g = lane >> 2, t = lane & 3;
    uint4 q[4];
#pragma unroll
    for (int pg = 0; pg < 4; pg++) q[pg] = lds128(ch + (pg * 32 + lane) * 16);
    const uint4 h0 = lds128(ch + 2048 + g * 16), h1 = lds128(ch + 2048 + (g + 8) * 16);
    const uint2 dd = lds64(ch + 2304 + g * 8);
    int acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0;
#pragma unroll
    for (int pg = 0; pg < 4; pg++) {
#pragma unroll
        for (int hs = 0; hs < 2; hs++) {
            const int sub = 2 * pg + hs;
            const uint32_t a0 = (hs ? q[pg].x >> 4 : q[pg].x) & 0x0F0F0F0Fu, a2 = (hs ? q[pg].y >> 4 : q[pg].y) & 0x0F0F0F0Fu;
            const uint32_t a1 = (hs ? q[pg].z >> 4 : q[pg].z) & 0x0F0F0F0Fu, a3 = (hs ? q[pg].w >> 4 : q[pg].w) & 0x0F0F0F0Fu;
            const int sc0 = (int)byte_of(sub < 4 ? h0.x : h0.y, sub & 3), sc1 = (int)byte_of(sub < 4 ? h1.x : h1.y, sub & 3);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const uint2 b = lds64(xb[nt] + 32 * sub);
                int c[4];
                imma16832<false>(c, a0, a1, a2, a3, b.x, b.y);
                acc[nt][0] += sc0 * c[0];
                acc[nt][1] += sc0 * c[1];
                acc[nt][2] += sc1 * c[2];
                acc[nt][3] += sc1 * c[3];
            }
        }
    }
    // mins: A = m_sub in k-slots 0..7 (rows g, g+8), B = the sub-block sums split as 64*hi + lo
    const uint32_t ma0 = t == 0 ? h0.z : (t == 1 ? h0.w : 0u), ma1 = t == 0 ? h1.z : (t == 1 ? h1.w : 0u);
    const __half2 dd0 = *reinterpret_cast<const __half2 *>(&dd.x), dd1 = *reinterpret_cast<const __half2 *>(&dd.y);
    const float d0 = __low2float(dd0), m0 = __high2float(dd0), d1 = __low2float(dd1), m1 = __high2float(dd1);
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        int chi[4], clo[4];
        imma16832<false>(chi, ma0, ma1, 0u, 0u, lds32(sb[nt] + 4 * (t & 1)), 0u);
        imma16832<false>(clo, ma0, ma1, 0u, 0u, lds32(sb[nt] + 8 + 4 * (t & 1)), 0u);
        const float k254 = 1.0f / 254.0f;
        const float f0 = fmaf((float)acc[nt][1], k254, (float)acc[nt][0]);
        const float f1 = fmaf((float)acc[nt][3], k254, (float)acc[nt][2]);
        const float n0 = fmaf((float)(64 * chi[1] + clo[1]), k254, (float)(64 * chi[0] + clo[0]));
        const float n1 = fmaf((float)(64 * chi[3] + clo[3]), k254, (float)(64 * chi[2] + clo[2]));
        tot[nt][0] = fmaf(xs[nt], fmaf(d0, f0, -(m0 * n0)), tot[nt][0]);
        tot[nt][1] = fmaf(xs[nt], fmaf(d1, f1, -(m1 * n1)), tot[nt][1]);
    }
}

// ---- one 16-row x 256-k chunk (8 blocks) of Q8_0; tot[nt][2h + digit] ------------------------
template <int NT>
__device__ __forceinline__ void q80_chunk(uint32_t ch, int lane, const uint32_t (&xb)[NT], const float (&xs)[NT],
                                          float (&tot)[NT][4]) {
    const int g = lane >> 2;
    const uint4 dg0 = lds128(ch + 4096 + g * 16), dg1 = lds128(ch + 4096 + (g + 8) * 16);
    const uint32_t dw0[4] = {dg0.x, dg0.y, dg0.z, dg0.w}, dw1[4] = {dg1.x, dg1.y, dg1.z, dg1.w};
    float cs[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) cs[nt][0] = cs[nt][1] = cs[nt][2] = cs[nt][3] = 0.f;
#pragma unroll
    for (int bb = 0; bb < 8; bb++) {
        const uint4 q = lds128(ch + (bb * 32 + lane) * 16);
        const __half2 h0 = *reinterpret_cast<const __half2 *>(&dw0[bb >> 1]), h1 = *reinterpret_cast<const __half2 *>(&dw1[bb >> 1]);
        const float d0 = (bb & 1) ? __high2float(h0) : __low2float(h0), d1 = (bb & 1) ? __high2float(h1) : __low2float(h1);
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const uint2 b = lds64(xb[nt] + 32 * bb);
            int c[4];
            imma16832<true>(c, q.x, q.z, q.y, q.w, b.x, b.y);
            cs[nt][0] = fmaf(d0, (float)c[0], cs[nt][0]);
            cs[nt][1] = fmaf(d0, (float)c[1], cs[nt][1]);
            cs[nt][2] = fmaf(d1, (float)c[2], cs[nt][2]);
            cs[nt][3] = fmaf(d1, (float)c[3], cs[nt][3]);
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int j = 0; j < 4; j++) tot[nt][j] = fmaf(xs[nt], cs[nt][j], tot[nt][j]);
}

// Completes this warp's tile: the last contributing CTA adds the partial sums in slot order (so the
// result does not depend on arrival order) and writes y.  Out of line: it runs once per row tile.
template <int NT>
__device__ __noinline__ void gemv_flush(const GemvParams &p, int tile, int slot, int nsl, float (&v)[NT][2]) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    bool finish = true;
    if (nsl > 1) {
        float *mine = p.partial + ((size_t)tile * p.maxslot + slot) * 256;
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            const int tok = nt * 4 + t;
            if (tok < p.m) {
                __stcg(mine + tok * 16 + g, v[nt][0]);
                __stcg(mine + tok * 16 + g + 8, v[nt][1]);
            }
        }
        __threadfence();
        __syncwarp();
        int arrived = 0;
        if (lane == 0) arrived = atomicAdd(p.counters + tile, 1);
        arrived = __shfl_sync(0xffffffffu, arrived, 0);
        finish = (arrived == nsl - 1);
        if (finish) {
            __threadfence();
            const float *base = p.partial + (size_t)tile * p.maxslot * 256;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const int tok = nt * 4 + t;
                float a0 = 0.f, a1 = 0.f;
                if (tok < p.m)
                    for (int s = 0; s < nsl; s++) {
                        a0 += __ldcg(base + s * 256 + tok * 16 + g);
                        a1 += __ldcg(base + s * 256 + tok * 16 + g + 8);
                    }
                v[nt][0] = a0;
                v[nt][1] = a1;
            }
            if (lane == 0) p.counters[tile] = 0;  // ready for the next launch
        }
    }
    if (!finish) return;
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        const int tok = nt * 4 + t;
        if (tok < p.m) {
#pragma unroll
            for (int hrow = 0; hrow < 2; hrow++) {
                const int64_t row = (int64_t)tile * 16 + g + 8 * hrow;
                if (row < p.n) {
                    float o = v[nt][hrow];
                    if (p.n_row_scales == 1) o *= p.row_scales[0];
                    else if (p.n_row_scales > 1) o *= p.row_scales[row];
                    const int64_t at = (int64_t)tok * p.yst + row * p.ysr;
                    p.y[at] = o;
                    // fused all-gather: the band also goes straight into the peers' copies of y over NVLink
                    for (int q = 0; q < p.npeer; q++) p.ypeer[q][at] = o;
                }
            }
        }
    }
}

// ---- FP4 (MXFP4 / NVFP4): 16 rows x 256 k of a swizzled tile image ------------------------------------
// Eight E2M1 codes of one word -> int8 values of TWICE the element (0, 1, 2, 3, 4, 6, 8, 12 with sign): byte
// tables through prmt (3-bit index), the sign picks between the positive and the negative table.
// lo = elements 0..3, hi = elements 4..7.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
__device__ __forceinline__ void fp4_to_s8(uint32_t w, uint32_t &lo, uint32_t &hi) {
    const uint32_t POS_A = 0x03020100u, POS_B = 0x0C080604u, NEG_A = 0xFDFEFF00u, NEG_B = 0xF4F8FAFCu;
    const uint32_t sel = w & 0x77777777u;
    const uint32_t te = (w << 4) & 0x80808080u;  // byte m, bit 7 = sign of nibble 2m
    const uint32_t to = w & 0x80808080u;         // byte m, bit 7 = sign of nibble 2m + 1
    // selector nibbles with bit 3 set replicate the chosen byte's sign bit: 0xFF where the element is negative
    const uint32_t m_lo = prmt(te, to, 0xD9C8u), m_hi = prmt(te, to, 0xFBEAu);
    lo = (prmt(POS_A, POS_B, sel) & ~m_lo) | (prmt(NEG_A, NEG_B, sel) & m_lo);
    hi = (prmt(POS_A, POS_B, sel >> 16) & ~m_hi) | (prmt(NEG_A, NEG_B, sel >> 16) & m_hi);
}
__device__ __forceinline__ float2 e4m3x2_to_f32(uint32_t two) {
    uint32_t h;
    asm("{\n.reg .b16 lo, hi;\nmov.b32 {lo, hi}, %1;\ncvt.rn.f16x2.e4m3x2 %0, lo;\n}\n" : "=r"(h) : "r"(two));
    return __half22float2(*reinterpret_cast<const __half2 *>(&h));
}
// st: the stage (tile image, then the scale atoms); the warp owns rows 16*warp .. +15 of the tile.  Lane
// (g, t) holds elements 8t..8t+7 of each 32-element block of rows g and g + 8: word t of 16-byte chunk bb.
// tot[nt][2h + digit] as for Q8_0.  NVFP4 has a scale per 16 elements = lanes t < 2 / t >= 2 of a block, so
// each block takes two MMAs with the other half's lanes supplying zeros.
template <int FMT, int NT>
__device__ __forceinline__ void fp4_chunk(uint32_t st, int warp, int lane, const uint32_t (&xb)[NT], const float (&xs)[NT],
                                          float (&tot)[NT][4]) {
    const int g = lane >> 2, t = lane & 3;
    const int r0 = 16 * warp + g;  // r0 & 7 == (r0 + 8) & 7 == g
    const uint32_t row0 = st + r0 * 128 + 4 * t, row1 = row0 + 8 * 128;
    const uint32_t sfa = st + 16384 + (r0 & 31) * 16 + (r0 >> 5) * 4;  // rows r0 and r0 + 8 share r >> 5
    float cs[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) cs[nt][0] = cs[nt][1] = cs[nt][2] = cs[nt][3] = 0.f;
    if constexpr (FMT == FMT_MXFP4) {
        // 8 scales per row: two atoms of 4
        const uint32_t s0w[2] = {lds32(sfa), lds32(sfa + 512)}, s1w[2] = {lds32(sfa + 8 * 16), lds32(sfa + 512 + 8 * 16)};
#pragma unroll
        for (int bb = 0; bb < 8; bb++) {
            uint32_t a0, a1, a2, a3;
            fp4_to_s8(lds32(row0 + ((bb ^ g) << 4)), a0, a2);
            fp4_to_s8(lds32(row1 + ((bb ^ g) << 4)), a1, a3);
            const float d0 = e8m0_to_f32((s0w[bb >> 2] >> (8 * (bb & 3))) & 0xFFu), d1 = e8m0_to_f32((s1w[bb >> 2] >> (8 * (bb & 3))) & 0xFFu);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const uint2 b = lds64(xb[nt] + 32 * bb);
                int c[4];
                imma16832<true>(c, a0, a1, a2, a3, b.x, b.y);
                cs[nt][0] = fmaf(d0, (float)c[0], cs[nt][0]);
                cs[nt][1] = fmaf(d0, (float)c[1], cs[nt][1]);
                cs[nt][2] = fmaf(d1, (float)c[2], cs[nt][2]);
                cs[nt][3] = fmaf(d1, (float)c[3], cs[nt][3]);
            }
        }
    } else {
        const bool first = t < 2;  // this lane's 8 elements belong to the block's first 16
#pragma unroll
        for (int bb = 0; bb < 8; bb++) {
            uint32_t a0, a1, a2, a3;
            fp4_to_s8(lds32(row0 + ((bb ^ g) << 4)), a0, a2);
            fp4_to_s8(lds32(row1 + ((bb ^ g) << 4)), a1, a3);
            // 16 scales per row: atom bb / 2, scales 2 * (bb % 2) and + 1
            const uint32_t s0 = lds32(sfa + (bb >> 1) * 512) >> (16 * (bb & 1)), s1 = lds32(sfa + (bb >> 1) * 512 + 8 * 16) >> (16 * (bb & 1));
            // two UE4M3 scales at once with the hardware conversion (exact; 0x7F / 0xFF are NaN as in the reference)
            const float2 dr0 = e4m3x2_to_f32(s0), dr1 = e4m3x2_to_f32(s1);
            const float d00 = dr0.x, d01 = dr0.y, d10 = dr1.x, d11 = dr1.y;
            const uint32_t f0 = first ? a0 : 0u, f1 = first ? a1 : 0u, f2 = first ? a2 : 0u, f3 = first ? a3 : 0u;
            const uint32_t e0 = first ? 0u : a0, e1 = first ? 0u : a1, e2 = first ? 0u : a2, e3 = first ? 0u : a3;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const uint2 b = lds64(xb[nt] + 32 * bb);
                int c[4], d[4];
                imma16832<true>(c, f0, f1, f2, f3, b.x, b.y);
                imma16832<true>(d, e0, e1, e2, e3, b.x, b.y);
                cs[nt][0] = fmaf(d00, (float)c[0], fmaf(d01, (float)d[0], cs[nt][0]));
                cs[nt][1] = fmaf(d00, (float)c[1], fmaf(d01, (float)d[1], cs[nt][1]));
                cs[nt][2] = fmaf(d10, (float)c[2], fmaf(d11, (float)d[2], cs[nt][2]));
                cs[nt][3] = fmaf(d10, (float)c[3], fmaf(d11, (float)d[3], cs[nt][3]));
            }
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int j = 0; j < 4; j++) tot[nt][j] = fmaf(xs[nt], cs[nt][j], tot[nt][j]);
}

// Balanced partition of the super-chunk sequence: CTA c owns [cta_first(c), cta_first(c + 1)).
__device__ __forceinline__ int64_t cta_first(const GemvParams &p, int c) {
    return (int64_t)c * p.per_cta + min(c, p.rem);
}
__device__ __forceinline__ int cta_of(const GemvParams &p, int64_t sc) {
    const int64_t big = (int64_t)p.rem * (p.per_cta + 1);
    return sc < big ? (int)(sc / (p.per_cta + 1)) : p.rem + (int)((sc - big) / p.per_cta);
}

// Stream-k over the flattened (tile group, k-step) sequence of super-chunks (8 row tiles x one k-step,
// contiguous in memory): CTA c owns super-chunks [c*per_cta, (c+1)*per_cta), one contiguous byte range.
// Thread 0 is the producer: per step it issues two bulk copies (the super-chunk and the activation slice
// of its k-step) into a ring stage; the 8 warps, each working on row tile 8*TG + warp, consume it.
template <int FMT, int NT, bool FUSE = false>
__global__ void __launch_bounds__(256) gemv_kernel(const __grid_constant__ GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ float wmax_s[2][8];
    __shared__ int wbad_s[2][8];
    constexpr int CHUNK = chunk_bytes<FMT>();
    constexpr int SFB = sf_bytes<FMT>();           // FP4 scale atoms of a super-chunk (own plane, own copy)
    constexpr int WDATA = GEMV_WARPS * CHUNK;      // weight bytes of a super-chunk in the main plane
    constexpr int SUPER = WDATA + SFB;             // weight bytes of a stage
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t xbytes = slice_bytes(p.m);
    const uint32_t stage_bytes = SUPER + (FUSE ? 0u : xbytes);
    const uint32_t smem_s = smem_u32(smem);
    const uint32_t slices_s = smem_s + GEMV_STAGES * stage_bytes;  // FUSE: this CTA's activation slices, in step order
    const uint32_t zero_s = slices_s + (FUSE ? (uint32_t)p.fuse_slices * xbytes : 0u);
    const uint32_t full = zero_s + GEMV_ZERO, empty = full + GEMV_STAGES * 8;

    // Whatever follows in the stream (the next call's staging kernel, then its GEMV grid) may be
    // scheduled as this grid's CTAs retire; it orders itself after this grid with griddepcontrol.wait.
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    const int nk = p.nk;
    const int64_t sc0 = cta_first(p, (int)blockIdx.x), sc1 = cta_first(p, (int)blockIdx.x + 1);
    const int n = (int)(sc1 - sc0);
    const uint8_t *wsrc = p.chunks + (size_t)sc0 * WDATA;
    const uint8_t *sfsrc = SFB ? p.sf + (size_t)sc0 * SFB : nullptr;
    int TG = (int)(sc0 / nk), b = (int)(sc0 % nk);

    if (threadIdx.x == 0) {
#pragma unroll
        for (int s = 0; s < GEMV_STAGES; s++) {
            mbar_init(full + 8 * s, 1);
            mbar_init(empty + 8 * s, GEMV_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        // weights of the first stages: independent of the activation staging kernel
#pragma unroll
        for (int s = 0; s < GEMV_STAGES; s++)
            if (s < n) {
                mbar_expect_tx(full + 8 * s, stage_bytes);
                bulk_g2s(smem_s + s * stage_bytes, wsrc + (size_t)s * WDATA, WDATA, full + 8 * s);
                if constexpr (SFB != 0) bulk_g2s(smem_s + s * stage_bytes + WDATA, sfsrc + (size_t)s * SFB, SFB, full + 8 * s);
            }
    }
    if (threadIdx.x < GEMV_ZERO / 4) reinterpret_cast<uint32_t *>(smem + (zero_s - smem_s))[threadIdx.x] = 0u;
    asm volatile("griddepcontrol.wait;\n" ::: "memory");  // everything before this grid in the stream is complete from here on
    if constexpr (FUSE) {
        if (p.xflags) {
            // exchange products: x may be the previous product's gathered y — wait (bounded) until every other rank
            // has completed as many exchange products as this rank; the weight copies above are already in flight
            if ((int)threadIdx.x < p.xnranks - 1) {
                const int src = (int)threadIdx.x < p.xrank ? (int)threadIdx.x : (int)threadIdx.x + 1;
                const uint32_t want = *reinterpret_cast<volatile const uint32_t *>(p.xflags + XF_EPOCH);
                bool seen = false;
                for (uint32_t it = 0; it < p.spins && !seen; it++) {
                    uint32_t v;
                    asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p.xflags + XF_FLAGS + src) : "memory");
                    seen = (int32_t)(v - want) >= 0;
                    if (!seen && it > 64) __nanosleep(100);
                }
                if (!seen) atomicExch(p.status, 32);
            }
            __syncthreads();
        }
        // this CTA's slices: all loads first (one L2 round trip for the lot), then the conversions
        const int nsl = min(n, p.fuse_slices);
        float xv[GEMV_FUSE_MAX_WORK];
#pragma unroll
        for (int j = 0; j < GEMV_FUSE_MAX_WORK; j++) {
            const int i = j / p.m, tok = j - i * p.m;  // slice, token
            xv[j] = 0.f;
            if (i < nsl) {
                int kb = b + i;
                if (kb >= nk) kb -= nk;
                const int64_t k = (int64_t)kb * 256 + threadIdx.x;
                if (k < p.K) {
                    xv[j] = __ldcg(p.x + (int64_t)tok * p.xst + k * p.xsk);
                    if (p.x_up) xv[j] = (xv[j] / (1.0f + expf(-xv[j]))) * __ldcg(p.x_up + (int64_t)tok * p.xst + k * p.xsk);
                }
            }
        }
        int par = 0;
#pragma unroll
        for (int j = 0; j < GEMV_FUSE_MAX_WORK; j++) {
            const int i = j / p.m, tok = j - i * p.m;
            if (i < nsl) stage_value_in_cta(xv[j], p.m, tok, smem + (slices_s - smem_s) + (size_t)i * xbytes, wmax_s, wbad_s, par);
        }
    } else if (threadIdx.x == 0) {
        int bb = b;
#pragma unroll
        for (int s = 0; s < GEMV_STAGES; s++) {
            if (s < n) bulk_g2s(smem_s + s * stage_bytes + SUPER, p.img + (size_t)bb * xbytes, xbytes, full + 8 * s);
            if (++bb == nk) bb = 0;
        }
    }
    __syncthreads();

    // Per-lane addresses inside stage 0.  Lanes of MMA columns >= 2m read the zero region (stride 0).
    uint32_t xb0[NT], sb0[NT], xs0[NT], xstride[NT], xsstride[NT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++) {
        const int col = nt * 8 + g, tok = nt * 4 + t;
        const bool act = col < 2 * p.m;
        // image path: the slice travels with its stage; fused path: slice i of the CTA's own area belongs to step i
        const uint32_t xbase = FUSE ? slices_s : smem_s + SUPER, xstep = FUSE ? xbytes : stage_bytes;
        xstride[nt] = act ? xstep : 0u;
        xb0[nt] = act ? xbase + col * 288 + 8 * t : zero_s;
        sb0[nt] = act ? xbase + (2 * p.m) * 288 + col * 16 : zero_s;
        xsstride[nt] = (tok < p.m) ? xstep : 0u;
        xs0[nt] = (tok < p.m) ? xbase + (2 * p.m) * 304 + tok * 4 : zero_s;
    }
    int sl = 0;  // FUSE: slice of step i
    int st = 0;                // stage of step i
    uint32_t ph = 0;           // its parity
    int bx = b + GEMV_STAGES;  // k-step of the next activation slice to request
    while (bx >= nk) bx -= nk;
    constexpr int NTOT = (FMT == FMT_Q4K) ? 2 : 4;
    float tot[NT][NTOT];
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int j = 0; j < NTOT; j++) tot[nt][j] = 0.f;

    int i = 0;
    while (i < n) {
        const int steps = min(nk - b, n - i);
        for (int s = 0; s < steps; s++, i++) {
            // producer: refill the stage released at step i-1 with step i-1+STAGES
            if (threadIdx.x == 0 && i > 0 && i - 1 + GEMV_STAGES < n) {
                const int ps = (st == 0) ? GEMV_STAGES - 1 : st - 1;
                const uint32_t pph = (st == 0) ? ph ^ 1u : ph;
                if (!mbar_wait(empty + 8 * ps, pph)) {
                    atomicExch(p.status, 2);
                } else {
                    mbar_expect_tx(full + 8 * ps, stage_bytes);
                    bulk_g2s(smem_s + ps * stage_bytes, wsrc + (size_t)(i - 1 + GEMV_STAGES) * WDATA, WDATA, full + 8 * ps);
                    if constexpr (SFB != 0)
                        bulk_g2s(smem_s + ps * stage_bytes + WDATA, sfsrc + (size_t)(i - 1 + GEMV_STAGES) * SFB, SFB, full + 8 * ps);
                    if constexpr (!FUSE) bulk_g2s(smem_s + ps * stage_bytes + SUPER, p.img + (size_t)bx * xbytes, xbytes, full + 8 * ps);
                }
                if (++bx == nk) bx = 0;
            }
            if (!mbar_wait(full + 8 * st, ph)) {
                if (lane == 0) atomicExch(p.status, 1);
                return;  // give up instead of hanging; the host sees the status word
            }
            uint32_t xb[NT], sb[NT];
            float xs[NT];
            const int xi = FUSE ? sl : st;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                xb[nt] = xb0[nt] + xi * xstride[nt];
                sb[nt] = sb0[nt] + xi * xstride[nt];
                xs[nt] = __uint_as_float(lds32(xs0[nt] + xi * xsstride[nt]));
            }
            if (FUSE && ++sl == p.fuse_slices) sl = 0;
            const uint32_t ch = smem_s + st * stage_bytes + warp * CHUNK;
            if constexpr (FMT == FMT_Q4K) q4k_chunk<NT>(ch, lane, xb, sb, xs, tot);
            else if constexpr (FMT == FMT_Q80) q80_chunk<NT>(ch, lane, xb, xs, tot);
            else fp4_chunk<FMT, NT>(smem_s + st * stage_bytes, warp, lane, xb, xs, tot);
            __syncwarp();
            if (lane == 0) mbar_arrive(empty + 8 * st);
            if (++st == GEMV_STAGES) { st = 0; ph ^= 1u; }
        }
        // ---- this CTA's share of tile group TG is complete; each warp finishes its own tile ----
        const int64_t first = (int64_t)TG * nk, last = first + nk - 1;
        const int slot0 = cta_of(p, first), nsl = cta_of(p, last) - slot0 + 1;
        float v[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
            if constexpr (FMT == FMT_Q4K) {
                v[nt][0] = tot[nt][0];
                v[nt][1] = tot[nt][1];
            } else {
                v[nt][0] = fmaf(tot[nt][1], 1.0f / 254.0f, tot[nt][0]);
                v[nt][1] = fmaf(tot[nt][3], 1.0f / 254.0f, tot[nt][2]);
                if constexpr (FMT == FMT_MXFP4 || FMT == FMT_NVFP4) {
                    v[nt][0] *= p.wscale;
                    v[nt][1] *= p.wscale;
                }
            }
#pragma unroll
            for (int j = 0; j < NTOT; j++) tot[nt][j] = 0.f;
        }
        gemv_flush<NT>(p, TG * 8 + warp, (int)blockIdx.x - slot0, nsl, v);
        TG++;
        b = 0;
    }
    if (p.xflags) {
        // Exchange products: every CTA orders its band stores (local and peer) before its arrival at GPU scope;
        // the CTA that makes the count complete has then observed all of them and tells the other ranks with system-scope
        // release stores (cumulative).  System-scope fences in every CTA, or in
        // every warp that finished a row tile, cost 12-16 us per product on two GPUs; a separate barrier launch 5.5 us.
        __syncthreads();
        if (threadIdx.x == 0) {
            int done;  // release: this CTA's stores before the arrival; acquire: the last arrival sees every CTA's stores
            asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;\n" : "=r"(done) : "l"(p.counters + p.ntiles) : "memory");
            if (done == (int)gridDim.x - 1) {
                p.counters[p.ntiles] = 0;  // ready for the next launch
                volatile uint32_t *epoch = p.xflags + XF_EPOCH;  // read and written through L2 only
                const uint32_t e = *epoch + 1u;
                *epoch = e;
                // the launch's one system-scope fence: every band store this CTA has observed (its own, and through the
                // counter every other CTA's) is visible to a rank that acquires a flag written after it.  One release store
                // per peer instead cost a fence each: 2 us per peer, 14 us per product on eight GPUs.
                __threadfence_system();
                for (int q = 0; q < p.npeer; q++)
                    asm volatile("st.relaxed.sys.global.u32 [%0], %1;\n" ::"l"(p.xflags_peer[q] + XF_FLAGS + p.xrank), "r"(e) : "memory");
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// workspace: the activation image, ceil(K/256) slices
size_t gemv_ws_bytes(const Weight *w, int m) {
    const size_t nk = ((size_t)w->k + 255) / 256;
    return align_up(nk * slice_bytes(m), 256);
}

template <typename Kern, typename Params>
static cudaError_t launch_pdl(Kern kern, dim3 grid, dim3 block, size_t smem, cudaStream_t s, bool pdl, const Params &p) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

// Resident CTAs per SM for (format, n-tiles, m): set up once per device, then cached.
template <int FMT, int NT>
static cudaError_t gemv_occupancy(int device, int m, size_t smem, int *per_sm) {
    static int cache[16][GLLMK_GEMV_MAX_M + 1];  // [device][m], 0 = not yet queried
    if (device >= 0 && device < 16 && cache[device][m]) {
        *per_sm = cache[device][m];
        return cudaSuccess;
    }
    cudaError_t e = cudaFuncSetAttribute(gemv_kernel<FMT, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)gemv_smem_bytes<FMT>(GLLMK_GEMV_MAX_M));
    if (e != cudaSuccess) return e;
    int n = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, gemv_kernel<FMT, NT>, 256, smem);
    if (e != cudaSuccess) return e;
    if (n < 1) n = 1;
    if (device >= 0 && device < 16) cache[device][m] = n;
    *per_sm = n;
    return cudaSuccess;
}


// Grid of a decode launch: resident CTAs, each with a contiguous share of the super-chunk sequence.
struct GemvGrid {
    int per_sm;
    int64_t ctas;
    int per_cta, rem;
};
template <int FMT, int NT>
static cudaError_t gemv_grid(Ctx *c, int m, int64_t nsuper, GemvGrid *g) {
    cudaError_t e = gemv_occupancy<FMT, NT>(c->device, m, gemv_smem_bytes<FMT>(m), &g->per_sm);
    if (e != cudaSuccess) return e;
    if (c->gemv_ctas_per_sm > 0 && c->gemv_ctas_per_sm < g->per_sm) g->per_sm = (int)c->gemv_ctas_per_sm;
    g->ctas = (int64_t)c->sm_count * g->per_sm;
    if (g->ctas > nsuper) g->ctas = nsuper;
    g->per_cta = (int)(nsuper / g->ctas);
    g->rem = (int)(nsuper % g->ctas);
    return cudaSuccess;
}

// Slices a CTA would stage itself (0 = use the staging kernel and its image): few enough, and the fused variant
// must keep as many CTAs resident as the image variant.
template <int FMT>
static cudaError_t gemv_fuse_plan(Ctx *c, int m, int64_t ntg, int nk, int *slices) {
    *slices = 0;
    if (!c->gemv_fuse || m > 4) return cudaSuccess;
    GemvGrid g;
    cudaError_t e = gemv_grid<FMT, 1>(c, m, ntg * nk, &g);
    if (e != cudaSuccess) return e;
    const int share = g.per_cta + (g.rem ? 1 : 0);
    const int nsl = share < nk ? share : nk;
    if (nsl * m > GEMV_FUSE_MAX_WORK) return cudaSuccess;
    static int occ[16][5][GEMV_FUSE_MAX_WORK + 1];  // [device][m][slices], 0 = not yet asked
    const int dv = c->device & 15;
    if (!occ[dv][m][nsl]) {
        e = cudaFuncSetAttribute(gemv_kernel<FMT, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)gemv_smem_bytes_fused<FMT>(4, GEMV_FUSE_MAX_WORK));
        if (e != cudaSuccess) return e;
        int nb = 0;
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, gemv_kernel<FMT, 1, true>, 256, gemv_smem_bytes_fused<FMT>(m, nsl));
        if (e != cudaSuccess) return e;
        occ[dv][m][nsl] = nb < 1 ? -1 : nb;
    }
    if (occ[dv][m][nsl] >= g.per_sm) *slices = nsl;
    return cudaSuccess;
}

template <int FMT, int NT>
static cudaError_t configure_and_launch(Ctx *c, GemvParams &p, int64_t ntg, cudaStream_t s, int32_t *rc_out, int fuse_slices) {
    p.nsuper = ntg * p.nk;
    GemvGrid g;
    cudaError_t e = gemv_grid<FMT, NT>(c, p.m, p.nsuper, &g);
    if (e != cudaSuccess) return e;
    p.per_cta = g.per_cta;
    p.rem = g.rem;
    const unsigned grid = (unsigned)g.ctas;
    p.maxslot = (p.nk - 1) / p.per_cta + 2;
    const int64_t tiles = ntg * 8;
    const size_t part_bytes = align_up((size_t)tiles * p.maxslot * 256 * sizeof(float), 256);
    *rc_out = ensure_red(c, part_bytes);
    if (!*rc_out) *rc_out = ensure_cnt(c, (size_t)(tiles + 1) * sizeof(int));
    if (*rc_out) return cudaSuccess;
    p.partial = static_cast<float *>(c->red);
    p.counters = static_cast<int *>(c->cnt);
    p.ntiles = (int)tiles;
    if constexpr (NT == 1 && (FMT == FMT_Q4K || FMT == FMT_Q80)) {
        if (fuse_slices > 0) {
            p.fuse_slices = fuse_slices;
            return launch_pdl(gemv_kernel<FMT, NT, true>, grid, 256, gemv_smem_bytes_fused<FMT>(p.m, fuse_slices), s, c->gemv_pdl != 0, p);
        }
    }
    return launch_pdl(gemv_kernel<FMT, NT>, grid, 256, gemv_smem_bytes<FMT>(p.m), s, c->gemv_pdl != 0, p);
}

int32_t gemv_launch(Ctx *c, const Weight *w, const float *x, int64_t xst, int64_t xsk, int m, float *y, int64_t yst,
                    int64_t ysr, const float *row_scales, int64_t n_row_scales, cudaStream_t s, void *const *y_peers,
                    int n_peers, const float *x_up, const Exchange *xch) {
    if (raw_format(w->qt)) {
        if (n_peers || x_up || xch) return fail(c, GLLMK_STATUS_UNSUPPORTED, "gemv: quant type %d has no fused exchange / SwiGLU input", w->qt);
        return raw_gemv_launch(c, w, x, xst, xsk, m, y, yst, ysr, row_scales, n_row_scales, s);
    }
    if (w->qt != GLLMK_QUANT_Q4K && w->qt != GLLMK_QUANT_Q8_0 && w->qt != GLLMK_QUANT_MXFP4 && w->qt != GLLMK_QUANT_NVFP4)
        return fail(c, GLLMK_STATUS_UNSUPPORTED, "gemv: quant type %d has no decode kernel", w->qt);
    // FP4 weights: the block-scaled tensor-core kernel (gemv_fp4.cu) unless the call needs what only this kernel
    // has (row scales, peer outputs, a fused SwiGLU input) or the context asks for the integer-decode kernel
    if ((w->qt == GLLMK_QUANT_MXFP4 || w->qt == GLLMK_QUANT_NVFP4) && !row_scales && n_peers == 0 && !x_up && !xch && !c->gemv_fp4_int)
        return gemv_fp4_launch(c, w, x, xst, xsk, m, y, yst, ysr, s);
    int32_t rc = ensure_ws(c, gemv_ws_bytes(w, m));
    if (rc) return rc;
    const int nk = (int)((w->k + 255) / 256);

    GemvParams p{};
    p.chunks = static_cast<const uint8_t *>(w->qs);
    p.img = static_cast<const uint8_t *>(c->ws);
    p.sf = static_cast<const uint8_t *>(w->aux);
    p.wscale = 0.5f * w->global_scale;
    p.y = y;
    p.yst = yst;
    p.ysr = ysr;
    p.npeer = n_peers;
    for (int q = 0; q < n_peers; q++) p.ypeer[q] = static_cast<float *>(y_peers[q]);
    p.row_scales = row_scales;
    p.n_row_scales = row_scales ? n_row_scales : 0;
    p.n = w->n;
    p.nk = nk;
    p.m = m;
    p.status = c->status_dev;
    if (xch && xch->flags_local) {
        p.xflags = xch->flags_local;
        for (int q = 0; q < xch->n_peers; q++) p.xflags_peer[q] = xch->flags_peer[q];
        p.xrank = xch->rank;
    }

    p.x = x;
    p.x_up = x_up;
    p.xst = xst;
    p.xsk = xsk;
    p.K = w->k;
    p.spins = (uint32_t)c->peer_wait_spins;
    p.xnranks = xch ? xch->n_peers + 1 : 1;

    StageParams sp{x, x_up, xst, xsk, m, w->k, static_cast<uint8_t *>(c->ws)};
    if (p.xflags) {
        sp.xflags = xch->flags_local;
        sp.nranks = xch->n_peers + 1;
        sp.rank = xch->rank;
        sp.spins = (uint32_t)c->peer_wait_spins;
        sp.status = c->status_dev;
    }
    dim3 sgrid((unsigned)(((size_t)nk * 256 + 1023) / 1024), (unsigned)m);
    static bool stage_carveout_set = false;
    if (!stage_carveout_set) {
        // same shared-memory carve-out as the GEMV grid that follows, so the SMs are not reconfigured in between
        (void)cudaFuncSetAttribute(stage_x_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        (void)cudaGetLastError();
        stage_carveout_set = true;
    }
    const int64_t ntg = w->n_pad / 128;
    const int NT = (2 * m + 7) / 8;
    // Small shares: the GEMV converts its activation slices itself and the staging kernel is not launched at all.
    // (Measured on one GPU the two-kernel form is as fast or faster even for small matrices — its staging kernel runs
    // under the previous product's tail — so by default only exchange products fuse: there the staging kernel would
    // also have to carry the wait for the other ranks.)
    int fuse = 0;
    const bool want_fuse = c->gemv_fuse == 2 || (c->gemv_fuse == 1 && xch != nullptr);
    if (want_fuse && NT == 1 && w->qt == GLLMK_QUANT_Q4K) GK_CUDA(c, gemv_fuse_plan<FMT_Q4K>(c, m, ntg, nk, &fuse));
    else if (want_fuse && NT == 1 && w->qt == GLLMK_QUANT_Q8_0) GK_CUDA(c, gemv_fuse_plan<FMT_Q80>(c, m, ntg, nk, &fuse));
    if (!fuse) GK_CUDA(c, launch_pdl(stage_x_kernel, sgrid, 256, 0, s, c->gemv_pdl != 0, sp));

    cudaError_t e;
    rc = 0;
    if (w->qt == GLLMK_QUANT_Q4K) {
        switch (NT) {
            case 1: e = configure_and_launch<FMT_Q4K, 1>(c, p, ntg, s, &rc, fuse); break;
            case 2: e = configure_and_launch<FMT_Q4K, 2>(c, p, ntg, s, &rc, 0); break;
            case 3: e = configure_and_launch<FMT_Q4K, 3>(c, p, ntg, s, &rc, 0); break;
            default: e = configure_and_launch<FMT_Q4K, 4>(c, p, ntg, s, &rc, 0); break;
        }
    } else if (w->qt == GLLMK_QUANT_Q8_0) {
        switch (NT) {
            case 1: e = configure_and_launch<FMT_Q80, 1>(c, p, ntg, s, &rc, fuse); break;
            case 2: e = configure_and_launch<FMT_Q80, 2>(c, p, ntg, s, &rc, 0); break;
            case 3: e = configure_and_launch<FMT_Q80, 3>(c, p, ntg, s, &rc, 0); break;
            default: e = configure_and_launch<FMT_Q80, 4>(c, p, ntg, s, &rc, 0); break;
        }
    } else if (w->qt == GLLMK_QUANT_MXFP4) {
        switch (NT) {
            case 1: e = configure_and_launch<FMT_MXFP4, 1>(c, p, ntg, s, &rc, 0); break;
            case 2: e = configure_and_launch<FMT_MXFP4, 2>(c, p, ntg, s, &rc, 0); break;
            case 3: e = configure_and_launch<FMT_MXFP4, 3>(c, p, ntg, s, &rc, 0); break;
            default: e = configure_and_launch<FMT_MXFP4, 4>(c, p, ntg, s, &rc, 0); break;
        }
    } else {
        switch (NT) {
            case 1: e = configure_and_launch<FMT_NVFP4, 1>(c, p, ntg, s, &rc, 0); break;
            case 2: e = configure_and_launch<FMT_NVFP4, 2>(c, p, ntg, s, &rc, 0); break;
            case 3: e = configure_and_launch<FMT_NVFP4, 3>(c, p, ntg, s, &rc, 0); break;
            default: e = configure_and_launch<FMT_NVFP4, 4>(c, p, ntg, s, &rc, 0); break;
        }
    }
    if (rc) return rc;
    GK_CUDA(c, e);
    return GLLMK_STATUS_OK;
}

// ---------------------------------------------------------------------------------------------
// Decode GEMV for callers that must not allocate.
//
// Some hosts of this library run their decode step where device allocation is off limits: inside a
// latency-critical serving loop that has pre-reserved all of HBM for weights and KV pages, under an
// allocator that owns the whole device, or in a callback where cudaMalloc's implicit synchronisation
// is not acceptable.  gllmk_gemv grows context-owned buffers on demand; this variant never does.  All of
// the kernel's scratch (activation image, split-k partial sums, arrival counters) lives in
// one fixed array inside the library image, so every GPU that loads the library holds these 8 MiB until
// the process exits.
// ---------------------------------------------------------------------------------------------
constexpr size_t GEMV_STATIC_BYTES = (size_t)8 << 20;
constexpr size_t GEMV_STATIC_MAX_TILES = 8192;  // counters area: rows up to 131072
static __device__ __align__(256) unsigned char g_gemv_static_scratch[GEMV_STATIC_BYTES];

// The array's name is only a host-side handle; the device address comes from cudaGetSymbolAddress,
// looked up once per device with that device current.
static cudaError_t gemv_static_base(int device, unsigned char **base) {
    static unsigned char *cached[16] = {};
    if (device < 0 || device >= 16) return cudaErrorInvalidDevice;
    if (!cached[device]) {
        void *ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_gemv_static_scratch);
        if (e != cudaSuccess) return e;
        cached[device] = static_cast<unsigned char *>(ptr);
    }
    *base = cached[device];
    return cudaSuccess;
}

template <int FMT, int NT>
static cudaError_t launch_static(Ctx *c, GemvParams &p, int64_t ntg, unsigned char *base, size_t img_bytes,
                                 cudaStream_t s, int32_t *rc_out) {
    const size_t smem = gemv_smem_bytes<FMT>(p.m);
    int per_sm = 0;
    cudaError_t e = gemv_occupancy<FMT, NT>(c->device, p.m, smem, &per_sm);
    if (e != cudaSuccess) return e;
    if (c->gemv_ctas_per_sm > 0 && c->gemv_ctas_per_sm < per_sm) per_sm = (int)c->gemv_ctas_per_sm;
    p.nsuper = ntg * p.nk;
    int64_t ctas = (int64_t)c->sm_count * per_sm;
    if (ctas > p.nsuper) ctas = p.nsuper;
    p.per_cta = (int)(p.nsuper / ctas);
    p.rem = (int)(p.nsuper % ctas);
    p.maxslot = (p.nk - 1) / p.per_cta + 2;
    const size_t tiles = (size_t)ntg * 8;
    // layout: reserved [256] | counters [GEMV_STATIC_MAX_TILES ints] | activation image | partial sums.  The status
    // word is NOT in the array: a give-up is reported through the context's own word (allocated when the context
    // was created), so gllmk_ctx_status sees it like any other kernel's.
    const size_t cnt_off = 256, img_off = cnt_off + GEMV_STATIC_MAX_TILES * sizeof(int);
    const size_t part_off = align_up(img_off + img_bytes, 256);
    const size_t part_bytes = tiles * (size_t)p.maxslot * 256 * sizeof(float);
    if (tiles > GEMV_STATIC_MAX_TILES || part_off + part_bytes > GEMV_STATIC_BYTES) {
        *rc_out = fail(c, GLLMK_STATUS_INVALID_ARG,
                       "gemv_static: this shape needs %zu bytes of scratch (%zu row tiles), the built-in area holds %zu "
                       "bytes (%zu row tiles); use gllmk_gemv",
                       part_off + part_bytes, tiles, GEMV_STATIC_BYTES, GEMV_STATIC_MAX_TILES);
        return cudaSuccess;
    }
    p.status = c->status_dev;
    p.counters = reinterpret_cast<int *>(base + cnt_off);
    p.img = base + img_off;
    p.partial = reinterpret_cast<float *>(base + part_off);
    // The area keeps whatever the previous call left: the counters must start at zero (a call that gave up
    // a bounded wait may have left some non-zero).  Stream-ordered, no allocation.
    e = cudaMemsetAsync(p.counters, 0, tiles * sizeof(int), s);
    if (e != cudaSuccess) return e;
    return launch_pdl(gemv_kernel<FMT, NT>, (unsigned)ctas, 256, smem, s, false, p);
}

}  // namespace gllmk

using namespace gllmk;

extern "C" int32_t gllmk_gemv_static(gllmk_ctx ctx, gllmk_weight wh, const float *x_dev, int64_t x_stride_t,
                                     int64_t x_stride_k, int32_t m, float *y_dev, int64_t y_stride_t, int64_t y_stride_r,
                                     const float *row_scales, int64_t n_row_scales, void *stream) {
    if (!ctx || !wh || !x_dev || !y_dev) return GLLMK_STATUS_INVALID_ARG;
    Ctx *c = static_cast<Ctx *>(ctx);
    const Weight *w = static_cast<const Weight *>(wh);
    if (m < 1 || m > GLLMK_GEMV_MAX_M)
        return fail(c, GLLMK_STATUS_INVALID_ARG, "gemv_static: m=%d outside 1..%d", m, GLLMK_GEMV_MAX_M);
    if (w->qt != GLLMK_QUANT_Q4K && w->qt != GLLMK_QUANT_Q8_0)
        return fail(c, GLLMK_STATUS_UNSUPPORTED, "gemv_static: quant type %d has no decode kernel", w->qt);
    if (w->device != c->device) return fail(c, GLLMK_STATUS_INVALID_ARG, "weight lives on another device");
    if (row_scales && n_row_scales != 1 && n_row_scales != w->n)
        return fail(c, GLLMK_STATUS_INVALID_ARG, "gemv_static: n_row_scales=%lld must be 1 or n=%lld", (long long)n_row_scales,
                    (long long)w->n);
    int prev = -1;
    GK_CUDA(c, cudaGetDevice(&prev));
    if (prev != c->device) GK_CUDA(c, cudaSetDevice(c->device));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned char *base = nullptr;
    cudaError_t e = gemv_static_base(c->device, &base);  // first call on a device: symbol address look-up
    int32_t rc = GLLMK_STATUS_OK;
    if (e == cudaSuccess) {
        const int nk = (int)((w->k + 255) / 256);
        const size_t img_bytes = align_up((size_t)nk * slice_bytes(m), 256);
        GemvParams p{};
        p.chunks = static_cast<const uint8_t *>(w->qs);
        p.y = y_dev;
        p.yst = y_stride_t;
        p.ysr = y_stride_r;
        p.row_scales = row_scales;
        p.n_row_scales = row_scales ? n_row_scales : 0;
        p.n = w->n;
        p.nk = nk;
        p.m = m;
        const size_t img_off = 256 + GEMV_STATIC_MAX_TILES * sizeof(int);
        if (img_off + img_bytes > GEMV_STATIC_BYTES) {
            rc = fail(c, GLLMK_STATUS_INVALID_ARG, "gemv_static: k=%lld with m=%d needs a %zu-byte activation image, "
                      "more than the built-in %zu-byte area; use gllmk_gemv", (long long)w->k, m, img_bytes, GEMV_STATIC_BYTES);
        } else {
            StageParams sp{x_dev, nullptr, x_stride_t, x_stride_k, m, w->k, base + img_off};  // no exchange: the other fields stay zero
            dim3 sgrid((unsigned)(((size_t)nk * 256 + 1023) / 1024), (unsigned)m);
            e = launch_pdl(stage_x_kernel, sgrid, 256, 0, s, false, sp);
            const int64_t ntg = w->n_pad / 128;
            const int NT = (2 * m + 7) / 8;
            if (e == cudaSuccess) {
                if (w->qt == GLLMK_QUANT_Q4K) {
                    switch (NT) {
                        case 1: e = launch_static<FMT_Q4K, 1>(c, p, ntg, base, img_bytes, s, &rc); break;
                        case 2: e = launch_static<FMT_Q4K, 2>(c, p, ntg, base, img_bytes, s, &rc); break;
                        case 3: e = launch_static<FMT_Q4K, 3>(c, p, ntg, base, img_bytes, s, &rc); break;
                        default: e = launch_static<FMT_Q4K, 4>(c, p, ntg, base, img_bytes, s, &rc); break;
                    }
                } else {
                    switch (NT) {
                        case 1: e = launch_static<FMT_Q80, 1>(c, p, ntg, base, img_bytes, s, &rc); break;
                        case 2: e = launch_static<FMT_Q80, 2>(c, p, ntg, base, img_bytes, s, &rc); break;
                        case 3: e = launch_static<FMT_Q80, 3>(c, p, ntg, base, img_bytes, s, &rc); break;
                        default: e = launch_static<FMT_Q80, 4>(c, p, ntg, base, img_bytes, s, &rc); break;
                    }
                }
            }
        }
    }
    if (prev != c->device) cudaSetDevice(prev);
    if (e != cudaSuccess) return cuda_fail(c, e, "gemv_static");
    return rc;
}
