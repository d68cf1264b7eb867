// Decode GEMV for MXFP4 / NVFP4 weights on the block-scaled tensor core: no instruction decodes a weight.
//
//   y[t, r] = gW * sum_k W4[r, k] * x[t, k]          t < m <= 16 tokens, r < n weight rows
//
// The weights stay what they are in HBM (E2M1 codes in 16 KB swizzled tile images + scale atoms) and are the A
// operand of tcgen05.mma.kind::mxf4 / kind::mxf4nvf4.block_scale straight from shared memory.  The f32
// activations become FP4 too, exactly enough: per token and scale block, x = s * sum_j 4^-j * d_j with eight
// E2M1 "digits" d_j (each digit rounds the residual of the previous ones, whose error is at most one unit of
// the next scale), written by a staging kernel as eight FP4 rows per token that share the block's scale.  The
// MMA therefore computes eight exact partial products per token (columns 8t .. 8t+7 of the accumulator) and
// the epilogue adds them with the weights 4^-j.  Representation error of x: <= s * 4^-7 ~ amax_block * 1e-5.
//
// HBM-bound by construction: per k-step (256 k) a CTA streams one weight tile (16 KB + 1-2 KB of scales) from
// HBM and the digit tile (<= 16 KB, L2 resident) beside it; four MMAs of K = 64 and N = 8m (rounded to 32) are
// negligible work.  Stream-k: one persistent CTA per SM owns a contiguous, balanced range of (row tile, k-step)
// units; a row tile shared between CTAs is summed from f32 partials (8 KB each) by the last CTA to arrive, in
// k order (deterministic).  No CTA waits for another; every mbarrier wait is bounded.
#include "common.cuh"
#include "tc05.cuh"

namespace gllmk {

constexpr int FD_DIGITS = 8;
constexpr int FD_MAX_STAGES = 12;     // a stage = weight tile (16 KB) + digit tile (128 B x MMA N) + both scale atoms, 1 KB aligned;
                                      // as many as fit: bytes in flight per SM are what hides the HBM latency
constexpr int FD_SMEM_BUDGET = 232448 - 2048;
constexpr int FD_THREADS = 320;       // warp 0: copies, warp 1: MMA + TMEM, warps 2-5: epilogue, warps 6-9: scale factors
constexpr int FD_SF_SETS = 4;         // scale-factor column sets in rotation
constexpr uint32_t FD_TMEM_COLS = 256;                        // 128 accumulator + 4 x (16 SFA + 16 SFB)

struct FdParams {
    const uint8_t *qw, *sfw;  // weight data / scale planes
    const uint8_t *qx, *sfx;  // digit data / scale planes (one 128-row tile: rows 8t + j)
    const float *gtok;        // per-token factor (NVFP4: the token's global scale; MXFP4: 1)
    float wscale;             // the weight's per-tensor scale
    int nv;                   // 1: NVFP4 (UE4M3 per 16), 0: MXFP4 (UE8M0 per 32)
    int64_t n;
    int nks;                  // k-steps of 256
    int m, ncol;              // tokens; MMA N = 8m rounded up to 32
    int stages, stage_bytes;  // shared-memory ring
    float *y;
    int64_t yst, ysr;
    int row_tiles;
    int64_t per_cta;          // units (row tile, k-step) per CTA: the first `rem` CTAs own one more
    int rem;
    float *partial;           // [grid][2][16 tokens][128 rows]
    int *counters;            // [row_tiles], zero between launches
    int *status;
};

__device__ __forceinline__ int64_t fd_first(const FdParams &p, int c) { return (int64_t)c * p.per_cta + min(c, p.rem); }
__device__ __forceinline__ int fd_cta_of(const FdParams &p, int64_t u) {
    const int64_t big = (int64_t)p.rem * (p.per_cta + 1);
    return u < big ? (int)(u / (p.per_cta + 1)) : p.rem + (int)((u - big) / p.per_cta);
}
__device__ __forceinline__ void fd_bulk(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ uint64_t fd_sf_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)(128 >> 4) << 32) | ((uint64_t)1 << 46);
}

// ---- activations -> eight FP4 digit rows per token ---------------------------------------------------------
// nearest E2M1 code of r (|r| <= 6 up to rounding); residual after it is at most 1 (between 4 and 6)
__device__ __forceinline__ uint32_t fd_e2m1(float r, float &val) {
    const float a = fabsf(r);
    uint32_t c;
    float v;
    if (a < 0.25f) c = 0, v = 0.0f;
    else if (a < 0.75f) c = 1, v = 0.5f;
    else if (a < 1.25f) c = 2, v = 1.0f;
    else if (a < 1.75f) c = 3, v = 1.5f;
    else if (a < 2.5f) c = 4, v = 2.0f;
    else if (a < 3.5f) c = 5, v = 3.0f;
    else if (a < 5.0f) c = 6, v = 4.0f;
    else c = 7, v = 6.0f;
    val = r < 0.0f ? -v : v;
    return c | (r < 0.0f ? 8u : 0u);
}
// smallest UE4M3 value >= v (0 < v <= 448): code, and its value in `dec`
__device__ __forceinline__ uint32_t fd_ue4m3_up(float v, float &dec) {
    if (!(v > 0.0f)) {
        dec = 0.0f;
        return 0u;
    }
    int e;
    (void)frexpf(v, &e);  // v = f * 2^e, f in [0.5, 1)
    e -= 1;               // v in [2^e, 2^(e+1))
    if (e < -6) {         // subnormal grid: multiples of 2^-9
        int mm = (int)ceilf(v * 512.0f);
        if (mm < 1) mm = 1;
        if (mm >= 8) {
            dec = 0.015625f;  // 2^-6, the smallest normal
            return 1u << 3;
        }
        dec = (float)mm * (1.0f / 512.0f);
        return (uint32_t)mm;
    }
    if (e > 8) e = 8;
    int mm = (int)ceilf((ldexpf(v, -e) - 1.0f) * 8.0f);
    if (mm >= 8) {
        mm = 0;
        e += 1;
    }
    if (e > 8 || (e == 8 && mm > 6)) {  // top of the range (0x7E = 448); the caller keeps v below it
        e = 8;
        mm = 6;
    }
    dec = ldexpf(1.0f + (float)mm * 0.125f, e);
    return (uint32_t)((e + 7) << 3) | (uint32_t)mm;
}

// grid (groups of 8 blocks of 32 elements, tokens): one warp per 32 elements: block scale(s), eight digits per
// element, packed into the token's eight rows of the digit tile.
__global__ void __launch_bounds__(256) fd_stage_kernel(const float *__restrict__ x, int64_t xst, int64_t xsk, int64_t K, int64_t k_pad,
                                                       int nv, uint8_t *__restrict__ qx, uint8_t *__restrict__ sfx,
                                                       float *__restrict__ gtok) {
    __shared__ float red[8];
    __shared__ int bad_s;
    // The GEMV grid behind this one may start now and stream its first weight tiles; it waits for this grid to
    // finish before it touches the digit planes.  This grid is itself launched early: it may read x and overwrite
    // the planes only once everything in front of it in the stream has completed.
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    const int tok = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float *xr = x + (int64_t)tok * xst;
    const float inf = __int_as_float(0x7F800000);
    float g = 1.0f;
    if (nv) {
        // The token's amax -> g = amax / (6 * 256), so that every block scale fits UE4M3 (NaN when the token
        // holds a non-finite value).  Every CTA of the token works it out for itself from the whole row (a few
        // tens of KB out of L2): cheaper than a reduction kernel of its own in front of this one.
        float a = 0.0f;
        int bad = 0;
        if (xsk == 1 && (K & 3) == 0 && (reinterpret_cast<uintptr_t>(xr) & 15) == 0) {
            // contiguous row: 16-byte loads, four in flight per thread (a 28672-element row is 7 rounds instead of 112)
            const float4 *x4 = reinterpret_cast<const float4 *>(xr);
            const int64_t n4 = K >> 2;
#pragma unroll 4
            for (int64_t k = threadIdx.x; k < n4; k += 256) {
                const float4 q = __ldg(x4 + k);
                const float v0 = fabsf(q.x), v1 = fabsf(q.y), v2 = fabsf(q.z), v3 = fabsf(q.w);
                bad |= !(v0 < inf) | !(v1 < inf) | !(v2 < inf) | !(v3 < inf);
                a = fmaxf(fmaxf(a, fmaxf(v0, v1)), fmaxf(v2, v3));
            }
        } else {
            for (int64_t k = threadIdx.x; k < K; k += 256) {
                const float v = fabsf(xr[k * xsk]);
                bad |= !(v < inf);
                a = fmaxf(a, v);
            }
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
        bad = __any_sync(0xffffffffu, bad);
        if (threadIdx.x == 0) bad_s = 0;
        __syncthreads();
        if (lane == 0) {
            red[warp] = a;
            if (bad) bad_s = 1;
        }
        __syncthreads();
        a = red[0];
#pragma unroll
        for (int i = 1; i < 8; i++) a = fmaxf(a, red[i]);
        g = bad_s ? __int_as_float(0x7FC00000) : (a > 0.0f ? a * (1.0f / 1536.0f) : 1.0f);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) gtok[tok] = g;
    const float ginv = (nv && g == g) ? 1.0f / g : 1.0f;
    const int64_t nblk = k_pad >> 5;
    const int64_t blk = (int64_t)blockIdx.x * 8 + warp;
    if (blk < nblk) {
        const int64_t k = blk * 32 + lane;
        const float v = (k < K) ? xr[k * xsk] * ginv : 0.0f;
        const bool fin = fabsf(v) < inf;
        // scale group: 32 lanes (MXFP4) or 16 lanes (NVFP4)
        float amax = fin ? fabsf(v) : 0.0f;
        int bad = !fin;
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) {
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            bad |= __shfl_xor_sync(0xffffffffu, bad, o);
        }
        if (!nv) {
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 16));
            bad |= __shfl_xor_sync(0xffffffffu, bad, 16);
        }
        float s;
        uint32_t sbyte;
        if (!nv) {
            int e = 0;
            if (amax > 0.0f) {
                int pw;
                const float f = frexpf(amax, &pw);  // smallest e with 6 * 2^e >= amax
                e = (f <= 0.75f) ? pw - 3 : pw - 2;
            }
            int byte = e + 127;
            byte = byte < 1 ? 1 : (byte > 254 ? 254 : byte);
            s = __int_as_float(byte << 23);
            sbyte = bad ? 255u : (uint32_t)byte;
        } else {
            sbyte = fd_ue4m3_up(amax * (1.0f / 6.0f), s);
            if (bad || g != g) sbyte = 0x7Fu;
        }
        // digits of r = v / s: d_j = nearest E2M1 of the residual, residual <- (residual - d_j) * 4
        float r = (s > 0.0f && fin) ? v / s : 0.0f;
        uint32_t codes = 0;
#pragma unroll
        for (int j = 0; j < FD_DIGITS; j++) {
            float val;
            codes |= fd_e2m1(r, val) << (4 * j);
            r = (r - val) * 4.0f;
        }
        // pack: element pairs (even lane = low nibble); digit j goes to row 8*tok + j
        const uint32_t other = __shfl_down_sync(0xffffffffu, codes, 1);
        if ((lane & 1) == 0) {
#pragma unroll
            for (int j = 0; j < FD_DIGITS; j++) {
                const uint8_t by = (uint8_t)(((codes >> (4 * j)) & 15u) | (((other >> (4 * j)) & 15u) << 4));
                qx[fp4_data_offset(8 * tok + j, blk * 16 + (lane >> 1), k_pad)] = by;
            }
        }
        const bool writer = nv ? (lane & 15) == 0 : lane == 0;
        if (writer) {
            const int64_t sidx = nv ? blk * 2 + (lane >> 4) : blk;
            const int64_t spr = nv ? (k_pad >> 4) : (k_pad >> 5);
#pragma unroll
            for (int j = 0; j < FD_DIGITS; j++) sfx[fp4_sf_offset(8 * tok + j, sidx, spr)] = (uint8_t)sbyte;
        }
    }
}

// ---- the kernel -------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(FD_THREADS, 1) gemv_fp4_tc_kernel(const __grid_constant__ FdParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * FD_MAX_STAGES + 2 + 2 * FD_SF_SETS];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s, last_s;
    const uint32_t smem_s = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t full = tc::smem_u32(&bars[0]), empty = full + 8 * FD_MAX_STAGES, accum = empty + 8 * FD_MAX_STAGES, tmem_free = accum + 8;
    const uint32_t sf_full = tmem_free + 8, sf_empty = sf_full + 8 * FD_SF_SETS;  // per scale set: written by the four scale warps / read by its MMAs
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int aps = p.nv ? 4 : 2;  // 512-byte scale atoms per k-step
    const uint32_t sf_bytes = (uint32_t)aps * 512u, bbytes = (uint32_t)p.ncol * 128u;
    const uint32_t b_off = 16384u, sfa_off = b_off + bbytes, sfb_off = sfa_off + sf_bytes;  // inside a stage
    const int64_t u_begin = fd_first(p, (int)blockIdx.x), u_end = fd_first(p, (int)blockIdx.x + 1);
    volatile int *abort_flag = &abort_s;

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < FD_MAX_STAGES; s++) {
            tc::mbar_init(full + 8 * s, 1);
            tc::mbar_init(empty + 8 * s, 1);
        }
        tc::mbar_init(accum, 1);
        tc::mbar_init(tmem_free, 4);
        for (int s = 0; s < FD_SF_SETS; s++) {
            tc::mbar_init(sf_full + 8 * s, 4);
            tc::mbar_init(sf_empty + 8 * s, 1);
        }
        tc::mbar_init_fence();
    }
    if (warp == 1) tc::tmem_alloc(tc::smem_u32(&tmem_base_s), FD_TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = tmem_base_s;

    if (warp == 0) {
        if (lane == 0) {
            // ---------------- copies ----------------
            // The weights do not depend on the staging kernel in front of this grid (programmatic dependent
            // launch): the first ring-full of weight tiles is requested before the dependency wait, the digit
            // tiles of those stages after it.
            const int64_t total = u_end - u_begin;
            const int pre = (int)(total < p.stages ? total : p.stages);
            for (int i = 0; i < pre; i++) {
                const int64_t u = u_begin + i;
                const int tile = (int)(u / p.nks), ks = (int)(u - (int64_t)tile * p.nks);
                const uint32_t st = smem_s + (uint32_t)(i * p.stage_bytes);
                tc::mbar_expect_tx(full + 8 * i, 16384u + bbytes + 2 * sf_bytes);
                const size_t wt = (size_t)tile * p.nks + ks;
                fd_bulk(st, p.qw + wt * 16384, 16384u, full + 8 * i);
                fd_bulk(st + sfa_off, p.sfw + wt * sf_bytes, sf_bytes, full + 8 * i);
            }
            asm volatile("griddepcontrol.wait;\n" ::: "memory");  // the digit planes and gtok are complete from here on
            for (int i = 0; i < pre; i++) {
                const int64_t u = u_begin + i;
                const int ks = (int)(u % p.nks);
                const uint32_t st = smem_s + (uint32_t)(i * p.stage_bytes);
                fd_bulk(st + b_off, p.qx + (size_t)ks * 16384, bbytes, full + 8 * i);
                fd_bulk(st + sfb_off, p.sfx + (size_t)ks * sf_bytes, sf_bytes, full + 8 * i);
            }
            int slot = pre == p.stages ? 0 : pre, round = pre == p.stages ? 1 : 0;
            for (int64_t u = u_begin + pre; u < u_end; u++) {
                const int tile = (int)(u / p.nks), ks = (int)(u - (int64_t)tile * p.nks);
                if (round > 0 && !tc::mbar_wait(empty + 8 * slot, (uint32_t)((round - 1) & 1), abort_flag)) {
                    abort_s = 1;
                    atomicExch(p.status, 51);
                    break;
                }
                const uint32_t st = smem_s + (uint32_t)(slot * p.stage_bytes);
                tc::mbar_expect_tx(full + 8 * slot, 16384u + bbytes + 2 * sf_bytes);
                const size_t wt = (size_t)tile * p.nks + ks;
                fd_bulk(st, p.qw + wt * 16384, 16384u, full + 8 * slot);
                fd_bulk(st + sfa_off, p.sfw + wt * sf_bytes, sf_bytes, full + 8 * slot);
                fd_bulk(st + b_off, p.qx + (size_t)ks * 16384, bbytes, full + 8 * slot);
                fd_bulk(st + sfb_off, p.sfx + (size_t)ks * sf_bytes, sf_bytes, full + 8 * slot);
                if (++slot == p.stages) slot = 0, round++;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- MMA issue ----------------
            // The scale factors are put into tensor memory by the scale warps (below), not by tcgen05.cp from this thread:
            // a copy occupies the tensor pipe for ~120 cycles here, eight of them per k-step (NVFP4) were more than half of
            // the k-step and held the kernel at 0.46 of the HBM bandwidth (MXFP4, four copies: 0.62).
            int slot = 0, round = 0, seg = 0;
            uint32_t g = 0;  // k-steps issued by this CTA so far
            bool ok = true;
            for (int64_t u = u_begin; u < u_end && ok; seg++) {
                const int tile = (int)(u / p.nks), j0 = (int)(u - (int64_t)tile * p.nks);
                const int j1 = (int)min((int64_t)p.nks, (int64_t)j0 + (u_end - u));
                // the accumulator is rewritten from the segment's first MMA on: the previous epilogue must be done
                if (seg > 0 && !tc::mbar_wait(tmem_free, (uint32_t)((seg - 1) & 1), abort_flag)) ok = false;
                tc::fence_after_sync();
                for (int ks = j0; ks < j1 && ok; ks++, g++) {
                    const uint32_t b = g % FD_SF_SETS;
                    if (!tc::mbar_wait(full + 8 * slot, (uint32_t)(round & 1), abort_flag) ||
                        !tc::mbar_wait(sf_full + 8 * b, (g / FD_SF_SETS) & 1u, abort_flag)) {
                        ok = false;
                        break;
                    }
                    tc::fence_after_sync();
                    const uint32_t st = smem_s + (uint32_t)(slot * p.stage_bytes);
                    const uint64_t ad = tc::smem_desc_sw128(st), bd = tc::smem_desc_sw128(st + b_off);
                    const uint32_t tsfa = tmem + 128u + 32u * b, tsfb = tsfa + 16u;
                    const uint32_t first = (uint32_t)(ks != j0);
                    if (p.nv) {
                        const uint32_t idesc = tc::idesc_fp4(128, p.ncol, 0, 0, 0);
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            tc::mma_nvf4(tmem, ad + 2 * j, bd + 2 * j, idesc, first | (uint32_t)(j != 0), tsfa + 4 * j, tsfb + 4 * j);
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const int id = (j & 1) * 2;
                            tc::mma_mxf4(tmem, ad + 2 * j, bd + 2 * j, tc::idesc_fp4(128, p.ncol, 1, id, id), first | (uint32_t)(j != 0),
                                         tsfa + 4 * (j >> 1), tsfb + 4 * (j >> 1));
                        }
                    }
                    tc::mma_commit(empty + 8 * slot);
                    tc::mma_commit(sf_empty + 8 * b);
                    if (++slot == p.stages) slot = 0, round++;
                }
                if (!ok) {
                    abort_s = 1;
                    atomicExch(p.status, 52);
                    break;
                }
                tc::mma_commit(accum);
                u += j1 - j0;
            }
        }
    } else if (warp >= 6) {
        // ---------------- scale warps: stage -> tensor memory, lane quadrant warp % 4 ----------------
        // An atom is 128 rows x 4 scale bytes: row r's bytes at (r % 32) * 16 + (r / 32) * 4.  Lane l reads its 16 bytes of
        // every atom (weight atoms -> columns 4j of the set, digit atoms -> columns 16 + 4j) and writes all 32 columns of
        // its own lane with ONE tcgen05.st: what tcgen05.cp.32x128b.warpx4 would leave there, every quadrant a copy.
        const uint32_t quad_lane = (uint32_t)(32 * (warp & 3)) << 16;
        int slot = 0, round = 0;
        uint32_t g = 0;
        bool ok = true;
        for (int64_t u = u_begin; u < u_end && ok; u++, g++) {
            const uint32_t b = g % FD_SF_SETS;
            ok = tc::mbar_wait(full + 8 * slot, (uint32_t)(round & 1), abort_flag) &&
                 (g < (uint32_t)FD_SF_SETS || tc::mbar_wait(sf_empty + 8 * b, (g / FD_SF_SETS - 1) & 1u, abort_flag));
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0 && !abort_s) {
                    abort_s = 1;
                    atomicExch(p.status, 54);
                }
                break;
            }
            tc::fence_after_sync();
            const uint32_t st = smem_s + (uint32_t)(slot * p.stage_bytes) + 16u * (uint32_t)lane;
            uint32_t w[32];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                // with two atoms per k-step (MXFP4) the upper columns take stale bytes that no MMA reads
                const uint32_t ja = (uint32_t)(j < aps ? j : 0);
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(w[4 * j]), "=r"(w[4 * j + 1]), "=r"(w[4 * j + 2]), "=r"(w[4 * j + 3]) : "r"(st + sfa_off + 512u * ja));
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(w[16 + 4 * j]), "=r"(w[17 + 4 * j]), "=r"(w[18 + 4 * j]), "=r"(w[19 + 4 * j]) : "r"(st + sfb_off + 512u * ja));
            }
            tc::tmem_st32(tmem + quad_lane + 128u + 32u * b, w);
            tc::tmem_st_wait();
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(sf_full + 8 * b);
            if (++slot == p.stages) slot = 0, round++;
        }
    } else {
        // ---------------- epilogue warps: TMEM lane quadrant = warp % 4 = 32 weight rows ----------------
        const int quad = warp & 3;
        bool ok = true;
        int seg = 0;
        for (int64_t u = u_begin; u < u_end && ok; seg++) {
            const int tile = (int)(u / p.nks), j0 = (int)(u - (int64_t)tile * p.nks);
            const int j1 = (int)min((int64_t)p.nks, (int64_t)j0 + (u_end - u));
            ok = __all_sync(0xffffffffu, tc::mbar_wait(accum, (uint32_t)(seg & 1), abort_flag));
            if (!ok) break;
            tc::fence_after_sync();
            // o[t] = sum_j 4^-j * column 8t + j
            float o[GLLMK_GEMV_MAX_M];
#pragma unroll
            for (int t = 0; t < GLLMK_GEMV_MAX_M; t++) o[t] = 0.0f;
#pragma unroll
            for (int c = 0; c < 128; c += 32) {
                if (c < p.ncol) {
                    uint32_t v[32];
                    tc::tmem_ld32(tmem + ((uint32_t)(32 * quad) << 16) + (uint32_t)c, v);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int tt = 0; tt < 4; tt++) {
                        float acc = 0.0f, wgt = 1.0f;
#pragma unroll
                        for (int j = 0; j < FD_DIGITS; j++) {
                            acc = fmaf(__uint_as_float(v[8 * tt + j]), wgt, acc);
                            wgt *= 0.25f;
                        }
                        o[c / 8 + tt] = acc;
                    }
                }
            }
            // the accumulator may be overwritten now
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(tmem_free);
            const bool whole = j0 == 0 && j1 == p.nks;
            const int rloc = 32 * quad + lane;
            bool store = whole;
            if (!whole) {
                // the row tile is shared: publish the partial, count arrivals; the last CTA to arrive sums all
                // partials in k order
                float *mine = p.partial + ((size_t)blockIdx.x * 2 + (j0 != 0 ? 0 : 1)) * (GLLMK_GEMV_MAX_M * 128);
#pragma unroll
                for (int t = 0; t < GLLMK_GEMV_MAX_M; t++)
                    if (t < p.m) __stcg(mine + t * 128 + rloc, o[t]);
                const int64_t ut = (int64_t)tile * p.nks;
                const int c_first = fd_cta_of(p, ut), nseg = fd_cta_of(p, ut + p.nks - 1) - c_first + 1;
                __threadfence();
                tc::named_bar_sync(1, 128);
                if (warp == 2 && lane == 0) {
                    const int old = atomicAdd(p.counters + tile, 1);
                    const int last = old == nseg - 1;
                    if (last) p.counters[tile] = 0;  // zero again for the next launch
                    last_s = last;
                }
                tc::named_bar_sync(1, 128);
                store = last_s != 0;
                if (store) {
                    __threadfence();
#pragma unroll
                    for (int t = 0; t < GLLMK_GEMV_MAX_M; t++) o[t] = 0.0f;
                    for (int sgi = 0; sgi < nseg; sgi++) {
                        // the tile's first segment is the head of its CTA's share (slot 1), the others are tails (slot 0)
                        const float *src = p.partial + ((size_t)(c_first + sgi) * 2 + (sgi == 0 ? 1 : 0)) * (GLLMK_GEMV_MAX_M * 128);
#pragma unroll
                        for (int t = 0; t < GLLMK_GEMV_MAX_M; t++)
                            if (t < p.m) o[t] += __ldcg(src + t * 128 + rloc);
                    }
                }
                tc::named_bar_sync(1, 128);  // last_s is rewritten by the next shared segment
            }
            if (store) {
                const int64_t row = (int64_t)tile * 128 + rloc;
                if (row < p.n) {
#pragma unroll
                    for (int t = 0; t < GLLMK_GEMV_MAX_M; t++)
                        if (t < p.m) p.y[(int64_t)t * p.yst + row * p.ysr] = o[t] * (p.wscale * __ldcg(p.gtok + t));
                }
            }
            u += j1 - j0;
        }
        if (!ok && !abort_s) {
            abort_s = 1;
            atomicExch(p.status, 53);
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem, FD_TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
int32_t gemv_fp4_launch(Ctx *c, const Weight *w, const float *x, int64_t xst, int64_t xsk, int m, float *y, int64_t yst, int64_t ysr,
                        cudaStream_t s) {
    static bool attr_set[64] = {};  // function attributes are per device
    const int dev_slot = c->device & 63;
    if (!attr_set[dev_slot]) {
        GK_CUDA(c, cudaFuncSetAttribute(gemv_fp4_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FD_SMEM_BUDGET));
        attr_set[dev_slot] = true;
    }
    const int nv = w->qt == GLLMK_QUANT_NVFP4;
    const size_t data_bytes = (size_t)128 * (size_t)(w->k_pad / 2), sf_bytes = (size_t)128 * (size_t)(w->k_pad / (nv ? 16 : 32));
    int32_t rc = ensure_act(c, data_bytes + sf_bytes + 256);
    if (rc) return rc;
    uint8_t *qx = static_cast<uint8_t *>(c->act), *sfx = qx + data_bytes;
    float *gtok = reinterpret_cast<float *>(sfx + sf_bytes);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    {
        cudaLaunchConfig_t scfg = {};
        scfg.gridDim = dim3((unsigned)((w->k_pad / 32 + 7) / 8), (unsigned)m);
        scfg.blockDim = dim3(256);
        scfg.stream = s;
        scfg.attrs = attr;
        scfg.numAttrs = c->gemv_pdl != 0 ? 1 : 0;
        GK_CUDA(c, cudaLaunchKernelEx(&scfg, fd_stage_kernel, x, xst, xsk, w->k, w->k_pad, nv, qx, sfx, gtok));
    }

    FdParams p{};
    p.qw = static_cast<const uint8_t *>(w->qs);
    p.sfw = static_cast<const uint8_t *>(w->aux);
    p.qx = qx;
    p.sfx = sfx;
    p.gtok = gtok;
    p.wscale = w->global_scale;
    p.nv = nv;
    p.n = w->n;
    p.nks = (int)(w->k_pad / 256);
    p.m = m;
    p.ncol = (FD_DIGITS * m + 31) / 32 * 32;
    p.stage_bytes = (16384 + p.ncol * 128 + 2 * (nv ? 2048 : 1024) + 1023) / 1024 * 1024;
    p.stages = (FD_SMEM_BUDGET - 1024) / p.stage_bytes;
    if (p.stages > FD_MAX_STAGES) p.stages = FD_MAX_STAGES;
    p.y = y;
    p.yst = yst;
    p.ysr = ysr;
    p.row_tiles = (int)(w->n_pad / 128);
    const int64_t units = (int64_t)p.row_tiles * p.nks;
    const int grid = (int)(units < c->sm_count ? units : c->sm_count);
    p.per_cta = units / grid;
    p.rem = (int)(units % grid);
    rc = ensure_red(c, (size_t)grid * 2 * GLLMK_GEMV_MAX_M * 128 * sizeof(float));
    if (!rc) rc = ensure_cnt(c, (size_t)p.row_tiles * sizeof(int));
    if (rc) return rc;
    p.partial = static_cast<float *>(c->red);
    p.counters = static_cast<int *>(c->cnt);
    p.status = c->status_dev;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(FD_THREADS);
    cfg.dynamicSmemBytes = (size_t)p.stages * p.stage_bytes + 1024;
    cfg.stream = s;
    cfg.attrs = attr;
    cfg.numAttrs = c->gemv_pdl != 0 ? 1 : 0;
    GK_CUDA(c, cudaLaunchKernelEx(&cfg, gemv_fp4_tc_kernel, p));
    return GLLMK_STATUS_OK;
}

}  // namespace gllmk
