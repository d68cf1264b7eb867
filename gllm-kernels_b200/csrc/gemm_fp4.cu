// Prefill GEMM with both operands in FP4: native block-scaled tcgen05 MMA.
//
//   Y[t, r] = gW * gX * sum_k W4[r, k] * X4[t, k]      (NVFP4: E2M1 values, UE4M3 scale per 16 elements)
//             (MXFP4: E2M1 values, UE8M0 scale per 32 elements, gW = gX = 1)
//
// Both operands are resident in the FP4 plane layout of common.cuh: packed nibbles stored as ready-made
// 128-byte-swizzled shared-memory tile images (128 rows x 256 elements = 16 KB, contiguous) + scale bytes in
// 128-row x 4-scale atoms.  Per k-step of 256 elements a CTA brings in, with plain bulk copies (no tensor
// map, no multicast):
//   A = one weight tile, B = one or two activation tiles, and their scale atoms;
// one thread copies the scale atoms to tensor memory (tcgen05.cp) and issues four
// tcgen05.mma.kind::mxf4nvf4.block_scale (K = 64 each; kind::mxf4 for MXFP4) into a 128 x 256 f32
// accumulator in TMEM; eight warps read it back, apply the two per-tensor scales and store Y (transposed through shared
// memory, 16 bytes per lane).
#include <cuda_bf16.h>

#include "common.cuh"
#include "tc05.cuh"

namespace gllmk {

constexpr int F4_BM = 128, F4_BN = 256;
constexpr int F4_STAGES = 4;
constexpr int F4_A_BYTES = F4_BM * 128, F4_B_BYTES = F4_BN * 128;
constexpr int F4_SFA_BYTES = 2048;          // 4 atoms (128 rows x 16 scales of 16 el; MXFP4 uses 2 of them)
constexpr int F4_SFB_BYTES = 4096;
constexpr int F4_STAGE_BYTES = F4_A_BYTES + F4_B_BYTES + F4_SFA_BYTES + F4_SFB_BYTES;
constexpr int F4_EPI_WARPS = 8;              // two per TMEM lane quadrant, each takes every other block of 32 tokens
constexpr int F4_THREADS = 64 + 32 * F4_EPI_WARPS;  // warp 0: copies, warp 1: MMA + TMEM, then the epilogue warps
constexpr size_t F4_SMEM = (size_t)F4_STAGES * F4_STAGE_BYTES + 1024;
constexpr uint32_t F4_TMEM_COLS = 512;      // 256 accumulator + 2 x (16 SFA + 32 SFB), power of two
constexpr uint32_t F4_TMEM_SF = 256;        // scale-factor columns, two sets of 48 used by alternate k-steps

struct Fp4Params {
    const uint8_t *qw, *qx;  // data planes (tile images)
    const uint8_t *sfw;  // weight scale plane
    const uint8_t *sfx;  // activation scale plane
    int nv;              // 1: NVFP4 (scale per 16, UE4M3), 0: MXFP4 (scale per 32, UE8M0)
    int64_t n, k;
    int m;
    int64_t x_row_tiles; // 128-row groups in the activation planes
    float scale;         // gW * gX
    void *y;
    int y_bf16;
    int64_t ldy;
    int vec;             // Y allows 16-byte stores
    int *status;
};

__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(bar)
                 : "memory");
}
// shared-memory descriptor of one 512-byte scale atom for tcgen05.cp: no swizzle, 8 x 16-byte core
// matrices 128 bytes apart (SBO = 128, LBO = 0)
__device__ __forceinline__ uint64_t sf_desc(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)(128 >> 4) << 32) | ((uint64_t)1 << 46);
}

__global__ void __launch_bounds__(F4_THREADS, 1)
gemm_fp4_kernel(const __grid_constant__ Fp4Params p, const int ntok) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[2 * F4_STAGES + 1];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    const uint32_t smem_s = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t full = tc::smem_u32(&bars[0]), empty = tc::smem_u32(&bars[F4_STAGES]), accum = tc::smem_u32(&bars[2 * F4_STAGES]);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t row0 = (int64_t)blockIdx.x * F4_BM, tok0 = (int64_t)blockIdx.y * F4_BN;
    const int nks = (int)(p.k / 256);
    const int64_t atoms_per_row_tile = p.nv ? (p.k >> 6) : (p.k >> 7);  // 512-byte atoms per 128 rows
    const int atoms_per_stage = p.nv ? 4 : 2;
    volatile int *abort_flag = &abort_s;

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < F4_STAGES; s++) {
            tc::mbar_init(full + 8 * s, 1);
            tc::mbar_init(empty + 8 * s, 1);
        }
        tc::mbar_init(accum, 1);
        tc::mbar_init_fence();
    }
    if (warp == 1) tc::tmem_alloc(tc::smem_u32(&tmem_base_s), F4_TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = tmem_base_s;

    if (warp == 0 && lane == 0) {
        // ---------------- TMA producer ----------------
        const uint32_t sf_bytes = (uint32_t)atoms_per_stage * 512u;
        // 128-row groups of the activation tile that exist in the planes (rows beyond them keep whatever the
        // stage held: they only reach output columns that are never stored)
        const int btiles = min((ntok + 127) / 128, (int)(p.x_row_tiles - (tok0 >> 7)));
        const uint32_t tx = F4_A_BYTES + (16384u + sf_bytes) * (uint32_t)btiles + sf_bytes;
        const size_t ktiles = (size_t)nks;
        for (int ks = 0; ks < nks; ks++) {
            const int s = ks % F4_STAGES;
            if (ks >= F4_STAGES && !tc::mbar_wait(empty + 8 * s, (uint32_t)((ks / F4_STAGES - 1) & 1), abort_flag)) {
                abort_s = 1;
                atomicExch(p.status, 21);
                break;
            }
            const uint32_t st = smem_s + s * F4_STAGE_BYTES;
            tc::mbar_expect_tx(full + 8 * s, tx);
            bulk_load(st, p.qw + ((size_t)blockIdx.x * ktiles + ks) * 16384, 16384u, full + 8 * s);
            for (int bt = 0; bt < btiles; bt++)
                bulk_load(st + F4_A_BYTES + bt * 16384, p.qx + (((size_t)(tok0 >> 7) + bt) * ktiles + ks) * 16384, 16384u, full + 8 * s);
            bulk_load(st + F4_A_BYTES + F4_B_BYTES,
                      p.sfw + ((size_t)blockIdx.x * atoms_per_row_tile + (size_t)ks * atoms_per_stage) * 512, sf_bytes, full + 8 * s);
            for (int bt = 0; bt < btiles; bt++)
                bulk_load(st + F4_A_BYTES + F4_B_BYTES + F4_SFA_BYTES + bt * 2048,
                          p.sfx + (((size_t)(tok0 >> 7) + bt) * atoms_per_row_tile + (size_t)ks * atoms_per_stage) * 512, sf_bytes,
                          full + 8 * s);
        }
    } else if (warp == 1 && lane == 0) {
        // ---------------- scale copies + MMA issue ----------------
        for (int ks = 0; ks < nks; ks++) {
            const int s = ks % F4_STAGES;
            if (!tc::mbar_wait(full + 8 * s, (uint32_t)((ks / F4_STAGES) & 1), abort_flag)) {
                abort_s = 1;
                atomicExch(p.status, 22);
                break;
            }
            tc::fence_after_sync();
            const uint32_t st = smem_s + s * F4_STAGE_BYTES;
            const uint32_t sfa = st + F4_A_BYTES + F4_B_BYTES, sfb = sfa + F4_SFA_BYTES;
            const uint64_t ad = tc::smem_desc_sw128(st), bd = tc::smem_desc_sw128(st + F4_A_BYTES);
            // alternate scale-factor column sets so the copies of this k-step do not have to wait for the
            // MMAs of the previous one to finish reading theirs
            const uint32_t F4_TMEM_SFA = F4_TMEM_SF + 48u * (uint32_t)(ks & 1), F4_TMEM_SFB = F4_TMEM_SFA + 16u;
            if (p.nv) {
                // atom j holds the four 16-element scales of MMA j (K = 64): 4 TMEM columns each
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    tc::tmem_cp_sf(tmem + F4_TMEM_SFA + 4 * j, sf_desc(sfa + 512 * j));
                    tc::tmem_cp_sf(tmem + F4_TMEM_SFB + 8 * j, sf_desc(sfb + 512 * j));
                    if (ntok > 128) tc::tmem_cp_sf(tmem + F4_TMEM_SFB + 8 * j + 4, sf_desc(sfb + 2048 + 512 * j));
                }
                const uint32_t idesc = tc::idesc_fp4(F4_BM, ntok, 0, 0, 0);
#pragma unroll
                for (int j = 0; j < 4; j++)
                    tc::mma_nvf4(tmem, ad + 2 * j, bd + 2 * j, idesc, (uint32_t)((ks | j) != 0), tmem + F4_TMEM_SFA + 4 * j,
                                 tmem + F4_TMEM_SFB + 8 * j);
            } else {
                // atom j holds the four 32-element scales of MMAs 2j and 2j+1 (two scales each: sf id 0 / 2)
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    tc::tmem_cp_sf(tmem + F4_TMEM_SFA + 4 * j, sf_desc(sfa + 512 * j));
                    tc::tmem_cp_sf(tmem + F4_TMEM_SFB + 8 * j, sf_desc(sfb + 512 * j));
                    if (ntok > 128) tc::tmem_cp_sf(tmem + F4_TMEM_SFB + 8 * j + 4, sf_desc(sfb + 2048 + 512 * j));
                }
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int id = (j & 1) * 2;
                    tc::mma_mxf4(tmem, ad + 2 * j, bd + 2 * j, tc::idesc_fp4(F4_BM, ntok, 1, id, id), (uint32_t)((ks | j) != 0),
                                 tmem + F4_TMEM_SFA + 4 * (j >> 1), tmem + F4_TMEM_SFB + 8 * (j >> 1));
                }
            }
            tc::mma_commit(empty + 8 * s);
        }
        tc::mma_commit(accum);
    }
    __syncwarp();

    if (warp >= 2) {
        // ---------------- epilogue: warp w reads TMEM lane quadrant w % 4 = weight rows ----------------
        const int quad = warp & 3;
        bool ok = !abort_s && tc::mbar_wait(accum, 0u, abort_flag);
        if (!ok && !abort_s) {
            abort_s = 1;
            atomicExch(p.status, 23);
        }
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc::fence_after_sync();
            // all MMAs have completed, so the pipeline stages are free: each epilogue warp stages its blocks in 4 KB
            // of stage 0
            uint8_t *stage = smem_raw + (smem_s - tc::smem_u32(smem_raw)) + (warp - 2) * 4096;
            for (int c = 32 * ((warp - 2) >> 2); c < ntok; c += 32 * (F4_EPI_WARPS / 4)) {
                uint32_t v[32];
                tc::tmem_ld32(tmem + ((uint32_t)(32 * quad) << 16) + (uint32_t)c, v);
                tc::tmem_ld_wait();
                float o[32];
#pragma unroll
                for (int j = 0; j < 32; j++) o[j] = __uint_as_float(v[j]) * p.scale;
                if (p.y_bf16) tc::store_block_32x32<true>(p.y, p.ldy, row0 + 32 * quad, tok0 + c, p.n, p.m, o, stage, lane, p.vec);
                else tc::store_block_32x32<false>(p.y, p.ldy, row0 + 32 * quad, tok0 + c, p.n, p.m, o, stage, lane, p.vec);
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem, F4_TMEM_COLS);
}


// ---------------------------------------------------------------------------------------------
// CTA-pair version (m > 128): persistent, two CTAs of a cluster on two SMs work on one 256-row x 256-token tile.
//
// Two things bound the one-CTA kernel above.  (1) What an SM can pull from L2: 54 KB per k-step for 8.4 M
// multiply-adds.  As a pair (tcgen05 cta_group::2, MMA M = 256) each CTA brings in its own 128 weight rows, HALF of
// the activation tile (the tensor core reads the other half from the partner's shared memory) and the scale atoms:
// 38 KB per k-step for the same multiply-adds per SM.  (2) The scale-factor copies: twelve tcgen05.cp per k-step run
// on the tensor pipe itself and take as long as the four MMAs they feed (measured with the MMA issued back to back
// on resident operands: 6.0 PFLOP/s without the copies, 3.1 with them).  Here the scale factors never touch that
// pipe: four "scale warps" per CTA (one per tensor-memory lane quadrant) read the atoms from the stage with 16-byte
// shared-memory loads and write them to tensor memory with tcgen05.st — the layout tcgen05.cp.32x128b.warpx4 would
// produce: lane = row % 32, one column per group of 32 rows, every quadrant a copy — three sets of columns in rotation.
//
// The kernel is persistent (grid = resident pairs, tiles dealt round robin), so the copy threads and the scale
// warps run ahead into the next tile while the accumulator of the finished one is stored.
//
// Per CTA: warp 0 lane 0 copies; warp 1 lane 0 issues the MMAs (leader = cluster rank 0) or forwards "my stage is
// full" to the leader (rank 1), because a wait on an mbarrier can only be done by its own CTA; warps 2..9 store the
// CTA's 128 rows x 256 tokens of the accumulator; warps 10..13 are the scale warps.  Loads are plain bulk copies:
// nothing is multicast.
// ---------------------------------------------------------------------------------------------
constexpr int P4_STAGES = 5;
constexpr int P4_A_BYTES = 16384, P4_B_BYTES = 16384, P4_SFA_BYTES = 2048, P4_SFB_BYTES = 4096;
constexpr int P4_STAGE_BYTES = P4_A_BYTES + P4_B_BYTES + P4_SFA_BYTES + P4_SFB_BYTES;
constexpr int P4_EPI_WARPS = 8, P4_SF_WARPS = 4;
constexpr int P4_THREADS = 64 + 32 * (P4_EPI_WARPS + P4_SF_WARPS);
constexpr size_t P4_SMEM = (size_t)P4_STAGES * P4_STAGE_BYTES + (size_t)P4_EPI_WARPS * 4096 + 1024;
constexpr uint32_t P4_TMEM_COLS = 512;                     // 256 accumulator + 3 x 48 scale-factor columns, power of two
constexpr int P4_SF_SETS = 3;                              // scale-factor column sets in rotation
constexpr uint32_t P4_TMEM_SF = 256, P4_SF_SET_COLS = 48;  // per set: SFA 16 columns, then SFB 32

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P4_THREADS, 1)
gemm_fp4_pair_kernel(const __grid_constant__ Fp4Params p, const int row_tiles, const int tok_tiles) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[4 * P4_STAGES + P4_SF_SETS + 2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    const uint32_t smem_s = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t full = tc::smem_u32(&bars[0]), empty = tc::smem_u32(&bars[P4_STAGES]), full2 = tc::smem_u32(&bars[2 * P4_STAGES]);
    const uint32_t sf_landed = tc::smem_u32(&bars[3 * P4_STAGES]);  // per stage: its scale atoms have landed (they are
                                                                     // requested first and are a sixth of the stage's bytes)
    const uint32_t sf_full = tc::smem_u32(&bars[4 * P4_STAGES]);
    const uint32_t accum_full = tc::smem_u32(&bars[4 * P4_STAGES + P4_SF_SETS]), accum_empty = accum_full + 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = tc::cluster_ctarank();
    const int pair = (int)(blockIdx.x >> 1), npairs = (int)(gridDim.x >> 1);
    const int row_pairs = (row_tiles + 1) >> 1;
    const int ntiles = row_pairs * tok_tiles;
    const int nks = (int)(p.k / 256);
    const int64_t atoms_per_row_tile = p.nv ? (p.k >> 6) : (p.k >> 7);
    const int atoms_per_stage = p.nv ? 4 : 2;
    volatile int *abort_flag = &abort_s;

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < P4_STAGES; s++) {
            tc::mbar_init(full + 8 * s, 1);
            tc::mbar_init(empty + 8 * s, 1);
            tc::mbar_init(full2 + 8 * s, 1);
            tc::mbar_init(sf_landed + 8 * s, 1);
        }
        for (int s = 0; s < P4_SF_SETS; s++) tc::mbar_init(sf_full + 8 * s, 2 * P4_SF_WARPS);  // the scale warps of both CTAs (leader only)
        tc::mbar_init(accum_full, 1);
        tc::mbar_init(accum_empty, 2 * P4_EPI_WARPS);
        tc::mbar_init_fence();
    }
    if (warp == 1) tc::tmem_alloc_pair(tc::smem_u32(&tmem_base_s), P4_TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    // both CTAs' barriers exist before either CTA arrives on the other's
    tc::cluster_arrive();
    tc::cluster_wait();
    tc::fence_after_sync();
    const uint32_t tmem = tmem_base_s;

    if (warp == 0 && lane == 0) {
        // ---------------- copies: own weight rows, own half of the activation tile, scale atoms ----------------
        const uint32_t sf_bytes = (uint32_t)atoms_per_stage * 512u;
        const size_t ktiles = (size_t)nks;
        uint32_t g = 0;
        for (int t = pair; t < ntiles && !*abort_flag; t += npairs) {
            const int rp = t / tok_tiles, tt = t % tok_tiles;
            const int64_t my_row_tile = 2 * (int64_t)rp + rank;
            const bool a_ok = my_row_tile < row_tiles;
            const int64_t b_tile0 = 2 * (int64_t)tt;  // 128-token groups of this tile: b_tile0 (leader's half), + 1 (partner's)
            const bool b_ok = b_tile0 + rank < p.x_row_tiles;
            const bool sfb_ok[2] = {b_tile0 < p.x_row_tiles, b_tile0 + 1 < p.x_row_tiles};
            // rows / tokens that do not exist are not copied: whatever the stage holds there only reaches accumulator
            // rows / columns that are never stored
            // The scale atoms go first and signal a barrier of their own: the scale warps turn them into tensor-memory
            // columns while the operand tiles of the same stage are still in flight (with one barrier for the whole
            // stage the MMA thread waited ~190 cycles per k-step for the scale sets after the operands had landed).
            const uint32_t tx_sf = (a_ok ? sf_bytes : 0u) + ((uint32_t)sfb_ok[0] + (uint32_t)sfb_ok[1]) * sf_bytes;
            const uint32_t tx = (a_ok ? 16384u : 0u) + (b_ok ? 16384u : 0u);
            for (int ks = 0; ks < nks; ks++, g++) {
                const uint32_t s = g % P4_STAGES;
                if (g >= P4_STAGES && !tc::mbar_wait_cluster(empty + 8 * s, (g / P4_STAGES - 1) & 1u, abort_flag)) {
                    abort_s = 1;
                    atomicExch(p.status, 24);
                    break;
                }
                const uint32_t st = smem_s + s * P4_STAGE_BYTES;
                tc::mbar_expect_tx(sf_landed + 8 * s, tx_sf);
                if (a_ok)
                    bulk_load(st + P4_A_BYTES + P4_B_BYTES, p.sfw + ((size_t)my_row_tile * atoms_per_row_tile + (size_t)ks * atoms_per_stage) * 512,
                              sf_bytes, sf_landed + 8 * s);
                for (int h = 0; h < 2; h++)
                    if (sfb_ok[h])
                        bulk_load(st + P4_A_BYTES + P4_B_BYTES + P4_SFA_BYTES + h * 2048,
                                  p.sfx + ((size_t)(b_tile0 + h) * atoms_per_row_tile + (size_t)ks * atoms_per_stage) * 512, sf_bytes,
                                  sf_landed + 8 * s);
                tc::mbar_expect_tx(full + 8 * s, tx);
                if (a_ok) bulk_load(st, p.qw + ((size_t)my_row_tile * ktiles + ks) * 16384, 16384u, full + 8 * s);
                if (b_ok) bulk_load(st + P4_A_BYTES, p.qx + ((size_t)(b_tile0 + rank) * ktiles + ks) * 16384, 16384u, full + 8 * s);
            }
        }
    } else if (warp == 1 && lane == 0 && rank != 0) {
        // ---------------- partner CTA: tell the leader when this CTA's stage has landed ----------------
        uint32_t g = 0;
        for (int t = pair; t < ntiles && !*abort_flag; t += npairs)
            for (int ks = 0; ks < nks; ks++, g++) {
                const uint32_t s = g % P4_STAGES;
                if (!tc::mbar_wait(full + 8 * s, (g / P4_STAGES) & 1u, abort_flag)) {
                    abort_s = 1;
                    atomicExch(p.status, 25);
                    t = ntiles;
                    break;
                }
                tc::mbar_arrive_cluster_relaxed(tc::map_to_cta(full2 + 8 * s, 0));
            }
    } else if (warp == 1 && lane == 0) {
        // ---------------- leader CTA: MMA issue for the pair ----------------
        const uint32_t idesc_nv = tc::idesc_fp4(256, 256, 0, 0, 0);
        uint32_t g = 0, it = 0;
        for (int t = pair; t < ntiles && !*abort_flag; t += npairs, it++) {
            // the accumulator of the previous tile has been read out by all sixteen epilogue warps of the pair
            if (it > 0 && !tc::mbar_wait_cluster(accum_empty, (it - 1) & 1u, abort_flag)) {
                abort_s = 1;
                atomicExch(p.status, 26);
                break;
            }
            tc::fence_after_sync();
            bool ok = true;
            for (int ks = 0; ks < nks; ks++, g++) {
                const uint32_t s = g % P4_STAGES, ph = (g / P4_STAGES) & 1u;
                const uint32_t b = g % P4_SF_SETS, bph = (g / P4_SF_SETS) & 1u;
                // both CTAs' operand tiles have landed, and both CTAs' scale warps have filled column set b
                if (!tc::mbar_wait(full + 8 * s, ph, abort_flag) || !tc::mbar_wait_cluster(full2 + 8 * s, ph, abort_flag) ||
                    !tc::mbar_wait_cluster(sf_full + 8 * b, bph, abort_flag)) {
                    abort_s = 1;
                    atomicExch(p.status, 22);
                    ok = false;
                    break;
                }
                tc::fence_after_sync();
                const uint32_t st = smem_s + s * P4_STAGE_BYTES;
                const uint64_t ad = tc::smem_desc_sw128(st), bd = tc::smem_desc_sw128(st + P4_A_BYTES);
                const uint32_t tsfa = tmem + P4_TMEM_SF + P4_SF_SET_COLS * b, tsfb = tsfa + 16;
                if (p.nv) {
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        tc::mma_nvf4_pair(tmem, ad + 2 * j, bd + 2 * j, idesc_nv, (uint32_t)((ks | j) != 0), tsfa + 4 * j, tsfb + 8 * j);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const int id = (j & 1) * 2;
                        tc::mma_mxf4_pair(tmem, ad + 2 * j, bd + 2 * j, tc::idesc_fp4(256, 256, 1, id, id), (uint32_t)((ks | j) != 0),
                                          tsfa + 4 * (j >> 1), tsfb + 8 * (j >> 1));
                    }
                }
                // once these MMAs have completed, stage s and column set b are free in BOTH CTAs
                tc::mma_commit_pair(empty + 8 * s);
                tc::mma_commit_pair(tc::map_to_cta(empty + 8 * s, 1));
            }
            if (!ok) break;
            tc::mma_commit_pair(accum_full);
            tc::mma_commit_pair(tc::map_to_cta(accum_full, 1));
        }
    } else if (warp >= 2 + P4_EPI_WARPS) {
        // ---------------- scale warps: stage -> tensor memory, lane quadrant warp % 4 ----------------
        // Atom = 128 rows x 4 scales as 512 bytes: row r's four bytes at (r % 32) * 16 + (r / 32) * 4.  Lane l reads
        // its 16 bytes (the scales of rows l, l + 32, l + 64, l + 96) and writes them to four columns of its own lane:
        // SFA atom j -> columns 4j; SFB atom j of token half h -> columns 16 + 8j + 4h.
        const uint32_t quad_lane = (uint32_t)(32 * (warp & 3)) << 16;
        const uint32_t sf_full_leader = tc::map_to_cta(sf_full, 0);
        uint32_t g = 0;
        bool ok = true;
        for (int t = pair; t < ntiles && ok; t += npairs)
            for (int ks = 0; ks < nks; ks++, g++) {
                const uint32_t s = g % P4_STAGES, b = g % P4_SF_SETS;
                ok = tc::mbar_wait(sf_landed + 8 * s, (g / P4_STAGES) & 1u, abort_flag) &&
                     // set b was last read by the MMAs of k-step g - 3, whose completion also released that k-step's stage
                     (g < P4_SF_SETS || tc::mbar_wait_cluster(empty + 8 * ((g - P4_SF_SETS) % P4_STAGES), ((g - P4_SF_SETS) / P4_STAGES) & 1u, abort_flag));
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    if (lane == 0 && !abort_s) {
                        abort_s = 1;
                        atomicExch(p.status, 28);
                    }
                    break;
                }
                tc::fence_after_sync();
                const uint32_t sfa = smem_s + s * P4_STAGE_BYTES + P4_A_BYTES + P4_B_BYTES + 16u * (uint32_t)lane, sfb = sfa + P4_SFA_BYTES;
                const uint32_t tsfa = tmem + quad_lane + P4_TMEM_SF + P4_SF_SET_COLS * b;
                // the set's 48 columns built in registers, two wide stores (with two atoms per stage the rest is never read)
                uint32_t w[48];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(w[4 * j]), "=r"(w[4 * j + 1]), "=r"(w[4 * j + 2]), "=r"(w[4 * j + 3]) : "r"(sfa + 512u * j));
#pragma unroll
                    for (int h = 0; h < 2; h++)
                        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                                     : "=r"(w[16 + 8 * j + 4 * h]), "=r"(w[17 + 8 * j + 4 * h]), "=r"(w[18 + 8 * j + 4 * h]), "=r"(w[19 + 8 * j + 4 * h])
                                     : "r"(sfb + 2048u * h + 512u * j));
                }
                tc::tmem_st32(tsfa, w);
                tc::tmem_st16(tsfa + 32, w + 32);
                tc::tmem_st_wait();
                tc::fence_before_sync();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive_cluster_relaxed(sf_full_leader + 8 * b);
            }
    }
    __syncwarp();

    if (warp >= 2 && warp < 2 + P4_EPI_WARPS) {
        // ---------------- epilogue: this CTA's 128 rows x 256 tokens; warp w reads TMEM lane quadrant w % 4 ----------------
        const int quad = warp & 3, half = (warp - 2) >> 2;
        uint8_t *stage = smem_raw + (smem_s - tc::smem_u32(smem_raw)) + (size_t)P4_STAGES * P4_STAGE_BYTES + (size_t)(warp - 2) * 4096;
        const uint32_t accum_empty_leader = tc::map_to_cta(accum_empty, 0);
        uint32_t it = 0;
        for (int t = pair; t < ntiles; t += npairs, it++) {
            bool ok = !abort_s && tc::mbar_wait_cluster(accum_full, it & 1u, abort_flag);
            if (!ok && !abort_s) {
                abort_s = 1;
                atomicExch(p.status, 23);
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc::fence_after_sync();
            const int rp = t / tok_tiles, tt = t % tok_tiles;
            const int64_t row0 = (2 * (int64_t)rp + rank) * 128 + 32 * quad, tok0 = (int64_t)tt * 256;
            const uint32_t tbase = tmem + ((uint32_t)(32 * quad) << 16) + (uint32_t)(128 * half);
            if (p.y_bf16) {
                // bf16 output: the warp's 32 rows x 128 tokens fit in registers as packed pairs (64 per thread), so the
                // accumulator is handed back to the MMA thread after four tensor-memory loads and the stores run under the
                // next tile's MMAs (with the stores in front of the hand-over the epilogue was ~23 % of a tile's time)
                uint32_t pk[4][16], v[2][32];
                tc::tmem_ld32(tbase, v[0]);
#pragma unroll
                for (int ci = 0; ci < 4; ci++) {
                    tc::tmem_ld_wait();
                    if (ci < 3) tc::tmem_ld32(tbase + 32 * (ci + 1), v[(ci + 1) & 1]);
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[ci & 1][2 * j]) * p.scale, __uint_as_float(v[ci & 1][2 * j + 1]) * p.scale);
                        pk[ci][j] = *reinterpret_cast<const uint32_t *>(&h);
                    }
                }
                tc::fence_before_sync();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive_cluster_relaxed(accum_empty_leader);  // the loads above have completed (wait::ld)
#pragma unroll
                for (int ci = 0; ci < 4; ci++) {
                    const int64_t tok = tok0 + 128 * half + 32 * ci;
                    if (row0 < p.n && tok < p.m) {
                        float o[32];
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            o[2 * j] = __uint_as_float(pk[ci][j] << 16);
                            o[2 * j + 1] = __uint_as_float(pk[ci][j] & 0xffff0000u);
                        }
                        tc::store_block_32x32<true>(p.y, p.ldy, row0, tok, p.n, p.m, o, stage, lane, p.vec);
                    }
                }
            } else {
                for (int c = 0; c < 128; c += 32) {
                    uint32_t v[32];
                    tc::tmem_ld32(tbase + (uint32_t)c, v);
                    tc::tmem_ld_wait();
                    const int64_t tok = tok0 + 128 * half + c;
                    if (row0 < p.n && tok < p.m) {
                        float o[32];
#pragma unroll
                        for (int j = 0; j < 32; j++) o[j] = __uint_as_float(v[j]) * p.scale;
                        tc::store_block_32x32<false>(p.y, p.ldy, row0, tok, p.n, p.m, o, stage, lane, p.vec);
                    }
                }
                // this warp's reads of the accumulator are complete: the leader may start the next tile
                tc::fence_before_sync();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive_cluster(accum_empty_leader);
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    // neither CTA may leave (or give TMEM back) while the pair's MMAs can still read its shared memory
    tc::cluster_arrive();
    tc::cluster_wait();
    if (warp == 1) tc::tmem_dealloc_pair(tmem, P4_TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// CTA-pair version with TWO accumulators (the default for m > 128): tiles of 256 rows x NT tokens, NT = 192 or 128.
//
// With one 256-column accumulator the epilogue of a tile (tensor memory -> bf16 -> global, ~10 k cycles) cannot
// overlap the next tile's MMAs: measured, it was 40 % of the launch.  Tensor memory has 512 columns: two accumulators of
// 192 columns and three 40-column scale-factor sets fit (2 x 192 + 3 x 40 = 504), so the epilogue warps drain
// accumulator (tile & 1) while the MMA thread fills the other one.  Everything else is the kernel above: own weight
// rows and own half of the activation tile per CTA, scale warps, relay of "stage full" to the leader.
//
// A 192-token tile does not line up with the 128-token groups the activation planes are stored in: a CTA's 96
// activation rows start at a multiple of 32 inside a group and may run into the next one (two bulk copies; the
// 128-byte swizzle only depends on row % 8, which a shift by a multiple of 8 rows keeps), and the scale warps pick the
// tile's 32-token column groups out of the (at most two) groups of scale atoms the tile touches.
// ---------------------------------------------------------------------------------------------
#ifdef GLLMK_FP4_PROF
// Development aid (not built by default): cycles each role of gemm_fp4_pair2_kernel spends in its waits.
__device__ unsigned long long g_fp4_prof[296 * 16];
#define PROF_DECL unsigned long long prof_t = 0, prof_a[4] = {0, 0, 0, 0}, prof_start = clock64()
#define PROF_T0() prof_t = clock64()
#define PROF_ACC(i) prof_a[i] += clock64() - prof_t
#define PROF_OUT(slot, i) g_fp4_prof[blockIdx.x * 16 + (slot)] = prof_a[i]
#define PROF_TOTAL(slot) g_fp4_prof[blockIdx.x * 16 + (slot)] = clock64() - prof_start
// timeline of the first 256 k-steps of CTA 0 (the leader of pair 0): row r, k-step g
__device__ unsigned long long g_fp4_tl[8 * 256];
#define PROF_TL(r, g) do { if (blockIdx.x == 0 && (g) < 256u) g_fp4_tl[(r) * 256 + (g)] = clock64(); } while (0)
#else
#define PROF_TL(r, g)
#define PROF_DECL
#define PROF_T0()
#define PROF_ACC(i)
#define PROF_OUT(slot, i)
#define PROF_TOTAL(slot)
#endif

template <int NT>
struct P2 {
    static constexpr int STAGES = 6;
    static constexpr int A_BYTES = 16384, B_BYTES = NT / 2 * 128, SFA_BYTES = 2048, SFB_BYTES = 4096;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
    static constexpr int EPI_WARPS = 4, SF_WARPS = 4, SF_SETS = 3;
    static constexpr int THREADS = 64 + 32 * (EPI_WARPS + SF_WARPS);
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + (size_t)EPI_WARPS * 4096 + 1024;
    static constexpr uint32_t TMEM_COLS = 512, ACC1 = NT, SF0 = 2 * NT, SFB_PER_MMA = NT / 32, SET_COLS = 16 + NT / 8;
    static_assert(SF0 + SF_SETS * SET_COLS <= TMEM_COLS, "tensor memory budget");
    static constexpr int CHUNKS = NT / 32;  // 32-token column groups of a tile
};

template <int NT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P2<NT>::THREADS, 1)
gemm_fp4_pair2_kernel(const __grid_constant__ Fp4Params p, const int row_tiles, const int tok_tiles) {
    using C = P2<NT>;
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[3 * C::STAGES + C::SF_SETS + 4];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    const uint32_t smem_s = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t full = tc::smem_u32(&bars[0]), empty = tc::smem_u32(&bars[C::STAGES]), full2 = tc::smem_u32(&bars[2 * C::STAGES]);
    const uint32_t sf_full = tc::smem_u32(&bars[3 * C::STAGES]);
    const uint32_t accum_full = sf_full + 8 * C::SF_SETS, accum_empty = accum_full + 16;  // two each
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = tc::cluster_ctarank();
    const int pair = (int)(blockIdx.x >> 1), npairs = (int)(gridDim.x >> 1);
    const int row_pairs = (row_tiles + 1) >> 1;
    const int ntiles = row_pairs * tok_tiles;
    const int nks = (int)(p.k / 256);
    const int64_t atoms_per_row_tile = p.nv ? (p.k >> 6) : (p.k >> 7);
    const int atoms_per_stage = p.nv ? 4 : 2;
    volatile int *abort_flag = &abort_s;

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < C::STAGES; s++) {
            tc::mbar_init(full + 8 * s, 1);
            tc::mbar_init(empty + 8 * s, 1);
            tc::mbar_init(full2 + 8 * s, 1);
        }
        for (int s = 0; s < C::SF_SETS; s++) tc::mbar_init(sf_full + 8 * s, 2 * C::SF_WARPS);  // the scale warps of both CTAs (leader only)
        for (int a = 0; a < 2; a++) {
            tc::mbar_init(accum_full + 8 * a, 1);
            tc::mbar_init(accum_empty + 8 * a, 2 * C::EPI_WARPS);  // the epilogue warps of both CTAs (used in the leader only)
        }
        tc::mbar_init_fence();
    }
    if (warp == 1) tc::tmem_alloc_pair(tc::smem_u32(&tmem_base_s), C::TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::cluster_arrive();
    tc::cluster_wait();
    tc::fence_after_sync();
    const uint32_t tmem = tmem_base_s;

    if (warp == 0 && lane == 0) {
        // ---------------- copies ----------------
        const uint32_t sf_bytes = (uint32_t)atoms_per_stage * 512u;
        const size_t ktiles = (size_t)nks;
        uint32_t g = 0;
        PROF_DECL;
        for (int t = pair; t < ntiles && !*abort_flag; t += npairs) {
            const int rp = t / tok_tiles, tt = t % tok_tiles;
            const int64_t my_row_tile = 2 * (int64_t)rp + rank;
            const bool a_ok = my_row_tile < row_tiles;
            // this CTA's NT / 2 activation rows: tokens [s0, s0 + NT / 2), in 128-token groups g0 (from row r0) and g0 + 1
            const int64_t tok_s = (int64_t)NT * tt, s0 = tok_s + (NT / 2) * (int64_t)rank;
            const int64_t g0 = s0 >> 7;
            const int r0 = (int)(s0 & 127);
            const int n1 = min(NT / 2, 128 - r0), n2 = NT / 2 - n1;
            const bool b1_ok = g0 < p.x_row_tiles, b2_ok = n2 > 0 && g0 + 1 < p.x_row_tiles;
            // the tile's scale atoms: groups G0 and (if the tile reaches into it) G0 + 1
            const int64_t G0 = tok_s >> 7, G1 = (tok_s + NT - 1) >> 7;
            const bool s1_ok = G0 < p.x_row_tiles, s2_ok = G1 != G0 && G1 < p.x_row_tiles;
            const uint32_t tx = (a_ok ? 16384u + sf_bytes : 0u) + (b1_ok ? (uint32_t)n1 * 128u : 0u) + (b2_ok ? (uint32_t)n2 * 128u : 0u) +
                                ((uint32_t)s1_ok + (uint32_t)s2_ok) * sf_bytes;
            for (int ks = 0; ks < nks; ks++, g++) {
                const uint32_t s = g % C::STAGES;
                PROF_T0();
                if (g >= (uint32_t)C::STAGES && !tc::mbar_wait_cluster(empty + 8 * s, (g / C::STAGES - 1) & 1u, abort_flag)) {
                    abort_s = 1;
                    atomicExch(p.status, 24);
                    break;
                }
                PROF_ACC(0);
                PROF_TL(0, g);
                const uint32_t st = smem_s + s * C::STAGE_BYTES, stb = st + C::A_BYTES, stsfa = stb + C::B_BYTES, stsfb = stsfa + C::SFA_BYTES;
                tc::mbar_expect_tx(full + 8 * s, tx);
                if (a_ok) {
                    bulk_load(st, p.qw + ((size_t)my_row_tile * ktiles + ks) * 16384, 16384u, full + 8 * s);
                    bulk_load(stsfa, p.sfw + ((size_t)my_row_tile * atoms_per_row_tile + (size_t)ks * atoms_per_stage) * 512, sf_bytes, full + 8 * s);
                }
                if (b1_ok) bulk_load(stb, p.qx + ((size_t)g0 * ktiles + ks) * 16384 + (size_t)r0 * 128, (uint32_t)n1 * 128u, full + 8 * s);
                if (b2_ok) bulk_load(stb + (uint32_t)n1 * 128u, p.qx + ((size_t)(g0 + 1) * ktiles + ks) * 16384, (uint32_t)n2 * 128u, full + 8 * s);
                if (s1_ok) bulk_load(stsfb, p.sfx + ((size_t)G0 * atoms_per_row_tile + (size_t)ks * atoms_per_stage) * 512, sf_bytes, full + 8 * s);
                if (s2_ok) bulk_load(stsfb + 2048, p.sfx + ((size_t)G1 * atoms_per_row_tile + (size_t)ks * atoms_per_stage) * 512, sf_bytes, full + 8 * s);
            }
        }
        PROF_OUT(0, 0);
        PROF_TOTAL(13);
    } else if (warp == 1 && lane == 0 && rank != 0) {
        // ---------------- partner CTA: tell the leader when this CTA's stage has landed ----------------
        uint32_t g = 0;
        for (int t = pair; t < ntiles && !*abort_flag; t += npairs)
            for (int ks = 0; ks < nks; ks++, g++) {
                const uint32_t s = g % C::STAGES;
                if (!tc::mbar_wait(full + 8 * s, (g / C::STAGES) & 1u, abort_flag)) {
                    abort_s = 1;
                    atomicExch(p.status, 25);
                    t = ntiles;
                    break;
                }
                tc::mbar_arrive_cluster_relaxed(tc::map_to_cta(full2 + 8 * s, 0));
            }
    } else if (warp == 1 && lane == 0) {
        // ---------------- leader CTA: MMA issue for the pair, accumulator (tile & 1) ----------------
        const uint32_t idesc_nv = tc::idesc_fp4(256, NT, 0, 0, 0);
        uint32_t g = 0, it = 0;
        PROF_DECL;
        for (int t = pair; t < ntiles && !*abort_flag; t += npairs, it++) {
            const uint32_t acc = it & 1u;
            PROF_T0();
            // the tile before last used this accumulator: all sixteen epilogue warps of the pair have read it out
            if (it >= 2 && !tc::mbar_wait_cluster(accum_empty + 8 * acc, ((it >> 1) - 1) & 1u, abort_flag)) {
                abort_s = 1;
                atomicExch(p.status, 26);
                break;
            }
            PROF_ACC(3);
            tc::fence_after_sync();
            const uint32_t td = tmem + acc * C::ACC1;
            bool ok = true;
            for (int ks = 0; ks < nks; ks++, g++) {
                const uint32_t s = g % C::STAGES, ph = (g / C::STAGES) & 1u;
                const uint32_t b = g % C::SF_SETS, bph = (g / C::SF_SETS) & 1u;
#ifdef GLLMK_FP4_PROF
                PROF_T0();
                bool w_ok = tc::mbar_wait(full + 8 * s, ph, abort_flag);
                PROF_ACC(0);
                PROF_T0();
                w_ok = w_ok && tc::mbar_wait_cluster(full2 + 8 * s, ph, abort_flag);
                PROF_ACC(1);
                PROF_TL(1, g);
                PROF_T0();
                w_ok = w_ok && tc::mbar_wait_cluster(sf_full + 8 * b, bph, abort_flag);
                PROF_ACC(2);
                PROF_TL(2, g);
                if (!w_ok) {
#else
                if (!tc::mbar_wait(full + 8 * s, ph, abort_flag) || !tc::mbar_wait_cluster(full2 + 8 * s, ph, abort_flag) ||
                    !tc::mbar_wait_cluster(sf_full + 8 * b, bph, abort_flag)) {
#endif
                    abort_s = 1;
                    atomicExch(p.status, 22);
                    ok = false;
                    break;
                }
                tc::fence_after_sync();
                const uint32_t st = smem_s + s * C::STAGE_BYTES;
                const uint64_t ad = tc::smem_desc_sw128(st), bd = tc::smem_desc_sw128(st + C::A_BYTES);
                const uint32_t tsfa = tmem + C::SF0 + C::SET_COLS * b, tsfb = tsfa + 16;
                if (p.nv) {
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        tc::mma_nvf4_pair(td, ad + 2 * j, bd + 2 * j, idesc_nv, (uint32_t)((ks | j) != 0), tsfa + 4 * j, tsfb + C::SFB_PER_MMA * j);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const int id = (j & 1) * 2;
                        tc::mma_mxf4_pair(td, ad + 2 * j, bd + 2 * j, tc::idesc_fp4(256, NT, 1, id, id), (uint32_t)((ks | j) != 0),
                                          tsfa + 4 * (j >> 1), tsfb + C::SFB_PER_MMA * (j >> 1));
                    }
                }
                tc::mma_commit_pair(empty + 8 * s);
                tc::mma_commit_pair(tc::map_to_cta(empty + 8 * s, 1));
                PROF_TL(3, g);
            }
            if (!ok) break;
            tc::mma_commit_pair(accum_full + 8 * acc);
            tc::mma_commit_pair(tc::map_to_cta(accum_full + 8 * acc, 1));
        }
        PROF_OUT(1, 0);
        PROF_OUT(2, 1);
        PROF_OUT(3, 2);
        PROF_OUT(4, 3);
        PROF_TOTAL(5);
    } else if (warp >= 2 + C::EPI_WARPS) {
        // ---------------- scale warps: stage -> tensor memory, lane quadrant warp % 4 ----------------
        // An atom holds 128 rows x 4 scales: row r's four bytes at (r % 32) * 16 + (r / 32) * 4.  SFA atom j -> columns 4j.. of
        // the set; SFB: the tile's 32-token group c is word (gt % 4) of 128-token group (gt / 4), gt = first token / 32 + c,
        // and goes to column 16 + (NT / 32) * j + c.
        const uint32_t quad_lane = (uint32_t)(32 * (warp & 3)) << 16;
        const uint32_t sf_full_leader = tc::map_to_cta(sf_full, 0);
        uint32_t g = 0;
        bool ok = true;
        PROF_DECL;
        for (int t = pair; t < ntiles && ok; t += npairs) {
            const bool tile_odd = NT == 192 && ((t % tok_tiles) & 1);
            for (int ks = 0; ks < nks; ks++, g++) {
                const uint32_t s = g % C::STAGES, b = g % C::SF_SETS;
                PROF_T0();
                ok = tc::mbar_wait(full + 8 * s, (g / C::STAGES) & 1u, abort_flag);
                PROF_ACC(0);
                PROF_T0();
                // set b was last read by the MMAs of k-step g - 3, whose completion also released that k-step's stage
                ok = ok && (g < (uint32_t)C::SF_SETS ||
                            tc::mbar_wait_cluster(empty + 8 * ((g - C::SF_SETS) % C::STAGES), ((g - C::SF_SETS) / C::STAGES) & 1u, abort_flag));
                PROF_ACC(1);
                ok = __all_sync(0xffffffffu, ok);
                PROF_T0();
                if (warp == 2 + C::EPI_WARPS && lane == 0) PROF_TL(4, g);
                if (!ok) {
                    if (lane == 0 && !abort_s) {
                        abort_s = 1;
                        atomicExch(p.status, 28);
                    }
                    break;
                }
                tc::fence_after_sync();
                const uint32_t sfa = smem_s + s * C::STAGE_BYTES + C::A_BYTES + C::B_BYTES + 16u * (uint32_t)lane, sfb = sfa + C::SFA_BYTES;
                const uint32_t tsfa = tmem + quad_lane + C::SF0 + C::SET_COLS * b;
                // the whole set is built in registers and stored with one (NT = 128) or two (192) wide tcgen05.st: per-atom
                // stores made this role the slowest of the kernel (1500 cycles per k-step, the MMA thread waiting on it half
                // of the time).  With two atoms per stage (MXFP4) the upper columns carry stale bytes nobody reads.
                uint32_t w[C::SET_COLS];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(w[4 * j]), "=r"(w[4 * j + 1]), "=r"(w[4 * j + 2]), "=r"(w[4 * j + 3]) : "r"(sfa + 512u * j));
                    if (NT == 128) {
                        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                                     : "=r"(w[16 + 4 * j]), "=r"(w[17 + 4 * j]), "=r"(w[18 + 4 * j]), "=r"(w[19 + 4 * j]) : "r"(sfb + 512u * j));
                    } else if (tile_odd) {  // the tile starts at token 64 of group G0: words 2, 3 of G0, then words 0..3 of G0 + 1
                        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(w[16 + 6 * j]), "=r"(w[17 + 6 * j]) : "r"(sfb + 512u * j + 8u));
                        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                                     : "=r"(w[18 + 6 * j]), "=r"(w[19 + 6 * j]), "=r"(w[20 + 6 * j]), "=r"(w[21 + 6 * j]) : "r"(sfb + 2048u + 512u * j));
                    } else {  // the tile starts at token 0 of group G0: words 0..3 of G0, then words 0, 1 of G0 + 1
                        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                                     : "=r"(w[16 + 6 * j]), "=r"(w[17 + 6 * j]), "=r"(w[18 + 6 * j]), "=r"(w[19 + 6 * j]) : "r"(sfb + 512u * j));
                        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(w[20 + 6 * j]), "=r"(w[21 + 6 * j]) : "r"(sfb + 2048u + 512u * j));
                    }
                }
#ifdef GLLMK_FP4_PROF
                {
                    uint32_t dep;
                    asm volatile("add.u32 %0, %1, %2;\n" : "=r"(dep) : "r"(w[C::SET_COLS - 1]), "r"(w[0]));
                    if (warp == 2 + C::EPI_WARPS && lane == 0) PROF_TL(5, g);
                }
#endif
                tc::tmem_st32(tsfa, w);
                if (NT == 192) tc::tmem_st8(tsfa + 32, w + 32);
                tc::tmem_st_wait();
                if (warp == 2 + C::EPI_WARPS && lane == 0) PROF_TL(6, g);
                tc::fence_before_sync();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive_cluster_relaxed(sf_full_leader + 8 * b);
                PROF_ACC(2);
                if (warp == 2 + C::EPI_WARPS && lane == 0) PROF_TL(7, g);
            }
        }
        if (warp == 2 + C::EPI_WARPS && lane == 0) {
            PROF_OUT(6, 0);
            PROF_OUT(7, 1);
            PROF_OUT(8, 2);
            PROF_TOTAL(9);
        }
    }
    __syncwarp();

    if (warp >= 2 && warp < 2 + C::EPI_WARPS) {
        // ---------------- epilogue: this CTA's 128 rows x NT tokens of accumulator (tile & 1) ----------------
        // warp w reads TMEM lane quadrant w % 4 and walks the tile's 32-token column groups with one tensor-memory load in
        // flight under the stores of the group before (the whole epilogue runs under the next tile's MMAs)
        const int quad = warp & 3;
        uint8_t *stage = smem_raw + (smem_s - tc::smem_u32(smem_raw)) + (size_t)C::STAGES * C::STAGE_BYTES + (size_t)(warp - 2) * 4096;
        const uint32_t accum_empty_leader = tc::map_to_cta(accum_empty, 0);
        uint32_t it = 0;
        PROF_DECL;
        for (int t = pair; t < ntiles; t += npairs, it++) {
            const uint32_t acc = it & 1u;
            PROF_T0();
            bool ok = !abort_s && tc::mbar_wait_cluster(accum_full + 8 * acc, (it >> 1) & 1u, abort_flag);
            PROF_ACC(0);
            if (!ok && !abort_s) {
                abort_s = 1;
                atomicExch(p.status, 23);
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            PROF_T0();
            tc::fence_after_sync();
            const int rp = t / tok_tiles, tt = t % tok_tiles;
            const int64_t row0 = (2 * (int64_t)rp + rank) * 128 + 32 * quad, tok0 = (int64_t)NT * tt;
            const uint32_t tbase = tmem + ((uint32_t)(32 * quad) << 16) + acc * C::ACC1;
            const auto emit = [&](const uint32_t (&v)[32], int ci) {
                const int64_t tok = tok0 + 32 * ci;
                if (row0 < p.n && tok < p.m) {
                    float o[32];
#pragma unroll
                    for (int j = 0; j < 32; j++) o[j] = __uint_as_float(v[j]) * p.scale;
                    if (p.y_bf16) tc::store_block_32x32<true>(p.y, p.ldy, row0, tok, p.n, p.m, o, stage, lane, p.vec);
                    else tc::store_block_32x32<false>(p.y, p.ldy, row0, tok, p.n, p.m, o, stage, lane, p.vec);
                }
            };
            uint32_t va[32], vb[32];
            tc::tmem_ld32(tbase, va);
#pragma unroll
            for (int ci = 0; ci < C::CHUNKS; ci += 2) {
                tc::tmem_ld_wait();
                tc::tmem_ld32(tbase + 32 * (ci + 1), vb);
                emit(va, ci);
                tc::tmem_ld_wait();
                if (ci + 2 < C::CHUNKS) tc::tmem_ld32(tbase + 32 * (ci + 2), va);
                emit(vb, ci + 1);
            }
            // this warp's reads of the accumulator are complete: the leader may reuse it for the tile after next
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive_cluster(accum_empty_leader + 8 * acc);
            PROF_ACC(1);
        }
        if (warp == 2 && lane == 0) {
            PROF_OUT(10, 0);
            PROF_OUT(11, 1);
            PROF_TOTAL(12);
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    tc::cluster_arrive();
    tc::cluster_wait();
    if (warp == 1) tc::tmem_dealloc_pair(tmem, C::TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// Ceiling probe: the block-scaled FP4 MMA of the kernels above issued back to back on operands that never leave
// shared memory (no copies from L2, no epilogue), one CTA (or CTA pair) per SM, k-steps of four MMAs committed to a
// ring of four barriers like the real pipelines.  What this reaches is the most the GEMM kernels can: it is the
// denominator bench.py reports beside the nominal 9 PFLOP/s.
// ---------------------------------------------------------------------------------------------
// sf_mode: 0 = no scale-factor traffic, 1 = twelve (six for MXFP4) tcgen05.cp per k-step issued by the MMA thread,
// 2 = the scale factors written by four scale warps with tcgen05.st into three column sets in rotation, as in
// gemm_fp4_pair_kernel.
template <bool PAIR>
__device__ __forceinline__ void probe_body(int nv, int sf_mode, int ksteps, int *status) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t bars[4 + 6];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    const uint32_t smem_s = (tc::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (smem_s - tc::smem_u32(smem_raw));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar0 = tc::smem_u32(&bars[0]), sf_full = tc::smem_u32(&bars[4]), sf_empty = tc::smem_u32(&bars[7]);
    const uint32_t rank = PAIR ? tc::cluster_ctarank() : 0u;
    constexpr int A = 16384, B = PAIR ? 16384 : 32768, SFA = 2048, SFB = 4096;
    // operands: every E2M1 code, scale bytes 0x38 (UE4M3 1.0; as UE8M0 2^-71: still finite)
    for (int i = threadIdx.x; i < (A + B) / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(smem)[i] = 0x76543210u * (uint32_t)(i | 1);
    for (int i = threadIdx.x; i < (SFA + SFB) / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(smem + A + B)[i] = 0x38383838u;
    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < 4; s++) tc::mbar_init(bar0 + 8 * s, 1);
        for (int s = 0; s < 3; s++) {
            tc::mbar_init(sf_full + 8 * s, PAIR ? 8 : 4);
            tc::mbar_init(sf_empty + 8 * s, 1);
        }
        tc::mbar_init_fence();
    }
    tc::fence_proxy_async();
    if (warp == 1) {
        if (PAIR) tc::tmem_alloc_pair(tc::smem_u32(&tmem_base_s), 512);
        else tc::tmem_alloc(tc::smem_u32(&tmem_base_s), 512);
    }
    tc::fence_before_sync();
    __syncthreads();
    if (PAIR) { tc::cluster_arrive(); tc::cluster_wait(); }
    tc::fence_after_sync();
    const uint32_t tmem = tmem_base_s;
    volatile int *abort_flag = &abort_s;
    const int atoms = nv ? 4 : 2;
    const uint32_t sfa = smem_s + A + B, sfb = sfa + SFA;
    if (threadIdx.x == 32 && rank == 0) {
        const uint64_t ad = tc::smem_desc_sw128(smem_s), bd = tc::smem_desc_sw128(smem_s + A);
        const uint32_t idesc_nv = tc::idesc_fp4(PAIR ? 256 : 128, 256, 0, 0, 0);
        for (int ks = 0; ks < ksteps; ks++) {
            const int s = ks & 3;
            const uint32_t b = sf_mode == 2 ? (uint32_t)(ks % 3) : 0u;
            if ((ks >= 4 && !tc::mbar_wait(bar0 + 8 * s, (uint32_t)((ks / 4 - 1) & 1), abort_flag)) ||
                (sf_mode == 2 && !tc::mbar_wait_cluster(sf_full + 8 * b, (uint32_t)((ks / 3) & 1), abort_flag))) {
                abort_s = 1;
                atomicExch(status, 27);
                break;
            }
            tc::fence_after_sync();
            const uint32_t tsfa = tmem + 256 + 48 * b, tsfb = tsfa + 16;
            if (sf_mode == 1)
                for (int j = 0; j < atoms; j++) {
                    if (PAIR) {
                        tc::tmem_cp_sf_pair(tsfa + 4 * j, sf_desc(sfa + 512 * j));
                        tc::tmem_cp_sf_pair(tsfb + 8 * j, sf_desc(sfb + 512 * j));
                        tc::tmem_cp_sf_pair(tsfb + 8 * j + 4, sf_desc(sfb + 2048 + 512 * j));
                    } else {
                        tc::tmem_cp_sf(tsfa + 4 * j, sf_desc(sfa + 512 * j));
                        tc::tmem_cp_sf(tsfb + 8 * j, sf_desc(sfb + 512 * j));
                        tc::tmem_cp_sf(tsfb + 8 * j + 4, sf_desc(sfb + 2048 + 512 * j));
                    }
                }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if (nv) {
                    if (PAIR) tc::mma_nvf4_pair(tmem, ad + 2 * j, bd + 2 * j, idesc_nv, (uint32_t)((ks | j) != 0), tsfa + 4 * j, tsfb + 8 * j);
                    else tc::mma_nvf4(tmem, ad + 2 * j, bd + 2 * j, idesc_nv, (uint32_t)((ks | j) != 0), tsfa + 4 * j, tsfb + 8 * j);
                } else {
                    const int id = (j & 1) * 2;
                    const uint32_t idm = tc::idesc_fp4(PAIR ? 256 : 128, 256, 1, id, id);
                    if (PAIR) tc::mma_mxf4_pair(tmem, ad + 2 * j, bd + 2 * j, idm, (uint32_t)((ks | j) != 0), tsfa + 4 * (j >> 1), tsfb + 8 * (j >> 1));
                    else tc::mma_mxf4(tmem, ad + 2 * j, bd + 2 * j, idm, (uint32_t)((ks | j) != 0), tsfa + 4 * (j >> 1), tsfb + 8 * (j >> 1));
                }
            }
            if (PAIR) {
                tc::mma_commit_pair(bar0 + 8 * s);
                if (sf_mode == 2) {
                    tc::mma_commit_pair(sf_empty + 8 * b);
                    tc::mma_commit_pair(tc::map_to_cta(sf_empty + 8 * b, 1));
                }
            } else {
                tc::mma_commit(bar0 + 8 * s);
                if (sf_mode == 2) tc::mma_commit(sf_empty + 8 * b);
            }
        }
        // drain: the last commits
        for (int ks = max(ksteps - 4, 0); ks < ksteps && !abort_s; ks++)
            if (!tc::mbar_wait(bar0 + 8 * (ks & 3), (uint32_t)((ks / 4) & 1), abort_flag)) {
                abort_s = 1;
                atomicExch(status, 27);
            }
    } else if (warp >= 2 && sf_mode == 2) {
        const uint32_t quad_lane = (uint32_t)(32 * (warp & 3)) << 16;
        const uint32_t sf_full_leader = PAIR ? tc::map_to_cta(sf_full, 0) : sf_full;
        for (int ks = 0; ks < ksteps; ks++) {
            const uint32_t b = (uint32_t)(ks % 3);
            bool ok = ks < 3 || tc::mbar_wait_cluster(sf_empty + 8 * b, (uint32_t)((ks / 3 - 1) & 1), abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) atomicExch(status, 27);
                break;
            }
            tc::fence_after_sync();
            const uint32_t tsfa = tmem + quad_lane + 256 + 48 * b;
            uint32_t w[48];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(w[4 * j]), "=r"(w[4 * j + 1]), "=r"(w[4 * j + 2]), "=r"(w[4 * j + 3]) : "r"(sfa + 16u * lane + 512u * j));
#pragma unroll
                for (int h = 0; h < 2; h++)
                    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                                 : "=r"(w[16 + 8 * j + 4 * h]), "=r"(w[17 + 8 * j + 4 * h]), "=r"(w[18 + 8 * j + 4 * h]), "=r"(w[19 + 8 * j + 4 * h])
                                 : "r"(sfb + 16u * lane + 2048u * h + 512u * j));
            }
            tc::tmem_st32(tsfa, w);
            tc::tmem_st16(tsfa + 32, w + 32);
            tc::tmem_st_wait();
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (PAIR) tc::mbar_arrive_cluster_relaxed(sf_full_leader + 8 * b);
                else tc::mbar_arrive(sf_full + 8 * b);
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (PAIR) { tc::cluster_arrive(); tc::cluster_wait(); }
    if (warp == 1) {
        if (PAIR) tc::tmem_dealloc_pair(tmem, 512);
        else tc::tmem_dealloc(tmem, 512);
    }
}
__global__ void __launch_bounds__(192, 1) probe_fp4_single_kernel(int nv, int sf_mode, int ksteps, int *status) { probe_body<false>(nv, sf_mode, ksteps, status); }
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1) probe_fp4_pair_kernel(int nv, int sf_mode, int ksteps, int *status) {
    probe_body<true>(nv, sf_mode, ksteps, status);
}

int32_t probe_fp4_mma(Ctx *c, int pair, int with_cp, int nv, int ksteps, float *tflops) {
    const size_t smem = 16384 + 32768 + 2048 + 4096 + 1024;
    // more shared memory than half an SM has: one CTA per SM, as in the GEMM kernels
    const size_t smem_req = smem < 120 * 1024 ? 120 * 1024 : smem;
    if (pair) GK_CUDA(c, cudaFuncSetAttribute(probe_fp4_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_req));
    else GK_CUDA(c, cudaFuncSetAttribute(probe_fp4_single_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_req));
    const unsigned grid = (unsigned)c->sm_count & ~1u;
    cudaEvent_t e0, e1;
    GK_CUDA(c, cudaEventCreate(&e0));
    GK_CUDA(c, cudaEventCreate(&e1));
    float best = 0.f;
    for (int rep = 0; rep < 4; rep++) {
        cudaEventRecord(e0, c->stream);
        if (pair) probe_fp4_pair_kernel<<<grid, 192, smem_req, c->stream>>>(nv, with_cp, ksteps, c->status_dev);
        else probe_fp4_single_kernel<<<grid, 192, smem_req, c->stream>>>(nv, with_cp, ksteps, c->status_dev);
        cudaEventRecord(e1, c->stream);
        cudaError_t e = cudaStreamSynchronize(c->stream);
        if (e == cudaSuccess) e = cudaGetLastError();
        if (e != cudaSuccess) {
            cudaEventDestroy(e0);
            cudaEventDestroy(e1);
            return cuda_fail(c, e, "probe_fp4_mma");
        }
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        // per k-step and CTA: four MMAs of 128 x 256 x 64 (a pair: 256 x 256 x 64 over two CTAs = the same per CTA)
        const double flops = (double)grid * ksteps * 4.0 * 2.0 * 128.0 * 256.0 * 64.0;
        const float tf = (float)(flops / (ms * 1e-3) / 1e12);
        if (rep > 0 && tf > best) best = tf;  // the first launch warms up
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *tflops = best;
    return GLLMK_STATUS_OK;
}

// ---------------------------------------------------------------------------------------------
// w: weights [n, k]; x: activations [m, k] in the same FP4 format, uploaded like a weight.
int32_t gemm_fp4_launch(Ctx *c, const Weight *w, const Weight *x, void *y, int y_bf16, int64_t ldy, cudaStream_t s) {
    if (w->qt != x->qt || (w->qt != GLLMK_QUANT_NVFP4 && w->qt != GLLMK_QUANT_MXFP4))
        return fail(c, GLLMK_STATUS_UNSUPPORTED, "gemm_fp4: both operands must be NVFP4 or both MXFP4");
    if (w->k != x->k) return fail(c, GLLMK_STATUS_INVALID_ARG, "gemm_fp4: k of the two operands must match");
    static bool attr_set[64] = {};  // function attributes are per device
    const int dev_slot = c->device & 63;
    if (!attr_set[dev_slot]) {
        GK_CUDA(c, cudaFuncSetAttribute(gemm_fp4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)F4_SMEM));
        attr_set[dev_slot] = true;
    }
    const int m = (int)x->n;
    const int ntok = (m > 128) ? 256 : 128;
    Fp4Params p{};
    p.qw = static_cast<const uint8_t *>(w->qs);
    p.qx = static_cast<const uint8_t *>(x->qs);
    p.sfw = static_cast<const uint8_t *>(w->aux);
    p.sfx = static_cast<const uint8_t *>(x->aux);
    p.nv = w->qt == GLLMK_QUANT_NVFP4;
    p.n = w->n;
    p.k = w->k_pad;
    p.m = m;
    p.x_row_tiles = x->n_pad / 128;
    p.scale = w->global_scale * x->global_scale;
    p.y = y;
    p.y_bf16 = y_bf16;
    p.ldy = ldy;
    p.vec = (((uintptr_t)y & 15) == 0 && (ldy * (y_bf16 ? 2 : 4)) % 16 == 0) ? 1 : 0;
    p.status = c->status_dev;
    if (m > 128 && c->gemm_fp4_pair) {
        // 1 (default): one 256-token accumulator; 2: two 192-token accumulators; 3: two 128-token accumulators
        const int variant = (c->gemm_fp4_pair == 2 || c->gemm_fp4_pair == 3) ? (int)c->gemm_fp4_pair : 1;
        const int tile_tok = variant == 3 ? 128 : (variant == 2 ? 192 : 256);
        const size_t smem_bytes = variant == 1 ? P4_SMEM : (variant == 3 ? P2<128>::SMEM : P2<192>::SMEM);
        const int threads = variant == 1 ? P4_THREADS : P2<192>::THREADS;
        const void *fn = variant == 1 ? (const void *)gemm_fp4_pair_kernel
                                      : (variant == 3 ? (const void *)gemm_fp4_pair2_kernel<128> : (const void *)gemm_fp4_pair2_kernel<192>);
        static int pairs_resident[64][4] = {};  // per device and variant: CTA pairs resident at once (0 = not yet asked)
        if (!pairs_resident[dev_slot][variant & 3]) {
            GK_CUDA(c, cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)c->sm_count & ~1u);
            cfg.blockDim = dim3((unsigned)threads);
            cfg.dynamicSmemBytes = smem_bytes;
            int nclusters = 0;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = 2;
            at[0].val.clusterDim.y = 1;
            at[0].val.clusterDim.z = 1;
            cfg.attrs = at;
            cfg.numAttrs = 1;
            if (cudaOccupancyMaxActiveClusters(&nclusters, fn, &cfg) != cudaSuccess || nclusters < 1) {
                (void)cudaGetLastError();
                nclusters = c->sm_count / 2;
            }
            pairs_resident[dev_slot][variant & 3] = nclusters < c->sm_count / 2 ? nclusters : c->sm_count / 2;
        }
        const int row_tiles = (int)(w->n_pad / 128), tok_tiles = (m + tile_tok - 1) / tile_tok;
        const int ntiles = ((row_tiles + 1) / 2) * tok_tiles;
        const int resident = pairs_resident[dev_slot][variant & 3];
        const int npairs = ntiles < resident ? ntiles : resident;
        if (variant == 1) gemm_fp4_pair_kernel<<<dim3(2u * (unsigned)npairs), P4_THREADS, P4_SMEM, s>>>(p, row_tiles, tok_tiles);
        else if (variant == 3) gemm_fp4_pair2_kernel<128><<<dim3(2u * (unsigned)npairs), P2<128>::THREADS, P2<128>::SMEM, s>>>(p, row_tiles, tok_tiles);
        else gemm_fp4_pair2_kernel<192><<<dim3(2u * (unsigned)npairs), P2<192>::THREADS, P2<192>::SMEM, s>>>(p, row_tiles, tok_tiles);
        GK_CUDA(c, cudaGetLastError());
        return GLLMK_STATUS_OK;
    }
    dim3 grid((unsigned)(w->n_pad / F4_BM), (unsigned)((m + F4_BN - 1) / F4_BN));
    gemm_fp4_kernel<<<grid, F4_THREADS, F4_SMEM, s>>>(p, ntok);
    GK_CUDA(c, cudaGetLastError());
    return GLLMK_STATUS_OK;
}

}  // namespace gllmk

#ifdef GLLMK_FP4_PROF
extern "C" __attribute__((visibility("default"))) int gllmk_debug_fp4_prof(unsigned long long *out) {
    return (int)cudaMemcpyFromSymbol(out, gllmk::g_fp4_prof, sizeof(gllmk::g_fp4_prof));
}
extern "C" __attribute__((visibility("default"))) int gllmk_debug_fp4_timeline(unsigned long long *out) {
    return (int)cudaMemcpyFromSymbol(out, gllmk::g_fp4_tl, sizeof(gllmk::g_fp4_tl));
}
#endif
