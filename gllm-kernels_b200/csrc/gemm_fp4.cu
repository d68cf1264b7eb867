// Prefill GEMM with both operands in FP4: native block-scaled tcgen05 MMA.
//
//   Y[t, r] = gW * gX * sum_k W4[r, k] * X4[t, k]      (NVFP4: E2M1 values, UE4M3 scale per 16 elements)
//             (MXFP4: E2M1 values, UE8M0 scale per 32 elements, gW = gX = 1)
//
// Both operands are resident in the FP4 plane layout of common.cuh (packed nibbles [rows][k/2] + scale
// bytes in 128-row x 4-scale atoms).  Per k-step of 256 elements (= one 128-byte swizzled row) a CTA
// brings in, with TMA tile loads and bulk copies (no multicast):
//   A = 128 weight rows x 128 B, B = up to 256 activation rows x 128 B, and their scale atoms;
// one thread copies the scale atoms to tensor memory (tcgen05.cp) and issues four
// tcgen05.mma.kind::mxf4nvf4.block_scale (K = 64 each; kind::mxf4 for MXFP4) into a 128 x 256 f32
// accumulator in TMEM; four warps read it back, apply the two per-tensor scales and store Y.
#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "tc05.cuh"

namespace gllmk {

constexpr int F4_BM = 128, F4_BN = 256;
constexpr int F4_BK_BYTES = 128;            // 256 FP4 elements per stage
constexpr int F4_STAGES = 4;
constexpr int F4_A_BYTES = F4_BM * 128, F4_B_BYTES = F4_BN * 128;
constexpr int F4_SFA_BYTES = 2048;          // 4 atoms (128 rows x 16 scales of 16 el; MXFP4 uses 2 of them)
constexpr int F4_SFB_BYTES = 4096;
constexpr int F4_STAGE_BYTES = F4_A_BYTES + F4_B_BYTES + F4_SFA_BYTES + F4_SFB_BYTES;
constexpr int F4_THREADS = 192;             // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: epilogue
constexpr size_t F4_SMEM = (size_t)F4_STAGES * F4_STAGE_BYTES + 1024;
constexpr uint32_t F4_TMEM_COLS = 512;      // 256 accumulator + 2 x (16 SFA + 32 SFB), power of two
constexpr uint32_t F4_TMEM_SF = 256;        // scale-factor columns, two sets of 48 used by alternate k-steps

struct Fp4Params {
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
    int *status;
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *tmap, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
                 "l"(tmap), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}
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
gemm_fp4_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                const __grid_constant__ Fp4Params p, const int ntok) {
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
        // 128-row groups of the activation tile that exist in the scale plane (the data rows beyond it are
        // zero-filled by TMA; their stale scales only reach output columns that are never stored)
        const int btiles = min((ntok + 127) / 128, (int)(p.x_row_tiles - (tok0 >> 7)));
        const uint32_t tx = F4_A_BYTES + (uint32_t)ntok * 128u + sf_bytes * (1u + (uint32_t)btiles);
        for (int ks = 0; ks < nks; ks++) {
            const int s = ks % F4_STAGES;
            if (ks >= F4_STAGES && !tc::mbar_wait(empty + 8 * s, (uint32_t)((ks / F4_STAGES - 1) & 1), abort_flag)) {
                abort_s = 1;
                atomicExch(p.status, 21);
                break;
            }
            const uint32_t st = smem_s + s * F4_STAGE_BYTES;
            tc::mbar_expect_tx(full + 8 * s, tx);
            tma_load_2d(st, &tmap_w, ks * 128, (int)row0, full + 8 * s);
            // the activation tensor map has a box of `ntok` rows (128 or 256): one load
            tma_load_2d(st + F4_A_BYTES, &tmap_x, ks * 128, (int)tok0, full + 8 * s);
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
            const int64_t row = row0 + 32 * quad + lane;
            for (int c = 0; c < ntok; c += 32) {
                uint32_t v[32];
                tc::tmem_ld32(tmem + ((uint32_t)(32 * quad) << 16) + (uint32_t)c, v);
                tc::tmem_ld_wait();
                if (row < p.n) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int64_t tok = tok0 + c + j;
                        if (tok < p.m) {
                            const float o = __uint_as_float(v[j]) * p.scale;
                            if (p.y_bf16) static_cast<__nv_bfloat16 *>(p.y)[tok * p.ldy + row] = __float2bfloat16_rn(o);
                            else static_cast<float *>(p.y)[tok * p.ldy + row] = o;
                        }
                    }
                }
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 1) tc::tmem_dealloc(tmem, F4_TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Tensor map over an FP4 data plane [rows][k/2] bytes: boxes of 128 bytes x box_rows rows, 128-byte swizzle.
static int32_t make_plane_tmap(Ctx *c, const Weight *w, int box_rows, CUtensorMap *out) {
    static EncodeTiledFn encode = nullptr;
    if (!encode) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        GK_CUDA(c, cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
        if (!fn || q != cudaDriverEntryPointSuccess) return fail(c, GLLMK_STATUS_RUNTIME_ERROR, "cuTensorMapEncodeTiled not available");
        encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    const cuuint64_t dims[2] = {(cuuint64_t)(w->k / 2), (cuuint64_t)w->n_pad};
    const cuuint64_t strides[1] = {(cuuint64_t)(w->k / 2)};
    const cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w->qs, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(c, GLLMK_STATUS_RUNTIME_ERROR, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    return GLLMK_STATUS_OK;
}

// w: weights [n, k]; x: activations [m, k] in the same FP4 format, uploaded like a weight.
int32_t gemm_fp4_launch(Ctx *c, const Weight *w, const Weight *x, void *y, int y_bf16, int64_t ldy, cudaStream_t s) {
    if (w->qt != x->qt || (w->qt != GLLMK_QUANT_NVFP4 && w->qt != GLLMK_QUANT_MXFP4))
        return fail(c, GLLMK_STATUS_UNSUPPORTED, "gemm_fp4: both operands must be NVFP4 or both MXFP4");
    if (w->k != x->k || (w->k % 256)) return fail(c, GLLMK_STATUS_INVALID_ARG, "gemm_fp4: k must match and be a multiple of 256");
    static bool attr_set = false;
    if (!attr_set) {
        GK_CUDA(c, cudaFuncSetAttribute(gemm_fp4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)F4_SMEM));
        attr_set = true;
    }
    const int m = (int)x->n;
    const int ntok = (m > 128) ? 256 : 128;
    CUtensorMap tw, tx;
    int32_t rc = make_plane_tmap(c, w, F4_BM, &tw);
    if (!rc) rc = make_plane_tmap(c, x, ntok, &tx);
    if (rc) return rc;
    Fp4Params p{};
    p.sfw = static_cast<const uint8_t *>(w->aux);
    p.sfx = static_cast<const uint8_t *>(x->aux);
    p.nv = w->qt == GLLMK_QUANT_NVFP4;
    p.n = w->n;
    p.k = w->k;
    p.m = m;
    p.x_row_tiles = x->n_pad / 128;
    p.scale = w->global_scale * x->global_scale;
    p.y = y;
    p.y_bf16 = y_bf16;
    p.ldy = ldy;
    p.status = c->status_dev;
    dim3 grid((unsigned)(w->n_pad / F4_BM), (unsigned)((m + F4_BN - 1) / F4_BN));
    gemm_fp4_kernel<<<grid, F4_THREADS, F4_SMEM, s>>>(tw, tx, p, ntok);
    GK_CUDA(c, cudaGetLastError());
    return GLLMK_STATUS_OK;
}

}  // namespace gllmk
