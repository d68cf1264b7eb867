// tcgen05 / TMEM / mbarrier building blocks for the prefill GEMM kernels (sm_100a inline PTX).
// Every wait is bounded: a wait that runs out returns false and the caller leaves through the
// kernel's common exit (which still releases TMEM).
#pragma once
#include <cuda_bf16.h>

#include <cstdint>

namespace gllmk {
namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier ----
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
// One try: the thread may be suspended by the hardware for up to `hint_ns` while the phase is pending.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity, uint32_t hint_ns = 2000u) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
// Bounded wait; also gives up early when another role of the CTA has raised `*abort_flag`.  The first tries
// are back to back (the common case: the phase completes within a few hundred cycles); after that the flag
// is looked at between tries.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
#pragma unroll 1
    for (uint32_t it = 0; it < (1u << 21); it++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (it >= 64u && *abort_flag) return false;
    }
    return false;
}

// The same with back-to-back probes that do not suspend the thread: for a role whose warp has nothing else to do and
// whose reaction time is on the critical path.
__device__ __forceinline__ bool mbar_spin(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
#pragma unroll 1
    for (uint32_t it = 0; it < (1u << 22); it++) {
        uint32_t ok;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
        if ((it & 255u) == 255u && *abort_flag) return false;
    }
    return false;
}

// named barrier among `nthreads` threads of the CTA (ids 1..15; 0 is __syncthreads)
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) { asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(nthreads) : "memory"); }

// generic-proxy writes to shared memory -> visible to the async proxy (tensor core / bulk copies)
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// ---- TMEM ----
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {  // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(dst_smem), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// 32 lanes x 32 columns of 32-bit: thread i of the warp gets lane (base_lane + i), columns c..c+31
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// 32 lanes x 4 columns of 32-bit from registers: thread i of the warp writes lane (base_lane + i), columns c..c+3
__device__ __forceinline__ void tmem_st4(uint32_t taddr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(taddr), "r"(r0), "r"(r1), "r"(r2), "r"(r3) : "memory");
}
__device__ __forceinline__ void tmem_st2(uint32_t taddr, uint32_t r0, uint32_t r1) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x2.b32 [%0], {%1, %2};\n" ::"r"(taddr), "r"(r0), "r"(r1) : "memory");
}
// wide forms: a tcgen05.st costs about the same whatever its width (~90 cycles measured beside running MMAs), so a role
// that fills many columns builds them in registers and stores once.  r[] indices must be compile-time after unrolling.
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t *r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};\n" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t *r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t *r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

// ---- UMMA descriptors ----
// K-major operand tile in shared memory, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes
// apart, tile base 1024-byte aligned.  Fields: start >> 4 [0,14) | LBO >> 4 [16,30) (unused with a
// swizzle, 1) | SBO >> 4 [32,46) = 64 | version 1 at [46,48) | layout type [61,64) = 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)1 << 16) | ((uint64_t)64 << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// Byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside such a tile.
__device__ __forceinline__ uint32_t sw128_offset(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

// Instruction descriptor, kind::f16, 16-bit operands (format 0 = f16, 1 = bf16) -> f32, both K-major.
__host__ __device__ constexpr uint32_t idesc_f16(int M, int N, int a_fmt, int b_fmt) {
    return (1u << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// kind::i8: 8-bit integer operands (format 0 = unsigned, 1 = signed) -> s32 (accumulator format 2), both K-major.
__host__ __device__ constexpr uint32_t idesc_i8(int M, int N, int a_signed, int b_signed) {
    return (2u << 4) | ((uint32_t)a_signed << 7) | ((uint32_t)b_signed << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// Block-scaled kinds (mxf4 / mxf4nvf4): E2M1 operands (format 1), scale format bit 23 (0 = UE4M3, 1 = UE8M0),
// scale-factor ids at [4,6) (B) and [29,31) (A).
__host__ __device__ constexpr uint32_t idesc_fp4(int M, int N, int scale_e8m0, int a_sf_id, int b_sf_id) {
    return ((uint32_t)b_sf_id << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)scale_e8m0 << 23) |
           ((uint32_t)(M >> 4) << 24) | ((uint32_t)a_sf_id << 29);
}

// D[tmem] (+)= A[smem] * B[smem]^T ; issued by ONE thread
__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_nvf4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
                                         uint32_t tmem_sfa, uint32_t tmem_sfb) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}
__device__ __forceinline__ void mma_mxf4(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
                                         uint32_t tmem_sfa, uint32_t tmem_sfb) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}
// all MMAs issued so far by this thread arrive on `bar` when they have completed
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
// scale factors: 32 lanes x 128 bits from shared memory (no-swizzle descriptor) to TMEM, replicated to the
// four 32-lane quadrants
__device__ __forceinline__ void tmem_cp_sf(uint32_t tmem_dst, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;\n" ::"r"(tmem_dst), "l"(sdesc) : "memory");
}

// ---- CTA pairs (cta_group::2): two CTAs of a cluster, one on each of two SMs, execute one MMA of M = 256 ----
// Each CTA supplies its own 128 rows of A and half of B's rows from its own shared memory (same offsets in both
// CTAs) and receives the accumulator of its own 128 rows x all N columns in its own TMEM.  One thread of the
// leader CTA (cluster rank 0) issues the instruction for both.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// shared::cluster address of the location at CTA-local shared address `addr` in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
// The same without the release: the release form stalls the arriving thread for ~1100 cycles (measured beside running
// bulk copies and MMAs).  For signals whose payload is already complete when the arrive is issued: tensor-memory stores
// after tcgen05.wait::st, bulk-copy data after its own mbarrier phase was observed.
__device__ __forceinline__ void mbar_arrive_cluster_relaxed(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_addr) : "memory");
}
// try_wait whose acquire covers arrivals from the other CTA of the cluster
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity, uint32_t hint_ns = 2000u) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
#pragma unroll 1
    for (uint32_t it = 0; it < (1u << 21); it++) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if (it >= 64u && *abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }
// TMEM of both CTAs of the pair: the same warp of BOTH CTAs executes these, with the same operands
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(dst_smem), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
// kind::i8 on a CTA pair: M = 256 (128 rows per CTA), each CTA supplies half of B
__device__ __forceinline__ void mma_i8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_nvf4_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
                                              uint32_t tmem_sfa, uint32_t tmem_sfb) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}
__device__ __forceinline__ void mma_mxf4_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
                                              uint32_t tmem_sfa, uint32_t tmem_sfb) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}
// All MMAs issued so far by this thread (executed by both CTAs) arrive on the barrier at shared::cluster address
// `cluster_bar` when complete.  One barrier per call: to tell both CTAs, call it once with each CTA's barrier.
__device__ __forceinline__ void mma_commit_pair(uint32_t cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(cluster_bar) : "memory");
}
// scale-factor atom from each CTA's shared memory (same offset) into each CTA's TMEM
__device__ __forceinline__ void tmem_cp_sf_pair(uint32_t tmem_dst, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;\n" ::"r"(tmem_dst), "l"(sdesc) : "memory");
}

// ---- epilogue store of a 32-row x 32-token accumulator block ----
// v[j] = value of (row row_base + lane, token tok_base + j), as tcgen05.ld hands it out (lane = row).  Y is
// [tokens][rows] row-major, so lanes writing their own row would store 2- or 4-byte elements one token at a
// time; instead the block goes through `stage` (4 KB of shared memory private to the warp) transposed, and
// every lane stores 16 bytes of consecutive rows of one token.  `vec` = the 16-byte path is legal (Y base and
// leading dimension 16-byte aligned); rows >= n or tokens >= m are skipped.
template <bool BF16>
__device__ __forceinline__ void store_block_32x32(void *y, int64_t ldy, int64_t row_base, int64_t tok_base, int64_t n, int64_t m,
                                                  const float (&v)[32], uint8_t *stage, int lane, bool vec) {
    if (!vec || row_base + 32 > n) {
        const int64_t row = row_base + lane;
        if (row < n) {
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const int64_t tok = tok_base + j;
                if (tok < m) {
                    if (BF16) static_cast<__nv_bfloat16 *>(y)[tok * ldy + row] = __float2bfloat16_rn(v[j]);
                    else static_cast<float *>(y)[tok * ldy + row] = v[j];
                }
            }
        }
        return;
    }
    if (BF16) {
        __nv_bfloat16 *st = reinterpret_cast<__nv_bfloat16 *>(stage);
#pragma unroll
        for (int j = 0; j < 32; j++) st[j * 32 + lane] = __float2bfloat16_rn(v[j]);
        __syncwarp();
        // a token's 32 rows are 64 bytes: 4 lanes x 16 bytes, 8 tokens per pass
        const int part = lane & 3;
#pragma unroll
        for (int pass = 0; pass < 4; pass++) {
            const int j = pass * 8 + (lane >> 2);
            const int64_t tok = tok_base + j;
            if (tok < m)
                *reinterpret_cast<uint4 *>(static_cast<__nv_bfloat16 *>(y) + tok * ldy + row_base + part * 8) =
                    *reinterpret_cast<const uint4 *>(st + j * 32 + part * 8);
        }
    } else {
        float *st = reinterpret_cast<float *>(stage);
#pragma unroll
        for (int j = 0; j < 32; j++) st[j * 32 + lane] = v[j];
        __syncwarp();
        // a token's 32 rows are 128 bytes: 8 lanes x 16 bytes, 4 tokens per pass
        const int part = lane & 7;
#pragma unroll
        for (int pass = 0; pass < 8; pass++) {
            const int j = pass * 4 + (lane >> 3);
            const int64_t tok = tok_base + j;
            if (tok < m)
                *reinterpret_cast<uint4 *>(static_cast<float *>(y) + tok * ldy + row_base + part * 4) =
                    *reinterpret_cast<const uint4 *>(st + j * 32 + part * 4);
        }
    }
    __syncwarp();  // the staging block is rewritten by the next call
}

}  // namespace tc
}  // namespace gllmk
