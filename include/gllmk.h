/*
 * gllmk — B200 (sm_100a) implementation of the quantized-matmul operators of gllm-kernels.
 *
 * C ABI in the conventions of the reference's own FFI (gllm-kernels src/ffi/mod.rs,
 * src/ffi/types.rs:4-14,31-41): every entry point returns an int32 status with the reference's
 * values, results come back through out-pointers, every pointer is null-checked first
 * (-> GLLMK_STATUS_INVALID_ARG), handles are opaque `void*`, `*_free(NULL)` is a no-op and no
 * function panics or throws across the boundary.  No existing `gllm_*` symbol is replaced: the
 * reference's FFI has no quant-matmul entry point, so these are the symbols a Rust
 * `impl Kernels<f32>` shim binds for the quant slice of the operator trait
 * (src/traits.rs:473-608).  Each declaration names the reference interface it stands in for.
 *
 * Dimension names follow the benchmark: M = tokens, N = weight rows (output features),
 * K = reduction length.  The reference's `kquant_matmul(m, n, k)` calls these (N, M, K).
 *
 * There is no CPU fallback: without a CUDA device every compute entry returns
 * GLLMK_STATUS_RUNTIME_ERROR.
 */
#ifndef GLLMK_H
#define GLLMK_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define GLLMK_API __attribute__((visibility("default")))
#else
#define GLLMK_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* src/ffi/types.rs:4-14 (GllmStatus), same integers. */
enum {
    GLLMK_STATUS_OK = 0,
    GLLMK_STATUS_INVALID_ARG = -1,
    GLLMK_STATUS_OUT_OF_MEMORY = -2,
    GLLMK_STATUS_COMPILE_ERROR = -3,
    GLLMK_STATUS_RUNTIME_ERROR = -4,
    GLLMK_STATUS_UNSUPPORTED = -5,
    GLLMK_STATUS_IO_ERROR = -6
};

/* The formats of the path out of src/quant.rs:8-87 (QuantType).  The Rust enum has no stable
 * discriminants, so the ids are this boundary's. */
enum {
    GLLMK_QUANT_Q4K = 1,   /* QuantType::Q4K    256 el / 144 B  (src/quant.rs:122-127) */
    GLLMK_QUANT_Q8_0 = 2,  /* QuantType::Q8_0    32 el /  34 B  (src/quant.rs:290-293) */
    GLLMK_QUANT_MXFP4 = 3, /* QuantType::Mxfp4{block_size}      (src/quant.rs:66-76)   */
    GLLMK_QUANT_NVFP4 = 4, /* QuantType::Nvfp4   64 el /  36 B  (src/quant.rs:366-371) */
    GLLMK_QUANT_INT8 = 5,  /* plain s8 matrix of the W8A8 path (gllmk_int8_weight_upload); not a block format */
    /* The other GGUF formats of the reference's CPU quant path.  Kept on the device as the reference stores them
     * (Q6_K in 224-byte slots) and served by a streaming CUDA-core integer-dot GEMV (f32 activations and outputs,
     * any m) plus decode / gather / unpack; gllmk_gemm with bf16 operands, gllmk_gemm_grouped, gllmk_gemv_allgather and gllmk_ffn_decode
     * answer GLLMK_STATUS_UNSUPPORTED for them. */
    GLLMK_QUANT_Q6_K = 6,  /* QuantType::Q6K    256 el / 210 B  (src/quant.rs:143-148) */
    GLLMK_QUANT_Q5_K = 7,  /* QuantType::Q5K    256 el / 176 B  (src/quant.rs:132-138) */
    GLLMK_QUANT_Q4_0 = 8,  /* QuantType::Q4_0    32 el /  18 B  (src/quant.rs:254-257) */
    GLLMK_QUANT_Q5_0 = 9,  /* QuantType::Q5_0    32 el /  22 B  (src/quant.rs:271-275) */
    GLLMK_QUANT_Q8_K = 10  /* QuantType::Q8K    256 el / 292 B  (src/quant.rs:153-157) */
};

/* Element type of an activation / output matrix handed to gllmk_gemm. */
enum { GLLMK_DTYPE_F32 = 0, GLLMK_DTYPE_BF16 = 1 };

typedef void *gllmk_ctx;    /* opaque, like GllmBackend (src/ffi/types.rs:31-32) */
typedef void *gllmk_weight; /* opaque, like GllmWeights (src/ffi/types.rs:40-41) */

/* ---- library / device information ------------------------------------------------------- */

/* gllm_version (src/ffi/mod.rs:198-201): static NUL-terminated string. */
GLLMK_API const char *gllmk_version(void);
/* gllm_hw_info (src/ffi/mod.rs:209-222): writes a NUL-terminated description of device 0 (or
 * "no CUDA device"), returns the bytes written (excluding NUL) or INVALID_ARG. */
GLLMK_API int32_t gllmk_hw_info(char *buf, size_t len);
/* QuantType::block_size / block_bytes (src/quant.rs:375-456); 0 for an unknown id.
 * `mx_block` is Mxfp4's block_size and ignored otherwise. */
GLLMK_API int32_t gllmk_quant_block_size(int32_t quant_type, int32_t mx_block);
GLLMK_API int32_t gllmk_quant_block_bytes(int32_t quant_type, int32_t mx_block);

/* ---- format descriptors ------------------------------------------------------------------------------- */

/* QuantFormatDescriptor (src/quant_format.rs:129-157), flattened for C: where a block of a format keeps its
 * scale(s), its zero point / min and its quantized data.  The enums mirror ScaleLayout (:159-199), ZeroLayout
 * (:202-225), DataLayout (:228-252), ScaleDType (:255-266), QuantDataKind (:94-121), StorageLayout (:19-30) and
 * NativeIsa (:53-91; only the variants these formats use).  Offsets are bytes from the start of the block, -1 =
 * the format has no such field.  The library's own kernels read their offsets from the same table. */
enum { GLLMK_SCALE_NONE = 0, GLLMK_SCALE_BLOCK_SCALAR, GLLMK_SCALE_BLOCK_SCALAR_WITH_MIN, GLLMK_SCALE_HIERARCHICAL,
       GLLMK_SCALE_Q6K_SCALES, GLLMK_SCALE_EXTERNAL_ARRAY, GLLMK_SCALE_SUB_BLOCK_SCALARS };
enum { GLLMK_ZERO_NONE = 0, GLLMK_ZERO_BLOCK_SCALAR, GLLMK_ZERO_HIERARCHICAL, GLLMK_ZERO_STATIC_BIAS, GLLMK_ZERO_BLOCK_MIN };
enum { GLLMK_DATA_PACKED_NIBBLES = 0, GLLMK_DATA_NIBBLE_WITH_HIGH_BITS, GLLMK_DATA_BYTES };
enum { GLLMK_SDT_F16 = 0, GLLMK_SDT_F32, GLLMK_SDT_BF16, GLLMK_SDT_U8RANGE, GLLMK_SDT_I8RANGE, GLLMK_SDT_F8E4M3, GLLMK_SDT_F8E5M2,
       GLLMK_SDT_E8M0 };
enum { GLLMK_KIND_INT8 = 0, GLLMK_KIND_PACKED_INT4, GLLMK_KIND_SIGNED_PACKED_INT4, GLLMK_KIND_PACKED_INT5, GLLMK_KIND_PACKED_INT6,
       GLLMK_KIND_FLOAT4, GLLMK_KIND_NVFP4 };
enum { GLLMK_STORAGE_ROW_MAJOR = 0, GLLMK_STORAGE_COL_INTERLEAVED, GLLMK_STORAGE_PACKED };
enum { GLLMK_ISA_NONE = 0, GLLMK_ISA_VPDPBUSD, GLLMK_ISA_TCGEN05_FP4 };
typedef struct gllmk_quant_format_descriptor {
    int32_t quant_type;          /* GLLMK_QUANT_*                                                              */
    int32_t block_size;          /* elements per block                                                          */
    int32_t block_bytes;         /* bytes per block                                                             */
    int32_t bits_per_element;
    int32_t scale_kind;          /* GLLMK_SCALE_*                                                               */
    int32_t scale_dtype;         /* GLLMK_SDT_* of the block / sub-block scale                                  */
    int32_t scale_offset;        /* BlockScalar.offset_bytes, Hierarchical.block_d_offset, Q6KScales.block_d_offset,
                                    SubBlockScalars.offset_bytes                                               */
    int32_t scale_min_offset;    /* Hierarchical.block_dmin_offset                                             */
    int32_t sub_scales_offset;   /* Hierarchical / Q6KScales sub_scales_offset; SubBlockScalars.offset_bytes   */
    int32_t sub_scales_bits;     /* 6 = KQuant6Bit packing (12 bytes -> 8 (scale, min) pairs); 8 = one byte each */
    int32_t sub_scales_count;
    int32_t sub_block_elements;
    int32_t zero_kind;           /* GLLMK_ZERO_*                                                               */
    int32_t zero_offset;         /* Hierarchical.dmin_offset                                                   */
    int32_t zero_sub_offset;     /* Hierarchical.sub_m_offset                                                  */
    int32_t static_bias;         /* StaticBias.value (subtracted from the code)                                */
    int32_t data_layout;         /* GLLMK_DATA_*                                                               */
    int32_t data_offset;         /* PackedNibbles.offset, NibbleWithHighBits.low_offset, Bytes.offset          */
    int32_t data_high_offset;    /* NibbleWithHighBits.high_offset                                             */
    int32_t data_high_bits;      /* NibbleWithHighBits.high_bits_per_elem                                      */
    int32_t data_low_first;      /* PackedNibbles.low_first                                                    */
    int32_t data_signed;         /* Bytes.signed                                                               */
    int32_t data_kind;           /* GLLMK_KIND_*                                                               */
    int32_t storage_layout;      /* GLLMK_STORAGE_*                                                            */
    int32_t native_isa;          /* GLLMK_ISA_* (Nvfp4: Tcgen05Fp4, src/quant_format.rs:1026)                  */
} gllmk_quant_format_descriptor;
/* QuantFormatDescriptor::for_type (src/quant_format.rs:36-44).  UNSUPPORTED for a type this library does not serve
 * (the reference panics for an unregistered type).  `mx_block` as in gllmk_quant_block_size.  Needs no device. */
GLLMK_API int32_t gllmk_quant_format_descriptor_for_type(int32_t quant_type, int32_t mx_block, gllmk_quant_format_descriptor *out);
/* registry() (src/quant_format.rs:1189-1193), restricted to the served formats: writes up to `cap` GLLMK_QUANT_* ids
 * and returns how many formats are registered. */
GLLMK_API int32_t gllmk_quant_format_registry(int32_t *quant_types, int32_t cap);

/* ---- context ---------------------------------------------------------------------------- */

/* gllm_backend_create / gllm_backend_free (src/ffi/mod.rs:25-57).  Binds to CUDA device
 * `device`; owns the activation staging workspace shared by all calls made with it.  Calls on
 * one context must not overlap in time (use one context per stream / thread). */
GLLMK_API int32_t gllmk_ctx_create(int32_t device, gllmk_ctx *out);
GLLMK_API void gllmk_ctx_free(gllmk_ctx ctx);
/* Text of the last error raised through this context ("" if none).  Never NULL. */
GLLMK_API const char *gllmk_last_error(gllmk_ctx ctx);
/* Waits for the device and reads the context's device-side status word: every wait inside a kernel
 * (on a bulk-copy barrier, a tensor-core completion, another GPU's flag) is bounded, and a kernel that
 * gives one up records a non-zero code there and returns instead of hanging.  Returns RUNTIME_ERROR if it
 * was set, and puts the context back into a usable state: the word and the decode kernels' split-k arrival
 * counters (which a kernel that gave up leaves non-zero) are cleared, so the next call on the context is
 * correct again.  Results of the call that gave up are incomplete.  Codes name the kernel and the wait: 1-2 decode GEMV (consumer, producer),
 * 10-14 fused-dequant prefill GEMM, 21-23 FP4 x FP4 GEMM, 31 gllmk_peer_barrier, 32 gllmk_gemv_exchange /
 * gllmk_exchange_wait (another rank's products), 41-46 W8A8 GEMM, 51-54 FP4
 * decode GEMV on the tensor core. */
GLLMK_API int32_t gllmk_ctx_status(gllmk_ctx ctx, int32_t *device_status);
/* Tuning knobs, for experiments.  key: "gemv_ctas_per_sm" (resident CTAs per SM the decode grid is
 * sized for; 0 = occupancy limit), "gemv_pdl" (1 = overlap the activation staging kernel with the
 * weight stream), "gemv_fp4_int" (1 = decode MXFP4 / NVFP4 weights on the integer-decode kernel instead of
 * the block-scaled tensor-core one), "gemv_fuse" (decode GEMV converting its own activation slices instead of a staging launch when a
 * block's share is small: 0 never (default), 1 products of an exchange chain only, 2 every product), "gemm_fp4_pair" (FP4 x FP4 GEMM with
 * m > 128: 0 the one-CTA kernel, 1 (default) CTA pairs with one 256-token accumulator, 2 CTA pairs with two 192-token
 * accumulators, 3 CTA pairs with two 128-token accumulators), "gemm_i8_pair" (W8A8 GEMM with m > 128 on the CTA-pair kernel: 0 never, 1 (default) when the estimate favours it, 2 always),
 * "host_batch_graph" (gllmk_matmul_host_batch replays a captured graph for a repeated
 * argument list: 1 default, 0 never), "gemm_tail_split" (prefill GEMM, last partial wave of tiles cut along k:
 * 0 automatic, 1 never, n into n), "gemm_row_tiles" (prefill GEMM, 128-row weight tiles per CTA: 0 estimated, 1, 2),
 * "gemm_raw_slots" (prefill GEMM, depth of the raw weight ring: 0 = what the shared-memory plan gives),
 * "raw_gemv_mma" (Q6_K products of 2 tokens and more on the mma.sync kernel: 1 default, 0 the dp2a kernel, 2 a single token too),
 * "gemm_pdl" (prefill GEMM launched programmatically behind its activation staging kernel: 1 default, 0 plain launch), "peer_wait_spins" (how many times a wait on another GPU's flag probes it
 * before it gives up with status 31; default 2^22, about a second), "inject_give_up" (testing aid, host side
 * only: leaves the context as a kernel that gave up a wait with that status code would — word set, arrival
 * counters dirty — without making any kernel wait). */
GLLMK_API int32_t gllmk_ctx_set(gllmk_ctx ctx, const char *key, int64_t value);

/* ---- weights: upload + repack, the inverse, and the bit-exact decode ----------------------- */

/* gllm_weights_create + gllm_weights_get_ptr fill (src/ffi/mod.rs:228-345): takes a weight
 * matrix of `n` rows x `k` columns as the reference stores it — row-major runs of k/block_size
 * blocks (src/cpu_kernels/mod.rs:476) — and repacks it on the device into the 16-byte-aligned
 * tiled layout the kernels stream.
 *   Q4K / Q8_0 / NVFP4: `blocks` holds n*(k/bs)*block_bytes bytes, `scales` must be NULL.
 *   MXFP4: split form of dequant_mxfp4 (src/quant_mxfp4.rs:72) — `blocks` holds n*k/2 nibble
 *          bytes and `scales` n*k/mx_block E8M0 bytes; or, with scales == NULL, the GGUF inline
 *          form (17-byte blocks, scale first; src/quant.rs:427).  mx_block must be 32.
 *   `global_scale` is NVFP4's out-of-band per-tensor f32 (src/quant.rs:77-86); pass 1 otherwise.
 *   `src_on_device` != 0 means `blocks`/`scales` are device pointers (16-byte aligned); the call then waits
 *   for all work already queued on the device (whatever stream produced the blocks) before it repacks.
 * Errors: INVALID_ARG (null, n<=0, k not a multiple of the block size, or of 128 for MXFP4),
 * UNSUPPORTED (unknown type, mx_block != 32), OUT_OF_MEMORY, RUNTIME_ERROR. */
GLLMK_API int32_t gllmk_weight_upload(gllmk_ctx ctx, int32_t quant_type, int64_t n, int64_t k, int32_t mx_block,
                            const void *blocks, const void *scales, float global_scale,
                            int32_t src_on_device, gllmk_weight *out);
/* gllm_weights_free (src/ffi/mod.rs:262-266). */
GLLMK_API void gllmk_weight_free(gllmk_weight w);
/* Shape / size query.  Any out-pointer may be NULL.  `ref_bytes` = bytes of the reference-format
 * blocks (the algorithmic weight bytes), `dev_bytes` = bytes held on the device. */
GLLMK_API int32_t gllmk_weight_info(gllmk_weight w, int32_t *quant_type, int64_t *n, int64_t *k, uint64_t *ref_bytes,
                          uint64_t *dev_bytes);
/* Inverse of the repack: writes the reference-format bytes back (same forms as upload; for MXFP4
 * always the split form).  Bit-exact round trip. `dst_on_device` as above. */
GLLMK_API int32_t gllmk_weight_unpack(gllmk_ctx ctx, gllmk_weight w, void *blocks, void *scales, int32_t dst_on_device);
/* Kernels::dequant_q4_k / dequant_q8_0 (src/traits.rs:476,488), dequant_mxfp4_scalar
 * (src/quant_mxfp4.rs:72-109) and the NVFP4 formula (src/quant.rs:77-86) over the whole matrix:
 * f32 [n, k] row-major into device memory, bit-exact with the reference's scalar decode. */
GLLMK_API int32_t gllmk_dequant(gllmk_ctx ctx, gllmk_weight w, float *out_dev, void *stream);

/* ---- decode: fused dequantize + GEMV (M <= 16 tokens) -------------------------------------- */

/* Quantized embedding lookup (the reference emits it inline in its JIT, emit_quant_gather_inline, tested at
 * src/compiler/codegen/x86_64/jit/quant_gemv_tests.inc.rs:541-828): out[r, :] = decode(weight row ids[r]) for
 * r < count, f32 [count, k] row-major, bit-exact with gllmk_dequant.  ids are on the device; an id outside
 * [0, n) yields a row of zeros. */
GLLMK_API int32_t gllmk_embedding_gather(gllmk_ctx ctx, gllmk_weight w, const int32_t *ids_dev, int64_t count, float *out_dev,
                               void *stream);

/* Kernels::kquant_matmul / classic_matmul (src/traits.rs:543-563) and gemm_q4
 * (src/traits.rs:511-520) for small batches, on device memory with resident weights.
 *   y[t, r] = sum_k W[r, k] * x[t, k],  t < m <= GLLMK_GEMV_MAX_M, r < n.
 * Element (t, k) of x is x_dev[t*x_stride_t + k*x_stride_k]; element (t, r) of y is
 * y_dev[t*y_stride_t + r*y_stride_r] — so the reference's [k, n]-input / [m, n]-output convention
 * is strides (1, n_ref) / (1, n_ref) and gemm_q4's [m, k] / [m, n] is (k, 1) / (n, 1).
 * `row_scales` (NULL, or 1 or n entries on the device; any other count is INVALID_ARG) multiplies row r's
 * result like gemm_q4's `scales`.  f32 accumulation; result within 2e-3 of the reference's sequential f32 sum.  All four
 * weight types (for MXFP4 / NVFP4 the reference has no matmul; the oracle is its dequant followed by the
 * same f32 sum). */
#define GLLMK_GEMV_MAX_M 16
GLLMK_API int32_t gllmk_gemv(gllmk_ctx ctx, gllmk_weight w, const float *x_dev, int64_t x_stride_t, int64_t x_stride_k,
                   int32_t m, float *y_dev, int64_t y_stride_t, int64_t y_stride_r, const float *row_scales,
                   int64_t n_row_scales, void *stream);

/* One gated feed-forward block for m <= GLLMK_GEMV_MAX_M tokens: the step on either side of the decode
 * products (Activation::is_gated, src/traits.rs:16-25; Kernels::swiglu, src/traits.rs:446;
 * scalar_swiglu, scalar-ops/src/activations.rs:57-66):
 *   h = W_gate_up x        h [m, 2f]: columns [0, f) = gate, [f, 2f) = up (gate and up stored as one weight)
 *   y = W_down (silu(gate) * up),  silu(g) = g / (1 + exp(-g)) in f32
 * Two decode products; SwiGLU is applied by the second product's activation staging while it reads h, so
 * there is no separate activation kernel and no third buffer.  x [m, k] and y [m, k] row-major, h is
 * caller-provided scratch of m * 2f floats (it holds gate || up afterwards). */
GLLMK_API int32_t gllmk_ffn_decode(gllmk_ctx ctx, gllmk_weight w_gate_up, gllmk_weight w_down, const float *x_dev, int32_t m,
                         float *h_dev, float *y_dev, void *stream);

/* The same block for any number of tokens (prefill): two tensor-core products with the intermediate kept in bf16,
 *   h = W_gate_up x   (bf16 [m, 2f], caller-provided scratch; it holds gate || up afterwards)
 *   y = W_down (silu(gate) * up)
 * SwiGLU (f32 arithmetic on the bf16 values of h) is applied by the second product's activation staging, so no
 * activation kernel runs and no third buffer exists.  x [m, k] f32 or bf16 (ldx), y [m, k] f32 or bf16 (ldy); the
 * Q4_K / Q8_0 / MXFP4 / NVFP4 weights of gllmk_gemm, and Q6_K / Q5_K / (k a multiple of 256:) Q4_0 / Q5_0; the two weights
 * may differ in format (a GGUF file often pairs Q4_K gate / up with a Q6_K down projection).  Each product is within 1e-2
 * of the reference's f32 evaluation. */
GLLMK_API int32_t gllmk_ffn_prefill(gllmk_ctx ctx, gllmk_weight w_gate_up, gllmk_weight w_down, const void *x_dev, int32_t x_dtype,
                                    int64_t ldx, int32_t m, void *h_dev, void *y_dev, int32_t y_dtype, int64_t ldy, void *stream);

/* ---- W8A8 integer path ------------------------------------------------------------------------------ */

/* avx512_int8::gemm_int8 and dequantize_i32_to_f32 (src/macros/matmul_x86_int8.rs:307-456; tests
 * src/tests_int8.rs:21-136):  C (s32) [m, n] = A (u8) [m, k] x B (s8) [k, n], exact integers, then
 * out = (C as f32) * scale_a * scale_b (+ bias[j]) followed by an activation.
 * gllmk_int8_weight_upload: B once -> resident tile images.  layout 0: B is [k, n] row-major as in the
 *   reference; layout 1: [n, k] row-major (one weight row after the other).  Freed with gllmk_weight_free.
 * gllmk_gemm_int8: device A (leading dimension lda, any alignment) and device C (ldc); tcgen05 kind::i8 with
 *   an s32 accumulator in tensor memory: bit-exact for every shape (|sum| stays below 2^31 for k < 66000).
 * gllmk_dequantize_i32_f32: element-wise epilogue on device buffers (contiguous [m, n]); bias_dev may be NULL;
 *   activation: GLLMK_ACT_* (the reference's Activation, src/traits.rs:7-15).
 * gllmk_gemm_int8_host: the reference call with host slices (its packed copy of B is not needed). */
enum { GLLMK_ACT_NONE = 0, GLLMK_ACT_RELU = 1, GLLMK_ACT_SILU = 2, GLLMK_ACT_GELU = 3, GLLMK_ACT_GEGLU = 4 };
GLLMK_API int32_t gllmk_int8_weight_upload(gllmk_ctx ctx, int64_t n, int64_t k, const int8_t *b, int32_t layout, int32_t src_on_device,
                                 gllmk_weight *out);
GLLMK_API int32_t gllmk_gemm_int8(gllmk_ctx ctx, gllmk_weight w, const uint8_t *a_dev, int64_t lda, int32_t m, int32_t *c_dev,
                        int64_t ldc, void *stream);
GLLMK_API int32_t gllmk_dequantize_i32_f32(gllmk_ctx ctx, const int32_t *c_dev, float *out_dev, int64_t m, int64_t n, float scale_a,
                                 float scale_b, const float *bias_dev, int32_t activation, void *stream);
GLLMK_API int32_t gllmk_gemm_int8_host(gllmk_ctx ctx, const uint8_t *a, const int8_t *b_kn, int32_t *c, size_t m, size_t n, size_t k);
/* The activation half of W8A8: quantize_from_fp32 with QuantFormat::Int8PerTensor (src/compiler/quant_convert.rs:17-20,
 * 165-177) on device memory: scale = max|x| / 127 over the whole [rows, k] tensor (leading dimension ldx),
 * q = (x / scale).round().clamp(-128, 127), round half away from zero, bit-exact with the reference's loop.
 * q_dev receives one byte per element (leading dimension ldq): the reference's signed values, or, with
 * as_unsigned != 0, q + 128 — the unsigned operand gllmk_gemm_int8 takes.  scale_dev: TWO 32-bit words of device
 * memory; word 0 receives the f32 scale (word 1 is the routine's running maximum). */
GLLMK_API int32_t gllmk_quantize_act_int8(gllmk_ctx ctx, const float *x_dev, int64_t rows, int64_t k, int64_t ldx, void *q_dev, int64_t ldq,
                                int32_t as_unsigned, float *scale_dev, void *stream);
/* A whole W8A8 linear layer on device memory: y = act((q_x . W) * scale_x * scale_b + bias), x f32 [m, k] quantized per
 * tensor as above, products on the tensor core (u8 = q_x + 128 against s8 weights), the 128 * sum_k W[k, j] the offset
 * adds taken off the exact s32 result with column sums computed at upload, then dequantize_i32_to_f32's epilogue. */
GLLMK_API int32_t gllmk_w8a8_linear_f32(gllmk_ctx ctx, gllmk_weight w, const float *x_dev, int64_t ldx, int32_t m, float *y_dev, int64_t ldy,
                              float scale_b, const float *bias_dev, int32_t activation, void *stream);

/* ---- multi-GPU: row-sharded decode with the all-gather fused into the GEMV -------------------------- */

/* No counterpart in the reference (single device).  Weights are sharded by rows over the GPUs of one node
 * (one process per GPU); every rank needs the whole y.  Instead of a collective after each product, the
 * decode kernel stores its band of y into EVERY rank's copy of y through peer-mapped pointers, and a flag
 * barrier tells each rank when all bands have landed.
 *
 * gllmk_shared_alloc: device buffer other processes of the node can map; `handle` (GLLMK_IPC_HANDLE_BYTES
 *   bytes) is what the host framework sends to the other ranks.  The buffer starts zeroed; its first
 *   GLLMK_PEER_FLAG_BYTES bytes are the barrier's flag words, the rest is the caller's (y copies).
 * gllmk_shared_open / _close: map / unmap another rank's buffer from its handle.  _free: release one's own.
 * gllmk_gemv_allgather: gllmk_gemv (no row scales) whose result element (t, r) is also stored at the same
 *   element offset from each of `y_peers[0..n_peers)`.  Every pointer is the position of this rank's band
 *   inside that rank's y.
 * gllmk_peer_barrier: on `stream`, after this rank's products: signal sequence number `seq` to every peer and
 *   wait (bounded, about a second; on time-out the context's status word becomes 31 and the kernel returns)
 *   until every peer has signalled `seq`.  `flags_peers[q]` is the q-th OTHER rank's flag words in rank
 *   order, `rank` this rank's number.  `seq` must grow by one per barrier, starting at 1; seq = 0 means
 *   "use and advance the counter kept in this rank's flag area", which is what a captured CUDA graph
 *   needs (every rank must then use 0 for every barrier).  After the barrier, y is complete on this rank.  A buffer may be rewritten by peers one barrier after its last reader finished. */
/* gllmk_gemv_exchange: the same product with the hand-shake built in, for chains of sharded products (a decode
 *   step): before it reads x it waits (bounded: "peer_wait_spins" probes per rank, then status 32) until every
 *   rank has completed as many exchange products as this rank — so an x that is the previous product's gathered y
 *   is complete — and the block that finishes last signals the new count to every rank (one system-scope fence per launch).  No
 *   barrier kernel between products: one staging + one GEMV launch per product, whose weight prefetch overlaps
 *   the wait.  Every rank must issue the same sequence of exchange products; flags_local / flags_peers are the
 *   flag words at the start of each rank's gllmk_shared_alloc buffer (this call uses words 32..48, the barrier
 *   words 0..16).  A buffer may be rewritten by peers one product after its last reader finished.
 *   x_up_dev != NULL: the activation is silu(x) * x_up (same strides) — the sharded form of gllmk_ffn_decode: a
 *   gate || up product gathered into h [m, 2f], then the down product with x = h, x_up = h + f.
 * gllmk_exchange_wait: after the last product of a chain, on `stream`: returns once every rank's bands of that
 *   product have landed here (what the next product's staging would otherwise wait for). */
#define GLLMK_MAX_PEERS 7
#define GLLMK_IPC_HANDLE_BYTES 64
#define GLLMK_PEER_FLAG_BYTES 256
GLLMK_API int32_t gllmk_shared_alloc(gllmk_ctx ctx, size_t bytes, void **dev_ptr, uint8_t *handle);
GLLMK_API int32_t gllmk_shared_open(gllmk_ctx ctx, const uint8_t *handle, void **peer_ptr);
GLLMK_API int32_t gllmk_shared_close(gllmk_ctx ctx, void *peer_ptr);
GLLMK_API int32_t gllmk_shared_free(gllmk_ctx ctx, void *dev_ptr);
GLLMK_API int32_t gllmk_gemv_allgather(gllmk_ctx ctx, gllmk_weight w, const float *x_dev, int64_t x_stride_t, int64_t x_stride_k,
                             int32_t m, float *y_local, int64_t y_stride_t, int64_t y_stride_r, void *const *y_peers,
                             int32_t n_peers, void *stream);
GLLMK_API int32_t gllmk_peer_barrier(gllmk_ctx ctx, void *flags_local, void *const *flags_peers, int32_t n_peers, int32_t rank,
                           uint32_t seq, void *stream);
GLLMK_API int32_t gllmk_gemv_exchange(gllmk_ctx ctx, gllmk_weight w, const float *x_dev, const float *x_up_dev, int64_t x_stride_t,
                                      int64_t x_stride_k, int32_t m, float *y_local, int64_t y_stride_t, int64_t y_stride_r,
                                      void *const *y_peers, void *flags_local, void *const *flags_peers, int32_t n_peers, int32_t rank,
                                      void *stream);
GLLMK_API int32_t gllmk_exchange_wait(gllmk_ctx ctx, void *flags_local, int32_t n_peers, int32_t rank, void *stream);

/* ---- prefill: fused dequantize + GEMM on tcgen05 tensor cores (any M) --------------------------- */

/* Kernels::gemm_q4 / kquant_matmul / classic_matmul for large batches, and the matmul the reference
 * leaves unimplemented for MXFP4 / NVFP4 weights (src/cpu_kernels/mod.rs:3347-3348; oracle = its dequant
 * followed by scalar_gemm, scalar-ops/src/blas.rs:116-135), on device memory with resident weights:
 *   y[t, r] = sum_k W[r, k] * a[t, k],  a [m, k] row-major (leading dimension lda), y [m, n] (ldy).
 * a_dtype / y_dtype: GLLMK_DTYPE_F32 or GLLMK_DTYPE_BF16.  Weights and activations are staged in fp16
 * (activations saturate at +-65504) and accumulated in f32: results within 1e-2 of the reference's f32
 * evaluation.  a and its rows must be 16-byte aligned.  With f32 in and out and
 * m <= GLLMK_GEMM_GEMV_MAX_M the call is one pass of the decode kernel (gllmk_gemv), which is faster
 * there and meets its tighter bound (from 17 tokens on the tensor-core kernel is the faster one:
 * W[28672, 8192] Q4_K at m = 32: 80 us against 113 us as two decode passes).  Of the other GGUF formats Q6_K and Q5_K
 * have a place in this kernel (Q6_K: more than 8 tokens, up to 8 its batch GEMV; Q5_K: 2 tokens and more; f32 only below),
 * and so have Q4_0 and Q5_0 when k is a multiple of 256 (2 tokens and more); Q8_K, and Q4_0 / Q5_0 with another k, run the
 * streaming GEMV over token tiles and take f32 only. */
#define GLLMK_GEMM_GEMV_MAX_M 16
GLLMK_API int32_t gllmk_gemm(gllmk_ctx ctx, gllmk_weight w, const void *a_dev, int32_t a_dtype, int64_t lda, int32_t m,
                             void *y_dev, int32_t y_dtype, int64_t ldy, void *stream);

/* A mixture-of-experts layer in one launch (no counterpart in the reference, which would loop over experts):
 * group g multiplies rows [row_offsets[g], row_offsets[g+1]) of a (tokens already gathered per expert) by
 * weights[g] and writes the same rows of y.  `row_offsets` is a HOST array of n_groups + 1 non-decreasing
 * entries; all weights must have one type and shape; empty groups are allowed.  Same numerics as gllmk_gemm. */
GLLMK_API int32_t gllmk_gemm_grouped(gllmk_ctx ctx, int32_t n_groups, const gllmk_weight *weights, const void *a_dev, int32_t a_dtype,
                           int64_t lda, const int64_t *row_offsets, void *y_dev, int32_t y_dtype, int64_t ldy, void *stream);

/* ---- mixture-of-experts routing conventions around gllmk_gemm_grouped -------------------------------- */

/* scalar_topk (scalar-ops/src/moe.rs:59-115) on device memory: for every row of gate_probs [seq_len,
 * num_experts] the top_k largest values (strict '>' insertion: the earlier expert wins a tie) and their
 * indices.  out holds 2 * seq_len * top_k floats: first the indices [seq_len * top_k] as u32 BIT PATTERNS in
 * f32 slots, then the weights [seq_len * top_k] renormalised to sum 1 (value * (1 / sum), 0 if sum <= 0).
 * Bit-exact with the reference's routine.  top_k <= 16. */
GLLMK_API int32_t gllmk_moe_topk(gllmk_ctx ctx, const float *gate_probs_dev, float *out_dev, int64_t seq_len, int32_t num_experts,
                                 int32_t top_k, void *stream);
/* Groups the (token, k) slots of a scalar_topk index section per expert — "rows grouped per expert", the order
 * gllmk_gemm_grouped takes its activation rows in.  Within an expert the slots keep their order.
 *   row_offsets_host [num_experts + 1]: rows of expert e are [row_offsets[e], row_offsets[e + 1])  (HOST, out)
 *   perm_dev [seq_len * top_k]: grouped row -> slot s * top_k + ki                                   (device, out)
 *   inv_dev  [seq_len * top_k]: slot -> grouped row, -1 for an index >= num_experts, which no expert serves
 *                               (scalar_moe_dispatch_packed skips it, scalar-ops/src/moe_dispatch_packed.rs:113-116)
 * Synchronises `stream` (the offsets come back to the host).  num_experts <= 1024. */
GLLMK_API int32_t gllmk_moe_route(gllmk_ctx ctx, const float *indices_dev, int64_t seq_len, int32_t num_experts, int32_t top_k,
                                  int64_t *row_offsets_host, int32_t *perm_dev, int32_t *inv_dev, void *stream);
/* out[g, :] = x[perm[g] / top_k, :] for g < rows: the activation rows in grouped order (f32 or bf16). */
GLLMK_API int32_t gllmk_moe_gather(gllmk_ctx ctx, const void *x_dev, int32_t dtype, int64_t ldx, const int32_t *perm_dev, int64_t rows,
                                   int32_t top_k, int64_t k, void *out_dev, int64_t ldo, void *stream);
/* scalar_weighted_sum (scalar-ops/src/moe.rs:127-157): out[s, d] = sum_ki weights[s, ki] * row(s, ki)[d], terms
 * added in ki order onto 0 with a separate multiply and add each (bit-exact with the reference's loop).
 *   inv_dev == NULL: expert_outputs is the reference's buffer [expert][seq_len][hidden] (ld = hidden);
 *   inv_dev != NULL: expert_outputs holds the grouped rows gllmk_gemm_grouped wrote (leading dimension ld) and
 *                    row(s, ki) = expert_outputs[inv[s * top_k + ki]]; slots with inv < 0 add nothing. */
GLLMK_API int32_t gllmk_moe_weighted_sum(gllmk_ctx ctx, const float *expert_outputs_dev, int64_t ld, const float *indices_dev,
                                         const float *weights_dev, const int32_t *inv_dev, float *out_dev, int64_t seq_len,
                                         int64_t hidden, int32_t top_k, int32_t num_experts, void *stream);

/* Both operands in FP4 (config "NVFP4 prefill GEMM": weights and activations quantized the same way;
 * the reference declares the format, src/quant.rs:357-371, and a native-FP4 capability,
 * DotProductCap::NativeFp4 / Tcgen05Fp4 in src/quant_format.rs:1007-1027, but ships no kernel).
 * `x` is the activation matrix [m, k] quantized with gllmk_quantize and uploaded with
 * gllmk_weight_upload like a weight (same type as `w`, NVFP4 or MXFP4).
 *   y[t, r] = gW * gX * sum_k W4[r, k] * X4[t, k]   -> y [m, n] row-major (ldy), f32 or bf16.
 * Products of the decoded FP4 values and their block scales are exact; accumulation is f32. */
GLLMK_API int32_t gllmk_gemm_fp4(gllmk_ctx ctx, gllmk_weight w, gllmk_weight x, void *y_dev, int32_t y_dtype, int64_t ldy,
                                 void *stream);

/* Measurement aid, no counterpart in the reference: the block-scaled FP4 MMA of gllmk_gemm_fp4 (kind::mxf4nvf4 scale_vec::4X
 * for nvfp4 != 0, kind::mxf4 scale_vec::2X otherwise; one CTA per SM, or CTA pairs with cta_pair != 0) issued back to
 * back on operands parked in shared memory.  with_scale_copies: 0 = no scale-factor traffic, 1 = the scale atoms copied to
 * tensor memory by tcgen05.cp from the MMA thread every k-step (what the one-CTA kernel does), 2 = written by four scale
 * warps with tcgen05.st into rotating column sets (what the CTA-pair kernel does).  Writes the TFLOP/s reached (best of three timed launches of `ksteps` k-steps of 256 per CTA): the practical ceiling
 * of the FP4 x FP4 GEMM on this device, which bench.py reports as the denominator beside the nominal peak.
 * Synchronous on the context's own stream. */
GLLMK_API int32_t gllmk_probe_fp4_mma(gllmk_ctx ctx, int32_t cta_pair, int32_t with_scale_copies, int32_t nvfp4, int32_t ksteps, float *tflops);

/* Same product as gllmk_gemv for callers that are not allowed to allocate device memory while they run:
 * a serving loop whose allocator has already claimed all of HBM for weights and KV pages, code running
 * under a pool allocator that owns the device, or a latency-critical section where cudaMalloc's implicit
 * device synchronisation is unacceptable.  This entry point has no counterpart in the reference (its CPU
 * path keeps scratch in a thread_local Vec).  It calls no cudaMalloc / cudaFree and no allocating library
 * routine: the activation image, the split-k partial sums and the arrival counters all live in one 8 MiB
 * array compiled into the library, which every GPU that loads the library holds until the process exits.
 * A bounded wait that gives up is reported through the context's own status word (allocated with the
 * context), i.e. by gllmk_ctx_status exactly as for gllmk_gemv.
 *   - Shapes whose scratch does not fit (more than 8192 row tiles = 131072 rows, or image + partial sums
 *     over 8 MiB; the message gives the byte count) are rejected with INVALID_ARG: use gllmk_gemv there.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress); make that
 *     first call before any stream capture begins.
 *   - All calls on a device share the array, whatever context they use.  Calls that overlap in time on
 *     the GPU (different streams, different contexts) race on it; serialise them.  The array keeps the
 *     previous call's contents; the part that must start at zero is cleared on the caller's stream.
 * Arguments, results and accuracy are those of gllmk_gemv (the same kernels run). */
GLLMK_API int32_t gllmk_gemv_static(gllmk_ctx ctx, gllmk_weight w, const float *x_dev, int64_t x_stride_t,
                                    int64_t x_stride_k, int32_t m, float *y_dev, int64_t y_stride_t,
                                    int64_t y_stride_r, const float *row_scales, int64_t n_row_scales, void *stream);

/* ---- host-pointer drop-ins of the reference operator API ----------------------------------- */

/* Kernels::kquant_matmul(weight_blocks, input, output, QuantType::Q4K, m, n, k) and
 * Kernels::classic_matmul(.., QuantType::Q8_0, ..) with E = f32 (src/traits.rs:543-563; CPU
 * implementation src/cpu_kernels/mod.rs:3226-3394).  All three pointers are HOST memory, exactly
 * as the reference takes slices: m weight rows, n batch columns, input [k, n], output [m, n].
 * Uploads and repacks the weight on every call; callers that reuse a weight should hold a
 * gllmk_weight and call gllmk_matmul_host.  UNSUPPORTED for a type of the other family
 * (the reference panics there, src/cpu_kernels/mod.rs:3335-3352). */
GLLMK_API int32_t gllmk_kquant_matmul_f32(gllmk_ctx ctx, const uint8_t *weight_blocks, const float *input, float *output,
                                int32_t quant_type, size_t m, size_t n, size_t k);
GLLMK_API int32_t gllmk_classic_matmul_f32(gllmk_ctx ctx, const uint8_t *weight_blocks, const float *input, float *output,
                                 int32_t quant_type, size_t m, size_t n, size_t k);
/* Kernels::gemm_q4 with E = f32 (src/traits.rs:511-520; src/cpu_kernels/mod.rs:2934-2981):
 * m batch rows, n output features, Q4_K rows of k/256 blocks, input [m, k], output [m, n],
 * scales: n_scales == n per channel, == 1 per tensor, else none.  INVALID_ARG if k % 256 != 0
 * (the reference asserts). */
GLLMK_API int32_t gllmk_gemm_q4_f32(gllmk_ctx ctx, const uint8_t *weight, const float *input, float *output,
                          const float *scales, size_t n_scales, size_t m, size_t n, size_t k);
/* Kernels::gemm_q8 with E = f32 (src/traits.rs:502-510; src/cpu_kernels/mod.rs:2983-3031): the same call over
 * Q8_K rows (`weight` is the reference's &[i8] view of 292-byte BlockQ8K blocks, k / 256 per row). */
GLLMK_API int32_t gllmk_gemm_q8_f32(gllmk_ctx ctx, const int8_t *weight, const float *input, float *output,
                          const float *scales, size_t n_scales, size_t m, size_t n, size_t k);
/* Kernels::gemv_q4 / gemv_q8 (src/traits.rs:500-501; src/cpu_kernels/mod.rs:2888-2932): ONE weight row of n
 * elements (n / 256 Q4_K or Q8_K blocks) dotted with input [n], times `scale`, into *out.  INVALID_ARG if
 * n % 256 != 0 (the reference asserts). */
GLLMK_API int32_t gllmk_gemv_q4_f32(gllmk_ctx ctx, const uint8_t *weight, const float *input, float scale, size_t n, float *out);
GLLMK_API int32_t gllmk_gemv_q8_f32(gllmk_ctx ctx, const int8_t *weight, const float *input, float scale, size_t n, float *out);
/* The same two conventions against a resident weight; x / y are HOST memory.
 * `ref_layout` != 0: kquant_matmul's input [k, m] / output [n, m]; 0: gemm_q4's [m, k] / [m, n]. */
GLLMK_API int32_t gllmk_matmul_host(gllmk_ctx ctx, gllmk_weight w, const float *x_host, int32_t m, float *y_host,
                          int32_t ref_layout);
/* The products of one decode step in ONE call: product i is gllmk_matmul_host(weights[i], x_host[i], m[i], y_host[i]).  All
 * of them are enqueued back to back on the context's stream, every activation is uploaded and every result downloaded on
 * a second stream beside the products (page-locked host buffers in place, pageable ones through the context's
 * page-locked staging area), and the call waits once, at the end.  An argument list (handles, host pointers, m) that is
 * passed twice in a row is captured as a CUDA graph and replayed on later calls with the same list: one launch per step
 * (gllmk_ctx_set "host_batch_graph" = 0 switches the replay off).  Outputs must not alias inputs of the same call.
 * No counterpart in the reference (its products are synchronous CPU calls). */
GLLMK_API int32_t gllmk_matmul_host_batch(gllmk_ctx ctx, int32_t count, const gllmk_weight *weights, const float *const *x_host,
                                          const int32_t *m, float *const *y_host, int32_t ref_layout);
/* Kernels::dequant_q4_k(block, out) / dequant_q8_0 (src/traits.rs:476,488): `nblocks` consecutive
 * blocks -> nblocks*block_size f32, host pointers. */
GLLMK_API int32_t gllmk_dequant_q4_k(gllmk_ctx ctx, const uint8_t *blocks, float *out, size_t nblocks);
GLLMK_API int32_t gllmk_dequant_q8_0(gllmk_ctx ctx, const uint8_t *blocks, float *out, size_t nblocks);
/* quant_mxfp4::dequant_mxfp4(blocks, scales, output, block_size) (src/quant_mxfp4.rs:267-292):
 * any even block_size; host pointers; INVALID_ARG where the reference returns Err / asserts. */
GLLMK_API int32_t gllmk_dequant_mxfp4(gllmk_ctx ctx, const uint8_t *blocks, const uint8_t *scales, float *out,
                            size_t num_blocks, size_t block_size);
/* NVFP4 decode of `nblocks` 36-byte blocks, formula of src/quant.rs:77-86 (host pointers). */
GLLMK_API int32_t gllmk_dequant_nvfp4(gllmk_ctx ctx, const uint8_t *blocks, float global_scale, float *out, size_t nblocks);
/* Kernels::dequant_q6_k / dequant_q5_k / dequant_q8_k / dequant_q4_0 / dequant_q5_0 (src/traits.rs, the dequant_*
 * family; scalar decoders src/macros/quant_primitive/k_quant.rs:92-101,381-472, classic.rs:15-29,484-504) behind one
 * entry point: `quant_type` is one of GLLMK_QUANT_Q6_K .. GLLMK_QUANT_Q8_K (Q4_K and Q8_0 are accepted too);
 * `nblocks` consecutive blocks -> nblocks*block_size f32, host pointers, bit-exact with the scalar decoders. */
GLLMK_API int32_t gllmk_dequant_gguf(gllmk_ctx ctx, int32_t quant_type, const uint8_t *blocks, float *out, size_t nblocks);

/* ---- on-device quantizers ------------------------------------------------------------------ */

/* f32 [rows, k] (device) -> reference-format blocks (device).  The reference has no encoder for
 * these formats (its only quantizer is per-tensor amax/127, src/compiler/quant_convert.rs:17-31);
 * these are this library's own, used for NVFP4 activations and to make synthetic weights.
 * MXFP4 writes the split form (blocks + scales).  NVFP4: *global_scale > 0 is used as given,
 * otherwise amax/(6*448) of the whole input is computed, used and written back. */
GLLMK_API int32_t gllmk_quantize(gllmk_ctx ctx, int32_t quant_type, const float *x_dev, int64_t rows, int64_t k,
                       int32_t mx_block, void *blocks_dev, void *scales_dev, float *global_scale, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* GLLMK_H */
