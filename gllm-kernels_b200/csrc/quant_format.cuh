// QuantFormatDescriptor of the reference (src/quant_format.rs:129-157) for the nine formats this library serves:
// where a block keeps its scale(s), its zero point / min and its quantized data.  The table below is the single
// source of those byte offsets on the device side: the repack kernels (repack.cu), the bit-exact decoders
// (repack.cu, gguf_raw.cu) and the raw-block GEMV read them from here, and gllmk_quant_format_descriptor hands the
// same table to the host (the Python mirror QuantFormatDescriptor.for_type / registry()).
// Values transcribed from the reference's registry: Q4_0 / Q5_0 / Q8_0 src/quant_format.rs:354-476,
// Q4_K / Q5_K / Q6_K / Q8_K :508-682, MXFP4 :982-1001, NVFP4 :1007-1027.
#pragma once
#include "../../include/gllmk.h"

namespace gllmk {

// The descriptor is the public C struct (include/gllmk.h); -1 marks a field the format does not have.
constexpr gllmk_quant_format_descriptor quant_format(int qt, int mx_block = 32) {
    gllmk_quant_format_descriptor d{};
    d.quant_type = qt;
    d.scale_offset = d.scale_min_offset = d.sub_scales_offset = -1;
    d.sub_scales_bits = d.sub_scales_count = d.sub_block_elements = 0;
    d.zero_offset = d.zero_sub_offset = -1;
    d.static_bias = 0;
    d.data_offset = d.data_high_offset = -1;
    d.data_high_bits = 0;
    d.data_low_first = d.data_signed = 0;
    d.storage_layout = GLLMK_STORAGE_ROW_MAJOR;
    d.native_isa = GLLMK_ISA_NONE;
    switch (qt) {
        case GLLMK_QUANT_Q4_0:  // d f16 @0 | qs[16] @2, nibble - 8
            d.block_size = 32; d.block_bytes = 18; d.bits_per_element = 4;
            d.scale_kind = GLLMK_SCALE_BLOCK_SCALAR; d.scale_dtype = GLLMK_SDT_F16; d.scale_offset = 0;
            d.zero_kind = GLLMK_ZERO_STATIC_BIAS; d.static_bias = 8;
            d.data_layout = GLLMK_DATA_PACKED_NIBBLES; d.data_offset = 2; d.data_low_first = 1;
            d.data_kind = GLLMK_KIND_SIGNED_PACKED_INT4;
            break;
        case GLLMK_QUANT_Q5_0:  // d f16 @0 | qh[4] @2 | qs[16] @6, q - 16
            d.block_size = 32; d.block_bytes = 22; d.bits_per_element = 5;
            d.scale_kind = GLLMK_SCALE_BLOCK_SCALAR; d.scale_dtype = GLLMK_SDT_F16; d.scale_offset = 0;
            d.zero_kind = GLLMK_ZERO_STATIC_BIAS; d.static_bias = 16;
            d.data_layout = GLLMK_DATA_NIBBLE_WITH_HIGH_BITS; d.data_offset = 6; d.data_high_offset = 2; d.data_high_bits = 1;
            d.data_kind = GLLMK_KIND_PACKED_INT5;
            break;
        case GLLMK_QUANT_Q8_0:  // d f16 @0 | qs[32] i8 @2
            d.block_size = 32; d.block_bytes = 34; d.bits_per_element = 8;
            d.scale_kind = GLLMK_SCALE_BLOCK_SCALAR; d.scale_dtype = GLLMK_SDT_F16; d.scale_offset = 0;
            d.zero_kind = GLLMK_ZERO_NONE;
            d.data_layout = GLLMK_DATA_BYTES; d.data_offset = 2; d.data_signed = 1;
            d.data_kind = GLLMK_KIND_INT8; d.native_isa = GLLMK_ISA_VPDPBUSD;
            break;
        case GLLMK_QUANT_Q4K:  // d f16 @0 | dmin f16 @2 | scales[12] 6-bit x 8 (sc, m) @4 | qs[128] @16
            d.block_size = 256; d.block_bytes = 144; d.bits_per_element = 4;
            d.scale_kind = GLLMK_SCALE_HIERARCHICAL; d.scale_dtype = GLLMK_SDT_F16; d.scale_offset = 0; d.scale_min_offset = 2;
            d.sub_scales_offset = 4; d.sub_scales_bits = 6; d.sub_scales_count = 8; d.sub_block_elements = 32;
            d.zero_kind = GLLMK_ZERO_HIERARCHICAL; d.zero_offset = 2; d.zero_sub_offset = 4;
            d.data_layout = GLLMK_DATA_PACKED_NIBBLES; d.data_offset = 16; d.data_low_first = 1;
            d.data_kind = GLLMK_KIND_PACKED_INT4;
            break;
        case GLLMK_QUANT_Q5_K:  // d @0 | dmin @2 | scales[12] @4 | qh[32] @16 | qs[128] @48
            d.block_size = 256; d.block_bytes = 176; d.bits_per_element = 5;
            d.scale_kind = GLLMK_SCALE_HIERARCHICAL; d.scale_dtype = GLLMK_SDT_F16; d.scale_offset = 0; d.scale_min_offset = 2;
            d.sub_scales_offset = 4; d.sub_scales_bits = 6; d.sub_scales_count = 8; d.sub_block_elements = 32;
            d.zero_kind = GLLMK_ZERO_HIERARCHICAL; d.zero_offset = 2; d.zero_sub_offset = 4;
            d.data_layout = GLLMK_DATA_NIBBLE_WITH_HIGH_BITS; d.data_offset = 48; d.data_high_offset = 16; d.data_high_bits = 1;
            d.data_kind = GLLMK_KIND_PACKED_INT5;
            break;
        case GLLMK_QUANT_Q6_K:  // ql[128] @0 | qh[64] @128 | scales[16] i8 @192 | d f16 @208, q - 32
            d.block_size = 256; d.block_bytes = 210; d.bits_per_element = 6;
            d.scale_kind = GLLMK_SCALE_Q6K_SCALES; d.scale_dtype = GLLMK_SDT_F16; d.scale_offset = 208;
            d.sub_scales_offset = 192; d.sub_scales_bits = 8; d.sub_scales_count = 16; d.sub_block_elements = 16;
            d.zero_kind = GLLMK_ZERO_STATIC_BIAS; d.static_bias = 32;
            d.data_layout = GLLMK_DATA_NIBBLE_WITH_HIGH_BITS; d.data_offset = 0; d.data_high_offset = 128; d.data_high_bits = 2;
            d.data_kind = GLLMK_KIND_PACKED_INT6;
            break;
        case GLLMK_QUANT_Q8_K:  // d f32 @0 | qs[256] i8 @4 | bsums[16] i16 @260
            d.block_size = 256; d.block_bytes = 292; d.bits_per_element = 8;
            d.scale_kind = GLLMK_SCALE_BLOCK_SCALAR; d.scale_dtype = GLLMK_SDT_F32; d.scale_offset = 0;
            d.zero_kind = GLLMK_ZERO_NONE;
            d.data_layout = GLLMK_DATA_BYTES; d.data_offset = 4; d.data_signed = 1;
            d.data_kind = GLLMK_KIND_INT8; d.native_isa = GLLMK_ISA_VPDPBUSD;
            break;
        case GLLMK_QUANT_MXFP4:  // E8M0 scale @0 | packed E2M1 @1 (inline GGUF form; the split API form keeps the scales apart)
            d.block_size = mx_block; d.block_bytes = 1 + mx_block / 2; d.bits_per_element = 4;
            d.scale_kind = GLLMK_SCALE_BLOCK_SCALAR; d.scale_dtype = GLLMK_SDT_E8M0; d.scale_offset = 0;
            d.zero_kind = GLLMK_ZERO_NONE;
            d.data_layout = GLLMK_DATA_PACKED_NIBBLES; d.data_offset = 1; d.data_low_first = 1;
            d.data_kind = GLLMK_KIND_FLOAT4;
            break;
        case GLLMK_QUANT_NVFP4:  // 4 x UE4M3 (one per 16 elements) @0 | packed E2M1 @4
            d.block_size = 64; d.block_bytes = 36; d.bits_per_element = 4;
            d.scale_kind = GLLMK_SCALE_SUB_BLOCK_SCALARS; d.scale_dtype = GLLMK_SDT_F8E4M3; d.scale_offset = 0;
            d.sub_scales_offset = 0; d.sub_scales_bits = 8; d.sub_scales_count = 4; d.sub_block_elements = 16;
            d.zero_kind = GLLMK_ZERO_NONE;
            d.data_layout = GLLMK_DATA_PACKED_NIBBLES; d.data_offset = 4; d.data_low_first = 1;
            d.data_kind = GLLMK_KIND_NVFP4; d.native_isa = GLLMK_ISA_TCGEN05_FP4;
            break;
        default:
            d.quant_type = 0;
            d.block_size = d.block_bytes = d.bits_per_element = 0;
            break;
    }
    return d;
}

// compile-time instances the kernels read their offsets from
constexpr gllmk_quant_format_descriptor FD_Q4K = quant_format(GLLMK_QUANT_Q4K), FD_Q8_0 = quant_format(GLLMK_QUANT_Q8_0),
                                        FD_MXFP4 = quant_format(GLLMK_QUANT_MXFP4, 32), FD_NVFP4 = quant_format(GLLMK_QUANT_NVFP4),
                                        FD_Q6K = quant_format(GLLMK_QUANT_Q6_K), FD_Q5K = quant_format(GLLMK_QUANT_Q5_K),
                                        FD_Q8K = quant_format(GLLMK_QUANT_Q8_K), FD_Q4_0 = quant_format(GLLMK_QUANT_Q4_0),
                                        FD_Q5_0 = quant_format(GLLMK_QUANT_Q5_0);

}  // namespace gllmk
