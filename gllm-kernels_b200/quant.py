"""Format metadata of the formats the library serves (mirror of src/quant.rs:8-87,375-456)."""
from __future__ import annotations

import struct
from dataclasses import dataclass

# ids of include/gllmk.h
Q4K, Q8_0, MXFP4, NVFP4 = 1, 2, 3, 4
Q6K, Q5K, Q4_0, Q5_0, Q8K = 6, 7, 8, 9, 10

_BS = {Q4K: 256, Q8_0: 32, NVFP4: 64, Q6K: 256, Q5K: 256, Q8K: 256, Q4_0: 32, Q5_0: 32}
_BB = {Q4K: 144, Q8_0: 34, NVFP4: 36, Q6K: 210, Q5K: 176, Q8K: 292, Q4_0: 18, Q5_0: 22}
_BITS = {Q4K: 4, Q8_0: 8, MXFP4: 4, NVFP4: 4, Q6K: 6, Q5K: 5, Q8K: 8, Q4_0: 4, Q5_0: 5}
_NAME = {Q4K: "Q4K", Q8_0: "Q8_0", NVFP4: "Nvfp4", Q6K: "Q6K", Q5K: "Q5K", Q8K: "Q8K", Q4_0: "Q4_0", Q5_0: "Q5_0"}

# src/quant.rs:90-93
QK_K = 256
K_SCALE_SIZE = 12
QK_NVFP4 = 64
QK_NVFP4_SUB = 16

# src/quant_mxfp4.rs:33-35
E2M1_LUT_F32 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


def decode_e8m0_scale(byte: int) -> float:
    """src/quant_mxfp4.rs:43-54: 2^(byte-127); 0 -> 2^-127 (f32 subnormal), 255 -> NaN."""
    byte &= 0xFF
    if byte == 255:
        return float("nan")
    bits = 0x00400000 if byte == 0 else byte << 23
    return struct.unpack("<f", struct.pack("<I", bits))[0]


@dataclass(frozen=True)
class QuantType:
    """One of QuantType::{Q4K, Q8_0, Mxfp4{block_size}, Nvfp4, Q6K, Q5K, Q4_0, Q5_0, Q8K}."""
    id: int
    mx_block: int = 0

    @staticmethod
    def q4k() -> "QuantType":
        return QuantType(Q4K)

    @staticmethod
    def q8_0() -> "QuantType":
        return QuantType(Q8_0)

    @staticmethod
    def mxfp4(block_size: int = 32) -> "QuantType":
        return QuantType(MXFP4, block_size)

    @staticmethod
    def nvfp4() -> "QuantType":
        return QuantType(NVFP4)

    @staticmethod
    def q6k() -> "QuantType":
        return QuantType(Q6K)

    @staticmethod
    def q5k() -> "QuantType":
        return QuantType(Q5K)

    @staticmethod
    def q8k() -> "QuantType":
        return QuantType(Q8K)

    @staticmethod
    def q4_0() -> "QuantType":
        return QuantType(Q4_0)

    @staticmethod
    def q5_0() -> "QuantType":
        return QuantType(Q5_0)

    def block_size(self) -> int:  # src/quant.rs:375-397
        return self.mx_block if self.id == MXFP4 else _BS[self.id]

    def block_bytes(self) -> int:  # src/quant.rs:399-431
        return 1 + self.mx_block // 2 if self.id == MXFP4 else _BB[self.id]

    def bits(self) -> int:  # src/quant.rs:433-456
        return _BITS[self.id]

    @property
    def name(self) -> str:
        return f"Mxfp4{{{self.mx_block}}}" if self.id == MXFP4 else _NAME[self.id]


# ---- QuantFormatDescriptor (src/quant_format.rs:129-157) -------------------------------------------------------
# Enum variant names of the reference, indexed by the integers of include/gllmk.h.
SCALE_KINDS = ("None", "BlockScalar", "BlockScalarWithMin", "Hierarchical", "Q6KScales", "ExternalArray", "SubBlockScalars")
ZERO_KINDS = ("None", "BlockScalar", "Hierarchical", "StaticBias", "BlockMin")
DATA_LAYOUTS = ("PackedNibbles", "NibbleWithHighBits", "Bytes")
SCALE_DTYPES = ("F16", "F32", "BF16", "U8Range", "I8Range", "F8E4M3", "F8E5M2", "E8M0")
DATA_KINDS = ("Int8", "PackedInt4", "SignedPackedInt4", "PackedInt5", "PackedInt6", "Float4", "Nvfp4")
STORAGE_LAYOUTS = ("RowMajor", "ColInterleaved", "Packed")
NATIVE_ISAS = (None, "Vpdpbusd", "Tcgen05Fp4")
_DESC_FIELDS = ("quant_type", "block_size", "block_bytes", "bits_per_element", "scale_kind", "scale_dtype", "scale_offset",
                "scale_min_offset", "sub_scales_offset", "sub_scales_bits", "sub_scales_count", "sub_block_elements", "zero_kind",
                "zero_offset", "zero_sub_offset", "static_bias", "data_layout", "data_offset", "data_high_offset", "data_high_bits",
                "data_low_first", "data_signed", "data_kind", "storage_layout", "native_isa")
_DESC_NAME = {Q4K: "Q4_K", Q8_0: "Q8_0", MXFP4: "MXFP4", NVFP4: "NVFP4", Q6K: "Q6_K", Q5K: "Q5_K", Q4_0: "Q4_0", Q5_0: "Q5_0", Q8K: "Q8_K"}


@dataclass(frozen=True)
class QuantFormatDescriptor:
    """Where a block of a format keeps its scales, zero point / min and data — the reference's descriptor, read from
    the table the library's own kernels use (gllmk_quant_format_descriptor_for_type).  Offsets are bytes from the
    start of the block; -1 = the format has no such field.  The `*_kind` / `*_layout` / dtype / isa fields are the
    reference's enum variant names."""
    name: str
    quant_type: QuantType
    block_size: int
    block_bytes: int
    bits_per_element: int
    scale_kind: str
    scale_dtype: str
    scale_offset: int
    scale_min_offset: int
    sub_scales_offset: int
    sub_scales_bits: int
    sub_scales_count: int
    sub_block_elements: int
    zero_kind: str
    zero_offset: int
    zero_sub_offset: int
    static_bias: int
    data_layout: str
    data_offset: int
    data_high_offset: int
    data_high_bits: int
    data_low_first: bool
    data_signed: bool
    data_kind: str
    storage_layout: str
    native_isa: object

    @staticmethod
    def for_type(quant_type: QuantType) -> "QuantFormatDescriptor":
        """QuantFormatDescriptor::for_type (src/quant_format.rs:36-44).  Raises for a type the library does not serve
        (the reference panics for an unregistered type)."""
        import ctypes as C
        from ._lib import GllmkError, lib
        raw = (C.c_int32 * len(_DESC_FIELDS))()
        rc = lib().gllmk_quant_format_descriptor_for_type(quant_type.id, quant_type.mx_block or 32, raw)
        if rc:
            raise GllmkError(rc, "QuantFormatDescriptor.for_type", f"no descriptor registered for quant type {quant_type.id}")
        v = dict(zip(_DESC_FIELDS, raw))
        return QuantFormatDescriptor(
            name=_DESC_NAME[v["quant_type"]], quant_type=quant_type, block_size=v["block_size"], block_bytes=v["block_bytes"],
            bits_per_element=v["bits_per_element"], scale_kind=SCALE_KINDS[v["scale_kind"]], scale_dtype=SCALE_DTYPES[v["scale_dtype"]],
            scale_offset=v["scale_offset"], scale_min_offset=v["scale_min_offset"], sub_scales_offset=v["sub_scales_offset"],
            sub_scales_bits=v["sub_scales_bits"], sub_scales_count=v["sub_scales_count"], sub_block_elements=v["sub_block_elements"],
            zero_kind=ZERO_KINDS[v["zero_kind"]], zero_offset=v["zero_offset"], zero_sub_offset=v["zero_sub_offset"],
            static_bias=v["static_bias"], data_layout=DATA_LAYOUTS[v["data_layout"]], data_offset=v["data_offset"],
            data_high_offset=v["data_high_offset"], data_high_bits=v["data_high_bits"], data_low_first=bool(v["data_low_first"]),
            data_signed=bool(v["data_signed"]), data_kind=DATA_KINDS[v["data_kind"]], storage_layout=STORAGE_LAYOUTS[v["storage_layout"]],
            native_isa=NATIVE_ISAS[v["native_isa"]])


def registry() -> dict:
    """registry() (src/quant_format.rs:1189-1193) restricted to the served formats: {format name: descriptor}."""
    import ctypes as C
    from ._lib import lib
    ids = (C.c_int32 * 32)()
    n = lib().gllmk_quant_format_registry(ids, 32)
    out = {}
    for i in range(n):
        qt = QuantType(ids[i], 32 if ids[i] == MXFP4 else 0)
        d = QuantFormatDescriptor.for_type(qt)
        out[d.name] = d
    return out
