"""Format metadata of the four formats on the path (mirror of src/quant.rs:8-87,375-456)."""
from __future__ import annotations

import struct
from dataclasses import dataclass

# ids of include/gllmk.h
Q4K, Q8_0, MXFP4, NVFP4 = 1, 2, 3, 4

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
    """One of QuantType::{Q4K, Q8_0, Mxfp4{block_size}, Nvfp4}."""
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

    def block_size(self) -> int:  # src/quant.rs:375-397
        return {Q4K: 256, Q8_0: 32, MXFP4: self.mx_block, NVFP4: 64}[self.id]

    def block_bytes(self) -> int:  # src/quant.rs:399-431
        return {Q4K: 144, Q8_0: 34, MXFP4: 1 + self.mx_block // 2, NVFP4: 36}[self.id]

    def bits(self) -> int:  # src/quant.rs:433-456
        return {Q4K: 4, Q8_0: 8, MXFP4: 4, NVFP4: 4}[self.id]

    @property
    def name(self) -> str:
        return {Q4K: "Q4K", Q8_0: "Q8_0", MXFP4: f"Mxfp4{{{self.mx_block}}}", NVFP4: "Nvfp4"}[self.id]
