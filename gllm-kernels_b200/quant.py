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
