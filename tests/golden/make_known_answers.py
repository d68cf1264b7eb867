"""Writes tests/golden/reference_known_answers.json.

Each case restates, as data, a known-answer test that lives in the reference's own test
suite (gllm-kernels, file:line given per case).  The inputs are rebuilt here byte by byte the
way the reference test builds them; the expected values are the literals the reference test
asserts.  Nothing is computed by the oracle or by this project's kernels: the file pins them.

Run:  python tests/golden/make_known_answers.py
"""
import json
import os
import struct

HERE = os.path.dirname(os.path.abspath(__file__))


def f16(v: float) -> bytes:
    return struct.pack("<e", v)


def q4k_block(d, dmin, scales=None, qs=None) -> list:
    b = bytearray(144)
    b[0:2] = f16(d)
    b[2:4] = f16(dmin)
    for i, v in (scales or {}).items():
        b[4 + i] = v
    for i, v in (qs or {}).items():
        b[16 + i] = v
    return list(b)


def q8_0_block(d, qs) -> list:
    b = bytearray(34)
    b[0:2] = f16(d)
    for i, v in qs.items():
        b[2 + i] = v & 0xFF
    return list(b)


cases = {}

# src/tests_quant.rs:14-43  test_dequant_q4_k_scalar
cases["q4k_decode_basic"] = {
    "cite": "src/tests_quant.rs:14-43",
    "block": q4k_block(1.0, 0.5, {0: 2, 4: 4}, {0: 0x05, 1: 0x03}),
    "expect": {"0": 8.0, "1": 4.0, "2": -2.0},
}

# src/asm/x86_64/quant_gemv.rs:2481-2533  test_q4k_decode_step_native_vs_llamacpp
# (sc, m) = (1, 1) for all eight sub-blocks, incl. the j >= 4 branch; expected = d*sc*q - dmin*m.
blk = bytearray(144)
blk[0:2] = f16(1.0)
blk[2:4] = f16(1.0)
for i in range(4, 12):
    blk[i] = 1
for i in range(12, 16):
    blk[i] = 0x11
qs = [0x32] + [0x11] * 31 + [0x22] * 32 + [0x33] * 32 + [0x44] * 32
blk[16:144] = bytes(qs)
exp = []
for g in range(4):
    exp += [float((qs[32 * g + l] & 15) - 1) for l in range(32)]
    exp += [float((qs[32 * g + l] >> 4) - 1) for l in range(32)]
cases["q4k_decode_all_subblocks"] = {
    "cite": "src/asm/x86_64/quant_gemv.rs:2481-2533",
    "block": list(blk),
    "expect_all": exp,
    "expect_scales": [1] * 8,
    "expect_mins": [1] * 8,
}

# src/tests_quant.rs:177-226  test_gemm_q4   (m=2 batch, n=2 features, k=256, no scales)
row0 = q4k_block(1.0, 0.0, {0: 1}, {0: 0x05, 1: 0x03})
row1 = q4k_block(2.0, 0.0, {0: 1}, {0: 0x05, 1: 0x03})
inp = [0.0] * 512
for i in (0, 1, 256, 257):
    inp[i] = 1.0
cases["gemm_q4_basic"] = {
    "cite": "src/tests_quant.rs:177-226",
    "weight": row0 + row1, "input": inp, "scales": [], "m": 2, "n": 2, "k": 256,
    "expect": [8.0, 16.0, 8.0, 16.0],
}
# src/tests_quant.rs:766-808  gemm_q4 with per-channel scales 10, 0.5 on one batch row -> 20, 1
row0 = q4k_block(1.0, 0.0, {0: 1}, {0: 0x02})
row1 = q4k_block(1.0, 0.0, {0: 1}, {0: 0x02})
inp = [0.0] * 256
inp[0] = 1.0
cases["gemm_q4_per_channel"] = {
    "cite": "src/tests_quant.rs:766-808",
    "weight": row0 + row1, "input": inp, "scales": [10.0, 0.5], "m": 1, "n": 2, "k": 256,
    "expect": [20.0, 1.0],
}

# src/tests_quant.rs:437-455  test_dequant_q8_0
cases["q8_0_decode_basic"] = {
    "cite": "src/tests_quant.rs:437-455",
    "block": q8_0_block(0.5, {0: 10, 1: -20, 31: 127}),
    "expect": {"0": 5.0, "1": -10.0, "31": 63.5},
}
# src/tests_quant.rs:457-480  test_dequant_q8_0_extreme
cases["q8_0_decode_extreme"] = {
    "cite": "src/tests_quant.rs:457-480",
    "block": q8_0_block(1.0, {i: (-128 if i % 2 == 0 else 127) for i in range(32)}),
    "expect_all": [(-128.0 if i % 2 == 0 else 127.0) for i in range(32)],
}
# src/tests_quant.rs:645-677  test_dot_q8_0 through classic_matmul(m=1, n=1, k=32)
inp = [0.0] * 32
inp[0], inp[1] = 3.0, 2.0
cases["q8_0_dot"] = {
    "cite": "src/tests_quant.rs:645-677",
    "weight": q8_0_block(0.5, {0: 10, 1: -4}), "input": inp, "m": 1, "n": 1, "k": 32,
    "expect": [11.0],
}

LUT = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]
mx = {}
# src/quant_mxfp4.rs:306-338
mx["all_16_codewords"] = {
    "cite": "src/quant_mxfp4.rs:306-338", "block_size": 32,
    "blocks": [((15 - i) << 4) | i for i in range(16)], "scales": [127],
    "expect": [v for i in range(16) for v in (LUT[i], LUT[15 - i])],
}
# src/quant_mxfp4.rs:392-413
mx["two_blocks_distinct_scales"] = {
    "cite": "src/quant_mxfp4.rs:392-413", "block_size": 32,
    "blocks": [0x21] * 16 + [0x67] * 16, "scales": [128, 126],
    "expect": [1.0, 2.0] * 16 + [3.0, 2.0] * 16,
}
# src/quant_mxfp4.rs:576-596
mx["scale_124"] = {"cite": "src/quant_mxfp4.rs:576-596", "block_size": 32,
                   "blocks": [0x22] * 16, "scales": [124], "expect": [0.125] * 32}
mx["scale_130"] = {"cite": "src/quant_mxfp4.rs:576-596", "block_size": 32,
                   "blocks": [0x22] * 16, "scales": [130], "expect": [8.0] * 32}
# src/quant_mxfp4.rs:638-672
mx["scale_independence"] = {
    "cite": "src/quant_mxfp4.rs:638-672", "block_size": 32,
    "blocks": [0x12] * 32, "scales": [127, 129],
    "expect": [1.0, 0.5] * 16 + [4.0, 2.0] * 16,
}
# src/quant_mxfp4.rs:674-702
mx["block_size_16"] = {
    "cite": "src/quant_mxfp4.rs:674-702", "block_size": 16,
    "blocks": [((15 - i) << 4) | i for i in range(8)], "scales": [127],
    "expect": [v for i in range(8) for v in (LUT[i], LUT[15 - i])],
}
# src/quant_mxfp4.rs:705-732
mx["block_size_64"] = {"cite": "src/quant_mxfp4.rs:705-732", "block_size": 64,
                       "blocks": [0x43] * 32, "scales": [125], "expect": [0.375, 0.5] * 32}
# src/quant_mxfp4.rs:1055-1074
mx["block_size_2"] = {"cite": "src/quant_mxfp4.rs:1055-1074", "block_size": 2,
                      "blocks": [0x95], "scales": [127], "expect": [3.0, -0.5]}
# src/quant_mxfp4.rs:1079-1098
mx["all_zero_varying_scales"] = {"cite": "src/quant_mxfp4.rs:1079-1098", "block_size": 32,
                                 "blocks": [0] * 64, "scales": [120, 127, 135, 254], "expect": [0.0] * 128}
# src/quant_mxfp4.rs:735-751 (every output NaN)
mx["nan_scale"] = {"cite": "src/quant_mxfp4.rs:735-751", "block_size": 32,
                   "blocks": [0x12] * 16, "scales": [255], "expect_all_nan": True}
cases["mxfp4"] = mx

# src/quant_mxfp4.rs:33-35 (table), :368-390, :498-535, :943-984 (E8M0 values as f32 bit patterns)
cases["e2m1_lut"] = {"cite": "src/quant_mxfp4.rs:33-35,342-362", "values": LUT}
cases["e8m0_bits"] = {
    "cite": "src/quant_mxfp4.rs:368-390,498-535,969-984",
    "byte_to_f32_bits": {"0": 0x00400000, "1": 1 << 23, "125": 125 << 23, "126": 126 << 23, "127": 127 << 23,
                         "128": 128 << 23, "129": 129 << 23, "254": 254 << 23},
    "nan_byte": 255,
}

# src/quant.rs:399-431,552-628,677-757 (block_size / block_bytes of the four formats of the path)
cases["metadata"] = {
    "cite": "src/quant.rs:399-431,552-628,677-757",
    "q4k": [256, 144], "q8_0": [32, 34], "mxfp4_32": [32, 17], "nvfp4": [64, 36],
}

# ---- the other GGUF formats of the reference's CPU quant path -------------------------------
# block layouts: src/quant.rs:132-157 (Q5_K, Q6_K, Q8_K), :254-275 (Q4_0, Q5_0)


def q4_0_block(d, qs_fill=0x88, qs=None) -> list:
    b = bytearray(18)
    b[0:2] = f16(d)
    b[2:18] = bytes([qs_fill] * 16)
    for i, v in (qs or {}).items():
        b[2 + i] = v
    return list(b)


def q5_0_block(d, qh=None, qs=None) -> list:
    b = bytearray(22)
    b[0:2] = f16(d)
    for i, v in (qh or {}).items():
        b[2 + i] = v
    for i, v in (qs or {}).items():
        b[6 + i] = v
    return list(b)


def q8_k_block(d, qs) -> list:
    b = bytearray(292)
    b[0:4] = struct.pack("<f", d)
    for i, v in qs.items():
        b[4 + i] = v & 0xFF
    return list(b)


# src/tests_quant.rs:46-61  test_dequant_q8_k
cases["q8_k_decode"] = {"cite": "src/tests_quant.rs:46-61", "qt": "q8_k",
                        "block": q8_k_block(2.0, {0: 10, 1: -5}), "expect": {"0": 20.0, "1": -10.0}}

# src/tests_quant.rs:122-149  test_dequant_q5_k   (d @0, dmin @2, scales @4, qh @16, qs @48)
blk = bytearray(176)
blk[0:2] = f16(1.0)
blk[4] = 1
blk[48] = 0x0F
blk[16] = 0x01
blk[49] = 0x0F
blk[17] = 0x01
cases["q5_k_decode"] = {"cite": "src/tests_quant.rs:122-149", "qt": "q5_k", "block": list(blk),
                        "expect": {"0": 31.0, "1": 31.0}}

# src/tests_quant.rs:152-174  test_dequant_q6_k   (ql @0, qh @128, scales @192, d @208)
blk = bytearray(210)
blk[208:210] = f16(1.0)
blk[192] = 1
blk[0] = 0x0F
blk[128] = 0x03
cases["q6_k_decode"] = {"cite": "src/tests_quant.rs:152-174", "qt": "q6_k", "block": list(blk), "expect": {"0": 31.0}}

# src/tests_quant.rs:233-246  test_dequant_q4_0_zero
cases["q4_0_decode_zero"] = {"cite": "src/tests_quant.rs:233-246", "qt": "q4_0", "block": q4_0_block(1.0),
                             "expect_all": [0.0] * 32}
# src/tests_quant.rs:249-279  test_dequant_q4_0_known_values
exp = [0.0] * 32
exp[0], exp[1], exp[16], exp[17] = -3.0, 1.0, -3.5, 3.5
cases["q4_0_decode_known"] = {"cite": "src/tests_quant.rs:249-279", "qt": "q4_0",
                              "block": q4_0_block(0.5, qs={0: 0x12, 1: 0xFA}), "expect_all": exp}
# src/tests_quant.rs:282-320  test_dequant_q4_0_full_range
cases["q4_0_decode_full_range"] = {
    "cite": "src/tests_quant.rs:282-320", "qt": "q4_0",
    "block": q4_0_block(2.0, 0, {j: j | ((15 - j) << 4) for j in range(16)}),
    "expect_all": [2.0 * (j - 8.0) for j in range(16)] + [2.0 * ((15 - j) - 8.0) for j in range(16)],
}
# src/tests_quant.rs:364-387  test_dequant_q5_0 ; :390-408 test_dequant_q5_0_all_bits
cases["q5_0_decode"] = {"cite": "src/tests_quant.rs:364-387", "qt": "q5_0",
                        "block": q5_0_block(1.0, {0: 0x01}, {0: 0x0F}), "expect": {"0": 15.0, "16": -16.0}}
cases["q5_0_decode_all_bits"] = {"cite": "src/tests_quant.rs:390-408", "qt": "q5_0",
                                 "block": q5_0_block(0.5, {1: 0x01}, {8: 0x07}), "expect": {"8": 3.5}}

# matmul known answers (reference layout: weight rows m, batch columns n, input [k, n], output [m, n])
inp = [0.0] * 32
inp[0], inp[1] = 3.0, 4.0
# src/tests_quant.rs:508-539  test_dot_q4_0.  The test's comment takes the high nibble of byte 0 as element 1;
# the decoder puts it at element 16, where the input is 0: the product is 2*3 = 6 and the test's own
# tolerance check (|out - 10| < 1e-2) would not hold for the scalar decoder.  Recorded with the decoder's value.
cases["q4_0_dot"] = {"cite": "src/tests_quant.rs:508-539", "qt": "q4_0", "weight": q4_0_block(1.0, qs={0: 0x9A}),
                     "input": inp, "m": 1, "n": 1, "k": 32, "expect": [6.0], "note": "decoder value; see generator"}
inp = [0.0] * 32
inp[0] = 2.0
# src/tests_quant.rs:577-607  test_dot_q5_0
cases["q5_0_dot"] = {"cite": "src/tests_quant.rs:577-607", "qt": "q5_0",
                     "weight": q5_0_block(1.0, {0: 0x01}, {0: 0x05}), "input": inp, "m": 1, "n": 1, "k": 32, "expect": [10.0]}
# src/tests_fragments/part1.inc.rs:1011-1024  test_kquant_matmul_q8_k
cases["q8_k_matmul"] = {"cite": "src/tests_fragments/part1.inc.rs:1011-1024", "qt": "q8_k",
                        "weight": q8_k_block(1.0, {i: 1 for i in range(256)}), "input": [1.0] * 256,
                        "m": 1, "n": 1, "k": 256, "expect": [256.0]}

# src/quant.rs:375-456 block_size / block_bytes
cases["metadata_gguf"] = {"cite": "src/quant.rs:375-456",
                          "q6_k": [256, 210], "q5_k": [256, 176], "q8_k": [256, 292], "q4_0": [32, 18], "q5_0": [32, 22]}

# src/tests_fragments/part2.inc.rs:161-176 test_gemv_q8 and :214-232 test_gemm_q8: one Q8_K block d = 0.5, qs = 1, input = 1
# -> 128 (tolerance 1.0 in the reference)
cases["gemv_q8"] = {"cite": "src/tests_fragments/part2.inc.rs:161-176", "weight": q8_k_block(0.5, {i: 1 for i in range(256)}),
                    "input": [1.0] * 256, "scale": 1.0, "n": 256, "expect": 128.0, "tol": 1.0}
cases["gemm_q8"] = {"cite": "src/tests_fragments/part2.inc.rs:214-232", "weight": q8_k_block(0.5, {i: 1 for i in range(256)}),
                    "input": [1.0] * 512, "scales": [1.0], "m": 2, "n": 1, "k": 256, "expect": [128.0, 128.0], "tol": 1.0}
# src/tests_fragments/part2.inc.rs:178-188 test_gemv_q4: an all-zero Q4_K block -> |result| < 1
cases["gemv_q4_zero"] = {"cite": "src/tests_fragments/part2.inc.rs:178-188", "weight": [0] * 144, "input": [1.0] * 256, "scale": 1.0,
                         "n": 256, "expect": 0.0, "tol": 1.0}

# scalar-ops/src/moe.rs:178-192  test_topk_selects_largest: 1 row, 4 experts, top_k = 2 -> experts 1 then 2, weights sum 1
cases["moe_topk"] = {"cite": "scalar-ops/src/moe.rs:178-192", "probs": [0.1, 0.5, 0.3, 0.1], "seq_len": 1, "num_experts": 4,
                     "top_k": 2, "expect_indices": [1, 2], "weights_sum": 1.0, "weights_sum_tol": 1e-5}
# scalar-ops/src/moe.rs:194-217  test_weighted_sum_identity: one expert, weight 1 -> the expert's row
cases["moe_weighted_sum"] = {"cite": "scalar-ops/src/moe.rs:194-217", "expert_outputs": [1.0, 2.0, 3.0], "indices": [0],
                             "weights": [1.0], "seq_len": 1, "hidden": 3, "top_k": 1, "expect": [1.0, 2.0, 3.0]}

with open(os.path.join(HERE, "reference_known_answers.json"), "w") as f:
    json.dump(cases, f, indent=0)
print("wrote", len(cases), "groups")
