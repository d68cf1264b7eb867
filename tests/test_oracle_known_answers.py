"""Pins the CPU oracle to the known-answer vectors of the reference's own tests.

The vectors live in tests/golden/reference_known_answers.json (written by
tests/golden/make_known_answers.py from the reference's test sources, cited per case).
"""
import json
import math
import os
import struct

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(HERE, "golden", "reference_known_answers.json")) as f:
    KA = json.load(f)


def bits(f):
    return struct.unpack("<I", struct.pack("<f", f))[0]


def test_q4k_decode_basic(oracle):
    c = KA["q4k_decode_basic"]
    out = oracle.dequant_q4_k(c["block"])
    for i, v in c["expect"].items():
        assert out[int(i)] == v


def test_q4k_decode_all_subblocks(oracle):
    c = KA["q4k_decode_all_subblocks"]
    out = oracle.dequant_q4_k(c["block"])
    assert out.tolist() == c["expect_all"]
    sc, m = oracle.q4k_scales(c["block"])
    assert sc.tolist() == c["expect_scales"] and m.tolist() == c["expect_mins"]
    blk = np.array(c["block"], np.uint8)
    import ctypes as C
    for e in range(256):  # element-indexed form of the same decode
        got = oracle.lib().gko_q4k_element(blk.ctypes.data_as(C.POINTER(C.c_uint8)), e)
        assert got == c["expect_all"][e]


@pytest.mark.parametrize("name", ["gemm_q4_basic", "gemm_q4_per_channel"])
def test_gemm_q4(oracle, name):
    c = KA[name]
    out = oracle.gemm_q4(c["weight"], c["input"], c["scales"], c["m"], c["n"], c["k"])
    assert out.reshape(-1).tolist() == c["expect"]


def test_q8_0_decode(oracle):
    c = KA["q8_0_decode_basic"]
    out = oracle.dequant_q8_0(c["block"])
    for i, v in c["expect"].items():
        assert out[int(i)] == v
    c = KA["q8_0_decode_extreme"]
    assert oracle.dequant_q8_0(c["block"]).tolist() == c["expect_all"]


def test_q8_0_dot_via_classic_matmul(oracle):
    c = KA["q8_0_dot"]
    out = oracle.quant_matmul(c["weight"], c["input"], oracle.Q8_0, c["m"], c["n"], c["k"])
    assert out.reshape(-1).tolist() == c["expect"]


@pytest.mark.parametrize("name", sorted(KA["mxfp4"].keys()))
def test_mxfp4_known_answers(oracle, name):
    c = KA["mxfp4"][name]
    out = oracle.dequant_mxfp4(c["blocks"], c["scales"], c["block_size"])
    if c.get("expect_all_nan"):
        assert np.isnan(out).all()
    else:
        exp = np.array(c["expect"], np.float32)
        assert out.shape == exp.shape
        # bit-exact, including the sign of zero
        assert (out.view(np.uint32) == exp.view(np.uint32)).all()


def test_e2m1_and_e8m0(oracle):
    lut = KA["e2m1_lut"]["values"]
    for i, v in enumerate(lut):
        assert bits(oracle.lib().gko_e2m1(i)) == bits(v)
    for b, u in KA["e8m0_bits"]["byte_to_f32_bits"].items():
        assert bits(oracle.lib().gko_decode_e8m0_scale(int(b))) == u
    assert math.isnan(oracle.lib().gko_decode_e8m0_scale(KA["e8m0_bits"]["nan_byte"]))


def test_metadata(oracle):
    md = KA["metadata"]
    L = oracle.lib()
    assert [L.gko_block_size(oracle.Q4K, 0), L.gko_block_bytes(oracle.Q4K, 0)] == md["q4k"]
    assert [L.gko_block_size(oracle.Q8_0, 0), L.gko_block_bytes(oracle.Q8_0, 0)] == md["q8_0"]
    assert [L.gko_block_size(oracle.MXFP4, 32), L.gko_block_bytes(oracle.MXFP4, 32)] == md["mxfp4_32"]
    assert [L.gko_block_size(oracle.NVFP4, 0), L.gko_block_bytes(oracle.NVFP4, 0)] == md["nvfp4"]


def test_f16_codec_against_numpy(oracle):
    L = oracle.lib()
    allh = np.arange(65536, dtype=np.uint16)
    ref = allh.view(np.float16).astype(np.float32)
    for h in range(0, 65536, 7):
        got = L.gko_f16_to_f32(h)
        assert bits(got) == int(ref[h:h + 1].view(np.uint32)[0]) or (math.isnan(got) and np.isnan(ref[h]))
    rng = np.random.default_rng(1)
    xs = np.concatenate([rng.standard_normal(4000).astype(np.float32) * 10.0 ** rng.integers(-9, 6, 4000),
                         np.array([0, -0.0, 65504, 65519.99, 65520, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8, np.inf],
                                  np.float32)]).astype(np.float32)
    want = xs.astype(np.float16).view(np.uint16)
    for x, w in zip(xs.tolist(), want.tolist()):
        assert L.gko_f32_to_f16(x) == w, x


def test_e4m3_codec_against_torch(oracle):
    """OCP E4M3 decode of all 256 bytes equals torch.float8_e4m3fn; encode round-trips every code."""
    import torch
    L = oracle.lib()
    allb = torch.arange(256, dtype=torch.uint8)
    ref = allb.view(torch.float8_e4m3fn).to(torch.float32).numpy()
    for b in range(256):
        got = L.gko_e4m3_to_f32(b)
        if math.isnan(ref[b]):
            assert math.isnan(got)
        else:
            assert bits(got) == bits(float(ref[b]))
            if (b & 0x7F) != 0 or b == 0:
                assert L.gko_f32_to_e4m3(float(ref[b])) == b
    assert L.gko_f32_to_e4m3(1000.0) == 0x7E  # saturates to 448
    assert L.gko_e4m3_to_f32(0x7E) == 448.0


# ---- the other GGUF formats (Q6_K, Q5_K, Q8_K, Q4_0, Q5_0) ------------------------------------
def _qt(oracle, name):
    return {"q6_k": oracle.Q6K, "q5_k": oracle.Q5K, "q8_k": oracle.Q8K, "q4_0": oracle.Q4_0, "q5_0": oracle.Q5_0}[name]


GGUF_DECODE_CASES = ["q8_k_decode", "q5_k_decode", "q6_k_decode", "q4_0_decode_zero", "q4_0_decode_known",
                     "q4_0_decode_full_range", "q5_0_decode", "q5_0_decode_all_bits"]


@pytest.mark.parametrize("name", GGUF_DECODE_CASES)
def test_gguf_decode_known_answers(oracle, name):
    c = KA[name]
    out = oracle.dequant_block(_qt(oracle, c["qt"]), c["block"])
    if "expect_all" in c:
        assert out.tolist() == c["expect_all"]
    for i, v in c.get("expect", {}).items():
        assert out[int(i)] == v


@pytest.mark.parametrize("name", ["q4_0_dot", "q5_0_dot", "q8_k_matmul"])
def test_gguf_matmul_known_answers(oracle, name):
    c = KA[name]
    out = oracle.quant_matmul(c["weight"], c["input"], _qt(oracle, c["qt"]), c["m"], c["n"], c["k"])
    assert out.reshape(-1).tolist() == c["expect"]


def test_gguf_metadata(oracle):
    c = KA["metadata_gguf"]
    for name in ("q6_k", "q5_k", "q8_k", "q4_0", "q5_0"):
        qt = _qt(oracle, name)
        assert [oracle.lib().gko_block_size(qt, 0), oracle.lib().gko_block_bytes(qt, 0)] == c[name]


@pytest.mark.parametrize("name", ["q6_k", "q5_k", "q8_k", "q4_0", "q5_0"])
def test_gguf_dot_is_decode_then_dot(oracle, name):
    """The block dot of each format equals the f32 dot with its own decode, term by term in element order
    (Q6_K and Q5_K visit elements in the order of their decode loops), so both agree to rounding."""
    qt = _qt(oracle, name)
    bs, bb = oracle.lib().gko_block_size(qt, 0), oracle.lib().gko_block_bytes(qt, 0)
    rng = np.random.default_rng(5)
    nb = 4
    w = rng.integers(0, 256, size=(nb, bb), dtype=np.uint8)
    for b in range(nb):  # finite scales
        if name == "q8_k":
            w[b, 0:4] = np.frombuffer(struct.pack("<f", 0.01 * (b + 1)), np.uint8)
        elif name == "q6_k":
            w[b, 208:210] = np.frombuffer(struct.pack("<e", 0.01 * (b + 1)), np.uint8)
        else:
            w[b, 0:2] = np.frombuffer(struct.pack("<e", 0.01 * (b + 1)), np.uint8)
            if name == "q5_k":
                w[b, 2:4] = np.frombuffer(struct.pack("<e", 0.02), np.uint8)
    x = rng.standard_normal(nb * bs).astype(np.float32)
    y = oracle.quant_matmul(w.reshape(-1), x, qt, 1, 1, nb * bs)
    dec = np.concatenate([oracle.dequant_block(qt, w[b]) for b in range(nb)])
    ref = float(np.dot(dec.astype(np.float64), x.astype(np.float64)))
    assert abs(float(y[0, 0]) - ref) <= 1e-4 * max(1.0, abs(ref))


def test_moe_topk_and_weighted_sum_known_answers(oracle):
    """scalar-ops/src/moe.rs:178-217 (the reference's own tests), plus the conventions the restatement must keep."""
    c = KA["moe_topk"]
    out = oracle.scalar_topk(np.array(c["probs"], np.float32).reshape(c["seq_len"], c["num_experts"]), c["top_k"])
    assert out[0].view(np.uint32).tolist() == c["expect_indices"]  # indices are u32 bit patterns in f32 slots
    assert abs(out[1].sum() - c["weights_sum"]) < c["weights_sum_tol"]
    assert out[1].tolist() == [np.float32(0.5) * (np.float32(1.0) / (np.float32(0.5) + np.float32(0.3))),
                               np.float32(0.3) * (np.float32(1.0) / (np.float32(0.5) + np.float32(0.3)))]
    c = KA["moe_weighted_sum"]
    routing = np.concatenate([np.array(c["indices"], np.uint32).view(np.float32), np.array(c["weights"], np.float32)])
    got = oracle.scalar_weighted_sum(np.array(c["expert_outputs"], np.float32).reshape(1, c["seq_len"], c["hidden"]), routing,
                                     c["seq_len"], c["top_k"])
    assert got.reshape(-1).tolist() == c["expect"]
    # ties go to the earlier expert; a NaN probability is never selected; all-zero rows give zero weights
    out = oracle.scalar_topk(np.array([[0.25, 0.25, 0.25, 0.25], [np.nan, 0.2, 0.7, 0.1], [0, 0, 0, 0]], np.float32), 2)
    assert out[0].view(np.uint32).reshape(3, 2).tolist() == [[0, 1], [2, 1], [0, 1]]
    assert out[1].reshape(3, 2)[2].tolist() == [0.0, 0.0]
    # the grouped-row form of the recombination is the same sum as the reference's [expert][seq][hidden] form
    rng = np.random.default_rng(5)
    E, T, H, top_k = 4, 9, 7, 2
    routing = oracle.scalar_topk(rng.random((T, E), dtype=np.float32), top_k)
    eo = rng.standard_normal((E, T, H)).astype(np.float32)
    idx = routing[0].view(np.uint32).reshape(T, top_k)
    rows = np.stack([eo[idx[t, ki], t] for t in range(T) for ki in range(top_k)])
    a = oracle.scalar_weighted_sum(eo, routing, T, top_k)
    b = oracle.scalar_weighted_sum_grouped(rows, routing, np.arange(T * top_k), T, top_k)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_gemv_q8_gemm_q8_gemv_q4_known_answers(oracle):
    """src/tests_fragments/part2.inc.rs:161-232."""
    c = KA["gemv_q8"]
    assert abs(oracle.gemv_q8(np.array(c["weight"], np.uint8), c["input"], c["scale"], c["n"]) - c["expect"]) < c["tol"]
    c = KA["gemm_q8"]
    out = oracle.gemm_q8(np.array(c["weight"], np.uint8), np.array(c["input"], np.float32).reshape(c["m"], c["k"]), c["scales"],
                         c["m"], c["n"], c["k"])
    assert np.abs(out.reshape(-1) - np.array(c["expect"])).max() < c["tol"]
    c = KA["gemv_q4_zero"]
    assert abs(oracle.gemv_q4(np.array(c["weight"], np.uint8), c["input"], c["scale"], c["n"]) - c["expect"]) < c["tol"]


def test_int8_per_tensor_quantizer_rule(oracle):
    """src/compiler/quant_convert.rs:17-20,165-177: scale = max|x| / 127, round half away from zero, clamp to
    [-128, 127]; an all-zero tensor gives scale 0 and zeros."""
    x = np.array([0.0, 1.27, -1.27, 0.005, -0.005, 0.015, 0.635, -0.645], np.float32)
    q, s = oracle.quantize_int8_per_tensor(x)
    assert s == np.float32(1.27) / np.float32(127.0)
    want = np.clip(np.sign(x / np.float32(s)) * np.floor(np.abs(x / np.float32(s)) + np.float32(0.5)), -128, 127).astype(np.int8)
    assert q.tolist() == want.tolist() and q[1] == 127 and q[2] == -127
    q, s = oracle.quantize_int8_per_tensor(np.zeros(5, np.float32))
    assert s == 0.0 and not q.any()
