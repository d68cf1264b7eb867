"""Parity of the CUDA path (through the C ABI) with the CPU oracle.  Needs a B200.

Bars: repack round trip, decoded weights, quantizer bytes — bit-exact.  GEMV outputs —
max_i |y_i - ref_i| / max(|ref_i|, rms(ref)) <= 2e-3 against the oracle's sequential f32 sum.
"""
import json
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 2e-3
HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(HERE, "golden", "reference_known_answers.json")) as f:
    KA = json.load(f)


@pytest.fixture(scope="module")
def K(gk):
    k = gk.GpuKernels(0)
    yield k
    k.close()


@pytest.fixture(scope="module")
def torch():
    import torch as t
    assert t.cuda.is_available()
    return t


def same_bits(a, b):
    a = np.ascontiguousarray(a, np.float32).reshape(-1)
    b = np.ascontiguousarray(b, np.float32).reshape(-1)
    nan = np.isnan(a) & np.isnan(b)
    return bool(((a.view(np.uint32) == b.view(np.uint32)) | nan).all())


def make(oracle, fmt, n, k, seed, random_bytes=False):
    """Returns (quant_type_name, oracle id, blocks, scales, global)."""
    rng = np.random.default_rng(seed)
    W = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    if fmt == "q4k":
        b = oracle.quantize_q4_k(W)
        if random_bytes:
            b = rng.integers(0, 256, b.size, dtype=np.uint8)
            v = b.reshape(-1, 144)
            v[:, 0:4] = np.frombuffer(rng.uniform(-0.05, 0.05, 2 * v.shape[0]).astype(np.float16).tobytes(),
                                      np.uint8).reshape(-1, 4)
        return oracle.Q4K, b, None, 1.0
    if fmt == "q8_0":
        b = oracle.quantize_q8_0(W)
        if random_bytes:
            b = rng.integers(0, 256, b.size, dtype=np.uint8)
            v = b.reshape(-1, 34)
            v[:, 0:2] = np.frombuffer(rng.uniform(-0.05, 0.05, v.shape[0]).astype(np.float16).tobytes(),
                                      np.uint8).reshape(-1, 2)
        return oracle.Q8_0, b, None, 1.0
    if fmt == "mxfp4":
        b, s = oracle.quantize_mxfp4(W)
        if random_bytes:
            b = rng.integers(0, 256, b.size, dtype=np.uint8)
            s = rng.integers(0, 256, s.size, dtype=np.uint8)  # includes 0 (2^-127) and 255 (NaN)
        return oracle.MXFP4, b, s, 1.0
    b, g = oracle.quantize_nvfp4(W)
    if random_bytes:
        b = rng.integers(0, 256, b.size, dtype=np.uint8)
        g = 0.37
    return oracle.NVFP4, b, None, g


def qt_of(gk, fmt):
    return {"q4k": gk.QuantType.q4k(), "q8_0": gk.QuantType.q8_0(), "mxfp4": gk.QuantType.mxfp4(32),
            "nvfp4": gk.QuantType.nvfp4()}[fmt]


# ---- repack / decode -------------------------------------------------------------------------
@pytest.mark.parametrize("fmt,n,k", [("q4k", 16, 256), ("q4k", 100, 1024), ("q4k", 1, 256), ("q8_0", 16, 32),
                                     ("q8_0", 37, 416), ("q8_0", 5, 2048), ("mxfp4", 128, 128), ("mxfp4", 70, 640),
                                     ("nvfp4", 128, 64), ("nvfp4", 200, 448)])
@pytest.mark.parametrize("random_bytes", [False, True])
def test_repack_roundtrip_and_decode_bit_exact(gk, K, oracle, fmt, n, k, random_bytes):
    oid, blocks, scales, g = make(oracle, fmt, n, k, seed=n * 7 + k, random_bytes=random_bytes)
    w = K.upload(qt_of(gk, fmt), n, k, blocks, scales, g)
    info = w.info()
    assert info["n"] == n and info["k"] == k and info["dev_bytes"] >= info["ref_bytes"] - n * (k // 32)
    back = K.unpack(w)
    if fmt == "mxfp4":
        assert np.array_equal(back[0], blocks) and np.array_equal(back[1], scales)
    else:
        assert np.array_equal(back, blocks)
    dec = K.dequant(w).cpu().numpy()
    ref = oracle.dequant_matrix(oid, blocks, n, k, scales=scales, global_scale=g)
    assert same_bits(dec, ref)
    w.free()


def test_mxfp4_inline_form_upload(gk, K, oracle):
    n, k = 130, 256
    _, blocks, scales, _ = make(oracle, "mxfp4", n, k, seed=4, random_bytes=True)
    inline = np.concatenate([scales.reshape(-1, 1), blocks.reshape(-1, 16)], axis=1).reshape(-1)
    w = K.upload(gk.QuantType.mxfp4(32), n, k, inline, None)
    b2, s2 = K.unpack(w)
    assert np.array_equal(b2, blocks) and np.array_equal(s2, scales)
    w.free()


def test_upload_from_device_memory(gk, K, oracle, torch):
    oid, blocks, _, _ = make(oracle, "q4k", 48, 512, seed=11)
    dev = torch.from_numpy(blocks).cuda()
    w = K.upload(gk.QuantType.q4k(), 48, 512, dev)
    assert np.array_equal(K.unpack(w), blocks)
    w.free()


def test_host_dropin_decoders_on_reference_known_answers(gk, K):
    c = KA["q4k_decode_basic"]
    out = np.zeros(256, np.float32)
    K.dequant_q4_k(np.array(c["block"], np.uint8), out)
    for i, v in c["expect"].items():
        assert out[int(i)] == v
    c = KA["q4k_decode_all_subblocks"]
    K.dequant_q4_k(np.array(c["block"], np.uint8), out)
    assert out.tolist() == c["expect_all"]
    out = np.zeros(32, np.float32)
    c = KA["q8_0_decode_basic"]
    K.dequant_q8_0(np.array(c["block"], np.uint8), out)
    for i, v in c["expect"].items():
        assert out[int(i)] == v
    c = KA["q8_0_decode_extreme"]
    K.dequant_q8_0(np.array(c["block"], np.uint8), out)
    assert out.tolist() == c["expect_all"]
    for name, c in KA["mxfp4"].items():
        exp_n = len(c["scales"]) * c["block_size"]
        out = np.zeros(exp_n, np.float32)
        K.dequant_mxfp4(np.array(c["blocks"], np.uint8), np.array(c["scales"], np.uint8), out, c["block_size"])
        if c.get("expect_all_nan"):
            assert np.isnan(out).all(), name
        else:
            assert same_bits(out, np.array(c["expect"], np.float32)), name
    with pytest.raises(gk.GllmkError):  # the reference returns Err on inconsistent lengths
        K.dequant_mxfp4(np.zeros(15, np.uint8), np.zeros(1, np.uint8), np.zeros(32, np.float32), 32)


def test_host_dropin_nvfp4_decode(gk, K, oracle):
    rng = np.random.default_rng(2)
    blocks = rng.integers(0, 256, 36 * 9, dtype=np.uint8)
    out = np.zeros(64 * 9, np.float32)
    K.dequant_nvfp4(blocks, 0.25, out)
    assert same_bits(out, oracle.dequant_nvfp4(blocks, 0.25))


# ---- quantizers ------------------------------------------------------------------------------
@pytest.mark.parametrize("fmt", ["q4k", "q8_0", "mxfp4", "nvfp4"])
def test_device_quantizers_match_oracle_bytes(gk, K, oracle, torch, fmt):
    rng = np.random.default_rng(21)
    n, k = 64, 1024
    W = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    W[3] = 0.0                      # all-zero blocks
    W[5, :256] = 0.013              # constant block
    W[7] *= 1e-6                    # tiny values
    W[9, 17] = 3.0                  # outlier
    Wd = torch.from_numpy(W).cuda()
    res = K.quantize(qt_of(gk, fmt), Wd)
    if fmt == "q4k":
        assert np.array_equal(res.cpu().numpy(), oracle.quantize_q4_k(W))
    elif fmt == "q8_0":
        assert np.array_equal(res.cpu().numpy(), oracle.quantize_q8_0(W))
    elif fmt == "mxfp4":
        b, s = oracle.quantize_mxfp4(W)
        assert np.array_equal(res[0].cpu().numpy(), b) and np.array_equal(res[1].cpu().numpy(), s)
    else:
        b, g = oracle.quantize_nvfp4(W)
        assert res[1] == pytest.approx(g, rel=0, abs=0)
        assert np.array_equal(res[0].cpu().numpy(), b)


# ---- GEMV ------------------------------------------------------------------------------------
def gemv_case(gk, K, oracle, torch, fmt, n, k, m, seed, ref_layout=False, ctas_per_sm=0, row_scales=None):
    oid, blocks, _, _ = make(oracle, fmt, n, k, seed)
    rng = np.random.default_rng(seed + 1)
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = K.upload(qt_of(gk, fmt), n, k, blocks)
    K.set("gemv_ctas_per_sm", ctas_per_sm)
    xin = torch.from_numpy(np.ascontiguousarray(x.T) if ref_layout else x).cuda()
    rs = None if row_scales is None else torch.from_numpy(row_scales).cuda()
    y = K.gemv(w, xin, ref_layout=ref_layout, row_scales=rs).cpu().numpy()
    K.set("gemv_ctas_per_sm", 0)
    ref = oracle.quant_matmul(blocks, np.ascontiguousarray(x.T), oid, n, m, k, threads=8)  # [n, m]
    if row_scales is not None:
        ref = ref * (row_scales.reshape(-1, 1) if row_scales.size > 1 else row_scales[0])
    if not ref_layout:
        ref = ref.T
    assert y.shape == ref.shape
    err = oracle.rel_err(y, ref)
    w.free()
    return err


def test_gemv_q4k_config1_shape(gk, K, oracle, torch):
    """BASELINE config 1: W[4096,4096] Q4_K, x[1,4096]."""
    assert gemv_case(gk, K, oracle, torch, "q4k", 4096, 4096, 1, seed=20240) <= TOL


@pytest.mark.parametrize("m", [1, 4, 8, 16])
def test_gemv_q8_0_config2_shape(gk, K, oracle, torch, m):
    """BASELINE config 2: W[11008,4096] Q8_0, x[M,4096], M in {1,4,8,16}."""
    assert gemv_case(gk, K, oracle, torch, "q8_0", 11008, 4096, m, seed=20241) <= TOL


@pytest.mark.parametrize("fmt,n,k,m", [("q4k", 1, 256, 1), ("q4k", 17, 512, 3), ("q4k", 100, 1280, 16),
                                       ("q4k", 333, 2048, 5), ("q8_0", 1, 32, 1), ("q8_0", 50, 96, 2),
                                       ("q8_0", 129, 4000, 16), ("q8_0", 16, 288, 9)])
@pytest.mark.parametrize("ref_layout", [False, True])
def test_gemv_ragged_shapes_both_layouts(gk, K, oracle, torch, fmt, n, k, m, ref_layout):
    assert gemv_case(gk, K, oracle, torch, fmt, n, k, m, seed=n + k + m, ref_layout=ref_layout) <= TOL


@pytest.mark.parametrize("ctas_per_sm", [1, 2, 3])
@pytest.mark.parametrize("fmt", ["q4k", "q8_0"])
def test_gemv_stream_k_partitions(gk, K, oracle, torch, fmt, ctas_per_sm):
    """Different grid sizes cut the (tile group, k-step) sequence at different places: row tiles are
    completed by 1, 2 or 3 CTAs and the slot-ordered reduction must give the same parity."""
    assert gemv_case(gk, K, oracle, torch, fmt, 5000, 4096, 3, seed=77, ctas_per_sm=ctas_per_sm) <= TOL


def test_gemv_row_scales(gk, K, oracle, torch):
    rs = np.random.default_rng(1).uniform(0.5, 2.0, 96).astype(np.float32)
    assert gemv_case(gk, K, oracle, torch, "q4k", 96, 512, 2, seed=5, row_scales=rs) <= TOL
    assert gemv_case(gk, K, oracle, torch, "q4k", 96, 512, 2, seed=5, row_scales=np.array([3.0], np.float32)) <= TOL


def test_gemv_is_deterministic_and_rejects_bad_m(gk, K, oracle, torch):
    oid, blocks, _, _ = make(oracle, "q4k", 256, 1024, 3)
    w = K.upload(gk.QuantType.q4k(), 256, 1024, blocks)
    x = torch.randn(4, 1024, device="cuda")
    a = K.gemv(w, x).clone()
    b = K.gemv(w, x)
    assert torch.equal(a, b)
    with pytest.raises(gk.GllmkError) as e:
        K.gemv(w, torch.randn(17, 1024, device="cuda"))
    assert e.value.status == gk.Status.INVALID_ARG
    w.free()


def test_gemv_scale_extremes_zero_and_nan(gk, K, oracle, torch):
    """Tokens of very different magnitude, an all-zero token, and a NaN that must reach every output."""
    n, k = 64, 512
    oid, blocks, _, _ = make(oracle, "q4k", n, k, 8)
    rng = np.random.default_rng(8)
    x = rng.standard_normal((4, k)).astype(np.float32)
    x[0] *= 1e-20
    x[1] *= 1e15
    x[2] = 0.0
    w = K.upload(gk.QuantType.q4k(), n, k, blocks)
    y = K.gemv(w, torch.from_numpy(x).cuda()).cpu().numpy()
    ref = oracle.quant_matmul(blocks, np.ascontiguousarray(x.T), oid, n, 4, k).T
    for t in (0, 1, 3):
        assert oracle.rel_err(y[t], ref[t]) <= TOL
    assert not y[2].any()
    x[3, 100] = np.nan
    y = K.gemv(w, torch.from_numpy(x).cuda()).cpu().numpy()
    assert np.isnan(y[3]).all() and not np.isnan(y[:3]).any()
    w.free()


def test_gemv_linearity_at_config5_size(gk, K, oracle, torch):
    """70B-shaped gate/up matrix W[28672, 8192] Q4_K quantized on the device: a sample of rows against the
    oracle, and linearity y(a*x1 + x2) = a*y(x1) + y(x2) over the whole output."""
    n, k = 28672, 8192
    g = torch.Generator(device="cuda").manual_seed(20244)
    W = torch.randn((n, k), generator=g, device="cuda") * 0.02
    qt = gk.QuantType.q4k()
    blocks = K.quantize(qt, W)
    del W
    w = K.upload(qt, n, k, blocks)
    x = torch.randn((2, k), generator=g, device="cuda")
    y = K.gemv(w, x)
    xc = (2.0 * x[0] + x[1]).reshape(1, k)
    yc = K.gemv(w, xc)
    # activations enter as two int8 digits per 256-block (error <= amax * 1.6e-5 per element), so
    # linearity holds to that precision, far inside the 2e-3 bar
    lin = (2.0 * y[0] + y[1] - yc[0]).abs().max().item() / yc.abs().max().item()
    assert lin < 2e-4
    rows = np.r_[0:16, 14000:14016, n - 16:n]
    hb = blocks.reshape(n, -1)[torch.from_numpy(rows).cuda()].cpu().numpy().reshape(-1)
    ref = oracle.quant_matmul(hb, np.ascontiguousarray(x.cpu().numpy().T), oracle.Q4K, rows.size, 2, k).T
    assert oracle.rel_err(y.cpu().numpy()[:, rows], ref) <= TOL
    w.free()


# ---- host-pointer drop-ins of the reference operator API --------------------------------------
def test_reference_known_answers_through_the_dropins(gk, K):
    c = KA["gemm_q4_basic"]
    out = np.zeros(c["m"] * c["n"], np.float32)
    K.gemm_q4(np.array(c["weight"], np.uint8), np.array(c["input"], np.float32), out, c["scales"], c["m"], c["n"], c["k"])
    assert out.tolist() == c["expect"]
    c = KA["gemm_q4_per_channel"]
    out = np.zeros(c["m"] * c["n"], np.float32)
    K.gemm_q4(np.array(c["weight"], np.uint8), np.array(c["input"], np.float32), out, c["scales"], c["m"], c["n"], c["k"])
    assert out.tolist() == c["expect"]
    c = KA["q8_0_dot"]
    out = np.zeros(1, np.float32)
    K.classic_matmul(np.array(c["weight"], np.uint8), np.array(c["input"], np.float32), out, gk.QuantType.q8_0(),
                     c["m"], c["n"], c["k"])
    assert abs(out[0] - c["expect"][0]) < 1e-2  # the reference's own tolerance (src/tests_quant.rs:672-676)


def test_kquant_and_classic_matmul_dropins(gk, K, oracle):
    rng = np.random.default_rng(31)
    for fmt, fn, qt in (("q4k", K.kquant_matmul, gk.QuantType.q4k()), ("q8_0", K.classic_matmul, gk.QuantType.q8_0())):
        m, n, k = 200, 21, 1024  # reference naming: m weight rows, n batch columns (> 16: chunked internally)
        oid, blocks, _, _ = make(oracle, fmt, m, k, 31)
        x = rng.standard_normal((k, n)).astype(np.float32)
        out = np.zeros((m, n), np.float32)
        fn(blocks, x, out, qt, m, n, k)
        ref = oracle.quant_matmul(blocks, x, oid, m, n, k)
        assert oracle.rel_err(out, ref) <= TOL
    # wrong family: the reference panics (unimplemented!), the C ABI returns Unsupported
    with pytest.raises(gk.GllmkError) as e:
        K.kquant_matmul(blocks, x, out, gk.QuantType.q8_0(), m, n, k)
    assert e.value.status == gk.Status.UNSUPPORTED
    with pytest.raises(gk.GllmkError) as e:
        K.gemm_q4(np.zeros(144, np.uint8), np.zeros(100, np.float32), np.zeros(1, np.float32), None, 1, 1, 100)
    assert e.value.status == gk.Status.INVALID_ARG  # k % 256 != 0: the reference asserts


def test_matmul_host_resident_weight(gk, K, oracle):
    oid, blocks, _, _ = make(oracle, "q4k", 512, 1024, 41)
    w = K.upload(gk.QuantType.q4k(), 512, 1024, blocks)
    x = np.random.default_rng(41).standard_normal((3, 1024)).astype(np.float32)
    y = K.matmul_host(w, x)
    ref = oracle.gemm_q4(blocks, x, None, 3, 512, 1024)
    assert oracle.rel_err(y, ref) <= TOL
    y2 = K.matmul_host(w, np.ascontiguousarray(x.T), ref_layout=True)
    assert oracle.rel_err(y2, ref.T) <= TOL
    assert K.gemv_q4(blocks[:4 * 144], x[0], 2.0, 1024) == pytest.approx(2.0 * ref[0, 0], rel=2e-3, abs=1e-6)
    w.free()


# ---- gated feed-forward block: two decode products with SwiGLU fused into the second one's staging ------
@pytest.mark.parametrize("fmt,d,f,m", [("q4k", 256, 512, 1), ("q4k", 512, 768, 5), ("q8_0", 128, 160, 16)])
def test_ffn_decode_swiglu(gk, K, oracle, torch, fmt, d, f, m):
    oid, b_gu, _, _ = make(oracle, fmt, 2 * f, d, 61)
    _, b_dn, _, _ = make(oracle, fmt, d, f, 62)
    qt = gk.QuantType.q4k() if fmt == "q4k" else gk.QuantType.q8_0()
    w_gu, w_dn = K.upload(qt, 2 * f, d, b_gu), K.upload(qt, d, f, b_dn)
    x = np.random.default_rng(63).standard_normal((m, d)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    h = torch.empty((m, 2 * f), dtype=torch.float32, device="cuda")
    y = K.ffn_decode(w_gu, w_dn, xd, h=h).cpu().numpy()
    # oracle chain: the reference's matmul, scalar_swiglu (g / (1 + exp(-g)) * u in f32), the reference's matmul
    h_ref = oracle.quant_matmul(b_gu, np.ascontiguousarray(x.T), oid, 2 * f, m, d).T
    g, u = h_ref[:, :f], h_ref[:, f:]
    act = ((g / (np.float32(1.0) + np.exp(-g, dtype=np.float32))) * u).astype(np.float32)
    y_ref = oracle.quant_matmul(b_dn, np.ascontiguousarray(act.T), oid, d, m, f).T
    assert oracle.rel_err(h.cpu().numpy(), h_ref) <= TOL
    assert oracle.rel_err(y, y_ref) <= TOL
    assert K.status() == 0
    with pytest.raises(gk.GllmkError) as e:  # shapes that do not chain
        K.ffn_decode(w_dn, w_dn, xd)
    assert e.value.status == gk.Status.INVALID_ARG
    w_gu.free()
    w_dn.free()


def test_swiglu_known_answers_through_ffn_decode(gk, K, oracle, torch):
    """scalar-ops/src/activations.rs:157-167: swiglu(0, 1) = 0, swiglu(1, 2) = 2 * silu(1).  Identity-like Q8_0
    weights (one 1.0 per row) pass x through the products unchanged, so y is the SwiGLU of x's two halves."""
    f = 32
    def unit_rows(rows, cols, picks):
        W = np.zeros((rows, cols), np.float32)
        for r, ccol in enumerate(picks):
            W[r, ccol] = 1.0
        return oracle.quantize_q8_0(W)
    qt = gk.QuantType.q8_0()
    w_gu = K.upload(qt, 2 * f, 2 * f, unit_rows(2 * f, 2 * f, range(2 * f)))  # h = x: gate = x[:f], up = x[f:]
    # the block maps back to the model width (2f here): rows 0..f-1 of the down weight copy act, the rest repeat act[0]
    w_dn = K.upload(qt, 2 * f, f, unit_rows(2 * f, f, list(range(f)) + [0] * f))
    x = np.zeros((1, 2 * f), np.float32)
    x[0, :4] = [0.0, 1.0, 2.0, -1.0]        # gate
    x[0, f:f + 4] = [1.0, 2.0, 3.0, 4.0]    # up
    y = K.ffn_decode(w_gu, w_dn, torch.from_numpy(x).cuda()).cpu().numpy()[0]
    silu = lambda g: g / (1.0 + np.exp(-g))
    want = [0.0, silu(1.0) * 2.0, silu(2.0) * 3.0, silu(-1.0) * 4.0]
    assert np.allclose(y[:4], want, rtol=2e-3, atol=1e-6), (y[:4], want)
    w_gu.free()
    w_dn.free()


# ---- quantized embedding lookup: decode of selected rows, bit-exact ---------------------------------------
@pytest.mark.parametrize("fmt,n,k", [("q4k", 300, 512), ("q8_0", 129, 96), ("mxfp4", 200, 320), ("nvfp4", 77, 192)])
def test_embedding_gather_bit_exact(gk, K, oracle, torch, fmt, n, k):
    oid, blocks, scales, g = make(oracle, fmt, n, k, 71)
    qt = {"q4k": gk.QuantType.q4k(), "q8_0": gk.QuantType.q8_0(), "mxfp4": gk.QuantType.mxfp4(32), "nvfp4": gk.QuantType.nvfp4()}[fmt]
    w = K.upload(qt, n, k, blocks, scales, g if g is not None else 1.0)
    full = oracle.dequant_matrix(oid, blocks, n, k, scales=scales, global_scale=g if g is not None else 1.0)
    ids = np.array([0, n - 1, 5, 5, n // 2, -1, n, 17], np.int32)  # repeats, both ends, two ids out of range
    out = K.embedding_gather(w, torch.from_numpy(ids).cuda()).cpu().numpy()
    for r, i in enumerate(ids):
        want = full[i] if 0 <= i < n else np.zeros(k, np.float32)
        assert np.array_equal(out[r].view(np.uint32), want.view(np.uint32)), (fmt, r, i)
    w.free()


def test_matmul_host_with_page_locked_buffers(gk, K, oracle, torch):
    """Pinned x / out are used in place (no staging copy); results equal the pageable-buffer call bit for bit."""
    oid, blocks, _, _ = make(oracle, "q4k", 512, 1024, 43)
    w = K.upload(gk.QuantType.q4k(), 512, 1024, blocks)
    x = np.random.default_rng(43).standard_normal((2, 1024)).astype(np.float32)
    xp = torch.empty((2, 1024), dtype=torch.float32, pin_memory=True)
    xp.copy_(torch.from_numpy(x))
    yp = torch.empty((2, 512), dtype=torch.float32, pin_memory=True)
    y_pinned = K.matmul_host(w, xp.numpy(), out=yp.numpy())
    y_plain = K.matmul_host(w, x)
    assert np.array_equal(y_pinned, y_plain) and np.array_equal(yp.numpy(), y_plain)
    assert oracle.rel_err(y_plain, oracle.gemm_q4(blocks, x, None, 2, 512, 1024)) <= TOL
    w.free()


# ---- small shares: the GEMV stages its activation slices itself (no staging launch) ---------------------------
@pytest.mark.parametrize("fmt,n,k,m", [("q4k", 4096, 4096, 1), ("q4k", 1024, 28672, 1), ("q4k", 7168, 8192, 1), ("q4k", 300, 1280, 3),
                                       ("q4k", 16, 256, 4), ("q8_0", 11008, 4096, 1), ("q8_0", 129, 4000, 2)])
def test_gemv_fused_staging_equals_the_staging_kernel(gk, K, oracle, torch, fmt, n, k, m):
    """Both variants do the same arithmetic on the same partition of the work: bit-identical outputs; and the
    oracle bar on top."""
    oid, blocks, _, _ = make(oracle, fmt, n, k, seed=n + k)
    w = K.upload(qt_of(gk, fmt), n, k, blocks)
    x = torch.from_numpy(np.random.default_rng(n).standard_normal((m, k)).astype(np.float32)).cuda()
    K.set("gemv_fuse", 0)
    try:
        y_img = K.gemv(w, x).clone()
        K.set("gemv_fuse", 2)  # every product (off by default)
        y_fused = K.gemv(w, x).clone()
        y_ref_layout = K.gemv(w, x.t().contiguous(), ref_layout=True)
    finally:
        K.set("gemv_fuse", 0)
    assert K.status() == 0
    assert torch.equal(y_img, y_fused)
    ref = oracle.quant_matmul(blocks, np.ascontiguousarray(x.cpu().numpy().T), oid, n, m, k, threads=8).T
    assert oracle.rel_err(y_fused.cpu().numpy(), ref) <= TOL
    # strided x (the reference's [k, m] layout) went through the same fused path
    assert torch.equal(y_ref_layout.t().contiguous(), y_fused)
    w.free()


def test_matmul_host_batch_equals_one_call_per_product(gk, K, oracle, torch):
    """The products of a step through one call (enqueued back to back, one wait): bit-identical with one synchronous call
    per product, with pageable and with page-locked host buffers, decode- and prefill-sized batches mixed."""
    rng = np.random.default_rng(81)
    specs = [("q4k", 512, 1024, 1), ("q8_0", 300, 416, 5), ("q4k", 256, 512, 70), ("q4k", 512, 1024, 2)]
    ws, xs, want = [], [], []
    for fmt, n, k, m in specs:
        oid, blocks, _, _ = make(oracle, fmt, n, k, seed=n + m)
        w = K.upload(qt_of(gk, fmt), n, k, blocks)
        x = rng.standard_normal((m, k)).astype(np.float32)
        ws.append(w), xs.append(x), want.append(K.matmul_host(w, x))
    outs = [np.full((x.shape[0], w.n), np.nan, np.float32) for w, x in zip(ws, xs)]
    K.matmul_host_batch(ws, xs, outs)
    for got, ref in zip(outs, want):
        assert np.array_equal(got, ref)
    xp = [torch.empty(x.shape, dtype=torch.float32, pin_memory=True) for x in xs]
    for t, x in zip(xp, xs):
        t.copy_(torch.from_numpy(x))
    yp = [torch.full(o.shape, float("nan"), dtype=torch.float32, pin_memory=True) for o in outs]
    K.matmul_host_batch(ws, [t.numpy() for t in xp], [t.numpy() for t in yp])
    for got, ref in zip(yp, want):
        assert np.array_equal(got.numpy(), ref)
    assert K.status() == 0
    # The same argument list again and again: from the third call on the step is replayed as a captured graph.  New
    # activations in the same buffers every time, page-locked and pageable buffers; then a different list (fresh
    # enqueue), the first list again, and the graph switched off.
    xn, yn = [t.numpy() for t in xp], [t.numpy() for t in yp]
    for rep in range(5):
        fresh = [rng.standard_normal(x.shape).astype(np.float32) for x in xs]
        ref = [K.matmul_host(w, x) for w, x in zip(ws, fresh)]
        for dst, x in zip(xn, fresh):
            dst[...] = x
        for y in yn:
            y[...] = np.nan
        K.matmul_host_batch(ws, xn, yn)
        for got, want_i in zip(yn, ref):
            assert np.array_equal(got, want_i), rep
    pageable_x = [x.copy() for x in xs]
    for rep in range(4):
        fresh = [rng.standard_normal(x.shape).astype(np.float32) for x in xs]
        ref = [K.matmul_host(w, x) for w, x in zip(ws, fresh)]
        for dst, x in zip(pageable_x, fresh):
            dst[...] = x
        for o in outs:
            o[...] = np.nan
        K.matmul_host_batch(ws, pageable_x, outs)
        for got, want_i in zip(outs, ref):
            assert np.array_equal(got, want_i), rep
    K.matmul_host_batch(ws[1:3], xn[1:3], yn[1:3])
    assert np.array_equal(yn[1], K.matmul_host(ws[1], xn[1])) and np.array_equal(yn[2], K.matmul_host(ws[2], xn[2]))
    plan = K.host_batch(ws, xn, yn)  # the argument arrays built once
    for rep in range(4):
        for dst in xn:
            dst[...] = rng.standard_normal(dst.shape).astype(np.float32)
        ref = [K.matmul_host(w, x) for w, x in zip(ws, xn)]
        for y in yn:
            y[...] = np.nan
        plan.run()
        for got, want_i in zip(yn, ref):
            assert np.array_equal(got, want_i), rep
    # a larger product in between makes the context grow its scratch buffers: the captured step must not be replayed
    # with the old ones (the cached graph is keyed on them), and the list is captured again later
    oid_big, blocks_big, _, _ = make(oracle, "q4k", 2048, 4096, seed=5)
    w_big = K.upload(qt_of(gk, "q4k"), 2048, 4096, blocks_big)
    x_big = rng.standard_normal((9, 4096)).astype(np.float32)
    y_big = K.matmul_host(w_big, x_big)
    ref_big = oracle.quant_matmul(blocks_big, np.ascontiguousarray(x_big.T), oid_big, 2048, 9, 4096, threads=8).T
    assert oracle.rel_err(y_big, ref_big) <= 2e-3
    for rep in range(4):
        for dst in xn:
            dst[...] = rng.standard_normal(dst.shape).astype(np.float32)
        ref = [K.matmul_host(w, x) for w, x in zip(ws, xn)]
        for y in yn:
            y[...] = np.nan
        plan.run()
        for got, want_i in zip(yn, ref):
            assert np.array_equal(got, want_i), rep
    w_big.free()
    K.set("host_batch_graph", 0)
    try:
        for y in yn:
            y[...] = np.nan
        K.matmul_host_batch(ws, xn, yn)
        for got, w, x in zip(yn, ws, xn):
            assert np.array_equal(got, K.matmul_host(w, x))
    finally:
        K.set("host_batch_graph", 1)
    assert K.status() == 0
    with pytest.raises(gk.GllmkError) as e:
        K.matmul_host_batch(ws[:1], [np.zeros((0, 1024), np.float32)], [np.zeros((0, 512), np.float32)])
    assert e.value.status == gk.Status.INVALID_ARG
    for w in ws:
        w.free()
