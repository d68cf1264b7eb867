"""Parity of the Q6_K / Q5_K / Q8_K / Q4_0 / Q5_0 path (through the C ABI) with the CPU oracle.  Needs a B200.

Bars: decoded values, unpack round trip, gathers — bit-exact.  GEMV / matmul outputs —
max_i |y_i - ref_i| / max(|ref_i|, rms(ref)) <= 2e-3 against the oracle's sequential f32 sum.
"""
import json
import os
import struct

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 2e-3
HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(HERE, "golden", "reference_known_answers.json")) as f:
    KA = json.load(f)

FORMATS = ["q6_k", "q5_k", "q8_k", "q4_0", "q5_0"]


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


def qtype(gk, name):
    Q = gk.QuantType
    return {"q6_k": Q.q6k(), "q5_k": Q.q5k(), "q8_k": Q.q8k(), "q4_0": Q.q4_0(), "q5_0": Q.q5_0()}[name]


def same_bits(a, b):
    a = np.ascontiguousarray(a, np.float32).reshape(-1)
    b = np.ascontiguousarray(b, np.float32).reshape(-1)
    return bool((a.view(np.uint32) == b.view(np.uint32)).all())


def random_blocks(name, qt, n, k, seed):
    """n rows of k / block_size blocks: random payload bytes, small finite scales (both signs)."""
    rng = np.random.default_rng(seed)
    bs, bb = qt.block_size(), qt.block_bytes()
    nblk = n * (k // bs)
    v = rng.integers(0, 256, size=(nblk, bb), dtype=np.uint8)
    if name == "q8_k":
        v[:, 0:4] = np.frombuffer(rng.uniform(-0.02, 0.02, nblk).astype(np.float32).tobytes(), np.uint8).reshape(-1, 4)
    else:
        d = np.frombuffer(rng.uniform(-0.02, 0.02, nblk).astype(np.float16).tobytes(), np.uint8).reshape(-1, 2)
        if name == "q6_k":
            v[:, 208:210] = d
        else:
            v[:, 0:2] = d
        if name == "q5_k":
            v[:, 2:4] = np.frombuffer(rng.uniform(-0.02, 0.02, nblk).astype(np.float16).tobytes(), np.uint8).reshape(-1, 2)
    return v.reshape(-1)


def oracle_matrix(oracle, qt, blocks, n, k):
    return oracle.dequant_matrix(qt.id, blocks, n, k)


@pytest.mark.parametrize("name", FORMATS)
def test_decode_unpack_gather_bit_exact(K, gk, oracle, torch, name):
    qt = qtype(gk, name)
    n, k = 37, 3 * 256  # ragged row count; row byte lengths that are not multiples of 16
    blocks = random_blocks(name, qt, n, k, 11)
    ref = oracle_matrix(oracle, qt, blocks, n, k)
    w = K.upload(qt, n, k, blocks)
    assert w.ref_bytes == blocks.size
    assert same_bits(K.dequant(w).cpu().numpy(), ref)
    assert np.array_equal(np.asarray(K.unpack(w)).reshape(-1), blocks)
    ids = torch.tensor([3, 36, -1, 0, 37, 3], dtype=torch.int32, device="cuda")
    got = K.embedding_gather(w, ids).cpu().numpy()
    want = np.stack([ref[i] if 0 <= i < n else np.zeros(k, np.float32) for i in ids.cpu().tolist()])
    assert same_bits(got, want)
    # host-pointer decode of a run of blocks
    out = np.empty(n * k, np.float32)
    K.dequant_gguf(qt, blocks, out)
    assert same_bits(out, ref)
    w.free()


@pytest.mark.parametrize("name", ["q8_k_decode", "q5_k_decode", "q6_k_decode", "q4_0_decode_zero", "q4_0_decode_known",
                                  "q4_0_decode_full_range", "q5_0_decode", "q5_0_decode_all_bits"])
def test_decode_known_answers(K, gk, name):
    c = KA[name]
    qt = qtype(gk, c["qt"])
    out = np.empty(qt.block_size(), np.float32)
    getattr(K, "dequant_" + c["qt"])(np.array(c["block"], np.uint8), out)
    if "expect_all" in c:
        assert out.tolist() == c["expect_all"]
    for i, v in c.get("expect", {}).items():
        assert out[int(i)] == v


@pytest.mark.parametrize("name", ["q4_0_dot", "q5_0_dot", "q8_k_matmul"])
def test_matmul_known_answers(K, gk, name):
    c = KA[name]
    qt = qtype(gk, c["qt"])
    out = np.zeros(c["m"] * c["n"], np.float32)
    fn = K.kquant_matmul if qt.block_size() == 256 else K.classic_matmul
    fn(np.array(c["weight"], np.uint8), np.array(c["input"], np.float32), out, qt, c["m"], c["n"], c["k"])
    # the activations pass through a 16-bit fixed-point form; the reference's own tests allow 1e-2 here
    assert np.max(np.abs(out - np.array(c["expect"], np.float32))) <= 1e-3


@pytest.mark.parametrize("name", FORMATS)
@pytest.mark.parametrize("m", [1, 3, 8, 16])
def test_gemv_parity(K, gk, oracle, torch, name, m):
    qt = qtype(gk, name)
    n, k = 203, 8 * 256  # rows not a multiple of the 8 a CTA takes per pass
    blocks = random_blocks(name, qt, n, k, 100 + m)
    rng = np.random.default_rng(7 + m)
    x = rng.standard_normal((m, k)).astype(np.float32)
    ref = oracle.quant_matmul(blocks, np.ascontiguousarray(x.T), qt.id, n, m, k, threads=4)  # [n, m]
    w = K.upload(qt, n, k, blocks)
    y = K.gemv(w, torch.from_numpy(x).cuda()).cpu().numpy()  # [m, n]
    assert oracle.rel_err(y.T, ref) <= TOL
    # reference layout (x [k, m] -> y [n, m]) reads the same tensors through strides
    y2 = K.gemv(w, torch.from_numpy(np.ascontiguousarray(x.T)).cuda(), ref_layout=True).cpu().numpy()
    assert oracle.rel_err(y2, ref) <= TOL
    assert K.status() == 0
    w.free()


@pytest.mark.parametrize("n,k,m", [(203, 8 * 256, 2), (16, 256, 8), (33, 3 * 256, 9), (64, 40 * 256, 16), (100, 5 * 256, 13)])
def test_q6k_batch_on_the_tensor_core(K, gk, oracle, torch, n, k, m):
    """Q6_K with two tokens and more: mma.sync over the same assembled s8 words and s16 activation digits as the dp2a
    kernel ("raw_gemv_mma" = 0), so both see the same integers; only the f32 summation order differs.  Shapes: rows not a
    multiple of the 16 a CTA owns, one block per row (seven of the eight warps idle), blocks not a multiple of eight,
    tokens not a multiple of eight; row scales and the reference's transposed layout."""
    qt = qtype(gk, "q6_k")
    blocks = random_blocks("q6_k", qt, n, k, 300 + m)
    rng = np.random.default_rng(31 + m)
    x = rng.standard_normal((m, k)).astype(np.float32)
    sc = rng.uniform(0.5, 2.0, n).astype(np.float32)
    ref = oracle.quant_matmul(blocks, np.ascontiguousarray(x.T), qt.id, n, m, k, threads=4)  # [n, m]
    w = K.upload(qt, n, k, blocks)
    xd = torch.from_numpy(x).cuda()
    run = (lambda: K.gemm(w, xd)) if m > 16 else (lambda: K.gemv(w, xd))
    try:
        K.set("raw_gemv_mma", 1)
        y_tc = run().cpu().numpy()
        K.set("raw_gemv_mma", 0)
        y_dp = run().cpu().numpy()
        K.set("raw_gemv_mma", 1)
        if m <= 16:
            y_sc = K.gemv(w, xd, row_scales=torch.from_numpy(sc).cuda()).cpu().numpy()
            y_t = K.gemv(w, torch.from_numpy(np.ascontiguousarray(x.T)).cuda(), ref_layout=True).cpu().numpy()
    finally:
        K.set("raw_gemv_mma", 1)
    assert K.status() == 0
    assert oracle.rel_err(y_tc.T, ref) <= TOL
    assert oracle.rel_err(y_tc.T, y_dp.T) <= 1e-5
    if m <= 16:
        assert oracle.rel_err(y_sc.T, ref * sc[:, None]) <= TOL
        assert oracle.rel_err(y_t, ref) <= TOL
    w.free()


def test_q6k_single_token_on_the_tensor_core(K, gk, oracle, torch):
    # "raw_gemv_mma" = 2 routes one token through the same kernel (seven of the eight MMA columns idle)
    qt = qtype(gk, "q6_k")
    n, k = 130, 6 * 256
    blocks = random_blocks("q6_k", qt, n, k, 77)
    x = np.random.default_rng(78).standard_normal((1, k)).astype(np.float32)
    ref = oracle.quant_matmul(blocks, np.ascontiguousarray(x.T), qt.id, n, 1, k, threads=4)
    w = K.upload(qt, n, k, blocks)
    try:
        K.set("raw_gemv_mma", 2)
        y = K.gemv(w, torch.from_numpy(x).cuda()).cpu().numpy()
    finally:
        K.set("raw_gemv_mma", 1)
    assert K.status() == 0 and oracle.rel_err(y.T, ref) <= TOL
    w.free()


@pytest.mark.parametrize("name", ["q6_k", "q4_0"])
def test_gemv_long_rows_and_row_scales(K, gk, oracle, torch, name):
    """k large enough for several staging passes per row (a pass holds 4 KB of blocks); per-row scales."""
    qt = qtype(gk, name)
    n, k = 64, 40 * 256
    blocks = random_blocks(name, qt, n, k, 5)
    rng = np.random.default_rng(6)
    x = rng.standard_normal((1, k)).astype(np.float32)
    sc = rng.uniform(0.5, 2.0, n).astype(np.float32)
    ref = oracle.quant_matmul(blocks, np.ascontiguousarray(x.T), qt.id, n, 1, k, threads=4) * sc[:, None]
    w = K.upload(qt, n, k, blocks)
    y = K.gemv(w, torch.from_numpy(x).cuda(), row_scales=torch.from_numpy(sc).cuda()).cpu().numpy()
    assert oracle.rel_err(y.T, ref) <= TOL
    w.free()


def test_gemm_many_tokens_f32(K, gk, oracle, torch):
    """gllmk_gemm with a format that has no tensor-core kernel runs the streaming kernel over token tiles; bf16 operands are refused."""
    qt = qtype(gk, "q8_k")
    n, k, m = 96, 512, 70
    blocks = random_blocks("q8_k", qt, n, k, 21)
    x = np.random.default_rng(22).standard_normal((m, k)).astype(np.float32)
    ref = oracle.quant_matmul(blocks, np.ascontiguousarray(x.T), qt.id, n, m, k, threads=4)
    w = K.upload(qt, n, k, blocks)
    y = K.gemm(w, torch.from_numpy(x).cuda()).cpu().numpy()
    assert oracle.rel_err(y.T, ref) <= TOL
    with pytest.raises(gk.GllmkError):
        K.gemm(w, torch.from_numpy(x).cuda().to(torch.bfloat16))
    w.free()


@pytest.mark.parametrize("n,k,m,bf16", [(96, 512, 70, False), (300, 5 * 256, 33, True), (64, 2 * 256, 9, False), (130, 256, 300, False), (1000, 12 * 256, 130, True),
                                        (20000, 512, 200, True)])
def test_q6k_prefill_on_the_tensor_core(K, gk, oracle, torch, n, k, m, bf16):
    """Q6_K with more than 8 tokens (gllmk_gemm): the fused-dequant tcgen05 GEMM, reference-layout blocks copied row by row into shared
    memory and converted to fp16 there (bar 1e-2 like the other weight-only formats).  Rows not a multiple of 128 (the
    last tile repeats the last row, results not stored), one and many k-blocks, one and two row tiles per CTA, f32 and bf16."""
    qt = qtype(gk, "q6_k")
    blocks = random_blocks("q6_k", qt, n, k, 400 + m)
    x = np.random.default_rng(41 + m).standard_normal((m, k)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    if bf16:
        xd = xd.to(torch.bfloat16)
        x = xd.to(torch.float32).cpu().numpy()
    w = K.upload(qt, n, k, blocks)
    y = K.gemm(w, xd, out_dtype=torch.bfloat16 if bf16 else torch.float32).to(torch.float32).cpu().numpy()
    assert K.status() == 0
    rows = np.random.default_rng(3).choice(n, size=min(n, 256), replace=False)
    wd = oracle_matrix(oracle, qt, blocks, n, k)[rows]
    ref = oracle.gemm_f32_nt(x, wd)
    assert oracle.rel_err(y[:, rows], ref) <= 1e-2 + (2.0 ** -8 if bf16 else 0.0)
    # the decode kernels on the same weight stay within their bar of the same reference
    y1 = K.gemv(w, torch.from_numpy(x[:4]).cuda()).cpu().numpy()
    assert oracle.rel_err(y1[:, rows], ref[:4]) <= TOL
    w.free()


@pytest.mark.parametrize("n,k,m,bf16", [(96, 512, 70, False), (300, 5 * 256, 17, True), (130, 256, 300, False), (1000, 12 * 256, 130, True),
                                        (20000, 512, 200, True), (64, 256, 2, False), (200, 3 * 256, 9, False)])
def test_q5k_prefill_on_the_tensor_core(K, gk, oracle, torch, n, k, m, bf16):
    """Q5_K with two tokens and more (gllmk_gemm) on the same kernel: reference-layout blocks (176 bytes), thread = weight row, the fifth
    bit from qh on top of the nibble, value = q * d*sc - dmin*m in fp16 as for Q4_K."""
    qt = qtype(gk, "q5_k")
    blocks = random_blocks("q5_k", qt, n, k, 600 + m)
    x = np.random.default_rng(61 + m).standard_normal((m, k)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    if bf16:
        xd = xd.to(torch.bfloat16)
        x = xd.to(torch.float32).cpu().numpy()
    w = K.upload(qt, n, k, blocks)
    y = K.gemm(w, xd, out_dtype=torch.bfloat16 if bf16 else torch.float32).to(torch.float32).cpu().numpy()
    assert K.status() == 0
    rows = np.random.default_rng(4).choice(n, size=min(n, 256), replace=False)
    ref = oracle.gemm_f32_nt(x, oracle_matrix(oracle, qt, blocks, n, k)[rows])
    assert oracle.rel_err(y[:, rows], ref) <= 1e-2 + (2.0 ** -8 if bf16 else 0.0)
    w.free()


@pytest.mark.parametrize("name", ["q4_0", "q5_0"])
@pytest.mark.parametrize("n,k,m,bf16", [(96, 512, 70, False), (300, 5 * 256, 2, False), (130, 256, 300, True), (1000, 12 * 256, 130, True),
                                        (20000, 512, 200, True)])
def test_classic_prefill_on_the_tensor_core(K, gk, oracle, torch, name, n, k, m, bf16):
    """Q4_0 / Q5_0 with k a multiple of 256 (a row's blocks then come in 16-byte aligned groups of eight) and more than
    one token: the same kernel; blocks start on 2-byte boundaries, so even blocks are read as words and shifted."""
    qt = qtype(gk, name)
    blocks = random_blocks(name, qt, n, k, 700 + m)
    x = np.random.default_rng(71 + m).standard_normal((m, k)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    if bf16:
        xd = xd.to(torch.bfloat16)
        x = xd.to(torch.float32).cpu().numpy()
    w = K.upload(qt, n, k, blocks)
    y = K.gemm(w, xd, out_dtype=torch.bfloat16 if bf16 else torch.float32).to(torch.float32).cpu().numpy()
    assert K.status() == 0
    rows = np.random.default_rng(5).choice(n, size=min(n, 256), replace=False)
    ref = oracle.gemm_f32_nt(x, oracle_matrix(oracle, qt, blocks, n, k)[rows])
    assert oracle.rel_err(y[:, rows], ref) <= 1e-2 + (2.0 ** -8 if bf16 else 0.0)
    w.free()


def test_classic_prefill_other_k_stays_on_the_streaming_kernel(K, gk, oracle, torch):
    # k = 5 * 32: rows are not 16-byte aligned; gllmk_gemm runs token tiles through the dp2a kernel (f32 only, 2e-3)
    qt = qtype(gk, "q4_0")
    n, k, m = 64, 160, 40
    blocks = random_blocks("q4_0", qt, n, k, 88)
    x = np.random.default_rng(89).standard_normal((m, k)).astype(np.float32)
    w = K.upload(qt, n, k, blocks)
    y = K.gemm(w, torch.from_numpy(x).cuda()).cpu().numpy()
    ref = oracle.quant_matmul(blocks, np.ascontiguousarray(x.T), qt.id, n, m, k, threads=4)
    assert oracle.rel_err(y.T, ref) <= TOL
    with pytest.raises(gk.GllmkError):
        K.gemm(w, torch.from_numpy(x).cuda().to(torch.bfloat16))
    w.free()


@pytest.mark.parametrize("gu,dn", [("q4k", "q6_k"), ("q5_k", "q5_k"), ("q4_0", "q6_k")])
def test_ffn_prefill_with_gguf_formats(K, gk, oracle, torch, gu, dn):
    """The gated feed-forward block for a batch with the formats a GGUF file mixes inside a block (Q4_K gate / up with a
    Q6_K down projection, all-Q5_K, legacy Q4_0): y = W_down (silu(gate) * up), each product within 1e-2 of the oracle's
    f32 product of the same inputs."""
    d, f, m = 512, 768, 96

    def make(name, n, k, seed):
        if name == "q4k":
            W = (np.random.default_rng(seed).standard_normal((n, k)) * 0.02).astype(np.float32)
            b = oracle.quantize_q4_k(W)
            return gk.QuantType.q4k(), b, oracle.dequant_matrix(oracle.Q4K, b, n, k)
        qt = qtype(gk, name)
        b = random_blocks(name, qt, n, k, seed)
        return qt, b, oracle_matrix(oracle, qt, b, n, k)
    qg, bg, wg_ref = make(gu, 2 * f, d, 91)
    qd, bd, wd_ref = make(dn, d, f, 92)
    w_gu, w_dn = K.upload(qg, 2 * f, d, bg), K.upload(qd, d, f, bd)
    scale = 2.5 if gu == "q4k" else 0.25  # random-byte blocks have weights of order 0.1 - 1: keep gate and up of order one
    xd = torch.from_numpy((np.random.default_rng(93).standard_normal((m, d)) * scale).astype(np.float32)).cuda().to(torch.bfloat16)
    x = xd.to(torch.float32).cpu().numpy()
    h = torch.empty((m, 2 * f), dtype=torch.bfloat16, device="cuda")
    y = K.ffn_prefill(w_gu, w_dn, xd, h=h).cpu().numpy()
    assert K.status() == 0
    def silu_mul(g):
        with np.errstate(over="ignore"):  # exp(-gate) may overflow to inf for a very negative gate: gate / inf = -0, the limit
            return ((g[:, :f] / (np.float32(1.0) + np.exp(-g[:, :f], dtype=np.float32))) * g[:, f:]).astype(np.float32)
    h_dev = h.to(torch.float32).cpu().numpy()
    assert oracle.rel_err(h_dev, oracle.gemm_f32_nt(x, wg_ref)) <= 1e-2 + 2.0 ** -8
    assert oracle.rel_err(y, oracle.gemm_f32_nt(silu_mul(h_dev), wd_ref)) <= 1e-2
    w_gu.free()
    w_dn.free()


def test_q6k_grouped_experts(K, gk, oracle, torch):
    """gllmk_gemm_grouped takes Q6_K experts through the same kernel (one launch for all groups); the formats without a
    tensor-core kernel are refused."""
    qt = qtype(gk, "q6_k")
    n, k, counts = 200, 3 * 256, [40, 0, 130, 7]
    blocks = [random_blocks("q6_k", qt, n, k, 500 + e) for e in range(len(counts))]
    ws = [K.upload(qt, n, k, b) for b in blocks]
    offs = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
    xd = torch.from_numpy(np.random.default_rng(51).standard_normal((int(offs[-1]), k)).astype(np.float32)).cuda().to(torch.bfloat16)
    x = xd.to(torch.float32).cpu().numpy()
    y = K.gemm_grouped(ws, xd, offs).to(torch.float32).cpu().numpy()
    assert K.status() == 0
    for e, b in enumerate(blocks):
        if counts[e]:
            ref = oracle.gemm_f32_nt(x[offs[e]:offs[e + 1]], oracle_matrix(oracle, qt, b, n, k))
            assert oracle.rel_err(y[offs[e]:offs[e + 1]], ref) <= 1e-2, e
    for w in ws:
        w.free()
    q8 = qtype(gk, "q8_k")
    w8 = K.upload(q8, 64, 256, random_blocks("q8_k", q8, 64, 256, 9))
    with pytest.raises(gk.GllmkError):
        K.gemm_grouped([w8], xd[:8, :256].contiguous(), [0, 8])
    w8.free()


@pytest.mark.parametrize("name", FORMATS)
def test_family_matmul_host(K, gk, oracle, name):
    """kquant_matmul / classic_matmul with host arrays: m weight rows, n batch columns, input [k, n], output [m, n]."""
    qt = qtype(gk, name)
    m, n, k = 50, 5, 2 * 256
    blocks = random_blocks(name, qt, m, k, 31)
    x = np.random.default_rng(32).standard_normal((k, n)).astype(np.float32)
    ref = oracle.quant_matmul(blocks, x, qt.id, m, n, k)
    out = np.empty((m, n), np.float32)
    fn = K.kquant_matmul if qt.block_size() == 256 else K.classic_matmul
    fn(blocks, x, out, qt, m, n, k)
    assert oracle.rel_err(out, ref) <= TOL
    wrong = K.classic_matmul if qt.block_size() == 256 else K.kquant_matmul
    with pytest.raises(gk.GllmkError):  # the reference panics for a format of the other family
        wrong(blocks, x, out, qt, m, n, k)


def test_linearity_large(K, gk, torch):
    """Size-independent property at a decode-sized Q6_K matrix: W(a x1 + b x2) = a W x1 + b W x2 to rounding."""
    qt = qtype(gk, "q6_k")
    n, k = 4096, 4096
    blocks = random_blocks("q6_k", qt, n, k, 41)
    w = K.upload(qt, n, k, blocks)
    g = torch.Generator(device="cuda").manual_seed(1)
    x1 = torch.randn(1, k, device="cuda", generator=g)
    x2 = torch.randn(1, k, device="cuda", generator=g)
    y = K.gemv(w, 0.5 * x1 - 2.0 * x2)
    y12 = 0.5 * K.gemv(w, x1) - 2.0 * K.gemv(w, x2)
    den = max(float(y12.abs().max()), 1e-6)
    assert float((y - y12).abs().max()) / den <= 1e-4
    # and against the f64 product with the decoded matrix
    ref = (K.dequant(w).double() @ x1.double().T).T
    assert float((K.gemv(w, x1).double() - ref).abs().max()) / float(ref.abs().max()) <= 1e-4
    w.free()


# ---- Kernels::gemv_q8 / gemm_q8 / gemv_q4 (src/traits.rs:500-510): Q8_K / Q4_K rows with optional scales -------------
def test_gemv_q8_gemm_q8_gemv_q4_reference_known_answers(gk, K):
    import json
    import os
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_known_answers.json")) as f:
        KA = json.load(f)
    c = KA["gemv_q8"]
    w_i8 = np.array(c["weight"], np.uint8).view(np.int8)  # the reference hands the blocks over as &[i8]
    assert abs(K.gemv_q8(w_i8, np.array(c["input"], np.float32), c["scale"], c["n"]) - c["expect"]) < c["tol"]
    c = KA["gemm_q8"]
    out = np.zeros(c["m"] * c["n"], np.float32)
    K.gemm_q8(np.array(c["weight"], np.uint8).view(np.int8), np.array(c["input"], np.float32), out, c["scales"], c["m"], c["n"], c["k"])
    assert np.abs(out - np.array(c["expect"], np.float32)).max() < c["tol"]
    c = KA["gemv_q4_zero"]
    assert abs(K.gemv_q4(np.array(c["weight"], np.uint8), np.array(c["input"], np.float32), c["scale"], c["n"]) - c["expect"]) < c["tol"]


@pytest.mark.parametrize("m,n,k,nscales", [(1, 64, 512, 0), (3, 100, 1024, 1), (20, 37, 768, 37), (5, 16, 256, 2)])
def test_gemm_q8_against_the_oracle(gk, K, oracle, m, n, k, nscales):
    """per-channel (n scales), per-tensor (1) and 'anything else = none' (src/cpu_kernels/mod.rs:2998-3026)."""
    rng = np.random.default_rng(m + n + k)
    nblk = n * (k // 256)
    b = rng.integers(0, 256, size=(nblk, 292), dtype=np.uint8)
    b[:, 0:4] = np.frombuffer(rng.uniform(-0.02, 0.02, nblk).astype(np.float32).tobytes(), np.uint8).reshape(nblk, 4)
    b = b.reshape(-1)
    x = rng.standard_normal((m, k)).astype(np.float32)
    scales = rng.uniform(0.5, 2.0, nscales).astype(np.float32) if nscales else None
    out = np.zeros((m, n), np.float32)
    K.gemm_q8(b.view(np.int8), x, out, scales, m, n, k)
    ref = oracle.gemm_q8(b, x, scales, m, n, k)
    assert oracle.rel_err(out, ref) <= 2e-3
    assert K.gemv_q8(b[: (k // 256) * 292].view(np.int8), x[0], 1.5, k) == pytest.approx(oracle.gemv_q8(b[: (k // 256) * 292], x[0], 1.5, k), rel=2e-3, abs=1e-5)
    with pytest.raises(gk.GllmkError) as e:  # k % 256 != 0: the reference asserts
        K.gemm_q8(b.view(np.int8), x, out, None, m, n, 100)
    assert e.value.status == gk.Status.INVALID_ARG
