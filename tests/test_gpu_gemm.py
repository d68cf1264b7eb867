"""Prefill GEMM (tcgen05) against the CPU oracle: decode of the packed bytes (reference formulas) followed by
the reference's f32 GEMM loop order.  Bar: max_i |y_i - ref_i| / max(|ref_i|, rms(ref)) <= 1e-2 (weights and
activations are staged in fp16, accumulation is f32)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
TOL = 1e-2


@pytest.fixture(scope="module")
def K(gk):
    k = gk.GpuKernels(0)
    yield k
    k.close()


def quantized(oracle, gk, fmt, n, k, seed):
    rng = np.random.default_rng(seed)
    W = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    if fmt == "q4k":
        b = oracle.quantize_q4_k(W)
        return gk.QuantType.q4k(), b, None, 1.0, oracle.dequant_matrix(oracle.Q4K, b, n, k)
    if fmt == "q8_0":
        b = oracle.quantize_q8_0(W)
        return gk.QuantType.q8_0(), b, None, 1.0, oracle.dequant_matrix(oracle.Q8_0, b, n, k)
    if fmt == "mxfp4":
        b, s = oracle.quantize_mxfp4(W)
        return gk.QuantType.mxfp4(32), b, s, 1.0, oracle.dequant_matrix(oracle.MXFP4, b, n, k, scales=s)
    b, g = oracle.quantize_nvfp4(W)
    return gk.QuantType.nvfp4(), b, None, g, oracle.dequant_matrix(oracle.NVFP4, b, n, k, global_scale=g)


def run_case(gk, K, oracle, fmt, n, k, m, seed, a_bf16=False, y_bf16=False):
    import torch
    qt, blocks, scales, g, wd = quantized(oracle, gk, fmt, n, k, seed)
    w = K.upload(qt, n, k, blocks, scales, g)
    x = np.random.default_rng(seed + 1).standard_normal((m, k)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    if a_bf16:
        xd = xd.to(torch.bfloat16)
        x = xd.to(torch.float32).cpu().numpy()
    y = K.gemm(w, xd, out_dtype=torch.bfloat16 if y_bf16 else torch.float32)
    torch.cuda.synchronize()
    assert K.status() == 0
    ref = oracle.gemm_f32_nt(x, wd) if m * n * k <= 2_000_000_000 else (x.astype(np.float64) @ wd.T.astype(np.float64))
    err = oracle.rel_err(y.to(torch.float32).cpu().numpy(), ref)
    w.free()
    return err


def test_gemm_single_tile_single_stage(gk, K, oracle):
    assert run_case(gk, K, oracle, "q8_0", 128, 64, 32, seed=1) <= TOL


def test_gemm_single_tile_pipeline_wraps(gk, K, oracle):
    assert run_case(gk, K, oracle, "q8_0", 128, 1024, 64, seed=2) <= TOL


@pytest.mark.parametrize("fmt", ["q4k", "q8_0", "mxfp4", "nvfp4"])
def test_gemm_formats(gk, K, oracle, fmt):
    assert run_case(gk, K, oracle, fmt, 384, 512, 256, seed=3) <= TOL


@pytest.mark.parametrize("fmt,n,k,m", [("q4k", 100, 256, 17), ("q4k", 300, 1280, 300), ("q8_0", 129, 192, 33),
                                       ("mxfp4", 200, 384, 513), ("nvfp4", 77, 448, 40)])
def test_gemm_ragged_shapes(gk, K, oracle, fmt, n, k, m):
    assert run_case(gk, K, oracle, fmt, n, k, m, seed=n + m) <= TOL


@pytest.mark.parametrize("fmt,n,k,m", [("q4k", 100, 256, 17), ("q8_0", 128, 1024, 32), ("q4k", 260, 768, 48), ("q8_0", 129, 192, 33)])
def test_gemm_few_tokens_tensor_core_path(gk, K, oracle, fmt, n, k, m):
    # with f32 in and out up to 16 tokens run as a pass of the decode kernel; bf16 activations keep the
    # call on the tcgen05 kernel with a narrow MMA N (32 / 64)
    assert run_case(gk, K, oracle, fmt, n, k, m, seed=n + m + 1, a_bf16=True) <= TOL


@pytest.mark.parametrize("m", [1, 7, 16])
def test_gemm_few_tokens_decode_pass(gk, K, oracle, m):
    # f32, m <= 16: one pass of the decode kernel, tighter bound
    assert run_case(gk, K, oracle, "q4k", 200, 512, m, seed=m) <= 2e-3
    assert run_case(gk, K, oracle, "q8_0", 200, 160, m, seed=m + 100) <= 2e-3


@pytest.mark.parametrize("m", [17, 32, 47, 48])
def test_gemm_few_tokens_f32_tensor_core(gk, K, oracle, m):
    # f32, 17 tokens and more: the tcgen05 kernel with a narrow MMA N (faster than two or three decode passes)
    assert run_case(gk, K, oracle, "q4k", 200, 512, m, seed=m) <= TOL
    assert run_case(gk, K, oracle, "q8_0", 200, 160, m, seed=m + 100) <= TOL


def test_gemm_bf16_in_bf16_out(gk, K, oracle):
    assert run_case(gk, K, oracle, "q4k", 256, 512, 96, seed=9, a_bf16=True, y_bf16=True) <= 1.5e-2


def test_gemm_rejects_bad_arguments(gk, K, oracle):
    import torch
    qt, blocks, _, _, _ = quantized(oracle, gk, "q8_0", 16, 96, 5)
    w = K.upload(qt, 16, 96, blocks)
    with pytest.raises(gk.GllmkError) as e:  # activation rows must be 16-byte aligned: lda % 4 for f32
        K.gemm(w, torch.zeros((64, 98), device="cuda")[:, :96])
    assert e.value.status == gk.Status.INVALID_ARG
    w.free()


@pytest.mark.parametrize("fmt,n,k,m", [("q4k", 37966, 256, 200), ("q8_0", 19008, 320, 300), ("nvfp4", 37966, 256, 130)])
def test_gemm_two_row_tiles_per_cta(gk, K, oracle, fmt, n, k, m):
    # enough 128-row tiles that a CTA takes two of them (one activation tile feeds two accumulators);
    # 297 tiles: the last CTA has a single tile
    assert run_case(gk, K, oracle, fmt, n, k, m, seed=n % 1000 + m, a_bf16=(fmt == "nvfp4")) <= TOL


def test_gemm_q8_0_ragged_k(gk, K, oracle):
    # k = 96: three blocks of a group of eight; the rest of the 256-wide k-step is zero padding
    assert run_case(gk, K, oracle, "q8_0", 144, 96, 40, seed=15) <= 1e-2


def test_gemm_fp4_weights_ragged_k(gk, K, oracle):
    # k not a multiple of 256: the FP4 planes are padded with zero codes
    assert run_case(gk, K, oracle, "mxfp4", 128, 320, 64, seed=16, a_bf16=True) <= 1e-2
    assert run_case(gk, K, oracle, "nvfp4", 128, 192, 64, seed=17, a_bf16=True) <= 1e-2


@pytest.mark.parametrize("fmt,n,k,m,split", [("q8_0", 19072, 2048, 64, 3), ("q4k", 38400, 1024, 300, 2), ("q4k", 19072, 2048, 200, 0),
                                             ("nvfp4", 19072, 1280, 96, 5)])
def test_gemm_tail_tiles_split_along_k(gk, K, oracle, fmt, n, k, m, split):
    """More tiles than SMs: the tiles of the last, partly filled wave are cut along k into units whose partial
    accumulators are added by the last unit to finish.  Forced split counts and the automatic choice, against the
    oracle and against the unsplit launch (same products, another summation order: f32 rounding apart)."""
    import torch
    qt, blocks, scales, g, wd = quantized(oracle, gk, fmt, n, k, seed=n % 977 + m)
    w = K.upload(qt, n, k, blocks, scales, g)
    x = torch.from_numpy(np.random.default_rng(m).standard_normal((m, k)).astype(np.float32)).cuda().to(torch.bfloat16)
    K.set("gemm_tail_split", 1)
    try:
        y_whole = K.gemm(w, x).clone()
        K.set("gemm_tail_split", split)
        y_split = K.gemm(w, x).clone()
        y_again = K.gemm(w, x)  # the arrival counters reset themselves; and the sum order is fixed: bit-identical
    finally:
        K.set("gemm_tail_split", 0)
    torch.cuda.synchronize()
    assert K.status() == 0
    assert torch.equal(y_split, y_again)
    scale = y_whole.abs().max().item()
    assert (y_split - y_whole).abs().max().item() <= 1e-5 * scale
    rows = np.r_[0:64, n // 2:n // 2 + 64, n - 64:n]  # the split tiles are the last ones
    ref = oracle.gemm_f32_nt(x.to(torch.float32).cpu().numpy(), wd[rows])
    assert oracle.rel_err(y_split.cpu().numpy()[:, rows], ref) <= TOL
    w.free()


# ---- both operands FP4: native block-scaled MMA ---------------------------------------------------
def run_fp4_case(gk, K, oracle, fmt, n, k, m, seed):
    import torch
    rng = np.random.default_rng(seed)
    W = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    X = rng.standard_normal((m, k)).astype(np.float32)
    if fmt == "nvfp4":
        qt = gk.QuantType.nvfp4()
        wb, gw = oracle.quantize_nvfp4(W)
        xb, gx = oracle.quantize_nvfp4(X)
        wd = oracle.dequant_matrix(oracle.NVFP4, wb, n, k, global_scale=gw)
        xd = oracle.dequant_matrix(oracle.NVFP4, xb, m, k, global_scale=gx)
        w, x = K.upload(qt, n, k, wb, None, gw), K.upload(qt, m, k, xb, None, gx)
    else:
        qt = gk.QuantType.mxfp4(32)
        wb, ws = oracle.quantize_mxfp4(W)
        xb, xs = oracle.quantize_mxfp4(X)
        wd = oracle.dequant_matrix(oracle.MXFP4, wb, n, k, scales=ws)
        xd = oracle.dequant_matrix(oracle.MXFP4, xb, m, k, scales=xs)
        w, x = K.upload(qt, n, k, wb, ws), K.upload(qt, m, k, xb, xs)
    y = K.gemm_fp4(w, x)
    torch.cuda.synchronize()
    assert K.status() == 0
    ref = oracle.gemm_f32_nt(xd, wd) if m * n * k <= 2_000_000_000 else (xd.astype(np.float64) @ wd.T.astype(np.float64))
    err = oracle.rel_err(y.cpu().numpy(), ref)
    w.free()
    x.free()
    return err


def test_gemm_fp4_nvfp4_single_tile(gk, K, oracle):
    assert run_fp4_case(gk, K, oracle, "nvfp4", 128, 256, 128, seed=1) <= 2e-3


def test_gemm_fp4_nvfp4_two_token_groups(gk, K, oracle):
    assert run_fp4_case(gk, K, oracle, "nvfp4", 128, 512, 256, seed=2) <= 2e-3


@pytest.mark.parametrize("n,k,m", [(384, 2048, 512), (200, 768, 300), (130, 1280, 77)])
def test_gemm_fp4_nvfp4_shapes(gk, K, oracle, n, k, m):
    assert run_fp4_case(gk, K, oracle, "nvfp4", n, k, m, seed=n + m) <= 2e-3


@pytest.mark.parametrize("n,k,m", [(128, 256, 128), (300, 1024, 384)])
def test_gemm_fp4_mxfp4(gk, K, oracle, n, k, m):
    assert run_fp4_case(gk, K, oracle, "mxfp4", n, k, m, seed=n + m) <= 2e-3


@pytest.mark.parametrize("fmt,n,k,m", [("nvfp4", 256, 256, 256), ("nvfp4", 128, 512, 300), ("nvfp4", 384, 1024, 129), ("nvfp4", 640, 768, 513),
                                       ("nvfp4", 1100, 2560, 777), ("mxfp4", 256, 512, 256), ("mxfp4", 900, 1280, 600),
                                       ("nvfp4", 512, 512, 193), ("nvfp4", 260, 1536, 1000)])
@pytest.mark.parametrize("variant", [1, 2, 3])
def test_gemm_fp4_cta_pair_kernel(gk, K, oracle, fmt, n, k, m, variant):
    """m > 128 runs on a persistent CTA-pair kernel (variant 1: one 256-token accumulator; 2: two of 192 tokens, whose tiles
    straddle the 128-token groups of the activation planes; 3: two of 128): an odd number of 128-row groups (the pair's
    second CTA has no rows), token counts that leave part of a tile empty or ragged, more k-steps than pipeline stages,
    several tiles per pair — against the oracle, and against the one-CTA kernel."""
    K.set("gemm_fp4_pair", variant)
    try:
        assert run_fp4_case(gk, K, oracle, fmt, n, k, m, seed=n + m) <= 2e-3
    finally:
        K.set("gemm_fp4_pair", 1)
    K.set("gemm_fp4_pair", variant)
    import torch
    rng = np.random.default_rng(n * m)
    W = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    X = rng.standard_normal((m, k)).astype(np.float32)
    if fmt == "nvfp4":
        qt = gk.QuantType.nvfp4()
        (wb, gw), (xb, gx) = oracle.quantize_nvfp4(W), oracle.quantize_nvfp4(X)
        w, x = K.upload(qt, n, k, wb, None, gw), K.upload(qt, m, k, xb, None, gx)
    else:
        qt = gk.QuantType.mxfp4(32)
        (wb, ws), (xb, xs) = oracle.quantize_mxfp4(W), oracle.quantize_mxfp4(X)
        w, x = K.upload(qt, n, k, wb, ws), K.upload(qt, m, k, xb, xs)
    y_pair = K.gemm_fp4(w, x, out_dtype=torch.bfloat16).clone()
    K.set("gemm_fp4_pair", 0)
    try:
        y_one = K.gemm_fp4(w, x, out_dtype=torch.bfloat16)
    finally:
        K.set("gemm_fp4_pair", 1)
    torch.cuda.synchronize()
    assert K.status() == 0
    # the same products in the same k order: equal up to the last bf16 bit of the output
    diff = (y_pair.float() - y_one.float()).abs().max().item()
    assert diff <= 2.0 ** -7 * y_one.float().abs().max().item(), diff
    w.free()
    x.free()


@pytest.mark.parametrize("variant", [1, 2, 3])
def test_gemm_fp4_cta_pair_kernel_many_tiles(gk, K, oracle, variant):
    """More tiles than resident pairs: every pair walks several tiles, the accumulator hand-over between the MMA
    thread and the sixteen epilogue warps of a pair is exercised over many rounds."""
    import torch
    n, k, m = 6144, 512, 2048  # 24 row pairs x 8 / 11 / 16 token tiles on 74 pairs
    qt = gk.QuantType.nvfp4()
    g = torch.Generator(device="cuda").manual_seed(5)
    W = torch.randn((n, k), generator=g, device="cuda") * 0.02
    X = torch.randn((m, k), generator=g, device="cuda")
    wb, gw = K.quantize(qt, W)
    xb, gx = K.quantize(qt, X)
    w, x = K.upload(qt, n, k, wb, None, gw), K.upload(qt, m, k, xb, None, gx)
    K.set("gemm_fp4_pair", variant)
    try:
        y = K.gemm_fp4(w, x)
    finally:
        K.set("gemm_fp4_pair", 1)
    torch.cuda.synchronize()
    assert K.status() == 0
    wd = oracle.dequant_matrix(oracle.NVFP4, wb.cpu().numpy(), n, k, global_scale=gw)
    xd = oracle.dequant_matrix(oracle.NVFP4, xb.cpu().numpy(), m, k, global_scale=gx)
    rows = np.r_[0:64, 3000:3064, n - 64:n]
    assert oracle.rel_err(y.cpu().numpy()[:, rows], oracle.gemm_f32_nt(xd, wd[rows])) <= 2e-3
    w.free()
    x.free()


# ---- FP4 weights on the decode kernel, and host batches that land on the tensor-core kernel -------------
@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
@pytest.mark.parametrize("n,k", [(200, 384), (128, 256), (1000, 2048)])
def test_fp4_weights_decode_kernel(gk, K, oracle, fmt, n, k):
    import torch
    qt, blocks, scales, g, wd = quantized(oracle, gk, fmt, n, k, 21 + n)
    w = K.upload(qt, n, k, blocks, scales, g)
    for m in (1, 3, 5, 8, 16):
        x = np.random.default_rng(m).standard_normal((m, k)).astype(np.float32)
        ref = oracle.gemm_f32_nt(x, wd)
        y = K.gemv(w, torch.from_numpy(x).cuda()).cpu().numpy()
        assert oracle.rel_err(y, ref) <= 2e-3, (fmt, m)
    x = np.random.default_rng(99).standard_normal((5, k)).astype(np.float32)
    ref = oracle.gemm_f32_nt(x, wd)
    assert oracle.rel_err(K.matmul_host(w, x), ref) <= 2e-3
    assert oracle.rel_err(K.matmul_host(w, np.ascontiguousarray(x.T), ref_layout=True), ref.T) <= 2e-3
    # 16 f32 tokens through gllmk_gemm: one pass of the decode kernel
    x = np.random.default_rng(98).standard_normal((16, k)).astype(np.float32)
    assert oracle.rel_err(K.gemm(w, torch.from_numpy(x).cuda()).cpu().numpy(), oracle.gemm_f32_nt(x, wd)) <= 2e-3
    assert K.status() == 0
    w.free()


def test_fp4_decode_negative_zero_codes_and_scale_specials(gk, K, oracle):
    """Every E2M1 code (incl. -0) in every position, E8M0 scales 0 (2^-127) and 254, NaN scale -> NaN row."""
    import torch
    n, k = 16, 256
    rng = np.random.default_rng(4)
    codes = rng.integers(0, 256, size=(n, k // 2), dtype=np.uint8)
    codes[0, :16] = np.arange(16, dtype=np.uint8) * 17  # both nibbles run through all 16 codes
    scales = rng.integers(118, 132, size=(n, k // 32), dtype=np.uint8)
    scales[1, 0], scales[2, 3], scales[3, 1] = 0, 200, 255
    w = K.upload(gk.QuantType.mxfp4(32), n, k, codes, scales)
    wd = oracle.dequant_matrix(oracle.MXFP4, codes, n, k, scales=scales)
    x = rng.standard_normal((2, k)).astype(np.float32)
    y = K.gemv(w, torch.from_numpy(x).cuda()).cpu().numpy()
    ref = oracle.gemm_f32_nt(x, wd)
    assert np.isnan(y[:, 3]).all() and np.isnan(ref[:, 3]).all()
    ok = [r for r in range(n) if r != 3]
    assert oracle.rel_err(y[:, ok], ref[:, ok]) <= 2e-3
    w.free()


def test_matmul_host_prefill_batch_uses_one_gemm(gk, K, oracle):
    n, k, m = 300, 512, 130
    qt, blocks, _, _, wd = quantized(oracle, gk, "q4k", n, k, 22)
    w = K.upload(qt, n, k, blocks)
    x = np.random.default_rng(5).standard_normal((m, k)).astype(np.float32)
    assert oracle.rel_err(K.matmul_host(w, x), oracle.gemm_f32_nt(x, wd)) <= TOL
    w.free()


# ---- mixture of experts: several weights, one launch ---------------------------------------------------
@pytest.mark.parametrize("fmt,counts,a_bf16", [("mxfp4", [70, 0, 128, 33, 129], True), ("q4k", [300, 17, 256], False),
                                               ("nvfp4", [5, 5, 5, 5], True), ("q8_0", [40] * 34, False)])
def test_gemm_grouped_matches_per_expert_products(gk, K, oracle, fmt, counts, a_bf16):
    import torch
    n, k = 200, 256
    experts = [quantized(oracle, gk, fmt, n, k, 100 + e) for e in range(len(counts))]
    ws = [K.upload(qt, n, k, b, s, g) for (qt, b, s, g, _) in experts]
    offs = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
    x = np.random.default_rng(77).standard_normal((int(offs[-1]), k)).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    if a_bf16:
        xd = xd.to(torch.bfloat16)
        x = xd.to(torch.float32).cpu().numpy()
    y = K.gemm_grouped(ws, xd, offs).cpu().numpy()
    torch.cuda.synchronize()
    assert K.status() == 0
    for e, (_, _, _, _, wd) in enumerate(experts):
        if counts[e]:
            ref = oracle.gemm_f32_nt(x[offs[e]:offs[e + 1]], wd)
            assert oracle.rel_err(y[offs[e]:offs[e + 1]], ref) <= TOL, (fmt, e)
    for w in ws:
        w.free()


@pytest.mark.parametrize("fmt,counts,split", [("mxfp4", [150, 97, 160], 0), ("q4k", [60, 1, 64, 33], 3), ("q8_0", [128, 128], 2)])
def test_gemm_grouped_tail_tiles_split_along_k(gk, K, oracle, fmt, counts, split):
    """A grouped launch with more tiles than SMs: the last wave's tiles are cut along k exactly as in a plain product (every
    unit finds its expert's weights and token tile through the same tables).  Against the unsplit launch and the oracle."""
    import torch
    n, k = 12800, 1280  # 100 row tiles per expert
    experts = [quantized(oracle, gk, fmt, n, k, 300 + e) for e in range(len(counts))]
    ws = [K.upload(qt, n, k, b, s, g) for (qt, b, s, g, _) in experts]
    offs = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
    xd = torch.from_numpy(np.random.default_rng(78).standard_normal((int(offs[-1]), k)).astype(np.float32)).cuda().to(torch.bfloat16)
    x = xd.to(torch.float32).cpu().numpy()
    K.set("gemm_tail_split", 1)
    try:
        y_whole = K.gemm_grouped(ws, xd, offs).cpu().numpy()
        K.set("gemm_tail_split", split)
        y_split = K.gemm_grouped(ws, xd, offs).cpu().numpy()
        y_again = K.gemm_grouped(ws, xd, offs).cpu().numpy()
    finally:
        K.set("gemm_tail_split", 0)
    assert K.status() == 0
    assert np.array_equal(y_split, y_again)
    rows = np.random.default_rng(9).choice(n, size=256, replace=False)
    for e, (_, _, _, _, wd) in enumerate(experts):
        ref = oracle.gemm_f32_nt(x[offs[e]:offs[e + 1]], wd[rows])
        assert oracle.rel_err(y_split[offs[e]:offs[e + 1]][:, rows], ref) <= TOL, (fmt, e)
        assert oracle.rel_err(y_split[offs[e]:offs[e + 1]], y_whole[offs[e]:offs[e + 1]]) <= 1e-5, (fmt, e)
    for w in ws:
        w.free()


def test_gemm_grouped_rejects_mismatched_weights(gk, K, oracle):
    import torch
    qa, ba, _, _, _ = quantized(oracle, gk, "q8_0", 64, 64, 1)
    qb, bb, _, _, _ = quantized(oracle, gk, "q8_0", 80, 64, 2)
    wa, wb = K.upload(qa, 64, 64, ba), K.upload(qb, 80, 64, bb)
    with pytest.raises(gk.GllmkError) as e:
        K.gemm_grouped([wa, wb], torch.zeros((8, 64), device="cuda"), [0, 4, 8])
    assert e.value.status == gk.Status.INVALID_ARG
    with pytest.raises(gk.GllmkError) as e:
        K.gemm_grouped([wa, wa], torch.zeros((8, 64), device="cuda"), [0, 5, 3])
    assert e.value.status == gk.Status.INVALID_ARG
    wa.free()
    wb.free()


def test_gemm_more_token_tiles_than_one_launch_holds(gk, K, oracle):
    # 17000 tokens = 67 tiles of 256: the launcher cuts the token range into launches of at most 64 tiles
    assert run_case(gk, K, oracle, "q8_0", 128, 64, 17000, seed=31) <= TOL


# ---- the gated feed-forward block for prefill batches: two tensor-core products, bf16 intermediate -------------------
@pytest.mark.parametrize("fmt,d,f,m,x_bf16", [("q4k", 512, 768, 96, False), ("q4k", 1024, 2048, 300, True), ("q8_0", 256, 384, 40, True),
                                              ("mxfp4", 512, 1024, 130, True)])
def test_ffn_prefill_swiglu(gk, K, oracle, fmt, d, f, m, x_bf16):
    """y = W_down (silu(gate) * up), [gate | up] = W_gate_up x, against the oracle's chain: the reference's f32 GEMM,
    scalar_swiglu, the reference's f32 GEMM.  The intermediate lives in bf16 and both products stage fp16 operands:
    each product holds the 1e-2 bar given the same inputs; the two-product chain against the all-f32 chain 2e-2."""
    import torch
    qt, b_gu, s_gu, g_gu, wd_gu = quantized(oracle, gk, fmt, 2 * f, d, 71)
    _, b_dn, s_dn, g_dn, wd_dn = quantized(oracle, gk, fmt, d, f, 72)
    w_gu, w_dn = K.upload(qt, 2 * f, d, b_gu, s_gu, g_gu), K.upload(qt, d, f, b_dn, s_dn, g_dn)
    # weights ~N(0, 0.02): scale x so that gate and up are of order one and SwiGLU is not linear
    x = (np.random.default_rng(73).standard_normal((m, d)) * 2.5).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    if x_bf16:
        xd = xd.to(torch.bfloat16)
        x = xd.to(torch.float32).cpu().numpy()
    h = torch.empty((m, 2 * f), dtype=torch.bfloat16, device="cuda")
    y = K.ffn_prefill(w_gu, w_dn, xd, h=h).cpu().numpy()
    torch.cuda.synchronize()
    assert K.status() == 0
    silu_mul = lambda gu: ((gu[:, :f] / (np.float32(1.0) + np.exp(-gu[:, :f], dtype=np.float32))) * gu[:, f:]).astype(np.float32)
    h_ref = oracle.gemm_f32_nt(x, wd_gu)
    assert oracle.rel_err(h.to(torch.float32).cpu().numpy(), h_ref) <= 1e-2
    # second product alone: from the h the device produced
    y_from_h = oracle.gemm_f32_nt(silu_mul(h.to(torch.float32).cpu().numpy()), wd_dn)
    assert oracle.rel_err(y, y_from_h) <= 1e-2
    # the whole chain in f32
    y_ref = oracle.gemm_f32_nt(silu_mul(h_ref), wd_dn)
    assert oracle.rel_err(y, y_ref) <= 2e-2
    with pytest.raises(gk.GllmkError) as e:  # shapes that do not chain
        K.ffn_prefill(w_dn, w_dn, xd)
    assert e.value.status == gk.Status.INVALID_ARG
    w_gu.free()
    w_dn.free()
