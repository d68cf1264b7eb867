"""W8A8 integer GEMM (tcgen05 kind::i8) and its dequantize epilogue.  The oracle is an exact integer matmul
(numpy int64), the same reference the project's own tests use (ref_matmul_i32, src/tests_int8.rs:8-20); the
first four cases are that file's test patterns (:21-108), the epilogue case its :110-136."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K(gk):
    k = gk.GpuKernels(0)
    yield k
    k.close()


def ref_i32(a, b):
    return (a.astype(np.int64) @ b.astype(np.int64)).astype(np.int32)


def pattern(m, n, k, amod, bmod, boff):
    a = (np.arange(m * k) % amod).astype(np.uint8).reshape(m, k)
    b = ((np.arange(k * n) % bmod) - boff).astype(np.int8).reshape(k, n)
    return a, b


@pytest.mark.parametrize("m,n,k,amod,bmod,boff", [(2, 4, 8, 128, 64, 32), (14, 32, 64, 200, 100, 50), (17, 37, 13, 250, 120, 60),
                                                 (64, 128, 512, 255, 127, 63)])
def test_reference_test_patterns_host_call(gk, K, m, n, k, amod, bmod, boff):
    a, b = pattern(m, n, k, amod, bmod, boff)
    c = K.gemm_int8_host(a, b)
    assert np.array_equal(c, ref_i32(a, b))
    assert K.status() == 0


@pytest.mark.parametrize("m,n,k", [(1, 128, 128), (33, 200, 300), (129, 257, 1000), (300, 130, 4096), (512, 1024, 2048)])
@pytest.mark.parametrize("layout_kn", [True, False])
def test_gemm_int8_resident_weight_bit_exact(gk, K, m, n, k, layout_kn):
    import torch
    rng = np.random.default_rng(m + n + k)
    a = rng.integers(0, 256, size=(m, k), dtype=np.uint8)
    b = rng.integers(-128, 128, size=(k, n), dtype=np.int8)
    w = K.upload_int8(b if layout_kn else np.ascontiguousarray(b.T), layout_kn=layout_kn)
    c = K.gemm_int8(w, torch.from_numpy(a).cuda()).cpu().numpy()
    assert np.array_equal(c, ref_i32(a, b))
    assert K.status() == 0
    w.free()


@pytest.mark.parametrize("pair", [0, 2])
def test_gemm_int8_two_row_tiles_per_cta(gk, K, pair):
    """299 row tiles and a 256-token tile.  One-CTA kernel: a CTA takes two row tiles (two accumulators share the
    activation stage), the last CTA has one.  CTA-pair kernel: 150 row pairs on 74 resident pairs, the last pair's second
    CTA has no rows."""
    import torch
    m, n, k = 200, 128 * 299 - 50, 256
    rng = np.random.default_rng(9)
    a = rng.integers(0, 256, size=(m, k), dtype=np.uint8)
    b = rng.integers(-128, 128, size=(k, n), dtype=np.int8)
    w = K.upload_int8(b)
    K.set("gemm_i8_pair", pair)
    try:
        c = K.gemm_int8(w, torch.from_numpy(a).cuda()).cpu().numpy()
    finally:
        K.set("gemm_i8_pair", 1)
    assert np.array_equal(c, ref_i32(a, b))
    assert K.status() == 0
    w.free()


@pytest.mark.parametrize("m,n,k", [(129, 128, 128), (257, 300, 1000), (700, 2500, 1152), (2048, 4000, 640), (513, 130, 4096)])
def test_gemm_int8_cta_pair_kernel(gk, K, m, n, k):
    """m > 128 runs on the persistent CTA-pair kernel: token counts that leave the second half of a tile empty or ragged,
    an odd number of 128-row groups, more k-steps than stages, more tiles than resident pairs (both accumulators in
    rotation over many tiles) — bit-exact, and equal to the one-CTA kernel."""
    import torch
    rng = np.random.default_rng(m + n + k)
    a = rng.integers(0, 256, size=(m, k), dtype=np.uint8)
    b = rng.integers(-128, 128, size=(k, n), dtype=np.int8)
    w = K.upload_int8(b)
    ad = torch.from_numpy(a).cuda()
    K.set("gemm_i8_pair", 2)  # always (the default picks the pair kernel when its estimate is lower)
    try:
        c_pair = K.gemm_int8(w, ad).clone()
        c_again = K.gemm_int8(w, ad).clone()
        K.set("gemm_i8_pair", 0)
        c_one = K.gemm_int8(w, ad).clone()
    finally:
        K.set("gemm_i8_pair", 1)
    assert K.status() == 0
    assert np.array_equal(c_pair.cpu().numpy(), ref_i32(a, b))
    assert torch.equal(c_pair, c_again) and torch.equal(c_pair, c_one)
    w.free()


def test_gemm_int8_extreme_values_and_strided_views(gk, K):
    """255 x -128 everywhere (the largest magnitude per product), and A / C that are column slices of wider buffers."""
    import torch
    m, n, k = 70, 96, 640
    a_full = torch.full((m, k + 7), 255, dtype=torch.uint8, device="cuda")
    b = np.full((k, n), -128, np.int8)
    w = K.upload_int8(b)
    c_full = torch.zeros((m, n + 4), dtype=torch.int32, device="cuda")
    K.gemm_int8(w, a_full[:, 3:3 + k], c=c_full[:, :n])
    assert (c_full[:, :n] == -128 * 255 * k).all().item() and (c_full[:, n:] == 0).all().item()
    w.free()


def test_dequantize_epilogue(gk, K):
    import torch
    n = 35
    c = (np.arange(n, dtype=np.int32) * 100 - 1700).reshape(1, n)
    cd = torch.from_numpy(c).cuda()
    out = K.dequantize_i32(cd, 0.5, 0.25).cpu().numpy()
    assert np.array_equal(out, (c.astype(np.float32) * np.float32(0.5)) * np.float32(0.25))
    bias = np.linspace(-1, 1, n, dtype=np.float32)
    v = (c.astype(np.float32) * np.float32(0.01)) * np.float32(0.1) + bias
    relu = K.dequantize_i32(cd, 0.01, 0.1, bias=torch.from_numpy(bias).cuda(), activation=1).cpu().numpy()
    assert np.array_equal(relu, np.where(v < 0, np.float32(0), v))
    silu = K.dequantize_i32(cd, 0.01, 0.1, bias=torch.from_numpy(bias).cuda(), activation=2).cpu().numpy()
    assert np.allclose(silu, v / (1.0 + np.exp(-v)), rtol=1e-6, atol=1e-7)
    gelu = K.dequantize_i32(cd, 0.01, 0.1, bias=torch.from_numpy(bias).cuda(), activation=3).cpu().numpy()
    inner = np.float32(0.7978845608) * (v + np.float32(0.044715) * v * v * v)
    assert np.allclose(gelu, 0.5 * v * (1.0 + np.tanh(inner)), rtol=1e-5, atol=1e-6)


def test_int8_argument_checks(gk, K, oracle):
    import torch
    with pytest.raises(gk.GllmkError) as e:
        K.dequantize_i32(torch.zeros((1, 4), dtype=torch.int32, device="cuda"), 1.0, 1.0, activation=9)
    assert e.value.status == gk.Status.UNSUPPORTED
    w = K.upload_int8(np.zeros((64, 32), np.int8))
    with pytest.raises(gk.GllmkError) as e:  # an int8 weight is not a block-quantized weight
        K.gemm(w, torch.zeros((64, 64), device="cuda"))
    assert e.value.status == gk.Status.UNSUPPORTED
    with pytest.raises(gk.GllmkError) as e:  # lda smaller than k
        K.gemm_int8(w, torch.zeros((4, 32), dtype=torch.uint8, device="cuda"))
    assert e.value.status == gk.Status.INVALID_ARG
    w.free()
    assert K.gemm_int8_host(np.zeros((0, 8), np.uint8), np.zeros((8, 4), np.int8)).shape == (0, 4)


# ---- the activation half of W8A8: per-tensor f32 -> int8 (src/compiler/quant_convert.rs:165-177) -------------------------
@pytest.mark.parametrize("rows,k", [(1, 7), (5, 64), (33, 1000), (257, 4096)])
def test_activation_quantizer_bit_exact(gk, K, oracle, rows, k):
    import torch
    rng = np.random.default_rng(rows + k)
    x = rng.standard_normal((rows, k)).astype(np.float32) * 3.0
    x[0, 0] = 0.0
    if k > 8:
        x[-1, 3] = -x.__abs__().max() * 1.5   # the maximum is negative: -127 after rounding
        x[0, 5] = np.float32(0.5) * np.float32(np.abs(x).max() / 127.0)  # a tie: rounds away from zero
    q_ref, s_ref = oracle.quantize_int8_per_tensor(x)
    xd = torch.from_numpy(x).cuda()
    q, s = K.quantize_act_int8(xd)
    assert s.item() == s_ref
    assert np.array_equal(q.cpu().numpy(), q_ref)
    qu, s2 = K.quantize_act_int8(xd, as_unsigned=True)
    assert s2.item() == s_ref
    assert np.array_equal(qu.cpu().numpy().astype(np.int16) - 128, q_ref.astype(np.int16))
    # a strided view (leading dimension larger than k) and an all-zero tensor
    wide = torch.zeros((rows, k + 9), device="cuda")
    wide[:, :k] = xd
    q3, _ = K.quantize_act_int8(wide[:, :k])
    assert np.array_equal(q3.cpu().numpy(), q_ref)
    qz, sz = K.quantize_act_int8(torch.zeros((rows, k), device="cuda"))
    assert sz.item() == 0.0 and not qz.cpu().numpy().any()


@pytest.mark.parametrize("m,n,k,act", [(1, 128, 256, 0), (37, 300, 1000, 0), (200, 513, 2048, 1), (64, 1024, 4096, 2)])
def test_w8a8_linear_against_the_reference_pipeline(gk, K, oracle, m, n, k, act):
    """quantize_from_fp32 -> gemm_int8 (exact s32) -> dequantize_i32_to_f32, as the reference chains them, evaluated with
    the oracle's quantizer, an int64 matmul and f32 arithmetic in the epilogue's order: bit-exact without an activation
    function, 1e-6 relative with one (expf / tanhf differ in the last bit between libm and the device)."""
    import torch
    rng = np.random.default_rng(m * n + k)
    x = (rng.standard_normal((m, k)) * 2.0).astype(np.float32)
    b = rng.integers(-128, 128, size=(k, n), dtype=np.int8)
    bias = rng.standard_normal(n).astype(np.float32)
    scale_b = np.float32(0.013)
    w = K.upload_int8(b, layout_kn=True)
    y = K.w8a8_linear(w, torch.from_numpy(x).cuda(), float(scale_b), bias=torch.from_numpy(bias).cuda(), activation=act).cpu().numpy()
    q, s = oracle.quantize_int8_per_tensor(x)
    c = (q.astype(np.int64) @ b.astype(np.int64)).astype(np.float32)
    ref = (c * np.float32(s)) * scale_b + bias
    if act == 1:
        ref = np.maximum(ref, 0)
    elif act == 2:
        ref = ref / (np.float32(1) + np.exp(-ref, dtype=np.float32))
    if act == 0:
        assert np.array_equal(y.view(np.uint32), ref.astype(np.float32).view(np.uint32))
    else:
        assert np.allclose(y, ref, rtol=2e-6, atol=1e-7)
    w.free()
