"""Properties of the CPU oracle and of this project's quantizers (CPU only)."""
import numpy as np
import pytest
from hypothesis import given, settings, strategies as st


def test_q4k_block_dot_equals_decode_dot(oracle):
    rng = np.random.default_rng(0)
    import ctypes as C
    for _ in range(50):
        blk = rng.integers(0, 256, 144, dtype=np.uint8)
        blk[0:2] = np.frombuffer(np.float16(rng.uniform(0.001, 0.1)).tobytes(), np.uint8)
        blk[2:4] = np.frombuffer(np.float16(rng.uniform(0.001, 0.1)).tobytes(), np.uint8)
        x = rng.standard_normal(256).astype(np.float32)
        w = oracle.dequant_q4_k(blk)
        acc = np.float32(0)
        for i in range(256):
            acc = np.float32(acc + np.float32(w[i] * x[i]))
        got = oracle.lib().gko_dot_q4_k(blk.ctypes.data_as(C.POINTER(C.c_uint8)), x.ctypes.data_as(C.POINTER(C.c_float)))
        assert np.float32(got) == acc
        for e in range(0, 256, 17):
            assert oracle.lib().gko_q4k_element(blk.ctypes.data_as(C.POINTER(C.c_uint8)), e) == w[e]


@settings(max_examples=50, deadline=None)
@given(st.binary(min_size=144, max_size=144))
def test_q4k_scale_pack_roundtrip(oracle, raw):
    """get_scale_min_k4 over random bytes yields 6-bit values and re-packing them gives the bytes back."""
    blk = np.frombuffer(raw, np.uint8).copy()
    sc, m = oracle.q4k_scales(blk)
    assert sc.max() < 64 and m.max() < 64
    s = np.zeros(12, np.uint8)
    for j in range(4):
        s[j] = sc[j] | ((sc[j + 4] >> 4) << 6)
        s[j + 4] = m[j] | ((m[j + 4] >> 4) << 6)
        s[j + 8] = (sc[j + 4] & 15) | ((m[j + 4] & 15) << 4)
    assert (s == blk[4:16]).all()


@pytest.mark.parametrize("fmt", ["q4k", "q8_0", "mxfp4", "nvfp4"])
def test_quantizers_reconstruct_within_format_precision(oracle, fmt):
    rng = np.random.default_rng(3)
    n, k = 8, 512
    W = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    if fmt == "q4k":
        wd = oracle.dequant_matrix(oracle.Q4K, oracle.quantize_q4_k(W), n, k)
        tol = 0.08
    elif fmt == "q8_0":
        wd = oracle.dequant_matrix(oracle.Q8_0, oracle.quantize_q8_0(W), n, k)
        tol = 0.01
    elif fmt == "mxfp4":
        b, s = oracle.quantize_mxfp4(W)
        wd = oracle.dequant_matrix(oracle.MXFP4, b, n, k, scales=s)
        tol = 0.2
        amax = np.abs(W.reshape(-1, 32)).max(1)
        scale = np.array([oracle.lib().gko_decode_e8m0_scale(int(v)) for v in s])
        assert (scale * 6.0 >= amax).all() and (scale * 3.0 < amax).all()  # smallest covering power of two
    else:
        b, g = oracle.quantize_nvfp4(W)
        wd = oracle.dequant_matrix(oracle.NVFP4, b, n, k, global_scale=g)
        tol = 0.15
    err = np.abs(wd - W).max() / np.abs(W).max()
    assert err < tol, err


def test_zero_and_constant_blocks(oracle):
    z = np.zeros((1, 256), np.float32)
    assert not oracle.dequant_matrix(oracle.Q4K, oracle.quantize_q4_k(z), 1, 256).any()
    assert not oracle.dequant_matrix(oracle.Q8_0, oracle.quantize_q8_0(z), 1, 256).any()
    b, s = oracle.quantize_mxfp4(z)
    assert (s == 127).all() and not oracle.dequant_matrix(oracle.MXFP4, b, 1, 256, scales=s).any()
    b, g = oracle.quantize_nvfp4(z)
    assert g == 1.0 and not oracle.dequant_matrix(oracle.NVFP4, b, 1, 256, global_scale=g).any()


def test_matmul_conventions_and_threads(oracle):
    rng = np.random.default_rng(5)
    n, k, m = 24, 512, 3
    W = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    for qt, blocks in ((oracle.Q4K, oracle.quantize_q4_k(W)), (oracle.Q8_0, oracle.quantize_q8_0(W))):
        y = oracle.quant_matmul(blocks, np.ascontiguousarray(x.T), qt, n, m, k)        # [n, m]
        y4 = oracle.quant_matmul(blocks, np.ascontiguousarray(x.T), qt, n, m, k, threads=4)
        assert (y == y4).all()
        wd = oracle.dequant_matrix(qt, blocks, n, k)
        truth = oracle.gemm_f64_nt(x, wd)                                              # [m, n]
        assert oracle.rel_err(y.T, truth) < 1e-5
        if qt == oracle.Q4K:
            assert (oracle.gemm_q4(blocks, x, None, m, n, k) == y.T).all()


def test_mxfp4_inline_split(oracle):
    import ctypes as C
    rng = np.random.default_rng(9)
    nb = 12
    inline = rng.integers(0, 256, nb * 17, dtype=np.uint8)
    blocks, scales = np.empty(nb * 16, np.uint8), np.empty(nb, np.uint8)
    p = lambda a: a.ctypes.data_as(C.POINTER(C.c_uint8))
    oracle.lib().gko_mxfp4_split(p(inline), p(blocks), p(scales), nb, 32)
    assert (scales == inline.reshape(nb, 17)[:, 0]).all()
    assert (blocks.reshape(nb, 16) == inline.reshape(nb, 17)[:, 1:]).all()
