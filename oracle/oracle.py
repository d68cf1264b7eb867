"""ctypes/numpy front end of the CPU oracle (oracle/gllmk_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by the
cpu-baseline / reference legs of bench.py.  The product package never imports it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

Q4K, Q8_0, MXFP4, NVFP4 = 1, 2, 3, 4
Q6K, Q5K, Q4_0, Q5_0, Q8K = 6, 7, 8, 9, 10


def build(force: bool = False) -> None:
    """Compile the C restatement (both optimisation levels) next to its source."""
    targets = [os.path.join(_HERE, n) for n in ("libgllmk_oracle.so", "libgllmk_oracle_o1.so")]
    src = os.path.join(_HERE, "gllmk_oracle.c")
    if not force and all(os.path.exists(t) and os.path.getmtime(t) >= os.path.getmtime(src) for t in targets):
        return
    subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True, capture_output=True)


_u8p = C.POINTER(C.c_uint8)
_f32p = C.POINTER(C.c_float)
_f64p = C.POINTER(C.c_double)


def _p(a, t):
    return a.ctypes.data_as(t)


def _load(name: str) -> C.CDLL:
    build()
    lib = C.CDLL(os.path.join(_HERE, name))
    z = C.c_size_t
    sig = {
        "gko_f16_to_f32": (C.c_float, [C.c_uint16]),
        "gko_f32_to_f16": (C.c_uint16, [C.c_float]),
        "gko_block_size": (C.c_int, [C.c_int, C.c_int]),
        "gko_block_bytes": (C.c_int, [C.c_int, C.c_int]),
        "gko_q4k_scales": (None, [_u8p, _u8p, _u8p]),
        "gko_dequant_q4_k": (None, [_u8p, _f32p]),
        "gko_dot_q4_k": (C.c_float, [_u8p, _f32p]),
        "gko_q4k_element": (C.c_float, [_u8p, C.c_int]),
        "gko_dequant_q8_0": (None, [_u8p, _f32p]),
        "gko_dequant_block": (C.c_int, [C.c_int, _u8p, _f32p]),
        "gko_dot_q8_0": (C.c_float, [_u8p, _f32p]),
        "gko_e2m1": (C.c_float, [C.c_int]),
        "gko_decode_e8m0_scale": (C.c_float, [C.c_uint8]),
        "gko_dequant_mxfp4": (None, [_u8p, _u8p, _f32p, z, z]),
        "gko_e4m3_to_f32": (C.c_float, [C.c_uint8]),
        "gko_f32_to_e4m3": (C.c_uint8, [C.c_float]),
        "gko_dequant_nvfp4": (None, [_u8p, C.c_float, _f32p, z]),
        "gko_quant_matmul": (C.c_int, [_u8p, _f32p, _f32p, C.c_int, z, z, z]),
        "gko_quant_matmul_mt": (C.c_int, [_u8p, _f32p, _f32p, C.c_int, z, z, z, C.c_int]),
        "gko_gemm_q4": (C.c_int, [_u8p, _f32p, _f32p, _f32p, z, z, z, z]),
        "gko_gemv_q4": (C.c_float, [_u8p, _f32p, C.c_float, z]),
        "gko_gemm_q8": (C.c_int, [_u8p, _f32p, _f32p, _f32p, z, z, z, z]),
        "gko_gemv_q8": (C.c_float, [_u8p, _f32p, C.c_float, z]),
        "gko_quantize_int8_per_tensor": (C.c_float, [_f32p, C.POINTER(C.c_int8), z]),
        "gko_gemm_f32_nt": (None, [_f32p, _f32p, _f32p, z, z, z]),
        "gko_gemm_f64_nt": (None, [_f32p, _f32p, _f64p, z, z, z]),
        "gko_dequant_matrix": (C.c_int, [C.c_int, _u8p, _u8p, C.c_float, z, z, C.c_int, _f32p]),
        "gko_scalar_gemv_q8": (C.c_float, [C.POINTER(C.c_int8), _f32p, C.c_float, z]),
        "gko_scalar_gemv_q4": (C.c_float, [_u8p, _f32p, C.c_float, z]),
        "gko_scalar_gemm_q8": (None, [C.POINTER(C.c_int8), _f32p, _f32p, _f32p, z, z, z]),
        "gko_scalar_gemm_q4": (None, [_u8p, _f32p, _f32p, _f32p, z, z, z]),
        "gko_scalar_kquant_matmul": (None, [_u8p, _f32p, _f32p, z, z, z, z, z]),
        "gko_quantize_q4_k": (None, [_f32p, _u8p, z]),
        "gko_quantize_q8_0": (None, [_f32p, _u8p, z]),
        "gko_quantize_mxfp4": (None, [_f32p, _u8p, _u8p, z, z]),
        "gko_nvfp4_global": (C.c_float, [_f32p, z]),
        "gko_quantize_nvfp4": (None, [_f32p, C.c_float, _u8p, z]),
        "gko_mxfp4_split": (None, [_u8p, _u8p, _u8p, z, z]),
        "gko_bench_gemv_q4_rows": (None, [_u8p, _f32p, _f32p, _f32p, z, z]),
        "gko_bench_gemv_q8_rows": (None, [C.POINTER(C.c_int8), _f32p, _f32p, _f32p, z, z]),
        "gko_scalar_topk": (None, [_f32p, _f32p, z, z, z]),
        "gko_scalar_weighted_sum": (None, [_f32p, _f32p, _f32p, C.POINTER(C.c_int64), _f32p, z, z, z]),
    }
    for k, (res, args) in sig.items():
        f = getattr(lib, k)
        f.restype, f.argtypes = res, args
    return lib


_libs: dict = {}


def lib(o1: bool = False) -> C.CDLL:
    name = "libgllmk_oracle_o1.so" if o1 else "libgllmk_oracle.so"
    if name not in _libs:
        _libs[name] = _load(name)
    return _libs[name]


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ---- decoders -------------------------------------------------------------------------------
def dequant_q4_k(block) -> np.ndarray:
    block = _u8(block)
    assert block.size == 144
    out = np.empty(256, np.float32)
    lib().gko_dequant_q4_k(_p(block, _u8p), _p(out, _f32p))
    return out


def dequant_q8_0(block) -> np.ndarray:
    block = _u8(block)
    assert block.size == 34
    out = np.empty(32, np.float32)
    lib().gko_dequant_q8_0(_p(block, _u8p), _p(out, _f32p))
    return out


def dequant_block(qt: int, block) -> np.ndarray:
    """One block of a GGUF format (Q4_K, Q8_0, Q6_K, Q5_K, Q8_K, Q4_0, Q5_0) -> block_size floats."""
    block = _u8(block)
    assert block.size == lib().gko_block_bytes(qt, 0)
    out = np.empty(lib().gko_block_size(qt, 0), np.float32)
    rc = lib().gko_dequant_block(qt, _p(block, _u8p), _p(out, _f32p))
    if rc:
        raise ValueError(f"gko_dequant_block: {rc}")
    return out


def q4k_scales(block):
    block = _u8(block)
    sc, m = np.empty(8, np.uint8), np.empty(8, np.uint8)
    lib().gko_q4k_scales(_p(block, _u8p), _p(sc, _u8p), _p(m, _u8p))
    return sc, m


def dequant_mxfp4(blocks, scales, block_size: int = 32) -> np.ndarray:
    blocks, scales = _u8(blocks), _u8(scales)
    nb = scales.size
    assert block_size % 2 == 0 and blocks.size == nb * block_size // 2
    out = np.empty(nb * block_size, np.float32)
    lib().gko_dequant_mxfp4(_p(blocks, _u8p), _p(scales, _u8p), _p(out, _f32p), nb, block_size)
    return out


def dequant_nvfp4(blocks, global_scale: float) -> np.ndarray:
    blocks = _u8(blocks)
    nb = blocks.size // 36
    out = np.empty(nb * 64, np.float32)
    lib().gko_dequant_nvfp4(_p(blocks, _u8p), global_scale, _p(out, _f32p), nb)
    return out


def dequant_matrix(qt, blocks, n, k, scales=None, global_scale=1.0, mx_block=32) -> np.ndarray:
    blocks = _u8(blocks)
    sc = _u8(scales) if scales is not None else np.zeros(1, np.uint8)
    out = np.empty((n, k), np.float32)
    rc = lib().gko_dequant_matrix(qt, _p(blocks, _u8p), _p(sc, _u8p), global_scale, n, k, mx_block, _p(out, _f32p))
    if rc:
        raise ValueError(f"gko_dequant_matrix rc={rc}")
    return out


# ---- matmuls --------------------------------------------------------------------------------
def quant_matmul(weight_blocks, inp, qt, m, n, k, threads: int = 1, o1: bool = False) -> np.ndarray:
    """Kernels::kquant_matmul / classic_matmul: m weight rows, n batch columns, input [k,n], output [m,n]."""
    w, x = _u8(weight_blocks), _f32(inp)
    assert x.size == k * n
    out = np.empty((m, n), np.float32)
    rc = lib(o1).gko_quant_matmul_mt(_p(w, _u8p), _p(x, _f32p), _p(out, _f32p), qt, m, n, k, threads)
    if rc:
        raise ValueError(f"gko_quant_matmul rc={rc}")
    return out


def gemm_q4(weight, inp, scales, m, n, k) -> np.ndarray:
    """Kernels::gemm_q4: m batch rows, n output features, input [m,k], output [m,n]."""
    w, x = _u8(weight), _f32(inp)
    s = _f32(scales) if scales is not None and len(scales) else np.zeros(0, np.float32)
    out = np.empty((m, n), np.float32)
    sp = _p(s, _f32p) if s.size else C.cast(None, _f32p)
    rc = lib().gko_gemm_q4(_p(w, _u8p), _p(x, _f32p), _p(out, _f32p), sp, s.size, m, n, k)
    if rc:
        raise ValueError(f"gko_gemm_q4 rc={rc}")
    return out


def gemm_q8(weight, inp, scales, m, n, k) -> np.ndarray:
    """Kernels::gemm_q8: Q8_K rows, input [m,k], output [m,n]."""
    w, x = _u8(np.ascontiguousarray(weight).view(np.uint8)), _f32(inp)
    s = _f32(scales) if scales is not None and len(scales) else np.zeros(0, np.float32)
    out = np.empty((m, n), np.float32)
    sp = _p(s, _f32p) if s.size else C.cast(None, _f32p)
    rc = lib().gko_gemm_q8(_p(w, _u8p), _p(x, _f32p), _p(out, _f32p), sp, s.size, m, n, k)
    if rc:
        raise ValueError(f"gko_gemm_q8 rc={rc}")
    return out


def gemv_q8(weight, inp, scale: float, n: int) -> float:
    w, x = _u8(np.ascontiguousarray(weight).view(np.uint8)), _f32(inp)
    return float(lib().gko_gemv_q8(_p(w, _u8p), _p(x, _f32p), scale, n))


def gemv_q4(weight, inp, scale: float, n: int) -> float:
    w, x = _u8(weight), _f32(inp)
    return float(lib().gko_gemv_q4(_p(w, _u8p), _p(x, _f32p), scale, n))


def quantize_int8_per_tensor(x):
    """quantize_from_fp32 / Int8PerTensor (src/compiler/quant_convert.rs:165-177): (int8 array, scale)."""
    x = _f32(x)
    q = np.empty(x.shape, np.int8)
    scale = lib().gko_quantize_int8_per_tensor(_p(x, _f32p), _p(q, C.POINTER(C.c_int8)), x.size)
    return q, float(scale)


def gemm_f32_nt(a, wd) -> np.ndarray:
    """C[m,n] = sum_p a[m,p]*wd[n,p], sequential f32 (scalar_gemm order)."""
    a, wd = _f32(a), _f32(wd)
    m, k = a.shape
    n = wd.shape[0]
    out = np.empty((m, n), np.float32)
    lib().gko_gemm_f32_nt(_p(a, _f32p), _p(wd, _f32p), _p(out, _f32p), m, n, k)
    return out


def gemm_f64_nt(a, wd) -> np.ndarray:
    a, wd = _f32(a), _f32(wd)
    m, k = a.shape
    n = wd.shape[0]
    out = np.empty((m, n), np.float64)
    lib().gko_gemm_f64_nt(_p(a, _f32p), _p(wd, _f32p), _p(out, _f64p), m, n, k)
    return out


# ---- mixture-of-experts conventions (scalar-ops/src/moe.rs) ----------------------------------
def scalar_topk(gate_probs, top_k: int) -> np.ndarray:
    """scalar_topk: [seq, experts] -> [2, seq*top_k] f32 (row 0: index bit patterns, row 1: weights)."""
    p = _f32(gate_probs)
    seq, ne = p.shape
    assert top_k <= 64
    out = np.empty((2, seq * top_k), np.float32)
    lib().gko_scalar_topk(_p(p, _f32p), _p(out, _f32p), seq, ne, top_k)
    return out


def scalar_weighted_sum(expert_outputs, routing, seq_len: int, top_k: int) -> np.ndarray:
    """scalar_weighted_sum over the reference's [experts, seq, hidden] buffer."""
    eo, r = _f32(expert_outputs), _f32(routing).reshape(2, -1)
    hidden = eo.shape[-1]
    out = np.empty((seq_len, hidden), np.float32)
    lib().gko_scalar_weighted_sum(_p(eo, _f32p), _p(r[0].copy(), _f32p), _p(r[1].copy(), _f32p), None, _p(out, _f32p), seq_len,
                                  hidden, top_k)
    return out


def scalar_weighted_sum_grouped(rows_buf, routing, inv, seq_len: int, top_k: int) -> np.ndarray:
    """The same sum over grouped rows [seq*top_k, hidden]; inv[slot] = row (negative: skipped)."""
    eo, r = _f32(rows_buf), _f32(routing).reshape(2, -1)
    inv = np.ascontiguousarray(inv, np.int64)
    hidden = eo.shape[-1]
    out = np.empty((seq_len, hidden), np.float32)
    lib().gko_scalar_weighted_sum(_p(eo, _f32p), _p(r[0].copy(), _f32p), _p(r[1].copy(), _f32p), _p(inv, C.POINTER(C.c_int64)),
                                  _p(out, _f32p), seq_len, hidden, top_k)
    return out


# ---- quantizers (this project's own; the reference has none for these formats) --------------
def quantize_q4_k(x) -> np.ndarray:
    x = _f32(x).reshape(-1)
    nb = x.size // 256
    out = np.empty(nb * 144, np.uint8)
    lib().gko_quantize_q4_k(_p(x, _f32p), _p(out, _u8p), nb)
    return out


def quantize_q8_0(x) -> np.ndarray:
    x = _f32(x).reshape(-1)
    nb = x.size // 32
    out = np.empty(nb * 34, np.uint8)
    lib().gko_quantize_q8_0(_p(x, _f32p), _p(out, _u8p), nb)
    return out


def quantize_mxfp4(x, block_size: int = 32):
    x = _f32(x).reshape(-1)
    nb = x.size // block_size
    blocks = np.empty(nb * block_size // 2, np.uint8)
    scales = np.empty(nb, np.uint8)
    lib().gko_quantize_mxfp4(_p(x, _f32p), _p(blocks, _u8p), _p(scales, _u8p), nb, block_size)
    return blocks, scales


def nvfp4_global(x) -> float:
    x = _f32(x).reshape(-1)
    return float(lib().gko_nvfp4_global(_p(x, _f32p), x.size))


def quantize_nvfp4(x, global_scale: float | None = None):
    x = _f32(x).reshape(-1)
    g = nvfp4_global(x) if global_scale is None else float(global_scale)
    nb = x.size // 64
    out = np.empty(nb * 36, np.uint8)
    lib().gko_quantize_nvfp4(_p(x, _f32p), g, _p(out, _u8p), nb)
    return out, g


def bench_gemv_q4_rows(w, x, scales, n: int, k: int, o1: bool = True) -> np.ndarray:
    """The loop benches/bench_quant.rs times for quant/gemv_q4 (simplified nibble-8 format, per-row scale),
    by default from the -O1 build that mirrors the reference's bench profile."""
    out = np.empty(n, np.float32)
    w, x, scales = _u8(w), _f32(x), _f32(scales)
    lib(o1).gko_bench_gemv_q4_rows(_p(w, _u8p), _p(x, _f32p), _p(scales, _f32p), _p(out, _f32p), n, k)
    return out


def bench_quant_kernel(kind: str, m: int, n: int, k: int, seed: int = 0, o1: bool = True):
    """One call of a benches/bench_quant.rs kernel on random data of its shape (the restated scalar-ops loops,
    built -O1 like the reference's bench profile).  Returns (seconds, rows of x actually run): GEMM kinds run
    min(m, 8) rows of x — the loops are `for i in 0..m` outermost, so the time per row does not depend on m."""
    import time
    rng = np.random.default_rng(seed)
    L = lib(o1)
    mi = min(m, 8)
    x = rng.standard_normal((mi, k), dtype=np.float32)
    sc = rng.random(n, dtype=np.float32)
    out = np.empty((mi, n), np.float32)
    i8p = C.POINTER(C.c_int8)
    if kind == "gemv_q8":
        w = rng.integers(-128, 128, size=n * k, dtype=np.int8)
        fn = lambda: L.gko_bench_gemv_q8_rows(_p(w, i8p), _p(x, _f32p), _p(sc, _f32p), _p(out, _f32p), n, k)
    elif kind == "gemv_q4":
        w = rng.integers(0, 256, size=n * k // 2, dtype=np.uint8)
        fn = lambda: L.gko_bench_gemv_q4_rows(_p(w, _u8p), _p(x, _f32p), _p(sc, _f32p), _p(out, _f32p), n, k)
    elif kind == "gemm_q8":
        w = rng.integers(-128, 128, size=n * k, dtype=np.int8)
        fn = lambda: L.gko_scalar_gemm_q8(_p(w, i8p), _p(x, _f32p), _p(out, _f32p), _p(sc, _f32p), mi, n, k)
    elif kind == "gemm_q4":
        w = rng.integers(0, 256, size=n * k // 2, dtype=np.uint8)
        fn = lambda: L.gko_scalar_gemm_q4(_p(w, _u8p), _p(x, _f32p), _p(out, _f32p), _p(sc, _f32p), mi, n, k)
    elif kind == "kquant_matmul":
        w = rng.integers(0, 256, size=n * (k // 256) * 144, dtype=np.uint8)
        w.reshape(-1, 144)[:, 0:4] = np.frombuffer(np.float32(0.01).tobytes(), np.uint8)
        fn = lambda: L.gko_scalar_kquant_matmul(_p(w, _u8p), _p(x, _f32p), _p(out, _f32p), 144, 256, mi, n, k)
    else:
        raise ValueError(kind)
    t0 = time.perf_counter()
    fn()
    return time.perf_counter() - t0, mi


def rel_err(y, ref) -> float:
    """Parity metric: max_i |y_i - ref_i| / max(|ref_i|, rms(ref))."""
    y = np.asarray(y, np.float64).reshape(-1)
    ref = np.asarray(ref, np.float64).reshape(-1)
    rms = float(np.sqrt(np.mean(ref * ref))) if ref.size else 0.0
    den = np.maximum(np.abs(ref), max(rms, 1e-30))
    return float(np.max(np.abs(y - ref) / den)) if ref.size else 0.0
