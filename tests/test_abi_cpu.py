"""CPU-side checks of the boundary: the library loads, exports every declared symbol, and the
entry points validate their arguments before touching a device (no compute without a GPU)."""
import ctypes as C
import importlib
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L(gk):
    if not os.path.exists(gk.lib_path()):
        gk.build_library()
    return gk.lib()


def test_header_symbols_are_exported(gk, L):
    hdr = open(os.path.join(ROOT, "include", "gllmk.h")).read()
    declared = sorted(set(re.findall(r"GLLMK_API[^;]*?\b(gllmk_\w+)\s*\(", hdr)))
    assert len(declared) >= 20
    bound = importlib.import_module("gllm-kernels_b200._lib").exported_symbols()
    assert declared == bound, "ctypes table and header disagree"
    raw = C.CDLL(gk.lib_path())
    for name in declared:
        assert hasattr(raw, name), f"{name} not exported"


def test_version_and_hw_info(L):
    assert L.gllmk_version().startswith(b"gllmk ")
    buf = C.create_string_buffer(256)
    n = L.gllmk_hw_info(buf, 256)
    assert n > 0 and len(buf.value) == n
    assert L.gllmk_hw_info(None, 10) == -1
    small = C.create_string_buffer(4)
    assert L.gllmk_hw_info(small, 4) == 3 and len(small.value) == 3  # truncated, NUL-terminated


def test_metadata_matches_reference_tables(gk, L):
    # src/quant.rs:375-456
    QT = gk.QuantType
    for qt in (QT.q4k(), QT.q8_0(), QT.mxfp4(32), QT.mxfp4(16), QT.nvfp4()):
        assert L.gllmk_quant_block_size(qt.id, qt.mx_block) == qt.block_size()
        assert L.gllmk_quant_block_bytes(qt.id, qt.mx_block) == qt.block_bytes()
    assert (QT.q4k().block_size(), QT.q4k().block_bytes(), QT.q4k().bits()) == (256, 144, 4)
    assert (QT.q8_0().block_size(), QT.q8_0().block_bytes(), QT.q8_0().bits()) == (32, 34, 8)
    assert (QT.mxfp4().block_size(), QT.mxfp4().block_bytes()) == (32, 17)
    assert (QT.nvfp4().block_size(), QT.nvfp4().block_bytes()) == (64, 36)
    assert L.gllmk_quant_block_size(99, 0) == 0


def test_null_and_free_conventions(L):
    # src/ffi/mod.rs:30-32,53-57: null -> InvalidArg, free(NULL) is a no-op
    assert L.gllmk_ctx_create(0, None) == -1
    L.gllmk_ctx_free(None)
    L.gllmk_weight_free(None)
    assert L.gllmk_last_error(None) == b""
    h = C.c_void_p()
    assert L.gllmk_weight_upload(None, 1, 16, 256, 0, None, None, 1.0, 0, C.byref(h)) == -1
    assert L.gllmk_gemv(None, None, None, 0, 0, 1, None, 0, 0, None, 0, None) == -1
    assert L.gllmk_kquant_matmul_f32(None, None, None, None, 1, 1, 1, 256) == -1
    assert L.gllmk_dequant_mxfp4(None, None, None, None, 1, 32) == -1
    assert L.gllmk_weight_info(None, None, None, None, None, None) == -1


def test_no_cpu_fallback_without_device(gk, L):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    h = C.c_void_p()
    assert L.gllmk_ctx_create(0, C.byref(h)) == gk.Status.RUNTIME_ERROR
    assert not h.value
    with pytest.raises(gk.GllmkError):
        gk.GpuKernels(0)


def test_e8m0_and_lut_mirror(gk, oracle):
    for b in range(256):
        a, r = gk.decode_e8m0_scale(b), oracle.lib().gko_decode_e8m0_scale(b)
        assert (np.isnan(a) and np.isnan(r)) or a == r
    assert [oracle.lib().gko_e2m1(i) for i in range(16)] == list(gk.E2M1_LUT_F32)


def test_rust_shim_declares_every_entry_point(gk):
    """gllm-kernels_b200/rust/gpu_b200.rs is shipped uncompiled (no Rust toolchain here): at least its extern block must
    name exactly the functions include/gllmk.h declares, and the header must declare what the binding binds."""
    import os
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    rs = open(os.path.join(root, "gllm-kernels_b200", "rust", "gpu_b200.rs")).read()
    ext = rs[rs.index('extern "C" {'):]
    ext = ext[:ext.index("\n}\n")]
    rust_syms = set(re.findall(r"fn (gllmk_\w+)\(", ext))
    header = open(os.path.join(root, "include", "gllmk.h")).read()
    header_syms = set(re.findall(r"GLLMK_API [\w \*]+?\b(gllmk_\w+)\(", header))
    assert header_syms == set(_lib_syms(gk)), (header_syms ^ set(_lib_syms(gk)))
    assert rust_syms == header_syms, (rust_syms ^ header_syms)


def _lib_syms(gk):
    import importlib
    return importlib.import_module("gllm-kernels_b200._lib").exported_symbols()
