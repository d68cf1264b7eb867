"""ctypes binding of libgllmk.so (include/gllmk.h).  No fallback: a missing library is an error."""
from __future__ import annotations

import ctypes as C
import enum
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_HERE)


class Status(enum.IntEnum):  # src/ffi/types.rs:4-14
    OK = 0
    INVALID_ARG = -1
    OUT_OF_MEMORY = -2
    COMPILE_ERROR = -3
    RUNTIME_ERROR = -4
    UNSUPPORTED = -5
    IO_ERROR = -6


class GllmkError(RuntimeError):
    def __init__(self, status: int, what: str, detail: str = ""):
        self.status = Status(status) if status in Status._value2member_map_ else status
        super().__init__(f"{what}: {getattr(self.status, 'name', self.status)}" + (f" — {detail}" if detail else ""))


def lib_path() -> str:
    return os.path.join(_HERE, "libgllmk.so")


def build_library(verbose: bool = False, jobs: int = 8) -> str:
    """Compile csrc/*.cu for sm_100a into libgllmk.so (nvcc cross-compiles without a GPU)."""
    r = subprocess.run(["make", "-C", os.path.join(_HERE, "csrc"), f"-j{jobs}"], capture_output=True, text=True)
    if verbose or r.returncode:
        print(r.stdout[-4000:], r.stderr[-4000:])
    if r.returncode:
        raise RuntimeError("building libgllmk.so failed")
    return lib_path()


_vp, _i32, _i64, _u64, _f32, _sz = C.c_void_p, C.c_int32, C.c_int64, C.c_uint64, C.c_float, C.c_size_t
_SIGS = {
    "gllmk_version": (C.c_char_p, []),
    "gllmk_hw_info": (_i32, [C.c_char_p, _sz]),
    "gllmk_quant_block_size": (_i32, [_i32, _i32]),
    "gllmk_quant_block_bytes": (_i32, [_i32, _i32]),
    "gllmk_ctx_create": (_i32, [_i32, C.POINTER(_vp)]),
    "gllmk_ctx_free": (None, [_vp]),
    "gllmk_last_error": (C.c_char_p, [_vp]),
    "gllmk_ctx_set": (_i32, [_vp, C.c_char_p, _i64]),
    "gllmk_ctx_status": (_i32, [_vp, C.POINTER(_i32)]),
    "gllmk_weight_upload": (_i32, [_vp, _i32, _i64, _i64, _i32, _vp, _vp, _f32, _i32, C.POINTER(_vp)]),
    "gllmk_weight_free": (None, [_vp]),
    "gllmk_weight_info": (_i32, [_vp, C.POINTER(_i32), C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_u64),
                                 C.POINTER(_u64)]),
    "gllmk_weight_unpack": (_i32, [_vp, _vp, _vp, _vp, _i32]),
    "gllmk_dequant": (_i32, [_vp, _vp, _vp, _vp]),
    "gllmk_gemv": (_i32, [_vp, _vp, _vp, _i64, _i64, _i32, _vp, _i64, _i64, _vp, _i64, _vp]),
    "gllmk_gemm": (_i32, [_vp, _vp, _vp, _i32, _i64, _i32, _vp, _i32, _i64, _vp]),
    "gllmk_gemm_fp4": (_i32, [_vp, _vp, _vp, _vp, _i32, _i64, _vp]),
    "gllmk_kquant_matmul_f32": (_i32, [_vp, _vp, _vp, _vp, _i32, _sz, _sz, _sz]),
    "gllmk_classic_matmul_f32": (_i32, [_vp, _vp, _vp, _vp, _i32, _sz, _sz, _sz]),
    "gllmk_gemm_q4_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz]),
    "gllmk_matmul_host": (_i32, [_vp, _vp, _vp, _i32, _vp, _i32]),
    "gllmk_dequant_q4_k": (_i32, [_vp, _vp, _vp, _sz]),
    "gllmk_dequant_q8_0": (_i32, [_vp, _vp, _vp, _sz]),
    "gllmk_dequant_mxfp4": (_i32, [_vp, _vp, _vp, _vp, _sz, _sz]),
    "gllmk_dequant_nvfp4": (_i32, [_vp, _vp, _f32, _vp, _sz]),
    "gllmk_quantize": (_i32, [_vp, _i32, _vp, _i64, _i64, _i32, _vp, _vp, C.POINTER(_f32), _vp]),
}
# Entry points added after the first release of the header are listed here as they land.
_OPTIONAL_SIGS: dict = {
    "gllmk_dequant_gguf": (_i32, [_vp, _i32, _vp, _vp, _sz]),
    "gllmk_gemv_static": (_i32, [_vp, _vp, _vp, _i64, _i64, _i32, _vp, _i64, _i64, _vp, _i64, _vp]),
    "gllmk_embedding_gather": (_i32, [_vp, _vp, _vp, _i64, _vp, _vp]),
    "gllmk_int8_weight_upload": (_i32, [_vp, _i64, _i64, _vp, _i32, _i32, C.POINTER(_vp)]),
    "gllmk_gemm_int8": (_i32, [_vp, _vp, _vp, _i64, _i32, _vp, _i64, _vp]),
    "gllmk_dequantize_i32_f32": (_i32, [_vp, _vp, _vp, _i64, _i64, _f32, _f32, _vp, _i32, _vp]),
    "gllmk_gemm_int8_host": (_i32, [_vp, _vp, _vp, _vp, _sz, _sz, _sz]),
    "gllmk_ffn_decode": (_i32, [_vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp]),
    "gllmk_matmul_host_batch": (_i32, [_vp, _i32, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_i32), C.POINTER(_vp), _i32]),
    "gllmk_ffn_prefill": (_i32, [_vp, _vp, _vp, _vp, _i32, _i64, _i32, _vp, _vp, _i32, _i64, _vp]),
    "gllmk_gemm_grouped": (_i32, [_vp, _i32, C.POINTER(_vp), _vp, _i32, _i64, C.POINTER(_i64), _vp, _i32, _i64, _vp]),
    "gllmk_shared_alloc": (_i32, [_vp, _sz, C.POINTER(_vp), _vp]),
    "gllmk_shared_open": (_i32, [_vp, _vp, C.POINTER(_vp)]),
    "gllmk_shared_close": (_i32, [_vp, _vp]),
    "gllmk_shared_free": (_i32, [_vp, _vp]),
    "gllmk_gemv_allgather": (_i32, [_vp, _vp, _vp, _i64, _i64, _i32, _vp, _i64, _i64, C.POINTER(_vp), _i32, _vp]),
    "gllmk_peer_barrier": (_i32, [_vp, _vp, C.POINTER(_vp), _i32, _i32, C.c_uint32, _vp]),
    "gllmk_probe_fp4_mma": (_i32, [_vp, _i32, _i32, _i32, _i32, C.POINTER(_f32)]),
    "gllmk_quantize_act_int8": (_i32, [_vp, _vp, _i64, _i64, _i64, _vp, _i64, _i32, _vp, _vp]),
    "gllmk_w8a8_linear_f32": (_i32, [_vp, _vp, _vp, _i64, _i32, _vp, _i64, _f32, _vp, _i32, _vp]),
    "gllmk_gemm_q8_f32": (_i32, [_vp, _vp, _vp, _vp, _vp, _sz, _sz, _sz, _sz]),
    "gllmk_gemv_q4_f32": (_i32, [_vp, _vp, _vp, _f32, _sz, _vp]),
    "gllmk_gemv_q8_f32": (_i32, [_vp, _vp, _vp, _f32, _sz, _vp]),
    "gllmk_quant_format_descriptor_for_type": (_i32, [_i32, _i32, _vp]),
    "gllmk_quant_format_registry": (_i32, [_vp, _i32]),
    "gllmk_gemv_exchange": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i32, _vp, _i64, _i64, C.POINTER(_vp), _vp, C.POINTER(_vp), _i32, _i32, _vp]),
    "gllmk_exchange_wait": (_i32, [_vp, _vp, _i32, _i32, _vp]),
    "gllmk_moe_topk": (_i32, [_vp, _vp, _vp, _i64, _i32, _i32, _vp]),
    "gllmk_moe_route": (_i32, [_vp, _vp, _i64, _i32, _i32, C.POINTER(_i64), _vp, _vp, _vp]),
    "gllmk_moe_gather": (_i32, [_vp, _vp, _i32, _i64, _vp, _i64, _i32, _i64, _vp, _i64, _vp]),
    "gllmk_moe_weighted_sum": (_i32, [_vp, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _vp]),
}

_lib = None


def exported_symbols() -> list:
    """Every function include/gllmk.h declares (used by the CPU-side symbol test)."""
    return sorted(list(_SIGS) + list(_OPTIONAL_SIGS))


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        p = lib_path()
        if not os.path.exists(p):
            raise ImportError(f"{p} is missing: build it with __graft_entry__.build() — there is no CPU fallback")
        L = C.CDLL(p)
        for name, (res, args) in {**_SIGS, **_OPTIONAL_SIGS}.items():
            f = getattr(L, name)
            f.restype, f.argtypes = res, args
        _lib = L
    return _lib
