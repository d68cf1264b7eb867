"""Host-side mirror of the quant slice of gllm-kernels' operator trait, bound to libgllmk.so.

`GpuKernels` carries the same method names, argument order and shape conventions as the reference's
`Kernels<f32>` quant methods (src/traits.rs:473-608; CPU implementation src/cpu_kernels/mod.rs) so
code and tests written against the reference read the same here.  Host-array methods take numpy
arrays where the reference takes slices.  The resident-weight methods (`upload`, `gemv`, ...) are
the additions a GPU needs: weights are repacked once and stay in HBM.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import quant as Q
from ._lib import GllmkError, Status, lib
from .quant import QuantType


def _np(a, dtype, writable=False):
    if not isinstance(a, np.ndarray) or a.dtype != dtype or not a.flags.c_contiguous:
        if writable:
            raise TypeError(f"output must be a C-contiguous numpy array of {np.dtype(dtype).name}")
        a = np.ascontiguousarray(a, dtype=dtype)
    return a


def _ptr(a) -> int:
    """Address of a numpy array, a torch tensor, or a raw integer device pointer."""
    if a is None:
        return 0
    if isinstance(a, np.ndarray):
        return a.ctypes.data
    if isinstance(a, int):
        return a
    return a.data_ptr()


def _stream(stream) -> int:
    if stream is None:
        import torch
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


class Weight:
    """A weight matrix resident on the device in the kernels' tiled layout (opaque gllmk_weight)."""

    def __init__(self, owner: "GpuKernels", handle: int, qt: QuantType, n: int, k: int):
        self._owner, self._h, self.quant_type, self.n, self.k = owner, handle, qt, n, k

    def info(self) -> dict:
        qt, n, k = C.c_int32(), C.c_int64(), C.c_int64()
        rb, db = C.c_uint64(), C.c_uint64()
        self._owner._check(lib().gllmk_weight_info(self._h, C.byref(qt), C.byref(n), C.byref(k), C.byref(rb),
                                                   C.byref(db)), "weight_info")
        return {"quant_type": qt.value, "n": n.value, "k": k.value, "ref_bytes": rb.value, "dev_bytes": db.value}

    @property
    def ref_bytes(self) -> int:
        return self.info()["ref_bytes"]

    def free(self) -> None:
        if self._h:
            lib().gllmk_weight_free(self._h)
            self._h = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class GpuKernels:
    """B200 implementation of the reference's quantized operators (one context = one device)."""

    GEMV_MAX_M = 16
    GEMM_GEMV_MAX_M = 16  # f32 products up to this many tokens run as a pass of the decode kernel

    def __init__(self, device: int = 0):
        h = C.c_void_p()
        rc = lib().gllmk_ctx_create(device, C.byref(h))
        if rc:
            raise GllmkError(rc, "gllmk_ctx_create", "no usable CUDA device (there is no CPU fallback)")
        self._ctx = h.value
        self.device = device

    # ---- plumbing ---------------------------------------------------------------------------
    def close(self) -> None:
        if getattr(self, "_ctx", None):
            lib().gllmk_ctx_free(self._ctx)
            self._ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int, what: str) -> None:
        if rc:
            raise GllmkError(rc, what, (lib().gllmk_last_error(self._ctx) or b"").decode())

    def status(self) -> int:
        """Synchronises and returns the device status word (0 = no kernel gave up a bounded wait)."""
        v = C.c_int32()
        self._check(lib().gllmk_ctx_status(self._ctx, C.byref(v)), "gllmk_ctx_status")
        return v.value

    def set(self, key: str, value: int) -> None:
        self._check(lib().gllmk_ctx_set(self._ctx, key.encode(), int(value)), "ctx_set")

    # ---- resident weights -------------------------------------------------------------------
    def upload(self, quant_type: QuantType, n: int, k: int, blocks, scales=None, global_scale: float = 1.0) -> Weight:
        """Repack reference-format blocks ([n rows][k/bs blocks]) into HBM.  `blocks`/`scales` may be numpy
        arrays (host) or CUDA torch tensors (device)."""
        on_dev = not isinstance(blocks, np.ndarray)
        if not on_dev:
            blocks = _np(blocks, np.uint8)
            scales = _np(scales, np.uint8) if scales is not None else None
            expect = n * (k // quant_type.block_size()) * quant_type.block_bytes() if quant_type.block_size() else 0
            if quant_type.id == Q.MXFP4 and scales is not None:
                expect = n * k // 2
            if expect and blocks.size != expect:
                raise GllmkError(Status.INVALID_ARG, "upload", f"blocks holds {blocks.size} bytes, expected {expect}")
        h = C.c_void_p()
        rc = lib().gllmk_weight_upload(self._ctx, quant_type.id, n, k, quant_type.mx_block, _ptr(blocks), _ptr(scales),
                                       float(global_scale), int(on_dev), C.byref(h))
        self._check(rc, "gllmk_weight_upload")
        return Weight(self, h.value, quant_type, n, k)

    def unpack(self, w: Weight):
        """Inverse of the repack: reference-format bytes (numpy).  MXFP4 returns (blocks, scales)."""
        qt = w.quant_type
        if qt.id == Q.MXFP4:
            blocks = np.empty(w.n * w.k // 2, np.uint8)
            scales = np.empty(w.n * w.k // 32, np.uint8)
            self._check(lib().gllmk_weight_unpack(self._ctx, w._h, _ptr(blocks), _ptr(scales), 0), "weight_unpack")
            return blocks, scales
        blocks = np.empty(w.n * (w.k // qt.block_size()) * qt.block_bytes(), np.uint8)
        self._check(lib().gllmk_weight_unpack(self._ctx, w._h, _ptr(blocks), 0, 0), "weight_unpack")
        return blocks

    def dequant(self, w: Weight, out=None, stream=None):
        """Whole-matrix decode to f32 [n, k] on the device (bit-exact with the reference's scalar decode)."""
        import torch
        if out is None:
            out = torch.empty((w.n, w.k), dtype=torch.float32, device=f"cuda:{self.device}")
        self._check(lib().gllmk_dequant(self._ctx, w._h, _ptr(out), _stream(stream)), "gllmk_dequant")
        return out

    def gemv(self, w: Weight, x, y=None, ref_layout: bool = False, row_scales=None, stream=None):
        """Decode product with device tensors.  ref_layout=False: x [m, k] -> y [m, n] (gemm_q4 convention);
        ref_layout=True: x [k, m] -> y [n, m] (kquant_matmul / classic_matmul convention)."""
        import torch
        m = x.shape[1] if ref_layout else x.shape[0]
        if y is None:
            y = torch.empty((w.n, m) if ref_layout else (m, w.n), dtype=torch.float32, device=x.device)
        # (token stride, k stride) of x and (token stride, row stride) of y, in elements: views are fine
        if ref_layout:
            xs, ys = (x.stride(1), x.stride(0)), (y.stride(1), y.stride(0))
        else:
            xs, ys = (x.stride(0), x.stride(1)), (y.stride(0), y.stride(1))
        ns = 0 if row_scales is None else row_scales.numel()
        rc = lib().gllmk_gemv(self._ctx, w._h, _ptr(x), xs[0], xs[1], m, _ptr(y), ys[0], ys[1], _ptr(row_scales), ns,
                              _stream(stream))
        self._check(rc, "gllmk_gemv")
        return y

    def gemm(self, w: Weight, a, y=None, out_dtype=None, stream=None):
        """Prefill product with device tensors: a [m, k] (f32 or bf16, row-major) -> y [m, n] (f32 or bf16)."""
        import torch
        m = a.shape[0]
        if y is None:
            y = torch.empty((m, w.n), dtype=out_dtype or torch.float32, device=a.device)
        dt = {torch.float32: 0, torch.bfloat16: 1}
        rc = lib().gllmk_gemm(self._ctx, w._h, _ptr(a), dt[a.dtype], a.stride(0), m, _ptr(y), dt[y.dtype], y.stride(0),
                              _stream(stream))
        self._check(rc, "gllmk_gemm")
        return y

    def embedding_gather(self, w: Weight, ids, out=None, stream=None):
        """out[r, :] = decoded weight row ids[r] (int32 CUDA tensor) -> f32 [len(ids), k]; bad ids give zero rows."""
        import torch
        count = ids.numel()
        if out is None:
            out = torch.empty((count, w.k), dtype=torch.float32, device=ids.device)
        self._check(lib().gllmk_embedding_gather(self._ctx, w._h, _ptr(ids), count, _ptr(out), _stream(stream)),
                    "gllmk_embedding_gather")
        return out

    # ---- W8A8 integer path (avx512_int8::gemm_int8 / dequantize_i32_to_f32, src/macros/matmul_x86_int8.rs) ----
    def upload_int8(self, b, layout_kn: bool = True) -> Weight:
        """s8 weight matrix -> resident tiles.  layout_kn=True: b is [k, n] row-major as in the reference's B;
        False: [n, k] row-major.  numpy (host) or CUDA torch int8 tensor."""
        on_dev = not isinstance(b, np.ndarray)
        if not on_dev:
            b = _np(b, np.int8)
        k, n = (b.shape[0], b.shape[1]) if layout_kn else (b.shape[1], b.shape[0])
        h = C.c_void_p()
        rc = lib().gllmk_int8_weight_upload(self._ctx, n, k, _ptr(b), 0 if layout_kn else 1, int(on_dev), C.byref(h))
        self._check(rc, "gllmk_int8_weight_upload")
        return Weight(self, h.value, None, n, k)

    def gemm_int8(self, w: Weight, a, c=None, stream=None):
        """C (int32) [m, n] = a (uint8 CUDA tensor [m, k]) x W, exact."""
        import torch
        m = a.shape[0]
        if c is None:
            c = torch.empty((m, w.n), dtype=torch.int32, device=a.device)
        rc = lib().gllmk_gemm_int8(self._ctx, w._h, _ptr(a), a.stride(0), m, _ptr(c), c.stride(0), _stream(stream))
        self._check(rc, "gllmk_gemm_int8")
        return c

    def dequantize_i32(self, c, scale_a: float, scale_b: float, bias=None, activation: int = 0, out=None, stream=None):
        """(c as f32) * scale_a * scale_b (+ bias[j]) then the activation (0 none, 1 relu, 2 silu, 3 gelu, 4 geglu)."""
        import torch
        m, n = c.shape
        if out is None:
            out = torch.empty((m, n), dtype=torch.float32, device=c.device)
        rc = lib().gllmk_dequantize_i32_f32(self._ctx, _ptr(c), _ptr(out), m, n, float(scale_a), float(scale_b), _ptr(bias),
                                            int(activation), _stream(stream))
        self._check(rc, "gllmk_dequantize_i32_f32")
        return out

    def quantize_act_int8(self, x, as_unsigned: bool = False, stream=None):
        """quantize_from_fp32 / Int8PerTensor on a CUDA f32 tensor [rows, k]: (int8 tensor — or uint8 = q + 128 —, scale
        as a 1-element CUDA tensor: no host synchronisation)."""
        import torch
        rows, k = x.shape
        q = torch.empty((rows, k), dtype=torch.uint8 if as_unsigned else torch.int8, device=x.device)
        sc = torch.zeros(2, dtype=torch.float32, device=x.device)
        self._check(lib().gllmk_quantize_act_int8(self._ctx, _ptr(x), rows, k, x.stride(0), _ptr(q), k, int(as_unsigned), _ptr(sc),
                                                  _stream(stream)), "gllmk_quantize_act_int8")
        return q, sc[:1]

    def w8a8_linear(self, w: Weight, x, scale_b: float, bias=None, activation: int = 0, y=None, stream=None):
        """y = act((quantize(x) . W) * scale_x * scale_b + bias): f32 in, f32 out, int8 tensor-core product."""
        import torch
        m = x.shape[0]
        if y is None:
            y = torch.empty((m, w.n), dtype=torch.float32, device=x.device)
        rc = lib().gllmk_w8a8_linear_f32(self._ctx, w._h, _ptr(x), x.stride(0), m, _ptr(y), y.stride(0), float(scale_b), _ptr(bias),
                                         int(activation), _stream(stream))
        self._check(rc, "gllmk_w8a8_linear_f32")
        return y

    def gemm_int8_host(self, a, b_kn) -> np.ndarray:
        """The reference call with host arrays: a uint8 [m, k], b int8 [k, n] -> int32 [m, n]."""
        a, b = _np(a, np.uint8), _np(b_kn, np.int8)
        m, k = a.shape
        n = b.shape[1]
        c = np.empty((m, n), np.int32)
        self._check(lib().gllmk_gemm_int8_host(self._ctx, _ptr(a), _ptr(b), _ptr(c), m, n, k), "gllmk_gemm_int8_host")
        return c

    def ffn_decode(self, w_gate_up: Weight, w_down: Weight, x, h=None, y=None, stream=None):
        """y = W_down (silu(gate) * up) with [gate | up] = W_gate_up x, for m <= 16 tokens (x [m, k] f32 CUDA)."""
        import torch
        m = x.shape[0]
        if h is None:
            h = torch.empty((m, w_gate_up.n), dtype=torch.float32, device=x.device)
        if y is None:
            y = torch.empty((m, w_down.n), dtype=torch.float32, device=x.device)
        rc = lib().gllmk_ffn_decode(self._ctx, w_gate_up._h, w_down._h, _ptr(x), m, _ptr(h), _ptr(y), _stream(stream))
        self._check(rc, "gllmk_ffn_decode")
        return y

    def ffn_prefill(self, w_gate_up: Weight, w_down: Weight, x, h=None, y=None, out_dtype=None, stream=None):
        """The gated block for any number of tokens: x [m, k] f32 / bf16 CUDA -> y [m, k]; h [m, 2f] bf16 scratch."""
        import torch
        m = x.shape[0]
        if h is None:
            h = torch.empty((m, w_gate_up.n), dtype=torch.bfloat16, device=x.device)
        if y is None:
            y = torch.empty((m, w_down.n), dtype=out_dtype or torch.float32, device=x.device)
        dt = {torch.float32: 0, torch.bfloat16: 1}
        rc = lib().gllmk_ffn_prefill(self._ctx, w_gate_up._h, w_down._h, _ptr(x), dt[x.dtype], x.stride(0), m, _ptr(h), _ptr(y),
                                     dt[y.dtype], y.stride(0), _stream(stream))
        self._check(rc, "gllmk_ffn_prefill")
        return y

    def gemm_grouped(self, weights, a, row_offsets, y=None, out_dtype=None, stream=None):
        """Mixture-of-experts product in one launch: rows [row_offsets[g], row_offsets[g+1]) of `a` times weights[g]."""
        import torch
        ng = len(weights)
        if y is None:
            y = torch.empty((a.shape[0], weights[0].n), dtype=out_dtype or torch.float32, device=a.device)
        dt = {torch.float32: 0, torch.bfloat16: 1}
        hs = (C.c_void_p * ng)(*[w._h for w in weights])
        offs = (C.c_int64 * (ng + 1))(*[int(o) for o in row_offsets])
        rc = lib().gllmk_gemm_grouped(self._ctx, ng, hs, _ptr(a), dt[a.dtype], a.stride(0), offs, _ptr(y), dt[y.dtype],
                                      y.stride(0), _stream(stream))
        self._check(rc, "gllmk_gemm_grouped")
        return y

    # ---- mixture-of-experts routing conventions (scalar-ops/src/moe.rs:59-157) ----
    def moe_topk(self, gate_probs, top_k: int, stream=None):
        """scalar_topk: gate_probs [seq, experts] f32 CUDA -> [2, seq * top_k] f32: row 0 the expert indices as u32
        bit patterns, row 1 the renormalised weights (the reference's output buffer, viewed as two rows)."""
        import torch
        seq, ne = gate_probs.shape
        out = torch.empty((2, seq * top_k), dtype=torch.float32, device=gate_probs.device)
        self._check(lib().gllmk_moe_topk(self._ctx, _ptr(gate_probs.contiguous()), _ptr(out), seq, ne, top_k, _stream(stream)),
                    "gllmk_moe_topk")
        return out

    def moe_route(self, routing, seq_len: int, num_experts: int, top_k: int, stream=None):
        """Groups the slots of a scalar_topk result per expert: (row_offsets list, perm int32 [seq * top_k],
        inv int32 [seq * top_k])."""
        import torch
        slots = seq_len * top_k
        perm = torch.empty(slots, dtype=torch.int32, device=routing.device)
        inv = torch.empty(slots, dtype=torch.int32, device=routing.device)
        offs = (C.c_int64 * (num_experts + 1))()
        self._check(lib().gllmk_moe_route(self._ctx, _ptr(routing), seq_len, num_experts, top_k, offs, _ptr(perm), _ptr(inv),
                                          _stream(stream)), "gllmk_moe_route")
        return list(offs), perm, inv

    def moe_gather(self, x, perm, top_k: int, rows: int = None, stream=None):
        """x [seq, k] (f32 or bf16) -> [rows, k] in grouped order."""
        import torch
        rows = perm.numel() if rows is None else rows
        out = torch.empty((rows, x.shape[1]), dtype=x.dtype, device=x.device)
        dt = {torch.float32: 0, torch.bfloat16: 1}
        self._check(lib().gllmk_moe_gather(self._ctx, _ptr(x), dt[x.dtype], x.stride(0), _ptr(perm), rows, top_k, x.shape[1],
                                           _ptr(out), out.stride(0), _stream(stream)), "gllmk_moe_gather")
        return out

    def moe_weighted_sum(self, expert_outputs, routing, inv, seq_len: int, top_k: int, num_experts: int = 1 << 30, stream=None):
        """scalar_weighted_sum.  inv=None: expert_outputs is the reference's [experts, seq, hidden] buffer; else the
        grouped rows [seq * top_k, hidden] and `inv` from moe_route."""
        import torch
        hidden = expert_outputs.shape[-1]
        if inv is None:
            num_experts = expert_outputs.shape[0]
        out = torch.empty((seq_len, hidden), dtype=torch.float32, device=expert_outputs.device)
        slots = seq_len * top_k
        flat = routing.reshape(-1)
        self._check(lib().gllmk_moe_weighted_sum(self._ctx, _ptr(expert_outputs), expert_outputs.stride(-2), _ptr(flat),
                                                 flat.data_ptr() + 4 * slots, _ptr(inv), _ptr(out), seq_len, hidden, top_k,
                                                 min(num_experts, (1 << 31) - 1), _stream(stream)), "gllmk_moe_weighted_sum")
        return out

    def probe_fp4_mma(self, cta_pair: bool = True, with_scale_copies: int = 2, nvfp4: bool = True, ksteps: int = 4096) -> float:
        """TFLOP/s of the block-scaled FP4 MMA issued back to back on shared-memory operands (the practical ceiling of
        gemm_fp4 on this device).  with_scale_copies: 0 none, 1 tcgen05.cp per k-step, 2 tcgen05.st by scale warps."""
        v = C.c_float()
        self._check(lib().gllmk_probe_fp4_mma(self._ctx, int(cta_pair), int(with_scale_copies), int(nvfp4), ksteps, C.byref(v)),
                    "gllmk_probe_fp4_mma")
        return v.value

    def gemm_fp4(self, w: Weight, x: Weight, y=None, out_dtype=None, stream=None):
        """Native FP4 x FP4 product: `x` is the activation matrix [m, k] quantized and uploaded like a weight."""
        import torch
        if y is None:
            y = torch.empty((x.n, w.n), dtype=out_dtype or torch.float32, device=f"cuda:{self.device}")
        dt = {torch.float32: 0, torch.bfloat16: 1}
        rc = lib().gllmk_gemm_fp4(self._ctx, w._h, x._h, _ptr(y), dt[y.dtype], y.stride(0), _stream(stream))
        self._check(rc, "gllmk_gemm_fp4")
        return y

    # ---- multi-GPU exchange buffers (one process per GPU, same node) ----
    def shared_alloc(self, nbytes: int):
        """Device buffer other ranks can map: returns (device pointer, 64-byte handle to send to them)."""
        ptr, handle = C.c_void_p(), C.create_string_buffer(64)
        self._check(lib().gllmk_shared_alloc(self._ctx, nbytes, C.byref(ptr), handle), "gllmk_shared_alloc")
        return ptr.value, handle.raw

    def shared_open(self, handle: bytes) -> int:
        ptr = C.c_void_p()
        self._check(lib().gllmk_shared_open(self._ctx, C.create_string_buffer(handle, 64), C.byref(ptr)), "gllmk_shared_open")
        return ptr.value

    def shared_close(self, ptr: int) -> None:
        self._check(lib().gllmk_shared_close(self._ctx, ptr), "gllmk_shared_close")

    def shared_free(self, ptr: int) -> None:
        self._check(lib().gllmk_shared_free(self._ctx, ptr), "gllmk_shared_free")

    def gemv_allgather(self, w: Weight, x, y_local: int, y_peers, y_stride_t: int, m: int, stream=None) -> None:
        """Decode product whose band of y is stored at `y_local` and at every pointer of `y_peers` (raw device
        addresses of the band's position in each rank's y; row stride 1, token stride y_stride_t)."""
        arr = (C.c_void_p * max(len(y_peers), 1))(*y_peers)
        rc = lib().gllmk_gemv_allgather(self._ctx, w._h, _ptr(x), x.stride(0), x.stride(1), m, y_local, y_stride_t, 1,
                                        arr, len(y_peers), _stream(stream))
        self._check(rc, "gllmk_gemv_allgather")

    def gemv_exchange(self, w: Weight, x, y_local: int, y_peers, y_stride_t: int, m: int, flags_local: int, flags_peers,
                      rank: int, stream=None, x_up=None) -> None:
        """gemv_allgather with the hand-shake built in: waits for every rank's previous exchange product before x
        is read, signals this one's completion from the GEMV's last block.  x_up: the activation is silu(x) * x_up."""
        ya = (C.c_void_p * max(len(y_peers), 1))(*y_peers)
        fa = (C.c_void_p * max(len(flags_peers), 1))(*flags_peers)
        rc = lib().gllmk_gemv_exchange(self._ctx, w._h, _ptr(x), _ptr(x_up), x.stride(0), x.stride(1), m, y_local, y_stride_t, 1, ya,
                                       flags_local, fa, len(y_peers), rank, _stream(stream))
        self._check(rc, "gllmk_gemv_exchange")

    def exchange_wait(self, flags_local: int, n_peers: int, rank: int, stream=None) -> None:
        self._check(lib().gllmk_exchange_wait(self._ctx, flags_local, n_peers, rank, _stream(stream)), "gllmk_exchange_wait")

    def peer_barrier(self, flags_local: int, flags_peers, rank: int, seq: int, stream=None) -> None:
        arr = (C.c_void_p * max(len(flags_peers), 1))(*flags_peers)
        rc = lib().gllmk_peer_barrier(self._ctx, flags_local, arr, len(flags_peers), rank, seq & 0xFFFFFFFF, _stream(stream))
        self._check(rc, "gllmk_peer_barrier")

    def gemv_static(self, w: Weight, x, y, ref_layout: bool = False, row_scales=None, stream=None):
        """gemv for callers that may not allocate device memory: scratch is a fixed 8 MiB area inside the
        library (shared by every call on the device — do not overlap calls).  `y` must be preallocated.
        Raises INVALID_ARG for shapes whose scratch does not fit."""
        m = x.shape[1] if ref_layout else x.shape[0]
        xs, ys = ((1, m), (1, m)) if ref_layout else ((w.k, 1), (w.n, 1))
        ns = 0 if row_scales is None else row_scales.numel()
        rc = lib().gllmk_gemv_static(self._ctx, w._h, _ptr(x), xs[0], xs[1], m, _ptr(y), ys[0], ys[1],
                                     _ptr(row_scales), ns, _stream(stream))
        self._check(rc, "gllmk_gemv_static")
        return y

    def matmul_host(self, w: Weight, x, ref_layout: bool = False, out=None) -> np.ndarray:
        """Resident weight, HOST activations and outputs (numpy): the call timed end to end.  Page-locked arrays
        (e.g. torch.empty(..., pin_memory=True).numpy()) for `x` and `out` are used without a staging copy."""
        x = _np(x, np.float32)
        m = x.shape[1] if ref_layout else x.shape[0]
        shape = (w.n, m) if ref_layout else (m, w.n)
        y = np.empty(shape, np.float32) if out is None else _np(out, np.float32, True)
        if y.shape != shape:
            raise ValueError(f"out has shape {y.shape}, expected {shape}")
        self._check(lib().gllmk_matmul_host(self._ctx, w._h, _ptr(x), m, _ptr(y), int(ref_layout)), "gllmk_matmul_host")
        return y

    def matmul_host_batch(self, weights, xs, outs, ref_layout: bool = False):
        """The products of one decode step in one call: outs[i] = product of weights[i] and xs[i] (numpy f32, [m, k] ->
        [m, n]; page-locked arrays are used in place), enqueued back to back and awaited once."""
        n = len(weights)
        ms = (C.c_int32 * n)(*[(x.shape[1] if ref_layout else x.shape[0]) for x in xs])
        wh = (C.c_void_p * n)(*[w._h for w in weights])
        xp = (C.c_void_p * n)(*[_ptr(_np(x, np.float32)) for x in xs])
        yp = (C.c_void_p * n)(*[_ptr(_np(y, np.float32, True)) for y in outs])
        self._check(lib().gllmk_matmul_host_batch(self._ctx, n, wh, xp, ms, yp, int(ref_layout)), "gllmk_matmul_host_batch")
        return outs

    def host_batch(self, weights, xs, outs, ref_layout: bool = False) -> "HostBatch":
        """The argument arrays of `matmul_host_batch` built once, for a step that is run many times on the same host
        buffers (a decode loop): `HostBatch.run()` is then one C call with nothing to convert."""
        return HostBatch(self, weights, xs, outs, ref_layout)

    def quantize(self, quant_type: QuantType, x, global_scale: float = 0.0, stream=None):
        """f32 [rows, k] CUDA tensor -> reference-format blocks (CUDA uint8 tensors).
        Returns blocks for Q4K/Q8_0, (blocks, scales) for MXFP4, (blocks, global_scale) for NVFP4."""
        import torch
        rows, k = x.shape
        bs, bb = quant_type.block_size(), quant_type.block_bytes()
        nblk = rows * k // bs
        g = C.c_float(global_scale)
        if quant_type.id == Q.MXFP4:
            blocks = torch.empty(nblk * bs // 2, dtype=torch.uint8, device=x.device)
            scales = torch.empty(nblk, dtype=torch.uint8, device=x.device)
        else:
            blocks = torch.empty(nblk * bb, dtype=torch.uint8, device=x.device)
            scales = None
        rc = lib().gllmk_quantize(self._ctx, quant_type.id, _ptr(x), rows, k, quant_type.mx_block, _ptr(blocks),
                                  _ptr(scales), C.byref(g), _stream(stream))
        self._check(rc, "gllmk_quantize")
        if quant_type.id == Q.MXFP4:
            return blocks, scales
        if quant_type.id == Q.NVFP4:
            return blocks, g.value
        return blocks

    # ---- the reference's operator methods (host arrays, E = f32) -------------------------------
    def dequant_q4_k(self, block, out) -> None:
        """Kernels::dequant_q4_k(block, out) (src/traits.rs:476)."""
        block, out = _np(block, np.uint8), _np(out, np.float32, True)
        self._check(lib().gllmk_dequant_q4_k(self._ctx, _ptr(block), _ptr(out), block.size // 144), "dequant_q4_k")

    def dequant_q8_0(self, block, out) -> None:
        """Kernels::dequant_q8_0(block, out) (src/traits.rs:488)."""
        block, out = _np(block, np.uint8), _np(out, np.float32, True)
        self._check(lib().gllmk_dequant_q8_0(self._ctx, _ptr(block), _ptr(out), block.size // 34), "dequant_q8_0")

    def dequant_mxfp4(self, blocks, scales, output, block_size: int) -> None:
        """quant_mxfp4::dequant_mxfp4(blocks, scales, output, block_size) (src/quant_mxfp4.rs:267-292)."""
        blocks, scales, output = _np(blocks, np.uint8), _np(scales, np.uint8), _np(output, np.float32, True)
        if block_size <= 0 or block_size % 2 or blocks.size != scales.size * block_size // 2 \
                or output.size != scales.size * block_size:
            raise GllmkError(Status.INVALID_ARG, "dequant_mxfp4", "length mismatch")  # reference returns Err
        self._check(lib().gllmk_dequant_mxfp4(self._ctx, _ptr(blocks), _ptr(scales), _ptr(output), scales.size,
                                              block_size), "dequant_mxfp4")

    def dequant_nvfp4(self, blocks, global_scale: float, output) -> None:
        blocks, output = _np(blocks, np.uint8), _np(output, np.float32, True)
        self._check(lib().gllmk_dequant_nvfp4(self._ctx, _ptr(blocks), float(global_scale), _ptr(output),
                                              blocks.size // 36), "dequant_nvfp4")

    def dequant_gguf(self, quant_type: QuantType, blocks, out) -> None:
        """Kernels::dequant_q6_k / dequant_q5_k / dequant_q8_k / dequant_q4_0 / dequant_q5_0 (block, out)
        (scalar decoders src/macros/quant_primitive/k_quant.rs:92-101,381-472, classic.rs:15-29,484-504)."""
        blocks, out = _np(blocks, np.uint8), _np(out, np.float32, True)
        self._check(lib().gllmk_dequant_gguf(self._ctx, quant_type.id, _ptr(blocks), _ptr(out),
                                             blocks.size // quant_type.block_bytes()), "dequant_gguf")

    def dequant_q6_k(self, block, out) -> None:
        self.dequant_gguf(QuantType.q6k(), block, out)

    def dequant_q5_k(self, block, out) -> None:
        self.dequant_gguf(QuantType.q5k(), block, out)

    def dequant_q8_k(self, block, out) -> None:
        self.dequant_gguf(QuantType.q8k(), block, out)

    def dequant_q4_0(self, block, out) -> None:
        self.dequant_gguf(QuantType.q4_0(), block, out)

    def dequant_q5_0(self, block, out) -> None:
        self.dequant_gguf(QuantType.q5_0(), block, out)

    def kquant_matmul(self, weight_blocks, input, output, quant_type: QuantType, m: int, n: int, k: int) -> None:
        """Kernels::kquant_matmul (src/traits.rs:543-551): m weight rows, n batch columns, input [k, n],
        output [m, n]."""
        w, x, y = _np(weight_blocks, np.uint8), _np(input, np.float32), _np(output, np.float32, True)
        self._check(lib().gllmk_kquant_matmul_f32(self._ctx, _ptr(w), _ptr(x), _ptr(y), quant_type.id, m, n, k),
                    "kquant_matmul")

    def classic_matmul(self, weight_blocks, input, output, quant_type: QuantType, m: int, n: int, k: int) -> None:
        """Kernels::classic_matmul (src/traits.rs:553-563)."""
        w, x, y = _np(weight_blocks, np.uint8), _np(input, np.float32), _np(output, np.float32, True)
        self._check(lib().gllmk_classic_matmul_f32(self._ctx, _ptr(w), _ptr(x), _ptr(y), quant_type.id, m, n, k),
                    "classic_matmul")

    def gemm_q4(self, weight, input, output, scales, m: int, n: int, k: int) -> None:
        """Kernels::gemm_q4 (src/traits.rs:511-520): m batch rows, n features, input [m, k], output [m, n]."""
        w, x, y = _np(weight, np.uint8), _np(input, np.float32), _np(output, np.float32, True)
        s = _np(scales, np.float32) if scales is not None and len(scales) else None
        self._check(lib().gllmk_gemm_q4_f32(self._ctx, _ptr(w), _ptr(x), _ptr(y), _ptr(s), 0 if s is None else s.size,
                                            m, n, k), "gemm_q4")

    def gemm_q8(self, weight, input, output, scales, m: int, n: int, k: int) -> None:
        """Kernels::gemm_q8 (src/traits.rs:502-510): Q8_K rows; `weight` is the reference's i8 (or u8) view of the blocks."""
        w = np.ascontiguousarray(weight).view(np.uint8)
        x, y = _np(input, np.float32), _np(output, np.float32, True)
        s = _np(scales, np.float32) if scales is not None and len(scales) else None
        self._check(lib().gllmk_gemm_q8_f32(self._ctx, _ptr(w), _ptr(x), _ptr(y), _ptr(s), 0 if s is None else s.size,
                                            m, n, k), "gemm_q8")

    def gemv_q4(self, weight, input, scale: float, n: int) -> float:
        """Kernels::gemv_q4 (src/traits.rs:501): one Q4_K row of n elements, result * scale."""
        out = np.empty(1, np.float32)
        w, x = _np(weight, np.uint8), _np(input, np.float32)
        self._check(lib().gllmk_gemv_q4_f32(self._ctx, _ptr(w), _ptr(x), float(scale), n, _ptr(out)), "gemv_q4")
        return float(out[0])

    def gemv_q8(self, weight, input, scale: float, n: int) -> float:
        """Kernels::gemv_q8 (src/traits.rs:500): one Q8_K row of n elements, result * scale."""
        out = np.empty(1, np.float32)
        w, x = np.ascontiguousarray(weight).view(np.uint8), _np(input, np.float32)
        self._check(lib().gllmk_gemv_q8_f32(self._ctx, _ptr(w), _ptr(x), float(scale), n, _ptr(out)), "gemv_q8")
        return float(out[0])


class HostBatch:
    """Prebuilt argument arrays of one `gllmk_matmul_host_batch` step (see GpuKernels.host_batch).  Keeps the weights and
    the host arrays alive; the arrays' contents may change between runs, their addresses may not."""

    def __init__(self, K: "GpuKernels", weights, xs, outs, ref_layout: bool = False):
        self.K, self.weights, self.ref_layout = K, list(weights), bool(ref_layout)
        self.xs = [_np(x, np.float32) for x in xs]
        self.outs = [_np(y, np.float32, True) for y in outs]
        n = self.n = len(self.weights)
        self._ms = (C.c_int32 * n)(*[(x.shape[1] if ref_layout else x.shape[0]) for x in self.xs])
        self._wh = (C.c_void_p * n)(*[w._h for w in self.weights])
        self._xp = (C.c_void_p * n)(*[_ptr(x) for x in self.xs])
        self._yp = (C.c_void_p * n)(*[_ptr(y) for y in self.outs])
        self._fn = lib().gllmk_matmul_host_batch

    def run(self):
        rc = self._fn(self.K._ctx, self.n, self._wh, self._xp, self._ms, self._yp, int(self.ref_layout))
        if rc:
            self.K._check(rc, "gllmk_matmul_host_batch")
        return self.outs
