//! `GpuKernels`: the quant slice of gllm-kernels' operator API on a B200, bound to libgllmk.so.
//!
//! Drop this file into gllm-kernels as `src/gpu_b200.rs` (behind a `b200` cargo feature, `mod gpu_b200;` in
//! `src/lib.rs`) and link `gllmk` (`cargo:rustc-link-lib=dylib=gllmk` + the search path of libgllmk.so in
//! `build.rs`).  Every method below has the name, the argument order, the shape conventions and the panics of
//! the method of `Kernels<f32>` it replaces (`src/traits.rs:473-608`; CPU implementation
//! `src/cpu_kernels/mod.rs:2888-3031, 3226-3394`), so callers switch by constructing a `GpuKernels` instead of a
//! `CpuKernels<f32>`.  The formats outside this library's scope (Q2_K, Q3_K, the `_1` formats, IQ*, AWQ / GPTQ /
//! Squeeze) are not declared here: keep calling `CpuKernels` for them.
//!
//! Written against include/gllmk.h; this image has no Rust toolchain, so the file is shipped uncompiled — the
//! signatures are transcribed from the header one to one.
//!
//! The reference's operator methods take host slices.  They work as they are (weights are uploaded and repacked
//! on every call, as the header says), but a decode loop should upload each tensor once (`upload`) and call
//! `matmul` / `gemv_dev` with the handle: that is the path the throughput numbers are measured on.

#![allow(clippy::too_many_arguments)]

use crate::quant::QuantType;
use std::ffi::{c_char, c_void, CStr};

// ---- status codes (src/ffi/types.rs:4-14, same integers) -------------------------------------------------------
pub const OK: i32 = 0;
pub const INVALID_ARG: i32 = -1;
pub const OUT_OF_MEMORY: i32 = -2;
pub const RUNTIME_ERROR: i32 = -4;
pub const UNSUPPORTED: i32 = -5;

/// `gllmk_quant_format_descriptor` of include/gllmk.h (QuantFormatDescriptor flattened for C).
#[repr(C)]
#[derive(Debug, Clone, Copy, Default, PartialEq, Eq)]
pub struct GllmkQuantFormatDescriptor {
    pub quant_type: i32,
    pub block_size: i32,
    pub block_bytes: i32,
    pub bits_per_element: i32,
    pub scale_kind: i32,
    pub scale_dtype: i32,
    pub scale_offset: i32,
    pub scale_min_offset: i32,
    pub sub_scales_offset: i32,
    pub sub_scales_bits: i32,
    pub sub_scales_count: i32,
    pub sub_block_elements: i32,
    pub zero_kind: i32,
    pub zero_offset: i32,
    pub zero_sub_offset: i32,
    pub static_bias: i32,
    pub data_layout: i32,
    pub data_offset: i32,
    pub data_high_offset: i32,
    pub data_high_bits: i32,
    pub data_low_first: i32,
    pub data_signed: i32,
    pub data_kind: i32,
    pub storage_layout: i32,
    pub native_isa: i32,
}

#[link(name = "gllmk")]
extern "C" {
    fn gllmk_version() -> *const c_char;
    fn gllmk_hw_info(buf: *mut c_char, len: usize) -> i32;
    fn gllmk_quant_block_size(quant_type: i32, mx_block: i32) -> i32;
    fn gllmk_quant_block_bytes(quant_type: i32, mx_block: i32) -> i32;
    fn gllmk_quant_format_descriptor_for_type(quant_type: i32, mx_block: i32, out: *mut GllmkQuantFormatDescriptor) -> i32;
    fn gllmk_quant_format_registry(quant_types: *mut i32, cap: i32) -> i32;

    fn gllmk_ctx_create(device: i32, out: *mut *mut c_void) -> i32;
    fn gllmk_ctx_free(ctx: *mut c_void);
    fn gllmk_last_error(ctx: *mut c_void) -> *const c_char;
    fn gllmk_ctx_status(ctx: *mut c_void, device_status: *mut i32) -> i32;
    fn gllmk_ctx_set(ctx: *mut c_void, key: *const c_char, value: i64) -> i32;

    fn gllmk_weight_upload(ctx: *mut c_void, quant_type: i32, n: i64, k: i64, mx_block: i32, blocks: *const c_void,
                           scales: *const c_void, global_scale: f32, src_on_device: i32, out: *mut *mut c_void) -> i32;
    fn gllmk_weight_free(w: *mut c_void);
    fn gllmk_weight_info(w: *mut c_void, quant_type: *mut i32, n: *mut i64, k: *mut i64, ref_bytes: *mut u64, dev_bytes: *mut u64) -> i32;
    fn gllmk_weight_unpack(ctx: *mut c_void, w: *mut c_void, blocks: *mut c_void, scales: *mut c_void, dst_on_device: i32) -> i32;
    fn gllmk_dequant(ctx: *mut c_void, w: *mut c_void, out_dev: *mut f32, stream: *mut c_void) -> i32;
    fn gllmk_embedding_gather(ctx: *mut c_void, w: *mut c_void, ids_dev: *const i32, count: i64, out_dev: *mut f32, stream: *mut c_void) -> i32;

    fn gllmk_gemv(ctx: *mut c_void, w: *mut c_void, x_dev: *const f32, x_stride_t: i64, x_stride_k: i64, m: i32, y_dev: *mut f32,
                  y_stride_t: i64, y_stride_r: i64, row_scales: *const f32, n_row_scales: i64, stream: *mut c_void) -> i32;
    fn gllmk_gemv_static(ctx: *mut c_void, w: *mut c_void, x_dev: *const f32, x_stride_t: i64, x_stride_k: i64, m: i32, y_dev: *mut f32,
                         y_stride_t: i64, y_stride_r: i64, row_scales: *const f32, n_row_scales: i64, stream: *mut c_void) -> i32;
    fn gllmk_ffn_decode(ctx: *mut c_void, w_gate_up: *mut c_void, w_down: *mut c_void, x_dev: *const f32, m: i32, h_dev: *mut f32,
                        y_dev: *mut f32, stream: *mut c_void) -> i32;
    fn gllmk_ffn_prefill(ctx: *mut c_void, w_gate_up: *mut c_void, w_down: *mut c_void, x_dev: *const c_void, x_dtype: i32, ldx: i64, m: i32,
                         h_dev: *mut c_void, y_dev: *mut c_void, y_dtype: i32, ldy: i64, stream: *mut c_void) -> i32;
    fn gllmk_gemm(ctx: *mut c_void, w: *mut c_void, a_dev: *const c_void, a_dtype: i32, lda: i64, m: i32, y_dev: *mut c_void,
                  y_dtype: i32, ldy: i64, stream: *mut c_void) -> i32;
    fn gllmk_gemm_grouped(ctx: *mut c_void, n_groups: i32, weights: *const *mut c_void, a_dev: *const c_void, a_dtype: i32, lda: i64,
                          row_offsets: *const i64, y_dev: *mut c_void, y_dtype: i32, ldy: i64, stream: *mut c_void) -> i32;
    fn gllmk_gemm_fp4(ctx: *mut c_void, w: *mut c_void, x: *mut c_void, y_dev: *mut c_void, y_dtype: i32, ldy: i64, stream: *mut c_void) -> i32;
    fn gllmk_probe_fp4_mma(ctx: *mut c_void, cta_pair: i32, with_scale_copies: i32, nvfp4: i32, ksteps: i32, tflops: *mut f32) -> i32;
    fn gllmk_quantize(ctx: *mut c_void, quant_type: i32, x_dev: *const f32, rows: i64, k: i64, mx_block: i32, blocks_dev: *mut c_void,
                      scales_dev: *mut c_void, global_scale: *mut f32, stream: *mut c_void) -> i32;

    fn gllmk_moe_topk(ctx: *mut c_void, gate_probs_dev: *const f32, out_dev: *mut f32, seq_len: i64, num_experts: i32, top_k: i32,
                      stream: *mut c_void) -> i32;
    fn gllmk_moe_route(ctx: *mut c_void, indices_dev: *const f32, seq_len: i64, num_experts: i32, top_k: i32, row_offsets_host: *mut i64,
                       perm_dev: *mut i32, inv_dev: *mut i32, stream: *mut c_void) -> i32;
    fn gllmk_moe_gather(ctx: *mut c_void, x_dev: *const c_void, dtype: i32, ldx: i64, perm_dev: *const i32, rows: i64, top_k: i32, k: i64,
                        out_dev: *mut c_void, ldo: i64, stream: *mut c_void) -> i32;
    fn gllmk_moe_weighted_sum(ctx: *mut c_void, expert_outputs_dev: *const f32, ld: i64, indices_dev: *const f32, weights_dev: *const f32,
                              inv_dev: *const i32, out_dev: *mut f32, seq_len: i64, hidden: i64, top_k: i32, num_experts: i32,
                              stream: *mut c_void) -> i32;

    fn gllmk_int8_weight_upload(ctx: *mut c_void, n: i64, k: i64, b: *const i8, layout: i32, src_on_device: i32, out: *mut *mut c_void) -> i32;
    fn gllmk_gemm_int8(ctx: *mut c_void, w: *mut c_void, a_dev: *const u8, lda: i64, m: i32, c_dev: *mut i32, ldc: i64, stream: *mut c_void) -> i32;
    fn gllmk_dequantize_i32_f32(ctx: *mut c_void, c_dev: *const i32, out_dev: *mut f32, m: i64, n: i64, scale_a: f32, scale_b: f32,
                                bias_dev: *const f32, activation: i32, stream: *mut c_void) -> i32;
    fn gllmk_gemm_int8_host(ctx: *mut c_void, a: *const u8, b_kn: *const i8, c: *mut i32, m: usize, n: usize, k: usize) -> i32;
    fn gllmk_quantize_act_int8(ctx: *mut c_void, x_dev: *const f32, rows: i64, k: i64, ldx: i64, q_dev: *mut c_void, ldq: i64,
                               as_unsigned: i32, scale_dev: *mut f32, stream: *mut c_void) -> i32;
    fn gllmk_w8a8_linear_f32(ctx: *mut c_void, w: *mut c_void, x_dev: *const f32, ldx: i64, m: i32, y_dev: *mut f32, ldy: i64, scale_b: f32,
                             bias_dev: *const f32, activation: i32, stream: *mut c_void) -> i32;

    fn gllmk_shared_alloc(ctx: *mut c_void, bytes: usize, dev_ptr: *mut *mut c_void, handle: *mut u8) -> i32;
    fn gllmk_shared_open(ctx: *mut c_void, handle: *const u8, peer_ptr: *mut *mut c_void) -> i32;
    fn gllmk_shared_close(ctx: *mut c_void, peer_ptr: *mut c_void) -> i32;
    fn gllmk_shared_free(ctx: *mut c_void, dev_ptr: *mut c_void) -> i32;
    fn gllmk_gemv_allgather(ctx: *mut c_void, w: *mut c_void, x_dev: *const f32, x_stride_t: i64, x_stride_k: i64, m: i32, y_local: *mut f32,
                            y_stride_t: i64, y_stride_r: i64, y_peers: *const *mut c_void, n_peers: i32, stream: *mut c_void) -> i32;
    fn gllmk_peer_barrier(ctx: *mut c_void, flags_local: *mut c_void, flags_peers: *const *mut c_void, n_peers: i32, rank: i32, seq: u32,
                          stream: *mut c_void) -> i32;
    fn gllmk_gemv_exchange(ctx: *mut c_void, w: *mut c_void, x_dev: *const f32, x_up_dev: *const f32, x_stride_t: i64, x_stride_k: i64, m: i32, y_local: *mut f32,
                           y_stride_t: i64, y_stride_r: i64, y_peers: *const *mut c_void, flags_local: *mut c_void,
                           flags_peers: *const *mut c_void, n_peers: i32, rank: i32, stream: *mut c_void) -> i32;
    fn gllmk_exchange_wait(ctx: *mut c_void, flags_local: *mut c_void, n_peers: i32, rank: i32, stream: *mut c_void) -> i32;

    fn gllmk_kquant_matmul_f32(ctx: *mut c_void, weight_blocks: *const u8, input: *const f32, output: *mut f32, quant_type: i32, m: usize,
                               n: usize, k: usize) -> i32;
    fn gllmk_classic_matmul_f32(ctx: *mut c_void, weight_blocks: *const u8, input: *const f32, output: *mut f32, quant_type: i32, m: usize,
                                n: usize, k: usize) -> i32;
    fn gllmk_gemm_q4_f32(ctx: *mut c_void, weight: *const u8, input: *const f32, output: *mut f32, scales: *const f32, n_scales: usize,
                         m: usize, n: usize, k: usize) -> i32;
    fn gllmk_gemm_q8_f32(ctx: *mut c_void, weight: *const i8, input: *const f32, output: *mut f32, scales: *const f32, n_scales: usize,
                         m: usize, n: usize, k: usize) -> i32;
    fn gllmk_gemv_q4_f32(ctx: *mut c_void, weight: *const u8, input: *const f32, scale: f32, n: usize, out: *mut f32) -> i32;
    fn gllmk_gemv_q8_f32(ctx: *mut c_void, weight: *const i8, input: *const f32, scale: f32, n: usize, out: *mut f32) -> i32;
    fn gllmk_matmul_host_batch(ctx: *mut c_void, count: i32, weights: *const *mut c_void, x_host: *const *const f32, m: *const i32,
                               y_host: *const *mut f32, ref_layout: i32) -> i32;
    fn gllmk_matmul_host(ctx: *mut c_void, w: *mut c_void, x_host: *const f32, m: i32, y_host: *mut f32, ref_layout: i32) -> i32;
    fn gllmk_dequant_q4_k(ctx: *mut c_void, blocks: *const u8, out: *mut f32, nblocks: usize) -> i32;
    fn gllmk_dequant_q8_0(ctx: *mut c_void, blocks: *const u8, out: *mut f32, nblocks: usize) -> i32;
    fn gllmk_dequant_mxfp4(ctx: *mut c_void, blocks: *const u8, scales: *const u8, out: *mut f32, num_blocks: usize, block_size: usize) -> i32;
    fn gllmk_dequant_nvfp4(ctx: *mut c_void, blocks: *const u8, global_scale: f32, out: *mut f32, nblocks: usize) -> i32;
    fn gllmk_dequant_gguf(ctx: *mut c_void, quant_type: i32, blocks: *const u8, out: *mut f32, nblocks: usize) -> i32;
}

/// Ids of include/gllmk.h for the formats this library serves; 0 for everything else.
pub fn quant_type_id(q: QuantType) -> (i32, i32) {
    match q {
        QuantType::Q4K => (1, 0),
        QuantType::Q8_0 => (2, 0),
        QuantType::Mxfp4 { block_size } => (3, block_size as i32),
        QuantType::Nvfp4 => (4, 0),
        QuantType::Q6K => (6, 0),
        QuantType::Q5K => (7, 0),
        QuantType::Q4_0 => (8, 0),
        QuantType::Q5_0 => (9, 0),
        QuantType::Q8K => (10, 0),
        _ => (0, 0),
    }
}

/// `QuantFormatDescriptor::for_type` (src/quant_format.rs:36-44) read from the table the device kernels use.
/// Panics for a type the library does not serve, as the reference does for an unregistered type.
pub fn format_descriptor(q: QuantType) -> GllmkQuantFormatDescriptor {
    let (id, mx) = quant_type_id(q);
    let mut d = GllmkQuantFormatDescriptor::default();
    let rc = unsafe { gllmk_quant_format_descriptor_for_type(id, if mx == 0 { 32 } else { mx }, &mut d) };
    if rc != OK {
        panic!("QuantFormatDescriptor::for_type: no descriptor registered for {:?}", q);
    }
    d
}

/// `registry()` (src/quant_format.rs:1189-1193), restricted to the served formats: their ids.
pub fn registry() -> Vec<i32> {
    let mut ids = vec![0i32; 32];
    let n = unsafe { gllmk_quant_format_registry(ids.as_mut_ptr(), ids.len() as i32) } as usize;
    ids.truncate(n.min(32));
    ids
}

pub fn version() -> String {
    unsafe { CStr::from_ptr(gllmk_version()) }.to_string_lossy().into_owned()
}

pub fn hw_info() -> String {
    let mut buf = vec![0u8; 256];
    let n = unsafe { gllmk_hw_info(buf.as_mut_ptr() as *mut c_char, buf.len()) };
    buf.truncate(n.max(0) as usize);
    String::from_utf8_lossy(&buf).into_owned()
}

/// A weight matrix resident in HBM in the kernels' tiled layout (gllmk_weight).
pub struct GpuWeight {
    h: *mut c_void,
    pub n: usize,
    pub k: usize,
}
unsafe impl Send for GpuWeight {}
unsafe impl Sync for GpuWeight {} // immutable after upload
impl Drop for GpuWeight {
    fn drop(&mut self) {
        unsafe { gllmk_weight_free(self.h) }
    }
}
impl GpuWeight {
    pub fn raw(&self) -> *mut c_void {
        self.h
    }
    /// (reference-format bytes, bytes held on the device)
    pub fn bytes(&self) -> (u64, u64) {
        let (mut r, mut d) = (0u64, 0u64);
        unsafe { gllmk_weight_info(self.h, std::ptr::null_mut(), std::ptr::null_mut(), std::ptr::null_mut(), &mut r, &mut d) };
        (r, d)
    }
}

/// One CUDA device's context.  `Send + Sync` like `Kernels` (src/traits.rs:387), but calls made through one
/// context must not overlap in time (they share scratch): keep one `GpuKernels` per inference thread / stream.
pub struct GpuKernels {
    ctx: *mut c_void,
}
unsafe impl Send for GpuKernels {}
unsafe impl Sync for GpuKernels {}
impl Drop for GpuKernels {
    fn drop(&mut self) {
        unsafe { gllmk_ctx_free(self.ctx) }
    }
}

impl GpuKernels {
    /// Err(RUNTIME_ERROR) without a CUDA device: there is no CPU fallback.
    pub fn new(device: i32) -> Result<Self, i32> {
        let mut ctx = std::ptr::null_mut();
        match unsafe { gllmk_ctx_create(device, &mut ctx) } {
            OK => Ok(Self { ctx }),
            e => Err(e),
        }
    }

    fn last_error(&self) -> String {
        unsafe { CStr::from_ptr(gllmk_last_error(self.ctx)) }.to_string_lossy().into_owned()
    }

    /// Panics with the library's message on any status but OK (the reference's methods panic on misuse too).
    fn check(&self, rc: i32, what: &str) {
        if rc == UNSUPPORTED {
            unimplemented!("{what}: {}", self.last_error()); // the reference: unimplemented!() for a wrong-family type
        }
        assert!(rc == OK, "{what} failed with status {rc}: {}", self.last_error());
    }

    /// Device status word: Err(code) if a kernel gave up a bounded wait since the last call (results of that call
    /// are incomplete; the context is usable again afterwards).
    pub fn status(&self) -> Result<(), i32> {
        let mut v = 0i32;
        match unsafe { gllmk_ctx_status(self.ctx, &mut v) } {
            OK => Ok(()),
            _ => Err(v),
        }
    }

    // ---- resident weights ------------------------------------------------------------------------------------
    /// `blocks`: the reference's row-major runs of k / block_size blocks.  MXFP4: `scales` = Some(E8M0 bytes) for the
    /// split form of quant_mxfp4::dequant_mxfp4, None for inline 17-byte blocks.  NVFP4: `global_scale`.
    pub fn upload(&self, q: QuantType, n: usize, k: usize, blocks: &[u8], scales: Option<&[u8]>, global_scale: f32) -> GpuWeight {
        let (id, mx) = quant_type_id(q);
        let mut h = std::ptr::null_mut();
        let rc = unsafe {
            gllmk_weight_upload(self.ctx, id, n as i64, k as i64, mx, blocks.as_ptr() as *const c_void,
                                scales.map_or(std::ptr::null(), |s| s.as_ptr() as *const c_void), global_scale, 0, &mut h)
        };
        self.check(rc, "gllmk_weight_upload");
        GpuWeight { h, n, k }
    }

    /// Host activations / outputs against a resident weight.  `ref_layout`: kquant_matmul's input [k, m] / output
    /// [n, m]; otherwise gemm_q4's [m, k] / [m, n].
    pub fn matmul(&self, w: &GpuWeight, x: &[f32], m: usize, y: &mut [f32], ref_layout: bool) {
        assert!(x.len() >= m * w.k && y.len() >= m * w.n);
        let rc = unsafe { gllmk_matmul_host(self.ctx, w.h, x.as_ptr(), m as i32, y.as_mut_ptr(), ref_layout as i32) };
        self.check(rc, "gllmk_matmul_host");
    }

    /// The products of one decode step in one call (enqueued back to back, one wait): `jobs[i] = (weight, x [m, k], m, y [m, n])`.
    pub fn matmul_batch(&self, jobs: &mut [(&GpuWeight, &[f32], usize, &mut [f32])]) {
        let ws: Vec<*mut c_void> = jobs.iter().map(|j| j.0.h).collect();
        let xs: Vec<*const f32> = jobs.iter().map(|j| j.1.as_ptr()).collect();
        let ms: Vec<i32> = jobs.iter().map(|j| j.2 as i32).collect();
        let ys: Vec<*mut f32> = jobs.iter_mut().map(|j| j.3.as_mut_ptr()).collect();
        let rc = unsafe { gllmk_matmul_host_batch(self.ctx, jobs.len() as i32, ws.as_ptr(), xs.as_ptr(), ms.as_ptr(), ys.as_ptr(), 0) };
        self.check(rc, "gllmk_matmul_host_batch");
    }

    /// Decode product on device memory (m <= 16): x [m, k] and y [m, n] row-major device pointers.
    ///
    /// # Safety
    /// `x_dev` / `y_dev` must be device pointers of at least m*k / m*n floats on this context's device.
    pub unsafe fn gemv_dev(&self, w: &GpuWeight, x_dev: *const f32, m: usize, y_dev: *mut f32, stream: *mut c_void) {
        let rc = gllmk_gemv(self.ctx, w.h, x_dev, w.k as i64, 1, m as i32, y_dev, w.n as i64, 1, std::ptr::null(), 0, stream);
        self.check(rc, "gllmk_gemv");
    }

    /// Prefill product on device memory (any m); dtype 0 = f32, 1 = bf16.
    ///
    /// # Safety
    /// Device pointers of m*lda / m*ldy elements of the stated types.
    pub unsafe fn gemm_dev(&self, w: &GpuWeight, a_dev: *const c_void, a_dtype: i32, lda: usize, m: usize, y_dev: *mut c_void, y_dtype: i32,
                           ldy: usize, stream: *mut c_void) {
        let rc = gllmk_gemm(self.ctx, w.h, a_dev, a_dtype, lda as i64, m as i32, y_dev, y_dtype, ldy as i64, stream);
        self.check(rc, "gllmk_gemm");
    }

    // ---- Kernels<f32>: dequantization (src/traits.rs:476-490) ------------------------------------------------
    pub fn dequant_q4_k(&self, block: &[u8], out: &mut [f32]) {
        let nb = block.len() / 144;
        assert!(out.len() >= nb * 256);
        self.check(unsafe { gllmk_dequant_q4_k(self.ctx, block.as_ptr(), out.as_mut_ptr(), nb) }, "dequant_q4_k");
    }
    pub fn dequant_q8_0(&self, block: &[u8], out: &mut [f32]) {
        let nb = block.len() / 34;
        assert!(out.len() >= nb * 32);
        self.check(unsafe { gllmk_dequant_q8_0(self.ctx, block.as_ptr(), out.as_mut_ptr(), nb) }, "dequant_q8_0");
    }
    fn dequant_gguf(&self, id: i32, bytes: usize, elems: usize, block: &[u8], out: &mut [f32], what: &str) {
        let nb = block.len() / bytes;
        assert!(out.len() >= nb * elems);
        self.check(unsafe { gllmk_dequant_gguf(self.ctx, id, block.as_ptr(), out.as_mut_ptr(), nb) }, what);
    }
    pub fn dequant_q6_k(&self, block: &[u8], out: &mut [f32]) {
        self.dequant_gguf(6, 210, 256, block, out, "dequant_q6_k")
    }
    pub fn dequant_q5_k(&self, block: &[u8], out: &mut [f32]) {
        self.dequant_gguf(7, 176, 256, block, out, "dequant_q5_k")
    }
    pub fn dequant_q8_k(&self, block: &[u8], out: &mut [f32]) {
        self.dequant_gguf(10, 292, 256, block, out, "dequant_q8_k")
    }
    pub fn dequant_q4_0(&self, block: &[u8], out: &mut [f32]) {
        self.dequant_gguf(8, 18, 32, block, out, "dequant_q4_0")
    }
    pub fn dequant_q5_0(&self, block: &[u8], out: &mut [f32]) {
        self.dequant_gguf(9, 22, 32, block, out, "dequant_q5_0")
    }
    /// quant_mxfp4::dequant_mxfp4 (src/quant_mxfp4.rs:267-292): Err on the length mismatches the reference rejects.
    pub fn dequant_mxfp4(&self, blocks: &[u8], scales: &[u8], output: &mut [f32], block_size: usize) -> Result<(), String> {
        if block_size == 0 || block_size % 2 != 0 || blocks.len() != scales.len() * block_size / 2 || output.len() != scales.len() * block_size {
            return Err("dequant_mxfp4: length mismatch".into());
        }
        match unsafe { gllmk_dequant_mxfp4(self.ctx, blocks.as_ptr(), scales.as_ptr(), output.as_mut_ptr(), scales.len(), block_size) } {
            OK => Ok(()),
            rc => Err(format!("dequant_mxfp4: status {rc}: {}", self.last_error())),
        }
    }
    /// NVFP4 decode: value = global * ue4m3(d[e / 16]) * E2M1[nibble] (src/quant.rs:77-86).
    pub fn dequant_nvfp4(&self, blocks: &[u8], global_scale: f32, out: &mut [f32]) {
        let nb = blocks.len() / 36;
        assert!(out.len() >= nb * 64);
        self.check(unsafe { gllmk_dequant_nvfp4(self.ctx, blocks.as_ptr(), global_scale, out.as_mut_ptr(), nb) }, "dequant_nvfp4");
    }

    // ---- Kernels<f32>: quantized GEMV / GEMM (src/traits.rs:500-523) --------------------------------------------
    pub fn gemv_q8(&self, weight: &[i8], input: &[f32], scale: f32, n: usize) -> f32 {
        assert!(n % 256 == 0);
        let mut out = 0f32;
        self.check(unsafe { gllmk_gemv_q8_f32(self.ctx, weight.as_ptr(), input.as_ptr(), scale, n, &mut out) }, "gemv_q8");
        out
    }
    pub fn gemv_q4(&self, weight: &[u8], input: &[f32], scale: f32, n: usize) -> f32 {
        assert!(n % 256 == 0);
        let mut out = 0f32;
        self.check(unsafe { gllmk_gemv_q4_f32(self.ctx, weight.as_ptr(), input.as_ptr(), scale, n, &mut out) }, "gemv_q4");
        out
    }
    pub fn gemm_q8(&self, weight: &[i8], input: &[f32], output: &mut [f32], scales: &[f32], m: usize, n: usize, k: usize) {
        assert!(k % 256 == 0);
        let rc = unsafe {
            gllmk_gemm_q8_f32(self.ctx, weight.as_ptr(), input.as_ptr(), output.as_mut_ptr(), scales.as_ptr(), scales.len(), m, n, k)
        };
        self.check(rc, "gemm_q8");
    }
    pub fn gemm_q4(&self, weight: &[u8], input: &[f32], output: &mut [f32], scales: &[f32], m: usize, n: usize, k: usize) {
        assert!(k % 256 == 0);
        let rc = unsafe {
            gllmk_gemm_q4_f32(self.ctx, weight.as_ptr(), input.as_ptr(), output.as_mut_ptr(), scales.as_ptr(), scales.len(), m, n, k)
        };
        self.check(rc, "gemm_q4");
    }

    // ---- Kernels<f32>: format-specific matmul (src/traits.rs:543-563) ---------------------------------------------
    /// m weight rows, n batch columns, input [k, n], output [m, n]; Q4K / Q5K / Q6K / Q8K.
    pub fn kquant_matmul(&self, weight_blocks: &[u8], input: &[f32], output: &mut [f32], quant_type: QuantType, m: usize, n: usize, k: usize) {
        let rc = unsafe {
            gllmk_kquant_matmul_f32(self.ctx, weight_blocks.as_ptr(), input.as_ptr(), output.as_mut_ptr(), quant_type_id(quant_type).0, m, n, k)
        };
        self.check(rc, "kquant_matmul");
    }
    /// Q8_0 / Q4_0 / Q5_0.
    pub fn classic_matmul(&self, weight_blocks: &[u8], input: &[f32], output: &mut [f32], quant_type: QuantType, m: usize, n: usize, k: usize) {
        let rc = unsafe {
            gllmk_classic_matmul_f32(self.ctx, weight_blocks.as_ptr(), input.as_ptr(), output.as_mut_ptr(), quant_type_id(quant_type).0, m, n, k)
        };
        self.check(rc, "classic_matmul");
    }

    // ---- avx512_int8::gemm_int8 (src/macros/matmul_x86_int8.rs:307): C (s32) = A (u8) x B (s8), host slices ---------
    pub fn gemm_int8(&self, a: &[u8], b_kn: &[i8], c: &mut [i32], m: usize, n: usize, k: usize) {
        assert!(a.len() >= m * k && b_kn.len() >= k * n && c.len() >= m * n);
        self.check(unsafe { gllmk_gemm_int8_host(self.ctx, a.as_ptr(), b_kn.as_ptr(), c.as_mut_ptr(), m, n, k) }, "gemm_int8");
    }
}

// The device-pointer entry points not wrapped above (gllmk_gemv_static, gllmk_ffn_decode, gllmk_gemm_grouped,
// gllmk_gemm_fp4, gllmk_quantize, gllmk_moe_*, gllmk_int8_weight_upload / gllmk_gemm_int8 / gllmk_dequantize_i32_f32 /
// gllmk_quantize_act_int8 / gllmk_w8a8_linear_f32, gllmk_embedding_gather, gllmk_dequant, gllmk_weight_unpack, the
// gllmk_shared_* / gllmk_gemv_allgather / gllmk_peer_barrier / gllmk_gemv_exchange / gllmk_exchange_wait group and
// gllmk_ctx_set) are declared in the extern block for callers that own device buffers and streams; they take raw
// device pointers, so gllm wraps them where it owns the corresponding tensors.
#[allow(dead_code)]
fn _declared_but_unwrapped() {
    let _ = (
        gllmk_quant_block_size as usize, gllmk_quant_block_bytes as usize, gllmk_ctx_set as usize, gllmk_weight_unpack as usize,
        gllmk_dequant as usize, gllmk_embedding_gather as usize, gllmk_gemv_static as usize, gllmk_ffn_decode as usize, gllmk_ffn_prefill as usize,
        gllmk_gemm_grouped as usize, gllmk_gemm_fp4 as usize, gllmk_probe_fp4_mma as usize, gllmk_quantize as usize, gllmk_moe_topk as usize, gllmk_moe_route as usize,
        gllmk_moe_gather as usize, gllmk_moe_weighted_sum as usize, gllmk_int8_weight_upload as usize, gllmk_gemm_int8 as usize,
        gllmk_dequantize_i32_f32 as usize, gllmk_quantize_act_int8 as usize, gllmk_w8a8_linear_f32 as usize, gllmk_shared_alloc as usize,
        gllmk_shared_open as usize, gllmk_shared_close as usize, gllmk_shared_free as usize, gllmk_gemv_allgather as usize,
        gllmk_peer_barrier as usize, gllmk_gemv_exchange as usize, gllmk_exchange_wait as usize,
    );
}
