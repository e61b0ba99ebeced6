//! CUDA (B200, sm_100a) backend glue for Tachyon's Granite mixture-of-experts
//! block: the `extern "C"` block over `libtachyon_cuda.so`
//! (`include/tachyon_cuda.h`), safe owners for its handles, and `CudaMoe`, which
//! runs `x += moe(rmsnorm(x))` of one layer on the device.
//!
//! It mirrors how `src/gpu/mod.rs` binds the Metal shim (`tm_*`): opaque
//! pointers, a context that is `Send` but not `Sync`, buffers dropped before
//! the context, construction errors as `Err`, a failed step as a panic.
//!
//! Where it plugs in (three small edits to Tachyon, none to `engine.rs`,
//! `scheduler.rs` or the server):
//!   * `src/lib.rs`: `#[cfg(feature = "cuda")] pub mod gpu_cuda;` with
//!     `#[path = "gpu/cuda/mod.rs"]` (the existing `gpu` module is macOS-only);
//!   * `src/model.rs`: `CpuBackend` gets `pub moe_on_device: Option<CudaMoe>`;
//!     in `forward`, where the MLP block starts, a layer with a router calls
//!     `gpu.block(l, &mut s.x[..t * dim], t)` and `continue`s instead of
//!     norm -> `moe()` -> residual add;
//!   * `src/main.rs`: the non-macOS `gpu_backend()` builds a `CpuBackend`,
//!     then `CudaMoe::new(&cfg, &weights, max_batch)?`, and sets the field.
//! Until attention, embeddings and the output head also run on the device, the
//! residual stream crosses PCIe around every block (`CudaMoe::block`); the
//! device-resident entry point is `tc_moe_block` itself.
//!
//! This file has not been compiled: the image this backend was built in has no
//! Rust toolchain. The C side it binds is exercised through the same entry
//! points from Python (`tachyon_b200/cuda.py`).

use std::ffi::{c_char, c_int, c_void, CStr};
use std::ptr;

use crate::config::Config;
use crate::model::{LayerWeights, Weights};
use crate::weights::Matrix;
use crate::{bail, Result};

#[repr(C)]
pub struct TcCtx {
    _private: [u8; 0],
}
#[repr(C)]
pub struct TcMatrix {
    _private: [u8; 0],
}
#[repr(C)]
pub struct TcMoeLayer {
    _private: [u8; 0],
}
#[repr(C)]
pub struct TcGraph {
    _private: [u8; 0],
}

pub const TC_BF16: c_int = 0;
pub const TC_Q8: c_int = 1;
pub const TC_Q4: c_int = 2;
pub const TC_ARITH_FAST: c_int = 0;
pub const TC_ARITH_CPU_LANES: c_int = 1;

#[link(name = "tachyon_cuda")]
extern "C" {
    fn tc_create(device: c_int, err: *mut c_char, errlen: usize) -> *mut TcCtx;
    fn tc_destroy(ctx: *mut TcCtx);
    fn tc_device_name(ctx: *mut TcCtx, out: *mut c_char, len: usize);
    fn tc_last_error(ctx: *mut TcCtx, out: *mut c_char, len: usize) -> usize;
    fn tc_sync(ctx: *mut TcCtx) -> c_int;
    fn tc_set_arithmetic(ctx: *mut TcCtx, mode: c_int) -> c_int;
    fn tc_set_prefill_threshold(ctx: *mut TcCtx, avg_tokens_per_expert: c_int) -> c_int;
    fn tc_set_decode_block(ctx: *mut TcCtx, on: c_int) -> c_int;
    fn tc_malloc(ctx: *mut TcCtx, bytes: usize) -> *mut c_void;
    fn tc_free(ctx: *mut TcCtx, dev: *mut c_void);
    fn tc_upload(ctx: *mut TcCtx, dst: *mut c_void, src: *const c_void, bytes: usize) -> c_int;
    fn tc_download(ctx: *mut TcCtx, dst: *mut c_void, src: *const c_void, bytes: usize) -> c_int;
    fn tc_matrix_upload(
        ctx: *mut TcCtx,
        kind: c_int,
        rows: usize,
        cols: usize,
        scales: *const c_void,
        scales_bytes: usize,
        data: *const c_void,
        data_bytes: usize,
    ) -> *mut TcMatrix;
    /// `Matrix::from_f32` on the device: same bytes as the host quantizers.
    fn tc_matrix_quantize(
        ctx: *mut TcCtx,
        kind: c_int,
        rows: usize,
        cols: usize,
        data: *const f32,
    ) -> *mut TcMatrix;
    fn tc_matrix_free(m: *mut TcMatrix);
    #[allow(clippy::too_many_arguments)]
    fn tc_moe_layer_create(
        ctx: *mut TcCtx,
        hidden: c_int,
        experts: c_int,
        experts_per_token: c_int,
        inter: c_int,
        router: *const TcMatrix,
        gate_up: *const TcMatrix,
        down: *const TcMatrix,
        max_tokens: c_int,
    ) -> *mut TcMoeLayer;
    fn tc_moe_layer_free(layer: *mut TcMoeLayer);
    fn tc_moe_layer_detach_experts(layer: *mut TcMoeLayer) -> c_int;
    fn tc_moe_forward(layer: *mut TcMoeLayer, x: *const f32, t: c_int, y: *mut f32) -> c_int;
    fn tc_moe_block(
        layer: *mut TcMoeLayer,
        norm_weight: *const f32,
        eps: f32,
        t: c_int,
        y: *mut f32,
    ) -> c_int;
    fn tc_capture_begin(ctx: *mut TcCtx) -> c_int;
    fn tc_capture_end(ctx: *mut TcCtx) -> *mut TcGraph;
    fn tc_graph_launch(g: *mut TcGraph) -> c_int;
    fn tc_graph_free(g: *mut TcGraph);
}

/// One device and one stream. Driven by one thread at a time, like the Metal
/// context (`src/gpu/mod.rs:440-442`).
struct Context(*mut TcCtx);

// SAFETY: the library keeps no thread-local state; a context may move between
// threads as long as one thread uses it at a time (`Backend: Send`).
unsafe impl Send for Context {}

impl Context {
    fn new(device: usize) -> Result<Context> {
        let mut err = [0 as c_char; 512];
        // SAFETY: `err` outlives the call and its length is passed.
        let p = unsafe { tc_create(device as c_int, err.as_mut_ptr(), err.len()) };
        if p.is_null() {
            // SAFETY: the library NUL-terminates what it writes.
            let why = unsafe { CStr::from_ptr(err.as_ptr()) }.to_string_lossy();
            bail!("CUDA backend: {why}");
        }
        Ok(Context(p))
    }

    fn last_error(&self) -> String {
        let mut buf = [0 as c_char; 512];
        // SAFETY: as above.
        unsafe { tc_last_error(self.0, buf.as_mut_ptr(), buf.len()) };
        unsafe { CStr::from_ptr(buf.as_ptr()) }
            .to_string_lossy()
            .into_owned()
    }

    fn name(&self) -> String {
        let mut buf = [0 as c_char; 256];
        // SAFETY: as above.
        unsafe { tc_device_name(self.0, buf.as_mut_ptr(), buf.len()) };
        unsafe { CStr::from_ptr(buf.as_ptr()) }
            .to_string_lossy()
            .into_owned()
    }
}

impl Drop for Context {
    fn drop(&mut self) {
        // SAFETY: created by tc_create, destroyed once.
        unsafe { tc_destroy(self.0) }
    }
}

/// A `Matrix` on the device, byte for byte (`GpuMatrix::upload`,
/// `src/gpu/mod.rs:222-251`).
struct DeviceMatrix(*mut TcMatrix);

impl DeviceMatrix {
    fn upload(ctx: &Context, m: &Matrix) -> Result<DeviceMatrix> {
        // SAFETY: every pointer/length pair describes a live Vec of `m`.
        let p = unsafe {
            match m {
                Matrix::Bf16 { rows, cols, data } => tc_matrix_upload(
                    ctx.0,
                    TC_BF16,
                    *rows,
                    *cols,
                    ptr::null(),
                    0,
                    data.as_ptr().cast(),
                    data.len() * 2,
                ),
                Matrix::Q8 {
                    rows,
                    cols,
                    scales,
                    qs,
                } => tc_matrix_upload(
                    ctx.0,
                    TC_Q8,
                    *rows,
                    *cols,
                    scales.as_ptr().cast(),
                    scales.len() * 2,
                    qs.as_ptr().cast(),
                    qs.len(),
                ),
                Matrix::Q4 {
                    rows,
                    cols,
                    scales,
                    qs,
                } => tc_matrix_upload(
                    ctx.0,
                    TC_Q4,
                    *rows,
                    *cols,
                    scales.as_ptr().cast(),
                    scales.len() * 4,
                    qs.as_ptr().cast(),
                    qs.len(),
                ),
            }
        };
        if p.is_null() {
            bail!("CUDA backend: {}", ctx.last_error());
        }
        Ok(DeviceMatrix(p))
    }
}

impl Drop for DeviceMatrix {
    fn drop(&mut self) {
        // SAFETY: created by tc_matrix_upload, freed once, before the context.
        unsafe { tc_matrix_free(self.0) }
    }
}

/// A plain device buffer of f32.
struct DeviceBuf {
    ctx: *mut TcCtx,
    ptr: *mut f32,
    len: usize,
}

impl DeviceBuf {
    fn new(ctx: &Context, len: usize) -> Result<DeviceBuf> {
        // SAFETY: the context is live.
        let p = unsafe { tc_malloc(ctx.0, len * 4) };
        if p.is_null() {
            bail!("CUDA backend: {}", ctx.last_error());
        }
        Ok(DeviceBuf {
            ctx: ctx.0,
            ptr: p.cast(),
            len,
        })
    }

    fn from_slice(ctx: &Context, data: &[f32]) -> Result<DeviceBuf> {
        let b = DeviceBuf::new(ctx, data.len())?;
        // SAFETY: both sides hold `data.len()` floats.
        if unsafe { tc_upload(ctx.0, b.ptr.cast(), data.as_ptr().cast(), data.len() * 4) } != 0 {
            bail!("CUDA backend: {}", ctx.last_error());
        }
        Ok(b)
    }
}

impl Drop for DeviceBuf {
    fn drop(&mut self) {
        // SAFETY: allocated by tc_malloc on this context, freed once.
        unsafe { tc_free(self.ctx, self.ptr.cast()) }
    }
}

/// One layer's MoE block on the device. Field order is drop order: the layer
/// handle goes before the matrices it refers to.
struct MoeLayer {
    handle: *mut TcMoeLayer,
    mlp_norm: DeviceBuf,
    _router: DeviceMatrix,
    gate_up: Option<DeviceMatrix>,
    down: Option<DeviceMatrix>,
}

impl Drop for MoeLayer {
    fn drop(&mut self) {
        // SAFETY: created by tc_moe_layer_create, freed once.
        unsafe { tc_moe_layer_free(self.handle) }
    }
}

/// The MoE blocks of a Granite-MoE model on one B200. Field order is drop
/// order: layers and buffers before the context (`src/gpu/mod.rs:427`).
pub struct CudaMoe {
    layers: Vec<Option<MoeLayer>>,
    x: DeviceBuf,
    eps: f32,
    hidden: usize,
    max_tokens: usize,
    ctx: Context,
}

// SAFETY: raw handles are only used through `&mut self`.
unsafe impl Send for CudaMoe {}

impl CudaMoe {
    /// Uploads every MoE layer's router and expert matrices (dense layers are
    /// left to the host). `max_tokens` bounds `t` of later blocks: all device
    /// scratch is allocated here, none during a forward pass.
    pub fn new(cfg: &Config, weights: &Weights, max_tokens: usize) -> Result<CudaMoe> {
        let ctx = Context::new(0)?;
        let mut layers = Vec::with_capacity(weights.layers.len());
        for layer in &weights.layers {
            layers.push(match &layer.router {
                Some(router) => Some(CudaMoe::layer(&ctx, cfg, layer, router, max_tokens)?),
                None => None,
            });
        }
        let x = DeviceBuf::new(&ctx, max_tokens * cfg.hidden)?;
        Ok(CudaMoe {
            layers,
            x,
            eps: cfg.norm_eps,
            hidden: cfg.hidden,
            max_tokens,
            ctx,
        })
    }

    fn layer(
        ctx: &Context,
        cfg: &Config,
        layer: &LayerWeights,
        router: &Matrix,
        max_tokens: usize,
    ) -> Result<MoeLayer> {
        let router = DeviceMatrix::upload(ctx, router)?;
        let gate_up = DeviceMatrix::upload(ctx, &layer.w_gate_up)?;
        let down = DeviceMatrix::upload(ctx, &layer.w_down)?;
        // SAFETY: the three matrices outlive the layer (see MoeLayer's field order).
        let handle = unsafe {
            tc_moe_layer_create(
                ctx.0,
                cfg.hidden as c_int,
                cfg.experts as c_int,
                cfg.experts_per_token as c_int,
                cfg.intermediate as c_int,
                router.0,
                gate_up.0,
                down.0,
                max_tokens as c_int,
            )
        };
        if handle.is_null() {
            bail!("CUDA backend: {}", ctx.last_error());
        }
        Ok(MoeLayer {
            handle,
            mlp_norm: DeviceBuf::from_slice(ctx, &layer.mlp_norm)?,
            _router: router,
            gate_up: Some(gate_up),
            down: Some(down),
        })
    }

    /// e.g. "cuda moe (NVIDIA B200)", for `Backend::name`.
    pub fn name(&self) -> String {
        format!("cuda moe ({})", self.ctx.name())
    }

    /// Whether layer `l` runs here (it has a router).
    pub fn has(&self, l: usize) -> bool {
        self.layers.get(l).is_some_and(|x| x.is_some())
    }

    /// `x[t, hidden] += moe(rmsnorm(x, mlp_norm, eps))` for layer `l`: what
    /// `src/model.rs:662-681` does on the host. `x` is the host residual stream
    /// (`s.x`); it crosses to the device and back.
    pub fn block(&mut self, l: usize, x: &mut [f32], t: usize) {
        assert!(t > 0 && t <= self.max_tokens, "batch of {t} tokens");
        assert_eq!(x.len(), t * self.hidden);
        let layer = self.layers[l].as_ref().expect("not a MoE layer");
        let bytes = x.len() * 4;
        // SAFETY: the device buffer holds max_tokens * hidden floats; `x` holds t * hidden.
        let ok = unsafe {
            tc_upload(self.ctx.0, self.x.ptr.cast(), x.as_ptr().cast(), bytes) == 0
                && tc_moe_block(
                    layer.handle,
                    layer.mlp_norm.ptr,
                    self.eps,
                    t as c_int,
                    self.x.ptr,
                ) == 0
                && tc_download(self.ctx.0, x.as_mut_ptr().cast(), self.x.ptr.cast(), bytes) == 0
                && tc_sync(self.ctx.0) == 0
        };
        if !ok {
            // As the Metal backend does for a failed command buffer (src/gpu/mod.rs:1049-1053).
            panic!("CUDA MoE block failed: {}", self.ctx.last_error());
        }
    }

    /// Frees the expert matrices as uploaded (a third of the experts' device
    /// memory): the layers compute from their own re-tiled copies. Afterwards
    /// `exact_cpu_order(true)` blocks are refused by the library.
    pub fn release_uploaded_experts(&mut self) -> Result<()> {
        for layer in self.layers.iter_mut().flatten() {
            // SAFETY: the layer is live; the matrices are dropped only after it lets go of them.
            if unsafe { tc_moe_layer_detach_experts(layer.handle) } != 0 {
                bail!("CUDA backend: {}", self.ctx.last_error());
            }
            layer.gate_up = None;
            layer.down = None;
        }
        Ok(())
    }

    /// Switches the expert products to the CPU path's own eight-lane order
    /// (bit-identical to `CpuBackend`), for validation runs.
    pub fn exact_cpu_order(&mut self, on: bool) {
        let mode = if on { TC_ARITH_CPU_LANES } else { TC_ARITH_FAST };
        // SAFETY: the context is live.
        unsafe { tc_set_arithmetic(self.ctx.0, mode) };
    }
}

#[allow(dead_code)]
fn _unused_entry_points() {
    // Bound for completeness; used by a backend that keeps the residual stream on the device.
    let _ = (
        tc_moe_forward as usize,
        tc_set_prefill_threshold as usize,
        tc_set_decode_block as usize,
        tc_capture_begin as usize,
        tc_capture_end as usize,
        tc_graph_launch as usize,
        tc_graph_free as usize,
        tc_matrix_quantize as usize,
    );
    let _ = DeviceBuf::len;
}

impl DeviceBuf {
    fn len(&self) -> usize {
        self.len
    }
}
