//! katsu-cuda: safe Rust over the C ABI of libkatsu_cuda.so (include/katsu_cuda.h), the sm_100a
//! replacement for katsu-core's dense loops (Conv2D forward / backward_buffers, matmul and its
//! VJP, the streaming ops that keep the autograd graph on the device).
//!
//! This is the only crate of the workspace that contains `unsafe`; katsu-core keeps
//! `#![forbid(unsafe_code)]` (crates/katsu-core/src/lib.rs:2) and calls the functions below.
//!
//! NOT COMPILED in the repository that carries the kernels (no Rust toolchain in its build image).
//! The same boundary is exercised there by the C++ mirror of katsu-core (katsu_b200/csrc/host) and
//! by ctypes tests; `ffi.rs` is generated from the header and checked against it by a test.
//!
//! Threading: `Context` is `!Send + !Sync` (it holds a raw pointer), matching katsu-core's
//! `Rc`-based, single-threaded `Tensor` (crates/katsu-core/src/tensor.rs:95-99).  One context is
//! one device and one stream; calls are asynchronous and ordered on it; `sync`, `DeviceBuf::to_host`
//! and `Event::elapsed_ms` wait.

pub mod ffi;

use std::ffi::CStr;
use std::fmt;
use std::marker::PhantomData;
use std::ptr;
use std::rc::Rc;

/// A failed call: the status code of include/katsu_cuda.h and the library's message.
#[derive(Debug, Clone, PartialEq, Eq)]
pub struct CudaError {
    pub code: i32,
    pub message: String,
}

impl CudaError {
    /// katsu-core maps this to `TensorError::Allocation`, everything else to `TensorError::Device`.
    pub fn is_allocation(&self) -> bool {
        self.code == ffi::KATSU_ERR_ALLOC
    }
    /// A bounded device-side wait gave up; results queued since the last check are undefined.
    pub fn is_timeout(&self) -> bool {
        self.code == ffi::KATSU_ERR_TIMEOUT
    }
}

impl fmt::Display for CudaError {
    fn fmt(&self, f: &mut fmt::Formatter<'_>) -> fmt::Result {
        write!(f, "katsu_cuda error {}: {}", self.code, self.message)
    }
}

impl std::error::Error for CudaError {}

fn check(code: i32) -> Result<(), CudaError> {
    if code == ffi::KATSU_OK {
        return Ok(());
    }
    // SAFETY: the library returns a pointer to a NUL-terminated thread-local buffer.
    let message = unsafe { CStr::from_ptr(ffi::katsu_cuda_last_error_string()) }.to_string_lossy().into_owned();
    Err(CudaError { code, message })
}

/// Arithmetic mode of the contraction kernels.
#[derive(Debug, Clone, Copy, PartialEq, Eq)]
pub enum Precision {
    /// Tensor cores, split precision (hi*hi + lo*hi + hi*lo): FP32-grade accuracy.  Default.
    ThreeXTf32,
    /// Tensor cores, one TF32 pass (relative error about 1e-3).
    Tf32,
    /// CUDA cores only.
    Fp32,
}

struct RawContext(*mut ffi::Ctx);

impl Drop for RawContext {
    fn drop(&mut self) {
        // SAFETY: created by katsu_cuda_init, dropped once (Rc), no buffer outlives it (they hold an Rc).
        unsafe { ffi::katsu_cuda_shutdown(self.0) };
    }
}

/// One device, one stream.  Cheap to clone (reference counted); buffers keep their context alive.
#[derive(Clone)]
pub struct Context {
    raw: Rc<RawContext>,
}

impl Context {
    pub fn device_count() -> Result<usize, CudaError> {
        let mut n = 0i32;
        check(unsafe { ffi::katsu_cuda_device_count(&mut n) })?;
        Ok(n.max(0) as usize)
    }

    pub fn new(device: usize) -> Result<Self, CudaError> {
        let mut raw = ptr::null_mut();
        check(unsafe { ffi::katsu_cuda_init(device as i32, &mut raw) })?;
        Ok(Self { raw: Rc::new(RawContext(raw)) })
    }

    fn ptr(&self) -> *mut ffi::Ctx {
        self.raw.0
    }

    pub fn set_precision(&self, mode: Precision) -> Result<(), CudaError> {
        let raw = match mode {
            Precision::ThreeXTf32 => ffi::KATSU_MODE_3XTF32,
            Precision::Tf32 => ffi::KATSU_MODE_TF32,
            Precision::Fp32 => ffi::KATSU_MODE_FP32,
        };
        check(unsafe { ffi::katsu_cuda_set_precision(self.ptr(), raw) })
    }

    /// Waits for everything queued; `Err(timeout)` once if a device-side wait gave up since the last check.
    pub fn sync(&self) -> Result<(), CudaError> {
        check(unsafe { ffi::katsu_cuda_sync(self.ptr()) })
    }

    pub fn launch_count(&self) -> Result<u64, CudaError> {
        let mut n = 0u64;
        check(unsafe { ffi::katsu_cuda_launch_count(self.ptr(), &mut n) })?;
        Ok(n)
    }
}

/// Owned device buffer of f32: the device variant of `TensorNode.data`
/// (crates/katsu-core/src/tensor.rs:101-107).  Freed (stream-ordered) on drop.
pub struct DeviceBuf {
    ctx: Context,
    ptr: *mut f32,
    len: usize,
    _not_send: PhantomData<*mut f32>,
}

impl DeviceBuf {
    /// Zero-filled, like `zeros_buffer` (tensor.rs:120-125).
    pub fn zeros(ctx: &Context, len: usize) -> Result<Self, CudaError> {
        let mut ptr = ptr::null_mut();
        check(unsafe { ffi::katsu_cuda_alloc(ctx.ptr(), len, &mut ptr) })?;
        Ok(Self { ctx: ctx.clone(), ptr, len, _not_send: PhantomData })
    }

    pub fn from_host(ctx: &Context, data: &[f32]) -> Result<Self, CudaError> {
        let buf = Self::zeros(ctx, data.len())?;
        check(unsafe { ffi::katsu_cuda_h2d(ctx.ptr(), buf.ptr, data.as_ptr(), data.len()) })?;
        ctx.sync()?; // `data` is pageable and may be dropped by the caller right away
        Ok(buf)
    }

    /// Synchronous copy back: what `Tensor::data()` / `Tensor::grad()` fill their host mirror with.
    pub fn to_host(&self) -> Result<Vec<f32>, CudaError> {
        let mut out = vec![0.0f32; self.len];
        check(unsafe { ffi::katsu_cuda_d2h(self.ctx.ptr(), out.as_mut_ptr(), self.ptr, self.len) })?;
        Ok(out)
    }

    pub fn len(&self) -> usize {
        self.len
    }
    pub fn is_empty(&self) -> bool {
        self.len == 0
    }
    pub fn as_ptr(&self) -> *const f32 {
        self.ptr
    }
    pub fn as_mut_ptr(&mut self) -> *mut f32 {
        self.ptr
    }
    pub fn context(&self) -> &Context {
        &self.ctx
    }
}

impl Drop for DeviceBuf {
    fn drop(&mut self) {
        // SAFETY: allocated by katsu_cuda_alloc on this context; freeing is ordered behind queued work.
        unsafe { ffi::katsu_cuda_free(self.ctx.ptr(), self.ptr) };
    }
}

fn opt_mut(buf: Option<&mut DeviceBuf>) -> *mut f32 {
    buf.map_or(ptr::null_mut(), |b| b.ptr)
}

fn opt_const(buf: Option<&DeviceBuf>) -> *const f32 {
    buf.map_or(ptr::null(), |b| b.ptr as *const f32)
}

/// Output of `Geometry::new` (crates/katsu-core/src/conv2d.rs:183-224); katsu-core validates, this
/// crate only carries the numbers across.
#[derive(Debug, Clone, Copy)]
pub struct ConvGeometry {
    pub batch: usize,
    pub cin: usize,
    pub h: usize,
    pub w: usize,
    pub cout: usize,
    pub kh: usize,
    pub kw: usize,
    pub oh: usize,
    pub ow: usize,
    pub stride: usize,
    pub padding: usize,
}

impl ConvGeometry {
    fn x_len(&self) -> usize {
        self.batch * self.cin * self.h * self.w
    }
    fn w_len(&self) -> usize {
        self.cout * self.cin * self.kh * self.kw
    }
    fn y_len(&self) -> usize {
        self.batch * self.cout * self.oh * self.ow
    }
}

fn length(what: &str, buf: &DeviceBuf, expected: usize) -> Result<(), CudaError> {
    if buf.len == expected {
        Ok(())
    } else {
        Err(CudaError { code: ffi::KATSU_ERR_INVALID_ARG, message: format!("{what}: expected {expected} elements, got {}", buf.len) })
    }
}

/// The visit closure of `Conv2D::forward` (conv2d.rs:95-103, 232-262); y is overwritten.
/// `bias` / `relu` are additions that ride in the kernel's epilogue.
pub fn conv2d_forward(ctx: &Context, x: &DeviceBuf, w: &DeviceBuf, bias: Option<&DeviceBuf>, relu: bool, y: &mut DeviceBuf,
                      g: &ConvGeometry) -> Result<(), CudaError> {
    length("x", x, g.x_len())?;
    length("w", w, g.w_len())?;
    length("y", y, g.y_len())?;
    if let Some(b) = bias {
        length("bias", b, g.cout)?;
    }
    check(unsafe {
        ffi::katsu_cuda_conv2d_fwd_bias_relu(ctx.ptr(), x.ptr, w.ptr, opt_const(bias), y.ptr, g.batch, g.cin, g.h, g.w, g.cout,
                                             g.kh, g.kw, g.stride, g.padding, relu as i32)
    })
}

/// Size in floats of the channels-innermost copy of x that this geometry's kernels read in the context's
/// current precision mode; 0 when they read x directly.
pub fn conv2d_staged_len(ctx: &Context, g: &ConvGeometry) -> Result<usize, CudaError> {
    let mut floats: usize = 0;
    check(unsafe {
        ffi::katsu_cuda_conv2d_staged_floats(ctx.ptr(), g.batch, g.cin, g.h, g.w, g.cout, g.kh, g.kw, g.stride, g.padding,
                                             &mut floats)
    })?;
    Ok(floats)
}

/// Writes that copy.  `Conv2D` holds its input from forward to backward (conv2d.rs:104-107, 130-136); holding
/// this copy beside it lets both calls skip their own staging pass.
pub fn conv2d_stage(ctx: &Context, x: &DeviceBuf, staged: &mut DeviceBuf, g: &ConvGeometry) -> Result<(), CudaError> {
    length("x", x, g.x_len())?;
    length("staged", staged, conv2d_staged_len(ctx, g)?)?;
    check(unsafe { ffi::katsu_cuda_conv2d_stage(ctx.ptr(), x.ptr, staged.ptr, g.batch, g.cin, g.h, g.w) })
}

/// `conv2d_forward` reading x through its staged copy (bit-identical to the plain call).
pub fn conv2d_forward_staged(ctx: &Context, x: &DeviceBuf, staged: Option<&DeviceBuf>, w: &DeviceBuf, bias: Option<&DeviceBuf>,
                             relu: bool, y: &mut DeviceBuf, g: &ConvGeometry) -> Result<(), CudaError> {
    length("x", x, g.x_len())?;
    length("w", w, g.w_len())?;
    length("y", y, g.y_len())?;
    check(unsafe {
        ffi::katsu_cuda_conv2d_fwd_staged(ctx.ptr(), x.ptr, opt_const(staged), w.ptr, opt_const(bias), y.ptr, g.batch, g.cin,
                                          g.h, g.w, g.cout, g.kh, g.kw, g.stride, g.padding, relu as i32)
    })
}

/// `conv2d_backward` reading x through its staged copy (dW).
pub fn conv2d_backward_staged(ctx: &Context, x: &DeviceBuf, staged: Option<&DeviceBuf>, w: &DeviceBuf, grad: &DeviceBuf,
                              scale: Option<GradScale<'_>>, dx: Option<&mut DeviceBuf>, dw: Option<&mut DeviceBuf>,
                              g: &ConvGeometry, accumulate: bool) -> Result<(), CudaError> {
    length("x", x, g.x_len())?;
    length("w", w, g.w_len())?;
    length("grad", grad, g.y_len())?;
    let (scalar, factor) = scale.map_or((ptr::null(), 1.0), |s| (opt_const(s.scalar), s.factor));
    check(unsafe {
        ffi::katsu_cuda_conv2d_bwd_staged(ctx.ptr(), x.ptr, opt_const(staged), w.ptr, grad.ptr, scalar, factor, opt_mut(dx),
                                          opt_mut(dw), g.batch, g.cin, g.h, g.w, g.cout, g.kh, g.kw, g.stride, g.padding,
                                          accumulate as i32)
    })
}

/// Scale of the upstream gradient handed to `conv2d_backward`: the gradient is `factor * scalar[0] * g`
/// without being stored (what the VJP of `sum(y * y)` sends: g = y, factor 2, scalar = the loss adjoint).
pub struct GradScale<'a> {
    pub scalar: Option<&'a DeviceBuf>,
    pub factor: f32,
}

/// One `backward_buffers` (conv2d.rs:269-292).  `dx` / `dw` may be `None`; `accumulate` adds to their
/// contents, which folds in the `pending[parent] += grad` pass of tensor.rs:383-390.
pub fn conv2d_backward(ctx: &Context, x: &DeviceBuf, w: &DeviceBuf, grad: &DeviceBuf, scale: Option<GradScale<'_>>,
                       dx: Option<&mut DeviceBuf>, dw: Option<&mut DeviceBuf>, g: &ConvGeometry, accumulate: bool)
                       -> Result<(), CudaError> {
    length("x", x, g.x_len())?;
    length("w", w, g.w_len())?;
    length("grad", grad, g.y_len())?;
    if let Some(b) = dx.as_deref() {
        length("dx", b, g.x_len())?;
    }
    if let Some(b) = dw.as_deref() {
        length("dw", b, g.w_len())?;
    }
    let (scalar, factor) = scale.map_or((ptr::null(), 1.0), |s| (opt_const(s.scalar), s.factor));
    check(unsafe {
        ffi::katsu_cuda_conv2d_bwd_scaled(ctx.ptr(), x.ptr, w.ptr, grad.ptr, scalar, factor, opt_mut(dx), opt_mut(dw), g.batch,
                                          g.cin, g.h, g.w, g.cout, g.kh, g.kw, g.stride, g.padding, accumulate as i32)
    })
}

/// VJP of the bias / ReLU epilogue: `dg` = grad where `y_act > 0` (else 0), `dbias[k]` (+)= its sum.
pub fn bias_relu_backward(ctx: &Context, y_act: &DeviceBuf, grad: &DeviceBuf, dg: Option<&mut DeviceBuf>,
                          dbias: Option<&mut DeviceBuf>, g: &ConvGeometry, relu: bool, accumulate_bias: bool)
                          -> Result<(), CudaError> {
    length("y", y_act, g.y_len())?;
    length("grad", grad, g.y_len())?;
    check(unsafe {
        ffi::katsu_cuda_bias_relu_bwd(ctx.ptr(), y_act.ptr, grad.ptr, opt_mut(dg), opt_mut(dbias), g.batch, g.cout, g.oh * g.ow,
                                      relu as i32, accumulate_bias as i32)
    })
}

/// `Tensor::matmul` (tensor.rs:264-273): c[m,n] = a[m,k] @ b[k,n].
pub fn matmul(ctx: &Context, a: &DeviceBuf, b: &DeviceBuf, c: &mut DeviceBuf, m: usize, k: usize, n: usize)
              -> Result<(), CudaError> {
    length("a", a, m * k)?;
    length("b", b, k * n)?;
    length("c", c, m * n)?;
    check(unsafe { ffi::katsu_cuda_matmul_fwd(ctx.ptr(), a.ptr, b.ptr, c.ptr, m, k, n) })
}

/// Matmul VJP (tensor.rs:418-445): da (+)= g @ b^T, db (+)= a^T @ g.
pub fn matmul_backward(ctx: &Context, a: &DeviceBuf, b: &DeviceBuf, grad: &DeviceBuf, da: Option<&mut DeviceBuf>,
                       db: Option<&mut DeviceBuf>, m: usize, k: usize, n: usize, accumulate: bool) -> Result<(), CudaError> {
    length("a", a, m * k)?;
    length("b", b, k * n)?;
    length("grad", grad, m * n)?;
    check(unsafe {
        ffi::katsu_cuda_matmul_bwd(ctx.ptr(), a.ptr, b.ptr, grad.ptr, opt_mut(da), opt_mut(db), m, k, n, accumulate as i32)
    })
}

macro_rules! same_len {
    ($($buf:expr),+ ; $len:expr) => { $( length(stringify!($buf), $buf, $len)?; )+ };
}

/// `Tensor::add` / `Tensor::mul` (tensor.rs:226-233).
pub fn add(ctx: &Context, a: &DeviceBuf, b: &DeviceBuf, out: &mut DeviceBuf) -> Result<(), CudaError> {
    same_len!(b, out; a.len);
    check(unsafe { ffi::katsu_cuda_add(ctx.ptr(), a.ptr, b.ptr, out.ptr, a.len) })
}
pub fn mul(ctx: &Context, a: &DeviceBuf, b: &DeviceBuf, out: &mut DeviceBuf) -> Result<(), CudaError> {
    same_len!(b, out; a.len);
    check(unsafe { ffi::katsu_cuda_mul(ctx.ptr(), a.ptr, b.ptr, out.ptr, a.len) })
}
/// `Tensor::sum` (tensor.rs:243-247) into a one-element buffer.
pub fn sum(ctx: &Context, a: &DeviceBuf, out: &mut DeviceBuf) -> Result<(), CudaError> {
    length("out", out, 1)?;
    check(unsafe { ffi::katsu_cuda_sum(ctx.ptr(), a.ptr, out.ptr, a.len) })
}
/// sum(a * a) in one pass, bit-identical to `mul` then `sum`.
pub fn sum_of_squares(ctx: &Context, a: &DeviceBuf, out: &mut DeviceBuf) -> Result<(), CudaError> {
    length("out", out, 1)?;
    check(unsafe { ffi::katsu_cuda_sumsq(ctx.ptr(), a.ptr, out.ptr, a.len) })
}
/// Both Mul VJP edges of y * y under a broadcast adjoint `scalar[0]` (tensor.rs:392-417).
pub fn square_vjp(ctx: &Context, dst: &mut DeviceBuf, src: &DeviceBuf, scalar: &DeviceBuf, accumulate: bool)
                  -> Result<(), CudaError> {
    same_len!(src; dst.len);
    length("scalar", scalar, 1)?;
    check(unsafe { ffi::katsu_cuda_square_vjp(ctx.ptr(), dst.ptr, src.ptr, scalar.ptr, dst.len, accumulate as i32) })
}
/// dst += g (tensor.rs:353-356, 387-389, 400-408).
pub fn axpy_acc(ctx: &Context, dst: &mut DeviceBuf, g: &DeviceBuf) -> Result<(), CudaError> {
    same_len!(g; dst.len);
    check(unsafe { ffi::katsu_cuda_axpy_acc(ctx.ptr(), dst.ptr, g.ptr, dst.len) })
}
/// dst += g * other (Mul VJP edge, tensor.rs:400-408).
pub fn mul_acc(ctx: &Context, dst: &mut DeviceBuf, g: &DeviceBuf, other: &DeviceBuf) -> Result<(), CudaError> {
    same_len!(g, other; dst.len);
    check(unsafe { ffi::katsu_cuda_mul_acc(ctx.ptr(), dst.ptr, g.ptr, other.ptr, dst.len) })
}
/// dst += g[0] (Sum VJP, tensor.rs:410-417).
pub fn bcast_acc(ctx: &Context, dst: &mut DeviceBuf, g: &DeviceBuf) -> Result<(), CudaError> {
    length("g", g, 1)?;
    check(unsafe { ffi::katsu_cuda_bcast_acc(ctx.ptr(), dst.ptr, g.ptr, dst.len) })
}
/// w -= lr * dw (docs/roadmap.md:21-22).
pub fn sgd_step(ctx: &Context, w: &mut DeviceBuf, dw: &DeviceBuf, lr: f32) -> Result<(), CudaError> {
    same_len!(dw; w.len);
    check(unsafe { ffi::katsu_cuda_sgd_step(ctx.ptr(), w.ptr, dw.ptr, lr, w.len) })
}

/// Data-parallel gradient exchange: one process per GPU, images sharded over ranks, only parameter
/// gradients cross devices (dW sums over the batch, conv2d.rs:289).
pub struct Comm {
    ctx: Context,
}

impl Comm {
    /// Rank 0 creates the id and ships its bytes to the other ranks by any means.
    pub fn unique_id() -> Result<[u8; ffi::KATSU_COMM_ID_BYTES], CudaError> {
        let mut id = [0u8; ffi::KATSU_COMM_ID_BYTES];
        check(unsafe { ffi::katsu_cuda_comm_unique_id(id.as_mut_ptr()) })?;
        Ok(id)
    }

    pub fn init(ctx: &Context, id: &[u8; ffi::KATSU_COMM_ID_BYTES], n_ranks: usize, rank: usize) -> Result<Self, CudaError> {
        check(unsafe { ffi::katsu_cuda_comm_init(ctx.ptr(), id.as_ptr(), n_ranks as i32, rank as i32) })?;
        Ok(Self { ctx: ctx.clone() })
    }

    /// In-place sum over all ranks of a flat gradient bucket, ordered on the context's stream.
    pub fn allreduce_sum(&self, bucket: &mut DeviceBuf) -> Result<(), CudaError> {
        check(unsafe { ffi::katsu_cuda_allreduce_sum(self.ctx.ptr(), bucket.ptr, bucket.len) })
    }
}

impl Drop for Comm {
    fn drop(&mut self) {
        unsafe { ffi::katsu_cuda_comm_destroy(self.ctx.ptr()) };
    }
}

/// A CUDA event on the context's stream, for timing and for ordering two contexts of one device.
pub struct Event {
    ctx: Context,
    raw: *mut ffi::Event,
}

impl Event {
    pub fn new(ctx: &Context) -> Result<Self, CudaError> {
        let mut raw = ptr::null_mut();
        check(unsafe { ffi::katsu_cuda_event_create(ctx.ptr(), &mut raw) })?;
        Ok(Self { ctx: ctx.clone(), raw })
    }
    pub fn record(&self) -> Result<(), CudaError> {
        check(unsafe { ffi::katsu_cuda_event_record(self.ctx.ptr(), self.raw) })
    }
    /// Makes `waiter`'s later work wait on the device for this event; the host does not block.
    pub fn make_wait(&self, waiter: &Context) -> Result<(), CudaError> {
        check(unsafe { ffi::katsu_cuda_wait_event(waiter.ptr(), self.raw) })
    }
    pub fn elapsed_ms(&self, stop: &Event) -> Result<f32, CudaError> {
        let mut ms = 0.0f32;
        check(unsafe { ffi::katsu_cuda_event_elapsed_ms(self.ctx.ptr(), self.raw, stop.raw, &mut ms) })?;
        Ok(ms)
    }
}

impl Drop for Event {
    fn drop(&mut self) {
        unsafe { ffi::katsu_cuda_event_destroy(self.ctx.ptr(), self.raw) };
    }
}
