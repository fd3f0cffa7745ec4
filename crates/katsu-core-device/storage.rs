// Device storage for katsu-core's TensorNode: the pieces a maintainer adds to
// crates/katsu-core/src/tensor.rs (behind a `cuda` cargo feature) so that Tensor keeps its public
// surface while its values live on the GPU.  Only new items are written out here; where an existing
// function changes, the comment names it by its line range in the reference and states the change.
//
// NOT COMPILED in the repository that carries the kernels (no Rust toolchain in its build image).
// The same design, compiled and tested there, is katsu_b200/csrc/host/katsu.{hpp,cpp}.
//
// katsu-core keeps #![forbid(unsafe_code)]: everything below is safe Rust over katsu_cuda's safe API.

use std::cell::{OnceCell, RefCell};

use katsu_cuda::{Context, DeviceBuf};

/// Replaces `data: Vec<f32>` in TensorNode (tensor.rs:101-107).  Values are immutable after
/// construction (the reference's own rule), so each side is filled lazily from the other, once.
pub(crate) enum Storage {
    /// What the reference has today.  Uploaded on first use by a device op.
    Host { values: Vec<f32>, device: OnceCell<DeviceBuf> },
    /// Result of a device op.  `mirror` is filled by the first `Tensor::data()`.
    Device { buf: DeviceBuf, mirror: OnceCell<Vec<f32>> },
}

impl Storage {
    /// `Tensor::data()` (tensor.rs:172-174) keeps returning `&[f32]`: a synchronous device-to-host
    /// copy on first access, never inside a timed region.
    pub(crate) fn host(&self) -> Result<&[f32], TensorError> {
        match self {
            Storage::Host { values, .. } => Ok(values),
            Storage::Device { buf, mirror } => {
                if mirror.get().is_none() {
                    let _ = mirror.set(buf.to_host().map_err(TensorError::from)?);
                }
                Ok(mirror.get().expect("just set"))
            }
        }
    }

    /// The device copy every kernel call reads (explicit `Tensor::to_device()` calls this early).
    pub(crate) fn device(&self, ctx: &Context) -> Result<&DeviceBuf, TensorError> {
        match self {
            Storage::Device { buf, .. } => Ok(buf),
            Storage::Host { values, device } => {
                if device.get().is_none() {
                    let _ = device.set(DeviceBuf::from_host(ctx, values).map_err(TensorError::from)?);
                }
                Ok(device.get().expect("just set"))
            }
        }
    }
}

/// Replaces `grad: RefCell<Option<Vec<f32>>>` (tensor.rs:104).  `Tensor::grad()` keeps its type
/// `Ref<'_, Option<Vec<f32>>>` by filling `host` from `device` under the borrow.
pub(crate) struct GradStorage {
    pub(crate) host: RefCell<Option<Vec<f32>>>,
    pub(crate) device: RefCell<Option<DeviceBuf>>,
}

/// New variant of TensorError (tensor.rs:9-20); the existing ones keep their meaning.
/// `KATSU_ERR_ALLOC` maps to the existing `Allocation` meaning through `is_allocation()`.
impl From<katsu_cuda::CudaError> for TensorError {
    fn from(e: katsu_cuda::CudaError) -> Self {
        TensorError::Device { code: e.code, message: e.message }
    }
}

// Call sites that change (line numbers of the reference):
//
//   conv2d.rs:99-103    Conv2D::forward, after Geometry::new:
//       katsu_cuda::conv2d_forward(ctx, x.device()?, w.device()?, None, false, &mut y, &geometry.into())?
//       wide layers (katsu_cuda::conv2d_staged_len(ctx, &g)? > 0): the input node keeps a second device buffer
//       beside `device`, `staged: OnceCell<(Precision, DeviceBuf)>`, written by katsu_cuda::conv2d_stage on the
//       first use in the current precision mode; forward and backward then call conv2d_forward_staged /
//       conv2d_backward_staged with it (one staging pass per step instead of two; values never change)
//   conv2d.rs:283-290   backward_buffers:
//       katsu_cuda::conv2d_backward(ctx, x, w, g, None, Some(&mut dx), Some(&mut dw), &geometry.into(), false)?
//   tensor.rs:374-391   Op::backward, Conv2D arm: the same call with the pending adjoints of the two
//                       parents as dx / dw and accumulate = true (skips the `+=` loop of 383-390);
//                       two calls, one output each, when x and w are the same node
//   tensor.rs:266-272   Tensor::matmul:            katsu_cuda::matmul(ctx, a, b, &mut c, m, k, n)?
//   tensor.rs:425-444   Matmul arm:                katsu_cuda::matmul_backward(.., accumulate = true)
//   tensor.rs:231-233   elementwise:               katsu_cuda::add / mul
//   tensor.rs:245       sum:                       katsu_cuda::sum (or sum_of_squares for y.mul(&y))
//   tensor.rs:387-389, 400-416, 353-356            katsu_cuda::axpy_acc / mul_acc / bcast_acc / square_vjp
//
// Additions to the public surface, as in the C++ mirror: Tensor::to_device(), Tensor::to_host(),
// Tensor::reshape(&[usize]) with Op::Reshape (BASELINE's small CNN needs [N,64,32,32] -> [N,65536] and
// the reference has no view op), TensorError::Device, a precision selector, Tensor::sgd_step(lr),
// Conv2D::from_weights_bias(weights, bias, stride, padding, relu).
