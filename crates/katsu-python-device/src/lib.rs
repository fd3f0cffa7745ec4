//! PyO3 binding of the device-backed Tensor and Conv2D: the tensor API the reference's Python
//! package does not have yet (crates/katsu-python/src/lib.rs:3-8 exports only `__version__`;
//! docs/roadmap.md:28-36 plans the rest).
//!
//! NOT COMPILED in the repository that carries the kernels (no Rust toolchain, no pyo3 crate in its
//! build image).  What runs and is tested there with the same surface is the ctypes package
//! katsu_b200/__init__.py over the C++ mirror.
//!
//! `Tensor` is `Rc`-based and `!Send` (crates/katsu-core/src/tensor.rs:95-99), so the classes are
//! `unsendable`: PyO3 then raises if an object is touched from another thread than its creator
//! (docs/architecture.md:54-56), which also keeps one host thread per device context.

use katsu_core::{Conv2D, Tensor, TensorError};
use pyo3::exceptions::{PyRuntimeError, PyValueError};
use pyo3::prelude::*;

fn to_py(e: TensorError) -> PyErr {
    match e {
        TensorError::Device { .. } | TensorError::Allocation(_) => PyRuntimeError::new_err(e.to_string()),
        _ => PyValueError::new_err(e.to_string()),
    }
}

#[pyclass(name = "Tensor", unsendable)]
#[derive(Clone)]
struct PyTensor(Tensor);

#[pymethods]
impl PyTensor {
    #[new]
    fn new(data: Vec<f32>, shape: Vec<usize>) -> PyResult<Self> {
        Tensor::new(data, &shape).map(Self).map_err(to_py)
    }
    #[staticmethod]
    fn zeros(shape: Vec<usize>) -> PyResult<Self> {
        Tensor::zeros(&shape).map(Self).map_err(to_py)
    }
    fn shape(&self) -> Vec<usize> {
        self.0.shape().to_vec()
    }
    /// Host copy of the values (one synchronous device-to-host transfer on first use).
    fn data(&self) -> Vec<f32> {
        self.0.data().to_vec()
    }
    fn grad(&self) -> PyResult<Option<Vec<f32>>> {
        Ok(self.0.grad().map_err(to_py)?.clone())
    }
    fn zero_grad(&self) -> PyResult<()> {
        self.0.zero_grad().map_err(to_py)
    }
    fn add(&self, rhs: &PyTensor) -> PyResult<Self> {
        self.0.add(&rhs.0).map(Self).map_err(to_py)
    }
    fn mul(&self, rhs: &PyTensor) -> PyResult<Self> {
        self.0.mul(&rhs.0).map(Self).map_err(to_py)
    }
    fn matmul(&self, rhs: &PyTensor) -> PyResult<Self> {
        self.0.matmul(&rhs.0).map(Self).map_err(to_py)
    }
    fn sum(&self) -> PyResult<Self> {
        self.0.sum().map(Self).map_err(to_py)
    }
    fn reshape(&self, shape: Vec<usize>) -> PyResult<Self> {
        self.0.reshape(&shape).map(Self).map_err(to_py)
    }
    fn backward(&self) -> PyResult<()> {
        self.0.backward().map_err(to_py)
    }
    fn backward_with(&self, seed: Vec<f32>) -> PyResult<()> {
        self.0.backward_with(&seed).map_err(to_py)
    }
    fn to_device(&self) -> PyResult<()> {
        self.0.to_device().map_err(to_py)
    }
    fn sgd_step(&self, lr: f32) -> PyResult<()> {
        self.0.sgd_step(lr).map_err(to_py)
    }
}

#[pyclass(name = "Conv2D", unsendable)]
struct PyConv2D(Conv2D);

#[pymethods]
impl PyConv2D {
    #[new]
    #[pyo3(signature = (in_channels, out_channels, kernel_size, stride, padding, seed = 42))]
    fn new(in_channels: usize, out_channels: usize, kernel_size: (usize, usize), stride: usize, padding: usize,
           seed: u64) -> PyResult<Self> {
        Conv2D::new_seeded(in_channels, out_channels, kernel_size, stride, padding, seed).map(Self).map_err(to_py)
    }
    #[staticmethod]
    fn from_weights(weights: &PyTensor, stride: usize, padding: usize) -> PyResult<Self> {
        Conv2D::from_weights(weights.0.clone(), stride, padding).map(Self).map_err(to_py)
    }
    fn weights(&self) -> PyTensor {
        PyTensor(self.0.weights().clone())
    }
    fn forward(&mut self, input: &PyTensor) -> PyResult<PyTensor> {
        self.0.forward(&input.0).map(PyTensor).map_err(to_py)
    }
    fn backward(&self, grad_output: &PyTensor) -> PyResult<(PyTensor, PyTensor)> {
        let (dx, dw) = self.0.backward(&grad_output.0).map_err(to_py)?;
        Ok((PyTensor(dx), PyTensor(dw)))
    }
    fn get_activation_map(&self) -> Option<PyTensor> {
        self.0.get_activation_map().map(PyTensor)
    }
    fn clear_cache(&mut self) {
        self.0.clear_cache()
    }
}

#[pymodule]
fn _native(module: &Bound<'_, PyModule>) -> PyResult<()> {
    module.add("__version__", env!("CARGO_PKG_VERSION"))?;
    module.add_class::<PyTensor>()?;
    module.add_class::<PyConv2D>()?;
    Ok(())
}
