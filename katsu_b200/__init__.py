"""katsu_b200 -- Python face of the B200-native Conv2D / matmul hot path.

The names mirror katsu_core's public surface (crates/katsu-core/src/lib.rs:5,8):
Tensor, Conv2D, Op and the TensorError variants.  Each object is a handle into
the C++ host mirror (csrc/host, libkatsu_host.so), which keeps the autograd
graph and runs every arithmetic loop through the C ABI of
include/katsu_cuda.h on the GPU.  Nothing here computes on the CPU; without
the built libraries or without a GPU, operations raise.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from . import cabi

_PKG = os.path.dirname(os.path.abspath(__file__))
HOST_LIB_PATH = os.path.join(_PKG, "lib", "libkatsu_host.so")

USIZE_MAX = (1 << 64) - 1

__all__ = [
    "Tensor", "Conv2D", "Op", "TensorError", "ShapeOverflow", "InvalidConv", "MissingForward",
    "NonScalarBackward", "GradientBorrowed", "DataLength", "ShapeMismatch", "RankMismatch",
    "MatmulMismatch", "Allocation", "DeviceError", "set_device", "set_precision", "synchronize",
    "set_loss_fusion", "loss_fusion",
    "context", "MODE_3XTF32", "MODE_TF32", "MODE_FP32",
]

MODE_3XTF32, MODE_TF32, MODE_FP32 = cabi.MODE_3XTF32, cabi.MODE_TF32, cabi.MODE_FP32


# ---------------------------------------------------------------------------
# errors (crates/katsu-core/src/tensor.rs:9-82)
# ---------------------------------------------------------------------------
class TensorError(Exception):
    def __init__(self, message="", a=0, b=0):
        super().__init__(message)
        self.message, self.a, self.b = message, a, b

    def __str__(self):
        return self.message


class ShapeOverflow(TensorError):
    pass


class InvalidConv(TensorError):
    pass


class MissingForward(TensorError):
    pass


class NonScalarBackward(TensorError):
    pass


class GradientBorrowed(TensorError):
    pass


class DataLength(TensorError):
    @property
    def expected(self):
        return self.a

    @property
    def actual(self):
        return self.b


class ShapeMismatch(TensorError):
    pass


class RankMismatch(TensorError):
    @property
    def left(self):
        return self.a

    @property
    def right(self):
        return self.b


class MatmulMismatch(TensorError):
    @property
    def left_columns(self):
        return self.a

    @property
    def right_rows(self):
        return self.b


class Allocation(TensorError):
    pass


class DeviceError(TensorError):
    """CUDA / library failure; has no counterpart in the CPU-only reference."""


_ERRORS = {1: ShapeOverflow, 2: InvalidConv, 3: MissingForward, 4: NonScalarBackward, 5: GradientBorrowed,
           6: DataLength, 7: ShapeMismatch, 8: RankMismatch, 9: MatmulMismatch, 10: Allocation, 11: DeviceError}

# ---------------------------------------------------------------------------
# library
# ---------------------------------------------------------------------------
_vp = ctypes.c_void_p
_sz = ctypes.c_size_t
_szp = ctypes.POINTER(ctypes.c_size_t)
_lib = None


def _load():
    global _lib
    if _lib is None:
        cabi.load()  # libkatsu_cuda.so first (libkatsu_host.so links against it)
        if not os.path.exists(HOST_LIB_PATH):
            raise OSError(f"{HOST_LIB_PATH} is missing: build it with `python -m katsu_b200.build`")
        lib = ctypes.CDLL(HOST_LIB_PATH)
        lib.kh_last_error_message.restype = ctypes.c_char_p
        lib.kh_last_error_numbers.argtypes = [_szp, _szp]
        lib.kh_last_error_numbers.restype = None
        sigs = {
            "kh_set_device": [ctypes.c_int], "kh_set_precision": [ctypes.c_int], "kh_synchronize": [],
            "kh_context": [ctypes.POINTER(_vp)],
            "kh_tensor_new": [_vp, _sz, _szp, _sz, ctypes.POINTER(_vp)],
            "kh_tensor_zeros": [_szp, _sz, ctypes.POINTER(_vp)],
            "kh_tensor_clone": [_vp, ctypes.POINTER(_vp)],
            "kh_tensor_data": [_vp, _vp, _sz],
            "kh_tensor_parent": [_vp, _sz, ctypes.POINTER(_vp)],
            "kh_tensor_grad": [_vp, _vp, _sz, ctypes.POINTER(ctypes.c_int)],
            "kh_tensor_borrow_grad": [_vp, ctypes.POINTER(_vp)],
            "kh_tensor_zero_grad": [_vp],
            "kh_tensor_add": [_vp, _vp, ctypes.POINTER(_vp)], "kh_tensor_mul": [_vp, _vp, ctypes.POINTER(_vp)],
            "kh_tensor_sum": [_vp, ctypes.POINTER(_vp)], "kh_tensor_matmul": [_vp, _vp, ctypes.POINTER(_vp)],
            "kh_tensor_reshape": [_vp, _szp, _sz, ctypes.POINTER(_vp)],
            "kh_tensor_backward": [_vp], "kh_tensor_backward_with": [_vp, _vp, _sz],
            "kh_tensor_to_device": [_vp], "kh_tensor_to_host": [_vp],
            "kh_tensor_sgd_step": [_vp, ctypes.c_float],
            "kh_conv_from_weights_bias": [_vp, _vp, _sz, _sz, ctypes.c_int, ctypes.POINTER(_vp)],
            "kh_conv_bias": [_vp, ctypes.POINTER(_vp)], "kh_conv_relu": [_vp], "kh_loss_fusion": [],
            "kh_tensor_device_data": [_vp, ctypes.POINTER(_vp)], "kh_tensor_device_grad": [_vp, ctypes.POINTER(_vp)],
            "kh_conv_new_seeded": [_sz, _sz, _sz, _sz, _sz, _sz, ctypes.c_uint64, ctypes.POINTER(_vp)],
            "kh_conv_from_weights": [_vp, _sz, _sz, ctypes.POINTER(_vp)],
            "kh_conv_weights": [_vp, ctypes.POINTER(_vp)],
            "kh_conv_forward": [_vp, _vp, ctypes.POINTER(_vp)],
            "kh_conv_backward": [_vp, _vp, ctypes.POINTER(_vp), ctypes.POINTER(_vp)],
            "kh_conv_activation_map": [_vp, ctypes.POINTER(_vp)],
        }
        for name, argtypes in sigs.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = argtypes, ctypes.c_int
        for name, argtypes, restype in [
            ("kh_tensor_free", [_vp], None), ("kh_tensor_rank", [_vp], _sz), ("kh_tensor_numel", [_vp], _sz),
            ("kh_tensor_shape", [_vp, _szp], None), ("kh_tensor_id", [_vp], _vp),
            ("kh_tensor_op", [_vp, ctypes.POINTER(ctypes.c_int), _szp, _szp], None),
            ("kh_tensor_parent_count", [_vp], _sz), ("kh_grad_borrow_release", [_vp], None),
            ("kh_conv_free", [_vp], None), ("kh_conv_stride", [_vp], _sz), ("kh_conv_padding", [_vp], _sz),
            ("kh_conv_clear_cache", [_vp], None), ("kh_set_loss_fusion", [ctypes.c_int], None),
            ("kh_tensor_op_flags", [_vp, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)], None),
        ]:
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = argtypes, restype
        _lib = lib
    return _lib


def _check(rc: int) -> None:
    if rc == 0:
        return
    lib = _load()
    a, b = _sz(), _sz()
    lib.kh_last_error_numbers(ctypes.byref(a), ctypes.byref(b))
    raise _ERRORS.get(rc, TensorError)(lib.kh_last_error_message().decode("utf-8", "replace"), a.value, b.value)


def _shape_args(shape):
    dims = [int(d) for d in shape]
    for d in dims:
        if d < 0 or d > USIZE_MAX:
            raise ShapeOverflow("shape exceeds addressable tensor storage")
    return (ctypes.c_size_t * len(dims))(*dims), len(dims)


def set_device(ordinal: int) -> None:
    """Device ordinal for this process (one process per GPU); call before the first op."""
    _check(_load().kh_set_device(int(ordinal)))


def set_precision(mode: int) -> None:
    _check(_load().kh_set_precision(int(mode)))


def synchronize() -> None:
    _check(_load().kh_synchronize())


def set_loss_fusion(on: bool) -> None:
    """Loss-graph fusion (default on): y.mul(y) defers its values, sum() of it reads y once, and
    backward hands the convolution "2 * s * y" symbolically instead of writing it out.  Values and
    gradients are those of node-by-node evaluation (tensor.rs:226-247, 392-417) either way."""
    _load().kh_set_loss_fusion(1 if on else 0)


def loss_fusion() -> bool:
    return bool(_load().kh_loss_fusion())


def context() -> int:
    """The raw katsu_cuda_ctx* the host mirror uses (for C-ABI level callers)."""
    out = _vp()
    _check(_load().kh_context(ctypes.byref(out)))
    return out.value


# ---------------------------------------------------------------------------
# Op (tensor.rs:85-93, plus Reshape)
# ---------------------------------------------------------------------------
class Op:
    _KINDS = ["Leaf", "Add", "Mul", "Matmul", "Conv2D", "Sum", "Reshape"]

    def __init__(self, kind, stride=None, padding=None, bias=False, relu=False):
        self.kind, self.stride, self.padding, self.bias, self.relu = kind, stride, padding, bias, relu

    def _key(self):
        return (self.kind, self.stride, self.padding, self.bias, self.relu)

    def __eq__(self, other):
        return isinstance(other, Op) and self._key() == other._key()

    def __hash__(self):
        return hash(self._key())

    def __repr__(self):
        if self.kind == "Conv2D":
            extra = (", bias" if self.bias else "") + (", relu" if self.relu else "")
            return f"Conv2D {{ stride: {self.stride}, padding: {self.padding}{extra} }}"
        return self.kind

    @staticmethod
    def Conv2D(stride, padding, bias=False, relu=False):
        """bias / relu are additions (the reference's roadmap lists them as not implemented yet)."""
        return Op("Conv2D", stride, padding, bias, relu)


Op.Leaf, Op.Add, Op.Mul, Op.Matmul, Op.Sum, Op.Reshape = (
    Op(k) for k in ("Leaf", "Add", "Mul", "Matmul", "Sum", "Reshape"))


class GradBorrow:
    """A held gradient borrow (the Ref guard of tensor.rs:200-206): backward and
    zero_grad fail with GradientBorrowed until release()."""

    def __init__(self, handle):
        self._handle = handle

    def release(self):
        if self._handle:
            _load().kh_grad_borrow_release(self._handle)
            self._handle = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.release()

    def __del__(self):
        self.release()


class Tensor:
    """Handle to one graph node (tensor.rs:98-107).  `clone()` and Python
    assignment both keep node identity."""

    def __init__(self, data, shape):
        lib = _load()
        array = np.ascontiguousarray(np.asarray(data, dtype=np.float32).reshape(-1))
        dims, rank = _shape_args(shape)
        out = _vp()
        _check(lib.kh_tensor_new(array.ctypes.data, array.size, dims, rank, ctypes.byref(out)))
        self._h = out.value

    @classmethod
    def _wrap(cls, handle):
        t = cls.__new__(cls)
        t._h = handle
        return t

    def __del__(self):
        h = getattr(self, "_h", None)
        if h and _lib is not None:
            _lib.kh_tensor_free(h)
            self._h = None

    @classmethod
    def zeros(cls, shape):
        dims, rank = _shape_args(shape)
        out = _vp()
        _check(_load().kh_tensor_zeros(dims, rank, ctypes.byref(out)))
        return cls._wrap(out.value)

    def clone(self):
        out = _vp()
        _check(_lib.kh_tensor_clone(self._h, ctypes.byref(out)))
        return Tensor._wrap(out.value)

    def id(self):
        return _lib.kh_tensor_id(self._h)

    def shape(self):
        rank = _lib.kh_tensor_rank(self._h)
        dims = (ctypes.c_size_t * max(rank, 1))()
        _lib.kh_tensor_shape(self._h, dims)
        return [int(dims[i]) for i in range(rank)]

    def rank(self):
        return int(_lib.kh_tensor_rank(self._h))

    def numel(self):
        return int(_lib.kh_tensor_numel(self._h))

    def data(self):
        """Host copy of the values (synchronous device-to-host on first use)."""
        out = np.empty(self.numel(), dtype=np.float32)
        _check(_lib.kh_tensor_data(self._h, out.ctypes.data, out.size))
        return out

    def op(self):
        kind, stride, padding = ctypes.c_int(), _sz(), _sz()
        _lib.kh_tensor_op(self._h, ctypes.byref(kind), ctypes.byref(stride), ctypes.byref(padding))
        name = Op._KINDS[kind.value]
        if name != "Conv2D":
            return Op(name)
        bias, relu = ctypes.c_int(), ctypes.c_int()
        _lib.kh_tensor_op_flags(self._h, ctypes.byref(bias), ctypes.byref(relu))
        return Op.Conv2D(stride.value, padding.value, bool(bias.value), bool(relu.value))

    def parents(self):
        result = []
        for i in range(_lib.kh_tensor_parent_count(self._h)):
            out = _vp()
            _check(_lib.kh_tensor_parent(self._h, i, ctypes.byref(out)))
            result.append(Tensor._wrap(out.value))
        return result

    def grad(self):
        """Host copy of the gradient, or None (tensor.rs:200-206)."""
        out = np.empty(self.numel(), dtype=np.float32)
        has = ctypes.c_int()
        _check(_lib.kh_tensor_grad(self._h, out.ctypes.data, out.size, ctypes.byref(has)))
        return out if has.value else None

    def borrow_grad(self):
        out = _vp()
        _check(_lib.kh_tensor_borrow_grad(self._h, ctypes.byref(out)))
        return GradBorrow(out.value)

    def zero_grad(self):
        _check(_lib.kh_tensor_zero_grad(self._h))

    def _binary(self, fn, rhs):
        out = _vp()
        _check(fn(self._h, rhs._h, ctypes.byref(out)))
        return Tensor._wrap(out.value)

    def add(self, rhs):
        return self._binary(_lib.kh_tensor_add, rhs)

    def mul(self, rhs):
        return self._binary(_lib.kh_tensor_mul, rhs)

    def matmul(self, rhs):
        return self._binary(_lib.kh_tensor_matmul, rhs)

    def sum(self):
        out = _vp()
        _check(_lib.kh_tensor_sum(self._h, ctypes.byref(out)))
        return Tensor._wrap(out.value)

    def reshape(self, shape):
        """Addition to the reference surface: same data, new shape, gradient passes through."""
        dims, rank = _shape_args(shape)
        out = _vp()
        _check(_lib.kh_tensor_reshape(self._h, dims, rank, ctypes.byref(out)))
        return Tensor._wrap(out.value)

    def backward(self):
        _check(_lib.kh_tensor_backward(self._h))

    def backward_with(self, seed):
        seed = np.ascontiguousarray(np.asarray(seed, dtype=np.float32).reshape(-1))
        _check(_lib.kh_tensor_backward_with(self._h, seed.ctypes.data, seed.size))

    def sgd_step(self, lr):
        """Addition (docs/roadmap.md:21-22): data -= lr * grad in place on the device."""
        _check(_lib.kh_tensor_sgd_step(self._h, float(lr)))

    def to_device(self):
        _check(_lib.kh_tensor_to_device(self._h))
        return self

    def to_host(self):
        _check(_lib.kh_tensor_to_host(self._h))
        return self

    def device_data(self) -> int:
        out = _vp()
        _check(_lib.kh_tensor_device_data(self._h, ctypes.byref(out)))
        return out.value or 0

    def device_grad(self) -> int:
        out = _vp()
        _check(_lib.kh_tensor_device_grad(self._h, ctypes.byref(out)))
        return out.value or 0


class Conv2D:
    """crates/katsu-core/src/conv2d.rs:14-154."""

    def __init__(self, in_channels, out_channels, kernel_size, stride, padding, seed=42):
        lib = _load()
        for v in (in_channels, out_channels, kernel_size[0], kernel_size[1], stride, padding):
            if v < 0 or v > USIZE_MAX:
                raise ShapeOverflow("shape exceeds addressable tensor storage")
        out = _vp()
        _check(lib.kh_conv_new_seeded(in_channels, out_channels, kernel_size[0], kernel_size[1], stride, padding,
                                      seed & USIZE_MAX, ctypes.byref(out)))
        self._h = out.value

    @classmethod
    def new_seeded(cls, in_channels, out_channels, kernel_size, stride, padding, seed):
        return cls(in_channels, out_channels, kernel_size, stride, padding, seed)

    @classmethod
    def from_weights(cls, weights, stride, padding, bias=None, relu=False):
        """bias (a rank-1 Tensor, one value per output channel) and relu are additions: they run in
        the convolution kernel's epilogue and take part in autograd as a third parent of the node."""
        out = _vp()
        if bias is None and not relu:
            _check(_load().kh_conv_from_weights(weights._h, stride, padding, ctypes.byref(out)))
        else:
            _check(_load().kh_conv_from_weights_bias(weights._h, bias._h if bias is not None else None, stride,
                                                     padding, 1 if relu else 0, ctypes.byref(out)))
        layer = cls.__new__(cls)
        layer._h = out.value
        return layer

    def bias(self):
        out = _vp()
        _check(_lib.kh_conv_bias(self._h, ctypes.byref(out)))
        return Tensor._wrap(out.value) if out.value else None

    def relu(self):
        return bool(_lib.kh_conv_relu(self._h))

    def __del__(self):
        h = getattr(self, "_h", None)
        if h and _lib is not None:
            _lib.kh_conv_free(h)
            self._h = None

    def weights(self):
        out = _vp()
        _check(_lib.kh_conv_weights(self._h, ctypes.byref(out)))
        return Tensor._wrap(out.value)

    def in_channels(self):
        return self.weights().shape()[1]

    def out_channels(self):
        return self.weights().shape()[0]

    def kernel_size(self):
        s = self.weights().shape()
        return (s[2], s[3])

    def stride(self):
        return int(_lib.kh_conv_stride(self._h))

    def padding(self):
        return int(_lib.kh_conv_padding(self._h))

    def forward(self, input):
        out = _vp()
        _check(_lib.kh_conv_forward(self._h, input._h, ctypes.byref(out)))
        return Tensor._wrap(out.value)

    def backward(self, grad_output):
        dx, dw = _vp(), _vp()
        _check(_lib.kh_conv_backward(self._h, grad_output._h, ctypes.byref(dx), ctypes.byref(dw)))
        return Tensor._wrap(dx.value), Tensor._wrap(dw.value)

    def get_activation_map(self):
        out = _vp()
        _check(_lib.kh_conv_activation_map(self._h, ctypes.byref(out)))
        return Tensor._wrap(out.value) if out.value else None

    def clear_cache(self):
        _lib.kh_conv_clear_cache(self._h)
