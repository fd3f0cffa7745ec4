"""CPU oracle for katsu-core's Tensor / Conv2D / autograd semantics.

TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and the
benchmark's CPU-baseline leg, never by the shipped package.

Arithmetic is done by oracle/katsu_oracle.c (same loop order and f32 rounding
as the reference); this module restates the graph logic around it:

* Tensor / TensorNode / Op            crates/katsu-core/src/tensor.rs:85-215
* add / mul / sum / matmul            crates/katsu-core/src/tensor.rs:217-280
* topological_order / backward_with   crates/katsu-core/src/tensor.rs:288-362
* Op::backward (per-op VJP arms)      crates/katsu-core/src/tensor.rs:365-449
* Conv2D layer, cache rules, init     crates/katsu-core/src/conv2d.rs:14-166

Parity pin: the reference cannot be compiled here (Rust), so this oracle is
pinned by restating every known-answer assertion of the reference's own tests
(tests/test_oracle_pins.py).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libkatsu_oracle.so")

USIZE_MAX = (1 << 64) - 1
ISIZE_MAX = (1 << 63) - 1


def build(force: bool = False) -> str:
    """Compile katsu_oracle.c with the flags in oracle/Makefile."""
    src = os.path.join(_HERE, "katsu_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B" if force else "-s"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None
_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)
_szp = ctypes.POINTER(ctypes.c_size_t)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.ko_sum.restype = ctypes.c_float
        _lib.ko_sum_f64.restype = ctypes.c_double
        _lib.ko_num_threads.restype = ctypes.c_int
    return _lib


def _p(a: np.ndarray):
    if a.dtype == np.float32:
        return a.ctypes.data_as(_f32p)
    if a.dtype == np.float64:
        return a.ctypes.data_as(_f64p)
    if a.dtype == np.uint64:
        return a.ctypes.data_as(_szp)
    raise TypeError(a.dtype)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32).reshape(-1))


def _sz(v: int):
    return ctypes.c_size_t(int(v))


# ---------------------------------------------------------------------------
# errors (tensor.rs:9-82)
# ---------------------------------------------------------------------------
class TensorError(Exception):
    pass


class ShapeOverflow(TensorError):
    def __str__(self):
        return "shape exceeds addressable tensor storage"


class InvalidConv(TensorError):
    def __str__(self):
        return "invalid Conv2D: " + (self.args[0] if self.args else "")


class MissingForward(TensorError):
    def __str__(self):
        return "Conv2D backward requires a successful forward"


class NonScalarBackward(TensorError):
    def __str__(self):
        return "backward requires one element; use sum() or backward_with(seed)"


class GradientBorrowed(TensorError):
    def __str__(self):
        return "release gradient borrows before backward or zero_grad"


class DataLength(TensorError):
    def __init__(self, expected, actual):
        super().__init__(expected, actual)
        self.expected, self.actual = expected, actual

    def __str__(self):
        return f"expected {self.expected} elements, got {self.actual}"


class ShapeMismatch(TensorError):
    def __str__(self):
        return "elementwise operations require identical shapes (no broadcasting)"


class RankMismatch(TensorError):
    def __init__(self, left, right):
        super().__init__(left, right)
        self.left, self.right = left, right

    def __str__(self):
        return f"matmul requires rank 2, got {self.left} and {self.right}"


class MatmulMismatch(TensorError):
    def __init__(self, left_columns, right_rows):
        super().__init__(left_columns, right_rows)
        self.left_columns, self.right_rows = left_columns, right_rows

    def __str__(self):
        return f"matmul inner dimensions differ: {self.left_columns} and {self.right_rows}"


def element_count(shape) -> int:
    """tensor.rs:127-138."""
    shape = [int(d) for d in shape]
    if 0 in shape:
        return 0
    count = 1
    for d in shape:
        count *= d
        if count > USIZE_MAX:
            raise ShapeOverflow()
    if count > ISIZE_MAX // 4:
        raise ShapeOverflow()
    return count


# ---------------------------------------------------------------------------
# raw kernels over numpy arrays
# ---------------------------------------------------------------------------
def conv_out_dims(h, w, kh, kw, stride, padding):
    return (h + 2 * padding - kh) // stride + 1, (w + 2 * padding - kw) // stride + 1


def conv2d_forward(x, w, xs, ws, stride, padding, mt=False):
    n, c, h, wd = xs
    k, _, r, s = ws
    oh, ow = conv_out_dims(h, wd, r, s, stride, padding)
    y = np.zeros(n * k * oh * ow, dtype=np.float32)
    fn = lib().ko_conv2d_forward_mt if mt else lib().ko_conv2d_forward
    fn(_p(x), _p(w), _p(y), _sz(n), _sz(c), _sz(h), _sz(wd), _sz(k), _sz(r), _sz(s), _sz(stride), _sz(padding))
    return y


def conv2d_backward(x, w, g, xs, ws, stride, padding, mt=False):
    n, c, h, wd = xs
    k, _, r, s = ws
    dx = np.zeros(n * c * h * wd, dtype=np.float32)
    dw = np.zeros(k * c * r * s, dtype=np.float32)
    fn = lib().ko_conv2d_backward_mt if mt else lib().ko_conv2d_backward
    fn(_p(x), _p(w), _p(g), _p(dx), _p(dw), _sz(n), _sz(c), _sz(h), _sz(wd), _sz(k), _sz(r), _sz(s),
       _sz(stride), _sz(padding))
    return dx, dw


def conv2d_forward_f64(x, w, xs, ws, stride, padding):
    n, c, h, wd = xs
    k, _, r, s = ws
    oh, ow = conv_out_dims(h, wd, r, s, stride, padding)
    y = np.zeros(n * k * oh * ow, dtype=np.float64)
    lib().ko_conv2d_forward_f64(_p(x), _p(w), _p(y), _sz(n), _sz(c), _sz(h), _sz(wd), _sz(k), _sz(r), _sz(s),
                                _sz(stride), _sz(padding))
    return y


def conv2d_backward_f64(x, w, g, xs, ws, stride, padding):
    n, c, h, wd = xs
    k, _, r, s = ws
    dx = np.zeros(n * c * h * wd, dtype=np.float64)
    dw = np.zeros(k * c * r * s, dtype=np.float64)
    lib().ko_conv2d_backward_f64(_p(x), _p(w), _p(g), _p(dx), _p(dw), _sz(n), _sz(c), _sz(h), _sz(wd), _sz(k),
                                 _sz(r), _sz(s), _sz(stride), _sz(padding))
    return dx, dw


def _sample(fn, a, b, idx, xs, ws, stride, padding):
    n, c, h, wd = xs
    k, _, r, s = ws
    idx = np.ascontiguousarray(np.asarray(idx, dtype=np.uint64))
    o32 = np.zeros(idx.size, dtype=np.float32)
    o64 = np.zeros(idx.size, dtype=np.float64)
    fn(_p(a), _p(b), _p(idx), _sz(idx.size), _p(o32), _p(o64), _sz(n), _sz(c), _sz(h), _sz(wd), _sz(k), _sz(r),
       _sz(s), _sz(stride), _sz(padding))
    return o32, o64


def sample_y(x, w, idx, xs, ws, stride, padding):
    return _sample(lib().ko_conv2d_sample_y, x, w, idx, xs, ws, stride, padding)


def sample_dx(w, g, idx, xs, ws, stride, padding):
    return _sample(lib().ko_conv2d_sample_dx, w, g, idx, xs, ws, stride, padding)


def sample_dw(x, g, idx, xs, ws, stride, padding):
    return _sample(lib().ko_conv2d_sample_dw, x, g, idx, xs, ws, stride, padding)


def matmul(a, b, m, k, n, mt=False):
    c = np.zeros(m * n, dtype=np.float32)
    (lib().ko_matmul_mt if mt else lib().ko_matmul)(_p(a), _p(b), _p(c), _sz(m), _sz(k), _sz(n))
    return c


def matmul_backward(a, b, g, da, db, m, k, n, mt=False):
    """Accumulates into da / db in place (either may be None)."""
    fn = lib().ko_matmul_backward_mt if mt else lib().ko_matmul_backward
    fn(_p(a), _p(b), _p(g), _p(da) if da is not None else None, _p(db) if db is not None else None,
       _sz(m), _sz(k), _sz(n))


def matmul_f64(a, b, m, k, n):
    c = np.zeros(m * n, dtype=np.float64)
    lib().ko_matmul_f64(_p(a), _p(b), _p(c), _sz(m), _sz(k), _sz(n))
    return c


def matmul_backward_f64(a, b, g, m, k, n):
    da = np.zeros(m * k, dtype=np.float64)
    db = np.zeros(k * n, dtype=np.float64)
    lib().ko_matmul_backward_f64(_p(a), _p(b), _p(g), _p(da), _p(db), _sz(m), _sz(k), _sz(n))
    return da, db


def splitmix_weights(seed, count, fan_in):
    out = np.zeros(count, dtype=np.float32)
    lib().ko_splitmix_weights(ctypes.c_uint64(seed & USIZE_MAX), _sz(count), _sz(fan_in), _p(out))
    return out


# ---------------------------------------------------------------------------
# graph (tensor.rs:85-449)
# ---------------------------------------------------------------------------
class Op:
    """tensor.rs:85-93.  Conv2D carries (stride, padding); equality is by value."""

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
        """bias / relu: not in the reference (docs/roadmap.md:18-26 lists them as planned); they
        restate the device mirror's extension with the textbook definitions."""
        return Op("Conv2D", stride, padding, bias, relu)


Op.Leaf, Op.Add, Op.Mul, Op.Matmul, Op.Sum, Op.Reshape = (
    Op(k) for k in ("Leaf", "Add", "Mul", "Matmul", "Sum", "Reshape"))


class GradBorrow:
    """Stand-in for the Ref guard returned by Tensor::grad (tensor.rs:200-206):
    while one is alive, backward and zero_grad fail with GradientBorrowed."""

    def __init__(self, node):
        self._node = node
        node._borrows += 1
        self.value = node._grad

    def release(self):
        if self._node is not None:
            self._node._borrows -= 1
            self._node = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.release()


class Tensor:
    """One graph node; Python object identity plays the part of Rc identity."""

    def __init__(self, data, shape):
        shape = [int(d) for d in shape]
        expected = element_count(shape)
        data = _f32(data)
        if data.size != expected:
            raise DataLength(expected, data.size)
        self._init(data, shape, Op.Leaf, [])

    def _init(self, data, shape, op, parents):
        self._data, self._shape, self._op, self._parents = data, list(shape), op, list(parents)
        self._grad = None
        self._borrows = 0

    @classmethod
    def _node(cls, data, shape, op, parents):
        t = cls.__new__(cls)
        t._init(data, shape, op, parents)
        return t

    @classmethod
    def zeros(cls, shape):
        shape = [int(d) for d in shape]
        return cls._node(np.zeros(element_count(shape), dtype=np.float32), shape, Op.Leaf, [])

    def clone(self):
        return self

    def shape(self):
        return list(self._shape)

    def data(self):
        return self._data

    def rank(self):
        return len(self._shape)

    def numel(self):
        return int(self._data.size)

    def op(self):
        return self._op

    def parents(self):
        return list(self._parents)

    def grad(self):
        """Copy of the stored gradient or None (the reference hands out a guard;
        use borrow_grad() to hold one)."""
        return None if self._grad is None else self._grad.copy()

    def borrow_grad(self):
        return GradBorrow(self)

    def zero_grad(self):
        if self._borrows:
            raise GradientBorrowed()
        self._grad = None

    # tensor.rs:217-240
    def _elementwise(self, rhs, op):
        if self._shape != rhs._shape:
            raise ShapeMismatch()
        out = np.zeros(self.numel(), dtype=np.float32)
        (lib().ko_add if op == Op.Add else lib().ko_mul)(_p(self._data), _p(rhs._data), _p(out), _sz(out.size))
        return Tensor._node(out, self._shape, op, [self, rhs])

    def add(self, rhs):
        return self._elementwise(rhs, Op.Add)

    def mul(self, rhs):
        return self._elementwise(rhs, Op.Mul)

    # tensor.rs:243-247
    def sum(self):
        total = lib().ko_sum(_p(self._data), _sz(self.numel()))
        return Tensor._node(np.array([total], dtype=np.float32), [], Op.Sum, [self])

    # tensor.rs:250-280
    def matmul(self, rhs):
        if self.rank() != 2 or rhs.rank() != 2:
            raise RankMismatch(self.rank(), rhs.rank())
        m, k, n = self._shape[0], self._shape[1], rhs._shape[1]
        if k != rhs._shape[0]:
            raise MatmulMismatch(k, rhs._shape[0])
        count = element_count([m, n])
        data = matmul(self._data, rhs._data, m, k, n) if count else np.zeros(0, dtype=np.float32)
        return Tensor._node(data, [m, n], Op.Matmul, [self, rhs])

    def reshape(self, shape):
        """Not in the reference (it has no view op): same flat data, new shape,
        VJP passes the gradient through.  Mirrors the extension of the device mirror."""
        shape = [int(d) for d in shape]
        count = element_count(shape)
        if count != self.numel():
            raise DataLength(self.numel(), count)
        return Tensor._node(self._data, shape, Op.Reshape, [self])

    def sgd_step(self, lr):
        """Not in the reference (docs/roadmap.md:21-22 plans it): data[i] -= fl(lr * grad[i]) in place,
        the multiply rounded to f32 before the subtraction."""
        if self._borrows:
            raise GradientBorrowed()
        if self._grad is None:
            raise TensorError("sgd_step needs a gradient: run backward first")
        step = (np.float32(lr) * self._grad).astype(np.float32)
        self._data -= step

    # tensor.rs:288-306
    def _topological_order(self):
        order, visited, stack = [], set(), [(self, False)]
        while stack:
            node, expanded = stack.pop()
            if expanded:
                order.append(node)
                continue
            if id(node) in visited:
                continue
            visited.add(id(node))
            stack.append((node, True))
            for parent in reversed(node._parents):
                stack.append((parent, False))
        return order

    # tensor.rs:309-314
    def backward(self):
        if self.numel() != 1:
            raise NonScalarBackward()
        self.backward_with([1.0])

    # tensor.rs:320-362
    def backward_with(self, seed):
        seed = _f32(seed)
        if seed.size != self.numel():
            raise DataLength(self.numel(), seed.size)
        order = self._topological_order()
        pending = {id(node): np.zeros(node.numel(), dtype=np.float32) for node in order}
        pending[id(self)][:] = seed
        for node in reversed(order):
            _op_backward(node, pending[id(node)], pending)
        for node in order:
            if node._borrows:
                raise GradientBorrowed()
        for node in order:
            gradient = pending[id(node)]
            if node._grad is not None:
                lib().ko_axpy_acc(_p(node._grad), _p(gradient), _sz(gradient.size))
            else:
                node._grad = gradient


def _op_backward(node, g, pending):
    """tensor.rs:365-449."""
    op = node._op
    if op == Op.Leaf:
        return
    if op.kind == "Conv2D":
        x, w = node._parents[0], node._parents[1]
        if op.relu:  # the gradient passes where the activation did (y > 0)
            g = np.where(node._data > 0, g, np.float32(0)).astype(np.float32)
        if op.bias:  # d bias[k] = sum over images, then rows, then columns, of g[:, k, :, :], f32 left to right
            cout = node._shape[1]
            planes = g.reshape(node._shape[0], cout, -1)
            db = np.zeros(cout, dtype=np.float32)
            for k in range(cout):
                db[k] = lib().ko_sum(_p(np.ascontiguousarray(planes[:, k, :].reshape(-1))), _sz(planes.shape[0] * planes.shape[2]))
            target = pending[id(node._parents[2])]
            lib().ko_axpy_acc(_p(target), _p(db), _sz(target.size))
        dx, dw = backward_buffers(x, w, g, op.stride, op.padding)
        for parent, gradient in zip((x, w), (dx, dw)):
            target = pending[id(parent)]
            lib().ko_axpy_acc(_p(target), _p(gradient), _sz(target.size))
    elif op in (Op.Add, Op.Mul):
        for side in range(2):
            parent, other = node._parents[side], node._parents[1 - side]
            target = pending[id(parent)]
            if op == Op.Add:
                lib().ko_axpy_acc(_p(target), _p(g), _sz(target.size))
            else:
                lib().ko_mul_acc(_p(target), _p(g), _p(other._data), _sz(target.size))
    elif op == Op.Sum:
        target = pending[id(node._parents[0])]
        lib().ko_bcast_acc(_p(target), _p(g), _sz(target.size))
    elif op == Op.Reshape:
        target = pending[id(node._parents[0])]
        lib().ko_axpy_acc(_p(target), _p(g), _sz(target.size))
    elif op == Op.Matmul:
        a, b = node._parents
        m, k, n = a._shape[0], a._shape[1], b._shape[1]
        if g.size == 0 or k == 0:
            return
        matmul_backward(a._data, b._data, g, pending[id(a)], None, m, k, n)
        matmul_backward(a._data, b._data, g, None, pending[id(b)], m, k, n)
    else:
        raise AssertionError(op)


# ---------------------------------------------------------------------------
# Conv2D layer (conv2d.rs)
# ---------------------------------------------------------------------------
def _validate_weights(shape, stride):
    """conv2d.rs:156-166"""
    if len(shape) != 4 or 0 in shape:
        raise InvalidConv("weights must have positive OIHW dimensions")
    if stride == 0:
        raise InvalidConv("stride must be positive")


def _check_padding(padding):
    if padding * 2 > USIZE_MAX:
        raise ShapeOverflow()


class Geometry:
    """conv2d.rs:183-224"""

    def __init__(self, input, weights, stride, padding):
        _validate_weights(weights._shape, stride)
        if input.rank() != 4:
            raise InvalidConv("input must be rank 4 (NCHW)")
        x, k = input._shape, weights._shape
        if x[1] != k[1] or x[2] == 0 or x[3] == 0:
            raise InvalidConv("input channels must match weights; H and W must be positive")
        element_count(x[1:])
        pad2 = padding * 2
        if pad2 > USIZE_MAX:
            raise ShapeOverflow()

        def output_dim(size, kernel):
            padded = size + pad2
            if padded > USIZE_MAX:
                raise ShapeOverflow()
            if padded < kernel:
                raise InvalidConv("kernel exceeds padded input")
            out = (padded - kernel) // stride + 1
            if out > USIZE_MAX:
                raise ShapeOverflow()
            return out

        self.oh, self.ow = output_dim(x[2], k[2]), output_dim(x[3], k[3])
        element_count([k[0], self.oh, self.ow])
        element_count([x[0], k[0], self.oh, self.ow])
        self.batch, self.cin, self.cout = x[0], x[1], k[0]
        self.h, self.w, self.kh, self.kw = x[2], x[3], k[2], k[3]
        self.stride, self.padding = stride, padding

    def output_shape(self):
        return [self.batch, self.cout, self.oh, self.ow]


def backward_buffers(input, weights, grad, stride, padding):
    """conv2d.rs:269-292"""
    geometry = Geometry(input, weights, stride, padding)
    expected = element_count(geometry.output_shape())
    grad = _f32(grad)
    if grad.size != expected:
        raise DataLength(expected, grad.size)
    return conv2d_backward(input._data, weights._data, grad, input._shape, weights._shape, stride, padding)


class Conv2D:
    def __init__(self, in_channels, out_channels, kernel_size, stride, padding, seed=42):
        """conv2d.rs:25-61 (new == new_seeded with seed 42)."""
        shape = [out_channels, in_channels, kernel_size[0], kernel_size[1]]
        _validate_weights(shape, stride)
        _check_padding(padding)
        count = element_count(shape)
        fan_in = element_count(shape[1:])
        data = splitmix_weights(seed, count, fan_in)
        self._setup(Tensor(data, shape), stride, padding)

    @classmethod
    def new_seeded(cls, in_channels, out_channels, kernel_size, stride, padding, seed):
        return cls(in_channels, out_channels, kernel_size, stride, padding, seed)

    @classmethod
    def from_weights(cls, weights, stride, padding, bias=None, relu=False):
        """conv2d.rs:65-74.  bias (rank 1, one value per output channel) and relu are not in the
        reference: y = max(conv(x, w) + bias[k], 0), each step rounded to f32."""
        _validate_weights(weights._shape, stride)
        _check_padding(padding)
        if bias is not None and bias._shape != [weights._shape[0]]:
            raise InvalidConv("bias must have one value per output channel")
        layer = cls.__new__(cls)
        layer._setup(weights, stride, padding)
        layer._bias, layer._relu = bias, bool(relu)
        return layer

    def bias(self):
        return self._bias

    def relu(self):
        return self._relu

    def _setup(self, weights, stride, padding):
        self._weights, self._stride, self._padding = weights, stride, padding
        self._bias, self._relu = None, False
        self._last_forward = None

    def weights(self):
        return self._weights

    def in_channels(self):
        return self._weights._shape[1]

    def out_channels(self):
        return self._weights._shape[0]

    def kernel_size(self):
        return (self._weights._shape[2], self._weights._shape[3])

    def stride(self):
        return self._stride

    def padding(self):
        return self._padding

    def forward(self, input):
        """conv2d.rs:95-115"""
        geometry = Geometry(input, self._weights, self._stride, self._padding)
        shape = geometry.output_shape()
        if element_count(shape):
            data = conv2d_forward(input._data, self._weights._data, input._shape, self._weights._shape,
                                  self._stride, self._padding)
        else:
            data = np.zeros(0, dtype=np.float32)
        parents = [input, self._weights]
        if self._bias is not None:
            data = (data.reshape(shape[0], shape[1], -1) + self._bias._data.reshape(1, -1, 1)).astype(np.float32).reshape(-1)
            parents.append(self._bias)
        if self._relu:
            data = np.maximum(data, np.float32(0)).astype(np.float32)
        op = Op.Conv2D(self._stride, self._padding, self._bias is not None, self._relu)
        output = Tensor._node(data, shape, op, parents)
        self._last_forward = (input, output)
        return output

    def backward(self, grad_output):
        """conv2d.rs:119-138"""
        if self._last_forward is None:
            raise MissingForward()
        input, output = self._last_forward
        if grad_output._shape != output._shape:
            raise InvalidConv("grad_output must match the output NCHW shape")
        grad = grad_output._data
        if self._relu:
            grad = np.where(output._data > 0, grad, np.float32(0)).astype(np.float32)
        dx, dw = backward_buffers(input, self._weights, grad, self._stride, self._padding)
        return Tensor(dx, input._shape), Tensor(dw, self._weights._shape)

    def get_activation_map(self):
        return None if self._last_forward is None else self._last_forward[1]

    def clear_cache(self):
        self._last_forward = None
