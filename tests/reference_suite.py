"""The reference's 19 integration tests, restated once and run against two
implementations of the same surface: the CPU oracle (oracle/katsu_ref.py, so
that the oracle is pinned by the reference's own known answers) and the device
host mirror (katsu_b200, so that the CUDA path meets the same assertions).

Each function takes `K`, a namespace with Tensor, Conv2D, Op and the error
classes, and follows one #[test] of
crates/katsu-core/tests/{conv2d,autograd,tensor}.rs (cited per function).
"""
import numpy as np
import pytest

USIZE_MAX = (1 << 64) - 1
ISIZE_MAX = (1 << 63) - 1


def close(a, b, tolerance):
    """tests/conv2d.rs:5-13"""
    a = np.asarray(a, dtype=np.float32).reshape(-1)
    b = np.asarray(b, dtype=np.float32).reshape(-1)
    assert a.size == b.size
    bound = np.float32(tolerance) * (np.float32(1.0) + np.maximum(np.abs(a), np.abs(b)))
    bad = np.nonzero(~(np.abs(a - b) <= bound))[0]
    assert bad.size == 0, f"element {bad[0]}: {a[bad[0]]} != {b[bad[0]]}"


def eq(a, b):
    assert list(np.asarray(a, dtype=np.float32).reshape(-1)) == [np.float32(v) for v in b]


# ---- tests/conv2d.rs -------------------------------------------------------
def known_forward_and_overlap_gradients(K):
    """tests/conv2d.rs:15-43"""
    x = K.Tensor([float(i) for i in range(1, 10)], [1, 1, 3, 3])
    layer = K.Conv2D.from_weights(K.Tensor([1., 2., 3., 4.], [1, 1, 2, 2]), 1, 0)
    assert layer.get_activation_map() is None
    y = layer.forward(x)
    assert y.shape() == [1, 1, 2, 2]
    eq(y.data(), [37., 47., 67., 77.])
    g = K.Tensor([1.] * 4, y.shape())
    dx, dw = layer.backward(g)
    eq(dx.data(), [1., 3., 2., 4., 10., 6., 3., 7., 4.])
    eq(dw.data(), [12., 16., 24., 28.])
    assert x.grad() is None
    y.sum().backward()
    close(x.grad(), dx.data(), 0.)
    close(layer.weights().grad(), dw.data(), 0.)
    amap = layer.get_activation_map()
    eq(amap.grad(), [1.] * 4)
    layer.clear_cache()
    assert layer.get_activation_map() is None
    with pytest.raises(K.MissingForward):
        layer.backward(g)
    y.sum().backward()
    assert x.grad()[0] == 2.


def finite_differences_input_and_weights(K):
    """tests/conv2d.rs:45-87"""
    f32 = np.float32
    for stride, padding in [(1, 0), (1, 1), (2, 1)]:
        xs, ws = [2, 2, 3, 4], [2, 2, 2, 3]
        xv = np.array([f32(i % 11) * f32(0.07) - f32(0.3) for i in range(48)], dtype=f32)
        wv = np.array([f32(i % 7) * f32(0.09) - f32(0.2) for i in range(24)], dtype=f32)
        x = K.Tensor(xv.copy(), xs)
        layer = K.Conv2D.from_weights(K.Tensor(wv.copy(), ws), stride, padding)
        y = layer.forward(x)
        seed = np.array([f32(i % 5) * f32(0.13) - f32(0.2) for i in range(y.numel())], dtype=f32)
        dx, dw = layer.backward(K.Tensor(seed.copy(), y.shape()))
        y.backward_with(seed)
        close(x.grad(), dx.data(), 1e-6)
        close(layer.weights().grad(), dw.data(), 1e-6)

        def evaluate(data, weights):
            conv = K.Conv2D.from_weights(K.Tensor(weights, ws), stride, padding)
            out = np.asarray(conv.forward(K.Tensor(data, xs)).data(), dtype=f32)
            acc = f32(0.0)
            for v, g in zip(out, seed):  # sequential f32 fold like iter().sum()
                acc = f32(acc + f32(v * g))
            return acc

        for side in range(2):
            analytical = np.asarray(dx.data() if side == 0 else dw.data())
            for i, expected in enumerate(analytical):
                xp, xm, wp, wm = xv.copy(), xv.copy(), wv.copy(), wv.copy()
                eps = f32(0.001)
                if side == 0:
                    xp[i] += eps
                    xm[i] -= eps
                else:
                    wp[i] += eps
                    wm[i] -= eps
                numerical = f32(evaluate(xp, wp) - evaluate(xm, wm)) / f32(f32(2.) * eps)
                close([expected], [numerical], 3e-4)


def reused_layer_keeps_independent_graphs(K):
    """tests/conv2d.rs:89-106"""
    layer = K.Conv2D.from_weights(K.Tensor([2.], [1, 1, 1, 1]), 1, 0)
    a = K.Tensor([3.], [1, 1, 1, 1])
    b = K.Tensor([5.], [1, 1, 1, 1])
    ya = layer.forward(a)
    yb = layer.forward(b)
    ya.add(yb).sum().backward()
    eq(layer.weights().grad(), [8.])
    eq(a.grad(), [2.])
    eq(b.grad(), [2.])
    _, dw = layer.backward(K.Tensor([1.], yb.shape()))
    eq(dw.data(), [5.])
    with pytest.raises(K.TensorError):
        layer.forward(K.Tensor.zeros([1]))
    eq(layer.get_activation_map().data(), [10.])


def shared_operand_and_chained_convolution(K):
    """tests/conv2d.rs:108-116"""
    x = K.Tensor([2.], [1, 1, 1, 1])
    layer = K.Conv2D.from_weights(x.clone(), 1, 0)
    y = layer.forward(x)
    layer.forward(y).sum().backward()
    eq(x.grad(), [12.])


def invalid_shapes_and_overflow(K):
    """tests/conv2d.rs:118-142"""
    for args in [(0, 1, (3, 3), 1, 0), (1, 1, (0, 3), 1, 0), (1, 1, (1, 1), 0, 0)]:
        with pytest.raises(K.TensorError):
            K.Conv2D(*args)
    with pytest.raises(K.TensorError):
        K.Conv2D.from_weights(K.Tensor.zeros([1, 1, 1]), 1, 0)
    with pytest.raises(K.TensorError):
        K.Conv2D(1, 1, (1, 1), 1, USIZE_MAX)
    layer = K.Conv2D(1, 1, (3, 3), 1, 0)
    with pytest.raises(K.MissingForward):
        layer.backward(K.Tensor.zeros([1]))
    for shape in ([1, 2, 3, 3], [1, 1, 2, 2], [1, 1, 0, 2]):
        with pytest.raises(K.TensorError):
            layer.forward(K.Tensor.zeros(shape))
    layer.forward(K.Tensor.zeros([1, 1, 3, 3]))
    with pytest.raises(K.TensorError):
        layer.backward(K.Tensor.zeros([1]))
    huge_pad = K.Conv2D(1, 1, (1, 1), 1, USIZE_MAX // 2)
    with pytest.raises(K.ShapeOverflow):
        huge_pad.forward(K.Tensor.zeros([0, 1, 2, 2]))


def empty_batch_and_seeded_initialization(K):
    """tests/conv2d.rs:144-169"""
    layer = K.Conv2D.new_seeded(3, 2, (3, 3), 1, 1, 7)
    same = K.Conv2D.new_seeded(3, 2, (3, 3), 1, 1, 7)
    other = K.Conv2D.new_seeded(3, 2, (3, 3), 1, 1, 8)
    assert np.array_equal(layer.weights().data(), same.weights().data())
    assert not np.array_equal(layer.weights().data(), other.weights().data())
    assert np.all(np.abs(layer.weights().data()) <= np.float32(1.) / np.sqrt(np.float32(27.)))
    x = K.Tensor.zeros([0, 3, 4, 5])
    y = layer.forward(x)
    assert y.shape() == [0, 2, 4, 5]
    y.sum().backward()
    assert len(x.grad()) == 0
    assert np.all(np.asarray(layer.weights().grad()) == 0.)


def known_stride_and_padding(K):
    """tests/conv2d.rs:171-179"""
    x = K.Tensor([float(i) for i in range(1, 10)], [1, 1, 3, 3])
    layer = K.Conv2D.from_weights(K.Tensor([1., 2., 3., 4.], [1, 1, 2, 2]), 2, 1)
    y = layer.forward(x)
    assert y.shape() == [1, 1, 2, 2]
    eq(y.data(), [4., 18., 36., 77.])


# ---- tests/autograd.rs -----------------------------------------------------
def squared_error_shared_nodes_and_repeated_backward(K):
    """tests/autograd.rs:7-28"""
    a = K.Tensor([1., 2.], [2])
    b = K.Tensor([3., 4.], [2])
    s = a.add(b)
    loss = s.mul(s).sum()
    assert s.op() == K.Op.Add
    assert len(s.parents()) == 2
    assert a.grad() is None
    loss.backward()
    eq(loss.data(), [52.])
    eq(a.grad(), [8., 12.])
    eq(b.grad(), [8., 12.])
    eq(s.grad(), [8., 12.])
    loss.backward()
    eq(a.grad(), [16., 24.])
    a.zero_grad()
    loss.backward()
    eq(a.grad(), [8., 12.])
    eq(b.grad(), [24., 36.])


def diamond_and_clone_identity(K):
    """tests/autograd.rs:30-39"""
    x = K.Tensor([2.], [])
    alias = x.clone()
    square = x.mul(alias)
    square.add(square.mul(x)).backward()
    eq(alias.grad(), [16.])
    eq(square.grad(), [3.])


def explicit_seed_and_errors_are_atomic(K):
    """tests/autograd.rs:41-60"""
    x = K.Tensor([2., 3.], [2])
    y = x.mul(x)
    with pytest.raises(K.NonScalarBackward):
        y.backward()
    with pytest.raises(K.DataLength):
        y.backward_with([1.])
    borrowed = x.borrow_grad()
    with pytest.raises(K.GradientBorrowed):
        y.backward_with([2., 4.])
    assert y.grad() is None
    borrowed.release()
    y.backward_with([2., 4.])
    eq(x.grad(), [8., 24.])


def matmul_finite_differences(K):
    """tests/autograd.rs:62-95"""
    f32 = np.float32
    av = np.array([0.2, -0.4, 0.7, 0.3, 0.8, -0.1], dtype=f32)
    bv = np.array([0.1, 0.5, -0.3, 0.6, 0.9, -0.2], dtype=f32)

    def evaluate(a, b):
        y = K.Tensor(a, [2, 3]).matmul(K.Tensor(b, [3, 2]))
        return f32(np.asarray(y.mul(y).sum().data())[0])

    a = K.Tensor(av.copy(), [2, 3])
    b = K.Tensor(bv.copy(), [3, 2])
    y = a.matmul(b)
    y.mul(y).sum().backward()
    for side in range(2):
        analytical = np.asarray(a.grad() if side == 0 else b.grad())
        for i in range(6):
            ap, am, bp, bm = av.copy(), av.copy(), bv.copy(), bv.copy()
            eps = f32(0.001)
            if side == 0:
                ap[i] += eps
                am[i] -= eps
            else:
                bp[i] += eps
                bm[i] -= eps
            numerical = f32(evaluate(ap, bp) - evaluate(am, bm)) / f32(f32(2.) * eps)
            assert abs(analytical[i] - numerical) < 0.001, (side, i, analytical[i], numerical)


def matmul_same_parent_accumulates_both_edges(K):
    """tests/autograd.rs:97-103"""
    a = K.Tensor([1., 2., 3., 4.], [2, 2])
    a.matmul(a).sum().backward()
    eq(a.grad(), [7., 11., 9., 13.])


def empty_graph_operations(K):
    """tests/autograd.rs:105-116"""
    a = K.Tensor.zeros([2, 0])
    b = K.Tensor.zeros([0, 3])
    a.matmul(b).sum().backward()
    assert len(a.grad()) == 0
    assert len(b.grad()) == 0
    x = K.Tensor.zeros([0])
    x.mul(x).add(x).sum().backward()
    assert len(x.grad()) == 0


# ---- tests/tensor.rs -------------------------------------------------------
def validates_data_and_storage_size(K):
    """tests/tensor.rs:3-17"""
    with pytest.raises(K.DataLength):
        K.Tensor([1.0], [2])
    with pytest.raises(K.ShapeOverflow):
        K.Tensor.zeros([USIZE_MAX, 2])
    with pytest.raises(K.ShapeOverflow):
        K.Tensor.zeros([ISIZE_MAX])


def scalar_and_empty_shapes(K):
    """tests/tensor.rs:19-25"""
    assert K.Tensor([3.0], []).rank() == 0
    eq(K.Tensor.zeros([]).data(), [0.0])
    assert K.Tensor.zeros([USIZE_MAX, 0]).numel() == 0


def addition_preserves_inputs(K):
    """tests/tensor.rs:27-38"""
    a = K.Tensor([1.0, 2.0], [2])
    b = K.Tensor([3.0, 4.0], [2])
    eq(a.add(b).data(), [4.0, 6.0])
    eq(a.data(), [1.0, 2.0])
    with pytest.raises(K.ShapeMismatch):
        a.add(K.Tensor.zeros([1, 2]))


def rectangular_matmul(K):
    """tests/tensor.rs:40-48"""
    a = K.Tensor([1., 2., 3., 4., 5., 6.], [2, 3])
    b = K.Tensor([7., 8., 9., 10., 11., 12.], [3, 2])
    c = a.matmul(b)
    assert c.shape() == [2, 2]
    eq(c.data(), [58., 64., 139., 154.])


def rejects_invalid_matmul(K):
    """tests/tensor.rs:50-62"""
    a = K.Tensor.zeros([2, 3])
    with pytest.raises(K.MatmulMismatch):
        a.matmul(K.Tensor.zeros([2, 2]))
    with pytest.raises(K.RankMismatch):
        a.matmul(K.Tensor.zeros([3]))


def empty_matmul_and_output_overflow(K):
    """tests/tensor.rs:64-86"""
    c = K.Tensor.zeros([2, 0]).matmul(K.Tensor.zeros([0, 3]))
    assert c.shape() == [2, 3]
    eq(c.data(), [0.] * 6)
    assert K.Tensor.zeros([0, 2]).matmul(K.Tensor.zeros([2, 3])).shape() == [0, 3]
    assert K.Tensor.zeros([USIZE_MAX, 0]).matmul(K.Tensor.zeros([0, 0])).numel() == 0
    with pytest.raises(K.ShapeOverflow):
        K.Tensor.zeros([USIZE_MAX, 0]).matmul(K.Tensor.zeros([0, 2]))


ALL = [
    known_forward_and_overlap_gradients,
    finite_differences_input_and_weights,
    reused_layer_keeps_independent_graphs,
    shared_operand_and_chained_convolution,
    invalid_shapes_and_overflow,
    empty_batch_and_seeded_initialization,
    known_stride_and_padding,
    squared_error_shared_nodes_and_repeated_backward,
    diamond_and_clone_identity,
    explicit_seed_and_errors_are_atomic,
    matmul_finite_differences,
    matmul_same_parent_accumulates_both_edges,
    empty_graph_operations,
    validates_data_and_storage_size,
    scalar_and_empty_shapes,
    addition_preserves_inputs,
    rectangular_matmul,
    rejects_invalid_matmul,
    empty_matmul_and_output_overflow,
]

# The subset that only exercises validation and never reaches arithmetic; it
# must pass on a machine without a GPU for the device mirror too.
NO_DEVICE = [
    validates_data_and_storage_size,
    rejects_invalid_matmul,
]
