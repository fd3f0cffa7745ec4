"""The loss sub-graph loss = sum(y * y) evaluated in fused form on the device.

With fusion on (the default) y.mul(y) stores nothing, sum() of it reads y once, and backward hands
the convolution the adjoint "2 * s * y" in symbolic form; the values every node and every gradient
finally shows are those of the reference's node-by-node evaluation
(crates/katsu-core/src/tensor.rs:226-247, 392-417), including the activation map's gradient
(crates/katsu-core/tests/conv2d.rs:31-32).  Checked against node-by-node evaluation on the device
(bit for bit where the arithmetic is the same) and against the oracle graph."""
import numpy as np
import pytest

from katsu_b200 import workloads
from parity_util import assert_parity

pytestmark = pytest.mark.gpu


@pytest.fixture
def K():
    import katsu_b200

    yield katsu_b200
    katsu_b200.set_loss_fusion(True)


def conv_loss_graph(lib, spec, x, w, seed=None):
    t = {"x": lib.Tensor(x, spec.x_shape), "w": lib.Tensor(w, spec.w_shape)}
    layer = lib.Conv2D.from_weights(t["w"], spec.stride, spec.pad)
    t["y"] = layer.forward(t["x"])
    t["q"] = t["y"].mul(t["y"])
    t["loss"] = t["q"].sum()
    if seed is None:
        t["loss"].backward()
    else:
        t["loss"].backward_with([seed])
    t["map"] = layer.get_activation_map()
    return t


SPECS = [workloads.CONV["stem_256x3x224"].with_batch(2),   # tensor-core kernels that scale their outputs
         workloads.CONV["cnn_conv2"].with_batch(2),        # implicit GEMM: the scaled gradient is written out once
         workloads.CONV["rgb_example"]]


@pytest.mark.parametrize("spec", SPECS, ids=lambda s: s.name)
def test_fused_equals_node_by_node_bit_for_bit(K, spec):
    """Seed 1 (loss.backward()): the fused form scales by exactly 2, which commutes with every
    rounding, so all values agree bit for bit with node-by-node evaluation on the device."""
    x, w = workloads.conv_inputs(spec)
    K.set_loss_fusion(False)
    plain = conv_loss_graph(K, spec, x, w)
    plain = {name: (t.data().copy(), t.grad().copy()) for name, t in plain.items()}
    K.set_loss_fusion(True)
    fused = conv_loss_graph(K, spec, x, w)
    for name in ("loss", "x", "w"):  # read before anything forces the lazy nodes to materialise
        assert np.array_equal(fused[name].data(), plain[name][0]), name
        assert np.array_equal(fused[name].grad(), plain[name][1]), name
    assert fused["map"].id() == fused["y"].id()
    assert np.array_equal(fused["map"].grad(), plain["y"][1])  # the activation map's gradient, written out on demand
    assert np.array_equal(fused["q"].grad(), plain["q"][1])    # broadcast of the loss adjoint
    assert np.array_equal(fused["q"].data(), plain["q"][0])    # y * y, computed when asked for
    assert np.array_equal(fused["y"].data(), plain["y"][0])


def test_fused_graph_matches_the_oracle_graph(K, oracle):
    spec = workloads.CONV["stem_256x3x224"].with_batch(2)
    x, w = workloads.conv_inputs(spec)
    dev = conv_loss_graph(K, spec, x, w, seed=0.37)
    ref = conv_loss_graph(oracle, spec, x, w, seed=0.37)
    terms = {"x": spec.k * 9, "w": spec.n * spec.oh * spec.ow, "y": spec.c * 9, "q": 1, "loss": 1}
    for name, count in terms.items():
        assert_parity(dev[name].grad(), ref[name].grad(), count, what=("grad", name))
    assert_parity(dev["y"].data(), ref["y"].data(), spec.c * 9, what="y")
    # the loss is a sum of 6.4 M squares; the device adds them in a tree, the reference left to right
    assert abs(float(dev["loss"].data()[0]) - float(np.sum(ref["y"].data().astype(np.float64) ** 2))) <= 1e-5 * abs(
        float(ref["loss"].data()[0]))


def test_repeated_backward_accumulates_through_the_symbolic_gradients(K, oracle):
    """tests/autograd.rs:8-28: a second backward adds to every stored gradient, also to those the
    first pass left in symbolic form."""
    spec = workloads.CONV["cnn_conv1"].with_batch(1)
    x, w = workloads.conv_inputs(spec)
    dev = conv_loss_graph(K, spec, x, w)
    ref = conv_loss_graph(oracle, spec, x, w)
    dev["loss"].backward()
    ref["loss"].backward()
    for name, count in (("x", spec.k * 9), ("w", spec.oh * spec.ow), ("y", spec.c * 9), ("q", 1), ("loss", 1)):
        assert_parity(dev[name].grad(), ref[name].grad(), count, what=name)
    dev["y"].zero_grad()
    assert dev["y"].grad() is None
    assert dev["map"].grad() is None  # same node


def test_second_consumer_of_y_mixes_symbolic_and_dense_adjoints(K, oracle):
    """loss = sum(y * y) + sum(y): y's adjoint receives the symbolic contribution and a dense one."""
    def graph(lib):
        x = lib.Tensor(np.linspace(-1, 1, 2 * 3 * 8 * 8, dtype=np.float32), [2, 3, 8, 8])
        w = lib.Tensor(np.linspace(-0.5, 0.7, 4 * 3 * 3 * 3, dtype=np.float32), [4, 3, 3, 3])
        y = lib.Conv2D.from_weights(w, 1, 1).forward(x)
        loss = y.mul(y).sum().add(y.sum())
        loss.backward()
        return x, w, y, loss

    dev, ref = graph(K), graph(oracle)
    for got, want, terms in zip(dev, ref, (36, 128, 27, 27 * 512)):
        assert_parity(got.data(), want.data(), 27, what="data")
        assert_parity(got.grad(), want.grad(), terms, what="grad")


def test_sum_of_squares_of_a_leaf_and_sgd_step(K, oracle):
    """Weight decay written as w.mul(w).sum(): the leaf's gradient stays symbolic until sgd_step reads
    it; data -= lr * grad then matches the oracle's in-place update."""
    values = np.linspace(-2, 3, 1003, dtype=np.float32)

    def run(lib):
        w = lib.Tensor(values.copy(), [1003])
        penalty = w.mul(w).sum()
        penalty.backward()
        w.sgd_step(0.125)
        return w, penalty

    (dw, dp), (rw, rp) = run(K), run(oracle)
    assert np.array_equal(dw.data(), rw.data())
    assert np.array_equal(dw.grad(), rw.grad())
    assert abs(float(dp.data()[0]) - float(rp.data()[0])) <= 1e-6 * abs(float(rp.data()[0]))
    fresh = K.Tensor(values, [1003])
    with pytest.raises(K.DeviceError):
        fresh.sgd_step(0.1)  # no gradient yet
    assert np.array_equal(fresh.data(), values)


def test_sumsq_and_square_vjp_through_the_c_abi(ctx):
    """katsu_cuda_sumsq == mul then sum, bit for bit; katsu_cuda_square_vjp == bcast_acc then two mul_acc."""
    from parity_util import DeviceArrays

    rng = np.random.default_rng(12)
    count = 1_000_003
    y = rng.standard_normal(count).astype(np.float32)
    start = rng.standard_normal(count).astype(np.float32)
    with DeviceArrays(ctx, y=y, s=np.array([0.7], np.float32), a=start, b=start) as d:
        d.alloc("q", count), d.alloc("one", 1), d.alloc("two", 1), d.alloc("gq", count)
        ctx.call("katsu_cuda_mul", d["y"], d["y"], d["q"], count)
        ctx.call("katsu_cuda_sum", d["q"], d["one"], count)
        ctx.call("katsu_cuda_sumsq", d["y"], d["two"], count)
        assert d.get("one")[0] == d.get("two")[0]
        ctx.call("katsu_cuda_bcast_acc", d["gq"], d["s"], count)
        for _ in range(2):
            ctx.call("katsu_cuda_mul_acc", d["a"], d["gq"], d["y"], count)
        ctx.call("katsu_cuda_square_vjp", d["b"], d["y"], d["s"], count, 1)
        assert np.array_equal(d.get("a"), d.get("b"))
        ctx.call("katsu_cuda_square_vjp", d["b"] + 4, d["y"] + 4, d["s"], count - 1, 0)  # unaligned, overwrite
        t = np.float32(0.7) * y[1:]
        assert np.array_equal(d.get("b")[1:], (t + t).astype(np.float32))


@pytest.mark.parametrize("name,batch", [("stem_256x3x224", 3), ("cnn_conv2", 2), ("cnn_conv1", 2)])
def test_scaled_backward_through_the_c_abi(ctx, oracle, name, batch):
    """katsu_cuda_conv2d_bwd_scaled(g = y, gscale, gfactor = 2) against the oracle's backward_buffers
    fed the written-out gradient 2 * s * y, overwrite and accumulate."""
    from parity_util import DeviceArrays

    spec = workloads.CONV[name].with_batch(batch)
    x, w = workloads.conv_inputs(spec)
    geom = (spec.n, spec.c, spec.h, spec.w, spec.k, spec.r, spec.s, spec.stride, spec.pad)
    y = oracle.conv2d_forward(x, w, spec.x_shape, spec.w_shape, spec.stride, spec.pad, mt=True)
    s = np.float32(0.3)
    g = (np.float32(2) * (s * y)).astype(np.float32)
    dx64, dw64 = oracle.conv2d_backward_f64(x, w, g, spec.x_shape, spec.w_shape, spec.stride, spec.pad)
    rng = np.random.default_rng(2)
    dx0, dw0 = rng.standard_normal(x.size).astype(np.float32), rng.standard_normal(w.size).astype(np.float32)
    with DeviceArrays(ctx, x=x, w=w, y=y, s=np.array([s], np.float32), dx=dx0, dw=dw0) as d:
        ctx.call("katsu_cuda_conv2d_bwd_scaled", d["x"], d["w"], d["y"], d["s"], 2.0, d["dx"], d["dw"], *geom, 1)
        assert_parity(d.get("dx"), dx64 + dx0, spec.k * 9, what="dx accumulate")
        assert_parity(d.get("dw"), dw64 + dw0, spec.n * spec.oh * spec.ow, what="dw accumulate")
        ctx.call("katsu_cuda_conv2d_bwd_scaled", d["x"], d["w"], d["y"], d["s"], 2.0, d["dx"], d["dw"], *geom, 0)
        assert_parity(d.get("dx"), dx64, spec.k * 9, what="dx")
        assert_parity(d.get("dw"), dw64, spec.n * spec.oh * spec.ow, what="dw")
        ctx.call("katsu_cuda_conv2d_bwd_scaled", d["x"], d["w"], d["y"], 0, 1.0, d["dx"], 0, *geom, 0)  # no scale at all
        dx_plain, _ = oracle.conv2d_backward_f64(x, w, y, spec.x_shape, spec.w_shape, spec.stride, spec.pad)
        assert_parity(d.get("dx"), dx_plain, spec.k * 9, what="dx unscaled")
