"""Bias, ReLU and the SGD update on the device.  The reference lists all three as not implemented
yet (docs/roadmap.md:18-26, README.md:53-56); they are checked here against their textbook
definitions restated in the oracle (oracle/katsu_ref.py: y = max(conv(x, w) + b[k], 0), the gradient
passes where y > 0, d b[k] = sum of it over images and pixels, w -= lr * dw)."""
import numpy as np
import pytest

from katsu_b200 import workloads
from parity_util import DeviceArrays, assert_parity

pytestmark = pytest.mark.gpu

# stem: bias and ReLU ride in the tensor-core forward kernel's epilogue; the others take the streaming pass
CASES = [("stem_256x3x224", 2), ("cnn_conv1", 3), ("cnn_conv2", 2), ("rgb_example", 1)]


def layer_graph(lib, spec, x, w, b, relu, upstream):
    t = {"x": lib.Tensor(x, spec.x_shape), "w": lib.Tensor(w, spec.w_shape)}
    t["b"] = lib.Tensor(b, [spec.k]) if b is not None else None
    layer = lib.Conv2D.from_weights(t["w"], spec.stride, spec.pad, bias=t["b"], relu=relu)
    t["y"] = layer.forward(t["x"])
    t["y"].backward_with(upstream)
    t["layer"] = layer
    return t


@pytest.mark.parametrize("name,batch", CASES)
@pytest.mark.parametrize("with_bias,relu", [(True, True), (True, False), (False, True)])
def test_conv_bias_relu_forward_and_gradients(oracle, name, batch, with_bias, relu):
    import katsu_b200 as K

    spec = workloads.CONV[name].with_batch(batch)
    x, w = workloads.conv_inputs(spec)
    rng = np.random.default_rng(spec.k + batch)
    b = rng.uniform(-0.5, 0.5, spec.k).astype(np.float32) if with_bias else None
    upstream = rng.standard_normal(spec.n * spec.k * spec.oh * spec.ow).astype(np.float32)
    dev = layer_graph(K, spec, x, w, b, relu, upstream)
    ref = layer_graph(oracle, spec, x, w, b, relu, upstream)
    assert dev["y"].op() == K.Op.Conv2D(spec.stride, spec.pad, with_bias, relu)
    assert len(dev["y"].parents()) == (3 if with_bias else 2)
    y_dev, y_ref = dev["y"].data(), ref["y"].data()
    assert_parity(y_dev, y_ref, spec.c * 9, what="y")
    if relu:
        assert y_dev.min() >= 0.0 and (y_dev == 0).mean() > 0.2
        # elements within rounding of zero may fall on either side of the clamp on the two machines;
        # the gradient mask follows each side's own y, so those are left out of the gradient check
        # by feeding the oracle's VJP the device's mask
        ref["y"]._data[:] = np.where(y_dev > 0, np.maximum(y_ref, np.float32(1e-30)), np.float32(0))
        for t in (ref["x"], ref["w"], ref["y"]) + ((ref["b"],) if with_bias else ()):
            t.zero_grad()
        ref["y"].backward_with(upstream)
    assert_parity(dev["x"].grad(), ref["x"].grad(), spec.k * 9, what="dx")
    assert_parity(dev["w"].grad(), ref["w"].grad(), spec.n * spec.oh * spec.ow, what="dw")
    if with_bias:
        masked = np.where(y_dev > 0, upstream, 0).astype(np.float64) if relu else upstream.astype(np.float64)
        db64 = masked.reshape(spec.n, spec.k, -1).sum(axis=(0, 2))
        assert_parity(dev["b"].grad(), db64, spec.n * spec.oh * spec.ow, what="db")
    # layer-local VJP (conv2d.rs:119-138) applies the same mask
    dx_local, dw_local = dev["layer"].backward(K.Tensor(upstream, spec.y_shape))
    assert_parity(dx_local.data(), dev["x"].grad(), spec.k * 9, what="local dx")
    assert_parity(dw_local.data(), dev["w"].grad(), spec.n * spec.oh * spec.ow, what="local dw")


def test_bias_shape_is_validated():
    import katsu_b200 as K

    w = K.Tensor(np.ones(4 * 3 * 9, np.float32), [4, 3, 3, 3])
    with pytest.raises(K.InvalidConv):
        K.Conv2D.from_weights(w, 1, 1, bias=K.Tensor(np.ones(5, np.float32), [5]))


def test_training_steps_stay_on_the_device(oracle):
    """Three SGD steps of conv + bias + ReLU under loss = sum(y * y): parameters after every step
    against the oracle running the same steps."""
    import katsu_b200 as K

    spec = workloads.CONV["cnn_conv1"].with_batch(2)
    x, w = workloads.conv_inputs(spec)
    b = np.linspace(-0.2, 0.2, spec.k, dtype=np.float32)

    def train(lib):
        tx, tw, tb = lib.Tensor(x, spec.x_shape), lib.Tensor(w.copy(), spec.w_shape), lib.Tensor(b.copy(), [spec.k])
        losses = []
        for _ in range(3):
            y = lib.Conv2D.from_weights(tw, 1, 1, bias=tb, relu=True).forward(tx)
            loss = y.mul(y).sum()
            loss.backward()
            losses.append(float(loss.data()[0]))
            for p in (tw, tb):
                p.sgd_step(1e-5)
                p.zero_grad()
            tx.zero_grad()
        return tw.data(), tb.data(), losses

    (dw, db, dl), (rw, rb, rl) = train(K), train(oracle)
    assert_parity(dw, rw, 1, tol=2e-5, what="w after 3 steps")
    assert_parity(db, rb, 1, tol=2e-5, what="b after 3 steps")
    assert dl[2] < dl[0] and np.allclose(dl, rl, rtol=1e-4)


def test_c_abi_entry_points(ctx, oracle):
    spec = workloads.CONV["stem_256x3x224"].with_batch(2)
    x, w = workloads.conv_inputs(spec)
    geom = (spec.n, spec.c, spec.h, spec.w, spec.k, spec.r, spec.s, spec.stride, spec.pad)
    rng = np.random.default_rng(8)
    b = rng.standard_normal(spec.k).astype(np.float32)
    y_count, plane = spec.n * spec.k * spec.oh * spec.ow, spec.oh * spec.ow
    g = rng.standard_normal(y_count).astype(np.float32)
    conv = oracle.conv2d_forward(x, w, spec.x_shape, spec.w_shape, spec.stride, spec.pad, mt=True)
    want = np.maximum(conv.reshape(spec.n, spec.k, -1) + b.reshape(1, -1, 1), 0).astype(np.float32).reshape(-1)
    with DeviceArrays(ctx, x=x, w=w, b=b, g=g, db=np.ones(spec.k, np.float32)) as d:
        d.alloc("y", y_count, fill=np.nan), d.alloc("dg", y_count, fill=np.nan)
        ctx.call("katsu_cuda_conv2d_fwd_bias_relu", d["x"], d["w"], d["b"], d["y"], *geom, 1)
        y = d.get("y")
        assert_parity(y, want, 27, what="y")
        ctx.call("katsu_cuda_bias_relu_bwd", d["y"], d["g"], d["dg"], d["db"], spec.n, spec.k, plane, 1, 1)
        masked = np.where(y > 0, g, np.float32(0))
        assert np.array_equal(d.get("dg"), masked)
        assert_parity(d.get("db"), 1.0 + masked.astype(np.float64).reshape(spec.n, spec.k, -1).sum(axis=(0, 2)),
                      spec.n * plane, what="db accumulate")
        ctx.call("katsu_cuda_bias_relu_bwd", 0, d["g"], 0, d["db"], spec.n, spec.k, plane, 0, 0)  # bias only, no mask
        assert_parity(d.get("db"), g.astype(np.float64).reshape(spec.n, spec.k, -1).sum(axis=(0, 2)), spec.n * plane,
                      what="db plain")
        before = d.get("w")
        ctx.call("katsu_cuda_sgd_step", d["w"], d["g"], 0.25, w.size)
        assert np.array_equal(d.get("w"), before - (np.float32(0.25) * g[:w.size]).astype(np.float32))
