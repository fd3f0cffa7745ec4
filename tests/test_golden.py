"""Committed golden vectors (tests/golden/, made by make_golden.py from the
pinned oracle, plus the reference's literal known answers) against the oracle
(CPU) and against the CUDA path through the C ABI (GPU)."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden  # noqa: E402

from parity_util import DeviceArrays, assert_parity  # noqa: E402

GOLDEN = np.load(os.path.join(HERE, "golden", "conv_matmul_golden.npz"))

LITERAL_CONV = {  # crates/katsu-core/tests/conv2d.rs:16-26 and 172-178
    "conv_s1p0": ((1, 1, 3, 3, 1, 2, 2, 1, 0), True),
    "conv_s2p1": ((1, 1, 3, 3, 1, 2, 2, 2, 1), False),
}


@pytest.mark.parametrize("name", sorted(make_golden.CONV_CASES))
def test_oracle_reproduces_conv_golden(oracle, name):
    n, c, h, w, k, r, s, stride, pad, _ = make_golden.CONV_CASES[name]
    x, wt, g = make_golden.conv_inputs(make_golden.CONV_CASES[name])
    assert np.array_equal(oracle.conv2d_forward(x, wt, [n, c, h, w], [k, c, r, s], stride, pad),
                          GOLDEN[f"conv/{name}/y"])
    dx, dw = oracle.conv2d_backward(x, wt, g, [n, c, h, w], [k, c, r, s], stride, pad, mt=True)
    assert np.array_equal(dx, GOLDEN[f"conv/{name}/dx"])  # threaded variant is bit-identical
    assert np.array_equal(dw, GOLDEN[f"conv/{name}/dw"])


@pytest.mark.parametrize("name", sorted(make_golden.MATMUL_CASES))
def test_oracle_reproduces_matmul_golden(oracle, name):
    m, k, n, _ = make_golden.MATMUL_CASES[name]
    a, b, g = make_golden.matmul_inputs(make_golden.MATMUL_CASES[name])
    assert np.array_equal(oracle.matmul(a, b, m, k, n, mt=True), GOLDEN[f"matmul/{name}/c"])


def test_oracle_reproduces_reference_literals(oracle):
    x = np.arange(1, 10, dtype=np.float32)
    w = np.array([1, 2, 3, 4], np.float32)
    for name, (shape, has_grads) in LITERAL_CONV.items():
        n, c, h, wd, k, r, s, stride, pad = shape
        y = oracle.conv2d_forward(x, w, [n, c, h, wd], [k, c, r, s], stride, pad)
        assert np.array_equal(y, GOLDEN[f"literal/{name}/y"])
        if has_grads:
            dx, dw = oracle.conv2d_backward(x, w, np.ones(4, np.float32), [n, c, h, wd], [k, c, r, s], stride, pad)
            assert np.array_equal(dx, GOLDEN[f"literal/{name}/dx"])
            assert np.array_equal(dw, GOLDEN[f"literal/{name}/dw"])
    a = np.arange(1, 7, dtype=np.float32)
    b = np.arange(7, 13, dtype=np.float32)
    assert np.array_equal(oracle.matmul(a, b, 2, 3, 2), GOLDEN["literal/matmul/c"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(make_golden.CONV_CASES))
def test_device_matches_conv_golden(ctx, name):
    n, c, h, w, k, r, s, stride, pad, _ = make_golden.CONV_CASES[name]
    x, wt, g = make_golden.conv_inputs(make_golden.CONV_CASES[name])
    with DeviceArrays(ctx, x=x, w=wt, g=g) as d:
        d.alloc("y", GOLDEN[f"conv/{name}/y"].size), d.alloc("dx", x.size), d.alloc("dw", wt.size)
        ctx.conv2d_fwd(d["x"], d["w"], d["y"], n, c, h, w, k, r, s, stride, pad)
        ctx.conv2d_bwd(d["x"], d["w"], d["g"], d["dx"], d["dw"], n, c, h, w, k, r, s, stride, pad, 0)
        oh, ow = (h + 2 * pad - r) // stride + 1, (w + 2 * pad - s) // stride + 1
        for key, terms in (("y", c * r * s), ("dx", k * r * s), ("dw", n * oh * ow)):
            assert_parity(d.get(key), GOLDEN[f"conv/{name}/{key}"], terms, what=(name, key))


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(make_golden.MATMUL_CASES))
def test_device_matches_matmul_golden(ctx, name):
    m, k, n, _ = make_golden.MATMUL_CASES[name]
    a, b, g = make_golden.matmul_inputs(make_golden.MATMUL_CASES[name])
    with DeviceArrays(ctx, a=a, b=b, g=g) as d:
        d.alloc("c", m * n), d.alloc("da", m * k), d.alloc("db", k * n)
        ctx.matmul_fwd(d["a"], d["b"], d["c"], m, k, n)
        ctx.matmul_bwd(d["a"], d["b"], d["g"], d["da"], d["db"], m, k, n, 0)
        for key, terms in (("c", k), ("da", n), ("db", m)):
            assert_parity(d.get(key), GOLDEN[f"matmul/{name}/{key}"], terms, what=(name, key))


@pytest.mark.gpu
def test_device_matches_reference_literals(ctx):
    """Small integers: the device results are exact, as the reference's assert_eq! demands."""
    x = np.arange(1, 10, dtype=np.float32)
    w = np.array([1, 2, 3, 4], np.float32)
    with DeviceArrays(ctx, x=x, w=w, g=np.ones(4, np.float32)) as d:
        d.alloc("y", 4), d.alloc("dx", 9), d.alloc("dw", 4)
        ctx.conv2d_fwd(d["x"], d["w"], d["y"], 1, 1, 3, 3, 1, 2, 2, 1, 0)
        ctx.conv2d_bwd(d["x"], d["w"], d["g"], d["dx"], d["dw"], 1, 1, 3, 3, 1, 2, 2, 1, 0, 0)
        assert np.array_equal(d.get("y"), GOLDEN["literal/conv_s1p0/y"])
        assert np.array_equal(d.get("dx"), GOLDEN["literal/conv_s1p0/dx"])
        assert np.array_equal(d.get("dw"), GOLDEN["literal/conv_s1p0/dw"])
        ctx.conv2d_fwd(d["x"], d["w"], d["y"], 1, 1, 3, 3, 1, 2, 2, 2, 1)
        assert np.array_equal(d.get("y"), GOLDEN["literal/conv_s2p1/y"])
