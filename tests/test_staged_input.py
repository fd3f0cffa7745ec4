"""A layer's input staged once for its forward and backward calls (katsu_cuda_conv2d_stage and the *_staged
entry points): same bits as the plain calls, which write the channels-innermost copy of x for themselves.
Conv2D caches its input between the two (crates/katsu-core/src/conv2d.rs:104-107, 130-136)."""
import numpy as np
import pytest

from parity_util import DeviceArrays

pytestmark = pytest.mark.gpu

# (n, c, h, w, k, r, s, stride, pad): wide tiles, ragged channels, a stride, a narrow layer
SHAPES = [(2, 64, 15, 17, 40, 3, 3, 2, 1), (1, 256, 9, 10, 256, 3, 3, 1, 1), (2, 32, 12, 12, 24, 3, 3, 1, 1),
          (1, 100, 8, 9, 36, 1, 1, 1, 0)]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("mode", [0, 1], ids=["3xtf32", "tf32"])
def test_staged_calls_match_the_plain_calls_bit_for_bit(ctx, oracle, shape, mode):
    n, c, h, w, k, r, s, stride, pad = shape
    oh, ow = oracle.conv_out_dims(h, w, r, s, stride, pad)
    rng = np.random.default_rng(sum(shape) + mode)
    x = rng.standard_normal(n * c * h * w).astype(np.float32)
    wt = rng.standard_normal(k * c * r * s).astype(np.float32)
    g = rng.standard_normal(n * k * oh * ow).astype(np.float32)
    dims = (n, c, h, w, k, r, s, stride, pad)
    ctx.set_precision(mode)
    try:
        floats = ctx.conv2d_staged_floats(*dims)
        assert floats >= n * c * h * w * (2 if mode == 0 else 1)
        with DeviceArrays(ctx, x=x, w=wt, g=g) as d:
            for name, size in (("y", g.size), ("dx", x.size), ("dw", wt.size), ("y2", g.size), ("dx2", x.size), ("dw2", wt.size)):
                d.alloc(name, size, fill=np.nan)
            d.alloc("staged", floats)
            ctx.conv2d_fwd(d["x"], d["w"], d["y"], *dims)
            ctx.conv2d_bwd(d["x"], d["w"], d["g"], d["dx"], d["dw"], *dims, 0)
            ctx.conv2d_stage(d["x"], d["staged"], n, c, h, w)
            ctx.conv2d_fwd_staged(d["x"], d["staged"], d["w"], None, d["y2"], *dims, 0)
            ctx.conv2d_bwd_staged(d["x"], d["staged"], d["w"], d["g"], None, 1.0, d["dx2"], d["dw2"], *dims, 0)
            for plain, staged in (("y", "y2"), ("dx", "dx2"), ("dw", "dw2")):
                assert np.array_equal(d.get(plain), d.get(staged)), (plain, shape)
            # a null copy is the plain call
            ctx.conv2d_fwd_staged(d["x"], None, d["w"], None, d["y2"], *dims, 0)
            assert np.array_equal(d.get("y"), d.get("y2"))
    finally:
        ctx.set_precision(0)


def test_shapes_that_stage_nothing_report_zero(ctx):
    assert ctx.conv2d_staged_floats(4, 3, 32, 32, 16, 3, 3, 1, 1) == 0     # stem kernels
    assert ctx.conv2d_staged_floats(2, 7, 13, 11, 9, 3, 3, 1, 1) == 0      # direct kernels
    ctx.set_precision(2)
    try:
        assert ctx.conv2d_staged_floats(2, 64, 15, 17, 40, 3, 3, 2, 1) == 0  # FP32 mode: CUDA cores
    finally:
        ctx.set_precision(0)
