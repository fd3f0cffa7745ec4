"""Tensors with more than 2^31 elements (the stem layer at N = 700: y and g hold 2.25e9 floats each): the
kernels' index arithmetic is 64-bit where it has to be.  Images are independent in forward and dX, so the last
images of the big call must equal, bit for bit, the same images run alone; dW must equal the sum of chunked
calls to rounding (conv2d.rs:283-290 sums over the batch)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_stem_layer_beyond_two_to_the_31_elements(ctx):
    n, c, h, w, k = 700, 3, 224, 224, 64
    plane = h * w
    assert n * k * plane > 2 ** 31
    rng = np.random.default_rng(0)
    x = rng.standard_normal(n * c * plane).astype(np.float32)
    wt = (rng.standard_normal(k * c * 9) / 5).astype(np.float32)
    px, pw = ctx.upload(x), ctx.upload(wt)
    py, pdx, pdw = ctx.alloc(n * k * plane), ctx.alloc(x.size), ctx.alloc(wt.size)
    tail, chunk = 6, 100
    first = n - tail
    qy, qdx, qdw = ctx.alloc(tail * k * plane), ctx.alloc(tail * c * plane), ctx.alloc(wt.size)
    try:
        ctx.conv2d_fwd(px, pw, py, n, c, h, w, k, 3, 3, 1, 1)
        ctx.conv2d_bwd(px, pw, py, pdx, pdw, n, c, h, w, k, 3, 3, 1, 1, 0)  # upstream gradient = y
        qx = px + 4 * first * c * plane
        ctx.conv2d_fwd(qx, pw, qy, tail, c, h, w, k, 3, 3, 1, 1)
        ctx.conv2d_bwd(qx, pw, qy, qdx, None, tail, c, h, w, k, 3, 3, 1, 1, 0)
        assert np.array_equal(ctx.download(py + 4 * first * k * plane, tail * k * plane), ctx.download(qy, tail * k * plane))
        assert np.array_equal(ctx.download(pdx + 4 * first * c * plane, tail * c * plane), ctx.download(qdx, tail * c * plane))
        ctx.call("katsu_cuda_zero", qdw, wt.size)
        for i in range(0, n, chunk):
            m = min(chunk, n - i)
            ctx.conv2d_bwd(px + 4 * i * c * plane, pw, py + 4 * i * k * plane, None, qdw, m, c, h, w, k, 3, 3, 1, 1, 1)
        whole, chunks = ctx.download(pdw, wt.size), ctx.download(qdw, wt.size)
        assert np.isfinite(whole).all()
        assert np.linalg.norm(whole.astype(np.float64) - chunks) <= 2e-6 * np.linalg.norm(chunks)
    finally:
        for p in (px, pw, py, pdx, pdw, qy, qdx, qdw):
            ctx.free(p)
