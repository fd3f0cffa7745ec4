"""Operands that are 4-byte but not 16-byte aligned (a caller's view into a larger buffer): every kernel family
either takes them or leaves them to one that does, and the results stay within the bars.  The CUDA-core
stencils once issued 128-bit accesses on such pointers (a misaligned-address fault), and the paired stores
of the strided dX need 8-byte alignment."""
import numpy as np
import pytest

from parity_util import rel_l2

pytestmark = pytest.mark.gpu

CONV_SHAPES = [(2, 3, 32, 32, 16, 3, 3, 1, 1), (2, 3, 30, 36, 64, 3, 3, 1, 1), (1, 64, 15, 17, 40, 3, 3, 2, 1),
               (1, 256, 9, 12, 256, 3, 3, 1, 1), (2, 32, 12, 12, 24, 3, 3, 1, 1)]
MATMUL_SHAPES = [(256, 512, 384), (2100, 516, 2304), (70, 33, 65), (512, 4096, 10)]
# which of the six operands is shifted, by how many floats
OFFSETS = [(1, 0, 0, 0, 0, 0), (0, 2, 0, 0, 0, 0), (0, 0, 3, 0, 0, 0), (0, 0, 0, 1, 0, 0), (0, 0, 0, 0, 2, 0),
           (0, 0, 0, 0, 0, 3), (1, 2, 3, 1, 2, 3)]


class Shifted:
    """Device copies of host arrays placed `offset` floats into their allocations."""

    def __init__(self, ctx):
        self.ctx, self.bases = ctx, []

    def put(self, values, offset):
        buffer = np.zeros(values.size + 4, np.float32)
        buffer[offset:offset + values.size] = values
        base = self.ctx.upload(buffer)
        self.bases.append(base)
        return base + 4 * offset

    def close(self):
        for base in self.bases:
            self.ctx.free(base)


@pytest.mark.parametrize("shape", CONV_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_convolution_with_shifted_operands(ctx, oracle, shape):
    n, c, h, w, k, r, s, stride, pad = shape
    oh, ow = oracle.conv_out_dims(h, w, r, s, stride, pad)
    rng = np.random.default_rng(sum(shape))
    x = rng.standard_normal(n * c * h * w).astype(np.float32)
    wt = rng.standard_normal(k * c * r * s).astype(np.float32)
    g = rng.standard_normal(n * k * oh * ow).astype(np.float32)
    y64 = oracle.conv2d_forward_f64(x, wt, [n, c, h, w], [k, c, r, s], stride, pad)
    dx64, dw64 = oracle.conv2d_backward_f64(x, wt, g, [n, c, h, w], [k, c, r, s], stride, pad)
    for offsets in OFFSETS:
        for mode, bar in ((0, 1e-5), (1, 2e-3)):
            mem = Shifted(ctx)
            ctx.set_precision(mode)
            try:
                px, pw, pg = mem.put(x, offsets[0]), mem.put(wt, offsets[1]), mem.put(g, offsets[2])
                py = mem.put(np.full(g.size, np.nan, np.float32), offsets[3])
                pdx = mem.put(np.full(x.size, np.nan, np.float32), offsets[4])
                pdw = mem.put(np.full(wt.size, np.nan, np.float32), offsets[5])
                ctx.conv2d_fwd(px, pw, py, *shape)
                ctx.conv2d_bwd(px, pw, pg, pdx, pdw, *shape, 0)
                errors = (rel_l2(ctx.download(py, g.size), y64), rel_l2(ctx.download(pdx, x.size), dx64),
                          rel_l2(ctx.download(pdw, wt.size), dw64))
            finally:
                ctx.set_precision(0)
                mem.close()
            assert max(errors) <= bar, (shape, offsets, mode, errors)


@pytest.mark.parametrize("shape", MATMUL_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_matmul_with_shifted_operands(ctx, oracle, shape):
    m, k, n = shape
    rng = np.random.default_rng(m + k + n)
    a = rng.standard_normal(m * k).astype(np.float32)
    b = rng.standard_normal(k * n).astype(np.float32)
    g = rng.standard_normal(m * n).astype(np.float32)
    c64 = oracle.matmul_f64(a, b, m, k, n)
    da64, db64 = oracle.matmul_backward_f64(a, b, g, m, k, n)
    for offsets in OFFSETS:
        for mode, bar in ((0, 1e-5), (1, 2e-3)):
            mem = Shifted(ctx)
            ctx.set_precision(mode)
            try:
                pa, pb, pg = mem.put(a, offsets[0]), mem.put(b, offsets[1]), mem.put(g, offsets[2])
                pc = mem.put(np.full(m * n, np.nan, np.float32), offsets[3])
                pda = mem.put(np.full(m * k, np.nan, np.float32), offsets[4])
                pdb = mem.put(np.full(k * n, np.nan, np.float32), offsets[5])
                ctx.matmul_fwd(pa, pb, pc, m, k, n)
                ctx.matmul_bwd(pa, pb, pg, pda, pdb, m, k, n, 0)
                errors = (rel_l2(ctx.download(pc, m * n), c64), rel_l2(ctx.download(pda, m * k), da64),
                          rel_l2(ctx.download(pdb, k * n), db64))
            finally:
                ctx.set_precision(0)
                mem.close()
            assert max(errors) <= bar, (shape, offsets, mode, errors)
