"""Several contexts (one stream each) of one device running the low-channel convolution kernels side by side.

Each stream's output must equal, bit for bit, what the same stream produced alone.  The element-wise kernel
between the convolutions is what puts another stream's memory traffic beside the pipelined kernels; without a
proxy fence before a TMA-written shared-memory stage is released for its refill, that timing made the forward
kernel compute whole pixels from the next tile's input window."""
import numpy as np
import pytest

from katsu_b200 import cabi, workloads
from parity_util import assert_parity

pytestmark = pytest.mark.gpu

LANES = 4
REPEATS = 5


def _lanes(spec):
    x, w = workloads.conv_inputs(spec)
    lanes = []
    for i in range(LANES):
        context = cabi.Context(0)
        xi = (x * np.float32(i + 1)).astype(np.float32)  # distinct inputs per stream
        lanes.append((context, context.upload(xi), context.upload(w)))
    return lanes


def _close(lanes, extra):
    for (context, px, pw), pointers in zip(lanes, extra):
        for p in (px, pw, *pointers):
            context.free(p)
        context.close()


def test_forward_beside_other_streams_is_bit_identical(oracle):
    spec = workloads.CONV["stem_256x3x224"].with_batch(16)
    geom = (spec.n, spec.c, spec.h, spec.w, spec.k, spec.r, spec.s, spec.stride, spec.pad)
    y_count = spec.n * spec.k * spec.oh * spec.ow
    lanes = _lanes(spec)
    extra, alone = [], []
    for context, px, pw in lanes:
        py, pg = context.alloc(y_count), context.alloc(y_count)
        context.conv2d_fwd(px, pw, py, *geom)
        context.sync()
        alone.append(context.download(py, y_count).copy())
        extra.append((py, pg))
    # "alone" is itself held to the oracle (sampled elements, reference visiting order), so that a
    # defect which shows with and without neighbours cannot pass as bit-identical
    x, w = workloads.conv_inputs(spec)
    idx = np.random.default_rng(3).integers(0, y_count, 4000)
    for i, y_alone in enumerate(alone):
        xi = (x * np.float32(i + 1)).astype(np.float32)
        y32, _ = oracle.sample_y(xi, w, idx, spec.x_shape, spec.w_shape, spec.stride, spec.pad)
        assert_parity(y_alone[idx], y32, spec.c * 9, what=("forward alone", i))
    try:
        for _ in range(REPEATS):
            for _ in range(3):
                for (context, px, pw), (py, pg) in zip(lanes, extra):
                    context.conv2d_fwd(px, pw, py, *geom)
                    context.call("katsu_cuda_add", py, py, pg, y_count)
            for context, _, _ in lanes:
                context.sync()
            for (context, _, _), (py, _), expect in zip(lanes, extra, alone):
                assert np.array_equal(context.download(py, y_count), expect)
    finally:
        _close(lanes, extra)


def test_backward_beside_other_streams_is_bit_identical(oracle):
    spec = workloads.CONV["stem_256x3x224"].with_batch(16)
    geom = (spec.n, spec.c, spec.h, spec.w, spec.k, spec.r, spec.s, spec.stride, spec.pad)
    x_count = spec.n * spec.c * spec.h * spec.w
    w_count = spec.k * spec.c * spec.r * spec.s
    y_count = spec.n * spec.k * spec.oh * spec.ow
    rng = np.random.default_rng(7)
    g = rng.standard_normal(y_count).astype(np.float32)
    lanes = _lanes(spec)
    extra, alone = [], []
    for context, px, pw in lanes:
        pg, pdx, pdw, ptmp = context.upload(g), context.alloc(x_count), context.alloc(w_count), context.alloc(y_count)
        context.conv2d_bwd(px, pw, pg, pdx, pdw, *geom)
        context.sync()
        alone.append((context.download(pdx, x_count).copy(), context.download(pdw, w_count).copy()))
        extra.append((pg, pdx, pdw, ptmp))
    x, w = workloads.conv_inputs(spec)
    idx_x = np.random.default_rng(4).integers(0, x_count, 4000)
    idx_w = np.random.default_rng(5).choice(w_count, 64, replace=False)
    for i, (dx_alone, dw_alone) in enumerate(alone):
        xi = (x * np.float32(i + 1)).astype(np.float32)
        _, dx64 = oracle.sample_dx(w, g, idx_x, spec.x_shape, spec.w_shape, spec.stride, spec.pad)
        _, dw64 = oracle.sample_dw(xi, g, idx_w, spec.x_shape, spec.w_shape, spec.stride, spec.pad)
        assert_parity(dx_alone[idx_x], dx64, spec.k * 9, what=("dX alone", i))
        assert_parity(dw_alone[idx_w], dw64, spec.n * spec.oh * spec.ow, what=("dW alone", i))
    try:
        for _ in range(REPEATS):
            for _ in range(2):
                for (context, px, pw), (pg, pdx, pdw, ptmp) in zip(lanes, extra):
                    context.conv2d_bwd(px, pw, pg, pdx, pdw, *geom)
                    context.call("katsu_cuda_add", pg, pg, ptmp, y_count)
            for context, _, _ in lanes:
                context.sync()
            for (context, _, _), (_, pdx, pdw, _), (dx_alone, dw_alone) in zip(lanes, extra, alone):
                assert np.array_equal(context.download(pdx, x_count), dx_alone)
                assert np.array_equal(context.download(pdw, w_count), dw_alone)
    finally:
        _close(lanes, extra)


def test_pair_gemms_and_wide_convolutions_side_by_side(oracle):
    """The kernels that run on pairs of thread blocks (large matmuls in both precision modes) and the wide
    implicit-GEMM convolutions, one per stream, all at once: every stream's results equal what it produced
    alone, bit for bit, and the matmul alone is held to the oracle."""
    rng = np.random.default_rng(5)
    m, k, n = 2100, 1024, 2332
    a = rng.standard_normal(m * k).astype(np.float32)
    b = rng.standard_normal(k * n).astype(np.float32)
    conv = (2, 256, 28, 28, 256, 3, 3, 1, 1)
    x = rng.standard_normal(conv[0] * conv[1] * conv[2] * conv[3]).astype(np.float32)
    w = rng.standard_normal(conv[4] * conv[1] * 9).astype(np.float32)
    y_count = conv[0] * conv[4] * conv[2] * conv[3]
    plans = [(0, "gemm"), (1, "gemm"), (0, "conv"), (1, "conv")]
    contexts = [cabi.Context(0) for _ in plans]
    runs, reads, frees = [], [], []
    for context, (mode, what) in zip(contexts, plans):
        context.set_precision(mode)
        if what == "gemm":
            pa, pb, pc = context.upload(a), context.upload(b), context.alloc(m * n)
            runs.append(lambda c=context, pa=pa, pb=pb, pc=pc: c.matmul_fwd(pa, pb, pc, m, k, n))
            reads.append(lambda c=context, pc=pc: c.download(pc, m * n))
            frees.append((pa, pb, pc))
        else:
            px, pw = context.upload(x), context.upload(w)
            py, pdx, pdw = context.alloc(y_count), context.alloc(x.size), context.alloc(w.size)

            def run(c=context, px=px, pw=pw, py=py, pdx=pdx, pdw=pdw):
                c.conv2d_fwd(px, pw, py, *conv)
                c.conv2d_bwd(px, pw, py, pdx, pdw, *conv, 0)

            runs.append(run)
            reads.append(lambda c=context, py=py, pdx=pdx, pdw=pdw: np.concatenate(
                [c.download(py, y_count), c.download(pdx, x.size), c.download(pdw, w.size)]))
            frees.append((px, pw, py, pdx, pdw))
    try:
        alone = []
        for context, run, read in zip(contexts, runs, reads):
            run()
            context.sync()
            alone.append(read())
        assert_parity(alone[0], oracle.matmul_f64(a, b, m, k, n), k, what="3xTF32 matmul alone")
        for _ in range(REPEATS):
            for _ in range(3):
                for run in runs:
                    run()
            for context in contexts:
                context.sync()
            for i, read in enumerate(reads):
                assert np.array_equal(read(), alone[i]), ("stream", i, plans[i])
    finally:
        for context, pointers in zip(contexts, frees):
            for p in pointers:
                context.free(p)
            context.close()
