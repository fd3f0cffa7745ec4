"""Conv2D forward / dX / dW through the C ABI against the CPU oracle
(crates/katsu-core/src/conv2d.rs:95-103, 232-262, 269-292 restated in
oracle/katsu_oracle.c)."""
import numpy as np
import pytest

from katsu_b200 import workloads
from parity_util import REL_L2_TOL, TF32_UNIT, DeviceArrays, assert_parity, rel_l2

pytestmark = pytest.mark.gpu

# (n, c, h, w, k, r, s, stride, pad): odd sizes, rectangular filters, strides
# with remainder, every low-channel count of the stencil path and shapes that
# fall outside it.
SHAPES = [
    (2, 2, 3, 4, 2, 2, 3, 1, 0), (2, 2, 3, 4, 2, 2, 3, 1, 1), (2, 2, 3, 4, 2, 2, 3, 2, 1),
    (1, 1, 3, 3, 1, 2, 2, 1, 0), (1, 1, 1, 1, 1, 1, 1, 1, 0), (3, 5, 9, 7, 6, 3, 3, 2, 1),
    (2, 8, 6, 6, 5, 1, 1, 1, 0), (1, 3, 10, 10, 4, 5, 5, 3, 2), (1, 7, 13, 11, 9, 3, 3, 1, 1),
    (2, 16, 12, 12, 24, 3, 3, 1, 1), (2, 16, 13, 12, 24, 3, 3, 2, 1), (1, 4, 5, 5, 3, 3, 3, 1, 2),
    # tensor-core implicit GEMM: channel counts that are multiples of 4 and >= 16; ragged tiles,
    # strides (parity classes in dX), rectangular and 1x1 / 5x5 filters, a stride larger than the filter
    (1, 32, 20, 20, 64, 3, 3, 1, 1), (2, 64, 15, 17, 40, 3, 3, 2, 1), (1, 20, 9, 9, 36, 5, 5, 1, 2),
    (1, 16, 8, 8, 16, 1, 1, 1, 0), (1, 16, 9, 9, 16, 1, 1, 3, 0), (2, 36, 10, 10, 132, 3, 3, 1, 1),
    (1, 16, 10, 12, 16, 2, 3, 1, 1), (3, 160, 7, 9, 144, 3, 3, 1, 1), (1, 24, 33, 32, 20, 3, 3, 2, 1),
    # narrow layers with more than 64 output channels (three and four 32-channel groups of g in the
    # all-taps dW kernel), and a wide layer whose channel counts fill only part of a 128-wide tile
    (1, 32, 12, 12, 100, 3, 3, 1, 1), (2, 20, 9, 11, 128, 3, 3, 2, 1), (1, 96, 10, 10, 80, 3, 3, 2, 1),
    # stencil path: C in 1..4, 3x3, stride 1, pad 1
    (1, 3, 8, 8, 8, 3, 3, 1, 1), (2, 3, 33, 37, 5, 3, 3, 1, 1), (1, 1, 40, 64, 70, 3, 3, 1, 1),
    (2, 4, 9, 36, 9, 3, 3, 1, 1), (3, 2, 17, 5, 64, 3, 3, 1, 1), (2, 3, 64, 64, 32, 3, 3, 1, 1),
    (1, 3, 31, 224, 64, 3, 3, 1, 1), (5, 3, 7, 3, 130, 3, 3, 1, 1),
    # low-channel tensor-core backward (C <= 3, width a multiple of 4): heights and widths that leave
    # partial 14x28 / 4x32 tiles, channel counts that leave partial 16- and 32-channel chunks, K beyond
    # the dW kernel's 64 (dX on tensor cores, dW on the stencil), every C
    (2, 3, 30, 36, 17, 3, 3, 1, 1), (1, 2, 45, 100, 64, 3, 3, 1, 1), (3, 1, 15, 60, 100, 3, 3, 1, 1),
    (1, 3, 57, 28, 33, 3, 3, 1, 1), (2, 3, 14, 28, 16, 3, 3, 1, 1),
    # three channels with 65..128 output channels: the dX kernel's filter operand takes three or four
    # 8 KiB blocks and it runs with three g stages so that its shared memory still fits the SM
    (1, 3, 16, 32, 96, 3, 3, 1, 1), (2, 3, 30, 36, 128, 3, 3, 1, 1), (1, 2, 20, 40, 80, 3, 3, 1, 1),
    # 256 or more channels on a side: 128 x 256 tiles with drained accumulators (forward when K >= 256, dX when
    # C >= 256), ragged pixel tiles, a stride, and an output-channel count that is not a whole number of
    # 32-channel groups (dW then keeps the kernel that loads operand tiles slab by slab)
    (1, 256, 9, 10, 256, 3, 3, 1, 1), (2, 64, 6, 7, 512, 3, 3, 2, 1), (1, 512, 8, 8, 272, 1, 1, 1, 0),
    # dW with 256-wide input-channel tiles whose second tile is a quarter full, half of an output-channel tile
    (2, 320, 6, 6, 64, 3, 3, 1, 1),
    # contractions of 3 000 .. 5 800 terms with fewer than 256 output channels: forward (C x taps) and dX
    # (K x taps) then take the kernel that folds its accumulators into registers every 192 accumulation steps
    # (the rotating accumulators alone measured 1.1e-5 .. 1.9e-5 on these); the last one also has a stride
    (2, 512, 10, 17, 132, 2, 3, 1, 1), (1, 132, 22, 11, 384, 5, 3, 1, 1), (4, 384, 19, 16, 128, 5, 3, 2, 1),
]


def run_case(ctx, oracle, shape, accumulate, rng):
    n, c, h, w, k, r, s, stride, pad = shape
    xs, ws = [n, c, h, w], [k, c, r, s]
    oh, ow = oracle.conv_out_dims(h, w, r, s, stride, pad)
    x = rng.standard_normal(n * c * h * w).astype(np.float32)
    wt = rng.standard_normal(k * c * r * s).astype(np.float32)
    g = rng.standard_normal(n * k * oh * ow).astype(np.float32)
    y_ref = oracle.conv2d_forward(x, wt, xs, ws, stride, pad, mt=True)
    dx_ref, dw_ref = oracle.conv2d_backward(x, wt, g, xs, ws, stride, pad, mt=True)
    dx0 = rng.standard_normal(dx_ref.size).astype(np.float32)
    dw0 = rng.standard_normal(dw_ref.size).astype(np.float32)
    with DeviceArrays(ctx, x=x, w=wt, g=g, dx=dx0, dw=dw0) as d:
        d.alloc("y", y_ref.size, fill=np.nan)
        if not accumulate:  # stale contents must be overwritten, not read
            ctx.free(d.ptr["dx"]), ctx.free(d.ptr["dw"])
            d.alloc("dx", dx_ref.size, fill=np.nan), d.alloc("dw", dw_ref.size, fill=np.nan)
        ctx.conv2d_fwd(d["x"], d["w"], d["y"], n, c, h, w, k, r, s, stride, pad)
        ctx.conv2d_bwd(d["x"], d["w"], d["g"], d["dx"], d["dw"], n, c, h, w, k, r, s, stride, pad, accumulate)
        y, dx, dw = d.get("y"), d.get("dx"), d.get("dw")
    if accumulate:
        dx_ref, dw_ref = dx_ref + dx0, dw_ref + dw0
    # terms summed per element: y over (c, r, s), dX over (k, r, s), dW over (n, oy, ox)
    return {"y": assert_parity(y, y_ref, c * r * s, what=("y", shape)),
            "dx": assert_parity(dx, dx_ref, k * r * s, what=("dx", shape)),
            "dw": assert_parity(dw, dw_ref, n * oh * ow, what=("dw", shape))}


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("accumulate", [0, 1])
def test_conv_matches_oracle(ctx, oracle, shape, accumulate):
    errors = run_case(ctx, oracle, shape, accumulate, np.random.default_rng(sum(shape) + accumulate))
    for name, err in errors.items():
        assert err <= REL_L2_TOL, (name, err, shape)


@pytest.mark.parametrize("shape", [(2, 32, 14, 14, 48, 3, 3, 1, 1), (1, 64, 16, 16, 32, 3, 3, 2, 1),
                                   (2, 3, 40, 64, 48, 3, 3, 1, 1), (1, 256, 9, 10, 256, 3, 3, 1, 1),
                                   (2, 320, 6, 6, 256, 3, 3, 1, 1)],
                         ids=lambda s: "x".join(map(str, s)))
def test_conv_tf32_mode(ctx, oracle, shape):
    """Opt-in single-pass TF32 mode on the tensor-core path: within 2e-3, and measurably
    coarser than the default split-precision mode (so the switch really selects it)."""
    n, c, h, w, k, r, s, stride, pad = shape
    rng = np.random.default_rng(17)
    xs, ws = [n, c, h, w], [k, c, r, s]
    oh, ow = oracle.conv_out_dims(h, w, r, s, stride, pad)
    x = rng.standard_normal(n * c * h * w).astype(np.float32)
    wt = rng.standard_normal(k * c * r * s).astype(np.float32)
    g = rng.standard_normal(n * k * oh * ow).astype(np.float32)
    y64 = oracle.conv2d_forward_f64(x, wt, xs, ws, stride, pad)
    dx64, dw64 = oracle.conv2d_backward_f64(x, wt, g, xs, ws, stride, pad)
    ctx.set_precision(1)
    try:
        with DeviceArrays(ctx, x=x, w=wt, g=g) as d:
            d.alloc("y", y64.size), d.alloc("dx", x.size), d.alloc("dw", wt.size)
            ctx.conv2d_fwd(d["x"], d["w"], d["y"], n, c, h, w, k, r, s, stride, pad)
            ctx.conv2d_bwd(d["x"], d["w"], d["g"], d["dx"], d["dw"], n, c, h, w, k, r, s, stride, pad, 0)
            errors = (rel_l2(d.get("y"), y64), rel_l2(d.get("dx"), dx64), rel_l2(d.get("dw"), dw64))
    finally:
        ctx.set_precision(0)
    assert max(errors) <= 2e-3, errors
    assert min(errors) > 1e-5, errors


@pytest.mark.parametrize("shape", [s for s in SHAPES if s[1] <= 4 and s[5:] == (3, 3, 1, 1)] + [(2, 32, 12, 12, 24, 3, 3, 1, 1)],
                         ids=lambda s: "x".join(map(str, s)))
def test_conv_fp32_mode_uses_cuda_cores(ctx, oracle, shape):
    """KATSU_MODE_FP32 keeps every contraction on the FP32 pipe (stencil and direct kernels)."""
    ctx.set_precision(2)
    try:
        errors = run_case(ctx, oracle, shape, 0, np.random.default_rng(sum(shape)))
    finally:
        ctx.set_precision(0)
    for name, err in errors.items():
        assert err <= REL_L2_TOL, (name, err, shape)


def test_skipping_one_output_leaves_the_other_unchanged(ctx, oracle):
    n, c, h, w, k, r, s, stride, pad = 2, 3, 20, 36, 16, 3, 3, 1, 1
    rng = np.random.default_rng(5)
    x = rng.standard_normal(n * c * h * w).astype(np.float32)
    wt = rng.standard_normal(k * c * r * s).astype(np.float32)
    g = rng.standard_normal(n * k * h * w).astype(np.float32)
    dx_ref, dw_ref = oracle.conv2d_backward(x, wt, g, [n, c, h, w], [k, c, r, s], stride, pad)
    with DeviceArrays(ctx, x=x, w=wt, g=g) as d:
        d.alloc("dx", dx_ref.size, fill=7.0), d.alloc("dw", dw_ref.size, fill=7.0)
        ctx.conv2d_bwd(d["x"], d["w"], d["g"], d["dx"], 0, n, c, h, w, k, r, s, stride, pad, 0)
        assert rel_l2(d.get("dx"), dx_ref) <= REL_L2_TOL
        assert np.all(d.get("dw") == 7.0)
        ctx.conv2d_bwd(d["x"], d["w"], d["g"], 0, d["dw"], n, c, h, w, k, r, s, stride, pad, 0)
        assert rel_l2(d.get("dw"), dw_ref) <= REL_L2_TOL


def test_results_are_bit_reproducible(ctx):
    """Two runs on the same inputs give identical bits (no atomics, fixed reduction trees)."""
    spec = workloads.CONV["stem_256x3x224"].with_batch(3)
    x, w = workloads.conv_inputs(spec)
    geom = (spec.n, spec.c, spec.h, spec.w, spec.k, spec.r, spec.s, spec.stride, spec.pad)
    y_count = spec.n * spec.k * spec.oh * spec.ow
    with DeviceArrays(ctx, x=x, w=w) as d:
        d.alloc("y", y_count), d.alloc("dx", x.size), d.alloc("dw", w.size)
        runs = []
        for _ in range(2):
            ctx.conv2d_fwd(d["x"], d["w"], d["y"], *geom)
            ctx.conv2d_bwd(d["x"], d["w"], d["y"], d["dx"], d["dw"], *geom, 0)
            runs.append((d.get("y"), d.get("dx"), d.get("dw")))
        for a, b in zip(*runs):
            assert np.array_equal(a, b)


def test_empty_batch(ctx):
    """N = 0 is legal (crates/katsu-core/tests/conv2d.rs:159-167): nothing to write, dW is zero."""
    with DeviceArrays(ctx, w=np.ones(54, np.float32)) as d:
        d.alloc("dw", 54, fill=3.0)
        ctx.conv2d_fwd(0, d["w"], 0, 0, 3, 4, 5, 2, 3, 3, 1, 1)
        ctx.conv2d_bwd(0, d["w"], 0, 0, d["dw"], 0, 3, 4, 5, 2, 3, 3, 1, 1, 0)
        assert np.all(d.get("dw") == 0.0)


def test_bad_arguments_are_refused(ctx):
    from katsu_b200 import cabi

    with DeviceArrays(ctx, x=np.ones(16, np.float32), w=np.ones(9, np.float32)) as d:
        d.alloc("y", 16)
        with pytest.raises(cabi.KatsuCudaError) as info:
            ctx.conv2d_fwd(d["x"], d["w"], d["y"], 1, 1, 4, 4, 1, 3, 3, 0, 1)  # stride 0
        assert info.value.code == cabi.ERR_INVALID_ARG
        with pytest.raises(cabi.KatsuCudaError):
            ctx.conv2d_fwd(d["x"], d["w"], d["y"], 1, 1, 2, 2, 1, 3, 3, 1, 0)  # kernel exceeds input
        ctx.sync()  # the context stays usable


def test_rgb_example_full_size(ctx, oracle):
    """Katsu's RGB example shape, whole tensors, against the single-threaded oracle."""
    spec = workloads.CONV["rgb_example"]
    x, w = workloads.conv_inputs(spec)
    geom = (spec.n, spec.c, spec.h, spec.w, spec.k, spec.r, spec.s, spec.stride, spec.pad)
    y_ref = oracle.conv2d_forward(x, w, spec.x_shape, spec.w_shape, spec.stride, spec.pad)
    g = (y_ref + y_ref).astype(np.float32)
    dx_ref, dw_ref = oracle.conv2d_backward(x, w, g, spec.x_shape, spec.w_shape, spec.stride, spec.pad)
    with DeviceArrays(ctx, x=x, w=w, g=g) as d:
        d.alloc("y", y_ref.size), d.alloc("dx", x.size), d.alloc("dw", w.size)
        ctx.conv2d_fwd(d["x"], d["w"], d["y"], *geom)
        ctx.conv2d_bwd(d["x"], d["w"], d["g"], d["dx"], d["dw"], *geom, 0)
        assert rel_l2(d.get("y"), y_ref) <= REL_L2_TOL
        assert rel_l2(d.get("dx"), dx_ref) <= REL_L2_TOL
        assert rel_l2(d.get("dw"), dw_ref) <= REL_L2_TOL


@pytest.mark.parametrize("name,batch", [("stem_256x3x224", 4), ("cnn_conv1", 8), ("cnn_conv2", 4),
                                        ("wide_128x256x56", 1), ("down_128x128x112_s2", 1)])
def test_named_workloads_at_reduced_batch(ctx, oracle, name, batch):
    """Each named shape, whole tensors, batch cut so the oracle finishes in seconds
    (the reference's cost is linear in N: conv2d.rs:233)."""
    spec = workloads.CONV[name].with_batch(batch)
    x, w = workloads.conv_inputs(spec)
    geom = (spec.n, spec.c, spec.h, spec.w, spec.k, spec.r, spec.s, spec.stride, spec.pad)
    y_ref = oracle.conv2d_forward(x, w, spec.x_shape, spec.w_shape, spec.stride, spec.pad, mt=True)
    g = (y_ref + y_ref).astype(np.float32)
    dx_ref, dw_ref = oracle.conv2d_backward(x, w, g, spec.x_shape, spec.w_shape, spec.stride, spec.pad, mt=True)
    dx64, dw64 = oracle.conv2d_backward_f64(x, w, g, spec.x_shape, spec.w_shape, spec.stride, spec.pad)
    with DeviceArrays(ctx, x=x, w=w, g=g) as d:
        d.alloc("y", y_ref.size), d.alloc("dx", x.size), d.alloc("dw", w.size)
        ctx.conv2d_fwd(d["x"], d["w"], d["y"], *geom)
        ctx.conv2d_bwd(d["x"], d["w"], d["g"], d["dx"], d["dw"], *geom, 0)
        y, dx, dw = d.get("y"), d.get("dx"), d.get("dw")
    assert rel_l2(y, y_ref) <= REL_L2_TOL
    assert rel_l2(dx, dx_ref) <= REL_L2_TOL
    # dW sums N*OH*OW terms per element; the reference's left-to-right f32 sum carries its
    # own rounding noise, so the device result is held to the bar against the exact (f64)
    # sum and to the bar plus that noise against the f32-order oracle.
    noise = rel_l2(dw_ref, dw64)
    assert rel_l2(dw, dw64) <= REL_L2_TOL
    assert rel_l2(dw, dw_ref) <= REL_L2_TOL + noise
    assert rel_l2(dx, dx64) <= REL_L2_TOL


def test_stem_full_size_sampled_and_adjoint(ctx, oracle):
    """The benchmark workload at its full size (x [256,3,224,224]).  The oracle
    cannot run 6.7e10 multiply-adds in test time, so: (1) randomly sampled
    elements of y, dX and dW are recomputed in reference order; (2) the
    size-independent adjoint identities <g, conv(x, w)> == <dX(g), x> == <dW(g), w>
    are checked on the device."""
    spec = workloads.CONV["stem_256x3x224"]
    x, w = workloads.conv_inputs(spec)
    geom = (spec.n, spec.c, spec.h, spec.w, spec.k, spec.r, spec.s, spec.stride, spec.pad)
    y_count = spec.n * spec.k * spec.oh * spec.ow
    rng = np.random.default_rng(11)
    with DeviceArrays(ctx, x=x, w=w) as d:
        d.alloc("y", y_count), d.alloc("g", y_count), d.alloc("dx", x.size), d.alloc("dw", w.size)
        d.alloc("tmp", y_count), d.alloc("s", 1)
        ctx.conv2d_fwd(d["x"], d["w"], d["y"], *geom)
        ctx.call("katsu_cuda_add", d["y"], d["y"], d["g"], y_count)
        ctx.conv2d_bwd(d["x"], d["w"], d["g"], d["dx"], d["dw"], *geom, 0)
        y, dx, dw = d.get("y"), d.get("dx"), d.get("dw")

        def dot(a, b, count):
            ctx.call("katsu_cuda_mul", d[a], d[b], d["tmp"], count)
            ctx.call("katsu_cuda_sum", d["tmp"], d["s"], count)
            return float(d.get("s")[0])

        lhs, via_dx, via_dw = dot("g", "y", y_count), dot("dx", "x", x.size), dot("dw", "w", w.size)
    g = y + y  # exact in f32
    idx_y = rng.integers(0, y_count, 20000)
    y32, y64 = oracle.sample_y(x, w, idx_y, spec.x_shape, spec.w_shape, spec.stride, spec.pad)
    assert rel_l2(y[idx_y], y32) <= REL_L2_TOL
    idx_x = rng.integers(0, x.size, 20000)
    dx32, dx64 = oracle.sample_dx(w, g, idx_x, spec.x_shape, spec.w_shape, spec.stride, spec.pad)
    assert rel_l2(dx[idx_x], dx32) <= REL_L2_TOL
    assert rel_l2(dx[idx_x], dx64) <= REL_L2_TOL
    idx_w = rng.choice(w.size, 48, replace=False)
    dw32, dw64 = oracle.sample_dw(x, g, idx_w, spec.x_shape, spec.w_shape, spec.stride, spec.pad)
    noise = rel_l2(dw32, dw64)  # the reference's own f32 left-fold error over 12.8 M terms
    assert rel_l2(dw[idx_w], dw64) <= REL_L2_TOL
    assert rel_l2(dw[idx_w], dw32) <= REL_L2_TOL + noise
    assert abs(via_dx - lhs) <= 1e-4 * abs(lhs)
    assert abs(via_dw - lhs) <= 1e-4 * abs(lhs)
