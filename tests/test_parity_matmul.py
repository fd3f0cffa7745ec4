"""Tensor::matmul and its VJP through the C ABI against the oracle
(crates/katsu-core/src/tensor.rs:264-273, 418-445)."""
import numpy as np
import pytest

from katsu_b200 import workloads
from parity_util import REL_L2_TOL, TF32_UNIT, DeviceArrays, assert_parity, max_abs_bound, rel_l2

pytestmark = pytest.mark.gpu

SHAPES = [(2, 3, 2), (1, 1, 1), (70, 33, 65), (64, 64, 64), (129, 17, 200), (37, 2100, 10), (5, 4099, 3),
          (66, 2048, 16), (33, 4096, 1), (3, 5000, 17), (200, 300, 12),
          # tensor-core tiles: full and ragged in every dimension, long K (split-K)
          (128, 128, 128), (256, 512, 384), (200, 260, 132), (1000, 96, 520), (64, 4100, 36), (130, 36, 4096),
          # 256-row tiles on pairs of thread blocks: odd pair count with a ragged last pair, ragged N, split K
          (384, 4100, 200), (256, 8192, 128), (700, 64, 1000)]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("accumulate", [0, 1])
def test_matmul_matches_oracle(ctx, oracle, shape, accumulate):
    m, k, n = shape
    rng = np.random.default_rng(m * 7 + k * 3 + n + accumulate)
    a = rng.standard_normal(m * k).astype(np.float32)
    b = rng.standard_normal(k * n).astype(np.float32)
    g = rng.standard_normal(m * n).astype(np.float32)
    c_ref = oracle.matmul(a, b, m, k, n, mt=True)
    da0 = rng.standard_normal(m * k).astype(np.float32) if accumulate else np.zeros(m * k, np.float32)
    db0 = rng.standard_normal(k * n).astype(np.float32) if accumulate else np.zeros(k * n, np.float32)
    da_ref, db_ref = da0.copy(), db0.copy()
    oracle.matmul_backward(a, b, g, da_ref, db_ref, m, k, n, mt=True)
    with DeviceArrays(ctx, a=a, b=b, g=g) as d:
        d.alloc("c", m * n, fill=np.nan)
        if accumulate:
            d.ptr["da"], d.ptr["db"] = ctx.upload(da0), ctx.upload(db0)
            d.size["da"], d.size["db"] = m * k, k * n
        else:
            d.alloc("da", m * k, fill=np.nan), d.alloc("db", k * n, fill=np.nan)
        ctx.matmul_fwd(d["a"], d["b"], d["c"], m, k, n)
        ctx.matmul_bwd(d["a"], d["b"], d["g"], d["da"], d["db"], m, k, n, accumulate)
        # terms per element: c over k, dA over n, dB over m
        assert_parity(d.get("c"), c_ref, k, what=("c", shape))
        assert_parity(d.get("da"), da_ref, n, what=("da", shape))
        assert_parity(d.get("db"), db_ref, m, what=("db", shape))


@pytest.mark.parametrize("size", [2, 48, 128, 200])
@pytest.mark.parametrize("accumulate", [0, 1])
def test_same_buffer_for_both_gradients(ctx, oracle, size, accumulate):
    """a.matmul(&a): both edges of the Matmul node lead to the same parent and its adjoint receives
    g @ b^T and a^T @ g (crates/katsu-core/src/tensor.rs:425-444, tests/autograd.rs:98-103).  With
    da == db one call delivers that sum, on top of the old contents only when accumulate != 0."""
    rng = np.random.default_rng(size + accumulate)
    a = rng.standard_normal(size * size).astype(np.float32)
    g = rng.standard_normal(size * size).astype(np.float32)
    start = rng.standard_normal(size * size).astype(np.float32)
    expect = start.copy() if accumulate else np.zeros(size * size, np.float32)
    oracle.matmul_backward(a, a, g, expect, expect, size, size, size)
    with DeviceArrays(ctx, a=a, g=g, d=start) as d:
        ctx.matmul_bwd(d["a"], d["a"], d["g"], d["d"], d["d"], size, size, size, accumulate)
        assert_parity(d.get("d"), expect, 2 * size, what=("same parent", size, accumulate))


@pytest.mark.parametrize("shape", [(1100, 2080, 2304), (1152, 520, 2332), (200, 96, 19200)],
                         ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("accumulate", [0, 1])
def test_large_single_pass_tf32(ctx, oracle, shape, accumulate):
    """Shapes with at least one 128 x 256 tile per two SMs take the single-pass kernels that read both operands
    from shared memory (256 x 256 tiles on pairs of thread blocks when there are 256 rows or more, else
    128 x 256): all four operand layouts (c: K-major x MN-major, dA: K x K, dB: MN x MN), ragged edges in
    every dimension, an N that is not a whole number of 32-column groups (second shape), and fewer than 256
    rows (third shape: the one-block kernel)."""
    m, k, n = shape
    rng = np.random.default_rng(m + k + n + accumulate)
    a = rng.standard_normal(m * k).astype(np.float32)
    b = rng.standard_normal(k * n).astype(np.float32)
    g = rng.standard_normal(m * n).astype(np.float32)
    c0 = rng.standard_normal(m * n).astype(np.float32)
    da0 = rng.standard_normal(m * k).astype(np.float32) if accumulate else np.zeros(m * k, np.float32)
    db0 = rng.standard_normal(k * n).astype(np.float32) if accumulate else np.zeros(k * n, np.float32)
    c64 = oracle.matmul_f64(a, b, m, k, n)
    da64, db64 = oracle.matmul_backward_f64(a, b, g, m, k, n)
    ctx.set_precision(1)
    try:
        with DeviceArrays(ctx, a=a, b=b, g=g, c=c0, da=da0, db=db0) as d:
            ctx.matmul_fwd(d["a"], d["b"], d["c"], m, k, n)
            ctx.matmul_bwd(d["a"], d["b"], d["g"], d["da"], d["db"], m, k, n, accumulate)
            c, da, db = d.get("c"), d.get("da"), d.get("db")
    finally:
        ctx.set_precision(0)
    errors = (rel_l2(c, c64), rel_l2(da, da0.astype(np.float64) + da64), rel_l2(db, db0.astype(np.float64) + db64))
    assert max(errors) <= 2e-3, errors
    assert min(errors) > 1e-5, errors  # really one TF32 pass
    # per-element bound with the TF32 unit roundoff
    for got, ref, terms in ((c, c64, k), (da, da0 + da64, n), (db, db0 + db64, m)):
        assert np.max(np.abs(got - ref)) <= max_abs_bound(ref, terms, unit=TF32_UNIT, sqrt_terms=False)


@pytest.mark.parametrize("accumulate", [0, 1])
def test_large_split_precision(ctx, oracle, accumulate):
    """At least one 256 x 256 tile per pair of SMs in the default mode: the kernel that reads both operands and
    their lo halves from shared memory on pairs of thread blocks, with alternating drained accumulators.  All
    three products of this shape take it (K-major x MN-major, K x K, MN x MN); N is ragged and not a whole
    number of 32-column groups.  Held to the 1e-5 bar against the exact (f64) products."""
    m, k, n = 2100, 2304, 2332
    rng = np.random.default_rng(77 + accumulate)
    a = rng.standard_normal(m * k).astype(np.float32)
    b = rng.standard_normal(k * n).astype(np.float32)
    g = rng.standard_normal(m * n).astype(np.float32)
    da0 = rng.standard_normal(m * k).astype(np.float32) if accumulate else np.zeros(m * k, np.float32)
    db0 = rng.standard_normal(k * n).astype(np.float32) if accumulate else np.zeros(k * n, np.float32)
    c64 = oracle.matmul_f64(a, b, m, k, n)
    da64, db64 = oracle.matmul_backward_f64(a, b, g, m, k, n)
    with DeviceArrays(ctx, a=a, b=b, g=g, da=da0, db=db0) as d:
        d.alloc("c", m * n, fill=np.nan)
        ctx.matmul_fwd(d["a"], d["b"], d["c"], m, k, n)
        ctx.matmul_bwd(d["a"], d["b"], d["g"], d["da"], d["db"], m, k, n, accumulate)
        c, da, db = d.get("c"), d.get("da"), d.get("db")
    assert_parity(c, c64, k, what="c")
    assert_parity(da, da0.astype(np.float64) + da64, n, what="da")
    assert_parity(db, db0.astype(np.float64) + db64, m, what="db")


@pytest.mark.parametrize("mode,bar", [(1, 2e-3), (2, REL_L2_TOL)], ids=["tf32", "fp32"])
def test_matmul_precision_modes(ctx, oracle, mode, bar):
    """TF32 mode (one tensor-core pass) holds the 2e-3 bar; FP32 mode stays on CUDA cores."""
    m, k, n = 256, 384, 192
    rng = np.random.default_rng(9)
    a = rng.standard_normal(m * k).astype(np.float32)
    b = rng.standard_normal(k * n).astype(np.float32)
    g = rng.standard_normal(m * n).astype(np.float32)
    c64 = oracle.matmul_f64(a, b, m, k, n)
    da64, db64 = oracle.matmul_backward_f64(a, b, g, m, k, n)
    ctx.set_precision(mode)
    try:
        with DeviceArrays(ctx, a=a, b=b, g=g) as d:
            d.alloc("c", m * n), d.alloc("da", m * k), d.alloc("db", k * n)
            ctx.matmul_fwd(d["a"], d["b"], d["c"], m, k, n)
            ctx.matmul_bwd(d["a"], d["b"], d["g"], d["da"], d["db"], m, k, n, 0)
            errors = (rel_l2(d.get("c"), c64), rel_l2(d.get("da"), da64), rel_l2(d.get("db"), db64))
    finally:
        ctx.set_precision(0)
    assert max(errors) <= bar, errors
    if mode == 1:
        assert max(errors) > 1e-5  # really a single TF32 pass, not the split-precision path


def test_empty_inner_dimension(ctx):
    """k == 0 gives a zero product and leaves the adjoints alone (tensor.rs:265, 421-423)."""
    with DeviceArrays(ctx) as d:
        d.alloc("c", 6, fill=5.0)
        ctx.matmul_fwd(0, 0, d["c"], 2, 0, 3)
        assert np.all(d.get("c") == 0.0)


@pytest.mark.parametrize("m", [64, 512])
def test_classifier_head_shape(ctx, oracle, m):
    """The small CNN's fully connected layer [m,65536] @ [65536,10] at a reduced batch and at the
    configured one (dB = a^T @ g then sums over all 512 batch rows)."""
    k, n = workloads.CNN["fc_in"], workloads.CNN["fc_out"]
    rng = np.random.default_rng(3)
    a = rng.standard_normal(m * k).astype(np.float32)
    b = workloads.cnn_fc_weights()
    g = rng.standard_normal(m * n).astype(np.float32)
    c_ref = oracle.matmul(a, b, m, k, n, mt=True)
    c64 = oracle.matmul_f64(a, b, m, k, n)
    da64, db64 = oracle.matmul_backward_f64(a, b, g, m, k, n)
    with DeviceArrays(ctx, a=a, b=b, g=g) as d:
        d.alloc("c", m * n), d.alloc("da", m * k), d.alloc("db", k * n)
        ctx.matmul_fwd(d["a"], d["b"], d["c"], m, k, n)
        ctx.matmul_bwd(d["a"], d["b"], d["g"], d["da"], d["db"], m, k, n, 0)
        c, da, db = d.get("c"), d.get("da"), d.get("db")
    noise = rel_l2(c_ref, c64)  # 65536-term f32 left fold
    assert_parity(c, c64, k, what="c")
    assert_parity(c, c_ref, k, tol=REL_L2_TOL + noise, what="c vs f32 order")
    assert_parity(da, da64, n, what="da")
    assert_parity(db, db64, m, what="db")
