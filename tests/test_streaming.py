"""Elementwise / reduction kernels through the C ABI against the oracle
(crates/katsu-core/src/tensor.rs:226-247, 353-356, 387-417)."""
import numpy as np
import pytest

from parity_util import DeviceArrays

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("count", [1, 3, 4, 5, 1023, 4096, 100003, 2_000_001])
def test_elementwise_and_accumulate(ctx, count):
    rng = np.random.default_rng(count)
    a = rng.standard_normal(count).astype(np.float32)
    b = rng.standard_normal(count).astype(np.float32)
    dst = rng.standard_normal(count).astype(np.float32)
    scalar = np.array([0.37], np.float32)
    with DeviceArrays(ctx, a=a, b=b, dst=dst, scalar=scalar) as d:
        d.alloc("out", count, fill=np.nan)
        ctx.call("katsu_cuda_add", d["a"], d["b"], d["out"], count)
        assert np.array_equal(d.get("out"), a + b)
        ctx.call("katsu_cuda_mul", d["a"], d["b"], d["out"], count)
        assert np.array_equal(d.get("out"), a * b)
        ctx.call("katsu_cuda_axpy_acc", d["dst"], d["a"], count)
        expect = dst + a
        assert np.array_equal(d.get("dst"), expect)
        ctx.call("katsu_cuda_mul_acc", d["dst"], d["a"], d["b"], count)
        got = d.get("dst")
        fused = (expect.astype(np.float64) + a.astype(np.float64) * b.astype(np.float64)).astype(np.float32)
        split = expect + a * b
        assert np.all((got == fused) | (got == split))  # fma or mul+add rounding
        expect = got
        ctx.call("katsu_cuda_bcast_acc", d["dst"], d["scalar"], count)
        assert np.array_equal(d.get("dst"), expect + scalar[0])


def test_unaligned_views(ctx):
    """Pointers into the middle of a buffer (a slice of a gradient bucket) take the scalar path."""
    count = 1001
    rng = np.random.default_rng(0)
    a = rng.standard_normal(count + 3).astype(np.float32)
    dst = rng.standard_normal(count + 3).astype(np.float32)
    with DeviceArrays(ctx, a=a, dst=dst) as d:
        ctx.call("katsu_cuda_axpy_acc", d["dst"] + 4, d["a"] + 8, count)
        got = d.get("dst")
        assert np.array_equal(got[1:1 + count], dst[1:1 + count] + a[2:2 + count])
        assert got[0] == dst[0] and np.array_equal(got[1 + count:], dst[1 + count:])


@pytest.mark.parametrize("count", [0, 1, 7, 1024, 99999, 5_000_003])
def test_sum(ctx, oracle, count):
    rng = np.random.default_rng(count)
    a = rng.standard_normal(count).astype(np.float32)
    exact = float(np.sum(a.astype(np.float64)))
    with DeviceArrays(ctx, a=a) as d:
        d.alloc("out", 1, fill=np.nan)
        ctx.call("katsu_cuda_sum", d["a"], d["out"], count)
        got = float(d.get("out")[0])
    scale = float(np.sum(np.abs(a.astype(np.float64)))) + 1e-30
    assert abs(got - exact) <= 1e-6 * scale
    if count:
        # the reference folds left to right in f32; the device tree sum must be at least as close to exact
        ref = float(oracle.lib().ko_sum(oracle._p(a), oracle._sz(count)))
        assert abs(got - exact) <= abs(ref - exact) + 1e-6 * scale


def test_wait_event_orders_two_contexts_of_one_device(ctx):
    """katsu_cuda_wait_event: work queued on a second context after the wait sees what the first
    context queued before the record, without a host synchronisation in between."""
    from katsu_b200 import cabi

    other = cabi.Context(0)
    try:
        n = 1 << 22
        a = ctx.upload(np.full(n, 1.5, np.float32))
        b, c = ctx.alloc(n), ctx.alloc(n)
        ctx.sync()
        ev = ctx.event()
        for _ in range(4):  # a little queue on the first stream
            ctx.call("katsu_cuda_add", a, a, b, n)
        ctx.record(ev)
        other.wait_event(ev)
        other.call("katsu_cuda_add", b, a, c, n)  # must see b = 3.0 everywhere
        out = other.download(c, n)
        assert np.all(out == 4.5)
        ctx.event_destroy(ev)
        for p in (a, b, c):
            ctx.free(p)
    finally:
        other.close()
