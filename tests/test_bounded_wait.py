"""Failure detection without a GPU fault: a device-side wait that nothing satisfies
runs out of its clock budget, the kernel returns, the host reads KATSU_ERR_TIMEOUT from
the context's status word, and the context keeps working."""
import numpy as np
import pytest

from katsu_b200 import cabi
from parity_util import DeviceArrays

pytestmark = pytest.mark.gpu


def test_wait_that_nothing_signals_times_out_and_context_survives(ctx):
    ctx.sync()
    ctx.call("katsu_cuda_selftest_wait_timeout", 2_000_000)  # ~1 ms of SM clocks
    with pytest.raises(cabi.KatsuCudaError) as info:
        ctx.sync()
    assert info.value.code == cabi.ERR_TIMEOUT
    ctx.sync()  # the status word was cleared: no second report
    with DeviceArrays(ctx, a=np.ones(1000, np.float32)) as d:
        d.alloc("out", 1)
        ctx.call("katsu_cuda_sum", d["a"], d["out"], 1000)
        assert float(d.get("out")[0]) == 1000.0


def test_budget_outside_the_allowed_range_is_refused(ctx):
    with pytest.raises(cabi.KatsuCudaError) as info:
        ctx.call("katsu_cuda_selftest_wait_timeout", 10)
    assert info.value.code == cabi.ERR_INVALID_ARG


def test_download_after_a_wait_that_gave_up_reports_it_too(ctx):
    """A caller that fetches results with katsu_cuda_d2h alone (never calling katsu_cuda_sync) must
    not receive the output of a launch whose wait ran out as if it were good."""
    with DeviceArrays(ctx, a=np.ones(16, np.float32)) as d:
        ctx.sync()
        ctx.call("katsu_cuda_selftest_wait_timeout", 2_000_000)
        with pytest.raises(cabi.KatsuCudaError) as info:
            d.get("a")
        assert info.value.code == cabi.ERR_TIMEOUT
        assert np.all(d.get("a") == 1.0)  # reported once; the context is re-armed


def test_elapsed_time_over_a_wait_that_gave_up_is_refused(ctx):
    ctx.sync()
    start, stop = ctx.event(), ctx.event()
    ctx.record(start)
    ctx.call("katsu_cuda_selftest_wait_timeout", 2_000_000)
    ctx.record(stop)
    with pytest.raises(cabi.KatsuCudaError) as info:
        ctx.elapsed_ms(start, stop)
    assert info.value.code == cabi.ERR_TIMEOUT
    ctx.sync()
    ctx.event_destroy(start), ctx.event_destroy(stop)
