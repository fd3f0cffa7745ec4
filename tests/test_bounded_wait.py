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
