"""The NCCL all-reduce entry points through the C ABI on one GPU: a communicator of
one rank must initialise, leave the bucket unchanged (a sum over one rank) and tear
down.  The multi-rank path is exercised by bench.py under torchrun and, for its host
logic, by tests/test_dp_gloo.py on CPU."""
import ctypes

import numpy as np
import pytest

from katsu_b200 import cabi, dp
from parity_util import DeviceArrays

pytestmark = pytest.mark.gpu


def test_single_rank_allreduce_and_bucket(ctx):
    ident = (ctypes.c_uint8 * cabi.COMM_ID_BYTES)()
    cabi.check(ctx.lib.katsu_cuda_comm_unique_id(ident))
    ctx.call("katsu_cuda_comm_init", ident, 1, 0)
    try:
        bucket = dp.GradBucket(ctx, {"conv1": 864, "fc": 1000})
        assert bucket.offsets["fc"] % dp.GradBucket.ALIGN == 0
        a = np.arange(864, dtype=np.float32)
        b = -np.arange(1000, dtype=np.float32)
        ctx.h2d(bucket.ptr("conv1"), a)
        ctx.h2d(bucket.ptr("fc"), b)
        bucket.allreduce()
        assert np.array_equal(bucket.read("conv1"), a)
        assert np.array_equal(bucket.read("fc"), b)
        bucket.free()
    finally:
        ctx.call("katsu_cuda_comm_destroy")


def test_allreduce_without_communicator_is_refused(ctx):
    with DeviceArrays(ctx, a=np.ones(4, np.float32)) as d:
        with pytest.raises(cabi.KatsuCudaError) as info:
            ctx.call("katsu_cuda_allreduce_sum", d["a"], 4)
        assert info.value.code == cabi.ERR_INVALID_ARG
