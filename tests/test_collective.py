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


@pytest.mark.parametrize("ranks,count", [(2, 1728), (4, 1729), (8, 1728), (8, 16384), (16, 5), (1, 100)])
def test_mailbox_allreduce_with_emulated_ranks(ctx, ranks, count):
    """The small-bucket all-reduce (one kernel per rank exchanging through mailboxes) with every rank
    emulated as one block of a cooperative launch on this device: every rank's bucket ends up holding
    the sum in rank order, bit for bit the same on all of them."""
    rng = np.random.default_rng(ranks * 100 + count)
    buckets = rng.standard_normal((ranks, count)).astype(np.float32)
    expect = np.zeros(count, np.float32)
    for r in range(ranks):
        expect = (expect + buckets[r]).astype(np.float32)
    with DeviceArrays(ctx, buf=buckets.reshape(-1)) as d:
        ctx.call("katsu_cuda_selftest_mailbox_allreduce", d["buf"], ranks, count, 0, 200_000_000)
        ctx.sync()
        out = d.get("buf").reshape(ranks, count)
    for r in range(ranks):
        assert np.array_equal(out[r], expect), r


def test_mailbox_allreduce_gives_up_on_a_rank_that_never_arrives(ctx):
    """Failure detection without a fault: one of four emulated ranks never runs; the others' bounded
    waits run out, the kernel returns, the host reads KATSU_ERR_TIMEOUT and the context works on."""
    from katsu_b200 import cabi

    buckets = np.ones(4 * 64, np.float32)
    with DeviceArrays(ctx, buf=buckets) as d:
        ctx.sync()
        ctx.call("katsu_cuda_selftest_mailbox_allreduce", d["buf"], 4, 64, 1, 2_000_000)  # ~1 ms of SM clocks
        with pytest.raises(cabi.KatsuCudaError) as info:
            ctx.sync()
        assert info.value.code == cabi.ERR_TIMEOUT
        ctx.sync()
        ctx.call("katsu_cuda_selftest_mailbox_allreduce", d["buf"], 2, 64, 0, 200_000_000)
        ctx.sync()
        assert np.all(d.get("buf")[:128] == 2.0)
