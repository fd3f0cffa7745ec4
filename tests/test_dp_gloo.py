"""Data-parallel host logic on CPU: two gloo ranks shard a batch, each computes
its partial dW (with the oracle standing in for the device), the partials are
all-reduced, and the sum must equal the unsharded dW.  Covers dp.shard and the
property the multi-GPU step relies on: dX / y stay sharded, only dW crosses ranks."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_covers_the_batch_exactly():
    from katsu_b200 import dp

    for total in (0, 1, 7, 8, 256, 513):
        for world in (1, 2, 3, 8):
            spans = [dp.shard(total, r, world) for r in range(world)]
            assert spans[0][0] == 0
            for (f0, c0), (f1, _) in zip(spans, spans[1:]):
                assert f0 + c0 == f1
            assert spans[-1][0] + spans[-1][1] == total
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1
    with pytest.raises(ValueError):
        dp.shard(8, 2, 2)


def _worker(rank, world, port, out_queue):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch
    import torch.distributed as dist

    from katsu_b200 import dp, workloads
    from oracle import katsu_ref as R

    dist.init_process_group(backend="gloo", rank=rank, world_size=world)
    spec = workloads.CONV["cnn_conv1"].with_batch(6)
    first, count = dp.shard(spec.n, rank, world)
    x, w = workloads.conv_inputs(spec, first, count)
    shard_spec = spec.with_batch(count)
    y = R.conv2d_forward(x, w, shard_spec.x_shape, spec.w_shape, 1, 1)
    dx, dw = R.conv2d_backward(x, w, y + y, shard_spec.x_shape, spec.w_shape, 1, 1)
    bucket = torch.from_numpy(dw.copy())
    dist.all_reduce(bucket)  # the one exchange of the step
    out_queue.put((rank, first, count, dx, bucket.numpy().copy()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_dw_allreduce_matches_unsharded():
    import torch.multiprocessing as mp

    from katsu_b200 import workloads
    from oracle import katsu_ref as R

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, queue)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted((queue.get(timeout=120) for _ in procs), key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0

    spec = workloads.CONV["cnn_conv1"].with_batch(6)
    x, w = workloads.conv_inputs(spec)
    y = R.conv2d_forward(x, w, spec.x_shape, spec.w_shape, 1, 1)
    dx_full, dw_full = R.conv2d_backward(x, w, y + y, spec.x_shape, spec.w_shape, 1, 1)
    per_image = spec.c * spec.h * spec.w
    for rank, first, count, dx, dw_sum in results:
        # dX of a shard is bit-identical to the same images' dX in the full batch
        assert np.array_equal(dx, dx_full[first * per_image:(first + count) * per_image])
        # dW differs from the unsharded sum only by summation order
        assert np.linalg.norm(dw_sum - dw_full) <= 1e-5 * np.linalg.norm(dw_full)
    assert np.array_equal(results[0][4], results[1][4])
