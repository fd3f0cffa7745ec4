"""katsu_cuda_sum_static, the entry point for callers that may not allocate
device memory (their pool owns all of it, or cudaMalloc's implicit device
synchronisation is unacceptable to them): its per-block partials sit in a fixed
array inside the library instead of cudaMalloc'ed scratch.  Checked here
against katsu_cuda_sum through the C ABI on two calls in a row -- the second
smaller than the first, so stale partials left in the shared array by the
first call would show -- and on its size limit.  The file name sorts last so a
run that stops at the first failure has already run every other test."""
import numpy as np
import pytest

from katsu_b200 import cabi
from parity_util import DeviceArrays

pytestmark = pytest.mark.gpu


def both_sums(ctx, d, name, count):
    ctx.call("katsu_cuda_sum", d[name], d["ref"], count)
    ctx.call("katsu_cuda_sum_static", d[name], d["out"], count)
    return float(d.get("out")[0]), float(d.get("ref")[0])


def test_static_scratch_sum_matches_allocating_sum_twice_in_a_row(ctx):
    rng = np.random.default_rng(42)
    big = rng.standard_normal(5_000_003).astype(np.float32)
    small = rng.standard_normal(70_001).astype(np.float32)
    with DeviceArrays(ctx, big=big, small=small) as d:
        d.alloc("out", 1, fill=np.nan), d.alloc("ref", 1, fill=np.nan)
        for name, host in (("big", big), ("small", small)):  # two calls in a row, shared scratch
            got, ref = both_sums(ctx, d, name, host.size)
            scale = float(np.sum(np.abs(host.astype(np.float64))))
            exact = float(np.sum(host.astype(np.float64)))
            assert abs(got - ref) <= 1e-6 * scale, (name, got, ref)
            assert abs(got - exact) <= 1e-6 * scale, (name, got, exact)
        # empty input: zero, like the reference's sum of an empty tensor (tensor.rs:243-247)
        ctx.call("katsu_cuda_sum_static", 0, d["out"], 0)
        assert float(d.get("out")[0]) == 0.0


def test_static_scratch_sum_reads_an_unaligned_input(ctx):
    """An input that does not start on a 16-byte boundary takes the kernel's scalar loads."""
    rng = np.random.default_rng(43)
    host = rng.standard_normal(3_000_001).astype(np.float32)
    with DeviceArrays(ctx, a=host) as d:
        d.alloc("out", 1, fill=np.nan)
        for skip in (1, 3):
            ctx.call("katsu_cuda_sum_static", d["a"] + 4 * skip, d["out"], host.size - skip)
            exact = float(np.sum(host[skip:].astype(np.float64)))
            scale = float(np.sum(np.abs(host[skip:].astype(np.float64))))
            assert abs(float(d.get("out")[0]) - exact) <= 1e-6 * scale, skip


def _free_device_memory_reader():
    """cudaMemGetInfo of the current device through the CUDA runtime's shared library (the C ABI has
    no memory query; a second copy of the runtime in the process shares the device's context)."""
    import ctypes

    runtime = None
    for name in ("libcudart.so.12", "libcudart.so", "/usr/local/cuda/lib64/libcudart.so.12"):
        try:
            runtime = ctypes.CDLL(name)
            break
        except OSError:
            continue
    if runtime is None:
        pytest.skip("no CUDA runtime shared library to query free memory with")

    def free_bytes():
        free, total = ctypes.c_size_t(), ctypes.c_size_t()
        assert runtime.cudaSetDevice(0) == 0
        assert runtime.cudaMemGetInfo(ctypes.byref(free), ctypes.byref(total)) == 0
        return free.value

    return free_bytes


def test_static_scratch_sum_leaves_free_device_memory_unchanged(ctx):
    """After its first call on the device (address lookup, kernels loaded) a call takes no device
    memory: the free byte count the driver reports is the same before and after."""
    free_bytes = _free_device_memory_reader()
    host = np.ones(1 << 20, np.float32)
    with DeviceArrays(ctx, a=host) as d:
        d.alloc("out", 1, fill=np.nan)
        ctx.call("katsu_cuda_sum_static", d["a"], d["out"], host.size)  # first use on this device
        ctx.sync()
        free_before = free_bytes()
        ctx.call("katsu_cuda_sum_static", d["a"], d["out"], host.size)
        ctx.sync()
        free_after = free_bytes()
        assert float(d.get("out")[0]) == float(host.size)
    assert free_after == free_before, (free_before, free_after)


def test_static_scratch_sum_refuses_sizes_beyond_its_maximum(ctx):
    with DeviceArrays(ctx, a=np.ones(8, np.float32)) as d:
        d.alloc("out", 1, fill=3.0)
        with pytest.raises(cabi.KatsuCudaError) as info:
            ctx.call("katsu_cuda_sum_static", d["a"], d["out"], cabi.SUM_STATIC_MAX_COUNT + 1)  # refused before any launch
        assert info.value.code == cabi.ERR_UNSUPPORTED
        assert "at most" in info.value.message
        assert float(d.get("out")[0]) == 3.0  # untouched
        ctx.call("katsu_cuda_sum_static", d["a"], d["out"], 8)  # the context still works
        assert float(d.get("out")[0]) == 8.0
