"""ctypes binding of the C ABI declared in include/katsu_cuda.h.

This is the same boundary a Rust `extern "C"` block (or any other FFI) binds;
Python is only one caller.  The library is loaded from katsu_b200/lib/ and
nowhere else, and loading fails loudly when it has not been built: there is
no CPU path behind these functions.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libkatsu_cuda.so")

OK = 0
ERR_INVALID_ARG, ERR_ALLOC, ERR_CUDA, ERR_NCCL, ERR_TIMEOUT, ERR_NO_DEVICE, ERR_UNSUPPORTED = range(1, 8)
MODE_3XTF32, MODE_TF32, MODE_FP32 = 0, 1, 2
SUM_STATIC_MAX_COUNT = 1 << 30
COMM_ID_BYTES = 128

_c_float_p = ctypes.POINTER(ctypes.c_float)
_sz = ctypes.c_size_t
_i32 = ctypes.c_int32
_ctx = ctypes.c_void_p
_ptr = ctypes.c_void_p  # device pointers travel as integers

# name -> argtypes (restype is int32 for all but last_error_string)
SIGNATURES = {
    "katsu_cuda_device_count": [ctypes.POINTER(_i32)],
    "katsu_cuda_init": [_i32, ctypes.POINTER(_ctx)],
    "katsu_cuda_shutdown": [_ctx],
    "katsu_cuda_set_precision": [_ctx, _i32],
    "katsu_cuda_get_precision": [_ctx, ctypes.POINTER(_i32)],
    "katsu_cuda_launch_count": [_ctx, ctypes.POINTER(ctypes.c_uint64)],
    "katsu_cuda_stream": [_ctx, ctypes.POINTER(ctypes.c_void_p)],
    "katsu_cuda_alloc": [_ctx, _sz, ctypes.POINTER(_ptr)],
    "katsu_cuda_free": [_ctx, _ptr],
    "katsu_cuda_zero": [_ctx, _ptr, _sz],
    "katsu_cuda_h2d": [_ctx, _ptr, ctypes.c_void_p, _sz],
    "katsu_cuda_d2h": [_ctx, ctypes.c_void_p, _ptr, _sz],
    "katsu_cuda_d2h_async": [_ctx, ctypes.c_void_p, _ptr, _sz],
    "katsu_cuda_d2d": [_ctx, _ptr, _ptr, _sz],
    "katsu_cuda_host_alloc": [_ctx, _sz, ctypes.POINTER(ctypes.c_void_p)],
    "katsu_cuda_host_free": [_ctx, ctypes.c_void_p],
    "katsu_cuda_sync": [_ctx],
    "katsu_cuda_conv2d_fwd": [_ctx, _ptr, _ptr, _ptr] + [_sz] * 9,
    "katsu_cuda_conv2d_bwd": [_ctx, _ptr, _ptr, _ptr, _ptr, _ptr] + [_sz] * 9 + [_i32],
    "katsu_cuda_conv2d_bwd_scaled": [_ctx, _ptr, _ptr, _ptr, _ptr, ctypes.c_float, _ptr, _ptr] + [_sz] * 9 + [_i32],
    "katsu_cuda_conv2d_fwd_bias_relu": [_ctx, _ptr, _ptr, _ptr, _ptr] + [_sz] * 9 + [_i32],
    "katsu_cuda_conv2d_staged_floats": [_ctx] + [_sz] * 9 + [ctypes.POINTER(ctypes.c_size_t)],
    "katsu_cuda_conv2d_stage": [_ctx, _ptr, _ptr, _sz, _sz, _sz, _sz],
    "katsu_cuda_conv2d_fwd_staged": [_ctx, _ptr, _ptr, _ptr, _ptr, _ptr] + [_sz] * 9 + [_i32],
    "katsu_cuda_conv2d_bwd_staged": [_ctx, _ptr, _ptr, _ptr, _ptr, _ptr, ctypes.c_float, _ptr, _ptr] + [_sz] * 9 + [_i32],
    "katsu_cuda_bias_relu_bwd": [_ctx, _ptr, _ptr, _ptr, _ptr, _sz, _sz, _sz, _i32, _i32],
    "katsu_cuda_sgd_step": [_ctx, _ptr, _ptr, ctypes.c_float, _sz],
    "katsu_cuda_sumsq": [_ctx, _ptr, _ptr, _sz],
    "katsu_cuda_square_vjp": [_ctx, _ptr, _ptr, _ptr, _sz, _i32],
    "katsu_cuda_matmul_fwd": [_ctx, _ptr, _ptr, _ptr, _sz, _sz, _sz],
    "katsu_cuda_matmul_bwd": [_ctx, _ptr, _ptr, _ptr, _ptr, _ptr, _sz, _sz, _sz, _i32],
    "katsu_cuda_add": [_ctx, _ptr, _ptr, _ptr, _sz],
    "katsu_cuda_mul": [_ctx, _ptr, _ptr, _ptr, _sz],
    "katsu_cuda_sum": [_ctx, _ptr, _ptr, _sz],
    "katsu_cuda_sum_static": [_ctx, _ptr, _ptr, _sz],
    "katsu_cuda_axpy_acc": [_ctx, _ptr, _ptr, _sz],
    "katsu_cuda_mul_acc": [_ctx, _ptr, _ptr, _ptr, _sz],
    "katsu_cuda_bcast_acc": [_ctx, _ptr, _ptr, _sz],
    "katsu_cuda_comm_unique_id": [ctypes.c_void_p],
    "katsu_cuda_comm_init": [_ctx, ctypes.c_void_p, _i32, _i32],
    "katsu_cuda_comm_destroy": [_ctx],
    "katsu_cuda_allreduce_sum": [_ctx, _ptr, _sz],
    "katsu_cuda_event_create": [_ctx, ctypes.POINTER(ctypes.c_void_p)],
    "katsu_cuda_event_record": [_ctx, ctypes.c_void_p],
    "katsu_cuda_event_elapsed_ms": [_ctx, ctypes.c_void_p, ctypes.c_void_p, _c_float_p],
    "katsu_cuda_event_destroy": [_ctx, ctypes.c_void_p],
    "katsu_cuda_wait_event": [_ctx, ctypes.c_void_p],
    "katsu_cuda_flush_l2": [_ctx],
    "katsu_cuda_selftest_wait_timeout": [_ctx, ctypes.c_uint64],
    "katsu_cuda_selftest_mailbox_allreduce": [_ctx, _ptr, _i32, _sz, _i32, ctypes.c_uint64],
}

_lib = None


class KatsuCudaError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"katsu_cuda error {code}: {message}")
        self.code = code
        self.message = message


def load() -> ctypes.CDLL:
    """Loads libkatsu_cuda.so; raises if it is not built (run `python -m katsu_b200.build`)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise OSError(f"{LIB_PATH} is missing: build it with `python -m katsu_b200.build`; "
                          "there is no CPU fallback")
        lib = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
        for name, argtypes in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _i32
        lib.katsu_cuda_last_error_string.argtypes = []
        lib.katsu_cuda_last_error_string.restype = ctypes.c_char_p
        _lib = lib
    return _lib


def check(rc: int) -> None:
    if rc != OK:
        raise KatsuCudaError(rc, load().katsu_cuda_last_error_string().decode("utf-8", "replace"))


class Context:
    """Thin owner of one katsu_cuda_ctx (one device, one stream)."""

    def __init__(self, device: int = 0):
        self.lib = load()
        handle = _ctx()
        check(self.lib.katsu_cuda_init(device, ctypes.byref(handle)))
        self.handle = handle
        self.device = device

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.katsu_cuda_shutdown(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # -- generic call ------------------------------------------------------
    def call(self, name: str, *args) -> None:
        check(getattr(self.lib, name)(self.handle, *args))

    # -- memory --------------------------------------------------------------
    def alloc(self, count: int) -> int:
        out = _ptr()
        self.call("katsu_cuda_alloc", count, ctypes.byref(out))
        return out.value or 0

    def free(self, ptr: int) -> None:
        if ptr:
            self.call("katsu_cuda_free", ptr)

    def upload(self, array) -> int:
        """Allocates a device buffer and copies a host f32 array into it."""
        array = np.ascontiguousarray(np.asarray(array, dtype=np.float32).reshape(-1))
        ptr = self.alloc(array.size)
        if array.size:
            self.call("katsu_cuda_h2d", ptr, array.ctypes.data, array.size)
            self.sync()  # the numpy source may be pageable and short-lived
        return ptr

    def h2d(self, ptr: int, array: np.ndarray) -> None:
        assert array.dtype == np.float32 and array.flags["C_CONTIGUOUS"]
        self.call("katsu_cuda_h2d", ptr, array.ctypes.data, array.size)

    def download(self, ptr: int, count: int) -> np.ndarray:
        out = np.empty(count, dtype=np.float32)
        self.call("katsu_cuda_d2h", out.ctypes.data, ptr, count)
        return out

    def d2h(self, array: np.ndarray, ptr: int) -> None:
        assert array.dtype == np.float32 and array.flags["C_CONTIGUOUS"]
        self.call("katsu_cuda_d2h", array.ctypes.data, ptr, array.size)

    def d2h_async(self, array: np.ndarray, ptr: int) -> None:
        """Stream-ordered copy into a page-locked array; valid after sync()."""
        assert array.dtype == np.float32 and array.flags["C_CONTIGUOUS"]
        self.call("katsu_cuda_d2h_async", array.ctypes.data, ptr, array.size)

    def pinned(self, count: int) -> np.ndarray:
        """A page-locked f32 numpy array of `count` elements (freed with free_pinned)."""
        out = ctypes.c_void_p()
        self.call("katsu_cuda_host_alloc", count, ctypes.byref(out))
        buf = (ctypes.c_float * count).from_address(out.value)
        arr = np.frombuffer(buf, dtype=np.float32, count=count)
        return arr

    def free_pinned(self, array: np.ndarray) -> None:
        self.call("katsu_cuda_host_free", array.ctypes.data)

    def sync(self) -> None:
        self.call("katsu_cuda_sync")

    def set_precision(self, mode: int) -> None:
        self.call("katsu_cuda_set_precision", mode)

    def launch_count(self) -> int:
        out = ctypes.c_uint64()
        self.call("katsu_cuda_launch_count", ctypes.byref(out))
        return out.value

    # -- timing ----------------------------------------------------------------
    def event(self) -> int:
        out = ctypes.c_void_p()
        self.call("katsu_cuda_event_create", ctypes.byref(out))
        return out.value

    def record(self, event: int) -> None:
        self.call("katsu_cuda_event_record", event)

    def elapsed_ms(self, start: int, stop: int) -> float:
        out = ctypes.c_float()
        self.call("katsu_cuda_event_elapsed_ms", start, stop, ctypes.byref(out))
        return out.value

    def wait_event(self, event: int) -> None:
        """Device-side wait of this context's queue for `event` (recorded on any context of the device)."""
        self.call("katsu_cuda_wait_event", event)

    def event_destroy(self, event: int) -> None:
        self.call("katsu_cuda_event_destroy", event)

    # -- kernels ---------------------------------------------------------------
    def conv2d_fwd(self, x, w, y, n, c, h, wd, k, r, s, stride, pad) -> None:
        self.call("katsu_cuda_conv2d_fwd", x, w, y, n, c, h, wd, k, r, s, stride, pad)

    def conv2d_bwd(self, x, w, g, dx, dw, n, c, h, wd, k, r, s, stride, pad, accumulate=0) -> None:
        self.call("katsu_cuda_conv2d_bwd", x, w, g, dx, dw, n, c, h, wd, k, r, s, stride, pad, accumulate)

    def conv2d_staged_floats(self, n, c, h, wd, k, r, s, stride, pad) -> int:
        """Floats of the channels-innermost copy of x that this shape's kernels read (0: none)."""
        out = ctypes.c_size_t(0)
        self.call("katsu_cuda_conv2d_staged_floats", n, c, h, wd, k, r, s, stride, pad, ctypes.byref(out))
        return int(out.value)

    def conv2d_stage(self, x, staged, n, c, h, wd) -> None:
        self.call("katsu_cuda_conv2d_stage", x, staged, n, c, h, wd)

    def conv2d_fwd_staged(self, x, x_staged, w, bias, y, n, c, h, wd, k, r, s, stride, pad, relu=0) -> None:
        self.call("katsu_cuda_conv2d_fwd_staged", x, x_staged, w, bias, y, n, c, h, wd, k, r, s, stride, pad, relu)

    def conv2d_bwd_staged(self, x, x_staged, w, g, gscale, gfactor, dx, dw, n, c, h, wd, k, r, s, stride, pad,
                          accumulate=0) -> None:
        self.call("katsu_cuda_conv2d_bwd_staged", x, x_staged, w, g, gscale, gfactor, dx, dw, n, c, h, wd, k, r, s,
                  stride, pad, accumulate)

    def matmul_fwd(self, a, b, c, m, k, n) -> None:
        self.call("katsu_cuda_matmul_fwd", a, b, c, m, k, n)

    def matmul_bwd(self, a, b, g, da, db, m, k, n, accumulate=0) -> None:
        self.call("katsu_cuda_matmul_bwd", a, b, g, da, db, m, k, n, accumulate)
