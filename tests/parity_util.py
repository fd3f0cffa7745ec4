"""Helpers shared by the GPU parity tests: one C-ABI context per session and
the error measures the tolerances are written in."""
import numpy as np

# Relative L2 bound for f32 results against the f32 reference-order oracle.
# Both sides carry about one f32 rounding per term, in different summation
# orders, so they agree to a few 1e-7; 1e-5 is the documented bar.
REL_L2_TOL = 1e-5


def rel_l2(a, b):
    a = np.asarray(a, dtype=np.float64).reshape(-1)
    b = np.asarray(b, dtype=np.float64).reshape(-1)
    assert a.size == b.size
    denom = np.linalg.norm(b)
    diff = np.linalg.norm(a - b)
    return float(diff / denom) if denom > 0 else float(diff)


class DeviceArrays:
    """Uploads named host arrays, frees them on exit."""

    def __init__(self, ctx, **arrays):
        self.ctx = ctx
        self.ptr = {name: ctx.upload(a) for name, a in arrays.items()}
        self.size = {name: int(np.asarray(a).size) for name, a in arrays.items()}

    def alloc(self, name, count, fill=None):
        if fill is None:
            self.ptr[name] = self.ctx.alloc(count)
        else:
            self.ptr[name] = self.ctx.upload(np.full(count, fill, dtype=np.float32))
        self.size[name] = count
        return self.ptr[name]

    def get(self, name):
        return self.ctx.download(self.ptr[name], self.size[name])

    def __getitem__(self, name):
        return self.ptr[name]

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        for p in self.ptr.values():
            self.ctx.free(p)
