"""Helpers shared by the GPU parity tests: one C-ABI context per session and
the error measures the tolerances are written in."""
import numpy as np

# Relative L2 bound for f32 results against the f32 reference-order oracle.
# Both sides carry about one f32 rounding per term, in different summation
# orders, so they agree to a few 1e-7; 1e-5 is the documented bar.
REL_L2_TOL = 1e-5


EPS32 = float(np.finfo(np.float32).eps)  # 2^-23
TF32_UNIT = 2.0 ** -10                   # spacing of TF32 (10 mantissa bits) relative to the value


def max_abs_bound(ref, terms, unit=EPS32, c=4.0, sqrt_terms=True):
    """Per-element bound that goes with the norm-wise bar.  An element that sums `terms` products
    of typical size s is about s * sqrt(terms) large and carries a rounding error of about
    unit * s * sqrt(terms) * sqrt(terms) / 5 in f32 (each add rounds the running sum), i.e.
    unit * sqrt(terms) / 5 of the largest element; c = 4 leaves a wide margin for that and is still
    orders of magnitude below one wrong element (which is off by about max|ref| / 4).  A single
    reduced-precision pass (TF32) errs by `unit` of each product instead, which does not grow with
    the term count relative to the result: sqrt_terms=False."""
    ref = np.asarray(ref, dtype=np.float64)
    scale = float(np.abs(ref).max()) if ref.size else 0.0
    growth = float(np.sqrt(max(int(terms), 1))) if sqrt_terms else 1.0
    return c * unit * growth * scale + 1e-30


def assert_parity(got, ref, terms, tol=REL_L2_TOL, what="", **bound_args):
    """rel-L2 within `tol` AND every element within max_abs_bound: a handful of wrong elements in a
    large tensor passes a norm-wise bar (whole wrong pixels once sat at 2e-6 .. 8e-5 in rel-L2)."""
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    ref64 = np.asarray(ref, dtype=np.float64).reshape(-1)
    err = rel_l2(got, ref64)
    assert err <= tol, (what, "rel-L2", err, tol)
    worst = float(np.abs(got - ref64).max()) if got.size else 0.0
    bound = max_abs_bound(ref64, terms, **bound_args)
    assert worst <= bound, (what, "max |diff|", worst, bound, int(np.abs(got - ref64).argmax()))
    return err


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
