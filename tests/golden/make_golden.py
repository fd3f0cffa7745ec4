"""Generates tests/golden/conv_matmul_golden.npz from the pinned CPU oracle.

The reference is Rust and cannot be run where this repository is built, so the
fixtures come from oracle/ (which is itself pinned by the reference's
known-answer tests, tests/test_oracle_pins.py).  Inputs are not stored: they are
regenerated from the seeds below with katsu_b200.synth; only the outputs of the
single-threaded, reference-order oracle are.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from katsu_b200 import synth  # noqa: E402
from oracle import katsu_ref as R  # noqa: E402

# name -> (n, c, h, w, k, r, s, stride, pad, seed)
CONV_CASES = {
    "rgb_stem_small": (2, 3, 20, 28, 8, 3, 3, 1, 1, 11),
    "rect_kernel_s1p0": (2, 2, 3, 4, 2, 2, 3, 1, 0, 12),
    "rect_kernel_s2p1": (2, 2, 3, 4, 2, 2, 3, 2, 1, 13),
    "wide_small": (1, 16, 9, 9, 12, 3, 3, 1, 1, 14),
    "strided_small": (1, 8, 11, 13, 6, 3, 3, 2, 1, 15),
    "pointwise": (3, 5, 4, 4, 7, 1, 1, 1, 0, 16),
}
# name -> (m, k, n, seed)
MATMUL_CASES = {
    "square": (16, 16, 16, 21),
    "skinny_head": (6, 2304, 10, 22),
    "rect": (5, 7, 3, 23),
}


def conv_inputs(case):
    n, c, h, w, k, r, s, stride, pad, seed = case
    oh, ow = R.conv_out_dims(h, w, r, s, stride, pad)
    x = synth.uniform(seed, n * c * h * w, -1.0, 1.0)
    wt = synth.normal(seed + 100, k * c * r * s, 0.3)
    g = synth.uniform(seed + 200, n * k * oh * ow, -1.0, 1.0)
    return x, wt, g


def matmul_inputs(case):
    m, k, n, seed = case
    return (synth.uniform(seed, m * k, -1.0, 1.0), synth.normal(seed + 100, k * n, 0.2),
            synth.uniform(seed + 200, m * n, -1.0, 1.0))


def main():
    out = {}
    for name, case in CONV_CASES.items():
        n, c, h, w, k, r, s, stride, pad, _ = case
        x, wt, g = conv_inputs(case)
        out[f"conv/{name}/y"] = R.conv2d_forward(x, wt, [n, c, h, w], [k, c, r, s], stride, pad)
        dx, dw = R.conv2d_backward(x, wt, g, [n, c, h, w], [k, c, r, s], stride, pad)
        out[f"conv/{name}/dx"], out[f"conv/{name}/dw"] = dx, dw
    for name, case in MATMUL_CASES.items():
        m, k, n, _ = case
        a, b, g = matmul_inputs(case)
        out[f"matmul/{name}/c"] = R.matmul(a, b, m, k, n)
        da, db = np.zeros(m * k, np.float32), np.zeros(k * n, np.float32)
        R.matmul_backward(a, b, g, da, db, m, k, n)
        out[f"matmul/{name}/da"], out[f"matmul/{name}/db"] = da, db
    # The reference's own literal vectors (crates/katsu-core/tests/conv2d.rs:16-26, 172-178; tests/tensor.rs:41-48)
    out["literal/conv_s1p0/y"] = np.array([37, 47, 67, 77], np.float32)
    out["literal/conv_s1p0/dx"] = np.array([1, 3, 2, 4, 10, 6, 3, 7, 4], np.float32)
    out["literal/conv_s1p0/dw"] = np.array([12, 16, 24, 28], np.float32)
    out["literal/conv_s2p1/y"] = np.array([4, 18, 36, 77], np.float32)
    out["literal/matmul/c"] = np.array([58, 64, 139, 154], np.float32)
    np.savez_compressed(os.path.join(HERE, "conv_matmul_golden.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
