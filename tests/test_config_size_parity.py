"""Every named workload at its full configured size, in both tensor-core precision modes.

The oracle cannot run 1e11..7e11 multiply-adds in test time, so each function of the path is
checked on randomly sampled output elements whose complete sums the oracle recomputes in the
reference's visiting order (crates/katsu-core/src/conv2d.rs:232-262, 269-292): y from (x, w),
dX from (w, g), dW from (x, g), with g = 2y exactly as the VJP of loss = sum(y*y) delivers it
(crates/katsu-core/src/tensor.rs:392-417).  dW at these sizes sums N*OH*OW = 401 408 (wide,
strided) or 12.8 M (stem) terms per element: the length at which the tensor-core accumulation
chains, the split of the reduction over blocks and the ordered fold of the slabs matter.

Three distances are reported per tensor (printed with -s): device vs the f32 reference-order sum,
device vs the exact (f64) sum, and the reference-order sum vs the exact one -- the reference's
own rounding noise, which no device result can be closer to the reference than.

Bars: 3xTF32 (default) 1e-5 against the exact sum, and 1e-5 plus the reference's own noise
against the reference-order sum; TF32 2e-3.  Each comes with a per-element bound
(parity_util.max_abs_bound) so that a few wrong elements cannot hide in the norm.
"""
import numpy as np
import pytest

from katsu_b200 import cabi, workloads
from parity_util import REL_L2_TOL, TF32_UNIT, DeviceArrays, assert_parity, rel_l2

pytestmark = pytest.mark.gpu

TF32_TOL = 2e-3
Y_SAMPLES, DX_SAMPLES = 20000, 20000


def sampled_parity(ctx, oracle, spec, modes, dw_samples, report):
    x, w = workloads.conv_inputs(spec)
    geom = (spec.n, spec.c, spec.h, spec.w, spec.k, spec.r, spec.s, spec.stride, spec.pad)
    y_count = spec.n * spec.k * spec.oh * spec.ow
    rng = np.random.default_rng(spec.x_seed * 1000 + 7)
    idx_y = rng.integers(0, y_count, Y_SAMPLES)
    idx_x = rng.integers(0, x.size, DX_SAMPLES)
    idx_w = rng.choice(w.size, min(dw_samples, w.size), replace=False)
    y32, y64 = oracle.sample_y(x, w, idx_y, spec.x_shape, spec.w_shape, spec.stride, spec.pad)
    terms = {"y": spec.c * spec.r * spec.s, "dx": spec.k * spec.r * spec.s, "dw": spec.n * spec.oh * spec.ow}
    with DeviceArrays(ctx, x=x, w=w) as d:
        d.alloc("y", y_count), d.alloc("g", y_count), d.alloc("dx", x.size), d.alloc("dw", w.size)
        for mode in modes:
            ctx.set_precision(mode)
            try:
                ctx.conv2d_fwd(d["x"], d["w"], d["y"], *geom)
                ctx.call("katsu_cuda_add", d["y"], d["y"], d["g"], y_count)
                ctx.conv2d_bwd(d["x"], d["w"], d["g"], d["dx"], d["dw"], *geom, 0)
                y, dx, dw = d.get("y"), d.get("dx"), d.get("dw")
            finally:
                ctx.set_precision(cabi.MODE_3XTF32)
            g = y + y  # exact in f32; the oracle differentiates the device's own y
            dx32, dx64 = oracle.sample_dx(w, g, idx_x, spec.x_shape, spec.w_shape, spec.stride, spec.pad)
            dw32, dw64 = oracle.sample_dw(x, g, idx_w, spec.x_shape, spec.w_shape, spec.stride, spec.pad)
            for name, got, r32, r64 in (("y", y[idx_y], y32, y64), ("dx", dx[idx_x], dx32, dx64),
                                        ("dw", dw[idx_w], dw32, dw64)):
                noise = rel_l2(r32, r64)
                report(f"{spec.name} mode={mode} {name}: relL2(gpu, f32-order)={rel_l2(got, r32):.3e} "
                       f"relL2(gpu, f64)={rel_l2(got, r64):.3e} relL2(f32-order, f64)={noise:.3e}")
                what = (spec.name, mode, name)
                if mode == cabi.MODE_TF32:
                    assert_parity(got, r64, terms[name], tol=TF32_TOL, unit=TF32_UNIT, sqrt_terms=False, what=what)
                    assert rel_l2(got, r64) > 1e-5, what  # the switch really selected the single pass
                else:
                    assert_parity(got, r64, terms[name], tol=REL_L2_TOL, what=what)
                    assert_parity(got, r32, terms[name], tol=REL_L2_TOL + noise, what=what)


@pytest.mark.parametrize("name,dw_samples", [("wide_128x256x56", 256), ("down_128x128x112_s2", 256),
                                             ("stem_256x3x224", 48)])
def test_named_config_full_batch_both_modes(ctx, oracle, name, dw_samples, capsys):
    spec = workloads.CONV[name]

    def report(line):
        with capsys.disabled():
            print("\n" + line, end="")

    sampled_parity(ctx, oracle, spec, (cabi.MODE_3XTF32, cabi.MODE_TF32), dw_samples, report)


def test_small_cnn_graph_at_batch_512(oracle, capsys):
    """BASELINE config 5 through the autograd graph at its configured batch of 512.  Each op of the
    graph is checked against the oracle GIVEN the device's own inputs to that op: the convolutions
    on sampled elements, the classifier head (matmul [512,65536] @ [65536,10], the add, and both
    matmul gradients, the one for the weights summing over all 512 batch rows) on whole tensors."""
    import katsu_b200 as K
    from test_small_cnn import build_graph

    batch = workloads.CNN["batch"]
    k_fc, n_fc = workloads.CNN["fc_in"], workloads.CNN["fc_out"]
    t = build_graph(K, batch)
    c1, c2 = workloads.CONV["cnn_conv1"].with_batch(batch), workloads.CONV["cnn_conv2"].with_batch(batch)
    host = {name: np.asarray(t[name].data(), dtype=np.float32) for name in ("x", "w1", "w2", "wfc", "const", "h1", "h2", "out")}
    grad = {name: np.asarray(t[name].grad(), dtype=np.float32) for name in ("x", "w1", "w2", "wfc", "const", "h1", "h2", "out")}
    rng = np.random.default_rng(55)

    def show(line):
        with capsys.disabled():
            print("\n" + line, end="")

    def conv_checks(tag, spec, x, w, y, gy, dx, dw, dw_samples):
        idx = rng.integers(0, y.size, Y_SAMPLES)
        r32, r64 = oracle.sample_y(x, w, idx, spec.x_shape, spec.w_shape, spec.stride, spec.pad)
        show(f"small_cnn {tag} y: relL2(gpu, f32-order)={rel_l2(y[idx], r32):.3e} relL2(gpu, f64)={rel_l2(y[idx], r64):.3e}")
        assert_parity(y[idx], r32, spec.c * 9, what=(tag, "y"))
        idx = rng.integers(0, x.size, DX_SAMPLES)
        r32, r64 = oracle.sample_dx(w, gy, idx, spec.x_shape, spec.w_shape, spec.stride, spec.pad)
        show(f"small_cnn {tag} dx: relL2(gpu, f32-order)={rel_l2(dx[idx], r32):.3e} relL2(gpu, f64)={rel_l2(dx[idx], r64):.3e}")
        assert_parity(dx[idx], r64, spec.k * 9, what=(tag, "dx"))
        idx = rng.choice(w.size, min(dw_samples, w.size), replace=False)
        r32, r64 = oracle.sample_dw(x, gy, idx, spec.x_shape, spec.w_shape, spec.stride, spec.pad)
        noise = rel_l2(r32, r64)
        show(f"small_cnn {tag} dw: relL2(gpu, f32-order)={rel_l2(dw[idx], r32):.3e} relL2(gpu, f64)={rel_l2(dw[idx], r64):.3e} "
             f"relL2(f32-order, f64)={noise:.3e}")
        assert_parity(dw[idx], r64, spec.n * spec.oh * spec.ow, what=(tag, "dw"))
        assert_parity(dw[idx], r32, spec.n * spec.oh * spec.ow, tol=REL_L2_TOL + noise, what=(tag, "dw vs f32 order"))

    conv_checks("conv1", c1, host["x"], host["w1"], host["h1"], grad["h1"], grad["x"], grad["w1"], 128)
    conv_checks("conv2", c2, host["h1"], host["w2"], host["h2"], grad["h2"], grad["h1"], grad["w2"], 256)

    # classifier head, whole tensors
    out64 = oracle.matmul_f64(host["h2"], host["wfc"], batch, k_fc, n_fc) + host["const"].astype(np.float64)
    out32 = oracle.matmul(host["h2"], host["wfc"], batch, k_fc, n_fc, mt=True) + host["const"]
    noise = rel_l2(out32, out64)
    show(f"small_cnn out: relL2(gpu, f32-order)={rel_l2(host['out'], out32):.3e} relL2(gpu, f64)={rel_l2(host['out'], out64):.3e} "
         f"relL2(f32-order, f64)={noise:.3e}")
    assert_parity(host["out"], out64, k_fc, what="out")
    assert_parity(host["out"], out32, k_fc, tol=REL_L2_TOL + noise, what="out vs f32 order")
    # Mul VJP on both edges of out*out, then the Sum VJP's broadcast of 1: exactly 2 * out
    assert np.array_equal(grad["out"], host["out"] + host["out"])
    assert np.array_equal(grad["const"], grad["out"])  # Add VJP passes the adjoint through
    dh2_64, dwfc_64 = oracle.matmul_backward_f64(host["h2"], host["wfc"], grad["out"], batch, k_fc, n_fc)
    show(f"small_cnn d(h2)={rel_l2(grad['h2'], dh2_64):.3e} d(wfc)={rel_l2(grad['wfc'], dwfc_64):.3e} (vs f64)")
    assert_parity(grad["h2"], dh2_64, n_fc, what="d h2")
    assert_parity(grad["wfc"], dwfc_64, batch, what="d wfc")
    assert t["h2"].shape() == [batch, 64, 32, 32] and t["out"].shape() == [batch, n_fc]
