"""Random shapes over every kernel family against the exact (f64) oracle, all three precision modes where they
apply.  Fixed seeds.  A sweep like this one found the accumulation-length problem of narrow layers with long
contractions and the vector accesses on unaligned operands; what it draws from: channel counts on both sides of
every tile width, filter sizes 1-5, strides 1-3, paddings 0-2, planes that leave partial tiles."""
import numpy as np
import pytest

from parity_util import rel_l2

pytestmark = pytest.mark.gpu

BARS = ((0, 1e-5), (1, 2e-3), (2, 1e-5))  # 3xTF32, TF32, FP32 (CUDA cores)


def run_conv(ctx, oracle, shape, rng, modes):
    n, c, h, w, k, r, s, stride, pad = shape
    oh, ow = oracle.conv_out_dims(h, w, r, s, stride, pad)
    x = rng.standard_normal(n * c * h * w).astype(np.float32)
    wt = rng.standard_normal(k * c * r * s).astype(np.float32)
    g = rng.standard_normal(n * k * oh * ow).astype(np.float32)
    y64 = oracle.conv2d_forward_f64(x, wt, [n, c, h, w], [k, c, r, s], stride, pad)
    dx64, dw64 = oracle.conv2d_backward_f64(x, wt, g, [n, c, h, w], [k, c, r, s], stride, pad)
    px, pw, pg = ctx.upload(x), ctx.upload(wt), ctx.upload(g)
    py = ctx.upload(np.full(g.size, np.nan, np.float32))
    pdx = ctx.upload(np.full(x.size, np.nan, np.float32))
    pdw = ctx.upload(np.full(wt.size, np.nan, np.float32))
    try:
        for mode, bar in modes:
            ctx.set_precision(mode)
            ctx.conv2d_fwd(px, pw, py, *shape)
            ctx.conv2d_bwd(px, pw, pg, pdx, pdw, *shape, 0)
            errors = (rel_l2(ctx.download(py, g.size), y64), rel_l2(ctx.download(pdx, x.size), dx64),
                      rel_l2(ctx.download(pdw, wt.size), dw64))
            assert all(np.isfinite(e) and e <= bar for e in errors), (shape, mode, errors)
    finally:
        ctx.set_precision(0)
        for p in (px, pw, pg, py, pdx, pdw):
            ctx.free(p)


@pytest.mark.parametrize("seed", [21, 22])
def test_wide_and_mid_channel_convolutions(ctx, oracle, seed):
    rng = np.random.default_rng(seed)
    channels = [16, 20, 24, 32, 36, 48, 64, 96, 100, 128, 132, 160, 192, 256, 260, 288, 320, 384, 512]
    done = 0
    while done < 40:
        c, k = int(rng.choice(channels)), int(rng.choice(channels))
        r, s = int(rng.choice([1, 2, 3, 3, 3, 5])), int(rng.choice([1, 3, 3, 3, 2]))
        stride, pad = int(rng.choice([1, 1, 1, 2, 2, 3])), int(rng.choice([0, 1, 1, 2]))
        h, w = int(rng.integers(max(r - 2 * pad, 1), 23)), int(rng.integers(max(s - 2 * pad, 1), 23))
        n = int(rng.integers(1, 5))
        if h + 2 * pad < r or w + 2 * pad < s:
            continue
        run_conv(ctx, oracle, (n, c, h, w, k, r, s, stride, pad), rng, BARS[:2])
        done += 1


@pytest.mark.parametrize("seed", [31, 32])
def test_low_channel_convolutions(ctx, oracle, seed):
    rng = np.random.default_rng(seed)
    done = 0
    while done < 60:
        c = int(rng.integers(1, 13))
        k = int(rng.choice([1, 3, 8, 16, 17, 31, 32, 33, 48, 64, 65, 96, 100, 128, 129, 130, 200]))
        r, s = (3, 3) if rng.random() < 0.8 else (int(rng.choice([1, 2, 3, 5])), int(rng.choice([1, 2, 3, 5])))
        stride = 1 if rng.random() < 0.8 else int(rng.choice([2, 3]))
        pad = 1 if rng.random() < 0.8 else int(rng.choice([0, 2]))
        h, w = int(rng.integers(3, 70)), int(rng.choice([4, 8, 12, 28, 32, 36, 60, 64, 100, 5, 7, 33, 50]))
        n = int(rng.integers(1, 4))
        if h + 2 * pad < r or w + 2 * pad < s:
            continue
        run_conv(ctx, oracle, (n, c, h, w, k, r, s, stride, pad), rng, BARS)
        done += 1


@pytest.mark.parametrize("seed", [41])
def test_matmuls(ctx, oracle, seed):
    rng = np.random.default_rng(seed)
    sizes = [1, 3, 10, 16, 33, 64, 100, 128, 200, 256, 260, 384, 512, 516, 1000, 1024, 1100, 2048, 2100, 2304, 2332]
    done = 0
    while done < 30:
        m, k, n = (int(rng.choice(sizes)) for _ in range(3))
        if m * k * n > 6e9:
            continue
        a = rng.standard_normal(m * k).astype(np.float32)
        b = rng.standard_normal(k * n).astype(np.float32)
        g = rng.standard_normal(m * n).astype(np.float32)
        c64 = oracle.matmul_f64(a, b, m, k, n)
        da64, db64 = oracle.matmul_backward_f64(a, b, g, m, k, n)
        pa, pb, pg = ctx.upload(a), ctx.upload(b), ctx.upload(g)
        pc = ctx.upload(np.full(m * n, np.nan, np.float32))
        pda = ctx.upload(np.full(m * k, np.nan, np.float32))
        pdb = ctx.upload(np.full(k * n, np.nan, np.float32))
        try:
            for mode, bar in BARS[:2]:
                ctx.set_precision(mode)
                ctx.matmul_fwd(pa, pb, pc, m, k, n)
                ctx.matmul_bwd(pa, pb, pg, pda, pdb, m, k, n, 0)
                errors = (rel_l2(ctx.download(pc, m * n), c64), rel_l2(ctx.download(pda, m * k), da64),
                          rel_l2(ctx.download(pdb, k * n), db64))
                assert all(np.isfinite(e) and e <= bar for e in errors), ((m, k, n), mode, errors)
        finally:
            ctx.set_precision(0)
            for p in (pa, pb, pg, pc, pda, pdb):
                ctx.free(p)
        done += 1
