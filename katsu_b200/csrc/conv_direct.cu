// General direct convolution on CUDA cores: any channel count, rectangular
// filters, any stride and padding.  This is the catch-all behind the
// specialised kernels (low-channel stencil, tensor-core implicit GEMM); it
// evaluates exactly the tap set of Geometry::visit,
// crates/katsu-core/src/conv2d.rs:232-262, with virtual zero padding.
#include "common.cuh"

namespace {

struct ConvDims {
    int n, c, h, w, k, r, s, stride, pad, oh, ow;
};

// One thread per output element, KB output channels per thread so each x load
// feeds KB FMAs.  ox is the fastest index: y stores and x loads coalesce.
template <int KB>
__global__ void __launch_bounds__(256) conv_fwd_direct_kernel(const float *__restrict__ x,
                                                              const float *__restrict__ w,
                                                              float *__restrict__ y, ConvDims d) {
    const int kgroups = (d.k + KB - 1) / KB;
    const size_t plane = size_t(d.oh) * d.ow;
    const size_t total = size_t(d.n) * kgroups * plane;
    for (size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += size_t(gridDim.x) * blockDim.x) {
        const int ox = int(idx % d.ow);
        const int oy = int((idx / d.ow) % d.oh);
        const int kg = int((idx / plane) % kgroups);
        const int n = int(idx / (plane * kgroups));
        const int k0 = kg * KB;
        float acc[KB];
#pragma unroll
        for (int j = 0; j < KB; ++j) acc[j] = 0.f;
        for (int c = 0; c < d.c; ++c) {
            const float *xc = x + (size_t(n) * d.c + c) * d.h * d.w;
            for (int r = 0; r < d.r; ++r) {
                const int iy = oy * d.stride + r - d.pad;
                if (iy < 0 || iy >= d.h) continue;
                for (int s = 0; s < d.s; ++s) {
                    const int ix = ox * d.stride + s - d.pad;
                    if (ix < 0 || ix >= d.w) continue;
                    const float xv = __ldg(xc + size_t(iy) * d.w + ix);
#pragma unroll
                    for (int j = 0; j < KB; ++j) {
                        if (k0 + j < d.k)
                            acc[j] = fmaf(xv, __ldg(w + ((size_t(k0 + j) * d.c + c) * d.r + r) * d.s + s), acc[j]);
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < KB; ++j)
            if (k0 + j < d.k) y[(size_t(n) * d.k + k0 + j) * plane + size_t(oy) * d.ow + ox] = acc[j];
    }
}

// One thread per dx element: gathers every (k, oy, ox) whose window covers it.
__global__ void __launch_bounds__(256) conv_dx_direct_kernel(const float *__restrict__ w,
                                                             const float *__restrict__ g, float *dx,
                                                             ConvDims d, int accumulate) {
    const size_t total = size_t(d.n) * d.c * d.h * d.w;
    const size_t gplane = size_t(d.oh) * d.ow;
    for (size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
         idx += size_t(gridDim.x) * blockDim.x) {
        const int ix = int(idx % d.w);
        const int iy = int((idx / d.w) % d.h);
        const int c = int((idx / (size_t(d.w) * d.h)) % d.c);
        const int n = int(idx / (size_t(d.w) * d.h * d.c));
        float acc = 0.f;
        for (int k = 0; k < d.k; ++k) {
            const float *gk = g + (size_t(n) * d.k + k) * gplane;
            const float *wk = w + (size_t(k) * d.c + c) * d.r * d.s;
            for (int r = 0; r < d.r; ++r) {
                const int py = iy + d.pad - r;
                if (py < 0 || py % d.stride != 0) continue;
                const int oy = py / d.stride;
                if (oy >= d.oh) continue;
                for (int s = 0; s < d.s; ++s) {
                    const int px = ix + d.pad - s;
                    if (px < 0 || px % d.stride != 0) continue;
                    const int ox = px / d.stride;
                    if (ox >= d.ow) continue;
                    acc = fmaf(__ldg(gk + size_t(oy) * d.ow + ox), __ldg(wk + r * d.s + s), acc);
                }
            }
        }
        dx[idx] = accumulate ? dx[idx] + acc : acc;
    }
}

// One block per dw element (k, c, r, s): threads stride over (n, oy, ox), then
// a fixed-shape tree reduction (bit-reproducible).
__global__ void __launch_bounds__(256) conv_dw_direct_kernel(const float *__restrict__ x,
                                                             const float *__restrict__ g, float *dw,
                                                             ConvDims d, int accumulate) {
    const size_t wi = blockIdx.x;
    const int s = int(wi % d.s);
    const int r = int((wi / d.s) % d.r);
    const int c = int((wi / (size_t(d.s) * d.r)) % d.c);
    const int k = int(wi / (size_t(d.s) * d.r * d.c));
    const size_t gplane = size_t(d.oh) * d.ow;
    const size_t terms = size_t(d.n) * gplane;
    float acc = 0.f;
    for (size_t t = threadIdx.x; t < terms; t += blockDim.x) {
        const int ox = int(t % d.ow);
        const int oy = int((t / d.ow) % d.oh);
        const int n = int(t / gplane);
        const int iy = oy * d.stride + r - d.pad;
        const int ix = ox * d.stride + s - d.pad;
        if (iy < 0 || iy >= d.h || ix < 0 || ix >= d.w) continue;
        acc = fmaf(__ldg(g + (size_t(n) * d.k + k) * gplane + size_t(oy) * d.ow + ox),
                   __ldg(x + ((size_t(n) * d.c + c) * d.h + iy) * d.w + ix), acc);
    }
    __shared__ float sh[256];
    sh[threadIdx.x] = acc;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if ((int)threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) dw[wi] = accumulate ? dw[wi] + sh[0] : sh[0];
}

int32_t make_dims(ConvDims *d, size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                  size_t stride, size_t pad, size_t oh, size_t ow) {
    const size_t lim = 0x7fffffff;
    if (n > lim || c > lim || h > lim || wd > lim || k > lim || r > lim || s > lim || stride > lim ||
        pad > lim || oh > lim || ow > lim)
        return katsu_set_error(KATSU_ERR_UNSUPPORTED, "a convolution dimension exceeds 2^31-1");
    d->n = (int)n; d->c = (int)c; d->h = (int)h; d->w = (int)wd; d->k = (int)k; d->r = (int)r; d->s = (int)s;
    d->stride = (int)stride; d->pad = (int)pad; d->oh = (int)oh; d->ow = (int)ow;
    return KATSU_OK;
}

unsigned grid_for(const katsu_cuda_ctx *ctx, size_t work_items, int threads) {
    size_t blocks = katsu_div_up(work_items, (size_t)threads);
    const size_t cap = size_t(ctx->num_sms) * 32;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    return (unsigned)blocks;
}

}  // namespace

int32_t katsu_conv_direct_fwd(katsu_cuda_ctx *ctx, const float *x, const float *w, float *y,
                              size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                              size_t stride, size_t pad, size_t oh, size_t ow) {
    ConvDims d;
    KATSU_TRY(make_dims(&d, n, c, h, wd, k, r, s, stride, pad, oh, ow));
    constexpr int KB = 4;
    const size_t total = n * katsu_div_up(k, (size_t)KB) * oh * ow;
    KATSU_LAUNCH(ctx, conv_fwd_direct_kernel<KB>, grid_for(ctx, total, 256), 256, 0, x, w, y, d);
    return KATSU_OK;
}

int32_t katsu_conv_direct_dx(katsu_cuda_ctx *ctx, const float *w, const float *g, float *dx,
                             size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                             size_t stride, size_t pad, size_t oh, size_t ow, int accumulate) {
    ConvDims d;
    KATSU_TRY(make_dims(&d, n, c, h, wd, k, r, s, stride, pad, oh, ow));
    KATSU_LAUNCH(ctx, conv_dx_direct_kernel, grid_for(ctx, n * c * h * wd, 256), 256, 0, w, g, dx, d, accumulate);
    return KATSU_OK;
}

int32_t katsu_conv_direct_dw(katsu_cuda_ctx *ctx, const float *x, const float *g, float *dw,
                             size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                             size_t stride, size_t pad, size_t oh, size_t ow, int accumulate) {
    ConvDims d;
    KATSU_TRY(make_dims(&d, n, c, h, wd, k, r, s, stride, pad, oh, ow));
    const size_t elems = k * c * r * s;
    if (elems > 0x7fffffff) return katsu_set_error(KATSU_ERR_UNSUPPORTED, "filter has more than 2^31-1 elements");
    KATSU_LAUNCH(ctx, conv_dw_direct_kernel, (unsigned)elems, 256, 0, x, g, dw, d, accumulate);
    return KATSU_OK;
}
