// Conv2D entry points of the C ABI: argument checks, output geometry and the
// choice of kernel family.  The arithmetic lives in conv_stencil.cu (low
// channel counts), conv_igemm.cu (wide channels, tensor cores) and
// conv_direct.cu (everything else, CUDA cores).
#include "common.cuh"

namespace {

struct Geometry {
    size_t oh, ow;
};

// Same output-size rule as Geometry::new, crates/katsu-core/src/conv2d.rs:197-210.
// The caller has normally validated already; this guards the kernels.
int32_t geometry(size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s, size_t stride, size_t pad,
                 Geometry *g) {
    if (c == 0 || k == 0 || r == 0 || s == 0)
        return katsu_set_error(KATSU_ERR_INVALID_ARG, "weights must have positive OIHW dimensions");
    if (stride == 0) return katsu_set_error(KATSU_ERR_INVALID_ARG, "stride must be positive");
    if (h == 0 || wd == 0) return katsu_set_error(KATSU_ERR_INVALID_ARG, "H and W must be positive");
    if (pad > (SIZE_MAX >> 2)) return katsu_set_error(KATSU_ERR_INVALID_ARG, "padding too large");
    if (h + 2 * pad < r || wd + 2 * pad < s)
        return katsu_set_error(KATSU_ERR_INVALID_ARG, "kernel exceeds padded input");
    g->oh = (h + 2 * pad - r) / stride + 1;
    g->ow = (wd + 2 * pad - s) / stride + 1;
    return KATSU_OK;
}

}  // namespace

namespace {

int32_t forward(katsu_cuda_ctx *ctx, const float *x, const float *w, const float *bias, float *y,
                size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s, size_t stride, size_t pad,
                int relu) {
    KATSU_TRY(katsu_bind(ctx));
    Geometry g;
    KATSU_TRY(geometry(c, h, wd, k, r, s, stride, pad, &g));
    if (n == 0) return KATSU_OK;  // empty batch: y has no elements (conv2d.rs:195-196)
    KATSU_REQUIRE(x != nullptr && w != nullptr && y != nullptr, "null tensor");
    int handled = 0;
    KATSU_TRY(katsu_conv_stem_tc_fwd(ctx, x, w, y, n, c, h, wd, k, r, s, stride, pad, bias, relu, &handled));
    if (handled) return KATSU_OK;  // bias and ReLU were applied in that kernel's epilogue
    KATSU_TRY(katsu_conv_stencil_fwd(ctx, x, w, y, n, c, h, wd, k, r, s, stride, pad, &handled));
    if (!handled) KATSU_TRY(katsu_conv_igemm_fwd(ctx, x, w, y, n, c, h, wd, k, r, s, stride, pad, g.oh, g.ow, &handled));
    if (!handled) KATSU_TRY(katsu_conv_direct_fwd(ctx, x, w, y, n, c, h, wd, k, r, s, stride, pad, g.oh, g.ow));
    return katsu_bias_relu_inplace(ctx, y, bias, n, k, g.oh * g.ow, relu);
}

// out[i] = factor * fl(s[0] * in[i]): the scaled upstream gradient written out, for the kernels that
// cannot apply the scale themselves.
__global__ void __launch_bounds__(256) scale_copy_kernel(float *__restrict__ out, const float *__restrict__ in,
                                                         const float *__restrict__ s, float factor, size_t count) {
    const float scalar = s != nullptr ? __ldg(s) : 1.f;
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride)
        out[i] = factor * __fmul_rn(scalar, in[i]);
}

int32_t scale_copy(katsu_cuda_ctx *ctx, float *out, const float *in, const float *s, float factor, size_t count) {
    size_t blocks = katsu_div_up(count, 256);
    if (blocks > size_t(ctx->num_sms) * 8) blocks = size_t(ctx->num_sms) * 8;
    KATSU_LAUNCH(ctx, scale_copy_kernel, (unsigned)blocks, 256, 0, out, in, s, factor, count);
    return KATSU_OK;
}

int32_t backward(katsu_cuda_ctx *ctx, const float *x, const float *w, const float *gr, const float *gscale,
                 float gfactor, float *dx, float *dw,
                 size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s, size_t stride, size_t pad,
                 int32_t accumulate) {
    KATSU_TRY(katsu_bind(ctx));
    Geometry g;
    KATSU_TRY(geometry(c, h, wd, k, r, s, stride, pad, &g));
    KATSU_REQUIRE(dx == nullptr || (const float *)dx != (const float *)dw, "dx and dw must not alias");
    if (n == 0) {
        // dx is empty; dw is a sum over no terms (conv2d.rs:283-284 leaves zeros).
        if (dw != nullptr && !accumulate)
            KATSU_CUDA_TRY(cudaMemsetAsync(dw, 0, k * c * r * s * sizeof(float), ctx->stream));
        return KATSU_OK;
    }
    KATSU_REQUIRE(gr != nullptr, "null upstream gradient");
    KATSU_REQUIRE(dx == nullptr || w != nullptr, "dx needs the weights");
    KATSU_REQUIRE(dw == nullptr || x != nullptr, "dw needs the input");
    int handled = 0;
    KATSU_TRY(katsu_conv_stencil_bwd(ctx, x, w, gr, dx, dw, n, c, h, wd, k, r, s, stride, pad, accumulate, gscale,
                                     gfactor, &handled));
    if (handled) return KATSU_OK;
    if (gscale != nullptr || gfactor != 1.f) {
        // no kernel for this shape applies the scale itself: write the scaled gradient out once
        const size_t count = n * k * g.oh * g.ow;
        void *scaled = nullptr;
        KATSU_TRY(katsu_pool_alloc(ctx, count * sizeof(float), &scaled));
        int32_t rc = scale_copy(ctx, (float *)scaled, gr, gscale, gfactor, count);
        if (rc == KATSU_OK)
            rc = backward(ctx, x, w, (const float *)scaled, nullptr, 1.f, dx, dw, n, c, h, wd, k, r, s, stride, pad,
                          accumulate);
        cudaFreeAsync(scaled, ctx->stream);
        return rc;
    }
    ctx->share_g_staging = (dx != nullptr && dw != nullptr) ? 1 : 0;
    ctx->g_staged = 0;
    if (dx != nullptr) {
        KATSU_TRY(katsu_conv_igemm_dx(ctx, w, gr, dx, n, c, h, wd, k, r, s, stride, pad, g.oh, g.ow, accumulate, &handled));
        if (!handled)
            KATSU_TRY(katsu_conv_direct_dx(ctx, w, gr, dx, n, c, h, wd, k, r, s, stride, pad, g.oh, g.ow, accumulate));
    }
    if (dw != nullptr) {
        KATSU_TRY(katsu_conv_igemm_dw(ctx, x, gr, dw, n, c, h, wd, k, r, s, stride, pad, g.oh, g.ow, accumulate, &handled));
        if (!handled)
            KATSU_TRY(katsu_conv_direct_dw(ctx, x, gr, dw, n, c, h, wd, k, r, s, stride, pad, g.oh, g.ow, accumulate));
    }
    ctx->share_g_staging = ctx->g_staged = 0;
    return KATSU_OK;
}

}  // namespace

extern "C" int32_t katsu_cuda_conv2d_fwd(katsu_cuda_ctx *ctx, const float *x, const float *w, float *y,
                                         size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                                         size_t stride, size_t pad) {
    return forward(ctx, x, w, nullptr, y, n, c, h, wd, k, r, s, stride, pad, 0);
}

extern "C" int32_t katsu_cuda_conv2d_fwd_bias_relu(katsu_cuda_ctx *ctx, const float *x, const float *w, const float *bias,
                                                   float *y, size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r,
                                                   size_t s, size_t stride, size_t pad, int32_t relu) {
    return forward(ctx, x, w, bias, y, n, c, h, wd, k, r, s, stride, pad, relu ? 1 : 0);
}

// ---- the layer's input staged once for forward and backward ---------------------------------------------
// Conv2D keeps its input between forward and backward (crates/katsu-core/src/conv2d.rs:104-107, 130-136), and
// the wide-channel kernels of both read x through a channels-innermost copy: a caller that holds the input
// anyway can hold that copy too and pay for the pass once per step instead of twice.
extern "C" int32_t katsu_cuda_conv2d_staged_floats(katsu_cuda_ctx *ctx, size_t n, size_t c, size_t h, size_t wd, size_t k,
                                                   size_t r, size_t s, size_t stride, size_t pad, size_t *floats) {
    KATSU_REQUIRE(ctx != nullptr && floats != nullptr, "null argument");
    Geometry g;
    KATSU_TRY(geometry(c, h, wd, k, r, s, stride, pad, &g));
    *floats = 0;
    if (n == 0) return KATSU_OK;
    *floats = katsu_conv_igemm_staged_floats(ctx, n, c, h, wd, k, r, s, stride, pad, g.oh, g.ow);
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_conv2d_stage(katsu_cuda_ctx *ctx, const float *x, float *staged, size_t n, size_t c,
                                           size_t h, size_t wd) {
    KATSU_TRY(katsu_bind(ctx));
    KATSU_REQUIRE(x != nullptr && staged != nullptr, "null tensor");
    KATSU_REQUIRE(n > 0 && c > 0 && h > 0 && wd > 0, "empty input");
    // inputs for which katsu_cuda_conv2d_staged_floats reports 0 whatever the filter: nothing to write
    if (ctx->precision == KATSU_MODE_FP32 || c < 16 || (c & 3) != 0) return KATSU_OK;
    return katsu_conv_igemm_stage(ctx, x, staged, n, c, h, wd);
}

extern "C" int32_t katsu_cuda_conv2d_fwd_staged(katsu_cuda_ctx *ctx, const float *x, const float *x_staged, const float *w,
                                                const float *bias, float *y, size_t n, size_t c, size_t h, size_t wd,
                                                size_t k, size_t r, size_t s, size_t stride, size_t pad, int32_t relu) {
    KATSU_REQUIRE(ctx != nullptr, "null context");
    ctx->x_prestaged = x_staged;
    const int32_t rc = forward(ctx, x, w, bias, y, n, c, h, wd, k, r, s, stride, pad, relu ? 1 : 0);
    ctx->x_prestaged = nullptr;
    return rc;
}

extern "C" int32_t katsu_cuda_conv2d_bwd_staged(katsu_cuda_ctx *ctx, const float *x, const float *x_staged, const float *w,
                                                const float *gr, const float *gscale, float gfactor, float *dx, float *dw,
                                                size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                                                size_t stride, size_t pad, int32_t accumulate) {
    KATSU_REQUIRE(ctx != nullptr, "null context");
    ctx->x_prestaged = x_staged;
    const int32_t rc = backward(ctx, x, w, gr, gscale, gfactor, dx, dw, n, c, h, wd, k, r, s, stride, pad, accumulate);
    ctx->x_prestaged = nullptr;
    return rc;
}

extern "C" int32_t katsu_cuda_conv2d_bwd(katsu_cuda_ctx *ctx, const float *x, const float *w, const float *gr,
                                         float *dx, float *dw,
                                         size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                                         size_t stride, size_t pad, int32_t accumulate) {
    return backward(ctx, x, w, gr, nullptr, 1.f, dx, dw, n, c, h, wd, k, r, s, stride, pad, accumulate);
}

extern "C" int32_t katsu_cuda_conv2d_bwd_scaled(katsu_cuda_ctx *ctx, const float *x, const float *w, const float *gr,
                                                const float *gscale, float gfactor, float *dx, float *dw,
                                                size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                                                size_t stride, size_t pad, int32_t accumulate) {
    return backward(ctx, x, w, gr, gscale, gfactor, dx, dw, n, c, h, wd, k, r, s, stride, pad, accumulate);
}
