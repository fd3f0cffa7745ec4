// Elementwise and reduction kernels that keep the autograd graph on the
// device: the loops of crates/katsu-core/src/tensor.rs:226-247 (add, mul, sum)
// and the streaming VJP arms / adjoint accumulation of tensor.rs:353-417.
// All are HBM-bound: 128-bit accesses, grid sized to a multiple of the SM count.
#include "common.cuh"

int32_t katsu_sum_impl(katsu_cuda_ctx *ctx, const float *a, float *out, size_t count, bool square);

namespace {

enum class Ew { Add, Mul, AxpyAcc, MulAcc, BcastAcc };

template <Ew OP>
__device__ __forceinline__ float ew_apply(float dst, float a, float b) {
    if (OP == Ew::Add) return a + b;
    if (OP == Ew::Mul) return a * b;
    if (OP == Ew::AxpyAcc) return dst + a;
    if (OP == Ew::MulAcc) return dst + __fmul_rn(a, b);  // product rounded on its own, as the reference's `+= g * other`
    return dst + a;  // BcastAcc: a is the broadcast scalar
}

// out[i] = f(out[i], a[i], b[i]).  `a` is a scalar pointer for BcastAcc.
// VEC = 4 uses 128-bit accesses on the 16-byte aligned body; the tail and
// unaligned buffers go through VEC = 1.
template <Ew OP, int VEC>
__global__ void __launch_bounds__(256) ew_kernel(float *out, const float *__restrict__ a,
                                                 const float *__restrict__ b, size_t count) {
    constexpr bool reads_dst = (OP == Ew::AxpyAcc || OP == Ew::MulAcc || OP == Ew::BcastAcc);
    constexpr bool reads_b = (OP == Ew::Add || OP == Ew::Mul || OP == Ew::MulAcc);
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    float scalar = 0.f;
    if (OP == Ew::BcastAcc) scalar = __ldg(a);
    if (VEC == 4) {
        const size_t nvec = count / 4;
        float4 *o4 = reinterpret_cast<float4 *>(out);
        const float4 *a4 = reinterpret_cast<const float4 *>(a);
        const float4 *b4 = reinterpret_cast<const float4 *>(b);
        for (; i < nvec; i += stride) {
            float4 d = reads_dst ? o4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            float4 av = (OP == Ew::BcastAcc) ? make_float4(scalar, scalar, scalar, scalar) : a4[i];
            float4 bv = reads_b ? b4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            d.x = ew_apply<OP>(d.x, av.x, bv.x);
            d.y = ew_apply<OP>(d.y, av.y, bv.y);
            d.z = ew_apply<OP>(d.z, av.z, bv.z);
            d.w = ew_apply<OP>(d.w, av.w, bv.w);
            o4[i] = d;
        }
    } else {
        for (; i < count; i += stride) {
            float d = reads_dst ? out[i] : 0.f;
            float av = (OP == Ew::BcastAcc) ? scalar : a[i];
            float bv = reads_b ? b[i] : 0.f;
            out[i] = ew_apply<OP>(d, av, bv);
        }
    }
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <Ew OP>
int32_t ew_launch(katsu_cuda_ctx *ctx, float *out, const float *a, const float *b, size_t count) {
    KATSU_TRY(katsu_bind(ctx));
    if (count == 0) return KATSU_OK;
    KATSU_REQUIRE(out != nullptr && a != nullptr, "null buffer");
    if (OP == Ew::Add || OP == Ew::Mul || OP == Ew::MulAcc) KATSU_REQUIRE(b != nullptr, "null buffer");
    const bool vec_ok = aligned16(out) && (OP == Ew::BcastAcc || aligned16(a)) && (b == nullptr || aligned16(b));
    const int threads = 256;
    const size_t max_blocks = size_t(ctx->num_sms) * 8;
    size_t body = vec_ok ? (count / 4) * 4 : 0;
    if (body) {
        size_t blocks = katsu_div_up(body / 4, threads);
        if (blocks > max_blocks) blocks = max_blocks;
        auto kernel = ew_kernel<OP, 4>;
        KATSU_LAUNCH(ctx, kernel, (unsigned)blocks, threads, 0, out, a, b, body);
    }
    if (body < count) {
        const size_t rest = count - body;
        size_t blocks = katsu_div_up(rest, threads);
        if (blocks > max_blocks) blocks = max_blocks;
        const float *a_tail = (OP == Ew::BcastAcc) ? a : a + body;
        auto kernel = ew_kernel<OP, 1>;
        KATSU_LAUNCH(ctx, kernel, (unsigned)blocks, threads, 0, out + body, a_tail, b ? b + body : nullptr, rest);
    }
    return KATSU_OK;
}

// ---- sum -------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Stage 1: block b folds elements b*chunk .. (b+1)*chunk into partial[b].
// Fixed assignment of elements to threads and a fixed tree make the result
// independent of scheduling (bit-reproducible run to run).
// SQUARE: every element is squared (one rounded multiply, as Tensor::mul would store it) on the way
// in, so sum(a * a) reads a once and the product tensor is never written.
template <bool SQUARE>
__device__ __forceinline__ float sum_term(float v) { return SQUARE ? __fmul_rn(v, v) : v; }

template <bool SQUARE>
__global__ void __launch_bounds__(256) sum_partial_kernel(const float *__restrict__ a, size_t count,
                                                          size_t chunk, float *__restrict__ partial) {
    const size_t begin = size_t(blockIdx.x) * chunk;
    size_t end = begin + chunk;
    if (end > count) end = count;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const bool vec = ((reinterpret_cast<uintptr_t>(a) & 15u) == 0) && (chunk % 4 == 0);
    if (vec) {
        const float4 *a4 = reinterpret_cast<const float4 *>(a);
        const size_t v_begin = begin / 4, v_end = end / 4;
        for (size_t i = v_begin + threadIdx.x; i < v_end; i += blockDim.x) {
            float4 v = a4[i];
            acc[0] += sum_term<SQUARE>(v.x); acc[1] += sum_term<SQUARE>(v.y);
            acc[2] += sum_term<SQUARE>(v.z); acc[3] += sum_term<SQUARE>(v.w);
        }
        for (size_t i = v_end * 4 + threadIdx.x; i < end; i += blockDim.x) acc[0] += sum_term<SQUARE>(a[i]);
    } else {
        for (size_t i = begin + threadIdx.x; i < end; i += blockDim.x) acc[0] += sum_term<SQUARE>(a[i]);
    }
    float v = warp_sum((acc[0] + acc[1]) + (acc[2] + acc[3]));
    __shared__ float warp_part[8];
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < 8 ? warp_part[threadIdx.x] : 0.f;
        t = warp_sum(t);
        if (threadIdx.x == 0) partial[blockIdx.x] = t;
    }
}

// Stage 2: one block folds the partials in f64 and writes out[0].
__global__ void __launch_bounds__(256) sum_final_kernel(const float *__restrict__ partial, int parts,
                                                        float *__restrict__ out) {
    double acc = 0.0;
    for (int i = threadIdx.x; i < parts; i += blockDim.x) acc += (double)partial[i];
    __shared__ double sh[256];
    sh[threadIdx.x] = acc;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) {
        if ((int)threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) out[0] = (float)sh[0];
}

// dst[i] (+)= t + t with t = fl(s[0] * src[i]): the two Mul VJP edges of q = y * y (both lead to y,
// tensor.rs:392-409) under an adjoint of q that is the broadcast scalar s[0] (the Sum VJP,
// tensor.rs:410-417).  The reference adds g*y into y's adjoint twice; (d + t) + t is kept in that order.
template <int VEC>
__global__ void __launch_bounds__(256) square_vjp_kernel(float *dst, const float *__restrict__ src,
                                                         const float *__restrict__ s, size_t count, int accumulate) {
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const float scalar = __ldg(s);
    if (VEC == 4) {
        const size_t nvec = count / 4;
        float4 *d4 = reinterpret_cast<float4 *>(dst);
        const float4 *s4 = reinterpret_cast<const float4 *>(src);
        for (; i < nvec; i += stride) {
            const float4 v = s4[i];
            float4 d = accumulate ? d4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            const float tx = __fmul_rn(scalar, v.x), ty = __fmul_rn(scalar, v.y), tz = __fmul_rn(scalar, v.z),
                        tw = __fmul_rn(scalar, v.w);
            d.x = (d.x + tx) + tx; d.y = (d.y + ty) + ty; d.z = (d.z + tz) + tz; d.w = (d.w + tw) + tw;
            d4[i] = d;
        }
    } else {
        for (; i < count; i += stride) {
            const float t = __fmul_rn(scalar, src[i]);
            const float d = accumulate ? dst[i] : 0.f;
            dst[i] = (d + t) + t;
        }
    }
}

// w[i] -= fl(lr * dw[i]): plain SGD (the multiply is rounded on its own so the step is defined
// independently of instruction selection).
template <int VEC>
__global__ void __launch_bounds__(256) sgd_kernel(float *w, const float *__restrict__ dw, float lr, size_t count) {
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (VEC == 4) {
        const size_t nvec = count / 4;
        float4 *w4 = reinterpret_cast<float4 *>(w);
        const float4 *g4 = reinterpret_cast<const float4 *>(dw);
        for (; i < nvec; i += stride) {
            float4 p = w4[i];
            const float4 g = g4[i];
            p.x -= __fmul_rn(lr, g.x); p.y -= __fmul_rn(lr, g.y); p.z -= __fmul_rn(lr, g.z); p.w -= __fmul_rn(lr, g.w);
            w4[i] = p;
        }
    } else {
        for (; i < count; i += stride) w[i] -= __fmul_rn(lr, dw[i]);
    }
}

// y[n, c, :] = act(y[n, c, :] + bias[c]) in place, act = max(., 0) when relu.  One block row per
// (n, c) plane segment; used behind the convolution kernels that have no fused epilogue.
__global__ void __launch_bounds__(256) bias_relu_kernel(float *y, const float *__restrict__ bias, size_t planes,
                                                        size_t plane, int channels, int relu) {
    const size_t total = planes * plane, stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int c = int((i / plane) % size_t(channels));
        float v = y[i] + (bias != nullptr ? __ldg(bias + c) : 0.f);
        if (relu) v = v > 0.f ? v : 0.f;
        y[i] = v;
    }
}

// Backward of act(conv + bias): dg = g where the activation passed (y_act > 0) else 0 (dg == g's
// values when there is no ReLU), and per block the sum of dg over its slice of one channel:
// partial[slice][c].  Slices are whole images, so the fold below adds them in image order.
__global__ void __launch_bounds__(256) bias_relu_bwd_kernel(const float *__restrict__ y_act, const float *__restrict__ g,
                                                            float *dg, float *__restrict__ partial, int n, int channels,
                                                            size_t plane, int images_per_slice, int relu) {
    const int c = blockIdx.x, slice = blockIdx.y;
    const int n0 = slice * images_per_slice;
    int n1 = n0 + images_per_slice;
    if (n1 > n) n1 = n;
    float acc = 0.f;
    for (int img = n0; img < n1; ++img) {
        const size_t base = (size_t(img) * channels + c) * plane;
        for (size_t p = threadIdx.x; p < plane; p += blockDim.x) {
            float v = g[base + p];
            if (relu && !(y_act[base + p] > 0.f)) v = 0.f;
            if (dg != nullptr) dg[base + p] = v;
            acc += v;
        }
    }
    acc = warp_sum(acc);
    __shared__ float warp_part[8];
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int q = 0; q < 8; ++q) t += warp_part[q];
        partial[size_t(slice) * channels + c] = t;
    }
}

__global__ void __launch_bounds__(256) bias_grad_fold_kernel(const float *__restrict__ partial, float *dbias, int channels,
                                                             int slices, int accumulate) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    float t = 0.f;
    for (int s = 0; s < slices; ++s) t += partial[size_t(s) * channels + c];
    dbias[c] = accumulate ? dbias[c] + t : t;
}

}  // namespace

int32_t katsu_bias_relu_inplace(katsu_cuda_ctx *ctx, float *y, const float *bias, size_t n, size_t k, size_t plane,
                                int relu) {
    if (n * k * plane == 0 || (bias == nullptr && !relu)) return KATSU_OK;
    size_t blocks = katsu_div_up(n * k * plane, 256);
    const size_t max_blocks = size_t(ctx->num_sms) * 8;
    if (blocks > max_blocks) blocks = max_blocks;
    KATSU_LAUNCH(ctx, bias_relu_kernel, (unsigned)blocks, 256, 0, y, bias, n * k, plane, (int)k, relu);
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_sumsq(katsu_cuda_ctx *ctx, const float *a, float *out, size_t count) {
    return katsu_sum_impl(ctx, a, out, count, true);
}

extern "C" int32_t katsu_cuda_square_vjp(katsu_cuda_ctx *ctx, float *dst, const float *src, const float *s, size_t count,
                                         int32_t accumulate) {
    KATSU_TRY(katsu_bind(ctx));
    if (count == 0) return KATSU_OK;
    KATSU_REQUIRE(dst != nullptr && src != nullptr && s != nullptr, "null buffer");
    const bool vec_ok = aligned16(dst) && aligned16(src);
    const size_t max_blocks = size_t(ctx->num_sms) * 8;
    const size_t body = vec_ok ? (count / 4) * 4 : 0;
    if (body) {
        size_t blocks = katsu_div_up(body / 4, 256);
        if (blocks > max_blocks) blocks = max_blocks;
        KATSU_LAUNCH(ctx, square_vjp_kernel<4>, (unsigned)blocks, 256, 0, dst, src, s, body, accumulate);
    }
    if (body < count) {
        size_t blocks = katsu_div_up(count - body, 256);
        if (blocks > max_blocks) blocks = max_blocks;
        KATSU_LAUNCH(ctx, square_vjp_kernel<1>, (unsigned)blocks, 256, 0, dst + body, src + body, s, count - body, accumulate);
    }
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_sgd_step(katsu_cuda_ctx *ctx, float *w, const float *dw, float lr, size_t count) {
    KATSU_TRY(katsu_bind(ctx));
    if (count == 0) return KATSU_OK;
    KATSU_REQUIRE(w != nullptr && dw != nullptr, "null buffer");
    KATSU_REQUIRE(w != dw, "w and dw must be different buffers");
    const bool vec_ok = aligned16(w) && aligned16(dw);
    const size_t max_blocks = size_t(ctx->num_sms) * 8;
    const size_t body = vec_ok ? (count / 4) * 4 : 0;
    if (body) {
        size_t blocks = katsu_div_up(body / 4, 256);
        if (blocks > max_blocks) blocks = max_blocks;
        KATSU_LAUNCH(ctx, sgd_kernel<4>, (unsigned)blocks, 256, 0, w, dw, lr, body);
    }
    if (body < count) {
        size_t blocks = katsu_div_up(count - body, 256);
        if (blocks > max_blocks) blocks = max_blocks;
        KATSU_LAUNCH(ctx, sgd_kernel<1>, (unsigned)blocks, 256, 0, w + body, dw + body, lr, count - body);
    }
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_bias_relu_bwd(katsu_cuda_ctx *ctx, const float *y_act, const float *g, float *dg,
                                            float *dbias, size_t n, size_t k, size_t plane, int32_t relu,
                                            int32_t accumulate_bias) {
    KATSU_TRY(katsu_bind(ctx));
    KATSU_REQUIRE(k >= 1 && k <= 65535 && n <= 0x7fffffff, "channel or batch count out of range");
    if (n * plane == 0) {
        if (dbias != nullptr && !accumulate_bias) KATSU_CUDA_TRY(cudaMemsetAsync(dbias, 0, k * sizeof(float), ctx->stream));
        return KATSU_OK;
    }
    KATSU_REQUIRE(g != nullptr, "null upstream gradient");
    KATSU_REQUIRE(!relu || y_act != nullptr, "the ReLU mask needs the activated output");
    KATSU_REQUIRE(dg != nullptr || dbias != nullptr, "nothing to compute");
    // slices of whole images: enough blocks to fill the GPU, folded in image order afterwards
    size_t slices = katsu_div_up(size_t(ctx->num_sms) * 4, k);
    if (slices > n) slices = n;
    if (slices > 65535) slices = 65535;
    const size_t per_slice = katsu_div_up(n, slices);
    slices = katsu_div_up(n, per_slice);
    float *partial = nullptr;
    KATSU_TRY(katsu_scratch(ctx, slices * k, &partial));
    dim3 grid((unsigned)k, (unsigned)slices);
    KATSU_LAUNCH(ctx, bias_relu_bwd_kernel, grid, 256, 0, y_act, g, dg, partial, (int)n, (int)k, plane, (int)per_slice,
                 relu);
    if (dbias != nullptr)
        KATSU_LAUNCH(ctx, bias_grad_fold_kernel, (unsigned)katsu_div_up(k, 256), 256, 0, partial, dbias, (int)k,
                     (int)slices, accumulate_bias);
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_add(katsu_cuda_ctx *ctx, const float *a, const float *b, float *out, size_t count) {
    return ew_launch<Ew::Add>(ctx, out, a, b, count);
}

extern "C" int32_t katsu_cuda_mul(katsu_cuda_ctx *ctx, const float *a, const float *b, float *out, size_t count) {
    return ew_launch<Ew::Mul>(ctx, out, a, b, count);
}

extern "C" int32_t katsu_cuda_axpy_acc(katsu_cuda_ctx *ctx, float *dst, const float *g, size_t count) {
    return ew_launch<Ew::AxpyAcc>(ctx, dst, g, nullptr, count);
}

extern "C" int32_t katsu_cuda_mul_acc(katsu_cuda_ctx *ctx, float *dst, const float *g, const float *other,
                                      size_t count) {
    return ew_launch<Ew::MulAcc>(ctx, dst, g, other, count);
}

extern "C" int32_t katsu_cuda_bcast_acc(katsu_cuda_ctx *ctx, float *dst, const float *g, size_t count) {
    return ew_launch<Ew::BcastAcc>(ctx, dst, g, nullptr, count);
}

int32_t katsu_sum_impl(katsu_cuda_ctx *ctx, const float *a, float *out, size_t count, bool square) {
    KATSU_TRY(katsu_bind(ctx));
    KATSU_REQUIRE(out != nullptr, "out is null");
    if (count == 0) {
        KATSU_CUDA_TRY(cudaMemsetAsync(out, 0, sizeof(float), ctx->stream));
        return KATSU_OK;
    }
    KATSU_REQUIRE(a != nullptr, "a is null");
    size_t parts = size_t(ctx->num_sms) * 8;
    size_t chunk = katsu_div_up(count, parts);
    chunk = katsu_div_up(chunk, 1024) * 1024;  // multiple of 4 so 128-bit loads stay aligned
    parts = katsu_div_up(count, chunk);
    float *partial = nullptr;
    KATSU_TRY(katsu_scratch(ctx, parts, &partial));
    if (square)
        KATSU_LAUNCH(ctx, sum_partial_kernel<true>, (unsigned)parts, 256, 0, a, count, chunk, partial);
    else
        KATSU_LAUNCH(ctx, sum_partial_kernel<false>, (unsigned)parts, 256, 0, a, count, chunk, partial);
    KATSU_LAUNCH(ctx, sum_final_kernel, 1, 256, 0, partial, (int)parts, out);
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_sum(katsu_cuda_ctx *ctx, const float *a, float *out, size_t count) {
    return katsu_sum_impl(ctx, a, out, count, false);
}
