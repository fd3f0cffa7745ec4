// Elementwise and reduction kernels that keep the autograd graph on the
// device: the loops of crates/katsu-core/src/tensor.rs:226-247 (add, mul, sum)
// and the streaming VJP arms / adjoint accumulation of tensor.rs:353-417.
// All are HBM-bound: 128-bit accesses, grid sized to a multiple of the SM count.
#include "common.cuh"

namespace {

enum class Ew { Add, Mul, AxpyAcc, MulAcc, BcastAcc };

template <Ew OP>
__device__ __forceinline__ float ew_apply(float dst, float a, float b) {
    if (OP == Ew::Add) return a + b;
    if (OP == Ew::Mul) return a * b;
    if (OP == Ew::AxpyAcc) return dst + a;
    if (OP == Ew::MulAcc) return dst + a * b;
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
            acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
        }
        for (size_t i = v_end * 4 + threadIdx.x; i < end; i += blockDim.x) acc[0] += a[i];
    } else {
        for (size_t i = begin + threadIdx.x; i < end; i += blockDim.x) acc[0] += a[i];
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

}  // namespace

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

extern "C" int32_t katsu_cuda_sum(katsu_cuda_ctx *ctx, const float *a, float *out, size_t count) {
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
    KATSU_LAUNCH(ctx, sum_partial_kernel, (unsigned)parts, 256, 0, a, count, chunk, partial);
    KATSU_LAUNCH(ctx, sum_final_kernel, 1, 256, 0, partial, (int)parts, out);
    return KATSU_OK;
}
