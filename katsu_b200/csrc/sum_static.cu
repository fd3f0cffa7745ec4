// katsu_cuda_sum_static: the sum reduction for callers that must not allocate.
//
// Who that is: a host program whose device memory is handed out entirely by
// its own pool (a framework allocator that has reserved all of HBM, so a
// cudaMalloc made behind its back fails), and latency-sensitive loops that
// cannot accept an allocation of any kind on their path.
// katsu_cuda_sum takes its partials from the context's scratch block, which
// grows on demand with an allocation from the context's memory pool; this
// variant keeps its per-block partial sums in a fixed array that is part of
// the library image instead, so it calls no cudaMalloc, cudaFree or any
// other allocating routine, ever.
//
// Cost and limits: every GPU that loads the library holds the 16 KiB array
// until the process exits.  At most KATSU_SUM_STATIC_MAX_COUNT elements per
// call.  All calls on a device share the one array: it keeps the previous
// call's partials (each call overwrites every slot it later reads, so nothing
// needs clearing), and two calls that overlap on the GPU -- different
// contexts or streams on the same device -- race on it.  Calls through one
// context are ordered by its stream and are safe.
//
// The first call on a device looks up the array's device address (a host-side
// lookup, no allocation by this library); make that first call before any
// stream capture, and before the host program's pool reserves whatever device
// memory is left: the driver loads the library's kernels onto the device at
// their first use and may take memory for the module image then.
#include "common.cuh"

namespace {

constexpr int kSlots = 4096;                 // floats in the static scratch (16 KiB)
constexpr size_t kMaxChunk = size_t(1) << 18;  // elements folded by one block at most

// In host code this name is only a handle for cudaGetSymbolAddress; kernels get the
// looked-up device pointer as an argument.
static __device__ __align__(256) float g_sum_static_scratch[kSlots];

constexpr int kMaxDevices = 64;
float *g_scratch_address[kMaxDevices] = {nullptr};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__global__ void __launch_bounds__(256) sum_static_partial_kernel(const float *__restrict__ a, size_t count,
                                                                 size_t chunk, float *__restrict__ partial) {
    const size_t begin = size_t(blockIdx.x) * chunk;
    size_t end = begin + chunk;
    if (end > count) end = count;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if ((reinterpret_cast<uintptr_t>(a) & 15u) == 0) {  // chunk is a multiple of 4
        const float4 *a4 = reinterpret_cast<const float4 *>(a);
        const size_t v_end = end / 4;
        for (size_t i = begin / 4 + threadIdx.x; i < v_end; i += blockDim.x) {
            const float4 v = a4[i];
            acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
        }
        for (size_t i = v_end * 4 + threadIdx.x; i < end; i += blockDim.x) acc[0] += a[i];
    } else {
        for (size_t i = begin + threadIdx.x; i < end; i += blockDim.x) acc[0] += a[i];
    }
    const float v = warp_sum((acc[0] + acc[1]) + (acc[2] + acc[3]));
    __shared__ float warp_part[8];
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < 8 ? warp_part[threadIdx.x] : 0.f;
        t = warp_sum(t);
        if (threadIdx.x == 0) partial[blockIdx.x] = t;
    }
}

__global__ void __launch_bounds__(256) sum_static_final_kernel(const float *__restrict__ partial, int parts,
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

// Once per device, with that device current (katsu_bind has just made it so).
int32_t scratch_for(const katsu_cuda_ctx *ctx, float **out) {
    if (ctx->device < 0 || ctx->device >= kMaxDevices)
        return katsu_set_error(KATSU_ERR_UNSUPPORTED, "device ordinal %d beyond %d", ctx->device, kMaxDevices - 1);
    if (g_scratch_address[ctx->device] == nullptr) {
        float *ptr = nullptr;
        KATSU_CUDA_TRY(cudaGetSymbolAddress((void **)&ptr, g_sum_static_scratch));
        g_scratch_address[ctx->device] = ptr;
    }
    *out = g_scratch_address[ctx->device];
    return KATSU_OK;
}

}  // namespace

extern "C" int32_t katsu_cuda_sum_static(katsu_cuda_ctx *ctx, const float *a, float *out, size_t count) {
    KATSU_TRY(katsu_bind(ctx));
    KATSU_REQUIRE(out != nullptr, "out is null");
    if (count > KATSU_SUM_STATIC_MAX_COUNT)
        return katsu_set_error(KATSU_ERR_UNSUPPORTED,
                               "katsu_cuda_sum_static handles at most %zu elements per call, got %zu "
                               "(use katsu_cuda_sum, which sizes its scratch on demand)",
                               (size_t)KATSU_SUM_STATIC_MAX_COUNT, count);
    if (count == 0) {
        KATSU_CUDA_TRY(cudaMemsetAsync(out, 0, sizeof(float), ctx->stream));
        return KATSU_OK;
    }
    KATSU_REQUIRE(a != nullptr, "a is null");
    float *partial = nullptr;
    KATSU_TRY(scratch_for(ctx, &partial));
    size_t chunk = katsu_div_up(count, size_t(ctx->num_sms) * 8);
    chunk = katsu_div_up(chunk, 1024) * 1024;
    if (chunk > kMaxChunk) chunk = kMaxChunk;
    const size_t parts = katsu_div_up(count, chunk);  // <= kSlots because count <= kSlots * kMaxChunk
    KATSU_LAUNCH(ctx, sum_static_partial_kernel, (unsigned)parts, 256, 0, a, count, chunk, partial);
    KATSU_LAUNCH(ctx, sum_static_final_kernel, 1, 256, 0, partial, (int)parts, out);
    return KATSU_OK;
}
