// Context, memory, transfer and timing entry points of the C ABI.
#include <stdarg.h>
#include <string.h>

#include <new>

#include "common.cuh"
#include <stdlib.h>

static thread_local char g_error[512] = "";

int32_t katsu_set_error(int32_t code, const char *fmt, ...) {
    va_list args;
    va_start(args, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, args);
    va_end(args);
    return code;
}

extern "C" const char *katsu_cuda_last_error_string(void) { return g_error; }

int32_t katsu_bind(katsu_cuda_ctx *ctx) {
    if (ctx == nullptr) return katsu_set_error(KATSU_ERR_INVALID_ARG, "null context");
    KATSU_CUDA_TRY(cudaSetDevice(ctx->device));
    return KATSU_OK;
}

int32_t katsu_pool_alloc(katsu_cuda_ctx *ctx, size_t bytes, void **out) {
    cudaError_t err = ctx->pool != nullptr ? cudaMallocFromPoolAsync(out, bytes, (cudaMemPool_t)ctx->pool, ctx->stream)
                                           : cudaMallocAsync(out, bytes, ctx->stream);
    if (err != cudaSuccess) {
        cudaGetLastError();
        *out = nullptr;
        return katsu_set_error(KATSU_ERR_ALLOC, "stream-ordered allocation of %zu bytes: %s", bytes,
                               cudaGetErrorString(err));
    }
    return KATSU_OK;
}

int32_t katsu_scratch(katsu_cuda_ctx *ctx, size_t floats, float **out) {
    if (floats > ctx->scratch_floats) {
        // Stream-ordered: launches already queued keep the old block until they have run, and the
        // new one comes from the context's pool, so growing the scratch does not stall the device.
        if (ctx->scratch) KATSU_CUDA_TRY(cudaFreeAsync(ctx->scratch, ctx->stream));
        ctx->scratch = nullptr;
        ctx->scratch_floats = 0;
        size_t want = floats < (size_t(1) << 20) ? (size_t(1) << 20) : floats;
        void *p = nullptr;
        KATSU_TRY(katsu_pool_alloc(ctx, want * sizeof(float), &p));
        ctx->scratch = (float *)p;
        ctx->scratch_floats = want;
    }
    *out = ctx->scratch;
    return KATSU_OK;
}

// Reads the status word of the bounded device-side waits after the host has waited for the stream
// (or for an event behind the kernels in question).  A non-zero word means some wait gave up: the
// results behind it are undefined, so every synchronising entry point reports it, and the word is
// cleared so that the context's next launches run normally again.
static int32_t katsu_report_status(katsu_cuda_ctx *ctx, int status) {
    if (status == 0) return KATSU_OK;
    cudaMemsetAsync(ctx->status, 0, sizeof(int), ctx->stream);
    cudaStreamSynchronize(ctx->stream);
    return katsu_set_error(KATSU_ERR_TIMEOUT, "a device-side wait gave up (status word %d)", status);
}

// Waits for the context's stream; the status word travels behind the queued work into a page-locked
// mirror, so the check costs no second synchronisation.
int32_t katsu_sync_and_check(katsu_cuda_ctx *ctx) {
    KATSU_CUDA_TRY(cudaMemcpyAsync(ctx->status_host, ctx->status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    KATSU_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return katsu_report_status(ctx, *ctx->status_host);
}

extern "C" int32_t katsu_cuda_device_count(int32_t *out_count) {
    KATSU_REQUIRE(out_count != nullptr, "out_count is null");
    int n = 0;
    cudaError_t err = cudaGetDeviceCount(&n);
    if (err != cudaSuccess) {
        *out_count = 0;
        return katsu_set_error(KATSU_ERR_NO_DEVICE, "cudaGetDeviceCount: %s", cudaGetErrorString(err));
    }
    *out_count = n;
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_init(int32_t device, katsu_cuda_ctx **out_ctx) {
    KATSU_REQUIRE(out_ctx != nullptr, "out_ctx is null");
    *out_ctx = nullptr;
    int n = 0;
    cudaError_t err = cudaGetDeviceCount(&n);
    if (err != cudaSuccess || n == 0)
        return katsu_set_error(KATSU_ERR_NO_DEVICE, "no CUDA device: %s", cudaGetErrorString(err));
    if (device < 0 || device >= n)
        return katsu_set_error(KATSU_ERR_NO_DEVICE, "device ordinal %d out of range (0..%d)", device, n - 1);
    KATSU_CUDA_TRY(cudaSetDevice(device));
    cudaDeviceProp prop;
    KATSU_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return katsu_set_error(KATSU_ERR_NO_DEVICE,
                               "device %d is sm_%d%d; this library only carries sm_100a code", device,
                               prop.major, prop.minor);
    katsu_cuda_ctx *ctx = new (std::nothrow) katsu_cuda_ctx();
    if (ctx == nullptr) return katsu_set_error(KATSU_ERR_ALLOC, "out of host memory");
    memset(ctx, 0, sizeof(*ctx));
    ctx->device = device;
    ctx->num_sms = prop.multiProcessorCount;
    ctx->precision = KATSU_MODE_3XTF32;
    // katsu_cuda_alloc / katsu_cuda_free and the kernels' scratch are stream-ordered allocations
    // from a pool private to this context that keeps freed blocks cached: an autograd step
    // allocates and frees the same few hundred MB of adjoint buffers every time, and cudaMalloc /
    // cudaFree each cost a device-wide synchronisation (measured: 34 ms -> a few ms per step of
    // the small CNN).  The pool is the context's own, so the host program's other users of the
    // device's default pool keep their release behaviour; it is destroyed at shutdown.
    {
        cudaMemPoolProps props;
        memset(&props, 0, sizeof(props));
        props.allocType = cudaMemAllocationTypePinned;
        props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice;
        props.location.id = device;
        cudaMemPool_t pool = nullptr;
        if (cudaMemPoolCreate(&pool, &props) == cudaSuccess) {
            unsigned long long keep = ~0ull;
            cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
            ctx->pool = pool;
        }
        cudaGetLastError();  // without a private pool the allocations fall back to cudaMallocAsync's default pool
    }
    err = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (err == cudaSuccess) err = cudaMalloc(&ctx->status, sizeof(int));
    if (err == cudaSuccess) err = cudaHostAlloc((void **)&ctx->status_host, sizeof(int), cudaHostAllocDefault);
    if (err == cudaSuccess) err = cudaMemsetAsync(ctx->status, 0, sizeof(int), ctx->stream);
    if (err != cudaSuccess) {
        if (ctx->status_host) cudaFreeHost(ctx->status_host);
        if (ctx->status) cudaFree(ctx->status);
        if (ctx->stream) cudaStreamDestroy(ctx->stream);
        if (ctx->pool) cudaMemPoolDestroy((cudaMemPool_t)ctx->pool);
        cudaGetLastError();
        delete ctx;
        return katsu_set_error(KATSU_ERR_CUDA, "context setup: %s", cudaGetErrorString(err));
    }
    *ctx->status_host = 0;
    *out_ctx = ctx;
    return KATSU_OK;
}

int32_t katsu_comm_destroy_impl(katsu_cuda_ctx *ctx);

extern "C" int32_t katsu_cuda_shutdown(katsu_cuda_ctx *ctx) {
    KATSU_TRY(katsu_bind(ctx));
    cudaStreamSynchronize(ctx->stream);
    if (ctx->comm) katsu_comm_destroy_impl(ctx);
    if (ctx->scratch) cudaFreeAsync(ctx->scratch, ctx->stream);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->flush) cudaFree(ctx->flush);
    if (ctx->status) cudaFree(ctx->status);
    if (ctx->status_host) cudaFreeHost(ctx->status_host);
    cudaStreamDestroy(ctx->stream);
    // blocks still held by the caller stay valid: the driver releases the pool with its last allocation
    if (ctx->pool) cudaMemPoolDestroy((cudaMemPool_t)ctx->pool);
    cudaGetLastError();
    delete ctx;
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_set_precision(katsu_cuda_ctx *ctx, int32_t mode) {
    KATSU_REQUIRE(ctx != nullptr, "null context");
    KATSU_REQUIRE(mode == KATSU_MODE_3XTF32 || mode == KATSU_MODE_TF32 || mode == KATSU_MODE_FP32,
                  "unknown precision mode");
    ctx->precision = mode;
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_get_precision(katsu_cuda_ctx *ctx, int32_t *out_mode) {
    KATSU_REQUIRE(ctx != nullptr && out_mode != nullptr, "null argument");
    *out_mode = ctx->precision;
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_launch_count(katsu_cuda_ctx *ctx, uint64_t *out_count) {
    KATSU_REQUIRE(ctx != nullptr && out_count != nullptr, "null argument");
    *out_count = ctx->launches;
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_stream(katsu_cuda_ctx *ctx, void **out_stream) {
    KATSU_REQUIRE(ctx != nullptr && out_stream != nullptr, "null argument");
    *out_stream = (void *)ctx->stream;
    return KATSU_OK;
}

// ---- memory ----------------------------------------------------------------
extern "C" int32_t katsu_cuda_alloc(katsu_cuda_ctx *ctx, size_t count, float **out_ptr) {
    KATSU_REQUIRE(out_ptr != nullptr, "out_ptr is null");
    *out_ptr = nullptr;
    KATSU_TRY(katsu_bind(ctx));
    if (count == 0) return KATSU_OK;
    if (count > SIZE_MAX / sizeof(float))
        return katsu_set_error(KATSU_ERR_ALLOC, "allocation of %zu floats overflows", count);
    float *p = nullptr;
    KATSU_TRY(katsu_pool_alloc(ctx, count * sizeof(float), (void **)&p));
    cudaError_t err = cudaMemsetAsync(p, 0, count * sizeof(float), ctx->stream);
    if (err != cudaSuccess) {
        cudaFreeAsync(p, ctx->stream);
        return katsu_set_error(KATSU_ERR_CUDA, "cudaMemsetAsync: %s", cudaGetErrorString(err));
    }
    *out_ptr = p;
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_free(katsu_cuda_ctx *ctx, float *ptr) {
    KATSU_TRY(katsu_bind(ctx));
    if (ptr == nullptr) return KATSU_OK;
    // Stream-ordered: work already queued on this context's stream may still use the block;
    // work queued on another context must have been synchronised by the caller.
    KATSU_CUDA_TRY(cudaFreeAsync(ptr, ctx->stream));
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_zero(katsu_cuda_ctx *ctx, float *dst, size_t count) {
    KATSU_TRY(katsu_bind(ctx));
    if (count == 0) return KATSU_OK;
    KATSU_REQUIRE(dst != nullptr, "dst is null");
    KATSU_CUDA_TRY(cudaMemsetAsync(dst, 0, count * sizeof(float), ctx->stream));
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_h2d(katsu_cuda_ctx *ctx, float *dst_device, const float *src_host, size_t count) {
    KATSU_TRY(katsu_bind(ctx));
    if (count == 0) return KATSU_OK;
    KATSU_REQUIRE(dst_device != nullptr && src_host != nullptr, "null buffer");
    KATSU_CUDA_TRY(cudaMemcpyAsync(dst_device, src_host, count * sizeof(float), cudaMemcpyHostToDevice,
                                   ctx->stream));
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_d2h(katsu_cuda_ctx *ctx, float *dst_host, const float *src_device, size_t count) {
    KATSU_TRY(katsu_bind(ctx));
    if (count != 0) {
        KATSU_REQUIRE(dst_host != nullptr && src_device != nullptr, "null buffer");
        KATSU_CUDA_TRY(cudaMemcpyAsync(dst_host, src_device, count * sizeof(float), cudaMemcpyDeviceToHost,
                                       ctx->stream));
    }
    // the data is only as good as the kernels that produced it: a wait that gave up is reported here too
    return katsu_sync_and_check(ctx);
}

extern "C" int32_t katsu_cuda_d2h_async(katsu_cuda_ctx *ctx, float *dst_host, const float *src_device, size_t count) {
    KATSU_TRY(katsu_bind(ctx));
    if (count == 0) return KATSU_OK;
    KATSU_REQUIRE(dst_host != nullptr && src_device != nullptr, "null buffer");
    KATSU_CUDA_TRY(cudaMemcpyAsync(dst_host, src_device, count * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_d2d(katsu_cuda_ctx *ctx, float *dst_device, const float *src_device, size_t count) {
    KATSU_TRY(katsu_bind(ctx));
    if (count == 0) return KATSU_OK;
    KATSU_REQUIRE(dst_device != nullptr && src_device != nullptr, "null buffer");
    KATSU_CUDA_TRY(cudaMemcpyAsync(dst_device, src_device, count * sizeof(float), cudaMemcpyDeviceToDevice,
                                   ctx->stream));
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_host_alloc(katsu_cuda_ctx *ctx, size_t count, float **out_ptr) {
    KATSU_REQUIRE(out_ptr != nullptr, "out_ptr is null");
    *out_ptr = nullptr;
    KATSU_TRY(katsu_bind(ctx));
    if (count == 0) return KATSU_OK;
    void *p = nullptr;
    cudaError_t err = cudaHostAlloc(&p, count * sizeof(float), cudaHostAllocDefault);
    if (err != cudaSuccess) {
        cudaGetLastError();
        return katsu_set_error(KATSU_ERR_ALLOC, "cudaHostAlloc(%zu bytes): %s", count * sizeof(float),
                               cudaGetErrorString(err));
    }
    *out_ptr = (float *)p;
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_host_free(katsu_cuda_ctx *ctx, float *ptr) {
    KATSU_TRY(katsu_bind(ctx));
    if (ptr == nullptr) return KATSU_OK;
    KATSU_CUDA_TRY(cudaFreeHost(ptr));
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_sync(katsu_cuda_ctx *ctx) {
    KATSU_TRY(katsu_bind(ctx));
    return katsu_sync_and_check(ctx);
}

// ---- timing ----------------------------------------------------------------
extern "C" int32_t katsu_cuda_event_create(katsu_cuda_ctx *ctx, katsu_cuda_event **out_event) {
    KATSU_REQUIRE(out_event != nullptr, "out_event is null");
    KATSU_TRY(katsu_bind(ctx));
    katsu_cuda_event *e = new (std::nothrow) katsu_cuda_event();
    if (e == nullptr) return katsu_set_error(KATSU_ERR_ALLOC, "out of host memory");
    cudaError_t err = cudaEventCreate(&e->ev);
    if (err != cudaSuccess) {
        delete e;
        return katsu_set_error(KATSU_ERR_CUDA, "cudaEventCreate: %s", cudaGetErrorString(err));
    }
    *out_event = e;
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_event_record(katsu_cuda_ctx *ctx, katsu_cuda_event *event) {
    KATSU_REQUIRE(event != nullptr, "event is null");
    KATSU_TRY(katsu_bind(ctx));
    KATSU_CUDA_TRY(cudaEventRecord(event->ev, ctx->stream));
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_wait_event(katsu_cuda_ctx *ctx, katsu_cuda_event *event) {
    KATSU_REQUIRE(event != nullptr, "event is null");
    KATSU_TRY(katsu_bind(ctx));
    KATSU_CUDA_TRY(cudaStreamWaitEvent(ctx->stream, event->ev, 0));
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_event_elapsed_ms(katsu_cuda_ctx *ctx, katsu_cuda_event *start,
                                               katsu_cuda_event *stop, float *out_ms) {
    KATSU_REQUIRE(start != nullptr && stop != nullptr && out_ms != nullptr, "null argument");
    KATSU_TRY(katsu_bind(ctx));
    KATSU_CUDA_TRY(cudaEventSynchronize(stop->ev));
    KATSU_CUDA_TRY(cudaEventElapsedTime(out_ms, start->ev, stop->ev));
    // The kernels in front of `stop` have run: a time measured over a wait that gave up is not a
    // measurement.  The word is read directly (work queued behind `stop` may still be running).
    int status = 0;
    KATSU_CUDA_TRY(cudaMemcpy(&status, ctx->status, sizeof(int), cudaMemcpyDeviceToHost));
    return katsu_report_status(ctx, status);
}

extern "C" int32_t katsu_cuda_event_destroy(katsu_cuda_ctx *ctx, katsu_cuda_event *event) {
    KATSU_TRY(katsu_bind(ctx));
    if (event == nullptr) return KATSU_OK;
    cudaEventDestroy(event->ev);
    delete event;
    return KATSU_OK;
}

extern "C" int32_t katsu_cuda_flush_l2(katsu_cuda_ctx *ctx) {
    KATSU_TRY(katsu_bind(ctx));
    const size_t floats = size_t(64) << 20;  // 256 MiB, twice the 126 MB L2
    if (ctx->flush == nullptr) {
        KATSU_CUDA_TRY(cudaMalloc(&ctx->flush, floats * sizeof(float)));
        ctx->flush_floats = floats;
    }
    KATSU_CUDA_TRY(cudaMemsetAsync(ctx->flush, 0, ctx->flush_floats * sizeof(float), ctx->stream));
    return KATSU_OK;
}
