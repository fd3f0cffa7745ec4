// Shared internals of libkatsu_cuda.so: the context object, error plumbing and
// small device helpers.  Nothing here is part of the C ABI (include/katsu_cuda.h).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include <stdio.h>

#include "katsu_cuda.h"

#define KATSU_NUM_SMS_B200 148

struct katsu_cuda_ctx {
    int device;
    int num_sms;
    int precision;
    cudaStream_t stream;
    uint64_t launches;
    // Scratch in global memory for per-block partial results (dW partials,
    // sum partials, split-K slabs).  Grown on demand, never shrunk, freed at
    // shutdown.  Only the context's stream touches it, so launches that use
    // it are serialised by stream order.
    float *scratch;
    size_t scratch_floats;
    // set by conv2d_bwd while one call computes both dX and dW on the implicit-GEMM path: the dX
    // launch stages g (channels-innermost copy) where the dW launch expects it, once for both
    int share_g_staging, g_staged;
    // set by the *_staged entry points for the duration of one call: the caller's channels-innermost copy
    // of x (hi, then lo in 3xTF32 mode), written by katsu_cuda_conv2d_stage; the forward and dW launches use
    // it instead of staging x themselves
    const float *x_prestaged;
    // Buffer written by katsu_cuda_flush_l2.
    float *flush;
    size_t flush_floats;
    // Device status word for bounded waits (0 = ok) and its page-locked host mirror.
    int *status;
    int *status_host;
    // cudaMemPool_t private to the context: katsu_cuda_alloc and the scratch come from it.
    void *pool;
    // NCCL communicator (void* so this header does not need nccl.h).
    void *comm;
    int comm_ranks;
    int comm_rank;
    // Mailbox all-reduce state of the communicator (collective.cu), null without a communicator.
    void *mailboxes;
};

struct katsu_cuda_event {
    cudaEvent_t ev;
};

// Records a message for katsu_cuda_last_error_string and returns `code`.
int32_t katsu_set_error(int32_t code, const char *fmt, ...);

// Makes the context's device current; returns a status.
int32_t katsu_bind(katsu_cuda_ctx *ctx);

// Ensures ctx->scratch holds at least `floats` floats.
int32_t katsu_scratch(katsu_cuda_ctx *ctx, size_t floats, float **out);

// Stream-ordered allocation from the context's pool.
int32_t katsu_pool_alloc(katsu_cuda_ctx *ctx, size_t bytes, void **out);

// cudaStreamSynchronize plus the status word of the bounded device-side waits: KATSU_ERR_TIMEOUT
// (once; the word is cleared) when a wait gave up in any launch since the last check.
int32_t katsu_sync_and_check(katsu_cuda_ctx *ctx);

#define KATSU_CUDA_TRY(expr)                                                              \
    do {                                                                                  \
        cudaError_t err__ = (expr);                                                       \
        if (err__ != cudaSuccess)                                                         \
            return katsu_set_error(err__ == cudaErrorMemoryAllocation ? KATSU_ERR_ALLOC   \
                                                                      : KATSU_ERR_CUDA,   \
                                   "%s failed: %s (%s:%d)", #expr,                        \
                                   cudaGetErrorString(err__), __FILE__, __LINE__);        \
    } while (0)

#define KATSU_TRY(expr)                   \
    do {                                  \
        int32_t rc__ = (expr);            \
        if (rc__ != KATSU_OK) return rc__; \
    } while (0)

#define KATSU_REQUIRE(cond, msg)                                          \
    do {                                                                  \
        if (!(cond)) return katsu_set_error(KATSU_ERR_INVALID_ARG, "%s", msg); \
    } while (0)

// After a <<<>>> launch: count it and surface launch-configuration errors.
#define KATSU_LAUNCHED(ctx)                                                        \
    do {                                                                           \
        (ctx)->launches += 1;                                                      \
        cudaError_t err__ = cudaGetLastError();                                    \
        if (err__ != cudaSuccess)                                                  \
            return katsu_set_error(KATSU_ERR_CUDA, "kernel launch failed: %s (%s:%d)", \
                                   cudaGetErrorString(err__), __FILE__, __LINE__); \
    } while (0)

// Launches `kernel` (a __global__ function or a pointer to one) on the
// context's stream, counts it and reports launch-configuration errors.
#ifndef KATSU_LAUNCH
#define KATSU_LAUNCH(ctx, kernel, grid, block, smem, ...)                   \
    do {                                                                    \
        kernel<<<(grid), (block), (smem), (ctx)->stream>>>(__VA_ARGS__);    \
        KATSU_LAUNCHED(ctx);                                                \
    } while (0)
#endif

// Start of the block's dynamic shared memory.
#ifndef KATSU_DYNAMIC_SMEM_DEFINED
__device__ __forceinline__ float *katsu_dynamic_smem() {
    extern __shared__ __align__(128) unsigned char katsu_smem_raw[];
    return reinterpret_cast<float *>(katsu_smem_raw);
}
#endif

static inline size_t katsu_div_up(size_t a, size_t b) { return (a + b - 1) / b; }

// Internal entry points shared between translation units.
int32_t katsu_conv_direct_fwd(katsu_cuda_ctx *ctx, const float *x, const float *w, float *y,
                              size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                              size_t stride, size_t pad, size_t oh, size_t ow);
int32_t katsu_conv_direct_dx(katsu_cuda_ctx *ctx, const float *w, const float *g, float *dx,
                             size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                             size_t stride, size_t pad, size_t oh, size_t ow, int accumulate);
int32_t katsu_conv_direct_dw(katsu_cuda_ctx *ctx, const float *x, const float *g, float *dw,
                             size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                             size_t stride, size_t pad, size_t oh, size_t ow, int accumulate);

// Tensor-core GEMM C[M,N] (+)= A * B (umma_gemm.cu).  a_mn / b_mn: the operand is stored
// with its M (resp. N) index contiguous rather than K.  *handled = 0 when the shape is not
// one it takes (alignment, size, FP32 mode); the caller then uses the CUDA-core kernels.
int32_t katsu_umma_gemm(katsu_cuda_ctx *ctx, const float *a, const float *b, float *c, size_t M, size_t N, size_t K,
                        bool a_mn, bool b_mn, int accumulate, int *handled);

// The same on pairs of thread blocks (umma_gemm_pair.cu): 256 x 128 tiles, half the B traffic per block.
// *handled = 0 when M is too small for that; operands already passed katsu_umma_gemm's alignment checks.
int32_t katsu_umma_gemm_pair(katsu_cuda_ctx *ctx, const float *a, const float *b, float *c, size_t M, size_t N, size_t K,
                             bool a_mn, bool b_mn, int accumulate, int *handled);
// Single-pass TF32 with 128 x 256 tiles (umma_gemm_wide.cu); *handled = 0 outside KATSU_MODE_TF32 or for small shapes.
int32_t katsu_umma_gemm_wide(katsu_cuda_ctx *ctx, const float *a, const float *b, float *c, size_t M, size_t N, size_t K,
                             bool a_mn, bool b_mn, int accumulate, int *handled);

// dW of a wide convolution through the GEMM kernel (umma_gemm.cu); maps and staging by the caller.
struct CUtensorMap_st;
int32_t katsu_umma_conv_dw(katsu_cuda_ctx *ctx, const CUtensorMap_st *map_g, const CUtensorMap_st *map_x,
                           const CUtensorMap_st *map_x_lo, float *partial, size_t k, size_t c, size_t taps,
                           size_t total_groups, size_t groups_x, size_t groups_per_img, size_t stride,
                           const short *off_y, const short *off_x, size_t splits, size_t groups_per_split,
                           int grouped_maps);

// Wide-channel implicit-GEMM convolution on the tensor cores (conv_igemm.cu); *handled = 0
// when the shape is outside what it takes.
// Floats of the staging copy of x that the implicit-GEMM kernels use for this shape in the context's precision
// mode (0 when the shape takes other kernels), and the pass that writes it.
size_t katsu_conv_igemm_staged_floats(const katsu_cuda_ctx *ctx, size_t n, size_t c, size_t h, size_t wd, size_t k,
                                      size_t r, size_t s, size_t stride, size_t pad, size_t oh, size_t ow);
int32_t katsu_conv_igemm_stage(katsu_cuda_ctx *ctx, const float *x, float *staged, size_t n, size_t c, size_t h,
                               size_t wd);
int32_t katsu_conv_igemm_fwd(katsu_cuda_ctx *ctx, const float *x, const float *w, float *y,
                             size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                             size_t stride, size_t pad, size_t oh, size_t ow, int *handled);
int32_t katsu_conv_igemm_dx(katsu_cuda_ctx *ctx, const float *w, const float *g, float *dx,
                            size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                            size_t stride, size_t pad, size_t oh, size_t ow, int accumulate, int *handled);
int32_t katsu_conv_igemm_dw(katsu_cuda_ctx *ctx, const float *x, const float *g, float *dw,
                            size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                            size_t stride, size_t pad, size_t oh, size_t ow, int accumulate, int *handled);

// Low-channel (C <= 3) 3x3 stride-1 pad-1 convolution on the tensor cores (conv_stem_tc.cu).
// bias (may be null) and relu are applied in the kernel's epilogue.
int32_t katsu_conv_stem_tc_fwd(katsu_cuda_ctx *ctx, const float *x, const float *w, float *y,
                               size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                               size_t stride, size_t pad, const float *bias, int relu, int *handled);

// y = act(y + bias[channel]) in place (streaming.cu), for the convolution kernels without a fused epilogue.
int32_t katsu_bias_relu_inplace(katsu_cuda_ctx *ctx, float *y, const float *bias, size_t n, size_t k, size_t plane,
                                int relu);

// dX of the same shape family on the tensor cores (conv_stem_tc_bwd.cu); *handled = 0 in FP32
// mode or when TMA cannot describe the tensors.
// The upstream gradient is gfactor * gscale[0] * g (gscale: device scalar or null for 1); the kernels
// apply the factor to their outputs, so g itself is only read.
int32_t katsu_conv_stem_tc_dx(katsu_cuda_ctx *ctx, const float *w, const float *g, float *dx, size_t n, size_t c,
                              size_t h, size_t wd, size_t k, int accumulate, const float *gscale, float gfactor,
                              int *handled);

int32_t katsu_conv_stem_tc_dw(katsu_cuda_ctx *ctx, const float *x, const float *g, float *dw, size_t n, size_t c,
                              size_t h, size_t wd, size_t k, int accumulate, const float *gscale, float gfactor,
                              int *handled);

// True when those two kernels take every output this backward call asks for.
bool katsu_conv_stem_tc_bwd_takes(const katsu_cuda_ctx *ctx, const float *x, const float *g, const float *dx,
                                  const float *dw, size_t n, size_t c, size_t h, size_t wd, size_t k);

// TMA-fed dX stencil (conv_stencil_tma.cu); *handled = 0 when TMA cannot describe g.
int32_t katsu_stencil_dx_tma(katsu_cuda_ctx *ctx, const float *w, const float *g, float *dx, size_t n, size_t c,
                             size_t h, size_t wd, size_t k, int accumulate, int *handled);

int32_t katsu_stencil_dw_tma(katsu_cuda_ctx *ctx, const float *x, const float *g, float *dw, size_t n, size_t c,
                             size_t h, size_t wd, size_t k, int accumulate, int *handled);

// Low-channel 3x3 stride-1 pad-1 stencil path; *handled = 0 when the shape is
// not one it covers (the caller then uses another kernel).
int32_t katsu_conv_stencil_fwd(katsu_cuda_ctx *ctx, const float *x, const float *w, float *y,
                               size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                               size_t stride, size_t pad, int *handled);
int32_t katsu_conv_stencil_bwd(katsu_cuda_ctx *ctx, const float *x, const float *w, const float *g,
                               float *dx, float *dw,
                               size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                               size_t stride, size_t pad, int accumulate, const float *gscale, float gfactor,
                               int *handled);
