/*
 * katsu_cuda.h -- C ABI of libkatsu_cuda.so, the sm_100a replacement for
 * katsu-core's dense CPU loops.
 *
 * The reference (pure Rust, crates/katsu-core) has no FFI of its own; these
 * are the entry points a `katsu-cuda` sys-crate binds with an `extern "C"`
 * block so that the arithmetic call sites of katsu-core can be redirected to
 * the GPU.  Each declaration cites the reference lines it stands in for.
 *
 * Conventions
 *  - every function returns an int32_t status (KATSU_OK == 0); nothing throws,
 *    aborts or prints.  katsu_cuda_last_error_string() describes the most
 *    recent failure on the calling thread.
 *  - all tensors are contiguous row-major f32; device pointers come from
 *    katsu_cuda_alloc (or any cudaMalloc'ed memory on the context's device).
 *  - sizes are size_t like the reference's usize; the caller has already run
 *    the reference's shape validation (Geometry::new, matmul rank checks);
 *    the library re-checks what it needs and never launches on bad input.
 *  - one context == one device == one stream; calls are asynchronous on that
 *    stream and ordered with each other; katsu_cuda_sync / katsu_cuda_d2h wait.
 *  - one host thread drives a context (the reference's Tensor is Rc-based and
 *    !Send, crates/katsu-core/src/tensor.rs:95-99).
 */
#ifndef KATSU_CUDA_H
#define KATSU_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KATSU_OK 0
#define KATSU_ERR_INVALID_ARG 1  /* null pointer, zero stride, inconsistent sizes */
#define KATSU_ERR_ALLOC 2        /* device or pinned allocation failed (TensorError::Allocation) */
#define KATSU_ERR_CUDA 3         /* a CUDA runtime call or launch failed */
#define KATSU_ERR_NCCL 4         /* NCCL missing or a collective failed */
#define KATSU_ERR_TIMEOUT 5      /* a bounded device-side wait ran out */
#define KATSU_ERR_NO_DEVICE 6    /* no usable CUDA device / bad ordinal */
#define KATSU_ERR_UNSUPPORTED 7  /* shape outside what the requested kernel handles */

/* Arithmetic modes for the contraction kernels.  FP32 = CUDA-core fma.rn.f32.
 * 3XTF32 = tensor-core split precision (hi*hi + lo*hi + hi*lo into an f32
 * accumulator), FP32-grade accuracy.  TF32 = single tensor-core pass. Kernels
 * that run on CUDA cores (low-channel stencils, streaming ops) ignore it. */
#define KATSU_MODE_3XTF32 0
#define KATSU_MODE_TF32 1
#define KATSU_MODE_FP32 2

typedef struct katsu_cuda_ctx katsu_cuda_ctx;
typedef struct katsu_cuda_event katsu_cuda_event;

/* ---- context ----------------------------------------------------------- */
int32_t katsu_cuda_device_count(int32_t *out_count);
/* Binds one context to one device ordinal and creates its stream. */
int32_t katsu_cuda_init(int32_t device, katsu_cuda_ctx **out_ctx);
int32_t katsu_cuda_shutdown(katsu_cuda_ctx *ctx);
int32_t katsu_cuda_set_precision(katsu_cuda_ctx *ctx, int32_t mode);
int32_t katsu_cuda_get_precision(katsu_cuda_ctx *ctx, int32_t *out_mode);
const char *katsu_cuda_last_error_string(void);
/* Number of kernels this context has launched so far (for benchmark reports). */
int32_t katsu_cuda_launch_count(katsu_cuda_ctx *ctx, uint64_t *out_count);
/* Raw cudaStream_t of the context, for callers that interleave their own work. */
int32_t katsu_cuda_stream(katsu_cuda_ctx *ctx, void **out_stream);

/* ---- memory ------------------------------------------------------------ */
/* Zero-filled device buffer of `count` floats: zeros_buffer,
 * crates/katsu-core/src/tensor.rs:120-125.  count == 0 yields a null pointer.
 * Allocation and release are ordered on the context's stream and served from a
 * cached pool, so a step that frees and re-allocates its buffers does not
 * synchronise the device.  A buffer must be freed through a context whose
 * stream has seen (or been synchronised with) its last use. */
int32_t katsu_cuda_alloc(katsu_cuda_ctx *ctx, size_t count, float **out_ptr);
int32_t katsu_cuda_free(katsu_cuda_ctx *ctx, float *ptr);
int32_t katsu_cuda_zero(katsu_cuda_ctx *ctx, float *dst, size_t count);
/* Explicit host<->device transfer for the device storage variant of
 * TensorNode.data (crates/katsu-core/src/tensor.rs:101-107).  d2h waits for the
 * stream (and, like katsu_cuda_sync, returns KATSU_ERR_TIMEOUT when a bounded
 * device-side wait gave up in a kernel before it: the data is then undefined).
 * h2d is ordered on the stream; from pageable memory it returns once the source
 * has been staged, a page-locked source (katsu_cuda_host_alloc) must stay
 * untouched until the next katsu_cuda_sync. */
int32_t katsu_cuda_h2d(katsu_cuda_ctx *ctx, float *dst_device, const float *src_host, size_t count);
int32_t katsu_cuda_d2h(katsu_cuda_ctx *ctx, float *dst_host, const float *src_device, size_t count);
/* d2h without the wait: ordered on the stream, dst_host (page-locked) is valid after the
 * next katsu_cuda_sync.  Lets a caller keep several contexts (streams) of one device busy,
 * e.g. copying one batch chunk out while the next one computes. */
int32_t katsu_cuda_d2h_async(katsu_cuda_ctx *ctx, float *dst_host, const float *src_device, size_t count);
int32_t katsu_cuda_d2d(katsu_cuda_ctx *ctx, float *dst_device, const float *src_device, size_t count);
/* Page-locked host staging buffers so h2d/d2h run at full PCIe rate. */
int32_t katsu_cuda_host_alloc(katsu_cuda_ctx *ctx, size_t count, float **out_ptr);
int32_t katsu_cuda_host_free(katsu_cuda_ctx *ctx, float *ptr);
/* Waits for everything queued on the context.  KATSU_ERR_TIMEOUT (once) when a bounded
 * device-side wait gave up in any kernel since the last synchronising call. */
int32_t katsu_cuda_sync(katsu_cuda_ctx *ctx);

/* ---- Conv2D ------------------------------------------------------------ */
/* y[n,k,oy,ox] = sum_{c,r,s} x[n,c,oy*stride+r-pad,ox*stride+s-pad] * w[k,c,r,s]
 * over the in-range taps.  Replaces the visit closure of Conv2D::forward,
 * crates/katsu-core/src/conv2d.rs:95-103 with 232-262.  x is [N,C,H,W], w is
 * [K,C,R,S], y is [N,K,OH,OW] with OH=(H+2*pad-R)/stride+1 (same for OW) and is
 * fully overwritten. */
int32_t katsu_cuda_conv2d_fwd(katsu_cuda_ctx *ctx, const float *x, const float *w, float *y,
                              size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                              size_t stride, size_t pad);
/* dx[xi] (+)= sum g[yi]*w[wi] and dw[wi] (+)= sum g[yi]*x[xi] over the same tap
 * set: one call == one backward_buffers, crates/katsu-core/src/conv2d.rs:269-292
 * (called from Conv2D::backward conv2d.rs:127-133 and the Conv2D VJP arm
 * tensor.rs:374-381).  dx or dw may be null to skip that output.  accumulate
 * != 0 adds the result to the existing contents, which folds in the
 * `pending[parent] += grad` pass of tensor.rs:383-390; dx and dw must not alias
 * each other. */
int32_t katsu_cuda_conv2d_bwd(katsu_cuda_ctx *ctx, const float *x, const float *w, const float *g,
                              float *dx, float *dw,
                              size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                              size_t stride, size_t pad, int32_t accumulate);

/* One backward_buffers (conv2d.rs:269-292) whose upstream gradient is gfactor * gscale[0] * g[i]
 * without that product ever being stored: gscale is a device scalar (null: 1).  The VJP of
 * loss = sum(y * y) hands the convolution exactly this, g = y with gfactor = 2 and gscale = the
 * adjoint of the loss (crates/katsu-core/src/tensor.rs:392-417), so the backward pass reads y where
 * it would otherwise write and re-read a gradient of y's size.  dX and dW are linear in the upstream
 * gradient; kernels that support it scale their outputs, others get the scaled gradient written
 * out once internally.  Same aliasing and accumulate rules as katsu_cuda_conv2d_bwd. */
int32_t katsu_cuda_conv2d_bwd_scaled(katsu_cuda_ctx *ctx, const float *x, const float *w, const float *g,
                                     const float *gscale, float gfactor, float *dx, float *dw,
                                     size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                                     size_t stride, size_t pad, int32_t accumulate);
/* y = act(conv(x, w) + bias[k]) with act = max(., 0) when relu != 0; bias may be null.  Bias and
 * ReLU are not in the reference yet (docs/roadmap.md:18-26 lists them as the next layer features);
 * here they ride in the convolution kernel's epilogue where it has one, so a layer's activation
 * costs no extra pass over y. */
int32_t katsu_cuda_conv2d_fwd_bias_relu(katsu_cuda_ctx *ctx, const float *x, const float *w, const float *bias,
                                        float *y, size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r,
                                        size_t s, size_t stride, size_t pad, int32_t relu);
/* The layer's input staged once for forward and backward.  Conv2D keeps its input between forward and
 * backward (crates/katsu-core/src/conv2d.rs:104-107, 130-136); the wide-channel kernels of both read x
 * through a channels-innermost copy that each call otherwise writes for itself.  A caller that holds x
 * anyway can hold that copy too:
 *   katsu_cuda_conv2d_staged_floats  *floats = size of the copy for this shape in the context's CURRENT
 *                                    precision mode, 0 when the shape's kernels use none;
 *   katsu_cuda_conv2d_stage          writes it into `staged` (device memory of that many floats);
 *   katsu_cuda_conv2d_fwd_staged     katsu_cuda_conv2d_fwd_bias_relu reading x through x_staged;
 *   katsu_cuda_conv2d_bwd_staged     katsu_cuda_conv2d_bwd_scaled reading x through x_staged (dW).
 * x_staged may be null (the plain calls).  The copy is only valid for the precision mode, x contents and
 * shape it was written for; results are bit-identical to the plain calls. */
int32_t katsu_cuda_conv2d_staged_floats(katsu_cuda_ctx *ctx, size_t n, size_t c, size_t h, size_t wd, size_t k,
                                        size_t r, size_t s, size_t stride, size_t pad, size_t *floats);
int32_t katsu_cuda_conv2d_stage(katsu_cuda_ctx *ctx, const float *x, float *staged, size_t n, size_t c, size_t h,
                                size_t wd);
int32_t katsu_cuda_conv2d_fwd_staged(katsu_cuda_ctx *ctx, const float *x, const float *x_staged, const float *w,
                                     const float *bias, float *y, size_t n, size_t c, size_t h, size_t wd,
                                     size_t k, size_t r, size_t s, size_t stride, size_t pad, int32_t relu);
int32_t katsu_cuda_conv2d_bwd_staged(katsu_cuda_ctx *ctx, const float *x, const float *x_staged, const float *w,
                                     const float *g, const float *gscale, float gfactor, float *dx, float *dw,
                                     size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                                     size_t stride, size_t pad, int32_t accumulate);
/* Backward of that epilogue over y_act [n, k, plane]: dg = g where y_act > 0 else 0 (relu != 0;
 * dg may alias g, or be null when only dbias is wanted), dbias[k] (+)= sum over n and the plane of
 * dg (null: skipped).  With relu == 0 the gradient passes through unchanged: pass dg = null and
 * feed g to katsu_cuda_conv2d_bwd. */
int32_t katsu_cuda_bias_relu_bwd(katsu_cuda_ctx *ctx, const float *y_act, const float *g, float *dg, float *dbias,
                                 size_t n, size_t k, size_t plane, int32_t relu, int32_t accumulate_bias);
/* w[i] -= lr * dw[i], the plain SGD update the roadmap names (docs/roadmap.md:21-22), so that a
 * training step's parameters never leave the device. */
int32_t katsu_cuda_sgd_step(katsu_cuda_ctx *ctx, float *w, const float *dw, float lr, size_t count);

/* ---- matmul ------------------------------------------------------------ */
/* c[m,n] = a[m,k] @ b[k,n]; Tensor::matmul, crates/katsu-core/src/tensor.rs:264-273.
 * c is fully overwritten (zero when k == 0). */
int32_t katsu_cuda_matmul_fwd(katsu_cuda_ctx *ctx, const float *a, const float *b, float *c,
                              size_t m, size_t k, size_t n);
/* da[m,k] (+)= g[m,n] @ b^T ; db[k,n] (+)= a^T @ g.  Matmul VJP arm,
 * crates/katsu-core/src/tensor.rs:418-445 (which accumulates into the pending
 * adjoints: pass accumulate != 0 for that behaviour).  da or db may be null.
 * da and db may be the same buffer only when m == k == n and the caller wants
 * the reference's "same parent, both edges" sum (tensor.rs:425-444): the buffer
 * then receives g @ b^T + a^T @ g (added to its contents when accumulate != 0). */
int32_t katsu_cuda_matmul_bwd(katsu_cuda_ctx *ctx, const float *a, const float *b, const float *g,
                              float *da, float *db, size_t m, size_t k, size_t n, int32_t accumulate);

/* ---- streaming ops that keep the autograd graph on the device ---------- */
/* out = a + b / out = a * b; Tensor::elementwise, tensor.rs:226-233. */
int32_t katsu_cuda_add(katsu_cuda_ctx *ctx, const float *a, const float *b, float *out, size_t count);
int32_t katsu_cuda_mul(katsu_cuda_ctx *ctx, const float *a, const float *b, float *out, size_t count);
/* out[0] = sum(a); Tensor::sum, tensor.rs:243-247.  Pairwise/tree order on the
 * device (the reference folds left to right). */
int32_t katsu_cuda_sum(katsu_cuda_ctx *ctx, const float *a, float *out, size_t count);
/* Same result as katsu_cuda_sum for callers that cannot allocate device memory (all of
 * it belongs to the host program's own pool, or the implicit synchronisation of
 * cudaMalloc is unacceptable).  Has no counterpart in the reference.  Its per-block
 * partial sums live in a 16 KiB array inside the library image, held by every GPU that
 * loads the library until exit; it calls no allocating routine.  At most
 * KATSU_SUM_STATIC_MAX_COUNT elements, more is refused with KATSU_ERR_UNSUPPORTED.  The
 * array is shared by all calls on a device and keeps the last call's partials: calls that
 * overlap on the GPU (other contexts or streams of the same device) race; calls through
 * one context are stream-ordered.  The first call on a device resolves the array's
 * address and should come before any stream capture, and before the host program's pool
 * takes the rest of the device memory (the driver may place the library's kernel image on
 * the device at that first use). */
#define KATSU_SUM_STATIC_MAX_COUNT ((size_t)1 << 30)
int32_t katsu_cuda_sum_static(katsu_cuda_ctx *ctx, const float *a, float *out, size_t count);
/* out[0] = sum_i a[i] * a[i]: Tensor::mul(a, a) followed by Tensor::sum (tensor.rs:226-247) in one
 * pass over a, every square rounded to f32 before it is added (as the product tensor would hold
 * it) and the same summation tree as katsu_cuda_sum, so the result equals the two-step one bit for
 * bit while the product tensor is never written. */
int32_t katsu_cuda_sumsq(katsu_cuda_ctx *ctx, const float *a, float *out, size_t count);
/* dst[i] (+)= s[0]*src[i] + s[0]*src[i]: both Mul VJP edges of q = y * y (tensor.rs:392-409) when
 * the adjoint of q is the broadcast of one device scalar s[0] (what the Sum VJP produces,
 * tensor.rs:410-417), without that broadcast being stored. */
int32_t katsu_cuda_square_vjp(katsu_cuda_ctx *ctx, float *dst, const float *src, const float *s, size_t count,
                              int32_t accumulate);
/* dst += g : Add VJP edge (tensor.rs:400-408), adjoint accumulation
 * (tensor.rs:387-389) and gradient publication (tensor.rs:353-356). */
int32_t katsu_cuda_axpy_acc(katsu_cuda_ctx *ctx, float *dst, const float *g, size_t count);
/* dst += g * other : Mul VJP edge, tensor.rs:400-408. */
int32_t katsu_cuda_mul_acc(katsu_cuda_ctx *ctx, float *dst, const float *g, const float *other, size_t count);
/* dst += g[0] : Sum VJP, tensor.rs:410-417. */
int32_t katsu_cuda_bcast_acc(katsu_cuda_ctx *ctx, float *dst, const float *g, size_t count);

/* ---- data-parallel gradient exchange (no counterpart in the reference,
 *      which is single-threaded; batch shards over GPUs and only dW sums) --- */
#define KATSU_COMM_ID_BYTES 128
int32_t katsu_cuda_comm_unique_id(uint8_t out_id[KATSU_COMM_ID_BYTES]);
int32_t katsu_cuda_comm_init(katsu_cuda_ctx *ctx, const uint8_t id[KATSU_COMM_ID_BYTES],
                             int32_t n_ranks, int32_t rank);
int32_t katsu_cuda_comm_destroy(katsu_cuda_ctx *ctx);
/* In-place sum over all ranks of a flat gradient bucket, on the context's stream.  Buckets of up to
 * 64 KiB on ranks that share a machine go through IPC-mapped mailboxes in one kernel per rank (a
 * bounded wait for the peers: a rank that never arrives shows as KATSU_ERR_TIMEOUT at the next
 * synchronising call); everything else is one ncclAllReduce.  Every rank receives the same bits. */
int32_t katsu_cuda_allreduce_sum(katsu_cuda_ctx *ctx, float *buf, size_t count);

/* ---- diagnostics (no counterpart in the reference) ------------------------ */
/* Launches one block that waits, for at most `cycles` SM clocks (1e3..2e8), on a barrier
 * nothing signals.  The wait gives up and the kernel returns; the next synchronising call
 * (katsu_cuda_sync, katsu_cuda_d2h, katsu_cuda_event_elapsed_ms) then returns
 * KATSU_ERR_TIMEOUT once and the context remains usable.  Exercises the bounded-wait path of
 * the pipelined kernels without faulting or hanging the device. */
int32_t katsu_cuda_selftest_wait_timeout(katsu_cuda_ctx *ctx, uint64_t cycles);
/* Runs the mailbox all-reduce with `ranks` (1..16) emulated ranks on this one device: buf holds
 * ranks * count floats (count <= 16384), rank r's bucket at r * count, and every bucket ends up
 * holding the sum.  absent > 0 leaves that many ranks out; the others give up after `cycles` SM
 * clocks (1e3..2e9) and the next synchronising call returns KATSU_ERR_TIMEOUT once. */
int32_t katsu_cuda_selftest_mailbox_allreduce(katsu_cuda_ctx *ctx, float *buf, int32_t ranks, size_t count,
                                              int32_t absent, uint64_t cycles);

/* ---- timing on the context's stream ------------------------------------ */
int32_t katsu_cuda_event_create(katsu_cuda_ctx *ctx, katsu_cuda_event **out_event);
int32_t katsu_cuda_event_record(katsu_cuda_ctx *ctx, katsu_cuda_event *event);
/* Waits for `stop`, then returns the milliseconds between the two records. */
int32_t katsu_cuda_event_elapsed_ms(katsu_cuda_ctx *ctx, katsu_cuda_event *start, katsu_cuda_event *stop,
                                    float *out_ms);
int32_t katsu_cuda_event_destroy(katsu_cuda_ctx *ctx, katsu_cuda_event *event);
/* Makes the work queued on `ctx` after this call wait, on the device, for everything that was
 * queued before `event` was last recorded (on this or another context of the same device).
 * The host does not block.  No counterpart in the reference (it has one thread and no queue);
 * it lets two contexts pipeline batch chunks without a host synchronisation per step. */
int32_t katsu_cuda_wait_event(katsu_cuda_ctx *ctx, katsu_cuda_event *event);
/* Overwrites a private buffer larger than L2 so the next kernel starts cold. */
int32_t katsu_cuda_flush_l2(katsu_cuda_ctx *ctx);

#ifdef __cplusplus
}
#endif
#endif /* KATSU_CUDA_H */
