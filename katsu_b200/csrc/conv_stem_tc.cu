// Low-channel (C_in <= 3) 3x3 stride-1 pad-1 convolution on the tensor cores.
//
// Why: this shape needs 27 multiply-adds per output element per pass; on the FP32 pipe
// that alone takes longer than moving the output through HBM (measured: the CUDA-core
// stencils of conv_stencil.cu sit at 22-48 % FMA-pipe utilisation and 9-24 % of HBM
// bandwidth).  As a GEMM with K = C_in*9 <= 27 padded to 32 the contraction is a few
// hundred tensor-pipe cycles per 128-pixel tile and the kernels become memory-bound.
//
// Reference loops: the visit closure of Conv2D::forward (crates/katsu-core/src/conv2d.rs:
// 95-103, 232-262) and backward_buffers (conv2d.rs:269-292).
//
// Forward:  Y[pixel, oc] = sum_tap Xcol[pixel, tap] * W[oc, tap]
//   A = Xcol, 128 pixels x 32 taps, held in TENSOR MEMORY (lane = pixel, column = tap) and
//       written there with tcgen05.st by "builder" threads from a halo tile of x that TMA
//       drops into shared memory (6 rows x 40 columns per channel, the start column rounded
//       down to a 16-byte boundary; out-of-image cells arrive as zeros == the reference's
//       skipped padding taps), as hi = trunc_tf32(v) and lo = v - hi; taps 27..31 are zero.
//   B = W, oc x 32 taps, K-major, built once per block (hi and lo).
//   D = 128 x oc f32 in tensor memory, several accumulators so epilogues overlap later MMAs.
//       3xTF32: lo*hi + hi*lo + hi*hi per k-step; TF32 mode: hi*hi.
// Blocks are persistent (two per SM up to 64 output channels, else one) and walk 4x32-pixel
// tiles with specialised warps (epilogue, builders, MMA issue, TMA loads of x; see the kernel).
// The backward kernels of the same shapes are in conv_stem_tc_bwd.cu.
// The output tile leaves through a shared-memory transpose and 128-bit global stores.
// Measured alternatives: 64 scalar 128-byte-per-warp stores per thread keep too few bytes
// in flight (6.5 B/clk per SM), and one TMA tensor store per tile (32 x 4 x K box, 128-byte
// inner rows) saturated near 16 B/clk per SM; the SM needs ~23 B/clk to fill HBM.
#include "common.cuh"
#include <string.h>

#include "sm100.cuh"

using namespace sm100;

namespace {

struct StemDims {
    int n, k, h, w;          // batch, output channels, image height / width
    int tiles_x, tiles_y;    // 32-pixel columns, 4-row bands
    int np;                  // output channels padded to a multiple of 32 (one TMEM load)
    int three_pass;
    int a_stages;            // 2 or 3 stages of the A tile
    int acc_buffers;         // 2 or 4 TMEM accumulators
    int *status;
    const float *bias;       // optional per-output-channel bias added in the epilogue (null: none)
    int relu;                // epilogue clamps at zero
};

__device__ __forceinline__ float tf32_hi(float v) { return __uint_as_float(__float_as_uint(v) & 0xFFFFE000u); }

// Writes one 16-byte chunk of a K-major 128-byte-swizzled row: chunk j of row r lands at
// chunk position j ^ (r & 7) (rows are 128 B apart, atoms of 8 rows are 1024 B aligned).
__device__ __forceinline__ void store_chunk(unsigned char *tile, int row, int chunk, float4 v) {
    st_shared_v4(tile + row * 128 + ((chunk ^ (row & 7)) << 4), v);
}

// Warp roles of the forward kernel, GROUPS = 1 or 2 (10 or 18 warps):
//   [0, 4G)      G epilogue groups (alternate tiles; warp % 4 selects the TMEM lane quarter)
//   [4G, 8G)     G builder groups (alternate tiles)
//   8G           MMA issue (one thread)      8G+1  TMA loads of the x halo tiles (one thread)
// GROUPS = 1 runs two blocks per SM (256 TMEM columns each) so that one block's hand-off
// latencies are covered by the other block's work; GROUPS = 2 is the single-block form for
// channel counts whose accumulators need more than 256 columns.
// Per-tile hand-offs cost several hundred cycles each, so every resource is buffered deeper
// than the role count: AS stages of A, NB accumulators, XS x tiles, one staging buffer per
// epilogue group.  A lives in tensor memory, not shared memory: with A in shared memory the
// block moved ~1450 128-byte shared-memory wavefronts per tile (A writes, three A operand
// reads, B reads, x reads, output staging) and was bound by that pipe; the tcgen05 form
// with A in TMEM leaves ~810.
//   TMEM columns: [NB accumulators x np][AS stages x {32 hi, 32 lo}]
constexpr int XS = 6;   // x halo tiles in flight

template <int CIN, int GROUPS>
__global__ void __launch_bounds__((8 * GROUPS + 2) * 32, GROUPS == 1 ? 2 : 1)
stem_fwd_tc_kernel(const float *__restrict__ w, float *__restrict__ y, const __grid_constant__ CUtensorMap map_x,
                   StemDims d) {
    constexpr int TAPS = CIN * 9;
    constexpr int XT = (CIN * 6 * 40 + 31) / 32 * 32;  // x stage pitch in floats: keeps stages 128-byte aligned
    constexpr int FWD_THREADS = (8 * GROUPS + 2) * 32;
    constexpr int MMA_WARP = 8 * GROUPS, TMA_WARP = 8 * GROUPS + 1;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // dynamic layout: B hi | B lo | output staging x 2 groups
    const int AS = d.a_stages, NB = d.acc_buffers;
    unsigned char *b_hi = smem;
    unsigned char *b_lo = b_hi + d.np * 128;
    float *out_stages = reinterpret_cast<float *>(b_lo + d.np * 128);  // group g: [64 oc][4 rows][32 px] at + g * 8192 floats
    __shared__ __align__(128) float x_tiles[XS][XT];                   // [c][6 rows][40 columns]
    __shared__ uint64_t full[3], empty[3], acc_full[4], acc_empty[4], x_full[XS], x_empty[XS];
    __shared__ uint32_t tmem_slot;
    __shared__ float bias_s[128];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tiles_per_img = d.tiles_x * d.tiles_y;
    const int total_tiles = d.n * tiles_per_img;
    const int my_tiles = (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const bool post_op = d.bias != nullptr || d.relu != 0;
    if (tid < 128) bias_s[tid] = (d.bias != nullptr && tid < d.k) ? __ldg(d.bias + tid) : 0.f;
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < NB * d.np + AS * 64) tmem_cols <<= 1;
    const uint32_t a_col0 = uint32_t(NB * d.np);  // first column of the A stages

    if (tid == 0) {
        for (int s = 0; s < 3; ++s) {
            mbar_init(&full[s], 4);  // one arrival per builder warp
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < 4; ++s) {
            mbar_init(&acc_full[s], 1);
            mbar_init(&acc_empty[s], 4);  // one arrival per epilogue warp
        }
        for (int s = 0; s < XS; ++s) {
            mbar_init(&x_full[s], 1);
            mbar_init(&x_empty[s], 4);
        }
        mbar_init_fence();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(&tmem_slot, tmem_cols);
        tmem_relinquish();
    }
    // filters -> B tiles (all threads)
    for (int i = tid; i < d.np * 8; i += FWD_THREADS) {
        const int oc = i >> 3, j = i & 7;
        float v[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int t = 4 * j + q;
            v[q] = (oc < d.k && t < TAPS) ? __ldg(w + size_t(oc) * TAPS + t) : 0.f;
        }
        const float4 hi = make_float4(tf32_hi(v[0]), tf32_hi(v[1]), tf32_hi(v[2]), tf32_hi(v[3]));
        store_chunk(b_hi, oc, j, hi);
        store_chunk(b_lo, oc, j, make_float4(v[0] - hi.x, v[1] - hi.y, v[2] - hi.z, v[3] - hi.w));
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;
    const size_t plane = size_t(d.h) * d.w;

    if (warp >= 4 * GROUPS && warp < 8 * GROUPS) {
        // ---- builders: one pixel (one A row) per thread, window read from the x halo tile ----
        const int group = (warp - 4 * GROUPS) >> 2;
        const int r = (warp & 3) * 32 + lane;
        const int win = (r >> 5) * 40 + (r & 31) + 3;  // window origin (ky = kx = 0) inside a channel's 6x40 tile
        for (int it = group; it < my_tiles; it += GROUPS) {
            const int s = it % AS, xs = it % XS;
            if (!mbar_wait_warp_ready(&x_full[xs], (it / XS) & 1, d.status, 45)) break;
            float v[32];
            const float *xt = x_tiles[xs] + win;
#pragma unroll
            for (int t = 0; t < 32; ++t) v[t] = 0.f;
#pragma unroll
            for (int c = 0; c < CIN; ++c)
#pragma unroll
                for (int ky = 0; ky < 3; ++ky)
#pragma unroll
                    for (int kx = 0; kx < 3; ++kx) v[(c * 3 + ky) * 3 + kx] = ld_shared_f32(xt + (c * 6 + ky) * 40 + kx);
            // Release the x stage: the window values are in registers.  The refill is an async-proxy
            // (TMA) write after generic-proxy reads, hence the proxy fence before the arrival.
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&x_empty[xs]);
            if (it >= AS && !mbar_wait_warp_ready(&empty[s], ((it / AS) - 1) & 1, d.status, 41)) break;
            tc_fence_after_sync();
            const uint32_t a_addr = tmem_base + (uint32_t((warp & 3) * 32) << 16) + a_col0 + uint32_t(s) * 64;
            float lo[32];
#pragma unroll
            for (int t = 0; t < 32; ++t) {
                const float hi = tf32_hi(v[t]);
                lo[t] = v[t] - hi;
                v[t] = hi;
            }
            tmem_st_32x32(a_addr, v);
            if (d.three_pass) tmem_st_32x32(a_addr + 32, lo);
            tmem_st_wait();
            tc_fence_before_sync();
            // tcgen05.wait::st is warp-wide: once it returns every lane's stores have landed, so one arrival per
            // warp does (128 single arrivals are 128 serialised shared-memory operations per tile)
            mbar_arrive_warp(&full[s]);
        }
    } else if (warp == TMA_WARP && lane == 0) {
        // ---- TMA loads of the x halo tiles ----
        for (int it = 0; it < my_tiles; ++it) {
            const int s = it % XS;
            if (it >= XS && !mbar_wait(&x_empty[s], ((it / XS) - 1) & 1, d.status, 46)) break;
            const int tile = blockIdx.x + it * gridDim.x;
            const int img = tile / tiles_per_img, tt = tile % tiles_per_img;
            mbar_arrive_expect_tx(&x_full[s], CIN * 6 * 40 * 4);
            tma_load_4d(x_tiles[s], &map_x, &x_full[s], (tt % d.tiles_x) * 32 - 4, (tt / d.tiles_x) * 4 - 1, 0, img);
        }
    } else if (warp == MMA_WARP) {
        // ---- MMA issue: descriptors are precomputed, this role is on the critical path.  The
        // whole warp runs the loop and the thread chosen by elect.sync issues; with warp-uniform
        // control flow the operands stay in uniform registers (measured: one small-N MMA per
        // ~22 cycles, against 44 behind a lane == 0 branch). ----
        const bool issue = elect_one();
        const uint32_t idesc = idesc_tf32(128, d.np, false, false);
        uint64_t db_hi[4], db_lo[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            db_hi[j] = smem_desc(smem_u32(b_hi) + j * 32, 16, 1024, kLayoutSw128);
            db_lo[j] = smem_desc(smem_u32(b_lo) + j * 32, 16, 1024, kLayoutSw128);
        }
        for (int it = 0; it < my_tiles; ++it) {
            const int s = it % AS, b = it % NB;
            if (!mbar_wait_warp_ready(&full[s], (it / AS) & 1, d.status, 42)) break;
            if (it >= NB && !mbar_wait_warp_ready(&acc_empty[b], ((it / NB) - 1) & 1, d.status, 43)) break;
            tc_fence_after_sync();
            const uint32_t acc = tmem_base + uint32_t(b) * d.np;
            const uint32_t a_hi = tmem_base + a_col0 + uint32_t(s) * 64, a_lo = a_hi + 32;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (issue) {
                    if (d.three_pass) {
                        mma_tf32_ts(acc, a_lo + 8 * j, db_hi[j], idesc, j != 0);
                        mma_tf32_ts(acc, a_hi + 8 * j, db_lo[j], idesc, true);
                        mma_tf32_ts(acc, a_hi + 8 * j, db_hi[j], idesc, true);
                    } else {
                        mma_tf32_ts(acc, a_hi + 8 * j, db_hi[j], idesc, j != 0);
                    }
                }
            }
            if (issue) {
                mma_commit(&empty[s]);
                mma_commit(&acc_full[b]);
            }
            __syncwarp();
        }
    } else if (warp < 4 * GROUPS) {
        // ---- epilogue: TMEM -> registers (thread = pixel) -> shared staging [oc][4 rows][32 px]
        // -> global with 128-bit stores (a warp writes the four 128-byte row segments of one
        // channel's tile per instruction), 64 channels per staging pass ----
        const int group = warp >> 2;
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const int bar_id = 1 + group;
        float *stage = out_stages + group * (64 * 128);
        bool alive = true;
        for (int it = group; it < my_tiles; it += GROUPS) {
            const int b = it % NB;
            // A warp whose wait ran out keeps meeting its group at the named barriers (the others
            // may have got through just before) and skips the work; once one wait of the launch
            // has failed all later waits return at once, so the rest of the loop is quick.
            if (alive) alive = mbar_wait_warp_ready(&acc_full[b], (it / NB) & 1, d.status, 44);
            tc_fence_after_sync();
            const int tile = blockIdx.x + it * gridDim.x;
            const int img = tile / tiles_per_img, tt = tile % tiles_per_img;
            const int oy0 = (tt / d.tiles_x) * 4, ox0 = (tt % d.tiles_x) * 32;
            for (int c0 = 0; c0 < d.np; c0 += 64) {
                named_barrier(bar_id, 128);  // the previous pass has been copied out of the staging buffer
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (alive && c0 + 32 * h < d.np) {
                        float v[32];
                        tmem_ld_32x32(tmem_base + (uint32_t(quarter * 32) << 16) + b * d.np + c0 + 32 * h, v);
                        if (post_op) {  // bias and ReLU fused behind the accumulator (block-uniform branch)
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                v[i] += bias_s[c0 + 32 * h + i];
                                if (d.relu) v[i] = fmaxf(v[i], 0.f);
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 32; ++i) st_shared_f32(stage + (32 * h + i) * 128 + r, v[i]);
                    }
                }
                if (alive && c0 + 64 >= d.np) {
                    tc_fence_before_sync();
                    mbar_arrive_warp(&acc_empty[b]);  // the loads above waited for their data (tcgen05.wait::ld, warp-wide)
                }
                named_barrier(bar_id, 128);
                const int chans = !alive ? 0 : (d.k - c0) < 64 ? (d.k - c0) : 64;
                for (int f = r; f < chans * 32; f += 128) {
                    const int oc = f >> 5, row = (f >> 3) & 3, col = (f & 7) * 4;
                    const int oy = oy0 + row, ox = ox0 + col;
                    if (oy < d.h && ox < d.w) {
                        const float4 q = ld_shared_v4(stage + f * 4);
                        __stcs(reinterpret_cast<float4 *>(y + (size_t(img) * d.k + c0 + oc) * plane + size_t(oy) * d.w + ox), q);
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == MMA_WARP) tmem_dealloc(tmem_base, tmem_cols);
}

bool stem_tc_shape(const katsu_cuda_ctx *ctx, size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                   size_t stride, size_t pad) {
    if (ctx->precision == KATSU_MODE_FP32) return false;
    if (c < 1 || c > 3 || r != 3 || s != 3 || stride != 1 || pad != 1) return false;
    if (k < 1 || k > 128 || h > 32768 || wd > 32768) return false;  // 2 accumulators + 2 A stages must fit 512 TMEM columns
    if (wd % 4 != 0) return false;  // TMA row pitch must be a multiple of 16 bytes
    return n * katsu_div_up(h, 4) * katsu_div_up(wd, 32) <= 0x7fffffffu;
}

template <int CIN, int GROUPS>
int32_t fwd_launch_groups(katsu_cuda_ctx *ctx, const float *x, const float *w, float *y, StemDims d) {
    // x as [N][C][H][W] with a box of one halo tile: 40 columns x 6 rows x all channels
    CUtensorMap map_x;
    {
        const uint64_t dims[4] = {(uint64_t)d.w, (uint64_t)d.h, (uint64_t)CIN, (uint64_t)d.n};
        const uint64_t strides[4] = {1, (uint64_t)d.w, (uint64_t)d.w * d.h, (uint64_t)d.w * d.h * CIN};
        const uint32_t box[4] = {40, 6, CIN, 1};
        if (!katsu_make_tensor_map(&map_x, x, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE))
            return katsu_set_error(KATSU_ERR_CUDA, "cuTensorMapEncodeTiled failed (stem forward x)");
    }
    // filters, one staging buffer per epilogue group, alignment slack.  The two-blocks-per-SM
    // form asks for at least 90 KiB so that a third block (which could not get TMEM columns)
    // is never co-resident.
    size_t smem = 2 * size_t(d.np) * 128 + size_t(GROUPS) * 64 * 512 + 1024;
    if (GROUPS == 1 && smem < 90 * 1024) smem = 90 * 1024;
    // tensor memory: accumulators first, then the A stages (64 columns each)
    const int cols = GROUPS == 1 ? 256 : 512;
    d.acc_buffers = (4 * d.np + 2 * 64 <= cols) ? 4 : 2;
    d.a_stages = (cols - d.acc_buffers * d.np) / 64;
    if (d.a_stages > 3) d.a_stages = 3;
    auto kernel = stem_fwd_tc_kernel<CIN, GROUPS>;
    KATSU_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const size_t total_tiles = size_t(d.n) * d.tiles_x * d.tiles_y;
    size_t grid = size_t(ctx->num_sms) * (GROUPS == 1 ? 2 : 1);
    if (grid > total_tiles) grid = total_tiles;
    KATSU_LAUNCH(ctx, kernel, (unsigned)grid, (8 * GROUPS + 2) * 32, smem, w, y, map_x, d);
    return KATSU_OK;
}

template <int CIN>
int32_t fwd_launch(katsu_cuda_ctx *ctx, const float *x, const float *w, float *y, StemDims d) {
    // two accumulators + two A stages in 256 TMEM columns: np <= 64
    if (d.np <= 64) return fwd_launch_groups<CIN, 1>(ctx, x, w, y, d);
    return fwd_launch_groups<CIN, 2>(ctx, x, w, y, d);
}

}  // namespace

int32_t katsu_conv_stem_tc_fwd(katsu_cuda_ctx *ctx, const float *x, const float *w, float *y,
                               size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                               size_t stride, size_t pad, const float *bias, int relu, int *handled) {
    *handled = 0;
    if (!stem_tc_shape(ctx, n, c, h, wd, k, r, s, stride, pad)) return KATSU_OK;
    if ((reinterpret_cast<uintptr_t>(x) & 15u) != 0 || (reinterpret_cast<uintptr_t>(y) & 15u) != 0) return KATSU_OK;
    *handled = 1;
    StemDims d;
    d.n = (int)n; d.k = (int)k; d.h = (int)h; d.w = (int)wd;
    d.tiles_x = (int)katsu_div_up(wd, 32);
    d.tiles_y = (int)katsu_div_up(h, 4);
    d.np = (int)katsu_div_up(k, 32) * 32;
    d.three_pass = ctx->precision == KATSU_MODE_3XTF32 ? 1 : 0;
    d.status = ctx->status;
    d.bias = bias;
    d.relu = relu;
    switch (c) {
        case 1: return fwd_launch<1>(ctx, x, w, y, d);
        case 2: return fwd_launch<2>(ctx, x, w, y, d);
        default: return fwd_launch<3>(ctx, x, w, y, d);
    }
}
