// Low-channel convolution (C_in <= 4, 3x3 filter, stride 1, padding 1) as
// shared-memory stencils on CUDA cores.  These shapes (RGB stems) move far
// more output than input: y and g are C_out/C_in times larger than x, so the
// kernels are organised around streaming y (forward) and g (backward) through
// HBM exactly once while x tiles and all filters sit in shared memory.
//
// Reference loops being replaced: the visit closure of Conv2D::forward
// (crates/katsu-core/src/conv2d.rs:95-103, 232-262) and backward_buffers
// (conv2d.rs:269-292).  Zero padding is virtual: halo cells outside the image
// are filled with 0 in shared memory, which contributes nothing, exactly like
// the reference's skipped taps.
#include "common.cuh"

namespace {

constexpr int TW = 32;         // tile width in pixels (one 128-byte line of f32)
constexpr int XP = 36;         // row pitch of halo tiles in floats (TW + 2, rounded up to 4)

struct StencilDims {
    int n, k, h, w;            // batch, output channels, image height/width (OH == H, OW == W)
    int tiles_x, tiles_y;
};

// ---------------------------------------------------------------------------
// forward: one block = 32x32 output pixels of one image, all output channels.
// Thread (tx, ty) owns pixels [4tx, 4tx+4) of row ty and keeps its
// CIN x 3 x 6 input window in registers; filters are read from shared memory
// as [tap][oc] so OCB consecutive channels come in as 128-bit broadcasts.
// ---------------------------------------------------------------------------
template <int CIN, int OCB>
__global__ void __launch_bounds__(256, 2)
stencil_fwd_kernel(const float *__restrict__ x, const float *__restrict__ w, float *__restrict__ y,
                   StencilDims d, int kp) {
    constexpr int TH = 32;
    constexpr int TAPS = CIN * 9;
    float *xs = katsu_dynamic_smem();              // [CIN][TH+2][XP]
    float *ws = xs + CIN * (TH + 2) * XP;          // [TAPS][kp]
    const int tid = threadIdx.x;
    const int tx = tid & 7, ty = tid >> 3;
    const int tiles = d.tiles_x * d.tiles_y;
    const int n = blockIdx.x / tiles;
    const int t = blockIdx.x % tiles;
    const int x0 = (t % d.tiles_x) * TW, y0 = (t / d.tiles_x) * TH;

    for (int i = tid; i < TAPS * kp; i += 256) {
        const int tap = i / kp, oc = i % kp;
        ws[i] = oc < d.k ? __ldg(w + size_t(oc) * TAPS + tap) : 0.f;
    }
    const float *xn = x + size_t(n) * CIN * d.h * d.w;
    for (int i = tid; i < CIN * (TH + 2) * (TW + 2); i += 256) {
        const int c = i / ((TH + 2) * (TW + 2));
        const int rem = i % ((TH + 2) * (TW + 2));
        const int r = rem / (TW + 2), col = rem % (TW + 2);
        const int gy = y0 - 1 + r, gx = x0 - 1 + col;
        float v = 0.f;
        if (gy >= 0 && gy < d.h && gx >= 0 && gx < d.w) v = __ldg(xn + (size_t(c) * d.h + gy) * d.w + gx);
        xs[(c * (TH + 2) + r) * XP + col] = v;
    }
    __syncthreads();

    float win[CIN][3][6];
#pragma unroll
    for (int c = 0; c < CIN; ++c)
#pragma unroll
        for (int r = 0; r < 3; ++r) {
            const float *row = xs + (c * (TH + 2) + ty + r) * XP + 4 * tx;
            const float4 a = *reinterpret_cast<const float4 *>(row);
            const float2 b = *reinterpret_cast<const float2 *>(row + 4);
            win[c][r][0] = a.x; win[c][r][1] = a.y; win[c][r][2] = a.z; win[c][r][3] = a.w;
            win[c][r][4] = b.x; win[c][r][5] = b.y;
        }

    const int oy = y0 + ty, ox = x0 + 4 * tx;
    const bool row_ok = oy < d.h;
    // 128-bit stores need rows that start on 16 bytes: W a multiple of 4 and the tensor itself aligned
    const bool vec_ok = (d.w % 4 == 0) && (ox + 3 < d.w) && (reinterpret_cast<uintptr_t>(y) & 15u) == 0;
    const size_t plane = size_t(d.h) * d.w;
    float *yrow = y + size_t(n) * d.k * plane + size_t(oy) * d.w + ox;

    for (int oc0 = 0; oc0 < kp; oc0 += OCB) {
        float acc[OCB][4];
#pragma unroll
        for (int j = 0; j < OCB; ++j)
#pragma unroll
            for (int p = 0; p < 4; ++p) acc[j][p] = 0.f;
#pragma unroll
        for (int c = 0; c < CIN; ++c)
#pragma unroll
            for (int r = 0; r < 3; ++r)
#pragma unroll
                for (int s = 0; s < 3; ++s) {
                    const float *wp = ws + ((c * 3 + r) * 3 + s) * kp + oc0;
                    float wv[OCB];
#pragma unroll
                    for (int j4 = 0; j4 < OCB / 4; ++j4) {
                        const float4 q = *reinterpret_cast<const float4 *>(wp + 4 * j4);
                        wv[4 * j4] = q.x; wv[4 * j4 + 1] = q.y; wv[4 * j4 + 2] = q.z; wv[4 * j4 + 3] = q.w;
                    }
#pragma unroll
                    for (int j = 0; j < OCB; ++j)
#pragma unroll
                        for (int p = 0; p < 4; ++p) acc[j][p] = fmaf(win[c][r][p + s], wv[j], acc[j][p]);
                }
        if (row_ok) {
#pragma unroll
            for (int j = 0; j < OCB; ++j) {
                const int oc = oc0 + j;
                if (oc < d.k) {
                    float *dst = yrow + size_t(oc) * plane;
                    if (vec_ok) {
                        *reinterpret_cast<float4 *>(dst) = make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]);
                    } else {
#pragma unroll
                        for (int p = 0; p < 4; ++p)
                            if (ox + p < d.w) dst[p] = acc[j][p];
                    }
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// dX: one block = 32x32 input pixels of one image, all CIN channels.  Output
// channels stream through shared memory OCB at a time as halo tiles of g.
// Thread (tx, ty) owns pixels [4tx, 4tx+4) of rows 2ty and 2ty+1.
//   dx[c, iy, ix] = sum_{oc, ky, kx} g[oc, iy+1-ky, ix+1-kx] * w[oc, c, ky, kx]
// ---------------------------------------------------------------------------
template <int CIN>
__global__ void __launch_bounds__(128, 4)
stencil_dx_kernel(const float *__restrict__ w, const float *__restrict__ g, float *dx, StencilDims d,
                  int kp, int accumulate) {
    constexpr int TH = 32;
    constexpr int OCB = 8;
    constexpr int TAPS = CIN * 9;
    constexpr int WP = (TAPS + 3) / 4 * 4;         // filter row pitch in floats
    float *gs = katsu_dynamic_smem();              // [OCB][TH+2][XP]
    float *ws = gs + OCB * (TH + 2) * XP;          // [kp][WP]
    const int tid = threadIdx.x;
    const int tx = tid & 7, ty = tid >> 3;
    const int tiles = d.tiles_x * d.tiles_y;
    const int n = blockIdx.x / tiles;
    const int t = blockIdx.x % tiles;
    const int x0 = (t % d.tiles_x) * TW, y0 = (t / d.tiles_x) * TH;
    const size_t plane = size_t(d.h) * d.w;

    for (int i = tid; i < kp * WP; i += 128) {
        const int oc = i / WP, tap = i % WP;
        ws[i] = (oc < d.k && tap < TAPS) ? __ldg(w + size_t(oc) * TAPS + tap) : 0.f;
    }

    float acc[CIN][2][4];
#pragma unroll
    for (int c = 0; c < CIN; ++c)
#pragma unroll
        for (int q = 0; q < 2; ++q)
#pragma unroll
            for (int p = 0; p < 4; ++p) acc[c][q][p] = 0.f;

    const float *gn = g + size_t(n) * d.k * plane;
    for (int oc0 = 0; oc0 < kp; oc0 += OCB) {
        __syncthreads();  // previous chunk fully consumed (also orders the ws fill)
        for (int i = tid; i < OCB * (TH + 2) * (TW + 2); i += 128) {
            const int j = i / ((TH + 2) * (TW + 2));
            const int rem = i % ((TH + 2) * (TW + 2));
            const int r = rem / (TW + 2), col = rem % (TW + 2);
            const int gy = y0 - 1 + r, gx = x0 - 1 + col;
            const int oc = oc0 + j;
            float v = 0.f;
            if (oc < d.k && gy >= 0 && gy < d.h && gx >= 0 && gx < d.w)
                v = __ldg(gn + size_t(oc) * plane + size_t(gy) * d.w + gx);
            gs[(j * (TH + 2) + r) * XP + col] = v;
        }
        __syncthreads();
#pragma unroll 1
        for (int j = 0; j < OCB; ++j) {
            float gw[4][6];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float *row = gs + (j * (TH + 2) + 2 * ty + r) * XP + 4 * tx;
                const float4 a = *reinterpret_cast<const float4 *>(row);
                const float2 b = *reinterpret_cast<const float2 *>(row + 4);
                gw[r][0] = a.x; gw[r][1] = a.y; gw[r][2] = a.z; gw[r][3] = a.w; gw[r][4] = b.x; gw[r][5] = b.y;
            }
            float wv[WP];
#pragma unroll
            for (int i4 = 0; i4 < WP / 4; ++i4) {
                const float4 q = *reinterpret_cast<const float4 *>(ws + (oc0 + j) * WP + 4 * i4);
                wv[4 * i4] = q.x; wv[4 * i4 + 1] = q.y; wv[4 * i4 + 2] = q.z; wv[4 * i4 + 3] = q.w;
            }
#pragma unroll
            for (int c = 0; c < CIN; ++c)
#pragma unroll
                for (int ky = 0; ky < 3; ++ky)
#pragma unroll
                    for (int kx = 0; kx < 3; ++kx)
#pragma unroll
                        for (int q = 0; q < 2; ++q)
#pragma unroll
                            for (int p = 0; p < 4; ++p)
                                acc[c][q][p] = fmaf(gw[q + 2 - ky][p + 2 - kx], wv[(c * 3 + ky) * 3 + kx], acc[c][q][p]);
        }
    }

    const int ix = x0 + 4 * tx;
    const bool vec_ok = (d.w % 4 == 0) && (ix + 3 < d.w) && (reinterpret_cast<uintptr_t>(dx) & 15u) == 0;
#pragma unroll
    for (int c = 0; c < CIN; ++c)
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int iy = y0 + 2 * ty + q;
            if (iy >= d.h) continue;
            float *dst = dx + (size_t(n) * CIN + c) * plane + size_t(iy) * d.w + ix;
            if (vec_ok) {
                float4 v = make_float4(acc[c][q][0], acc[c][q][1], acc[c][q][2], acc[c][q][3]);
                if (accumulate) {
                    const float4 o = *reinterpret_cast<const float4 *>(dst);
                    v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                *reinterpret_cast<float4 *>(dst) = v;
            } else {
#pragma unroll
                for (int p = 0; p < 4; ++p)
                    if (ix + p < d.w) dst[p] = accumulate ? dst[p] + acc[c][q][p] : acc[c][q][p];
            }
        }
}

// ---------------------------------------------------------------------------
// dW: persistent blocks walk 8x32 pixel tiles.  Within a warp the lanes are
// output channels (lane and lane+32 of a 64-channel group), every lane keeps
// the CIN x 9 filter-gradient sums of its two channels in registers for the
// block's whole share of the batch, and the x window it multiplies with is a
// warp-wide shared-memory broadcast.  Each block then writes one partial
// filter gradient to scratch; stencil_dw_reduce_kernel folds the partials in
// a fixed order, so the result is bit-reproducible.
//   dw[oc, c, ky, kx] = sum_{n, oy, ox} g[n, oc, oy, ox] * x[n, c, oy+ky-1, ox+kx-1]
// ---------------------------------------------------------------------------
constexpr int DW_TH = 8;       // tile rows == warps per block
constexpr int DW_GP = DW_TH * TW + 4;  // g plane pitch: 260 floats, == 4 mod 32 so 8 lanes hit 8 bank groups

template <int CIN>
__global__ void __launch_bounds__(256, 2)
stencil_dw_kernel(const float *__restrict__ x, const float *__restrict__ g, float *__restrict__ partial,
                  StencilDims d, int groups) {
    constexpr int TAPS = CIN * 9;
    float *gs = katsu_dynamic_smem();              // [64][DW_GP]; reused as [8][64][TAPS] for the block reduce
    constexpr int GS_FLOATS = (64 * DW_GP > 8 * 64 * TAPS) ? 64 * DW_GP : 8 * 64 * TAPS;
    float *xs = gs + GS_FLOATS;                    // [CIN][DW_TH+2][XP]
    const int tid = threadIdx.x;
    const int lane = tid & 31, wp = tid >> 5;
    const int tiles_per_image = d.tiles_x * d.tiles_y;
    const int total_tiles = d.n * tiles_per_image;
    const size_t plane = size_t(d.h) * d.w;
    const bool w_vec = (d.w % 4 == 0) && (reinterpret_cast<uintptr_t>(g) & 15u) == 0;

    for (int grp = 0; grp < groups; ++grp) {
        float acc0[TAPS], acc1[TAPS];
#pragma unroll
        for (int i = 0; i < TAPS; ++i) { acc0[i] = 0.f; acc1[i] = 0.f; }

        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            const int n = tile / tiles_per_image;
            const int t = tile % tiles_per_image;
            const int x0 = (t % d.tiles_x) * TW, y0 = (t / d.tiles_x) * DW_TH;
            __syncthreads();  // the previous tile is fully consumed
            // g tile: 64 planes x 8 rows x 8 quads
            const float *gn = g + (size_t(n) * d.k + size_t(grp) * 64) * plane;
            for (int i = tid; i < 64 * DW_TH * (TW / 4); i += 256) {
                const int j = i / (DW_TH * (TW / 4));
                const int r = (i / (TW / 4)) % DW_TH;
                const int q = i % (TW / 4);
                const int oc = grp * 64 + j;
                const int gy = y0 + r, gx = x0 + 4 * q;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (oc < d.k && gy < d.h) {
                    const float *src = gn + size_t(j) * plane + size_t(gy) * d.w + gx;
                    if (w_vec && gx + 3 < d.w) {
                        v = __ldg(reinterpret_cast<const float4 *>(src));
                    } else {
                        if (gx < d.w) v.x = __ldg(src);
                        if (gx + 1 < d.w) v.y = __ldg(src + 1);
                        if (gx + 2 < d.w) v.z = __ldg(src + 2);
                        if (gx + 3 < d.w) v.w = __ldg(src + 3);
                    }
                }
                *reinterpret_cast<float4 *>(gs + j * DW_GP + r * TW + 4 * q) = v;
            }
            const float *xn = x + size_t(n) * CIN * plane;
            for (int i = tid; i < CIN * (DW_TH + 2) * (TW + 2); i += 256) {
                const int c = i / ((DW_TH + 2) * (TW + 2));
                const int rem = i % ((DW_TH + 2) * (TW + 2));
                const int r = rem / (TW + 2), col = rem % (TW + 2);
                const int gy = y0 - 1 + r, gx = x0 - 1 + col;
                float v = 0.f;
                if (gy >= 0 && gy < d.h && gx >= 0 && gx < d.w) v = __ldg(xn + (size_t(c) * d.h + gy) * d.w + gx);
                xs[(c * (DW_TH + 2) + r) * XP + col] = v;
            }
            __syncthreads();
            // warp wp owns tile row wp
#pragma unroll 1
            for (int q = 0; q < TW / 4; ++q) {
                const float4 ga = *reinterpret_cast<const float4 *>(gs + lane * DW_GP + wp * TW + 4 * q);
                const float4 gb = *reinterpret_cast<const float4 *>(gs + (lane + 32) * DW_GP + wp * TW + 4 * q);
                const float g0[4] = {ga.x, ga.y, ga.z, ga.w};
                const float g1[4] = {gb.x, gb.y, gb.z, gb.w};
#pragma unroll
                for (int c = 0; c < CIN; ++c)
#pragma unroll
                    for (int ky = 0; ky < 3; ++ky) {
                        const float *row = xs + (c * (DW_TH + 2) + wp + ky) * XP + 4 * q;
                        const float4 a = *reinterpret_cast<const float4 *>(row);
                        const float2 b = *reinterpret_cast<const float2 *>(row + 4);
                        const float xw[6] = {a.x, a.y, a.z, a.w, b.x, b.y};
#pragma unroll
                        for (int kx = 0; kx < 3; ++kx)
#pragma unroll
                            for (int p = 0; p < 4; ++p) {
                                acc0[(c * 3 + ky) * 3 + kx] = fmaf(g0[p], xw[p + kx], acc0[(c * 3 + ky) * 3 + kx]);
                                acc1[(c * 3 + ky) * 3 + kx] = fmaf(g1[p], xw[p + kx], acc1[(c * 3 + ky) * 3 + kx]);
                            }
                    }
            }
        }

        // block reduce: red[warp][oc][tap], summed over warps in a fixed order
        __syncthreads();
        float *red = gs;
#pragma unroll
        for (int i = 0; i < TAPS; ++i) {
            red[(wp * 64 + lane) * TAPS + i] = acc0[i];
            red[(wp * 64 + lane + 32) * TAPS + i] = acc1[i];
        }
        __syncthreads();
        for (int i = tid; i < 64 * TAPS; i += 256) {
            float s = 0.f;
#pragma unroll
            for (int v = 0; v < 8; ++v) s += red[v * 64 * TAPS + i];
            const int oc = grp * 64 + i / TAPS;
            if (oc < d.k) partial[size_t(blockIdx.x) * d.k * TAPS + size_t(oc) * TAPS + i % TAPS] = s;
        }
    }
}

__global__ void __launch_bounds__(256)
stencil_dw_reduce_kernel(const float *__restrict__ partial, float *dw, int elems, int parts, int accumulate) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= elems) return;
    float s = 0.f;
    for (int p = 0; p < parts; ++p) s += partial[size_t(p) * elems + i];
    dw[i] = accumulate ? dw[i] + s : s;
}

bool stencil_shape(size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s, size_t stride,
                   size_t pad) {
    if (c < 1 || c > 4 || r != 3 || s != 3 || stride != 1 || pad != 1) return false;
    if (k < 1 || k > 256) return false;
    if (h > 32768 || wd > 32768) return false;
    const size_t tiles = n * katsu_div_up(h, 8) * katsu_div_up(wd, (size_t)TW);
    return tiles <= 0x7fffffffu;
}

template <typename Kernel>
int32_t allow_smem(Kernel kernel, size_t bytes) {
    if (bytes > 48 * 1024)
        KATSU_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    return KATSU_OK;
}

template <int CIN>
int32_t fwd_launch(katsu_cuda_ctx *ctx, const float *x, const float *w, float *y, StencilDims d) {
    constexpr int OCB = 8;
    const int kp = (d.k + OCB - 1) / OCB * OCB;
    const size_t smem = (size_t(CIN) * 34 * XP + size_t(CIN) * 9 * kp) * sizeof(float);
    auto kernel = stencil_fwd_kernel<CIN, OCB>;
    KATSU_TRY(allow_smem(kernel, smem));
    d.tiles_y = (d.h + 31) / 32;
    const unsigned grid = (unsigned)(size_t(d.n) * d.tiles_x * d.tiles_y);
    KATSU_LAUNCH(ctx, kernel, grid, 256, smem, x, w, y, d, kp);
    return KATSU_OK;
}

template <int CIN>
int32_t dx_launch(katsu_cuda_ctx *ctx, const float *w, const float *g, float *dx, StencilDims d, int accumulate) {
    const int kp = (d.k + 7) / 8 * 8;
    constexpr int WP = (CIN * 9 + 3) / 4 * 4;
    const size_t smem = (size_t(8) * 34 * XP + size_t(kp) * WP) * sizeof(float);
    auto kernel = stencil_dx_kernel<CIN>;
    KATSU_TRY(allow_smem(kernel, smem));
    d.tiles_y = (d.h + 31) / 32;
    const unsigned grid = (unsigned)(size_t(d.n) * d.tiles_x * d.tiles_y);
    KATSU_LAUNCH(ctx, kernel, grid, 128, smem, w, g, dx, d, kp, accumulate);
    return KATSU_OK;
}

template <int CIN>
int32_t dw_launch(katsu_cuda_ctx *ctx, const float *x, const float *g, float *dw, StencilDims d, int accumulate) {
    constexpr int TAPS = CIN * 9;
    constexpr size_t GS_FLOATS = (64 * DW_GP > 8 * 64 * TAPS) ? 64 * DW_GP : 8 * 64 * TAPS;
    const size_t smem = (GS_FLOATS + size_t(CIN) * (DW_TH + 2) * XP) * sizeof(float);
    auto kernel = stencil_dw_kernel<CIN>;
    KATSU_TRY(allow_smem(kernel, smem));
    d.tiles_y = (d.h + DW_TH - 1) / DW_TH;
    const size_t total_tiles = size_t(d.n) * d.tiles_x * d.tiles_y;
    size_t grid = size_t(ctx->num_sms) * 2;
    if (grid > total_tiles) grid = total_tiles;
    const int groups = (d.k + 63) / 64;
    const int elems = d.k * TAPS;
    float *partial = nullptr;
    KATSU_TRY(katsu_scratch(ctx, grid * elems, &partial));
    KATSU_LAUNCH(ctx, kernel, (unsigned)grid, 256, smem, x, g, partial, d, groups);
    KATSU_LAUNCH(ctx, stencil_dw_reduce_kernel, (unsigned)katsu_div_up(elems, 256), 256, 0, partial, dw, elems,
                 (int)grid, accumulate);
    return KATSU_OK;
}

}  // namespace

int32_t katsu_conv_stencil_fwd(katsu_cuda_ctx *ctx, const float *x, const float *w, float *y,
                               size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                               size_t stride, size_t pad, int *handled) {
    *handled = 0;
    if (!stencil_shape(n, c, h, wd, k, r, s, stride, pad)) return KATSU_OK;
    *handled = 1;
    StencilDims d = {(int)n, (int)k, (int)h, (int)wd, (int)katsu_div_up(wd, (size_t)TW), 0};
    switch (c) {
        case 1: return fwd_launch<1>(ctx, x, w, y, d);
        case 2: return fwd_launch<2>(ctx, x, w, y, d);
        case 3: return fwd_launch<3>(ctx, x, w, y, d);
        default: return fwd_launch<4>(ctx, x, w, y, d);
    }
}

int32_t katsu_conv_stencil_bwd(katsu_cuda_ctx *ctx, const float *x, const float *w, const float *g,
                               float *dx, float *dw,
                               size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                               size_t stride, size_t pad, int accumulate, const float *gscale, float gfactor,
                               int *handled) {
    *handled = 0;
    if (!stencil_shape(n, c, h, wd, k, r, s, stride, pad)) return KATSU_OK;
    // only the tensor-core kernels scale the upstream gradient themselves (the caller checks)
    const bool scaled = gscale != nullptr || gfactor != 1.f;
    if (scaled && !katsu_conv_stem_tc_bwd_takes(ctx, x, g, dx, dw, n, c, h, wd, k)) return KATSU_OK;
    *handled = 1;
    StencilDims d = {(int)n, (int)k, (int)h, (int)wd, (int)katsu_div_up(wd, (size_t)TW), 0};
    int dx_done = 0;
    if (dx != nullptr)
        KATSU_TRY(katsu_conv_stem_tc_dx(ctx, w, g, dx, n, c, h, wd, k, accumulate, gscale, gfactor, &dx_done));
    if (dx != nullptr && !dx_done) KATSU_TRY(katsu_stencil_dx_tma(ctx, w, g, dx, n, c, h, wd, k, accumulate, &dx_done));
    if (dx != nullptr && !dx_done) {
        switch (c) {
            case 1: KATSU_TRY(dx_launch<1>(ctx, w, g, dx, d, accumulate)); break;
            case 2: KATSU_TRY(dx_launch<2>(ctx, w, g, dx, d, accumulate)); break;
            case 3: KATSU_TRY(dx_launch<3>(ctx, w, g, dx, d, accumulate)); break;
            default: KATSU_TRY(dx_launch<4>(ctx, w, g, dx, d, accumulate)); break;
        }
    }
    int dw_done = 0;
    if (dw != nullptr)
        KATSU_TRY(katsu_conv_stem_tc_dw(ctx, x, g, dw, n, c, h, wd, k, accumulate, gscale, gfactor, &dw_done));
    if (dw != nullptr && !dw_done) KATSU_TRY(katsu_stencil_dw_tma(ctx, x, g, dw, n, c, h, wd, k, accumulate, &dw_done));
    if (dw != nullptr && !dw_done) {
        switch (c) {
            case 1: KATSU_TRY(dw_launch<1>(ctx, x, g, dw, d, accumulate)); break;
            case 2: KATSU_TRY(dw_launch<2>(ctx, x, g, dw, d, accumulate)); break;
            case 3: KATSU_TRY(dw_launch<3>(ctx, x, g, dw, d, accumulate)); break;
            default: KATSU_TRY(dw_launch<4>(ctx, x, g, dw, d, accumulate)); break;
        }
    }
    return KATSU_OK;
}
