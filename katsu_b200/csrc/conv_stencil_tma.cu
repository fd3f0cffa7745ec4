// TMA-fed variant of the low-channel dX stencil (conv_stencil.cu: stencil_dx_kernel).
//
// The first dX kernel filled its halo tiles of g with a synchronous, division-heavy
// per-element loop: ncu showed 2.2 non-FMA instructions per FMA and long-scoreboard
// stalls.  Here one thread asks TMA for the whole [8 oc][34 rows][40 columns] tile (the
// start column is rounded down to a 16-byte boundary, cells outside the image arrive as
// zeros == the reference's skipped padding taps, crates/katsu-core/src/conv2d.rs:242-252),
// two tiles are in flight, and the compute loop contains nothing but shared-memory
// window loads and FMAs.
//   dx[c, iy, ix] = sum_{oc, ky, kx} g[oc, iy+1-ky, ix+1-kx] * w[oc, c, ky, kx]   (conv2d.rs:288)
#include "common.cuh"
#include "sm100.cuh"

using namespace sm100;

namespace {

constexpr int TWD = 32;            // dx tile width
constexpr int OCB = 4;             // output channels per g tile
constexpr int GP = 40;             // g tile pitch: columns x0-4 .. x0+35

struct DxDims {
    int n, k, h, w, tiles_x, tiles_y, kp, accumulate;
    int *status;
};

// TH = tile height (56 or 64): a thread owns two rows, so a block has 8 * TH / 2 threads
// (7 or 8 warps) and two blocks fit an SM -- the first version (TH = 32, 4 warps per block)
// ran at 12 % occupancy and 67 % issue utilisation.
template <int CIN, int TH>
__global__ void __launch_bounds__(4 * TH, 2)
stencil_dx_tma_kernel(const __grid_constant__ CUtensorMap map_g, const float *__restrict__ w, float *dx, DxDims d) {
    constexpr int TAPS = CIN * 9;
    constexpr int WP = (TAPS + 3) / 4 * 4;
    constexpr int GR = TH + 2;                 // g tile rows
    constexpr int G_STAGE = OCB * GR * GP;     // floats per stage
    constexpr int THREADS = 4 * TH;
    float *gs = katsu_dynamic_smem();          // [2][OCB][GR][GP], 128-byte aligned stages
    float *ws = gs + 2 * G_STAGE;              // [kp][WP]
    __shared__ uint64_t full[2];
    const int tid = threadIdx.x;
    const int tx = tid & 7, ty = tid >> 3;
    const int tiles = d.tiles_x * d.tiles_y;
    const int n = blockIdx.x / tiles;
    const int t = blockIdx.x % tiles;
    const int x0 = (t % d.tiles_x) * TWD, y0 = (t / d.tiles_x) * TH;
    const size_t plane = size_t(d.h) * d.w;
    const int chunks = d.kp / OCB;

    if (tid == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        mbar_init_fence();
        mbar_arrive_expect_tx(&full[0], G_STAGE * 4);
        tma_load_4d(gs, &map_g, &full[0], x0 - 4, y0 - 1, 0, n);
    }
    for (int i = tid; i < d.kp * WP; i += THREADS) {
        const int oc = i / WP, tap = i % WP;
        st_shared_f32(ws + i, (oc < d.k && tap < TAPS) ? __ldg(w + size_t(oc) * TAPS + tap) : 0.f);
    }
    __syncthreads();

    float acc[CIN][2][4];
#pragma unroll
    for (int c = 0; c < CIN; ++c)
#pragma unroll
        for (int q = 0; q < 2; ++q)
#pragma unroll
            for (int p = 0; p < 4; ++p) acc[c][q][p] = 0.f;

    bool alive = true;
    for (int ch = 0; ch < chunks; ++ch) {
        const int s = ch & 1;
        if (tid == 0 && ch + 1 < chunks) {  // the other stage was released by the barrier ending the last iteration
            mbar_arrive_expect_tx(&full[s ^ 1], G_STAGE * 4);
            tma_load_4d(gs + (s ^ 1) * G_STAGE, &map_g, &full[s ^ 1], x0 - 4, y0 - 1, (ch + 1) * OCB, n);
        }
        alive = mbar_wait_warp(&full[s], (ch >> 1) & 1, d.status, 51);
        if (!alive) break;  // whole block leaves: every warp sees the same barrier time out
        const float *stage = gs + s * G_STAGE;
#pragma unroll 1
        for (int j = 0; j < OCB; ++j) {
            float gw[4][6];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float *row = stage + (j * GR + 2 * ty + r) * GP + 4 * tx + 3;
                gw[r][0] = ld_shared_f32(row);
                const float4 a = ld_shared_v4(row + 1);
                gw[r][1] = a.x; gw[r][2] = a.y; gw[r][3] = a.z; gw[r][4] = a.w;
                gw[r][5] = ld_shared_f32(row + 5);
            }
            float wv[WP];
#pragma unroll
            for (int i4 = 0; i4 < WP / 4; ++i4) {
                const float4 q = ld_shared_v4(ws + (ch * OCB + j) * WP + 4 * i4);
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
        fence_proxy_async_smem();  // ordinary reads of the stage before its TMA refill
        __syncthreads();  // stage s may be refilled from the next iteration on
    }
    if (!alive) return;

    const int ix = x0 + 4 * tx;
    if (ix >= d.w) return;  // w is a multiple of 4: a float4 is either fully inside or fully outside
#pragma unroll
    for (int c = 0; c < CIN; ++c)
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int iy = y0 + 2 * ty + q;
            if (iy >= d.h) continue;
            float4 *dst = reinterpret_cast<float4 *>(dx + (size_t(n) * CIN + c) * plane + size_t(iy) * d.w + ix);
            float4 v = make_float4(acc[c][q][0], acc[c][q][1], acc[c][q][2], acc[c][q][3]);
            if (d.accumulate) {
                const float4 o = *dst;
                v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
            }
            *dst = v;
        }
}

template <int CIN, int TH>
int32_t launch_th(katsu_cuda_ctx *ctx, const float *g, const float *w, float *dx, DxDims d) {
    constexpr int WP = (CIN * 9 + 3) / 4 * 4;
    constexpr int G_STAGE = OCB * (TH + 2) * GP;
    CUtensorMap map_g;
    const uint64_t dims[4] = {(uint64_t)d.w, (uint64_t)d.h, (uint64_t)d.k, (uint64_t)d.n};
    const uint64_t strides[4] = {1, (uint64_t)d.w, (uint64_t)d.w * d.h, (uint64_t)d.w * d.h * d.k};
    const uint32_t box[4] = {GP, TH + 2, OCB, 1};
    if (!katsu_make_tensor_map(&map_g, g, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE))
        return katsu_set_error(KATSU_ERR_CUDA, "cuTensorMapEncodeTiled failed (stencil dX)");
    d.tiles_y = (d.h + TH - 1) / TH;
    const size_t smem = (2 * size_t(G_STAGE) + size_t(d.kp) * WP) * sizeof(float);
    auto kernel = stencil_dx_tma_kernel<CIN, TH>;
    KATSU_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const unsigned grid = (unsigned)(size_t(d.n) * d.tiles_x * d.tiles_y);
    KATSU_LAUNCH(ctx, kernel, grid, 4 * TH, smem, map_g, w, dx, d);
    return KATSU_OK;
}

template <int CIN>
int32_t launch(katsu_cuda_ctx *ctx, const float *g, const float *w, float *dx, DxDims d) {
    // 56-row tiles when they divide the image (224 = 4 x 56), else 64-row tiles
    if (d.h % 56 == 0) return launch_th<CIN, 56>(ctx, g, w, dx, d);
    return launch_th<CIN, 64>(ctx, g, w, dx, d);
}

}  // namespace

namespace {

// ---------------------------------------------------------------------------
// dW:  dw[oc, c, ky, kx] = sum_{n, oy, ox} g[n, oc, oy, ox] * x[n, c, oy+ky-1, ox+kx-1]   (conv2d.rs:289)
//
// Persistent blocks walk 4x32-pixel tiles; per tile TMA delivers g [64 oc][4][32] (dense)
// and the x halo [CIN][6][40].  A thread owns one pair of output channels (t >> 3 and
// +32) and one 4-pixel quad of every tile row (t & 7): the eight lanes of a quarter warp
// read eight different 16-byte quads of g (conflict-free on the dense TMA layout) and the
// x window slides down the rows in registers.  The CIN*9 sums of both channels stay in
// registers for the block's whole share of the batch; at the end the eight quad lanes are
// folded with shuffles and each block writes one partial filter gradient to scratch, which
// a second kernel folds in block order (bit-reproducible, no atomics).
// ---------------------------------------------------------------------------
constexpr int DW_ROWS = 4;
constexpr int DW_G_STAGE = 64 * DW_ROWS * 32;          // floats
constexpr int DW_XR = DW_ROWS + 2;

struct DwDims {
    int n, k, h, w, tiles_x, tiles_y, groups;
    int *status;
};

template <int CIN>
__global__ void __launch_bounds__(256, 2)
stencil_dw_tma_kernel(const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_x,
                      float *__restrict__ partial, DwDims d) {
    constexpr int TAPS = CIN * 9;
    constexpr int XT = (CIN * DW_XR * GP + 31) / 32 * 32;  // x stage pitch (128-byte aligned stages)
    float *gs = katsu_dynamic_smem();                   // [2][64][DW_ROWS][32]
    float *xs = gs + 2 * DW_G_STAGE;                    // [2][CIN][DW_XR][GP]
    __shared__ uint64_t full[2];
    const int tid = threadIdx.x, lane = tid & 31;
    const int quad = tid & 7, pair = tid >> 3;          // pixels 4*quad.., channels pair and pair + 32
    const int tiles_per_img = d.tiles_x * d.tiles_y;
    const int total_tiles = d.n * tiles_per_img;
    const int my_tiles = (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const uint32_t tile_bytes = (DW_G_STAGE + CIN * DW_XR * GP) * 4;

    if (tid == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        mbar_init_fence();
    }
    __syncthreads();

    uint32_t uses = 0;  // tiles consumed so far across all groups (stage = uses & 1, parity = (uses >> 1) & 1)
    for (int grp = 0; grp < d.groups; ++grp) {
        auto issue = [&](int it, int stage) {
            const int tile = blockIdx.x + it * gridDim.x;
            const int img = tile / tiles_per_img, tt = tile % tiles_per_img;
            const int x0 = (tt % d.tiles_x) * 32, y0 = (tt / d.tiles_x) * DW_ROWS;
            mbar_arrive_expect_tx(&full[stage], tile_bytes);
            tma_load_4d(gs + stage * DW_G_STAGE, &map_g, &full[stage], x0, y0, grp * 64, img);
            tma_load_4d(xs + stage * XT, &map_x, &full[stage], x0 - 4, y0 - 1, 0, img);
        };
        float acc0[TAPS], acc1[TAPS];
#pragma unroll
        for (int i = 0; i < TAPS; ++i) { acc0[i] = 0.f; acc1[i] = 0.f; }
        if (tid == 0 && my_tiles > 0) issue(0, uses & 1);
        bool alive = true;
        for (int it = 0; it < my_tiles; ++it, ++uses) {
            const int s = uses & 1;
            if (tid == 0 && it + 1 < my_tiles) issue(it + 1, s ^ 1);  // released by the barrier ending the last tile
            alive = mbar_wait_warp(&full[s], (uses >> 1) & 1, d.status, 52);
            if (!alive) break;
            const float *gt = gs + s * DW_G_STAGE + 4 * quad;
            const float *xt = xs + s * XT + 4 * quad + 3;
            float xw[CIN][3][6];  // sliding window: rows r, r+1, r+2 of the halo tile
#pragma unroll
            for (int c = 0; c < CIN; ++c)
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                    const float *row = xt + (c * DW_XR + rr) * GP;
                    xw[c][rr + 1][0] = ld_shared_f32(row);
                    const float4 a = ld_shared_v4(row + 1);
                    xw[c][rr + 1][1] = a.x; xw[c][rr + 1][2] = a.y; xw[c][rr + 1][3] = a.z; xw[c][rr + 1][4] = a.w;
                    xw[c][rr + 1][5] = ld_shared_f32(row + 5);
                }
#pragma unroll
            for (int r = 0; r < DW_ROWS; ++r) {
#pragma unroll
                for (int c = 0; c < CIN; ++c) {
#pragma unroll
                    for (int e = 0; e < 6; ++e) { xw[c][0][e] = xw[c][1][e]; xw[c][1][e] = xw[c][2][e]; }
                    const float *row = xt + (c * DW_XR + r + 2) * GP;
                    xw[c][2][0] = ld_shared_f32(row);
                    const float4 a = ld_shared_v4(row + 1);
                    xw[c][2][1] = a.x; xw[c][2][2] = a.y; xw[c][2][3] = a.z; xw[c][2][4] = a.w;
                    xw[c][2][5] = ld_shared_f32(row + 5);
                }
                const float4 ga = ld_shared_v4(gt + (pair * DW_ROWS + r) * 32);
                const float4 gb = ld_shared_v4(gt + ((pair + 32) * DW_ROWS + r) * 32);
                const float g0[4] = {ga.x, ga.y, ga.z, ga.w};
                const float g1[4] = {gb.x, gb.y, gb.z, gb.w};
#pragma unroll
                for (int c = 0; c < CIN; ++c)
#pragma unroll
                    for (int ky = 0; ky < 3; ++ky)
#pragma unroll
                        for (int kx = 0; kx < 3; ++kx)
#pragma unroll
                            for (int p = 0; p < 4; ++p) {
                                acc0[(c * 3 + ky) * 3 + kx] = fmaf(g0[p], xw[c][ky][p + kx], acc0[(c * 3 + ky) * 3 + kx]);
                                acc1[(c * 3 + ky) * 3 + kx] = fmaf(g1[p], xw[c][ky][p + kx], acc1[(c * 3 + ky) * 3 + kx]);
                            }
            }
            fence_proxy_async_smem();  // ordinary reads of the stage before its TMA refill
            __syncthreads();  // stage s may be refilled
        }
        if (!alive) return;
        // fold the eight quad lanes (lanes l, l^1, l^2, l^4 share a channel pair)
#pragma unroll
        for (int i = 0; i < TAPS; ++i) {
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) {
                acc0[i] += __shfl_xor_sync(0xffffffffu, acc0[i], o);
                acc1[i] += __shfl_xor_sync(0xffffffffu, acc1[i], o);
            }
        }
        if ((lane & 7) == 0) {
            float *dst = partial + size_t(blockIdx.x) * d.k * TAPS;
            const int oc0 = grp * 64 + pair, oc1 = oc0 + 32;
#pragma unroll
            for (int i = 0; i < TAPS; ++i) {
                if (oc0 < d.k) dst[size_t(oc0) * TAPS + i] = acc0[i];
                if (oc1 < d.k) dst[size_t(oc1) * TAPS + i] = acc1[i];
            }
        }
    }
}

__global__ void __launch_bounds__(256)
dw_partials_fold_kernel(const float *__restrict__ partial, float *dw, int elems, int parts, int accumulate) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= elems) return;
    float s = 0.f;
    for (int p = 0; p < parts; ++p) s += partial[size_t(p) * elems + i];
    dw[i] = accumulate ? dw[i] + s : s;
}

template <int CIN>
int32_t dw_launch(katsu_cuda_ctx *ctx, const CUtensorMap &map_g, const CUtensorMap &map_x, float *dw, DwDims d,
                  int accumulate) {
    constexpr int XT = (CIN * DW_XR * GP + 31) / 32 * 32;
    const size_t smem = (2 * size_t(DW_G_STAGE) + 2 * size_t(XT)) * sizeof(float);
    auto kernel = stencil_dw_tma_kernel<CIN>;
    KATSU_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const size_t total_tiles = size_t(d.n) * d.tiles_x * d.tiles_y;
    size_t grid = size_t(ctx->num_sms) * 2;
    if (grid > total_tiles) grid = total_tiles;
    const int elems = d.k * CIN * 9;
    float *partial = nullptr;
    KATSU_TRY(katsu_scratch(ctx, grid * elems, &partial));
    KATSU_LAUNCH(ctx, kernel, (unsigned)grid, 256, smem, map_g, map_x, partial, d);
    KATSU_LAUNCH(ctx, dw_partials_fold_kernel, (unsigned)katsu_div_up((size_t)elems, (size_t)256), 256, 0, partial, dw,
                 elems, (int)grid, accumulate);
    return KATSU_OK;
}

}  // namespace

// dW of the C_in <= 4, 3x3, stride 1, pad 1 convolution through TMA-fed tiles; *handled = 0
// when TMA cannot describe the operands.
int32_t katsu_stencil_dw_tma(katsu_cuda_ctx *ctx, const float *x, const float *g, float *dw, size_t n, size_t c,
                             size_t h, size_t wd, size_t k, int accumulate, int *handled) {
    *handled = 0;
    if (wd % 4 != 0 || c < 1 || c > 4 || k > 256 || n == 0) return KATSU_OK;
    if ((reinterpret_cast<uintptr_t>(g) & 15u) || (reinterpret_cast<uintptr_t>(x) & 15u)) return KATSU_OK;
    if (katsu_tensor_map_encoder() == nullptr) return KATSU_OK;
    CUtensorMap map_g, map_x;
    {
        const uint64_t dims[4] = {wd, h, k, n};
        const uint64_t strides[4] = {1, wd, wd * h, wd * h * k};
        const uint32_t box[4] = {32, DW_ROWS, 64, 1};
        if (!katsu_make_tensor_map(&map_g, g, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE)) return KATSU_OK;
    }
    {
        const uint64_t dims[4] = {wd, h, c, n};
        const uint64_t strides[4] = {1, wd, wd * h, wd * h * c};
        const uint32_t box[4] = {GP, DW_XR, (uint32_t)c, 1};
        if (!katsu_make_tensor_map(&map_x, x, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE)) return KATSU_OK;
    }
    *handled = 1;
    DwDims d;
    d.n = (int)n; d.k = (int)k; d.h = (int)h; d.w = (int)wd;
    d.tiles_x = (int)katsu_div_up(wd, 32);
    d.tiles_y = (int)katsu_div_up(h, (size_t)DW_ROWS);
    d.groups = (int)katsu_div_up(k, 64);
    d.status = ctx->status;
    switch (c) {
        case 1: return dw_launch<1>(ctx, map_g, map_x, dw, d, accumulate);
        case 2: return dw_launch<2>(ctx, map_g, map_x, dw, d, accumulate);
        case 3: return dw_launch<3>(ctx, map_g, map_x, dw, d, accumulate);
        default: return dw_launch<4>(ctx, map_g, map_x, dw, d, accumulate);
    }
}

// dX of the C_in <= 4, 3x3, stride 1, pad 1 convolution; *handled = 0 when TMA cannot
// describe g (width not a multiple of 4, unaligned pointers) and the caller keeps the
// plain-load kernel.
int32_t katsu_stencil_dx_tma(katsu_cuda_ctx *ctx, const float *w, const float *g, float *dx, size_t n, size_t c,
                             size_t h, size_t wd, size_t k, int accumulate, int *handled) {
    *handled = 0;
    if (wd % 4 != 0 || c < 1 || c > 4 || k > 256) return KATSU_OK;
    if ((reinterpret_cast<uintptr_t>(g) & 15u) || (reinterpret_cast<uintptr_t>(dx) & 15u)) return KATSU_OK;
    if (katsu_tensor_map_encoder() == nullptr) return KATSU_OK;
    *handled = 1;
    DxDims d;
    d.n = (int)n; d.k = (int)k; d.h = (int)h; d.w = (int)wd;
    d.tiles_x = (int)katsu_div_up(wd, (size_t)TWD);
    d.tiles_y = 0;
    d.kp = (int)katsu_div_up(k, (size_t)OCB) * OCB;
    d.accumulate = accumulate;
    d.status = ctx->status;
    switch (c) {
        case 1: return launch<1>(ctx, g, w, dx, d);
        case 2: return launch<2>(ctx, g, w, dx, d);
        case 3: return launch<3>(ctx, g, w, dx, d);
        default: return launch<4>(ctx, g, w, dx, d);
    }
}
