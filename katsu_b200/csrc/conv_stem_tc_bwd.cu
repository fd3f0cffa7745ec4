// Backward of the low-channel (C_in <= 3) 3x3 stride-1 pad-1 convolution on the tensor cores.
//
// Reference loops: backward_buffers (crates/katsu-core/src/conv2d.rs:269-292), i.e. for every
// visited (n, oc, oy, ox, ic, ky, kx): dX[n,ic,iy,ix] += g[n,oc,oy,ox] * W[oc,ic,ky,kx] and
// dW[oc,ic,ky,kx] += g[n,oc,oy,ox] * x[n,ic,iy,ix].
//
// On the FP32 pipe each of the two needs 27 * C_out multiply-adds per pixel, more time than
// reading g from HBM once.  As contractions over oc (dX) and over pixels (dW) they are a few
// hundred tensor-pipe cycles per 128 pixels and the kernels become bound by the read of g.
//
// dX:  Z[pixel, tap] = sum_oc g[oc, pixel] * W[oc, tap]         (a GEMM, K = C_out, N = 27 -> 32)
//      dX[c, iy, ix] = sum_{ky,kx} Z[(iy + 1 - ky, ix + 1 - kx), (c, ky, kx)]   (col2im)
//   A = g^T, 128 pixels x 16 oc per stage, held in TENSOR MEMORY (lane = pixel, column = oc) as
//       hi = trunc_tf32(v) and lo = v - hi, written by builder warps from the g tile TMA
//       dropped into shared memory ([16 oc][16 rows][36 columns], start column rounded down
//       to a 16-byte boundary, out-of-image cells arrive as zeros).
//   B = W as [tap][oc], K-major 128-byte-swizzled rows, built once per block (hi and lo).
//   D = four 128 x 32 accumulators per tile (a 16 x 32 pixel region of g), double buffered.
//   Every Z value is used exactly once, so the col2im is a gather through shared memory:
//   Z leaves TMEM as [tap][pixel] planes, each output pixel adds its nine (ky, kx) terms per
//   channel in a fixed order, and the 14 x 28 output tile goes out with one TMA store.
//   The region overlaps its neighbours by one pixel on each side (recomputed, not exchanged),
//   so no two blocks ever add into the same dX element and results are bit-reproducible.
//   Two warps issue MMAs (two M-tiles each): the elect.sync thread of one converged warp
//   sustains one N = 32 MMA per ~22 cycles, two such warps reach the pipe's 16 (measured).
#include "common.cuh"
#include <string.h>

#include "sm100.cuh"

using namespace sm100;

namespace {

__device__ __forceinline__ float tf32_hi(float v) { return __uint_as_float(__float_as_uint(v) & 0xFFFFE000u); }

__device__ __forceinline__ void store_chunk(unsigned char *tile, int row, int chunk, float4 v) {
    st_shared_v4(tile + row * 128 + ((chunk ^ (row & 7)) << 4), v);
}

struct StemDxDims {
    int n, k, h, w;
    int tiles_x, tiles_y;   // 28-column, 14-row output tiles
    int chunks;             // 16-oc chunks of g per tile
    int kblocks;            // 32-oc blocks of the filter operand
    int gs;                 // g stages in shared memory (DX_GS, or fewer when the filter operand is large)
    int three_pass;
    int accumulate;
    int *status;
    // The upstream gradient is gfactor * gscale[0] * g (gscale may be null: 1).  dX is linear in it,
    // so the factor is applied once per output element in the epilogue.
    const float *gscale;
    float gfactor;
};

constexpr int DX_TW = 28, DX_TH = 14;          // output tile
constexpr int DX_RW = 32, DX_RH = 16;          // g region that is multiplied (one halo pixel each side, padded)
constexpr int DX_GW = 36;                      // g columns TMA loads per row (region starts at column 3)
constexpr int DX_OC = 16;                      // oc per chunk
constexpr int DX_GSTAGE = DX_OC * DX_RH * DX_GW;  // floats per g stage
constexpr int DX_GS = 4;                       // g stages at most (StemDxDims::gs of them are used)
constexpr int DX_ZP = DX_RW * DX_RH;           // pixels per Z plane
constexpr int DX_THREADS = 15 * 32;

// Warp roles: 0-3 epilogue (TMEM lane quarter = warp), 4-11 builders (quarter = warp & 3,
// M-tiles {0,1} for warps 4-7 and {2,3} for warps 8-11), 12-13 MMA issue (M-tiles {0,1} and
// {2,3}), 14 TMA loads of g.
// TMEM columns: [2 D buffers x 4 M-tiles x 32][2 A stages x 4 M-tiles x {16 hi, 16 lo}] = 512.
template <int CIN>
__global__ void __launch_bounds__(DX_THREADS, 1)
stem_dx_tc_kernel(const float *__restrict__ w, float *dx, const __grid_constant__ CUtensorMap map_g,
                  const __grid_constant__ CUtensorMap map_dx, StemDxDims d) {
    constexpr int TAPS = CIN * 9;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // dynamic layout: B hi | B lo | g stages | Z planes | output tile
    unsigned char *b_hi = smem;
    unsigned char *b_lo = b_hi + d.kblocks * 4096;
    float *g_stages = reinterpret_cast<float *>(b_lo + d.kblocks * 4096);
    float *zs = g_stages + d.gs * DX_GSTAGE;
    float *outs = zs + TAPS * DX_ZP;
    __shared__ uint64_t g_full[DX_GS], g_empty[DX_GS], a_full[2], a_empty[2], d_full[2], d_empty[2];
    __shared__ uint32_t tmem_slot;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tiles_per_img = d.tiles_x * d.tiles_y;
    const int total_tiles = d.n * tiles_per_img;
    const int my_tiles = (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int NCH = d.chunks, GS = d.gs;

    if (tid == 0) {
        for (int s = 0; s < DX_GS; ++s) {
            mbar_init(&g_full[s], 1);
            mbar_init(&g_empty[s], 8);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&a_full[s], 8);    // one arrival per builder warp
            mbar_init(&a_empty[s], 2);
            mbar_init(&d_full[s], 2);
            mbar_init(&d_empty[s], 4);   // one arrival per epilogue warp
        }
        mbar_init_fence();
    }
    if (warp == 12) {
        tmem_alloc(&tmem_slot, 512);
        tmem_relinquish();
    }
    // filters -> B tiles: row = tap, 32 oc per 128-byte row, one tile of 32 rows per oc block
    for (int i = tid; i < d.kblocks * 32 * 8; i += DX_THREADS) {
        const int blk = i >> 8, t = (i >> 3) & 31, j = i & 7;
        float v[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int oc = blk * 32 + 4 * j + q;
            v[q] = (oc < d.k && t < TAPS) ? __ldg(w + size_t(oc) * TAPS + t) : 0.f;
        }
        const float4 hi = make_float4(tf32_hi(v[0]), tf32_hi(v[1]), tf32_hi(v[2]), tf32_hi(v[3]));
        store_chunk(b_hi + blk * 4096, t, j, hi);
        store_chunk(b_lo + blk * 4096, t, j, make_float4(v[0] - hi.x, v[1] - hi.y, v[2] - hi.z, v[3] - hi.w));
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;
    constexpr uint32_t A_COL0 = 256;

    if (warp >= 4 && warp < 12) {
        // ---- builders: thread = one pixel of two M-tiles; 16 oc per chunk -> TMEM A (hi | lo) ----
        const int quarter = warp & 3, half = (warp - 4) >> 2;
        for (int it = 0; it < my_tiles; ++it) {
            bool ok = true;
            for (int q = 0; q < NCH; ++q) {
                const int cc = it * NCH + q, gs = cc % GS, as = cc & 1;
                if (!mbar_wait_warp_ready(&g_full[gs], (cc / GS) & 1, d.status, 61)) { ok = false; break; }
                const float *st = g_stages + gs * DX_GSTAGE + 3 + lane;
                float v[2][32];
#pragma unroll
                for (int m = 0; m < 2; ++m) {
                    const int row = 4 * (2 * half + m) + quarter;
#pragma unroll
                    for (int oc = 0; oc < DX_OC; ++oc) {
                        const float val = ld_shared_f32(st + (oc * DX_RH + row) * DX_GW);
                        const float hi = tf32_hi(val);
                        v[m][oc] = hi;
                        v[m][16 + oc] = val - hi;
                    }
                }
                fence_proxy_async_smem();  // ordinary reads of the stage before its TMA refill
                __syncwarp();
                if (lane == 0) mbar_arrive(&g_empty[gs]);
                if (cc >= 2 && !mbar_wait_warp_ready(&a_empty[as], ((cc >> 1) - 1) & 1, d.status, 62)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t a_addr = tmem_base + (uint32_t(quarter * 32) << 16) + A_COL0 + uint32_t(as) * 128 + uint32_t(2 * half) * 32;
                tmem_st_32x32(a_addr, v[0]);
                tmem_st_32x32(a_addr + 32, v[1]);
                tmem_st_wait();
                tc_fence_before_sync();
                mbar_arrive_warp(&a_full[as]);  // tcgen05.wait::st above is warp-wide
            }
            if (!ok) break;
        }
    } else if (warp == 14 && lane == 0) {
        // ---- TMA loads of the g chunks ----
        for (int it = 0; it < my_tiles; ++it) {
            const int tile = blockIdx.x + it * gridDim.x;
            const int img = tile / tiles_per_img, tt = tile % tiles_per_img;
            const int x0 = (tt % d.tiles_x) * DX_TW, y0 = (tt / d.tiles_x) * DX_TH;
            bool ok = true;
            for (int q = 0; q < NCH; ++q) {
                const int cc = it * NCH + q, gs = cc % GS;
                if (cc >= GS && !mbar_wait(&g_empty[gs], ((cc / GS) - 1) & 1, d.status, 63)) { ok = false; break; }
                mbar_arrive_expect_tx(&g_full[gs], DX_GSTAGE * 4);
                tma_load_4d(g_stages + gs * DX_GSTAGE, &map_g, &g_full[gs], x0 - 4, y0 - 1, q * DX_OC, img);
            }
            if (!ok) break;
        }
    } else if (warp == 12 || warp == 13) {
        // ---- MMA issue: this warp's two M-tiles, every chunk.  The whole warp runs the loop and
        // the thread chosen by elect.sync issues: with warp-uniform control flow the operands
        // stay in uniform registers and one warp issues a small-N MMA every ~22 cycles
        // (measured; 44 behind a lane == 0 branch, 81 with a per-instruction lane test). ----
        const int mw = warp - 12;
        const bool issue = elect_one();
        const uint32_t idesc = idesc_tf32(128, 32, false, false);
        const uint64_t db_hi0 = smem_desc(smem_u32(b_hi), 16, 1024, kLayoutSw128);
        const uint64_t db_lo0 = smem_desc(smem_u32(b_lo), 16, 1024, kLayoutSw128);
        for (int it = 0; it < my_tiles; ++it) {
            const int db = it & 1;
            bool ok = true;
            for (int q = 0; q < NCH; ++q) {
                const int cc = it * NCH + q, as = cc & 1;
                if (!mbar_wait_warp_ready(&a_full[as], (cc >> 1) & 1, d.status, 64)) { ok = false; break; }
                if (q == 0 && it >= 2 && !mbar_wait_warp_ready(&d_empty[db], ((it >> 1) - 1) & 1, d.status, 65)) { ok = false; break; }
                tc_fence_after_sync();
#pragma unroll
                for (int m = 0; m < 2; ++m) {
                    const int j = 2 * mw + m;
                    const uint32_t acc = tmem_base + uint32_t(db) * 128 + uint32_t(j) * 32;
                    const uint32_t a_hi = tmem_base + A_COL0 + uint32_t(as) * 128 + uint32_t(j) * 32, a_lo = a_hi + 16;
#pragma unroll
                    for (int ks = 0; ks < 2; ++ks) {
                        const uint64_t off = uint64_t(((q >> 1) * 4096 + ((q & 1) * 2 + ks) * 32) >> 4);
                        const bool first = q == 0 && ks == 0;
                        if (issue) {
                            if (d.three_pass) {
                                mma_tf32_ts(acc, a_lo + 8 * ks, db_hi0 + off, idesc, !first);
                                mma_tf32_ts(acc, a_hi + 8 * ks, db_lo0 + off, idesc, true);
                                mma_tf32_ts(acc, a_hi + 8 * ks, db_hi0 + off, idesc, true);
                            } else {
                                mma_tf32_ts(acc, a_hi + 8 * ks, db_hi0 + off, idesc, !first);
                            }
                        }
                    }
                }
                if (issue) {
                    mma_commit(&a_empty[as]);
                    if (q == NCH - 1) mma_commit(&d_full[db]);
                }
                __syncwarp();
            }
            if (!ok) break;
        }
    } else if (warp < 4) {
        // ---- epilogue: Z out of TMEM into [tap][pixel] planes, col2im gather, TMA store ----
        const int quarter = warp;
        const size_t plane = size_t(d.h) * d.w;
        const float alpha = d.gfactor * (d.gscale != nullptr ? __ldg(d.gscale) : 1.f);
        bool alive = true;
        for (int it = 0; it < my_tiles; ++it) {
            const int db = it & 1;
            // A warp whose wait ran out keeps meeting the others at the named barriers (they may
            // have got through just before) and skips the work; once one wait of the launch has
            // failed all later waits return at once, so the rest of the loop is quick.
            if (alive) alive = mbar_wait_warp_ready(&d_full[db], (it >> 1) & 1, d.status, 66);
            tc_fence_after_sync();
            const int tile = blockIdx.x + it * gridDim.x;
            const int img = tile / tiles_per_img, tt = tile % tiles_per_img;
            const int x0 = (tt % d.tiles_x) * DX_TW, y0 = (tt / d.tiles_x) * DX_TH;
            if (alive) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float v[32];
                    tmem_ld_32x32(tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(db) * 128 + uint32_t(j) * 32, v);
                    float *zp = zs + (4 * j + quarter) * DX_RW + lane;
#pragma unroll
                    for (int t = 0; t < TAPS; ++t) st_shared_f32(zp + t * DX_ZP, v[t]);
                }
                tc_fence_before_sync();
                mbar_arrive_warp(&d_empty[db]);
            }
            if (tid == 0) tma_store_wait_read<0>();  // the previous tile's store has read `outs`
            named_barrier(1, 128);
            if (alive && lane < DX_TW) {
                for (int iy = warp; iy < DX_TH; iy += 4) {
                    const float *zr = zs + (iy + 2) * DX_RW + lane + 2;
#pragma unroll
                    for (int c = 0; c < CIN; ++c) {
                        float acc = 0.f;
#pragma unroll
                        for (int ky = 0; ky < 3; ++ky)
#pragma unroll
                            for (int kx = 0; kx < 3; ++kx)
                                acc += ld_shared_f32(zr + ((c * 3 + ky) * 3 + kx) * DX_ZP - ky * DX_RW - kx);
                        acc *= alpha;
                        if (d.accumulate) {
                            const int gy = y0 + iy, gx = x0 + lane;
                            if (gy < d.h && gx < d.w) acc = dx[(size_t(img) * CIN + c) * plane + size_t(gy) * d.w + gx] + acc;
                        }
                        st_shared_f32(outs + (c * DX_TH + iy) * DX_TW + lane, acc);
                    }
                }
            }
            fence_proxy_async_smem();
            named_barrier(1, 128);
            if (tid == 0 && alive) {
                tma_store_4d(&map_dx, outs, x0, y0, 0, img);
                tma_store_commit();
            }
        }
        if (tid == 0) tma_store_wait_all<0>();
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 12) tmem_dealloc(tmem_base, 512);
}

// Dynamic shared memory of the dX kernel with `gs` g stages.
template <int CIN>
size_t dx_smem_bytes(int kblocks, int gs) {
    return size_t(kblocks) * 8192 + size_t(gs) * DX_GSTAGE * 4 + size_t(CIN) * 9 * DX_ZP * 4 +
           size_t(CIN) * DX_TH * DX_TW * 4 + 1024;
}

// The most g stages (4, else 3) whose shared-memory request the SM can grant; 0 when neither fits
// (the caller then uses the CUDA-core kernel).  Three channels with more than 64 output channels
// need 233 056 B with four stages, above the 232 448 B a block may opt in to.
template <int CIN>
int dx_stages(int kblocks) {
    constexpr size_t kMaxOptIn = 232448 - 256;  // the kernel's barriers are static shared memory
    for (int gs = DX_GS; gs >= 3; --gs)
        if (dx_smem_bytes<CIN>(kblocks, gs) <= kMaxOptIn) return gs;
    return 0;
}

template <int CIN>
int32_t dx_launch(katsu_cuda_ctx *ctx, const float *w, const float *g, float *dx, StemDxDims d) {
    CUtensorMap map_g, map_dx;
    {
        const uint64_t dims[4] = {(uint64_t)d.w, (uint64_t)d.h, (uint64_t)d.k, (uint64_t)d.n};
        const uint64_t strides[4] = {1, (uint64_t)d.w, (uint64_t)d.w * d.h, (uint64_t)d.w * d.h * d.k};
        const uint32_t box[4] = {DX_GW, DX_RH, DX_OC, 1};
        if (!katsu_make_tensor_map(&map_g, g, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE))
            return katsu_set_error(KATSU_ERR_CUDA, "cuTensorMapEncodeTiled failed (stem dX g)");
    }
    {
        const uint64_t dims[4] = {(uint64_t)d.w, (uint64_t)d.h, (uint64_t)CIN, (uint64_t)d.n};
        const uint64_t strides[4] = {1, (uint64_t)d.w, (uint64_t)d.w * d.h, (uint64_t)d.w * d.h * CIN};
        const uint32_t box[4] = {DX_TW, DX_TH, CIN, 1};
        if (!katsu_make_tensor_map(&map_dx, dx, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE))
            return katsu_set_error(KATSU_ERR_CUDA, "cuTensorMapEncodeTiled failed (stem dX out)");
    }
    const size_t smem = dx_smem_bytes<CIN>(d.kblocks, d.gs);
    auto kernel = stem_dx_tc_kernel<CIN>;
    KATSU_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const size_t total_tiles = size_t(d.n) * d.tiles_x * d.tiles_y;
    size_t grid = size_t(ctx->num_sms);
    if (grid > total_tiles) grid = total_tiles;
    KATSU_LAUNCH(ctx, kernel, (unsigned)grid, DX_THREADS, smem, w, dx, map_g, map_dx, d);
    return KATSU_OK;
}


// ---------------------------------------------------------------------------------------
// dW:  dW[oc, tap] = sum_pixel g[oc, pixel] * Xcol[tap, pixel]   (a GEMM whose K is the pixel index)
//   A = [g_hi ; g_lo], 128 rows (64 oc twice) x 32 pixels per K-block, in TENSOR MEMORY
//       (lane = row, column = pixel), written by builder warps from the g row segment TMA
//       dropped into shared memory ([64 oc][32 px], 128-byte-swizzled rows so that 32 lanes
//       reading 32 different rows do not collide on banks).
//   B = [Xcol_hi ; Xcol_lo], 64 rows (32 taps twice) x 32 pixels, K-major swizzled rows in
//       shared memory, built from the x halo tile (the shifted windows cannot be loaded by
//       TMA: a shift of one pixel is not a 16-byte step).
//   D = 128 x 64: rows 0-63 hold hi*hi | hi*lo, rows 64-127 hold lo*hi | (lo*lo, unused).
//       One MMA per 8 pixels does all of 3xTF32.  Two accumulators alternate K-blocks and are
//       drained into running sums (shared memory) every DW_DRAIN K-blocks, which bounds the
//       length of any tensor-core accumulation chain (its f32 adds lose a little per step) to
//       2048 pixels.
//   Each block ends with one partial dW in scratch; a second kernel folds the partials in a
//   fixed order (bit-reproducible, no atomics).
struct StemDwDims {
    int n, k, h, w;
    int tiles_x, tiles_y;   // 32-pixel columns, 4-row bands
    int three_pass;
    int *status;
};

constexpr int DW_GS = 6;                 // g K-block stages (8 KiB each)
constexpr int DW_BS = 4;                 // B stages (8 KiB each); must equal DW_AS (shared barriers)
constexpr int DW_AS = 4;                 // A stages in TMEM (32 columns each)
constexpr int DW_XS = 3;                 // x halo tiles in flight
constexpr int DW_DRAIN = 128;            // K-blocks per drain period
constexpr int DW_THREADS = 13 * 32;
constexpr uint32_t DW_A_COL0 = 128;      // TMEM: [2 accumulators x 64][4 A stages x 32] = 256 columns
constexpr int DW_MMA_WARP = 11;  // warp 12 issues the TMA loads

// Warp roles: 0-3 and 4-7 two groups of A builders that alternate K-blocks (TMEM lane quarter
// = warp & 3; a group's chain load -> split -> tcgen05.st -> wait is several hundred cycles
// per K-block, two chains in flight per block hide it); group 0 also drains the accumulators.
// 8-10 B builders, 11 MMA issue, 12 TMA loads.  Two blocks share an SM (256 TMEM columns each),
// so the running sums of the drains live in shared memory, not registers.
template <int CIN>
__global__ void __launch_bounds__(DW_THREADS, 2)
stem_dw_tc_kernel(const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_x,
                  float *__restrict__ partial, StemDwDims d) {
    constexpr int TAPS = CIN * 9;
    constexpr int XT = (CIN * 6 * 40 + 31) / 32 * 32;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char *g_stages = smem;                           // DW_GS x 8 KiB
    unsigned char *b_stages = g_stages + DW_GS * 8192;        // DW_BS x 8 KiB
    float *sums = reinterpret_cast<float *>(b_stages + DW_BS * 8192);  // [32 columns][128 rows]
    float *x_tiles = sums + 32 * 128;                         // DW_XS x XT floats
    __shared__ uint64_t g_full[DW_GS], g_empty[DW_GS], ab_full[DW_AS], ab_empty[DW_AS], x_full[DW_XS], x_empty[DW_XS], d_full,
        d_empty;
    __shared__ uint32_t tmem_slot;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tiles_per_img = d.tiles_x * d.tiles_y;
    const int total_tiles = d.n * tiles_per_img;
    const int my_tiles = (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int my_kblocks = my_tiles * 4;

    if (tid == 0) {
        for (int s = 0; s < DW_GS; ++s) { mbar_init(&g_full[s], 1); mbar_init(&g_empty[s], 4); }
        // one barrier pair per stage for A and B together (the four A-builder warps of the K-block's group
        // + the three B-builder warps fill it, one commit frees it): every wait in the MMA warp's loop
        // costs ~90 cycles.  A warp arrives once, after tcgen05.wait::st (A, warp-wide) or after every
        // lane's proxy fence (B): 224 single arrivals per K-block were 224 serialised shared-memory
        // operations in a kernel that is bound by the shared-memory pipe.
        for (int s = 0; s < DW_AS; ++s) { mbar_init(&ab_full[s], 4 + 3); mbar_init(&ab_empty[s], 1); }
        for (int s = 0; s < DW_XS; ++s) { mbar_init(&x_full[s], 1); mbar_init(&x_empty[s], 3); }
        mbar_init(&d_full, 1);
        mbar_init(&d_empty, 4);
        mbar_init_fence();
    }
    if (warp == DW_MMA_WARP) {
        tmem_alloc(&tmem_slot, 256);
        tmem_relinquish();
    }
    // rows of B that no tap writes (27..31 and 59..63) stay zero for the whole kernel; sums start at zero
    for (int i = tid; i < (DW_BS * 8192 + 32 * 128 * 4) / 16; i += DW_THREADS)
        st_shared_v4(b_stages + i * 16, make_float4(0.f, 0.f, 0.f, 0.f));
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;

    if (warp < 8) {
        // ---- A builders: thread = one row of A (oc = row % 64; rows >= 64 carry the lo parts) ----
        const int group = warp >> 2, quarter = warp & 3, row = quarter * 32 + lane, oc = row & 63;
        const bool is_lo = quarter >= 2;
        const uint32_t lane_addr = tmem_base + (uint32_t(quarter * 32) << 16);
        // drain of period p (group 0 only): fold both accumulators into the running sums in
        // shared memory, then hand the accumulators back to the MMA warp
        auto drain = [&](int p) -> bool {
            if (!mbar_wait_warp_ready(&d_full, p & 1, d.status, 73)) return false;
            tc_fence_after_sync();
            const int in_period = (my_kblocks - p * DW_DRAIN) < DW_DRAIN ? (my_kblocks - p * DW_DRAIN) : DW_DRAIN;
            for (int a = 0; a < 2 && a < in_period; ++a) {
                // rows < 64: hi*hi (columns 0-31) and hi*lo (32-63); rows >= 64: lo*hi (0-31)
                for (int h = 0; h < (is_lo ? 1 : 2); ++h) {
                    float t0[32];
                    tmem_ld_32x32(lane_addr + uint32_t(a) * 64 + uint32_t(h) * 32, t0);
#pragma unroll
                    for (int t = 0; t < 32; ++t) st_shared_f32(sums + t * 128 + row, ld_shared_f32(sums + t * 128 + row) + t0[t]);
                }
            }
            tc_fence_before_sync();
            mbar_arrive_warp(&d_empty);
            return true;
        };
        bool ok = true;
        for (int kb = group; kb < my_kblocks; kb += 2) {
            if (group == 0 && kb > 0 && kb % DW_DRAIN == 0 && !drain(kb / DW_DRAIN - 1)) { ok = false; break; }
            const int gs = kb % DW_GS, as = kb % DW_AS;
            if (!mbar_wait_warp_ready(&g_full[gs], (kb / DW_GS) & 1, d.status, 71)) { ok = false; break; }
            const unsigned char *grow = g_stages + gs * 8192 + oc * 128;
            float v[32];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const float4 q = ld_shared_v4(grow + ((c ^ (oc & 7)) << 4));
                v[4 * c] = q.x; v[4 * c + 1] = q.y; v[4 * c + 2] = q.z; v[4 * c + 3] = q.w;
            }
            // hi rows go in as they are: the tensor core reads only the TF32 part of an operand
            // (it truncates), so the explicit split is needed for the lo rows alone
            if (is_lo) {
                if (d.three_pass) {
#pragma unroll
                    for (int t = 0; t < 32; ++t) v[t] -= tf32_hi(v[t]);
                } else {
#pragma unroll
                    for (int t = 0; t < 32; ++t) v[t] = 0.f;
                }
            }
            fence_proxy_async_smem();  // ordinary reads of the stage before its TMA refill
            __syncwarp();
            if (lane == 0) mbar_arrive(&g_empty[gs]);
            if (kb >= DW_AS && !mbar_wait_warp_ready(&ab_empty[as], ((kb / DW_AS) - 1) & 1, d.status, 72)) { ok = false; break; }
            tc_fence_after_sync();
            tmem_st_32x32(lane_addr + DW_A_COL0 + uint32_t(as) * 32, v);
            tmem_st_wait();
            tc_fence_before_sync();
            mbar_arrive_warp(&ab_full[as]);
        }
        if (group == 0) {
            if (ok) drain((my_kblocks - 1) / DW_DRAIN);
            // combine the hi rows with the lo rows of the same oc and write this block's partial
            named_barrier(1, 128);
            if (!is_lo && oc < d.k) {
                float *dst = partial + (size_t(blockIdx.x) * d.k + oc) * TAPS;
#pragma unroll
                for (int t = 0; t < TAPS; ++t) dst[t] = ld_shared_f32(sums + t * 128 + oc) + ld_shared_f32(sums + t * 128 + 64 + oc);
            }
        }
    } else if (warp < DW_MMA_WARP) {
        // ---- B builders: task = (channel, ky, 4-pixel chunk); writes the three kx taps, hi and lo ----
        const int task = (warp - 8) * 32 + lane;
        const int cky = task >> 3, j = task & 7;
        const bool active = cky < CIN * 3;
        const int c = cky / 3, ky = cky - 3 * c;
        int off_hi[3];  // byte offsets of this task's three chunks inside a B stage (lo rows: + 4096)
#pragma unroll
        for (int kx = 0; kx < 3; ++kx) {
            const int t = cky * 3 + kx;
            off_hi[kx] = t * 128 + ((j ^ (t & 7)) << 4);
        }
        const int src_off = (c * 6 + ky) * 40 + 4 * j + 3;
        for (int it = 0; it < my_tiles; ++it) {
            const int xs = it % DW_XS;
            if (!mbar_wait_warp_ready(&x_full[xs], (it / DW_XS) & 1, d.status, 74)) break;
            bool ok = true;
            for (int r = 0; r < 4; ++r) {
                const int kb = it * 4 + r, bs = kb % DW_BS;
                float f[6];
                if (active) {
                    const float *src = x_tiles + xs * XT + src_off + r * 40;
                    f[0] = ld_shared_f32(src);
                    const float4 q = ld_shared_v4(src + 1);
                    f[1] = q.x; f[2] = q.y; f[3] = q.z; f[4] = q.w;
                    f[5] = ld_shared_f32(src + 5);
                }
                if (kb >= DW_BS && !mbar_wait_warp_ready(&ab_empty[bs], ((kb / DW_BS) - 1) & 1, d.status, 75)) { ok = false; break; }
                if (active) {
                    unsigned char *bt = b_stages + bs * 8192;
                    float lo[6];
#pragma unroll
                    for (int e = 0; e < 6; ++e) lo[e] = d.three_pass ? f[e] - tf32_hi(f[e]) : 0.f;
#pragma unroll
                    for (int kx = 0; kx < 3; ++kx) {
                        st_shared_v4(bt + off_hi[kx], make_float4(f[kx], f[kx + 1], f[kx + 2], f[kx + 3]));
                        st_shared_v4(bt + off_hi[kx] + 4096, make_float4(lo[kx], lo[kx + 1], lo[kx + 2], lo[kx + 3]));
                    }
                }
                fence_proxy_async_smem();
                mbar_arrive_warp(&ab_full[bs]);
            }
            if (!ok) break;
            fence_proxy_async_smem();  // ordinary reads of the stage before its TMA refill
            __syncwarp();
            if (lane == 0) mbar_arrive(&x_empty[xs]);
        }
    } else if (warp == DW_MMA_WARP) {
        // ---- MMA issue (whole warp runs the loop, the elected thread issues) ----
        const bool issue = elect_one();
        const uint32_t idesc = idesc_tf32(128, 64, false, false);
        const uint64_t bdesc0 = smem_desc(smem_u32(b_stages), 16, 1024, kLayoutSw128);
        for (int kb = 0; kb < my_kblocks; ++kb) {
            const int as = kb % DW_AS, bs = kb % DW_BS;
            if (!mbar_wait_warp_ready(&ab_full[as], (kb / DW_AS) & 1, d.status, 76)) break;
            const int period = kb / DW_DRAIN, in_period = kb - period * DW_DRAIN;
            if (in_period == 0 && period > 0 && !mbar_wait_warp_ready(&d_empty, (period - 1) & 1, d.status, 78)) break;
            tc_fence_after_sync();
            const uint32_t acc = tmem_base + uint32_t(kb & 1) * 64;
            const uint32_t a_addr = tmem_base + DW_A_COL0 + uint32_t(as) * 32;
            const uint64_t bdesc = bdesc0 + uint64_t((bs * 8192) >> 4);
            if (issue) {
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                    mma_tf32_ts(acc, a_addr + 8 * ks, bdesc + uint64_t(2 * ks), idesc, !(in_period < 2 && ks == 0));
                mma_commit(&ab_empty[as]);
                if (in_period == DW_DRAIN - 1 || kb + 1 == my_kblocks) mma_commit(&d_full);
            }
            __syncwarp();
        }
    } else if (lane == 0) {
        // ---- TMA loads: one x halo tile per 4-row tile, one g row segment per K-block ----
        for (int it = 0; it < my_tiles; ++it) {
            const int tile = blockIdx.x + it * gridDim.x;
            const int img = tile / tiles_per_img, tt = tile % tiles_per_img;
            const int ox0 = (tt % d.tiles_x) * 32, oy0 = (tt / d.tiles_x) * 4;
            const int xs = it % DW_XS;
            if (it >= DW_XS && !mbar_wait(&x_empty[xs], ((it / DW_XS) - 1) & 1, d.status, 79)) break;
            mbar_arrive_expect_tx(&x_full[xs], CIN * 6 * 40 * 4);
            tma_load_4d(x_tiles + xs * XT, &map_x, &x_full[xs], ox0 - 4, oy0 - 1, 0, img);
            bool ok = true;
            for (int r = 0; r < 4; ++r) {
                const int kb = it * 4 + r, gs = kb % DW_GS;
                if (kb >= DW_GS && !mbar_wait(&g_empty[gs], ((kb / DW_GS) - 1) & 1, d.status, 80)) { ok = false; break; }
                mbar_arrive_expect_tx(&g_full[gs], 8192);
                tma_load_4d(g_stages + gs * 8192, &map_g, &g_full[gs], ox0, oy0 + r, 0, img);
            }
            if (!ok) break;
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == DW_MMA_WARP) tmem_dealloc(tmem_base, 256);
}

// dw (+)= sum over blocks of partial[block][oc][tap].  32 elements per block; eight thread groups
// each add every eighth partial, one group then adds the eight sums: a fixed order (bit-
// reproducible) with eight loads per element in flight instead of one (21 -> a few microseconds,
// which matters when a GPU's share of the batch makes the whole kernel 100 microseconds).
__global__ void __launch_bounds__(256)
stem_dw_fold_kernel(const float *__restrict__ partial, float *dw, int elems, int parts, int accumulate,
                    const float *__restrict__ gscale, float gfactor) {
    __shared__ float sums[8][32];
    const int i = blockIdx.x * 32 + (threadIdx.x & 31), part = threadIdx.x >> 5;
    float s = 0.f;
    if (i < elems)
        for (int p = part; p < parts; p += 8) s += partial[size_t(p) * elems + i];
    sums[part][threadIdx.x & 31] = s;
    __syncthreads();
    if (part == 0 && i < elems) {
        float total = sums[0][threadIdx.x];
#pragma unroll
        for (int q = 1; q < 8; ++q) total += sums[q][threadIdx.x];
        total *= gfactor * (gscale != nullptr ? __ldg(gscale) : 1.f);  // dW is linear in the upstream gradient
        dw[i] = accumulate ? dw[i] + total : total;
    }
}

template <int CIN>
int32_t dw_launch(katsu_cuda_ctx *ctx, const float *x, const float *g, float *dw, StemDwDims d, int accumulate,
                  const float *gscale, float gfactor) {
    CUtensorMap map_g, map_x;
    {
        const uint64_t dims[4] = {(uint64_t)d.w, (uint64_t)d.h, (uint64_t)d.k, (uint64_t)d.n};
        const uint64_t strides[4] = {1, (uint64_t)d.w, (uint64_t)d.w * d.h, (uint64_t)d.w * d.h * d.k};
        const uint32_t box[4] = {32, 1, 64, 1};
        if (!katsu_make_tensor_map(&map_g, g, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B))
            return katsu_set_error(KATSU_ERR_CUDA, "cuTensorMapEncodeTiled failed (stem dW g)");
    }
    {
        const uint64_t dims[4] = {(uint64_t)d.w, (uint64_t)d.h, (uint64_t)CIN, (uint64_t)d.n};
        const uint64_t strides[4] = {1, (uint64_t)d.w, (uint64_t)d.w * d.h, (uint64_t)d.w * d.h * CIN};
        const uint32_t box[4] = {40, 6, CIN, 1};
        if (!katsu_make_tensor_map(&map_x, x, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE))
            return katsu_set_error(KATSU_ERR_CUDA, "cuTensorMapEncodeTiled failed (stem dW x)");
    }
    constexpr int XT = (CIN * 6 * 40 + 31) / 32 * 32;
    // at least 100 KiB so that a third block (which could not get TMEM columns) is never co-resident
    size_t smem = size_t(DW_GS + DW_BS) * 8192 + 32 * 128 * 4 + size_t(DW_XS) * XT * 4 + 1024;
    if (smem < 100 * 1024) smem = 100 * 1024;
    auto kernel = stem_dw_tc_kernel<CIN>;
    KATSU_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const size_t total_tiles = size_t(d.n) * d.tiles_x * d.tiles_y;
    size_t grid = size_t(ctx->num_sms) * 2;
    if (grid > total_tiles) grid = total_tiles;
    const int elems = d.k * CIN * 9;
    float *partial = nullptr;
    KATSU_TRY(katsu_scratch(ctx, grid * elems, &partial));
    KATSU_LAUNCH(ctx, kernel, (unsigned)grid, DW_THREADS, smem, map_g, map_x, partial, d);
    KATSU_LAUNCH(ctx, stem_dw_fold_kernel, (unsigned)katsu_div_up((size_t)elems, (size_t)32), 256, 0, partial, dw, elems,
                 (int)grid, accumulate, gscale, gfactor);
    return KATSU_OK;
}

}  // namespace

namespace {

int dx_stages_for(size_t c, int kblocks) {
    return c == 1 ? dx_stages<1>(kblocks) : c == 2 ? dx_stages<2>(kblocks) : dx_stages<3>(kblocks);
}

bool dx_takes(const katsu_cuda_ctx *ctx, const float *g, const float *dx, size_t n, size_t c, size_t h, size_t wd,
              size_t k) {
    if (ctx->precision == KATSU_MODE_FP32) return false;
    if (c < 1 || c > 3 || k < 1 || k > 128 || h > 32768 || wd > 32768 || wd % 4 != 0) return false;
    if ((reinterpret_cast<uintptr_t>(g) & 15u) != 0 || (reinterpret_cast<uintptr_t>(dx) & 15u) != 0) return false;
    if (n * katsu_div_up(wd, DX_TW) * katsu_div_up(h, DX_TH) > 0x3fffffffu / 8) return false;  // chunk counters stay in int
    return katsu_tensor_map_encoder() != nullptr && dx_stages_for(c, (int)katsu_div_up(k, 32)) != 0;
}

bool dw_takes(const katsu_cuda_ctx *ctx, const float *x, const float *g, size_t n, size_t c, size_t h, size_t wd,
              size_t k) {
    if (ctx->precision == KATSU_MODE_FP32) return false;
    if (c < 1 || c > 3 || k < 1 || k > 64 || n == 0 || h > 32768 || wd > 32768 || wd % 4 != 0) return false;
    if ((reinterpret_cast<uintptr_t>(g) & 15u) != 0 || (reinterpret_cast<uintptr_t>(x) & 15u) != 0) return false;
    if (n * katsu_div_up(wd, 32) * katsu_div_up(h, 4) > 0x3fffffffu / 4) return false;  // K-block counters stay in int
    return katsu_tensor_map_encoder() != nullptr;
}

}  // namespace

// Whether the tensor-core kernels below take this backward call (the outputs that are asked for);
// they apply a scale on the upstream gradient themselves, other kernels need it materialised.
bool katsu_conv_stem_tc_bwd_takes(const katsu_cuda_ctx *ctx, const float *x, const float *g, const float *dx,
                                  const float *dw, size_t n, size_t c, size_t h, size_t wd, size_t k) {
    return (dx == nullptr || dx_takes(ctx, g, dx, n, c, h, wd, k)) && (dw == nullptr || dw_takes(ctx, x, g, n, c, h, wd, k));
}

int32_t katsu_conv_stem_tc_dx(katsu_cuda_ctx *ctx, const float *w, const float *g, float *dx, size_t n, size_t c,
                              size_t h, size_t wd, size_t k, int accumulate, const float *gscale, float gfactor,
                              int *handled) {
    *handled = 0;
    if (!dx_takes(ctx, g, dx, n, c, h, wd, k)) return KATSU_OK;
    StemDxDims d;
    d.n = (int)n; d.k = (int)k; d.h = (int)h; d.w = (int)wd;
    d.tiles_x = (int)katsu_div_up(wd, DX_TW);
    d.tiles_y = (int)katsu_div_up(h, DX_TH);
    d.chunks = (int)katsu_div_up(k, DX_OC);
    d.kblocks = (int)katsu_div_up(k, 32);
    d.three_pass = ctx->precision == KATSU_MODE_3XTF32 ? 1 : 0;
    d.accumulate = accumulate;
    d.status = ctx->status;
    d.gs = dx_stages_for(c, d.kblocks);
    d.gscale = gscale;
    d.gfactor = gfactor;
    *handled = 1;
    switch (c) {
        case 1: return dx_launch<1>(ctx, w, g, dx, d);
        case 2: return dx_launch<2>(ctx, w, g, dx, d);
        default: return dx_launch<3>(ctx, w, g, dx, d);
    }
}

int32_t katsu_conv_stem_tc_dw(katsu_cuda_ctx *ctx, const float *x, const float *g, float *dw, size_t n, size_t c,
                              size_t h, size_t wd, size_t k, int accumulate, const float *gscale, float gfactor,
                              int *handled) {
    *handled = 0;
    if (!dw_takes(ctx, x, g, n, c, h, wd, k)) return KATSU_OK;
    StemDwDims d;
    d.n = (int)n; d.k = (int)k; d.h = (int)h; d.w = (int)wd;
    d.tiles_x = (int)katsu_div_up(wd, 32);
    d.tiles_y = (int)katsu_div_up(h, 4);
    d.three_pass = ctx->precision == KATSU_MODE_3XTF32 ? 1 : 0;
    d.status = ctx->status;
    *handled = 1;
    switch (c) {
        case 1: return dw_launch<1>(ctx, x, g, dw, d, accumulate, gscale, gfactor);
        case 2: return dw_launch<2>(ctx, x, g, dw, d, accumulate, gscale, gfactor);
        default: return dw_launch<3>(ctx, x, g, dw, d, accumulate, gscale, gfactor);
    }
}
