// Wide-channel convolution as implicit GEMM on tcgen05 (forward, dX, dW).
//
// Reference loops: Conv2D::forward's visit closure (crates/katsu-core/src/conv2d.rs:95-103,
// 232-262) and backward_buffers (conv2d.rs:269-292).
//
// Layout problem and its answer.  The reference layout is NCHW with W innermost, and a
// filter tap shifts the window by +-1 pixel along W.  TMA cannot start a tile at an
// address that is not 16-byte aligned, so shifted NCHW tiles cannot be fetched directly.
// Each call therefore first copies its activation operand (x for forward and dW, g for
// dX and dW) into a channels-innermost staging buffer [N][H][W][C]; there a tap shift
// moves along outer dimensions (no alignment rule, out-of-range coordinates are
// zero-filled == the reference's skipped padding taps) and a pixel's channels are one
// contiguous K-major row.  The same pass writes the "lo" halves for 3xTF32
// (lo = v - trunc_tf32(v); the tensor core itself truncates the raw value to "hi").
// The transform costs 2-3 |x| of HBM traffic against a tensor-bound contraction.
//
//   forward : Y[pixel, oc]  = sum_tap  X[pixel + tap, c]  * Wf[tap][oc][c]     (A, B K-major)
//   dX      : dX[pixel, c]  = sum_tap  G[(pixel + p - tap) / s, oc] * Wb[tap][c][oc]
//             one launch per stride-parity class of input pixels      (A, B K-major)
//   dW      : dW[tap][oc, c] = sum_pixel G[pixel, oc] * X[pixel*s + tap - p, c] (A, B MN-major)
//
// Tiles are 128 (two 64-pixel blocks, or 128 output channels for dW) x 32..256 by channel count, k-blocks of
// 32 channels or pixels, both operands read by the tensor core from shared memory.  In 3xTF32 the stages carry
// hi and lo halves and accumulation chains are kept short (rotating accumulators; beyond ~300 accumulation steps,
// or with 256-wide tiles, two accumulators that are folded into registers in turn); in single-pass TF32 the
// stages carry hi only, the ring is deeper and tiles are as wide as the layer allows (256 channels, or several
// filter taps side by side in dW), because that mode is bound by getting operands into shared memory.
#include "common.cuh"
#include "sm100.cuh"

using namespace sm100;

namespace {

constexpr int BM = 128, BN = 128, BK = 32, NACC = 4, STAGES = 3;
constexpr int TILE_BYTES = BM * BK * 4;
constexpr int MAX_TAPS = 49;

__device__ __forceinline__ float lo_part(float v) { return v - __uint_as_float(__float_as_uint(v) & 0xFFFFE000u); }

// ---- staging passes ---------------------------------------------------------------
// [N][C][HW] -> [N][HW][C] through 32x33 shared tiles; optionally also the lo halves.  A block
// moves four 32-pixel x 32-channel tiles and issues all of its loads before the first store, so
// that enough bytes are in flight per SM (one tile per block ran at 3.8 TB/s of traffic).
constexpr int NHWC_TILES = 4;

__global__ void __launch_bounds__(256)
nchw_to_nhwc_kernel(const float *__restrict__ src, float *__restrict__ dst, float *__restrict__ dst_lo, int c, int hw) {
    __shared__ float tile[NHWC_TILES][32][33];
    const int n = blockIdx.z;
    const int p0 = blockIdx.x * (32 * NHWC_TILES), c0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    const float *s = src + size_t(n) * c * hw;
#pragma unroll
    for (int t = 0; t < NHWC_TILES; ++t)
#pragma unroll
        for (int i = ty; i < 32; i += 8) {
            const int cc = c0 + i, pp = p0 + 32 * t + tx;
            tile[t][i][tx] = (cc < c && pp < hw) ? __ldg(s + size_t(cc) * hw + pp) : 0.f;
        }
    __syncthreads();
#pragma unroll
    for (int t = 0; t < NHWC_TILES; ++t)
#pragma unroll
        for (int i = ty; i < 32; i += 8) {
            const int pp = p0 + 32 * t + i, cc = c0 + tx;
            if (pp < hw && cc < c) {
                const float v = tile[t][tx][i];
                const size_t o = (size_t(n) * hw + pp) * c + cc;
                dst[o] = v;
                if (dst_lo != nullptr) dst_lo[o] = lo_part(v);
            }
        }
}

// w[K][C][taps] -> wf[tap][K][C] (forward B, rows = oc) and/or wb[tap][C][K] (dX B, rows = c), with lo halves.
__global__ void __launch_bounds__(256)
weights_to_taps_kernel(const float *__restrict__ w, float *wf, float *wf_lo, float *wb, float *wb_lo, int k, int c,
                       int taps) {
    const size_t total = size_t(k) * c * taps;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
        const int t = int(i % taps);
        const int cc = int((i / taps) % c);
        const int kk = int(i / (size_t(taps) * c));
        const float v = w[i];
        if (wf != nullptr) {
            const size_t o = (size_t(t) * k + kk) * c + cc;
            wf[o] = v;
            if (wf_lo != nullptr) wf_lo[o] = lo_part(v);
        }
        if (wb != nullptr) {
            const size_t o = (size_t(t) * c + cc) * k + kk;
            wb[o] = v;
            if (wb_lo != nullptr) wb_lo[o] = lo_part(v);
        }
    }
}

// ---- forward / dX kernel ------------------------------------------------------------
struct IgemmParams {
    float *out;                 // NCHW output
    int n_img, out_c, out_h, out_w;
    int blocks_x, blocks_y, bw, bh;  // 64-pixel blocks (bw * bh == 64) over this launch's pixel grid
    int grid_h, grid_w;         // extent of the pixel grid (all output pixels, or one parity class)
    int out_sy, out_oy, out_sx, out_ox;  // output pixel = (out_sy * jy + out_oy, out_sx * jx + out_ox)
    int in_step;                // operand coordinate = j * in_step + tap offset
    int kc;                     // channels of the operand (GEMM K per tap)
    int ntaps;
    int accumulate, three_pass;
    int *status;
    short off_y[MAX_TAPS], off_x[MAX_TAPS], b_tap[MAX_TAPS];
    // merge_x = 1 (dX of a stride-2 layer): every pixel tile is computed twice in a row, once per x-parity
    // class (the second with the tap table below), into the two accumulator sets; the epilogue keeps the first
    // class's results in registers and writes the two results of a pixel pair side by side (output x = 2 jx
    // and 2 jx + 1).  One launch per class left every 32-byte sector of dX half written, twice.
    int merge_x, ntaps2, grid_w2;
    short off_y2[MAX_TAPS], off_x2[MAX_TAPS], b_tap2[MAX_TAPS];
};

// Persistent: one block per SM walks (pixel tile, channel tile) pairs.  BNT = 128 / 64 / 32 output
// channels per tile, chosen by the launch from the channel count so that narrow layers do not
// pay for 128-wide MMAs and operand tiles.  Warps 0-3 are the epilogue (TMEM lane quarter =
// warp), warp 4 issues the TMA loads, warp 5 the MMAs.  Two accumulator sets alternate between
// tiles so a tile's epilogue runs under the next tile's k-loop; a set is NACC_T rotating
// accumulators (2 of 128 columns, or 4 of 64 / 32).
// SINGLE = single-pass TF32: no lo halves are loaded, a stage is A | B only, so the ring is twice as deep in
// the same shared memory (the k-loop is bound by getting operands in, not by the pipe), and with 256 or more
// output channels the tile is 128 x 256 (one accumulator of 256 columns per set): the pixel operand is then
// fetched once per 256 instead of per 128 output channels.
template <int BNT, bool SINGLE>
struct IgemmCfg {
    static constexpr int NACC_T = BNT == 256 ? 1 : BNT == 128 ? 2 : 4;
    static constexpr int SET_COLS = NACC_T * BNT;
    static constexpr int TMEM_COLS = 2 * SET_COLS;                 // 512, 512, 512, 256
    static constexpr int B_BYTES = BNT * BK * 4;
    static constexpr int B_OFF = SINGLE ? TILE_BYTES : 2 * TILE_BYTES;  // A hi | (A lo) | B hi | (B lo)
    static constexpr int STAGE_BYTES = SINGLE ? TILE_BYTES + B_BYTES : 2 * TILE_BYTES + 2 * B_BYTES;
    static constexpr int FIT = (200 * 1024) / STAGE_BYTES;
    static constexpr int STAGES_T = SINGLE ? (FIT > 8 ? 8 : FIT) : (BNT == 128 ? 3 : 4);
    static constexpr size_t SMEM = size_t(STAGES_T) * STAGE_BYTES + 1024;
    static_assert(SINGLE || BNT <= 128, "the split-precision stage of a 256-wide tile does not fit twice");
};

template <int BNT, bool SINGLE, bool MERGE>
__global__ void __launch_bounds__(192, 1)
conv_igemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_a_lo,
                  const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_b_lo,
                  const __grid_constant__ IgemmParams p, int m_tiles, int n_tiles) {
    using Cfg = IgemmCfg<BNT, SINGLE>;
    constexpr int NACC_T = Cfg::NACC_T, STAGES_T = Cfg::STAGES_T;
    constexpr int PARTS = SINGLE ? 1 : 2;  // hi, lo
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full[STAGES_T], empty[STAGES_T], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int blocks_per_img = p.blocks_x * p.blocks_y;
    const int kchunks = (p.kc + BK - 1) / BK;
    const int kblocks_cls[2] = {p.ntaps * kchunks, p.ntaps2 * kchunks};
    const int total_tiles = m_tiles * n_tiles;
    // passes over the accumulator sets: one per tile, or two per tile (class 0, class 1) with merge_x
    constexpr int shift = MERGE ? 1 : 0;
    const int my_tiles = ((total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x) << shift;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES_T; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 128);
        }
        mbar_init_fence();
    }
    if (warp == 5) {
        tmem_alloc(&tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;

    if (warp == 4 && lane == 0) {
        // ---- TMA producer ----
        bool ok = true;
        int g = 0;  // stages filled so far
        for (int it = 0; it < my_tiles && ok; ++it) {
            const int tile = blockIdx.x + (it >> shift) * gridDim.x, cls = it & shift;
            const int kblocks = kblocks_cls[cls];
            const int mt = tile / n_tiles, n0 = (tile % n_tiles) * BNT;
            // block coordinates of the tile's two 64-pixel halves
            int bn[2], by[2], bx[2];
            for (int h = 0; h < 2; ++h) {
                const long long gb = 2ll * mt + h;
                bn[h] = int(gb / blocks_per_img);  // == n_img for a block past the end: TMA zero-fills it
                const int r = int(gb % blocks_per_img);
                by[h] = r / p.blocks_x;
                bx[h] = r % p.blocks_x;
            }
            for (int i = 0; i < kblocks; ++i, ++g) {
                const int s = g % STAGES_T;
                if (g >= STAGES_T && !mbar_wait(&empty[s], ((g / STAGES_T) - 1) & 1, p.status, 21)) { ok = false; break; }
                mbar_arrive_expect_tx(&full[s], PARTS * (TILE_BYTES + Cfg::B_BYTES));
                unsigned char *st = smem + s * Cfg::STAGE_BYTES;
                const int t = i / kchunks, k0 = (i % kchunks) * BK;
                const int ox = cls ? p.off_x2[t] : p.off_x[t], oy = cls ? p.off_y2[t] : p.off_y[t];
                const int bt = cls ? p.b_tap2[t] : p.b_tap[t];
                for (int part = 0; part < PARTS; ++part) {
                    const CUtensorMap *ma = part ? &map_a_lo : &map_a;
                    const CUtensorMap *mb = part ? &map_b_lo : &map_b;
                    for (int h = 0; h < 2; ++h)
                        tma_load_4d(st + part * TILE_BYTES + h * (TILE_BYTES / 2), ma, &full[s], k0,
                                    bx[h] * p.bw * p.in_step + ox, by[h] * p.bh * p.in_step + oy, bn[h]);
                    tma_load_4d(st + Cfg::B_OFF + part * Cfg::B_BYTES, mb, &full[s], k0, n0, bt, 0);
                }
            }
        }
    } else if (warp == 5) {
        // ---- MMA issue: whole warp in the loop, the elect.sync thread issues (uniform control
        // flow keeps operands in uniform registers and makes waits on full stages cheap) ----
        const bool issue = elect_one();
        const uint32_t idesc = idesc_tf32(BM, BNT, false, false);
        bool ok = true;
        int g = 0;  // stages consumed so far
        for (int it = 0; it < my_tiles && ok; ++it) {
            const int b = it & 1;
            const int kblocks = kblocks_cls[it & shift];
            if (it >= 2 && !mbar_wait_warp(&acc_empty[b], ((it >> 1) - 1) & 1, p.status, 24)) break;
            tc_fence_after_sync();
            for (int i = 0; i < kblocks; ++i, ++g) {
                const int s = g % STAGES_T;
                if (!mbar_wait_warp_ready(&full[s], (g / STAGES_T) & 1, p.status, 22)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t st = smem_u32(smem + s * Cfg::STAGE_BYTES);
                const uint32_t acc = tmem_base + uint32_t(b) * Cfg::SET_COLS + uint32_t(i % NACC_T) * BNT;
                const bool first = i < NACC_T;
                if (issue) {
#pragma unroll
                    for (int j = 0; j < BK / 8; ++j) {
                        const uint64_t a_hi = smem_desc(st + j * 32, 16, 1024, kLayoutSw128);
                        const uint64_t b_hi = smem_desc(st + Cfg::B_OFF + j * 32, 16, 1024, kLayoutSw128);
                        if (!SINGLE) {
                            const uint64_t a_lo = smem_desc(st + TILE_BYTES + j * 32, 16, 1024, kLayoutSw128);
                            const uint64_t b_lo = smem_desc(st + Cfg::B_OFF + Cfg::B_BYTES + j * 32, 16, 1024, kLayoutSw128);
                            mma_tf32(acc, a_lo, b_hi, idesc, !(first && j == 0));
                            mma_tf32(acc, a_hi, b_lo, idesc, true);
                            mma_tf32(acc, a_hi, b_hi, idesc, true);
                        } else {
                            mma_tf32(acc, a_hi, b_hi, idesc, !(first && j == 0));
                        }
                    }
                    mma_commit(&empty[s]);
                    if (i == kblocks - 1) mma_commit(&acc_full[b]);
                }
                __syncwarp();
            }
        }
    } else if (warp < 4) {
        // ---- epilogue: thread = pixel; accumulators summed in registers, 32 channels at a time ----
        const int r = warp * 32 + lane;
        const size_t plane = size_t(p.out_h) * p.out_w;
        // merge_x: the first class's results of this thread's pixel, kept until the second class's are ready
        constexpr int HELD = MERGE ? BNT : 1;
        float held[HELD];
        for (int it = 0; it < my_tiles; ++it) {
            const int b = it & 1;
            const int cls = it & shift;
            const int kblocks = kblocks_cls[cls];
            const int used_acc = kblocks < NACC_T ? kblocks : NACC_T;
            if (!mbar_wait_warp(&acc_full[b], (it >> 1) & 1, p.status, 23)) break;
            tc_fence_after_sync();
            const int tile = blockIdx.x + (it >> shift) * gridDim.x;
            const int mt = tile / n_tiles, n0 = (tile % n_tiles) * BNT;
            const long long gb = 2ll * mt + (r >> 6);
            const int img = int(gb / blocks_per_img);
            const int rb = int(gb % blocks_per_img);
            const int jy = (rb / p.blocks_x) * p.bh + (r & 63) / p.bw;
            const int jx = (rb % p.blocks_x) * p.bw + (r & 63) % p.bw;
            const bool pixel_ok = img < p.n_img && jy < p.grid_h && jx < p.grid_w;
            const int oy = p.out_sy * jy + p.out_oy, ox = p.out_sx * jx + p.out_ox;
            float *dst_px = p.out + size_t(img) * p.out_c * plane + size_t(oy) * p.out_w + ox;
            const uint32_t set = tmem_base + (uint32_t(warp * 32) << 16) + uint32_t(b) * Cfg::SET_COLS;
            if constexpr (MERGE) {
                {
                    // pixel pair (oy, 2 jx), (oy, 2 jx + 1): class 0 is held, class 1 completes the pair
                    const bool ok2 = pixel_ok && jx < p.grid_w2;
                    // (pairs start at even x: 8-byte aligned when the rows and the tensor itself are)
                    const bool vec = ok2 && ((p.out_w & 1) == 0) && !p.accumulate && (reinterpret_cast<uintptr_t>(p.out) & 7u) == 0;
#pragma unroll
                    for (int c0 = 0; c0 < BNT; c0 += 32) {
                        float v[32];
                        tmem_ld_32x32(set + c0, v);
                        for (int a = 1; a < used_acc; ++a) {
                            float t[32];
                            tmem_ld_32x32(set + a * BNT + c0, t);
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] += t[i];
                        }
                        if (c0 + 32 >= BNT) {
                            tc_fence_before_sync();
                            mbar_arrive(&acc_empty[b]);
                        }
                        if (cls == 0) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) held[c0 + i] = v[i];
                        } else if (pixel_ok) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                const int ch = n0 + c0 + i;
                                if (ch < p.out_c) {
                                    float *dst = dst_px + size_t(ch) * plane;
                                    if (vec) {
                                        *reinterpret_cast<float2 *>(dst) = make_float2(held[c0 + i], v[i]);
                                    } else {
                                        dst[0] = p.accumulate ? dst[0] + held[c0 + i] : held[c0 + i];
                                        if (ok2) dst[1] = p.accumulate ? dst[1] + v[i] : v[i];
                                    }
                                }
                            }
                        }
                    }
                    continue;
                }
            }
            for (int c0 = 0; c0 < BNT; c0 += 32) {
                const bool last_group = c0 + 32 >= BNT || n0 + c0 + 32 >= p.out_c;
                float v[32];
                tmem_ld_32x32(set + c0, v);
                for (int a = 1; a < used_acc; ++a) {
                    float t[32];
                    tmem_ld_32x32(set + a * BNT + c0, t);
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] += t[i];
                }
                if (last_group) {
                    // everything this tile needs from the accumulators is in registers now
                    tc_fence_before_sync();
                    mbar_arrive(&acc_empty[b]);
                }
                if (pixel_ok) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int ch = n0 + c0 + i;
                        if (ch < p.out_c) {
                            float *dst = dst_px + size_t(ch) * plane;
                            *dst = p.accumulate ? *dst + v[i] : v[i];
                        }
                    }
                }
                if (last_group) break;
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 5) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// ---- forward / dX, 3xTF32, 256 or more output channels ---------------------------------------
// The k-loop of the split-precision kernel above is bound by shared-memory bandwidth: a stage's bytes are
// written once by TMA and every MMA reads its A and B tiles from there, and with 128 x 128 tiles the twelve
// MMAs of a k-block read 96 KiB for 64 KiB of fill.  A 128 x 256 tile needs 144 KiB of reads and 96 KiB of
// fill for twice the work.  Tensor memory then holds exactly two 256-column accumulators, which take turns:
// one receives DRAIN3 k-blocks (16 x 12 = 192 accumulations, shorter than the 216 of the rotating
// accumulators above, so the split-precision error bar is kept) while the other is folded into f32
// registers by eight epilogue warps (lane quarter = warp % 4, column half = warp / 4, 128 running sums per
// thread).  Warp 8 issues the TMA loads, warp 9 the MMAs.  A k-block is 16 channels (64-byte rows, 64-byte
// swizzle), so that four stages of 48 KiB fit: with two stages of 96 KiB a stage's fill and its MMAs cannot
// overlap and the loop ran at 2480 clocks per 32 channels.
constexpr int BK3 = 16;
constexpr int DRAIN3 = 32;  // k-blocks of 16 channels
constexpr int WIDE3_A_BYTES = BM * BK3 * 4;
constexpr uint32_t kLayoutSw64 = 4;
// BNT = 256 for layers with that many output channels; BNT = 128 is the same kernel for narrower layers whose
// contraction is too long for the rotating accumulators of conv_igemm_kernel (see drained_kernel_needed).
template <int BNT>
struct Wide3Cfg {
    static constexpr int B_BYTES = BNT * BK3 * 4;
    static constexpr int STAGE_BYTES = 2 * WIDE3_A_BYTES + 2 * B_BYTES;   // 48 / 32 KiB
    static constexpr int STAGES = BNT == 256 ? 4 : 6;
    static constexpr size_t SMEM = size_t(STAGES) * STAGE_BYTES + 1024;
    static constexpr int HALF = BNT / 2;   // columns folded by one epilogue thread
};

template <int BNT>
__global__ void __launch_bounds__(320, 1)
conv_igemm_wide3_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_a_lo,
                        const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_b_lo,
                        const __grid_constant__ IgemmParams p, int m_tiles, int n_tiles) {
    using Cfg = Wide3Cfg<BNT>;
    constexpr int A_BYTES = WIDE3_A_BYTES, B_BYTES = Cfg::B_BYTES, B_OFF = 2 * A_BYTES;
    constexpr int WIDE3_STAGES = Cfg::STAGES, WIDE3_STAGE_BYTES = Cfg::STAGE_BYTES, HALF = Cfg::HALF;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full[WIDE3_STAGES], empty[WIDE3_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int blocks_per_img = p.blocks_x * p.blocks_y;
    const int kchunks = (p.kc + BK3 - 1) / BK3;
    const int kblocks = p.ntaps * kchunks;
    const int batches = (kblocks + DRAIN3 - 1) / DRAIN3;
    const int total_tiles = m_tiles * n_tiles;
    const int my_tiles = (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < WIDE3_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 8);
        }
        mbar_init_fence();
    }
    if (warp == 9) {
        tmem_alloc(&tmem_slot, 2 * BNT);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;

    if (warp == 8 && lane == 0) {
        // ---- TMA producer ----
        bool ok = true;
        for (int it = 0; it < my_tiles && ok; ++it) {
            const int tile = blockIdx.x + it * gridDim.x;
            const int mt = tile / n_tiles, n0 = (tile % n_tiles) * BNT;
            int bn[2], by[2], bx[2];
            for (int h = 0; h < 2; ++h) {
                const long long gb = 2ll * mt + h;
                bn[h] = int(gb / blocks_per_img);  // == n_img for a block past the end: TMA zero-fills it
                const int r = int(gb % blocks_per_img);
                by[h] = r / p.blocks_x;
                bx[h] = r % p.blocks_x;
            }
            for (int i = 0; i < kblocks; ++i) {
                const int g = it * kblocks + i, s = g % WIDE3_STAGES;
                if (g >= WIDE3_STAGES && !mbar_wait(&empty[s], ((g / WIDE3_STAGES) - 1) & 1, p.status, 25)) { ok = false; break; }
                mbar_arrive_expect_tx(&full[s], WIDE3_STAGE_BYTES);
                unsigned char *st = smem + s * WIDE3_STAGE_BYTES;
                const int t = i / kchunks, k0 = (i % kchunks) * BK3;
                for (int part = 0; part < 2; ++part) {
                    const CUtensorMap *ma = part ? &map_a_lo : &map_a;
                    const CUtensorMap *mb = part ? &map_b_lo : &map_b;
                    for (int h = 0; h < 2; ++h)
                        tma_load_4d(st + part * A_BYTES + h * (A_BYTES / 2), ma, &full[s], k0,
                                    bx[h] * p.bw * p.in_step + p.off_x[t], by[h] * p.bh * p.in_step + p.off_y[t], bn[h]);
                    tma_load_4d(st + B_OFF + part * B_BYTES, mb, &full[s], k0, n0, p.b_tap[t], 0);
                }
            }
        }
    } else if (warp == 9) {
        // ---- MMA issue: whole warp in the loop, the elect.sync thread issues ----
        const bool issue = elect_one();
        const uint32_t idesc = idesc_tf32(BM, BNT, false, false);
        bool ok = true;
        int q = 0;  // accumulator hand-overs so far (batches of all tiles)
        for (int it = 0; it < my_tiles && ok; ++it) {
            for (int bi = 0; bi < batches && ok; ++bi, ++q) {
                const int b = q & 1;
                if (q >= 2 && !mbar_wait_warp(&acc_empty[b], ((q >> 1) - 1) & 1, p.status, 26)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t acc = tmem_base + uint32_t(b) * BNT;
                const int i_end = (bi + 1) * DRAIN3 < kblocks ? (bi + 1) * DRAIN3 : kblocks;
                for (int i = bi * DRAIN3; i < i_end; ++i) {
                    const int g = it * kblocks + i, s = g % WIDE3_STAGES;
                    if (!mbar_wait_warp_ready(&full[s], (g / WIDE3_STAGES) & 1, p.status, 27)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t st = smem_u32(smem + s * WIDE3_STAGE_BYTES);
                    const bool first = i == bi * DRAIN3;
                    if (issue) {
#pragma unroll
                        for (int j = 0; j < BK3 / 8; ++j) {
                            const uint64_t a_hi = smem_desc(st + j * 32, 16, 512, kLayoutSw64);
                            const uint64_t b_hi = smem_desc(st + B_OFF + j * 32, 16, 512, kLayoutSw64);
                            const uint64_t a_lo = smem_desc(st + A_BYTES + j * 32, 16, 512, kLayoutSw64);
                            const uint64_t b_lo = smem_desc(st + B_OFF + B_BYTES + j * 32, 16, 512, kLayoutSw64);
                            mma_tf32(acc, a_lo, b_hi, idesc, !(first && j == 0));
                            mma_tf32(acc, a_hi, b_lo, idesc, true);
                            mma_tf32(acc, a_hi, b_hi, idesc, true);
                        }
                        mma_commit(&empty[s]);
                        if (i == i_end - 1) mma_commit(&acc_full[b]);
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp < 8) {
        // ---- epilogue: thread = pixel x column half; running sums in registers ----
        const int quarter = warp & 3, half = warp >> 2;
        const int r = quarter * 32 + lane;
        const size_t plane = size_t(p.out_h) * p.out_w;
        int q = 0;
        bool alive = true;
        for (int it = 0; it < my_tiles && alive; ++it) {
            float run[HALF];
#pragma unroll
            for (int i = 0; i < HALF; ++i) run[i] = 0.f;
            for (int bi = 0; bi < batches; ++bi, ++q) {
                const int b = q & 1;
                if (!mbar_wait_warp(&acc_full[b], (q >> 1) & 1, p.status, 28)) { alive = false; break; }
                tc_fence_after_sync();
                const uint32_t acc = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(b) * BNT + uint32_t(half) * HALF;
#pragma unroll
                for (int c0 = 0; c0 < HALF; c0 += 32) {
                    float t[32];
                    tmem_ld_32x32(acc + c0, t);
#pragma unroll
                    for (int i = 0; i < 32; ++i) run[c0 + i] += t[i];
                }
                tc_fence_before_sync();
                mbar_arrive_warp(&acc_empty[b]);
            }
            if (!alive) break;
            const int tile = blockIdx.x + it * gridDim.x;
            const int mt = tile / n_tiles, n0 = (tile % n_tiles) * BNT + half * HALF;
            const long long gb = 2ll * mt + (r >> 6);
            const int img = int(gb / blocks_per_img);
            const int rb = int(gb % blocks_per_img);
            const int jy = (rb / p.blocks_x) * p.bh + (r & 63) / p.bw;
            const int jx = (rb % p.blocks_x) * p.bw + (r & 63) % p.bw;
            if (img < p.n_img && jy < p.grid_h && jx < p.grid_w) {
                const int oy = p.out_sy * jy + p.out_oy, ox = p.out_sx * jx + p.out_ox;
                float *dst_px = p.out + size_t(img) * p.out_c * plane + size_t(oy) * p.out_w + ox;
#pragma unroll
                for (int i = 0; i < HALF; ++i) {
                    const int ch = n0 + i;
                    if (ch < p.out_c) {
                        float *dst = dst_px + size_t(ch) * plane;
                        *dst = p.accumulate ? *dst + run[i] : run[i];
                    }
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 9) tmem_dealloc(tmem_base, 2 * BNT);
}

// ---- dW kernel ------------------------------------------------------------------------
// One block: output tile [128 oc x 128 c] of one tap, over a range of 32-pixel groups
// (4 rows x 8 pixels of one image).  A = G staged [pixel][oc], B = X staged
// [pixel][c]; both MN-major (32-byte-atom swizzle).  Every DRAIN k-blocks the four
// accumulators are folded into f32 registers so no accumulation chain exceeds 512 terms.
struct DwParams {
    float *partial;             // [splits][taps][K][C]
    int n_img, k, c, taps;
    int groups_x, groups_y;     // 8 x 4 pixel groups over the output plane
    int groups_per_split;
    int stride;
    int three_pass;
    int grouped;                // 1: the maps are 5-D (channel groups as a dimension), one load per operand tile
    // Single-pass TF32 on layers of at most 128 input channels: a block's 256 accumulator columns hold
    // taps_per_block filter taps side by side (cpad = 256 / taps_per_block columns each), all fed by the same g
    // tile, so that tile is fetched and read once per 2 or 4 taps instead of once per tap.
    int taps_per_block, cpad;
    int *status;
    short off_y[MAX_TAPS], off_x[MAX_TAPS];
};

constexpr int DRAIN = NACC * 16;

// 192 threads: warps 0-3 fold the accumulators (one TMEM lane quarter each), warp 4 feeds TMA,
// warp 5 issues the MMAs.  The roles never share a thread, so the drain hand-shake cannot
// wait on itself.
// SINGLE = single-pass TF32: no lo tiles, so a stage is g | x only and the ring is two to three times as deep
// in the same shared memory; tiles are 256 input channels wide where the layer has them; and the whole
// pixel range of a block accumulates in tensor memory without drains (the 2e-3 bar of that mode leaves room
// for the tensor core's accumulation loss over ~40 000 terms), so no running sums are kept in registers.
template <int BNT, bool SINGLE>
struct DwCfg {
    static constexpr int NACC_D = BNT == 256 ? 2 : NACC;
    static constexpr int B_OFF = SINGLE ? TILE_BYTES : 2 * TILE_BYTES;
    static constexpr int STAGE_BYTES = SINGLE ? TILE_BYTES + BNT * BK * 4 : 4 * TILE_BYTES;
    static constexpr int FIT = (200 * 1024) / STAGE_BYTES;
    static constexpr int STAGES_D = SINGLE ? (FIT > 8 ? 8 : FIT) : STAGES;
    static constexpr size_t SMEM = size_t(STAGES_D) * STAGE_BYTES + 1024;
    static_assert(SINGLE || BNT <= 128, "256-wide tiles are for the single-pass form");
};

template <int BNT, bool SINGLE>
__global__ void __launch_bounds__(192, 1)
conv_dw_igemm_kernel(const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_g_lo,
                     const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_x_lo,
                     const __grid_constant__ DwParams p) {
    using Cfg = DwCfg<BNT, SINGLE>;
    constexpr int NACC_D = Cfg::NACC_D, STAGES_D = Cfg::STAGES_D, PARTS = SINGLE ? 1 : 2;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full[STAGES_D], empty[STAGES_D], drained, batch_done;
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tpb = (SINGLE && BNT == 256) ? p.taps_per_block : 1;   // > 1: one channel tile, several taps
    const int ctiles = tpb > 1 ? 1 : (p.c + BNT - 1) / BNT;
    const int c0 = (blockIdx.x % ctiles) * BNT, k0 = (blockIdx.x / ctiles) * BM;
    const int tap = blockIdx.y * tpb;
    const int taps_here = (p.taps - tap) < tpb ? (p.taps - tap) : tpb;
    const int groups_per_img = p.groups_x * p.groups_y;
    const long long total_groups = (long long)p.n_img * groups_per_img;
    const long long g_begin = (long long)blockIdx.z * p.groups_per_split;
    long long g_end = g_begin + p.groups_per_split;
    if (g_end > total_groups) g_end = total_groups;
    const int kblocks = g_end > g_begin ? int(g_end - g_begin) : 0;
    constexpr uint32_t stage_bytes = Cfg::STAGE_BYTES;
    const int drain_every = SINGLE ? (kblocks > 0 ? kblocks : 1) : DRAIN;  // single pass: one batch, no drains
    const int batches = (kblocks + drain_every - 1) / drain_every;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES_D; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(&drained, 128);
        mbar_init(&batch_done, 1);
        mbar_init_fence();
    }
    if (warp == 4) {
        tmem_alloc(&tmem_slot, NACC_D * BNT);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;

    if (warp == 4 && lane == 0) {
        for (int i = 0; i < kblocks; ++i) {
            const int s = i % STAGES_D;
            if (i >= STAGES_D && !mbar_wait(&empty[s], ((i / STAGES_D) - 1) & 1, p.status, 31)) break;
            mbar_arrive_expect_tx(&full[s], tpb > 1 ? TILE_BYTES + taps_here * p.cpad * BK * 4 : PARTS * (TILE_BYTES + BNT * BK * 4));
            unsigned char *st = smem + s * stage_bytes;
            const long long gidx = g_begin + i;
            const int img = int(gidx / groups_per_img);
            const int r = int(gidx % groups_per_img);
            const int oy0 = (r / p.groups_x) * 4, ox0 = (r % p.groups_x) * 8;
            for (int part = 0; part < PARTS; ++part) {
                const CUtensorMap *mg = part ? &map_g_lo : &map_g;
                const CUtensorMap *mx = part ? &map_x_lo : &map_x;
                if (tpb > 1) {
                    // (only reached with grouped maps and one part) the g tile once, one x tile per tap
                    tma_load_5d(st, mg, &full[s], 0, ox0, oy0, k0 / 32, img);
                    for (int tt = 0; tt < taps_here; ++tt)
                        tma_load_5d(st + Cfg::B_OFF + tt * p.cpad * BK * 4, mx, &full[s], 0,
                                    ox0 * p.stride + p.off_x[tap + tt], oy0 * p.stride + p.off_y[tap + tt], 0, img);
                    continue;
                }
                if (p.grouped) {
                    // one instruction per operand tile: the TMA unit's per-instruction cost, not its
                    // bandwidth, bounds a stage made of twelve 4 KiB boxes
                    tma_load_5d(st + part * TILE_BYTES, mg, &full[s], 0, ox0, oy0, k0 / 32, img);
                    tma_load_5d(st + Cfg::B_OFF + part * TILE_BYTES, mx, &full[s], 0, ox0 * p.stride + p.off_x[tap],
                                oy0 * p.stride + p.off_y[tap], c0 / 32, img);
                    continue;
                }
                for (int j = 0; j < BM / 32; ++j)
                    tma_load_4d(st + part * TILE_BYTES + j * 4096, mg, &full[s], k0 + 32 * j, ox0, oy0, img);
                for (int j = 0; j < BNT / 32; ++j)
                    tma_load_4d(st + Cfg::B_OFF + part * TILE_BYTES + j * 4096, mx, &full[s], c0 + 32 * j,
                                ox0 * p.stride + p.off_x[tap], oy0 * p.stride + p.off_y[tap], img);
            }
        }
    } else if (warp == 5) {
        // MMA issue: whole warp in the loop, the elect.sync thread issues
        const bool issue = elect_one();
        const uint32_t idesc = idesc_tf32(BM, BNT, true, true);
        bool ok = true;
        for (int b = 0; b < batches && ok; ++b) {
            // the previous batch's accumulators must have been read out by all 128 threads
            if (b > 0 && !mbar_wait_warp(&drained, (b - 1) & 1, p.status, 33)) break;
            tc_fence_after_sync();
            const int i_end = (b + 1) * drain_every < kblocks ? (b + 1) * drain_every : kblocks;
            for (int i = b * drain_every; i < i_end; ++i) {
                const int s = i % STAGES_D;
                if (!mbar_wait_warp_ready(&full[s], (i / STAGES_D) & 1, p.status, 32)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t st = smem_u32(smem + s * stage_bytes);
                const int li = i - b * drain_every;
                const uint32_t acc = tmem_base + uint32_t(li % NACC_D) * BNT;
                const bool first = li < NACC_D;
                if (issue) {
#pragma unroll
                    for (int j = 0; j < BK / 8; ++j) {
                        const uint64_t a_hi = smem_desc(st + j * 1024, 4096, 512, kLayoutSw128Base32);
                        const uint64_t b_hi = smem_desc(st + Cfg::B_OFF + j * 1024, 4096, 512, kLayoutSw128Base32);
                        if (!SINGLE) {
                            const uint64_t a_lo = smem_desc(st + TILE_BYTES + j * 1024, 4096, 512, kLayoutSw128Base32);
                            const uint64_t b_lo = smem_desc(st + 3 * TILE_BYTES + j * 1024, 4096, 512, kLayoutSw128Base32);
                            mma_tf32(acc, a_lo, b_hi, idesc, !(first && j == 0));
                            mma_tf32(acc, a_hi, b_lo, idesc, true);
                            mma_tf32(acc, a_hi, b_hi, idesc, true);
                        } else {
                            mma_tf32(acc, a_hi, b_hi, idesc, !(first && j == 0));
                        }
                    }
                    mma_commit(&empty[s]);
                }
                __syncwarp();
            }
            if (ok && issue) mma_commit(&batch_done);
            __syncwarp();
        }
    }
    __syncwarp();

    if constexpr (SINGLE) {
      if (warp < 4) {
        // single pass: one batch; the accumulators are added 32 columns at a time and go straight out
        const int oc = k0 + warp * 32 + lane;
        const bool alive = kblocks == 0 || mbar_wait(&batch_done, 0, p.status, 34);
        tc_fence_after_sync();
        const int used_acc = kblocks < NACC_D ? kblocks : NACC_D;
        for (int q = 0; q < BNT / 32; ++q) {
            // columns q * 32 .. + 31: of tap `tap + tt`, channels ch0 .. (one tap and c0 + q * 32 without tap packing)
            const int tt = tpb > 1 ? (q * 32) / p.cpad : 0;
            const int ch0 = tpb > 1 ? (q * 32) % p.cpad : c0 + q * 32;
            if (tt >= taps_here) break;
            float *dst = p.partial + ((size_t(blockIdx.z) * p.taps + tap + tt) * p.k + (oc < p.k ? oc : 0)) * p.c;
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0.f;
            for (int a = 0; a < used_acc && alive; ++a) {
                float t[32];
                tmem_ld_32x32(tmem_base + (uint32_t(warp * 32) << 16) + a * BNT + q * 32, t);
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] += t[i];
            }
            if (oc < p.k) {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (ch0 + i < p.c) dst[ch0 + i] = v[i];
            }
        }
      }
    } else if (warp < 4) {
    // running sums of this thread's output row (oc = k0 + 32*warp + lane), BNT columns
    float run[BNT];
#pragma unroll
    for (int i = 0; i < BNT; ++i) run[i] = 0.f;
    bool alive = true;
    for (int b = 0; b < batches && alive; ++b) {
        alive = mbar_wait(&batch_done, b & 1, p.status, 34);
        tc_fence_after_sync();
        if (alive) {
            const int in_batch = (kblocks - b * DRAIN) < DRAIN ? (kblocks - b * DRAIN) : DRAIN;
            const int used_acc = in_batch < NACC ? in_batch : NACC;
#pragma unroll
            for (int q = 0; q < BNT / 32; ++q) {
                for (int a = 0; a < used_acc; ++a) {
                    float t[32];
                    tmem_ld_32x32(tmem_base + (uint32_t(warp * 32) << 16) + a * BNT + q * 32, t);
#pragma unroll
                    for (int i = 0; i < 32; ++i) run[q * 32 + i] += t[i];
                }
            }
        }
        tc_fence_before_sync();
        mbar_arrive(&drained);
    }
    {
        const int oc = k0 + warp * 32 + lane;
        if (oc < p.k) {
            float *dst = p.partial + ((size_t(blockIdx.z) * p.taps + tap) * p.k + oc) * p.c;
#pragma unroll
            for (int i = 0; i < BNT; ++i)
                if (c0 + i < p.c) dst[c0 + i] = alive ? run[i] : 0.f;
        }
    }
    }  // epilogue warps
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 4) tmem_dealloc(tmem_base, NACC_D * BNT);
}

// ---- dW for narrow layers (C <= 32): all taps in one block ---------------------------------
// The kernel above gives every tap its own blocks, so the g tile (the larger operand when C is
// small) is fetched and read by the MMAs once per tap.  Here one block holds g once per 32-pixel
// k-block and the x tiles of ALL taps side by side along N (tap t occupies accumulator columns
// 32 t .. 32 t + 31), so one MMA per k-step covers up to eight taps.  The accumulators (taps x 32
// columns) leave no room for a second set, so a block works in chunks of CHUNK k-blocks (512
// pixels, the longest accumulation chain): after a chunk the four epilogue warps write the
// accumulators as that chunk's partial dW and the fold kernel adds the chunks in order.
constexpr int TAPS_MAX = 16;   // taps x 32 accumulator columns <= 512
constexpr int CHUNK = 16;      // k-blocks per chunk
constexpr int TAPS_STAGES = 2;

struct DwTapsParams {
    float *partial;             // [chunks][taps][K][C]
    int n_img, k, c, taps;
    int groups_x, groups_y;     // 8 x 4 pixel groups over the output plane
    long long total_groups;
    int chunks;
    int stride;
    int three_pass;
    int a_groups;               // 32-channel groups of g that exist (ceil(k / 32))
    int grouped;                // 1: the g maps are 5-D (channel groups as a dimension): one load for the g tile
    int *status;
    short off_y[TAPS_MAX], off_x[TAPS_MAX];
};

__global__ void __launch_bounds__(192, 1)
conv_dw_taps_kernel(const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_g_lo,
                    const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_x_lo,
                    const __grid_constant__ DwTapsParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full[TAPS_STAGES], empty[TAPS_STAGES], acc_full, acc_empty;
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int groups_per_img = p.groups_x * p.groups_y;
    const int parts = p.three_pass ? 2 : 1;
    // stage: g hi | g lo (4 groups x 4 KiB each) | x hi per tap | x lo per tap
    const uint32_t a_bytes = TILE_BYTES, b_bytes = uint32_t(p.taps) * 4096;
    const uint32_t stage_bytes = 2 * a_bytes + 2 * b_bytes;
    const int my_chunks = (p.chunks - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    uint32_t tmem_cols = 32;
    while ((int)tmem_cols < p.taps * 32) tmem_cols <<= 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TAPS_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(&acc_full, 1);
        mbar_init(&acc_empty, 128);
        mbar_init_fence();
    }
    if (warp == 5) {
        tmem_alloc(&tmem_slot, tmem_cols);
        tmem_relinquish();
    }
    // g groups beyond the layer's channels are never loaded: they must hold finite values
    for (uint32_t i = threadIdx.x; i < TAPS_STAGES * stage_bytes / 16; i += blockDim.x)
        st_shared_v4(smem + i * 16, make_float4(0.f, 0.f, 0.f, 0.f));
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;

    auto chunk_kblocks = [&](int chunk) {
        const long long first = (long long)chunk * CHUNK;
        const long long left = p.total_groups - first;
        return int(left < CHUNK ? left : CHUNK);
    };

    if (warp == 4 && lane == 0) {
        // ---- TMA producer ----
        int g = 0;
        bool ok = true;
        for (int it = 0; it < my_chunks && ok; ++it) {
            const int chunk = blockIdx.x + it * gridDim.x, nkb = chunk_kblocks(chunk);
            for (int i = 0; i < nkb; ++i, ++g) {
                const int s = g % TAPS_STAGES;
                if (g >= TAPS_STAGES && !mbar_wait(&empty[s], ((g / TAPS_STAGES) - 1) & 1, p.status, 35)) { ok = false; break; }
                mbar_arrive_expect_tx(&full[s], parts * (p.a_groups * 4096 + p.taps * 4096));
                unsigned char *st = smem + s * stage_bytes;
                const long long gidx = (long long)chunk * CHUNK + i;
                const int img = int(gidx / groups_per_img);
                const int r = int(gidx % groups_per_img);
                const int oy0 = (r / p.groups_x) * 4, ox0 = (r % p.groups_x) * 8;
                for (int part = 0; part < parts; ++part) {
                    const CUtensorMap *mg = part ? &map_g_lo : &map_g;
                    const CUtensorMap *mx = part ? &map_x_lo : &map_x;
                    if (p.grouped) {
                        tma_load_5d(st + part * a_bytes, mg, &full[s], 0, ox0, oy0, 0, img);
                    } else {
                        for (int j = 0; j < p.a_groups; ++j)
                            tma_load_4d(st + part * a_bytes + j * 4096, mg, &full[s], 32 * j, ox0, oy0, img);
                    }
                    for (int t = 0; t < p.taps; ++t)
                        tma_load_4d(st + 2 * a_bytes + part * b_bytes + t * 4096, mx, &full[s], 0,
                                    ox0 * p.stride + p.off_x[t], oy0 * p.stride + p.off_y[t], img);
                }
            }
        }
    } else if (warp == 5) {
        // ---- MMA issue: one MMA per k-step and pass covers up to eight taps (N = 256) ----
        const bool issue = elect_one();
        int g = 0;
        bool ok = true;
        for (int it = 0; it < my_chunks && ok; ++it) {
            const int chunk = blockIdx.x + it * gridDim.x, nkb = chunk_kblocks(chunk);
            if (it >= 1 && !mbar_wait_warp(&acc_empty, (it - 1) & 1, p.status, 36)) break;
            tc_fence_after_sync();
            for (int i = 0; i < nkb; ++i, ++g) {
                const int s = g % TAPS_STAGES;
                if (!mbar_wait_warp_ready(&full[s], (g / TAPS_STAGES) & 1, p.status, 37)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t st = smem_u32(smem + s * stage_bytes);
                if (issue) {
                    for (int t0 = 0; t0 < p.taps; t0 += 8) {
                        const int nt = (p.taps - t0) < 8 ? (p.taps - t0) : 8;
                        const uint32_t idesc = idesc_tf32(BM, nt * 32, true, true);
                        const uint32_t acc = tmem_base + uint32_t(t0) * 32;
#pragma unroll
                        for (int j = 0; j < BK / 8; ++j) {
                            const uint64_t a_hi = smem_desc(st + j * 1024, 4096, 512, kLayoutSw128Base32);
                            const uint64_t b_hi = smem_desc(st + 2 * a_bytes + t0 * 4096 + j * 1024, 4096, 512, kLayoutSw128Base32);
                            const bool acc_flag = !(i == 0 && j == 0);
                            if (p.three_pass) {
                                const uint64_t a_lo = smem_desc(st + a_bytes + j * 1024, 4096, 512, kLayoutSw128Base32);
                                const uint64_t b_lo = smem_desc(st + 2 * a_bytes + b_bytes + t0 * 4096 + j * 1024, 4096, 512, kLayoutSw128Base32);
                                mma_tf32(acc, a_lo, b_hi, idesc, acc_flag);
                                mma_tf32(acc, a_hi, b_lo, idesc, true);
                                mma_tf32(acc, a_hi, b_hi, idesc, true);
                            } else {
                                mma_tf32(acc, a_hi, b_hi, idesc, acc_flag);
                            }
                        }
                    }
                    mma_commit(&empty[s]);
                    if (i == nkb - 1) mma_commit(&acc_full);
                }
                __syncwarp();
            }
        }
    } else if (warp < 4) {
        // ---- epilogue: this chunk's accumulators become its partial dW (thread = oc) ----
        const int oc = warp * 32 + lane;
        for (int it = 0; it < my_chunks; ++it) {
            const int chunk = blockIdx.x + it * gridDim.x;
            if (!mbar_wait_warp(&acc_full, it & 1, p.status, 38)) break;
            tc_fence_after_sync();
            for (int t = 0; t < p.taps; ++t) {
                float v[32];
                tmem_ld_32x32(tmem_base + (uint32_t(warp * 32) << 16) + uint32_t(t) * 32, v);
                if (t == p.taps - 1) {
                    tc_fence_before_sync();
                    mbar_arrive(&acc_empty);
                }
                if (oc < p.k) {
                    float *dst = p.partial + ((size_t(chunk) * p.taps + t) * p.k + oc) * p.c;
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        if (i < p.c) *reinterpret_cast<float4 *>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 5) tmem_dealloc(tmem_base, tmem_cols);
}

// dw[k][c][tap] (+)= sum over splits of partial[split][tap][k][c].  A block handles 32 elements:
// eight thread groups each add every eighth partial, then one group adds the eight sums -- a fixed
// order (bit-reproducible) with eight times the loads in flight of a flat loop, which matters when
// the all-taps kernel leaves a thousand chunks to fold.
__global__ void __launch_bounds__(256)
dw_fold_kernel(const float *__restrict__ partial, float *dw, int k, int c, int taps, int splits, int accumulate) {
    __shared__ float sums[8][32];
    const size_t elems = size_t(k) * c * taps;
    // walk the partials in their own order ([tap][k][c], contiguous loads); dw is [k][c][tap]
    const size_t j = size_t(blockIdx.x) * 32 + (threadIdx.x & 31);
    const int part = threadIdx.x >> 5;
    float s = 0.f;
    if (j < elems)
        for (int q = part; q < splits; q += 8) s += partial[size_t(q) * elems + j];
    sums[part][threadIdx.x & 31] = s;
    __syncthreads();
    if (part == 0 && j < elems) {
        float total = sums[0][threadIdx.x];
#pragma unroll
        for (int q = 1; q < 8; ++q) total += sums[q][threadIdx.x];
        const size_t kc = size_t(k) * c;
        const size_t i = (j % kc) * taps + j / kc;
        dw[i] = accumulate ? dw[i] + total : total;
    }
}

// ---- host side --------------------------------------------------------------------------
struct Scratch {
    float *base;
    size_t cursor;
    float *take(size_t n) {
        float *ptr = base + cursor;
        cursor += (n + 63) / 64 * 64;  // keeps every array 256-byte aligned
        return ptr;
    }
};

size_t padded(size_t n) { return (n + 63) / 64 * 64; }

// [N][H][W][C] staging array as a 4-D tensor map, box {32 channels, bw, bh, 1}; step > 1 walks every step-th pixel.
bool nhwc_map(CUtensorMap *map, const float *base, size_t n, size_t h, size_t w, size_t c, int bw, int bh, int step,
              CUtensorMapSwizzle swizzle, int box_c = 32) {
    katsu_tensor_map_encode_fn encode = katsu_tensor_map_encoder();
    if (encode == nullptr) return false;
    cuuint64_t dims[4] = {c, w, h, n};
    cuuint64_t strides[3] = {c * sizeof(float), w * c * sizeof(float), h * w * c * sizeof(float)};
    cuuint32_t box[4] = {cuuint32_t(box_c), cuuint32_t((bw - 1) * step + 1), cuuint32_t((bh - 1) * step + 1), 1};
    cuuint32_t estr[4] = {1, cuuint32_t(step), cuuint32_t(step), 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The same array with its channel groups as a dimension of their own: 5-D {32 channels, W, H, C/32, N},
// box {32, bw, bh, groups, 1}, so that one load brings `groups` 32-channel slabs, 4 KiB apart in shared
// memory as the MN-major operand layout wants them.  C must be a multiple of 32.
bool nhwc_grouped_map(CUtensorMap *map, const float *base, size_t n, size_t h, size_t w, size_t c, int bw, int bh,
                      int step, int groups, CUtensorMapSwizzle swizzle) {
    katsu_tensor_map_encode_fn encode = katsu_tensor_map_encoder();
    if (encode == nullptr || (c & 31)) return false;
    cuuint64_t dims[5] = {32, w, h, c / 32, n};
    cuuint64_t strides[4] = {c * sizeof(float), w * c * sizeof(float), 32 * sizeof(float), h * w * c * sizeof(float)};
    cuuint32_t box[5] = {32, cuuint32_t((bw - 1) * step + 1), cuuint32_t((bh - 1) * step + 1), cuuint32_t(groups), 1};
    cuuint32_t estr[5] = {1, cuuint32_t(step), cuuint32_t(step), 1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<float *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// [taps][rows][inner] weight staging array, box {32, box_rows, 1, 1} (4-D with a unit last dimension).
bool taps_map(CUtensorMap *map, const float *base, size_t taps, size_t rows, size_t inner, int box_rows,
              int box_inner = 32, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
    katsu_tensor_map_encode_fn encode = katsu_tensor_map_encoder();
    if (encode == nullptr) return false;
    cuuint64_t dims[4] = {inner, rows, taps, 1};
    cuuint64_t strides[3] = {inner * sizeof(float), rows * inner * sizeof(float), taps * rows * inner * sizeof(float)};
    cuuint32_t box[4] = {cuuint32_t(box_inner), cuuint32_t(box_rows), 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int32_t stage_nhwc(katsu_cuda_ctx *ctx, const float *src, float *dst, float *dst_lo, size_t n, size_t c, size_t hw) {
    dim3 grid((unsigned)katsu_div_up(hw, (size_t)32 * NHWC_TILES), (unsigned)katsu_div_up(c, 32), (unsigned)n);
    KATSU_LAUNCH(ctx, nchw_to_nhwc_kernel, grid, 256, 0, src, dst, dst_lo, (int)c, (int)hw);
    return KATSU_OK;
}

void pick_block(size_t width, int *bw, int *bh) {
    *bw = (width % 32 == 0) ? 32 : (width % 16 == 0) ? 16 : 8;
    *bh = 64 / *bw;
}

constexpr size_t kSmemBytes = size_t(STAGES) * 4 * TILE_BYTES + 1024;  // dW kernel

struct Shape {
    size_t n, c, h, w, k, r, s, stride, pad, oh, ow;
};

bool igemm_shape(const katsu_cuda_ctx *ctx, const Shape &g) {
    if (ctx->precision == KATSU_MODE_FP32) return false;
    if (g.c < 16 || g.k < 16 || (g.c & 3) || (g.k & 3)) return false;  // TMA needs 16-byte channel rows
    if (g.r * g.s > (size_t)MAX_TAPS || g.stride > 8 || g.pad > 1024) return false;
    if (g.n > 65535 || g.h > 32768 || g.w > 32768) return false;
    // too little work for 128x128 tiles: leave it to the direct kernels
    if (g.n * g.oh * g.ow < 64) return false;
    return katsu_tensor_map_encoder() != nullptr;
}

// Split of the dW contraction over pixel groups and the scratch it needs.
struct DwPlan {
    size_t bnt, splits, groups_per_split, partial_floats, scratch_floats;
    size_t taps_per_block;  // > 1: single-pass TF32 with several taps side by side in a 256-column tile
    bool all_taps;  // narrow layer: conv_dw_taps_kernel, `splits` counts its chunks
};

DwPlan dw_plan(const katsu_cuda_ctx *ctx, const Shape &g) {
    DwPlan plan;
    const size_t taps = g.r * g.s;
    const size_t total_groups = g.n * katsu_div_up(g.ow, 8) * katsu_div_up(g.oh, 4);
    // channel-tile width of the c side: narrow layers get narrow MMAs and operand tiles
    const bool three = ctx->precision == KATSU_MODE_3XTF32;
    plan.bnt = g.c <= 32 ? 32 : g.c <= 64 ? 64 : (!three && g.c >= 256 && g.c % 32 == 0 && g.k % 32 == 0) ? 256 : 128;
    plan.taps_per_block = 1;
    if (!three && g.c > 32 && g.c <= 128 && g.c % 32 == 0 && g.k % 32 == 0 && taps > 1) {
        plan.taps_per_block = g.c <= 64 ? 4 : 2;
        plan.bnt = 256;
    }
    // two stages of (g hi/lo 32 KiB + x hi/lo 8 KiB per tap) must fit in shared memory: taps <= 10
    plan.all_taps = g.c <= 32 && g.k <= (size_t)BM && taps <= 10 && total_groups <= 0x7fffffffu;
    if (plan.all_taps) {
        plan.splits = katsu_div_up(total_groups, (size_t)CHUNK);
        plan.groups_per_split = CHUNK;
        plan.partial_floats = plan.splits * taps * g.k * g.c;
        plan.scratch_floats = (padded(g.n * g.c * g.h * g.w) + padded(g.n * g.k * g.oh * g.ow)) * (three ? 2 : 1) + padded(plan.partial_floats);
        return plan;
    }
    const size_t out_tiles = plan.taps_per_block > 1
                                 ? katsu_div_up(g.k, (size_t)BM) * katsu_div_up(taps, plan.taps_per_block)
                                 : katsu_div_up(g.k, (size_t)BM) * katsu_div_up(g.c, plan.bnt) * taps;
    // Split the pixel range so that the grid fills whole waves of the GPU: the smallest split
    // count (at least two blocks' worth of work per SM) whose last wave is >= 95 % full.
    size_t splits = katsu_div_up(size_t(ctx->num_sms) * 2, out_tiles);
    for (size_t cand = splits; cand < splits + size_t(ctx->num_sms); ++cand) {
        const size_t blocks = out_tiles * cand, waves = katsu_div_up(blocks, (size_t)ctx->num_sms);
        if (blocks * 100 >= waves * ctx->num_sms * 95) { splits = cand; break; }
    }
    // single-pass TF32 keeps a block's whole pixel range in tensor memory: at most 2048 k-blocks (65 536 pixels,
    // ~4 000 accumulation steps per accumulator, ~1e-4 of accumulation loss against the 2e-3 bar of that mode)
    if (!three && splits < katsu_div_up(total_groups, (size_t)2048)) splits = katsu_div_up(total_groups, (size_t)2048);
    if (splits > total_groups) splits = total_groups;
    if (splits < 1) splits = 1;
    plan.groups_per_split = katsu_div_up(total_groups, splits);
    plan.splits = katsu_div_up(total_groups, plan.groups_per_split);
    plan.partial_floats = plan.splits * taps * g.k * g.c;
    plan.scratch_floats = (padded(g.n * g.c * g.h * g.w) + padded(g.n * g.k * g.oh * g.ow)) * (three ? 2 : 1) + padded(plan.partial_floats);
    return plan;
}

// Forward / dX launch: picks the channel-tile width, builds the B maps for it and starts one
// persistent block per SM (or per tile, if there are fewer).
template <int BNT, bool SINGLE>
int32_t launch_igemm_bn(katsu_cuda_ctx *ctx, const CUtensorMap &ma, const CUtensorMap &ma_lo, const float *b_hi,
                        const float *b_lo, size_t taps, size_t rows, size_t inner, const IgemmParams &p,
                        size_t total_blocks) {
    CUtensorMap mb, mb_lo;
    if (!taps_map(&mb, b_hi, taps, rows, inner, BNT) || !taps_map(&mb_lo, b_lo, taps, rows, inner, BNT))
        return katsu_set_error(KATSU_ERR_CUDA, "cuTensorMapEncodeTiled failed (conv weights)");
    auto kernel = p.merge_x ? conv_igemm_kernel<BNT, SINGLE, (BNT <= 128)> : conv_igemm_kernel<BNT, SINGLE, false>;
    if (p.merge_x && BNT > 128) return katsu_set_error(KATSU_ERR_UNSUPPORTED, "merged dX classes need tiles of at most 128 channels");
    KATSU_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)IgemmCfg<BNT, SINGLE>::SMEM));
    const size_t m_tiles = katsu_div_up(total_blocks, 2), n_tiles = katsu_div_up(rows, (size_t)BNT);
    if (m_tiles * n_tiles > 0x7fffffffu / 64) return katsu_set_error(KATSU_ERR_UNSUPPORTED, "convolution too large for the tile counter");
    size_t grid = m_tiles * n_tiles;
    if (grid > (size_t)ctx->num_sms) grid = (size_t)ctx->num_sms;
    KATSU_LAUNCH(ctx, kernel, (unsigned)grid, 192, (IgemmCfg<BNT, SINGLE>::SMEM), ma, ma_lo, mb, mb_lo, p, (int)m_tiles, (int)n_tiles);
    return KATSU_OK;
}

// 256-wide tiles do a third more work per unit of shared-memory traffic; they pay unless padding the
// channel count to a multiple of 256 adds more than a fifth over padding it to a multiple of 128.
bool wide_tiles_pay(size_t rows) {
    return rows >= 256 && katsu_div_up(rows, (size_t)256) * 256 * 10 <= katsu_div_up(rows, (size_t)128) * 128 * 12;
}

// The staged activation operand of a forward / dX launch, for kernels that build their own maps of it.
struct Activation {
    const float *hi, *lo;
    size_t n, h, w, c;
    int step;
};

// The tensor core's f32 accumulation loses about 3e-8 (relative) per accumulation step, and conv_igemm_kernel in
// 3xTF32 makes 12 steps per 32-channel k-block into one of its 2 (128-wide tiles) or 4 (64- and 32-wide tiles)
// rotating accumulators: 72 k-blocks (a 3x3 layer over 256 channels) measured 8.4e-6 against the 1e-5 bar with
// two accumulators, 180 k-blocks 1.9e-5.  Beyond 300 steps per accumulator the layer goes to the kernel that
// folds its accumulators into registers every 192 steps.
bool drained_kernel_needed(size_t rows, const IgemmParams &p) {
    const size_t kblocks = size_t(p.ntaps) * katsu_div_up((size_t)p.kc, (size_t)BK);
    const size_t accumulators = rows <= 64 ? 4 : 2;
    return katsu_div_up(kblocks, accumulators) * 12 > 300;
}

int32_t launch_igemm(katsu_cuda_ctx *ctx, const CUtensorMap &ma, const CUtensorMap &ma_lo, const float *b_hi,
                     const float *b_lo, size_t taps, size_t rows, size_t inner, const IgemmParams &p, size_t total_blocks,
                     const Activation &act) {
    if (!p.three_pass) {
        if (rows <= 32) return launch_igemm_bn<32, true>(ctx, ma, ma_lo, b_hi, b_lo, taps, rows, inner, p, total_blocks);
        if (rows <= 64) return launch_igemm_bn<64, true>(ctx, ma, ma_lo, b_hi, b_lo, taps, rows, inner, p, total_blocks);
        if (!wide_tiles_pay(rows)) return launch_igemm_bn<128, true>(ctx, ma, ma_lo, b_hi, b_lo, taps, rows, inner, p, total_blocks);
        return launch_igemm_bn<256, true>(ctx, ma, ma_lo, b_hi, b_lo, taps, rows, inner, p, total_blocks);
    }
    if (rows <= 32) return launch_igemm_bn<32, false>(ctx, ma, ma_lo, b_hi, b_lo, taps, rows, inner, p, total_blocks);
    if (rows <= 64) return launch_igemm_bn<64, false>(ctx, ma, ma_lo, b_hi, b_lo, taps, rows, inner, p, total_blocks);
    const bool wide = wide_tiles_pay(rows);
    if (!p.merge_x && (wide || drained_kernel_needed(rows, p))) {
        const int bnt = wide ? 256 : 128;
        CUtensorMap mb, mb_lo, wa, wa_lo;
        const CUtensorMapSwizzle sw64 = CU_TENSOR_MAP_SWIZZLE_64B;
        if (!taps_map(&mb, b_hi, taps, rows, inner, bnt, BK3, sw64) || !taps_map(&mb_lo, b_lo, taps, rows, inner, bnt, BK3, sw64) ||
            !nhwc_map(&wa, act.hi, act.n, act.h, act.w, act.c, p.bw, p.bh, act.step, sw64, BK3) ||
            !nhwc_map(&wa_lo, act.lo, act.n, act.h, act.w, act.c, p.bw, p.bh, act.step, sw64, BK3))
            return katsu_set_error(KATSU_ERR_CUDA, "cuTensorMapEncodeTiled failed (wide conv operands)");
        auto kernel = wide ? conv_igemm_wide3_kernel<256> : conv_igemm_wide3_kernel<128>;
        const size_t smem = wide ? Wide3Cfg<256>::SMEM : Wide3Cfg<128>::SMEM;
        KATSU_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        const size_t m_tiles = katsu_div_up(total_blocks, 2), n_tiles = katsu_div_up(rows, (size_t)bnt);
        if (m_tiles * n_tiles > 0x7fffffffu / 64) return katsu_set_error(KATSU_ERR_UNSUPPORTED, "convolution too large for the tile counter");
        size_t grid = m_tiles * n_tiles;
        if (grid > (size_t)ctx->num_sms) grid = (size_t)ctx->num_sms;
        KATSU_LAUNCH(ctx, kernel, (unsigned)grid, 320, smem, wa, wa_lo, mb, mb_lo, p, (int)m_tiles, (int)n_tiles);
        return KATSU_OK;
    }
    return launch_igemm_bn<128, false>(ctx, ma, ma_lo, b_hi, b_lo, taps, rows, inner, p, total_blocks);
}

}  // namespace

size_t katsu_conv_igemm_staged_floats(const katsu_cuda_ctx *ctx, size_t n, size_t c, size_t h, size_t wd, size_t k,
                                      size_t r, size_t s, size_t stride, size_t pad, size_t oh, size_t ow) {
    const Shape g = {n, c, h, wd, k, r, s, stride, pad, oh, ow};
    if (!igemm_shape(ctx, g)) return 0;
    return padded(n * c * h * wd) * (ctx->precision == KATSU_MODE_3XTF32 ? 2 : 1);
}

int32_t katsu_conv_igemm_stage(katsu_cuda_ctx *ctx, const float *x, float *staged, size_t n, size_t c, size_t h,
                               size_t wd) {
    const bool three = ctx->precision == KATSU_MODE_3XTF32;
    return stage_nhwc(ctx, x, staged, three ? staged + padded(n * c * h * wd) : nullptr, n, c, h * wd);
}

int32_t katsu_conv_igemm_fwd(katsu_cuda_ctx *ctx, const float *x, const float *w, float *y,
                             size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                             size_t stride, size_t pad, size_t oh, size_t ow, int *handled) {
    *handled = 0;
    const Shape g = {n, c, h, wd, k, r, s, stride, pad, oh, ow};
    if (!igemm_shape(ctx, g)) return KATSU_OK;
    *handled = 1;
    const bool three = ctx->precision == KATSU_MODE_3XTF32;
    const size_t xe = n * c * h * wd, we = k * c * r * s, taps = r * s;
    float *base = nullptr;
    KATSU_TRY(katsu_scratch(ctx, (padded(xe) + padded(we)) * (three ? 2 : 1), &base));
    Scratch sc = {base, 0};
    float *xt = sc.take(xe), *xt_lo = three ? sc.take(xe) : nullptr;
    float *wf = sc.take(we), *wf_lo = three ? sc.take(we) : nullptr;
    if (ctx->x_prestaged != nullptr) {
        xt = const_cast<float *>(ctx->x_prestaged);
        xt_lo = three ? xt + padded(xe) : nullptr;
    } else {
        KATSU_TRY(stage_nhwc(ctx, x, xt, xt_lo, n, c, h * wd));
    }
    KATSU_LAUNCH(ctx, weights_to_taps_kernel, (unsigned)katsu_div_up(we, 256), 256, 0, w, wf, wf_lo, (float *)nullptr,
                 (float *)nullptr, (int)k, (int)c, (int)taps);

    IgemmParams p;
    p.out = y;
    p.n_img = (int)n; p.out_c = (int)k; p.out_h = (int)oh; p.out_w = (int)ow;
    pick_block(ow, &p.bw, &p.bh);
    p.blocks_x = (int)katsu_div_up(ow, (size_t)p.bw);
    p.blocks_y = (int)katsu_div_up(oh, (size_t)p.bh);
    p.grid_h = (int)oh; p.grid_w = (int)ow;
    p.out_sy = 1; p.out_oy = 0; p.out_sx = 1; p.out_ox = 0;
    p.in_step = (int)stride;
    p.kc = (int)c;
    p.ntaps = (int)taps;
    p.accumulate = 0;
    p.three_pass = three ? 1 : 0;
    p.status = ctx->status;
    p.merge_x = 0; p.ntaps2 = 0; p.grid_w2 = 0;
    for (size_t t = 0; t < taps; ++t) {
        p.off_y[t] = (short)((int)(t / s) - (int)pad);
        p.off_x[t] = (short)((int)(t % s) - (int)pad);
        p.b_tap[t] = (short)t;
    }
    CUtensorMap ma, ma_lo;
    bool ok = nhwc_map(&ma, xt, n, h, wd, c, p.bw, p.bh, (int)stride, CU_TENSOR_MAP_SWIZZLE_128B) &&
              nhwc_map(&ma_lo, three ? xt_lo : xt, n, h, wd, c, p.bw, p.bh, (int)stride, CU_TENSOR_MAP_SWIZZLE_128B);
    if (!ok) return katsu_set_error(KATSU_ERR_CUDA, "cuTensorMapEncodeTiled failed (conv forward)");
    const size_t total_blocks = n * p.blocks_x * p.blocks_y;
    const Activation act = {xt, three ? xt_lo : xt, n, h, wd, c, (int)stride};
    return launch_igemm(ctx, ma, ma_lo, wf, three ? wf_lo : wf, taps, k, c, p, total_blocks, act);
}

int32_t katsu_conv_igemm_dx(katsu_cuda_ctx *ctx, const float *w, const float *gr, float *dx,
                            size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                            size_t stride, size_t pad, size_t oh, size_t ow, int accumulate, int *handled) {
    *handled = 0;
    const Shape g = {n, c, h, wd, k, r, s, stride, pad, oh, ow};
    if (!igemm_shape(ctx, g)) return KATSU_OK;
    *handled = 1;
    const bool three = ctx->precision == KATSU_MODE_3XTF32;
    const size_t ge = n * k * oh * ow, we = k * c * r * s, taps = r * s;
    float *base = nullptr;
    size_t need = (padded(ge) + padded(we)) * (three ? 2 : 1);
    // a dW launch of the same backward call follows: size the scratch for it now, so that it is
    // not reallocated in between and the staged g can be shared
    if (ctx->share_g_staging) need = need > dw_plan(ctx, g).scratch_floats ? need : dw_plan(ctx, g).scratch_floats;
    KATSU_TRY(katsu_scratch(ctx, need, &base));
    Scratch sc = {base, 0};
    float *gt = sc.take(ge), *gt_lo = three ? sc.take(ge) : nullptr;
    float *wb = sc.take(we), *wb_lo = three ? sc.take(we) : nullptr;
    KATSU_TRY(stage_nhwc(ctx, gr, gt, gt_lo, n, k, oh * ow));
    if (ctx->share_g_staging) ctx->g_staged = 1;
    KATSU_LAUNCH(ctx, weights_to_taps_kernel, (unsigned)katsu_div_up(we, 256), 256, 0, w, (float *)nullptr,
                 (float *)nullptr, wb, wb_lo, (int)k, (int)c, (int)taps);

    // One launch per parity class (py, px) of input pixels: iy = stride*jy + py receives
    // only taps with (py + pad - ky) divisible by stride, from g row jy + (py + pad - ky)/stride.
    const int st = (int)stride;
    // A class no tap reaches (stride larger than the filter) receives nothing: zero dx once
    // and let every launch add.
    bool some_class_empty = false;
    for (int py = 0; py < st; ++py) {
        bool any = false;
        for (int ky = 0; ky < (int)r; ++ky) any |= (((py + (int)pad - ky) % st) + st) % st == 0;
        some_class_empty |= !any;
    }
    for (int px = 0; px < st; ++px) {
        bool any = false;
        for (int kx = 0; kx < (int)s; ++kx) any |= (((px + (int)pad - kx) % st) + st) % st == 0;
        some_class_empty |= !any;
    }
    if (some_class_empty && !accumulate) {
        KATSU_CUDA_TRY(cudaMemsetAsync(dx, 0, n * c * h * wd * sizeof(float), ctx->stream));
        accumulate = 1;
    }
    // taps of parity class (py, px) into the given tables; returns their number
    auto class_taps = [&](int py, int px, short *oy, short *ox, short *bt) {
        int nt = 0;
        for (int ky = 0; ky < (int)r; ++ky) {
            const int ty = py + (int)pad - ky;
            if (((ty % st) + st) % st != 0) continue;
            for (int kx = 0; kx < (int)s; ++kx) {
                const int tx = px + (int)pad - kx;
                if (((tx % st) + st) % st != 0) continue;
                // floor division (ty, tx may be negative)
                oy[nt] = (short)((ty >= 0) ? ty / st : -((-ty + st - 1) / st));
                ox[nt] = (short)((tx >= 0) ? tx / st : -((-tx + st - 1) / st));
                bt[nt] = (short)(ky * (int)s + kx);
                ++nt;
            }
        }
        return nt;
    };
    // Stride 2, every class reached by some tap, tiles of at most 128 channels: one launch per ROW parity
    // computes both x-parity classes and writes them interleaved (IgemmParams::merge_x).
    // (... unless a class's contraction is long enough to need the drained-accumulator kernel, which the
    // per-class launches below can be routed to)
    bool merged_ok = st == 2 && !some_class_empty && wd >= 2 && !wide_tiles_pay(c);
    if (merged_ok && three) {
        IgemmParams probe;
        probe.kc = (int)k;
        for (int py = 0; py < 2; ++py)
            for (int px = 0; px < 2; ++px) {
                probe.ntaps = class_taps(py, px, probe.off_y, probe.off_x, probe.b_tap);
                merged_ok = merged_ok && !drained_kernel_needed(c, probe);
            }
    }
    if (merged_ok) {
        for (int py = 0; py < 2 && py < (int)h; ++py) {
            IgemmParams p;
            p.out = dx;
            p.n_img = (int)n; p.out_c = (int)c; p.out_h = (int)h; p.out_w = (int)wd;
            p.grid_h = (int)((h - py + 1) / 2);
            p.grid_w = (int)((wd + 1) / 2);
            p.grid_w2 = (int)(wd / 2);
            pick_block((size_t)p.grid_w, &p.bw, &p.bh);
            p.blocks_x = (p.grid_w + p.bw - 1) / p.bw;
            p.blocks_y = (p.grid_h + p.bh - 1) / p.bh;
            p.out_sy = 2; p.out_oy = py; p.out_sx = 2; p.out_ox = 0;
            p.in_step = 1;
            p.kc = (int)k;
            p.accumulate = accumulate;
            p.three_pass = three ? 1 : 0;
            p.status = ctx->status;
            p.merge_x = 1;
            p.ntaps = class_taps(py, 0, p.off_y, p.off_x, p.b_tap);
            p.ntaps2 = class_taps(py, 1, p.off_y2, p.off_x2, p.b_tap2);
            const size_t total_blocks = n * p.blocks_x * p.blocks_y;
            CUtensorMap ma, ma_lo;
            bool ok = nhwc_map(&ma, gt, n, oh, ow, k, p.bw, p.bh, 1, CU_TENSOR_MAP_SWIZZLE_128B) &&
                      nhwc_map(&ma_lo, three ? gt_lo : gt, n, oh, ow, k, p.bw, p.bh, 1, CU_TENSOR_MAP_SWIZZLE_128B);
            if (!ok) return katsu_set_error(KATSU_ERR_CUDA, "cuTensorMapEncodeTiled failed (conv dX)");
            const Activation act = {gt, three ? gt_lo : gt, n, oh, ow, k, 1};
            KATSU_TRY(launch_igemm(ctx, ma, ma_lo, wb, three ? wb_lo : wb, taps, c, k, p, total_blocks, act));
        }
        return KATSU_OK;
    }
    for (int py = 0; py < st && py < (int)h; ++py)
        for (int px = 0; px < st && px < (int)wd; ++px) {
            IgemmParams p;
            p.merge_x = 0; p.ntaps2 = 0; p.grid_w2 = 0;
            p.out = dx;
            p.n_img = (int)n; p.out_c = (int)c; p.out_h = (int)h; p.out_w = (int)wd;
            p.grid_h = (int)((h - py + st - 1) / st);
            p.grid_w = (int)((wd - px + st - 1) / st);
            pick_block((size_t)p.grid_w, &p.bw, &p.bh);
            p.blocks_x = (p.grid_w + p.bw - 1) / p.bw;
            p.blocks_y = (p.grid_h + p.bh - 1) / p.bh;
            p.out_sy = st; p.out_oy = py; p.out_sx = st; p.out_ox = px;
            p.in_step = 1;
            p.kc = (int)k;
            p.accumulate = accumulate;
            p.three_pass = three ? 1 : 0;
            p.status = ctx->status;
            const int nt = class_taps(py, px, p.off_y, p.off_x, p.b_tap);
            p.ntaps = nt;
            if (nt == 0) continue;
            const size_t total_blocks = n * p.blocks_x * p.blocks_y;
            CUtensorMap ma, ma_lo;
            bool ok = nhwc_map(&ma, gt, n, oh, ow, k, p.bw, p.bh, 1, CU_TENSOR_MAP_SWIZZLE_128B) &&
                      nhwc_map(&ma_lo, three ? gt_lo : gt, n, oh, ow, k, p.bw, p.bh, 1, CU_TENSOR_MAP_SWIZZLE_128B);
            if (!ok) return katsu_set_error(KATSU_ERR_CUDA, "cuTensorMapEncodeTiled failed (conv dX)");
            const Activation act = {gt, three ? gt_lo : gt, n, oh, ow, k, 1};
            KATSU_TRY(launch_igemm(ctx, ma, ma_lo, wb, three ? wb_lo : wb, taps, c, k, p, total_blocks, act));
        }
    return KATSU_OK;
}

int32_t katsu_conv_igemm_dw(katsu_cuda_ctx *ctx, const float *x, const float *gr, float *dw,
                            size_t n, size_t c, size_t h, size_t wd, size_t k, size_t r, size_t s,
                            size_t stride, size_t pad, size_t oh, size_t ow, int accumulate, int *handled) {
    *handled = 0;
    const Shape g = {n, c, h, wd, k, r, s, stride, pad, oh, ow};
    if (!igemm_shape(ctx, g)) return KATSU_OK;
    *handled = 1;
    const bool three = ctx->precision == KATSU_MODE_3XTF32;
    const size_t xe = n * c * h * wd, ge = n * k * oh * ow, taps = r * s;
    DwParams p;
    p.n_img = (int)n; p.k = (int)k; p.c = (int)c; p.taps = (int)taps;
    p.groups_x = (int)katsu_div_up(ow, 8);
    p.groups_y = (int)katsu_div_up(oh, 4);
    p.stride = (int)stride;
    p.three_pass = three ? 1 : 0;
    p.status = ctx->status;
    for (size_t t = 0; t < taps; ++t) {
        p.off_y[t] = (short)((int)(t / s) - (int)pad);
        p.off_x[t] = (short)((int)(t % s) - (int)pad);
    }
    const DwPlan plan = dw_plan(ctx, g);
    const size_t bnt = plan.bnt, splits = plan.splits;
    p.taps_per_block = (int)plan.taps_per_block;
    p.cpad = 256 / (int)plan.taps_per_block;
    p.groups_per_split = (int)plan.groups_per_split;
    float *base = nullptr;
    KATSU_TRY(katsu_scratch(ctx, plan.scratch_floats, &base));
    // g first: a backward call that also computes dX has already staged it at the same place
    Scratch sc = {base, 0};
    float *gt = sc.take(ge), *gt_lo = three ? sc.take(ge) : nullptr;
    float *xt = sc.take(xe), *xt_lo = three ? sc.take(xe) : nullptr;
    p.partial = sc.take(plan.partial_floats);
    if (ctx->x_prestaged != nullptr) {
        xt = const_cast<float *>(ctx->x_prestaged);
        xt_lo = three ? xt + padded(xe) : nullptr;
    } else {
        KATSU_TRY(stage_nhwc(ctx, x, xt, xt_lo, n, c, h * wd));
    }
    if (!ctx->g_staged) KATSU_TRY(stage_nhwc(ctx, gr, gt, gt_lo, n, k, oh * ow));

    CUtensorMap mg, mg_lo, mx, mx_lo;
    const CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
    // wide layers: the GEMM kernel's convolution mode (g goes through tensor memory, its tiles
    // are read by builder threads and arrive as dense boxes; its lo halves are not needed)
    // (only for channel counts that rule out one-load tiles: with one load per operand tile the kernel
    // below, which reads both operands from shared memory, is faster in both precision modes: the wide
    // layer's dW 3.1 -> 2.5 ms in 3xTF32, 1.89 -> 1.14 ms in TF32)
    const bool whole_groups = (c % 32 == 0) && (k % 32 == 0);
    const bool via_gemm = !plan.all_taps && bnt == 128 && !whole_groups;
    bool ok = nhwc_map(&mg, gt, n, oh, ow, k, 8, 4, 1, via_gemm ? CU_TENSOR_MAP_SWIZZLE_NONE : sw) &&
              nhwc_map(&mg_lo, three ? gt_lo : gt, n, oh, ow, k, 8, 4, 1, sw) &&
              nhwc_map(&mx, xt, n, h, wd, c, 8, 4, (int)stride, sw) &&
              nhwc_map(&mx_lo, three ? xt_lo : xt, n, h, wd, c, 8, 4, (int)stride, sw);
    if (!ok) return katsu_set_error(KATSU_ERR_CUDA, "cuTensorMapEncodeTiled failed (conv dW)");
    p.grouped = 0;
    if (!plan.all_taps && whole_groups) {
        CUtensorMap ng, ng_lo, nx, nx_lo;
        const bool grouped = nhwc_grouped_map(&ng, gt, n, oh, ow, k, 8, 4, 1, BM / 32, via_gemm ? CU_TENSOR_MAP_SWIZZLE_NONE : sw) &&
                             nhwc_grouped_map(&ng_lo, three ? gt_lo : gt, n, oh, ow, k, 8, 4, 1, BM / 32, sw) &&
                             nhwc_grouped_map(&nx, xt, n, h, wd, c, 8, 4, (int)stride, (plan.taps_per_block > 1 ? p.cpad : (int)bnt) / 32, sw) &&
                             nhwc_grouped_map(&nx_lo, three ? xt_lo : xt, n, h, wd, c, 8, 4, (int)stride, (plan.taps_per_block > 1 ? p.cpad : (int)bnt) / 32, sw);
        if (!grouped && plan.taps_per_block > 1) return katsu_set_error(KATSU_ERR_CUDA, "cuTensorMapEncodeTiled failed (conv dW, grouped)");
        if (grouped) { mg = ng; mg_lo = ng_lo; mx = nx; mx_lo = nx_lo; p.grouped = 1; }
    }
    if (via_gemm) {
        KATSU_TRY(katsu_umma_conv_dw(ctx, &mg, &mx, &mx_lo, p.partial, k, c, taps, n * p.groups_x * p.groups_y,
                                     (size_t)p.groups_x, size_t(p.groups_x) * p.groups_y, stride, p.off_y, p.off_x,
                                     splits, (size_t)p.groups_per_split, p.grouped));
    } else
    if (plan.all_taps) {
        DwTapsParams q;
        q.partial = p.partial;
        q.n_img = (int)n; q.k = (int)k; q.c = (int)c; q.taps = (int)taps;
        q.groups_x = p.groups_x; q.groups_y = p.groups_y;
        q.total_groups = (long long)(n * p.groups_x * p.groups_y);
        q.chunks = (int)splits;
        q.stride = (int)stride;
        q.three_pass = three ? 1 : 0;
        q.a_groups = (int)katsu_div_up(k, (size_t)32);
        q.status = ctx->status;
        q.grouped = 0;
        if (k % 32 == 0) {
            // box = exactly the groups that exist, so the bytes counted on the stage barrier stay a_groups * 4 KiB
            CUtensorMap ng, ng_lo;
            if (nhwc_grouped_map(&ng, gt, n, oh, ow, k, 8, 4, 1, q.a_groups, sw) &&
                nhwc_grouped_map(&ng_lo, three ? gt_lo : gt, n, oh, ow, k, 8, 4, 1, q.a_groups, sw)) {
                mg = ng; mg_lo = ng_lo; q.grouped = 1;
            }
        }
        for (size_t t = 0; t < taps; ++t) { q.off_y[t] = p.off_y[t]; q.off_x[t] = p.off_x[t]; }
        const size_t smem = size_t(TAPS_STAGES) * (2 * TILE_BYTES + 2 * taps * 4096) + 1024;
        KATSU_CUDA_TRY(cudaFuncSetAttribute(conv_dw_taps_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        size_t grid = splits < (size_t)ctx->num_sms ? splits : (size_t)ctx->num_sms;
        KATSU_LAUNCH(ctx, conv_dw_taps_kernel, (unsigned)grid, 192, smem, mg, mg_lo, mx, mx_lo, q);
    } else {
        dim3 grid((unsigned)(katsu_div_up(k, (size_t)BM) * (plan.taps_per_block > 1 ? 1 : katsu_div_up(c, bnt))),
                  (unsigned)katsu_div_up(taps, plan.taps_per_block), (unsigned)splits);
        if (three) {
            auto kernel = bnt == 32 ? conv_dw_igemm_kernel<32, false> : bnt == 64 ? conv_dw_igemm_kernel<64, false>
                                                                                  : conv_dw_igemm_kernel<128, false>;
            KATSU_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
            KATSU_LAUNCH(ctx, kernel, grid, 192, kSmemBytes, mg, mg_lo, mx, mx_lo, p);
        } else {
            auto kernel = bnt == 32 ? conv_dw_igemm_kernel<32, true> : bnt == 64 ? conv_dw_igemm_kernel<64, true>
                          : bnt == 128 ? conv_dw_igemm_kernel<128, true> : conv_dw_igemm_kernel<256, true>;
            const size_t smem = bnt == 32 ? DwCfg<32, true>::SMEM : bnt == 64 ? DwCfg<64, true>::SMEM
                                : bnt == 128 ? DwCfg<128, true>::SMEM : DwCfg<256, true>::SMEM;
            KATSU_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            KATSU_LAUNCH(ctx, kernel, grid, 192, smem, mg, mg_lo, mx, mx_lo, p);
        }
    }
    KATSU_LAUNCH(ctx, dw_fold_kernel, (unsigned)katsu_div_up(k * c * taps, (size_t)32), 256, 0, p.partial, dw, (int)k,
                 (int)c, (int)taps, (int)splits, accumulate);
    return KATSU_OK;
}
