// Tensor-core GEMM for Tensor::matmul and its VJP (crates/katsu-core/src/tensor.rs:264-273,
// 418-445) on tcgen05: TMA-fed 128x128 tiles, f32 accumulators in tensor memory.
//
//   C[M,N] (+)= A * B with either operand K-major (K contiguous) or MN-major
//   (M resp. N contiguous), so a@b, g@b^T and a^T@g all run without a transpose.
//
// Precision.  kind::tf32 truncates its f32 inputs to TF32.  TF32 mode issues one
// MMA per k-step on the raw data.  3xTF32 mode restores FP32-grade accuracy with
// the split x = hi + lo, hi = trunc_tf32(x) (what the hardware sees when given x),
// lo = x - hi: three MMAs per k-step, lo*hi + hi*lo + hi*hi, into the same f32
// accumulator.
//
// Where the operands live.  With both operands in shared memory a 128x128x8 MMA reads 8 KiB
// in its 64 pipe cycles -- the whole 128 B/clk of the SM's shared memory, before TMA has
// written anything -- and every k-block pulled 64 KiB (hi and lo tiles of both operands)
// through L2; that form topped out at 48 % of the pipe.  So A goes through TENSOR MEMORY: TMA drops the raw A tile in shared memory, four
// builder warps (thread = tile row) read it once, compute lo on the fly and write hi | lo
// with tcgen05.st; the MMAs then read only B (hi and lo tiles, lo produced by a streaming
// pre-pass) from shared memory.  A needs no lo array in HBM at all and a k-block pulls 48 KiB.
// Measured 8192^3: 203 TFLOP/s useful = 608 issued (3xTF32), 175 before.  No pipe is saturated at
// that point (tensor 67 %, L2 38 %, DRAM 20 % at 4096^3): the hand-off ring bounds it.  A 256-row
// tile would halve the B traffic per MMA but leaves no tensor-memory columns for the A stages.
//
// Accumulation.  The tensor core's f32 accumulate loses a little on every k-step
// (measured: relative error grows about linearly with K, 1.2e-6 at K = 512), so k-blocks
// alternate between two accumulators and every DRAIN k-blocks four epilogue warps fold both
// into f32 registers (chains of at most 512 terms).  Split-K over blockIdx.z only fills the
// GPU when there are fewer tiles than SMs; slabs are folded in a fixed order
// (bit-reproducible, no atomics).
#include "common.cuh"
#include "sm100.cuh"

using namespace sm100;

namespace {

constexpr int BM = 128;      // tile rows == TMEM lanes
constexpr int BN = 128;      // tile columns
constexpr int BK = 32;       // f32 per 128-byte swizzle row
constexpr int AS = 4;          // shared-memory slots of the raw A tile (free as soon as the builders have read it)
constexpr int BS = 4;          // shared-memory slots of the B tiles, hi | lo (free when the MMAs that read them are done)
constexpr int TS = 4;          // tensor-memory stages of A, hi | lo
constexpr int TILE_BYTES = BM * BK * 4;  // 16 KiB, same for A and B tiles (BM == BN)

struct GemmParams {
    float *c;          // output, or partial slabs [splits][M][N] when splits > 1
    int M, N, K;
    int kblocks_per_split;
    int splits;
    int accumulate;    // only used when splits == 1
    int three_pass;    // 3xTF32
    int *status;
    // MN-major operand maps with the 32-wide column groups as a dimension of their own (3-D; 5-D in conv_dw
    // mode): one load brings a whole operand tile.  The TMA unit's cost per instruction, not its bandwidth,
    // is what a stage made of 4 KiB boxes pays for.
    int a_grouped, b_grouped;
    // conv_dw = 1: the dW contraction of a convolution.  A = g and B = x are channels-innermost
    // staging arrays [N][H][W][C] (both MN-major), a k-block is one 8 x 4 group of output pixels,
    // blockIdx.z = split * taps + tap selects the filter tap whose shifted x window is B, and
    // every block writes a slab (M = output channels, N = input channels).
    int conv_dw, taps, groups_x, groups_per_img, stride;
    short off_y[49], off_x[49];
};

__global__ void __launch_bounds__(256) split_lo_kernel(const float *__restrict__ x, float *__restrict__ lo, size_t count) {
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
        const float v = x[i];
        lo[i] = v - __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
    }
}

constexpr int DRAIN = 32;            // k-blocks per accumulator batch (2 accumulators x 16 k-blocks x 32)
constexpr uint32_t A_COL0 = 2 * BN;  // TMEM: [2 accumulators x 128][TS A stages x {32 hi, 32 lo}]

// Warps 0-3: drains and the epilogue (TMEM lane quarter = warp).  Warps 4-7: A builders
// (quarter = warp & 3).  Warp 8: TMA loads of A.  Warp 9: MMA issue.  Warp 10: TMA loads of B.
// A and B have separate rings because their slots live differently long: an A slot is free once
// the builders have read it, a B slot only when the MMAs that read it have completed.
// (A second builder group with eight drain warps was measured slower, 183 against 193 TFLOP/s at
// 8192^3: the builders are not what bounds the kernel.)
constexpr int RASTER_W = 16;
constexpr int GEMM_THREADS = 11 * 32, TMA_A_WARP = 8, MMA_WARP = 9, TMA_B_WARP = 10;

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_b_lo, GemmParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t a_full[AS], a_read[AS], b_full[BS], b_free[BS], t_free[TS], a_ready[TS], batch_done, drained;
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Tile order: bands of RASTER_W column tiles, row tiles fastest inside a band, so that the
    // tiles in flight at one time (one per SM) share few distinct A and B panels and those stay
    // in L2 (x-fastest order re-read all of B, hi and lo, for every 2-3 tile rows).
    int tile_m, tile_n;
    {
        const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
        const int band = blockIdx.x / (RASTER_W * m_tiles), within = blockIdx.x % (RASTER_W * m_tiles);
        const int width = (n_tiles - band * RASTER_W) < RASTER_W ? (n_tiles - band * RASTER_W) : RASTER_W;
        tile_n = band * RASTER_W + within % width;
        tile_m = within / width;
    }
    const int m0 = tile_m * BM, n0 = tile_n * BN;
    const int kb_total = (p.K + BK - 1) / BK;
    const int tap = p.conv_dw ? int(blockIdx.z) % p.taps : 0;
    const int kb_begin = (p.conv_dw ? int(blockIdx.z) / p.taps : int(blockIdx.z)) * p.kblocks_per_split;
    int kb_end = kb_begin + p.kblocks_per_split;
    if (kb_end > kb_total) kb_end = kb_total;
    const int kblocks = kb_end > kb_begin ? kb_end - kb_begin : 0;
    const int batches = (kblocks + DRAIN - 1) / DRAIN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < AS; ++s) {
            mbar_init(&a_full[s], 1);
            mbar_init(&a_read[s], 4);
        }
        for (int s = 0; s < BS; ++s) {
            mbar_init(&b_full[s], 1);
            mbar_init(&b_free[s], 1);
        }
        for (int s = 0; s < TS; ++s) {
            mbar_init(&t_free[s], 1);
            mbar_init(&a_ready[s], 128);
        }
        mbar_init(&batch_done, 1);
        mbar_init(&drained, 128);
        mbar_init_fence();
    }
    if (warp == MMA_WARP) {
        tmem_alloc(&tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;

    unsigned char *a_slots = smem, *b_slots = smem + AS * TILE_BYTES;
    if (warp == TMA_A_WARP && lane == 0) {
        // ---- TMA producer of A ----
        for (int i = 0; i < kblocks; ++i) {
            const int sa = i % AS;
            if (i >= AS && !mbar_wait(&a_read[sa], ((i / AS) - 1) & 1, p.status, 11)) break;
            mbar_arrive_expect_tx(&a_full[sa], TILE_BYTES);
            unsigned char *ad = a_slots + sa * TILE_BYTES;
            const int k0 = (kb_begin + i) * BK;
            if (A_MN && p.conv_dw) {
                const int gidx = kb_begin + i, img = gidx / p.groups_per_img, r = gidx % p.groups_per_img;
                if (p.a_grouped) {
                    tma_load_5d(ad, &map_a, &a_full[sa], 0, (r % p.groups_x) * 8, (r / p.groups_x) * 4, m0 / 32, img);
                    continue;
                }
                for (int j = 0; j < BM / 32; ++j)
                    tma_load_4d(ad + j * 4096, &map_a, &a_full[sa], m0 + 32 * j, (r % p.groups_x) * 8, (r / p.groups_x) * 4, img);
            } else if (!A_MN) {
                tma_load_2d(ad, &map_a, &a_full[sa], k0, m0);
            } else if (p.a_grouped) {
                tma_load_3d(ad, &map_a, &a_full[sa], 0, k0, m0 / 32);
            } else {
                for (int j = 0; j < BM / 32; ++j) tma_load_2d(ad + j * 4096, &map_a, &a_full[sa], m0 + 32 * j, k0);
            }
        }
    } else if (warp == TMA_B_WARP && lane == 0) {
        // ---- TMA producer of B (hi and lo tiles) ----
        for (int i = 0; i < kblocks; ++i) {
            const int sb = i % BS;
            if (i >= BS && !mbar_wait(&b_free[sb], ((i / BS) - 1) & 1, p.status, 17)) break;
            mbar_arrive_expect_tx(&b_full[sb], (p.three_pass ? 2 : 1) * TILE_BYTES);
            unsigned char *bd = b_slots + sb * 2 * TILE_BYTES;
            const int k0 = (kb_begin + i) * BK;
            for (int part = 0; part < (p.three_pass ? 2 : 1); ++part) {
                const CUtensorMap *mb = part ? &map_b_lo : &map_b;
                if (B_MN && p.conv_dw) {
                    const int gidx = kb_begin + i, img = gidx / p.groups_per_img, r = gidx % p.groups_per_img;
                    const int x0 = (r % p.groups_x) * 8 * p.stride + p.off_x[tap], y0 = (r / p.groups_x) * 4 * p.stride + p.off_y[tap];
                    if (p.b_grouped) {
                        tma_load_5d(bd + part * TILE_BYTES, mb, &b_full[sb], 0, x0, y0, n0 / 32, img);
                        continue;
                    }
                    for (int j = 0; j < BN / 32; ++j)
                        tma_load_4d(bd + part * TILE_BYTES + j * 4096, mb, &b_full[sb], n0 + 32 * j, x0, y0, img);
                } else if (!B_MN) {
                    tma_load_2d(bd + part * TILE_BYTES, mb, &b_full[sb], k0, n0);
                } else if (p.b_grouped) {
                    tma_load_3d(bd + part * TILE_BYTES, mb, &b_full[sb], 0, k0, n0 / 32);
                } else {
                    for (int j = 0; j < BN / 32; ++j) tma_load_2d(bd + part * TILE_BYTES + j * 4096, mb, &b_full[sb], n0 + 32 * j, k0);
                }
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // ---- A builders: thread = one row of the tile; hi goes in raw (the tensor core truncates) ----
        const int quarter = warp & 3, row = quarter * 32 + lane;
        const uint32_t lane_addr = tmem_base + (uint32_t(quarter * 32) << 16) + A_COL0;
        for (int i = 0; i < kblocks; ++i) {
            const int sa = i % AS, s = i % TS;
            if (!mbar_wait_warp_ready(&a_full[sa], (i / AS) & 1, p.status, 14)) break;
            const unsigned char *ad = a_slots + sa * TILE_BYTES;
            float v[32];
            if (!A_MN) {
                // K-major tile, 128-byte-swizzled rows: chunk c of row r sits at chunk c ^ (r & 7)
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const float4 q = ld_shared_v4(ad + row * 128 + ((c ^ (row & 7)) << 4));
                    v[4 * c] = q.x; v[4 * c + 1] = q.y; v[4 * c + 2] = q.z; v[4 * c + 3] = q.w;
                }
            } else {
                // MN-major tile: four dense [32 k][32 m] sub-tiles; a warp reads one 128-byte k-row per load
#pragma unroll
                for (int k = 0; k < 32; ++k) v[k] = ld_shared_f32(ad + quarter * 4096 + k * 128 + lane * 4);
            }
            fence_proxy_async_smem();  // ordinary reads of the slot before its TMA refill
            mbar_arrive_warp(&a_read[sa]);
            if (i >= TS && !mbar_wait_warp_ready(&t_free[s], ((i / TS) - 1) & 1, p.status, 15)) break;
            tc_fence_after_sync();
            tmem_st_32x32(lane_addr + uint32_t(s) * 64, v);
            if (p.three_pass) {
#pragma unroll
                for (int t = 0; t < 32; ++t) v[t] -= __uint_as_float(__float_as_uint(v[t]) & 0xFFFFE000u);
                tmem_st_32x32(lane_addr + uint32_t(s) * 64 + 32, v);
            }
            tmem_st_wait();
            tc_fence_before_sync();
            mbar_arrive(&a_ready[s]);
        }
    } else if (warp == MMA_WARP) {
        // ---- MMA issue: the whole warp runs the loop, the thread chosen by elect.sync issues ----
        const bool issue = elect_one();
        const uint32_t idesc = idesc_tf32(BM, BN, false, B_MN);
        bool ok = true;
        for (int b = 0; b < batches && ok; ++b) {
            // the previous batch's accumulators must have been folded into registers
            if (b > 0 && !mbar_wait_warp(&drained, (b - 1) & 1, p.status, 16)) break;
            tc_fence_after_sync();
            const int i_end = (b + 1) * DRAIN < kblocks ? (b + 1) * DRAIN : kblocks;
            for (int i = b * DRAIN; i < i_end; ++i) {
                const int s = i % TS, sb = i % BS;
                if (!mbar_wait_warp_ready(&a_ready[s], (i / TS) & 1, p.status, 12)) { ok = false; break; }
                if (!mbar_wait_warp_ready(&b_full[sb], (i / BS) & 1, p.status, 18)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t bd = smem_u32(b_slots + sb * 2 * TILE_BYTES);
                const int li = i - b * DRAIN;
                const uint32_t acc = tmem_base + uint32_t(li & 1) * BN;
                const uint32_t a_hi = tmem_base + A_COL0 + uint32_t(s) * 64, a_lo = a_hi + 32;
                if (issue) {
#pragma unroll
                    for (int j = 0; j < BK / 8; ++j) {
                        const uint32_t b_off = B_MN ? j * 1024 : j * 32;
                        const uint64_t b_hi = B_MN ? smem_desc(bd + b_off, 4096, 512, kLayoutSw128Base32)
                                                   : smem_desc(bd + b_off, 16, 1024, kLayoutSw128);
                        const bool acc_flag = !(li < 2 && j == 0);
                        if (p.three_pass) {
                            const uint64_t b_lo = B_MN ? smem_desc(bd + TILE_BYTES + b_off, 4096, 512, kLayoutSw128Base32)
                                                       : smem_desc(bd + TILE_BYTES + b_off, 16, 1024, kLayoutSw128);
                            mma_tf32_ts(acc, a_lo + 8 * j, b_hi, idesc, acc_flag);
                            mma_tf32_ts(acc, a_hi + 8 * j, b_lo, idesc, true);
                            mma_tf32_ts(acc, a_hi + 8 * j, b_hi, idesc, true);
                        } else {
                            mma_tf32_ts(acc, a_hi + 8 * j, b_hi, idesc, acc_flag);
                        }
                    }
                    mma_commit(&t_free[s]);
                    mma_commit(&b_free[sb]);
                    if (i == i_end - 1) mma_commit(&batch_done);
                }
                __syncwarp();
            }
        }
    } else if (warp < 4) {
        // ---- drains and epilogue: warp w owns tile rows 32w .. 32w+31 ----
        float run[BN];
#pragma unroll
        for (int i = 0; i < BN; ++i) run[i] = 0.f;
        bool alive = true;
        for (int b = 0; b < batches && alive; ++b) {
            alive = mbar_wait_warp(&batch_done, b & 1, p.status, 13);
            tc_fence_after_sync();
            if (alive) {
                const int in_batch = (kblocks - b * DRAIN) < DRAIN ? (kblocks - b * DRAIN) : DRAIN;
#pragma unroll
                for (int q = 0; q < BN / 32; ++q) {
                    if (n0 + q * 32 >= p.N) break;  // warp-uniform
                    for (int a = 0; a < 2 && a < in_batch; ++a) {
                        float t[32];
                        tmem_ld_32x32(tmem_base + (uint32_t(warp * 32) << 16) + a * BN + q * 32, t);
#pragma unroll
                        for (int i = 0; i < 32; ++i) run[q * 32 + i] += t[i];
                    }
                }
                tc_fence_before_sync();
                mbar_arrive(&drained);
            }
        }
        const int row = m0 + warp * 32 + lane;
        if (alive && row < p.M) {
            const bool slabs = p.splits > 1 || p.conv_dw;
            float *out = p.c + (slabs ? size_t(blockIdx.z) * p.M * p.N : 0);
            const bool acc_out = p.accumulate && !slabs;
#pragma unroll
            for (int q = 0; q < BN / 32; ++q) {
                const int c0 = q * 32;
                if (n0 + c0 >= p.N) break;
                float *dst = out + size_t(row) * p.N + n0 + c0;
                if (n0 + c0 + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        float4 o = make_float4(run[c0 + i], run[c0 + i + 1], run[c0 + i + 2], run[c0 + i + 3]);
                        if (acc_out) {
                            const float4 old = *reinterpret_cast<const float4 *>(dst + i);
                            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                        }
                        *reinterpret_cast<float4 *>(dst + i) = o;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (n0 + c0 + i < p.N) dst[i] = acc_out ? dst[i] + run[c0 + i] : run[c0 + i];
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == MMA_WARP) tmem_dealloc(tmem_base, 512);
}

__global__ void __launch_bounds__(256)
fold_slabs_kernel(const float *__restrict__ partial, float *out, size_t elems, int parts, int accumulate) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= elems) return;
    float s = 0.f;
    for (int q = 0; q < parts; ++q) s += partial[size_t(q) * elems + i];
    out[i] = accumulate ? out[i] + s : s;
}

bool aligned16(const void *ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

// Tensor map of one operand.  K-major: storage [rows][K] (K contiguous), box 32 x 128.
// MN-major: storage [K][cols] (cols contiguous), box 32 x 32 with the 32-byte-atom swizzle.
// When the MN extent is a multiple of 32 the MN-major map is 3-D {32, K, extent / 32} with box {32, 32, 4}:
// the four 32-column slabs of a tile, 4 KiB apart in shared memory, arrive by one load (*grouped = 1).
bool mn_major_map(CUtensorMap *map, const float *base, size_t mn_extent, size_t k_extent, CUtensorMapSwizzle swizzle,
                  int *grouped) {
    *grouped = (mn_extent & 31) == 0;
    if (*grouped) {
        const uint64_t dims[3] = {32, k_extent, mn_extent / 32}, strides[3] = {1, mn_extent, 32};
        const uint32_t box[3] = {32, BK, BM / 32};
        if (katsu_make_tensor_map(map, base, 3, dims, strides, box, swizzle)) return true;
        *grouped = 0;
    }
    const uint64_t dims[2] = {mn_extent, k_extent}, strides[2] = {1, mn_extent};
    const uint32_t box[2] = {32, BK};
    return katsu_make_tensor_map(map, base, 2, dims, strides, box, swizzle);
}

bool operand_map(CUtensorMap *map, const float *base, bool mn_major, size_t mn_extent, size_t k_extent, int *grouped) {
    *grouped = 0;
    if (!mn_major) {
        const uint64_t dims[2] = {k_extent, mn_extent}, strides[2] = {1, k_extent};
        const uint32_t box[2] = {BK, BM};
        return katsu_make_tensor_map(map, base, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    }
    return mn_major_map(map, base, mn_extent, k_extent, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, grouped);
}

// MN-major A is read by the builder threads, not by the tensor core: dense 32 x 32 boxes.
bool builder_map_mn(CUtensorMap *map, const float *base, size_t mn_extent, size_t k_extent, int *grouped) {
    return mn_major_map(map, base, mn_extent, k_extent, CU_TENSOR_MAP_SWIZZLE_NONE, grouped);
}

template <bool A_MN, bool B_MN>
int32_t launch(katsu_cuda_ctx *ctx, const float *a, const float *b, float *c, size_t M, size_t N, size_t K,
               int accumulate) {
    const bool three_pass = ctx->precision == KATSU_MODE_3XTF32;
    const size_t b_count = K * N;
    const int kb_total = (int)katsu_div_up(K, (size_t)BK);
    // K split only to fill the GPU when there are fewer tiles than SMs (chains are kept short by
    // the in-kernel drains); every split gets at least DRAIN k-blocks.
    const size_t tiles = katsu_div_up(M, (size_t)BM) * katsu_div_up(N, (size_t)BN);
    int splits = (int)katsu_div_up((size_t)ctx->num_sms, tiles);
    if (splits > kb_total / DRAIN) splits = kb_total / DRAIN;
    if (splits < 1) splits = 1;
    if (splits > 1024) splits = 1024;
    int kb_per_split = (int)katsu_div_up((size_t)kb_total, (size_t)splits);
    splits = (int)katsu_div_up((size_t)kb_total, (size_t)kb_per_split);

    size_t scratch_floats = (three_pass ? b_count : 0) + (splits > 1 ? size_t(splits) * M * N : 0);
    float *scratch = nullptr;
    if (scratch_floats) KATSU_TRY(katsu_scratch(ctx, scratch_floats + 64, &scratch));
    float *b_lo = nullptr, *slabs = nullptr;
    size_t cursor = 0;
    auto take = [&](size_t n) { float *ptr = scratch + cursor; cursor += (n + 31) / 32 * 32; return ptr; };
    if (three_pass) {
        b_lo = take(b_count);
        const unsigned blocks = (unsigned)(size_t(ctx->num_sms) * 8);
        KATSU_LAUNCH(ctx, split_lo_kernel, blocks, 256, 0, b, b_lo, b_count);
    }
    if (splits > 1) slabs = take(size_t(splits) * M * N);

    CUtensorMap map_a, map_b, map_b_lo;
    GemmParams p;
    int b_lo_grouped = 0;
    bool ok = (A_MN ? builder_map_mn(&map_a, a, M, K, &p.a_grouped) : operand_map(&map_a, a, false, M, K, &p.a_grouped)) &&
              operand_map(&map_b, b, B_MN, N, K, &p.b_grouped) &&
              operand_map(&map_b_lo, three_pass ? b_lo : b, B_MN, N, K, &b_lo_grouped);
    if (!ok || b_lo_grouped != p.b_grouped)
        return katsu_set_error(KATSU_ERR_CUDA, "cuTensorMapEncodeTiled failed for a matmul operand");

    p.c = splits > 1 ? slabs : c;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.kblocks_per_split = kb_per_split;
    p.splits = splits;
    p.accumulate = accumulate;
    p.three_pass = three_pass ? 1 : 0;
    p.status = ctx->status;
    p.conv_dw = 0;
    const size_t smem = size_t(AS + 2 * BS) * TILE_BYTES + 1024;
    auto kernel = umma_gemm_kernel<A_MN, B_MN>;
    KATSU_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)(katsu_div_up(N, (size_t)BN) * katsu_div_up(M, (size_t)BM)), 1, (unsigned)splits);
    KATSU_LAUNCH(ctx, kernel, grid, GEMM_THREADS, smem, map_a, map_b, map_b_lo, p);
    if (splits > 1)
        KATSU_LAUNCH(ctx, fold_slabs_kernel, (unsigned)katsu_div_up(M * N, (size_t)256), 256, 0, slabs, c, M * N, splits,
                     accumulate);
    return KATSU_OK;
}

}  // namespace

// Diagnostic: one block waits, with a budget of `cycles` SM clocks, on an mbarrier that
// nothing ever arrives on.  The wait gives up, records code 99 in the context's status word
// and the kernel returns normally; the next katsu_cuda_sync reports KATSU_ERR_TIMEOUT and
// the context stays usable.  This is the path every pipeline wait in the tensor-core
// kernels takes if a hand-off is ever missed.
__global__ void wait_timeout_probe_kernel(int *status, long long cycles) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_init_fence();
    }
    __syncthreads();
    mbar_wait_budget(&bar, 0, status, 99, cycles);
}

extern "C" int32_t katsu_cuda_selftest_wait_timeout(katsu_cuda_ctx *ctx, uint64_t cycles) {
    KATSU_TRY(katsu_bind(ctx));
    KATSU_REQUIRE(cycles >= 1000 && cycles <= 200000000ull, "cycle budget must be between 1e3 and 2e8");
    KATSU_LAUNCH(ctx, wait_timeout_probe_kernel, 1, 32, 0, ctx->status, (long long)cycles);
    return KATSU_OK;
}

// dW of a wide convolution through the same kernel (see GemmParams::conv_dw).  The caller has
// staged g and x (and x's lo halves) channels-innermost and built their tensor maps: g with
// dense 32-channel x 8 x 4 boxes (read by the builders), x with the 32-byte-atom swizzle (read
// by the tensor core), stepping `stride` pixels; grouped_maps = 1 when they are the 5-D maps whose
// fourth dimension counts 32-channel groups (box: four groups).  partial receives [splits][taps][k][c].
int32_t katsu_umma_conv_dw(katsu_cuda_ctx *ctx, const CUtensorMap *map_g, const CUtensorMap *map_x,
                           const CUtensorMap *map_x_lo, float *partial, size_t k, size_t c, size_t taps,
                           size_t total_groups, size_t groups_x, size_t groups_per_img, size_t stride,
                           const short *off_y, const short *off_x, size_t splits, size_t groups_per_split,
                           int grouped_maps) {
    if (taps > 49 || total_groups > 0x3ffffffu || splits * taps > 65535)
        return katsu_set_error(KATSU_ERR_UNSUPPORTED, "convolution too large for the dW contraction");
    GemmParams p;
    p.c = partial;
    p.M = (int)k; p.N = (int)c; p.K = (int)(total_groups * BK);
    p.kblocks_per_split = (int)groups_per_split;
    p.splits = (int)splits;
    p.accumulate = 0;
    p.three_pass = ctx->precision == KATSU_MODE_3XTF32 ? 1 : 0;
    p.status = ctx->status;
    p.conv_dw = 1;
    p.a_grouped = p.b_grouped = grouped_maps;
    p.taps = (int)taps; p.groups_x = (int)groups_x; p.groups_per_img = (int)groups_per_img; p.stride = (int)stride;
    for (size_t t = 0; t < taps; ++t) { p.off_y[t] = off_y[t]; p.off_x[t] = off_x[t]; }
    const size_t smem = size_t(AS + 2 * BS) * TILE_BYTES + 1024;
    auto kernel = umma_gemm_kernel<true, true>;
    KATSU_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)(katsu_div_up(c, (size_t)BN) * katsu_div_up(k, (size_t)BM)), 1, (unsigned)(splits * taps));
    KATSU_LAUNCH(ctx, kernel, grid, GEMM_THREADS, smem, *map_g, *map_x, *map_x_lo, p);
    return KATSU_OK;
}

// C[M,N] (+)= A * B on the tensor cores.  a_mn / b_mn: operand stored with its
// M (resp. N) index contiguous instead of K.  *handled = 0 when the shape does
// not meet TMA's alignment rules or is too small to be worth a 128x128 tile;
// the caller then uses the CUDA-core kernels.
int32_t katsu_umma_gemm(katsu_cuda_ctx *ctx, const float *a, const float *b, float *c, size_t M, size_t N, size_t K,
                        bool a_mn, bool b_mn, int accumulate, int *handled) {
    *handled = 0;
    if (ctx->precision == KATSU_MODE_FP32) return KATSU_OK;
    if (M < 64 || N < 32 || K < 32) return KATSU_OK;
    if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff || katsu_div_up(M, (size_t)BM) > 65535) return KATSU_OK;
    // TMA: 16-byte aligned bases and row pitches
    const size_t a_pitch = a_mn ? M : K, b_pitch = b_mn ? N : K;
    if ((a_pitch & 3) || (b_pitch & 3) || !aligned16(a) || !aligned16(b) || !aligned16(c)) return KATSU_OK;
    if (katsu_tensor_map_encoder() == nullptr) return KATSU_OK;
    // single-pass TF32, large: 128 x 256 tiles straight from shared memory
    KATSU_TRY(katsu_umma_gemm_wide(ctx, a, b, c, M, N, K, a_mn, b_mn, accumulate, handled));
    if (*handled) return KATSU_OK;
    // tall enough for a 256-row tile: two thread blocks share each MMA and each loads half of B
    KATSU_TRY(katsu_umma_gemm_pair(ctx, a, b, c, M, N, K, a_mn, b_mn, accumulate, handled));
    if (*handled) return KATSU_OK;
    *handled = 1;
    if (!a_mn && !b_mn) return launch<false, false>(ctx, a, b, c, M, N, K, accumulate);
    if (!a_mn && b_mn) return launch<false, true>(ctx, a, b, c, M, N, K, accumulate);
    if (a_mn && !b_mn) return launch<true, false>(ctx, a, b, c, M, N, K, accumulate);
    return launch<true, true>(ctx, a, b, c, M, N, K, accumulate);
}
