// Single-pass TF32 GEMM with 128 x 256 tiles, both operands read by the tensor core from shared memory.
//
// Replaces, for KATSU_MODE_TF32 and large shapes, the loops of Tensor::matmul
// (crates/katsu-core/src/tensor.rs:265-273) and of its VJP (tensor.rs:425-444).
//
// Why a kernel of its own.  The split-precision kernel (umma_gemm.cu) routes A through tensor memory, where
// builder threads split it into hi | lo, and spends its tensor-memory budget on those stages; in single-pass
// mode that detour only costs time (the builders, not the pipe, set the pace: 358 TFLOP/s at 8192^3).  Single
// pass needs no lo halves and no A in tensor memory: a stage is A (16 KiB) | B (32 KiB) read straight from shared
// memory, four stages deep, and tensor memory holds two 256-column accumulators so that a tile's epilogue runs
// under the next tile's k-loop.  The tile is 128 x 256 because what bounds the k-loop is the traffic through
// shared memory (every operand byte is written once by TMA and read once per MMA that uses it): back-to-back
// MMAs on resident operands run at the pipe's rate for N = 128 and N = 256 alike (64 and 128 clocks), but per
// flop a 128 x 256 tile moves three quarters of the bytes of a 128 x 128 one.
//
// Persistent: one block per SM walks the tiles band by band (bands of RASTER_M tile rows, column-major
// inside a band) so that blocks running together share operand tiles in L2.  Warps 0-3 are the epilogue
// (TMEM lane quarter = warp), warp 4 issues the TMA loads, warp 5 the MMAs.  K is not split: the dispatcher
// only sends shapes with at least one tile per two SMs here.
#include <cstring>

#include "common.cuh"
#include "sm100.cuh"
#include "sm100_pair.cuh"

using namespace sm100;

namespace {

constexpr int BM = 128, BN = 256, BK = 32, STAGES = 4, RASTER_M = 16;
constexpr int A_BYTES = BM * BK * 4, B_BYTES = BN * BK * 4, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr size_t SMEM = size_t(STAGES) * STAGE_BYTES + 1024;

struct WideParams {
    float *c;
    int M, N, K;
    int m_tiles, n_tiles;
    int accumulate;
    int a_grouped, b_grouped;  // MN-major maps are 3-D {32, K, extent / 32}: one load per operand tile
    int *status;
};

__device__ __forceinline__ void tile_of(int tile, int m_tiles, int n_tiles, int *mt, int *nt) {
    const int band_tiles = RASTER_M * n_tiles;
    const int band = tile / band_tiles, r = tile % band_tiles;
    const int rows = m_tiles - band * RASTER_M < RASTER_M ? m_tiles - band * RASTER_M : RASTER_M;
    *mt = band * RASTER_M + r % rows;
    *nt = r / rows;
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(192, 1)
umma_gemm_wide_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const __grid_constant__ WideParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kblocks = (p.K + BK - 1) / BK;
    const int total_tiles = p.m_tiles * p.n_tiles;
    const int my_tiles = (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 4);
        }
        mbar_init_fence();
    }
    if (warp == 5) {
        tmem_alloc(&tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;

    if (warp == 4 && lane == 0) {
        // ---- TMA producer ----
        bool ok = true;
        for (int it = 0; it < my_tiles && ok; ++it) {
            int mt, nt;
            tile_of(blockIdx.x + it * gridDim.x, p.m_tiles, p.n_tiles, &mt, &nt);
            const int m0 = mt * BM, n0 = nt * BN;
            for (int i = 0; i < kblocks; ++i) {
                const int g = it * kblocks + i, s = g % STAGES;
                if (g >= STAGES && !mbar_wait(&empty[s], ((g / STAGES) - 1) & 1, p.status, 131)) { ok = false; break; }
                mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
                unsigned char *ad = smem + s * STAGE_BYTES, *bd = ad + A_BYTES;
                const int k0 = i * BK;
                if (!A_MN) {
                    tma_load_2d(ad, &map_a, &full[s], k0, m0);
                } else if (p.a_grouped) {
                    tma_load_3d(ad, &map_a, &full[s], 0, k0, m0 / 32);
                } else {
                    for (int j = 0; j < BM / 32; ++j) tma_load_2d(ad + j * 4096, &map_a, &full[s], m0 + 32 * j, k0);
                }
                if (!B_MN) {
                    tma_load_2d(bd, &map_b, &full[s], k0, n0);
                } else if (p.b_grouped) {
                    tma_load_3d(bd, &map_b, &full[s], 0, k0, n0 / 32);
                } else {
                    for (int j = 0; j < BN / 32; ++j) tma_load_2d(bd + j * 4096, &map_b, &full[s], n0 + 32 * j, k0);
                }
            }
        }
    } else if (warp == 5) {
        // ---- MMA issue: whole warp in the loop, the elect.sync thread issues ----
        const bool issue = elect_one();
        const uint32_t idesc = idesc_tf32(BM, BN, A_MN, B_MN);
        bool ok = true;
        for (int it = 0; it < my_tiles && ok; ++it) {
            const int b = it & 1;
            if (it >= 2 && !mbar_wait_warp(&acc_empty[b], ((it >> 1) - 1) & 1, p.status, 134)) break;
            tc_fence_after_sync();
            const uint32_t acc = tmem_base + uint32_t(b) * BN;
            for (int i = 0; i < kblocks; ++i) {
                const int g = it * kblocks + i, s = g % STAGES;
                if (!mbar_wait_warp_ready(&full[s], (g / STAGES) & 1, p.status, 132)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t ad = smem_u32(smem + s * STAGE_BYTES), bd = ad + A_BYTES;
                if (issue) {
#pragma unroll
                    for (int j = 0; j < BK / 8; ++j) {
                        const uint64_t a_desc = A_MN ? smem_desc(ad + j * 1024, 4096, 512, kLayoutSw128Base32)
                                                     : smem_desc(ad + j * 32, 16, 1024, kLayoutSw128);
                        const uint64_t b_desc = B_MN ? smem_desc(bd + j * 1024, 4096, 512, kLayoutSw128Base32)
                                                     : smem_desc(bd + j * 32, 16, 1024, kLayoutSw128);
                        mma_tf32(acc, a_desc, b_desc, idesc, !(i == 0 && j == 0));
                    }
                    mma_commit(&empty[s]);
                    if (i == kblocks - 1) mma_commit(&acc_full[b]);
                }
                __syncwarp();
            }
        }
    } else if (warp < 4) {
        // ---- epilogue: thread = row of the tile; 32 columns at a time, one 128-byte line per thread ----
        const bool vec = (p.N & 3) == 0;
        for (int it = 0; it < my_tiles; ++it) {
            const int b = it & 1;
            if (!mbar_wait_warp(&acc_full[b], (it >> 1) & 1, p.status, 133)) break;
            tc_fence_after_sync();
            int mt, nt;
            tile_of(blockIdx.x + it * gridDim.x, p.m_tiles, p.n_tiles, &mt, &nt);
            const int row = mt * BM + warp * 32 + lane, n0 = nt * BN;
            float *dst_row = p.c + size_t(row < p.M ? row : 0) * p.N;
            const uint32_t acc = tmem_base + (uint32_t(warp * 32) << 16) + uint32_t(b) * BN;
            for (int c0 = 0; c0 < BN; c0 += 32) {
                const bool last_group = c0 + 32 >= BN || n0 + c0 + 32 >= p.N;
                float v[32];
                tmem_ld_32x32(acc + c0, v);
                if (last_group) {
                    // everything this tile needs from the accumulator is in registers now
                    tc_fence_before_sync();
                    mbar_arrive_warp(&acc_empty[b]);
                }
                if (row < p.M) {
                    float *dst = dst_row + n0 + c0;
                    if (vec && n0 + c0 + 32 <= p.N) {
                        float4 *d4 = reinterpret_cast<float4 *>(dst);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            float4 o = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                            if (p.accumulate) {
                                const float4 old = d4[i];
                                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                            }
                            d4[i] = o;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (n0 + c0 + i < p.N) dst[i] = p.accumulate ? dst[i] + v[i] : v[i];
                    }
                }
                if (last_group) break;
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 5) tmem_dealloc(tmem_base, 512);
}

// ---- the same on pairs of thread blocks: 256 x 256 tiles ---------------------------------------------
// In the kernel above a stage's bytes cross the SM's shared memory twice, written by TMA and read by the MMAs
// (12 KiB each per 128 x 256 x 8 MMA), and the k-loop runs at about 210 clocks per MMA against the pipe's 128.
// With cta_group::2 one MMA spans two SMs: each block supplies its own 128 rows of A and HALF of the 256
// columns of B, so a block moves 8 KiB in and 8 KiB out per MMA for the same tensor work.  Each block's tensor
// memory holds its 128 rows of the result (two 256-column accumulators, alternating between tiles).
//
// Roles per block as above (warps 0-3 epilogue, warp 4 TMA, warp 5 MMA issue in the leader only).  Across the
// pair: both blocks' loads complete on the LEADER's full barrier, the leader's commits release a stage and
// publish an accumulator on both blocks' barriers, and both blocks' epilogue warps free an accumulator on the
// leader's barrier.  Every wait is bounded; both blocks always reach the cluster barrier at the end.
constexpr int PAIR_STAGES = 6, BH = BN / 2;
constexpr int PAIR_B_BYTES = BH * BK * 4, PAIR_STAGE_BYTES = A_BYTES + PAIR_B_BYTES;
constexpr size_t PAIR_SMEM = size_t(PAIR_STAGES) * PAIR_STAGE_BYTES + 1024;

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(192, 1)
umma_gemm_wide_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                           const __grid_constant__ WideParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full[PAIR_STAGES], empty[PAIR_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int kblocks = (p.K + BK - 1) / BK;
    const int total_tiles = p.m_tiles * p.n_tiles;  // m_tiles counts 256-row pair tiles here
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int my_tiles = (total_tiles - pair + pairs - 1) / pairs;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s) {
            mbar_init(&full[s], 1);    // the leader's: its own expect_tx arrival, both blocks' bytes
            mbar_init(&empty[s], 1);   // each block's own copy, released by the leader's commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);   // each block's own copy
            mbar_init(&acc_empty[b], 8);  // the leader's: four epilogue warps of each block
        }
        mbar_init_fence();
    }
    if (warp == 5) {
        tmem_alloc_pair(&tmem_slot, 512);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // both blocks' barriers exist before anything is signalled across the pair
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;

    if (warp == 4 && lane == 0) {
        // ---- TMA producer of this block's rows of A and half of B; bytes are counted on the leader's barrier ----
        bool ok = true;
        for (int it = 0; it < my_tiles && ok; ++it) {
            int mt, nt;
            tile_of(pair + it * pairs, p.m_tiles, p.n_tiles, &mt, &nt);
            const int m0 = (2 * mt + (int)rank) * BM, nb0 = nt * BN + (int)rank * BH;
            for (int i = 0; i < kblocks; ++i) {
                const int g = it * kblocks + i, s = g % PAIR_STAGES;
                if (g >= PAIR_STAGES && !mbar_wait(&empty[s], ((g / PAIR_STAGES) - 1) & 1, p.status, 141)) { ok = false; break; }
                if (leader) mbar_arrive_expect_tx(&full[s], 2 * PAIR_STAGE_BYTES);
                const uint32_t bar = map_to_rank(&full[s], 0);
                unsigned char *ad = smem + s * PAIR_STAGE_BYTES, *bd = ad + A_BYTES;
                const int k0 = i * BK;
                if (!A_MN) {
                    tma_load_2d_pair(ad, &map_a, bar, k0, m0);
                } else if (p.a_grouped) {
                    tma_load_3d_pair(ad, &map_a, bar, 0, k0, m0 / 32);
                } else {
                    for (int j = 0; j < BM / 32; ++j) tma_load_2d_pair(ad + j * 4096, &map_a, bar, m0 + 32 * j, k0);
                }
                if (!B_MN) {
                    tma_load_2d_pair(bd, &map_b, bar, k0, nb0);
                } else if (p.b_grouped) {
                    tma_load_3d_pair(bd, &map_b, bar, 0, k0, nb0 / 32);
                } else {
                    for (int j = 0; j < BH / 32; ++j) tma_load_2d_pair(bd + j * 4096, &map_b, bar, nb0 + 32 * j, k0);
                }
            }
        }
    } else if (warp == 5 && leader) {
        // ---- MMA issue for the pair: whole warp in the loop, the elect.sync thread issues ----
        const bool issue = elect_one();
        const uint32_t idesc = idesc_tf32(2 * BM, BN, A_MN, B_MN);
        bool ok = true;
        for (int it = 0; it < my_tiles && ok; ++it) {
            const int b = it & 1;
            if (it >= 2 && !mbar_wait_warp(&acc_empty[b], ((it >> 1) - 1) & 1, p.status, 144)) break;
            tc_fence_after_sync();
            const uint32_t acc = tmem_base + uint32_t(b) * BN;
            for (int i = 0; i < kblocks; ++i) {
                const int g = it * kblocks + i, s = g % PAIR_STAGES;
                if (!mbar_wait_warp_ready(&full[s], (g / PAIR_STAGES) & 1, p.status, 142)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t ad = smem_u32(smem + s * PAIR_STAGE_BYTES), bd = ad + A_BYTES;
                if (issue) {
#pragma unroll
                    for (int j = 0; j < BK / 8; ++j) {
                        const uint64_t a_desc = A_MN ? smem_desc(ad + j * 1024, 4096, 512, kLayoutSw128Base32)
                                                     : smem_desc(ad + j * 32, 16, 1024, kLayoutSw128);
                        const uint64_t b_desc = B_MN ? smem_desc(bd + j * 1024, 4096, 512, kLayoutSw128Base32)
                                                     : smem_desc(bd + j * 32, 16, 1024, kLayoutSw128);
                        mma_tf32_pair(acc, a_desc, b_desc, idesc, !(i == 0 && j == 0));
                    }
                    // every release goes to this block's barrier and to the peer's copy of it
                    mma_commit_pair(smem_u32(&empty[s]));
                    mma_commit_pair(map_to_rank(&empty[s], 1));
                    if (i == kblocks - 1) {
                        mma_commit_pair(smem_u32(&acc_full[b]));
                        mma_commit_pair(map_to_rank(&acc_full[b], 1));
                    }
                }
                __syncwarp();
            }
        }
    } else if (warp < 4) {
        // ---- epilogue: thread = row of this block's half of the tile ----
        const bool vec = (p.N & 3) == 0;
        for (int it = 0; it < my_tiles; ++it) {
            const int b = it & 1;
            if (!mbar_wait_warp(&acc_full[b], (it >> 1) & 1, p.status, 143)) break;
            tc_fence_after_sync();
            int mt, nt;
            tile_of(pair + it * pairs, p.m_tiles, p.n_tiles, &mt, &nt);
            const int row = (2 * mt + (int)rank) * BM + warp * 32 + lane, n0 = nt * BN;
            float *dst_row = p.c + size_t(row < p.M ? row : 0) * p.N;
            const uint32_t acc = tmem_base + (uint32_t(warp * 32) << 16) + uint32_t(b) * BN;
            for (int c0 = 0; c0 < BN; c0 += 32) {
                const bool last_group = c0 + 32 >= BN || n0 + c0 + 32 >= p.N;
                float v[32];
                tmem_ld_32x32(acc + c0, v);
                if (last_group) {
                    // everything this tile needs from the accumulator is in registers now
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) {
                        if (leader) mbar_arrive(&acc_empty[b]);
                        else mbar_arrive_cluster(map_to_rank(&acc_empty[b], 0));
                    }
                }
                if (row < p.M) {
                    float *dst = dst_row + n0 + c0;
                    if (vec && n0 + c0 + 32 <= p.N) {
                        float4 *d4 = reinterpret_cast<float4 *>(dst);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            float4 o = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                            if (p.accumulate) {
                                const float4 old = d4[i];
                                o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                            }
                            d4[i] = o;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (n0 + c0 + i < p.N) dst[i] = p.accumulate ? dst[i] + v[i] : v[i];
                    }
                }
                if (last_group) break;
            }
        }
    }
    // Neither block leaves (or gives its tensor memory back) while the other may still signal its barriers,
    // read its half of B or hold accumulators: every path above ends here.
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    if (warp == 5) tmem_dealloc_pair(tmem_base, 512);
}

// ---- 3xTF32 on pairs of thread blocks, both operands and their lo halves from shared memory ---------------
// The split-precision kernels that build A in tensor memory (umma_gemm.cu, umma_gemm_pair.cu) are paced by
// their builder warps.  Here the lo halves of BOTH operands are written once by a streaming pre-pass
// (lo = v - trunc_tf32(v); the tensor core truncates the raw values to the hi parts itself) and a stage is
// A hi | A lo | B-half hi | B-half lo (4 x 16 KiB, three stages); the leader issues lo*hi + hi*lo + hi*hi for
// the pair.  Tensor memory holds exactly two 256-column accumulators, which take turns: one receives DRAIN3
// k-blocks (16 x 12 = 192 accumulations: the tensor core's f32 accumulation loses ~3e-8 per step, so chains
// stay short) while eight epilogue warps (lane quarter = warp % 4, column half = warp / 4) fold the other
// into 128 f32 running sums per thread.  Warp 8 issues the TMA loads, warp 9 the MMAs (leader only).
constexpr int DRAIN3 = 16, W3_STAGES = 3;
constexpr int W3_STAGE_BYTES = 2 * A_BYTES + 2 * PAIR_B_BYTES;   // 64 KiB
constexpr size_t W3_SMEM = size_t(W3_STAGES) * W3_STAGE_BYTES + 1024;

__global__ void __launch_bounds__(256) split_lo_wide_kernel(const float *__restrict__ x, float *__restrict__ lo, size_t count) {
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
        const float v = x[i];
        lo[i] = v - __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
    }
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(320, 1)
umma_gemm_wide3_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_a_lo,
                            const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_b_lo,
                            const __grid_constant__ WideParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t full[W3_STAGES], empty[W3_STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int kblocks = (p.K + BK - 1) / BK;
    const int batches = (kblocks + DRAIN3 - 1) / DRAIN3;
    const int total_tiles = p.m_tiles * p.n_tiles;  // m_tiles counts 256-row pair tiles
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int my_tiles = (total_tiles - pair + pairs - 1) / pairs;

    if (threadIdx.x == 0) {
        for (int s = 0; s < W3_STAGES; ++s) {
            mbar_init(&full[s], 1);    // the leader's: its own expect_tx arrival, both blocks' bytes
            mbar_init(&empty[s], 1);   // each block's own copy, released by the leader's commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);    // each block's own copy
            mbar_init(&acc_empty[b], 16);  // the leader's: eight epilogue warps of each block
        }
        mbar_init_fence();
    }
    if (warp == 9) {
        tmem_alloc_pair(&tmem_slot, 512);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // both blocks' barriers exist before anything is signalled across the pair
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;

    if (warp == 8 && lane == 0) {
        // ---- TMA producer: this block's rows of A and half of B, hi and lo ----
        bool ok = true;
        for (int it = 0; it < my_tiles && ok; ++it) {
            int mt, nt;
            tile_of(pair + it * pairs, p.m_tiles, p.n_tiles, &mt, &nt);
            const int m0 = (2 * mt + (int)rank) * BM, nb0 = nt * BN + (int)rank * BH;
            for (int i = 0; i < kblocks; ++i) {
                const int g = it * kblocks + i, s = g % W3_STAGES;
                if (g >= W3_STAGES && !mbar_wait(&empty[s], ((g / W3_STAGES) - 1) & 1, p.status, 151)) { ok = false; break; }
                if (leader) mbar_arrive_expect_tx(&full[s], 2 * W3_STAGE_BYTES);
                const uint32_t bar = map_to_rank(&full[s], 0);
                unsigned char *st = smem + s * W3_STAGE_BYTES;
                const int k0 = i * BK;
                for (int part = 0; part < 2; ++part) {
                    const CUtensorMap *ma = part ? &map_a_lo : &map_a;
                    const CUtensorMap *mb = part ? &map_b_lo : &map_b;
                    unsigned char *ad = st + part * A_BYTES, *bd = st + 2 * A_BYTES + part * PAIR_B_BYTES;
                    if (!A_MN) {
                        tma_load_2d_pair(ad, ma, bar, k0, m0);
                    } else if (p.a_grouped) {
                        tma_load_3d_pair(ad, ma, bar, 0, k0, m0 / 32);
                    } else {
                        for (int j = 0; j < BM / 32; ++j) tma_load_2d_pair(ad + j * 4096, ma, bar, m0 + 32 * j, k0);
                    }
                    if (!B_MN) {
                        tma_load_2d_pair(bd, mb, bar, k0, nb0);
                    } else if (p.b_grouped) {
                        tma_load_3d_pair(bd, mb, bar, 0, k0, nb0 / 32);
                    } else {
                        for (int j = 0; j < BH / 32; ++j) tma_load_2d_pair(bd + j * 4096, mb, bar, nb0 + 32 * j, k0);
                    }
                }
            }
        }
    } else if (warp == 9 && leader) {
        // ---- MMA issue for the pair: whole warp in the loop, the elect.sync thread issues ----
        const bool issue = elect_one();
        const uint32_t idesc = idesc_tf32(2 * BM, BN, A_MN, B_MN);
        bool ok = true;
        int q = 0;  // accumulator hand-overs so far (batches of all tiles)
        for (int it = 0; it < my_tiles && ok; ++it) {
            for (int bi = 0; bi < batches && ok; ++bi, ++q) {
                const int b = q & 1;
                if (q >= 2 && !mbar_wait_warp(&acc_empty[b], ((q >> 1) - 1) & 1, p.status, 152)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t acc = tmem_base + uint32_t(b) * BN;
                const int i_end = (bi + 1) * DRAIN3 < kblocks ? (bi + 1) * DRAIN3 : kblocks;
                for (int i = bi * DRAIN3; i < i_end; ++i) {
                    const int g = it * kblocks + i, s = g % W3_STAGES;
                    if (!mbar_wait_warp_ready(&full[s], (g / W3_STAGES) & 1, p.status, 153)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t ah = smem_u32(smem + s * W3_STAGE_BYTES), al = ah + A_BYTES;
                    const uint32_t bh = ah + 2 * A_BYTES, bl = bh + PAIR_B_BYTES;
                    const bool first = i == bi * DRAIN3;
                    if (issue) {
#pragma unroll
                        for (int j = 0; j < BK / 8; ++j) {
                            const uint32_t ao = A_MN ? j * 1024 : j * 32, bo = B_MN ? j * 1024 : j * 32;
                            const uint64_t a_hi = A_MN ? smem_desc(ah + ao, 4096, 512, kLayoutSw128Base32) : smem_desc(ah + ao, 16, 1024, kLayoutSw128);
                            const uint64_t a_lo = A_MN ? smem_desc(al + ao, 4096, 512, kLayoutSw128Base32) : smem_desc(al + ao, 16, 1024, kLayoutSw128);
                            const uint64_t b_hi = B_MN ? smem_desc(bh + bo, 4096, 512, kLayoutSw128Base32) : smem_desc(bh + bo, 16, 1024, kLayoutSw128);
                            const uint64_t b_lo = B_MN ? smem_desc(bl + bo, 4096, 512, kLayoutSw128Base32) : smem_desc(bl + bo, 16, 1024, kLayoutSw128);
                            mma_tf32_pair(acc, a_lo, b_hi, idesc, !(first && j == 0));
                            mma_tf32_pair(acc, a_hi, b_lo, idesc, true);
                            mma_tf32_pair(acc, a_hi, b_hi, idesc, true);
                        }
                        // every release goes to this block's barrier and to the peer's copy of it
                        mma_commit_pair(smem_u32(&empty[s]));
                        mma_commit_pair(map_to_rank(&empty[s], 1));
                        if (i == i_end - 1) {
                            mma_commit_pair(smem_u32(&acc_full[b]));
                            mma_commit_pair(map_to_rank(&acc_full[b], 1));
                        }
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp < 8) {
        // ---- drains and epilogue: thread = row of this block's half of the tile x column half ----
        const int quarter = warp & 3, half = warp >> 2;
        const bool vec = (p.N & 3) == 0;
        int q = 0;
        bool alive = true;
        for (int it = 0; it < my_tiles && alive; ++it) {
            float run[128];
#pragma unroll
            for (int i = 0; i < 128; ++i) run[i] = 0.f;
            for (int bi = 0; bi < batches; ++bi, ++q) {
                const int b = q & 1;
                if (!mbar_wait_warp(&acc_full[b], (q >> 1) & 1, p.status, 154)) { alive = false; break; }
                tc_fence_after_sync();
                const uint32_t acc = tmem_base + (uint32_t(quarter * 32) << 16) + uint32_t(b) * BN + uint32_t(half) * 128;
#pragma unroll
                for (int c0 = 0; c0 < 128; c0 += 32) {
                    float t[32];
                    tmem_ld_32x32(acc + c0, t);
#pragma unroll
                    for (int i = 0; i < 32; ++i) run[c0 + i] += t[i];
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if (leader) mbar_arrive(&acc_empty[b]);
                    else mbar_arrive_cluster(map_to_rank(&acc_empty[b], 0));
                }
            }
            if (!alive) break;
            int mt, nt;
            tile_of(pair + it * pairs, p.m_tiles, p.n_tiles, &mt, &nt);
            const int row = (2 * mt + (int)rank) * BM + quarter * 32 + lane, n0 = nt * BN + half * 128;
            if (row < p.M) {
                float *dst = p.c + size_t(row) * p.N + n0;
                if (vec && n0 + 128 <= p.N) {
                    float4 *d4 = reinterpret_cast<float4 *>(dst);
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        float4 o = make_float4(run[4 * i], run[4 * i + 1], run[4 * i + 2], run[4 * i + 3]);
                        if (p.accumulate) {
                            const float4 old = d4[i];
                            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                        }
                        d4[i] = o;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 128; ++i)
                        if (n0 + i < p.N) dst[i] = p.accumulate ? dst[i] + run[i] : run[i];
                }
            }
        }
    }
    // Neither block leaves (or gives its tensor memory back) while the other may still signal its barriers,
    // read its half of B or hold accumulators: every path above ends here.
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    if (warp == 9) tmem_dealloc_pair(tmem_base, 512);
}

bool wide_map(CUtensorMap *map, const float *base, bool mn_major, size_t mn_extent, size_t k_extent, uint32_t tile,
              int *grouped) {
    *grouped = 0;
    if (!mn_major) {
        const uint64_t dims[2] = {k_extent, mn_extent}, strides[2] = {1, k_extent};
        const uint32_t box[2] = {BK, tile};
        return katsu_make_tensor_map(map, base, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    }
    if ((mn_extent & 31) == 0) {
        const uint64_t dims[3] = {32, k_extent, mn_extent / 32}, strides[3] = {1, mn_extent, 32};
        const uint32_t box[3] = {32, BK, tile / 32};
        if (katsu_make_tensor_map(map, base, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B)) {
            *grouped = 1;
            return true;
        }
    }
    const uint64_t dims[2] = {mn_extent, k_extent}, strides[2] = {1, mn_extent};
    const uint32_t box[2] = {32, BK};
    return katsu_make_tensor_map(map, base, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
}

template <bool A_MN, bool B_MN>
int32_t launch_wide(katsu_cuda_ctx *ctx, const float *a, const float *b, float *c, size_t M, size_t N, size_t K,
                    int accumulate) {
    WideParams p;
    CUtensorMap map_a, map_b;
    if (!wide_map(&map_a, a, A_MN, M, K, BM, &p.a_grouped) || !wide_map(&map_b, b, B_MN, N, K, BN, &p.b_grouped))
        return katsu_set_error(KATSU_ERR_CUDA, "cuTensorMapEncodeTiled failed for a matmul operand");
    p.c = c;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.m_tiles = (int)katsu_div_up(M, (size_t)BM);
    p.n_tiles = (int)katsu_div_up(N, (size_t)BN);
    p.accumulate = accumulate;
    p.status = ctx->status;
    auto kernel = umma_gemm_wide_kernel<A_MN, B_MN>;
    KATSU_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
    size_t grid = size_t(p.m_tiles) * p.n_tiles;
    if (grid > (size_t)ctx->num_sms) grid = (size_t)ctx->num_sms;
    KATSU_LAUNCH(ctx, kernel, (unsigned)grid, 192, SMEM, map_a, map_b, p);
    return KATSU_OK;
}

template <bool A_MN, bool B_MN>
int32_t launch_wide_pair(katsu_cuda_ctx *ctx, const float *a, const float *b, float *c, size_t M, size_t N, size_t K,
                         int accumulate) {
    WideParams p;
    CUtensorMap map_a, map_b;
    if (!wide_map(&map_a, a, A_MN, M, K, BM, &p.a_grouped) || !wide_map(&map_b, b, B_MN, N, K, BH, &p.b_grouped))
        return katsu_set_error(KATSU_ERR_CUDA, "cuTensorMapEncodeTiled failed for a matmul operand");
    p.c = c;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.m_tiles = (int)katsu_div_up(M, (size_t)(2 * BM));
    p.n_tiles = (int)katsu_div_up(N, (size_t)BN);
    p.accumulate = accumulate;
    p.status = ctx->status;
    auto kernel = umma_gemm_wide_pair_kernel<A_MN, B_MN>;
    KATSU_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PAIR_SMEM));
    size_t pairs = size_t(p.m_tiles) * p.n_tiles;
    if (pairs > (size_t)ctx->num_sms / 2) pairs = (size_t)ctx->num_sms / 2;
    cudaLaunchConfig_t config;
    memset(&config, 0, sizeof(config));
    config.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
    config.blockDim = dim3(192, 1, 1);
    config.dynamicSmemBytes = PAIR_SMEM;
    config.stream = ctx->stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = 2;
    attribute.val.clusterDim.y = 1;
    attribute.val.clusterDim.z = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    cudaError_t err = cudaLaunchKernelEx(&config, kernel, map_a, map_b, p);
    ctx->launches += 1;
    if (err != cudaSuccess)
        return katsu_set_error(KATSU_ERR_CUDA, "pair GEMM launch failed: %s", cudaGetErrorString(err));
    return KATSU_OK;
}

template <bool A_MN, bool B_MN>
int32_t launch_wide3_pair(katsu_cuda_ctx *ctx, const float *a, const float *b, float *c, size_t M, size_t N, size_t K,
                          int accumulate) {
    const size_t a_count = M * K, b_count = K * N;
    float *scratch = nullptr;
    KATSU_TRY(katsu_scratch(ctx, a_count + b_count + 128, &scratch));
    float *a_lo = scratch, *b_lo = scratch + (a_count + 63) / 64 * 64;
    const unsigned split_blocks = (unsigned)(size_t(ctx->num_sms) * 8);
    KATSU_LAUNCH(ctx, split_lo_wide_kernel, split_blocks, 256, 0, a, a_lo, a_count);
    KATSU_LAUNCH(ctx, split_lo_wide_kernel, split_blocks, 256, 0, b, b_lo, b_count);
    WideParams p;
    CUtensorMap map_a, map_a_lo, map_b, map_b_lo;
    int a_lo_grouped = 0, b_lo_grouped = 0;
    if (!wide_map(&map_a, a, A_MN, M, K, BM, &p.a_grouped) || !wide_map(&map_a_lo, a_lo, A_MN, M, K, BM, &a_lo_grouped) ||
        !wide_map(&map_b, b, B_MN, N, K, BH, &p.b_grouped) || !wide_map(&map_b_lo, b_lo, B_MN, N, K, BH, &b_lo_grouped) ||
        a_lo_grouped != p.a_grouped || b_lo_grouped != p.b_grouped)
        return katsu_set_error(KATSU_ERR_CUDA, "cuTensorMapEncodeTiled failed for a matmul operand");
    p.c = c;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.m_tiles = (int)katsu_div_up(M, (size_t)(2 * BM));
    p.n_tiles = (int)katsu_div_up(N, (size_t)BN);
    p.accumulate = accumulate;
    p.status = ctx->status;
    auto kernel = umma_gemm_wide3_pair_kernel<A_MN, B_MN>;
    KATSU_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)W3_SMEM));
    size_t pairs = size_t(p.m_tiles) * p.n_tiles;
    if (pairs > (size_t)ctx->num_sms / 2) pairs = (size_t)ctx->num_sms / 2;
    cudaLaunchConfig_t config;
    memset(&config, 0, sizeof(config));
    config.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
    config.blockDim = dim3(320, 1, 1);
    config.dynamicSmemBytes = W3_SMEM;
    config.stream = ctx->stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = 2;
    attribute.val.clusterDim.y = 1;
    attribute.val.clusterDim.z = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    cudaError_t err = cudaLaunchKernelEx(&config, kernel, map_a, map_a_lo, map_b, map_b_lo, p);
    ctx->launches += 1;
    if (err != cudaSuccess)
        return katsu_set_error(KATSU_ERR_CUDA, "pair GEMM launch failed: %s", cudaGetErrorString(err));
    return KATSU_OK;
}

}  // namespace

// C[M,N] (+)= A * B in single-pass TF32 with 128 x 256 tiles.  *handled = 0 unless the context is in
// KATSU_MODE_TF32 and the shape gives at least one tile per two SMs (smaller shapes need the K split of the
// 128 x 128 kernel to fill the GPU).  Alignment has been checked by the caller (katsu_umma_gemm).
int32_t katsu_umma_gemm_wide(katsu_cuda_ctx *ctx, const float *a, const float *b, float *c, size_t M, size_t N,
                             size_t K, bool a_mn, bool b_mn, int accumulate, int *handled) {
    *handled = 0;
    if (ctx->precision == KATSU_MODE_3XTF32) {
        // split precision: only the pair form, and only with a 256 x 256 tile for every pair of SMs
        const size_t tiles3 = katsu_div_up(M, (size_t)(2 * BM)) * katsu_div_up(N, (size_t)BN);
        if (M < 256 || N < 256 || K < 32 || tiles3 < (size_t)ctx->num_sms / 2 || tiles3 > 0x3fffffffu) return KATSU_OK;
        if (katsu_div_up(K, (size_t)BK) * tiles3 > 0x7fffffffu) return KATSU_OK;
        // room for the lo halves of both operands; without it the tensor-memory pair kernel (which needs b's
        // only) takes the shape
        float *room = nullptr;
        if (katsu_scratch(ctx, M * K + K * N + 128, &room) != KATSU_OK) {
            cudaGetLastError();
            return KATSU_OK;
        }
        *handled = 1;
        if (!a_mn && !b_mn) return launch_wide3_pair<false, false>(ctx, a, b, c, M, N, K, accumulate);
        if (!a_mn && b_mn) return launch_wide3_pair<false, true>(ctx, a, b, c, M, N, K, accumulate);
        if (a_mn && !b_mn) return launch_wide3_pair<true, false>(ctx, a, b, c, M, N, K, accumulate);
        return launch_wide3_pair<true, true>(ctx, a, b, c, M, N, K, accumulate);
    }
    if (ctx->precision != KATSU_MODE_TF32) return KATSU_OK;
    if (M < 128 || N < 256 || K < 32) return KATSU_OK;
    // the whole contraction accumulates in tensor memory, which loses ~3e-8 per accumulation step: measured
    // 1.17e-3 at K = 200 000 against 7.7e-4 for the kernel that drains every 32 k-blocks (bar of this mode:
    // 2e-3).  Up to 2^16 columns the loss stays a small part of the mode's own rounding; longer ones go there.
    if (K > (size_t(1) << 16)) return KATSU_OK;
    const size_t tiles = katsu_div_up(M, (size_t)BM) * katsu_div_up(N, (size_t)BN);
    if (tiles * 2 < (size_t)ctx->num_sms || tiles > 0x3fffffffu) return KATSU_OK;
    if (katsu_div_up(K, (size_t)BK) * tiles > 0x7fffffffu) return KATSU_OK;  // the ring counter is an int
    *handled = 1;
    // tall enough for 256-row tiles on pairs of thread blocks, and enough of them for every pair of SMs
    const size_t pair_tiles = katsu_div_up(M, (size_t)(2 * BM)) * katsu_div_up(N, (size_t)BN);
    if (M >= 256 && pair_tiles * 2 >= (size_t)ctx->num_sms / 2) {
        if (!a_mn && !b_mn) return launch_wide_pair<false, false>(ctx, a, b, c, M, N, K, accumulate);
        if (!a_mn && b_mn) return launch_wide_pair<false, true>(ctx, a, b, c, M, N, K, accumulate);
        if (a_mn && !b_mn) return launch_wide_pair<true, false>(ctx, a, b, c, M, N, K, accumulate);
        return launch_wide_pair<true, true>(ctx, a, b, c, M, N, K, accumulate);
    }
    if (!a_mn && !b_mn) return launch_wide<false, false>(ctx, a, b, c, M, N, K, accumulate);
    if (!a_mn && b_mn) return launch_wide<false, true>(ctx, a, b, c, M, N, K, accumulate);
    if (a_mn && !b_mn) return launch_wide<true, false>(ctx, a, b, c, M, N, K, accumulate);
    return launch_wide<true, true>(ctx, a, b, c, M, N, K, accumulate);
}
