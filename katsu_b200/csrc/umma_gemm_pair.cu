// Tensor-core GEMM on CTA pairs (tcgen05 cta_group::2) for Tensor::matmul and its VJP
// (crates/katsu-core/src/tensor.rs:264-273, 418-445): a 256 x 128 tile per pair of thread blocks.
//
// Why pairs.  The single-block kernel (umma_gemm.cu) is bound by operand delivery into shared memory:
// its 128 x 128 tile pulls 48 KiB per 32-wide k-block in 3xTF32 (raw A, B hi and lo) and the time per
// k-block follows the bytes, not the tensor pipe (measured: about 290 clk + 18.75 clk per KiB).  With
// cta_group::2 one MMA spans two SMs: each block supplies its own 128 rows of A and HALF of the 128
// columns of B, and each block's tensor memory receives its 128 rows of the result.  Every block then
// loads 16 KiB of A and 2 x 8 KiB of B per k-block, 32 KiB instead of 48, for the same tensor work.
// No load is shared between blocks by the copy engine: each block issues its own plain TMA loads
// (the cta_group::2 form only lets a block's copy signal the pair leader's barrier).
//
// Structure per block (same roles as umma_gemm.cu): warps 0-3 drain accumulators and write the result,
// warps 4-7 build A in tensor memory (hi | lo), warp 8 loads A, warp 9 issues MMAs (leader block only),
// warp 10 loads this block's half of B.  Across the pair: the builders and drain warps of both blocks
// arrive on the LEADER's barriers (remote mbarrier arrive), both blocks' B copies complete on the
// leader's barrier, and the leader commits every stage release to both blocks' barriers (two commits).
// Every wait is bounded; both blocks always reach the cluster barriers at the end, whatever gave up.
#include <string.h>

#include "common.cuh"
#include "sm100.cuh"
#include "sm100_pair.cuh"

using namespace sm100;

namespace {

constexpr int BM = 128;   // rows per block (256 per pair)
constexpr int BN = 128;   // tile columns
constexpr int BH = 64;    // B columns (tile N half) this block loads
constexpr int BK = 32;    // f32 per 128-byte swizzle row
constexpr int AS = 6, TS_MAX = 8;   // A slots in shared memory; stages (A in tensor memory + B slot) at most
constexpr int A_BYTES = BM * BK * 4;   // 16 KiB
constexpr int B_BYTES = BH * BK * 4;   // 8 KiB (hi) + 8 KiB (lo) per slot
constexpr int DRAIN = 32;              // k-blocks per accumulator batch (2 accumulators x 16 k-blocks x 32)
constexpr uint32_t A_COL0 = 2 * BN;    // TMEM: [2 accumulators x 128][TS A stages x {32 hi, 32 lo}]
constexpr int RASTER_W = 16;
// Two MMA-issue warps in the leader: warp 9 takes the even k-blocks (accumulator 0), warp 11 the odd ones
// (accumulator 1), so the waits, commits and address mapping of a k-block are spread over two threads.
constexpr int PAIR_THREADS = 12 * 32, TMA_A_WARP = 8, MMA_WARP = 9, TMA_B_WARP = 10, MMA_WARP2 = 11;

struct PairParams {
    float *c;          // output, or partial slabs [splits][M][N] when splits > 1
    int M, N, K;
    int m_pairs, n_tiles;
    int kblocks_per_split;
    int splits;
    int accumulate;    // only used when splits == 1
    int three_pass;
    int a_grouped, b_grouped;  // MN-major maps are 3-D {32, K, extent / 32}: one load per operand tile
    int *status;
};

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
umma_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const __grid_constant__ CUtensorMap map_b_lo, PairParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // stage_free[s] releases tensor-memory A stage s AND shared-memory B slot s together (TS == BS): one commit per
    // block instead of two, which matters to the one thread that issues everything for the pair
    __shared__ uint64_t a_full[AS], a_read[AS], b_full[TS_MAX], stage_free[TS_MAX], a_ready[TS_MAX], batch_done, drained;
    // Stages in flight: a 3xTF32 stage holds hi | lo (64 columns), four fit beside the accumulators; single-pass
    // TF32 needs hi only (32 columns), so eight do.  The ring's round trip crosses the pair twice (peer's arrival,
    // leader's commit), and it is the number of stages in flight that hides it.
    const int TS = p.three_pass ? 4 : 8;
    const uint32_t stage_cols = p.three_pass ? 64 : 32;
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    // Tile order: bands of RASTER_W column tiles, pair rows fastest inside a band (see umma_gemm.cu).
    int tile_mp, tile_n;
    {
        const int pair = blockIdx.x >> 1;
        const int band = pair / (RASTER_W * p.m_pairs), within = pair % (RASTER_W * p.m_pairs);
        const int width = (p.n_tiles - band * RASTER_W) < RASTER_W ? (p.n_tiles - band * RASTER_W) : RASTER_W;
        tile_n = band * RASTER_W + within % width;
        tile_mp = within / width;
    }
    const int m0 = (2 * tile_mp + (int)rank) * BM, n0 = tile_n * BN, nb0 = n0 + (int)rank * BH;
    const int kb_total = (p.K + BK - 1) / BK;
    const int kb_begin = int(blockIdx.z) * p.kblocks_per_split;
    int kb_end = kb_begin + p.kblocks_per_split;
    if (kb_end > kb_total) kb_end = kb_total;
    const int kblocks = kb_end > kb_begin ? kb_end - kb_begin : 0;
    const int batches = (kblocks + DRAIN - 1) / DRAIN;
    const int parts = p.three_pass ? 2 : 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < AS; ++s) {
            mbar_init(&a_full[s], 1);
            mbar_init(&a_read[s], 4);
        }
        for (int s = 0; s < TS_MAX; ++s) {
            mbar_init(&b_full[s], 1);   // the leader's: its own expect_tx arrival, both blocks' bytes
            mbar_init(&stage_free[s], 1);  // released by the leader's commit (to each block's own copy)
            mbar_init(&a_ready[s], 8);     // the leader's: four builder warps of each block
        }
        mbar_init(&batch_done, 2);      // one arrival per MMA-issue warp of the leader
        mbar_init(&drained, 8);         // the leader's: four drain warps of each block
        mbar_init_fence();
    }
    if (warp == MMA_WARP) {
        tmem_alloc_pair(&tmem_slot, 512);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // both blocks' barriers exist before anything is signalled across the pair
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;

    unsigned char *a_slots = smem, *b_slots = smem + AS * A_BYTES;
    if (warp == TMA_A_WARP && lane == 0) {
        // ---- TMA producer of this block's rows of A (all local) ----
        for (int i = 0; i < kblocks; ++i) {
            const int sa = i % AS;
            if (i >= AS && !mbar_wait(&a_read[sa], ((i / AS) - 1) & 1, p.status, 111)) break;
            mbar_arrive_expect_tx(&a_full[sa], A_BYTES);
            unsigned char *ad = a_slots + sa * A_BYTES;
            const int k0 = (kb_begin + i) * BK;
            if (!A_MN) {
                tma_load_2d(ad, &map_a, &a_full[sa], k0, m0);
            } else if (p.a_grouped) {
                tma_load_3d(ad, &map_a, &a_full[sa], 0, k0, m0 / 32);
            } else {
                for (int j = 0; j < BM / 32; ++j) tma_load_2d(ad + j * 4096, &map_a, &a_full[sa], m0 + 32 * j, k0);
            }
        }
    } else if (warp == TMA_B_WARP && lane == 0) {
        // ---- TMA producer of this block's half of B; the bytes are counted on the leader's barrier ----
        for (int i = 0; i < kblocks; ++i) {
            const int sb = i % TS;
            if (i >= TS && !mbar_wait(&stage_free[sb], ((i / TS) - 1) & 1, p.status, 117)) break;
            if (leader) mbar_arrive_expect_tx(&b_full[sb], 2 * parts * B_BYTES);
            const uint32_t bar = map_to_rank(&b_full[sb], 0);
            unsigned char *bd = b_slots + sb * 2 * B_BYTES;
            const int k0 = (kb_begin + i) * BK;
            for (int part = 0; part < parts; ++part) {
                const CUtensorMap *mb = part ? &map_b_lo : &map_b;
                if (!B_MN) {
                    tma_load_2d_pair(bd + part * B_BYTES, mb, bar, k0, nb0);
                } else if (p.b_grouped) {
                    tma_load_3d_pair(bd + part * B_BYTES, mb, bar, 0, k0, nb0 / 32);
                } else {
                    for (int j = 0; j < BH / 32; ++j) tma_load_2d_pair(bd + part * B_BYTES + j * 4096, mb, bar, nb0 + 32 * j, k0);
                }
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // ---- A builders: thread = one row of this block's tile; hi goes in raw (the tensor core truncates) ----
        const int quarter = warp & 3, row = quarter * 32 + lane;
        const uint32_t lane_addr = tmem_base + (uint32_t(quarter * 32) << 16) + A_COL0;
        for (int i = 0; i < kblocks; ++i) {
            const int sa = i % AS, s = i % TS;
            if (!mbar_wait_warp_ready(&a_full[sa], (i / AS) & 1, p.status, 114)) break;
            const unsigned char *ad = a_slots + sa * A_BYTES;
            float v[32];
            if (!A_MN) {
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const float4 q = ld_shared_v4(ad + row * 128 + ((c ^ (row & 7)) << 4));
                    v[4 * c] = q.x; v[4 * c + 1] = q.y; v[4 * c + 2] = q.z; v[4 * c + 3] = q.w;
                }
            } else {
#pragma unroll
                for (int k = 0; k < 32; ++k) v[k] = ld_shared_f32(ad + quarter * 4096 + k * 128 + lane * 4);
            }
            fence_proxy_async_smem();  // ordinary reads of the slot before its TMA refill
            mbar_arrive_warp(&a_read[sa]);
            if (i >= TS && !mbar_wait_warp_ready(&stage_free[s], ((i / TS) - 1) & 1, p.status, 115)) break;
            tc_fence_after_sync();
            tmem_st_32x32(lane_addr + uint32_t(s) * stage_cols, v);
            if (p.three_pass) {
#pragma unroll
                for (int t = 0; t < 32; ++t) v[t] -= __uint_as_float(__float_as_uint(v[t]) & 0xFFFFE000u);
                tmem_st_32x32(lane_addr + uint32_t(s) * stage_cols + 32, v);
            }
            tmem_st_wait();  // warp-wide: every lane's stores have landed when it returns
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                if (leader)
                    mbar_arrive(&a_ready[s]);
                else
                    mbar_arrive_cluster(map_to_rank(&a_ready[s], 0));
            }
        }
    } else if ((warp == MMA_WARP || warp == MMA_WARP2) && leader) {
        // ---- MMA issue for the pair: the whole warp runs the loop, the thread chosen by elect.sync issues ----
        const int mine = warp == MMA_WARP ? 0 : 1;  // parity of the k-blocks (and the accumulator) this warp owns
        const bool issue = elect_one();
        const uint32_t idesc = idesc_tf32(2 * BM, BN, false, B_MN);
        const uint32_t peer = 1;
        bool ok = true;
        for (int b = 0; b < batches && ok; ++b) {
            // both blocks have folded the previous batch's accumulators into registers
            if (b > 0 && !mbar_wait_warp(&drained, (b - 1) & 1, p.status, 116)) break;
            tc_fence_after_sync();
            const int i_end = (b + 1) * DRAIN < kblocks ? (b + 1) * DRAIN : kblocks;
            // last k-block of this batch that is this warp's; none when the batch is one k-block of the other parity
            const int i_last = ((i_end - 1) & 1) == mine ? i_end - 1 : i_end - 2;
            if (i_last < b * DRAIN) {
                if (lane == 0) {
                    mbar_arrive(&batch_done);
                    mbar_arrive_cluster(map_to_rank(&batch_done, peer));
                }
                __syncwarp();
                continue;
            }
            for (int i = b * DRAIN + mine; i < i_end; i += 2) {
                const int s = i % TS, sb = s;
                if (!mbar_wait_warp_ready(&a_ready[s], (i / TS) & 1, p.status, 112)) { ok = false; break; }
                if (!mbar_wait_warp_ready(&b_full[sb], (i / TS) & 1, p.status, 118)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t bd = smem_u32(b_slots + sb * 2 * B_BYTES);
                const int li = i - b * DRAIN;
                const uint32_t acc = tmem_base + uint32_t(li & 1) * BN;
                const uint32_t a_hi = tmem_base + A_COL0 + uint32_t(s) * stage_cols, a_lo = a_hi + 32;
                if (issue) {
#pragma unroll
                    for (int j = 0; j < BK / 8; ++j) {
                        const uint32_t b_off = B_MN ? j * 1024 : j * 32;
                        const uint64_t b_hi = B_MN ? smem_desc(bd + b_off, 4096, 512, kLayoutSw128Base32)
                                                   : smem_desc(bd + b_off, 16, 1024, kLayoutSw128);
                        const bool acc_flag = !(li < 2 && j == 0);
                        if (p.three_pass) {
                            const uint64_t b_lo = B_MN ? smem_desc(bd + B_BYTES + b_off, 4096, 512, kLayoutSw128Base32)
                                                       : smem_desc(bd + B_BYTES + b_off, 16, 1024, kLayoutSw128);
                            mma_tf32_ts_pair(acc, a_lo + 8 * j, b_hi, idesc, acc_flag);
                            mma_tf32_ts_pair(acc, a_hi + 8 * j, b_lo, idesc, true);
                            mma_tf32_ts_pair(acc, a_hi + 8 * j, b_hi, idesc, true);
                        } else {
                            mma_tf32_ts_pair(acc, a_hi + 8 * j, b_hi, idesc, acc_flag);
                        }
                    }
                    // every release goes to this block's barrier and to the peer's copy of it
                    mma_commit_pair(smem_u32(&stage_free[s]));
                    mma_commit_pair(map_to_rank(&stage_free[s], peer));
                    if (i == i_last) {
                        mma_commit_pair(smem_u32(&batch_done));
                        mma_commit_pair(map_to_rank(&batch_done, peer));
                    }
                }
                __syncwarp();
            }
        }
    } else if (warp < 4) {
        // ---- drains and epilogue: warp w owns rows 32w .. 32w+31 of this block's tile ----
        float run[BN];
#pragma unroll
        for (int i = 0; i < BN; ++i) run[i] = 0.f;
        bool alive = true;
        for (int b = 0; b < batches && alive; ++b) {
            alive = mbar_wait_warp(&batch_done, b & 1, p.status, 113);
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
                __syncwarp();
                if (lane == 0) {
                    if (leader)
                        mbar_arrive(&drained);
                    else
                        mbar_arrive_cluster(map_to_rank(&drained, 0));
                }
            }
        }
        const int row = m0 + warp * 32 + lane;
        if (alive && row < p.M) {
            const bool slabs = p.splits > 1;
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
    // Neither block leaves (or gives its tensor memory back) while the other may still signal its barriers,
    // read its half of B or hold accumulators: every path above ends here.
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    if (warp == MMA_WARP) tmem_dealloc_pair(tmem_base, 512);
}

__global__ void __launch_bounds__(256)
fold_pair_slabs_kernel(const float *__restrict__ partial, float *out, size_t elems, int parts, int accumulate) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= elems) return;
    float s = 0.f;
    for (int q = 0; q < parts; ++q) s += partial[size_t(q) * elems + i];
    out[i] = accumulate ? out[i] + s : s;
}

__global__ void __launch_bounds__(256) split_lo_pair_kernel(const float *__restrict__ x, float *__restrict__ lo, size_t count) {
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
        const float v = x[i];
        lo[i] = v - __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
    }
}

// K-major: storage [rows][K] (K contiguous), box 32 x rows.  MN-major: storage [K][cols] (cols contiguous),
// box 32 x 32 with the 32-byte-atom swizzle (tensor-core reads) or none (builder reads).
bool map_kmajor(CUtensorMap *map, const float *base, size_t rows_extent, size_t k_extent, uint32_t rows_box) {
    const uint64_t dims[2] = {k_extent, rows_extent}, strides[2] = {1, k_extent};
    const uint32_t box[2] = {BK, rows_box};
    return katsu_make_tensor_map(map, base, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

// `slabs` 32-column slabs per tile; when the extent is a multiple of 32 they are a third dimension and one load
// brings them all (*grouped = 1).
bool map_mnmajor(CUtensorMap *map, const float *base, size_t mn_extent, size_t k_extent, bool for_tensor_core,
                 uint32_t slabs, int *grouped) {
    const CUtensorMapSwizzle swizzle = for_tensor_core ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
    *grouped = (mn_extent & 31) == 0;
    if (*grouped) {
        const uint64_t dims[3] = {32, k_extent, mn_extent / 32}, strides[3] = {1, mn_extent, 32};
        const uint32_t box[3] = {32, BK, slabs};
        if (katsu_make_tensor_map(map, base, 3, dims, strides, box, swizzle)) return true;
        *grouped = 0;
    }
    const uint64_t dims[2] = {mn_extent, k_extent}, strides[2] = {1, mn_extent};
    const uint32_t box[2] = {32, BK};
    return katsu_make_tensor_map(map, base, 2, dims, strides, box, swizzle);
}

template <bool A_MN, bool B_MN>
int32_t launch_pair(katsu_cuda_ctx *ctx, const float *a, const float *b, float *c, size_t M, size_t N, size_t K,
                    int accumulate) {
    const bool three_pass = ctx->precision == KATSU_MODE_3XTF32;
    const size_t b_count = K * N;
    const int kb_total = (int)katsu_div_up(K, (size_t)BK);
    const size_t m_pairs = katsu_div_up(M, (size_t)(2 * BM)), n_tiles = katsu_div_up(N, (size_t)BN);
    const size_t blocks = 2 * m_pairs * n_tiles;
    int splits = (int)katsu_div_up((size_t)ctx->num_sms, blocks);
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
        KATSU_LAUNCH(ctx, split_lo_pair_kernel, (unsigned)(size_t(ctx->num_sms) * 8), 256, 0, b, b_lo, b_count);
    }
    if (splits > 1) slabs = take(size_t(splits) * M * N);

    CUtensorMap map_a, map_b, map_b_lo;
    const float *b_lo_src = three_pass ? b_lo : b;
    PairParams p;
    p.a_grouped = p.b_grouped = 0;
    int b_lo_grouped = 0;
    const bool ok = (A_MN ? map_mnmajor(&map_a, a, M, K, false, BM / 32, &p.a_grouped) : map_kmajor(&map_a, a, M, K, BM)) &&
                    (B_MN ? map_mnmajor(&map_b, b, N, K, true, BH / 32, &p.b_grouped) : map_kmajor(&map_b, b, N, K, BH)) &&
                    (B_MN ? map_mnmajor(&map_b_lo, b_lo_src, N, K, true, BH / 32, &b_lo_grouped)
                          : map_kmajor(&map_b_lo, b_lo_src, N, K, BH));
    if (!ok || b_lo_grouped != p.b_grouped)
        return katsu_set_error(KATSU_ERR_CUDA, "cuTensorMapEncodeTiled failed for a matmul operand");

    p.c = splits > 1 ? slabs : c;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.m_pairs = (int)m_pairs; p.n_tiles = (int)n_tiles;
    p.kblocks_per_split = kb_per_split;
    p.splits = splits;
    p.accumulate = accumulate;
    p.three_pass = three_pass ? 1 : 0;
    p.status = ctx->status;
    const size_t smem = size_t(AS) * A_BYTES + size_t(TS_MAX) * 2 * B_BYTES + 1024;
    auto kernel = umma_gemm_pair_kernel<A_MN, B_MN>;
    KATSU_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaLaunchConfig_t config;
    memset(&config, 0, sizeof(config));
    config.gridDim = dim3((unsigned)blocks, 1, (unsigned)splits);
    config.blockDim = dim3(PAIR_THREADS, 1, 1);
    config.dynamicSmemBytes = smem;
    config.stream = ctx->stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = 2;
    attribute.val.clusterDim.y = 1;
    attribute.val.clusterDim.z = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    cudaError_t err = cudaLaunchKernelEx(&config, kernel, map_a, map_b, map_b_lo, p);
    ctx->launches += 1;
    if (err != cudaSuccess)
        return katsu_set_error(KATSU_ERR_CUDA, "pair GEMM launch failed: %s", cudaGetErrorString(err));
    if (splits > 1)
        KATSU_LAUNCH(ctx, fold_pair_slabs_kernel, (unsigned)katsu_div_up(M * N, (size_t)256), 256, 0, slabs, c, M * N, splits,
                     accumulate);
    return KATSU_OK;
}

}  // namespace

// C[M,N] (+)= A * B on CTA pairs.  *handled = 0 when the shape is not worth a 256-row tile (the caller then
// uses the single-block kernel).
int32_t katsu_umma_gemm_pair(katsu_cuda_ctx *ctx, const float *a, const float *b, float *c, size_t M, size_t N, size_t K,
                             bool a_mn, bool b_mn, int accumulate, int *handled) {
    *handled = 0;
    // Measured at 8192^3 / 4096^3: 238 / 229-234 TFLOP/s useful in 3xTF32 against 206-219 / 199-207 for the
    // single-block kernel.  Shapes with a 256 x 256 tile for every pair of SMs have been taken by
    // umma_gemm_wide.cu before this is called (both modes); what arrives here in 3xTF32 is the rest with 256
    // rows or more, which needs this kernel's K split to fill the GPU.
    if (ctx->precision != KATSU_MODE_3XTF32) return KATSU_OK;
    if (M < 256 || N < 64 || K < 32) return KATSU_OK;
    if (katsu_div_up(M, (size_t)(2 * BM)) * katsu_div_up(N, (size_t)BN) > 0x3fffffffu) return KATSU_OK;
    *handled = 1;
    if (!a_mn && !b_mn) return launch_pair<false, false>(ctx, a, b, c, M, N, K, accumulate);
    if (!a_mn && b_mn) return launch_pair<false, true>(ctx, a, b, c, M, N, K, accumulate);
    if (a_mn && !b_mn) return launch_pair<true, false>(ctx, a, b, c, M, N, K, accumulate);
    return launch_pair<true, true>(ctx, a, b, c, M, N, K, accumulate);
}
