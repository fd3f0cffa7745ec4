// Tensor-core GEMM for Tensor::matmul and its VJP (crates/katsu-core/src/tensor.rs:264-273,
// 418-445) on tcgen05: TMA-fed 128x128 tiles, f32 accumulators in tensor memory.
//
//   C[M,N] (+)= A * B with either operand K-major (K contiguous) or MN-major
//   (M resp. N contiguous), so a@b, g@b^T and a^T@g all run without a transpose.
//
// Precision.  kind::tf32 truncates its f32 inputs to TF32.  TF32 mode issues one
// MMA per k-step on the raw data.  3xTF32 mode restores FP32-grade accuracy with
// the split x = hi + lo, hi = trunc_tf32(x) (what the hardware sees when given x),
// lo = x - hi: three MMAs per k-step, hi*hi + lo*hi + hi*lo, into the same f32
// accumulator.  The lo arrays are produced by a streaming pre-pass into scratch.
//
// Accumulation.  The tensor core's f32 accumulate loses a little on every k-step
// (measured: relative error grows about linearly with K, 1.2e-6 at K = 512), so a
// tile rotates its k-blocks over four TMEM accumulators that are added in f32 at
// the end, and long K is split over blockIdx.z with an ordered fold of the
// partial tiles (bit-reproducible, no atomics).
#include "common.cuh"
#include "sm100.cuh"

using namespace sm100;

namespace {

constexpr int BM = 128;      // tile rows == TMEM lanes
constexpr int BN = 128;      // tile columns
constexpr int BK = 32;       // f32 per 128-byte swizzle row
constexpr int NACC = 4;      // rotating accumulators (4 x 128 columns = all of TMEM)
constexpr int STAGES = 3;
constexpr int TILE_BYTES = BM * BK * 4;  // 16 KiB, same for A and B tiles (BM == BN)

struct GemmParams {
    float *c;          // output, or partial slabs [splits][M][N] when splits > 1
    int M, N, K;
    int kblocks_per_split;
    int splits;
    int accumulate;    // only used when splits == 1
    int three_pass;    // 3xTF32
    int *status;
};

__global__ void __launch_bounds__(256) split_lo_kernel(const float *__restrict__ x, float *__restrict__ lo, size_t count) {
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
        const float v = x[i];
        lo[i] = v - __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
    }
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(128, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_a_lo,
                 const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_b_lo,
                 GemmParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // stage layout: [A hi][A lo][B hi][B lo], 16 KiB each
    __shared__ uint64_t full[STAGES], empty[STAGES], done;
    __shared__ uint32_t tmem_slot;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int kb_total = (p.K + BK - 1) / BK;
    const int kb_begin = blockIdx.z * p.kblocks_per_split;
    int kb_end = kb_begin + p.kblocks_per_split;
    if (kb_end > kb_total) kb_end = kb_total;
    const int kblocks = kb_end - kb_begin;
    const int tiles_per_stage = p.three_pass ? 4 : 2;
    const uint32_t stage_bytes = 4 * TILE_BYTES;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(&done, 1);
        mbar_init_fence();
    }
    if (warp == 0) {
        tmem_alloc(&tmem_slot, NACC * BN);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_slot;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer ----
        for (int i = 0; i < kblocks; ++i) {
            const int s = i % STAGES;
            if (i >= STAGES && !mbar_wait(&empty[s], ((i / STAGES) - 1) & 1, p.status, 11)) break;
            mbar_arrive_expect_tx(&full[s], tiles_per_stage * TILE_BYTES);
            unsigned char *st = smem + s * stage_bytes;
            const int k0 = (kb_begin + i) * BK;
            for (int part = 0; part < (p.three_pass ? 2 : 1); ++part) {
                const CUtensorMap *ma = part ? &map_a_lo : &map_a;
                const CUtensorMap *mb = part ? &map_b_lo : &map_b;
                unsigned char *ad = st + part * TILE_BYTES, *bd = st + (2 + part) * TILE_BYTES;
                if (!A_MN) {
                    tma_load_2d(ad, ma, &full[s], k0, m0);
                } else {
                    for (int j = 0; j < BM / 32; ++j) tma_load_2d(ad + j * 4096, ma, &full[s], m0 + 32 * j, k0);
                }
                if (!B_MN) {
                    tma_load_2d(bd, mb, &full[s], k0, n0);
                } else {
                    for (int j = 0; j < BN / 32; ++j) tma_load_2d(bd + j * 4096, mb, &full[s], n0 + 32 * j, k0);
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer: the whole warp runs the loop, the thread chosen by elect.sync issues.
        // With warp-uniform control flow the operands stay in uniform registers, and a wait on
        // an already-full stage costs ~90 cycles instead of ~300 behind a lane == 0 branch
        // (measured); at 768 tensor-pipe cycles per 3xTF32 k-block that is the difference
        // between ~70 % and ~90 % of the pipe. ----
        const bool issue = elect_one();
        const uint32_t idesc = idesc_tf32(BM, BN, A_MN, B_MN);
        for (int i = 0; i < kblocks; ++i) {
            const int s = i % STAGES;
            if (!mbar_wait_warp_ready(&full[s], (i / STAGES) & 1, p.status, 12)) break;
            tc_fence_after_sync();
            const uint32_t st = smem_u32(smem + s * stage_bytes);
            const uint32_t acc = tmem_base + uint32_t(i % NACC) * BN;
            const bool first = i < NACC;
            if (issue) {
#pragma unroll
                for (int j = 0; j < BK / 8; ++j) {
                    const uint32_t a_off = A_MN ? j * 1024 : j * 32, b_off = B_MN ? j * 1024 : j * 32;
                    auto desc = [&](uint32_t addr, bool mn) {
                        return mn ? smem_desc(addr, 4096, 512, kLayoutSw128Base32) : smem_desc(addr, 16, 1024, kLayoutSw128);
                    };
                    const uint64_t a_hi = desc(st + a_off, A_MN), b_hi = desc(st + 2 * TILE_BYTES + b_off, B_MN);
                    if (p.three_pass) {
                        const uint64_t a_lo = desc(st + TILE_BYTES + a_off, A_MN);
                        const uint64_t b_lo = desc(st + 3 * TILE_BYTES + b_off, B_MN);
                        mma_tf32(acc, a_lo, b_hi, idesc, !(first && j == 0));
                        mma_tf32(acc, a_hi, b_lo, idesc, true);
                        mma_tf32(acc, a_hi, b_hi, idesc, true);
                    } else {
                        mma_tf32(acc, a_hi, b_hi, idesc, !(first && j == 0));
                    }
                }
                mma_commit(&empty[s]);  // frees the stage once these MMAs have read it
            }
            __syncwarp();
        }
        if (issue) mma_commit(&done);
    }
    __syncwarp();

    // ---- epilogue: warp w owns tile rows 32w .. 32w+31 ----
    const bool finished = mbar_wait(&done, 0, p.status, 13);
    tc_fence_after_sync();
    if (finished && kblocks > 0) {
        const int row = m0 + warp * 32 + lane;
        const int used_acc = kblocks < NACC ? kblocks : NACC;
        float *out = p.c + (p.splits > 1 ? size_t(blockIdx.z) * p.M * p.N : 0);
        for (int c0 = 0; c0 < BN; c0 += 32) {
            if (n0 + c0 >= p.N) break;  // warp-uniform
            float v[32];
            tmem_ld_32x32(tmem_base + (uint32_t(warp * 32) << 16) + c0, v);
            for (int a = 1; a < used_acc; ++a) {
                float t[32];
                tmem_ld_32x32(tmem_base + (uint32_t(warp * 32) << 16) + a * BN + c0, t);
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] += t[i];
            }
            if (row < p.M) {
                float *dst = out + size_t(row) * p.N + n0 + c0;
                const bool acc_out = p.accumulate && p.splits == 1;
                if (n0 + c0 + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4) {
                        float4 q = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                        if (acc_out) {
                            const float4 o = *reinterpret_cast<const float4 *>(dst + i);
                            q.x += o.x; q.y += o.y; q.z += o.z; q.w += o.w;
                        }
                        *reinterpret_cast<float4 *>(dst + i) = q;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (n0 + c0 + i < p.N) dst[i] = acc_out ? dst[i] + v[i] : v[i];
                }
            }
        }
    } else if (finished && kblocks == 0 && p.splits > 1) {
        // an empty K range still owns a partial slab: it must read as zero
        const int row = m0 + warp * 32 + lane;
        if (row < p.M)
            for (int c = n0; c < n0 + BN && c < p.N; ++c) p.c[(size_t(blockIdx.z) * p.M + row) * p.N + c] = 0.f;
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_base, NACC * BN);
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
bool operand_map(CUtensorMap *map, const float *base, bool mn_major, size_t mn_extent, size_t k_extent) {
    uint64_t dims[2], strides[2] = {1, 0};
    uint32_t box[2];
    if (!mn_major) {
        dims[0] = k_extent; dims[1] = mn_extent; strides[1] = k_extent; box[0] = BK; box[1] = BM;
        return katsu_make_tensor_map(map, base, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    }
    dims[0] = mn_extent; dims[1] = k_extent; strides[1] = mn_extent; box[0] = 32; box[1] = BK;
    return katsu_make_tensor_map(map, base, 2, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
}

template <bool A_MN, bool B_MN>
int32_t launch(katsu_cuda_ctx *ctx, const float *a, const float *b, float *c, size_t M, size_t N, size_t K,
               int accumulate) {
    const bool three_pass = ctx->precision == KATSU_MODE_3XTF32;
    const size_t a_count = M * K, b_count = K * N;
    const int kb_total = (int)katsu_div_up(K, (size_t)BK);
    // K split: keep each accumulator's chain short (<= 16 k-blocks = 512 terms) and fill the GPU.
    const size_t tiles = katsu_div_up(M, (size_t)BM) * katsu_div_up(N, (size_t)BN);
    int splits = (int)katsu_div_up((size_t)kb_total, (size_t)(NACC * 16));
    const int fill = (int)katsu_div_up((size_t)ctx->num_sms, tiles);
    if (splits < fill) splits = fill;
    if (splits > kb_total) splits = kb_total;
    if (splits > 1024) splits = 1024;
    int kb_per_split = (int)katsu_div_up((size_t)kb_total, (size_t)splits);
    splits = (int)katsu_div_up((size_t)kb_total, (size_t)kb_per_split);

    size_t scratch_floats = (three_pass ? a_count + b_count : 0) + (splits > 1 ? size_t(splits) * M * N : 0);
    float *scratch = nullptr;
    if (scratch_floats) KATSU_TRY(katsu_scratch(ctx, scratch_floats + 64, &scratch));
    float *a_lo = nullptr, *b_lo = nullptr, *slabs = nullptr;
    size_t cursor = 0;
    auto take = [&](size_t n) { float *ptr = scratch + cursor; cursor += (n + 31) / 32 * 32; return ptr; };
    if (three_pass) {
        a_lo = take(a_count);
        b_lo = take(b_count);
        const unsigned blocks = (unsigned)(size_t(ctx->num_sms) * 8);
        KATSU_LAUNCH(ctx, split_lo_kernel, blocks, 256, 0, a, a_lo, a_count);
        KATSU_LAUNCH(ctx, split_lo_kernel, blocks, 256, 0, b, b_lo, b_count);
    }
    if (splits > 1) slabs = take(size_t(splits) * M * N);

    CUtensorMap map_a, map_a_lo, map_b, map_b_lo;
    bool ok = operand_map(&map_a, a, A_MN, M, K) && operand_map(&map_b, b, B_MN, N, K);
    ok = ok && operand_map(&map_a_lo, three_pass ? a_lo : a, A_MN, M, K) &&
         operand_map(&map_b_lo, three_pass ? b_lo : b, B_MN, N, K);
    if (!ok) return katsu_set_error(KATSU_ERR_CUDA, "cuTensorMapEncodeTiled failed for a matmul operand");

    GemmParams p;
    p.c = splits > 1 ? slabs : c;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.kblocks_per_split = kb_per_split;
    p.splits = splits;
    p.accumulate = accumulate;
    p.three_pass = three_pass ? 1 : 0;
    p.status = ctx->status;
    const size_t smem = size_t(STAGES) * 4 * TILE_BYTES + 1024;
    auto kernel = umma_gemm_kernel<A_MN, B_MN>;
    KATSU_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)katsu_div_up(N, (size_t)BN), (unsigned)katsu_div_up(M, (size_t)BM), (unsigned)splits);
    KATSU_LAUNCH(ctx, kernel, grid, 128, smem, map_a, map_a_lo, map_b, map_b_lo, p);
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
    *handled = 1;
    if (!a_mn && !b_mn) return launch<false, false>(ctx, a, b, c, M, N, K, accumulate);
    if (!a_mn && b_mn) return launch<false, true>(ctx, a, b, c, M, N, K, accumulate);
    if (a_mn && !b_mn) return launch<true, false>(ctx, a, b, c, M, N, K, accumulate);
    return launch<true, true>(ctx, a, b, c, M, N, K, accumulate);
}
