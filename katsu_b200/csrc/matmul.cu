// Tensor::matmul and its VJP on CUDA cores.
//
//   fwd : c[m,n]   = a[m,k] @ b[k,n]          crates/katsu-core/src/tensor.rs:264-273
//   dA  : da[m,k] (+)= g[m,n] @ b^T           tensor.rs:425-434
//   dB  : db[k,n] (+)= a^T @ g                tensor.rs:435-444
//
// Two families:
//  * "skinny" kernels for n <= 16 (a classifier head such as [512,65536]@[65536,10]):
//    the big operand (a, or da) is streamed through HBM exactly once with
//    128-bit accesses while the small ones live in registers / shared memory;
//  * a general 64x64-tile kernel with arbitrary element strides, so the same
//    code serves a@b, g@b^T and a^T@g without materialising a transpose.
#include "common.cuh"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// ---------------------------------------------------------------------------
// general strided GEMM: C[i,j] (+)= sum_p A(i,p) * B(p,j)
//   A(i,p) = a[i*sa_i + p*sa_p],  B(p,j) = b[p*sb_p + j*sb_j],  C row-major [M,N]
// 64x64 tile, 16-deep slices, 256 threads x (4x4) micro tiles.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gemm_strided_kernel(const float *__restrict__ a, const float *__restrict__ b, float *c, int M, int N, int K,
                    size_t sa_i, size_t sa_p, size_t sb_p, size_t sb_j, int accumulate) {
    __shared__ float As[16][64 + 4];
    __shared__ float Bs[16][64 + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int i0 = blockIdx.y * 64, j0 = blockIdx.x * 64;
    float acc[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int v = 0; v < 4; ++v) acc[u][v] = 0.f;

    for (int p0 = 0; p0 < K; p0 += 16) {
        // Pick the thread->element map that walks the unit-stride axis fastest.
        for (int e = tid; e < 64 * 16; e += 256) {
            int ii, pp;
            if (sa_p == 1) { pp = e & 15; ii = e >> 4; } else { ii = e & 63; pp = e >> 6; }
            const int gi = i0 + ii, gp = p0 + pp;
            As[pp][ii] = (gi < M && gp < K) ? __ldg(a + size_t(gi) * sa_i + size_t(gp) * sa_p) : 0.f;
        }
        for (int e = tid; e < 64 * 16; e += 256) {
            int jj, pp;
            if (sb_j == 1) { jj = e & 63; pp = e >> 6; } else { pp = e & 15; jj = e >> 4; }
            const int gj = j0 + jj, gp = p0 + pp;
            Bs[pp][jj] = (gj < N && gp < K) ? __ldg(b + size_t(gp) * sb_p + size_t(gj) * sb_j) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int pp = 0; pp < 16; ++pp) {
            const float4 av = *reinterpret_cast<const float4 *>(&As[pp][ty * 4]);
            const float4 bv = *reinterpret_cast<const float4 *>(&Bs[pp][tx * 4]);
            const float ar[4] = {av.x, av.y, av.z, av.w};
            const float br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int v = 0; v < 4; ++v) acc[u][v] = fmaf(ar[u], br[v], acc[u][v]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int gi = i0 + ty * 4 + u;
        if (gi >= M) continue;
#pragma unroll
        for (int v = 0; v < 4; ++v) {
            const int gj = j0 + tx * 4 + v;
            if (gj >= N) continue;
            float *dst = c + size_t(gi) * N + gj;
            *dst = accumulate ? *dst + acc[u][v] : acc[u][v];
        }
    }
}

// ---------------------------------------------------------------------------
// skinny forward, n <= NP <= 16.  grid = (k slabs of SK_KC columns, row splits).
// A block stages its [SK_KC x n] slab of b in shared memory once, then streams
// its rows of a: a warp takes four rows at a time, its lanes cover the slab's
// columns as float4s (all sixteen loads of an iteration are issued before the
// first use, which is what keeps enough bytes in flight for HBM), and the
// per-row sums over the slab go to scratch as [slab][m][n]; a second kernel
// folds the slabs in order.
// ---------------------------------------------------------------------------
constexpr int SK_RW = 4;     // rows per warp and iteration
// k columns per shared-memory slab: as many as 48 KiB hold, at most 1024.  A longer slab means fewer
// cross-lane reductions (one per row and slab) for the same bytes of a.
template <int NP>
constexpr int sk_kc() { return NP <= 12 ? 1024 : 512; }

template <int NP>
__global__ void __launch_bounds__(256, 2)
skinny_fwd_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ partial,
                  int m, size_t k, int n, int rows_per_block, int vec_ok) {
    // the slab transposed, [NP][SK_KC]: a lane's four consecutive k for one output column are one 128-bit
    // shared-memory read, and consecutive lanes read consecutive float4s (the [k][n] order put sixteen lanes
    // on one bank)
    constexpr int SK_KC = sk_kc<NP>();
    __shared__ __align__(16) float bs[NP * SK_KC];
    const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
    const size_t kc = size_t(blockIdx.x) * SK_KC;
    const int span = (int)((k - kc) < (size_t)SK_KC ? (k - kc) : (size_t)SK_KC);
    // rows kc .. kc + span of b are one contiguous run of span * n floats: read it in order (coalesced),
    // scatter into the transposed slab; columns n .. NP and rows past the end of k are zero
    for (int e = tid; e < SK_KC * NP; e += 256) bs[e] = 0.f;
    __syncthreads();
    {
        const float *slab = b + kc * n;
        const int count = span * n;
        for (int e = tid; e < count; e += 256) {
            const int pp = e / n, j = e - pp * n;
            bs[j * SK_KC + pp] = __ldg(slab + e);
        }
    }
    __syncthreads();
    const int r_begin = blockIdx.y * rows_per_block;
    const int r_end = (r_begin + rows_per_block) < m ? (r_begin + rows_per_block) : m;
    const bool whole = vec_ok && span == SK_KC;
    for (int row0 = r_begin + wp * SK_RW; row0 < r_end; row0 += 8 * SK_RW) {
        float acc[SK_RW][NP];
#pragma unroll
        for (int r = 0; r < SK_RW; ++r)
#pragma unroll
            for (int j = 0; j < NP; ++j) acc[r][j] = 0.f;
        for (int base = 0; base < SK_KC; base += 512) {   // sixteen loads in flight per lane at a time
        float av[4][SK_RW][4];
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int pp = base + lane * 4 + it * 128;
#pragma unroll
            for (int r = 0; r < SK_RW; ++r) {
                const int row = row0 + r;
                const float *src = a + size_t(row < r_end ? row : r_begin) * k + kc + pp;
                if (whole) {
                    const float4 q = __ldg(reinterpret_cast<const float4 *>(src));
                    av[it][r][0] = q.x; av[it][r][1] = q.y; av[it][r][2] = q.z; av[it][r][3] = q.w;
                } else {
#pragma unroll
                    for (int u = 0; u < 4; ++u) av[it][r][u] = (pp + u < span) ? __ldg(src + u) : 0.f;
                }
            }
        }
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int pp = base + lane * 4 + it * 128;
#pragma unroll
            for (int j = 0; j < NP; ++j) {
                const float4 bq = *reinterpret_cast<const float4 *>(&bs[j * SK_KC + pp]);
                const float bv[4] = {bq.x, bq.y, bq.z, bq.w};
                // k order within the lane as before: u = 0, 1, 2, 3
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int r = 0; r < SK_RW; ++r) acc[r][j] = fmaf(av[it][r][u], bv[u], acc[r][j]);
            }
        }
        }  // halves of the slab
#pragma unroll
        for (int r = 0; r < SK_RW; ++r)
#pragma unroll
            for (int j = 0; j < NP; ++j) {
                const float sum = warp_sum(acc[r][j]);
                const int row = row0 + r;
                if (lane == 0 && row < r_end && j < n) partial[(size_t(blockIdx.x) * m + row) * n + j] = sum;
            }
    }
}

// out[i] (+)= sum over `parts` slabs of `elems` floats, in slab order.
__global__ void __launch_bounds__(256)
fold_partials_kernel(const float *__restrict__ partial, float *out, size_t elems, int parts, int accumulate) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= elems) return;
    float s = 0.f;
    int p = 0;
    // sixteen loads in flight, added in slab order (a plain loop waits out one L2 round trip per slab)
    for (; p + 16 <= parts; p += 16) {
        float v[16];
#pragma unroll
        for (int q = 0; q < 16; ++q) v[q] = __ldg(partial + size_t(p + q) * elems + i);
#pragma unroll
        for (int q = 0; q < 16; ++q) s += v[q];
    }
    for (; p < parts; ++p) s += partial[size_t(p) * elems + i];
    out[i] = accumulate ? out[i] + s : s;
}

// ---------------------------------------------------------------------------
// skinny dA: da[i, p] (+)= sum_j g[i,j] * b[p,j].  A thread owns four
// consecutive p (one float4 of every da row it touches) and keeps b[p..p+3][:]
// in registers; g rows come from shared memory as broadcasts.
// grid = (k / 1024, row chunks of 64).
// ---------------------------------------------------------------------------
template <int NP>
__global__ void __launch_bounds__(256)
skinny_da_kernel(const float *__restrict__ g, const float *__restrict__ b, float *da, int m, size_t k, int n,
                 int vec_ok, int accumulate) {
    __shared__ __align__(16) float gs[64 * NP];
    const int tid = threadIdx.x;
    const int row0 = blockIdx.y * 64;
    const int rows = (m - row0) < 64 ? (m - row0) : 64;
    for (int e = tid; e < 64 * NP; e += 256) {
        const int r = e / NP, j = e % NP;
        gs[e] = (r < rows && j < n) ? __ldg(g + size_t(row0 + r) * n + j) : 0.f;
    }
    __syncthreads();
    const size_t p = (size_t(blockIdx.x) * 256 + tid) * 4;
    if (p >= k) return;
    float bv[4][NP];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int j = 0; j < NP; ++j) bv[u][j] = (p + u < k && j < n) ? __ldg(b + (p + u) * n + j) : 0.f;
    const bool full = vec_ok && (p + 3 < k);
    for (int r = 0; r < rows; ++r) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < NP; ++j) {
            const float gv = gs[r * NP + j];
#pragma unroll
            for (int u = 0; u < 4; ++u) acc[u] = fmaf(gv, bv[u][j], acc[u]);
        }
        float *dst = da + size_t(row0 + r) * k + p;
        if (full) {
            float4 v = make_float4(acc[0], acc[1], acc[2], acc[3]);
            if (accumulate) {
                const float4 o = *reinterpret_cast<const float4 *>(dst);
                v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
            }
            *reinterpret_cast<float4 *>(dst) = v;
        } else {
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (p + u < k) dst[u] = accumulate ? dst[u] + acc[u] : acc[u];
        }
    }
}

// ---------------------------------------------------------------------------
// skinny dB: db[p, j] (+)= sum_i a[i,p] * g[i,j].  A thread owns four
// consecutive p and NP columns; it streams its float4 column strip of a over
// the block's row range, eight rows per iteration with all eight loads issued
// before the first use.  The g rows of the range sit in shared memory
// (broadcast reads).  grid = (k / 512, row splits); partials [split][k][n] go
// to scratch and are folded in order.
// ---------------------------------------------------------------------------
constexpr int SK_GROWS = 256;  // g rows staged at a time

template <int NP>
__global__ void __launch_bounds__(128)
skinny_db_kernel(const float *__restrict__ a, const float *__restrict__ g, float *__restrict__ partial, int m,
                 size_t k, int n, int rows_per_split, int vec_ok) {
    __shared__ __align__(16) float gs[SK_GROWS * NP];
    const int tid = threadIdx.x;
    const size_t p = (size_t(blockIdx.x) * 128 + tid) * 4;
    const int r_begin = blockIdx.y * rows_per_split;
    const int r_end = (r_begin + rows_per_split) < m ? (r_begin + rows_per_split) : m;
    const bool full = vec_ok && (p + 3 < k);
    float acc[4][NP];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int j = 0; j < NP; ++j) acc[u][j] = 0.f;
    for (int rc = r_begin; rc < r_end; rc += SK_GROWS) {
        const int rows = (r_end - rc) < SK_GROWS ? (r_end - rc) : SK_GROWS;
        __syncthreads();
        for (int e = tid; e < SK_GROWS * NP; e += 128) {
            const int r = e / NP, j = e % NP;
            gs[e] = (r < rows && j < n) ? __ldg(g + size_t(rc + r) * n + j) : 0.f;
        }
        __syncthreads();
        if (p < k) {
            for (int r0 = 0; r0 < rows; r0 += 8) {
                float av[8][4];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int r = r0 + q;
                    const float *src = a + size_t(rc + (r < rows ? r : 0)) * k + p;
                    if (full) {
                        const float4 v = __ldg(reinterpret_cast<const float4 *>(src));
                        av[q][0] = v.x; av[q][1] = v.y; av[q][2] = v.z; av[q][3] = v.w;
                    } else {
#pragma unroll
                        for (int u = 0; u < 4; ++u) av[q][u] = (p + u < k) ? __ldg(src + u) : 0.f;
                    }
                }
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    if (r0 + q < rows) {
#pragma unroll
                        for (int j = 0; j < NP; ++j) {
                            const float gv = gs[(r0 + q) * NP + j];
#pragma unroll
                            for (int u = 0; u < 4; ++u) acc[u][j] = fmaf(av[q][u], gv, acc[u][j]);
                        }
                    }
                }
            }
        }
    }
    if (p < k) {
        float *dst = partial + size_t(blockIdx.y) * k * n;
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (p + u < k)
#pragma unroll
                for (int j = 0; j < NP; ++j)
                    if (j < n) dst[(p + u) * n + j] = acc[u][j];
    }
}

bool aligned16(const void *ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; }

int32_t gemm_strided(katsu_cuda_ctx *ctx, const float *a, const float *b, float *c, size_t M, size_t N, size_t K,
                     size_t sa_i, size_t sa_p, size_t sb_p, size_t sb_j, int accumulate) {
    if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff)
        return katsu_set_error(KATSU_ERR_UNSUPPORTED, "a matmul dimension exceeds 2^31-1");
    const size_t gy = katsu_div_up(M, 64), gx = katsu_div_up(N, 64);
    if (gy > 65535) return katsu_set_error(KATSU_ERR_UNSUPPORTED, "matmul output has too many row tiles");
    dim3 grid((unsigned)gx, (unsigned)gy);
    KATSU_LAUNCH(ctx, gemm_strided_kernel, grid, 256, 0, a, b, c, (int)M, (int)N, (int)K, sa_i, sa_p, sb_p, sb_j,
                 accumulate);
    return KATSU_OK;
}

template <int NP>
int32_t skinny_fwd(katsu_cuda_ctx *ctx, const float *a, const float *b, float *c, size_t m, size_t k, size_t n) {
    // one block per (slab of SK_KC columns, range of rows); the row ranges only exist to fill the GPU
    const size_t slabs = katsu_div_up(k, (size_t)sk_kc<NP>());
    size_t row_splits = katsu_div_up(size_t(ctx->num_sms) * 2, slabs);
    const size_t max_row_splits = katsu_div_up(m, (size_t)(8 * SK_RW));
    if (row_splits > max_row_splits) row_splits = max_row_splits;
    if (row_splits > 65535) row_splits = 65535;
    const size_t rows_per_block = katsu_div_up(katsu_div_up(m, row_splits), (size_t)(8 * SK_RW)) * (8 * SK_RW);
    row_splits = katsu_div_up(m, rows_per_block);
    float *partial = nullptr;
    KATSU_TRY(katsu_scratch(ctx, slabs * m * n, &partial));
    const int vec_ok = aligned16(a) && (k % 4 == 0);
    dim3 grid((unsigned)slabs, (unsigned)row_splits);
    KATSU_LAUNCH(ctx, skinny_fwd_kernel<NP>, grid, 256, 0, a, b, partial, (int)m, k, (int)n, (int)rows_per_block, vec_ok);
    KATSU_LAUNCH(ctx, fold_partials_kernel, (unsigned)katsu_div_up(m * n, 256), 256, 0, partial, c, m * n,
                 (int)slabs, 0);
    return KATSU_OK;
}

template <int NP>
int32_t skinny_da(katsu_cuda_ctx *ctx, const float *g, const float *b, float *da, size_t m, size_t k, size_t n,
                  int accumulate) {
    const int vec_ok = aligned16(da) && (k % 4 == 0);
    dim3 grid((unsigned)katsu_div_up(k, 1024), (unsigned)katsu_div_up(m, 64));
    KATSU_LAUNCH(ctx, skinny_da_kernel<NP>, grid, 256, 0, g, b, da, (int)m, k, (int)n, vec_ok, accumulate);
    return KATSU_OK;
}

template <int NP>
int32_t skinny_db(katsu_cuda_ctx *ctx, const float *a, const float *g, float *db, size_t m, size_t k, size_t n,
                  int accumulate) {
    const size_t col_blocks = katsu_div_up(k, 512);
    size_t splits = katsu_div_up(size_t(ctx->num_sms) * 4, col_blocks);
    const size_t max_splits = katsu_div_up(m, 64);
    if (splits > max_splits) splits = max_splits;
    size_t rows_per_split = katsu_div_up(katsu_div_up(m, splits), 64) * 64;
    splits = katsu_div_up(m, rows_per_split);
    float *partial = nullptr;
    KATSU_TRY(katsu_scratch(ctx, splits * k * n, &partial));
    const int vec_ok = aligned16(a) && (k % 4 == 0);
    dim3 grid((unsigned)col_blocks, (unsigned)splits);
    KATSU_LAUNCH(ctx, skinny_db_kernel<NP>, grid, 128, 0, a, g, partial, (int)m, k, (int)n, (int)rows_per_split,
                 vec_ok);
    KATSU_LAUNCH(ctx, fold_partials_kernel, (unsigned)katsu_div_up(k * n, 256), 256, 0, partial, db, k * n,
                 (int)splits, accumulate);
    return KATSU_OK;
}

bool skinny_shape(size_t m, size_t k, size_t n) {
    // (the forward kernel keeps one [m x n] partial per 512-column slab of k: at most 256 MiB of scratch)
    return n >= 1 && n <= 16 && k >= 2048 && m <= 0x7fffffff && katsu_div_up(k, 512) <= 0x7fffffff &&
           katsu_div_up(m, 32) <= 0x7fffffff && katsu_div_up(m, 64) <= 65535 &&
           katsu_div_up(k, 512) * m * n <= (size_t(1) << 26);
}

}  // namespace

#define KATSU_NP_SWITCH(n, CALL)            \
    do {                                    \
        if ((n) <= 4) return CALL(4);       \
        if ((n) <= 8) return CALL(8);       \
        if ((n) <= 12) return CALL(12);     \
        return CALL(16);                    \
    } while (0)

extern "C" int32_t katsu_cuda_matmul_fwd(katsu_cuda_ctx *ctx, const float *a, const float *b, float *c,
                                         size_t m, size_t k, size_t n) {
    KATSU_TRY(katsu_bind(ctx));
    if (m == 0 || n == 0) return KATSU_OK;
    KATSU_REQUIRE(c != nullptr, "c is null");
    if (k == 0) {
        KATSU_CUDA_TRY(cudaMemsetAsync(c, 0, m * n * sizeof(float), ctx->stream));
        return KATSU_OK;
    }
    KATSU_REQUIRE(a != nullptr && b != nullptr, "null operand");
    if (skinny_shape(m, k, n)) {
#define CALL(NP) skinny_fwd<NP>(ctx, a, b, c, m, k, n)
        KATSU_NP_SWITCH(n, CALL);
#undef CALL
    }
    int handled = 0;
    KATSU_TRY(katsu_umma_gemm(ctx, a, b, c, m, n, k, false, true, 0, &handled));
    if (handled) return KATSU_OK;
    return gemm_strided(ctx, a, b, c, m, n, k, k, 1, n, 1, 0);
}

extern "C" int32_t katsu_cuda_matmul_bwd(katsu_cuda_ctx *ctx, const float *a, const float *b, const float *g,
                                         float *da, float *db, size_t m, size_t k, size_t n,
                                         int32_t accumulate) {
    KATSU_TRY(katsu_bind(ctx));
    // tensor.rs:421-423: nothing to do when g is empty or k == 0 (the adjoints keep their contents).
    if (m == 0 || n == 0 || k == 0) {
        if (!accumulate) {
            if (da != nullptr && m * k != 0) KATSU_CUDA_TRY(cudaMemsetAsync(da, 0, m * k * sizeof(float), ctx->stream));
            if (db != nullptr && k * n != 0) KATSU_CUDA_TRY(cudaMemsetAsync(db, 0, k * n * sizeof(float), ctx->stream));
        }
        return KATSU_OK;
    }
    KATSU_REQUIRE(a != nullptr && b != nullptr && g != nullptr, "null operand");
    const bool skinny = skinny_shape(m, k, n);
    // da == db (the reference's "same parent on both edges", tensor.rs:425-444, possible when
    // m == k == n): the second product is added to the first whatever `accumulate` says.
    const int accumulate_db = (da != nullptr && da == db) ? 1 : accumulate;
    if (da != nullptr) {
        if (skinny) {
#define CALL(NP) skinny_da<NP>(ctx, g, b, da, m, k, n, accumulate)
            int32_t rc = [&]() -> int32_t { KATSU_NP_SWITCH(n, CALL); }();
#undef CALL
            KATSU_TRY(rc);
        } else {
            // da[m,k] = g[m,n] @ b^T : A(i,p)=g[i*n+p], B(p,j)=b[j*n+p]  (both K-major for the tensor cores)
            int handled = 0;
            KATSU_TRY(katsu_umma_gemm(ctx, g, b, da, m, k, n, false, false, accumulate, &handled));
            if (!handled) KATSU_TRY(gemm_strided(ctx, g, b, da, m, k, n, n, 1, 1, n, accumulate));
        }
    }
    if (db != nullptr) {
        if (skinny) {
#define CALL(NP) skinny_db<NP>(ctx, a, g, db, m, k, n, accumulate_db)
            int32_t rc = [&]() -> int32_t { KATSU_NP_SWITCH(n, CALL); }();
#undef CALL
            KATSU_TRY(rc);
        } else {
            // db[k,n] = a^T @ g : A(i,p)=a[p*k+i], B(p,j)=g[p*n+j]  (both MN-major for the tensor cores)
            int handled = 0;
            KATSU_TRY(katsu_umma_gemm(ctx, a, g, db, k, n, m, true, true, accumulate_db, &handled));
            if (!handled) KATSU_TRY(gemm_strided(ctx, a, g, db, k, n, m, 1, k, n, 1, accumulate_db));
        }
    }
    return KATSU_OK;
}
