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
// skinny forward, n <= NP <= 16.  grid = (row blocks of 32, k splits).  Each
// warp owns 4 rows; lanes walk the split's k range four columns at a time
// (one float4 of a per row).  The matching [KC x n] slab of b is staged in
// shared memory.  Partials go to scratch as [split][m][n]; a second kernel
// folds the splits in order.
// ---------------------------------------------------------------------------
constexpr int SK_KC = 512;   // k columns per shared-memory slab
constexpr int SK_RW = 4;     // rows per warp

template <int NP>
__global__ void __launch_bounds__(256)
skinny_fwd_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ partial,
                  int m, size_t k, int n, size_t k_per_split, int vec_ok) {
    __shared__ float bs[SK_KC * NP];
    const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
    const int row0 = blockIdx.x * 32 + wp * SK_RW;
    const size_t k_begin = size_t(blockIdx.y) * k_per_split;
    size_t k_end = k_begin + k_per_split;
    if (k_end > k) k_end = k;
    float acc[SK_RW][NP];
#pragma unroll
    for (int r = 0; r < SK_RW; ++r)
#pragma unroll
        for (int j = 0; j < NP; ++j) acc[r][j] = 0.f;

    for (size_t kc = k_begin; kc < k_end; kc += SK_KC) {
        const int span = (int)((k_end - kc) < (size_t)SK_KC ? (k_end - kc) : (size_t)SK_KC);
        __syncthreads();
        for (int e = tid; e < SK_KC * NP; e += 256) {
            const int pp = e / NP, j = e % NP;
            bs[e] = (pp < span && j < n) ? __ldg(b + (kc + pp) * n + j) : 0.f;
        }
        __syncthreads();
        for (int pp = lane * 4; pp < span; pp += 128) {
            float av[SK_RW][4];
#pragma unroll
            for (int r = 0; r < SK_RW; ++r) {
                const int row = row0 + r;
                if (row < m) {
                    const float *src = a + size_t(row) * k + kc + pp;
                    if (vec_ok && pp + 3 < span) {
                        const float4 q = __ldg(reinterpret_cast<const float4 *>(src));
                        av[r][0] = q.x; av[r][1] = q.y; av[r][2] = q.z; av[r][3] = q.w;
                    } else {
#pragma unroll
                        for (int u = 0; u < 4; ++u) av[r][u] = (pp + u < span) ? __ldg(src + u) : 0.f;
                    }
                } else {
#pragma unroll
                    for (int u = 0; u < 4; ++u) av[r][u] = 0.f;
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                float bv[NP];
#pragma unroll
                for (int j = 0; j < NP; ++j) bv[j] = bs[(pp + u) * NP + j];
#pragma unroll
                for (int r = 0; r < SK_RW; ++r)
#pragma unroll
                    for (int j = 0; j < NP; ++j) acc[r][j] = fmaf(av[r][u], bv[j], acc[r][j]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < SK_RW; ++r)
#pragma unroll
        for (int j = 0; j < NP; ++j) {
            const float s = warp_sum(acc[r][j]);
            const int row = row0 + r;
            if (lane == 0 && row < m && j < n) partial[(size_t(blockIdx.y) * m + row) * n + j] = s;
        }
}

// out[i] (+)= sum over `parts` slabs of `elems` floats, in slab order.
__global__ void __launch_bounds__(256)
fold_partials_kernel(const float *__restrict__ partial, float *out, size_t elems, int parts, int accumulate) {
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= elems) return;
    float s = 0.f;
    for (int p = 0; p < parts; ++p) s += partial[size_t(p) * elems + i];
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
// the block's row range.  grid = (k / 512, row splits); partials [split][k][n]
// go to scratch and are folded in order.
// ---------------------------------------------------------------------------
template <int NP>
__global__ void __launch_bounds__(128)
skinny_db_kernel(const float *__restrict__ a, const float *__restrict__ g, float *__restrict__ partial, int m,
                 size_t k, int n, int rows_per_split, int vec_ok) {
    __shared__ __align__(16) float gs[64 * NP];
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
    for (int rc = r_begin; rc < r_end; rc += 64) {
        const int rows = (r_end - rc) < 64 ? (r_end - rc) : 64;
        __syncthreads();
        for (int e = tid; e < 64 * NP; e += 128) {
            const int r = e / NP, j = e % NP;
            gs[e] = (r < rows && j < n) ? __ldg(g + size_t(rc + r) * n + j) : 0.f;
        }
        __syncthreads();
        if (p < k) {
            for (int r = 0; r < rows; ++r) {
                const float *src = a + size_t(rc + r) * k + p;
                float av[4];
                if (full) {
                    const float4 q = __ldg(reinterpret_cast<const float4 *>(src));
                    av[0] = q.x; av[1] = q.y; av[2] = q.z; av[3] = q.w;
                } else {
#pragma unroll
                    for (int u = 0; u < 4; ++u) av[u] = (p + u < k) ? __ldg(src + u) : 0.f;
                }
#pragma unroll
                for (int j = 0; j < NP; ++j) {
                    const float gv = gs[r * NP + j];
#pragma unroll
                    for (int u = 0; u < 4; ++u) acc[u][j] = fmaf(av[u], gv, acc[u][j]);
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
    const size_t row_blocks = katsu_div_up(m, 32);
    size_t splits = katsu_div_up(size_t(ctx->num_sms) * 4, row_blocks);
    const size_t max_splits = katsu_div_up(k, (size_t)SK_KC);
    if (splits > max_splits) splits = max_splits;
    if (splits > 65535) splits = 65535;
    size_t k_per_split = katsu_div_up(katsu_div_up(k, splits), (size_t)SK_KC) * SK_KC;
    splits = katsu_div_up(k, k_per_split);
    float *partial = nullptr;
    KATSU_TRY(katsu_scratch(ctx, splits * m * n, &partial));
    const int vec_ok = aligned16(a) && (k % 4 == 0);
    dim3 grid((unsigned)row_blocks, (unsigned)splits);
    KATSU_LAUNCH(ctx, skinny_fwd_kernel<NP>, grid, 256, 0, a, b, partial, (int)m, k, (int)n, k_per_split, vec_ok);
    KATSU_LAUNCH(ctx, fold_partials_kernel, (unsigned)katsu_div_up(m * n, 256), 256, 0, partial, c, m * n,
                 (int)splits, 0);
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
    return n >= 1 && n <= 16 && k >= 2048 && m <= 0x7fffffff && katsu_div_up(k, 512) <= 0x7fffffff &&
           katsu_div_up(m, 32) <= 0x7fffffff && katsu_div_up(m, 64) <= 65535;
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
