/*
 * katsu_oracle.c -- CPU restatement of katsu-core's dense hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing the library ships may call into this
 * file: it exists so the tests, the smoke check and the benchmark's CPU
 * baseline leg have an independent statement of what the reference computes.
 *
 * Every loop below follows the reference's loop order and arithmetic:
 * f32 storage, f32 accumulators, a rounded multiply followed by a rounded
 * add (build with -ffp-contract=off and without -ffast-math so the compiler
 * neither fuses nor reorders), left-to-right sums.  The reference is Rust and
 * cannot be compiled where this file is built, so parity is pinned by the
 * known-answer vectors of the reference's own integration tests
 * (crates/katsu-core/tests/{conv2d,autograd,tensor}.rs), restated under
 * tests/test_oracle_pins.py.
 *
 * Entry points (all extern "C"-style, plain pointers and sizes):
 *   ko_conv2d_geometry       crates/katsu-core/src/conv2d.rs:183-224
 *   ko_conv2d_forward        crates/katsu-core/src/conv2d.rs:95-103, 232-262
 *   ko_conv2d_backward       crates/katsu-core/src/conv2d.rs:269-292
 *   ko_matmul                crates/katsu-core/src/tensor.rs:264-273
 *   ko_matmul_backward       crates/katsu-core/src/tensor.rs:418-445
 *   ko_add / ko_mul / ko_sum crates/katsu-core/src/tensor.rs:226-247
 *   ko_*_acc                 crates/katsu-core/src/tensor.rs:387-417, 353-356
 *   ko_splitmix_weights      crates/katsu-core/src/conv2d.rs:46-58
 *   *_mt variants            same sums, same order per element, threads over
 *                            independent elements only (bit-identical output)
 *   *_f64 variants           same index set, f64 accumulation ("exact" answer)
 *   ko_conv2d_sample_*       one element's full sum in reference order
 */
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define KO_OK 0
#define KO_INVALID_CONV 1
#define KO_SHAPE_OVERFLOW 2
#define KO_DATA_LENGTH 3

typedef struct {
    size_t batch, cin, cout, h, w, kh, kw, oh, ow, stride, padding;
} ko_geometry;

/* tensor.rs:127-138: zero if any dim is zero, else checked product capped at
 * isize::MAX / 4. */
static int ko_element_count(const size_t *shape, size_t rank, size_t *out) {
    size_t i, count = 1;
    for (i = 0; i < rank; ++i)
        if (shape[i] == 0) { *out = 0; return KO_OK; }
    for (i = 0; i < rank; ++i) {
        if (__builtin_mul_overflow(count, shape[i], &count)) return KO_SHAPE_OVERFLOW;
    }
    if (count > ((size_t)INTPTR_MAX) / sizeof(float)) return KO_SHAPE_OVERFLOW;
    *out = count;
    return KO_OK;
}

int ko_element_count_checked(const size_t *shape, size_t rank, size_t *out) {
    return ko_element_count(shape, rank, out);
}

/* conv2d.rs:183-224 (Geometry::new) with validate_weights (conv2d.rs:156-166).
 * x_shape / w_shape carry their ranks so that rank errors are reproduced. */
int ko_conv2d_geometry(const size_t *x_shape, size_t x_rank,
                       const size_t *w_shape, size_t w_rank,
                       size_t stride, size_t padding, ko_geometry *g) {
    size_t i, pad2, tmp, dims[4];
    int rc;
    if (w_rank != 4) return KO_INVALID_CONV;
    for (i = 0; i < 4; ++i) if (w_shape[i] == 0) return KO_INVALID_CONV;
    if (stride == 0) return KO_INVALID_CONV;
    if (x_rank != 4) return KO_INVALID_CONV;
    if (x_shape[1] != w_shape[1] || x_shape[2] == 0 || x_shape[3] == 0) return KO_INVALID_CONV;
    rc = ko_element_count(x_shape + 1, 3, &tmp);
    if (rc) return rc;
    if (__builtin_mul_overflow(padding, (size_t)2, &pad2)) return KO_SHAPE_OVERFLOW;
    {
        size_t sizes[2] = { x_shape[2], x_shape[3] };
        size_t kernels[2] = { w_shape[2], w_shape[3] };
        size_t outs[2];
        for (i = 0; i < 2; ++i) {
            size_t padded;
            if (__builtin_add_overflow(sizes[i], pad2, &padded)) return KO_SHAPE_OVERFLOW;
            if (padded < kernels[i]) return KO_INVALID_CONV;
            outs[i] = (padded - kernels[i]) / stride;
            if (__builtin_add_overflow(outs[i], (size_t)1, &outs[i])) return KO_SHAPE_OVERFLOW;
        }
        g->oh = outs[0];
        g->ow = outs[1];
    }
    dims[0] = w_shape[0]; dims[1] = g->oh; dims[2] = g->ow;
    rc = ko_element_count(dims, 3, &tmp);
    if (rc) return rc;
    dims[0] = x_shape[0]; dims[1] = w_shape[0]; dims[2] = g->oh; dims[3] = g->ow;
    rc = ko_element_count(dims, 4, &tmp);
    if (rc) return rc;
    g->batch = x_shape[0]; g->cin = x_shape[1]; g->cout = w_shape[0];
    g->h = x_shape[2]; g->w = x_shape[3]; g->kh = w_shape[2]; g->kw = w_shape[3];
    g->stride = stride; g->padding = padding;
    return KO_OK;
}

static ko_geometry ko_geom(size_t n, size_t c, size_t h, size_t w, size_t k,
                           size_t r, size_t s, size_t stride, size_t padding) {
    ko_geometry g;
    g.batch = n; g.cin = c; g.cout = k; g.h = h; g.w = w; g.kh = r; g.kw = s;
    g.stride = stride; g.padding = padding;
    g.oh = (h + 2 * padding - r) / stride + 1;
    g.ow = (w + 2 * padding - s) / stride + 1;
    return g;
}

/*
 * The visit loop (conv2d.rs:232-262), order n, oc, oy, ox, ic, ky, kx, with
 * the padding test written as the reference writes it: p = o*stride + k,
 * skip unless p >= padding and p - padding < size.  BODY is the closure the
 * reference passes to visit; it sees xi, wi and yi.  N0/N1 and OC0/OC1
 * restrict the two outer loops for the threaded variants.
 */
#define KO_VISIT(G, N0, N1, OC0, OC1, BODY)                                            \
    do {                                                                               \
        size_t n_, oc_, oy_, ox_, ic_, ky_, kx_;                                       \
        for (n_ = (N0); n_ < (N1); ++n_)                                               \
        for (oc_ = (OC0); oc_ < (OC1); ++oc_)                                          \
        for (oy_ = 0; oy_ < (G).oh; ++oy_)                                             \
        for (ox_ = 0; ox_ < (G).ow; ++ox_) {                                           \
            const size_t yi = ((n_ * (G).cout + oc_) * (G).oh + oy_) * (G).ow + ox_;   \
            for (ic_ = 0; ic_ < (G).cin; ++ic_)                                        \
            for (ky_ = 0; ky_ < (G).kh; ++ky_) {                                       \
                const size_t py_ = oy_ * (G).stride + ky_;                             \
                size_t iy_, xbase_, wbase_;                                            \
                if (py_ < (G).padding) continue;                                       \
                iy_ = py_ - (G).padding;                                               \
                if (iy_ >= (G).h) continue;                                            \
                xbase_ = ((n_ * (G).cin + ic_) * (G).h + iy_) * (G).w;                 \
                wbase_ = ((oc_ * (G).cin + ic_) * (G).kh + ky_) * (G).kw;              \
                for (kx_ = 0; kx_ < (G).kw; ++kx_) {                                   \
                    const size_t px_ = ox_ * (G).stride + kx_;                         \
                    if (px_ >= (G).padding && px_ - (G).padding < (G).w) {             \
                        const size_t xi = xbase_ + (px_ - (G).padding);                \
                        const size_t wi = wbase_ + kx_;                                \
                        BODY                                                           \
                    }                                                                  \
                }                                                                      \
            }                                                                          \
        }                                                                              \
    } while (0)

/* conv2d.rs:95-103: y starts at zero, y[yi] += x[xi] * w[wi]. */
void ko_conv2d_forward(const float *x, const float *w, float *y,
                       size_t n, size_t c, size_t h, size_t wd, size_t k,
                       size_t r, size_t s, size_t stride, size_t padding) {
    ko_geometry g = ko_geom(n, c, h, wd, k, r, s, stride, padding);
    memset(y, 0, sizeof(float) * n * k * g.oh * g.ow);
    KO_VISIT(g, 0, g.batch, 0, g.cout, { y[yi] += x[xi] * w[wi]; });
}

/* conv2d.rs:283-290: fresh zero dx and dw, one visit doing both updates. */
void ko_conv2d_backward(const float *x, const float *w, const float *grad,
                        float *dx, float *dw,
                        size_t n, size_t c, size_t h, size_t wd, size_t k,
                        size_t r, size_t s, size_t stride, size_t padding) {
    ko_geometry g = ko_geom(n, c, h, wd, k, r, s, stride, padding);
    memset(dx, 0, sizeof(float) * n * c * h * wd);
    memset(dw, 0, sizeof(float) * k * c * r * s);
    KO_VISIT(g, 0, g.batch, 0, g.cout, {
        dx[xi] += grad[yi] * w[wi];
        dw[wi] += grad[yi] * x[xi];
    });
}

/*
 * Threaded variants.  They split only over loop indices that never share an
 * output element (n and oc for y; n for dx; oc for dw), so each element still
 * receives its terms in the reference's order and the results are bit-equal
 * to the single-threaded functions above.  Used to generate full-size golden
 * data in reasonable time and as the "all host threads" reference arm.
 */
void ko_conv2d_forward_mt(const float *x, const float *w, float *y,
                          size_t n, size_t c, size_t h, size_t wd, size_t k,
                          size_t r, size_t s, size_t stride, size_t padding) {
    ko_geometry g = ko_geom(n, c, h, wd, k, r, s, stride, padding);
    long job, jobs = (long)(n * k);
    memset(y, 0, sizeof(float) * n * k * g.oh * g.ow);
#pragma omp parallel for schedule(dynamic, 1)
    for (job = 0; job < jobs; ++job) {
        size_t nn = (size_t)job / k, oc = (size_t)job % k;
        KO_VISIT(g, nn, nn + 1, oc, oc + 1, { y[yi] += x[xi] * w[wi]; });
    }
}

void ko_conv2d_backward_mt(const float *x, const float *w, const float *grad,
                           float *dx, float *dw,
                           size_t n, size_t c, size_t h, size_t wd, size_t k,
                           size_t r, size_t s, size_t stride, size_t padding) {
    ko_geometry g = ko_geom(n, c, h, wd, k, r, s, stride, padding);
    long job;
    memset(dx, 0, sizeof(float) * n * c * h * wd);
    memset(dw, 0, sizeof(float) * k * c * r * s);
#pragma omp parallel
    {
#pragma omp for schedule(dynamic, 1) nowait
        for (job = 0; job < (long)n; ++job) {
            size_t nn = (size_t)job;
            KO_VISIT(g, nn, nn + 1, 0, g.cout, { dx[xi] += grad[yi] * w[wi]; });
        }
#pragma omp for schedule(dynamic, 1)
        for (job = 0; job < (long)k; ++job) {
            size_t oc = (size_t)job;
            KO_VISIT(g, 0, g.batch, oc, oc + 1, { dw[wi] += grad[yi] * x[xi]; });
        }
    }
}

/* Same index set with f64 accumulators: the answer the f32 sums approximate. */
void ko_conv2d_forward_f64(const float *x, const float *w, double *y,
                           size_t n, size_t c, size_t h, size_t wd, size_t k,
                           size_t r, size_t s, size_t stride, size_t padding) {
    ko_geometry g = ko_geom(n, c, h, wd, k, r, s, stride, padding);
    long job, jobs = (long)(n * k);
    memset(y, 0, sizeof(double) * n * k * g.oh * g.ow);
#pragma omp parallel for schedule(dynamic, 1)
    for (job = 0; job < jobs; ++job) {
        size_t nn = (size_t)job / k, oc = (size_t)job % k;
        KO_VISIT(g, nn, nn + 1, oc, oc + 1, { y[yi] += (double)x[xi] * (double)w[wi]; });
    }
}

void ko_conv2d_backward_f64(const float *x, const float *w, const float *grad,
                            double *dx, double *dw,
                            size_t n, size_t c, size_t h, size_t wd, size_t k,
                            size_t r, size_t s, size_t stride, size_t padding) {
    ko_geometry g = ko_geom(n, c, h, wd, k, r, s, stride, padding);
    long job;
    memset(dx, 0, sizeof(double) * n * c * h * wd);
    memset(dw, 0, sizeof(double) * k * c * r * s);
#pragma omp parallel
    {
#pragma omp for schedule(dynamic, 1) nowait
        for (job = 0; job < (long)n; ++job) {
            size_t nn = (size_t)job;
            KO_VISIT(g, nn, nn + 1, 0, g.cout, { dx[xi] += (double)grad[yi] * (double)w[wi]; });
        }
#pragma omp for schedule(dynamic, 1)
        for (job = 0; job < (long)k; ++job) {
            size_t oc = (size_t)job;
            KO_VISIT(g, 0, g.batch, oc, oc + 1, { dw[wi] += (double)grad[yi] * (double)x[xi]; });
        }
    }
}

/*
 * Sampled oracle: the full sum of single elements, visited in the order the
 * reference's loop nest reaches them.  out32 gets the f32 left-to-right sum,
 * out64 the f64 sum of the same terms.  Lets full-size tensors be checked
 * without running the whole 7-deep loop on the CPU.
 */
void ko_conv2d_sample_y(const float *x, const float *w, const size_t *idx, size_t count,
                        float *out32, double *out64,
                        size_t n, size_t c, size_t h, size_t wd, size_t k,
                        size_t r, size_t s, size_t stride, size_t padding) {
    ko_geometry g = ko_geom(n, c, h, wd, k, r, s, stride, padding);
    long q;
#pragma omp parallel for schedule(static)
    for (q = 0; q < (long)count; ++q) {
        size_t yi = idx[q];
        size_t ox = yi % g.ow, oy = (yi / g.ow) % g.oh;
        size_t oc = (yi / (g.ow * g.oh)) % g.cout, nn = yi / (g.ow * g.oh * g.cout);
        float a32 = 0.0f; double a64 = 0.0;
        size_t ic, ky, kx;
        for (ic = 0; ic < g.cin; ++ic)
        for (ky = 0; ky < g.kh; ++ky) {
            size_t py = oy * g.stride + ky, iy;
            if (py < g.padding) continue;
            iy = py - g.padding;
            if (iy >= g.h) continue;
            for (kx = 0; kx < g.kw; ++kx) {
                size_t px = ox * g.stride + kx, ix;
                if (px < g.padding) continue;
                ix = px - g.padding;
                if (ix >= g.w) continue;
                {
                    float xv = x[((nn * g.cin + ic) * g.h + iy) * g.w + ix];
                    float wv = w[((oc * g.cin + ic) * g.kh + ky) * g.kw + kx];
                    a32 += xv * wv;
                    a64 += (double)xv * (double)wv;
                }
            }
        }
        out32[q] = a32; out64[q] = a64;
    }
}

void ko_conv2d_sample_dx(const float *w, const float *grad, const size_t *idx, size_t count,
                         float *out32, double *out64,
                         size_t n, size_t c, size_t h, size_t wd, size_t k,
                         size_t r, size_t s, size_t stride, size_t padding) {
    ko_geometry g = ko_geom(n, c, h, wd, k, r, s, stride, padding);
    long q;
#pragma omp parallel for schedule(static)
    for (q = 0; q < (long)count; ++q) {
        size_t xi = idx[q];
        size_t ix = xi % g.w, iy = (xi / g.w) % g.h;
        size_t ic = (xi / (g.w * g.h)) % g.cin, nn = xi / (g.w * g.h * g.cin);
        float a32 = 0.0f; double a64 = 0.0;
        size_t oc, oy, ox;
        /* visit order for a fixed (n, ic, iy, ix): oc, oy, ox ascending; each
         * (oy, ox) reaches this input element through at most one (ky, kx). */
        for (oc = 0; oc < g.cout; ++oc)
        for (oy = 0; oy < g.oh; ++oy) {
            size_t py = iy + g.padding, ky;
            if (oy * g.stride > py) break;
            ky = py - oy * g.stride;
            if (ky >= g.kh) continue;
            for (ox = 0; ox < g.ow; ++ox) {
                size_t px = ix + g.padding, kx;
                if (ox * g.stride > px) break;
                kx = px - ox * g.stride;
                if (kx >= g.kw) continue;
                {
                    float gv = grad[((nn * g.cout + oc) * g.oh + oy) * g.ow + ox];
                    float wv = w[((oc * g.cin + ic) * g.kh + ky) * g.kw + kx];
                    a32 += gv * wv;
                    a64 += (double)gv * (double)wv;
                }
            }
        }
        out32[q] = a32; out64[q] = a64;
    }
}

void ko_conv2d_sample_dw(const float *x, const float *grad, const size_t *idx, size_t count,
                         float *out32, double *out64,
                         size_t n, size_t c, size_t h, size_t wd, size_t k,
                         size_t r, size_t s, size_t stride, size_t padding) {
    ko_geometry g = ko_geom(n, c, h, wd, k, r, s, stride, padding);
    long q;
#pragma omp parallel for schedule(dynamic, 1)
    for (q = 0; q < (long)count; ++q) {
        size_t wi = idx[q];
        size_t kx = wi % g.kw, ky = (wi / g.kw) % g.kh;
        size_t ic = (wi / (g.kw * g.kh)) % g.cin, oc = wi / (g.kw * g.kh * g.cin);
        float a32 = 0.0f; double a64 = 0.0;
        size_t nn, oy, ox;
        for (nn = 0; nn < g.batch; ++nn)
        for (oy = 0; oy < g.oh; ++oy) {
            size_t py = oy * g.stride + ky, iy;
            if (py < g.padding) continue;
            iy = py - g.padding;
            if (iy >= g.h) continue;
            for (ox = 0; ox < g.ow; ++ox) {
                size_t px = ox * g.stride + kx, ix;
                if (px < g.padding) continue;
                ix = px - g.padding;
                if (ix >= g.w) continue;
                {
                    float gv = grad[((nn * g.cout + oc) * g.oh + oy) * g.ow + ox];
                    float xv = x[((nn * g.cin + ic) * g.h + iy) * g.w + ix];
                    a32 += gv * xv;
                    a64 += (double)gv * (double)xv;
                }
            }
        }
        out32[q] = a32; out64[q] = a64;
    }
}

/* tensor.rs:264-273: c zero-filled, loops i, p, j; skipped when m*n == 0 or k == 0. */
void ko_matmul(const float *a, const float *b, float *c, size_t m, size_t k, size_t n) {
    size_t i, p, j;
    memset(c, 0, sizeof(float) * m * n);
    if (m * n == 0 || k == 0) return;
    for (i = 0; i < m; ++i)
        for (p = 0; p < k; ++p)
            for (j = 0; j < n; ++j)
                c[i * n + j] += a[i * k + p] * b[p * n + j];
}

/* tensor.rs:418-445: da and db are the pending adjoints and are accumulated
 * into (not overwritten); early-out when g is empty or k == 0.  Either output
 * may be NULL to skip it.  When a and b are the same node the caller passes the
 * same buffer for da and db and both loops add into it, da first. */
void ko_matmul_backward(const float *a, const float *b, const float *g,
                        float *da, float *db, size_t m, size_t k, size_t n) {
    size_t i, p, j;
    if (m * n == 0 || k == 0) return;
    if (da)
        for (i = 0; i < m; ++i)
            for (p = 0; p < k; ++p)
                for (j = 0; j < n; ++j)
                    da[i * k + p] += g[i * n + j] * b[p * n + j];
    if (db)
        for (i = 0; i < m; ++i)
            for (p = 0; p < k; ++p)
                for (j = 0; j < n; ++j)
                    db[p * n + j] += a[i * k + p] * g[i * n + j];
}

/* Threaded, bit-identical: rows of c / da are independent; db[p,:] sums over i
 * ascending for every p, so threads split p. */
void ko_matmul_mt(const float *a, const float *b, float *c, size_t m, size_t k, size_t n) {
    long i;
    memset(c, 0, sizeof(float) * m * n);
    if (m * n == 0 || k == 0) return;
#pragma omp parallel for schedule(static)
    for (i = 0; i < (long)m; ++i) {
        size_t p, j;
        for (p = 0; p < k; ++p)
            for (j = 0; j < n; ++j)
                c[i * n + j] += a[i * k + p] * b[p * n + j];
    }
}

void ko_matmul_backward_mt(const float *a, const float *b, const float *g,
                           float *da, float *db, size_t m, size_t k, size_t n) {
    long q;
    if (m * n == 0 || k == 0) return;
    if (da) {
#pragma omp parallel for schedule(static)
        for (q = 0; q < (long)m; ++q) {
            size_t i = (size_t)q, p, j;
            for (p = 0; p < k; ++p)
                for (j = 0; j < n; ++j)
                    da[i * k + p] += g[i * n + j] * b[p * n + j];
        }
    }
    if (db) {
#pragma omp parallel for schedule(static)
        for (q = 0; q < (long)k; ++q) {
            size_t p = (size_t)q, i, j;
            for (i = 0; i < m; ++i)
                for (j = 0; j < n; ++j)
                    db[p * n + j] += a[i * k + p] * g[i * n + j];
        }
    }
}

void ko_matmul_f64(const float *a, const float *b, double *c, size_t m, size_t k, size_t n) {
    long i;
    memset(c, 0, sizeof(double) * m * n);
    if (m * n == 0 || k == 0) return;
#pragma omp parallel for schedule(static)
    for (i = 0; i < (long)m; ++i) {
        size_t p, j;
        for (p = 0; p < k; ++p)
            for (j = 0; j < n; ++j)
                c[i * n + j] += (double)a[i * k + p] * (double)b[p * n + j];
    }
}

/* f64 VJP of matmul, overwriting (not accumulating) da and db. */
void ko_matmul_backward_f64(const float *a, const float *b, const float *g,
                            double *da, double *db, size_t m, size_t k, size_t n) {
    long q;
    if (da) memset(da, 0, sizeof(double) * m * k);
    if (db) memset(db, 0, sizeof(double) * k * n);
    if (m * n == 0 || k == 0) return;
    if (da) {
#pragma omp parallel for schedule(static)
        for (q = 0; q < (long)m; ++q) {
            size_t i = (size_t)q, p, j;
            for (p = 0; p < k; ++p)
                for (j = 0; j < n; ++j)
                    da[i * k + p] += (double)g[i * n + j] * (double)b[p * n + j];
        }
    }
    if (db) {
#pragma omp parallel for schedule(static)
        for (q = 0; q < (long)k; ++q) {
            size_t p = (size_t)q, i, j;
            for (i = 0; i < m; ++i)
                for (j = 0; j < n; ++j)
                    db[p * n + j] += (double)a[i * k + p] * (double)g[i * n + j];
        }
    }
}

/* tensor.rs:226-233 */
void ko_add(const float *a, const float *b, float *out, size_t count) {
    size_t i;
    for (i = 0; i < count; ++i) out[i] = a[i] + b[i];
}

void ko_mul(const float *a, const float *b, float *out, size_t count) {
    size_t i;
    for (i = 0; i < count; ++i) out[i] = a[i] * b[i];
}

/* tensor.rs:245: iter().sum() is a sequential left fold in f32. */
float ko_sum(const float *a, size_t count) {
    size_t i;
    float acc = 0.0f;
    for (i = 0; i < count; ++i) acc += a[i];
    return acc;
}

double ko_sum_f64(const float *a, size_t count) {
    size_t i;
    double acc = 0.0;
    for (i = 0; i < count; ++i) acc += (double)a[i];
    return acc;
}

/* tensor.rs:387-389 and 353-356 and the Add arm of 400-408: dst[i] += g[i]. */
void ko_axpy_acc(float *dst, const float *g, size_t count) {
    size_t i;
    for (i = 0; i < count; ++i) dst[i] += g[i];
}

/* Mul arm of tensor.rs:400-408: dst[i] += g[i] * other[i]. */
void ko_mul_acc(float *dst, const float *g, const float *other, size_t count) {
    size_t i;
    for (i = 0; i < count; ++i) dst[i] += g[i] * other[i];
}

/* tensor.rs:410-417: dst[i] += g[0]. */
void ko_bcast_acc(float *dst, const float *g, size_t count) {
    size_t i;
    for (i = 0; i < count; ++i) dst[i] += g[0];
}

/* SplitMix64 step of conv2d.rs:49-56; returns u in [0, 1) with 24 bits. */
static float ko_splitmix_uniform(uint64_t *state) {
    uint64_t z;
    *state += 0x9e3779b97f4a7c15ULL;
    z = *state;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
    z ^= z >> 31;
    return (float)(z >> 40) / 16777216.0f;
}

/* conv2d.rs:46-58: bound = 1/sqrt(fan_in as f32); w = (2u - 1) * bound. */
void ko_splitmix_weights(uint64_t seed, size_t count, size_t fan_in, float *out) {
    size_t i;
    float bound = 1.0f / sqrtf((float)fan_in);
    uint64_t state = seed;
    for (i = 0; i < count; ++i) {
        float u = ko_splitmix_uniform(&state);
        out[i] = (2.0f * u - 1.0f) * bound;
    }
}

int ko_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void ko_set_num_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}
