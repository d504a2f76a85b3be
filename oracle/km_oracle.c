/*
 * CPU oracle for the kernel-matmul hot path.  TEST INFRASTRUCTURE ONLY: nothing in the
 * shipped package may link, load or call this file; it is the checker that the CUDA path is
 * compared against (tests, the smoke check, and the CPU-baseline leg of the benchmark).
 *
 * It restates, in plain C with fp64 arithmetic, the algorithm of the reference project
 * Turakar/kernel-matmul.  Inputs are the same fp32 / int32 arrays the GPU path sees; every
 * intermediate and every output is double.  Each function cites the reference source it
 * follows (path within the reference project : lines).
 *
 * Parity pinning: the band routines below are checked bit-for-bit against the reference's own
 * native/ranges/ranges.cpp compiled unmodified (oracle/build_ref.py), and the products and
 * gradients against the reference's CUDA kernels run on a B200 (fixtures in tests/golden/).
 *
 * Layout convention: every array has a flattened leading batch index b in [0, B) and a
 * per-array batch stride in elements (0 = the same data for every batch); the trailing
 * dimensions are contiguous.
 *
 * Build:  gcc -O2 -fopenmp -fPIC -shared -o libkm_oracle.so km_oracle.c -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define KMO_RBF 0
#define KMO_SPECTRAL 1
#define KMO_LOCALLY_PERIODIC 2
#define KMO_MAX_PARAMS 4

static const double KMO_PI = 3.14159265358979323846;

int kmo_num_params(int kernel_type) {
    /* native/common/kernel_function.cuh:3-9 */
    switch (kernel_type) {
    case KMO_RBF: return 2;
    case KMO_SPECTRAL: return 3;
    case KMO_LOCALLY_PERIODIC: return 4;
    default: return -1;
    }
}

/* theta (user parameters) -> p (device parameters).
 * native/common/kernel_function.cuh:198-219 (transform_params). */
static void kmo_transform(int kt, const double *theta, double *p) {
    switch (kt) {
    case KMO_RBF:
        p[0] = 0.5 / (theta[0] * theta[0]);
        p[1] = theta[1];
        break;
    case KMO_SPECTRAL:
        p[0] = 0.5 / (theta[0] * theta[0]);
        p[1] = 2.0 * theta[1];
        p[2] = theta[2];
        break;
    case KMO_LOCALLY_PERIODIC:
        p[0] = 0.5 / (theta[0] * theta[0]);
        p[1] = 2.0 / theta[1];
        p[2] = 1.0 / theta[2];
        p[3] = theta[3];
        break;
    }
}

/* Gradient wrt p -> gradient wrt theta.
 * native/common/kernel_function.cuh:221-251 (transform_params_grad). */
static void kmo_transform_grad(int kt, const double *theta, const double *gp, double *gt) {
    switch (kt) {
    case KMO_RBF:
        gt[0] = gp[0] * (-1.0 / (theta[0] * theta[0] * theta[0]));
        gt[1] = gp[1];
        break;
    case KMO_SPECTRAL:
        gt[0] = gp[0] * (-1.0 / (theta[0] * theta[0] * theta[0]));
        gt[1] = gp[1] * 2.0;
        gt[2] = gp[2];
        break;
    case KMO_LOCALLY_PERIODIC:
        gt[0] = gp[0] * (-1.0 / (theta[0] * theta[0] * theta[0]));
        gt[1] = gp[1] * (-2.0 / (theta[1] * theta[1]));
        gt[2] = gp[2] * (-1.0 / (theta[2] * theta[2]));
        gt[3] = gp[3];
        break;
    }
}

/* kappa(x1, x2; p).  native/common/kernel_function.cuh:25-58 (kernel_function). */
static double kmo_value(int kt, double x1, double x2, const double *p) {
    const double d = x1 - x2;
    switch (kt) {
    case KMO_RBF:
        return p[1] * exp(-(d * d) * p[0]);
    case KMO_SPECTRAL:
        return p[2] * exp(-p[0] * d * d) * cos(KMO_PI * (p[1] * d));
    case KMO_LOCALLY_PERIODIC: {
        const double s = sin(KMO_PI * (p[2] * d));
        return p[3] * exp(-(d * d * p[0] + s * s * p[1]));
    }
    }
    return 0.0;
}

/* d kappa / d p_i.  native/common/kernel_function.cuh:92-163 (kernel_function_bwd). */
static void kmo_value_bwd(int kt, double x1, double x2, const double *p, double *g) {
    const double d = x1 - x2;
    const double dsq = d * d;
    switch (kt) {
    case KMO_RBF: {
        const double e = exp(-dsq * p[0]);
        g[0] = -(p[1] * e) * dsq;
        g[1] = e;
        break;
    }
    case KMO_SPECTRAL: {
        const double a = KMO_PI * (p[1] * d);
        const double sn = sin(a), cs = cos(a);
        const double e = exp(-p[0] * dsq);
        g[0] = -(p[2] * e * cs) * dsq;
        g[1] = -KMO_PI * p[2] * e * sn * d;
        g[2] = e * cs;
        break;
    }
    case KMO_LOCALLY_PERIODIC: {
        const double a = KMO_PI * (p[2] * d);
        const double sn = sin(a), cs = cos(a);
        const double e = exp(-(dsq * p[0] + sn * sn * p[1]));
        const double v = p[3] * e;
        g[0] = -v * dsq;
        g[1] = -v * sn * sn;
        g[2] = -(2.0 * KMO_PI) * v * p[1] * sn * cs * d;
        g[3] = e;
        break;
    }
    }
}

static void kmo_load_params(int kt, const float *theta32, double *theta, double *p) {
    const int P = kmo_num_params(kt);
    for (int i = 0; i < P; i++) theta[i] = (double)theta32[i];
    kmo_transform(kt, theta, p);
}

static inline int kmo_min(int a, int b) { return a < b ? a : b; }
static inline int kmo_max(int a, int b) { return a > b ? a : b; }

/* Clamp a band to the valid column range.  The symmetric band routine may return
 * end[0] = block_size > n when n < block_size (native/ranges/ranges.cpp:83,93); the reference
 * kernels never dereference beyond it only because their tests avoid that case. */
static inline void kmo_band(const int32_t *start, const int32_t *end, int r, int n, int *s, int *e) {
    *s = kmo_max(0, kmo_min(start[r], n));
    *e = kmo_max(*s, kmo_min(end[r], n));
}

/*
 * out[b, m, :] = sum_{j in [start[b,r], end[b,r])} kappa(x1[b,m], x2[b,j]) * rhs[b, j, :],
 * r = m / block.  The semantics of the reference product kernel
 * (native/matmul/matmul.cu:13-157: one row block sees one column range; rows >= m and
 * columns >= end are masked) followed by its column-slab sum (matmul.cu:202), which is the
 * dense formulation "materialise K, zero outside the ranges, matmul" of the reference tests
 * (tests/conftest.py:243-249, tests/native/test_matmul.py:27).
 *
 * row_blocks == NULL: all R = ceil(m/block) row blocks, out is (B, m, k).
 * row_blocks != NULL: only the listed n_row_blocks blocks, out is (B, n_row_blocks, block, k)
 *                     (rows past m are left zero).
 */
void kmo_matmul(int kt, int64_t B, int m, int n, int k, int block,
                const float *x1, int64_t x1_bs, const float *x2, int64_t x2_bs,
                const float *rhs, int64_t rhs_bs, const float *theta, int64_t theta_bs,
                const int32_t *start, const int32_t *end, int64_t range_bs,
                const int32_t *row_blocks, int n_row_blocks, double *out) {
    const int R = (m + block - 1) / block;
    const int nblk = row_blocks ? n_row_blocks : R;
    const int64_t total = B * (int64_t)nblk;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t w = 0; w < total; w++) {
        const int64_t b = w / nblk;
        const int bi = (int)(w % nblk);
        const int r = row_blocks ? row_blocks[bi] : bi;
        double th[KMO_MAX_PARAMS], p[KMO_MAX_PARAMS];
        kmo_load_params(kt, theta + b * theta_bs, th, p);
        int s, e;
        kmo_band(start + b * range_bs, end + b * range_bs, r, n, &s, &e);
        const float *x1b = x1 + b * x1_bs, *x2b = x2 + b * x2_bs, *rb = rhs + b * rhs_bs;
        const int row0 = r * block, row1 = kmo_min(row0 + block, m);
        for (int i = row0; i < row1; i++) {
            double *o = row_blocks ? out + ((b * nblk + bi) * (int64_t)block + (i - row0)) * k
                                   : out + (b * (int64_t)m + i) * k;
            for (int c = 0; c < k; c++) o[c] = 0.0;
            const double xi = (double)x1b[i];
            for (int j = s; j < e; j++) {
                const double v = kmo_value(kt, xi, (double)x2b[j], p);
                const float *rr = rb + (int64_t)j * k;
                for (int c = 0; c < k; c++) o[c] += v * (double)rr[c];
            }
        }
    }
}

/*
 * grad[b, q] = d/d theta_q  sum_{m, j in band, c} left[b,m,c] * kappa(x1[b,m], x2[b,j]) * right[b,j,c].
 *
 * This one contraction is both reference gradient ops:
 *  - native/bilinear_derivative/bilinear_derivative.cu:12-183 (left = left_vecs, right = right_vecs),
 *  - native/matmul_bwd/matmul_bwd.cu:12-221 (left = out_grad, right = rhs),
 * each followed by the chain rule transform_params_grad (kernel_function.cuh:221-251).
 * It equals autograd through the masked dense formulation used by the reference tests
 * (tests/native/test_matmul_bwd.py:26-27, tests/native/test_bilinear_derivative.py:35-40).
 * out: (B, P) doubles.  absolute != 0 returns the sum of the MAGNITUDES of the terms instead
 * (the scale that bounds the rounding error of any finite-precision evaluation of the sum;
 * used by the tests to assess results whose terms cancel).
 */
void kmo_bilinear_derivative(int kt, int64_t B, int m, int n, int k, int block,
                             const float *x1, int64_t x1_bs, const float *x2, int64_t x2_bs,
                             const float *left, int64_t left_bs, const float *right, int64_t right_bs,
                             const float *theta, int64_t theta_bs,
                             const int32_t *start, const int32_t *end, int64_t range_bs,
                             int absolute, double *out) {
    const int P = kmo_num_params(kt);
    const int R = (m + block - 1) / block;
    for (int64_t b = 0; b < B; b++) {
        double th[KMO_MAX_PARAMS], p[KMO_MAX_PARAMS];
        kmo_load_params(kt, theta + b * theta_bs, th, p);
        const float *x1b = x1 + b * x1_bs, *x2b = x2 + b * x2_bs;
        const float *lb = left + b * left_bs, *rb = right + b * right_bs;
        double acc0 = 0, acc1 = 0, acc2 = 0, acc3 = 0;
#pragma omp parallel for schedule(dynamic, 1) reduction(+ : acc0, acc1, acc2, acc3)
        for (int r = 0; r < R; r++) {
            int s, e;
            kmo_band(start + b * range_bs, end + b * range_bs, r, n, &s, &e);
            const int row1 = kmo_min((r + 1) * block, m);
            double a[KMO_MAX_PARAMS] = {0, 0, 0, 0};
            for (int i = r * block; i < row1; i++) {
                const double xi = (double)x1b[i];
                const float *li = lb + (int64_t)i * k;
                for (int j = s; j < e; j++) {
                    const float *rj = rb + (int64_t)j * k;
                    double coeff = 0.0;
                    for (int c = 0; c < k; c++) coeff += (double)li[c] * (double)rj[c];
                    double g[KMO_MAX_PARAMS];
                    kmo_value_bwd(kt, xi, (double)x2b[j], p, g);
                    for (int q = 0; q < P; q++) a[q] += absolute ? fabs(coeff * g[q]) : coeff * g[q];
                }
            }
            acc0 += a[0]; acc1 += a[1]; acc2 += a[2]; acc3 += a[3];
        }
        const double gp[KMO_MAX_PARAMS] = {acc0, acc1, acc2, acc3};
        double gt[KMO_MAX_PARAMS];
        kmo_transform_grad(kt, th, gp, gt);
        for (int q = 0; q < P; q++) out[b * P + q] = absolute ? fabs(gt[q]) : gt[q];
    }
}

/* Masked dense K, (B, m, n) doubles, exact zeros outside the band.
 * native/dense/dense.cu:12-98; masking loop of tests/conftest.py:243-249. */
void kmo_dense(int kt, int64_t B, int m, int n, int block,
               const float *x1, int64_t x1_bs, const float *x2, int64_t x2_bs,
               const float *theta, int64_t theta_bs,
               const int32_t *start, const int32_t *end, int64_t range_bs, double *out) {
    const int R = (m + block - 1) / block;
    memset(out, 0, sizeof(double) * (size_t)B * (size_t)m * (size_t)n);
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t w = 0; w < B * (int64_t)R; w++) {
        const int64_t b = w / R;
        const int r = (int)(w % R);
        double th[KMO_MAX_PARAMS], p[KMO_MAX_PARAMS];
        kmo_load_params(kt, theta + b * theta_bs, th, p);
        int s, e;
        kmo_band(start + b * range_bs, end + b * range_bs, r, n, &s, &e);
        const int row1 = kmo_min((r + 1) * block, m);
        for (int i = r * block; i < row1; i++)
            for (int j = s; j < e; j++)
                out[(b * (int64_t)m + i) * n + j] =
                    kmo_value(kt, (double)x1[b * x1_bs + i], (double)x2[b * x2_bs + j], p);
    }
}

/* grad[b, q] = d/d theta_q sum_{m, j in band} out_grad[b,m,j] * kappa.
 * native/dense_bwd/dense_bwd.cu:12-116; tests/native/test_dense_bwd.py:23-24. */
void kmo_dense_bwd(int kt, int64_t B, int m, int n, int block,
                   const float *x1, int64_t x1_bs, const float *x2, int64_t x2_bs,
                   const float *theta, int64_t theta_bs,
                   const int32_t *start, const int32_t *end, int64_t range_bs,
                   const float *out_grad, int64_t og_bs, int absolute, double *out) {
    const int P = kmo_num_params(kt);
    const int R = (m + block - 1) / block;
    for (int64_t b = 0; b < B; b++) {
        double th[KMO_MAX_PARAMS], p[KMO_MAX_PARAMS];
        kmo_load_params(kt, theta + b * theta_bs, th, p);
        double gp[KMO_MAX_PARAMS] = {0, 0, 0, 0};
        for (int r = 0; r < R; r++) {
            int s, e;
            kmo_band(start + b * range_bs, end + b * range_bs, r, n, &s, &e);
            const int row1 = kmo_min((r + 1) * block, m);
            for (int i = r * block; i < row1; i++)
                for (int j = s; j < e; j++) {
                    double g[KMO_MAX_PARAMS];
                    kmo_value_bwd(kt, (double)x1[b * x1_bs + i], (double)x2[b * x2_bs + j], p, g);
                    const double og = (double)out_grad[b * og_bs + (int64_t)i * n + j];
                    for (int q = 0; q < P; q++) gp[q] += absolute ? fabs(og * g[q]) : og * g[q];
                }
        }
        double gt[KMO_MAX_PARAMS];
        kmo_transform_grad(kt, th, gp, gt);
        for (int q = 0; q < P; q++) out[b * P + q] = absolute ? fabs(gt[q]) : gt[q];
    }
}

/*
 * Gather: out[l] = K[batch[l], row[l], col[l]] if start <= col < end for the row's block,
 * else 0.  native/index/index.cu:12-57.  batch[] holds flattened batch indices.
 * x1/x2/theta/ranges are addressed with per-array batch strides as elsewhere.
 */
void kmo_index(int kt, int64_t L, int block,
               const float *x1, int64_t x1_bs, const float *x2, int64_t x2_bs,
               const float *theta, int64_t theta_bs,
               const int32_t *start, const int32_t *end, int64_t range_bs,
               const int64_t *batch, const int32_t *row, const int32_t *col, double *out) {
#pragma omp parallel for
    for (int64_t l = 0; l < L; l++) {
        const int64_t b = batch[l];
        const int r = row[l] / block;
        const int s = start[b * range_bs + r], e = end[b * range_bs + r];
        double v = 0.0;
        if (s <= col[l] && col[l] < e) {
            double th[KMO_MAX_PARAMS], p[KMO_MAX_PARAMS];
            kmo_load_params(kt, theta + b * theta_bs, th, p);
            v = kmo_value(kt, (double)x1[b * x1_bs + row[l]], (double)x2[b * x2_bs + col[l]], p);
        }
        out[l] = v;
    }
}

/* grad[b, q] = d/d theta_q sum_l [batch[l]==b] out_grad[l] * K[b,row[l],col[l]] (in band).
 * native/index_bwd/index_bwd.cu:12-112; tests/native/test_index_bwd.py:27-28.  out: (B, P). */
void kmo_index_bwd(int kt, int64_t B, int64_t L, int block,
                   const float *x1, int64_t x1_bs, const float *x2, int64_t x2_bs,
                   const float *theta, int64_t theta_bs,
                   const int32_t *start, const int32_t *end, int64_t range_bs,
                   const int64_t *batch, const int32_t *row, const int32_t *col,
                   const float *out_grad, int absolute, double *out) {
    const int P = kmo_num_params(kt);
    double *gp = (double *)calloc((size_t)B * KMO_MAX_PARAMS, sizeof(double));
    for (int64_t l = 0; l < L; l++) {
        const int64_t b = batch[l];
        const int r = row[l] / block;
        const int s = start[b * range_bs + r], e = end[b * range_bs + r];
        if (s <= col[l] && col[l] < e) {
            double th[KMO_MAX_PARAMS], p[KMO_MAX_PARAMS], g[KMO_MAX_PARAMS];
            kmo_load_params(kt, theta + b * theta_bs, th, p);
            kmo_value_bwd(kt, (double)x1[b * x1_bs + row[l]], (double)x2[b * x2_bs + col[l]], p, g);
            for (int q = 0; q < P; q++) {
                const double t = (double)out_grad[l] * g[q];
                gp[b * KMO_MAX_PARAMS + q] += absolute ? fabs(t) : t;
            }
        }
    }
    for (int64_t b = 0; b < B; b++) {
        double th[KMO_MAX_PARAMS], p[KMO_MAX_PARAMS], gt[KMO_MAX_PARAMS];
        kmo_load_params(kt, theta + b * theta_bs, th, p);
        kmo_transform_grad(kt, th, gp + b * KMO_MAX_PARAMS, gt);
        for (int q = 0; q < P; q++) out[b * P + q] = absolute ? fabs(gt[q]) : gt[q];
    }
    free(gp);
}

/* ------------------------------------------------------------------------------------------
 * Band construction.  Sequential scans, all comparisons in fp32 exactly as the reference does
 * them (the cutoff arrives as a C float), so the integer outputs can be compared bit-for-bit.
 * x1: (B, m), x2: (B, n) contiguous; start/end: (B, R) with R = ceil(m / block).
 * ---------------------------------------------------------------------------------------- */

static inline int kmo_advance(int j, int step, int n) { return kmo_min(j + step, n); }

/* native/ranges/ranges.cpp:8-62 (make_ranges). */
void kmo_make_ranges(int64_t B, int m, int n, const float *x1, const float *x2, float cutoff,
                     int block, int align, int32_t *start, int32_t *end) {
    const int R = (m + block - 1) / block;
    const int step = align ? block : 1;
    for (int64_t b = 0; b < B; b++) {
        const float *a = x1 + b * (int64_t)m, *c = x2 + b * (int64_t)n;
        int32_t *S = start + b * (int64_t)R, *E = end + b * (int64_t)R;
        int prev_start = 0, prev_end = 0;
        for (int r = 0; r < R; r++) {
            const float first = a[r * block];
            const float last = a[kmo_min((r + 1) * block, m) - 1];
            int j = prev_start;
            while (j < n && !(first - c[j] <= cutoff)) j = kmo_advance(j, step, n);
            S[r] = j;
            int q = kmo_max(prev_end, j);
            while (q < n && !(c[q] - last > cutoff)) q = kmo_advance(q, step, n);
            E[r] = q;
            prev_start = j;
            prev_end = q;
        }
    }
}

/* native/ranges/ranges.cpp:64-101 (make_ranges_symmetric). */
void kmo_make_ranges_symmetric(int64_t B, int n, const float *x, float cutoff, int block,
                               int32_t *start, int32_t *end) {
    const int R = (n + block - 1) / block;
    for (int64_t b = 0; b < B; b++) {
        const float *a = x + b * (int64_t)n;
        int32_t *S = start + b * (int64_t)R, *E = end + b * (int64_t)R;
        for (int r = 0; r < R; r++) S[r] = n;
        if (R > 0) S[0] = 0;
        int j = block;
        for (int r = 0; r < R; r++) {
            const float last = a[kmo_min((r + 1) * block, n) - 1];
            while (j < n && !(a[j] - last >= cutoff)) j = kmo_advance(j, block, n);
            E[r] = j;
            const int reach = (j + block - 1) / block;
            for (int t = r; t < reach && t < R; t++) S[t] = kmo_min(S[t], r * block);
        }
    }
}

/* native/ranges/ranges.cpp:103-150 (transpose_ranges).  start/end: (B, R); outputs (B, C),
 * C = ceil(x2_size / block). */
void kmo_transpose_ranges(int64_t B, int R, const int32_t *start, const int32_t *end,
                          int x1_size, int x2_size, int block, int32_t *start_t, int32_t *end_t) {
    const int C = (x2_size + block - 1) / block;
    for (int64_t b = 0; b < B; b++) {
        const int32_t *S = start + b * (int64_t)R, *E = end + b * (int64_t)R;
        int32_t *St = start_t + b * (int64_t)C, *Et = end_t + b * (int64_t)C;
        for (int c = 0; c < C; c++) { St[c] = x1_size; Et[c] = 0; }
        for (int r = 0; r < R; r++) {
            if (S[r] == E[r]) continue;
            const int c0 = S[r] / block;
            const int c1 = (E[r] + block - 1) / block;
            const int row0 = r * block, row1 = kmo_min(row0 + block, x1_size);
            for (int c = c0; c < c1 && c < C; c++) {
                St[c] = kmo_min(St[c], row0);
                Et[c] = kmo_max(Et[c], row1);
            }
        }
        if (C > 0 && St[0] == x1_size) { St[0] = 0; Et[0] = 0; }
        for (int c = 1; c < C; c++)
            if (St[c] == x1_size) { St[c] = St[c - 1]; Et[c] = St[c - 1]; }
    }
}

/* Visited entries: sum_b sum_r rows(r) * (end - start), bands clamped to [0, n]. */
int64_t kmo_count_entries(int64_t B, int m, int n, int block, const int32_t *start,
                          const int32_t *end, int64_t range_bs) {
    const int R = (m + block - 1) / block;
    int64_t total = 0;
    for (int64_t b = 0; b < B; b++)
        for (int r = 0; r < R; r++) {
            int s, e;
            kmo_band(start + b * range_bs, end + b * range_bs, r, n, &s, &e);
            total += (int64_t)(kmo_min((r + 1) * block, m) - r * block) * (e - s);
        }
    return total;
}
