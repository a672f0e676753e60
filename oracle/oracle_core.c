/*
 * TEST INFRASTRUCTURE, not product code: a plain-C restatement, on the CPU, of
 * the algorithms on the elementwise/reduction path of dpnp.  It is the checker
 * the tests and the measurement harness compare the CUDA path with; the
 * product never calls it.  Each function names the reference code it restates
 * (paths relative to the root of IntelPython/dpnp).
 *
 * Parity status: the reference cannot be built or imported here (it needs
 * DPC++/SYCL, dpctl and oneMKL), so these functions are pinned against the
 * known-answer cases of the reference's own tests and against NumPy, which the
 * reference's tests use as their oracle.  For exp/log/erf at the 2-ulp level
 * parity is unpinned: the reference delegates those to oneMKL VM / the SYCL
 * device library, whose bits are not available.
 *
 * The *_mt variants run the same loops with OpenMP over all host cores; they
 * are the timed CPU baseline.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* Thread count of the multi-threaded variants (launchers such as torchrun export
 * OMP_NUM_THREADS=1, which would silently turn the all-cores baseline into one core). */
void orc_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int orc_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Element displacement of the i-th element (C order over `shape`) of an array
 * with the given strides: the computation of CIndexer_vector::get_displacement
 * (dpnp/tensor/libtensor/include/utils/strided_iters.hpp:91-214), i.e. peel
 * indices from the last dimension with div/mod. */
static int64_t displacement(int nd, const int64_t *shape, const int64_t *strides, int64_t i)
{
    int64_t d = 0;
    for (int k = nd - 1; k > 0; --k) {
        const int64_t q = i / shape[k];
        d += (i - q * shape[k]) * strides[k];
        i = q;
    }
    if (nd > 0) d += i * strides[0];
    return d;
}

/* out[o3(i)] = a[o1(i)] (op) b[o2(i)], one element per index as in
 * BinaryStridedFunctor (include/kernels/elementwise_functions/common.hpp:528-558).
 * op: 0 add, 1 subtract, 2 multiply, 3 divide.  type: 0 f32, 1 f64, 2 i32, 3 i64. */
int orc_binary_strided(int op, int type, int64_t n, int nd, const int64_t *shape, const int64_t *sa,
                       const int64_t *sb, const int64_t *so, const void *a, const void *b, void *out)
{
    for (int64_t i = 0; i < n; ++i) {
        const int64_t ia = displacement(nd, shape, sa, i), ib = displacement(nd, shape, sb, i),
                      io = displacement(nd, shape, so, i);
#define ORC_APPLY(T)                                                   \
    {                                                                  \
        const T x = ((const T *)a)[ia], y = ((const T *)b)[ib];        \
        T r;                                                           \
        switch (op) {                                                  \
        case 0: r = x + y; break;                                      \
        case 1: r = x - y; break;                                      \
        case 2: r = x * y; break;                                      \
        default: r = x / y; break;                                     \
        }                                                              \
        ((T *)out)[io] = r;                                            \
    }
        switch (type) {
        case 0: ORC_APPLY(float) break;
        case 1: ORC_APPLY(double) break;
        case 2: ORC_APPLY(int32_t) break;
        case 3: ORC_APPLY(int64_t) break;
        default: return 1;
        }
#undef ORC_APPLY
    }
    return 0;
}

/* dst = cond ? x1 : x2 on f64 values with a one-byte condition where any
 * non-zero byte is true (include/kernels/where.hpp:67-161; byte rule of
 * include/utils/type_utils.hpp:63-114). */
void orc_where_f64(int64_t n, const uint8_t *cond, const double *x1, const double *x2, double *dst)
{
    for (int64_t i = 0; i < n; ++i) dst[i] = cond[i] ? x1[i] : x2[i];
}

/* Row sums of a C-contiguous (rows x cols) f32 matrix in extended precision:
 * the "float128/Kahan" oracle the tolerance of floating sums is stated against.
 * What is reduced is what reduction_axis1_over_group_temps_contig_impl reduces
 * (include/kernels/reductions.hpp:1396-1624). */
void orc_sum_axis1_f32(int64_t rows, int64_t cols, const float *x, double *sum, double *abs_sum)
{
    for (int64_t r = 0; r < rows; ++r) {
        long double s = 0.0L, a = 0.0L;
        for (int64_t c = 0; c < cols; ++c) {
            const long double v = x[r * cols + c];
            s += v;
            a += fabsl(v);
        }
        sum[r] = (double)s;
        abs_sum[r] = (double)a;
    }
}

/* Column sums (reduction_axis0_over_group_temps_contig_impl, reductions.hpp:1626-1856). */
void orc_sum_axis0_f32(int64_t rows, int64_t cols, const float *x, double *sum, double *abs_sum)
{
    for (int64_t c = 0; c < cols; ++c) {
        long double s = 0.0L, a = 0.0L;
        for (int64_t r = 0; r < rows; ++r) {
            const long double v = x[r * cols + c];
            s += v;
            a += fabsl(v);
        }
        sum[c] = (double)s;
        abs_sum[c] = (double)a;
    }
}

/* Maximum and index of its first occurrence per row of an int32 matrix
 * (index operator = minimum, source/reductions/argmax.cpp:139-141;
 * include/kernels/reductions.hpp:2062-2117). */
void orc_max_argmax_axis1_i32(int64_t rows, int64_t cols, const int32_t *x, int32_t *mx, int64_t *arg)
{
    for (int64_t r = 0; r < rows; ++r) {
        int32_t best = x[r * cols];
        int64_t at = 0;
        for (int64_t c = 1; c < cols; ++c)
            if (x[r * cols + c] > best) {
                best = x[r * cols + c];
                at = c;
            }
        mx[r] = best;
        arg[r] = at;
    }
}

/* f32 version: a NaN is the extreme value and the first NaN wins
 * (include/utils/sycl_utils.hpp:332-376; reductions.hpp:1933-1963). */
void orc_max_argmax_axis1_f32(int64_t rows, int64_t cols, const float *x, float *mx, int64_t *arg)
{
    for (int64_t r = 0; r < rows; ++r) {
        float best = x[r * cols];
        int64_t at = 0;
        for (int64_t c = 1; c < cols && !isnan(best); ++c) {
            const float v = x[r * cols + c];
            if (isnan(v) || v > best) {
                best = v;
                at = c;
            }
        }
        mx[r] = best;
        arg[r] = at;
    }
}

/* One option of the Black-Scholes chain of examples/example_bs.py:50-75, every
 * operation rounded on its own as the 26 separate ufunc calls round it. */
static void bs_one(double P, double S, double T, double rate, double vol, double *call, double *put)
{
    const double mr = -rate;
    const double sst = vol * vol * 2;
    const double a = log(P / S);
    const double b = T * mr;
    const double z = T * sst;
    const double c = 0.25 * z;
    const double y = 1.0 / sqrt(z);
    const double w1 = (a - b + c) * y;
    const double w2 = (a - b - c) * y;
    const double d1 = 0.5 + 0.5 * erf(w1);
    const double d2 = 0.5 + 0.5 * erf(w2);
    const double Se = exp(b) * S;
    const double r = P * d1 - Se * d2;
    *call = r;
    *put = r - P + Se;
}

void orc_black_scholes_f64(int64_t n, const double *price, const double *strike, const double *t,
                           double rate, double vol, double *call, double *put)
{
    for (int64_t i = 0; i < n; ++i) bs_one(price[i], strike[i], t[i], rate, vol, &call[i], &put[i]);
}

/* ------------------------------------------------------------------------
 * Multi-threaded variants: the timed CPU baseline (all host cores).
 * ---------------------------------------------------------------------- */
void orc_black_scholes_f64_mt(int64_t n, const double *price, const double *strike, const double *t,
                              double rate, double vol, double *call, double *put)
{
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) bs_one(price[i], strike[i], t[i], rate, vol, &call[i], &put[i]);
}

void orc_add_f32_mt(int64_t n, const float *a, const float *b, float *out)
{
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = a[i] + b[i];
}

void orc_multiply_transposed_f32_mt(int64_t ni, int64_t nj, int64_t nk, const float *a /* (nj,nk,ni) */,
                                    const float *b /* (ni,1,nk) */, float *out /* (ni,nj,nk) */)
{
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t i = 0; i < ni; ++i)
        for (int64_t j = 0; j < nj; ++j)
            for (int64_t k = 0; k < nk; ++k)
                out[(i * nj + j) * nk + k] = a[(j * nk + k) * ni + i] * b[i * nk + k];
}

void orc_sum_axis1_f32_mt(int64_t rows, int64_t cols, const float *x, float *sum)
{
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        double s = 0.0;
        for (int64_t c = 0; c < cols; ++c) s += x[r * cols + c];
        sum[r] = (float)s;
    }
}

void orc_max_argmax_axis1_i32_mt(int64_t rows, int64_t cols, const int32_t *x, int32_t *mx, int64_t *arg)
{
    /* rows are few and long: split every row into chunks, combine in order */
    enum { CHUNKS = 256 };
    for (int64_t r = 0; r < rows; ++r) {
        int32_t bests[CHUNKS];
        int64_t ats[CHUNKS];
        const int64_t len = (cols + CHUNKS - 1) / CHUNKS;
#pragma omp parallel for schedule(static)
        for (int ch = 0; ch < CHUNKS; ++ch) {
            const int64_t lo = ch * len, hi = (lo + len < cols) ? lo + len : cols;
            int32_t best = INT32_MIN;
            int64_t at = -1;
            for (int64_t c = lo; c < hi; ++c)
                if (at < 0 || x[r * cols + c] > best) {
                    best = x[r * cols + c];
                    at = c;
                }
            bests[ch] = best;
            ats[ch] = at;
        }
        int32_t best = bests[0];
        int64_t at = ats[0];
        for (int ch = 1; ch < CHUNKS; ++ch)
            if (ats[ch] >= 0 && bests[ch] > best) {
                best = bests[ch];
                at = ats[ch];
            }
        mx[r] = best;
        arg[r] = at;
    }
}
