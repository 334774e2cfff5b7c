/*
 * Test infrastructure (y oracle and timed CPU baseline). NOT part of the product: only tests,
 * the smoke check and bench.py's CPU-baseline leg load the library built from this file.
 *
 * The reference has no host SpMV of its own: the meaning of y is fixed by its emitted
 * kernels, y[row] (+)= sum_k val[k] * x[col[k]] over the non-zeros of the row (e.g. the ELL-like
 * emitter direct_atom_op_warp_block_compress.cc:777-1010; input grammar struct.cc:92-174:
 * 1-based "row col val", sorted by row then column). This file restates that as the plain
 * row-major CSR loop over the ORIGINAL matrix:
 *   - asp_oracle_spmv_*_ref: accumulation in double whatever the value type, plus the per-row
 *     scale sum_k |val[k]|*|x[col[k]]| that the tolerance is relative to;
 *   - asp_oracle_spmv_*_native: accumulation in the value type, OpenMP row-parallel with
 *     schedule(dynamic, 1024): the timed CPU baseline.
 * parity unpinned: the reference ships no golden vectors or known-answer tests for y.
 */
#include <math.h>
#include <stdint.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int asp_oracle_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

#define DEF_REF(NAME, VT)                                                                                   \
    void NAME(int64_t n_rows, const int64_t *indptr, const uint32_t *indices, const VT *values, const VT *x, \
              double *y_ref, double *scale)                                                                 \
    {                                                                                                       \
        _Pragma("omp parallel for schedule(dynamic, 1024)") for (int64_t r = 0; r < n_rows; r++)            \
        {                                                                                                   \
            double acc = 0.0, sc = 0.0;                                                                     \
            for (int64_t k = indptr[r]; k < indptr[r + 1]; k++)                                             \
            {                                                                                               \
                const double a = (double)values[k], b = (double)x[indices[k]];                              \
                acc += a * b;                                                                               \
                sc += fabs(a) * fabs(b);                                                                    \
            }                                                                                               \
            y_ref[r] = acc;                                                                                 \
            if (scale) scale[r] = sc;                                                                       \
        }                                                                                                   \
    }

#define DEF_NATIVE(NAME, VT)                                                                           \
    void NAME(int64_t n_rows, const int64_t *indptr, const uint32_t *indices, const VT *values, const VT *x, VT *y) \
    {                                                                                                  \
        _Pragma("omp parallel for schedule(dynamic, 1024)") for (int64_t r = 0; r < n_rows; r++)       \
        {                                                                                              \
            VT acc = 0;                                                                                \
            for (int64_t k = indptr[r]; k < indptr[r + 1]; k++) acc += values[k] * x[indices[k]];      \
            y[r] = acc;                                                                                \
        }                                                                                              \
    }

DEF_REF(asp_oracle_spmv_f32_ref, float)
DEF_REF(asp_oracle_spmv_f64_ref, double)
DEF_NATIVE(asp_oracle_spmv_f32_native, float)
DEF_NATIVE(asp_oracle_spmv_f64_native, double)

/* first-touch helper: copies src to dst with the same OpenMP schedule the SpMV uses, so that
 * pages of the timed arrays land on the NUMA node of the thread that will read them. */
void asp_oracle_first_touch_copy(void *dst, const void *src, int64_t bytes)
{
    char *d = (char *)dst;
    const char *s = (const char *)src;
    _Pragma("omp parallel for schedule(static)") for (int64_t i = 0; i < bytes; i += 4096)
    {
        int64_t e = i + 4096 < bytes ? i + 4096 : bytes;
        for (int64_t j = i; j < e; j++) d[j] = s[j];
    }
}
