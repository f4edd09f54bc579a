/*
 * TEST INFRASTRUCTURE — CPU restatement of the reference's CBM compute path in plain C.
 *
 * This file is the checker the CUDA engine is compared against and the CPU baseline that bench.py
 * times beside it.  It is never linked into, imported by or called from the product
 * (cbm4gnn_b200/); only tests/, the smoke check and bench.py's cpu_baseline / reference legs load it.
 *
 * Parity status: pinned.  The reference holds no golden vectors for this path (its tests are
 * differential against torch.sparse on random inputs, tests/test_matmul_correctness.py:30-61), so
 * the pins are outputs of the reference itself: its unmodified cbm/cbm_extensions.cpp compiled into
 * oracle/_ref (build_ref.py: stand-in headers for oneMKL and arbok, the sparse product forwarded to
 * the oneMKL inside libtorch).  The update loops below reproduce the reference's bit for bit
 * (committed fixtures tests/golden/cbm_reference.npz and live against oracle/_ref); the products
 * agree within the reference's own atol = rtol = 1e-4.  For the tree SHAPE (an output of the
 * arborescence solver's tie-breaking) parity is unpinned; validity and total weight are pinned.
 *
 * Each function names the reference lines (cbm/cbm_extensions.cpp) it follows.
 */
#include <stdint.h>
#include <stdlib.h>
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* dst = M * rhs for a CSR in the reference's 4-array form; alpha = 1, beta = 0, row-major, ld = f.
 * Follows the mkl_sparse_s_mm call at cbm/cbm_extensions.cpp:694-704 (seq) and :1149-1159 /
 * :1744-1754 (omp).  MKL is closed source: this is the textbook row-wise product in the same
 * storage, summed in column order. */
void oracle_csr_spmm(int32_t n_rows, const int32_t* row_b, const int32_t* row_e, const int32_t* col,
                     const float* val, const float* rhs, int32_t f, float* dst, int32_t parallel) {
#pragma omp parallel for schedule(dynamic, 64) if (parallel)
    for (int32_t r = 0; r < n_rows; ++r) {
        float* y = dst + (size_t)r * f;
        for (int32_t i = 0; i < f; ++i) y[i] = 0.0f;
        for (int32_t k = row_b[r]; k < row_e[r]; ++k) {
            const float w = val[k];
            const float* x = rhs + (size_t)col[k] * f;
            for (int32_t i = 0; i < f; ++i) y[i] += w * x[i];
        }
    }
}

/* y_v += y_u for a tree edge u -> v (cblas_saxpy with a = 1, cbm/cbm_extensions.cpp:734;
 * AVX2 add, :1190-1213). */
static void add_row(const float* x, float* y, int32_t f) {
    for (int32_t i = 0; i < f; ++i) y[i] += x[i];
}

/* Depth-first walk of one subtree with an explicit stack: children are visited in mst_col order
 * and pushed, the last pushed is expanded first (cbm/cbm_extensions.cpp:719-738, 1172-1217). */
static void walk_plain(int32_t top, const int32_t* mst_row, const int32_t* mst_col, float* dst,
                       int32_t f, int32_t* stack) {
    int32_t sp = 0;
    stack[sp++] = top;
    while (sp > 0) {
        const int32_t u = stack[--sp];
        for (int32_t k = mst_row[u]; k < mst_row[u + 1]; ++k) {
            const int32_t v = mst_col[k];
            add_row(dst + (size_t)u * f, dst + (size_t)v * f, f);
            stack[sp++] = v;
        }
    }
}

/* Unnormalized tree update in place.  parallel == 0: seq_s_update_csr_int32_
 * (cbm/cbm_extensions.cpp:742-786; one stack seeded with every child of the virtual root n).
 * parallel != 0: omp_s_update_csr_int32_ / the update half of omp_s_spmm_update_csr_int32_
 * (cbm/cbm_extensions.cpp:1166-1218, 1579-1609): one subtree of the virtual root per task,
 * schedule(dynamic, 50). */
int oracle_update(int32_t n, const int32_t* mst_row, const int32_t* mst_col, float* dst, int32_t f,
                  int32_t parallel) {
    const int32_t b = mst_row[n], e = mst_row[n + 1];
    int failed = 0;
#pragma omp parallel if (parallel)
    {
        int32_t* stack = (int32_t*)malloc(sizeof(int32_t) * (size_t)(n + 1));
        if (!stack) {
#pragma omp atomic write
            failed = 1;
        }
#pragma omp for schedule(dynamic, 50)
        for (int32_t j = b; j < e; ++j)
            if (stack) walk_plain(mst_col[j], mst_row, mst_col, dst, f, stack);
        free(stack);
    }
    return failed;
}

/* Normalized walk of one subtree (cbm/cbm_extensions.cpp:910-995 seq, 1288-1373 omp):
 * the root child is scaled by its own multiplier (:914-940); along an edge u -> v the body of the
 * row, in blocks of 8 floats, is y = fma(x, 1/s_u, y) * s_v (:966-986) and the tail of fewer than
 * 8 floats is y = (y + x / s_u) * s_v (:988-990). */
static void walk_fused(int32_t top, const int32_t* mst_row, const int32_t* mst_col,
                       const float* mult, float* dst, int32_t f, int32_t* stack) {
    const int32_t body = f - (f % 8);
    {
        float* x = dst + (size_t)top * f;
        const float s = mult[top];
        for (int32_t i = 0; i < f; ++i) x[i] *= s;
    }
    int32_t sp = 0;
    stack[sp++] = top;
    while (sp > 0) {
        const int32_t u = stack[--sp];
        const float u_scale = mult[u];
        const float u_inv = 1.0f / u_scale;
        for (int32_t k = mst_row[u]; k < mst_row[u + 1]; ++k) {
            const int32_t v = mst_col[k];
            const float v_scale = mult[v];
            const float* x = dst + (size_t)u * f;
            float* y = dst + (size_t)v * f;
            int32_t i = 0;
            for (; i < body; ++i) y[i] = fmaf(x[i], u_inv, y[i]) * v_scale;
            for (; i < f; ++i) y[i] = (y[i] + (x[i] / u_scale)) * v_scale;
            stack[sp++] = v;
        }
    }
}

/* Normalized tree update in place: seq_s_fused_update_csr_int32_ (cbm/cbm_extensions.cpp:998-1105)
 * and omp_s_fused_update_csr_int32_ (:1376-1483); also the update half of the fused
 * spmm+update functions (:908-995, :1285-1373). */
int oracle_fused_update(int32_t n, const int32_t* mst_row, const int32_t* mst_col,
                        const float* mult, float* dst, int32_t f, int32_t parallel) {
    const int32_t b = mst_row[n], e = mst_row[n + 1];
    int failed = 0;
#pragma omp parallel if (parallel)
    {
        int32_t* stack = (int32_t*)malloc(sizeof(int32_t) * (size_t)(n + 1));
        if (!stack) {
#pragma omp atomic write
            failed = 1;
        }
#pragma omp for schedule(dynamic, 50)
        for (int32_t j = b; j < e; ++j)
            if (stack) walk_fused(mst_col[j], mst_row, mst_col, mult, dst, f, stack);
        free(stack);
    }
    return failed;
}

/* dst = deltas * rhs, then the tree update: seq_/omp_s_spmm_update_csr_int32_
 * (cbm/cbm_extensions.cpp:650-740, 1108-1219). */
int oracle_spmm_update(int32_t n, const int32_t* row_b, const int32_t* row_e, const int32_t* col,
                       const float* val, const float* rhs, const int32_t* mst_row,
                       const int32_t* mst_col, float* dst, int32_t f, int32_t parallel) {
    oracle_csr_spmm(n, row_b, row_e, col, val, rhs, f, dst, parallel);
    return oracle_update(n, mst_row, mst_col, dst, f, parallel);
}

/* seq_/omp_s_fused_spmm_update_csr_int32_ (cbm/cbm_extensions.cpp:845-996, 1224-1374). */
int oracle_fused_spmm_update(int32_t n, const int32_t* row_b, const int32_t* row_e,
                             const int32_t* col, const float* val, const float* rhs,
                             const int32_t* mst_row, const int32_t* mst_col, const float* mult,
                             float* dst, int32_t f, int32_t parallel) {
    oracle_csr_spmm(n, row_b, row_e, col, val, rhs, f, dst, parallel);
    return oracle_fused_update(n, mst_row, mst_col, mult, dst, f, parallel);
}

int oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void oracle_set_threads(int32_t t) {
#ifdef _OPENMP
    if (t > 0) omp_set_num_threads(t);
#else
    (void)t;
#endif
}
