// TEST INFRASTRUCTURE — the functions behind the stand-in headers mkl.h / mkl_spblas.h of this
// folder.  Linked with the reference's unmodified cbm/cbm_extensions.cpp into oracle/_ref.
//
// Compute path (what the parity tests pin): create_csr, s_mm, destroy and cblas_saxpy go to the real
// Intel oneMKL routines that libtorch_cpu.so exports (the same library the reference links,
// cbm/setup.py:35-47), so `dst = deltas * rhs` (cbm/cbm_extensions.cpp:694-704 and the other ten
// compute entry points) is computed by oneMKL itself.
//
// Builder path: create_coo, convert_csr and syrk are not exported by libtorch and are written out
// here from their documented semantics — COO to CSR by a stable counting sort over rows, and
// C = A * A^T restricted to its upper triangle with ascending columns per row (the reference skips
// the first entry of each row as the diagonal, cbm/cbm_extensions.cpp:87).
#define REFSHIM_IMPLEMENTATION
#include "mkl.h"

#include <ATen/Parallel.h>
#include <omp.h>

#include <algorithm>
#include <new>
#include <vector>

// the real oneMKL handle type is opaque; only pointers to it pass through here
extern "C" {
sparse_status_t mkl_sparse_s_create_csr(void** A, sparse_index_base_t indexing, MKL_INT rows, MKL_INT cols,
                                        MKL_INT* rows_start, MKL_INT* rows_end, MKL_INT* col_indx, float* values);
sparse_status_t mkl_sparse_s_mm(sparse_operation_t operation, float alpha, void* A, struct matrix_descr descr,
                                sparse_layout_t layout, const float* B, MKL_INT columns, MKL_INT ldb, float beta,
                                float* C, MKL_INT ldc);
sparse_status_t mkl_sparse_s_export_csr(void* source, sparse_index_base_t* indexing, MKL_INT* rows, MKL_INT* cols,
                                        MKL_INT** rows_start, MKL_INT** rows_end, MKL_INT** col_indx, float** values);
sparse_status_t mkl_sparse_destroy(void* A);
}

struct refshim_matrix {
    void* mkl = nullptr;  // non-null: a real oneMKL handle, everything else unused
    bool coo = false;
    MKL_INT rows = 0, cols = 0;
    std::vector<MKL_INT> ri, ci;   // COO
    std::vector<MKL_INT> ptr, col; // CSR (ptr has rows + 1 entries)
    std::vector<float> val;
};

extern "C" {

int refshim_get_max_threads(void) { return at::get_num_threads(); }

void refshim_set_num_threads(int n) {
    const int team = omp_get_max_threads();
    at::set_num_threads(n);      // sets the thread count of the oneMKL inside libtorch (and OpenMP's)
    omp_set_num_threads(team);   // the reference changes only MKL's count, so OpenMP's is put back
}

sparse_status_t refshim_sparse_s_create_coo(sparse_matrix_t* A, sparse_index_base_t indexing, MKL_INT rows,
                                            MKL_INT cols, MKL_INT nnz, MKL_INT* row_indx, MKL_INT* col_indx,
                                            float* values) {
    if (!A || indexing != SPARSE_INDEX_BASE_ZERO || rows < 0 || cols < 0 || nnz < 0) return SPARSE_STATUS_INVALID_VALUE;
    refshim_matrix* m = new (std::nothrow) refshim_matrix();
    if (!m) return SPARSE_STATUS_ALLOC_FAILED;
    m->coo = true;
    m->rows = rows;
    m->cols = cols;
    m->ri.assign(row_indx, row_indx + nnz);
    m->ci.assign(col_indx, col_indx + nnz);
    m->val.assign(values, values + nnz);
    *A = m;
    return SPARSE_STATUS_SUCCESS;
}

sparse_status_t refshim_sparse_convert_csr(sparse_matrix_t src, sparse_operation_t operation, sparse_matrix_t* dest) {
    if (!src || !dest || !src->coo || operation != SPARSE_OPERATION_NON_TRANSPOSE) return SPARSE_STATUS_NOT_SUPPORTED;
    refshim_matrix* m = new (std::nothrow) refshim_matrix();
    if (!m) return SPARSE_STATUS_ALLOC_FAILED;
    m->rows = src->rows;
    m->cols = src->cols;
    const size_t nnz = src->ri.size();
    m->ptr.assign((size_t)m->rows + 1, 0);
    for (size_t k = 0; k < nnz; ++k) {
        if (src->ri[k] < 0 || src->ri[k] >= m->rows || src->ci[k] < 0 || src->ci[k] >= m->cols) {
            delete m;
            return SPARSE_STATUS_INVALID_VALUE;
        }
        ++m->ptr[(size_t)src->ri[k] + 1];
    }
    for (MKL_INT r = 0; r < m->rows; ++r) m->ptr[(size_t)r + 1] += m->ptr[r];
    m->col.resize(nnz);
    m->val.resize(nnz);
    std::vector<MKL_INT> fill(m->ptr.begin(), m->ptr.end() - 1);
    for (size_t k = 0; k < nnz; ++k) {
        const MKL_INT at_ = fill[src->ri[k]]++;
        m->col[at_] = src->ci[k];
        m->val[at_] = src->val[k];
    }
    *dest = m;
    return SPARSE_STATUS_SUCCESS;
}

sparse_status_t refshim_sparse_syrk(sparse_operation_t operation, sparse_matrix_t A, sparse_matrix_t* C) {
    if (!A || !C || A->mkl || A->coo || operation != SPARSE_OPERATION_NON_TRANSPOSE) return SPARSE_STATUS_NOT_SUPPORTED;
    const MKL_INT n = A->rows;
    // column lists of A (= rows of A^T), rows ascending inside each list
    std::vector<MKL_INT> tptr((size_t)A->cols + 1, 0);
    for (MKL_INT c : A->col) ++tptr[(size_t)c + 1];
    for (MKL_INT c = 0; c < A->cols; ++c) tptr[(size_t)c + 1] += tptr[c];
    std::vector<MKL_INT> trow(A->col.size());
    std::vector<float> tval(A->col.size());
    {
        std::vector<MKL_INT> fill(tptr.begin(), tptr.end() - 1);
        for (MKL_INT r = 0; r < n; ++r)
            for (MKL_INT k = A->ptr[r]; k < A->ptr[(size_t)r + 1]; ++k) {
                const MKL_INT at_ = fill[A->col[k]]++;
                trow[at_] = r;
                tval[at_] = A->val[k];
            }
    }
    refshim_matrix* m = new (std::nothrow) refshim_matrix();
    if (!m) return SPARSE_STATUS_ALLOC_FAILED;
    m->rows = n;
    m->cols = n;
    m->ptr.assign((size_t)n + 1, 0);
    std::vector<float> acc((size_t)n, 0.f);
    std::vector<char> hit((size_t)n, 0);
    std::vector<MKL_INT> touched;
    for (MKL_INT i = 0; i < n; ++i) {
        touched.clear();
        for (MKL_INT k = A->ptr[i]; k < A->ptr[(size_t)i + 1]; ++k) {
            const MKL_INT c = A->col[k];
            const float a = A->val[k];
            // rows j >= i that also hold column c
            const MKL_INT* lo = std::lower_bound(trow.data() + tptr[c], trow.data() + tptr[(size_t)c + 1], i);
            for (const MKL_INT* p = lo; p < trow.data() + tptr[(size_t)c + 1]; ++p) {
                const MKL_INT j = *p;
                if (!hit[j]) {
                    hit[j] = 1;
                    touched.push_back(j);
                }
                acc[j] += a * tval[p - trow.data()];
            }
        }
        std::sort(touched.begin(), touched.end());
        for (MKL_INT j : touched) {
            m->col.push_back(j);
            m->val.push_back(acc[j]);
            acc[j] = 0.f;
            hit[j] = 0;
        }
        m->ptr[(size_t)i + 1] = (MKL_INT)m->col.size();
    }
    *C = m;
    return SPARSE_STATUS_SUCCESS;
}

sparse_status_t refshim_sparse_s_create_csr(sparse_matrix_t* A, sparse_index_base_t indexing, MKL_INT rows,
                                            MKL_INT cols, MKL_INT* rows_start, MKL_INT* rows_end,
                                            MKL_INT* col_indx, float* values) {
    if (!A) return SPARSE_STATUS_INVALID_VALUE;
    refshim_matrix* m = new (std::nothrow) refshim_matrix();
    if (!m) return SPARSE_STATUS_ALLOC_FAILED;
    const sparse_status_t s = mkl_sparse_s_create_csr(&m->mkl, indexing, rows, cols, rows_start, rows_end, col_indx, values);
    if (s != SPARSE_STATUS_SUCCESS || !m->mkl) {
        delete m;
        return s != SPARSE_STATUS_SUCCESS ? s : SPARSE_STATUS_INTERNAL_ERROR;
    }
    *A = m;
    return SPARSE_STATUS_SUCCESS;
}

sparse_status_t refshim_sparse_s_export_csr(sparse_matrix_t src, sparse_index_base_t* indexing, MKL_INT* rows,
                                            MKL_INT* cols, MKL_INT** rows_start, MKL_INT** rows_end,
                                            MKL_INT** col_indx, float** values) {
    if (!src) return SPARSE_STATUS_NOT_INITIALIZED;
    if (src->mkl) return mkl_sparse_s_export_csr(src->mkl, indexing, rows, cols, rows_start, rows_end, col_indx, values);
    if (src->coo) return SPARSE_STATUS_INVALID_VALUE;
    *indexing = SPARSE_INDEX_BASE_ZERO;
    *rows = src->rows;
    *cols = src->cols;
    *rows_start = src->ptr.data();
    *rows_end = src->ptr.data() + 1;
    *col_indx = src->col.data();
    *values = src->val.data();
    return SPARSE_STATUS_SUCCESS;
}

sparse_status_t refshim_sparse_s_mm(sparse_operation_t operation, float alpha, sparse_matrix_t A,
                                    struct matrix_descr descr, sparse_layout_t layout, const float* B,
                                    MKL_INT columns, MKL_INT ldb, float beta, float* C, MKL_INT ldc) {
    if (!A || !A->mkl) return SPARSE_STATUS_NOT_INITIALIZED;
    return mkl_sparse_s_mm(operation, alpha, A->mkl, descr, layout, B, columns, ldb, beta, C, ldc);
}

sparse_status_t refshim_sparse_destroy(sparse_matrix_t A) {
    if (!A) return SPARSE_STATUS_NOT_INITIALIZED;
    sparse_status_t s = SPARSE_STATUS_SUCCESS;
    if (A->mkl) s = mkl_sparse_destroy(A->mkl);
    delete A;
    return s;
}

}  // extern "C"
