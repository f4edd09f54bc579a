/* TEST INFRASTRUCTURE — stand-in for Intel oneMKL's <mkl_spblas.h>, just wide enough for the
 * reference's cbm/cbm_extensions.cpp and cbm/helpers.hpp to compile UNMODIFIED where no oneMKL
 * development files are installed.
 *
 * Types, enumerators and argument lists follow the published oneMKL Inspector-Executor Sparse BLAS
 * C interface (LP64: MKL_INT = int).  Every routine the reference calls is renamed to a
 * refshim_* function (ref_shim.cpp).  The routines of the compute path
 * (create_csr, s_mm, export_csr of such a handle, destroy) are forwarded there to the REAL oneMKL
 * entry points that libtorch_cpu.so exports, so the arithmetic of `deltas * rhs` is Intel's.
 * The routines only the builder calls (create_coo, convert_csr, syrk), which libtorch does not
 * export, are written out in ref_shim.cpp from their documented semantics. */
#ifndef REFSHIM_MKL_SPBLAS_H
#define REFSHIM_MKL_SPBLAS_H

#ifdef __cplusplus
extern "C" {
#endif

#ifndef MKL_INT
#define MKL_INT int
#endif

typedef enum {
    SPARSE_STATUS_SUCCESS = 0,
    SPARSE_STATUS_NOT_INITIALIZED = 1,
    SPARSE_STATUS_ALLOC_FAILED = 2,
    SPARSE_STATUS_INVALID_VALUE = 3,
    SPARSE_STATUS_EXECUTION_FAILED = 4,
    SPARSE_STATUS_INTERNAL_ERROR = 5,
    SPARSE_STATUS_NOT_SUPPORTED = 6
} sparse_status_t;

typedef enum {
    SPARSE_OPERATION_NON_TRANSPOSE = 10,
    SPARSE_OPERATION_TRANSPOSE = 11,
    SPARSE_OPERATION_CONJUGATE_TRANSPOSE = 12
} sparse_operation_t;

typedef enum {
    SPARSE_MATRIX_TYPE_GENERAL = 20,
    SPARSE_MATRIX_TYPE_SYMMETRIC = 21,
    SPARSE_MATRIX_TYPE_HERMITIAN = 22,
    SPARSE_MATRIX_TYPE_TRIANGULAR = 23,
    SPARSE_MATRIX_TYPE_DIAGONAL = 24,
    SPARSE_MATRIX_TYPE_BLOCK_TRIANGULAR = 25,
    SPARSE_MATRIX_TYPE_BLOCK_DIAGONAL = 26
} sparse_matrix_type_t;

typedef enum { SPARSE_INDEX_BASE_ZERO = 0, SPARSE_INDEX_BASE_ONE = 1 } sparse_index_base_t;
typedef enum { SPARSE_FILL_MODE_LOWER = 40, SPARSE_FILL_MODE_UPPER = 41, SPARSE_FILL_MODE_FULL = 42 } sparse_fill_mode_t;
typedef enum { SPARSE_DIAG_NON_UNIT = 50, SPARSE_DIAG_UNIT = 51 } sparse_diag_type_t;
typedef enum { SPARSE_LAYOUT_ROW_MAJOR = 101, SPARSE_LAYOUT_COLUMN_MAJOR = 102 } sparse_layout_t;

struct matrix_descr {
    sparse_matrix_type_t type;
    sparse_fill_mode_t mode;
    sparse_diag_type_t diag;
};

/* A handle of the shim: either wraps a real oneMKL handle (compute path) or owns a COO/CSR copy
 * (builder path). */
struct refshim_matrix;
typedef struct refshim_matrix* sparse_matrix_t;

sparse_status_t refshim_sparse_s_create_coo(sparse_matrix_t* A, sparse_index_base_t indexing, MKL_INT rows,
                                            MKL_INT cols, MKL_INT nnz, MKL_INT* row_indx, MKL_INT* col_indx,
                                            float* values);
sparse_status_t refshim_sparse_s_create_csr(sparse_matrix_t* A, sparse_index_base_t indexing, MKL_INT rows,
                                            MKL_INT cols, MKL_INT* rows_start, MKL_INT* rows_end,
                                            MKL_INT* col_indx, float* values);
sparse_status_t refshim_sparse_convert_csr(sparse_matrix_t source, sparse_operation_t operation,
                                           sparse_matrix_t* dest);
sparse_status_t refshim_sparse_s_export_csr(sparse_matrix_t source, sparse_index_base_t* indexing, MKL_INT* rows,
                                            MKL_INT* cols, MKL_INT** rows_start, MKL_INT** rows_end,
                                            MKL_INT** col_indx, float** values);
sparse_status_t refshim_sparse_syrk(sparse_operation_t operation, sparse_matrix_t A, sparse_matrix_t* C);
sparse_status_t refshim_sparse_s_mm(sparse_operation_t operation, float alpha, sparse_matrix_t A,
                                    struct matrix_descr descr, sparse_layout_t layout, const float* B,
                                    MKL_INT columns, MKL_INT ldb, float beta, float* C, MKL_INT ldc);
sparse_status_t refshim_sparse_destroy(sparse_matrix_t A);

#ifndef REFSHIM_IMPLEMENTATION
#define mkl_sparse_s_create_coo refshim_sparse_s_create_coo
#define mkl_sparse_s_create_csr refshim_sparse_s_create_csr
#define mkl_sparse_convert_csr refshim_sparse_convert_csr
#define mkl_sparse_s_export_csr refshim_sparse_s_export_csr
#define mkl_sparse_syrk refshim_sparse_syrk
#define mkl_sparse_s_mm refshim_sparse_s_mm
#define mkl_sparse_destroy refshim_sparse_destroy
#endif

#ifdef __cplusplus
}
#endif
#endif
