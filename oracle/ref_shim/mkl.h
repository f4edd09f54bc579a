/* TEST INFRASTRUCTURE — stand-in for Intel oneMKL's <mkl.h> (see mkl_spblas.h beside this file):
 * the service and BLAS level-1 routines the reference's cbm/cbm_extensions.cpp calls. */
#ifndef REFSHIM_MKL_H
#define REFSHIM_MKL_H
#include "mkl_spblas.h"

#ifdef __cplusplus
extern "C" {
#endif

/* The thread-count pair is routed through torch's own setter (which drives the oneMKL inside
 * libtorch) with the OpenMP team size put back afterwards, since libtorch exports no
 * mkl_set_num_threads. */
int refshim_get_max_threads(void);
void refshim_set_num_threads(int n);
/* Real oneMKL routine, exported by libtorch_cpu.so. */
void cblas_saxpy(const MKL_INT n, const float a, const float* x, const MKL_INT incx, float* y, const MKL_INT incy);

#ifndef REFSHIM_IMPLEMENTATION
#define mkl_get_max_threads refshim_get_max_threads
#define mkl_set_num_threads refshim_set_num_threads
#endif

#ifdef __cplusplus
}
#endif
#endif
