/* Stand-in for the OpenBLAS header the reference includes
 * (csrc/cpu/matmul.hpp:2); OpenBLAS is not installed here. Only the generic
 * matmul_ker<T> template is used from that file; the float/double
 * specialisations that call these functions are never invoked. */
#pragma once
#include <cstdlib>
enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 };
enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112 };
static inline void cblas_sgemm(int, int, int, int, int, int, float, const float *, int, const float *, int, float, float *, int) { std::abort(); }
static inline void cblas_dgemm(int, int, int, int, int, int, double, const double *, int, const double *, int, double, double *, int) { std::abort(); }
static inline float cblas_sdot(int, const float *, int, const float *, int) { std::abort(); }
static inline double cblas_ddot(int, const double *, int, const double *, int) { std::abort(); }
