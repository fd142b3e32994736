// Builds the REFERENCE's legacy path-tracking routine into a shared library, for use as a checker only.
//
// test/regress/include/fwgpu/cpu_srgemm.hpp of the reference (cpu_fwgemm_naive: distances and the contraction
// index that last improved them) is included unmodified from the reference checkout and exported for float and
// double with 32-bit indices.  The routine is written for square column-major matrices (its loops run to n in
// every dimension), and that is how it is called.  The output of the build goes to oracle/_ref/, which is not
// committed.
//
// TEST INFRASTRUCTURE ONLY.
#include <algorithm>   // the header uses std::min without including it
#include <cstdint>

#include "fwgpu/cpu_srgemm.hpp"

extern "C" __attribute__((visibility("default"))) int cuasr_ref_fwgemm(int is_double, int n, void const *A, int lda,
                                                                        void const *B, int ldb, void *dist, int ldc,
                                                                        int32_t *parent) {
  if (is_double)
    fwgpu::cpu_fwgemm_naive<double, int32_t>(n, n, n, static_cast<double const *>(A), lda,
                                             static_cast<double const *>(B), ldb, static_cast<double *>(dist), ldc, parent);
  else
    fwgpu::cpu_fwgemm_naive<float, int32_t>(n, n, n, static_cast<float const *>(A), lda, static_cast<float const *>(B),
                                            ldb, static_cast<float *>(dist), ldc, parent);
  return 0;
}
