// Runs the REFERENCE's own device test bed against this library's drop-in headers.
//
// test/device/testbed.h of the reference (TestAllGemm: the M/N/K grid, the data, the comparison with the
// reference's host SRGEMM by cutlass TensorEquals) is included unmodified from the reference checkout; the only
// thing swapped underneath it is cuasr::gemm::device::Srgemm, which here is include/cuasr/gemm/device/srgemm.h of
// this repository (the include path lists this repository's include/ and the reference's tools/include, but NOT the
// reference's include/).  The instantiation list below plays the part of the reference's generated test files
// (test/device/simt_sm50.py:27-55): every pre-tuned ring x {float, double} x the eight layout combinations.
// The output of the build goes to oracle/_ref/, which is not committed.
//
// TEST INFRASTRUCTURE ONLY.
#include <cstdio>
#include <iostream>

// The two spellings of EXPECT_TRUE the test bed uses (`EXPECT_TRUE(x);` and `EXPECT_TRUE(x) << message;`),
// without googletest: count failures, print the message.
static int g_expect_failures = 0;
struct ExpectSink {
  bool ok;
  template <typename T>
  ExpectSink &operator<<(T const &v) {
    if (!ok) std::cerr << v;
    return *this;
  }
  ~ExpectSink() {
    if (!ok) std::cerr << std::endl;
  }
};
#define EXPECT_TRUE(cond) \
  ExpectSink { (cond) ? true : (++g_expect_failures, std::cerr << "EXPECT_TRUE(" #cond ") failed ", false) }

#define CUASR_B200_USE_CUTLASS
#include "cuasr/functional.h"
#include "cuasr/gemm/device/default_srgemm_configuration.h"
#include "cuasr/gemm/device/srgemm.h"

#include "testbed.h"   // the reference's test/device/testbed.h

using Col = cutlass::layout::ColumnMajor;
using Row = cutlass::layout::RowMajor;

static int g_cases = 0, g_failed = 0;

template <template <typename, int> class Add, template <typename, int> class Mul, typename T, typename LA, typename LB,
          typename LC>
void one(char const *ring, char const *type, char const *layouts) {
  using Op = cuasr::gemm::device::Srgemm<Add<T, 1>, Mul<T, 1>, T, LA, T, LB, T, LC, T>;
  bool ok = cuasr::test::gemm::device::TestAllGemm<Op>();
  ++g_cases;
  if (!ok) {
    ++g_failed;
    std::printf("FAILED %s %s %s\n", ring, type, layouts);
  }
}

template <template <typename, int> class Add, template <typename, int> class Mul, typename T>
void all_layouts(char const *ring, char const *type) {
  one<Add, Mul, T, Col, Col, Col>(ring, type, "nn_n");
  one<Add, Mul, T, Col, Col, Row>(ring, type, "nn_t");
  one<Add, Mul, T, Col, Row, Col>(ring, type, "nt_n");
  one<Add, Mul, T, Col, Row, Row>(ring, type, "nt_t");
  one<Add, Mul, T, Row, Col, Col>(ring, type, "tn_n");
  one<Add, Mul, T, Row, Col, Row>(ring, type, "tn_t");
  one<Add, Mul, T, Row, Row, Col>(ring, type, "tt_n");
  one<Add, Mul, T, Row, Row, Row>(ring, type, "tt_t");
}

template <typename T>
void all_rings(char const *type) {
  all_layouts<cuasr::plus, cuasr::multiplies, T>("plus_multiplies", type);
  all_layouts<cuasr::minimum, cuasr::plus, T>("minimum_plus", type);
  all_layouts<cuasr::maximum, cuasr::plus, T>("maximum_plus", type);
  all_layouts<cuasr::minimum, cuasr::maximum, T>("minimum_maximum", type);
  all_layouts<cuasr::maximum, cuasr::minimum, T>("maximum_minimum", type);
  all_layouts<cuasr::minimum, cuasr::multiplies, T>("minimum_multiplies", type);
  all_layouts<cuasr::maximum, cuasr::multiplies, T>("maximum_multiplies", type);
  all_layouts<cuasr::binary_or, cuasr::binary_and, T>("binary_or_binary_and", type);
}

int main() {
  all_rings<float>("float");
  all_rings<double>("double");
  std::printf("reference test bed: %d operator instantiations, %d failed, %d EXPECT_TRUE failures\n", g_cases, g_failed,
              g_expect_failures);
  std::printf("%s\n", (g_failed == 0 && g_expect_failures == 0) ? "ALL OK" : "FAILURES");
  return (g_failed == 0 && g_expect_failures == 0) ? 0 : 1;
}
