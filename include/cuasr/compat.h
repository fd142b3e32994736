// Minimal stand-ins for the few CUTLASS types that appear in cuASR's public interface, so that code written
// against the reference (cutlass::Status, cutlass::gemm::GemmCoord, cutlass::TensorRef, layout and tag types)
// compiles against this library without a CUTLASS checkout.  Define CUASR_B200_USE_CUTLASS before including
// any cuasr header to use the real CUTLASS types instead.
#pragma once

#ifdef CUASR_B200_USE_CUTLASS
#include "cutlass/cutlass.h"
#include "cutlass/gemm/gemm.h"
#include "cutlass/layout/matrix.h"
#include "cutlass/tensor_ref.h"
#include "cutlass/arch/arch.h"
#include "cutlass/arch/mma.h"
#include "cutlass/numeric_conversion.h"   // the reference's device headers bring it in; its tools rely on that
#ifdef __CUDACC__   // device intrinsics inside: only a CUDA compiler can read it
#include "cutlass/gemm/threadblock/threadblock_swizzle.h"
#endif
#else

#include <cstdint>

namespace cutlass {

// Same numbering as cutlass::Status; the C ABI returns these values.
enum class Status {
  kSuccess = 0,
  kErrorMisalignedOperand,
  kErrorInvalidDataType,
  kErrorInvalidLayout,
  kErrorInvalidProblem,
  kErrorNotSupported,
  kErrorWorkspaceNull,
  kErrorInternal,
  kErrorArchMismatch,
  kErrorInsufficientDriver,
  kErrorMemoryAllocation,
  kInvalid
};

namespace layout {
struct RowMajor {
  static int const kRank = 2;
};
struct ColumnMajor {
  static int const kRank = 2;
};
}  // namespace layout

namespace arch {
struct OpClassSimt {};
struct Sm50 {};
struct Sm100 {};
}  // namespace arch

namespace gemm {
struct GemmCoord {
  int extent[3];
  GemmCoord() : extent{0, 0, 0} {}
  GemmCoord(int m, int n, int k) : extent{m, n, k} {}
  int m() const { return extent[0]; }
  int n() const { return extent[1]; }
  int k() const { return extent[2]; }
};
template <int M, int N, int K>
struct GemmShape {
  static int const kM = M;
  static int const kN = N;
  static int const kK = K;
};
// Names that code written against the reference passes as the ThreadblockSwizzle argument
// (examples/01_userdefined_semiring/userdefined_semiring.cu:131-132); this library rasterises tiles itself.
namespace threadblock {
template <int N = 1> struct GemmIdentityThreadblockSwizzle {};
struct GemmHorizontalThreadblockSwizzle {};
template <int N = 1> struct GemmSplitKIdentityThreadblockSwizzle {};
struct GemmSplitKHorizontalThreadblockSwizzle {};
}  // namespace threadblock
}  // namespace gemm

// A pointer and one leading dimension, in elements.
template <typename Element_, typename Layout_>
class TensorRef {
 public:
  using Element = Element_;
  using Layout = Layout_;
  TensorRef() : ptr_(nullptr), ld_(0) {}
  TensorRef(Element* ptr, int64_t ld) : ptr_(ptr), ld_(ld) {}
  // a reference to mutable data converts to a reference to const data
  template <typename Other, typename = decltype(static_cast<Element*>(static_cast<Other*>(nullptr)))>
  TensorRef(TensorRef<Other, Layout> const& other) : ptr_(other.data()), ld_(other.stride(0)) {}
  Element* data() const { return ptr_; }
  int64_t stride(int = 0) const { return ld_; }
  void reset(Element* ptr, int64_t ld) { ptr_ = ptr; ld_ = ld; }

 private:
  Element* ptr_;
  int64_t ld_;
};

}  // namespace cutlass
#endif  // CUASR_B200_USE_CUTLASS
