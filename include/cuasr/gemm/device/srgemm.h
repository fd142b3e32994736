// cuasr::gemm::device::Srgemm with the public surface of the reference
// (include/cuasr/gemm/device/srgemm.h:28-357; the column-major-C specialisation :398-567 needs no counterpart
// because the library transposes internally): same template parameter list, Arguments, can_implement,
// get_workspace_size, initialize, update, run and both operator() forms, same status codes.  Every member
// forwards to the C ABI of libcuasr_b200 (include/cuasr_b200.h); tile-shape parameters are accepted and unused.
#pragma once

#include <cstddef>
#include <cstring>

#include <cuda_runtime_api.h>

#include "../../../cuasr_b200.h"
#include "../../compat.h"
#include "../../functional.h"
#include "default_srgemm_configuration.h"
#include "user_functor_srgemm.h"

namespace cuasr {
namespace gemm {
namespace device {

namespace detail {
template <typename Layout> struct LayoutCode;
template <> struct LayoutCode<cutlass::layout::ColumnMajor> { static constexpr int value = CUASR_COLUMN_MAJOR; };
template <> struct LayoutCode<cutlass::layout::RowMajor>    { static constexpr int value = CUASR_ROW_MAJOR; };

template <typename T>
inline cuasr_b200_scalar_t scalar(T v) {
  cuasr_b200_scalar_t s;
  std::memset(s.bytes, 0, sizeof s.bytes);
  std::memcpy(s.bytes, &v, sizeof v);
  return s;
}
template <typename T>
inline T unscalar(cuasr_b200_scalar_t const& s) {
  T v;
  std::memcpy(&v, s.bytes, sizeof v);
  return v;
}

// Launch of the caller-compiled kernel for functors without an operator code.  The primary template is what a
// host-only translation unit, or an operator whose functors both declare their codes, sees: it never names the
// kernel, so nothing is instantiated for it.
template <bool kCompileKernel, typename AdditionOp, typename MultiplicationOp, typename T, typename LayoutA,
          typename LayoutB, typename LayoutC>
struct UserFunctorPath {
  static constexpr bool kAvailable = false;
  static int run(cuasr_b200_args_t const&, cudaStream_t) { return CUASR_STATUS_ERROR_NOT_SUPPORTED; }
};
#if defined(__CUDACC__)
template <typename AdditionOp, typename MultiplicationOp, typename T, typename LayoutA, typename LayoutB,
          typename LayoutC>
struct UserFunctorPath<true, AdditionOp, MultiplicationOp, T, LayoutA, LayoutB, LayoutC> {
  static constexpr bool kAvailable = true;
  static int run(cuasr_b200_args_t const& a, cudaStream_t stream) {
    return run_user_functor_srgemm<AdditionOp, MultiplicationOp, T>(
        a.m, a.n, a.k, static_cast<const T*>(a.A), a.lda, LayoutCode<LayoutA>::value == CUASR_ROW_MAJOR,
        static_cast<const T*>(a.B), a.ldb, LayoutCode<LayoutB>::value == CUASR_ROW_MAJOR, static_cast<const T*>(a.C),
        a.ldc, static_cast<T*>(a.D), a.ldd, LayoutCode<LayoutC>::value == CUASR_ROW_MAJOR, unscalar<T>(a.alpha),
        unscalar<T>(a.beta), stream);
  }
};
#endif
}  // namespace detail

template <typename AdditionOp_, typename MultiplicationOp_, typename ElementA_, typename LayoutA_,
          typename ElementB_, typename LayoutB_, typename ElementC_, typename LayoutC_,
          typename ElementAccumulator_ = ElementC_, typename OperatorClass_ = cutlass::arch::OpClassSimt,
          typename ArchTag_ = cutlass::arch::Sm50,
          typename ThreadblockShape_ = typename DefaultSemiRingConfiguration<
              ElementA_, ElementB_, ElementC_, ElementAccumulator_, OperatorClass_, AdditionOp_, MultiplicationOp_,
              ArchTag_>::ThreadblockShape,
          typename WarpShape_ = typename DefaultSemiRingConfiguration<
              ElementA_, ElementB_, ElementC_, ElementAccumulator_, OperatorClass_, AdditionOp_, MultiplicationOp_,
              ArchTag_>::WarpShape,
          typename InstructionShape_ = typename DefaultSemiRingConfiguration<
              ElementA_, ElementB_, ElementC_, ElementAccumulator_, OperatorClass_, AdditionOp_, MultiplicationOp_,
              ArchTag_>::InstructionShape,
          typename EpilogueOutputOp_ = typename DefaultSemiRingConfiguration<
              ElementA_, ElementB_, ElementC_, ElementAccumulator_, OperatorClass_, AdditionOp_, MultiplicationOp_,
              ArchTag_>::EpilogueOutputOp,
          typename ThreadblockSwizzle_ = IdentityThreadblockSwizzle,
          int Stages = DefaultSemiRingConfiguration<ElementA_, ElementB_, ElementC_, ElementAccumulator_, OperatorClass_,
                                                    AdditionOp_, MultiplicationOp_, ArchTag_>::kStages,
          int AlignmentA = 1, int AlignmentB = 1, bool SplitKSerial = false>
class Srgemm {
 public:
  using AdditionOp = AdditionOp_;
  using MultiplicationOp = MultiplicationOp_;
  using ElementA = ElementA_;
  using LayoutA = LayoutA_;
  using ElementB = ElementB_;
  using LayoutB = LayoutB_;
  using ElementC = ElementC_;
  using LayoutC = LayoutC_;
  using ElementAccumulator = ElementAccumulator_;
  using OperatorClass = OperatorClass_;
  using ArchTag = ArchTag_;
  using ThreadblockShape = ThreadblockShape_;
  using WarpShape = WarpShape_;
  using InstructionShape = InstructionShape_;
  using EpilogueOutputOp = EpilogueOutputOp_;
  using ThreadblockSwizzle = ThreadblockSwizzle_;
  using TensorRefA = cutlass::TensorRef<ElementA const, LayoutA>;
  using TensorRefB = cutlass::TensorRef<ElementB const, LayoutB>;
  using TensorRefC = cutlass::TensorRef<ElementC const, LayoutC>;
  using TensorRefD = cutlass::TensorRef<ElementC, LayoutC>;
  static int const kStages = Stages;
  static int const kAlignmentA = AlignmentA;
  static int const kAlignmentB = AlignmentB;
  static bool const kSplitKSerial = SplitKSerial;
  static int const kAlignmentC = EpilogueOutputOp::kCount;
  // The reference's test bed and bench harness name the epilogue functor through the kernel type
  // (test/device/testbed.h:52-54, bench/device/harness.h:49-50); there is no kernel type here, only that path.
  struct SrgemmKernel {
    struct Epilogue {
      using OutputOp = EpilogueOutputOp;
    };
  };

  static_assert(std::is_same<ElementA, ElementC>::value && std::is_same<ElementB, ElementC>::value &&
                    std::is_same<ElementAccumulator, ElementC>::value,
                "the B200 library computes in one element type for A, B, C, D and the accumulator");

  struct Arguments {
    cutlass::gemm::GemmCoord problem_size;
    TensorRefA ref_A;
    TensorRefB ref_B;
    TensorRefC ref_C;
    TensorRefD ref_D;
    typename EpilogueOutputOp::Params epilogue;
    int split_k_slices;
    Arguments() : problem_size(0, 0, 0), split_k_slices(1) {}
    Arguments(cutlass::gemm::GemmCoord problem_size_, TensorRefA ref_A_, TensorRefB ref_B_, TensorRefC ref_C_,
              TensorRefD ref_D_, typename EpilogueOutputOp::Params epilogue_ = typename EpilogueOutputOp::Params(),
              int split_k_slices_ = 1)
        : problem_size(problem_size_), ref_A(ref_A_), ref_B(ref_B_), ref_C(ref_C_), ref_D(ref_D_),
          epilogue(epilogue_), split_k_slices(split_k_slices_) {}
  };

  Srgemm() : initialized_(false) { std::memset(&args_, 0, sizeof args_); }

  static cutlass::Status can_implement(Arguments const& args) {
    cuasr_b200_desc_t d = desc();
    cuasr_b200_args_t a = pack(args, nullptr, 0, nullptr);
    if (user_functors()) return user_can_implement(a, SplitKSerial);
    return static_cast<cutlass::Status>(cuasr_b200_srgemm_can_implement(&d, &a));
  }

  static size_t get_workspace_size(Arguments const& args) {
    cuasr_b200_desc_t d = desc();
    cuasr_b200_args_t a = pack(args, nullptr, 0, nullptr);
    if (user_functors()) return 0;
    return cuasr_b200_srgemm_workspace_size(&d, &a);
  }

  // Not in the reference: bytes of an OPTIONAL workspace that makes an unsplit launch faster (balanced last wave,
  // packed adds on re-packed operands, unaligned operands kept on the fast kernel); 0 = nothing to gain.  Pass the
  // buffer and its size to initialize() / operator() through their last parameter.  Needs a current device.
  static size_t get_optional_workspace_size(Arguments const& args) {
    cuasr_b200_desc_t d = desc();
    cuasr_b200_args_t a = pack(args, nullptr, 0, nullptr);
    if (user_functors()) return 0;
    return cuasr_b200_srgemm_optional_workspace_size(&d, &a);
  }

  // workspace_bytes: size of `workspace` when it is larger than get_workspace_size() asks for (the optional
  // workspace above); 0 = exactly the required size, as in the reference.
  cutlass::Status initialize(Arguments const& args, void* workspace = nullptr, cudaStream_t stream = nullptr,
                             size_t workspace_bytes = 0) {
    cuasr_b200_desc_t d = desc();
    const size_t required = get_workspace_size(args);
    cuasr_b200_args_t a = pack(args, workspace, workspace_bytes > required ? workspace_bytes : required, stream);
    cutlass::Status st = user_functors() ? user_can_implement(a, SplitKSerial)
                                         : static_cast<cutlass::Status>(cuasr_b200_srgemm_can_implement(&d, &a));
    if (st != cutlass::Status::kSuccess) return st;
    if (required > 0 && workspace == nullptr) return cutlass::Status::kErrorWorkspaceNull;
    if (workspace == nullptr) a.workspace_bytes = 0;
    args_ = a;
    initialized_ = true;
    return cutlass::Status::kSuccess;
  }

  // refreshes the operand pointers and the workspace of an initialised operator
  cutlass::Status update(Arguments const& args, void* workspace = nullptr) {
    if (!initialized_) return cutlass::Status::kErrorInternal;
    if (args_.workspace_bytes > 0 && workspace == nullptr) return cutlass::Status::kErrorWorkspaceNull;
    args_.A = args.ref_A.data();
    args_.B = args.ref_B.data();
    args_.C = args.ref_C.data();
    args_.D = args.ref_D.data();
    args_.workspace = workspace;
    return cutlass::Status::kSuccess;
  }

  cutlass::Status run(cudaStream_t stream = nullptr) {
    if (!initialized_) return cutlass::Status::kErrorInternal;
    cuasr_b200_desc_t d = desc();
    args_.stream = stream;
    if (user_functors()) return static_cast<cutlass::Status>(UserPath::run(args_, stream));
    return static_cast<cutlass::Status>(cuasr_b200_srgemm(&d, &args_));
  }

  cutlass::Status operator()(cudaStream_t stream = nullptr) { return run(stream); }

  cutlass::Status operator()(Arguments const& args, void* workspace = nullptr, cudaStream_t stream = nullptr,
                             size_t workspace_bytes = 0) {
    cutlass::Status st = initialize(args, workspace, stream, workspace_bytes);
    return st == cutlass::Status::kSuccess ? run(stream) : st;
  }

 protected:
  // A functor pair the library has no operator codes for runs in a kernel compiled here from the functors themselves
  // (user_functor_srgemm.h); that needs a CUDA compiler, so elsewhere such a pair is refused as not supported.
  using UserPath = detail::UserFunctorPath<!(HasOpCode<AdditionOp>::value && HasOpCode<MultiplicationOp>::value),
                                           AdditionOp, MultiplicationOp, ElementC, LayoutA, LayoutB, LayoutC>;
  static bool user_functors() {
    return UserPath::kAvailable &&
           (OpCodeOf<AdditionOp, ElementC>::get() < 0 || OpCodeOf<MultiplicationOp, ElementC>::get() < 0);
  }
  static cutlass::Status user_can_implement(cuasr_b200_args_t const& a, bool slices_allowed) {
    if (a.m <= 0 || a.n <= 0 || a.k <= 0 || a.A == nullptr || a.B == nullptr || a.D == nullptr || a.split_k_slices < 1)
      return cutlass::Status::kErrorInvalidProblem;
    if (a.split_k_slices > 1 && !slices_allowed) return cutlass::Status::kErrorInvalidProblem;
    return cutlass::Status::kSuccess;
  }

  static cuasr_b200_desc_t desc() {
    cuasr_b200_desc_t d;
    d.add_op = OpCodeOf<AdditionOp, ElementC>::get();
    d.mul_op = OpCodeOf<MultiplicationOp, ElementC>::get();
    d.dtype = DTypeCode<ElementC>::value;
    d.layout_a = detail::LayoutCode<LayoutA>::value;
    d.layout_b = detail::LayoutCode<LayoutB>::value;
    d.layout_c = detail::LayoutCode<LayoutC>::value;
    d.split_k_serial = SplitKSerial ? 1 : 0;
    d.reserved = 0;
    return d;
  }

  static cuasr_b200_args_t pack(Arguments const& args, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    cuasr_b200_args_t a;
    std::memset(&a, 0, sizeof a);
    a.m = args.problem_size.m();
    a.n = args.problem_size.n();
    a.k = args.problem_size.k();
    a.split_k_slices = args.split_k_slices;
    a.A = args.ref_A.data(); a.lda = args.ref_A.stride(0);
    a.B = args.ref_B.data(); a.ldb = args.ref_B.stride(0);
    a.C = args.ref_C.data(); a.ldc = args.ref_C.stride(0);
    a.D = args.ref_D.data(); a.ldd = args.ref_D.stride(0);
    a.alpha = detail::scalar<ElementC>(args.epilogue.alpha_value());
    a.beta = detail::scalar<ElementC>(args.epilogue.beta_value());
    a.add_identity = detail::scalar<ElementC>(AdditionOp::Identity);
    a.mul_identity = detail::scalar<ElementC>(MultiplicationOp::Identity);
    a.workspace = workspace;
    a.workspace_bytes = workspace_bytes;
    a.stream = stream;
    return a;
  }

  cuasr_b200_args_t args_;
  bool initialized_;
};

}  // namespace device
}  // namespace gemm
}  // namespace cuasr
