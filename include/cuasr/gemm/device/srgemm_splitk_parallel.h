// cuasr::gemm::device::SrgemmSplitKParallel with the public surface of the reference
// (include/cuasr/gemm/device/srgemm_splitk_parallel.h:36-378, column-major specialisation :424-607): the K
// range is cut into Arguments::split_k_slices slices.  The reference runs a partitioned GEMM and a second
// reduction kernel; the library does both in one launch (cuasr_b200_srgemm_splitk).  ConvertScaledOp and
// ReductionOp are accepted for source compatibility: the reduction is always the ring's addition.
#pragma once

#include "srgemm.h"

namespace cuasr {
namespace gemm {
namespace device {

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
          typename ConvertScaledOp_ = void, typename ReductionOp_ = void,
          typename ThreadblockSwizzle_ = SplitKHorizontalThreadblockSwizzle,
          int Stages = DefaultSemiRingConfiguration<ElementA_, ElementB_, ElementC_, ElementAccumulator_, OperatorClass_,
                                                    AdditionOp_, MultiplicationOp_, ArchTag_>::kStages,
          int kAlignmentA_ = 1, int kAlignmentB_ = 1>
class SrgemmSplitKParallel
    : private Srgemm<AdditionOp_, MultiplicationOp_, ElementA_, LayoutA_, ElementB_, LayoutB_, ElementC_, LayoutC_,
                     ElementAccumulator_, OperatorClass_, ArchTag_, ThreadblockShape_, WarpShape_, InstructionShape_,
                     EpilogueOutputOp_, ThreadblockSwizzle_, Stages, kAlignmentA_, kAlignmentB_, false> {
  using Base = Srgemm<AdditionOp_, MultiplicationOp_, ElementA_, LayoutA_, ElementB_, LayoutB_, ElementC_, LayoutC_,
                      ElementAccumulator_, OperatorClass_, ArchTag_, ThreadblockShape_, WarpShape_, InstructionShape_,
                      EpilogueOutputOp_, ThreadblockSwizzle_, Stages, kAlignmentA_, kAlignmentB_, false>;

 public:
  using typename Base::AdditionOp;
  using typename Base::MultiplicationOp;
  using typename Base::ElementA;
  using typename Base::ElementB;
  using typename Base::ElementC;
  using typename Base::LayoutA;
  using typename Base::LayoutB;
  using typename Base::LayoutC;
  using typename Base::ElementAccumulator;
  using typename Base::EpilogueOutputOp;
  using typename Base::ThreadblockShape;
  using typename Base::WarpShape;
  using typename Base::Arguments;
  using ConvertScaledOp = ConvertScaledOp_;
  using ReductionOp = ReductionOp_;
  static int const kStages = Stages;

  SrgemmSplitKParallel() {}

  static cutlass::Status can_implement(Arguments const& args) {
    cuasr_b200_desc_t d = Base::desc();
    cuasr_b200_args_t a = Base::pack(args, nullptr, 0, nullptr);
    if (Base::user_functors()) return Base::user_can_implement(a, true);
    return static_cast<cutlass::Status>(cuasr_b200_srgemm_splitk_can_implement(&d, &a));
  }

  static size_t get_workspace_size(Arguments const& args) {
    cuasr_b200_desc_t d = Base::desc();
    cuasr_b200_args_t a = Base::pack(args, nullptr, 0, nullptr);
    if (Base::user_functors()) return 0;    // the caller-compiled kernel contracts all of K in one pass
    return cuasr_b200_srgemm_splitk_workspace_size(&d, &a);
  }

  cutlass::Status initialize(Arguments const& args, void* workspace, cudaStream_t stream = nullptr) {
    cuasr_b200_desc_t d = Base::desc();
    cuasr_b200_args_t a = Base::pack(args, workspace, get_workspace_size(args), stream);
    cutlass::Status st = Base::user_functors()
                             ? Base::user_can_implement(a, true)
                             : static_cast<cutlass::Status>(cuasr_b200_srgemm_splitk_can_implement(&d, &a));
    if (st != cutlass::Status::kSuccess) return st;
    if (a.workspace_bytes > 0 && workspace == nullptr) return cutlass::Status::kErrorWorkspaceNull;
    this->args_ = a;
    this->initialized_ = true;
    return cutlass::Status::kSuccess;
  }

  cutlass::Status update(Arguments const& args, void* workspace = nullptr) { return Base::update(args, workspace); }

  cutlass::Status run(cudaStream_t stream = nullptr) {
    if (!this->initialized_) return cutlass::Status::kErrorInternal;
    cuasr_b200_desc_t d = Base::desc();
    this->args_.stream = stream;
    if (Base::user_functors()) return static_cast<cutlass::Status>(Base::UserPath::run(this->args_, stream));
    return static_cast<cutlass::Status>(cuasr_b200_srgemm_splitk(&d, &this->args_));
  }

  cutlass::Status operator()(cudaStream_t stream = nullptr) { return run(stream); }

  cutlass::Status operator()(Arguments const& args, void* workspace = nullptr, cudaStream_t stream = nullptr) {
    cutlass::Status st = initialize(args, workspace, stream);
    return st == cutlass::Status::kSuccess ? run(stream) : st;
  }
};

}  // namespace device
}  // namespace gemm
}  // namespace cuasr
