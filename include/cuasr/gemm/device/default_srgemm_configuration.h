// Tile presets kept for source compatibility with
// include/cuasr/gemm/device/default_srgemm_configuration.h:38-275 of the reference.  The B200 library chooses
// its own tiling (one persistent 128 x 128 CTA tile per SM, TMA-fed), so the shapes below only describe it; they
// are accepted as template arguments of Srgemm and otherwise ignored.
#pragma once

#include "../../compat.h"
#include "../epilogue/thread/semiring_linear_combination.h"

namespace cuasr {
namespace gemm {
namespace device {

struct IdentityThreadblockSwizzle {};
struct SplitKHorizontalThreadblockSwizzle {};

template <typename ElementA, typename ElementB, typename ElementC, typename ElementAccumulator,
          typename OperatorClass, typename AdditionOp_, typename MultiplicationOp_, typename ArchTag>
struct DefaultSemiRingConfiguration {
  // the ring the configuration was asked for (bench/device/simt_*_sm50.cu read these back)
  using AdditionOp = AdditionOp_;
  using MultiplicationOp = MultiplicationOp_;
  static int const kAlignmentA = 1;
  static int const kAlignmentB = 1;
  using ThreadblockShape = cutlass::gemm::GemmShape<128, 128, int(128 / sizeof(ElementA))>;
  using WarpShape = cutlass::gemm::GemmShape<64, 32, int(128 / sizeof(ElementA))>;
  using InstructionShape = cutlass::gemm::GemmShape<1, 1, 1>;
  static int const kStages = 5;
  using EpilogueOutputOp =
      cuasr::epilogue::thread::SemiringLinearCombination<AdditionOp, MultiplicationOp, ElementC, 1>;
};

}  // namespace device
}  // namespace gemm
}  // namespace cuasr
