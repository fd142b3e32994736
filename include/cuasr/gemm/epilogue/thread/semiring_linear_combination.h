// Host-side counterpart of the reference's epilogue functor
// (include/cuasr/gemm/epilogue/thread/semiring_linear_combination.h:37-184): the Params aggregate with its five
// constructors and defaults (alpha = mult identity, beta = mult annihilator, :67-100), and is_source_needed()
// (:118-125).  The arithmetic D = add(mult(alpha, acc), mult(beta, C)) itself runs inside the library's kernels.
#pragma once

#include "../../../functional.h"

namespace cuasr {
namespace epilogue {
namespace thread {

template <typename AdditionOp_, typename MultiplicationOp_, typename ElementOutput_, int Count = 1,
          typename ElementAccumulator_ = ElementOutput_, typename ElementCompute_ = ElementOutput_>
class SemiringLinearCombination {
 public:
  using AdditionOp = AdditionOp_;
  using MultiplicationOp = MultiplicationOp_;
  using ElementOutput = ElementOutput_;
  using ElementAccumulator = ElementAccumulator_;
  using ElementCompute = ElementCompute_;
  static int const kCount = Count;

  struct Params {
    ElementCompute alpha;
    ElementCompute beta;
    ElementCompute const* alpha_ptr;  // host pointers; when set they override the values
    ElementCompute const* beta_ptr;
    Params() : alpha(MultiplicationOp::Identity), beta(MultiplicationOp::Annihilator), alpha_ptr(nullptr), beta_ptr(nullptr) {}
    Params(ElementCompute a, ElementCompute b) : alpha(a), beta(b), alpha_ptr(nullptr), beta_ptr(nullptr) {}
    Params(ElementCompute a) : alpha(a), beta(MultiplicationOp::Annihilator), alpha_ptr(nullptr), beta_ptr(nullptr) {}
    Params(ElementCompute const* a, ElementCompute const* b)
        : alpha(MultiplicationOp::Identity), beta(MultiplicationOp::Annihilator), alpha_ptr(a), beta_ptr(b) {}
    Params(ElementCompute const* a)
        : alpha(MultiplicationOp::Identity), beta(MultiplicationOp::Annihilator), alpha_ptr(a), beta_ptr(nullptr) {}
    ElementCompute alpha_value() const { return alpha_ptr ? *alpha_ptr : alpha; }
    ElementCompute beta_value() const { return beta_ptr ? *beta_ptr : beta; }
  };

  explicit SemiringLinearCombination(Params const& params) : alpha_(params.alpha_value()), beta_(params.beta_value()) {}

  // C takes part unless mult(beta, mult identity) is the additive identity
  bool is_source_needed() const {
    ElementCompute add_identity = AdditionOp::Identity;
    ElementCompute mult_identity = MultiplicationOp::Identity;
    return add_identity != MultiplicationOp()(beta_, mult_identity);
  }

  // the formula, for host-side checks
  ElementOutput operator()(ElementAccumulator acc, ElementOutput source) const {
    return AdditionOp()(MultiplicationOp()(alpha_, acc), MultiplicationOp()(beta_, source));
  }

 private:
  ElementCompute alpha_, beta_;
};

}  // namespace thread
}  // namespace epilogue
}  // namespace cuasr
