// A few dozen lines standing in for the part of google-benchmark that the reference's generated benchmark files
// (bench/device/simt_*_sm50.cu) use, so that those files compile UNMODIFIED where google-benchmark is not installed:
// benchmark::State (range, the `for (auto _ : state)` loop, counters), benchmark::Counter with
// kIsIterationInvariantRate, benchmark::DoNotOptimize, and BENCHMARK(fn)->RangeMultiplier(m)->Range(lo, hi).
// Written for this repository (no google-benchmark code); the runner is oracle/ref_bench_main.cpp.
// TEST AND MEASUREMENT INFRASTRUCTURE ONLY.
#pragma once

#include <chrono>
#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace benchmark {

struct Counter {
  enum Flags { kDefaults = 0, kIsRate = 1, kIsIterationInvariant = 2, kIsIterationInvariantRate = 3 };
  double value = 0.0;
  int flags = kDefaults;
  Counter() = default;
  Counter(double v, int f = kDefaults) : value(v), flags(f) {}
};

class State {
 public:
  State(int64_t range0, int64_t iterations) : range0_(range0), left_(iterations), iterations_(iterations) {}
  int64_t range(int = 0) const { return range0_; }
  std::map<std::string, Counter> counters;

  // `for (auto _ : state)`: the clock runs from the first test of the loop condition to the last
  struct Token {};
  struct Iterator {
    State *state;
    bool operator!=(Iterator const &) {
      if (state->left_ == state->iterations_) state->start_ = std::chrono::steady_clock::now();
      if (state->left_ > 0) return true;
      state->seconds_ = std::chrono::duration<double>(std::chrono::steady_clock::now() - state->start_).count();
      return false;
    }
    Iterator &operator++() {
      --state->left_;
      return *this;
    }
    Token operator*() const { return Token(); }
  };
  Iterator begin() { return Iterator{this}; }
  Iterator end() { return Iterator{this}; }

  int64_t iterations() const { return iterations_; }
  double seconds() const { return seconds_; }

 private:
  int64_t range0_, left_, iterations_;
  std::chrono::steady_clock::time_point start_;
  double seconds_ = 0.0;
};

template <typename T>
inline void DoNotOptimize(T const &value) {
  asm volatile("" : : "r,m"(value) : "memory");
}

struct Registration {
  std::string name;
  void (*fn)(State &);
  int multiplier = 2;
  int64_t lo = 0, hi = 0;
  Registration *RangeMultiplier(int m) {
    multiplier = m;
    return this;
  }
  Registration *Range(int64_t lo_, int64_t hi_) {
    lo = lo_;
    hi = hi_;
    return this;
  }
};

inline std::vector<Registration *> &registry() {
  static std::vector<Registration *> all;
  return all;
}
inline Registration *Register(char const *name, void (*fn)(State &)) {
  Registration *r = new Registration{name, fn};
  registry().push_back(r);
  return r;
}

}  // namespace benchmark

#define BENCHMARK_SHIM_CONCAT2(a, b) a##b
#define BENCHMARK_SHIM_CONCAT(a, b) BENCHMARK_SHIM_CONCAT2(a, b)
#define BENCHMARK(fn) \
  static ::benchmark::Registration *BENCHMARK_SHIM_CONCAT(benchmark_shim_reg_, __LINE__) = ::benchmark::Register(#fn, fn)
