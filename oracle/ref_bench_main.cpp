// Runner for the reference's generated benchmark files compiled against oracle/shim/benchmark/benchmark.h and this
// library's drop-in headers: every registered benchmark at every size of its range, one warm-up pass and then
// `iterations` timed ones (argv[1], default 5; argv[2] caps the size).  Prints one line per (benchmark, size) with
// the counter the files define ("Flop/s" = 2 N^3 per iteration; each iteration is harness.run(): argument set-up,
// initialize and the launch, as the reference times it).
// TEST AND MEASUREMENT INFRASTRUCTURE ONLY.
#include <cstdio>
#include <cstdlib>

#include "benchmark/benchmark.h"

int main(int argc, char **argv) {
  const int iterations = argc > 1 ? std::atoi(argv[1]) : 5;
  const long long cap = argc > 2 ? std::atoll(argv[2]) : (1LL << 40);
  int ran = 0;
  for (benchmark::Registration *r : benchmark::registry()) {
    for (long long n = r->lo; n <= r->hi && n <= cap; n *= r->multiplier) {
      benchmark::State warm(n, 1);
      r->fn(warm);
      benchmark::State state(n, iterations);
      r->fn(state);
      double rate = 0.0;
      auto it = state.counters.find("Flop/s");
      if (it != state.counters.end() && state.seconds() > 0) rate = it->second.value * iterations / state.seconds();
      std::printf("%s/%lld  %.3f ms/iteration  %.4g Flop/s\n", r->name.c_str(), n,
                  1e3 * state.seconds() / iterations, rate);
      ++ran;
    }
  }
  std::printf("ran %d benchmark cases\n", ran);
  return ran > 0 ? 0 : 1;
}
