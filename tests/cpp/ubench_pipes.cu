// Micro-benchmarks of the instruction mix of the fp32 min-plus contraction on one SM sub-partition: what the
// two pipes involved sustain alone and together, and what the register file delivers.  They back the roofline
// discussion of the hot kernel (packed add + three-input min per two products) with numbers measured on the GPU
// the library runs on.  Every kernel runs one CTA per SM with 256 threads (two warps per scheduler, like the
// kernel's consumer warps), times its loop with clock64 and reports clocks per group of instructions per scheduler.
//
// All recurrences are in place and all "volatile", so nothing is hoisted, merged or removed:
//   a constant operand repeated in the same operand slot of consecutive instructions can be served by the operand
//   reuse cache; a "fresh" operand is a different register every time and has to come from the register file.
//
// Output: one line per case, "name : clocks".  tests/test_hardware_model_gpu.py checks the lines the design
// relies on against loose bands.
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::printf("CUDA error %s line %d\n", cudaGetErrorString(e_), __LINE__); return 1; } } while (0)
typedef unsigned long long u64;

__device__ __forceinline__ u64 pack2(float lo, float hi) { u64 r; asm("mov.b64 %0, {%1,%2};" : "=l"(r) : "f"(lo), "f"(hi)); return r; }
__device__ __forceinline__ void unpack2(u64 v, float& lo, float& hi) { asm("mov.b64 {%0,%1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }

constexpr int kIters = 2048;
constexpr int kChains = 32;

enum Case {
  kAdd2Alone, kMin3Alone, kFaddAlone, kFfmaAlone,            // one pipe, second operands constant
  kAdd2Min3SharedConst,                                      // both pipes; the constants of both are the same registers
  kAdd2Min3OwnConst,                                         // both pipes; each instruction has its own constants
  kTwoFaddMin3,                                              // scalar form of the pair: two adds + one min3
  kFfmaFresh, kFaddFresh, kMin3Fresh,                        // every source operand a different register each time
  kRealPair,                                                 // t = a[i] + b[j] (packed); acc[i][j] = min3(acc, t.lo, t.hi), 8 x 8
  kRealPairScalar,                                           // the same with two scalar adds
  kMaxMinPair,                                               // acc = max3(acc, min(a0, b0), min(a1, b1)), 8 x 8
  kCases
};

template <int CASE>
__global__ void __launch_bounds__(256, 1) kern(float* out, long long* cyc, float seed) {
  float x[kChains], y[kChains], z[kChains];
  u64 px[kChains];
  const float c0 = seed * 1.5f, c1 = seed * 2.5f;
  // halves ARE c0 and c1 (built with integer operations: the compiler then keeps the three in one register pair)
  const u64 pc_shared = (static_cast<u64>(__float_as_uint(c0)) << 32) | __float_as_uint(c1);
  const u64 pc_own = pack2(seed * 3.5f, seed * 4.5f);
#pragma unroll
  for (int i = 0; i < kChains; ++i) {
    x[i] = seed + i + threadIdx.x; y[i] = 1.0f + seed * 1e-6f * i; z[i] = seed * 1e-3f * i + threadIdx.x;
    px[i] = pack2(seed + i, seed - i + threadIdx.x);
  }
  // operands of the 8 x 8 outer-product cases
  u64 a[8], b[8];
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    a[i] = pack2(seed + i + threadIdx.x, seed * 2 + i);
    b[i] = pack2(seed * 3 + i, seed * 5 + i + threadIdx.x);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 1e30f + i + j;
  }
  const long long t0 = clock64();
#pragma unroll 1
  for (int it = 0; it < kIters; ++it) {
    if (CASE == kRealPair || CASE == kRealPairScalar || CASE == kMaxMinPair) {
      // keep the operands loop-variant at the cost of 16 packed adds per 64 pairs (counted in the divisor below)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        asm volatile("add.rn.f32x2 %0,%0,%1;" : "+l"(a[i]) : "l"(pc_own));
        asm volatile("add.rn.f32x2 %0,%0,%1;" : "+l"(b[i]) : "l"(pc_own));
      }
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (CASE == kRealPair) {
            u64 t; float lo, hi;
            asm volatile("add.rn.f32x2 %0,%1,%2;" : "=l"(t) : "l"(a[i]), "l"(b[j]));
            unpack2(t, lo, hi);
            asm volatile("min.f32 %0,%0,%1,%2;" : "+f"(acc[i][j]) : "f"(lo), "f"(hi));
          } else {
            float a0, a1, b0, b1, p0, p1;
            unpack2(a[i], a0, a1); unpack2(b[j], b0, b1);
            if (CASE == kRealPairScalar) {
              asm volatile("add.f32 %0,%1,%2;" : "=f"(p0) : "f"(a0), "f"(b0));
              asm volatile("add.f32 %0,%1,%2;" : "=f"(p1) : "f"(a1), "f"(b1));
              asm volatile("min.f32 %0,%0,%1,%2;" : "+f"(acc[i][j]) : "f"(p0), "f"(p1));
            } else {
              asm volatile("min.f32 %0,%1,%2;" : "=f"(p0) : "f"(a0), "f"(b0));
              asm volatile("min.f32 %0,%1,%2;" : "=f"(p1) : "f"(a1), "f"(b1));
              asm volatile("max.f32 %0,%0,%1,%2;" : "+f"(acc[i][j]) : "f"(p0), "f"(p1));
            }
          }
        }
    } else {
#pragma unroll
      for (int i = 0; i < kChains; ++i) {
        if (CASE == kAdd2Alone) asm volatile("add.rn.f32x2 %0,%0,%1;" : "+l"(px[i]) : "l"(pc_own));
        if (CASE == kMin3Alone) asm volatile("min.f32 %0,%0,%1,%2;" : "+f"(x[i]) : "f"(c0), "f"(c1));
        if (CASE == kFaddAlone) asm volatile("add.f32 %0,%0,%1;" : "+f"(x[i]) : "f"(c0));
        if (CASE == kFfmaAlone) asm volatile("fma.rn.f32 %0,%0,%1,%2;" : "+f"(x[i]) : "f"(c0), "f"(c1));
        if (CASE == kAdd2Min3SharedConst) {
          asm volatile("add.rn.f32x2 %0,%0,%1;" : "+l"(px[i]) : "l"(pc_shared));
          asm volatile("min.f32 %0,%0,%1,%2;" : "+f"(x[i]) : "f"(c0), "f"(c1));
        }
        if (CASE == kAdd2Min3OwnConst) {
          asm volatile("add.rn.f32x2 %0,%0,%1;" : "+l"(px[i]) : "l"(pc_own));
          asm volatile("min.f32 %0,%0,%1,%2;" : "+f"(x[i]) : "f"(c0), "f"(c1));
        }
        if (CASE == kTwoFaddMin3) {
          asm volatile("add.f32 %0,%0,%1;" : "+f"(y[i]) : "f"(c0));
          asm volatile("add.f32 %0,%0,%1;" : "+f"(z[i]) : "f"(c1));
          asm volatile("min.f32 %0,%0,%1,%2;" : "+f"(x[i]) : "f"(c0), "f"(c1));
        }
        if (CASE == kFfmaFresh) asm volatile("fma.rn.f32 %0,%0,%1,%2;" : "+f"(x[i]) : "f"(y[(i + 1) % kChains]), "f"(z[(i + 2) % kChains]));
        if (CASE == kFaddFresh) asm volatile("add.f32 %0,%0,%1;" : "+f"(x[i]) : "f"(y[(i + 1) % kChains]));
        if (CASE == kMin3Fresh) asm volatile("min.f32 %0,%0,%1,%2;" : "+f"(x[i]) : "f"(y[(i + 1) % kChains]), "f"(z[(i + 2) % kChains]));
      }
    }
  }
  const long long t1 = clock64();
  // only what the case touched is summed, so that the other arrays are dead and take no registers
  float s = 0;
  constexpr bool outer_case = CASE == kRealPair || CASE == kRealPairScalar || CASE == kMaxMinPair;
  if (!outer_case) {
#pragma unroll
    for (int i = 0; i < kChains; ++i) {
      float lo, hi; unpack2(px[i], lo, hi);
      s += x[i];
      if (CASE == kAdd2Alone || CASE == kAdd2Min3SharedConst || CASE == kAdd2Min3OwnConst) s += lo + hi;
      if (CASE == kTwoFaddMin3 || CASE == kFfmaFresh || CASE == kFaddFresh || CASE == kMin3Fresh) s += y[i] + z[i];
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float lo, hi; unpack2(a[i], lo, hi); s += lo + hi; unpack2(b[i], lo, hi); s += lo + hi;
#pragma unroll
      for (int j = 0; j < 8; ++j) s += acc[i][j];
    }
  }
  out[blockIdx.x * blockDim.x + threadIdx.x] = s;
  if (threadIdx.x == 0) cyc[blockIdx.x] = t1 - t0;
}

template <int CASE>
static int run(const char* name, int nsm, float* out, long long* cyc) {
  for (int rep = 0; rep < 2; ++rep) {
    kern<CASE><<<nsm, 256>>>(out, cyc, 1.0f);
    CK(cudaDeviceSynchronize());
  }
  long long h[512];
  CK(cudaMemcpy(h, cyc, sizeof(long long) * nsm, cudaMemcpyDeviceToHost));
  double avg = 0;
  for (int i = 0; i < nsm; ++i) avg += static_cast<double>(h[i]);
  avg /= nsm;
  const bool outer = CASE == kRealPair || CASE == kRealPairScalar || CASE == kMaxMinPair;
  // outer-product cases: 64 pairs + 16 operand updates (each as long as a packed add) per iteration
  const double groups = outer ? 64.0 : static_cast<double>(kChains);
  const double overhead = outer ? 16.0 * 2.0 * 2.0 : 0.0;       // 16 packed adds x 2 clk x 2 warps, per iteration
  std::printf("%-28s : %.2f\n", name, (avg / kIters - overhead) / groups / 2.0);
  return 0;
}

int main() {
  cudaDeviceProp prop;
  CK(cudaGetDeviceProperties(&prop, 0));
  const int nsm = prop.multiProcessorCount < 512 ? prop.multiProcessorCount : 512;
  float* out = nullptr;
  long long* cyc = nullptr;
  CK(cudaMalloc(&out, sizeof(float) * nsm * 256));
  CK(cudaMalloc(&cyc, sizeof(long long) * 512));
  std::printf("# %s, %d SMs; clocks per instruction group per scheduler, 2 warps per scheduler\n", prop.name, nsm);
  run<kAdd2Alone>("add2_alone", nsm, out, cyc);
  run<kMin3Alone>("min3_alone", nsm, out, cyc);
  run<kFaddAlone>("fadd_alone", nsm, out, cyc);
  run<kFfmaAlone>("ffma_alone", nsm, out, cyc);
  run<kAdd2Min3SharedConst>("add2_min3_shared_constants", nsm, out, cyc);
  run<kAdd2Min3OwnConst>("add2_min3_own_constants", nsm, out, cyc);
  run<kTwoFaddMin3>("two_fadd_min3", nsm, out, cyc);
  run<kFfmaFresh>("ffma_three_fresh_operands", nsm, out, cyc);
  run<kFaddFresh>("fadd_two_fresh_operands", nsm, out, cyc);
  run<kMin3Fresh>("min3_three_fresh_operands", nsm, out, cyc);
  run<kRealPair>("pair_add2_min3_8x8", nsm, out, cyc);
  run<kRealPairScalar>("pair_two_fadd_min3_8x8", nsm, out, cyc);
  run<kMaxMinPair>("pair_two_min_max3_8x8", nsm, out, cyc);
  return 0;
}
