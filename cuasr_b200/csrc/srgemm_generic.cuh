// Fallback SRGEMM kernel: any ring, any element type, any alignment and leading dimension.
//
// It plays the role of the reference's only kernel (include/cuasr/gemm/kernel/srgemm.h:156-321 with the
// mainloop of include/cuasr/gemm/threadblock/srmma_pipelined.h:153-288) for the cases the TMA kernel
// cannot take: operands that are not 16-byte aligned, leading dimensions that are not multiples of
// 16 bytes, rings with no safe padding value, and tiny problems.  Out-of-range elements are never
// loaded and never enter the contraction, exactly like the host SRGEMM that only loops over k < K.
#pragma once

#include "ring.cuh"

namespace cuasr_b200 {

template <typename T>
struct GenericParams {
  int M, N, K;               // row-major-C view of the problem
  const T* A;  long long a_row, a_col;   // element (m, k) of A at A[m * a_row + k * a_col]
  const T* B;  long long b_row, b_col;   // element (k, n) of B at B[k * b_row + n * b_col]
  const T* C;  long long ldc;            // row-major, may alias D, may be null when !read_c
  T* D;        long long ldd;            // row-major
  int n_extra;               // further copies of the output (same ld), possibly in peer-GPU memory
  T* extra_d[7];
  T alpha, beta, add_identity;
  int read_c;                // epilogue uses C: D = add(mul(alpha, acc), mul(beta, C)); else D = mul(alpha, acc)
  // split-K: slice z of gridDim.z covers k in [z * k_per_slice, min(K, (z + 1) * k_per_slice)) and writes
  // its raw accumulators to partial + z * M * N (row-major, ld N) instead of running the epilogue.
  int k_per_slice;
  T* partial;
  int tiles_n;               // tiles along N: the tile index runs along grid.x (2^31 - 1 tiles), slices along grid.z
};

constexpr int kGenTile = 64;     // CTA tile 64 x 64
constexpr int kGenK = 16;        // K step held in shared memory
constexpr int kGenThreads = 256; // 16 x 16 threads, 4 x 4 outputs each

template <typename RingT>
__global__ void __launch_bounds__(kGenThreads)
srgemm_generic_kernel(GenericParams<typename RingT::Element> p) {
  using T = typename RingT::Element;
  __shared__ T As[kGenK][kGenTile + 1];
  __shared__ T Bs[kGenK][kGenTile + 1];

  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;
  const int m0 = (blockIdx.x / p.tiles_n) * kGenTile, n0 = (blockIdx.x % p.tiles_n) * kGenTile;

  int k_begin = 0, k_end = p.K;
  if (p.partial != nullptr) {
    k_begin = blockIdx.z * p.k_per_slice;
    k_end = min(p.K, k_begin + p.k_per_slice);
    if (blockIdx.z == gridDim.z - 1) k_end = p.K;
  }

  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = p.add_identity;

  for (int k0 = k_begin; k0 < k_end; k0 += kGenK) {
    const int kt = min(kGenK, k_end - k0);
    // stage the A and B tiles; an element outside the matrix is simply not used below
    for (int e = tid; e < kGenK * kGenTile; e += kGenThreads) {
      // let the contiguous dimension of each operand vary fastest across threads
      int kk, mm;
      if (p.a_col == 1) { kk = e % kGenK; mm = e / kGenK; } else { mm = e % kGenTile; kk = e / kGenTile; }
      if (kk < kt && m0 + mm < p.M) As[kk][mm] = p.A[(long long)(m0 + mm) * p.a_row + (long long)(k0 + kk) * p.a_col];
      int nn;
      if (p.b_row == 1) { kk = e % kGenK; nn = e / kGenK; } else { nn = e % kGenTile; kk = e / kGenTile; }
      if (kk < kt && n0 + nn < p.N) Bs[kk][nn] = p.B[(long long)(k0 + kk) * p.b_row + (long long)(n0 + nn) * p.b_col];
    }
    __syncthreads();
    for (int kk = 0; kk < kt; ++kk) {
      T a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty + 16 * i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx + 16 * j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = RingT::add(RingT::mul(a[i], b[j]), acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty + 16 * i;
    if (m >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx + 16 * j;
      if (n >= p.N) continue;
      if (p.partial != nullptr) {
        p.partial[((long long)blockIdx.z * p.M + m) * p.N + n] = acc[i][j];
      } else {
        T v = RingT::mul(p.alpha, acc[i][j]);
        if (p.read_c) v = RingT::add(v, RingT::mul(p.beta, p.C[(long long)m * p.ldc + n]));
        p.D[(long long)m * p.ldd + n] = v;
        for (int x = 0; x < p.n_extra; ++x) p.extra_d[x][(long long)m * p.ldd + n] = v;
      }
    }
  }
}

// Folds the slices of a split-K run in slice order and applies the epilogue: one thread per output.
template <typename RingT>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(GenericParams<typename RingT::Element> p, int slices) {
  using T = typename RingT::Element;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long total = static_cast<long long>(p.M) * p.N;
  if (idx >= total) return;
  const int m = static_cast<int>(idx / p.N), n = static_cast<int>(idx % p.N);
  T r = p.add_identity;
  for (int z = 0; z < slices; ++z) r = RingT::add(p.partial[z * total + idx], r);
  T v = RingT::mul(p.alpha, r);
  if (p.read_c) v = RingT::add(v, RingT::mul(p.beta, p.C[(long long)m * p.ldc + n]));
  p.D[(long long)m * p.ldd + n] = v;
  for (int x = 0; x < p.n_extra; ++x) p.extra_d[x][(long long)m * p.ldd + n] = v;
}

// Re-packs a rows x K operand into K-contiguous storage (dst[r * ld_dst + k]) through 32 x 32 shared-memory tiles.
// The source is either MN-contiguous (element (r, k) at src[r + k * ld_src]: a transposition, reads and writes both
// coalesced) or K-contiguous with a leading dimension or address TMA cannot use (src[r * ld_src + k]: a copy).
// W is an unsigned integer of the element's width: the data is only moved.  Tiles are numbered along grid.x
// (rows fastest), so neither extent is limited by the 65535 of the other grid dimensions.
template <typename W>
__global__ void __launch_bounds__(256)
repack_to_kcontig_kernel(const W* __restrict__ src, long long ld_src, int src_kcontig, int rows, int K, int K_out,
                         W pad, W* __restrict__ dst, long long ld_dst, int tiles_r) {
  __shared__ W tile[32][33];
  const int r0 = (blockIdx.x % tiles_r) * 32, k0 = (blockIdx.x / tiles_r) * 32;
  const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;   // 32 x 8
  if (!src_kcontig) {
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      const int r = r0 + tx, k = k0 + ty + i;
      if (r < rows && k < K) tile[ty + i][tx] = src[r + (long long)k * ld_src];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 32; i += 8) {
    const int r = r0 + ty + i, k = k0 + tx;
    if (r < rows && k < K_out)
      dst[(long long)r * ld_dst + k] = k >= K ? pad : src_kcontig ? src[(long long)r * ld_src + k] : tile[tx][ty + i];
  }
}

}  // namespace cuasr_b200
