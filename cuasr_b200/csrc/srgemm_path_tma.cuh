// Path-tracking tropical SRGEMM on the TMA pipeline: dist <- min/max(dist, A (x) B) in place, and for every element
// the contraction index k that first produced its final value (parent), fp32.
//
// Same role as srgemm_path_kernel (the device counterpart of the reference's legacy routine cpu_fwgemm_naive,
// test/regress/include/fwgpu/cpu_srgemm.hpp:20-48), same staging as srgemm_tma_kernel: one persistent CTA per SM,
// a producer lane that feeds a ring of shared-memory stages with TMA tile loads, eight consumer warps over a
// 128 x 128 tile with an 8 x 8 micro-tile per lane.
//
// The contraction is the plain kernel's: per element and four k, two packed (or four scalar) adds and two
// three-input min/max.  A product that IMPROVES an element is rare after the first few k (the n-th product of a
// random sequence is a new minimum with probability 1/n), so nothing per product is spent on the index: each row
// of eight elements is followed by one test "did any bit of this row change over these four k" (one three-input
// logic instruction per element), and only then the improved elements of the row are noted in a bit mask.  After
// the last row a loop runs once per noted element: it forms the four products again from the stage, takes the first
// k that attains their best, and stores that k straight to the parent matrix.  Every output element
// lives in one lane, and that lane meets the K range in ascending order, so its stores to one parent element are
// ordered and "the first k that gives the best value" needs no comparison between lanes; K is never split over
// CTAs here for the same reason.  An element that never improves keeps the parent it came with: the parent matrix
// is not read at all.
// Ragged K and ragged tiles: out-of-range operand elements are NaN (TMA fill), and a NaN product never compares as
// an improvement.
#pragma once

#include "srgemm_tma.cuh"

namespace cuasr_b200 {

__device__ __forceinline__ float lds4(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}

struct PathTmaParams {
  int M, N, K;
  float* dist;      long long d_row, d_col;     // dist(m, n) at dist[m * d_row + n * d_col], read and written
  int32_t* parent;  long long p_row, p_col;     // same shape; written where an element improves, never read
  int k_offset;                                 // added to every recorded k
  int tiles_m, tiles_n;
  unsigned int* status;
};

constexpr int kPathTmaSmemBytes = kStages * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;

template <bool kMaximize, bool kAK, bool kBK>
__global__ void __launch_bounds__(kTmaThreads, 1)
srgemm_path_tma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const PathTmaParams p) {
  constexpr int TK = kTileKBytes / 4;   // 32 k per stage
  constexpr int kChunks = TK / 4;       // 8 chunks of 16 bytes

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  volatile unsigned int* abandoned = reinterpret_cast<unsigned int*>(empty_bar + kStages);   // see ptx.cuh

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kConsumerWarps);
    }
    *abandoned = 0;
    fence_barrier_init();
  }
  __syncthreads();

  const int k_tiles = (p.K + TK - 1) / TK;
  const int num_tiles = p.tiles_m * p.tiles_n;

  if (warp >= kConsumerWarps) {
    // ---------------------------------------------------------------- producer
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kProducerRegs));
    if (warp == kConsumerWarps && lane == 0) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
        int tm, tn;
        tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
        for (int kt = 0; kt < k_tiles; ++kt, ++it) {
          const int s = it % kStages;
          const uint32_t round = it / kStages;
          if (round > 0 && !mbar_wait(&empty_bar[s], (round - 1) & 1, p.status, kDeviceTimeoutEmpty)) return;
          mbar_arrive_expect_tx(&full_bar[s], kStageBytes);
          uint8_t* sa = smem + s * kStageBytes;
          uint8_t* sb = sa + kOperandStageBytes;
          if (kAK) tma_load_2d(sa, &map_a, &full_bar[s], kt * TK, tm * kTileM);
          else     tma_load_2d(sa, &map_a, &full_bar[s], tm * kTileM, kt * TK);
          if (kBK) tma_load_2d(sb, &map_b, &full_bar[s], kt * TK, tn * kTileN);
          else     tma_load_2d(sb, &map_b, &full_bar[s], tn * kTileN, kt * TK);
        }
      }
    }
    return;
  }

  // ------------------------------------------------------------------ consumers
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kConsumerRegs));
  const int wm = warp / 4, wn = warp % 4;
  const int lr = lane / 4, lc = lane % 4;
  auto row_of = [&](int i) { return kAK ? (lr + 8 * i) : (4 * lr + (i % 4) + 32 * (i / 4)); };
  auto col_of = [&](int j) { return kBK ? (lc + 4 * j) : (4 * lc + (j % 4) + 16 * (j / 4)); };
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t a_base = kAK ? (wm * 64 + lr) * 128 : (wm * 64 + 4 * lr) * 4;
  const uint32_t b_base = kBK ? (wn * 32 + lc) * 128 : (wn * 32 + 4 * lc) * 4;
  auto better = [](float candidate, float current) { return kMaximize ? candidate > current : candidate < current; };
  auto best3 = [](float x, float y, float z) { return kMaximize ? max3(x, y, z) : min3(x, y, z); };

  float acc[8][8];

  uint32_t it = 0;
  for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
    int tm, tn;
    tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
    const int m_base = tm * kTileM + wm * 64, n_base = tn * kTileN + wn * 32;

    // the running best starts from what is stored: an element outside the matrix can never improve (NaN operands)
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int m = m_base + row_of(i), n = n_base + col_of(j);
        acc[i][j] = (m < p.M && n < p.N) ? p.dist[m * p.d_row + n * p.d_col] : 0.0f;
      }

    for (int kt = 0; kt < k_tiles; ++kt, ++it) {
      const int s = it % kStages;
      mbar_wait_or_abandon(&full_bar[s], (it / kStages) & 1, p.status, kDeviceTimeoutFull, abandoned);
      const uint32_t sa = smem_base + s * kStageBytes;
      const uint32_t sb = sa + kOperandStageBytes;
#pragma unroll 1
      for (int chunk = 0; chunk < kChunks; ++chunk) {
        // a[i][e] = A(row i, k = 4 * chunk + e), b[j][e] = B(k = 4 * chunk + e, column j)
        float a[8][4], b[8][4];
        if (kAK) {
          const uint32_t base = sa + a_base + (((chunk ^ lr) & 7) << 4);
#pragma unroll
          for (int i = 0; i < 8; ++i) lds16(base + i * 1024, a[i]);
        } else {
          const uint32_t base = sa + a_base + chunk * (4 * kTileM * 4);
#pragma unroll
          for (int e = 0; e < 4; ++e)
#pragma unroll
            for (int g = 0; g < 2; ++g) {
              float v[4];
              lds16(base + e * (kTileM * 4) + g * 128, v);
#pragma unroll
              for (int t = 0; t < 4; ++t) a[g * 4 + t][e] = v[t];
            }
        }
        if (kBK) {
          const uint32_t base0 = sb + b_base + (((chunk ^ lc) & 7) << 4);
          const uint32_t base1 = sb + b_base + (((chunk ^ (lc + 4)) & 7) << 4);
#pragma unroll
          for (int j = 0; j < 8; ++j) lds16(((j & 1) ? base1 : base0) + j * 512, b[j]);
        } else {
          const uint32_t base = sb + b_base + chunk * (4 * kTileN * 4);
#pragma unroll
          for (int e = 0; e < 4; ++e)
#pragma unroll
            for (int g = 0; g < 2; ++g) {
              float v[4];
              lds16(base + e * (kTileN * 4) + g * 64, v);
#pragma unroll
              for (int t = 0; t < 4; ++t) b[g * 4 + t][e] = v[t];
            }
        }
        const int32_t k0 = kt * TK + chunk * 4 + p.k_offset;
        float next[4][8];
        uint32_t any[4];
        uint32_t improved_lo = 0, improved_hi = 0;     // bit 8 i + j: element (i, j) improved in this chunk
        auto fold_row = [&](int i, int buf) {
          uint32_t changed = 0;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float s0, s1, s2, s3;
            if constexpr (kAK && kBK) {
              unpack2(add2(pack2(a[i][0], a[i][1]), pack2(b[j][0], b[j][1])), s0, s1);
              unpack2(add2(pack2(a[i][2], a[i][3]), pack2(b[j][2], b[j][3])), s2, s3);
            } else {
              s0 = a[i][0] + b[j][0]; s1 = a[i][1] + b[j][1];
              s2 = a[i][2] + b[j][2]; s3 = a[i][3] + b[j][3];
            }
            next[buf][j] = best3(best3(acc[i][j], s0, s1), s2, s3);
            // the folds only ever move a value in one direction, so the bit patterns differ exactly where a
            // value improved
            changed |= __float_as_uint(next[buf][j]) ^ __float_as_uint(acc[i][j]);
          }
          any[buf] = changed;
        };
        // Two rows per test, and the test on one pair of rows is issued after the folds of the next pair, so that
        // the chain add -> fold -> "anything changed?" -> branch runs under the arithmetic of other rows.
        fold_row(0, 0);
        fold_row(1, 1);
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
          const int buf = i & 2;
          if (i + 2 < 8) {
            fold_row(i + 2, buf ^ 2);
            fold_row(i + 3, (buf ^ 2) + 1);
          }
          if (__builtin_expect((any[buf] | any[buf + 1]) != 0, 0)) {
            // something in these rows improved: note which elements, the k are looked up after the last row
            uint32_t bits = 0;
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (better(next[buf + r][j], acc[i + r][j])) bits |= 1u << (8 * r + j);
            if (i < 4) improved_lo |= bits << (8 * i);
            else       improved_hi |= bits << (8 * (i - 4));
          }
#pragma unroll
          for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[i + r][j] = next[buf + r][j];
        }
        // One pass per improved element of this lane; most chunks have none.  The improvements of an element are
        // strict, so its new value is the best of the four products and the k of the last improvement is the
        // first k that attains it.  The operands are read again from the stage (it stays put until this warp
        // releases it): the loop is ordinary code with computed addresses, one copy of it per chunk.
        while (__builtin_expect((improved_lo | improved_hi) != 0, 0)) {
          int bit;
          if (improved_lo != 0) { bit = __ffs(improved_lo) - 1; improved_lo &= improved_lo - 1; }
          else                  { bit = 31 + __ffs(improved_hi); improved_hi &= improved_hi - 1; }
          const int i = bit >> 3, j = bit & 7;
          float ar[4], br[4];
          if (kAK) {
            lds16(sa + a_base + (((chunk ^ lr) & 7) << 4) + i * 1024, ar);
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              ar[e] = lds4(sa + a_base + (chunk * 4 + e) * (kTileM * 4) + ((i % 4) + 32 * (i / 4)) * 4);
          }
          if (kBK) {
            lds16(sb + b_base + (((chunk ^ (lc + 4 * (j & 1))) & 7) << 4) + j * 512, br);
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              br[e] = lds4(sb + b_base + (chunk * 4 + e) * (kTileN * 4) + ((j % 4) + 16 * (j / 4)) * 4);
          }
          float best = ar[0] + br[0];
          int e_first = 0;
#pragma unroll
          for (int e = 1; e < 4; ++e) {
            const float sum = ar[e] + br[e];
            if (better(sum, best)) { best = sum; e_first = e; }
          }
          const int m = m_base + row_of(i), n = n_base + col_of(j);
          if (m < p.M && n < p.N) p.parent[m * p.p_row + n * p.p_col] = k0 + e_first;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
    }

    // (the opaque zero: the addresses are computed here again instead of being carried through the loop above)
    int zero;
    asm volatile("mov.s32 %0, 0;" : "=r"(zero));
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int m = m_base + row_of(i) + zero, n = n_base + col_of(j) + zero;
        if (m < p.M && n < p.N) p.dist[m * p.d_row + n * p.d_col] = acc[i][j];
      }
  }
}

// Launches srgemm_path_tma_kernel<maximize, a_kcontig, b_kcontig> on `grid` persistent CTAs.
cudaError_t launch_path_tma(bool maximize, bool a_kcontig, bool b_kcontig, const CUtensorMap& map_a,
                            const CUtensorMap& map_b, const PathTmaParams& params, int grid, cudaStream_t stream);

}  // namespace cuasr_b200
