// Path-tracking tropical SRGEMM on the TMA pipeline: dist <- min/max(dist, A (x) B) in place, and for every element
// the contraction index k that first produced its final value (parent), fp32.
//
// Same role as srgemm_path_kernel (the device counterpart of the reference's legacy routine cpu_fwgemm_naive,
// test/regress/include/fwgpu/cpu_srgemm.hpp:20-48), same staging as srgemm_tma_kernel: one persistent CTA per SM,
// a producer lane that feeds a ring of shared-memory stages with TMA tile loads, eight consumer warps over a
// 128 x 128 tile with an 8 x 8 micro-tile per lane.  What is new is the second accumulator set: idx[8][8] holds the
// k of the best product so far.  Every output element lives in one lane, and that lane meets the K range in
// ascending order (stage after stage, chunk after chunk), so "the first k that gives the best value" needs no
// comparison between lanes; K is never split over CTAs here for the same reason.
//
// The contraction keeps the two-instruction form of the plain kernel (one packed or two scalar adds and one
// three-input min/max per two products).  A product that IMPROVES an element is rare after the first few k (the
// n-th product of a random sequence is a new minimum with probability 1/n), so the index is not updated with
// selects in every step: each row of eight folds is followed by one test "did anything in this row change", and
// only then the row is replayed element by element in k order to find out which k it was.
// Ragged K: out-of-range operand elements are NaN (TMA fill), and a NaN product never compares as an improvement.
#pragma once

#include "srgemm_tma.cuh"

namespace cuasr_b200 {

__device__ __forceinline__ void lds8(uint32_t addr, float (&v)[2]) {
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v[0]), "=f"(v[1]) : "r"(addr));
}

struct PathTmaParams {
  int M, N, K;
  float* dist;      long long d_row, d_col;     // dist(m, n) at dist[m * d_row + n * d_col], read and written
  int32_t* parent;  long long p_row, p_col;     // same shape, read and written
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
  int32_t idx[8][8];

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
        const bool in = m < p.M && n < p.N;
        acc[i][j] = in ? p.dist[m * p.d_row + n * p.d_col] : 0.0f;
        idx[i][j] = in ? p.parent[m * p.p_row + n * p.p_col] : 0;
      }

    for (int kt = 0; kt < k_tiles; ++kt, ++it) {
      const int s = it % kStages;
      mbar_wait_or_abandon(&full_bar[s], (it / kStages) & 1, p.status, kDeviceTimeoutFull, abandoned);
      const uint32_t sa = smem_base + s * kStageBytes;
      const uint32_t sb = sa + kOperandStageBytes;
#pragma unroll 1
      for (int step = 0; step < 2 * kChunks; ++step) {
        // two k per step (the two accumulator sets leave room for no more operand registers):
        // a[i][e] = A(row i, k = 2 * step + e)
        const int chunk = step >> 1, half = step & 1;
        float a[8][2], b[8][2];
        if (kAK) {
          const uint32_t base = sa + a_base + (((chunk ^ lr) & 7) << 4) + half * 8;
#pragma unroll
          for (int i = 0; i < 8; ++i) lds8(base + i * 1024, a[i]);
        } else {
          const uint32_t base = sa + a_base + step * (2 * kTileM * 4);
#pragma unroll
          for (int e = 0; e < 2; ++e)
#pragma unroll
            for (int g = 0; g < 2; ++g) {
              float v[4];
              lds16(base + e * (kTileM * 4) + g * 128, v);
#pragma unroll
              for (int t = 0; t < 4; ++t) a[g * 4 + t][e] = v[t];
            }
        }
        if (kBK) {
          const uint32_t base0 = sb + b_base + (((chunk ^ lc) & 7) << 4) + half * 8;
          const uint32_t base1 = sb + b_base + (((chunk ^ (lc + 4)) & 7) << 4) + half * 8;
#pragma unroll
          for (int j = 0; j < 8; ++j) lds8(((j & 1) ? base1 : base0) + j * 512, b[j]);
        } else {
          const uint32_t base = sb + b_base + step * (2 * kTileN * 4);
#pragma unroll
          for (int e = 0; e < 2; ++e)
#pragma unroll
            for (int g = 0; g < 2; ++g) {
              float v[4];
              lds16(base + e * (kTileN * 4) + g * 64, v);
#pragma unroll
              for (int t = 0; t < 4; ++t) b[g * 4 + t][e] = v[t];
            }
        }
        const int32_t k0 = kt * TK + step * 2 + p.k_offset;
        // The rows are software-pipelined by one: the folds of row i + 1 are issued before the test on row i, so
        // that the chain add -> fold -> "anything changed?" -> branch of one row runs under the arithmetic of the next.
        float lo[2][8], hi[2][8], next[2][8];
        uint32_t any[2];
        auto fold_row = [&](int i, int buf) {
          uint32_t diff[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            if constexpr (kAK && kBK) {
              unpack2(add2(pack2(a[i][0], a[i][1]), pack2(b[j][0], b[j][1])), lo[buf][j], hi[buf][j]);
            } else {
              lo[buf][j] = a[i][0] + b[j][0];
              hi[buf][j] = a[i][1] + b[j][1];
            }
            next[buf][j] = best3(acc[i][j], lo[buf][j], hi[buf][j]);
            // the folds only ever move a value in one direction, so the bit patterns differ exactly where a
            // value improved
            diff[j] = __float_as_uint(next[buf][j]) ^ __float_as_uint(acc[i][j]);
          }
          any[buf] = ((diff[0] | diff[1]) | (diff[2] | diff[3])) | ((diff[4] | diff[5]) | (diff[6] | diff[7]));
        };
        fold_row(0, 0);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int buf = i & 1;
          if (i + 1 < 8) fold_row(i + 1, buf ^ 1);
          if (any[buf] != 0) {
            // something in this row improved: replay its two k steps in order to see which one it was
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float cur = acc[i][j];
              if (better(lo[buf][j], cur)) { cur = lo[buf][j]; idx[i][j] = k0; }
              if (better(hi[buf][j], cur)) { idx[i][j] = k0 + 1; }
            }
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[i][j] = next[buf][j];
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
    }

#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int m = m_base + row_of(i), n = n_base + col_of(j);
        if (m < p.M && n < p.N) {
          p.dist[m * p.d_row + n * p.d_col] = acc[i][j];
          p.parent[m * p.p_row + n * p.p_col] = idx[i][j];
        }
      }
  }
}

// Launches srgemm_path_tma_kernel<maximize, a_kcontig, b_kcontig> on `grid` persistent CTAs.
cudaError_t launch_path_tma(bool maximize, bool a_kcontig, bool b_kcontig, const CUtensorMap& map_a,
                            const CUtensorMap& map_b, const PathTmaParams& params, int grid, cudaStream_t stream);

}  // namespace cuasr_b200
