// The B200 SRGEMM kernel: D = (alpha (x) (A (x)(+) B)) (+) (beta (x) C), row-major D.
//
// It replaces, as one kernel, the reference's kernel::Srgemm (include/cuasr/gemm/kernel/srgemm.h:156-321),
// its threadblock mainloop SrmmaPipelined (include/cuasr/gemm/threadblock/srmma_pipelined.h:153-288),
// the warp/thread level (include/cuasr/gemm/warp/srmma_simt.h:139-199,
// include/cuasr/gemm/thread/srmma_sm50.h:118-146) and the epilogue functor
// (include/cuasr/gemm/epilogue/thread/semiring_linear_combination.h:118-183); with `partial` set it is
// also the first half of kernel::SrgemmSplitKParallel (include/cuasr/gemm/kernel/srgemm_splitk_parallel.h:86-219).
//
// Structure (one persistent CTA per SM, 12 warps = 2 consumer warpgroups + 1 producer warpgroup that
// hands most of its registers to the consumers with setmaxnreg):
//   warp 8, lane 0      producer: for every K tile of every output tile this CTA owns, waits for a free
//                       stage and issues two TMA tile loads (A, B) that complete on the stage's mbarrier.
//   warps 0..7          consumers: 2 x 4 warps over a 128 x 128 output tile, 8 x 4 lanes per warp, an
//                       8 x 8 register micro-tile per lane.  They wait for a stage, read 16-byte vectors
//                       from shared memory and run the contraction two k steps at a time:
//                       acc = add(acc, a0 (x) b0, a1 (x) b1)  — for fp32 min/max rings one add per product
//                       plus ONE three-input min/max per two products.
// Shared-memory tile layouts (per stage, 16 KiB per operand):
//   K-contiguous operand  (row-major A, column-major B): [128 rows][128 bytes of k], TMA 128-byte swizzle;
//                         a lane owns rows lane_row + 8 i (A) / lane_col + 4 j (B) and loads 16 bytes of k.
//   MN-contiguous operand (column-major A, row-major B): [k][128 rows], no swizzle; a lane owns groups of
//                         16/sizeof(T) adjacent rows and loads one k of a group per 16-byte vector.
// Ragged edges: TMA fills out-of-range elements with NaN (fp min/max rings; min/max never select a NaN
// product) or zero (rings where 0 (x) 0 is neutral); stores are predicated on m < M, n < N.
#pragma once

#include "ring.cuh"

namespace cuasr_b200 {

constexpr int kTileM = 128;
constexpr int kTileN = 128;
constexpr int kTileKBytes = 128;                 // bytes of k per stage and row
constexpr int kStages = 5;
constexpr int kConsumerWarps = 8;
constexpr int kProducerWarps = 4;                 // one warpgroup; only its first lane issues TMA
constexpr int kTmaThreads = (kConsumerWarps + kProducerWarps) * 32;
// Registers per thread after the warpgroups re-balance with setmaxnreg: the two consumer warps and
// the one producer warp that share an SM sub-partition fit its 16384 registers (2 * 232 + 40 = 504 <= 512).
constexpr int kConsumerRegs = 232;
constexpr int kProducerRegs = 40;
constexpr int kOperandStageBytes = kTileM * kTileKBytes;   // 16 KiB
constexpr int kStageBytes = 2 * kOperandStageBytes;
constexpr int kEpilogueWarpBytes = 8192;          // per consumer warp: staging for coalesced output rows
constexpr int kEpilogueBytes = kConsumerWarps * kEpilogueWarpBytes;
constexpr int kMaxDestinations = 8;               // output copies one launch can write (this GPU + peers)
constexpr int kTmaSmemBytes =
    kStages * kStageBytes + kEpilogueBytes + 1024 /* alignment slack */ + 256 /* barriers */;

template <typename T>
struct TmaParams {
  int M, N, K;
  const T* C;  long long ldc;   // row-major; may alias D; may be null when !read_c
  T* D;        long long ldd;   // row-major
  // Extra copies of the output: when n_extra > 0 every element of D is also stored to extra_d[i] (same
  // leading dimension).  The pointers may be peer-GPU memory; this is how the sharded squaring step pushes
  // its block of the result into every rank's next-iteration matrix while the tile is still in registers.
  int n_extra;
  T* extra_d[kMaxDestinations - 1];
  T alpha, beta, add_identity;
  int read_c;
  int vector_epilogue;          // D, C and every extra_d are 16-byte aligned, ld * sizeof(T) % 16 == 0, N % EV == 0
  int tiles_m, tiles_n;
  unsigned int* status;         // device status word (see DeviceStatus)
  // Work decomposition.  Tiles [0, whole_tiles) are computed whole by one CTA each.  Every later tile is cut
  // along K into `slices` pieces: piece z handles K tiles [z * k_tiles_per_slice, ...), the last piece takes the
  // rest, and writes its raw accumulators to partial + ((tile - whole_tiles) * slices + z) * 128 * 128 (a full
  // 128 x 128 block, row-major).  tickets[tile - whole_tiles] counts the pieces written; the CTA that draws the
  // last ticket folds the pieces in slice order and runs the epilogue, so nobody ever waits and the result does
  // not depend on which CTA finishes last.  tickets must be zero at launch; the kernel leaves them zero.
  // Explicit split-K is whole_tiles = 0; a balanced launch splits only the tiles of the last, partial wave.
  int whole_tiles, slices, k_tiles_per_slice;
  T* partial;
  unsigned int* tickets;
};

// One 16-byte shared-memory load into EV = 16 / sizeof(T) elements.
__device__ __forceinline__ void lds16(uint32_t addr, float (&v)[4]) {
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]) : "r"(addr));
}
__device__ __forceinline__ void lds16(uint32_t addr, uint32_t (&v)[4]) {
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(addr));
}
__device__ __forceinline__ void lds16(uint32_t addr, int32_t (&v)[4]) {
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(addr));
}
__device__ __forceinline__ void lds16(uint32_t addr, double (&v)[2]) {
  asm volatile("ld.shared.v2.f64 {%0,%1}, [%2];" : "=d"(v[0]), "=d"(v[1]) : "r"(addr));
}

// Tile rasterisation: bands of kBand tile columns, rows fastest inside a band, so that the CTAs that
// run at the same time share A row-panels and B column-panels in L2.
constexpr int kBand = 16;
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_band = kBand * tiles_m;
  const int band = t / per_band;
  const int in_band = t - band * per_band;
  const int width = min(kBand, tiles_n - band * kBand);
  tm = in_band / width;
  tn = band * kBand + in_band % width;
}

// Work item w of a launch -> (tile, K piece z, number of pieces of that tile).
__device__ __forceinline__ void decode_work(int w, int num_tiles, int whole_tiles, int slices, int& tile, int& z,
                                            int& pieces) {
  if (w < whole_tiles) {
    tile = w; z = 0; pieces = 1;
  } else {
    const int tail = num_tiles - whole_tiles;
    const int v = w - whole_tiles;
    z = v / tail;
    tile = whole_tiles + (v - z * tail);
    pieces = slices;
  }
}

template <typename RingT, bool kAK, bool kBK>
__global__ void __launch_bounds__(kTmaThreads, 1)
srgemm_tma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const TmaParams<typename RingT::Element> p) {
  using T = typename RingT::Element;
  constexpr int EV = 16 / sizeof(T);              // elements per 16-byte vector: 4 (fp32/int32) or 2 (fp64)
  constexpr int TK = kTileKBytes / sizeof(T);     // k per stage: 32 or 16
  constexpr int kChunks = TK / EV;                // 16-byte k chunks per stage: 8

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* epi_smem = smem + kStages * kStageBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(epi_smem + kEpilogueBytes);
  uint64_t* empty_bar = full_bar + kStages;
  unsigned int* ticket_smem = reinterpret_cast<unsigned int*>(empty_bar + kStages);
  volatile unsigned int* abandoned = ticket_smem + 1;     // raised when a consumer's wait ran out (see ptx.cuh)

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

  const int k_tiles_total = (p.K + TK - 1) / TK;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_work = p.whole_tiles + (num_tiles - p.whole_tiles) * p.slices;

  if (warp >= kConsumerWarps) {
    // ---------------------------------------------------------------- producer
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kProducerRegs));
    if (warp == kConsumerWarps && lane == 0) {
      prefetch_tensormap(&map_a);
      prefetch_tensormap(&map_b);
      uint32_t it = 0;  // running K-tile counter across all work items: stage = it % kStages
      for (int w = blockIdx.x; w < num_work; w += gridDim.x) {
        int tile, z, pieces, tm, tn;
        decode_work(w, num_tiles, p.whole_tiles, p.slices, tile, z, pieces);
        tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
        const int kt_begin = pieces == 1 ? 0 : z * p.k_tiles_per_slice;
        const int kt_end = (z == pieces - 1) ? k_tiles_total : min(k_tiles_total, kt_begin + p.k_tiles_per_slice);
        for (int kt = kt_begin; kt < kt_end; ++kt, ++it) {
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
  const int wm = warp / 4, wn = warp % 4;        // 2 x 4 warps
  const int lr = lane / 4, lc = lane % 4;        // 8 x 4 lanes
  // Row i (0..7) of this lane inside the warp's 64 rows; column j (0..7) inside the warp's 32 columns.
  // Plus-times fp64 runs on the tensor cores (DMMA): acc[mb][2 nb + e] is then element e of the lane's
  // accumulator pair of the 8 x 8 block (mb, nb) of the warp tile; its row inside the block is lr, its column
  // 2 lc + e.  Blocks fed from an MN-contiguous operand are interleaved in pairs (see the loaders below).
  constexpr bool kDmma = std::is_same<T, double>::value && RingT::kAdd == CUASR_OP_PLUS &&
                         RingT::kMul == CUASR_OP_MULTIPLIES;
  auto row_of = [&](int i) {
    if (kDmma) return kAK ? (8 * i + lr) : (16 * (i / 2) + 2 * lr + (i % 2));
    return kAK ? (lr + 8 * i) : (EV * lr + (i % EV) + 8 * EV * (i / EV));
  };
  auto col_of = [&](int j) {
    if (kDmma) return kBK ? (8 * (j / 2) + 2 * lc + (j % 2)) : (16 * (j / 4) + 4 * lc + 2 * (j % 2) + ((j / 2) % 2));
    return kBK ? (lc + 4 * j) : (EV * lc + (j % EV) + 4 * EV * (j / EV));
  };

  // Byte offset of this lane's first operand vector inside a stage; every other vector of the lane is a
  // compile-time constant away from it.
  //   K-contiguous:  row * 128 + ((chunk ^ (row & 7)) * 16)        (TMA 128-byte swizzle)
  //                  A rows are lr + 8 i  -> + i * 1024 bytes, row & 7 == lr for every i
  //                  B rows are lc + 4 j  -> + j * 512 bytes,  row & 7 == lc + 4 (j & 1)
  //   MN-contiguous: k * (128 * sizeof(T)) + first_row_of_group * sizeof(T); groups are 8 EV (A) or
  //                  4 EV (B) rows apart -> + g * 128 / + g * 64 bytes
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t a_base = kAK ? (wm * 64 + lr) * 128 : (wm * 64 + EV * lr) * (int)sizeof(T);
  const uint32_t b_base = kBK ? (wn * 32 + lc) * 128 : (wn * 32 + EV * lc) * (int)sizeof(T);

  T acc[8][8];

  // Per-lane byte offsets of the eight 16-byte k chunks of a K-contiguous operand row, swizzle applied: computed
  // once, so that inside the contraction an operand vector is addressed as (stage base + one of these + a constant).
  // Only for 4-byte elements: with 8-byte elements the accumulators leave no registers for the table, and the
  // offsets are computed where they are used.
  constexpr bool kOffsetTable = sizeof(T) == 4;
  // chunks unrolled in the contraction loop; the table holds the offsets of that many chunks, and chunk c + kUnroll
  // of a stage is reached by flipping bit 6 of the offset (bit 2 of the chunk index; a_base and b_base are
  // multiples of 128, so the flip commutes with adding them)
  // (four chunks keep the loop body near 16 KiB of instructions; unrolling all eight measured the same on min-plus
  // and 25 % slower on max-min, whose body is half as large again)
  constexpr int kUnroll = 4;
  uint32_t a_off[kOffsetTable ? kUnroll : 1], b_off[kOffsetTable ? 8 : 1];
  if constexpr (kOffsetTable) {
#pragma unroll
    for (int c = 0; c < kUnroll; ++c) a_off[c] = a_base + (((c ^ lr) & 7) << 4);
#pragma unroll
    for (int c = 0; c < 8; ++c) b_off[c] = b_base + (((c ^ lc) & 7) << 4);      // rows lc + 4 j with odd j use b_off[c ^ 4]
  }

  uint32_t it = 0;
  for (int w = blockIdx.x; w < num_work; w += gridDim.x) {
    int tile, z, pieces, tm, tn;
    decode_work(w, num_tiles, p.whole_tiles, p.slices, tile, z, pieces);
    tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
    const int kt_begin = pieces == 1 ? 0 : z * p.k_tiles_per_slice;
    const int kt_end = (z == pieces - 1) ? k_tiles_total : min(k_tiles_total, kt_begin + p.k_tiles_per_slice);

#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[i][j] = p.add_identity;

    for (int kt = kt_begin; kt < kt_end; ++kt, ++it) {
      const int s = it % kStages;
      mbar_wait_or_abandon(&full_bar[s], (it / kStages) & 1, p.status, kDeviceTimeoutFull, abandoned);
      const uint32_t sa = smem_base + s * kStageBytes;
      const uint32_t sb = sa + kOperandStageBytes;

      // fragment loaders for one 16-byte k chunk: a[i][e] = A(row i, k = chunk * EV + e).  With the offset table the
      // chunk is given as (c, h): chunk = h * kUnroll + c with c a compile-time constant; without it h is 0.
      auto load_a = [&](T (&a)[8][EV], int c, int h = 0) {
        const int chunk = kOffsetTable ? h * kUnroll + c : c;
        if (kAK) {
          uint32_t base;
          if constexpr (kOffsetTable) base = sa + (a_off[c] ^ (h << 6));
          else base = sa + a_base + (((chunk ^ lr) & 7) << 4);
#pragma unroll
          for (int i = 0; i < 8; ++i) lds16(base + i * 1024, a[i]);
        } else {
          const uint32_t base = sa + a_base + chunk * (EV * kTileM * (int)sizeof(T));
#pragma unroll
          for (int e = 0; e < EV; ++e) {
#pragma unroll
            for (int g = 0; g < 8 / EV; ++g) {
              T v[EV];
              lds16(base + e * (kTileM * (int)sizeof(T)) + g * 128, v);
#pragma unroll
              for (int t = 0; t < EV; ++t) a[g * EV + t][e] = v[t];
            }
          }
        }
      };
      auto load_b = [&](T (&b)[8][EV], int c, int h = 0) {
        const int chunk = kOffsetTable ? h * kUnroll + c : c;
        if (kBK) {
          uint32_t base0, base1;
          if constexpr (kOffsetTable) {
            base0 = sb + (b_off[c] ^ (h << 6));
            base1 = sb + (b_off[c ^ 4] ^ (h << 6));
          } else {
            base0 = sb + b_base + (((chunk ^ lc) & 7) << 4);
            base1 = sb + b_base + (((chunk ^ (lc + 4)) & 7) << 4);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) lds16(((j & 1) ? base1 : base0) + j * 512, b[j]);
        } else {
          const uint32_t base = sb + b_base + chunk * (EV * kTileN * (int)sizeof(T));
#pragma unroll
          for (int e = 0; e < EV; ++e) {
#pragma unroll
            for (int g = 0; g < 8 / EV; ++g) {
              T v[EV];
              lds16(base + e * (kTileN * (int)sizeof(T)) + g * 64, v);
#pragma unroll
              for (int t = 0; t < EV; ++t) b[g * EV + t][e] = v[t];
            }
          }
        }
      };
      auto compute = [&](const T (&a)[8][EV], const T (&b)[8][EV]) {
        if constexpr (kAK && kBK && RingT::kPackedPairs) {
          // both fragments came from 16-byte loads along k: (k, k+1) are adjacent registers, so the pairs below
          // are register renames, not moves
#pragma unroll
          for (int e = 0; e < EV; e += 2) {
            uint64_t pa[8], pb[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) { pa[i] = pack2(a[i][e], a[i][e + 1]); pb[i] = pack2(b[i][e], b[i][e + 1]); }
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[i][j] = RingT::mac_packed(acc[i][j], pa[i], pb[j]);
          }
          return;
        }
#pragma unroll
        for (int e = 0; e < EV; e += 2)
#pragma unroll
          for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j)
              acc[i][j] = RingT::mac2(acc[i][j], a[i][e], b[j][e], a[i][e + 1], b[j][e + 1]);
      };

      if constexpr (kDmma) {
        // Tensor-core path.  The fp64 mma takes, per lane, A(row lr [+8], k slot lc [+4]) and B(k slot lc [+4], column lr).
        // The contraction index may be permuted freely as long as A and B agree: within a group of 8 k the
        // slot lc of step s (s = 0, 1) stands for k = 2 lc + s, so a K-contiguous operand delivers both steps of
        // a block with one 16-byte load.  An MN-contiguous operand delivers two adjacent rows with one 16-byte
        // load; they feed the two blocks of an interleaved pair (block rows 2 lr and 2 lr + 1).
        static_assert(!kDmma || TK == 16, "two groups of 8 k per stage");
        auto load_group = [&](double (&a)[8][2], double (&b)[4][2], int group) {
          if (kAK) {
            const uint32_t base = sa + (wm * 64 + lr) * 128 + ((((group * 4 + lc) ^ lr) & 7) << 4);
#pragma unroll
            for (int mb = 0; mb < 8; ++mb) lds16(base + mb * 1024, a[mb]);
          } else {
#pragma unroll
            for (int sstep = 0; sstep < 2; ++sstep) {
              const uint32_t base = sa + (group * 8 + 2 * lc + sstep) * (kTileM * 8) + (wm * 64 + 2 * lr) * 8;
#pragma unroll
              for (int pr = 0; pr < 4; ++pr) {
                double v[2];
                lds16(base + pr * 128, v);
                a[2 * pr][sstep] = v[0];
                a[2 * pr + 1][sstep] = v[1];
              }
            }
          }
          if (kBK) {
            const uint32_t base = sb + (wn * 32 + lr) * 128 + ((((group * 4 + lc) ^ lr) & 7) << 4);
#pragma unroll
            for (int nb = 0; nb < 4; ++nb) lds16(base + nb * 1024, b[nb]);
          } else {
#pragma unroll
            for (int sstep = 0; sstep < 2; ++sstep) {
              const uint32_t base = sb + (group * 8 + 2 * lc + sstep) * (kTileN * 8) + (wn * 32 + 2 * lr) * 8;
#pragma unroll
              for (int pr = 0; pr < 2; ++pr) {
                double v[2];
                lds16(base + pr * 128, v);
                b[2 * pr][sstep] = v[0];
                b[2 * pr + 1][sstep] = v[1];
              }
            }
          }
        };
        auto mma_group = [&](const double (&a)[8][2], const double (&b)[4][2]) {
          // m16n8k8: rows lr and lr + 8 of the instruction are the two 8-row blocks 2 h and 2 h + 1, k slots lc and
          // lc + 4 are the two steps of this group
#pragma unroll
          for (int h = 0; h < 4; ++h)
#pragma unroll
            for (int nb = 0; nb < 4; ++nb)
              asm volatile(
                  "mma.sync.aligned.m16n8k8.row.col.f64.f64.f64.f64 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                  "{%0, %1, %2, %3};"
                  : "+d"(acc[2 * h][2 * nb]), "+d"(acc[2 * h][2 * nb + 1]), "+d"(acc[2 * h + 1][2 * nb]),
                    "+d"(acc[2 * h + 1][2 * nb + 1])
                  : "d"(a[2 * h][0]), "d"(a[2 * h + 1][0]), "d"(a[2 * h][1]), "d"(a[2 * h + 1][1]), "d"(b[nb][0]),
                    "d"(b[nb][1]));
        };
        double a0[8][2], b0[4][2], a1[8][2], b1[4][2];
        load_group(a0, b0, 0);
        load_group(a1, b1, 1);
        mma_group(a0, b0);
        mma_group(a1, b1);
      } else if constexpr (sizeof(T) == 4) {
        // 4-byte elements: operand fragments are double-buffered in registers (64 + 4 x 32 registers)
        T a0[8][EV], b0[8][EV], a1[8][EV], b1[8][EV];
        load_a(a0, 0, 0);
        load_b(b0, 0, 0);
        // kUnroll chunks at a time with compile-time chunk indices, so that the only integer work left per chunk is
        // combining the stage base with a table entry (integer instructions share the half-rate pipe with the
        // three-input min: each one costs as much as a product pair)
#pragma unroll 1
        for (int h = 0; h < kChunks / kUnroll; ++h) {
#pragma unroll
          for (int c = 0; c < kUnroll; c += 2) {
            load_a(a1, c + 1, h);
            load_b(b1, c + 1, h);
            compute(a0, b0);
            if (c + 2 < kUnroll) {
              load_a(a0, c + 2, h);
              load_b(b0, c + 2, h);
            } else if (h + 1 < kChunks / kUnroll) {
              load_a(a0, 0, h + 1);
              load_b(b0, 0, h + 1);
            }
            compute(a1, b1);
          }
        }
      } else {
        // 8-byte elements: the 8 x 8 accumulators alone take 128 registers, so one fragment set is live
        T a0[8][EV], b0[8][EV];
#pragma unroll 1
        for (int chunk = 0; chunk < kChunks; ++chunk) {
          load_a(a0, chunk);
          load_b(b0, chunk);
          compute(a0, b0);
        }
      }
      // Release the stage only after the math that consumed its last fragments: every value loaded from it is
      // then in registers for certain (a release placed right after the loads leaves the compiler free to sink
      // not-yet-needed loads below it, and the refill would race with them).
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
    }

    // ---------------------------------------------------------------- epilogue
    const int m_base = tm * kTileM + wm * 64, n_base = tn * kTileN + wn * 32;
    if (pieces > 1) {
      // A piece of a split tile: park the raw accumulators in the tile's scratch block, in "fragment order"
      // ([16 vectors][256 consumer threads][16 bytes], so that every access is a coalesced 16-byte vector and the
      // thread that folds reads exactly the layout it would have written), then take a ticket.
      constexpr int kVecPerThread = 64 / EV;
      const int split = tile - p.whole_tiles;                     // index among the split tiles
      T* block = p.partial + (long long)split * pieces * (kTileM * kTileN);
      uint4* mine = reinterpret_cast<uint4*>(block + (long long)z * (kTileM * kTileN)) + threadIdx.x;
#pragma unroll
      for (int v = 0; v < kVecPerThread; ++v) {
        alignas(16) T tmp[EV];
#pragma unroll
        for (int e = 0; e < EV; ++e) tmp[e] = acc[(v * EV + e) / 8][(v * EV + e) % 8];
        mine[v * (kConsumerWarps * 32)] = *reinterpret_cast<const uint4*>(tmp);
      }
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
      if (threadIdx.x == 0) *ticket_smem = atomicAdd(&p.tickets[split], 1u);
      asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
      const bool last = (*ticket_smem == (unsigned)pieces - 1);
      asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
      if (!last) continue;
      // This CTA completed the tile: fold all pieces in slice order (a fixed order, whoever comes last), then
      // fall through to the ordinary epilogue with the folded accumulators.
      __threadfence();
      if (threadIdx.x == 0) p.tickets[split] = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = p.add_identity;
      for (int zz = 0; zz < pieces; ++zz) {
        const uint4* theirs = reinterpret_cast<const uint4*>(block + (long long)zz * (kTileM * kTileN)) + threadIdx.x;
        uint4 raw[kVecPerThread];
#pragma unroll
        for (int v = 0; v < kVecPerThread; ++v) raw[v] = __ldcg(theirs + v * (kConsumerWarps * 32));
#pragma unroll
        for (int v = 0; v < kVecPerThread; ++v) {
          alignas(16) T tmp[EV];
          *reinterpret_cast<uint4*>(tmp) = raw[v];
#pragma unroll
          for (int e = 0; e < EV; ++e) {
            T& a = acc[(v * EV + e) / 8][(v * EV + e) % 8];
            a = RingT::add(tmp[e], a);
          }
        }
      }
    }
    if (p.vector_epilogue) {

      // Coalesced path: the warp's 64 x 32 block goes through its private staging area (rows of 32
      // elements, the 16-byte column groups XOR-swizzled by row & 7), then every lane handles 16 bytes of
      // a row: C is read, the epilogue applied and the vector stored to D and to every extra copy.
      constexpr int kRowsPerPass = kEpilogueWarpBytes / (32 * (int)sizeof(T));   // 64 (4-byte) or 32 (8-byte)
      constexpr int kGroups = 32 / EV;                                            // 16-byte groups per row
      T* stage = reinterpret_cast<T*>(epi_smem + warp * kEpilogueWarpBytes);
#pragma unroll
      for (int pass = 0; pass < 64 / kRowsPerPass; ++pass) {
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = row_of(i) - pass * kRowsPerPass;
          if (r < 0 || r >= kRowsPerPass) continue;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int c = col_of(j);
            const int group = ((c / EV) ^ (r & 7)) & (kGroups - 1);
            stage[r * 32 + group * EV + (c % EV)] = acc[i][j];
          }
        }
        __syncwarp();
#pragma unroll 4
        for (int idx = lane; idx < kRowsPerPass * kGroups; idx += 32) {
          const int r = idx / kGroups, g = idx % kGroups;
          const int m = m_base + pass * kRowsPerPass + r;
          const int n = n_base + g * EV;
          if (m >= p.M || n >= p.N) continue;
          const int group = (g ^ (r & 7)) & (kGroups - 1);
          alignas(16) T v[EV];
          *reinterpret_cast<uint4*>(v) = *reinterpret_cast<const uint4*>(stage + r * 32 + group * EV);
#pragma unroll
          for (int e = 0; e < EV; ++e) v[e] = RingT::mul(p.alpha, v[e]);
          if (p.read_c) {
            alignas(16) T c[EV];
            *reinterpret_cast<uint4*>(c) = *reinterpret_cast<const uint4*>(p.C + (long long)m * p.ldc + n);
#pragma unroll
            for (int e = 0; e < EV; ++e) v[e] = RingT::add(v[e], RingT::mul(p.beta, c[e]));
          }
          const long long off = (long long)m * p.ldd + n;
          *reinterpret_cast<uint4*>(p.D + off) = *reinterpret_cast<const uint4*>(v);
          for (int x = 0; x < p.n_extra; ++x) *reinterpret_cast<uint4*>(p.extra_d[x] + off) = *reinterpret_cast<const uint4*>(v);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int m = m_base + row_of(i);
        if (m >= p.M) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int n = n_base + col_of(j);
          if (n >= p.N) continue;
          T v = RingT::mul(p.alpha, acc[i][j]);
          if (p.read_c) v = RingT::add(v, RingT::mul(p.beta, p.C[(long long)m * p.ldc + n]));
          const long long off = (long long)m * p.ldd + n;
          p.D[off] = v;
          for (int x = 0; x < p.n_extra; ++x) p.extra_d[x][off] = v;
        }
      }
    }
  }
}

}  // namespace cuasr_b200
