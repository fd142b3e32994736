// extern "C" boundary of the library: validation, layout normalisation, kernel choice and launch.
//
// Host-side counterpart of the reference's device::Srgemm (include/cuasr/gemm/device/srgemm.h:85-357 and
// its column-major specialisation :398-567) and device::SrgemmSplitKParallel
// (include/cuasr/gemm/device/srgemm_splitk_parallel.h:101-378, :424-607).
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>

#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/cuasr_b200.h"
#include "../../include/cuasr_b200_apsp.h"
#include "srgemm_launch.h"
#include "srgemm_path.cuh"
#include "srgemm_path_tma.cuh"

namespace cuasr_b200 {
namespace {

std::atomic<uint64_t> g_launches{0};
thread_local const char* t_last_kernel = "none";

// ---- per-device state: SM count and the device status word --------------------------------------
__device__ unsigned int g_status_word;  // zero-initialised when the module loads

struct DeviceState {
  bool ready = false;
  int sms = 0;
  unsigned int* status = nullptr;
};
constexpr int kMaxDevices = 64;
DeviceState g_devices[kMaxDevices];
std::mutex g_device_mutex;

// First call on a device looks up the SM count and the address of the status word; no allocation.
bool device_state(DeviceState** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return false;
  std::lock_guard<std::mutex> lock(g_device_mutex);
  DeviceState& st = g_devices[dev];
  if (!st.ready) {
    if (cudaDeviceGetAttribute(&st.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return false;
    void* addr = nullptr;
    if (cudaGetSymbolAddress(&addr, g_status_word) != cudaSuccess) return false;
    st.status = static_cast<unsigned int*>(addr);
    st.ready = true;
  }
  *out = &st;
  return true;
}

// ---- cuTensorMapEncodeTiled through the runtime, so that the library does not link libcuda --------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

template <typename T> struct TmaType;
template <> struct TmaType<float>    { static constexpr CUtensorMapDataType v = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; };
template <> struct TmaType<double>   { static constexpr CUtensorMapDataType v = CU_TENSOR_MAP_DATA_TYPE_FLOAT64; };
template <> struct TmaType<int32_t>  { static constexpr CUtensorMapDataType v = CU_TENSOR_MAP_DATA_TYPE_INT32; };
template <> struct TmaType<uint32_t> { static constexpr CUtensorMapDataType v = CU_TENSOR_MAP_DATA_TYPE_UINT32; };

// Describes one operand of `rows` x K elements to TMA.
//   K-contiguous:  tensor {K, rows}, box {128 bytes of k, 128 rows}, 128-byte swizzle
//   MN-contiguous: tensor {rows, K}, box {128 rows, 128 bytes worth of k}, no swizzle
template <typename T>
bool make_operand_map(CUtensorMap* map, const T* ptr, long long ld, int rows, int K, bool kcontig, bool nan_fill) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (encode == nullptr) return false;
  const cuuint32_t tk = kTileKBytes / sizeof(T);
  cuuint64_t dims[2];
  cuuint32_t box[2];
  if (kcontig) { dims[0] = K; dims[1] = rows; box[0] = tk; box[1] = kTileM; }
  else         { dims[0] = rows; dims[1] = K; box[0] = kTileM; box[1] = tk; }
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * sizeof(T)};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult r = encode(map, TmaType<T>::v, 2, const_cast<T*>(ptr), dims, strides, box, elem_strides,
                            CU_TENSOR_MAP_INTERLEAVE_NONE,
                            kcontig ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            nan_fill ? CU_TENSOR_MAP_FLOAT_OOB_FILL_NAN_REQUEST_ZERO_FMA
                                     : CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// ---- host evaluation of ring operators (only for the "is C needed" decision) ----------------------
template <typename T>
T host_op(int op, T l, T r) {
  switch (op) {
    case CUASR_OP_PLUS: return l + r;
    case CUASR_OP_MULTIPLIES: return l * r;
    case CUASR_OP_MINIMUM: return r < l ? r : l;
    case CUASR_OP_MAXIMUM: return l < r ? r : l;
    case CUASR_OP_BINARY_AND: return static_cast<T>(l && r);
    case CUASR_OP_BINARY_OR: return static_cast<T>(l || r);
    default: break;
  }
  if constexpr (std::is_integral<T>::value) {
    switch (op) {
      case CUASR_OP_BIT_AND: return l & r;
      case CUASR_OP_BIT_OR: return l | r;
      case CUASR_OP_BIT_XOR: return l ^ r;
      default: break;
    }
  }
  return l;
}

template <typename T>
T load_scalar(const cuasr_b200_scalar_t& s) {
  T v;
  std::memcpy(&v, s.bytes, sizeof(T));
  return v;
}

bool ring_supported(int add, int mul, int dtype) {
  const bool is_int = (dtype == CUASR_S32 || dtype == CUASR_U32);
  auto is = [&](int a, int m) { return add == a && mul == m; };
  if (is(CUASR_OP_PLUS, CUASR_OP_MULTIPLIES) || is(CUASR_OP_MINIMUM, CUASR_OP_PLUS) ||
      is(CUASR_OP_MAXIMUM, CUASR_OP_PLUS) || is(CUASR_OP_MINIMUM, CUASR_OP_MAXIMUM) ||
      is(CUASR_OP_MAXIMUM, CUASR_OP_MINIMUM) || is(CUASR_OP_MINIMUM, CUASR_OP_MULTIPLIES) ||
      is(CUASR_OP_MAXIMUM, CUASR_OP_MULTIPLIES) || is(CUASR_OP_BINARY_OR, CUASR_OP_BINARY_AND))
    return true;
  if (is_int && (is(CUASR_OP_BIT_XOR, CUASR_OP_BIT_AND) || is(CUASR_OP_BIT_OR, CUASR_OP_BIT_AND) ||
                 is(CUASR_OP_BIT_XOR, CUASR_OP_BINARY_AND)))
    return true;
  return false;
}

// The problem after the column-major-C transposition of device/srgemm.h:432-453, :513-523: always a
// row-major D (m x n), A' (m x k) and B' (k x n), each operand either K-contiguous or MN-contiguous.
struct Normalised {
  int m, n, k;
  const void* a; long long lda; bool a_kcontig;
  const void* b; long long ldb; bool b_kcontig;
  const void* c; long long ldc;
  void* d;       long long ldd;
};

Normalised normalise(const cuasr_b200_desc_t& desc, const cuasr_b200_args_t& args) {
  Normalised p;
  p.k = args.k;
  p.c = args.C; p.ldc = args.ldc; p.d = args.D; p.ldd = args.ldd;
  if (desc.layout_c == CUASR_ROW_MAJOR) {
    p.m = args.m; p.n = args.n;
    p.a = args.A; p.lda = args.lda; p.a_kcontig = (desc.layout_a == CUASR_ROW_MAJOR);
    p.b = args.B; p.ldb = args.ldb; p.b_kcontig = (desc.layout_b == CUASR_COLUMN_MAJOR);
  } else {
    // D^T = B^T (x)(+) A^T; a column-major matrix is the row-major storage of its transpose
    p.m = args.n; p.n = args.m;
    p.a = args.B; p.lda = args.ldb; p.a_kcontig = (desc.layout_b == CUASR_COLUMN_MAJOR);
    p.b = args.A; p.ldb = args.lda; p.b_kcontig = (desc.layout_a == CUASR_ROW_MAJOR);
  }
  return p;
}

int validate(const cuasr_b200_desc_t* desc, const cuasr_b200_args_t* args) {
  if (desc == nullptr || args == nullptr) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  if (desc->dtype < CUASR_F32 || desc->dtype > CUASR_U32) return CUASR_STATUS_ERROR_INVALID_DATA_TYPE;
  for (int l : {desc->layout_a, desc->layout_b, desc->layout_c})
    if (l != CUASR_ROW_MAJOR && l != CUASR_COLUMN_MAJOR) return CUASR_STATUS_ERROR_INVALID_LAYOUT;
  if (!ring_supported(desc->add_op, desc->mul_op, desc->dtype)) return CUASR_STATUS_ERROR_NOT_SUPPORTED;
  if (args->m <= 0 || args->n <= 0 || args->k <= 0) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  if (args->split_k_slices < 1) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  if (args->A == nullptr || args->B == nullptr || args->D == nullptr) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  // A leading dimension shorter than the contiguous extent makes storage lines overlap.  For D (and C, which may
  // alias it) that would be a race, so it is refused.  A and B are only read: the reference never looks at their
  // leading dimensions (its own examples/02_splitk_srgemm/splitk_srgemm.cu:247-248 passes 128 for a row-major
  // 128 x 4096 operand), and an overlapping view is well defined, so any positive value is accepted; such views
  // run on the generic kernel.
  const long long c_min = desc->layout_c == CUASR_ROW_MAJOR ? args->n : args->m;
  if (args->lda < 1 || args->ldb < 1 || args->ldd < c_min) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  if (args->C != nullptr && args->ldc < c_min) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  const size_t es = desc->dtype == CUASR_F64 ? 8 : 4;
  for (const void* ptr : {args->A, args->B, args->C, static_cast<const void*>(args->D)})
    if (reinterpret_cast<uintptr_t>(ptr) % es != 0) return CUASR_STATUS_ERROR_MISALIGNED_OPERAND;
  return CUASR_STATUS_SUCCESS;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

size_t tile_count(const cuasr_b200_args_t& args) {
  return static_cast<size_t>((args.m + kTileM - 1) / kTileM) * ((args.n + kTileN - 1) / kTileN);
}
size_t ticket_bytes_for(const cuasr_b200_args_t& args) { return align_up(tile_count(args) * sizeof(unsigned int), 256); }

// Scratch layout: [tickets: one u32 per 128 x 128 tile, padded to 256 B][partials: one full 128 x 128 block per
// (split tile, slice)].  With every tile split (explicit split-K) that is tiles * slices blocks, which also
// covers the slices * m * n elements the fallback kernel needs.
size_t splitk_bytes_for_pieces(const cuasr_b200_desc_t& desc, const cuasr_b200_args_t& args, long long pieces) {
  const size_t es = desc.dtype == CUASR_F64 ? 8 : 4;
  return ticket_bytes_for(args) + es * tile_count(args) * kTileM * kTileN * static_cast<size_t>(pieces);
}

// Explicit split-K: into how many pieces of consecutive K tiles every output tile is really cut.  The reference
// launches exactly tiles x slices CTAs (include/cuasr/gemm/kernel/srgemm_splitk_parallel.h:86-89), whatever the GPU;
// here a slice count that leaves SMs idle (4 tiles x 16 slices = 64 work items on 148 SMs, or 4 x 32 = 128) is
// refined to the piece count in [slices, 8 x slices] that the cost model likes best (4 x 37 = 148).  That is only
// done where (+) is exact and order-independent (everything but floating-point plus): the pieces are folded in K
// order and the result cannot depend on how K was cut, hence not on the SM count either.  The cost model counts K
// tiles: waves x (K tiles per piece) for the contraction, plus half a K tile per piece for parking and folding a
// 128 x 128 partial.
bool splitk_order_independent(const cuasr_b200_desc_t& desc) {
  return !(desc.add_op == CUASR_OP_PLUS && (desc.dtype == CUASR_F32 || desc.dtype == CUASR_F64));
}
long long splitk_pieces(const cuasr_b200_desc_t& desc, const cuasr_b200_args_t& args, int sms, long long max_pieces) {
  const long long slices = args.split_k_slices;
  if (sms <= 0 || slices <= 1 || !splitk_order_independent(desc)) return slices;
  const int tk = kTileKBytes / (desc.dtype == CUASR_F64 ? 8 : 4);
  const long long k_tiles = (args.k + tk - 1) / tk;
  const long long tiles = static_cast<long long>(tile_count(args));
  auto cost = [&](long long pieces) {
    const long long waves = (tiles * pieces + sms - 1) / sms;
    return static_cast<double>(waves * ((k_tiles + pieces - 1) / pieces)) + 0.5 * static_cast<double>(pieces);
  };
  long long best = slices;
  double best_cost = cost(slices);
  const long long limit = std::min<long long>(std::min<long long>(8 * slices, max_pieces), k_tiles / 4);
  for (long long pieces = slices + 1; pieces <= limit; ++pieces) {
    const double c = cost(pieces);
    if (c < 0.97 * best_cost) { best = pieces; best_cost = c; }
  }
  return best;
}

// Workspace the split-K entry points ask for: room for the refined plan on the current GPU (the plain
// tiles x slices layout where no GPU is visible).  A smaller workspace, down to the plain layout, is accepted at run
// time and simply limits the refinement.
size_t splitk_workspace_bytes(const cuasr_b200_desc_t& desc, const cuasr_b200_args_t& args) {
  if (args.split_k_slices <= 1) return 0;
  return splitk_bytes_for_pieces(desc, args, args.split_k_slices);
}
size_t splitk_workspace_bytes_refined(const cuasr_b200_desc_t& desc, const cuasr_b200_args_t& args) {
  if (args.split_k_slices <= 1) return 0;
  DeviceState* dev = nullptr;
  const long long pieces = device_state(&dev) ? splitk_pieces(desc, args, dev->sms, 1LL << 30) : args.split_k_slices;
  return splitk_bytes_for_pieces(desc, args, pieces);
}

// Load balancing of a launch that was not asked to split K: the tiles of the last, partial wave are cut along K
// so that their pieces fill the SMs.  Returns the number of pieces (1 = leave the launch alone) and the number of
// tiles that stay whole.
struct BalancePlan {
  int whole_tiles;
  int pieces;
};
BalancePlan balance_plan(long long tiles, int sms, int k_tiles) {
  BalancePlan plan{static_cast<int>(tiles), 1};
  if (sms <= 0 || tiles <= 0) return plan;
  const long long rem = tiles % sms;
  if (rem == 0) return plan;
  double best = 1.0;    // time of the last wave in units of one whole tile
  const int max_pieces = k_tiles / 4 < 16 ? k_tiles / 4 : 16;
  for (int s = 2; s <= max_pieces; ++s) {
    const double t = static_cast<double>((rem * s + sms - 1) / sms) / s + 0.02 * s;   // + a little per piece for the fold
    if (t < best - 0.05) { best = t; plan.pieces = s; }
  }
  if (plan.pieces > 1) plan.whole_tiles = static_cast<int>(tiles - rem);
  return plan;
}
size_t balance_workspace_bytes(const cuasr_b200_desc_t& desc, const cuasr_b200_args_t& args, int sms) {
  const size_t es = desc.dtype == CUASR_F64 ? 8 : 4;
  const int tk = kTileKBytes / static_cast<int>(es);
  const BalancePlan plan = balance_plan(static_cast<long long>(tile_count(args)), sms, (args.k + tk - 1) / tk);
  if (plan.pieces <= 1) return 0;
  return ticket_bytes_for(args) + es * (tile_count(args) - plan.whole_tiles) * kTileM * kTileN * plan.pieces;
}

// Dispatch over rings.  X(ADD, MUL) is expanded for each ring the element type supports.
#define CUASR_FLOAT_RINGS(X)                   \
  X(CUASR_OP_PLUS, CUASR_OP_MULTIPLIES)        \
  X(CUASR_OP_MINIMUM, CUASR_OP_PLUS)           \
  X(CUASR_OP_MAXIMUM, CUASR_OP_PLUS)           \
  X(CUASR_OP_MINIMUM, CUASR_OP_MAXIMUM)        \
  X(CUASR_OP_MAXIMUM, CUASR_OP_MINIMUM)        \
  X(CUASR_OP_MINIMUM, CUASR_OP_MULTIPLIES)     \
  X(CUASR_OP_MAXIMUM, CUASR_OP_MULTIPLIES)     \
  X(CUASR_OP_BINARY_OR, CUASR_OP_BINARY_AND)
#define CUASR_BIT_RINGS(X)                     \
  X(CUASR_OP_BIT_XOR, CUASR_OP_BIT_AND)        \
  X(CUASR_OP_BIT_OR, CUASR_OP_BIT_AND)         \
  X(CUASR_OP_BIT_XOR, CUASR_OP_BINARY_AND)

// Further destinations of the output (cuasr_b200_srgemm_push); empty for the ordinary entry points.
struct ExtraOutputs {
  int count = 0;
  void* ptr[kMaxDestinations - 1] = {};
};

// Re-packing of MN-contiguous fp32 operands into K-contiguous scratch, so that the kernel variant with packed
// fp32x2 adds (both operands deliver (k, k+1) register pairs) can run.  Worth it only for the rings that variant
// speeds up, for problems large enough for the TMA kernel, and when the copy is cheap against what it buys: the
// variant is about 7 % faster (8192^3: 31.0 ms against 33.4), the copy moves 8 bytes per re-packed element, which
// breaks even near m n = 700 x (re-packed rows).  One rank's share of a sharded SRGEMM or one chunk of the host
// pipeline (8192 x 1024 x 8192) passes that test, thinner slices do not; copies of less than 16 MB are always taken
// (512^3: 0.076 -> 0.050 ms).
bool repack_pays(const cuasr_b200_desc_t& desc, const Normalised& p) {
  const bool ring = (desc.add_op == CUASR_OP_MINIMUM || desc.add_op == CUASR_OP_MAXIMUM) &&
                    (desc.mul_op == CUASR_OP_PLUS || desc.mul_op == CUASR_OP_MULTIPLIES);
  if (!(desc.dtype == CUASR_F32 && ring && static_cast<long long>(p.m) * p.n >= 256 * 256 && p.k >= 256 &&
        (!p.a_kcontig || !p.b_kcontig)))
    return false;
  const long long rows = (p.a_kcontig ? 0LL : p.m) + (p.b_kcontig ? 0LL : p.n);
  const bool small_copy = rows * p.k < 4LL * 1024 * 1024;
  return small_copy || static_cast<long long>(p.m) * p.n >= 700LL * rows;
}
// Which operands a launch copies into K-contiguous, 16-byte aligned scratch before the TMA kernel runs:
//   * an operand TMA cannot describe (its address or its leading dimension is not a multiple of 16 bytes; the
//     reference accepts alignment 1, include/cuasr/gemm/device/default_srgemm_configuration.h:88-89) - otherwise the
//     whole product would fall back to the generic kernel;
//   * an MN-contiguous fp32 operand of a ring with a packed-add variant, where that pays (repack_pays).
// Rows are padded to a multiple of 16 bytes; the padding is never read (the tensor map ends at K).
struct RepackPlan {
  bool a = false, b = false;
  int k_padded = 0;      // > 0: both copies are extended along K to this length (a multiple of the kernel's K step)
  size_t bytes = 0;
};
bool tma_describable(const void* ptr, long long ld, size_t es) {
  return reinterpret_cast<uintptr_t>(ptr) % 16 == 0 && (ld * static_cast<long long>(es)) % 16 == 0;
}
size_t repack_operand_bytes(int rows, int k, size_t es) {
  return align_up(static_cast<size_t>(rows) * align_up(static_cast<size_t>(k), 16 / es) * es, 256);
}
// Rings whose ragged last K step the TMA kernel pads by itself: floating min/max rings (out-of-range elements are
// filled with NaN, which min and max ignore) and rings where 0 (x) 0 is neutral (zero fill).
bool ring_pads_itself(const cuasr_b200_desc_t& desc, const cuasr_b200_args_t& args) {
  const bool is_float = desc.dtype == CUASR_F32 || desc.dtype == CUASR_F64;
  if (is_float && (desc.add_op == CUASR_OP_MINIMUM || desc.add_op == CUASR_OP_MAXIMUM)) return true;
  if (desc.add_op == CUASR_OP_PLUS && desc.mul_op == CUASR_OP_MULTIPLIES) return true;
  if ((desc.add_op == CUASR_OP_BIT_OR || desc.add_op == CUASR_OP_BIT_XOR) &&
      (desc.mul_op == CUASR_OP_BINARY_AND || desc.mul_op == CUASR_OP_BIT_AND))
    return true;
  if (desc.add_op == CUASR_OP_BINARY_OR && desc.mul_op == CUASR_OP_BINARY_AND) {
    // zero fill is neutral when the accumulator starts at 0 or 1
    switch (desc.dtype) {
      case CUASR_F32: { const float v = load_scalar<float>(args.add_identity); return v == 0.0f || v == 1.0f; }
      case CUASR_F64: { const double v = load_scalar<double>(args.add_identity); return v == 0.0 || v == 1.0; }
      default:        { const uint32_t v = load_scalar<uint32_t>(args.add_identity); return v == 0u || v == 1u; }
    }
  }
  return false;
}
// Every other ring (the integer min/max rings) has no value TMA could fill in.  With the optional workspace both
// operands are copied and their K range is extended to a whole number of K steps: A with the additive identity, B
// with the multiplicative one, so that every padded product is the additive identity.
RepackPlan repack_plan(const cuasr_b200_desc_t& desc, const cuasr_b200_args_t& args, const Normalised& p) {
  RepackPlan plan;
  const size_t es = desc.dtype == CUASR_F64 ? 8 : 4;
  // only problems the TMA kernel would take: not tiny, storage lines that do not overlap
  if (static_cast<long long>(p.m) * p.n < 64 * 64) return plan;
  if (p.lda < (p.a_kcontig ? p.k : p.m) || p.ldb < (p.b_kcontig ? p.k : p.n)) return plan;
  const int tk = kTileKBytes / static_cast<int>(es);
  if (p.k % tk != 0 && !ring_pads_itself(desc, args)) {
    plan.a = plan.b = true;
    plan.k_padded = (p.k + tk - 1) / tk * tk;
  } else {
    const bool pays = repack_pays(desc, p);
    plan.a = !tma_describable(p.a, p.lda, es) || (pays && !p.a_kcontig);
    plan.b = !tma_describable(p.b, p.ldb, es) || (pays && !p.b_kcontig);
  }
  const int k_copy = plan.k_padded > 0 ? plan.k_padded : p.k;
  plan.bytes = (plan.a ? repack_operand_bytes(p.m, k_copy, es) : 0) + (plan.b ? repack_operand_bytes(p.n, k_copy, es) : 0);
  return plan;
}

template <typename T>
int run_typed(const cuasr_b200_desc_t& desc, const cuasr_b200_args_t& args, int slices, const ExtraOutputs& extra) {
  DeviceState* dev = nullptr;
  if (!device_state(&dev)) return CUASR_STATUS_ERROR_INTERNAL;
  cudaStream_t stream = static_cast<cudaStream_t>(args.stream);
  Normalised p = normalise(desc, args);

  const T alpha = load_scalar<T>(args.alpha), beta = load_scalar<T>(args.beta);
  const T add_id = load_scalar<T>(args.add_identity), mul_id = load_scalar<T>(args.mul_identity);
  // semiring_linear_combination.h:118-125: C is read unless mult(beta, mult-identity) is the add-identity
  const bool read_c = !(host_op<T>(desc.mul_op, beta, mul_id) == add_id);
  if (read_c && p.c == nullptr) return CUASR_STATUS_ERROR_INVALID_PROBLEM;

  // split-K scratch
  unsigned int* tickets = nullptr;
  T* partial = nullptr;
  BalancePlan plan{static_cast<int>(tile_count(args)), 1};
  // partials are moved 16 bytes at a time and re-packed operands are read by TMA: a workspace that does not start
  // on a 16-byte boundary is an error where it is required and is left unused where it is optional
  const bool workspace_aligned = reinterpret_cast<uintptr_t>(args.workspace) % 16 == 0;
  if (slices > 1) {
    const size_t need = splitk_workspace_bytes(desc, args);
    if (args.workspace == nullptr) return CUASR_STATUS_ERROR_WORKSPACE_NULL;
    if (args.workspace_bytes < need) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
    if (!workspace_aligned) return CUASR_STATUS_ERROR_MISALIGNED_OPERAND;
    // as many pieces as the workspace at hand has room for (it always has room for `slices`)
    const size_t per_piece = splitk_bytes_for_pieces(desc, args, 1) - splitk_bytes_for_pieces(desc, args, 0);
    const long long room = static_cast<long long>((args.workspace_bytes - splitk_bytes_for_pieces(desc, args, 0)) / per_piece);
    plan = BalancePlan{0, static_cast<int>(splitk_pieces(desc, args, dev->sms, room))};
  } else if (args.workspace != nullptr && workspace_aligned) {
    // an optional workspace on an unsplit launch buys load balancing, if it is large enough for the plan
    constexpr int tk = kTileKBytes / sizeof(T);
    const BalancePlan wish = balance_plan(static_cast<long long>(tile_count(args)), dev->sms, (args.k + tk - 1) / tk);
    if (wish.pieces > 1 && args.workspace_bytes >= balance_workspace_bytes(desc, args, dev->sms)) plan = wish;
  }
  // the rest of an optional workspace holds K-contiguous, aligned copies of operands (see RepackPlan)
  bool repacked = false;
  int k_map = p.k;              // K extent the tensor maps describe
  if (slices == 1 && args.workspace != nullptr && workspace_aligned) {
    const size_t first = align_up(balance_workspace_bytes(desc, args, dev->sms), 256);
    const RepackPlan rp = repack_plan(desc, args, p);
    if (rp.bytes > 0 && args.workspace_bytes >= first + rp.bytes) {
      char* cursor = static_cast<char*>(args.workspace) + first;
      const int k_copy = rp.k_padded > 0 ? rp.k_padded : p.k;
      const long long ldt = static_cast<long long>(align_up(static_cast<size_t>(k_copy), 16 / sizeof(T)));
      unsigned long long pad_a = 0, pad_b = 0;
      std::memcpy(&pad_a, &add_id, sizeof(T));
      std::memcpy(&pad_b, &mul_id, sizeof(T));
      if (rp.a) {
        if (launch_repack(p.a, p.lda, p.a_kcontig, p.m, p.k, k_copy, pad_a, cursor, ldt, sizeof(T), stream) != cudaSuccess)
          return CUASR_STATUS_ERROR_INTERNAL;
        g_launches.fetch_add(1);
        p.a = cursor; p.lda = ldt; p.a_kcontig = true;
        cursor += repack_operand_bytes(p.m, k_copy, sizeof(T));
      }
      if (rp.b) {
        if (launch_repack(p.b, p.ldb, p.b_kcontig, p.n, p.k, k_copy, pad_b, cursor, ldt, sizeof(T), stream) != cudaSuccess)
          return CUASR_STATUS_ERROR_INTERNAL;
        g_launches.fetch_add(1);
        p.b = cursor; p.ldb = ldt; p.b_kcontig = true;
      }
      repacked = true;
      k_map = k_copy;
    }
  }
  if (plan.pieces > 1) {
    const size_t ticket_bytes = ticket_bytes_for(args);
    tickets = static_cast<unsigned int*>(args.workspace);
    partial = reinterpret_cast<T*>(static_cast<char*>(args.workspace) + ticket_bytes);
    // same role as the semaphore memset of device/srgemm.h:253-259
    if (cudaMemsetAsync(tickets, 0, ticket_bytes, stream) != cudaSuccess) return CUASR_STATUS_ERROR_INTERNAL;
  }

  constexpr int TK = kTileKBytes / sizeof(T);
  const bool is_float = std::is_floating_point<T>::value;
  const bool min_or_max = desc.add_op == CUASR_OP_MINIMUM || desc.add_op == CUASR_OP_MAXIMUM;
  const bool zero_pad_ok =
      (desc.add_op == CUASR_OP_PLUS && desc.mul_op == CUASR_OP_MULTIPLIES) ||
      ((desc.add_op == CUASR_OP_BIT_OR || desc.add_op == CUASR_OP_BIT_XOR) &&
       (desc.mul_op == CUASR_OP_BINARY_AND || desc.mul_op == CUASR_OP_BIT_AND)) ||
      (desc.add_op == CUASR_OP_BINARY_OR && desc.mul_op == CUASR_OP_BINARY_AND && (add_id == T(0) || add_id == T(1)));
  const bool nan_pad = is_float && min_or_max;
  const bool paddable = nan_pad || zero_pad_ok || (k_map % TK == 0);
  auto tma_ok = [&](const void* ptr, long long ld) {
    return reinterpret_cast<uintptr_t>(ptr) % 16 == 0 && (ld * (long long)sizeof(T)) % 16 == 0;
  };
  const bool small = static_cast<long long>(p.m) * p.n < 64 * 64;
  // operands whose storage lines overlap (leading dimension below the contiguous extent) stay off the TMA path
  const bool dense = p.lda >= (p.a_kcontig ? p.k : p.m) && p.ldb >= (p.b_kcontig ? p.k : p.n);
  bool use_tma = paddable && !small && dense && tma_ok(p.a, p.lda) && tma_ok(p.b, p.ldb) && encode_tiled_fn() != nullptr;

  cudaError_t err = cudaErrorInvalidValue;
  bool launched = false;
  if (use_tma) {
    CUtensorMap map_a, map_b;
    if (make_operand_map<T>(&map_a, static_cast<const T*>(p.a), p.lda, p.m, k_map, p.a_kcontig, nan_pad) &&
        make_operand_map<T>(&map_b, static_cast<const T*>(p.b), p.ldb, p.n, k_map, p.b_kcontig, nan_pad)) {
      TmaParams<T> tp;
      tp.M = p.m; tp.N = p.n; tp.K = p.k;
      tp.C = static_cast<const T*>(p.c); tp.ldc = p.ldc;
      tp.D = static_cast<T*>(p.d); tp.ldd = p.ldd;
      tp.alpha = alpha; tp.beta = beta; tp.add_identity = add_id; tp.read_c = read_c;
      tp.n_extra = extra.count;
      bool vec = tma_ok(p.d, p.ldd) && (!read_c || tma_ok(p.c, p.ldc)) && p.n % (16 / (int)sizeof(T)) == 0;
      for (int x = 0; x < extra.count; ++x) {
        tp.extra_d[x] = static_cast<T*>(extra.ptr[x]);
        vec = vec && reinterpret_cast<uintptr_t>(extra.ptr[x]) % 16 == 0;
      }
      tp.vector_epilogue = vec;
      tp.tiles_m = (p.m + kTileM - 1) / kTileM; tp.tiles_n = (p.n + kTileN - 1) / kTileN;
      tp.status = dev->status;
      tp.whole_tiles = plan.whole_tiles;
      tp.slices = plan.pieces;
      const int k_tiles = (p.k + TK - 1) / TK;
      tp.k_tiles_per_slice = (k_tiles + plan.pieces - 1) / plan.pieces;
      tp.partial = partial; tp.tickets = tickets;
      const long long all_tiles = static_cast<long long>(tp.tiles_m) * tp.tiles_n;
      const long long work = plan.whole_tiles + (all_tiles - plan.whole_tiles) * plan.pieces;
      const int grid = static_cast<int>(work < dev->sms ? work : dev->sms);
#define X(ADD, MUL)                                                                                       \
      if (!launched && desc.add_op == ADD && desc.mul_op == MUL) {                                        \
        if constexpr (tma_instantiated<ADD, MUL, T>()) {                                                  \
          err = launch_tma<ADD, MUL, T>(p.a_kcontig, p.b_kcontig, map_a, map_b, tp, grid, stream);        \
          launched = true;                                                                                \
        }                                                                                                 \
      }
      CUASR_FLOAT_RINGS(X)
      if constexpr (std::is_integral<T>::value) { CUASR_BIT_RINGS(X) }
#undef X
      if (launched)
        t_last_kernel = slices > 1 ? "tma_splitk" : plan.pieces > 1 ? "tma_balanced" : repacked ? "tma_repacked" : "tma";
    }
  }
  if (!launched) {
    GenericParams<T> gp;
    gp.M = p.m; gp.N = p.n; gp.K = p.k;
    gp.A = static_cast<const T*>(p.a); gp.a_row = p.a_kcontig ? p.lda : 1; gp.a_col = p.a_kcontig ? 1 : p.lda;
    gp.B = static_cast<const T*>(p.b); gp.b_row = p.b_kcontig ? 1 : p.ldb; gp.b_col = p.b_kcontig ? p.ldb : 1;
    gp.C = static_cast<const T*>(p.c); gp.ldc = p.ldc;
    gp.D = static_cast<T*>(p.d); gp.ldd = p.ldd;
    gp.n_extra = extra.count;
    for (int x = 0; x < extra.count; ++x) gp.extra_d[x] = static_cast<T*>(extra.ptr[x]);
    gp.alpha = alpha; gp.beta = beta; gp.add_identity = add_id; gp.read_c = read_c;
    gp.k_per_slice = (p.k + slices - 1) / slices;
    gp.partial = slices > 1 ? partial : nullptr;
#define X(ADD, MUL)                                                   \
    if (!launched && desc.add_op == ADD && desc.mul_op == MUL) {      \
      err = launch_generic<ADD, MUL, T>(gp, slices, stream);          \
      launched = true;                                                \
    }
    CUASR_FLOAT_RINGS(X)
    if constexpr (std::is_integral<T>::value) { CUASR_BIT_RINGS(X) }
#undef X
    if (launched && err == cudaSuccess && slices > 1) {
      g_launches.fetch_add(1);
      bool reduced = false;
#define X(ADD, MUL)                                                   \
      if (!reduced && desc.add_op == ADD && desc.mul_op == MUL) {     \
        err = launch_generic_reduce<ADD, MUL, T>(gp, slices, stream); \
        reduced = true;                                               \
      }
      CUASR_FLOAT_RINGS(X)
      if constexpr (std::is_integral<T>::value) { CUASR_BIT_RINGS(X) }
#undef X
    }
    if (launched) t_last_kernel = slices > 1 ? "generic_splitk" : "generic";
  }
  if (!launched) return CUASR_STATUS_ERROR_NOT_SUPPORTED;
  if (err != cudaSuccess) return CUASR_STATUS_ERROR_INTERNAL;
  g_launches.fetch_add(1);
  return CUASR_STATUS_SUCCESS;
}

int run(const cuasr_b200_desc_t* desc, const cuasr_b200_args_t* args, int slices,
        const ExtraOutputs& extra = ExtraOutputs()) {
  switch (desc->dtype) {
    case CUASR_F32: return run_typed<float>(*desc, *args, slices, extra);
    case CUASR_F64: return run_typed<double>(*desc, *args, slices, extra);
    case CUASR_S32: return run_typed<int32_t>(*desc, *args, slices, extra);
    case CUASR_U32: return run_typed<uint32_t>(*desc, *args, slices, extra);
    default: return CUASR_STATUS_ERROR_INVALID_DATA_TYPE;
  }
}

// ---- one-sided flags between GPUs --------------------------------------------------------------------------
// A producer raises a word in every consumer's memory after the kernel whose peer stores it announces; a consumer
// waits for its own copy of the word on its own stream.  Neither side ever waits for the other to ARRIVE at a
// collective, which is what lets the owner of a panel run ahead of the ranks that only consume it.
constexpr int kMaxFlagTargets = 8;
constexpr int kMaxFlagWords = 64;
struct FlagTargets {
  unsigned int* ptr[kMaxFlagTargets];
};

// Stream order puts this kernel after the stores it announces; the fence makes them visible system-wide first.
// atomicMax keeps the word monotonic when several producers raise it in turn.
__global__ void flag_raise_kernel(FlagTargets targets, int count, unsigned int value) {
  const int i = threadIdx.x;
  if (i < count) {
    __threadfence_system();
    atomicMax_system(targets.ptr[i], value);
  }
}

// Thread i waits until word i is at least `value`.  The wait is bounded twice (wall time and iterations); when it
// runs out the kernel records kDeviceTimeoutPeerFlag in the status word and returns, so the stream keeps moving and
// the host finds the code with cuasr_b200_device_status.
__global__ void flag_wait_kernel(const unsigned int* words, int count, unsigned int value, unsigned long long limit_ns,
                                 unsigned int* status) {
  const int i = threadIdx.x;
  if (i >= count) return;
  unsigned long long start, now;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(start));
  for (unsigned int spin = 0; spin < (1u << 26); ++spin) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(words + i) : "memory");
    if (v >= value) return;
    __nanosleep(256);
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (now - start > limit_ns) break;
  }
  report_device_error(status, kDeviceTimeoutPeerFlag);
}

// ---- built-in scratch for cuasr_b200_srgemm_splitk_static --------------------------------------------
// The array is device memory that belongs to the loaded module.  Its name is only a host-side handle: a
// kernel must be given the address cudaGetSymbolAddress returns for the CURRENT device, never the name.
static __device__ __align__(256) unsigned char g_static_scratch[CUASR_B200_STATIC_SCRATCH_BYTES];
void* g_static_scratch_ptr[kMaxDevices] = {};
std::mutex g_static_scratch_mutex;

// Device address of the static scratch on the current device; looked up once per device.
cudaError_t static_scratch_address(void** out) {
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return err;
  if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    err = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_scratch);
    if (err != cudaSuccess) return err;
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return cudaSuccess;
}

}  // namespace
}  // namespace cuasr_b200

using namespace cuasr_b200;

extern "C" {

int cuasr_b200_srgemm_can_implement(const cuasr_b200_desc_t* desc, const cuasr_b200_args_t* args) {
  const int st = validate(desc, args);
  if (st != CUASR_STATUS_SUCCESS) return st;
  // device/srgemm.h:198-200
  if (!desc->split_k_serial && args->split_k_slices > 1) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  return CUASR_STATUS_SUCCESS;
}

size_t cuasr_b200_srgemm_workspace_size(const cuasr_b200_desc_t* desc, const cuasr_b200_args_t* args) {
  if (desc == nullptr || args == nullptr) return 0;
  if (desc->split_k_serial && args->split_k_slices > 1) return splitk_workspace_bytes_refined(*desc, *args);
  return 0;
}

size_t cuasr_b200_srgemm_optional_workspace_size(const cuasr_b200_desc_t* desc, const cuasr_b200_args_t* args) {
  if (desc == nullptr || args == nullptr || validate(desc, args) != CUASR_STATUS_SUCCESS) return 0;
  if (args->split_k_slices > 1) return 0;
  DeviceState* dev = nullptr;
  if (!device_state(&dev)) return 0;
  const size_t repack = repack_plan(*desc, *args, normalise(*desc, *args)).bytes;
  const size_t balance = balance_workspace_bytes(*desc, *args, dev->sms);
  return repack > 0 ? align_up(balance, 256) + repack : balance;
}

int cuasr_b200_srgemm(const cuasr_b200_desc_t* desc, const cuasr_b200_args_t* args) {
  const int st = cuasr_b200_srgemm_can_implement(desc, args);
  if (st != CUASR_STATUS_SUCCESS) return st;
  return run(desc, args, args->split_k_slices);
}

int cuasr_b200_srgemm_push(const cuasr_b200_desc_t* desc, const cuasr_b200_args_t* args, int n_extra,
                           void* const* extra_d) {
  const int st = cuasr_b200_srgemm_can_implement(desc, args);
  if (st != CUASR_STATUS_SUCCESS) return st;
  if (n_extra < 0 || n_extra > kMaxDestinations - 1 || (n_extra > 0 && extra_d == nullptr))
    return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  ExtraOutputs extra;
  extra.count = n_extra;
  const size_t es = desc->dtype == CUASR_F64 ? 8 : 4;
  for (int x = 0; x < n_extra; ++x) {
    if (extra_d[x] == nullptr) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
    if (reinterpret_cast<uintptr_t>(extra_d[x]) % es != 0) return CUASR_STATUS_ERROR_MISALIGNED_OPERAND;
    extra.ptr[x] = extra_d[x];
  }
  return run(desc, args, args->split_k_slices, extra);
}

int cuasr_b200_srgemm_splitk_can_implement(const cuasr_b200_desc_t* desc, const cuasr_b200_args_t* args) {
  return validate(desc, args);
}

size_t cuasr_b200_srgemm_splitk_workspace_size(const cuasr_b200_desc_t* desc, const cuasr_b200_args_t* args) {
  if (desc == nullptr || args == nullptr) return 0;
  return splitk_workspace_bytes_refined(*desc, *args);
}

int cuasr_b200_srgemm_splitk(const cuasr_b200_desc_t* desc, const cuasr_b200_args_t* args) {
  const int st = validate(desc, args);
  if (st != CUASR_STATUS_SUCCESS) return st;
  // device/srgemm_splitk_parallel.h:247-249
  if (args->split_k_slices > 1 && args->workspace == nullptr) return CUASR_STATUS_ERROR_WORKSPACE_NULL;
  return run(desc, args, args->split_k_slices);
}

int cuasr_b200_srgemm_splitk_static(const cuasr_b200_desc_t* desc, const cuasr_b200_args_t* args) {
  const int st = validate(desc, args);
  if (st != CUASR_STATUS_SUCCESS) return st;
  if (splitk_workspace_bytes(*desc, *args) > CUASR_B200_STATIC_SCRATCH_BYTES)
    return CUASR_STATUS_ERROR_STATIC_SCRATCH_TOO_SMALL;
  void* scratch = nullptr;
  if (static_scratch_address(&scratch) != cudaSuccess) return CUASR_STATUS_ERROR_INTERNAL;
  cuasr_b200_args_t with_scratch = *args;
  with_scratch.workspace = scratch;
  with_scratch.workspace_bytes = CUASR_B200_STATIC_SCRATCH_BYTES;
  return run(desc, &with_scratch, with_scratch.split_k_slices);
}

int cuasr_b200_srgemm_path(const cuasr_b200_desc_t* desc, const cuasr_b200_args_t* args, int32_t* parent,
                           int64_t ld_parent, int32_t k_offset) {
  const int st = validate(desc, args);
  if (st != CUASR_STATUS_SUCCESS) return st;
  const bool minimize = desc->add_op == CUASR_OP_MINIMUM, maximize = desc->add_op == CUASR_OP_MAXIMUM;
  if (!(minimize || maximize) || desc->mul_op != CUASR_OP_PLUS) return CUASR_STATUS_ERROR_NOT_SUPPORTED;
  if (desc->dtype != CUASR_F32 && desc->dtype != CUASR_F64) return CUASR_STATUS_ERROR_INVALID_DATA_TYPE;
  if (args->split_k_slices != 1) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  if (parent == nullptr || reinterpret_cast<uintptr_t>(parent) % 4 != 0) return CUASR_STATUS_ERROR_MISALIGNED_OPERAND;
  const bool row_c = desc->layout_c == CUASR_ROW_MAJOR;
  if (ld_parent < (row_c ? args->n : args->m)) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  auto fill = [&](auto* pp) {
    pp->M = args->m; pp->N = args->n; pp->K = args->k;
    const bool row_a = desc->layout_a == CUASR_ROW_MAJOR, row_b = desc->layout_b == CUASR_ROW_MAJOR;
    pp->a_row = row_a ? args->lda : 1; pp->a_col = row_a ? 1 : args->lda;
    pp->b_row = row_b ? args->ldb : 1; pp->b_col = row_b ? 1 : args->ldb;
    pp->d_row = row_c ? args->ldd : 1; pp->d_col = row_c ? 1 : args->ldd;
    pp->p_row = row_c ? ld_parent : 1; pp->p_col = row_c ? 1 : ld_parent;
    pp->parent = parent; pp->k_offset = k_offset;
  };
  cudaStream_t stream = static_cast<cudaStream_t>(args->stream);
  cudaError_t err;
  // fp32 operands TMA can describe take the pipelined kernel; everything else the any-layout one
  if (desc->dtype == CUASR_F32 && static_cast<long long>(args->m) * args->n >= 64 * 64 && encode_tiled_fn() != nullptr) {
    const Normalised p = normalise(*desc, *args);
    const bool dense = p.lda >= (p.a_kcontig ? p.k : p.m) && p.ldb >= (p.b_kcontig ? p.k : p.n);
    DeviceState* dev = nullptr;
    CUtensorMap map_a, map_b;
    if (dense && tma_describable(p.a, p.lda, 4) && tma_describable(p.b, p.ldb, 4) && device_state(&dev) &&
        make_operand_map<float>(&map_a, static_cast<const float*>(p.a), p.lda, p.m, p.k, p.a_kcontig, true) &&
        make_operand_map<float>(&map_b, static_cast<const float*>(p.b), p.ldb, p.n, p.k, p.b_kcontig, true)) {
      PathTmaParams tp;
      tp.M = p.m; tp.N = p.n; tp.K = p.k;
      // the normalised problem has a row-major D: element (m, n) at D[m * ldd + n], whatever the caller's layout
      tp.dist = static_cast<float*>(args->D); tp.d_row = args->ldd; tp.d_col = 1;
      tp.parent = parent; tp.p_row = ld_parent; tp.p_col = 1;
      tp.k_offset = k_offset;
      tp.tiles_m = (p.m + kTileM - 1) / kTileM; tp.tiles_n = (p.n + kTileN - 1) / kTileN;
      tp.status = dev->status;
      const long long tiles = static_cast<long long>(tp.tiles_m) * tp.tiles_n;
      const int grid = static_cast<int>(tiles < dev->sms ? tiles : dev->sms);
      if (launch_path_tma(maximize, p.a_kcontig, p.b_kcontig, map_a, map_b, tp, grid, stream) != cudaSuccess)
        return CUASR_STATUS_ERROR_INTERNAL;
      g_launches.fetch_add(1);
      t_last_kernel = "path_tma";
      return CUASR_STATUS_SUCCESS;
    }
  }
  if (desc->dtype == CUASR_F32) {
    PathParams<float> pp;
    fill(&pp);
    pp.A = static_cast<const float*>(args->A); pp.B = static_cast<const float*>(args->B);
    pp.dist = static_cast<float*>(args->D);
    err = launch_path<float>(pp, maximize, stream);
  } else {
    PathParams<double> pp;
    fill(&pp);
    pp.A = static_cast<const double*>(args->A); pp.B = static_cast<const double*>(args->B);
    pp.dist = static_cast<double*>(args->D);
    err = launch_path<double>(pp, maximize, stream);
  }
  if (err != cudaSuccess) return CUASR_STATUS_ERROR_INTERNAL;
  g_launches.fetch_add(1);
  t_last_kernel = "path";
  return CUASR_STATUS_SUCCESS;
}

int cuasr_b200_pack_k_contiguous(int32_t dtype, const void* src, int64_t ld_src, int32_t src_k_contiguous, int32_t rows,
                                 int32_t k, void* dst, int64_t ld_dst, void* stream) {
  if (dtype != CUASR_F32 && dtype != CUASR_F64 && dtype != CUASR_S32 && dtype != CUASR_U32)
    return CUASR_STATUS_ERROR_INVALID_DATA_TYPE;
  if (src == nullptr || dst == nullptr || rows <= 0 || k <= 0 || ld_dst < k) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  if (ld_src < (src_k_contiguous ? k : rows)) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  const size_t es = dtype == CUASR_F64 ? 8 : 4;
  if (reinterpret_cast<uintptr_t>(src) % es != 0 || reinterpret_cast<uintptr_t>(dst) % es != 0)
    return CUASR_STATUS_ERROR_MISALIGNED_OPERAND;
  if (launch_repack(src, ld_src, src_k_contiguous != 0, rows, k, k, 0ull, dst, ld_dst, es,
                    static_cast<cudaStream_t>(stream)) != cudaSuccess)
    return CUASR_STATUS_ERROR_INTERNAL;
  g_launches.fetch_add(1);
  t_last_kernel = "pack";
  return CUASR_STATUS_SUCCESS;
}

int cuasr_b200_device_status(void* stream) {
  DeviceState* dev = nullptr;
  if (!device_state(&dev)) return -1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  unsigned int host = 0;
  if (cudaMemcpyAsync(&host, dev->status, sizeof(host), cudaMemcpyDeviceToHost, s) != cudaSuccess) return -1;
  if (cudaStreamSynchronize(s) != cudaSuccess) return -1;
  if (host != 0) cudaMemsetAsync(dev->status, 0, sizeof(unsigned int), s);
  return static_cast<int>(host);
}

int cuasr_b200_flag_raise(void* const* words, int count, uint32_t value, void* stream) {
  if (words == nullptr || count < 1 || count > kMaxFlagTargets) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  FlagTargets targets = {};
  for (int i = 0; i < count; ++i) {
    if (words[i] == nullptr) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
    if (reinterpret_cast<uintptr_t>(words[i]) % 4 != 0) return CUASR_STATUS_ERROR_MISALIGNED_OPERAND;
    targets.ptr[i] = static_cast<unsigned int*>(words[i]);
  }
  flag_raise_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(targets, count, value);
  if (cudaGetLastError() != cudaSuccess) return CUASR_STATUS_ERROR_INTERNAL;
  g_launches.fetch_add(1);
  return CUASR_STATUS_SUCCESS;
}

int cuasr_b200_flag_wait(const void* words, int count, uint32_t value, uint32_t timeout_ms, void* stream) {
  if (words == nullptr || count < 1 || count > kMaxFlagWords || timeout_ms == 0 || timeout_ms > 10000)
    return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  if (reinterpret_cast<uintptr_t>(words) % 4 != 0) return CUASR_STATUS_ERROR_MISALIGNED_OPERAND;
  DeviceState* dev = nullptr;
  if (!device_state(&dev)) return CUASR_STATUS_ERROR_INTERNAL;
  flag_wait_kernel<<<1, kMaxFlagWords, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned int*>(words), count, value, 1000000ull * timeout_ms, dev->status);
  if (cudaGetLastError() != cudaSuccess) return CUASR_STATUS_ERROR_INTERNAL;
  g_launches.fetch_add(1);
  return CUASR_STATUS_SUCCESS;
}

const char* cuasr_b200_last_kernel(void) { return t_last_kernel; }

uint64_t cuasr_b200_launch_count(void) { return g_launches.load(); }

const char* cuasr_b200_status_string(int status) {
  switch (status) {
    case CUASR_STATUS_SUCCESS: return "success";
    case CUASR_STATUS_ERROR_MISALIGNED_OPERAND: return "misaligned operand";
    case CUASR_STATUS_ERROR_INVALID_DATA_TYPE: return "invalid data type";
    case CUASR_STATUS_ERROR_INVALID_LAYOUT: return "invalid layout";
    case CUASR_STATUS_ERROR_INVALID_PROBLEM: return "invalid problem";
    case CUASR_STATUS_ERROR_NOT_SUPPORTED: return "not supported";
    case CUASR_STATUS_ERROR_WORKSPACE_NULL: return "workspace null";
    case CUASR_STATUS_ERROR_INTERNAL: return "internal error";
    case CUASR_STATUS_ERROR_STATIC_SCRATCH_TOO_SMALL:
      return "problem needs more scratch than the library's static scratch array holds";
    default: return "unknown status";
  }
}

const char* cuasr_b200_version(void) { return "cuasr_b200 0.1 (sm_100a)"; }

}  // extern "C"
