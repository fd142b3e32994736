// All-pairs shortest paths as sequences of min-plus SRGEMM launches (include/cuasr_b200_apsp.h).
//
// Host code only: every product goes through the public entry points of this library, so the kernels, their
// validation and their load balancing are the ones every other caller gets.  The reference has no counterpart
// (README.md:338-342 motivates APSP and stops there).
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <limits>
#include <mutex>
#include <thread>
#include <vector>

#include "../../include/cuasr_b200_apsp.h"

namespace {

constexpr int kDefaultBlock = 1024;

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
size_t elem_size(int dtype) { return dtype == CUASR_F64 ? 8 : 4; }

int ceil_log2(int v) {
  int r = 0;
  while ((1LL << r) < v) ++r;
  return r;
}

cuasr_b200_scalar_t scalar(int dtype, double v) {
  cuasr_b200_scalar_t s;
  std::memset(&s, 0, sizeof(s));
  if (dtype == CUASR_F64) {
    std::memcpy(s.bytes, &v, sizeof(double));
  } else {
    const float f = static_cast<float>(v);
    std::memcpy(s.bytes, &f, sizeof(float));
  }
  return s;
}

cuasr_b200_desc_t minplus_desc(int dtype) {
  cuasr_b200_desc_t d;
  std::memset(&d, 0, sizeof(d));
  d.add_op = CUASR_OP_MINIMUM;
  d.mul_op = CUASR_OP_PLUS;
  d.dtype = dtype;
  d.layout_a = d.layout_b = d.layout_c = CUASR_COLUMN_MAJOR;
  return d;
}

// D = min(C, A (x) B): alpha = beta = 0 (the identity of +), accumulators start at +infinity.
cuasr_b200_args_t minplus_args(int dtype, int m, int n, int k, const void* A, long long lda, const void* B,
                               long long ldb, const void* C, long long ldc, void* D, long long ldd, void* ws,
                               size_t ws_bytes, void* stream) {
  cuasr_b200_args_t a;
  std::memset(&a, 0, sizeof(a));
  a.m = m; a.n = n; a.k = k;
  a.split_k_slices = 1;
  a.A = A; a.lda = lda;
  a.B = B; a.ldb = ldb;
  a.C = C; a.ldc = ldc;
  a.D = D; a.ldd = ldd;
  a.alpha = a.beta = a.mul_identity = scalar(dtype, 0.0);
  a.add_identity = scalar(dtype, std::numeric_limits<double>::infinity());
  a.workspace = ws;
  a.workspace_bytes = ws_bytes;
  a.stream = stream;
  return a;
}

bool valid(const cuasr_b200_apsp_args_t* a) {
  if (a == nullptr || (a->dtype != CUASR_F32 && a->dtype != CUASR_F64)) return false;
  if (a->algorithm != CUASR_APSP_REPEATED_SQUARING && a->algorithm != CUASR_APSP_BLOCKED_FLOYD_WARSHALL) return false;
  if (a->n <= 0 || a->iterations < 0 || a->block < 0 || a->block % 4 != 0) return false;
  return true;
}

int block_of(const cuasr_b200_apsp_args_t& a) { return std::min(a.block > 0 ? a.block : kDefaultBlock, (a.n + 3) / 4 * 4); }

// Scratch of the Floyd-Warshall solve, as offsets into the workspace.
struct FwLayout {
  size_t p_col, p_row, diag[2], srgemm, total;
};

// What the SRGEMM launches of a solve can use, at most, as their optional workspace.  0 without a current device.
size_t srgemm_scratch(const cuasr_b200_apsp_args_t& a) {
  const cuasr_b200_desc_t desc = minplus_desc(a.dtype);
  // the size query looks at null-ness and alignment of the pointers only and never dereferences them
  const void* any = reinterpret_cast<const void*>(static_cast<uintptr_t>(256));
  auto need = [&](int m, int n, int k, long long lda, long long ldb, long long ldc) {
    cuasr_b200_args_t s = minplus_args(a.dtype, m, n, k, any, lda, any, ldb, any, ldc, const_cast<void*>(any), ldc,
                                       nullptr, 0, nullptr);
    return cuasr_b200_srgemm_optional_workspace_size(&desc, &s);
  };
  const int n = a.n;
  if (a.algorithm == CUASR_APSP_REPEATED_SQUARING) return need(n, n, n, n, n, n);
  const int b = block_of(a);
  return std::max(std::max(need(b, b, b, b, b, b), need(n, b, b, n, b, n)),
                  std::max(need(b, n, b, b, n, b), need(n, n, b, n, b, n)));
}

FwLayout fw_layout(const cuasr_b200_apsp_args_t& a) {
  const size_t es = elem_size(a.dtype), n = a.n, b = block_of(a);
  FwLayout l;
  size_t off = 0;
  l.p_col = off;   off = align_up(off + n * b * es, 256);
  l.p_row = off;   off = align_up(off + b * n * es, 256);
  l.diag[0] = off; off = align_up(off + b * b * es, 256);
  l.diag[1] = off; off = align_up(off + b * b * es, 256);
  l.srgemm = off;
  l.total = off + srgemm_scratch(a);
  return l;
}

// The path-tracking product of the solves with predecessors: dist <- min(dist, A (x) B) in place, the k of every
// improvement (plus k_offset) to `parent`.
int path_product(const cuasr_b200_apsp_args_t& a, int m, int nn, int k, const void* A, long long lda, const void* B,
                 long long ldb, void* dist, long long ldd, int32_t* parent, int k_offset) {
  const cuasr_b200_desc_t desc = minplus_desc(a.dtype);
  cuasr_b200_args_t s = minplus_args(a.dtype, m, nn, k, A, lda, B, ldb, dist, ldd, dist, ldd, nullptr, 0, a.stream);
  return cuasr_b200_srgemm_path(&desc, &s, parent, a.ld_parent, k_offset);
}

cudaError_t copy_block(const cuasr_b200_apsp_args_t& a, void* dst, size_t ld_dst, const void* src, size_t ld_src,
                       size_t rows, size_t cols) {
  const size_t es = elem_size(a.dtype);
  return cudaMemcpy2DAsync(dst, ld_dst * es, src, ld_src * es, rows * es, cols, cudaMemcpyDeviceToDevice,
                           static_cast<cudaStream_t>(a.stream));
}

// Repeated squaring with predecessors: D <- min(D, D' (x) D') in place, D' a copy of D taken before each squaring.
int squaring_with_parents(const cuasr_b200_apsp_args_t& a) {
  void* copy = a.workspace;               // n x n, leading dimension n
  const int iterations = a.iterations > 0 ? a.iterations : std::max(1, ceil_log2(a.n));
  for (int it = 0; it < iterations; ++it) {
    if (copy_block(a, copy, a.n, a.D, a.ldd, a.n, a.n) != cudaSuccess) return CUASR_STATUS_ERROR_INTERNAL;
    const int st = path_product(a, a.n, a.n, a.n, copy, a.n, copy, a.n, a.D, a.ldd, a.parent, 0);
    if (st != CUASR_STATUS_SUCCESS) return st;
  }
  return CUASR_STATUS_SUCCESS;
}

// Blocked Floyd-Warshall with predecessors.  Same phases as below, every product the path-tracking one, and every
// finished piece is copied back into D before the next phase reads D: the path-tracking product records a k only
// for a STRICT improvement, so a phase that meets values an earlier phase has already produced (the diagonal block
// inside the panels, the panels inside the full update) records nothing for them, in particular not the trivial
// "improvement" through an end point of the pair itself (D[i, i] == 0).
int floyd_warshall_with_parents(const cuasr_b200_apsp_args_t& a) {
  const size_t es = elem_size(a.dtype);
  const int n = a.n, b = block_of(a);
  const FwLayout l = fw_layout(a);
  char* ws = static_cast<char*>(a.workspace);
  char* D = static_cast<char*>(a.D);
  void* p_col = ws + l.p_col;             // n x bk, leading dimension n
  void* p_row = ws + l.p_row;             // bk x n, leading dimension b
  void* diag[2] = {ws + l.diag[0], ws + l.diag[1]};   // bk x bk, leading dimension b
  for (int k0 = 0; k0 < n; k0 += b) {
    const int bk = std::min(b, n - k0);
    char* dkk = D + (static_cast<size_t>(k0) + static_cast<size_t>(k0) * a.ldd) * es;
    char* col = D + static_cast<size_t>(k0) * a.ldd * es;
    char* row = D + static_cast<size_t>(k0) * es;
    int32_t* parent_kk = a.parent + k0 + static_cast<size_t>(k0) * a.ld_parent;
    int32_t* parent_col = a.parent + static_cast<size_t>(k0) * a.ld_parent;
    int32_t* parent_row = a.parent + k0;
    // phase 1: paths inside the block, by squaring the diagonal block in place against a copy of itself
    for (int it = 0; it < std::max(1, ceil_log2(bk)); ++it) {
      if (copy_block(a, diag[0], b, dkk, a.ldd, bk, bk) != cudaSuccess) return CUASR_STATUS_ERROR_INTERNAL;
      const int st = path_product(a, bk, bk, bk, diag[0], b, diag[0], b, dkk, a.ldd, parent_kk, k0);
      if (st != CUASR_STATUS_SUCCESS) return st;
    }
    if (copy_block(a, diag[0], b, dkk, a.ldd, bk, bk) != cudaSuccess) return CUASR_STATUS_ERROR_INTERNAL;   // the closed block
    // phase 2: both panels through the closed block, in place against copies of themselves
    if (copy_block(a, p_col, n, col, a.ldd, n, bk) != cudaSuccess) return CUASR_STATUS_ERROR_INTERNAL;
    int st = path_product(a, n, bk, bk, p_col, n, diag[0], b, col, a.ldd, parent_col, k0);
    if (st != CUASR_STATUS_SUCCESS) return st;
    if (copy_block(a, p_row, b, row, a.ldd, bk, n) != cudaSuccess) return CUASR_STATUS_ERROR_INTERNAL;
    st = path_product(a, bk, n, bk, diag[0], b, p_row, b, row, a.ldd, parent_row, k0);
    if (st != CUASR_STATUS_SUCCESS) return st;
    // phase 3: everything through the two finished panels, in place (the operands are copies)
    if (copy_block(a, p_col, n, col, a.ldd, n, bk) != cudaSuccess) return CUASR_STATUS_ERROR_INTERNAL;
    if (copy_block(a, p_row, b, row, a.ldd, bk, n) != cudaSuccess) return CUASR_STATUS_ERROR_INTERNAL;
    st = path_product(a, n, n, bk, p_col, n, p_row, b, D, a.ldd, a.parent, k0);
    if (st != CUASR_STATUS_SUCCESS) return st;
  }
  return CUASR_STATUS_SUCCESS;
}

int squaring(const cuasr_b200_apsp_args_t& a) {
  if (a.parent != nullptr) return squaring_with_parents(a);
  const cuasr_b200_desc_t desc = minplus_desc(a.dtype);
  const size_t es = elem_size(a.dtype), n = a.n;
  const size_t matrix = align_up(n * n * es, 256);
  char* ws = static_cast<char*>(a.workspace);
  void* other = ws;                       // n x n, leading dimension n
  void* scratch = ws + matrix;
  const size_t scratch_bytes = a.workspace_bytes - matrix;
  const int iterations = a.iterations > 0 ? a.iterations : std::max(1, ceil_log2(a.n));
  void* cur = a.D;
  long long ld_cur = a.ldd;
  void* next = other;
  long long ld_next = a.n;
  for (int it = 0; it < iterations; ++it) {
    cuasr_b200_args_t s = minplus_args(a.dtype, a.n, a.n, a.n, cur, ld_cur, cur, ld_cur, cur, ld_cur, next, ld_next,
                                       scratch_bytes ? scratch : nullptr, scratch_bytes, a.stream);
    const int st = cuasr_b200_srgemm(&desc, &s);
    if (st != CUASR_STATUS_SUCCESS) return st;
    std::swap(cur, next);
    std::swap(ld_cur, ld_next);
  }
  if (cur != a.D) {
    const cudaError_t err = cudaMemcpy2DAsync(a.D, a.ldd * es, cur, n * es, n * es, n, cudaMemcpyDeviceToDevice,
                                              static_cast<cudaStream_t>(a.stream));
    if (err != cudaSuccess) return CUASR_STATUS_ERROR_INTERNAL;
  }
  return CUASR_STATUS_SUCCESS;
}

int floyd_warshall(const cuasr_b200_apsp_args_t& a) {
  if (a.parent != nullptr) return floyd_warshall_with_parents(a);
  const cuasr_b200_desc_t desc = minplus_desc(a.dtype);
  const size_t es = elem_size(a.dtype);
  const int n = a.n, b = block_of(a);
  const FwLayout l = fw_layout(a);
  char* ws = static_cast<char*>(a.workspace);
  char* D = static_cast<char*>(a.D);
  void* p_col = ws + l.p_col;             // n x bk, leading dimension n
  void* p_row = ws + l.p_row;             // bk x n, leading dimension b
  void* diag[2] = {ws + l.diag[0], ws + l.diag[1]};   // bk x bk, leading dimension b
  void* scratch = a.workspace_bytes > l.srgemm ? ws + l.srgemm : nullptr;
  const size_t scratch_bytes = a.workspace_bytes - l.srgemm;
  cudaStream_t stream = static_cast<cudaStream_t>(a.stream);
  auto product = [&](int m, int nn, int k, const void* A, long long lda, const void* B, long long ldb, const void* C,
                     long long ldc, void* out, long long ldo) {
    cuasr_b200_args_t s = minplus_args(a.dtype, m, nn, k, A, lda, B, ldb, C, ldc, out, ldo, scratch, scratch_bytes,
                                       a.stream);
    return cuasr_b200_srgemm(&desc, &s);
  };
  for (int k0 = 0; k0 < n; k0 += b) {
    const int bk = std::min(b, n - k0);
    // phase 1: paths inside the block, by squaring a private copy of the diagonal block
    const char* dkk = D + (static_cast<size_t>(k0) + static_cast<size_t>(k0) * a.ldd) * es;
    if (cudaMemcpy2DAsync(diag[0], b * es, dkk, a.ldd * es, bk * es, bk, cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
      return CUASR_STATUS_ERROR_INTERNAL;
    int cur = 0;
    for (int it = 0; it < std::max(1, ceil_log2(bk)); ++it, cur = 1 - cur) {
      const int st = product(bk, bk, bk, diag[cur], b, diag[cur], b, diag[cur], b, diag[1 - cur], b);
      if (st != CUASR_STATUS_SUCCESS) return st;
    }
    const void* star = diag[cur];
    // phase 2: the column panel D[:, K] and the row panel D[K, :] through the closed block, out of place
    const char* col = D + static_cast<size_t>(k0) * a.ldd * es;
    const char* row = D + static_cast<size_t>(k0) * es;
    int st = product(n, bk, bk, col, a.ldd, star, b, col, a.ldd, p_col, n);
    if (st != CUASR_STATUS_SUCCESS) return st;
    st = product(bk, n, bk, star, b, row, a.ldd, row, a.ldd, p_row, b);
    if (st != CUASR_STATUS_SUCCESS) return st;
    // phase 3: everything through the two panels, in place (the operands are copies)
    st = product(n, n, bk, p_col, n, p_row, b, D, a.ldd, D, a.ldd);
    if (st != CUASR_STATUS_SUCCESS) return st;
  }
  return CUASR_STATUS_SUCCESS;
}

}  // namespace

extern "C" {

size_t cuasr_b200_apsp_workspace_size(const cuasr_b200_apsp_args_t* args) {
  if (!valid(args)) return 0;
  if (args->algorithm == CUASR_APSP_REPEATED_SQUARING)
    return align_up(static_cast<size_t>(args->n) * args->n * elem_size(args->dtype), 256) + srgemm_scratch(*args);
  return fw_layout(*args).total;
}

int cuasr_b200_apsp(const cuasr_b200_apsp_args_t* args) {
  if (!valid(args) || args->D == nullptr || args->ldd < args->n) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  if (reinterpret_cast<uintptr_t>(args->D) % elem_size(args->dtype) != 0) return CUASR_STATUS_ERROR_MISALIGNED_OPERAND;
  // the part of the workspace the solve cannot do without; the SRGEMM scratch behind it is used when it is there
  const size_t required = args->algorithm == CUASR_APSP_REPEATED_SQUARING
                              ? align_up(static_cast<size_t>(args->n) * args->n * elem_size(args->dtype), 256)
                              : fw_layout(*args).srgemm;
  if (args->workspace == nullptr || args->workspace_bytes < required) return CUASR_STATUS_ERROR_WORKSPACE_NULL;
  if (reinterpret_cast<uintptr_t>(args->workspace) % 256 != 0) return CUASR_STATUS_ERROR_MISALIGNED_OPERAND;
  if (args->parent != nullptr) {
    if (args->ld_parent < args->n) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
    if (reinterpret_cast<uintptr_t>(args->parent) % 4 != 0) return CUASR_STATUS_ERROR_MISALIGNED_OPERAND;
  }
  return args->algorithm == CUASR_APSP_REPEATED_SQUARING ? squaring(*args) : floyd_warshall(*args);
}

int cuasr_b200_apsp_shard_squaring(const cuasr_b200_apsp_shard_args_t* a) {
  if (a == nullptr || (a->dtype != CUASR_F32 && a->dtype != CUASR_F64)) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  if (a->n <= 0 || a->cols <= 0 || a->col0 < 0 || static_cast<long long>(a->col0) + a->cols > a->n)
    return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  if (a->D_cur == nullptr || a->D_next == nullptr || a->ld_cur < a->n || a->ld_next < a->n)
    return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  if (a->n_peers < 0 || a->n_peers > 7 || (a->n_peers > 0 && a->peer_next == nullptr))
    return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  const cuasr_b200_desc_t desc = minplus_desc(a->dtype);
  const size_t es = elem_size(a->dtype);
  const size_t block_cur = static_cast<size_t>(a->col0) * a->ld_cur * es;
  const size_t block_next = static_cast<size_t>(a->col0) * a->ld_next * es;
  const char* cur = static_cast<const char*>(a->D_cur);
  cuasr_b200_args_t s = minplus_args(a->dtype, a->n, a->cols, a->n, cur, a->ld_cur, cur + block_cur, a->ld_cur,
                                     cur + block_cur, a->ld_cur, static_cast<char*>(a->D_next) + block_next, a->ld_next,
                                     a->workspace, a->workspace ? a->workspace_bytes : 0, a->stream);
  void* peers[7] = {};
  for (int p = 0; p < a->n_peers; ++p) {
    if (a->peer_next[p] == nullptr) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
    peers[p] = static_cast<char*>(a->peer_next[p]) + block_next;
  }
  return cuasr_b200_srgemm_push(&desc, &s, a->n_peers, peers);
}

int cuasr_b200_apsp_multi_partition(int32_t n, int32_t n_devices, int32_t g, int32_t* col0, int32_t* cols) {
  if (n <= 0 || n_devices < 1 || n_devices > 8 || g < 0 || g >= n_devices || n % n_devices != 0 || col0 == nullptr ||
      cols == nullptr)
    return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  *cols = n / n_devices;
  *col0 = g * *cols;
  return CUASR_STATUS_SUCCESS;
}

namespace {
constexpr int kDefaultMultiBlock = 512;
int multi_block(const cuasr_b200_apsp_multi_args_t& a) { return a.block > 0 ? a.block : kDefaultMultiBlock; }
bool multi_valid(const cuasr_b200_apsp_multi_args_t* a) {
  if (a == nullptr || (a->dtype != CUASR_F32 && a->dtype != CUASR_F64)) return false;
  if (a->algorithm != CUASR_APSP_REPEATED_SQUARING && a->algorithm != CUASR_APSP_BLOCKED_FLOYD_WARSHALL) return false;
  if (a->n <= 0 || a->n_devices < 1 || a->n_devices > 8 || a->n % a->n_devices != 0 || a->ldd < a->n) return false;
  if (a->iterations < 0 || a->block < 0 || a->block % 4 != 0) return false;
  if (a->algorithm == CUASR_APSP_BLOCKED_FLOYD_WARSHALL &&
      a->n % (static_cast<long long>(a->n_devices) * multi_block(*a)) != 0)
    return false;
  return true;
}
// Per-GPU scratch of the sharded Floyd-Warshall solve, as offsets into the workspace.
constexpr int kPanelBuffers = 3;
struct MultiFwLayout {
  size_t p_col[kPanelBuffers], p_row, diag[2], srgemm, total;
};
// What the SRGEMM launches of one GPU's share can use, at most, as their optional workspace (they run one after
// the other on one stream, so one region serves all of them).  0 without a current device.
size_t multi_srgemm_scratch(const cuasr_b200_apsp_multi_args_t& a) {
  const cuasr_b200_desc_t desc = minplus_desc(a.dtype);
  const void* any = reinterpret_cast<const void*>(static_cast<uintptr_t>(256));   // never dereferenced by the query
  auto need = [&](int m, int nn, int k, long long lda, long long ldb, long long ldc) {
    cuasr_b200_args_t s = minplus_args(a.dtype, m, nn, k, any, lda, any, ldb, any, ldc, const_cast<void*>(any), ldc,
                                       nullptr, 0, nullptr);
    return cuasr_b200_srgemm_optional_workspace_size(&desc, &s);
  };
  const int n = a.n, b = multi_block(a), cols = n / a.n_devices;
  const long long ld = a.ldd;
  return std::max(std::max(need(b, b, b, b, b, b), need(n, b, b, ld, b, ld)),
                  std::max(need(b, cols, b, n, ld, ld), need(n, cols, b, n, b, ld)));
}
MultiFwLayout multi_fw_layout(const cuasr_b200_apsp_multi_args_t& a) {
  const size_t es = elem_size(a.dtype), n = a.n, b = multi_block(a), cols = n / a.n_devices;
  MultiFwLayout l;
  size_t off = 0;
  for (int i = 0; i < kPanelBuffers; ++i) { l.p_col[i] = off; off = align_up(off + n * b * es, 256); }
  l.p_row = off; off = align_up(off + b * cols * es, 256);
  for (int i = 0; i < 2; ++i) { l.diag[i] = off; off = align_up(off + b * b * es, 256); }
  l.srgemm = off;
  l.total = off + multi_srgemm_scratch(a);
  return l;
}
}  // namespace

size_t cuasr_b200_apsp_multi_workspace_size(const cuasr_b200_apsp_multi_args_t* a) {
  if (!multi_valid(a) || a->algorithm != CUASR_APSP_BLOCKED_FLOYD_WARSHALL) return 0;
  return multi_fw_layout(*a).total;
}

int cuasr_b200_apsp_multi(const cuasr_b200_apsp_multi_args_t* a) {
  if (!multi_valid(a)) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  const bool fw = a->algorithm == CUASR_APSP_BLOCKED_FLOYD_WARSHALL;
  if (a->devices == nullptr || a->buf0 == nullptr || (!fw && a->buf1 == nullptr) || a->result_buffer == nullptr)
    return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  const int G = a->n_devices;
  for (int g = 0; g < G; ++g) {
    if (a->buf0[g] == nullptr || (!fw && a->buf1[g] == nullptr)) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
    for (int h = 0; h < g; ++h)
      if (a->devices[g] == a->devices[h]) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  }
  if (fw) {
    // the part of the workspace the solve cannot do without; the SRGEMM scratch behind it is used when it is there
    if (a->workspace == nullptr || a->workspace_bytes < multi_fw_layout(*a).srgemm) return CUASR_STATUS_ERROR_WORKSPACE_NULL;
    for (int g = 0; g < G; ++g) {
      if (a->workspace[g] == nullptr) return CUASR_STATUS_ERROR_WORKSPACE_NULL;
      if (reinterpret_cast<uintptr_t>(a->workspace[g]) % 256 != 0) return CUASR_STATUS_ERROR_MISALIGNED_OPERAND;
    }
  }
  const int steps = a->iterations > 0 ? a->iterations : std::max(1, ceil_log2(a->n));

  // A reusable barrier of the G host threads that also makes them agree: the thread that completes a round takes
  // a snapshot of the shared status and every thread of that round gets the same snapshot back, so either all of
  // them go on or all of them stop (a thread that looked at the status by itself could see a failure of the NEXT
  // step, leave, and strand the others at the next barrier).
  std::atomic<int> failed{CUASR_STATUS_SUCCESS};
  struct Barrier {
    std::mutex m;
    std::condition_variable cv;
    int waiting = 0, generation = 0, count, agreed = CUASR_STATUS_SUCCESS;
    std::atomic<int>& status;
    Barrier(int c, std::atomic<int>& st) : count(c), status(st) {}
    int arrive_and_wait() {
      std::unique_lock<std::mutex> lock(m);
      const int gen = generation;
      if (++waiting == count) {
        waiting = 0;
        agreed = status.load();
        ++generation;
        cv.notify_all();
        return agreed;
      }
      cv.wait(lock, [&] { return gen != generation; });
      return agreed;
    }
  } barrier(G, failed);
  auto fail = [&](int status) { int expected = CUASR_STATUS_SUCCESS; failed.compare_exchange_strong(expected, status); };

  // one squaring per step: every GPU computes its block of columns and stores it into every GPU's next iterate
  auto squaring_steps = [&](int g, cudaStream_t stream) {
    int32_t col0 = 0, cols = 0;
    cuasr_b200_apsp_multi_partition(a->n, G, g, &col0, &cols);
    for (int s = 0; s < steps; ++s) {
      void* const* cur = (s % 2 == 0) ? a->buf0 : a->buf1;
      void* const* nxt = (s % 2 == 0) ? a->buf1 : a->buf0;
      void* peers[7];
      int np = 0;
      for (int h = 0; h < G; ++h)
        if (h != g) peers[np++] = nxt[h];
      cuasr_b200_apsp_shard_args_t sa;
      std::memset(&sa, 0, sizeof(sa));
      sa.dtype = a->dtype; sa.n = a->n; sa.col0 = col0; sa.cols = cols;
      sa.D_cur = cur[g]; sa.ld_cur = a->ldd;
      sa.D_next = nxt[g]; sa.ld_next = a->ldd;
      sa.n_peers = np; sa.peer_next = peers;
      sa.workspace = a->workspace != nullptr ? a->workspace[g] : nullptr;
      sa.workspace_bytes = sa.workspace != nullptr ? a->workspace_bytes : 0;
      sa.stream = stream;
      const int st = cuasr_b200_apsp_shard_squaring(&sa);
      if (st != CUASR_STATUS_SUCCESS) fail(st);
      // the step is over when every GPU's kernel, and with it every store into every next iterate, is complete
      if (cudaStreamSynchronize(stream) != cudaSuccess) fail(CUASR_STATUS_ERROR_INTERNAL);
      if (barrier.arrive_and_wait() != CUASR_STATUS_SUCCESS) break;   // the same answer on every thread
    }
  };

  // Blocked Floyd-Warshall, one block of vertices per step, with the column panel of the NEXT step computed first:
  // in step kb the owner of block kb + 1 brings that block up to date, closes its diagonal block, computes the
  // column panel and stores it into every GPU's panel buffer (kb + 1) % 3, and only then updates the rest of its
  // columns, so the other GPUs find the panel waiting when they finish step kb.
  // Who waits for what, on the host: before the barrier of step kb every thread waits until its own GPU has
  // finished step kb - 2, and the owner of block kb until its panel has been stored everywhere.  After the barrier,
  // then, panel kb is complete on every GPU, and the buffer the owner of block kb + 1 is about to fill (it last held
  // panel kb - 2, read in step kb - 2) has no reader left.  The GPUs always have a step queued ahead.
  auto floyd_warshall_steps = [&](int g, cudaStream_t stream) {
    const cuasr_b200_desc_t desc = minplus_desc(a->dtype);
    const size_t es = elem_size(a->dtype);
    const int n = a->n, b = multi_block(*a), cols = n / G, blocks = n / b;
    const MultiFwLayout l = multi_fw_layout(*a);
    char* ws = static_cast<char*>(a->workspace[g]);
    char* D = static_cast<char*>(a->buf0[g]);
    void* p_row = ws + l.p_row;                               // b x cols, leading dimension b
    void* diag[2] = {ws + l.diag[0], ws + l.diag[1]};         // b x b
    void* scratch = a->workspace_bytes > l.srgemm ? ws + l.srgemm : nullptr;
    const size_t scratch_bytes = a->workspace_bytes - l.srgemm;
    cudaEvent_t done[kPanelBuffers] = {}, pushed = nullptr;
    bool events = cudaEventCreateWithFlags(&pushed, cudaEventDisableTiming) == cudaSuccess;
    for (int i = 0; i < kPanelBuffers; ++i)
      events = events && cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming) == cudaSuccess;
    if (!events) fail(CUASR_STATUS_ERROR_INTERNAL);
    auto product = [&](int m, int nn, int k, const void* A, long long lda, const void* B, long long ldb, const void* C,
                       long long ldc, void* out, long long ldo, int n_extra, void* const* extra) {
      cuasr_b200_args_t s = minplus_args(a->dtype, m, nn, k, A, lda, B, ldb, C, ldc, out, ldo, scratch, scratch_bytes, stream);
      return n_extra > 0 ? cuasr_b200_srgemm_push(&desc, &s, n_extra, extra) : cuasr_b200_srgemm(&desc, &s);
    };
    // phases 1 and 2 (column part) of block kb, by its owner: the closed diagonal block from a private copy, then
    // P_col = min(D[:, K], D[:, K] (x) D[K, K]*) into every GPU's panel buffer; `pushed` marks the end of it
    auto make_panel = [&](int kb) {
      const int k0 = kb * b;
      char* panel = D + static_cast<size_t>(kb / G) * b * a->ldd * es;      // my columns of block kb
      if (cudaMemcpy2DAsync(diag[0], b * es, panel + static_cast<size_t>(k0) * es, a->ldd * es, b * es, b,
                            cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
        return static_cast<int>(CUASR_STATUS_ERROR_INTERNAL);
      int cur = 0, st = CUASR_STATUS_SUCCESS;
      for (int it = 0; st == CUASR_STATUS_SUCCESS && it < std::max(1, ceil_log2(b)); ++it, cur = 1 - cur)
        st = product(b, b, b, diag[cur], b, diag[cur], b, diag[cur], b, diag[1 - cur], b, 0, nullptr);
      if (st != CUASR_STATUS_SUCCESS) return st;
      void* peers[7];
      int np = 0;
      for (int h = 0; h < G; ++h)
        if (h != g) peers[np++] = static_cast<char*>(a->workspace[h]) + l.p_col[kb % kPanelBuffers];
      st = product(n, b, b, panel, a->ldd, diag[cur], b, panel, a->ldd, ws + l.p_col[kb % kPanelBuffers], n, np, peers);
      if (st == CUASR_STATUS_SUCCESS && cudaEventRecord(pushed, stream) != cudaSuccess) st = CUASR_STATUS_ERROR_INTERNAL;
      return st;
    };
    bool wait_for_push = false;
    if (events && g == 0) {                                   // block 0 has no step before it
      const int st = make_panel(0);
      if (st != CUASR_STATUS_SUCCESS) fail(st);
      wait_for_push = true;
    }
    for (int kb = 0; kb < blocks; ++kb) {    // without events the status is a failure already: everybody leaves at the first barrier
      if (wait_for_push && cudaEventSynchronize(pushed) != cudaSuccess) fail(CUASR_STATUS_ERROR_INTERNAL);
      wait_for_push = false;
      if (kb >= 2 && cudaEventSynchronize(done[(kb - 2) % kPanelBuffers]) != cudaSuccess) fail(CUASR_STATUS_ERROR_INTERNAL);
      if (barrier.arrive_and_wait() != CUASR_STATUS_SUCCESS) break;
      const int k0 = kb * b;
      const char* p_col = ws + l.p_col[kb % kPanelBuffers];   // n x b, leading dimension n; rows K of it = D[K, K]*
      // phase 2, my piece of the row panel: P_row = min(D[K, mine], D[K, K]* (x) D[K, mine])
      const char* rows = D + static_cast<size_t>(k0) * es;
      int st = product(b, cols, b, p_col + static_cast<size_t>(k0) * es, n, rows, a->ldd, rows, a->ldd, p_row, b, 0, nullptr);
      // phase 3: my columns [c0, c1) through the two panels, in place (the operands are copies)
      auto update = [&](size_t c0, size_t c1) {
        if (c1 <= c0) return static_cast<int>(CUASR_STATUS_SUCCESS);
        char* part = D + c0 * a->ldd * es;
        return product(n, static_cast<int>(c1 - c0), b, p_col, n, static_cast<char*>(p_row) + c0 * b * es, b, part,
                       a->ldd, part, a->ldd, 0, nullptr);
      };
      if (st == CUASR_STATUS_SUCCESS && kb + 1 < blocks && (kb + 1) % G == g) {
        // the next block is mine: phase 3 on it alone, then its panel goes out before the rest of phase 3
        const size_t lc = static_cast<size_t>((kb + 1) / G) * b;
        st = update(lc, lc + b);
        if (st == CUASR_STATUS_SUCCESS) st = make_panel(kb + 1);
        wait_for_push = true;
        if (st == CUASR_STATUS_SUCCESS) st = update(0, lc);
        if (st == CUASR_STATUS_SUCCESS) st = update(lc + b, cols);
      } else if (st == CUASR_STATUS_SUCCESS) {
        st = update(0, cols);
      }
      if (st == CUASR_STATUS_SUCCESS && cudaEventRecord(done[kb % kPanelBuffers], stream) != cudaSuccess)
        st = CUASR_STATUS_ERROR_INTERNAL;
      if (st != CUASR_STATUS_SUCCESS) fail(st);
    }
    if (cudaStreamSynchronize(stream) != cudaSuccess) fail(CUASR_STATUS_ERROR_INTERNAL);
    if (pushed != nullptr) cudaEventDestroy(pushed);
    for (int i = 0; i < kPanelBuffers; ++i)
      if (done[i] != nullptr) cudaEventDestroy(done[i]);
  };

  auto worker = [&](int g) {
    bool ok = cudaSetDevice(a->devices[g]) == cudaSuccess;
    if (!ok) fail(CUASR_STATUS_ERROR_INTERNAL);
    for (int h = 0; ok && h < G; ++h) {
      if (h == g) continue;
      int can = 0;
      if (cudaDeviceCanAccessPeer(&can, a->devices[g], a->devices[h]) != cudaSuccess || !can) {
        fail(CUASR_STATUS_ERROR_NOT_SUPPORTED);
        ok = false;
        break;
      }
      const cudaError_t e = cudaDeviceEnablePeerAccess(a->devices[h], 0);
      if (e == cudaErrorPeerAccessAlreadyEnabled) (void)cudaGetLastError();
      else if (e != cudaSuccess) { fail(CUASR_STATUS_ERROR_INTERNAL); ok = false; }
    }
    cudaStream_t stream = a->streams != nullptr ? static_cast<cudaStream_t>(a->streams[g]) : nullptr;
    // every GPU has its peers mapped, or somebody failed
    if (barrier.arrive_and_wait() == CUASR_STATUS_SUCCESS) {
      if (fw) floyd_warshall_steps(g, stream);
      else squaring_steps(g, stream);
    }
    if (a->device_status != nullptr) a->device_status[g] = cuasr_b200_device_status(stream);
  };

  std::vector<std::thread> threads;
  threads.reserve(G);
  for (int g = 0; g < G; ++g) threads.emplace_back(worker, g);
  for (auto& t : threads) t.join();
  *a->result_buffer = fw ? 0 : steps % 2;
  return failed.load();
}

}  // extern "C"
