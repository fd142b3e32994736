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

int squaring(const cuasr_b200_apsp_args_t& a) {
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

int cuasr_b200_apsp_multi(const cuasr_b200_apsp_multi_args_t* a) {
  if (a == nullptr || (a->dtype != CUASR_F32 && a->dtype != CUASR_F64)) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  if (a->n <= 0 || a->n_devices < 1 || a->n_devices > 8 || a->n % a->n_devices != 0 || a->ldd < a->n)
    return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  if (a->devices == nullptr || a->buf0 == nullptr || a->buf1 == nullptr || a->result_buffer == nullptr)
    return CUASR_STATUS_ERROR_INVALID_PROBLEM;
  const int G = a->n_devices;
  for (int g = 0; g < G; ++g) {
    if (a->buf0[g] == nullptr || a->buf1[g] == nullptr) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
    for (int h = 0; h < g; ++h)
      if (a->devices[g] == a->devices[h]) return CUASR_STATUS_ERROR_INVALID_PROBLEM;
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
    int32_t col0 = 0, cols = 0;
    cuasr_b200_apsp_multi_partition(a->n, G, g, &col0, &cols);
    // every GPU has its peers mapped, or somebody failed
    const bool run = barrier.arrive_and_wait() == CUASR_STATUS_SUCCESS;
    for (int s = 0; run && s < steps; ++s) {
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
    if (a->device_status != nullptr) a->device_status[g] = cuasr_b200_device_status(stream);
  };

  std::vector<std::thread> threads;
  threads.reserve(G);
  for (int g = 0; g < G; ++g) threads.emplace_back(worker, g);
  for (auto& t : threads) t.join();
  *a->result_buffer = steps % 2;
  return failed.load();
}

}  // extern "C"
