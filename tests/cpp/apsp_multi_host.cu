// All-pairs shortest paths on every GPU of the machine from one plain C++ process: cudaMalloc'ed buffers, the C entry
// point cuasr_b200_apsp_multi, nothing else (no Python, no NCCL, no MPI).  The reference motivates the distributed
// case (README.md:338-342) and ships no code for it; this is what a C++ user of the library writes.
//
// Both algorithms are run on min(device count, 4) GPUs that divide the problem (one GPU works too: the same code
// path without peers) and compared, value for value, with a Floyd-Warshall on the host:
//   repeated squaring         every GPU holds the n x n matrix; each squaring, a GPU computes its block of columns
//                             and its epilogue stores it into every GPU's next iterate
//   blocked Floyd-Warshall    every GPU holds n / G columns, dealt out in blocks; the column panel of each step is
//                             stored into every GPU's panel buffer by its owner's epilogue
// Exit code 0 = every check passed.
#include <cstdio>
#include <cstdlib>
#include <limits>
#include <random>
#include <vector>

#include <cuda_runtime.h>

#include "cuasr_b200.h"
#include "cuasr_b200_apsp.h"

#define CHECK_CUDA(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::printf("CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__); std::exit(2); } } while (0)

// column-major n x n weights: w[i + j * n] = weight of the edge i -> j, +inf where there is none, 0 on the diagonal
static std::vector<float> random_graph(int n, unsigned seed) {
  std::mt19937 rng(seed);
  std::uniform_int_distribution<int> weight(1, 100);
  std::uniform_real_distribution<float> coin(0.0f, 1.0f);
  std::vector<float> w(static_cast<size_t>(n) * n, std::numeric_limits<float>::infinity());
  for (int j = 0; j < n; ++j)
    for (int i = 0; i < n; ++i)
      if (i == j) w[i + static_cast<size_t>(j) * n] = 0.0f;
      else if (coin(rng) < 0.03f) w[i + static_cast<size_t>(j) * n] = static_cast<float>(weight(rng));
  return w;
}

static void host_floyd_warshall(std::vector<float>& d, int n) {
  for (int k = 0; k < n; ++k)
    for (int j = 0; j < n; ++j) {
      const float kj = d[k + static_cast<size_t>(j) * n];
      if (kj == std::numeric_limits<float>::infinity()) continue;
      for (int i = 0; i < n; ++i) {
        const float through = d[i + static_cast<size_t>(k) * n] + kj;
        if (through < d[i + static_cast<size_t>(j) * n]) d[i + static_cast<size_t>(j) * n] = through;
      }
    }
}

static int squaring(const std::vector<float>& w, const std::vector<float>& want, int n, int G) {
  std::vector<int32_t> devices(G);
  std::vector<void*> buf0(G), buf1(G);
  const size_t bytes = sizeof(float) * n * n;
  for (int g = 0; g < G; ++g) {
    devices[g] = g;
    CHECK_CUDA(cudaSetDevice(g));
    CHECK_CUDA(cudaMalloc(&buf0[g], bytes));
    CHECK_CUDA(cudaMalloc(&buf1[g], bytes));
    CHECK_CUDA(cudaMemcpy(buf0[g], w.data(), bytes, cudaMemcpyHostToDevice));
  }
  int32_t which = -1;
  std::vector<int32_t> status(G, -1);
  cuasr_b200_apsp_multi_args_t a = {};
  a.dtype = CUASR_F32; a.algorithm = CUASR_APSP_REPEATED_SQUARING; a.n = n; a.n_devices = G;
  a.devices = devices.data(); a.buf0 = buf0.data(); a.buf1 = buf1.data(); a.ldd = n;
  a.result_buffer = &which; a.device_status = status.data();
  const int st = cuasr_b200_apsp_multi(&a);
  int bad = st != CUASR_STATUS_SUCCESS;
  std::vector<float> got(static_cast<size_t>(n) * n);
  for (int g = 0; g < G && !bad; ++g) {
    CHECK_CUDA(cudaSetDevice(g));
    CHECK_CUDA(cudaMemcpy(got.data(), which == 0 ? buf0[g] : buf1[g], bytes, cudaMemcpyDeviceToHost));
    bad += status[g] != 0 || got != want;          // every GPU ends up with the whole closure
  }
  for (int g = 0; g < G; ++g) { CHECK_CUDA(cudaSetDevice(g)); cudaFree(buf0[g]); cudaFree(buf1[g]); }
  std::printf("repeated squaring, n = %d on %d GPU(s): %s (status %d)\n", n, G, bad ? "FAILED" : "ok", st);
  return bad;
}

static int floyd_warshall(const std::vector<float>& w, const std::vector<float>& want, int n, int G, int block) {
  const int cols = n / G, blocks = n / block;
  std::vector<int32_t> devices(G);
  std::vector<void*> buf(G), ws(G);
  cuasr_b200_apsp_multi_args_t a = {};
  a.dtype = CUASR_F32; a.algorithm = CUASR_APSP_BLOCKED_FLOYD_WARSHALL; a.n = n; a.block = block; a.n_devices = G; a.ldd = n;
  const size_t need = cuasr_b200_apsp_multi_workspace_size(&a);
  if (need == 0) { std::printf("Floyd-Warshall: no workspace size for n = %d, %d GPUs, block %d\n", n, G, block); return 1; }
  // GPU g owns the column blocks g, g + G, ...; its buffer holds them one after the other
  std::vector<float> piece(static_cast<size_t>(n) * cols);
  for (int g = 0; g < G; ++g) {
    devices[g] = g;
    int local = 0;
    for (int kb = g; kb < blocks; kb += G, ++local)
      std::copy(w.begin() + static_cast<size_t>(kb) * block * n, w.begin() + static_cast<size_t>(kb + 1) * block * n,
                piece.begin() + static_cast<size_t>(local) * block * n);
    CHECK_CUDA(cudaSetDevice(g));
    CHECK_CUDA(cudaMalloc(&buf[g], sizeof(float) * piece.size()));
    CHECK_CUDA(cudaMalloc(&ws[g], need));
    CHECK_CUDA(cudaMemcpy(buf[g], piece.data(), sizeof(float) * piece.size(), cudaMemcpyHostToDevice));
  }
  int32_t which = -1;
  std::vector<int32_t> status(G, -1);
  a.devices = devices.data(); a.buf0 = buf.data(); a.workspace = ws.data(); a.workspace_bytes = need;
  a.result_buffer = &which; a.device_status = status.data();
  const int st = cuasr_b200_apsp_multi(&a);
  int bad = st != CUASR_STATUS_SUCCESS || which != 0;
  for (int g = 0; g < G && !bad; ++g) {
    CHECK_CUDA(cudaSetDevice(g));
    CHECK_CUDA(cudaMemcpy(piece.data(), buf[g], sizeof(float) * piece.size(), cudaMemcpyDeviceToHost));
    bad += status[g] != 0;
    int local = 0;
    for (int kb = g; kb < blocks; kb += G, ++local)
      bad += !std::equal(piece.begin() + static_cast<size_t>(local) * block * n,
                         piece.begin() + static_cast<size_t>(local + 1) * block * n,
                         want.begin() + static_cast<size_t>(kb) * block * n);
  }
  for (int g = 0; g < G; ++g) { CHECK_CUDA(cudaSetDevice(g)); cudaFree(buf[g]); cudaFree(ws[g]); }
  std::printf("blocked Floyd-Warshall, n = %d, block %d on %d GPU(s): %s (status %d)\n", n, block, G, bad ? "FAILED" : "ok", st);
  return bad;
}

int main() {
  int count = 0;
  CHECK_CUDA(cudaGetDeviceCount(&count));
  const int n = 1024, block = 128;
  int G = count < 4 ? count : 4;
  while (G > 1 && n % (G * block) != 0) --G;
  const std::vector<float> w = random_graph(n, 2024);
  std::vector<float> want = w;
  host_floyd_warshall(want, n);          // integer weights: every sum is exact, so equality is bit for bit
  int failures = 0;
  for (int g = 1; g <= G; g *= 2) {
    failures += squaring(w, want, n, g);
    failures += floyd_warshall(w, want, n, g, block);
  }
  // what is refused before any GPU is touched
  cuasr_b200_apsp_multi_args_t bad_args = {};
  failures += cuasr_b200_apsp_multi(&bad_args) != CUASR_STATUS_ERROR_INVALID_PROBLEM;
  failures += cuasr_b200_apsp_multi(nullptr) != CUASR_STATUS_ERROR_INVALID_PROBLEM;
  std::printf("%s\n", failures == 0 ? "ALL OK" : "FAILURES");
  return failures == 0 ? 0 : 1;
}
