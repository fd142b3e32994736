/*
 * All-pairs shortest paths on top of the min-plus SRGEMM of cuasr_b200.h, as C entry points.
 *
 * The reference has no such layer: its README.md:338-342 names APSP as what the semiring GEMM and its
 * epilogue (+) are for and leaves the driver to the user.  These calls are that driver: a sequence of
 * cuasr_b200_srgemm launches on the caller's stream, nothing else.  Like the SRGEMM entry points they take
 * DEVICE pointers owned by the caller, allocate nothing, never synchronise with the host and return
 * cutlass::Status numbering (cuasr_status_t).
 *
 * Distances: n x n, element (i, j) = length of the best known path i -> j, stored at D[i + j * ldd].  The
 * closure of a transposed matrix is the transpose of the closure, so a row-major matrix is passed as it is.
 * Absent edges hold +infinity (or any value that stays larger than every path length under addition), the
 * diagonal holds 0.
 */
#ifndef CUASR_B200_APSP_H
#define CUASR_B200_APSP_H

#include "cuasr_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef enum cuasr_apsp_algorithm {
  /* D <- min(D, D (x) D), ceil(log2 n) times (or `iterations` times): 2 n^3 log2 n operations, every launch one
   * large SRGEMM.  Shards over GPUs with one exchange per squaring (cuasr_b200_apsp_shard_squaring). */
  CUASR_APSP_REPEATED_SQUARING = 0,
  /* Three-phase blocked Floyd-Warshall: per block of `block` vertices close the diagonal block, update the
   * column and the row panel through it, then D <- min(D, column panel (x) row panel).  2 n^3 operations. */
  CUASR_APSP_BLOCKED_FLOYD_WARSHALL = 1
} cuasr_apsp_algorithm_t;

typedef struct cuasr_b200_apsp_args {
  int32_t dtype;       /* CUASR_F32 or CUASR_F64 */
  int32_t algorithm;   /* cuasr_apsp_algorithm_t */
  int32_t n;           /* vertices */
  int32_t block;       /* Floyd-Warshall block size, a multiple of 4; 0 = 1024 (the measured optimum at n = 16384) */
  int32_t iterations;  /* repeated squaring: number of squarings; 0 = ceil(log2 n), enough for any graph */
  int32_t reserved;
  void *D;             /* distances, read and overwritten with the closure */
  int64_t ldd;         /* >= n, in elements */
  void *workspace;     /* at least cuasr_b200_apsp_workspace_size bytes, 256-byte aligned */
  size_t workspace_bytes;
  void *stream;        /* cudaStream_t */
  int32_t *parent;     /* optional (NULL = distances only): n x n, column-major like D, see below */
  int64_t ld_parent;   /* >= n, in elements */
} cuasr_b200_apsp_args_t;

/* Bytes of device scratch cuasr_b200_apsp needs: a second n x n matrix for repeated squaring; two panels and two
 * diagonal blocks for Floyd-Warshall; plus, when a device is current, what the SRGEMM launches can use to balance
 * their last wave (cuasr_b200_srgemm_optional_workspace_size).  0 for invalid arguments. */
CUASR_B200_API size_t cuasr_b200_apsp_workspace_size(const cuasr_b200_apsp_args_t *args);

/* Enqueues the whole solve on args->stream and returns.  CUASR_STATUS_ERROR_WORKSPACE_NULL when the workspace is
 * missing or too small, CUASR_STATUS_ERROR_INVALID_PROBLEM for bad sizes or pointers.
 *
 * With `parent` set the solve also says how to walk the shortest paths: every product of the solve is the
 * path-tracking one (cuasr_b200_srgemm_path), and whenever D[i, j] improves to D[i, k] + D[k, j] the vertex k goes
 * to parent[i + j * ld_parent].  Entries that never improve keep what the caller put there (fill the matrix with a
 * value that is no vertex, say -1, before the call).  Afterwards, for every pair with parent k >= 0:
 * D[i, j] == D[i, k] + D[k, j] with k different from i and j, so the path i -> j is the path i -> k followed by the
 * path k -> j, down to pairs without a parent, which are edges of the input.  This needs what shortest paths need
 * anyway: D[i, i] == 0 and positive weights elsewhere (a zero-weight cycle would make the walk circular).
 * The distances are the same bits as without `parent`; the same workspace size serves both. */
CUASR_B200_API int cuasr_b200_apsp(const cuasr_b200_apsp_args_t *args);

/* One squaring of a solve whose columns are sharded over GPUs: this rank owns columns [col0, col0 + cols) and
 * computes  D_next[:, own] = min(D_cur[:, own], D_cur (x) D_cur[:, own])  from its full local copy D_cur, storing
 * the block into its own D_next and, from the same epilogue, into the D_next of up to 7 peers (addresses this
 * device can write: peer access or symmetric memory).  After every rank's launch and a barrier that orders them
 * (for example a one-word NCCL all-reduce on the same streams) each D_next holds the complete next iterate and
 * the roles of D_cur and D_next swap.  The workspace is optional (load balance only) and may be NULL. */
typedef struct cuasr_b200_apsp_shard_args {
  int32_t dtype;
  int32_t n;
  int32_t col0, cols;
  const void *D_cur;  int64_t ld_cur;
  void *D_next;       int64_t ld_next;   /* same leading dimension on every rank */
  int32_t n_peers;    int32_t reserved;
  void *const *peer_next;                /* n_peers base addresses of the other ranks' D_next */
  void *workspace;    size_t workspace_bytes;
  void *stream;
} cuasr_b200_apsp_shard_args_t;

CUASR_B200_API int cuasr_b200_apsp_shard_squaring(const cuasr_b200_apsp_shard_args_t *args);

/* The whole sharded solve on the GPUs of one machine, from one host process: one host thread per GPU, plain peer
 * access between the GPUs (no other library), the push epilogue of the SRGEMM as the only exchange, and a barrier of
 * the host threads between steps (each waits for its own GPU's part first; the barrier also makes the threads agree
 * on the status, so a failure on one GPU stops all of them at the same step).  Every tensor map a kernel reads
 * through describes memory of the GPU that runs it; only plain stores cross NVLink.
 *
 * The caller owns all memory.  n_devices is 1..8, `devices` their CUDA ordinals; per GPU g, in that order:
 *   streams[g]         a stream of device devices[g], or NULL for its default stream;
 *   workspace[g]       device scratch of workspace_bytes.
 * CUASR_APSP_REPEATED_SQUARING (n divisible by n_devices): GPU g owns the contiguous columns
 *   [g n / G, (g + 1) n / G) (cuasr_b200_apsp_multi_partition).  buf0[g] and buf1[g] are two n x n matrices
 *   (leading dimension ldd) on GPU g; before the call buf0[g] holds the whole distance matrix on EVERY GPU.  Each
 *   squaring is one cuasr_b200_apsp_shard_squaring per GPU, which stores the GPU's block into every GPU's next
 *   iterate.  On return every GPU holds the complete closure in buf0[g] or buf1[g]; *result_buffer says which.
 *   The workspace is optional here (load balance; may be NULL).
 * CUASR_APSP_BLOCKED_FLOYD_WARSHALL (n divisible by n_devices x block): the column blocks of `block` vertices are
 *   dealt out cyclically, GPU g owns blocks g, g + G, g + 2 G, ... and buf0[g] holds exactly those columns, one
 *   block after the other, as an n x (n / G) matrix with leading dimension ldd >= n; buf1 is not used.  Per block
 *   the owner closes the diagonal block, computes the column panel and stores it into every GPU's panel buffer
 *   (one step ahead: the owner of the next block does this before the bulk of its own update, so the panel is
 *   waiting when the others get there); every GPU updates its piece of the row panel and its own columns in
 *   place.  The closure ends up in buf0 (*result_buffer = 0), distributed as it came.  The workspace is REQUIRED:
 *   cuasr_b200_apsp_multi_workspace_size bytes per GPU, 256-byte aligned.
 * The call blocks the calling host thread until the solve is done; peer access between the GPUs is switched on by
 * it and left on.  Status: CUASR_STATUS_ERROR_NOT_SUPPORTED when a
 * GPU cannot reach a peer's memory, otherwise the first error any GPU met; `device_status` (n_devices entries, may
 * be NULL) receives each GPU's cuasr_b200_device_status after the solve. */
typedef struct cuasr_b200_apsp_multi_args {
  int32_t dtype;            /* CUASR_F32 or CUASR_F64 */
  int32_t algorithm;        /* cuasr_apsp_algorithm_t */
  int32_t n;
  int32_t block;            /* Floyd-Warshall block size, a multiple of 4; 0 = 512 */
  int32_t iterations;       /* repeated squaring: squarings; 0 = ceil(log2 n) */
  int32_t n_devices;
  const int32_t *devices;   /* CUDA device ordinals */
  void *const *buf0;
  void *const *buf1;        /* repeated squaring only */
  int64_t ldd;
  void *const *workspace;   /* n_devices entries (repeated squaring: NULL, or entries that may be NULL) */
  size_t workspace_bytes;
  void *const *streams;     /* NULL, or n_devices entries */
  int32_t *result_buffer;   /* out */
  int32_t *device_status;   /* out, may be NULL */
} cuasr_b200_apsp_multi_args_t;

CUASR_B200_API int cuasr_b200_apsp_multi(const cuasr_b200_apsp_multi_args_t *args);

/* Bytes of per-GPU scratch cuasr_b200_apsp_multi needs (0 for repeated squaring, whose workspace is optional, and
 * for invalid arguments): three column panels, one row-panel piece and two diagonal blocks for Floyd-Warshall, plus,
 * when a device is current, what the SRGEMM launches can use to balance their last wave (that part is optional: a
 * smaller workspace that still holds the panels and blocks is accepted). */
CUASR_B200_API size_t cuasr_b200_apsp_multi_workspace_size(const cuasr_b200_apsp_multi_args_t *args);

/* How the columns are dealt out by the repeated-squaring form of cuasr_b200_apsp_multi: first column and number of
 * columns of GPU `g` of `n_devices`.  Returns 0, or CUASR_STATUS_ERROR_INVALID_PROBLEM when n does not divide or an
 * index is out of range. */
CUASR_B200_API int cuasr_b200_apsp_multi_partition(int32_t n, int32_t n_devices, int32_t g, int32_t *col0, int32_t *cols);

/* One-sided ordering between GPUs, for solves in which one rank produces what the others consume (the column
 * panels of the sharded Floyd-Warshall solve).  A barrier makes the producer wait for the slowest consumer to
 * arrive; with these two calls the producer only announces, and each consumer waits for the announcement alone.
 *
 * cuasr_b200_flag_raise: after everything already enqueued on `stream` (in particular a cuasr_b200_srgemm_push
 * whose peer stores it announces), raise each of `count` (at most 8) 32-bit words to at least `value`.  The
 * words are device addresses this GPU can write: its own memory or peers'.  Values only grow.
 *
 * cuasr_b200_flag_wait: hold `stream` until each of `count` (at most 64) consecutive words of THIS GPU's memory
 * is at least `value`.  The wait gives up after `timeout_ms` (1..10000): the kernel then records code 3 in the
 * device status word (cuasr_b200_device_status) and lets the stream continue.  The word must be raised by another
 * GPU or by an earlier operation of the same stream; never wait on one stream of a GPU for a kernel that has to
 * run on another stream of the same GPU. */
CUASR_B200_API int cuasr_b200_flag_raise(void *const *words, int count, uint32_t value, void *stream);
CUASR_B200_API int cuasr_b200_flag_wait(const void *words, int count, uint32_t value, uint32_t timeout_ms, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* CUASR_B200_APSP_H */
