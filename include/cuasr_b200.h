/*
 * C ABI of the B200 (sm_100a) semiring-GEMM library.
 *
 * These entry points are what a binding of the reference's device-level API
 *   cuasr::gemm::device::Srgemm               (include/cuasr/gemm/device/srgemm.h:85-357, :398-567)
 *   cuasr::gemm::device::SrgemmSplitKParallel (include/cuasr/gemm/device/srgemm_splitk_parallel.h:101-378, :424-607)
 * calls: the template parameters of those classes travel in a descriptor (operator codes, element type,
 * layouts), their `Arguments` in an argument block.  All pointers are DEVICE pointers owned by the
 * caller; nothing here allocates, frees or synchronises with the host (the reference keeps only a
 * Params copy: device/srgemm.h:188), and every launch is asynchronous on the given stream.
 * Return values use cutlass::Status numbering (cuasr_status_t), 0 = success.
 *
 * The header-only C++ facade in include/cuasr/ turns `Srgemm<AdditionOp, MultiplicationOp, ...>` objects
 * into calls of these functions.
 */
#ifndef CUASR_B200_H
#define CUASR_B200_H

#include <stddef.h>
#include <stdint.h>

#include "cuasr_b200_types.h"

#if defined(__GNUC__)
#define CUASR_B200_API __attribute__((visibility("default")))
#else
#define CUASR_B200_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* The compile-time half of the reference's interface: template parameters of device::Srgemm
 * (device/srgemm.h:28-84).  Element type is one type for A, B, C, D, accumulator and scalars. */
typedef struct cuasr_b200_desc {
  int32_t add_op;    /* cuasr_op_t: AdditionOp        */
  int32_t mul_op;    /* cuasr_op_t: MultiplicationOp  */
  int32_t dtype;     /* cuasr_dtype_t                 */
  int32_t layout_a;  /* cuasr_layout_t of A (M x K)   */
  int32_t layout_b;  /* cuasr_layout_t of B (K x N)   */
  int32_t layout_c;  /* cuasr_layout_t of C and D (M x N) */
  /* kSplitKSerial of device::Srgemm (device/srgemm.h:83, :198-200): when 0, split_k_slices > 1 is an
   * invalid problem for cuasr_b200_srgemm; when 1, the K range is split and combined inside one launch. */
  int32_t split_k_serial;
  int32_t reserved;
} cuasr_b200_desc_t;

/* One element of the descriptor's dtype, stored in the first sizeof(element) bytes. */
typedef struct cuasr_b200_scalar {
  unsigned char bytes[8];
} cuasr_b200_scalar_t;

/* The run-time half: device::Srgemm::Arguments (device/srgemm.h:139-183) plus the workspace and stream
 * that initialize()/run() take (device/srgemm.h:237, :303).  Leading dimensions are in elements. */
typedef struct cuasr_b200_args {
  int32_t m, n, k;                  /* GemmCoord problem_size */
  int32_t split_k_slices;           /* Arguments::split_k_slices, default 1 */
  const void *A; int64_t lda;       /* ref_A */
  const void *B; int64_t ldb;       /* ref_B */
  const void *C; int64_t ldc;       /* ref_C; may be NULL when the epilogue does not need the source */
  void *D;       int64_t ldd;       /* ref_D; may alias C */
  cuasr_b200_scalar_t alpha;        /* EpilogueOutputOp::Params::alpha (semiring_linear_combination.h:54-100) */
  cuasr_b200_scalar_t beta;         /* EpilogueOutputOp::Params::beta  */
  cuasr_b200_scalar_t add_identity; /* AdditionOp::Identity of the caller's functor: start value of every
                                       accumulator (kernel/srgemm.h:220-221) */
  cuasr_b200_scalar_t mul_identity; /* MultiplicationOp::Identity: used only to decide whether C is read
                                       (semiring_linear_combination.h:118-125) */
  void *workspace;                  /* device scratch of at least cuasr_b200_*_workspace_size bytes, 16-byte
                                       aligned (any cudaMalloc result is), or NULL */
  size_t workspace_bytes;
  void *stream;                     /* cudaStream_t */
} cuasr_b200_args_t;

/* Srgemm::can_implement (device/srgemm.h:196-215): validates sizes, pointers and the split-K setting. */
CUASR_B200_API int cuasr_b200_srgemm_can_implement(const cuasr_b200_desc_t *desc, const cuasr_b200_args_t *args);

/* Srgemm::get_workspace_size (device/srgemm.h:218-234): bytes of device scratch the call needs
 * (0 unless desc->split_k_serial and split_k_slices > 1). */
CUASR_B200_API size_t cuasr_b200_srgemm_workspace_size(const cuasr_b200_desc_t *desc, const cuasr_b200_args_t *args);

/* Srgemm::operator()(args, workspace, stream) = initialize + run (device/srgemm.h:237-336, :344-356):
 * enqueues D = add(mul(alpha, A (x)(+) B), mul(beta, C)) and returns without waiting. */
CUASR_B200_API int cuasr_b200_srgemm(const cuasr_b200_desc_t *desc, const cuasr_b200_args_t *args);

/* Optional.  The reference's unsplit Srgemm needs no workspace (device/srgemm.h:218-234 returns 0) and neither
 * does cuasr_b200_srgemm.  A caller who passes a workspace of at least this many bytes (0 = nothing to gain) to
 * cuasr_b200_srgemm or cuasr_b200_srgemm_push with split_k_slices == 1 gets two things, with identical results:
 *  - load balance: when the tile count is not a multiple of the SM count, the tiles of the last wave are cut along
 *    K, their pieces fill the SMs, and the CTA that finishes a tile last folds the pieces in a fixed order;
 *  - fp32 min/max-plus and min/max-times rings: operands whose contiguous dimension is not K are first copied into
 *    K-contiguous scratch (a bandwidth-bound pre-pass of well under 1 % of the run time), which lets the kernel use
 *    packed fp32x2 adds for both products of a three-input min/max;
 *  - operands the fast kernel cannot read in place are copied into scratch it can read: an operand whose address
 *    or leading dimension is not a multiple of 16 bytes (the reference accepts alignment 1,
 *    device/default_srgemm_configuration.h:88-89; without the workspace such a product runs on the slower generic
 *    kernel), and both operands of an integer min/max ring whose K is not a multiple of the kernel's K step (the
 *    copies are extended along K: A by the additive identity, B by the multiplicative one).
 * The size depends on the operand addresses in `args`.  Needs a current device. */
CUASR_B200_API size_t cuasr_b200_srgemm_optional_workspace_size(const cuasr_b200_desc_t *desc, const cuasr_b200_args_t *args);

/* cuasr_b200_srgemm whose epilogue also stores every element of D to `n_extra` (at most 7) further
 * matrices with the same layout and leading dimension as D.  The extra pointers may be peer-GPU memory that
 * this device can address (peer access enabled): this is the fused "compute + all-gather" step of the sharded
 * repeated-squaring solve, where each rank pushes its block of D into every rank's next-iteration matrix while
 * the tile is still on chip.  New in this library: the reference has no multi-GPU code (README.md:338-342 only
 * motivates it).  Ordering across GPUs is the caller's job (a stream-ordered barrier after the launch). */
CUASR_B200_API int cuasr_b200_srgemm_push(const cuasr_b200_desc_t *desc, const cuasr_b200_args_t *args, int n_extra,
                                          void *const *extra_d);

/* Path-tracking tropical product, in place: D[m, n] <- min (or max) of D[m, n] and A[m, k] + B[k, n] over k, and
 * parent[m, n] <- k_offset + the first k whose product was strictly better than everything before it (parent is
 * left alone where nothing improved).  Device form of the reference's legacy CPU routine cpu_fwgemm_naive
 * (test/regress/include/fwgpu/cpu_srgemm.hpp:20-48), generalised to both layouts, M x N x K and max-plus.
 * desc: add_op MINIMUM or MAXIMUM, mul_op PLUS, dtype F32 or F64.  args: A, B, D (= the distances, read and
 * written; C, alpha, beta, workspace are ignored), split_k_slices = 1.  parent has D's layout, leading dimension
 * ld_parent, 32-bit signed entries.  fp32 operands with 16-byte aligned storage lines run on the TMA pipeline (the
 * index is looked up, and parent written, only for elements that improved; parent is never read there), everything
 * else on an any-layout kernel. */
CUASR_B200_API int cuasr_b200_srgemm_path(const cuasr_b200_desc_t *desc, const cuasr_b200_args_t *args, int32_t *parent,
                                          int64_t ld_parent, int32_t k_offset);

/* SrgemmSplitKParallel::can_implement / get_workspace_size / operator()
 * (device/srgemm_splitk_parallel.h:220-235, :238-279, :333-348).  The reference needs
 * sizeof(element) * M * N * slices bytes of workspace and two launches; this library needs a little more
 * (per-tile arrival counters) and one launch: the CTA that completes a tile last combines the slices
 * in K order and applies the epilogue.  Where the slice count leaves SMs idle (tiles x slices below or badly
 * off a multiple of the SM count) and (+) is exact and order-independent (everything but floating-point plus), K is
 * cut into more pieces than asked, up to 8 x slices (256 x 256 outputs on 148 SMs: 37 pieces per tile whether 16 or
 * 32 slices were asked for); the result does not depend on the cutting.  The workspace size reported with a current
 * device has room for that; a workspace of only the reference's size is accepted and limits the cutting. */
CUASR_B200_API int cuasr_b200_srgemm_splitk_can_implement(const cuasr_b200_desc_t *desc, const cuasr_b200_args_t *args);
CUASR_B200_API size_t cuasr_b200_srgemm_splitk_workspace_size(const cuasr_b200_desc_t *desc, const cuasr_b200_args_t *args);
CUASR_B200_API int cuasr_b200_srgemm_splitk(const cuasr_b200_desc_t *desc, const cuasr_b200_args_t *args);

/* Split-K SRGEMM for callers that cannot allocate device memory.  (No counterpart in the reference, whose
 * SrgemmSplitKParallel always takes a caller-allocated workspace.)
 *
 * Some hosts of this library may not call cudaMalloc at the point where they need a split-K product: code
 * running inside a framework that owns all device memory and hands out none for scratch, plugins invoked
 * under a "no allocation after start-up" rule (real-time or long-running services that must not fragment or
 * fail on memory late), and callers that only hold the operand buffers they were given.  For them this entry
 * point does what cuasr_b200_srgemm_splitk does, but the slice partials and tile counters live in a static
 * device array that is part of the library image, so `workspace` / `workspace_bytes` in `args` are ignored
 * and no cudaMalloc, cudaFree or other allocating call is made.  Inputs and outputs are still the caller's.
 *
 * Limits and rules:
 *  - the array holds CUASR_B200_STATIC_SCRATCH_BYTES bytes; every GPU that loads the library carries it
 *    until the process exits.  A problem that needs more (see cuasr_b200_srgemm_splitk_workspace_size)
 *    is refused with CUASR_STATUS_ERROR_STATIC_SCRATCH_TOO_SMALL and nothing is launched;
 *  - the first call on each device looks up the array's device address (a one-time, synchronous set-up, done
 *    with that device current); make that first call before starting any stream capture;
 *  - every call on a device shares the one array, which keeps whatever the previous call left in it: the
 *    counters are cleared on the stream at the start of each call, the partials are fully overwritten
 *    before they are read; two calls that overlap on the GPU (different streams) race on it -- serialise them.
 *    That holds for a call with split_k_slices == 1 too: it hands the array to the ordinary path as its optional
 *    workspace (balanced last wave, re-packed operands), so it also writes the array;
 *  - the address found by the first call is kept for the life of the process.  Do not destroy the device's
 *    context in between (cudaDeviceReset): the array would be loaded anew at another address and later calls
 *    would write through the old one. */
#define CUASR_B200_STATIC_SCRATCH_BYTES (16u * 1024u * 1024u + 4096u)
CUASR_B200_API int cuasr_b200_srgemm_splitk_static(const cuasr_b200_desc_t *desc, const cuasr_b200_args_t *args);

/* Copies a rows x k operand of 4- or 8-byte elements (dtype: any cuasr_dtype_t) into storage that is contiguous
 * along k: the element with row index r and contraction index kk, found at src[r + kk * ld_src]
 * (src_k_contiguous == 0: a column-major A, a row-major B) or at src[r * ld_src + kk] (src_k_contiguous != 0), goes
 * to dst[r * ld_dst + kk].  Any leading dimensions (ld_dst >= k) and alignments; src and dst must not overlap.
 * New in this library.  The kernels run fastest on operands that are contiguous along k and otherwise make such
 * a copy themselves, per call, when they are given the optional workspace; a caller that multiplies by the same
 * column-major A (row-major B) many times can make the copy once with this call and pass it as a row-major A
 * (column-major B) with leading dimension ld_dst.  The result of the product is the same bits either way.
 * Enqueues on `stream` and returns. */
CUASR_B200_API int cuasr_b200_pack_k_contiguous(int32_t dtype, const void *src, int64_t ld_src, int32_t src_k_contiguous,
                                                int32_t rows, int32_t k, void *dst, int64_t ld_dst, void *stream);

/* Reads (and clears) the device-side status word of the current device after synchronising `stream`:
 * 0 = every kernel of this library ran to completion; otherwise a bounded wait inside a kernel expired
 * (1: tile never arrived, 2: stage never released, 3: peer flag never set).  This call blocks. */
CUASR_B200_API int cuasr_b200_device_status(void *stream);

/* Name of the kernel the last cuasr_b200_srgemm* call on this thread launched ("tma", "generic", ...). */
CUASR_B200_API const char *cuasr_b200_last_kernel(void);

/* Number of kernels this library has launched in this process so far. */
CUASR_B200_API uint64_t cuasr_b200_launch_count(void);

CUASR_B200_API const char *cuasr_b200_status_string(int status);
CUASR_B200_API const char *cuasr_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* CUASR_B200_H */
