/*
 * km_b200 -- C ABI of the B200 (sm_100a) kernel-matmul hot path.
 *
 * One shared library, plain pointers and sizes, no framework types.  Every entry point is the
 * drop-in for one native op of the reference project Turakar/kernel-matmul (one pybind11
 * module per op there); the reference interface it replaces is cited above each declaration
 * (path within the reference project : lines).
 *
 * Conventions shared by all entry points
 *  - All data pointers are DEVICE pointers on the current CUDA device.  Floats are fp32,
 *    ranges and indices are int32 (the reference's dtypes, native/common/entrypoint.h:3-14).
 *  - Tensors are described by `km_view`: a base pointer plus ELEMENT strides (int64, so that
 *    batch x rows x columns may exceed 2^31 elements; the reference's accessors use int32
 *    offsets, native/common/accessor.cuh:13-24).  Up to KM_MAX_BATCH_DIMS leading batch
 *    dimensions, shared by all arguments of a call and given once in `km_batch`; a batch
 *    stride of 0 broadcasts the same data to every batch (the reference receives such views
 *    from `Tensor.expand`, kernel_matmul/linear_operator.py:170-183).
 *  - Inputs are borrowed and never written.  Outputs and workspaces are caller-allocated; the
 *    library never calls an allocator.  The only device state it holds is the fixed scratch
 *    array of km_bilinear_derivative_static_f32 (compiled into the library, 4 MiB per device)
 *    and the cached device address of that array; every other entry point is stateless.
 *  - Launches are asynchronous on the `stream` argument (a cudaStream_t passed as void*).
 *    The band-construction calls do not synchronise either.
 *  - Return value: KM_OK or an error code; km_last_error() gives a message for the calling
 *    thread.  Nothing traps or aborts.  Arguments are validated before anything is launched.
 *  - Row blocks are KM_BLOCK_SIZE = 128 rows (kernel_matmul/__init__.py:1).  Row block r of
 *    batch b sees columns [start[b,r], end[b,r]) only; every other entry of K is exactly 0.
 *    Bands are clamped to [0, n].
 */
#ifndef KM_B200_H
#define KM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define KM_API __attribute__((visibility("default")))
#else
#define KM_API
#endif

#define KM_BLOCK_SIZE 128
#define KM_MAX_BATCH_DIMS 4
#define KM_MAX_PARAMS 4
/* the product of the batch sizes of a call may not exceed this (refused with KM_ERR_UNSUPPORTED) */
#define KM_MAX_BATCH_COUNT (1LL << 40)

/* status codes */
#define KM_OK 0
#define KM_ERR_INVALID_ARGUMENT 1
#define KM_ERR_UNSUPPORTED 2
#define KM_ERR_WORKSPACE 3
#define KM_ERR_CUDA 4

/* kernel types; parameter order as the reference's callers stack them
 * (native/common/kernel_function.cuh:3-9, kernel_matmul/gpytorch/rbf.py:78-79,
 *  spectral.py:102-103, locally_periodic.py:130-134) */
#define KM_KERNEL_RBF 0              /* theta = [lengthscale, outputscale]                  */
#define KM_KERNEL_SPECTRAL 1         /* theta = [lengthscale, frequency, outputscale]       */
#define KM_KERNEL_LOCALLY_PERIODIC 2 /* theta = [l_rbf, l_periodic, period, outputscale]    */

typedef struct km_batch {
    int32_t ndim;                    /* 0 .. KM_MAX_BATCH_DIMS */
    int64_t size[KM_MAX_BATCH_DIMS]; /* unused entries ignored */
} km_batch;

typedef struct km_view {
    void *data;                              /* device pointer                              */
    int64_t batch_stride[KM_MAX_BATCH_DIMS]; /* element strides of the batch dims (0 = broadcast) */
    int64_t stride[2];                       /* element strides of the trailing dims        */
} km_view;

KM_API const char *km_last_error(void);
KM_API int km_num_params(int kernel_type); /* 2 / 3 / 4, or -1 */
KM_API const char *km_version(void);

/* ---------------------------------------------------------------------------------------
 * out[b, i, :] = sum_{j in band(b, i/128)} kappa(x1[b,i], x2[b,j]; theta[b]) * rhs[b, j, :]
 * Replaces matmul.call(x1, x2, rhs, params, start, end) (native/matmul/matmul.cpp:6-17,
 * native/matmul/matmul.cu:160-203).
 *   x1 (B.., m)  x2 (B.., n)  rhs (B.., n, k)  params (B.., P)  start,end (B.., ceil(m/128)) i32
 *   out (B.., m, k), every element written.
 * Single-stride views (x1, x2, params, start, end) use stride[0].
 * ------------------------------------------------------------------------------------- */
KM_API int km_matmul_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n, int64_t k,
                  const km_view *x1, const km_view *x2, const km_view *rhs,
                  const km_view *params, const km_view *start, const km_view *end,
                  const km_view *out, void *stream);

/* ---------------------------------------------------------------------------------------
 * The same product on the tensor cores (tcgen05.mma, fp32 accumulators in tensor memory): any
 * number of columns, GEMM width 16 / 32 / 64 / 128.  Same arguments and result as km_matmul_f32
 * (to fp32 accuracy: kernel entries and rhs as fp16 hi + lo pairs, 22 significant bits each, rhs
 * columns scaled by a power of two; sine and cosine of a phase difference from per-row and
 * per-column factors around the row block's middle point, per-entry evaluation for row blocks
 * that span too wide a range), plus a workspace of
 * km_matmul_tc_workspace_bytes(...) bytes, 256-byte aligned, contents irrelevant on entry: a
 * pre-pass writes the rhs there as hi / lo fp16 tile images in the tensor core's shared-memory
 * layout, preceded by a 4-byte status word (0 = ok, non-zero = a bounded wait inside the
 * kernel gave up and the output is invalid; read it with km_workspace_status, which
 * synchronises the stream).  A CTA whose wait gave up also writes NaN to its rows of `out`, so a
 * failure shows in everything computed from the result even if nobody reads the status word.
 * Replaces the same reference call as km_matmul_f32.
 * ------------------------------------------------------------------------------------- */
KM_API size_t km_matmul_tc_workspace_bytes(const km_batch *batch, int64_t n, int64_t k,
                                           const km_view *rhs);

KM_API int km_matmul_tc_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n,
                            int64_t k, const km_view *x1, const km_view *x2, const km_view *rhs,
                            const km_view *params, const km_view *start, const km_view *end,
                            const km_view *out, void *workspace, size_t workspace_bytes,
                            void *stream);

/* The tensor-core product restricted to a window of row blocks (as km_matmul_rows_f32 without
 * the batch sum): how a single-kernel product is sharded by rows over GPUs. */
KM_API int km_matmul_tc_rows_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n,
                                 int64_t k, const km_view *x1, const km_view *x2,
                                 const km_view *rhs, const km_view *params, const km_view *start,
                                 const km_view *end, const km_view *out, int64_t row_block_begin,
                                 int64_t row_block_count, void *workspace, size_t workspace_bytes,
                                 void *stream);

KM_API int km_workspace_status(const void *workspace, int32_t *status_out, void *stream);

/* ---------------------------------------------------------------------------------------
 * The same product for a window of row blocks, optionally summed over the batch:
 *   rows [row_block_begin * 128, (row_block_begin + row_block_count) * 128) (clipped to m) only;
 *   out row 0 is row row_block_begin * 128, i.e. out is (B.., rows_in_window, k);
 *   sum_batches != 0: out (rows_in_window, k) = sum_b K_b . rhs_b, accumulated in registers
 *   inside one CTA per row block -- no (B.., m, k) intermediate.  out's batch strides are ignored.
 *   Spectral components that share x1, x2, rhs and the band (batch stride 0) and have one
 *   common lengthscale are summed with the Gaussian envelope evaluated once per entry.
 * row_block_count < 0 means "to the last row block".
 * The window is how the product is sharded by rows over GPUs: every rank holds x, rhs and the
 * bands in full and computes its own row blocks (there is no dependence between row blocks).
 * The batch sum is the product with the reference's SumKernel operator
 * (kernel_matmul/gpytorch/sum.py:16-24: the batched operator summed over its batch dim), which
 * the reference evaluates as B separate products followed by a sum.
 * Up to 1024 spectral components with one common lengthscale and k <= 16 take the tensor-core form
 * of the sum (the sum over the components as a dot product of per-point phase vectors).  Two
 * environment variables, read at every launch, select other arrangements of that kernel; they
 * exist for the tests and for comparison, every setting gives the same result to fp32 accuracy:
 *   KM_SUM_TC_VARIANT = 1 (default) | 2 (rhs contraction on the tensor core too) | 3 (two row
 *   blocks per CTA, k <= 8);  KM_SUM_TC_GROUPS = 2 (default) | 1 (row groups per CTA, variant 1);
 *   KM_SUM_TC_WARP_MMA = 0 (default) | 1 (variant 1, k <= 8: rhs contraction by mma.sync).
 * ------------------------------------------------------------------------------------- */
KM_API int km_matmul_rows_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n,
                              int64_t k, const km_view *x1, const km_view *x2,
                              const km_view *rhs, const km_view *params, const km_view *start,
                              const km_view *end, const km_view *out, int64_t row_block_begin,
                              int64_t row_block_count, int32_t sum_batches, void *stream);

/* ---------------------------------------------------------------------------------------
 * The batch sum of spectral components with the per-point phase vectors written ONCE per
 * operator.  The tensor-core form of the sum evaluates, for every tile of band columns and every
 * row block again, the vectors (cos, sin)(2 pi f_b x_j) of the columns -- values that depend on
 * the operator (x2, the frequencies) and not on rhs.  A solver that applies one operator many
 * times calls km_sum_phases_prepare_f32 once: it writes those vectors for all n columns and the
 * vectors s_b (cos, sin)(2 pi f_b x_i) of all m rows into `workspace` (fp16 hi / lo images in the
 * tensor core's operand layouts; sine and cosine in fp64 with exact range reduction), and
 * km_matmul_rows_phases_f32 -- km_matmul_rows_f32 with sum_batches != 0 and the same arguments --
 * copies them (one bulk copy of 32 KB per tile).  x1, x2 must be shared by all components (batch
 * stride 0); the workspace is valid for these x1, x2, frequencies and output scales; size from
 * km_sum_phases_workspace_bytes (about (m + n) * 8 bytes per component), 256-byte aligned.  Where
 * the tensor-core form does not apply (another kernel type, more than 1024 components, k > 16,
 * different lengthscales) the call computes what km_matmul_rows_f32 computes and ignores the
 * workspace.  No reference counterpart: the reference evaluates every component's kernel entries
 * inside every product (native/matmul/matmul.cu).
 * ------------------------------------------------------------------------------------- */
KM_API size_t km_sum_phases_workspace_bytes(const km_batch *batch, int64_t m, int64_t n);

/* Only the rows [row_begin, row_end) and the columns [col_begin, col_end) (widened to whole tiles of
 * 64) are written -- what a rank of a row-sharded solve reads: its own rows and the columns of
 * their bands; row_end / col_end < 0 mean m / n.  The workspace has the full size either way. */
KM_API int km_sum_phases_prepare_f32(const km_batch *batch, int64_t m, int64_t n, const km_view *x1,
                                     const km_view *x2, const km_view *params, int64_t row_begin,
                                     int64_t row_end, int64_t col_begin, int64_t col_end,
                                     void *workspace, size_t workspace_bytes, void *stream);

KM_API int km_matmul_rows_phases_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n,
                                     int64_t k, const km_view *x1, const km_view *x2,
                                     const km_view *rhs, const km_view *params, const km_view *start,
                                     const km_view *end, const km_view *out, int64_t row_block_begin,
                                     int64_t row_block_count, const void *phases, size_t phases_bytes,
                                     void *stream);


/* ---------------------------------------------------------------------------------------
 * grad[b, q] = d/d theta_q  sum_{i, j in band, c} left[b,i,c] * kappa(x1[b,i], x2[b,j]) * right[b,j,c]
 * Replaces bilinear_derivative.call(x1, x2, left, right, params, start, end)
 * (native/bilinear_derivative/bilinear_derivative.cpp:6-21, .cu:138-183) and, with
 * left = out_grad and right = rhs, matmul_bwd.call(x1, x2, rhs, params, start, end, out_grad)
 * (native/matmul_bwd/matmul_bwd.cpp:6-19, matmul_bwd.cu:182-221): both are this contraction.
 *   left (B.., m, k)  right (B.., n, k)  grad (B.., P) fp32, every element written.
 * workspace: km_grad_workspace_bytes(...) bytes of device memory, 256-byte aligned, contents
 * irrelevant on entry; per-row-block partial sums are written there and reduced in a fixed
 * order, so results are deterministic.
 * ------------------------------------------------------------------------------------- */
KM_API size_t km_grad_workspace_bytes(int kernel_type, const km_batch *batch, int64_t m);

KM_API int km_bilinear_derivative_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n,
                               int64_t k, const km_view *x1, const km_view *x2,
                               const km_view *left, const km_view *right, const km_view *params,
                               const km_view *start, const km_view *end, const km_view *grad,
                               void *workspace, size_t workspace_bytes, void *stream);

KM_API int km_matmul_bwd_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n, int64_t k,
                      const km_view *x1, const km_view *x2, const km_view *rhs,
                      const km_view *params, const km_view *start, const km_view *end,
                      const km_view *out_grad, const km_view *grad, void *workspace,
                      size_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------------------------------
 * The same gradients with the coefficients <left[i, :], right[j, :]> computed on the tensor
 * cores (tcgen05.mma, 3xTF32 = fp32-level accuracy) while the threads evaluate the factors of
 * d kappa / d p: the FP32 pipe no longer pays k FMAs per entry.  Sine and cosine of a phase
 * difference come from per-row and per-column factors, as in km_matmul_tc_f32.  Up to 64 columns
 * per pass; wider operands are processed in column blocks of 64.  Replaces the same reference calls as
 * km_bilinear_derivative_f32 / km_matmul_bwd_f32.
 * workspace: km_grad_tc_workspace_bytes(...) bytes of device memory, 256-byte aligned: a 4-byte
 * status word (0 = ok, non-zero = a bounded wait inside the kernel gave up and the gradient is
 * invalid; read it with km_workspace_status; the gradient of the affected batch is NaN as
 * well), the per-row-block partial sums, and the hi / lo TF32 images of `right` written by a
 * pre-pass.
 * ------------------------------------------------------------------------------------- */
KM_API size_t km_grad_tc_workspace_bytes(const km_batch *batch, int64_t m, int64_t n, int64_t k,
                                         const km_view *right);

KM_API int km_bilinear_derivative_tc_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n,
                                         int64_t k, const km_view *x1, const km_view *x2,
                                         const km_view *left, const km_view *right,
                                         const km_view *params, const km_view *start,
                                         const km_view *end, const km_view *grad, void *workspace,
                                         size_t workspace_bytes, void *stream);

KM_API int km_matmul_bwd_tc_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n,
                                int64_t k, const km_view *x1, const km_view *x2, const km_view *rhs,
                                const km_view *params, const km_view *start, const km_view *end,
                                const km_view *out_grad, const km_view *grad, void *workspace,
                                size_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------------------------------
 * km_bilinear_derivative_f32 for callers that cannot hand over a workspace.  It has no
 * counterpart in the reference (whose ops allocate their temporaries through ATen).
 *
 * Some hosts may not allocate device memory at the point where they need this gradient: an
 * application that has given all of HBM to its own pool has nothing left for cudaMalloc to
 * return, and a latency-critical loop may forbid allocation calls because they can serialise
 * the device.  For them the per-row-block partial sums go to a fixed array compiled into the
 * library instead of a caller buffer.  Same arguments (minus the workspace), same results,
 * bit for bit, as km_bilinear_derivative_f32; pass left = out_grad and right = rhs for the
 * matmul_bwd gradient.  The call itself allocates nothing and frees nothing.
 *
 * Limits and rules
 *  - batch count x ceil(m / 128) must not exceed KM_STATIC_GRAD_UNITS (262144 records, 4 MiB);
 *    larger problems are refused with KM_ERR_UNSUPPORTED and a message, nothing is launched.
 *  - The array exists once per device and is shared by every call on that device.  Nothing in
 *    it has to be cleared (each call writes every record it later reads), but two calls whose
 *    kernels may run at the same time (different streams, different host threads) race on
 *    it: serialise them.  It occupies its 4 MiB on every GPU that loads the library, until
 *    the process exits.
 *  - The first call on each device looks up the array's device address
 *    (cudaGetSymbolAddress, with that device current) and keeps it.  Make that first call
 *    before starting any stream capture on that device.  Device ordinals up to
 *    KM_STATIC_MAX_DEVICES - 1.
 *  - The array is part of the library's device code: the CUDA runtime places it in device
 *    memory when that code is first loaded on a device (with the default lazy loading: at the
 *    first use of any gradient entry point there).  A host that hands all of HBM to its own
 *    pool must make one gradient call on each device BEFORE doing so, or the load fails with
 *    an out-of-memory error.
 *  - The cached address belongs to the device's primary context.  After cudaDeviceReset, or
 *    under another context, it is stale: this entry point supports the primary context of a
 *    process that does not reset its devices.
 * ------------------------------------------------------------------------------------- */
#define KM_STATIC_GRAD_UNITS 262144
#define KM_STATIC_MAX_DEVICES 64

KM_API int km_bilinear_derivative_static_f32(int kernel_type, const km_batch *batch, int64_t m,
                                             int64_t n, int64_t k, const km_view *x1,
                                             const km_view *x2, const km_view *left,
                                             const km_view *right, const km_view *params,
                                             const km_view *start, const km_view *end,
                                             const km_view *grad, void *stream);

/* ---------------------------------------------------------------------------------------
 * Masked dense K: out (B.., m, n), exact zeros outside the band; every element written (no
 * separate zero fill).  Replaces dense.call(x1, x2, params, start, end)
 * (native/dense/dense.cpp:6-17, native/dense/dense.cu:73-98).
 * ------------------------------------------------------------------------------------- */
KM_API int km_dense_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n,
                 const km_view *x1, const km_view *x2, const km_view *params,
                 const km_view *start, const km_view *end, const km_view *out, void *stream);

/* grad[b, q] = d/d theta_q sum_{i, j in band} out_grad[b,i,j] * kappa.  Replaces
 * dense_bwd.call(x1, x2, params, start, end, out_grad) (native/dense_bwd/dense_bwd.cpp:6-17,
 * dense_bwd.cu:86-116).  Workspace as for km_bilinear_derivative_f32. */
KM_API int km_dense_bwd_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n,
                     const km_view *x1, const km_view *x2, const km_view *params,
                     const km_view *start, const km_view *end, const km_view *out_grad,
                     const km_view *grad, void *workspace, size_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------------------------------
 * Gather: out[l] = K[bidx_0[l], .., row[l], col[l]] if the column lies in the band of the
 * row's block, else 0; every element written.  Replaces
 * index.call(x1, x2, params, start, end, batch_indices, row_index, col_index)
 * (native/index/index.cpp:6-24, native/index/index.cu:69-101).
 *   batch_indices: batch->ndim device pointers to int32 arrays of L entries (contiguous);
 *   row, col: int32[L] contiguous; out: float[L].  The index tensors' own leading shape is
 *   flattened by the caller (L = number of lookups).
 * ------------------------------------------------------------------------------------- */
KM_API int km_index_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n, int64_t L,
                 const km_view *x1, const km_view *x2, const km_view *params,
                 const km_view *start, const km_view *end,
                 const int32_t *const *batch_indices, const int32_t *row, const int32_t *col,
                 float *out, void *stream);

/* grad[b, q] = d/d theta_q sum_l [batch(l) == b] out_grad[l] * K[b, row[l], col[l]].  Replaces
 * index_bwd.call(..., out_grad) (native/index_bwd/index_bwd.cpp:6-27, index_bwd.cu:65-112).
 * grad (B.., P) every element written.  workspace: km_index_bwd_workspace_bytes(...) bytes. */
KM_API size_t km_index_bwd_workspace_bytes(int kernel_type, const km_batch *batch);

KM_API int km_index_bwd_f32(int kernel_type, const km_batch *batch, int64_t m, int64_t n, int64_t L,
                     const km_view *x1, const km_view *x2, const km_view *params,
                     const km_view *start, const km_view *end,
                     const int32_t *const *batch_indices, const int32_t *row,
                     const int32_t *col, const float *out_grad, const km_view *grad,
                     void *workspace, size_t workspace_bytes, void *stream);

/* ---------------------------------------------------------------------------------------
 * Band construction on the device (the reference runs these on one CPU thread after a
 * device-to-host copy, native/ranges/ranges.cpp:8-150).  x1 (B, m), x2 (B, n) contiguous fp32;
 * start, end (B, ceil(m/block)) contiguous int32, every element written.  Results are
 * bit-identical to the reference's sequential scans for any input: non-decreasing x2 (the
 * case every caller produces) takes a parallel search, anything else a sequential scan on the
 * device.  `flags` is a device int32[B] scratch (contents irrelevant on entry).
 * ------------------------------------------------------------------------------------- */

/* ranges.make_ranges(x1, x2, cutoff, block_size, align)  (native/ranges/ranges.cpp:8-62) */
KM_API int km_make_ranges_f32(int64_t B, int64_t m, int64_t n, const float *x1, const float *x2,
                       float cutoff, int32_t block_size, int32_t align, int32_t *start,
                       int32_t *end, int32_t *flags, void *stream);

/* ranges.make_ranges_symmetric(x, cutoff, block_size)  (native/ranges/ranges.cpp:64-101) */
KM_API int km_make_ranges_symmetric_f32(int64_t B, int64_t n, const float *x, float cutoff,
                                 int32_t block_size, int32_t *start, int32_t *end,
                                 int32_t *flags, void *stream);

/* The symmetric pattern for B kernels with their own cutoffs in one call: cutoffs (device, B
 * fp32); x (B rows, x_batch_stride elements apart; 0 = one x shared by all).  Equals B calls of
 * km_make_ranges_symmetric_f32 -- a mixture of components with different lengthscales over the
 * same inputs builds its bands with one set of launches instead of B.  No reference counterpart
 * (the reference takes one cutoff per call). */
KM_API int km_make_ranges_symmetric_cutoffs_f32(int64_t B, int64_t n, const float *x,
                                         int64_t x_batch_stride, const float *cutoffs,
                                         int32_t block_size, int32_t *start, int32_t *end,
                                         int32_t *flags, void *stream);

/* ranges.transpose_ranges(start, end, x1_size, x2_size, block_size)
 * (native/ranges/ranges.cpp:103-150).  start, end (B, R); start_t, end_t (B, ceil(x2_size/block)).
 * The caller checks block alignment (kernel_matmul/ranges.py:110-113). */
KM_API int km_transpose_ranges_i32(int64_t B, int64_t R, const int32_t *start, const int32_t *end,
                            int64_t x1_size, int64_t x2_size, int32_t block_size,
                            int32_t *start_t, int32_t *end_t, void *stream);

/* Visited entries sum_b sum_r rows(r) * (end - start) (bands clamped), written to *count
 * (device int64).  No reference counterpart; used for throughput accounting. */
KM_API int km_count_entries(const km_batch *batch, int64_t m, int64_t n, const km_view *start,
                     const km_view *end, int64_t *count, void *stream);

/* `iters` of the two calibration calls below may not exceed this (a mistaken argument must not
 * become a kernel that never ends on a shared GPU). */
#define KM_PROBE_MAX_ITERS (1LL << 24)

/* FP32-pipe calibration: runs `iters` dependent-chain-free FFMA rounds on every SM and writes a
 * checksum to *sink (device float, may be NULL).  flops = 2 * threads * iters * 64 are returned
 * in *flops_out (host).  No reference counterpart; bench.py times it to obtain the measured
 * FP32 FMA peak the roofline fractions are quoted against. */
KM_API int km_probe_fp32_peak(int64_t iters, float *sink, double *flops_out, void *stream);

/* Special-function-unit calibration: `iters` rounds of 8 independent ex2.approx chains per thread
 * on every SM; the number of SFU operations is returned in *ops_out (host).  No reference
 * counterpart; bench.py times it to obtain the measured SFU rate, which bounds the tensor-core
 * kernels (their FP32-pipe work per entry is small; kappa costs 1-3 SFU operations per entry). */
KM_API int km_probe_sfu_peak(int64_t iters, float *sink, double *ops_out, void *stream);

/* ---------------------------------------------------------------------------------------
 * Vector kernels of the row-sharded conjugate-gradient solve (K + sigma^2 I) X = Y.  No reference
 * counterpart: the reference has no CG, it inherits LinearOperator.solve from the third-party
 * linear_operator package (tests/test_linear_operator.py:9-38).  One iteration is
 *     km_matmul_rows_f32 (K p on the rank's rows)  ->  km_cg_q_dots_f32  ->  km_cg_segment_sums_f32
 *     -> [all-gather]  ->  km_cg_update_xr_f32  ->  km_cg_segment_sums_f32  ->  [all-gather]
 *     ->  km_cg_update_p_f32.
 * All vectors are fp32, (n, k) row-major with row stride k, indexed by GLOBAL row; a rank owns
 * the rows [row0, row1) (row0 a multiple of 128) and keeps r and p valid on [lo, hi), the columns
 * its band reads.  Inner products: one fp32 partial per 128-row block, fp64 sums per segment of
 * `seg_blocks` consecutive row blocks, and the gathered segment sums (seg_ranks records,
 * seg_rank_stride_bytes apart, of seg_slots x k doubles each; unused slots zero) added in record
 * order -- the same numbers for any number of ranks whose windows are whole segments.
 * ------------------------------------------------------------------------------------- */

/* block_partials[(row - row0) / 128][c] = sum over the block's rows of a[row, c] * b[row, c] */
KM_API int km_cg_block_dots_f32(int64_t k, const float *a, const float *b, int64_t row0, int64_t row1,
                                float *block_partials, void *stream);

/* kp[row, :] (in: K p) becomes q = K p + sigma2 * p on the own rows; block partials of p . q; the
 * first top_rows and the last bottom_rows rows of q are also copied to send_top / send_bottom
 * (what the neighbouring ranks need of q). */
KM_API int km_cg_q_dots_f32(int64_t k, float *kp, const float *p, float sigma2, int64_t row0, int64_t row1,
                            float *block_partials, float *send_top, int64_t top_rows, float *send_bottom,
                            int64_t bottom_rows, void *stream);

/* seg_sums[s][c] = sum of block_partials[blk][c] over the blocks [s * seg_blocks, (s + 1) * seg_blocks) */
KM_API int km_cg_segment_sums_f32(int64_t k, const float *block_partials, int64_t blocks, int64_t seg_blocks,
                                  double *seg_sums, void *stream);

/* start of a solve: rs[c] = total of the gathered segment sums of y . y, ynorm[c] = sqrt(rs[c]) */
KM_API int km_cg_init_scalars_f32(int64_t k, const void *seg_sums, int64_t seg_rank_stride_bytes, int32_t seg_ranks,
                                  int32_t seg_slots, float *rs, float *ynorm, void *stream);

/* alpha = rs / (p . q) from the gathered sums; x += alpha p on the own rows; r -= alpha q on
 * [lo, hi), with q of a row below / above the own window read from
 * q_below[(row - below_origin) * k + c] / q_above[(row - above_origin) * k + c]; block partials of
 * the new r . r over the own rows.  alpha_row (may be NULL): alpha[k] of this iteration is stored
 * there (with the betas, the Lanczos coefficients of the solve: log-determinant estimates). */
KM_API int km_cg_update_xr_f32(int64_t k, float *x, float *r, const float *p, const float *q_own,
                               const float *q_below, int64_t below_origin, const float *q_above,
                               int64_t above_origin, int64_t row0, int64_t row1, int64_t lo, int64_t hi,
                               const void *pq_seg_sums, int64_t seg_rank_stride_bytes, int32_t seg_ranks,
                               int32_t seg_slots, const float *rs, float *block_partials, float *alpha_row,
                               void *stream);

/* rs_new = total of the gathered sums of r . r; beta = rs_new / rs_old; p = r + beta p on [lo, hi);
 * rs_new[k] is stored (rs_old and rs_new must be different buffers) and, if history_row is not
 * NULL, history_row[c] = sqrt(rs_new[c]) / ynorm[c]; if beta_row is not NULL, beta_row[c] = beta. */
KM_API int km_cg_update_p_f32(int64_t k, float *p, const float *r, int64_t lo, int64_t hi, const void *rr_seg_sums,
                              int64_t seg_rank_stride_bytes, int32_t seg_ranks, int32_t seg_slots,
                              const float *rs_old, float *rs_new, const float *ynorm, float *history_row,
                              float *beta_row, void *stream);

/* ---------------------------------------------------------------------------------------
 * Self-tests of the give-up path of the tensor-core kernels.  No reference counterpart (the
 * reference's debug build synchronises and throws on a CUDA error,
 * native/common/gpu_assert.cuh:6-23; its kernels have no hand-offs that could stall).
 *
 * Every hand-off inside km_matmul_tc_f32, the *_tc_f32 gradients and the tensor-core batch sum
 * of km_matmul_rows_f32 is an mbarrier wait with a poll limit.  When the limit runs out the CTA
 * stops, waits for its own copies and MMAs in flight, releases its tensor memory, sets the
 * status word and writes NaN results; it never spins for ever and never traps.
 *
 * km_selftest_bounded_wait launches one warp that waits, with `polls` polls, on a barrier nobody
 * arrives at and writes 1 to *status (device int32) when the wait gave up, 0 if it did not.
 * km_selftest_set_wait_polls(polls) sets the poll limit that later launches of the tensor-core
 * kernels of this process use: 0 makes every wait that is not complete at its first test give
 * up at once, -1 restores the default.  A process-wide setting for tests; not thread-safe with
 * respect to launches in flight on other host threads.
 * ------------------------------------------------------------------------------------- */
KM_API int km_selftest_bounded_wait(int64_t polls, int32_t *status, void *stream);
KM_API int km_selftest_set_wait_polls(int64_t polls);

#ifdef __cplusplus
}
#endif
#endif /* KM_B200_H */
