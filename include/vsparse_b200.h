/*
 * vsparse_b200 — C ABI of the column-vector-sparse (CVSE) SpMM / SDDMM library for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain pointers and sizes.  Unless a function says "host", pointers are DEVICE
 * pointers owned by the caller; the library enqueues its kernels on `stream` (a cudaStream_t passed as void*)
 * and returns without synchronising.  One piece of device memory is the library's own: the tensor-path
 * operators keep a plan scratch per calling stream (cudaMallocAsync at the first call on a stream, and again
 * when a larger matrix needs more — make those calls outside stream capture; vs_release_scratch frees it).
 * A caller that hands over a buffer with vs_set_workspace gets a library that never allocates.
 *
 * Return value of every function: 0 on success, a negative VS_ERR_* code when the arguments are rejected
 * before anything is launched, or a positive cudaError_t if the CUDA runtime reported one.
 *
 * Naming follows the vectorSparse reference, whose operator headers these entry points replace:
 *   SpMM   A[m x n] * B[n x k] = C[m x k]      reference argument `k` = dense width, `n` = columns of A
 *   SDDMM  out = (lhs[m x k] * rhs[n x k]^T) sampled at the CVSE mask of an m x n matrix
 * CVSE: m_vec vector-rows of `vec_length` (V) real rows each (m = m_vec*V); row_offsets[m_vec+1] and
 * col_indices[nnz_vec] count column VECTORS; values[j*V+v] belongs to real row i*V+v, column col_indices[j];
 * row_indices[m_vec] is the order in which vector-rows are scheduled (a load-balancing hint that never
 * changes the result).
 */
#ifndef VSPARSE_B200_H
#define VSPARSE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types */
#define VS_F16 0
#define VS_F32 1

/* kernel families: the reference's wmma* entry points map to TENSOR, its cuda* entry points to CUDA_CORE */
#define VS_PATH_TENSOR 0
#define VS_PATH_CUDA_CORE 1

/* validation errors (nothing was launched) */
#define VS_OK 0
#define VS_ERR_VEC_LENGTH (-1)   /* vec_length not in {1,2,4,8} (tensor path: {2,4,8}) */
#define VS_ERR_DTYPE (-2)        /* unsupported (path, in_dtype, out_dtype) combination */
#define VS_ERR_SHAPE (-3)        /* negative size, or a size the path cannot tile (see each function) */
#define VS_ERR_NULL (-4)         /* a required pointer is null */
#define VS_ERR_ALIGN (-5)        /* a pointer or stride is not 16-byte aligned */
#define VS_ERR_STRUCTURE (-6)    /* host-side CVSE check failed: offsets not monotone, column out of range */
#define VS_ERR_IO (-7)           /* file could not be opened or parsed */
#define VS_ERR_ARG (-8)          /* any other rejected argument (unknown mode, batch < 1, ...) */
#define VS_ERR_DEVICE (-9)       /* a kernel reported a bounded wait that ran out (see vs_device_status) */

const char *vs_error_string(int code);

/* Library / build identification: "vsparse_b200 <version> sm_100a". */
const char *vs_version(void);

/* ------------------------------------------------------------------------------------------------------
 * SpMM.  Replaces spmm::wmmaSpmm (include/wmma_spmm.cuh:7-29, path = VS_PATH_TENSOR) and spmm::cudaSpmm
 * (include/cuda_spmm.cuh:7-29, path = VS_PATH_CUDA_CORE).
 *
 *   C[(i*V+v)*k + l] = sum_{j in row i} values[j*V+v] * rhs[col_indices[j]*k + l],  every row of C written
 *   (vector-rows without nonzeros produce zeros).
 *
 * (in_dtype, out_dtype): (F16,F16), (F16,F32) on both paths; (F32,F32) on VS_PATH_CUDA_CORE only (the
 * reference's float wmmaSpmm prints "doesn't support" and computes nothing, src/wmma_spmm.cu:412-422; here it
 * returns VS_ERR_DTYPE).  fp16 products are accumulated in fp32.
 * vec_length: {2,4,8} on the tensor path, {1,2,4,8} on the CUDA-core path, else VS_ERR_VEC_LENGTH.
 * k (dense width): tensor path needs k % 64 == 0 (as the reference, src/wmma_spmm.cu:327,396); CUDA-core path
 * needs k % 8 == 0 for fp16 and k % 4 == 0 for fp32.  values, rhs, out must be 16-byte aligned.
 *
 * Tensor path: two formulations, chosen on the device (the signature carries no nonzero count) by comparing
 * their measured costs: zero-filled 256 x 64 tiles of the sparse matrix multiplied with whole tiles of rhs cost
 * the same whatever the tiles hold; where that is more than a per-row overhead plus a cost per nonzero vector
 * (wide, very sparse matrices), and whenever the dense kernel produced a non-finite sum
 * (0 * Inf from a row of rhs that no nonzero names), one row of rhs is gathered per nonzero vector as in the
 * reference.  A matrix that names a column twice in one vector-row (the reference's generator pads rows that
 * way, include/bm_test_utils.h:110-124, and its kernels add both values) is recognised on the device and goes
 * to the gather kernel, which adds them too.
 * Environment variable VSPARSE_B200_SPMM = "dense" | "gather" forces one formulation.  The first tensor-path
 * call on a stream allocates a plan scratch buffer with cudaMallocAsync on that stream (8 bytes per nonzero
 * vector, bounded by m_vec * n and by 512 MB; reused and grown by later calls on the stream, never freed): make
 * that call outside stream capture.  Everything else about the call is asynchronous and allocation-free.
 * ---------------------------------------------------------------------------------------------------- */
int vs_spmm(int path, int in_dtype, int out_dtype, int m_vec, int vec_length, int k, int n,
            const int32_t *row_indices, const int32_t *row_offsets, const int32_t *col_indices,
            const void *values, const void *rhs_matrix, void *output_matrix, void *stream);

/* `batch` independent products that share one CVSE structure (row_indices/row_offsets/col_indices) and differ
 * in values, rhs and output, found at element strides stride_values / stride_rhs / stride_out from the first
 * (a stride of 0 shares that operand; stride_out must not be 0).  Strides must keep 16-byte alignment.
 * One launch covers the whole batch.  The reference has no batched call; this is the batch x head form of its
 * SpMM for fixed-mask sparse attention. */
int vs_spmm_batched(int path, int in_dtype, int out_dtype, int m_vec, int vec_length, int k, int n,
                    const int32_t *row_indices, const int32_t *row_offsets, const int32_t *col_indices,
                    const void *values, const void *rhs_matrix, void *output_matrix, int batch,
                    int64_t stride_values, int64_t stride_rhs, int64_t stride_out, void *stream);

/* ------------------------------------------------------------------------------------------------------
 * SpMM with the transposed sparse matrix:  out[n x k] = A^T . rhs,  A the m_vec*V x n CVSE matrix, rhs m_vec*V x k.
 *
 *   out[c*k + l] = sum over the nonzero vectors (i, j) with col_indices[j] == c of
 *                  sum_v values[j*V+v] * rhs[(i*V+v)*k + l];       every row of out written (zeros for a column
 *                                                                   no vector names)
 *
 * No counterpart in the reference, whose kernels cover the forward products (src/wmma_spmm.cu,
 * src/cuda_spmm.cu); this is the product on the other side of them in a training step of fixed-mask sparse
 * attention (dV = P^T dO, dK = dS^T Q), kept to the conventions of vs_spmm: device pointers, caller-owned
 * buffers, asynchronous on `stream`, nothing allocated.  `values` is the SAME array the forward operators use;
 * only the structure is transposed, once, on the host, by vs_cvse_transpose below.
 * (in_dtype, out_dtype): (F16,F16), (F16,F32); fp32 accumulation in the listed order (reproducible).
 * vec_length in {1,2,4,8}; k % 8 == 0; values, rhs, out 16-byte aligned.  Two kernels, chosen on the device from
 * their measured costs: A^T through the densifying tensor-core kernel of vs_spmm
 * (plan built from the transposed structure, the V values of a vector side by side in one row of the tile; same plan scratch rules as vs_spmm: per-stream buffer or
 * vs_set_workspace, first call on a stream outside capture), or CUDA cores (one warp per 256 columns of an
 * output row: very sparse matrices, a column named twice by one vector-row, non-finite sums, no scratch).
 * VSPARSE_B200_SPMM_T = "dense" | "gather" forces one.  The batched form shares the structure and strides
 * values / rhs / out as vs_spmm_batched.
 * ---------------------------------------------------------------------------------------------------- */
int vs_spmm_t(int in_dtype, int out_dtype, int m_vec, int vec_length, int k, int n, const int32_t *t_offsets,
              const int32_t *t_rows, const int32_t *t_src, const void *values, const void *rhs_matrix,
              void *output_matrix, void *stream);
int vs_spmm_t_batched(int in_dtype, int out_dtype, int m_vec, int vec_length, int k, int n, const int32_t *t_offsets,
                      const int32_t *t_rows, const int32_t *t_src, const void *values, const void *rhs_matrix,
                      void *output_matrix, int batch, int64_t stride_values, int64_t stride_rhs, int64_t stride_out,
                      void *stream);

/* ------------------------------------------------------------------------------------------------------
 * SDDMM.  Replaces sddmm::wmmaSddmm (include/wmma_sddmm.cuh:7-33, path = VS_PATH_TENSOR) and
 * sddmm::cudaSddmm (include/cuda_sddmm.cuh:7-32, path = VS_PATH_CUDA_CORE; `algorithm` ignored).
 *
 *   out[j*V+v] = sum_l lhs[(i*V+v)*k + l] * rhs[col_indices[j]*k + l]   for row_offsets[i] <= j < row_offsets[i+1]
 *
 * Exactly nonzeros_vec*V outputs are written; the structure arrays are read-only.
 * (in_dtype, out_dtype): (F16,F16), (F16,F32).  (F32,F32) is VS_ERR_DTYPE on both paths (the reference prints
 * "doesn't support", src/cuda_sddmm.cu:1333-1344, src/wmma_sddmm.cu:3204-3215).
 * k (contraction length): tensor path needs k % 64 == 0 (the reference's main loop, src/wmma_sddmm.cu:147);
 * CUDA-core path needs k % 8 == 0.
 * algorithm: 0..3 accepted on the tensor path and all computed by the same kernel — in the reference they are
 * implementation variants of one function, and variant 3 returns deliberately wrong values
 * (src/wmma_sddmm.cu:769-771); here it returns correct ones.  Other values: VS_ERR_ARG.
 *
 * Tensor path: two formulations, chosen on the host from nonzeros_vec, the shape and k.  Dense 256 x 128 tiles
 * of lhs . rhs^T sampled at the mask (denser masks, k >= 128), or one gathered row of rhs per mask entry as in
 * the reference.  Environment variable VSPARSE_B200_SDDMM = "dense" | "gather" forces one.  The dense
 * formulation keeps a plan scratch buffer per calling stream exactly as the tensor-path SpMM does (see vs_spmm);
 * with it, a mask entry whose column lies outside [0, n) is skipped instead of written as zero.
 * ---------------------------------------------------------------------------------------------------- */
int vs_sddmm(int path, int in_dtype, int out_dtype, int m_vec, int k, int n, int nonzeros_vec,
             const int32_t *row_indices, const int32_t *row_offsets, const int32_t *col_indices,
             const void *lhs_matrix, const void *rhs_matrix, void *output_values, int vec_length,
             void *stream, int algorithm);

/* Batched twin: shared structure; lhs, rhs, out at element strides (stride_out must not be 0). */
int vs_sddmm_batched(int path, int in_dtype, int out_dtype, int m_vec, int k, int n, int nonzeros_vec,
                     const int32_t *row_indices, const int32_t *row_offsets, const int32_t *col_indices,
                     const void *lhs_matrix, const void *rhs_matrix, void *output_values, int vec_length,
                     int batch, int64_t stride_lhs, int64_t stride_rhs, int64_t stride_out, void *stream,
                     int algorithm);

/* ------------------------------------------------------------------------------------------------------
 * Masked row softmax over CVSE values, in place or out of place (probs may equal scores):
 *   probs[j*V+v] = exp(scale*scores[j*V+v] - max) / sum,  max and sum over the entries j of vector-row i.
 * fp32 arithmetic; dtype is VS_F16 or VS_F32 for both arrays.  No counterpart in the reference (its README
 * points to an external repository for attention); it is the step between SDDMM and SpMM in fixed-mask
 * sparse attention.
 * ---------------------------------------------------------------------------------------------------- */
int vs_softmax_cvse(int dtype, int m_vec, int vec_length, const int32_t *row_indices,
                    const int32_t *row_offsets, const void *scores, void *probs, float scale, int batch,
                    int64_t stride, void *stream);

/* Fixed-mask sparse attention for `batch` (batch x head) problems sharing one mask:
 *   O_b = softmax(scale * SDDMM(Q_b, K_b)) . V_b, fp16 in and out, head dimension d (d % 64 == 0).
 * q [batch][m][d], kmat / vmat [batch][n][d], out [batch][m][d], all contiguous.
 * `workspace` must hold batch * nonzeros_vec * V fp16 values (the probabilities); the caller owns it.
 * One call for the whole batch (the batched form of the pipeline): it enqueues the SDDMM, the masked softmax and
 * the SpMM on `stream` (up to five kernels with their plan and fallback kernels); they are not fused into one. */
int vs_attention_cvse(int path, int m_vec, int vec_length, int n, int d, int nonzeros_vec,
                      const int32_t *row_indices, const int32_t *row_offsets, const int32_t *col_indices,
                      const void *q, const void *kmat, const void *vmat, void *out, void *workspace,
                      float scale, int batch, void *stream);

/* Backward of vs_softmax_cvse: grad_scores[j*V+v] = scale * probs[j*V+v] * (grad_probs[j*V+v] - sum over the row's
 * entries of probs * grad_probs), the gradient with respect to the scores the forward call was given (it applies
 * `scale` inside).  Same layout, dtype (F16 or F32, fp32 sums), batch and alignment rules as vs_softmax_cvse;
 * grad_scores may be grad_probs.  No counterpart in the reference (it has no softmax, README.md:76). */
int vs_softmax_cvse_backward(int dtype, int m_vec, int vec_length, const int32_t *row_offsets, const void *probs,
                             const void *grad_probs, void *grad_scores, float scale, int batch, int64_t stride,
                             void *stream);

/* Backward of vs_attention_cvse for fp16 q [m x d], kmat, vmat [n x d] per batch entry and one shared mask:
 * given grad_out [m x d] it writes grad_q [m x d], grad_k and grad_v [n x d] (fp16).  The probabilities are
 * recomputed (SDDMM + softmax into probs_workspace), then dV = P^T dO (vs_spmm_t), dP = dO V^T at the mask
 * (SDDMM), dS = softmax backward (in grad_workspace), dQ = dS K (SpMM), dK = dS^T Q (vs_spmm_t): seven calls of
 * the operators above on `stream`.  t_offsets / t_rows / t_src: the mask's transposed structure from
 * vs_cvse_transpose.  Both workspaces hold batch * nonzeros_vec * vec_length fp16 values and must differ.
 * No counterpart in the reference. */
int vs_attention_cvse_backward(int path, int m_vec, int vec_length, int n, int d, int nonzeros_vec,
                               const int32_t *row_indices, const int32_t *row_offsets, const int32_t *col_indices,
                               const int32_t *t_offsets, const int32_t *t_rows, const int32_t *t_src, const void *q,
                               const void *kmat, const void *vmat, const void *grad_out, void *grad_q, void *grad_k,
                               void *grad_v, void *probs_workspace, void *grad_workspace, float scale, int batch,
                               void *stream);

/* vs_attention_cvse for callers that may not allocate device memory.  No counterpart in the reference.
 *
 * Some hosts of this library cannot hand it a workspace: an inference runtime that plans all device memory
 * ahead of time and gives plug-ins no allocator, a service loop that must never hit the implicit device-wide
 * synchronisation of cudaMalloc / cudaFree, a caller that simply has no allocation hook at the point where
 * attention runs.  For them the probabilities (batch * nonzeros_vec * vec_length fp16 values) live in an
 * 8 MiB (8 388 608 byte) array that is part of the library image; every GPU that loads the library holds it
 * until the process exits.  Same arguments and results as vs_attention_cvse, minus `workspace`.
 *
 *  - Larger requests are refused with VS_ERR_SHAPE and a message on stderr; nothing is launched.
 *  - The call itself, and everything it calls, uses no cudaMalloc, cudaFree or allocating library routine: its
 *    SDDMM and SpMM steps always run the row-gather kernels, never the formulations that keep plan scratch.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *    current).  Make that first call outside any stream capture.
 *  - All calls on a device share the one array, and it keeps what the last call left in it.  Nothing in it has
 *    to start at zero: each call writes every probability before it reads it.  Two calls that overlap on the
 *    GPU (different streams, or graphs replayed concurrently) race on it: serialise them. */
int vs_attention_cvse_static(int path, int m_vec, int vec_length, int n, int d, int nonzeros_vec,
                             const int32_t *row_indices, const int32_t *row_offsets, const int32_t *col_indices,
                             const void *q, const void *kmat, const void *vmat, void *out, float scale, int batch,
                             void *stream);

/* ------------------------------------------------------------------------------------------------------
 * Host-buffer convenience forms (every pointer is a HOST pointer).  They allocate device buffers, copy the
 * operands in, run the operator, copy the result back and free the buffers, synchronising before returning:
 * what the reference drivers do around their kernel call (spmm_benchmark.cpp:100-216,
 * sddmm_benchmark.cpp:222-283).
 * ---------------------------------------------------------------------------------------------------- */
int vs_spmm_host(int path, int in_dtype, int out_dtype, int m_vec, int vec_length, int k, int n,
                 const int32_t *row_indices, const int32_t *row_offsets, const int32_t *col_indices,
                 const void *values, const void *rhs_matrix, void *output_matrix);

int vs_sddmm_host(int path, int in_dtype, int out_dtype, int m_vec, int k, int n, int nonzeros_vec,
                  const int32_t *row_indices, const int32_t *row_offsets, const int32_t *col_indices,
                  const void *lhs_matrix, const void *rhs_matrix, void *output_values, int vec_length,
                  int algorithm);

/* ------------------------------------------------------------------------------------------------------
 * Device status.  Kernels that wait on hardware barriers bound every wait; one that ran out records a code
 * in a per-device status word instead of hanging.  Reads the word of the current device (synchronises the
 * device), optionally clearing it.  0 = no kernel ever gave up.
 * ---------------------------------------------------------------------------------------------------- */
int vs_device_status(int clear, uint32_t *status);

/* ------------------------------------------------------------------------------------------------------
 * Plan scratch in the caller's hands (no counterpart in the reference, whose kernels keep no workspace:
 * src/wmma_spmm.cu:317-350).  The dense formulations of the tensor path bucket the nonzeros once per call and
 * need device memory for that.  By default the library keeps one buffer per calling stream (see vs_spmm).  A
 * caller that plans its own device memory can instead hand over a buffer:
 *
 *   vs_spmm_workspace_bytes / vs_sddmm_workspace_bytes / vs_spmm_t_workspace_bytes
 *                                                        bytes the dense formulation needs for such a call
 *                                                        (0: it is never used for this problem); no device needed
 *   vs_set_workspace(ptr, bytes)                         from now on the tensor-path calls made by THIS host
 *                                                        thread put their plan in [ptr, ptr + bytes) when it
 *                                                        fits and run the row-gather formulation when it does
 *                                                        not: with a workspace set the library never allocates.
 *                                                        (NULL, 0) returns to the library's own buffers.
 *
 * ptr must be 16-byte aligned device memory and stay valid until the work enqueued with it has completed; calls
 * that may overlap on the GPU (different streams) need different workspaces.
 * ---------------------------------------------------------------------------------------------------- */
int64_t vs_spmm_workspace_bytes(int m_vec, int vec_length, int n, int batch, int64_t stride_values);
int64_t vs_sddmm_workspace_bytes(int m_vec, int n, int nonzeros_vec);
int64_t vs_spmm_t_workspace_bytes(int m_vec, int vec_length, int n, int batch, int64_t stride_values);
int vs_set_workspace(void *workspace, int64_t bytes);

/* Frees the plan scratch the library keeps on the current device for `stream` (stream-ordered: behind the work
 * already enqueued there), or for every stream when every_stream != 0.  The next tensor-path call on such a
 * stream allocates again.  With the per-thread default stream handle (cudaStreamPerThread) the buffer of the
 * calling thread is meant: each host thread has its own.  No counterpart in the reference. */
int vs_release_scratch(void *stream, int every_stream);

/* Times the multiplying kernels of the dense tensor-core paths (the pair kernels of SpMM, the transposed product and
 * SDDMM) with CUDA events on their own streams.  enable != 0 switches the bracketing on for the calls that follow,
 * 0 off; either way the call first waits for the kernels bracketed so far and returns the sum of their durations
 * and their number (either pointer may be NULL), then forgets them.  A bracketed kernel does not overlap its
 * neighbours in the stream, so a call is slower while this is on: it measures the kernel, not the call.
 * Diagnostic, no counterpart in the reference. */
int vs_kernel_timing(int enable, double *total_ms, int *launches);

/* Measures the fp32 fused-multiply-add throughput of the current device (TFLOP/s, 2 flops per FMA) with a
 * register-only kernel: the roofline denominator for the fp32 CUDA-core SpMM, which is bound by FMA issue and not by
 * memory.  Synchronous (times three short launches on the legacy default stream and returns the best); diagnostic,
 * no counterpart in the reference. */
int vs_measure_fp32_fma(double *tflops);

/* Which tensor-path SDDMM formulation vs_sddmm / vs_sddmm_batched would run for this problem: 1 = dense tiles
 * sampled at the mask, 0 = row gather (environment override included).  Diagnostic, no counterpart in the
 * reference; lets a benchmark name the kernels it measures.  Needs no device. */
int vs_sddmm_formulation(int m_vec, int k, int n, int nonzeros_vec, int vec_length);

/* ------------------------------------------------------------------------------------------------------
 * Tensor-core encoding self-test (diagnostic; no counterpart in the reference).  Copies `image_bytes` of a
 * caller-built shared-memory image (device pointer) to the start of a 1024-byte aligned buffer, issues n_mma
 * (1..64) tcgen05.mma kind::f16 instructions with the given 64-bit (A, B) descriptor pairs — a HOST array of
 * 2 * n_mma descriptors, their start-address field relative to the image — accumulating into one tile, and
 * copies the accumulator, pre-filled with `fill`, to out[lane * ncols + col] (128 lanes, ncols a multiple of 8,
 * at most 128).  Lets the host confirm an operand layout convention against a plain matrix product before
 * trusting a kernel built on it.  Nothing is launched unless every operand lies inside the image: idesc must be
 * fp16 x fp16 -> fp32 with M = 128 and N <= ncols, descriptors unswizzled or with the 128-byte swizzle, and
 * start + extent (from the leading / stride byte offsets) <= image_bytes, else VS_ERR_SHAPE.
 * ---------------------------------------------------------------------------------------------------- */
int vs_selftest_mma(const void *image, int image_bytes, const uint64_t *descs, int n_mma, uint32_t idesc,
                    int ncols, float fill, float *out, void *stream);

/* The same for a PAIR of CTAs (tcgen05 cta_group::2, M = 256): each CTA of the pair loads its own image (128
 * rows of A and N / 2 columns of B at the offsets the shared descriptors name), the first CTA issues the MMAs for
 * both, and CTA r copies its accumulator lanes to out[(r * 128 + lane) * ncols + col]; ncols <= 256, N % 32 == 0.
 * Same host-side checks. */
int vs_selftest_mma_pair(const void *image0, const void *image1, int image_bytes, const uint64_t *descs, int n_mma,
                         uint32_t idesc, int ncols, float fill, float *out, void *stream);

/* Row-gather self-test (diagnostic; no counterpart in the reference): `groups` (1..32) hardware row gathers of
 * four rows each — indices from row_indices[4*groups] (device), rows >= `rows` read as zeros — 64 fp16 columns
 * wide starting at column x (a multiple of 8) of the row-major fp16 matrix [rows x cols]; the 512-byte blocks
 * land consecutively in a 1024-byte aligned shared-memory buffer with the 128-byte swizzle, which is copied raw
 * to out[groups * 512] bytes. */
int vs_selftest_gather4(const void *matrix, int rows, int cols, const int32_t *row_indices, int groups, int x,
                        void *out, void *stream);

/* ------------------------------------------------------------------------------------------------------
 * CVSE builder, row swizzle and generators — HOST functions on HOST arrays.
 * ---------------------------------------------------------------------------------------------------- */

/* Checks a CVSE structure: row_offsets[0]==0, non-decreasing, row_offsets[m_vec]==nonzeros_vec, every
 * column in [0, n).  Returns VS_OK or VS_ERR_STRUCTURE. */
int vs_cvse_validate(int m_vec, int n, int nonzeros_vec, const int32_t *row_offsets,
                     const int32_t *col_indices);

/* mode 0: identity (IdentityRowSwizzle, include/bm_test_utils.h:196-198).
 * mode 1: vector-rows by nonzero count, descending (SortedRowSwizzle, :200-215); ties by ascending index. */
int vs_row_swizzle(int mode, int m_vec, const int32_t *row_offsets, int32_t *row_indices);

/* .smtx pattern files (spmm_benchmark.cpp:21-54): line 1 "rows, cols, nnz"; line 2 rows+1 offsets; line 3 nnz
 * column indices.  The header call returns the three sizes; the body call fills caller arrays of
 * rows+1 and nnz ints. */
int vs_smtx_read_header(const char *path, int *rows, int *cols, int *nnz);
int vs_smtx_read(const char *path, int rows, int nnz, int32_t *row_offsets, int32_t *col_indices);
int vs_smtx_write(const char *path, int rows, int cols, int nnz, const int32_t *row_offsets,
                  const int32_t *col_indices);

/* Dense 0/1 mask [m_vec x n] (one byte per vector slot) -> CVSE structure.  Pass col_indices == NULL to
 * count only (row_offsets is still filled).  Returns nonzeros_vec or a negative error. */
int vs_cvse_from_dense_mask(int m_vec, int n, const uint8_t *mask, int32_t *row_offsets,
                            int32_t *col_indices);

/* HOST.  Structure of A^T for vs_spmm_t: for each column c of A, t_offsets[c] .. t_offsets[c+1] delimit its
 * nonzero vectors in t_rows (vector-row i, ascending) and t_src (index j of the vector in col_indices / values).
 * t_offsets holds n + 1 ints, t_rows and t_src nonzeros_vec each.  The input is validated first
 * (VS_ERR_STRUCTURE).  No counterpart in the reference. */
int vs_cvse_transpose(int m_vec, int n, int nonzeros_vec, const int32_t *row_offsets, const int32_t *col_indices,
                      int32_t *t_offsets, int32_t *t_rows, int32_t *t_src);

/* Vector-wise magnitude pruning of a dense row-major weight [m_vec * vec_length x n] (fp32) into CVSE: every
 * vec_length x 1 column vector is scored by the sum of its absolute values and the highest-scoring vectors are
 * kept — scope 0: round((1 - sparsity) * m_vec * n) of them over the whole matrix; scope 1: round((1 -
 * sparsity) * n) in every vector-row.  Ties go to the lower (vector-row, column).  Two-call protocol like the
 * generators: col_indices == NULL fills row_offsets and returns nonzeros_vec; the second call fills col_indices
 * (ascending within a row) and, when `values` is not NULL, the kept weights in the CVSE value layout
 * (values[j * vec_length + v]).  The reference has no pruning step: it reads patterns pruned elsewhere (DLMC
 * .smtx files, spmm_benchmark.cpp:21-54); this is the way in for a weight held in memory. */
int vs_cvse_prune_dense(int m_vec, int n, int vec_length, const float *weight, double sparsity, int scope,
                        int32_t *row_offsets, int32_t *col_indices, float *values);

/* Seeded pattern generators; two-call protocol: col_indices == NULL fills row_offsets and returns nnz_vec,
 * the second call (same arguments) fills col_indices too.  Columns ascend within a row.
 *   kind 0 "fixed"  : every vector-row gets exactly round((1-sparsity)*n) columns, uniform without replacement
 *   kind 1 "beta"   : row density = clip(2*(1-sparsity)*beta_i, 0, 1), beta_i ~ Beta(2,2); columns as above
 *   kind 2 "uniform": exactly round(m_vec*n*(1-sparsity)) slots uniform over the whole m_vec x n grid
 *                     (the recipe of MakeSparseMatrixRandomUniform, include/bm_test_utils.h:70-127)
 *   kind 3 "band"   : attention mask: a band of `band` columns centred on the vector-row's diagonal position
 *                     plus random columns on a stride-16 lattice until the row holds round((1-sparsity)*n)
 */
int vs_cvse_generate(int kind, uint64_t seed, int m_vec, int n, int vec_length, double sparsity, int band,
                     int32_t *row_offsets, int32_t *col_indices);

/* Seeded value generators (counter-based, identical on every platform).
 *   dist 0: uniform(-1, 1)  (the law of MakeDenseMatrix, include/bm_test_utils.h:130-142)
 *   dist 1: normal(0, sigma)
 * dtype VS_F32 writes floats; VS_F16 writes the fp32 draw rounded to nearest-even fp16. */
int vs_fill_random(int dtype, int dist, uint64_t seed, double sigma, int64_t count, void *out);

#ifdef __cplusplus
}
#endif
#endif /* VSPARSE_B200_H */
