// C++ source compatibility with the vectorSparse operator headers.
//
// Including this file gives a translation unit the twelve overloads the reference declares in
//   include/wmma_spmm.cuh:7-29   spmm::wmmaSpmm   (half->float, half->half, float->float)
//   include/cuda_spmm.cuh:7-29   spmm::cudaSpmm   (same three)
//   include/wmma_sddmm.cuh:7-33  sddmm::wmmaSddmm (same three, + vec_length, stream, algorithm)
//   include/cuda_sddmm.cuh:7-32  sddmm::cudaSddmm (same three, + vec_length, stream)
// with identical names, argument order and meaning, implemented inline on the C ABI of libvsparse_b200.so, so
// a caller written against the reference (its benchmark drivers, for instance) recompiles unchanged and links
// with -lvsparse_b200 instead of the reference's object files.
//
// Behaviour kept from the reference: one asynchronous launch, no synchronisation, the "V=<n>" line on stdout
// (src/wmma_spmm.cu:330-343), the "Unsupported Vector Length!" line for other vector lengths (:345-346) and the
// "doesn't support" lines of the float tensor-core / float SDDMM overloads, which compute nothing and return
// cudaSuccess (src/wmma_spmm.cu:412-422, src/cuda_sddmm.cu:1333-1344, src/wmma_sddmm.cu:3204-3215).
// Behaviour that differs: the float cudaSpmm overload, an empty stub in the reference
// (src/cuda_spmm.cu:328-338), computes the product; `stream` is honoured (the reference ignores it);
// rejected arguments return cudaErrorInvalidValue instead of launching with them.
#ifndef VSPARSE_COMPAT_H
#define VSPARSE_COMPAT_H

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdio.h>

#include "vsparse_b200.h"

namespace vsparse_compat_detail {
inline cudaError_t to_cuda(int rc) {
    if (rc == VS_OK) return cudaSuccess;
    if (rc > 0) return static_cast<cudaError_t>(rc);
    if (rc == VS_ERR_VEC_LENGTH) {
        printf("Unsupported Vector Length!\n");
        return cudaGetLastError();  // what the reference returns after printing: nothing was launched
    }
    fprintf(stderr, "vsparse_b200: %s\n", vs_error_string(rc));
    return cudaErrorInvalidValue;
}
inline void announce(int vec_length) {
    if (vec_length == 1 || vec_length == 2 || vec_length == 4 || vec_length == 8) printf("V=%d\n", vec_length);
}
}  // namespace vsparse_compat_detail

namespace spmm {

inline cudaError_t wmmaSpmm(int m_vec, int vec_length, int k, int n, const int* __restrict__ row_indices,
                            const int* __restrict__ row_offsets, const int* __restrict__ column_indices,
                            const half* __restrict__ values, const half* __restrict__ rhs_matrix,
                            float* __restrict__ output_matrix) {
    if (vec_length != 1) vsparse_compat_detail::announce(vec_length);
    return vsparse_compat_detail::to_cuda(vs_spmm(VS_PATH_TENSOR, VS_F16, VS_F32, m_vec, vec_length, k, n, row_indices,
                                                  row_offsets, column_indices, values, rhs_matrix, output_matrix, 0));
}

inline cudaError_t wmmaSpmm(int m_vec, int vec_length, int k, int n, const int* __restrict__ row_indices,
                            const int* __restrict__ row_offsets, const int* __restrict__ column_indices,
                            const half* __restrict__ values, const half* __restrict__ rhs_matrix,
                            half* __restrict__ output_matrix) {
    if (vec_length != 1) vsparse_compat_detail::announce(vec_length);
    return vsparse_compat_detail::to_cuda(vs_spmm(VS_PATH_TENSOR, VS_F16, VS_F16, m_vec, vec_length, k, n, row_indices,
                                                  row_offsets, column_indices, values, rhs_matrix, output_matrix, 0));
}

inline cudaError_t wmmaSpmm(int, int, int, int, const int* __restrict__, const int* __restrict__,
                            const int* __restrict__, const float* __restrict__, const float* __restrict__,
                            float* __restrict__) {
    printf("wmmaSpmm doesn't support float input.\n");
    return cudaSuccess;
}

inline cudaError_t cudaSpmm(int m_vec, int vec_length, int k, int n, const int* __restrict__ row_indices,
                            const int* __restrict__ row_offsets, const int* __restrict__ column_indices,
                            const half* __restrict__ values, const half* __restrict__ rhs_matrix,
                            float* __restrict__ output_matrix) {
    vsparse_compat_detail::announce(vec_length);
    return vsparse_compat_detail::to_cuda(vs_spmm(VS_PATH_CUDA_CORE, VS_F16, VS_F32, m_vec, vec_length, k, n,
                                                  row_indices, row_offsets, column_indices, values, rhs_matrix,
                                                  output_matrix, 0));
}

inline cudaError_t cudaSpmm(int m_vec, int vec_length, int k, int n, const int* __restrict__ row_indices,
                            const int* __restrict__ row_offsets, const int* __restrict__ column_indices,
                            const half* __restrict__ values, const half* __restrict__ rhs_matrix,
                            half* __restrict__ output_matrix) {
    vsparse_compat_detail::announce(vec_length);
    return vsparse_compat_detail::to_cuda(vs_spmm(VS_PATH_CUDA_CORE, VS_F16, VS_F16, m_vec, vec_length, k, n,
                                                  row_indices, row_offsets, column_indices, values, rhs_matrix,
                                                  output_matrix, 0));
}

inline cudaError_t cudaSpmm(int m_vec, int vec_length, int k, int n, const int* __restrict__ row_indices,
                            const int* __restrict__ row_offsets, const int* __restrict__ column_indices,
                            const float* __restrict__ values, const float* __restrict__ rhs_matrix,
                            float* __restrict__ output_matrix) {
    vsparse_compat_detail::announce(vec_length);
    return vsparse_compat_detail::to_cuda(vs_spmm(VS_PATH_CUDA_CORE, VS_F32, VS_F32, m_vec, vec_length, k, n,
                                                  row_indices, row_offsets, column_indices, values, rhs_matrix,
                                                  output_matrix, 0));
}

}  // namespace spmm

namespace sddmm {

inline cudaError_t wmmaSddmm(int m_vec, int k, int n, int nonzeros_vec, const int* __restrict__ row_indices,
                             const int* __restrict__ row_offsets, const int* __restrict__ col_indices,
                             const half* __restrict__ lhs_matrix, const half* __restrict__ rhs_matrix,
                             float* __restrict__ output_values, int vec_length, cudaStream_t stream, int algorithm) {
    return vsparse_compat_detail::to_cuda(vs_sddmm(VS_PATH_TENSOR, VS_F16, VS_F32, m_vec, k, n, nonzeros_vec,
                                                   row_indices, row_offsets, col_indices, lhs_matrix, rhs_matrix,
                                                   output_values, vec_length, stream, algorithm));
}

inline cudaError_t wmmaSddmm(int m_vec, int k, int n, int nonzeros_vec, const int* __restrict__ row_indices,
                             const int* __restrict__ row_offsets, const int* __restrict__ col_indices,
                             const half* __restrict__ lhs_matrix, const half* __restrict__ rhs_matrix,
                             half* __restrict__ output_values, int vec_length, cudaStream_t stream, int algorithm) {
    return vsparse_compat_detail::to_cuda(vs_sddmm(VS_PATH_TENSOR, VS_F16, VS_F16, m_vec, k, n, nonzeros_vec,
                                                   row_indices, row_offsets, col_indices, lhs_matrix, rhs_matrix,
                                                   output_values, vec_length, stream, algorithm));
}

inline cudaError_t wmmaSddmm(int, int, int, int, const int* __restrict__, const int* __restrict__,
                             const int* __restrict__, const float* __restrict__, const float* __restrict__,
                             float* __restrict__, int, cudaStream_t, int) {
    printf("wmmaSddmm doesn't support float input.\n");
    return cudaSuccess;
}

inline cudaError_t cudaSddmm(int m_vec, int k, int n, int nonzeros_vec, const int* __restrict__ row_indices,
                             const int* __restrict__ row_offsets, const int* __restrict__ col_indices,
                             const half* __restrict__ lhs_matrix, const half* __restrict__ rhs_matrix,
                             float* __restrict__ output_values, int vec_length, cudaStream_t stream) {
    return vsparse_compat_detail::to_cuda(vs_sddmm(VS_PATH_CUDA_CORE, VS_F16, VS_F32, m_vec, k, n, nonzeros_vec,
                                                   row_indices, row_offsets, col_indices, lhs_matrix, rhs_matrix,
                                                   output_values, vec_length, stream, 0));
}

inline cudaError_t cudaSddmm(int m_vec, int k, int n, int nonzeros_vec, const int* __restrict__ row_indices,
                             const int* __restrict__ row_offsets, const int* __restrict__ col_indices,
                             const half* __restrict__ lhs_matrix, const half* __restrict__ rhs_matrix,
                             half* __restrict__ output_values, int vec_length, cudaStream_t stream) {
    return vsparse_compat_detail::to_cuda(vs_sddmm(VS_PATH_CUDA_CORE, VS_F16, VS_F16, m_vec, k, n, nonzeros_vec,
                                                   row_indices, row_offsets, col_indices, lhs_matrix, rhs_matrix,
                                                   output_values, vec_length, stream, 0));
}

inline cudaError_t cudaSddmm(int, int, int, int, const int* __restrict__, const int* __restrict__,
                             const int* __restrict__, const float* __restrict__, const float* __restrict__,
                             float* __restrict__, int, cudaStream_t) {
    printf("cudaSddmm doesn't support float input.\n");
    return cudaSuccess;
}

}  // namespace sddmm

#endif  // VSPARSE_COMPAT_H
