// extern "C" doors to the reference's operator overloads (include/wmma_spmm.cuh:7-29, cuda_spmm.cuh:7-29,
// wmma_sddmm.cuh:7-33, cuda_sddmm.cuh:7-32), so that a Python harness can launch the reference's own kernels —
// compiled unmodified for sm_100a by the Makefile next to this file — for context timing.  Device pointers in, one
// asynchronous launch on the legacy default stream (the reference ignores its stream argument), the reference's
// return value out.  Benchmark infrastructure: nothing in the library links or loads this.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "wmma_spmm.cuh"
#include "cuda_spmm.cuh"
#include "wmma_sddmm.cuh"
#include "cuda_sddmm.cuh"

#define REFK_EXPORT extern "C" __attribute__((visibility("default")))

// out_f32 != 0 selects the half -> float overload, else half -> half.
REFK_EXPORT int refk_wmma_spmm(int m_vec, int vec_length, int k, int n, const int *row_indices, const int *row_offsets,
                               const int *column_indices, const void *values, const void *rhs, void *out, int out_f32) {
    return out_f32 ? (int)spmm::wmmaSpmm(m_vec, vec_length, k, n, row_indices, row_offsets, column_indices, (const half *)values,
                                         (const half *)rhs, (float *)out)
                   : (int)spmm::wmmaSpmm(m_vec, vec_length, k, n, row_indices, row_offsets, column_indices, (const half *)values,
                                         (const half *)rhs, (half *)out);
}

REFK_EXPORT int refk_cuda_spmm(int m_vec, int vec_length, int k, int n, const int *row_indices, const int *row_offsets,
                               const int *column_indices, const void *values, const void *rhs, void *out, int out_f32) {
    return out_f32 ? (int)spmm::cudaSpmm(m_vec, vec_length, k, n, row_indices, row_offsets, column_indices, (const half *)values,
                                         (const half *)rhs, (float *)out)
                   : (int)spmm::cudaSpmm(m_vec, vec_length, k, n, row_indices, row_offsets, column_indices, (const half *)values,
                                         (const half *)rhs, (half *)out);
}

REFK_EXPORT int refk_wmma_sddmm(int m_vec, int k, int n, int nonzeros_vec, const int *row_indices, const int *row_offsets,
                                const int *col_indices, const void *lhs, const void *rhs, void *out, int vec_length, int algorithm,
                                int out_f32) {
    return out_f32 ? (int)sddmm::wmmaSddmm(m_vec, k, n, nonzeros_vec, row_indices, row_offsets, col_indices, (const half *)lhs,
                                           (const half *)rhs, (float *)out, vec_length, 0, algorithm)
                   : (int)sddmm::wmmaSddmm(m_vec, k, n, nonzeros_vec, row_indices, row_offsets, col_indices, (const half *)lhs,
                                           (const half *)rhs, (half *)out, vec_length, 0, algorithm);
}

REFK_EXPORT int refk_cuda_sddmm(int m_vec, int k, int n, int nonzeros_vec, const int *row_indices, const int *row_offsets,
                                const int *col_indices, const void *lhs, const void *rhs, void *out, int vec_length, int out_f32) {
    return out_f32 ? (int)sddmm::cudaSddmm(m_vec, k, n, nonzeros_vec, row_indices, row_offsets, col_indices, (const half *)lhs,
                                           (const half *)rhs, (float *)out, vec_length, 0)
                   : (int)sddmm::cudaSddmm(m_vec, k, n, nonzeros_vec, row_indices, row_offsets, col_indices, (const half *)lhs,
                                           (const half *)rhs, (half *)out, vec_length, 0);
}
