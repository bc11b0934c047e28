// Shim that compiles the vectorSparse reference's OWN host verification code, where it lies in the
// reference checkout, into a small shared library used only to pin the oracle.
//
// TEST INFRASTRUCTURE ONLY: never linked or loaded by the shipped library.
//
// What is taken from the reference, at build time, without copying it into this repository:
//   * include/bm_test_utils.h (whole header, via -I<reference>): Host_sddmm (:171-193),
//     IdentityRowSwizzle / SortedRowSwizzle (:196-215), MakeDenseMatrix (:130-142).
//   * the inline host SpMM loop of spmm_benchmark.cpp:66-86.  That file cannot be compiled as a unit
//     (it includes sputnik, which is not vendored), so oracle/Makefile extracts exactly that line range
//     into the build directory as `spmm_host_loop.inc` and it is #included below inside a function whose
//     local names match the driver's (func, m, k, m_vec, vec_length, row_offsets, col_indices, values,
//     rhs_matrix, output_value_host).
#include <cstdint>
#include <random>
#include <string>
#include <vector>
#include <numeric>

#include "include/bm_test_utils.h"

template <typename InType>
static void reference_spmm_host_loop(int m_vec, int vec_length, int k, const int *row_offsets,
                                     const int *col_indices, const InType *values, const InType *rhs_matrix,
                                     float *output_value_host) {
    const bool func = true;
    const int m = m_vec * vec_length;
    {
#include "spmm_host_loop.inc"
    }
}

extern "C" {

__attribute__((visibility("default"))) void ref_spmm_host_f32(int m_vec, int V, int N, const int *row_offsets,
                                                               const int *col_indices, const float *values,
                                                               const float *B, float *C) {
    reference_spmm_host_loop<float>(m_vec, V, N, row_offsets, col_indices, values, B, C);
}

// fp16 operands arrive as raw 16-bit patterns; `half` on the host has the same storage.
__attribute__((visibility("default"))) void ref_spmm_host_h16(int m_vec, int V, int N, const int *row_offsets,
                                                               const int *col_indices, const uint16_t *values,
                                                               const uint16_t *B, float *C) {
    static_assert(sizeof(half) == 2, "half must be 16 bits");
    reference_spmm_host_loop<half>(m_vec, V, N, row_offsets, col_indices, reinterpret_cast<const half *>(values),
                                   reinterpret_cast<const half *>(B), C);
}

__attribute__((visibility("default"))) void ref_sddmm_host_f32(int m_vec, int k, int V, const int *row_offsets,
                                                                const int *col_indices, const float *lhs,
                                                                const float *rhs, float *out) {
    Host_sddmm<float, float>(m_vec, k, V, row_offsets, col_indices, lhs, rhs, out);
}

__attribute__((visibility("default"))) void ref_sddmm_host_h16(int m_vec, int k, int V, const int *row_offsets,
                                                                const int *col_indices, const uint16_t *lhs,
                                                                const uint16_t *rhs, float *out) {
    Host_sddmm<half, float>(m_vec, k, V, row_offsets, col_indices, reinterpret_cast<const half *>(lhs),
                            reinterpret_cast<const half *>(rhs), out);
}

// Same, rounding each output to fp16 the way the half-output driver does (OutType = half).
__attribute__((visibility("default"))) void ref_sddmm_host_h16_out16(int m_vec, int k, int V,
                                                                      const int *row_offsets,
                                                                      const int *col_indices, const uint16_t *lhs,
                                                                      const uint16_t *rhs, uint16_t *out) {
    Host_sddmm<half, half>(m_vec, k, V, row_offsets, col_indices, reinterpret_cast<const half *>(lhs),
                           reinterpret_cast<const half *>(rhs), reinterpret_cast<half *>(out));
}

__attribute__((visibility("default"))) void ref_row_swizzle(int sorted, int m_vec, const int *row_offsets,
                                                             int *row_indices) {
    if (sorted) SortedRowSwizzle(m_vec, row_offsets, row_indices);
    else IdentityRowSwizzle(m_vec, row_indices);
}

// MakeDenseMatrix with the default-constructed engine the drivers use (spmm_benchmark.cpp:38,59-60).
__attribute__((visibility("default"))) void ref_make_dense_f32(int rows, int cols, float *out) {
    std::default_random_engine generator;
    MakeDenseMatrix<float>(rows, cols, out, generator);
}

__attribute__((visibility("default"))) void ref_make_dense_h16(int rows, int cols, uint16_t *out) {
    std::default_random_engine generator;
    MakeDenseMatrix<half>(rows, cols, reinterpret_cast<half *>(out), generator);
}

}  // extern "C"
