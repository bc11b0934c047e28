// Shared by spmm_benchmark.cpp and sddmm_benchmark.cpp: benchmark-spec parsing, CVSE loading, checked CUDA
// calls and the verification summary.  The drivers keep the positional command lines of the reference
// (spmm_benchmark.cpp:480-509, sddmm_benchmark.cpp:399-432) so harnesses that shell out to them keep working.
#pragma once
#include <cuda_fp16.h>
#include <cuda_profiler_api.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "vsparse_b200.h"

inline void check_cuda(cudaError_t e, const char *what) {
    if (e != cudaSuccess) {
        fprintf(stderr, "CUDA Runtime Error: %s (%s)\n", cudaGetErrorString(e), what);
        exit(1);
    }
}
inline void check_vs(int rc, const char *what) {
    if (rc < 0) {
        fprintf(stderr, "%s: %s\n", what, vs_error_string(rc));
        exit(1);
    }
    if (rc > 0) check_cuda(static_cast<cudaError_t>(rc), what);
}

struct HostCvse {
    int m_vec = 0, n = 0, nnz_vec = 0;
    std::vector<int32_t> row_offsets, col_indices, row_indices;
};

// `bm` is either a path to a .smtx pattern file, or a synthetic pattern
//     synthetic:<kind>:<m_vec>x<n>:s=<sparsity>[:seed=<u64>][:band=<cols>]
// with kind in {fixed, beta, uniform, band} (see vs_cvse_generate).  The .smtx row count is the number of
// VECTOR rows, as in the reference (spmm_benchmark.cpp:26-33), and so is <m_vec> here.
inline HostCvse load_benchmark(const std::string &bm, int vec_length, bool sorted) {
    HostCvse a;
    if (bm.rfind("synthetic:", 0) == 0) {
        char kind[32] = {0};
        double sparsity = 0.9;
        unsigned long long seed = 0;
        int band = 0;
        if (sscanf(bm.c_str(), "synthetic:%31[a-z]:%dx%d", kind, &a.m_vec, &a.n) != 3) {
            fprintf(stderr, "bad synthetic spec: %s\n", bm.c_str());
            exit(1);
        }
        const char *p;
        if ((p = strstr(bm.c_str(), ":s="))) sparsity = atof(p + 3);
        if ((p = strstr(bm.c_str(), ":seed="))) seed = strtoull(p + 6, nullptr, 10);
        if ((p = strstr(bm.c_str(), ":band="))) band = atoi(p + 6);
        int k = !strcmp(kind, "fixed") ? 0 : !strcmp(kind, "beta") ? 1 : !strcmp(kind, "uniform") ? 2 : !strcmp(kind, "band") ? 3 : -1;
        if (k < 0) {
            fprintf(stderr, "unknown synthetic kind: %s\n", kind);
            exit(1);
        }
        // a vector length the operators do not support still gets a pattern, so that the call is made and answers
        // "Unsupported Vector Length!" itself, as the reference's dispatch does (src/wmma_spmm.cu:345-346)
        if (!(vec_length == 1 || vec_length == 2 || vec_length == 4 || vec_length == 8)) vec_length = 1;
        a.row_offsets.resize((size_t)a.m_vec + 1);
        int nnz = vs_cvse_generate(k, seed, a.m_vec, a.n, vec_length, sparsity, band, a.row_offsets.data(), nullptr);
        check_vs(nnz < 0 ? nnz : 0, "vs_cvse_generate");
        a.nnz_vec = nnz;
        a.col_indices.resize((size_t)nnz + 1);
        check_vs(vs_cvse_generate(k, seed, a.m_vec, a.n, vec_length, sparsity, band, a.row_offsets.data(), a.col_indices.data()) < 0 ? VS_ERR_ARG : 0,
                 "vs_cvse_generate");
    } else {
        check_vs(vs_smtx_read_header(bm.c_str(), &a.m_vec, &a.n, &a.nnz_vec), bm.c_str());
        a.row_offsets.resize((size_t)a.m_vec + 1);
        a.col_indices.resize((size_t)a.nnz_vec + 1);
        check_vs(vs_smtx_read(bm.c_str(), a.m_vec, a.nnz_vec, a.row_offsets.data(), a.col_indices.data()), bm.c_str());
    }
    a.row_indices.resize((size_t)a.m_vec + 1);
    check_vs(vs_row_swizzle(sorted ? 1 : 0, a.m_vec, a.row_offsets.data(), a.row_indices.data()), "vs_row_swizzle");
    return a;
}

template <typename T> struct Elem;
template <> struct Elem<float> {
    static constexpr int kDtype = VS_F32;
    static float to_float(float x) { return x; }
};
template <> struct Elem<half> {
    static constexpr int kDtype = VS_F16;
    static float to_float(half x) { return __half2float(x); }
};

template <typename T> T *to_device(const std::vector<T> &h, size_t count) {
    T *d = nullptr;
    check_cuda(cudaMalloc(&d, (count ? count : 1) * sizeof(T)), "cudaMalloc");
    if (count) check_cuda(cudaMemcpy(d, h.data(), count * sizeof(T), cudaMemcpyHostToDevice), "cudaMemcpy");
    return d;
}

// The reference's pass criterion (abs difference <= 0.5 per element, spmm_benchmark.cpp:214) and its two
// messages, followed by one line with the tighter error norms against a double-precision host result.
inline void report(const char *op, size_t count, const std::vector<float> &device, const std::vector<float> &host32,
                   const std::vector<double> &host64) {
    int errors = 0;
    double num = 0, den = 0, max_abs = 0;
    for (size_t j = 0; j < count; ++j) {
        if (std::fabs(device[j] - host32[j]) > 0.5f || !std::isfinite(device[j])) ++errors;
        double d = (double)device[j] - host64[j];
        num += d * d;
        den += host64[j] * host64[j];
        if (std::fabs(d) > max_abs) max_abs = std::fabs(d);
    }
    if (errors > 0) printf("%s does not agree with SEQUENTIAL! %d errors!\n", op, errors);
    else printf("Results verified: they agree.\n");
    printf("rel_l2 %.3e max_abs %.3e (against a double-precision host result)\n", den > 0 ? std::sqrt(num / den) : std::sqrt(num), max_abs);
}
