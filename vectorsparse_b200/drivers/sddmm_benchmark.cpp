// sddmm_benchmark — D = (A[m x k] * B[n x k]^T) sampled at a CVSE mask, on one B200 through libvsparse_b200.
//
// Same positional command line and stdout lines as the reference driver (sddmm_benchmark.cpp:392-435):
//     ./sddmm_benchmark [bm] [k] [v] [kernel] [alg] [sort] [function] [sparse] [mixed]
// It calls sddmm::wmmaSddmm / sddmm::cudaSddmm through include/vsparse_compat.h exactly as the reference
// driver does (sddmm_benchmark.cpp:255-262).
#include "driver_common.h"
#include "vsparse_compat.h"

template <typename InType, typename OutType>
void BmFN(const std::string &benchmark, int dimK, int vec_length, int kernel, int alg, bool sorted, bool func) {
    HostCvse a = load_benchmark(benchmark, vec_length, sorted);
    const int m_vec = a.m_vec, n = a.n, k = dimK;
    const int m = m_vec * vec_length;
    const size_t nonzeros = (size_t)a.nnz_vec * vec_length;
    printf("Problem size: M: %d, N: %d, nnz: %zu, K: %d\n", m, n, nonzeros, k);

    std::vector<InType> lhs((size_t)m * k + 1), rhs((size_t)n * k + 1);
    check_vs(vs_fill_random(Elem<InType>::kDtype, 0, 1, 1.0, (int64_t)m * k, lhs.data()), "vs_fill_random");
    check_vs(vs_fill_random(Elem<InType>::kDtype, 0, 2, 1.0, (int64_t)n * k, rhs.data()), "vs_fill_random");

    std::vector<float> host32;
    std::vector<double> host64;
    if (func) {  // one dot product per mask entry and element of the vector, fp32 accumulator (and a double one)
        host32.assign(nonzeros, 0.f);
        host64.assign(nonzeros, 0.0);
        for (int i = 0; i < m_vec; ++i)
            for (int j = a.row_offsets[i]; j < a.row_offsets[i + 1]; ++j)
                for (int v = 0; v < vec_length; ++v) {
                    float acc = 0.f;
                    double acc64 = 0.0;
                    const InType *pa = &lhs[((size_t)i * vec_length + v) * k];
                    const InType *pb = &rhs[(size_t)a.col_indices[j] * k];
                    for (int l = 0; l < k; ++l) {
                        const float x = Elem<InType>::to_float(pa[l]), y = Elem<InType>::to_float(pb[l]);
                        acc += x * y;
                        acc64 += (double)x * (double)y;
                    }
                    host32[(size_t)j * vec_length + v] = acc;
                    host64[(size_t)j * vec_length + v] = acc64;
                }
    }

    int *d_row_offsets = to_device(a.row_offsets, (size_t)m_vec + 1);
    int *d_col_indices = to_device(a.col_indices, (size_t)a.nnz_vec);
    int *d_row_indices = to_device(a.row_indices, (size_t)m_vec);
    InType *d_lhs_matrix = to_device(lhs, (size_t)m * k);
    InType *d_rhs_matrix = to_device(rhs, (size_t)n * k);
    OutType *d_output_value = nullptr;
    check_cuda(cudaMalloc(&d_output_value, (nonzeros + 1) * sizeof(OutType)), "cudaMalloc");

    cudaEvent_t t0, t1;
    check_cuda(cudaEventCreate(&t0), "event");
    check_cuda(cudaEventCreate(&t1), "event");
    cudaProfilerStart();
    check_cuda(cudaEventRecord(t0), "event");
    cudaError_t launched = cudaSuccess;
    if (kernel == 0) {
        printf("Using WMMA \n");
        launched = sddmm::wmmaSddmm(m_vec, k, n, a.nnz_vec, d_row_indices, d_row_offsets, d_col_indices, d_lhs_matrix, d_rhs_matrix, d_output_value, vec_length, 0, alg);
    } else if (kernel == 1) {
        printf("Using CUDA \n");
        launched = sddmm::cudaSddmm(m_vec, k, n, a.nnz_vec, d_row_indices, d_row_offsets, d_col_indices, d_lhs_matrix, d_rhs_matrix, d_output_value, vec_length, 0);
    } else if (kernel == 2 || kernel == 3) {
        printf("%s is a third-party baseline of the reference and is not built here.\n", kernel == 2 ? "Sputnik" : "cuSPARSE");
    } else {
        printf("unsupported kernel\n");
    }
    check_cuda(cudaEventRecord(t1), "event");
    cudaProfilerStop();
    check_cuda(launched, "kernel launch");
    check_cuda(cudaDeviceSynchronize(), "kernel execution");
    float ms = 0;
    check_cuda(cudaEventElapsedTime(&ms, t0, t1), "event");
    if (kernel == 0 || kernel == 1) printf("first launch %.3f ms\n", ms);

    if (func && (kernel == 0 || kernel == 1)) {
        std::vector<OutType> out(nonzeros + 1);
        check_cuda(cudaMemcpy(out.data(), d_output_value, nonzeros * sizeof(OutType), cudaMemcpyDeviceToHost), "cudaMemcpy");
        std::vector<float> dev(nonzeros);
        for (size_t j = 0; j < nonzeros; ++j) dev[j] = Elem<OutType>::to_float(out[j]);
        report("SDDMM", nonzeros, dev, host32, host64);
    }
    cudaFree(d_row_offsets); cudaFree(d_col_indices); cudaFree(d_row_indices);
    cudaFree(d_lhs_matrix); cudaFree(d_rhs_matrix); cudaFree(d_output_value);
}

int main(int argc, char **argv) {
    if (argc != 10 || !strcmp(argv[1], "-h") || !strcmp(argv[1], "--help")) {
        printf("This program does a D_mxn = A_mxk * B_nxk^T o C_mxn sampled matrix multiplication.\n");
        printf("C_mxn is a column-vector sparse mask whose pattern comes from the benchmark [bm]; A and B are row-major dense.\n\n");
        printf("usage: ./sddmm_benchmark [bm] [k] [v] [kernel] [alg] [sort] [function] [sparse] [mixed]\n");
        printf("bm      :   path to a .smtx pattern, or synthetic:<fixed|beta|uniform|band>:<m_vec>x<n>:s=<sparsity>[:seed=<n>][:band=<cols>]\n");
        printf("k       :   the length of the contraction.\n");
        printf("v       :   the vector length, one of {1, 2, 4, 8}.\n");
        printf("kernel  :   0 = tensor-core SDDMM (v = 2, 4, 8); 1 = CUDA-core SDDMM (v = 1, 2, 4, 8); 2, 3 not built.\n");
        printf("alg     :   0..3, kept for command-line compatibility: all select the same tensor-core kernel.\n");
        printf("sort    :   1 = vector rows are scheduled longest first; 0 = in order.\n");
        printf("function:   1 = verify against a sequential host result; 0 = skip.\n");
        printf("sparse  :   1 = SDDMM. 0 (dense cuBLAS) is not built.\n");
        printf("mixed   :   1 = half precision. 0 = single precision, which neither SDDMM family supports.\n");
        return (argc == 2 || argc == 10) ? 0 : 1;
    }
    std::string benchmark(argv[1]);
    int dimK = std::atoi(argv[2]), vec_length = std::atoi(argv[3]), kernel = std::atoi(argv[4]), alg = std::atoi(argv[5]);
    int sorted = std::atoi(argv[6]), func = std::atoi(argv[7]), sparse = std::atoi(argv[8]), mixed = std::atoi(argv[9]);
    if (sparse != 1) {
        printf("sparse = %d (dense cuBLAS) is a third-party baseline of the reference and is not built here.\n", sparse);
        return 0;
    }
    if (mixed) BmFN<half, half>(benchmark, dimK, vec_length, kernel, alg, sorted, func);
    else BmFN<float, float>(benchmark, dimK, vec_length, kernel, alg, sorted, func);
    return 0;
}
