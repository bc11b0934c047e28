// spmm_benchmark — A[m x n] (CVSE) * B[n x k] = C[m x k] on one B200 through libvsparse_b200.
//
// Same positional command line and stdout lines as the reference driver (spmm_benchmark.cpp:473-513):
//     ./spmm_benchmark [bm] [k] [v] [kernel] [sort] [function] [sparse] [mixed]
// Built against include/vsparse_compat.h, i.e. it calls spmm::wmmaSpmm / spmm::cudaSpmm exactly as the
// reference driver does (spmm_benchmark.cpp:124-132).  kernel 2 (sputnik), 3 (cuSPARSE) and sparse 0 / 2
// (dense cuBLAS, Blocked-ELL) are third-party baselines of the reference and are not built here.
#include "driver_common.h"
#include "vsparse_compat.h"

template <typename InType, typename OutType>
void BmFN(const std::string &benchmark, int dimK, int vec_length, int kernel, bool sorted, bool func) {
    HostCvse a = load_benchmark(benchmark, vec_length, sorted);
    const int m_vec = a.m_vec, n = a.n, k = dimK;
    const int m = m_vec * vec_length;
    const size_t nonzeros = (size_t)a.nnz_vec * vec_length;

    // operands: uniform(-1, 1), the law of the reference's MakeDenseMatrix
    std::vector<InType> values(nonzeros + 1), rhs((size_t)n * k + 1);
    check_vs(vs_fill_random(Elem<InType>::kDtype, 0, 1, 1.0, (int64_t)n * k, rhs.data()), "vs_fill_random");
    check_vs(vs_fill_random(Elem<InType>::kDtype, 0, 2, 1.0, (int64_t)nonzeros, values.data()), "vs_fill_random");

    std::vector<float> host32;
    std::vector<double> host64;
    if (func) {  // the sequential host product: vector-row, nonzero vector, element of the vector, dense column
        host32.assign((size_t)m * k, 0.f);
        host64.assign((size_t)m * k, 0.0);
        for (int i = 0; i < m_vec; ++i)
            for (int j = a.row_offsets[i]; j < a.row_offsets[i + 1]; ++j) {
                const size_t col = (size_t)a.col_indices[j];
                for (int v = 0; v < vec_length; ++v) {
                    const float av = Elem<InType>::to_float(values[(size_t)j * vec_length + v]);
                    float *o32 = &host32[((size_t)i * vec_length + v) * k];
                    double *o64 = &host64[((size_t)i * vec_length + v) * k];
                    for (int l = 0; l < k; ++l) {
                        const float bv = Elem<InType>::to_float(rhs[col * k + l]);
                        o32[l] += av * bv;
                        o64[l] += (double)av * (double)bv;
                    }
                }
            }
    }

    int *d_row_offsets = to_device(a.row_offsets, (size_t)m_vec + 1);
    int *d_col_indices = to_device(a.col_indices, (size_t)a.nnz_vec);
    int *d_row_indices = to_device(a.row_indices, (size_t)m_vec);
    InType *d_value = to_device(values, nonzeros);
    InType *d_rhs_matrix = to_device(rhs, (size_t)n * k);
    OutType *d_output_value = nullptr;
    check_cuda(cudaMalloc(&d_output_value, ((size_t)m * k + 1) * sizeof(OutType)), "cudaMalloc");

    cudaEvent_t t0, t1;
    check_cuda(cudaEventCreate(&t0), "event");
    check_cuda(cudaEventCreate(&t1), "event");
    cudaProfilerStart();
    check_cuda(cudaEventRecord(t0), "event");
    cudaError_t launched = cudaSuccess;
    if (kernel == 0) {
        printf("Using WMMA \n");
        launched = spmm::wmmaSpmm(m_vec, vec_length, k, n, d_row_indices, d_row_offsets, d_col_indices, d_value, d_rhs_matrix, d_output_value);
    } else if (kernel == 1) {
        printf("Using CUDA \n");
        launched = spmm::cudaSpmm(m_vec, vec_length, k, n, d_row_indices, d_row_offsets, d_col_indices, d_value, d_rhs_matrix, d_output_value);
    } else if (kernel == 2 || kernel == 3) {
        printf("%s is a third-party baseline of the reference and is not built here.\n", kernel == 2 ? "Sputnik" : "cuSPARSE");
    } else {
        printf("Unsupported Kernel \n");
    }
    check_cuda(cudaEventRecord(t1), "event");
    cudaProfilerStop();
    check_cuda(launched, "kernel launch");
    check_cuda(cudaDeviceSynchronize(), "kernel execution");
    float ms = 0;
    check_cuda(cudaEventElapsedTime(&ms, t0, t1), "event");
    if (kernel == 0 || kernel == 1)
        printf("Problem size: M: %d, N: %d, nnz: %zu, K: %d; first launch %.3f ms\n", m, n, nonzeros, k, ms);

    if (func && (kernel == 0 || kernel == 1)) {
        std::vector<OutType> out((size_t)m * k + 1);
        check_cuda(cudaMemcpy(out.data(), d_output_value, (size_t)m * k * sizeof(OutType), cudaMemcpyDeviceToHost), "cudaMemcpy");
        std::vector<float> dev((size_t)m * k);
        for (size_t j = 0; j < dev.size(); ++j) dev[j] = Elem<OutType>::to_float(out[j]);
        report("SPMM", dev.size(), dev, host32, host64);
    }
    cudaFree(d_row_offsets); cudaFree(d_col_indices); cudaFree(d_row_indices);
    cudaFree(d_value); cudaFree(d_rhs_matrix); cudaFree(d_output_value);
}

int main(int argc, char **argv) {
    if (argc != 9 || !strcmp(argv[1], "-h") || !strcmp(argv[1], "--help")) {
        printf("This program does a A_mxn * B_nxk = C_mxk matrix multiplication.\n");
        printf("A_mxn is a column-vector sparse matrix whose pattern comes from the benchmark [bm]; B and C are row-major dense.\n\n");
        printf("usage: ./spmm_benchmark [bm] [k] [v] [kernel] [sort] [function] [sparse] [mixed]\n");
        printf("bm      :   path to a .smtx pattern (its row count is the number of vector rows), or\n");
        printf("            synthetic:<fixed|beta|uniform|band>:<m_vec>x<n>:s=<sparsity>[:seed=<n>][:band=<cols>]\n");
        printf("k       :   the dense width (columns of B and C).\n");
        printf("v       :   the vector length of the column vector sparsity, one of {1, 2, 4, 8}.\n");
        printf("kernel  :   0 = tensor-core SpMM (v = 2, 4, 8); 1 = CUDA-core SpMM (v = 1, 2, 4, 8);\n");
        printf("            2 (sputnik) and 3 (cusparse) are not built.\n");
        printf("sort    :   1 = vector rows are scheduled longest first; 0 = in order.\n");
        printf("function:   1 = verify the result against a sequential host product; 0 = skip.\n");
        printf("sparse  :   1 = SpMM. 0 (dense cuBLAS) and 2 (Blocked-ELL) are not built.\n");
        printf("mixed   :   1 = half precision; 0 = single precision.\n");
        return argc == 9 ? 0 : (argc == 2 ? 0 : 1);
    }
    std::string benchmark(argv[1]);
    int dimK = std::atoi(argv[2]), vec_length = std::atoi(argv[3]), kernel = std::atoi(argv[4]);
    int sorted = std::atoi(argv[5]), func = std::atoi(argv[6]), sparse = std::atoi(argv[7]), mixed = std::atoi(argv[8]);
    if (sparse != 1) {
        printf("sparse = %d (%s) is a third-party baseline of the reference and is not built here.\n", sparse,
               sparse == 0 ? "dense cuBLAS" : "Blocked-ELL");
        return 0;
    }
    if (mixed) BmFN<half, half>(benchmark, dimK, vec_length, kernel, sorted, func);
    else BmFN<float, float>(benchmark, dimK, vec_length, kernel, sorted, func);
    return 0;
}
