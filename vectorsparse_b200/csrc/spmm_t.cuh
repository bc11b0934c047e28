// SpMM with the TRANSPOSE of a column-vector sparse matrix: out[n x N] = A^T . rhs, A being m_vec * V x n in CVSE
// and rhs m_vec * V x N, row-major fp16.  It is the step behind the forward SpMM / SDDMM pair in the backward
// pass of fixed-mask sparse attention (dV = P^T dO, dK = dS^T Q); the reference has no such operator — its
// kernels cover the forward products only (src/wmma_spmm.cu, src/cuda_spmm.cu).
//
// The caller transposes the STRUCTURE once on the host (vs_cvse_transpose): for every column c of A the nonzero
// vectors that name it, as (vector-row i, index j of the vector in the CVSE arrays), ascending in i.  The values
// stay where they are: a nonzero vector (i, c) contributes  sum_v values[j*V+v] * rhs[i*V+v][:]  to row c of the
// output, and its V rows of rhs are adjacent.  No atomics: one warp owns 256 columns of one output row and adds
// its entries in the listed order, fp32 accumulate of exact fp16 products, so results are reproducible.
//
// Bound: every nonzero vector pulls V rows of rhs (V * N * 2 bytes) through L2 -> shared/registers, V times the
// gather traffic of the forward product, with no reuse between output rows; HBM traffic is the operands once
// (rhs of one batch entry stays in L2 while its output rows are produced).
#pragma once

#include <cuda_fp16.h>
#include <cstdint>

#include "common.cuh"

namespace vs {
namespace spmmt {

struct Params {
    int n;          // columns of A = rows of the output
    int N;          // dense width
    int batch;
    const int32_t *t_offsets;   // [n + 1]
    const int32_t *t_rows;      // [nnz_vec] vector-row of each entry
    const int32_t *t_src;       // [nnz_vec] index of the entry's vector in `values` (in vectors)
    const __half *values;
    const __half *rhs;
    void *out;
    int64_t stride_values, stride_rhs, stride_out;   // in elements
};

constexpr int kWarps = 4;
constexpr int kThreads = 32 * kWarps;
constexpr int kChunk = 256;   // output columns per warp: 8 per lane
constexpr int kAhead = 2;     // entries whose loads are issued together

template <int V> struct Vals { __half v[V]; };
template <int V> __device__ __forceinline__ Vals<V> load_vals(const __half *p);
template <> __device__ __forceinline__ Vals<8> load_vals<8>(const __half *p) {
    Vals<8> r; *reinterpret_cast<uint4 *>(r.v) = __ldg(reinterpret_cast<const uint4 *>(p)); return r;
}
template <> __device__ __forceinline__ Vals<4> load_vals<4>(const __half *p) {
    Vals<4> r; *reinterpret_cast<uint2 *>(r.v) = __ldg(reinterpret_cast<const uint2 *>(p)); return r;
}
template <> __device__ __forceinline__ Vals<2> load_vals<2>(const __half *p) {
    Vals<2> r; *reinterpret_cast<uint32_t *>(r.v) = __ldg(reinterpret_cast<const uint32_t *>(p)); return r;
}
template <> __device__ __forceinline__ Vals<1> load_vals<1>(const __half *p) {
    Vals<1> r; r.v[0] = __ldg(p); return r;
}

__device__ __forceinline__ void fma8(float (&acc)[8], float a, const uint4 &b) {
    const __half2 *h = reinterpret_cast<const __half2 *>(&b);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float2 f = __half22float2(h[q]);
        acc[2 * q] = fmaf(a, f.x, acc[2 * q]);
        acc[2 * q + 1] = fmaf(a, f.y, acc[2 * q + 1]);
    }
}

__device__ __forceinline__ void store8(__half *dst, const float (&acc)[8]) {
    uint4 o;
    __half2 *h = reinterpret_cast<__half2 *>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) h[q] = __floats2half2_rn(acc[2 * q], acc[2 * q + 1]);
    *reinterpret_cast<uint4 *>(dst) = o;
}
__device__ __forceinline__ void store8(float *dst, const float (&acc)[8]) {
    *reinterpret_cast<float4 *>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4 *>(dst + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
}

// Work item = (batch entry, 256-column chunk, group of kWarps output rows); items are walked grid-stride so that
// a launch never needs more CTAs than fit the machine a few times over.
template <typename TOut, int V>
__global__ void __launch_bounds__(kThreads) spmm_t_kernel(const Params p, int64_t items, int row_groups, int chunks,
                                                          const int32_t *plan_hdr, int plan_checks) {
    // Enqueued behind the tensor-core kernel (plan_hdr != null): wait for its end, then leave unless it handed the
    // call over (a matrix it cannot hold, or a non-finite sum it would not vouch for).
    pdl_launch_dependents();   // the next call's plan kernel may queue up behind this one
    pdl_wait();
    if (plan_hdr && plan_dense_chosen(plan_hdr, plan_checks)) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int64_t w = blockIdx.x; w < items; w += gridDim.x) {
        const int rg = (int)(w % row_groups);
        const int64_t rest = w / row_groups;
        const int chunk = (int)(rest % chunks);
        const int b = (int)(rest / chunks);
        const int c = rg * kWarps + warp;
        const int col = chunk * kChunk + lane * 8;
        if (c >= p.n) continue;   // warp-uniform
        const bool live = col < p.N;   // N is a multiple of 8: a lane holds eight columns or none
        const __half *vals = p.values + (int64_t)b * p.stride_values;
        const __half *rhs = p.rhs + (int64_t)b * p.stride_rhs + col;
        float acc[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] = 0.0f;
        const int e0 = __ldg(p.t_offsets + c), e1 = __ldg(p.t_offsets + c + 1);
        for (int base = e0; base < e1; base += 32) {
            // 32 entries' indices in one coalesced load, handed round by shuffles
            const int mine = base + lane;
            const int my_row = mine < e1 ? __ldg(p.t_rows + mine) : 0;
            const int my_src = mine < e1 ? __ldg(p.t_src + mine) : 0;
            const int count = min(32, e1 - base);
            for (int t = 0; t < count; t += kAhead) {
                Vals<V> a[kAhead];
                uint4 bv[kAhead][V];
#pragma unroll
                for (int u = 0; u < kAhead; ++u) {
                    const int src_lane = min(t + u, count - 1);
                    const int i = __shfl_sync(0xffffffffu, my_row, src_lane);
                    const int j = __shfl_sync(0xffffffffu, my_src, src_lane);
                    a[u] = load_vals<V>(vals + (int64_t)j * V);
                    if (live) {
#pragma unroll
                        for (int v = 0; v < V; ++v)
                            bv[u][v] = __ldg(reinterpret_cast<const uint4 *>(rhs + ((int64_t)i * V + v) * p.N));
                    }
                }
                if (live) {
#pragma unroll
                    for (int u = 0; u < kAhead; ++u) {
                        if (t + u >= count) break;   // warp-uniform: the clamped repeat of the last entry is not added
#pragma unroll
                        for (int v = 0; v < V; ++v) fma8(acc, __half2float(a[u].v[v]), bv[u][v]);
                    }
                }
            }
        }
        if (live) store8(reinterpret_cast<TOut *>(p.out) + (int64_t)b * p.stride_out + (int64_t)c * p.N + col, acc);
    }
}

}  // namespace spmmt
}  // namespace vs
