// CUDA-core kernels: SpMM and SDDMM for V = 1/2/4/8 in fp32 or fp16 (fp32 accumulate), and the masked row
// softmax.  These are the `cudaSpmm` / `cudaSddmm` family of the reference (src/cuda_spmm.cu,
// src/cuda_sddmm.cu) including the fp32 SpMM the reference leaves as a stub (src/cuda_spmm.cu:328-338).
//
// Design: no shared memory and no intra-CTA cooperation.  Each thread (SpMM) or 8-lane group (SDDMM) owns an
// independent piece of output, dense operands are read with 16-byte loads that coalesce across neighbouring
// threads, and the per-nonzero index / value-vector loads are warp-uniform broadcasts served by L1.
#pragma once
#include "common.cuh"

namespace vs {

constexpr int kCcThreads = 128;

// ---- SpMM ---------------------------------------------------------------------------------------------------
// Work item = (vector-row in row_indices order, 16-byte chunk of the dense width).  The thread keeps V x E
// fp32 accumulators (E = elements per 16 bytes) and walks the row's nonzero vectors four at a time so that
// four independent gathers of B are in flight.
template <typename TIn, typename TOut, int V>
__global__ void __launch_bounds__(kCcThreads) spmm_cc_kernel(const SpmmParams p) {
    constexpr int E = Chunk<TIn>::kElems;
    constexpr int U = 4;
    const int chunks = p.N / E;
    const int64_t item = (int64_t)blockIdx.x * kCcThreads + threadIdx.x;
    if (item >= (int64_t)p.m_vec * chunks) return;
    const int order = (int)(item / chunks);
    const int chunk = (int)(item - (int64_t)order * chunks);
    const int row = __ldg(p.row_indices + order);
    const int b = blockIdx.y;

    const TIn *values = static_cast<const TIn *>(p.values) + (int64_t)b * p.stride_values;
    const TIn *rhs = static_cast<const TIn *>(p.rhs) + (int64_t)b * p.stride_rhs + (int64_t)chunk * E;
    TOut *out = static_cast<TOut *>(p.out) + (int64_t)b * p.stride_out + (int64_t)chunk * E;

    float acc[V][E];
#pragma unroll
    for (int v = 0; v < V; ++v)
#pragma unroll
        for (int e = 0; e < E; ++e) acc[v][e] = 0.f;

    int j = __ldg(p.row_offsets + row);
    const int end = __ldg(p.row_offsets + row + 1);

    for (; j + U <= end; j += U) {
        int col[U];
        float a[U][V];
        Chunk<TIn> bt[U];
#pragma unroll
        for (int u = 0; u < U; ++u) col[u] = __ldg(p.col_indices + j + u);
#pragma unroll
        for (int u = 0; u < U; ++u) bt[u].load(rhs + (int64_t)col[u] * p.N);
#pragma unroll
        for (int u = 0; u < U; ++u) VecLoad<TIn, V>::load(values + (int64_t)(j + u) * V, a[u]);
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int v = 0; v < V; ++v)
#pragma unroll
                for (int e = 0; e < E; ++e) acc[v][e] = fmaf(a[u][v], bt[u].f[e], acc[v][e]);
    }
    for (; j < end; ++j) {
        const int col = __ldg(p.col_indices + j);
        float a[V];
        Chunk<TIn> bt;
        bt.load(rhs + (int64_t)col * p.N);
        VecLoad<TIn, V>::load(values + (int64_t)j * V, a);
#pragma unroll
        for (int v = 0; v < V; ++v)
#pragma unroll
            for (int e = 0; e < E; ++e) acc[v][e] = fmaf(a[v], bt.f[e], acc[v][e]);
    }

#pragma unroll
    for (int v = 0; v < V; ++v) store_chunk(out + ((int64_t)row * V + v) * p.N, acc[v]);
}

// ---- SDDMM --------------------------------------------------------------------------------------------------
// Eight lanes share one mask entry j: lane g takes the 16-byte chunks g, g+8, ... of the contraction, keeps V
// partial sums (one per real row of the vector), and the eight partials are folded with three xor-shuffles.
// The vector-row of entry j is found by bisection in row_offsets, so the grid is exactly nnz_vec entries and
// no thread block is launched for empty parts of the mask.
template <typename TIn, typename TOut, int V>
__global__ void __launch_bounds__(kCcThreads) sddmm_cc_kernel(const SddmmParams p) {
    constexpr int E = Chunk<TIn>::kElems;
    constexpr int L = 8;
    const int g = threadIdx.x & (L - 1);
    const int64_t entry = ((int64_t)blockIdx.x * kCcThreads + threadIdx.x) / L;
    const bool valid = entry < p.nnz_vec;
    const int j = valid ? (int)entry : 0;
    const int b = blockIdx.y;

    int lo = 0, hi = p.m_vec;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(p.row_offsets + mid) <= j) lo = mid; else hi = mid;
    }
    const int i = lo;
    const int col = __ldg(p.col_indices + j);

    const TIn *lhs = static_cast<const TIn *>(p.lhs) + (int64_t)b * p.stride_lhs + (int64_t)i * V * p.k;
    const TIn *rhs = static_cast<const TIn *>(p.rhs) + (int64_t)b * p.stride_rhs + (int64_t)col * p.k;
    TOut *out = static_cast<TOut *>(p.out) + (int64_t)b * p.stride_out + (int64_t)j * V;

    float acc[V];
#pragma unroll
    for (int v = 0; v < V; ++v) acc[v] = 0.f;

    const int chunks = p.k / E;
    for (int c = g; c < chunks; c += L) {
        Chunk<TIn> r;
        r.load(rhs + c * E);
#pragma unroll
        for (int v = 0; v < V; ++v) {
            Chunk<TIn> l;
            l.load(lhs + (int64_t)v * p.k + c * E);
#pragma unroll
            for (int e = 0; e < E; ++e) acc[v] = fmaf(l.f[e], r.f[e], acc[v]);
        }
    }
#pragma unroll
    for (int off = L / 2; off > 0; off >>= 1)
#pragma unroll
        for (int v = 0; v < V; ++v) acc[v] += __shfl_xor_sync(0xffffffffu, acc[v], off);

    if (valid && g == 0) {
        if constexpr (V >= 4) {
            store_chunk(out, acc);
        } else {
#pragma unroll
            for (int v = 0; v < V; ++v) store_scalar(out + v, acc[v]);
        }
    }
}

// ---- masked row softmax -----------------------------------------------------------------------------------
// One warp per vector-row: lanes stride over the row's entries, each entry carrying the V real rows, so the V
// softmaxes of a vector-row run side by side on contiguous loads.  fp32 arithmetic, three passes over a row
// that stays in L1/L2.  probs may alias scores.
template <typename T, int V>
__global__ void __launch_bounds__(kCcThreads) softmax_cvse_kernel(const SoftmaxParams p) {
    const int warp = (blockIdx.x * kCcThreads + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= p.m_vec) return;
    const int b = blockIdx.y;
    const T *s = static_cast<const T *>(p.scores) + (int64_t)b * p.stride;
    T *o = static_cast<T *>(p.probs) + (int64_t)b * p.stride;
    const int beg = __ldg(p.row_offsets + warp), end = __ldg(p.row_offsets + warp + 1);
    if (beg == end) return;

    float mx[V], sum[V];
#pragma unroll
    for (int v = 0; v < V; ++v) { mx[v] = -INFINITY; sum[v] = 0.f; }
    for (int j = beg + lane; j < end; j += 32) {
#pragma unroll
        for (int v = 0; v < V; ++v) mx[v] = fmaxf(mx[v], p.scale * load_scalar(s + (int64_t)j * V + v));
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
#pragma unroll
        for (int v = 0; v < V; ++v) mx[v] = fmaxf(mx[v], __shfl_xor_sync(0xffffffffu, mx[v], off));
    for (int j = beg + lane; j < end; j += 32) {
#pragma unroll
        for (int v = 0; v < V; ++v) sum[v] += expf(p.scale * load_scalar(s + (int64_t)j * V + v) - mx[v]);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
#pragma unroll
        for (int v = 0; v < V; ++v) sum[v] += __shfl_xor_sync(0xffffffffu, sum[v], off);
    for (int j = beg + lane; j < end; j += 32) {
#pragma unroll
        for (int v = 0; v < V; ++v) {
            const float x = expf(p.scale * load_scalar(s + (int64_t)j * V + v) - mx[v]) / sum[v];
            store_scalar(o + (int64_t)j * V + v, x);
        }
    }
}

}  // namespace vs
