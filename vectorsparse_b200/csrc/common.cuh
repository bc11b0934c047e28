// Shared device helpers and launch parameter blocks for the CVSE kernels.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace vs {

// One SpMM problem, or `batch` of them sharing the structure arrays.
struct SpmmParams {
    int m_vec;       // vector-rows
    int N;           // dense width (reference argument `k`)
    int K;           // columns of the sparse matrix (reference argument `n`)
    int batch;
    const int32_t *row_indices;
    const int32_t *row_offsets;
    const int32_t *col_indices;
    const void *values;
    const void *rhs;
    void *out;
    int64_t stride_values, stride_rhs, stride_out;  // in elements
};

// Programmatic dependent launch (a kernel launched with cudaLaunchAttributeProgrammaticStreamSerialization may
// start before the kernel ahead of it in the stream has finished).  pdl_launch_dependents(): "the kernel behind
// me may be scheduled now" — its CTAs become resident as room appears and run their set-up.  pdl_wait(): blocks
// until the kernel ahead has COMPLETED and its writes are visible; everything that reads what that kernel (or
// anything before it) wrote comes after this call.  Both are no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Header of the plan scratch of the densifying SpMM, read by the kernels enqueued behind the plan kernel:
// word 0 = the plan kernel chose the dense kernel; words 4 .. 4 + checks = one verdict per duplicate-checking CTA
// of the plan kernel, set when it met the same column twice in one vector-row (the dense tile would keep one of
// the two values, the reference adds them: such matrices go to the gather kernel).  Block-uniform result; every
// thread of the block must call it.  The early way out ahead of the barrier is deliberate (word 0 is the same for
// every thread): with the barrier reached on every path the multiplying kernel came out 14 % slower at 50 %
// sparsity, for the same instructions.
__device__ __forceinline__ bool plan_dense_chosen(const int32_t *hdr, int checks) {
    if (*reinterpret_cast<const volatile int32_t *>(hdr) == 0) return false;
    int dup = 0;
    for (int i = threadIdx.x; i < checks; i += blockDim.x) dup |= hdr[4 + i];
    return __syncthreads_or(dup) == 0;
}

struct SddmmParams {
    int m_vec;
    int k;           // contraction length
    int n;           // columns of the mask
    int nnz_vec;
    int batch;
    const int32_t *row_indices;
    const int32_t *row_offsets;
    const int32_t *col_indices;
    const void *lhs;
    const void *rhs;
    void *out;
    int64_t stride_lhs, stride_rhs, stride_out;  // in elements
};

struct SoftmaxParams {
    int m_vec;
    int batch;
    const int32_t *row_offsets;
    const void *scores;
    void *probs;
    int64_t stride;  // in elements
    float scale;
};

// ---- 16-byte chunks as fp32 lanes ------------------------------------------------------------------------

template <typename T> struct Chunk;  // one 16-byte global load worth of T, widened to float

template <> struct Chunk<float> {
    static constexpr int kElems = 4;
    float f[4];
    __device__ __forceinline__ void load(const float *p) {
        float4 v = __ldg(reinterpret_cast<const float4 *>(p));
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
};

template <> struct Chunk<__half> {
    static constexpr int kElems = 8;
    float f[8];
    __device__ __forceinline__ void load(const __half *p) {
        uint4 v = __ldg(reinterpret_cast<const uint4 *>(p));
        const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 t = __half22float2(h[i]);
            f[2 * i] = t.x;
            f[2 * i + 1] = t.y;
        }
    }
};

// Loads the V values of one nonzero vector (V * sizeof(T) bytes, naturally aligned) widened to float.
template <typename T, int V> struct VecLoad;

template <int V> struct VecLoad<float, V> {
    __device__ __forceinline__ static void load(const float *p, float (&a)[V]) {
        if constexpr (V == 1) {
            a[0] = __ldg(p);
        } else if constexpr (V == 2) {
            float2 t = __ldg(reinterpret_cast<const float2 *>(p));
            a[0] = t.x; a[1] = t.y;
        } else {
#pragma unroll
            for (int q = 0; q < V / 4; ++q) {
                float4 t = __ldg(reinterpret_cast<const float4 *>(p) + q);
                a[4 * q] = t.x; a[4 * q + 1] = t.y; a[4 * q + 2] = t.z; a[4 * q + 3] = t.w;
            }
        }
    }
};

template <int V> struct VecLoad<__half, V> {
    __device__ __forceinline__ static void load(const __half *p, float (&a)[V]) {
        if constexpr (V == 1) {
            a[0] = __half2float(__ldg(p));
        } else if constexpr (V == 2) {
            float2 t = __half22float2(__ldg(reinterpret_cast<const __half2 *>(p)));
            a[0] = t.x; a[1] = t.y;
        } else if constexpr (V == 4) {
            uint2 r = __ldg(reinterpret_cast<const uint2 *>(p));
            const __half2 *h = reinterpret_cast<const __half2 *>(&r);
            float2 t0 = __half22float2(h[0]), t1 = __half22float2(h[1]);
            a[0] = t0.x; a[1] = t0.y; a[2] = t1.x; a[3] = t1.y;
        } else {
            uint4 r = __ldg(reinterpret_cast<const uint4 *>(p));
            const __half2 *h = reinterpret_cast<const __half2 *>(&r);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float2 t = __half22float2(h[i]);
                a[2 * i] = t.x; a[2 * i + 1] = t.y;
            }
        }
    }
};

// Stores kElems consecutive outputs from float lanes.
__device__ __forceinline__ void store_chunk(float *p, const float (&f)[4]) {
    *reinterpret_cast<float4 *>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
__device__ __forceinline__ void store_chunk(float *p, const float (&f)[8]) {
    reinterpret_cast<float4 *>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
    reinterpret_cast<float4 *>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
}
__device__ __forceinline__ void store_chunk(__half *p, const float (&f)[8]) {
    uint4 v;
    __half2 *h = reinterpret_cast<__half2 *>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4 *>(p) = v;
}
__device__ __forceinline__ void store_chunk(__half *p, const float (&f)[4]) {
    uint2 v;
    __half2 *h = reinterpret_cast<__half2 *>(&v);
    h[0] = __floats2half2_rn(f[0], f[1]);
    h[1] = __floats2half2_rn(f[2], f[3]);
    *reinterpret_cast<uint2 *>(p) = v;
}

__device__ __forceinline__ void store_scalar(float *p, float x) { *p = x; }
__device__ __forceinline__ void store_scalar(__half *p, float x) { *p = __float2half_rn(x); }
__device__ __forceinline__ float load_scalar(const float *p) { return *p; }
__device__ __forceinline__ float load_scalar(const __half *p) { return __half2float(*p); }

}  // namespace vs
