// extern "C" entry points of libvsparse_b200: argument validation and kernel dispatch.
//
// Each operator entry point checks its arguments on the host, picks the template instantiation for
// (path, element types, vector length) and enqueues the kernel(s) on the caller's stream.  Nothing here
// synchronises; the *_host convenience forms allocate and say so, and the tensor-core SpMM keeps one plan
// scratch buffer per calling stream, taken from the stream-ordered allocator the first time (and when a larger
// matrix needs a larger one).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <algorithm>
#include <cstring>
#include <cmath>
#include <mutex>
#include <thread>
#include <functional>
#include <unordered_map>
#include <utility>
#include <vector>

#include "vsparse_b200.h"
#include "common.cuh"
#include "cuda_core.cuh"
#include "spmm_tc.cuh"
#include "spmm_tma.cuh"
#include "spmm_dense.cuh"
#include "sddmm_pair.cuh"
#include "spmm_pair.cuh"
#include "spmm_t.cuh"
#include "sddmm_tc.cuh"
#include "sddmm_tma.cuh"
#include "sddmm_dense.cuh"
#include "tc_selftest.cuh"

#define VS_EXPORT extern "C" __attribute__((visibility("default")))
#define VS_CUDA_TRY(expr)                      \
    do {                                       \
        cudaError_t e__ = (expr);              \
        if (e__ != cudaSuccess) return (int)e__; \
    } while (0)

namespace {

using namespace vs;

// Per-device status word, OR-ed into by kernels whose bounded waits ran out.
__device__ uint32_t g_device_status = 0;

constexpr int kMaxDevices = 64;
struct Scratch {
    void *ptr = nullptr;
    size_t bytes = 0;
};
struct DeviceInfo {
    bool ready = false;
    int sm_count = 0;
    uint32_t *status = nullptr;
    // Plan scratch of the densifying SpMM, one buffer per stream that has called it: calls on one stream run
    // in order, so they can share a buffer; calls on different streams cannot.  cudaStreamPerThread is one handle
    // value that names a different stream in every host thread, so there the calling thread is part of the key.
    struct Key {
        cudaStream_t stream;
        std::thread::id thread;
        bool operator==(const Key &o) const { return stream == o.stream && thread == o.thread; }
    };
    struct KeyHash {
        size_t operator()(const Key &k) const {
            return std::hash<const void *>()(static_cast<const void *>(k.stream)) ^ (std::hash<std::thread::id>()(k.thread) * 0x9e3779b97f4a7c15ull);
        }
    };
    std::unordered_map<Key, Scratch, KeyHash> scratch;
    static Key key_of(cudaStream_t s) { return Key{s, s == cudaStreamPerThread ? std::this_thread::get_id() : std::thread::id()}; }
};
DeviceInfo g_devices[kMaxDevices];
std::mutex g_devices_mutex;

int device_info(DeviceInfo **out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return VS_ERR_ARG;
    std::lock_guard<std::mutex> lock(g_devices_mutex);
    DeviceInfo &d = g_devices[dev];
    if (!d.ready) {
        e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return (int)e;
        e = cudaGetSymbolAddress(reinterpret_cast<void **>(&d.status), g_device_status);
        if (e != cudaSuccess) return (int)e;
        d.ready = true;
    }
    *out = &d;
    return VS_OK;
}

// Set for the duration of an entry point that promises not to allocate: the tensor-core formulations that need
// plan scratch are skipped on this thread, the gather kernels (which need none) take the call.
thread_local bool t_no_scratch = false;
struct NoScratchScope {
    bool saved;
    NoScratchScope() : saved(t_no_scratch) { t_no_scratch = true; }
    ~NoScratchScope() { t_no_scratch = saved; }
};

// A workspace handed over by the caller (vs_set_workspace) for the calls of this host thread.
thread_local bool t_ws_set = false;
thread_local void *t_ws_ptr = nullptr;
thread_local int64_t t_ws_bytes = 0;

// Scratch of at least `bytes` for work enqueued on `stream`.  Grows by stream-ordered allocation (the old buffer
// is released behind the work already enqueued); in the steady state this makes no CUDA call.  Buffers live
// until vs_release_scratch or the end of the process.
int stream_scratch(DeviceInfo *d, cudaStream_t stream, size_t bytes, void **out) {
    if (t_ws_set) {   // the caller's buffer or nothing: never allocate behind a caller that manages memory itself
        if ((int64_t)bytes > t_ws_bytes) return VS_ERR_SHAPE;
        *out = t_ws_ptr;
        return VS_OK;
    }
    std::lock_guard<std::mutex> lock(g_devices_mutex);
    Scratch &sc = d->scratch[DeviceInfo::key_of(stream)];
    if (sc.bytes < bytes) {
        size_t want = 1u << 20;
        while (want < bytes) want <<= 1;
        void *fresh = nullptr;
        cudaError_t e = cudaMallocAsync(&fresh, want, stream);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            return (int)e;
        }
        if (sc.ptr) (void)cudaFreeAsync(sc.ptr, stream);
        sc.ptr = fresh;
        sc.bytes = want;
    }
    *out = sc.ptr;
    return VS_OK;
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool valid_v(int v) { return v == 1 || v == 2 || v == 4 || v == 8; }
inline int elem_size(int dtype) { return dtype == VS_F16 ? 2 : 4; }
inline bool stride_ok(int64_t stride, int dtype) { return stride >= 0 && (stride * elem_size(dtype)) % 16 == 0; }

template <typename K> int set_smem(K kernel, int bytes) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    return e == cudaSuccess ? VS_OK : (int)e;
}

// Launches `kernel` so that it may start while the kernel ahead of it in the stream is still running (programmatic
// dependent launch); such a kernel calls pdl_wait() before it reads anything written earlier in the stream.
// VSPARSE_B200_PDL=0 launches the ordinary way.
template <typename... Exp, typename... Act>
cudaError_t launch_overlapped(void (*kernel)(Exp...), unsigned grid, unsigned block, size_t smem, cudaStream_t s, Act &&...args) {
    static const bool overlap = []() {
        const char *e = std::getenv("VSPARSE_B200_PDL");
        return !(e && !std::strcmp(e, "0"));
    }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Act>(args)...);
}

// Launches `pairs` clusters of two CTAs (tcgen05 cta_group::2 kernels), optionally as a programmatic dependent.
template <typename... Exp, typename... Act>
cudaError_t launch_pairs(void (*kernel)(Exp...), unsigned pairs, unsigned block, size_t smem, cudaStream_t s, bool overlapped,
                         Act &&...args) {
    static const bool overlap = []() {
        const char *e = std::getenv("VSPARSE_B200_PDL");
        return !(e && !std::strcmp(e, "0"));
    }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (overlapped && overlap) ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Act>(args)...);
}

// Diagnostic: CUDA events around the multiplying kernels of the dense tensor-core paths (vs_kernel_timing).  Off by
// default; while on, every such kernel is bracketed by two events on its stream, which also keeps it from
// overlapping the kernels before and behind it (it is timed alone, as a profiler's launch list shows it).
struct KernelTiming {
    std::mutex lock;
    bool on = false;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> pairs;
};
KernelTiming &kernel_timing() {
    static KernelTiming t;
    return t;
}
struct TimedLaunch {   // records the opening event on construction, the closing one on destruction
    cudaStream_t s;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    explicit TimedLaunch(cudaStream_t stream) : s(stream) {
        KernelTiming &t = kernel_timing();
        std::lock_guard<std::mutex> g(t.lock);
        if (!t.on) return;
        if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) { e0 = e1 = nullptr; (void)cudaGetLastError(); return; }
        cudaEventRecord(e0, s);
    }
    ~TimedLaunch() {
        if (!e0) return;
        cudaEventRecord(e1, s);
        KernelTiming &t = kernel_timing();
        std::lock_guard<std::mutex> g(t.lock);
        t.pairs.emplace_back(e0, e1);
    }
};

// cuTensorMapEncodeTiled, fetched from the driver at first use (the library does not link libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
        return q == cudaDriverEntryPointSuccess ? reinterpret_cast<EncodeTiledFn>(p) : nullptr;
    }();
    return fn;
}

// Tensor map of a row-major fp16 matrix [rows x cols] for row gathers: box = 64 columns x 1 row, 128-byte
// swizzle, zero fill outside the matrix.
int make_gather_map(CUtensorMap *map, const void *ptr, uint64_t rows, uint64_t cols) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return VS_ERR_DEVICE;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {64, 1};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? VS_OK : VS_ERR_ARG;
}

// Tensor map of a batch of row-major matrices, dimensions {cols, rows, batch}, for tile loads / stores of
// box_cols x box_rows elements, swizzled over the bytes of a box row (128 or 64); loads read zeros outside the
// matrix, stores are clipped there.
int make_tile_map(CUtensorMap *map, const void *ptr, bool f32, uint64_t rows, uint64_t cols, uint64_t batch,
                  uint64_t batch_stride, uint32_t box_cols, uint32_t box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return VS_ERR_DEVICE;
    const uint64_t es = f32 ? 4 : 2;
    const cuuint64_t dims[3] = {cols, rows, batch};
    const cuuint64_t strides[2] = {cols * es, (batch > 1 ? batch_stride : rows * cols) * es};
    const cuuint32_t box[3] = {box_cols, box_rows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUtensorMapSwizzle swizzle = box_cols * es == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
    CUresult r = fn(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void *>(ptr), dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? VS_OK : VS_ERR_ARG;
}

// The dense operand of a batch seen as {64 columns, rows, cols / 64 column blocks, batch}: one copy fetches
// 64 rows of `blocks` neighbouring 64-column blocks, each block landing as its own 64 x 128-byte slab.
// cols must be a multiple of 64.
int make_blocked_map(CUtensorMap *map, const void *ptr, uint64_t rows, uint64_t cols, uint64_t batch, uint64_t batch_stride,
                     uint32_t blocks) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return VS_ERR_DEVICE;
    const cuuint64_t dims[4] = {64, rows, cols / 64, batch};
    const cuuint64_t strides[3] = {cols * 2, 128, (batch > 1 ? batch_stride : rows * cols) * 2};
    const cuuint32_t box[4] = {64, 64, blocks, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? VS_OK : VS_ERR_ARG;
}

// ---- SpMM dispatch ----------------------------------------------------------------------------------------
template <typename TIn, typename TOut, int V> int launch_spmm_cc(const SpmmParams &p, cudaStream_t s) {
    constexpr int E = Chunk<TIn>::kElems;
    // several 16-byte chunks per thread where the dense width allows it and the accumulators stay in registers (64 at
    // most); VSPARSE_B200_SPMM_CC_CHUNKS=1|2|4 caps them
    const char *e = std::getenv("VSPARSE_B200_SPMM_CC_CHUNKS");
    const int cap = e ? std::atoi(e) : 4;
    const int want = (V * E <= 16 && cap >= 4 && p.N % (128 * E) == 0) ? 4 : (V * E <= 32 && cap >= 2 && p.N % (64 * E) == 0) ? 2 : 1;
    const int64_t items = (int64_t)p.m_vec * (p.N / E) / want;
    const int64_t blocks = (items + kCcThreads - 1) / kCcThreads;
    if (blocks > 0x7fffffffll) return VS_ERR_SHAPE;
    dim3 grid((unsigned)blocks, (unsigned)p.batch, 1);
    if constexpr (V * E <= 16) {
        if (want == 4) {
            spmm_cc_kernel<TIn, TOut, V, 4><<<grid, kCcThreads, 0, s>>>(p);
            return (int)cudaGetLastError();
        }
    }
    if constexpr (V * E <= 32) {
        if (want == 2) {
            spmm_cc_kernel<TIn, TOut, V, 2><<<grid, kCcThreads, 0, s>>>(p);
            return (int)cudaGetLastError();
        }
    }
    spmm_cc_kernel<TIn, TOut, V, 1><<<grid, kCcThreads, 0, s>>>(p);
    return (int)cudaGetLastError();
}

template <typename TIn, typename TOut> int spmm_cc_by_v(int V, const SpmmParams &p, cudaStream_t s) {
    switch (V) {
        case 1: return launch_spmm_cc<TIn, TOut, 1>(p, s);
        case 2: return launch_spmm_cc<TIn, TOut, 2>(p, s);
        case 4: return launch_spmm_cc<TIn, TOut, 4>(p, s);
        case 8: return launch_spmm_cc<TIn, TOut, 8>(p, s);
    }
    return VS_ERR_VEC_LENGTH;
}

// Software (cp.async) gather: works for any batch stride.
template <typename TOut, int V>
int launch_spmm_tc_cpasync(const SpmmParams &p, cudaStream_t s, DeviceInfo *d, const int32_t *plan_hdr = nullptr, int plan_checks = 0) {
    auto kernel = tcspmm::spmm_tc_kernel<TOut, V>;
    int rc = set_smem(kernel, tcspmm::kSmemBytes);
    if (rc != VS_OK) return rc;
    const int n_tiles = (p.N + tcspmm::kTileN - 1) / tcspmm::kTileN;
    const int64_t items = (int64_t)p.batch * n_tiles * p.m_vec;
    const int64_t cap = (int64_t)tcspmm::kCtasPerSm * d->sm_count;  // persistent CTAs
    const unsigned grid = (unsigned)(items < cap ? items : cap);
    if (plan_hdr) return (int)launch_overlapped(kernel, grid, tcspmm::kThreads, tcspmm::kSmemBytes, s, p, d->status, plan_hdr, plan_checks);
    kernel<<<grid, tcspmm::kThreads, tcspmm::kSmemBytes, s>>>(p, d->status, plan_hdr, plan_checks);
    return (int)cudaGetLastError();
}

// TMA row gather: the dense operand of all batch entries must be addressable as one matrix of N-wide rows,
// i.e. the batch stride is a multiple of N (or zero / a single entry).  With `plan_hdr` the kernel returns at
// once when that plan header says that the densifying kernel has taken the call.
template <typename TOut, int V>
int launch_spmm_gather(const SpmmParams &p, cudaStream_t s, DeviceInfo *d, const int32_t *plan_hdr, int plan_checks) {
    static const bool force_cpasync = []() {
        const char *e = std::getenv("VSPARSE_B200_GATHER");
        return e && !std::strcmp(e, "cpasync");
    }();
    const bool one = p.batch == 1 || p.stride_rhs == 0;
    const int64_t rows_per_batch = one ? 0 : p.stride_rhs / p.N;
    const int64_t total_rows = (one ? 0 : (int64_t)(p.batch - 1) * rows_per_batch) + p.K;
    const bool tma_ok = !force_cpasync && p.K > 0 && (one || p.stride_rhs % p.N == 0) && total_rows < 0x7fffffffll;
    if (!tma_ok) return launch_spmm_tc_cpasync<TOut, V>(p, s, d, plan_hdr, plan_checks);
    CUtensorMap map;
    int rc = make_gather_map(&map, p.rhs, (uint64_t)total_rows, (uint64_t)p.N);
    if (rc != VS_OK) return launch_spmm_tc_cpasync<TOut, V>(p, s, d, plan_hdr, plan_checks);
    auto kernel = tmaspmm::spmm_tma_kernel<TOut, V>;
    rc = set_smem(kernel, tmaspmm::kSmemBytes);
    if (rc != VS_OK) return rc;
    const int n_tiles = (p.N + tmaspmm::kTileN - 1) / tmaspmm::kTileN;
    const int64_t items = (int64_t)p.batch * n_tiles * p.m_vec;
    const int64_t cap = (int64_t)tmaspmm::kCtasPerSm * d->sm_count;  // persistent CTAs
    const unsigned grid = (unsigned)(items < cap ? items : cap);
    if (plan_hdr)
        return (int)launch_overlapped(kernel, grid, tmaspmm::kThreads, tmaspmm::kSmemBytes, s, p, map, (int)rows_per_batch,
                                      (int)total_rows, d->status, plan_hdr, plan_checks);
    kernel<<<grid, tmaspmm::kThreads, tmaspmm::kSmemBytes, s>>>(p, map, (int)rows_per_batch, (int)total_rows, d->status,
                                                                plan_hdr, plan_checks);
    return (int)cudaGetLastError();
}

// Which tensor-core SpMM runs.  The densifying kernel multiplies zero-filled 256 x 64 tiles of A, the gather
// kernels fetch one row of B per nonzero vector: the first costs the same whatever the sparsity, the second is
// proportional to the nonzeros.  The number of nonzeros is only known on the device (the reference signature
// does not pass it), so the choice is made there: the plan kernel compares the two costs (see there) and
// leaves a flag that one of the two kernels, both enqueued, finds set against it and returns at once.  The
// densifying kernel clears the flag again if it produced a non-finite sum, so that the gather kernel redoes the
// call with the reference's semantics for Inf / NaN in rows of B that no nonzero names.
enum class SpmmMode { kAuto, kDense, kGather };
SpmmMode spmm_mode() {   // read at every call, so that a test can switch kernels inside one process
    const char *e = std::getenv("VSPARSE_B200_SPMM");
    if (e && !std::strcmp(e, "dense")) return SpmmMode::kDense;
    if (e && !std::strcmp(e, "gather")) return SpmmMode::kGather;
    return SpmmMode::kAuto;
}
constexpr int64_t kMaxPlanBytes = 512ll << 20;

// Bytes of plan scratch the densifying SpMM needs: the header (verdict + one word per duplicate-checking CTA of
// the plan kernel), the bucket offsets, 8 bytes per possible entry.
inline int spmm_plan_checks(int m_vec) {   // duplicate-checking CTAs: a vector-row per warp, a few rows each at most
    const int want = (m_vec + densespmm::kPlanWarps - 1) / densespmm::kPlanWarps;
    return want < densespmm::kMaxCheckCtas ? want : densespmm::kMaxCheckCtas;
}
inline int64_t spmm_plan_header_bytes(int checks) { return ((int64_t)(4 + checks) * 4 + 15) & ~15ll; }
int64_t spmm_plan_bytes(int m_vec, int V, int K, int batch, int64_t stride_values, int64_t *capacity_out, int64_t *offsets_out) {
    const int k_blocks = (K + densespmm::kBlockK - 1) / densespmm::kBlockK;
    const int m_tiles = (int)(((int64_t)m_vec * V + densespmm::kTileM - 1) / densespmm::kTileM);
    const int groups = m_tiles * (densespmm::kTileM / densespmm::kGroupRows);
    const int plan_blocks = k_blocks * (densespmm::kBlockK / densespmm::kPlanCols);
    // entries are addressed like the nonzero vectors: at most one per (vector-row, column), and never more than
    // fit between two matrices of a batch
    int64_t capacity = (int64_t)m_vec * K;
    if (batch > 1 && stride_values > 0 && stride_values / V < capacity) capacity = stride_values / V;
    const int64_t offsets_bytes = (((int64_t)groups * (plan_blocks + 1) * 4) + 15) & ~15ll;
    if (capacity_out) *capacity_out = capacity;
    if (offsets_out) *offsets_out = offsets_bytes;
    return spmm_plan_header_bytes(spmm_plan_checks(m_vec)) + offsets_bytes + capacity * 8;
}
// The plan of A^T for the transposed product: n rows over m_vec * V columns, one entry per nonzero VECTOR of A.
int64_t spmm_t_plan_bytes(int n, int m_vec, int V, int batch, int64_t stride_values, int64_t *capacity_out, int64_t *offsets_out) {
    const int64_t M = (int64_t)m_vec * V;
    const int k_blocks = (int)((M + densespmm::kBlockK - 1) / densespmm::kBlockK);
    const int m_tiles = (n + densespmm::kTileM - 1) / densespmm::kTileM;
    const int groups = m_tiles * (densespmm::kTileM / densespmm::kGroupRows);
    const int plan_blocks = k_blocks * (densespmm::kBlockK / densespmm::kPlanCols);
    int64_t capacity = (int64_t)n * m_vec;   // at most one vector per (column of A, vector-row)
    if (batch > 1 && stride_values > 0 && stride_values / V < capacity) capacity = stride_values / V;
    const int64_t offsets_bytes = (((int64_t)groups * (plan_blocks + 1) * 4) + 15) & ~15ll;
    if (capacity_out) *capacity_out = capacity;
    if (offsets_out) *offsets_out = offsets_bytes;
    return spmm_plan_header_bytes(spmm_plan_checks(n)) + offsets_bytes + capacity * 8;
}
// The same for the dense SDDMM: per-row chunk offsets and 8 bytes per mask entry.
int64_t sddmm_plan_bytes(int m_vec, int n, int nnz_vec, int64_t *offsets_out) {
    const int chunks = (n + densesddmm::kChunk - 1) / densesddmm::kChunk;
    const int64_t offsets_bytes = (((int64_t)m_vec * (chunks + 1) * 4) + 15) & ~15ll;
    if (offsets_out) *offsets_out = offsets_bytes;
    return offsets_bytes + (int64_t)nnz_vec * 8;
}

// How many pairs of CTAs of `kernel` the device holds at once (one CTA per SM, two neighbouring SMs per pair).
template <typename K> int max_resident_pairs(K kernel, int block, size_t smem, DeviceInfo *d) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (unsigned)d->sm_count);
    cfg.blockDim = dim3((unsigned)block);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
        (void)cudaGetLastError();
        return 0;
    }
    return n;
}

// The densified product by pairs of CTAs (spmm_pair.cuh) takes dense widths that are multiples of 128; the
// single-CTA kernel (spmm_dense.cuh) the other widths.  VSPARSE_B200_SPMM_PAIR=0 keeps every width on the latter.
inline bool spmm_pair_enabled() {
    const char *e = std::getenv("VSPARSE_B200_SPMM_PAIR");
    return !(e && !std::strcmp(e, "0"));
}
// Enqueues the pair kernel for a call whose plan kernel has been enqueued; false if this device cannot hold it.
template <typename TOut, int V, bool kTransposed>
bool launch_spmm_pair(const SpmmParams &q, cudaStream_t s, DeviceInfo *d, const CUtensorMap &map, const CUtensorMap &map_out,
                      const CUtensorMap &map_b2, const int32_t *blk_offsets, const uint2 *blk_entries, int m_tiles, int k_blocks,
                      int32_t *flag, int checks, int *rc_out) {
    static int resident[kMaxDevices];   // 0 = not asked yet, -1 = the kernel cannot run here
    auto kernel = pairspmm::spmm_pair_kernel<TOut, V, kTransposed>;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return false;
    if (resident[dev] == 0) {
        if (set_smem(kernel, pairspmm::kSmemBytes) != VS_OK) {
            resident[dev] = -1;
        } else {
            const int n = max_resident_pairs(kernel, pairspmm::kThreads, pairspmm::kSmemBytes, d);
            resident[dev] = n > 0 ? n : -1;
        }
    }
    if (resident[dev] < 0) return false;
    const int tn = q.N % 256 == 0 ? 256 : 128;
    const int n_tiles = q.N / tn;
    const int64_t items = (int64_t)q.batch * n_tiles * m_tiles;
    const unsigned pairs = (unsigned)(items < resident[dev] ? items : resident[dev]);
    TimedLaunch timed(s);
    *rc_out = (int)launch_pairs(kernel, pairs, pairspmm::kThreads, (size_t)pairspmm::kSmemBytes, s, true, q, map, map_out, map_b2, tn,
                                blk_offsets, blk_entries, m_tiles, n_tiles, k_blocks, d->status, flag, checks);
    return true;
}

template <typename TOut, int V> int launch_spmm_tc(const SpmmParams &p, cudaStream_t s) {
    DeviceInfo *d;
    int rc = device_info(&d);
    if (rc != VS_OK) return rc;
    const SpmmMode mode = spmm_mode();
    const int k_blocks = (p.K + densespmm::kBlockK - 1) / densespmm::kBlockK;
    const int m_tiles = (p.m_vec * V + densespmm::kTileM - 1) / densespmm::kTileM;
    const int n_tiles = (p.N + densespmm::kTileN - 1) / densespmm::kTileN;
    const int groups = m_tiles * (densespmm::kTileM / densespmm::kGroupRows);
    const int plan_blocks = k_blocks * (densespmm::kBlockK / densespmm::kPlanCols);
    const int rows_per_group = densespmm::kGroupRows / V;
    int64_t capacity = 0, offsets_bytes = 0;
    const int64_t plan_bytes = spmm_plan_bytes(p.m_vec, V, p.K, p.batch, p.stride_values, &capacity, &offsets_bytes);
    const int checks = spmm_plan_checks(p.m_vec);
    const size_t plan_words = (size_t)(2 * plan_blocks + rows_per_group + 1), check_words = (size_t)densespmm::kPlanWarps * plan_blocks;
    const size_t plan_smem = (plan_words > check_words ? plan_words : check_words) * 4;
    const bool dense_ok = !t_no_scratch && mode != SpmmMode::kGather && p.K > 0 && p.m_vec > 0 && p.N % 8 == 0 && plan_bytes <= kMaxPlanBytes &&
                          plan_smem <= 40 * 1024 && (p.batch == 1 || (p.stride_rhs * 2) % 16 == 0) &&
                          (p.batch == 1 || (p.stride_out * sizeof(TOut)) % 16 == 0) && aligned16(p.rhs) && aligned16(p.out);
    if (!dense_ok) return launch_spmm_gather<TOut, V>(p, s, d, nullptr, 0);

    constexpr bool kOutF32 = sizeof(TOut) == 4;
    CUtensorMap map, map_out;
    if (make_tile_map(&map, p.rhs, false, (uint64_t)p.K, (uint64_t)p.N, (uint64_t)p.batch, (uint64_t)p.stride_rhs, 64, 64) != VS_OK ||
        make_tile_map(&map_out, p.out, kOutF32, (uint64_t)p.m_vec * V, (uint64_t)p.N, (uint64_t)p.batch,
                      (uint64_t)p.stride_out, densespmm::kStoreCols, 32) != VS_OK)
        return launch_spmm_gather<TOut, V>(p, s, d, nullptr, 0);
    CUtensorMap map_b4 = map;
    const int use_b4 = (p.N % 64 == 0 && make_blocked_map(&map_b4, p.rhs, (uint64_t)p.K, (uint64_t)p.N, (uint64_t)p.batch,
                                                          (uint64_t)p.stride_rhs, densespmm::kTileN / 64) == VS_OK) ? 1 : 0;
    auto kernel = densespmm::spmm_dense_kernel<TOut, V, false>;
    rc = set_smem(kernel, densespmm::kSmemBytes);
    if (rc != VS_OK) return rc;
    uint8_t *plan = nullptr;
    if (stream_scratch(d, s, (size_t)plan_bytes, reinterpret_cast<void **>(&plan)) != VS_OK)
        return launch_spmm_gather<TOut, V>(p, s, d, nullptr, 0);
    int32_t *flag = reinterpret_cast<int32_t *>(plan);
    const int64_t header_bytes = spmm_plan_header_bytes(checks);
    int32_t *blk_offsets = reinterpret_cast<int32_t *>(plan + header_bytes);
    uint2 *blk_entries = reinterpret_cast<uint2 *>(plan + header_bytes + offsets_bytes);
    const int force_dense = mode == SpmmMode::kDense ? 1 : 0;
    // a dependent launch as well: in a stream of calls the plan kernel queues up behind the previous call's last kernel
    rc = (int)launch_overlapped(densespmm::dense_plan_kernel<false>, (unsigned)(groups + checks), densespmm::kPlanThreads, plan_smem, s,
                                p.row_offsets, p.col_indices, (const int32_t *)nullptr, 0, p.m_vec, p.K, groups, rows_per_group,
                                plan_blocks, blk_offsets, blk_entries, capacity, force_dense, 370.0f, 4.7f, 0.0f, flag);
    if (rc != VS_OK) return rc;
    const int64_t items = (int64_t)p.batch * n_tiles * m_tiles;
    const unsigned grid = (unsigned)(items < d->sm_count ? items : d->sm_count);   // one persistent CTA per SM
    rc = (int)cudaGetLastError();
    if (rc == VS_OK) {
        int rc_pair = VS_OK;
        if (use_b4 && p.N % 128 == 0 && spmm_pair_enabled() &&
            launch_spmm_pair<TOut, V, false>(p, s, d, map, map_out, map_b4, blk_offsets, blk_entries, m_tiles, k_blocks, flag, checks, &rc_pair))
            rc = rc_pair;
        else
            rc = (int)launch_overlapped(kernel, grid, densespmm::kThreads, densespmm::kSmemBytes, s, p, map, map_out, map_b4, use_b4,
                                        blk_offsets, blk_entries, m_tiles, n_tiles, k_blocks, d->status, flag, checks);
    }
    if (rc == VS_OK) rc = launch_spmm_gather<TOut, V>(p, s, d, flag, checks);
    return rc;
}

template <typename TOut> int spmm_tc_by_v(int V, const SpmmParams &p, cudaStream_t s) {
    switch (V) {
        case 2: return launch_spmm_tc<TOut, 2>(p, s);
        case 4: return launch_spmm_tc<TOut, 4>(p, s);
        case 8: return launch_spmm_tc<TOut, 8>(p, s);
    }
    return VS_ERR_VEC_LENGTH;
}

// ---- SDDMM dispatch ---------------------------------------------------------------------------------------
// CUDA-core SDDMM: a group of lanes per vector-row with the lhs rows in registers when the contraction length fits
// 32 chunks of 16 bytes (k <= 256 in fp16, 128 in fp32), a group of eight lanes per mask entry otherwise.
// VSPARSE_B200_SDDMM_CC=entry keeps the latter.
template <typename TIn, typename TOut, int V, int L> int launch_sddmm_cc_row(const SddmmParams &p, cudaStream_t s) {
    const int64_t blocks = ((int64_t)p.m_vec * L + kCcThreads - 1) / kCcThreads;
    if (blocks > 0x7fffffffll) return VS_ERR_SHAPE;
    dim3 grid((unsigned)blocks, (unsigned)p.batch, 1);
    sddmm_cc_row_kernel<TIn, TOut, V, L><<<grid, kCcThreads, 0, s>>>(p);
    return (int)cudaGetLastError();
}
template <typename TIn, typename TOut, int V> int launch_sddmm_cc(const SddmmParams &p, cudaStream_t s) {
    const int chunks = p.k / Chunk<TIn>::kElems;
    const char *e = std::getenv("VSPARSE_B200_SDDMM_CC");
    if (chunks >= 1 && chunks <= 32 && p.m_vec > 0 && !(e && !std::strcmp(e, "entry"))) {
        if (chunks > 16) return launch_sddmm_cc_row<TIn, TOut, V, 32>(p, s);
        if (chunks > 8) return launch_sddmm_cc_row<TIn, TOut, V, 16>(p, s);
        return launch_sddmm_cc_row<TIn, TOut, V, 8>(p, s);
    }
    const int64_t blocks = ((int64_t)p.nnz_vec * 8 + kCcThreads - 1) / kCcThreads;
    if (blocks > 0x7fffffffll) return VS_ERR_SHAPE;
    dim3 grid((unsigned)blocks, (unsigned)p.batch, 1);
    sddmm_cc_kernel<TIn, TOut, V><<<grid, kCcThreads, 0, s>>>(p);
    return (int)cudaGetLastError();
}

template <typename TIn, typename TOut> int sddmm_cc_by_v(int V, const SddmmParams &p, cudaStream_t s) {
    switch (V) {
        case 1: return launch_sddmm_cc<TIn, TOut, 1>(p, s);
        case 2: return launch_sddmm_cc<TIn, TOut, 2>(p, s);
        case 4: return launch_sddmm_cc<TIn, TOut, 4>(p, s);
        case 8: return launch_sddmm_cc<TIn, TOut, 8>(p, s);
    }
    return VS_ERR_VEC_LENGTH;
}

// Software (cp.async) gather: works for any batch stride.
template <typename TOut, int V> int launch_sddmm_tc_cpasync(const SddmmParams &p, cudaStream_t s, DeviceInfo *d) {
    auto kernel = tcsddmm::sddmm_tc_kernel<TOut, V>;
    int rc = set_smem(kernel, tcsddmm::kSmemBytes);
    if (rc != VS_OK) return rc;
    const int64_t items = (int64_t)p.batch * p.m_vec;
    const int64_t cap = 2ll * d->sm_count;
    const unsigned grid = (unsigned)(items < cap ? items : cap);
    kernel<<<grid, tcsddmm::kThreads, tcsddmm::kSmemBytes, s>>>(p, d->status);
    return (int)cudaGetLastError();
}

// TMA row gather: lhs and rhs of all batch entries must each be addressable as one matrix of k-wide rows, i.e.
// their batch strides are multiples of k (or zero / a single entry).
template <typename TOut, int V> int launch_sddmm_gather(const SddmmParams &p, cudaStream_t s, DeviceInfo *d) {
    static const bool force_cpasync = []() {
        const char *e = std::getenv("VSPARSE_B200_GATHER");
        return e && !std::strcmp(e, "cpasync");
    }();
    const int64_t m = (int64_t)p.m_vec * V;
    const bool one_r = p.batch == 1 || p.stride_rhs == 0, one_l = p.batch == 1 || p.stride_lhs == 0;
    const int64_t rpb_r = one_r ? 0 : p.stride_rhs / p.k, rpb_l = one_l ? 0 : p.stride_lhs / p.k;
    const int64_t rows_r = (one_r ? 0 : (int64_t)(p.batch - 1) * rpb_r) + p.n;
    const int64_t rows_l = (one_l ? 0 : (int64_t)(p.batch - 1) * rpb_l) + m;
    const bool tma_ok = !force_cpasync && p.n > 0 && (one_r || p.stride_rhs % p.k == 0) && (one_l || p.stride_lhs % p.k == 0) &&
                        rows_r < 0x7fffffffll && rows_l < 0x7fffffffll;
    if (!tma_ok) return launch_sddmm_tc_cpasync<TOut, V>(p, s, d);
    CUtensorMap map_r, map_l;
    if (make_gather_map(&map_r, p.rhs, (uint64_t)rows_r, (uint64_t)p.k) != VS_OK ||
        make_gather_map(&map_l, p.lhs, (uint64_t)rows_l, (uint64_t)p.k) != VS_OK)
        return launch_sddmm_tc_cpasync<TOut, V>(p, s, d);
    auto kernel = tmasddmm::sddmm_tma_kernel<TOut, V>;
    int rc = set_smem(kernel, tmasddmm::kSmemBytes);
    if (rc != VS_OK) return rc;
    const int64_t items = (int64_t)p.batch * p.m_vec;
    const int64_t cap = (int64_t)tmasddmm::kCtasPerSm * d->sm_count;
    const unsigned grid = (unsigned)(items < cap ? items : cap);
    kernel<<<grid, tmasddmm::kThreads, tmasddmm::kSmemBytes, s>>>(p, map_r, map_l, (int)rpb_r, (int)rows_r, (int)rpb_l,
                                                                  (int)rows_l, d->status);
    return (int)cudaGetLastError();
}

// Which tensor-core SDDMM runs: dense tiles of lhs . rhs^T sampled at the mask cost the same whatever the sparsity,
// the gather kernel a fixed amount per vector-row plus a little per mask entry.  The number of entries is an argument
// here, so the choice is made on the host, in SM-cycles per product, fitted to measurements on B200 (lhs 2048 x 256,
// rhs 512 x 256, 90 % and 98 % sparse; 4096 x 4096 masks of 410 entries per row at k = 64): gather ~306 per vector-row
// and 64 contraction elements + ~4 per entry; dense ~2230 per 256 x 256 tile and 64 contraction elements over the two
// SMs of a pair, and not less than ~4250 per tile (reading the accumulator out).
// VSPARSE_B200_SDDMM = "dense" | "gather" (read at every call) forces one.
bool sddmm_use_dense(const SddmmParams &p, int V) {
    const char *e = std::getenv("VSPARSE_B200_SDDMM");
    if (e && !std::strcmp(e, "dense")) return true;
    if (e && !std::strcmp(e, "gather")) return false;
    const double k_blocks = (double)(p.k / densesddmm::kBlockK);
    const double tiles = std::ceil((double)p.m_vec * V / 256.0) * std::ceil((double)p.n / 256.0);
    const double gather = (double)p.m_vec * 306.0 * k_blocks + (double)p.nnz_vec * 4.0;
    const double dense = tiles * std::max(2230.0 * k_blocks, 4250.0);
    return dense * 1.1 < gather;
}

// The dense SDDMM by pairs of CTAs (sddmm_pair.cuh) serves masks of up to pairsddmm::kMaxPlanColumns columns whose
// outputs can be written with vector stores; VSPARSE_B200_SDDMM_PAIR=0 keeps the single-CTA kernel.
inline bool sddmm_pair_enabled() {
    const char *e = std::getenv("VSPARSE_B200_SDDMM_PAIR");
    return !(e && !std::strcmp(e, "0"));
}
// Scratch of the pair kernel's plan: cells, entry order, the twins flag.
int64_t sddmm_pair_plan_bytes(int m_vec, int n, int nnz_vec, int64_t *cells_out, int64_t *order_out) {
    const int64_t blocks = (m_vec + pairsddmm::kBlockVecRows - 1) / pairsddmm::kBlockVecRows;
    const int64_t cells_bytes = (blocks * n * 8 + 15) & ~15ll, order_bytes = ((int64_t)nnz_vec * 4 + 15) & ~15ll;
    if (cells_out) *cells_out = cells_bytes;
    if (order_out) *order_out = order_bytes;
    return cells_bytes + order_bytes + 16;
}
// Plan, multiplying kernel and the fix-up for repeated columns; false if this call or this device cannot take them
// (nothing has been enqueued then).
template <typename TOut, int V> bool launch_sddmm_pair(const SddmmParams &p, cudaStream_t s, DeviceInfo *d, int *rc_out) {
    static int resident[kMaxDevices];   // 0 = not asked yet, -1 = the kernels cannot run here
    auto kernel = pairsddmm::sddmm_pair_kernel<TOut, V>;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return false;
    if (resident[dev] == 0) {
        if (set_smem(kernel, pairsddmm::kSmemBytes) != VS_OK ||
            set_smem(pairsddmm::sddmm_cell_plan_kernel, 8 * pairsddmm::kMaxPlanColumns) != VS_OK) {
            resident[dev] = -1;
        } else {
            const int n = max_resident_pairs(kernel, pairsddmm::kThreads, pairsddmm::kSmemBytes, d);
            resident[dev] = n > 0 ? n : -1;
        }
    }
    if (resident[dev] < 0) return false;
    int64_t cells_bytes = 0, order_bytes = 0;
    const int64_t plan_bytes = sddmm_pair_plan_bytes(p.m_vec, p.n, p.nnz_vec, &cells_bytes, &order_bytes);
    if (p.n > pairsddmm::kMaxPlanColumns || plan_bytes > kMaxPlanBytes || !aligned16(p.out) ||
        (p.batch > 1 && (p.stride_out * sizeof(TOut)) % 16 != 0))
        return false;
    CUtensorMap map_l, map_r;
    if (make_tile_map(&map_l, p.lhs, false, (uint64_t)p.m_vec * V, (uint64_t)p.k, (uint64_t)p.batch, (uint64_t)p.stride_lhs, 64,
                      pairsddmm::kCtaRows) != VS_OK ||
        make_tile_map(&map_r, p.rhs, false, (uint64_t)p.n, (uint64_t)p.k, (uint64_t)p.batch, (uint64_t)p.stride_rhs, 64,
                      pairsddmm::kCtaRows) != VS_OK)
        return false;
    uint8_t *plan = nullptr;
    if (stream_scratch(d, s, (size_t)plan_bytes, reinterpret_cast<void **>(&plan)) != VS_OK) return false;
    uint2 *cells = reinterpret_cast<uint2 *>(plan);
    int32_t *order = reinterpret_cast<int32_t *>(plan + cells_bytes);
    int32_t *twins = reinterpret_cast<int32_t *>(plan + cells_bytes + order_bytes);
    const int blocks = (p.m_vec + pairsddmm::kBlockVecRows - 1) / pairsddmm::kBlockVecRows;
    pairsddmm::sddmm_cell_plan_kernel<<<blocks, pairsddmm::kPlanThreads, (size_t)8 * p.n, s>>>(p.row_offsets, p.col_indices, p.m_vec, p.n,
                                                                                              p.nnz_vec, cells, order, twins);
    int rc = (int)cudaGetLastError();
    if (rc == VS_OK) {
        const int m_tiles = (p.m_vec * V + pairsddmm::kTile - 1) / pairsddmm::kTile;
        const int n_tiles = (p.n + pairsddmm::kTile - 1) / pairsddmm::kTile;
        const int64_t items = (int64_t)p.batch * n_tiles * m_tiles;
        const unsigned pairs = (unsigned)(items < resident[dev] ? items : resident[dev]);
        // rhs of a batch entry fits the resident slots (VSPARSE_B200_SDDMM_RESIDENT=0: stream both operands anyway)
        const char *res_env = std::getenv("VSPARSE_B200_SDDMM_RESIDENT");
        const int resident = (n_tiles * (p.k / densesddmm::kBlockK) <= pairsddmm::kMaxResident && !(res_env && !std::strcmp(res_env, "0"))) ? 1 : 0;
        TimedLaunch timed(s);
        rc = (int)launch_pairs(kernel, pairs, pairsddmm::kThreads, (size_t)pairsddmm::kSmemBytes, s, true, p, map_l, map_r, cells, order,
                               blocks, m_tiles, n_tiles, resident, d->status);
    }
    if (rc == VS_OK)
        rc = (int)launch_overlapped(pairsddmm::sddmm_twin_kernel<TOut, V>, (unsigned)((p.nnz_vec + pairsddmm::kPlanThreads - 1) / pairsddmm::kPlanThreads),
                                    pairsddmm::kPlanThreads, 0, s, p, cells, order, twins);
    *rc_out = rc;
    return true;
}

template <typename TOut, int V> int launch_sddmm_tc(const SddmmParams &p, cudaStream_t s) {
    DeviceInfo *d;
    int rc = device_info(&d);
    if (rc != VS_OK) return rc;
    const int chunks = (p.n + densesddmm::kChunk - 1) / densesddmm::kChunk;
    int64_t offsets_bytes = 0;
    const int64_t plan_bytes = sddmm_plan_bytes(p.m_vec, p.n, p.nnz_vec, &offsets_bytes);
    const size_t plan_smem = (size_t)2 * chunks * 4;
    const bool dense_ok = !t_no_scratch && p.n > 0 && p.m_vec > 0 && p.nnz_vec > 0 && p.k >= densesddmm::kBlockK && plan_bytes <= kMaxPlanBytes &&
                          plan_smem <= 40 * 1024 && aligned16(p.lhs) && aligned16(p.rhs) &&
                          (p.batch == 1 || ((p.stride_lhs * 2) % 16 == 0 && (p.stride_rhs * 2) % 16 == 0)) &&
                          sddmm_use_dense(p, V);
    if (!dense_ok) return launch_sddmm_gather<TOut, V>(p, s, d);
    if (sddmm_pair_enabled() && launch_sddmm_pair<TOut, V>(p, s, d, &rc)) return rc;
    CUtensorMap map_l, map_r;
    if (make_tile_map(&map_l, p.lhs, false, (uint64_t)p.m_vec * V, (uint64_t)p.k, (uint64_t)p.batch, (uint64_t)p.stride_lhs, 64,
                      densesddmm::kTileM) != VS_OK ||
        make_tile_map(&map_r, p.rhs, false, (uint64_t)p.n, (uint64_t)p.k, (uint64_t)p.batch, (uint64_t)p.stride_rhs, 64,
                      densesddmm::kTileN) != VS_OK)
        return launch_sddmm_gather<TOut, V>(p, s, d);
    auto kernel = densesddmm::sddmm_dense_kernel<TOut, V>;
    rc = set_smem(kernel, densesddmm::kSmemBytes);
    if (rc != VS_OK) return rc;
    uint8_t *plan = nullptr;
    if (stream_scratch(d, s, (size_t)plan_bytes, reinterpret_cast<void **>(&plan)) != VS_OK)
        return launch_sddmm_gather<TOut, V>(p, s, d);
    int32_t *chunk_offsets = reinterpret_cast<int32_t *>(plan);
    uint2 *chunk_entries = reinterpret_cast<uint2 *>(plan + offsets_bytes);
    densesddmm::sddmm_plan_kernel<<<p.m_vec, densesddmm::kPlanThreads, plan_smem, s>>>(p.row_offsets, p.col_indices, p.n, chunks,
                                                                                   p.nnz_vec, chunk_offsets, chunk_entries);
    const int m_tiles = (p.m_vec * V + densesddmm::kTileM - 1) / densesddmm::kTileM;
    const int n_tiles = (p.n + densesddmm::kTileN - 1) / densesddmm::kTileN;
    const int64_t items = (int64_t)p.batch * m_tiles * n_tiles;
    const unsigned grid = (unsigned)(items < d->sm_count ? items : d->sm_count);   // one persistent CTA per SM
    rc = (int)cudaGetLastError();
    if (rc != VS_OK) return rc;
    return (int)launch_overlapped(kernel, grid, densesddmm::kThreads, densesddmm::kSmemBytes, s, p, map_l, map_r, chunk_offsets,
                                  chunk_entries, m_tiles, n_tiles, chunks, d->status);
}

template <typename TOut> int sddmm_tc_by_v(int V, const SddmmParams &p, cudaStream_t s) {
    switch (V) {
        case 2: return launch_sddmm_tc<TOut, 2>(p, s);
        case 4: return launch_sddmm_tc<TOut, 4>(p, s);
        case 8: return launch_sddmm_tc<TOut, 8>(p, s);
    }
    return VS_ERR_VEC_LENGTH;
}

template <typename T> int softmax_by_v(int V, const SoftmaxParams &p, cudaStream_t s) {
    const int64_t blocks = ((int64_t)p.m_vec * 32 + kCcThreads - 1) / kCcThreads;
    dim3 grid((unsigned)blocks, (unsigned)p.batch, 1);
    switch (V) {
        case 1: softmax_cvse_kernel<T, 1><<<grid, kCcThreads, 0, s>>>(p); break;
        case 2: softmax_cvse_kernel<T, 2><<<grid, kCcThreads, 0, s>>>(p); break;
        case 4: softmax_cvse_kernel<T, 4><<<grid, kCcThreads, 0, s>>>(p); break;
        case 8: softmax_cvse_kernel<T, 8><<<grid, kCcThreads, 0, s>>>(p); break;
        default: return VS_ERR_VEC_LENGTH;
    }
    return (int)cudaGetLastError();
}

template <typename T> int softmax_backward_by_v(int V, const SoftmaxBackwardParams &p, int batch, cudaStream_t s) {
    const int64_t blocks = ((int64_t)p.m_vec * 32 + kCcThreads - 1) / kCcThreads;
    dim3 grid((unsigned)blocks, (unsigned)batch, 1);
    switch (V) {
        case 1: softmax_cvse_backward_kernel<T, 1><<<grid, kCcThreads, 0, s>>>(p); break;
        case 2: softmax_cvse_backward_kernel<T, 2><<<grid, kCcThreads, 0, s>>>(p); break;
        case 4: softmax_cvse_backward_kernel<T, 4><<<grid, kCcThreads, 0, s>>>(p); break;
        case 8: softmax_cvse_backward_kernel<T, 8><<<grid, kCcThreads, 0, s>>>(p); break;
        default: return VS_ERR_VEC_LENGTH;
    }
    return (int)cudaGetLastError();
}

constexpr int kMaxBatch = 65535;  // grid.y of the CUDA-core kernels

}  // namespace

// =============================================================================================================

VS_EXPORT int vs_spmm_batched(int path, int in_dtype, int out_dtype, int m_vec, int vec_length, int k, int n,
                              const int32_t *row_indices, const int32_t *row_offsets, const int32_t *col_indices,
                              const void *values, const void *rhs_matrix, void *output_matrix, int batch,
                              int64_t stride_values, int64_t stride_rhs, int64_t stride_out, void *stream) {
    if (path != VS_PATH_TENSOR && path != VS_PATH_CUDA_CORE) return VS_ERR_ARG;
    if (path == VS_PATH_TENSOR ? !(vec_length == 2 || vec_length == 4 || vec_length == 8) : !valid_v(vec_length))
        return VS_ERR_VEC_LENGTH;
    const bool f16 = (in_dtype == VS_F16) && (out_dtype == VS_F16 || out_dtype == VS_F32);
    const bool f32 = (in_dtype == VS_F32) && (out_dtype == VS_F32) && path == VS_PATH_CUDA_CORE;
    if (!f16 && !f32) return VS_ERR_DTYPE;
    if (m_vec < 0 || k < 0 || n < 0) return VS_ERR_SHAPE;
    if (batch < 1 || batch > kMaxBatch) return VS_ERR_ARG;
    if (path == VS_PATH_TENSOR ? (k % 64 != 0) : (k % (in_dtype == VS_F16 ? 8 : 4) != 0)) return VS_ERR_SHAPE;
    if ((int64_t)m_vec * vec_length > 0x7fffffffll) return VS_ERR_SHAPE;
    if (m_vec == 0 || k == 0) return VS_OK;
    if (!row_indices || !row_offsets || !col_indices || !values || !rhs_matrix || !output_matrix) return VS_ERR_NULL;
    if (!aligned16(values) || !aligned16(rhs_matrix) || !aligned16(output_matrix)) return VS_ERR_ALIGN;
    if (!stride_ok(stride_values, in_dtype) || !stride_ok(stride_rhs, in_dtype) || !stride_ok(stride_out, out_dtype))
        return VS_ERR_ALIGN;
    if (batch > 1 && stride_out == 0) return VS_ERR_ARG;

    SpmmParams p;
    p.m_vec = m_vec; p.N = k; p.K = n; p.batch = batch;
    p.row_indices = row_indices; p.row_offsets = row_offsets; p.col_indices = col_indices;
    p.values = values; p.rhs = rhs_matrix; p.out = output_matrix;
    p.stride_values = stride_values; p.stride_rhs = stride_rhs; p.stride_out = stride_out;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    if (path == VS_PATH_TENSOR) {
        return out_dtype == VS_F16 ? spmm_tc_by_v<__half>(vec_length, p, s) : spmm_tc_by_v<float>(vec_length, p, s);
    }
    if (in_dtype == VS_F32) return spmm_cc_by_v<float, float>(vec_length, p, s);
    return out_dtype == VS_F16 ? spmm_cc_by_v<__half, __half>(vec_length, p, s)
                               : spmm_cc_by_v<__half, float>(vec_length, p, s);
}

VS_EXPORT int vs_spmm(int path, int in_dtype, int out_dtype, int m_vec, int vec_length, int k, int n,
                      const int32_t *row_indices, const int32_t *row_offsets, const int32_t *col_indices,
                      const void *values, const void *rhs_matrix, void *output_matrix, void *stream) {
    return vs_spmm_batched(path, in_dtype, out_dtype, m_vec, vec_length, k, n, row_indices, row_offsets,
                           col_indices, values, rhs_matrix, output_matrix, 1, 0, 0, 0, stream);
}

// ---- SpMM with the transposed sparse matrix ------------------------------------------------------------------
namespace {
// CUDA-core kernel.  With `plan_hdr` it is enqueued behind the dense kernel and returns at once unless that kernel
// left the call to it.
template <typename TOut, int V>
int launch_spmm_t_cc(const spmmt::Params &p, cudaStream_t s, DeviceInfo *d, const int32_t *plan_hdr, int plan_checks) {
    const int row_groups = (p.n + spmmt::kWarps - 1) / spmmt::kWarps;
    const int chunks = (p.N + spmmt::kChunk - 1) / spmmt::kChunk;
    const int64_t items = (int64_t)p.batch * chunks * row_groups;
    const int64_t cap = (int64_t)d->sm_count * 16;   // as many 128-thread CTAs as are resident at once; the rest by grid stride
                                                      // (behind the dense kernel the launch usually returns at once: 9472 CTAs
                                                      // took 14 us to do so, a quarter of them a quarter of that)
    const unsigned grid = (unsigned)(items < cap ? items : cap);
    auto kernel = spmmt::spmm_t_kernel<TOut, V>;
    if (plan_hdr) return (int)launch_overlapped(kernel, grid, spmmt::kThreads, 0, s, p, items, row_groups, chunks, plan_hdr, plan_checks);
    kernel<<<grid, spmmt::kThreads, 0, s>>>(p, items, row_groups, chunks, plan_hdr, plan_checks);
    return (int)cudaGetLastError();
}

enum class SpmmTMode { kAuto, kDense, kGather };
SpmmTMode spmm_t_mode() {   // read at every call, so that a test can switch kernels inside one process
    const char *e = std::getenv("VSPARSE_B200_SPMM_T");
    if (e && !std::strcmp(e, "dense")) return SpmmTMode::kDense;
    if (e && !std::strcmp(e, "gather")) return SpmmTMode::kGather;
    return SpmmTMode::kAuto;
}

// Tensor path of the transposed product: A^T (n x m_vec * V) goes through the densifying SpMM kernel, its plan
// built straight from the transposed structure (dense_plan_kernel<true>), the values read where the forward
// operators keep them; a vector's V values land side by side in one row of the tile.  Costs for the choice, in the
// plan kernel's units (SM-cycles per 128 columns): the CUDA-core kernel ~5 per value (0.92 ms for 256 products of
// 2048 x 512, 90 % sparse, V = 8), the dense kernel ~1100 per stage plus ~1.5 per vector of fill work (0.170 ms on
// the same problem against 0.137 for the forward product with the same tiles).
template <typename TOut, int V> int launch_spmm_t(const spmmt::Params &p, int m_vec, cudaStream_t s) {
    DeviceInfo *d;
    int rc = device_info(&d);
    if (rc != VS_OK) return rc;
    const SpmmTMode mode = spmm_t_mode();
    const int shift = V == 8 ? 3 : V == 4 ? 2 : V == 2 ? 1 : 0;
    const int64_t M = (int64_t)m_vec * V;   // columns of A^T: the contraction
    SpmmParams q;
    q.m_vec = p.n; q.N = p.N; q.K = (int)M; q.batch = p.batch;
    q.row_indices = nullptr; q.row_offsets = p.t_offsets; q.col_indices = p.t_rows;
    q.values = p.values; q.rhs = p.rhs; q.out = p.out;
    q.stride_values = p.stride_values; q.stride_rhs = p.stride_rhs; q.stride_out = p.stride_out;
    const int k_blocks = (q.K + densespmm::kBlockK - 1) / densespmm::kBlockK;
    const int m_tiles = (q.m_vec + densespmm::kTileM - 1) / densespmm::kTileM;
    const int n_tiles = (q.N + densespmm::kTileN - 1) / densespmm::kTileN;
    const int groups = m_tiles * (densespmm::kTileM / densespmm::kGroupRows);
    const int plan_blocks = k_blocks * (densespmm::kBlockK / densespmm::kPlanCols);
    const int rows_per_group = densespmm::kGroupRows;
    int64_t capacity = 0, offsets_bytes = 0;
    const int64_t plan_bytes = spmm_t_plan_bytes(p.n, m_vec, V, q.batch, q.stride_values, &capacity, &offsets_bytes);
    const int checks = spmm_plan_checks(q.m_vec);
    const size_t plan_words = (size_t)(2 * plan_blocks + rows_per_group + 1), check_words = (size_t)densespmm::kPlanWarps * plan_blocks;
    const size_t plan_smem = (plan_words > check_words ? plan_words : check_words) * 4;
    const bool dense_ok = !t_no_scratch && mode != SpmmTMode::kGather && q.K > 0 && q.m_vec > 0 && plan_bytes <= kMaxPlanBytes &&
                          plan_smem <= 40 * 1024 && (q.batch == 1 || (q.stride_rhs * 2) % 16 == 0) &&
                          (q.batch == 1 || (q.stride_out * sizeof(TOut)) % 16 == 0);
    if (!dense_ok) return launch_spmm_t_cc<TOut, V>(p, s, d, nullptr, 0);

    constexpr bool kOutF32 = sizeof(TOut) == 4;
    CUtensorMap map, map_out;
    if (make_tile_map(&map, q.rhs, false, (uint64_t)q.K, (uint64_t)q.N, (uint64_t)q.batch, (uint64_t)q.stride_rhs, 64, 64) != VS_OK ||
        make_tile_map(&map_out, q.out, kOutF32, (uint64_t)q.m_vec, (uint64_t)q.N, (uint64_t)q.batch, (uint64_t)q.stride_out,
                      densespmm::kStoreCols, 32) != VS_OK)
        return launch_spmm_t_cc<TOut, V>(p, s, d, nullptr, 0);
    CUtensorMap map_b4 = map;
    const int use_b4 = (q.N % 64 == 0 && make_blocked_map(&map_b4, q.rhs, (uint64_t)q.K, (uint64_t)q.N, (uint64_t)q.batch,
                                                          (uint64_t)q.stride_rhs, densespmm::kTileN / 64) == VS_OK) ? 1 : 0;
    auto kernel = densespmm::spmm_dense_kernel<TOut, V, true>;
    rc = set_smem(kernel, densespmm::kSmemBytes);
    if (rc != VS_OK) return rc;
    uint8_t *plan = nullptr;
    if (stream_scratch(d, s, (size_t)plan_bytes, reinterpret_cast<void **>(&plan)) != VS_OK)
        return launch_spmm_t_cc<TOut, V>(p, s, d, nullptr, 0);
    int32_t *flag = reinterpret_cast<int32_t *>(plan);
    const int64_t header_bytes = spmm_plan_header_bytes(checks);
    int32_t *blk_offsets = reinterpret_cast<int32_t *>(plan + header_bytes);
    uint2 *blk_entries = reinterpret_cast<uint2 *>(plan + header_bytes + offsets_bytes);
    rc = (int)launch_overlapped(densespmm::dense_plan_kernel<true>, (unsigned)(groups + checks), densespmm::kPlanThreads, plan_smem, s,
                                p.t_offsets, p.t_rows, p.t_src, shift, q.m_vec, q.K, groups, rows_per_group, plan_blocks, blk_offsets,
                                blk_entries, capacity, mode == SpmmTMode::kDense ? 1 : 0, 0.0f, 5.0f * V, 1.5f, flag);
    const int64_t items = (int64_t)q.batch * n_tiles * m_tiles;
    const unsigned grid = (unsigned)(items < d->sm_count ? items : d->sm_count);   // one persistent CTA per SM
    if (rc == VS_OK) {
        int rc_pair = VS_OK;
        if (use_b4 && q.N % 128 == 0 && spmm_pair_enabled() &&
            launch_spmm_pair<TOut, V, true>(q, s, d, map, map_out, map_b4, blk_offsets, blk_entries, m_tiles, k_blocks, flag, checks, &rc_pair))
            rc = rc_pair;
        else
            rc = (int)launch_overlapped(kernel, grid, densespmm::kThreads, densespmm::kSmemBytes, s, q, map, map_out, map_b4, use_b4,
                                        blk_offsets, blk_entries, m_tiles, n_tiles, k_blocks, d->status, flag, checks);
    }
    if (rc == VS_OK) rc = launch_spmm_t_cc<TOut, V>(p, s, d, flag, checks);
    return rc;
}
template <typename TOut> int spmm_t_by_v(int V, const spmmt::Params &p, int m_vec, cudaStream_t s) {
    switch (V) {
        case 1: return launch_spmm_t<TOut, 1>(p, m_vec, s);
        case 2: return launch_spmm_t<TOut, 2>(p, m_vec, s);
        case 4: return launch_spmm_t<TOut, 4>(p, m_vec, s);
        case 8: return launch_spmm_t<TOut, 8>(p, m_vec, s);
    }
    return VS_ERR_VEC_LENGTH;
}
}  // namespace

VS_EXPORT int vs_spmm_t_batched(int in_dtype, int out_dtype, int m_vec, int vec_length, int k, int n,
                                const int32_t *t_offsets, const int32_t *t_rows, const int32_t *t_src,
                                const void *values, const void *rhs_matrix, void *output_matrix, int batch,
                                int64_t stride_values, int64_t stride_rhs, int64_t stride_out, void *stream) {
    if (!valid_v(vec_length)) return VS_ERR_VEC_LENGTH;
    if (!(in_dtype == VS_F16 && (out_dtype == VS_F16 || out_dtype == VS_F32))) return VS_ERR_DTYPE;
    if (m_vec < 0 || k < 0 || n < 0 || k % 8 != 0) return VS_ERR_SHAPE;
    if ((int64_t)m_vec * vec_length > 0x7fffffffll) return VS_ERR_SHAPE;
    if (batch < 1 || batch > kMaxBatch) return VS_ERR_ARG;
    if (n == 0 || k == 0) return VS_OK;
    if (!t_offsets || !t_rows || !t_src || !values || !rhs_matrix || !output_matrix) return VS_ERR_NULL;
    if (!aligned16(values) || !aligned16(rhs_matrix) || !aligned16(output_matrix)) return VS_ERR_ALIGN;
    if (!stride_ok(stride_values, in_dtype) || !stride_ok(stride_rhs, in_dtype) || !stride_ok(stride_out, out_dtype))
        return VS_ERR_ALIGN;
    if (batch > 1 && stride_out == 0) return VS_ERR_ARG;
    spmmt::Params p;
    p.n = n; p.N = k; p.batch = batch;
    p.t_offsets = t_offsets; p.t_rows = t_rows; p.t_src = t_src;
    p.values = static_cast<const __half *>(values); p.rhs = static_cast<const __half *>(rhs_matrix); p.out = output_matrix;
    p.stride_values = stride_values; p.stride_rhs = stride_rhs; p.stride_out = stride_out;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return out_dtype == VS_F16 ? spmm_t_by_v<__half>(vec_length, p, m_vec, s) : spmm_t_by_v<float>(vec_length, p, m_vec, s);
}

VS_EXPORT int vs_spmm_t(int in_dtype, int out_dtype, int m_vec, int vec_length, int k, int n, const int32_t *t_offsets,
                        const int32_t *t_rows, const int32_t *t_src, const void *values, const void *rhs_matrix,
                        void *output_matrix, void *stream) {
    return vs_spmm_t_batched(in_dtype, out_dtype, m_vec, vec_length, k, n, t_offsets, t_rows, t_src, values, rhs_matrix,
                             output_matrix, 1, 0, 0, 0, stream);
}

VS_EXPORT int vs_sddmm_batched(int path, int in_dtype, int out_dtype, int m_vec, int k, int n, int nonzeros_vec,
                               const int32_t *row_indices, const int32_t *row_offsets, const int32_t *col_indices,
                               const void *lhs_matrix, const void *rhs_matrix, void *output_values,
                               int vec_length, int batch, int64_t stride_lhs, int64_t stride_rhs,
                               int64_t stride_out, void *stream, int algorithm) {
    if (path != VS_PATH_TENSOR && path != VS_PATH_CUDA_CORE) return VS_ERR_ARG;
    if (path == VS_PATH_TENSOR ? !(vec_length == 2 || vec_length == 4 || vec_length == 8) : !valid_v(vec_length))
        return VS_ERR_VEC_LENGTH;
    if (!(in_dtype == VS_F16 && (out_dtype == VS_F16 || out_dtype == VS_F32))) return VS_ERR_DTYPE;
    if (path == VS_PATH_TENSOR && (algorithm < 0 || algorithm > 3)) return VS_ERR_ARG;
    if (m_vec < 0 || k < 0 || n < 0 || nonzeros_vec < 0) return VS_ERR_SHAPE;
    if (batch < 1 || batch > kMaxBatch) return VS_ERR_ARG;
    if (path == VS_PATH_TENSOR ? (k % 64 != 0) : (k % 8 != 0)) return VS_ERR_SHAPE;
    if ((int64_t)nonzeros_vec * vec_length > 0x7fffffffll) return VS_ERR_SHAPE;
    if (m_vec == 0 || nonzeros_vec == 0) return VS_OK;
    if (!row_indices || !row_offsets || !col_indices || !lhs_matrix || !rhs_matrix || !output_values)
        return VS_ERR_NULL;
    if (!aligned16(lhs_matrix) || !aligned16(rhs_matrix) || !aligned16(output_values)) return VS_ERR_ALIGN;
    if (!stride_ok(stride_lhs, in_dtype) || !stride_ok(stride_rhs, in_dtype) || !stride_ok(stride_out, out_dtype))
        return VS_ERR_ALIGN;
    if (batch > 1 && stride_out == 0) return VS_ERR_ARG;

    SddmmParams p;
    p.m_vec = m_vec; p.k = k; p.n = n; p.nnz_vec = nonzeros_vec; p.batch = batch;
    p.row_indices = row_indices; p.row_offsets = row_offsets; p.col_indices = col_indices;
    p.lhs = lhs_matrix; p.rhs = rhs_matrix; p.out = output_values;
    p.stride_lhs = stride_lhs; p.stride_rhs = stride_rhs; p.stride_out = stride_out;
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    if (k == 0) {  // empty contraction: every output is zero
        for (int b = 0; b < batch; ++b) {
            cudaError_t e = cudaMemsetAsync(static_cast<char *>(output_values) + (size_t)b * stride_out * elem_size(out_dtype),
                                            0, (size_t)nonzeros_vec * vec_length * elem_size(out_dtype), s);
            if (e != cudaSuccess) return (int)e;
        }
        return VS_OK;
    }
    if (path == VS_PATH_TENSOR) {
        return out_dtype == VS_F16 ? sddmm_tc_by_v<__half>(vec_length, p, s) : sddmm_tc_by_v<float>(vec_length, p, s);
    }
    return out_dtype == VS_F16 ? sddmm_cc_by_v<__half, __half>(vec_length, p, s)
                               : sddmm_cc_by_v<__half, float>(vec_length, p, s);
}

VS_EXPORT int vs_sddmm(int path, int in_dtype, int out_dtype, int m_vec, int k, int n, int nonzeros_vec,
                       const int32_t *row_indices, const int32_t *row_offsets, const int32_t *col_indices,
                       const void *lhs_matrix, const void *rhs_matrix, void *output_values, int vec_length,
                       void *stream, int algorithm) {
    return vs_sddmm_batched(path, in_dtype, out_dtype, m_vec, k, n, nonzeros_vec, row_indices, row_offsets,
                            col_indices, lhs_matrix, rhs_matrix, output_values, vec_length, 1, 0, 0, 0, stream,
                            algorithm);
}

VS_EXPORT int vs_softmax_cvse(int dtype, int m_vec, int vec_length, const int32_t *row_indices,
                              const int32_t *row_offsets, const void *scores, void *probs, float scale, int batch,
                              int64_t stride, void *stream) {
    (void)row_indices;  // rows are independent and equally cheap to reach: the order is not needed
    if (!valid_v(vec_length)) return VS_ERR_VEC_LENGTH;
    if (dtype != VS_F16 && dtype != VS_F32) return VS_ERR_DTYPE;
    if (m_vec < 0) return VS_ERR_SHAPE;
    if (batch < 1 || batch > kMaxBatch) return VS_ERR_ARG;
    if (m_vec == 0) return VS_OK;
    if (!row_offsets || !scores || !probs) return VS_ERR_NULL;
    if (stride < 0 || (batch > 1 && stride == 0)) return VS_ERR_ARG;
    {   // one entry (V values) is read and written as one vector of up to 16 bytes
        const size_t entry = (size_t)vec_length * elem_size(dtype), al = entry < 16 ? entry : 16;
        if (reinterpret_cast<uintptr_t>(scores) % al || reinterpret_cast<uintptr_t>(probs) % al ||
            ((size_t)stride * elem_size(dtype)) % al)
            return VS_ERR_ALIGN;
    }
    SoftmaxParams p;
    p.m_vec = m_vec; p.batch = batch; p.row_offsets = row_offsets; p.scores = scores; p.probs = probs;
    p.stride = stride; p.scale = scale;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return dtype == VS_F16 ? softmax_by_v<__half>(vec_length, p, s) : softmax_by_v<float>(vec_length, p, s);
}

VS_EXPORT int vs_softmax_cvse_backward(int dtype, int m_vec, int vec_length, const int32_t *row_offsets, const void *probs,
                                       const void *grad_probs, void *grad_scores, float scale, int batch, int64_t stride,
                                       void *stream) {
    if (!valid_v(vec_length)) return VS_ERR_VEC_LENGTH;
    if (dtype != VS_F16 && dtype != VS_F32) return VS_ERR_DTYPE;
    if (m_vec < 0) return VS_ERR_SHAPE;
    if (batch < 1 || batch > kMaxBatch) return VS_ERR_ARG;
    if (m_vec == 0) return VS_OK;
    if (!row_offsets || !probs || !grad_probs || !grad_scores) return VS_ERR_NULL;
    if (stride < 0 || (batch > 1 && stride == 0)) return VS_ERR_ARG;
    {   // one entry (V values) is read and written as one vector of up to 16 bytes
        const size_t entry = (size_t)vec_length * elem_size(dtype), al = entry < 16 ? entry : 16;
        if (reinterpret_cast<uintptr_t>(probs) % al || reinterpret_cast<uintptr_t>(grad_probs) % al ||
            reinterpret_cast<uintptr_t>(grad_scores) % al || ((size_t)stride * elem_size(dtype)) % al)
            return VS_ERR_ALIGN;
    }
    SoftmaxBackwardParams p;
    p.m_vec = m_vec; p.row_offsets = row_offsets; p.probs = probs; p.grad_probs = grad_probs; p.grad_scores = grad_scores;
    p.stride = stride; p.scale = scale;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return dtype == VS_F16 ? softmax_backward_by_v<__half>(vec_length, p, batch, s)
                           : softmax_backward_by_v<float>(vec_length, p, batch, s);
}

VS_EXPORT int vs_attention_cvse_backward(int path, int m_vec, int vec_length, int n, int d, int nonzeros_vec,
                                         const int32_t *row_indices, const int32_t *row_offsets, const int32_t *col_indices,
                                         const int32_t *t_offsets, const int32_t *t_rows, const int32_t *t_src, const void *q,
                                         const void *kmat, const void *vmat, const void *grad_out, void *grad_q, void *grad_k,
                                         void *grad_v, void *probs_workspace, void *grad_workspace, float scale, int batch,
                                         void *stream) {
    if ((!probs_workspace || !grad_workspace) && nonzeros_vec > 0) return VS_ERR_NULL;
    if (probs_workspace && probs_workspace == grad_workspace) return VS_ERR_ARG;
    const int64_t m = (int64_t)m_vec * vec_length;
    const int64_t s_ws = (int64_t)nonzeros_vec * vec_length;
    if ((s_ws * 2) % 16 != 0 && batch > 1) return VS_ERR_ALIGN;
    const int64_t s_q = m * d, s_k = (int64_t)n * d;
    if (nonzeros_vec == 0) {   // an empty mask: the output does not depend on q, k or v
        if (m_vec < 0 || n < 0 || d < 0 || batch < 1 || !valid_v(vec_length)) return VS_ERR_ARG;
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        if (s_q > 0 && !grad_q) return VS_ERR_NULL;
        if (s_k > 0 && (!grad_k || !grad_v)) return VS_ERR_NULL;
        if (s_q > 0) VS_CUDA_TRY(cudaMemsetAsync(grad_q, 0, (size_t)batch * s_q * 2, st));
        if (s_k > 0) VS_CUDA_TRY(cudaMemsetAsync(grad_k, 0, (size_t)batch * s_k * 2, st));
        if (s_k > 0) VS_CUDA_TRY(cudaMemsetAsync(grad_v, 0, (size_t)batch * s_k * 2, st));
        return VS_OK;
    }
    // P = softmax(scale * Q K^T) at the mask, recomputed rather than kept from the forward pass
    int rc = vs_sddmm_batched(path, VS_F16, VS_F16, m_vec, d, n, nonzeros_vec, row_indices, row_offsets, col_indices, q, kmat,
                              probs_workspace, vec_length, batch, s_q, s_k, s_ws, stream, 0);
    if (rc != VS_OK) return rc;
    rc = vs_softmax_cvse(VS_F16, m_vec, vec_length, row_indices, row_offsets, probs_workspace, probs_workspace, scale, batch,
                         s_ws, stream);
    if (rc != VS_OK) return rc;
    // dV = P^T dO
    rc = vs_spmm_t_batched(VS_F16, VS_F16, m_vec, vec_length, d, n, t_offsets, t_rows, t_src, probs_workspace, grad_out, grad_v,
                           batch, s_ws, s_q, s_k, stream);
    if (rc != VS_OK) return rc;
    // dP = dO V^T at the mask; dS = scale * P o (dP - rowsum(P o dP))
    rc = vs_sddmm_batched(path, VS_F16, VS_F16, m_vec, d, n, nonzeros_vec, row_indices, row_offsets, col_indices, grad_out, vmat,
                          grad_workspace, vec_length, batch, s_q, s_k, s_ws, stream, 0);
    if (rc != VS_OK) return rc;
    rc = vs_softmax_cvse_backward(VS_F16, m_vec, vec_length, row_offsets, probs_workspace, grad_workspace, grad_workspace, scale,
                                  batch, s_ws, stream);
    if (rc != VS_OK) return rc;
    // dQ = dS K,  dK = dS^T Q
    rc = vs_spmm_batched(path, VS_F16, VS_F16, m_vec, vec_length, d, n, row_indices, row_offsets, col_indices, grad_workspace,
                         kmat, grad_q, batch, s_ws, s_k, s_q, stream);
    if (rc != VS_OK) return rc;
    return vs_spmm_t_batched(VS_F16, VS_F16, m_vec, vec_length, d, n, t_offsets, t_rows, t_src, grad_workspace, q, grad_k, batch,
                             s_ws, s_q, s_k, stream);
}

VS_EXPORT int vs_attention_cvse(int path, int m_vec, int vec_length, int n, int d, int nonzeros_vec,
                                const int32_t *row_indices, const int32_t *row_offsets, const int32_t *col_indices,
                                const void *q, const void *kmat, const void *vmat, void *out, void *workspace,
                                float scale, int batch, void *stream) {
    if (!workspace && nonzeros_vec > 0) return VS_ERR_NULL;
    const int64_t m = (int64_t)m_vec * vec_length;
    const int64_t s_ws = (int64_t)nonzeros_vec * vec_length;
    if ((s_ws * 2) % 16 != 0 && batch > 1) return VS_ERR_ALIGN;
    if (nonzeros_vec == 0) {   // an empty mask: no scores, no probabilities, every output row is zero
        if (m_vec < 0 || d < 0 || batch < 1 || !valid_v(vec_length)) return VS_ERR_ARG;
        if (m == 0 || d == 0) return VS_OK;
        if (!out) return VS_ERR_NULL;
        return (int)cudaMemsetAsync(out, 0, (size_t)batch * m * d * 2, static_cast<cudaStream_t>(stream));
    }
    int rc = vs_sddmm_batched(path, VS_F16, VS_F16, m_vec, d, n, nonzeros_vec, row_indices, row_offsets,
                              col_indices, q, kmat, workspace, vec_length, batch, m * d, (int64_t)n * d, s_ws,
                              stream, 0);
    if (rc != VS_OK) return rc;
    rc = vs_softmax_cvse(VS_F16, m_vec, vec_length, row_indices, row_offsets, workspace, workspace, scale, batch,
                         s_ws, stream);
    if (rc != VS_OK) return rc;
    return vs_spmm_batched(path, VS_F16, VS_F16, m_vec, vec_length, d, n, row_indices, row_offsets, col_indices,
                           workspace, vmat, out, batch, s_ws, (int64_t)n * d, m * d, stream);
}

// ---- attention without a caller workspace --------------------------------------------------------------------
//
// Scratch for vs_attention_cvse_static: the probabilities between its SDDMM, softmax and SpMM steps.  The array
// is part of the library image, so every GPU that loads the library carries these 8 MiB until the process exits.
// In host code the NAME below is only a handle; the device address comes from cudaGetSymbolAddress.
constexpr size_t kStaticScratchBytes = size_t(8) << 20;
static __device__ __align__(256) unsigned char g_attention_scratch[kStaticScratchBytes];

namespace {
void *g_attention_scratch_ptr[kMaxDevices];   // device address of the array, looked up once per device
std::mutex g_attention_scratch_mutex;

// Must run with the target device current.  The look-up is a runtime query, not an allocation.
int attention_scratch(void **out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= kMaxDevices) return VS_ERR_ARG;
    std::lock_guard<std::mutex> lock(g_attention_scratch_mutex);
    if (!g_attention_scratch_ptr[dev]) {
        void *ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_attention_scratch);
        if (e != cudaSuccess) return (int)e;
        g_attention_scratch_ptr[dev] = ptr;
    }
    *out = g_attention_scratch_ptr[dev];
    return VS_OK;
}
}  // namespace

VS_EXPORT int vs_attention_cvse_static(int path, int m_vec, int vec_length, int n, int d, int nonzeros_vec,
                                       const int32_t *row_indices, const int32_t *row_offsets,
                                       const int32_t *col_indices, const void *q, const void *kmat, const void *vmat,
                                       void *out, float scale, int batch, void *stream) {
    if (batch < 1) return VS_ERR_ARG;
    if (nonzeros_vec < 0) return VS_ERR_SHAPE;
    if (!valid_v(vec_length)) return VS_ERR_VEC_LENGTH;
    const unsigned long long need = 2ull * (unsigned long long)batch * (unsigned long long)nonzeros_vec * (unsigned long long)vec_length;
    if (need > kStaticScratchBytes) {
        fprintf(stderr,
                "vs_attention_cvse_static: batch * nonzeros_vec * vec_length = %llu fp16 probabilities need %llu bytes, "
                "the built-in scratch holds %zu; use vs_attention_cvse with a workspace of your own\n",
                need / 2, need, kStaticScratchBytes);
        return VS_ERR_SHAPE;
    }
    void *scratch = nullptr;
    int rc = attention_scratch(&scratch);
    if (rc != VS_OK) return rc;
    NoScratchScope no_allocation;   // SDDMM and SpMM below: the formulations without plan scratch
    return vs_attention_cvse(path, m_vec, vec_length, n, d, nonzeros_vec, row_indices, row_offsets, col_indices, q, kmat,
                             vmat, out, scratch, scale, batch, stream);
}

// ---- host-buffer forms -------------------------------------------------------------------------------------

namespace {
struct DeviceBuffers {  // frees whatever was allocated when it goes out of scope
    void *ptr[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    int count = 0;
    cudaError_t alloc(void **out, size_t bytes) {
        cudaError_t e = cudaMalloc(out, bytes ? bytes : 16);
        if (e == cudaSuccess) ptr[count++] = *out;
        return e;
    }
    ~DeviceBuffers() {
        for (int i = 0; i < count; ++i) cudaFree(ptr[i]);
    }
};
}  // namespace

VS_EXPORT int vs_spmm_host(int path, int in_dtype, int out_dtype, int m_vec, int vec_length, int k, int n,
                           const int32_t *row_indices, const int32_t *row_offsets, const int32_t *col_indices,
                           const void *values, const void *rhs_matrix, void *output_matrix) {
    if (m_vec < 0 || k < 0 || n < 0) return VS_ERR_SHAPE;
    if (!valid_v(vec_length)) return VS_ERR_VEC_LENGTH;
    if ((in_dtype != VS_F16 && in_dtype != VS_F32) || (out_dtype != VS_F16 && out_dtype != VS_F32)) return VS_ERR_DTYPE;
    if (!row_indices || !row_offsets || !output_matrix) return VS_ERR_NULL;
    const int nnz_vec = row_offsets[m_vec];
    int rc = vs_cvse_validate(m_vec, n, nnz_vec, row_offsets, col_indices);
    if (rc != VS_OK) return rc;
    if (nnz_vec > 0 && (!values || !rhs_matrix)) return VS_ERR_NULL;
    const size_t si = elem_size(in_dtype), so = elem_size(out_dtype);
    const size_t b_idx = (size_t)m_vec * 4, b_off = (size_t)(m_vec + 1) * 4, b_col = (size_t)nnz_vec * 4;
    const size_t b_val = (size_t)nnz_vec * vec_length * si, b_rhs = (size_t)n * k * si;
    const size_t b_out = (size_t)m_vec * vec_length * k * so;
    DeviceBuffers bufs;
    int32_t *d_idx, *d_off, *d_col;
    void *d_val, *d_rhs, *d_out;
    VS_CUDA_TRY(bufs.alloc((void **)&d_idx, b_idx));
    VS_CUDA_TRY(bufs.alloc((void **)&d_off, b_off));
    VS_CUDA_TRY(bufs.alloc((void **)&d_col, b_col));
    VS_CUDA_TRY(bufs.alloc(&d_val, b_val));
    VS_CUDA_TRY(bufs.alloc(&d_rhs, b_rhs));
    VS_CUDA_TRY(bufs.alloc(&d_out, b_out));
    VS_CUDA_TRY(cudaMemcpy(d_idx, row_indices, b_idx, cudaMemcpyHostToDevice));
    VS_CUDA_TRY(cudaMemcpy(d_off, row_offsets, b_off, cudaMemcpyHostToDevice));
    if (b_col) VS_CUDA_TRY(cudaMemcpy(d_col, col_indices, b_col, cudaMemcpyHostToDevice));
    if (b_val) VS_CUDA_TRY(cudaMemcpy(d_val, values, b_val, cudaMemcpyHostToDevice));
    if (b_rhs) VS_CUDA_TRY(cudaMemcpy(d_rhs, rhs_matrix, b_rhs, cudaMemcpyHostToDevice));
    rc = vs_spmm(path, in_dtype, out_dtype, m_vec, vec_length, k, n, d_idx, d_off, d_col, d_val, d_rhs, d_out, nullptr);
    if (rc != VS_OK) return rc;
    VS_CUDA_TRY(cudaDeviceSynchronize());
    if (b_out) VS_CUDA_TRY(cudaMemcpy(output_matrix, d_out, b_out, cudaMemcpyDeviceToHost));
    return VS_OK;
}

VS_EXPORT int vs_sddmm_host(int path, int in_dtype, int out_dtype, int m_vec, int k, int n, int nonzeros_vec,
                            const int32_t *row_indices, const int32_t *row_offsets, const int32_t *col_indices,
                            const void *lhs_matrix, const void *rhs_matrix, void *output_values, int vec_length,
                            int algorithm) {
    if (m_vec < 0 || k < 0 || n < 0 || nonzeros_vec < 0) return VS_ERR_SHAPE;
    if (!valid_v(vec_length)) return VS_ERR_VEC_LENGTH;
    if ((in_dtype != VS_F16 && in_dtype != VS_F32) || (out_dtype != VS_F16 && out_dtype != VS_F32)) return VS_ERR_DTYPE;
    if (!row_indices || !row_offsets) return VS_ERR_NULL;
    int rc = vs_cvse_validate(m_vec, n, nonzeros_vec, row_offsets, col_indices);
    if (rc != VS_OK) return rc;
    if (nonzeros_vec > 0 && (!lhs_matrix || !rhs_matrix || !output_values)) return VS_ERR_NULL;
    const size_t si = elem_size(in_dtype), so = elem_size(out_dtype);
    const size_t b_idx = (size_t)m_vec * 4, b_off = (size_t)(m_vec + 1) * 4, b_col = (size_t)nonzeros_vec * 4;
    const size_t b_lhs = (size_t)m_vec * vec_length * k * si, b_rhs = (size_t)n * k * si;
    const size_t b_out = (size_t)nonzeros_vec * vec_length * so;
    DeviceBuffers bufs;
    int32_t *d_idx, *d_off, *d_col;
    void *d_lhs, *d_rhs, *d_out;
    VS_CUDA_TRY(bufs.alloc((void **)&d_idx, b_idx));
    VS_CUDA_TRY(bufs.alloc((void **)&d_off, b_off));
    VS_CUDA_TRY(bufs.alloc((void **)&d_col, b_col));
    VS_CUDA_TRY(bufs.alloc(&d_lhs, b_lhs));
    VS_CUDA_TRY(bufs.alloc(&d_rhs, b_rhs));
    VS_CUDA_TRY(bufs.alloc(&d_out, b_out));
    VS_CUDA_TRY(cudaMemcpy(d_idx, row_indices, b_idx, cudaMemcpyHostToDevice));
    VS_CUDA_TRY(cudaMemcpy(d_off, row_offsets, b_off, cudaMemcpyHostToDevice));
    if (b_col) VS_CUDA_TRY(cudaMemcpy(d_col, col_indices, b_col, cudaMemcpyHostToDevice));
    if (b_lhs) VS_CUDA_TRY(cudaMemcpy(d_lhs, lhs_matrix, b_lhs, cudaMemcpyHostToDevice));
    if (b_rhs) VS_CUDA_TRY(cudaMemcpy(d_rhs, rhs_matrix, b_rhs, cudaMemcpyHostToDevice));
    rc = vs_sddmm(path, in_dtype, out_dtype, m_vec, k, n, nonzeros_vec, d_idx, d_off, d_col, d_lhs, d_rhs, d_out,
                  vec_length, nullptr, algorithm);
    if (rc != VS_OK) return rc;
    VS_CUDA_TRY(cudaDeviceSynchronize());
    if (b_out) VS_CUDA_TRY(cudaMemcpy(output_values, d_out, b_out, cudaMemcpyDeviceToHost));
    return VS_OK;
}

VS_EXPORT int64_t vs_spmm_workspace_bytes(int m_vec, int vec_length, int n, int batch, int64_t stride_values) {
    if (m_vec <= 0 || n <= 0 || batch < 1 || !(vec_length == 2 || vec_length == 4 || vec_length == 8)) return 0;
    const int64_t bytes = spmm_plan_bytes(m_vec, vec_length, n, batch, stride_values, nullptr, nullptr);
    return bytes <= kMaxPlanBytes ? bytes : 0;
}

VS_EXPORT int64_t vs_spmm_t_workspace_bytes(int m_vec, int vec_length, int n, int batch, int64_t stride_values) {
    if (m_vec <= 0 || n <= 0 || batch < 1 || !valid_v(vec_length) || (int64_t)m_vec * vec_length > 0x7fffffffll) return 0;
    const int64_t bytes = spmm_t_plan_bytes(n, m_vec, vec_length, batch, stride_values, nullptr, nullptr);
    return bytes <= kMaxPlanBytes ? bytes : 0;
}

VS_EXPORT int64_t vs_sddmm_workspace_bytes(int m_vec, int n, int nonzeros_vec) {
    if (m_vec <= 0 || n <= 0 || nonzeros_vec <= 0) return 0;
    const int64_t bytes = sddmm_plan_bytes(m_vec, n, nonzeros_vec, nullptr);
    return bytes <= kMaxPlanBytes ? bytes : 0;
}

VS_EXPORT int vs_set_workspace(void *workspace, int64_t bytes) {
    if (bytes < 0 || (workspace == nullptr && bytes != 0)) return VS_ERR_ARG;
    if (!aligned16(workspace)) return VS_ERR_ALIGN;
    t_ws_set = workspace != nullptr;
    t_ws_ptr = workspace;
    t_ws_bytes = bytes;
    return VS_OK;
}

VS_EXPORT int vs_release_scratch(void *stream, int every_stream) {
    DeviceInfo *d;
    int rc = device_info(&d);
    if (rc != VS_OK) return rc;
    std::lock_guard<std::mutex> lock(g_devices_mutex);
    if (every_stream) {
        for (auto &kv : d->scratch)
            if (kv.second.ptr) (void)cudaFreeAsync(kv.second.ptr, kv.first.stream);
        d->scratch.clear();
        return VS_OK;
    }
    auto it = d->scratch.find(DeviceInfo::key_of(static_cast<cudaStream_t>(stream)));
    if (it != d->scratch.end()) {
        if (it->second.ptr) (void)cudaFreeAsync(it->second.ptr, it->first.stream);
        d->scratch.erase(it);
    }
    return VS_OK;
}

VS_EXPORT int vs_sddmm_formulation(int m_vec, int k, int n, int nonzeros_vec, int vec_length) {
    if (m_vec <= 0 || n <= 0 || k < densesddmm::kBlockK || nonzeros_vec <= 0 || !(vec_length == 2 || vec_length == 4 || vec_length == 8))
        return 0;
    SddmmParams p{};
    p.m_vec = m_vec; p.k = k; p.n = n; p.nnz_vec = nonzeros_vec;
    return sddmm_use_dense(p, vec_length) ? 1 : 0;
}

VS_EXPORT int vs_kernel_timing(int enable, double *total_ms, int *launches) {
    KernelTiming &t = kernel_timing();
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> done;
    {
        std::lock_guard<std::mutex> g(t.lock);
        done.swap(t.pairs);
        t.on = enable != 0;
    }
    double ms = 0.0;
    int n = 0, rc = VS_OK;
    for (auto &pr : done) {
        float x = 0.0f;
        cudaError_t e = cudaEventSynchronize(pr.second);
        if (e == cudaSuccess) e = cudaEventElapsedTime(&x, pr.first, pr.second);
        if (e == cudaSuccess) { ms += x; ++n; } else { rc = (int)e; (void)cudaGetLastError(); }
        cudaEventDestroy(pr.first);
        cudaEventDestroy(pr.second);
    }
    if (total_ms) *total_ms = ms;
    if (launches) *launches = n;
    return rc;
}

VS_EXPORT int vs_measure_fp32_fma(double *tflops) {
    if (!tflops) return VS_ERR_NULL;
    DeviceInfo *d;
    int rc = device_info(&d);
    if (rc != VS_OK) return rc;
    const int iters = 1 << 14, blocks = d->sm_count * 8, threads = 256;
    cudaEvent_t e0, e1;
    VS_CUDA_TRY(cudaEventCreate(&e0));
    VS_CUDA_TRY(cudaEventCreate(&e1));
    float *sink = nullptr;
    fp32_fma_probe_kernel<<<blocks, threads>>>(iters, 1.0f, sink);   // warm-up
    double best = 0.0;
    for (int rep = 0; rep < 3; ++rep) {
        cudaEventRecord(e0);
        fp32_fma_probe_kernel<<<blocks, threads>>>(iters, 1.0f, sink);
        cudaEventRecord(e1);
        cudaError_t e = cudaEventSynchronize(e1);
        float ms = 0.0f;
        if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
        if (e != cudaSuccess) {
            cudaEventDestroy(e0);
            cudaEventDestroy(e1);
            return (int)e;
        }
        const double t = 2.0 * 8.0 * iters * (double)blocks * threads / (ms * 1e-3) / 1e12;
        if (t > best) best = t;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *tflops = best;
    return VS_OK;
}

VS_EXPORT int vs_device_status(int clear, uint32_t *status) {
    if (!status) return VS_ERR_NULL;
    DeviceInfo *d;
    int rc = device_info(&d);
    if (rc != VS_OK) return rc;
    VS_CUDA_TRY(cudaDeviceSynchronize());
    VS_CUDA_TRY(cudaMemcpy(status, d->status, sizeof(uint32_t), cudaMemcpyDeviceToHost));
    if (clear) VS_CUDA_TRY(cudaMemset(d->status, 0, sizeof(uint32_t)));
    return VS_OK;
}

VS_EXPORT int vs_selftest_gather4(const void *matrix, int rows, int cols, const int32_t *row_indices, int groups,
                                  int x, void *out, void *stream) {
    if (!matrix || !row_indices || !out) return VS_ERR_NULL;
    if (rows < 1 || cols < 64 || cols % 8 != 0 || groups < 1 || groups > 32 || x < 0 || x % 8 != 0) return VS_ERR_SHAPE;
    if (!aligned16(matrix) || !aligned16(out)) return VS_ERR_ALIGN;
    DeviceInfo *d;
    int rc = device_info(&d);
    if (rc != VS_OK) return rc;
    CUtensorMap map;
    rc = make_gather_map(&map, matrix, (uint64_t)rows, (uint64_t)cols);
    if (rc != VS_OK) return rc;
    const int smem = groups * 512 + 64 + 1024;
    tcselftest::gather4_kernel<<<1, 32, smem, static_cast<cudaStream_t>(stream)>>>(
        map, row_indices, groups, x, static_cast<uint8_t *>(out), d->status);
    return (int)cudaGetLastError();
}



namespace {
// Whether the 16 contraction elements x `rows` fp16 operand a shared-memory descriptor names lies inside an image
// of `image_bytes` (descriptor start relative to the image).  Only the layouts the kernels use are accepted:
// no swizzle or the 128-byte swizzle, either major.
bool selftest_operand_fits(uint64_t desc, int rows, bool mn_major, int image_bytes) {
    const int64_t start = (int64_t)(desc & 0x3fffu) << 4, lbo = (int64_t)((desc >> 16) & 0x3fffu) << 4,
                  sbo = (int64_t)((desc >> 32) & 0x3fffu) << 4;
    const unsigned swizzle = (unsigned)(desc >> 61) & 7u;
    if (swizzle != 0 && swizzle != 2) return false;
    if (rows < 8 || rows % 8 != 0) return false;
    int64_t end;
    if (swizzle == 2 && mn_major) {          // atoms of 64 rows x 8 contraction elements (1 KiB): LBO between atoms along the rows, SBO along the contraction
        if (rows % 64 != 0) return false;
        end = start + (rows / 64 - 1) * lbo + sbo + 1024;
    } else if (swizzle == 2) {               // rows of 128 bytes, eight to a 1 KiB block, SBO between blocks; the 32 bytes of a step stay inside a row
        if (start % 128 + 32 > 128) return false;
        end = start - start % 128 + (rows / 8 - 1) * sbo + 1024;
    } else {                                 // unswizzled: 128-byte core matrices, LBO between them along the contraction, SBO along the rows
        end = start + (rows / 8 - 1) * sbo + lbo + 128;
    }
    return start >= 0 && end <= image_bytes;
}
// Decodes what the self-test kernels rely on from an instruction descriptor; false for anything else.
bool selftest_idesc(uint32_t idesc, int max_m, int *M, int *N, bool *a_mn, bool *b_mn) {
    *N = (int)((idesc >> 17) & 0x3fu) << 3;
    *M = (int)((idesc >> 24) & 0x1fu) << 4;
    *a_mn = (idesc >> 15) & 1u;
    *b_mn = (idesc >> 16) & 1u;
    if ((idesc & ~((0x3fu << 17) | (0x1fu << 24) | (1u << 15) | (1u << 16))) != (1u << 4)) return false;   // fp16 x fp16 -> fp32 only
    return *M == max_m && *N >= 16 && *N <= 256 && *N % 16 == 0;
}
}  // namespace

VS_EXPORT int vs_selftest_mma(const void *image, int image_bytes, const uint64_t *descs_host, int n_mma,
                              uint32_t idesc, int ncols, float fill, float *out, void *stream) {
    if (!image || !descs_host || !out) return VS_ERR_NULL;
    if (image_bytes <= 0 || image_bytes > 128 * 1024 || n_mma < 1 || n_mma > 64) return VS_ERR_SHAPE;
    if (ncols < 8 || ncols > tcselftest::kTmemCols || ncols % 8 != 0) return VS_ERR_SHAPE;
    if (!aligned16(image)) return VS_ERR_ALIGN;
    int M, N;
    bool a_mn, b_mn;
    if (!selftest_idesc(idesc, 128, &M, &N, &a_mn, &b_mn) || N > ncols) return VS_ERR_SHAPE;
    for (int i = 0; i < n_mma; ++i)
        if (!selftest_operand_fits(descs_host[2 * i], M, a_mn, image_bytes) || !selftest_operand_fits(descs_host[2 * i + 1], N, b_mn, image_bytes))
            return VS_ERR_SHAPE;
    DeviceInfo *d;
    int rc = device_info(&d);
    if (rc != VS_OK) return rc;
    const int smem = ((image_bytes + 15) & ~15) + 16 + 1024;
    rc = set_smem(tcselftest::sandbox_kernel, smem);
    if (rc != VS_OK) return rc;
    tcselftest::DescList descs;
    std::memcpy(descs.d, descs_host, sizeof(uint64_t) * 2 * n_mma);
    tcselftest::sandbox_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t *>(image), image_bytes, descs, n_mma, idesc, ncols, fill, out, d->status);
    return (int)cudaGetLastError();
}

VS_EXPORT int vs_selftest_mma_pair(const void *image0, const void *image1, int image_bytes, const uint64_t *descs_host,
                                   int n_mma, uint32_t idesc, int ncols, float fill, float *out, void *stream) {
    if (!image0 || !image1 || !descs_host || !out) return VS_ERR_NULL;
    if (image_bytes <= 0 || image_bytes > 128 * 1024 || n_mma < 1 || n_mma > 64) return VS_ERR_SHAPE;
    if (ncols < 8 || ncols > tcselftest::kPairTmemCols || ncols % 8 != 0) return VS_ERR_SHAPE;
    if (!aligned16(image0) || !aligned16(image1)) return VS_ERR_ALIGN;
    int M, N;
    bool a_mn, b_mn;
    if (!selftest_idesc(idesc, 256, &M, &N, &a_mn, &b_mn) || N > ncols || N % 32 != 0) return VS_ERR_SHAPE;
    for (int i = 0; i < n_mma; ++i)   // per CTA: 128 rows of A, N / 2 columns of B
        if (!selftest_operand_fits(descs_host[2 * i], 128, a_mn, image_bytes) || !selftest_operand_fits(descs_host[2 * i + 1], N / 2, b_mn, image_bytes))
            return VS_ERR_SHAPE;
    DeviceInfo *d;
    int rc = device_info(&d);
    if (rc != VS_OK) return rc;
    const int smem = ((image_bytes + 15) & ~15) + 16 + 1024;
    rc = set_smem(tcselftest::sandbox_pair_kernel, smem);
    if (rc != VS_OK) return rc;
    tcselftest::DescList descs;
    std::memcpy(descs.d, descs_host, sizeof(uint64_t) * 2 * n_mma);
    return (int)launch_pairs(tcselftest::sandbox_pair_kernel, 1, 128, (size_t)smem, static_cast<cudaStream_t>(stream), false,
                             static_cast<const uint8_t *>(image0), static_cast<const uint8_t *>(image1), image_bytes, descs, n_mma,
                             idesc, ncols, fill, out, d->status);
}
