// Self-test of the tcgen05 operand encodings: runs a handful of MMAs on a caller-built shared-memory image and
// returns the raw accumulator, so that the host can check a descriptor / layout convention against a plain
// matrix product.  Used by the GPU tests; never on a product path.
#pragma once
#include <cuda.h>

#include "tc_ptx.cuh"

namespace vs {
namespace tcselftest {

constexpr uint32_t kStatusTimeout = 4u;
constexpr int kTmemCols = 128;
constexpr int kMaxMma = 64;
struct DescList {   // (A, B) descriptor pairs, passed by value: the host has checked every one against the image
    uint64_t d[2 * kMaxMma];
};

__device__ __forceinline__ void tmem_st_x8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// image: bytes copied to the 1024-byte aligned start of shared memory.  descs: n_mma pairs (A, B) of 64-bit
// descriptors whose start-address field is RELATIVE to the image start (checked on the host to stay inside it).  The accumulator (128 lanes x ncols
// fp32 columns, ncols a multiple of 8 up to 128) is pre-filled with `fill`, so lanes an instruction shape does
// not write can be told apart, and copied to out[lane * ncols + col].
__global__ void __launch_bounds__(128) sandbox_kernel(const uint8_t *image, int image_bytes, const DescList descs,
                                                      int n_mma, uint32_t idesc, int ncols, float fill, float *out,
                                                      uint32_t *status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = tc::smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);
    const int padded = (image_bytes + 15) & ~15;
    const uint32_t bar = base + padded;          // 8-byte mbarrier
    const uint32_t holder = bar + 8;             // tensor-memory base address
    const int t = threadIdx.x, warp = t >> 5;

    for (int i = t; i < padded / 16; i += 128) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (i * 16 + 16 <= image_bytes) v = reinterpret_cast<const uint4 *>(image)[i];
        reinterpret_cast<uint4 *>(sm)[i] = v;
    }
    if (t == 0) {
        tc::mbar_init(bar, 1);
        tc::fence_mbar_init();
    }
    if (warp == 0) {
        tc::tmem_alloc(holder, kTmemCols);
        tc::tmem_relinquish();
    }
    tc::fence_proxy_async();
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(sm + padded + 8);
    const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);

    uint32_t f[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = __float_as_uint(fill);
    for (int c = 0; c < ncols; c += 8) tmem_st_x8(lane_addr + c, f);
    tmem_st_wait();
    tc::tc_fence_before_sync();
    __syncthreads();

    if (t == 0) {
        tc::tc_fence_after_sync();
        for (int i = 0; i < n_mma; ++i) {
            const uint64_t a = descs.d[2 * i] + (uint64_t)(base >> 4);
            const uint64_t b = descs.d[2 * i + 1] + (uint64_t)(base >> 4);
            tc::mma_f16_ss(tmem_base, a, b, idesc, i > 0 ? 1u : 0u);
        }
        tc::mma_commit(bar);
    }
    const bool ok = tc::mbar_wait(bar, 0);
    tc::tc_fence_after_sync();
    for (int c = 0; c < ncols; c += 8) {
        uint32_t r[8];
        tc::tmem_ld_x8(lane_addr + c, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) out[(size_t)t * ncols + c + i] = __uint_as_float(r[i]);
    }
    if (!ok) atomicOr(status, kStatusTimeout);
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem_base, kTmemCols);
}

// The same sandbox for a PAIR of CTAs (a cluster of two, tcgen05 cta_group::2): each CTA copies its own image to
// the same shared-memory offsets, the leader CTA issues the MMAs for both and tells each CTA's barrier with a
// commit of its own; every CTA then copies its 128 accumulator lanes to out[(rank * 128 + lane) * ncols + col].
// Pins what the pair kernels rely on: with M = 256 CTA r owns rows 128 r .. 128 r + 127 of A and of the
// accumulator, and holds columns r * N / 2 .. of B.  ncols: a multiple of 8 up to 256.
constexpr int kPairTmemCols = 256;
constexpr uint32_t kStatusPairTimeout = 16u;
__global__ void __launch_bounds__(128) sandbox_pair_kernel(const uint8_t *image0, const uint8_t *image1, int image_bytes,
                                                           const DescList descs, int n_mma, uint32_t idesc, int ncols,
                                                           float fill, float *out, uint32_t *status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = tc::smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);
    const int padded = (image_bytes + 15) & ~15;
    const uint32_t bar = base + padded;          // 8-byte mbarrier
    const uint32_t holder = bar + 8;             // tensor-memory base address
    const int t = threadIdx.x, warp = t >> 5;
    const uint32_t rank = tc::cluster_ctarank();
    const uint8_t *image = rank == 0 ? image0 : image1;

    for (int i = t; i < padded / 16; i += 128) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (i * 16 + 16 <= image_bytes) v = reinterpret_cast<const uint4 *>(image)[i];
        reinterpret_cast<uint4 *>(sm)[i] = v;
    }
    if (t == 0) {
        tc::mbar_init(bar, 1);
        tc::fence_mbar_init();
    }
    if (warp == 0) {
        tc::tmem_alloc_pair(holder, kPairTmemCols);
        tc::tmem_relinquish_pair();
    }
    tc::fence_proxy_async();
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(sm + padded + 8);
    const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);

    uint32_t f[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = __float_as_uint(fill);
    for (int c = 0; c < ncols; c += 8) tmem_st_x8(lane_addr + c, f);
    tmem_st_wait();
    tc::tc_fence_before_sync();
    tc::cluster_sync();   // both images, both barriers and both accumulators are in place
    tc::tc_fence_after_sync();

    if (rank == 0 && t == 0) {
        for (int i = 0; i < n_mma; ++i) {
            const uint64_t a = descs.d[2 * i] + (uint64_t)(base >> 4);
            const uint64_t b = descs.d[2 * i + 1] + (uint64_t)(base >> 4);
            tc::mma_f16_ss_pair(tmem_base, a, b, idesc, i > 0 ? 1u : 0u);
        }
        tc::mma_commit_pair(tc::map_to_cta(bar, 0));
        tc::mma_commit_pair(tc::map_to_cta(bar, 1));
    }
    bool ok = false;
    for (uint32_t i = 0; i < tc::kMaxPolls && !ok; ++i) ok = tc::mbar_try_wait_cluster(bar, 0);
    tc::tc_fence_after_sync();
    for (int c = 0; c < ncols; c += 8) {
        uint32_t r[8];
        tc::tmem_ld_x8(lane_addr + c, r);
#pragma unroll
        for (int i = 0; i < 8; ++i) out[((size_t)rank * 128 + t) * ncols + c + i] = __uint_as_float(r[i]);
    }
    if (!ok) atomicOr(status, kStatusPairTimeout << rank);
    tc::tc_fence_before_sync();
    tc::cluster_sync();   // neither CTA leaves (or frees tensor memory) while the other may still be read by an MMA
    if (warp == 0) tc::tmem_dealloc_pair(tmem_base, kPairTmemCols);
}

// Row-gather self-test: `groups` gather4 operations (4 row indices each, from `rows`) at column x into
// consecutive 512-byte blocks of a 1024-byte aligned buffer, which is then copied out raw.
constexpr uint32_t kStatusGatherTimeout = 8u;
__global__ void __launch_bounds__(32) gather4_kernel(const __grid_constant__ CUtensorMap map, const int *rows, int groups,
                                                    int x, uint8_t *out, uint32_t *status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = tc::smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);
    const int lane = threadIdx.x;
    const uint32_t bar = base + groups * 512;
    for (int i = lane; i < groups * 512 / 16; i += 32) reinterpret_cast<uint4 *>(sm)[i] = make_uint4(0xdeadbeefu, 0xdeadbeefu, 0xdeadbeefu, 0xdeadbeefu);
    if (lane == 0) {
        tc::mbar_init(bar, 1);
        tc::fence_mbar_init();
    }
    tc::fence_proxy_async();
    __syncwarp();
    if (lane == 0) tc::mbar_expect_tx(bar, (uint32_t)groups * 512u);
    __syncwarp();
    if (lane < groups)
        tc::tma_gather4(base + lane * 512, &map, bar, x, rows[4 * lane], rows[4 * lane + 1], rows[4 * lane + 2], rows[4 * lane + 3]);
    const bool ok = tc::mbar_wait(bar, 0);
    __syncwarp();
    for (int i = lane; i < groups * 512 / 16; i += 32) reinterpret_cast<uint4 *>(out)[i] = reinterpret_cast<uint4 *>(sm)[i];
    if (!ok && lane == 0) atomicOr(status, kStatusGatherTimeout);
}

}  // namespace tcselftest
}  // namespace vs
