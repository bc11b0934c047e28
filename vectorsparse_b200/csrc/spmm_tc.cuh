// Tensor-core SpMM for fp16 CVSE matrices on sm_100a: the `wmmaSpmm` entry point of the reference
// (src/wmma_spmm.cu:13-314 are its three Volta mma.m8n8k4 kernels) rebuilt on tcgen05.
//
// Formulation.  For one vector-row r and one tile of 128 dense columns the kernel computes, transposed,
//     D[128 cols x 16] (+)= Bg^T[128 cols x 16 nnz] * Ar^T[16 nnz x 16]
// Bg = the rows of the dense operand selected by col_indices, Ar = the row's value vectors (V <= 8 of the 16
// columns are real, the rest are a constant zero block).  Both operands are MN-major in shared memory:
// a gathered row of B is contiguous along the 128 columns (MMA-M), a value vector is contiguous along V
// (MMA-N).  The accumulator lives in tensor memory, 16 fp32 columns per work item.
//
// Pipeline.  One CTA = 128 threads, persistent over work items (batch, column tile, vector-row in
// row_indices order), dealt round-robin so that the descending-length order the row swizzle produces becomes
// a longest-first schedule.  All threads gather: cp.async 16-byte chunks of B rows straight into the
// 128-byte-swizzled operand layout (zero-filled past the end of a row), 32 nonzero vectors per stage, several
// stages in flight.  Thread 0 issues the MMAs of a landed stage and commits them to that stage's mbarrier
// (slot reuse) and, at the end of a row, to the accumulator's mbarrier.  The epilogue of a row (tcgen05.ld,
// convert, store to C) runs two rows late so the tensor core's latency never stalls the gather.
// Every wait is bounded; a wait that runs out raises a status bit and the CTA leaves through the normal
// teardown (drain cp.async, free tensor memory).
#pragma once
#include "common.cuh"
#include "tc_ptx.cuh"

namespace vs {
namespace tcspmm {

constexpr int kThreads = 128;
constexpr int kTileN = 128;                              // dense columns per work item (MMA M)
constexpr int kStageNnz = 32;                            // nonzero vectors per stage (two K=16 MMAs)
constexpr int kStages = 8;                               // shared-memory ring
constexpr int kInflight = 5;                             // cp.async groups in flight behind the newest
constexpr int kAStageBytes = kStageNnz * kTileN * 2;     // 8 KiB
constexpr int kVStageBytes = kStageNnz * 16;             // 512 B: one 16-byte slot per nonzero vector
constexpr int kAccCols = 16;                             // TMEM columns per accumulator
constexpr int kTmemCols = 128;
constexpr int kAccSlots = kTmemCols / kAccCols;          // 8
constexpr int kEpiLag = 2;                               // rows between MMA issue and epilogue
constexpr int kMetaRing = 16;
constexpr int kItemsPerPhase = 256;

constexpr uint32_t kStatusTimeout = 1u;  // bit raised in the status word when a bounded wait ran out

struct StageMeta {
    int row, b, n0, n_mma, accslot, flags;  // flags: bit0 first stage of the row, bit1 last, bit2 acc parity
};

struct Smem {  // offsets from the 1024-byte aligned base
    static constexpr int kA = 0;
    static constexpr int kV = kA + kStages * kAStageBytes;
    static constexpr int kZ = kV + kStages * kVStageBytes;       // zero block: the N = 8..15 half of operand B
    static constexpr int kRow = kZ + kStages * kVStageBytes;
    static constexpr int kJ0 = kRow + kItemsPerPhase * 4;
    static constexpr int kEnd = kJ0 + kItemsPerPhase * 4;
    static constexpr int kMeta = kEnd + kItemsPerPhase * 4;
    static constexpr int kBarEmpty = kMeta + kMetaRing * (int)sizeof(StageMeta);
    static constexpr int kBarAcc = kBarEmpty + kStages * 8;
    static constexpr int kTmemHolder = kBarAcc + kAccSlots * 8;
    static constexpr int kTotal = kTmemHolder + 16;
};
constexpr int kSmemBytes = Smem::kTotal + 1024;  // + slack for the manual 1024-byte alignment

struct Pending {
    int row, b, n0, accslot, parity;
};

template <typename TOut, int V>
__global__ void __launch_bounds__(kThreads) spmm_tc_kernel(const SpmmParams p, uint32_t *status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = tc::smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);

    const int t = threadIdx.x;
    const int warp = t >> 5;
    int *l_row = reinterpret_cast<int *>(sm + Smem::kRow);
    int *l_j0 = reinterpret_cast<int *>(sm + Smem::kJ0);
    int *l_end = reinterpret_cast<int *>(sm + Smem::kEnd);
    StageMeta *meta = reinterpret_cast<StageMeta *>(sm + Smem::kMeta);
    volatile uint32_t *tmem_holder = reinterpret_cast<volatile uint32_t *>(sm + Smem::kTmemHolder);
    const uint32_t bar_empty = base + Smem::kBarEmpty;
    const uint32_t bar_acc = base + Smem::kBarAcc;

    // ---- set-up: zero the value slots and the zero block, barriers, tensor memory -------------------------
    for (int i = t; i < 2 * kStages * kVStageBytes / 16; i += kThreads)
        reinterpret_cast<uint4 *>(sm + Smem::kV)[i] = make_uint4(0, 0, 0, 0);
    if (t == 0) {
        for (int s = 0; s < kStages; ++s) tc::mbar_init(bar_empty + 8 * s, 1);
        for (int s = 0; s < kAccSlots; ++s) tc::mbar_init(bar_acc + 8 * s, 1);
        tc::fence_mbar_init();
    }
    if (warp == 0) {
        tc::tmem_alloc(base + Smem::kTmemHolder, kTmemCols);
        tc::tmem_relinquish();
    }
    tc::fence_proxy_async();
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    const int n_tiles = (p.N + kTileN - 1) / kTileN;
    const int64_t total_items = (int64_t)p.batch * n_tiles * p.m_vec;
    const int64_t G = gridDim.x;
    const int64_t my_items = (total_items > blockIdx.x) ? (total_items - blockIdx.x + G - 1) / G : 0;

    constexpr uint32_t kIdesc = tc::make_idesc_f16(kTileN, 16, 1, 1);
    const int chunk = t & 15;       // 16-byte chunk of the 256-byte row segment this thread copies
    const int rsub = t >> 4;        // row within each group of eight
    // destination of this thread's chunk inside a stage, for row group i add i*1024
    const uint32_t a_dst0 = (uint32_t)((chunk >> 3) * (kAStageBytes / 2) + rsub * 128 + (((chunk & 7) ^ rsub) << 4));

    uint32_t g_stage = 0;   // stages issued so far by this CTA (ring position and barrier parity)
    uint32_t g_item = 0;    // rows started so far (accumulator slot and parity)
    int timeout = 0;
    bool aborted = false;

    for (int64_t ph0 = 0; ph0 < my_items && !aborted; ph0 += kItemsPerPhase) {
        const int cnt = (int)((my_items - ph0 < kItemsPerPhase) ? (my_items - ph0) : kItemsPerPhase);
        // ---- phase set-up: decode this CTA's next rows in bulk (one round of global latency) ------------
        for (int q = t; q < cnt; q += kThreads) {
            const int64_t w = blockIdx.x + (ph0 + q) * G;
            const int o = (int)(w % p.m_vec);
            const int row = __ldg(p.row_indices + o);
            l_row[q] = row;
            l_j0[q] = __ldg(p.row_offsets + row);
            l_end[q] = __ldg(p.row_offsets + row + 1);
        }
        __syncthreads();

        // ---- stage iterator (identical in every thread) ------------------------------------------------
        int q = 0;                       // item within the phase
        int j = l_j0[0], jend = l_end[0];
        bool first = true;
        int idx[4];
        auto prefetch = [&]() {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int jj = j + rsub + 8 * i;
                idx[i] = (jj < jend) ? __ldg(p.col_indices + jj) : 0;
            }
        };
        prefetch();

        Pending fifo[kEpiLag];  // fifo[kEpiLag - fifo_n .. kEpiLag) are valid, oldest first
#pragma unroll
        for (int i = 0; i < kEpiLag; ++i) fifo[i] = Pending{0, 0, 0, 0, 0};
        int fifo_n = 0;
        const uint32_t g_base = g_stage;
        int phase_stages = -1;  // known once the iterator runs dry

        auto epilogue = [&](const Pending &e) {
            if (!tc::mbar_wait(bar_acc + 8 * e.accslot, (uint32_t)e.parity)) timeout = 1;
            tc::tc_fence_after_sync();
            uint32_t r[8];
            tc::tmem_ld_x8(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(e.accslot * kAccCols), r);
            tc::tmem_ld_wait();
            tc::tc_fence_before_sync();
            const int col = e.n0 + t;
            if (col < p.N) {
                TOut *o = static_cast<TOut *>(p.out) + (int64_t)e.b * p.stride_out + (int64_t)e.row * V * p.N + col;
#pragma unroll
                for (int v = 0; v < V; ++v) store_scalar(o + (int64_t)v * p.N, __uint_as_float(r[v]));
            }
        };

        for (int it = 0;; ++it) {
            // ---- issue side ---------------------------------------------------------------------------
            if (q < cnt) {
                const uint32_t slot = g_stage % kStages;
                if (g_stage >= (uint32_t)kStages) {
                    if (!tc::mbar_wait(bar_empty + 8 * slot, ((g_stage / kStages) - 1u) & 1u)) timeout = 1;
                }
                const int64_t w = blockIdx.x + (ph0 + q) * G;
                const int tile = (int)((w / p.m_vec) % n_tiles);
                const int b = (int)(w / ((int64_t)p.m_vec * n_tiles));
                const int n0 = tile * kTileN;
                const int nnz = min(kStageNnz, max(0, jend - j));
                const int n_mma = max(1, (nnz + 15) >> 4);
                const bool last = (j + kStageNnz >= jend);

                const __half *rhs = static_cast<const __half *>(p.rhs) + (int64_t)b * p.stride_rhs;
                const bool col_ok = (n0 + chunk * 8) < p.N;
                const uint32_t a_dst = base + Smem::kA + slot * kAStageBytes + a_dst0;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (i < 2 * n_mma) {
                        const bool ok = col_ok && (rsub + 8 * i) < nnz;
                        const __half *src = ok ? rhs + (int64_t)idx[i] * p.N + n0 + chunk * 8 : rhs;
                        tc::cp_async_16(a_dst + i * 1024, src, ok ? 16u : 0u);
                    }
                }
                if (t < 16 * n_mma) {
                    const __half *vals = static_cast<const __half *>(p.values) + (int64_t)b * p.stride_values;
                    const bool ok = t < nnz;
                    tc::cp_async_small<V * 2>(base + Smem::kV + slot * kVStageBytes + t * 16,
                                              ok ? vals + (int64_t)(j + t) * V : vals, ok ? (uint32_t)(V * 2) : 0u);
                }
                if (t == 0) {
                    StageMeta m;
                    m.row = l_row[q]; m.b = b; m.n0 = n0; m.n_mma = n_mma;
                    m.accslot = (int)(g_item % kAccSlots);
                    m.flags = (first ? 1 : 0) | (last ? 2 : 0) | ((int)((g_item / kAccSlots) & 1u) << 2);
                    meta[g_stage % kMetaRing] = m;
                }
                ++g_stage;
                if (last) {
                    ++g_item;
                    ++q;
                    first = true;
                    if (q < cnt) { j = l_j0[q]; jend = l_end[q]; }
                } else {
                    j += kStageNnz;
                    first = false;
                }
                if (q < cnt) prefetch();
                else phase_stages = (int)(g_stage - g_base);
            }
            tc::cp_async_commit();

            // ---- consume side: the stage issued kInflight iterations ago has landed ----------------------
            const int cs = it - kInflight;
            if (cs >= 0) {
                tc::cp_async_wait<kInflight>();
                tc::fence_proxy_async();
            }
            tc::tc_fence_before_sync();
            if (__syncthreads_or(timeout)) { aborted = true; break; }
            if (cs >= 0) {
                const uint32_t gs = g_base + (uint32_t)cs;
                const uint32_t slot = gs % kStages;
                const StageMeta m = meta[gs % kMetaRing];
                if (t == 0) {
                    tc::tc_fence_after_sync();
                    const uint32_t d = tmem_base + (uint32_t)(m.accslot * kAccCols);
#pragma unroll 1
                    for (int mm = 0; mm < m.n_mma; ++mm) {
                        const uint64_t ad = tc::make_smem_desc(base + Smem::kA + slot * kAStageBytes + mm * 2048,
                                                               kAStageBytes / 2, 1024, tc::kSwizzle128B);
                        const uint64_t bd = tc::make_smem_desc(base + Smem::kV + slot * kVStageBytes + mm * 256, 128,
                                                               kStages * kVStageBytes, tc::kSwizzleNone);
                        tc::mma_f16_ss(d, ad, bd, kIdesc, ((m.flags & 1) && mm == 0) ? 0u : 1u);
                    }
                    tc::mma_commit(bar_empty + 8 * slot);
                    if (m.flags & 2) tc::mma_commit(bar_acc + 8 * m.accslot);
                }
                if (m.flags & 2) {
                    // shift register of rows whose epilogue is owed: the oldest one is served now
                    const Pending oldest = fifo[0];
#pragma unroll
                    for (int i = 0; i + 1 < kEpiLag; ++i) fifo[i] = fifo[i + 1];
                    fifo[kEpiLag - 1].row = m.row; fifo[kEpiLag - 1].b = m.b; fifo[kEpiLag - 1].n0 = m.n0;
                    fifo[kEpiLag - 1].accslot = m.accslot; fifo[kEpiLag - 1].parity = (m.flags >> 2) & 1;
                    if (fifo_n == kEpiLag) epilogue(oldest);
                    else ++fifo_n;
                }
                if (phase_stages >= 0 && cs == phase_stages - 1) break;
            }
        }
        // ---- drain the rows whose epilogue is still owed ---------------------------------------------------
        if (!aborted) {
#pragma unroll
            for (int i = 0; i < kEpiLag; ++i)
                if (i >= kEpiLag - fifo_n) epilogue(fifo[i]);
        }
        tc::tc_fence_before_sync();
        if (__syncthreads_or(timeout)) aborted = true;
    }

    // ---- teardown ---------------------------------------------------------------------------------------
    tc::cp_async_wait<0>();
    if (aborted && t == 0) atomicOr(status, kStatusTimeout);
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace tcspmm
}  // namespace vs
