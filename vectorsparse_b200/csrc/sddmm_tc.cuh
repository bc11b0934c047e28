// Tensor-core SDDMM for fp16 operands on sm_100a: the `wmmaSddmm` entry point of the reference
// (src/wmma_sddmm.cu holds its twelve Volta kernels: V = 8/4/2 times the four `algorithm` variants, all
// computing the same function; all four values map to this one kernel).
//
// Formulation.  For one vector-row i and one tile of 128 of its mask entries the kernel computes
//     D[128 entries x 16] (+)= Rg[128 entries x 64] * L_i^T[64 x 16]
// per 64-wide block of the contraction: Rg = rows of rhs selected by col_indices, L_i = the V (<= 8) lhs rows
// of the vector-row, zero-padded to 16.  Both operands are K-major in shared memory with the 128-byte swizzle
// (a gathered row is 64 fp16 = 128 bytes).  D row e, column v is out[(j0 + e) * V + v]: each thread of the
// epilogue owns one mask entry and stores its V outputs with one vector store, neighbouring threads writing
// neighbouring addresses.
//
// The pipeline is the one of the tensor-core SpMM: persistent CTAs of 128 threads over (batch, vector-row)
// items in row_indices order, cp.async gathers with zero fill for entries past the end of a row, one thread
// issuing MMAs, per-stage and per-accumulator mbarriers, epilogues two tiles late, every wait bounded.
#pragma once
#include "common.cuh"
#include "tc_ptx.cuh"

namespace vs {
namespace tcsddmm {

constexpr int kThreads = 128;
constexpr int kTileE = 128;                       // mask entries per tile (MMA M)
constexpr int kBlockK = 64;                       // contraction elements per stage (four K=16 MMAs)
constexpr int kStages = 5;
constexpr int kInflight = 3;
constexpr int kAStageBytes = kTileE * kBlockK * 2;  // 16 KiB gathered rhs rows
constexpr int kBStageBytes = 16 * kBlockK * 2;      // 2 KiB lhs rows (V real + zero padding)
constexpr int kAccCols = 16;
constexpr int kTmemCols = 128;
constexpr int kAccSlots = kTmemCols / kAccCols;
constexpr int kEpiLag = 2;
constexpr int kMetaRing = 16;
constexpr int kItemsPerPhase = 256;

constexpr uint32_t kStatusTimeout = 2u;

struct StageMeta {
    int jt, jend, b, accslot, flags;  // flags: bit0 first k-block of the tile, bit1 last, bit2 acc parity
};

struct Smem {
    static constexpr int kA = 0;
    static constexpr int kB = kA + kStages * kAStageBytes;
    static constexpr int kRow = kB + kStages * kBStageBytes;
    static constexpr int kJ0 = kRow + kItemsPerPhase * 4;
    static constexpr int kEnd = kJ0 + kItemsPerPhase * 4;
    static constexpr int kItemB = kEnd + kItemsPerPhase * 4;
    static constexpr int kMeta = kItemB + kItemsPerPhase * 4;
    static constexpr int kBarEmpty = kMeta + kMetaRing * (int)sizeof(StageMeta);
    static constexpr int kBarAcc = kBarEmpty + kStages * 8;
    static constexpr int kTmemHolder = kBarAcc + kAccSlots * 8;
    static constexpr int kTotal = kTmemHolder + 16;
};
constexpr int kSmemBytes = Smem::kTotal + 1024;

struct Pending {
    int jt, jend, b, accslot, parity;
};

template <typename TOut, int V>
__global__ void __launch_bounds__(kThreads) sddmm_tc_kernel(const SddmmParams p, uint32_t *status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = tc::smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);

    const int t = threadIdx.x;
    const int warp = t >> 5;
    int *l_row = reinterpret_cast<int *>(sm + Smem::kRow);
    int *l_j0 = reinterpret_cast<int *>(sm + Smem::kJ0);
    int *l_end = reinterpret_cast<int *>(sm + Smem::kEnd);
    int *l_b = reinterpret_cast<int *>(sm + Smem::kItemB);
    StageMeta *meta = reinterpret_cast<StageMeta *>(sm + Smem::kMeta);
    volatile uint32_t *tmem_holder = reinterpret_cast<volatile uint32_t *>(sm + Smem::kTmemHolder);
    const uint32_t bar_empty = base + Smem::kBarEmpty;
    const uint32_t bar_acc = base + Smem::kBarAcc;

    if (t == 0) {
        for (int s = 0; s < kStages; ++s) tc::mbar_init(bar_empty + 8 * s, 1);
        for (int s = 0; s < kAccSlots; ++s) tc::mbar_init(bar_acc + 8 * s, 1);
        tc::fence_mbar_init();
    }
    if (warp == 0) {
        tc::tmem_alloc(base + Smem::kTmemHolder, kTmemCols);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_holder;

    const int nkb = p.k / kBlockK;
    const int64_t total_items = (int64_t)p.batch * p.m_vec;
    const int64_t G = gridDim.x;
    const int64_t my_items = (total_items > blockIdx.x) ? (total_items - blockIdx.x + G - 1) / G : 0;

    constexpr uint32_t kIdesc = tc::make_idesc_f16(kTileE, 16, 0, 0);
    const int chunk = t & 7;          // 16-byte chunk of the 128-byte row block
    const int r0 = t >> 3;            // rows r0 + 16*i, i = 0..7
    const int rsw = r0 & 7;
    const uint32_t a_dst0 = (uint32_t)((r0 >> 3) * 1024 + rsw * 128 + ((chunk ^ rsw) << 4));  // + i*2048
    const uint32_t b_dst = (uint32_t)((r0 >> 3) * 1024 + rsw * 128 + ((chunk ^ rsw) << 4));   // lhs row r0

    uint32_t g_stage = 0, g_tile = 0;
    int timeout = 0;
    bool aborted = false;

    for (int64_t ph0 = 0; ph0 < my_items && !aborted; ph0 += kItemsPerPhase) {
        const int cnt = (int)((my_items - ph0 < kItemsPerPhase) ? (my_items - ph0) : kItemsPerPhase);
        for (int q = t; q < cnt; q += kThreads) {
            const int64_t w = blockIdx.x + (ph0 + q) * G;
            const int64_t b = w / p.m_vec;  // the only 64-bit division: once per item, not per stage
            const int o = (int)(w - b * p.m_vec);
            const int row = __ldg(p.row_indices + o);
            l_row[q] = row;
            l_b[q] = (int)b;
            l_j0[q] = __ldg(p.row_offsets + row);
            l_end[q] = __ldg(p.row_offsets + row + 1);
        }
        __syncthreads();

        // ---- tile iterator: (q, j) = item and first entry of the tile; rows without entries are skipped ----
        int q = 0;
        while (q < cnt && l_j0[q] >= l_end[q]) ++q;
        int j = 0, jend = 0, kb = 0;
        if (q < cnt) { j = l_j0[q]; jend = l_end[q]; }
        int idx[8], idx_next[8];
        auto load_idx = [&](int (&dst)[8], int jj0, int jje) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int jj = jj0 + r0 + 16 * i;
                dst[i] = (jj < jje) ? __ldg(p.col_indices + jj) : 0;
            }
        };
        // the tile after (qq, jj): next tile of the same row, else the first tile of the next non-empty row
        auto peek = [&](int qq, int jj, int jje, int &nq, int &nj, int &nje) {
            if (jj + kTileE < jje) { nq = qq; nj = jj + kTileE; nje = jje; return; }
            nq = qq + 1;
            while (nq < cnt && l_j0[nq] >= l_end[nq]) ++nq;
            if (nq < cnt) { nj = l_j0[nq]; nje = l_end[nq]; } else { nj = 0; nje = 0; }
        };
        if (q < cnt) load_idx(idx, j, jend);

        Pending fifo[kEpiLag];
#pragma unroll
        for (int i = 0; i < kEpiLag; ++i) fifo[i] = Pending{0, 0, 0, 0, 0};
        int fifo_n = 0;
        const uint32_t g_base = g_stage;
        int phase_stages = (q < cnt) ? -1 : 0;

        auto epilogue = [&](const Pending &e) {
            if (!tc::mbar_wait(bar_acc + 8 * e.accslot, (uint32_t)e.parity)) timeout = 1;
            tc::tc_fence_after_sync();
            uint32_t r[8];
            tc::tmem_ld_x8(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(e.accslot * kAccCols), r);
            tc::tc_fence_before_sync();
            const int jj = e.jt + t;
            if (jj < e.jend) {
                TOut *o = static_cast<TOut *>(p.out) + (int64_t)e.b * p.stride_out + (int64_t)jj * V;
                float f[V];
#pragma unroll
                for (int v = 0; v < V; ++v) f[v] = __uint_as_float(r[v]);
                if constexpr (V >= 4) {
                    store_chunk(o, f);
                } else {
#pragma unroll
                    for (int v = 0; v < V; ++v) store_scalar(o + v, f[v]);
                }
            }
        };

        for (int it = 0; phase_stages != 0; ++it) {
            // ---- issue side ---------------------------------------------------------------------------
            if (q < cnt) {
                const uint32_t slot = g_stage % kStages;
                if (g_stage >= (uint32_t)kStages) {
                    if (!tc::mbar_wait(bar_empty + 8 * slot, ((g_stage / kStages) - 1u) & 1u)) timeout = 1;
                }
                const int b = l_b[q];
                const int row = l_row[q];
                const __half *rhs = static_cast<const __half *>(p.rhs) + (int64_t)b * p.stride_rhs;
                const __half *lhs = static_cast<const __half *>(p.lhs) + (int64_t)b * p.stride_lhs;
                const int koff = kb * kBlockK + chunk * 8;
                const int n_ent = min(kTileE, jend - j);

                const uint32_t a_dst = base + Smem::kA + slot * kAStageBytes + a_dst0;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const bool ok = (r0 + 16 * i) < n_ent;
                    const __half *src = ok ? rhs + (int64_t)idx[i] * p.k + koff : rhs;
                    tc::cp_async_16(a_dst + i * 2048, src, ok ? 16u : 0u);
                }
                {
                    const bool ok = r0 < V;
                    const __half *src = ok ? lhs + ((int64_t)row * V + r0) * p.k + koff : lhs;
                    tc::cp_async_16(base + Smem::kB + slot * kBStageBytes + b_dst, src, ok ? 16u : 0u);
                }
                const bool first = (kb == 0), last = (kb == nkb - 1);
                if (t == 0) {
                    StageMeta m;
                    m.jt = j; m.jend = jend; m.b = b;
                    m.accslot = (int)(g_tile % kAccSlots);
                    m.flags = (first ? 1 : 0) | (last ? 2 : 0) | ((int)((g_tile / kAccSlots) & 1u) << 2);
                    meta[g_stage % kMetaRing] = m;
                }
                ++g_stage;
                if (first) {  // fetch the indices of the tile after this one while this one is in flight
                    int nq, nj, nje;
                    peek(q, j, jend, nq, nj, nje);
                    if (nq < cnt) load_idx(idx_next, nj, nje);
                }
                if (last) {
                    ++g_tile;
                    int nq, nj, nje;
                    peek(q, j, jend, nq, nj, nje);
                    q = nq; j = nj; jend = nje; kb = 0;
#pragma unroll
                    for (int i = 0; i < 8; ++i) idx[i] = idx_next[i];
                    if (q >= cnt) phase_stages = (int)(g_stage - g_base);
                } else {
                    ++kb;
                }
            }
            tc::cp_async_commit();

            // ---- consume side -------------------------------------------------------------------------
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
#pragma unroll
                    for (int mm = 0; mm < kBlockK / 16; ++mm) {
                        const uint64_t ad = tc::make_smem_desc(base + Smem::kA + slot * kAStageBytes + mm * 32, 16,
                                                               1024, tc::kSwizzle128B);
                        const uint64_t bd = tc::make_smem_desc(base + Smem::kB + slot * kBStageBytes + mm * 32, 16,
                                                               1024, tc::kSwizzle128B);
                        tc::mma_f16_ss(d, ad, bd, kIdesc, ((m.flags & 1) && mm == 0) ? 0u : 1u);
                    }
                    tc::mma_commit(bar_empty + 8 * slot);
                    if (m.flags & 2) tc::mma_commit(bar_acc + 8 * m.accslot);
                }
                if (m.flags & 2) {
                    const Pending oldest = fifo[0];
#pragma unroll
                    for (int i = 0; i + 1 < kEpiLag; ++i) fifo[i] = fifo[i + 1];
                    fifo[kEpiLag - 1] = Pending{m.jt, m.jend, m.b, m.accslot, (m.flags >> 2) & 1};
                    if (fifo_n == kEpiLag) epilogue(oldest);
                    else ++fifo_n;
                }
                if (phase_stages >= 0 && cs == phase_stages - 1) break;
            }
        }
        if (!aborted) {
#pragma unroll
            for (int i = 0; i < kEpiLag; ++i)
                if (i >= kEpiLag - fifo_n) epilogue(fifo[i]);
        }
        tc::tc_fence_before_sync();
        if (__syncthreads_or(timeout)) aborted = true;
    }

    tc::cp_async_wait<0>();
    if (aborted && t == 0) atomicOr(status, kStatusTimeout);
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace tcsddmm
}  // namespace vs
