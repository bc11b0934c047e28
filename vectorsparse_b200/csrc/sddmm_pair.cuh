// Tensor-core SDDMM on dense tiles sampled at the mask, computed by PAIRS of CTAs (a cluster of two SMs, tcgen05
// cta_group::2): the `wmmaSddmm` entry point of the reference (src/wmma_sddmm.cu:3175-3202).  Same formulation as
// sddmm_dense.cuh next to this file; what changes is the tile, its orientation and the way it is sampled:
//
//     D^T[256 mask columns x 256 rows of lhs] += rhs[256 x 64] . lhs[256 x 64]^T        per 64 contraction elements
//
// is ONE stream of 256 x 256 x 16 MMAs issued by one thread of the pair's first CTA.  CTA r of the pair loads rows
// 128 r .. of the rhs tile (its half of the M operand) and rows 128 r .. of the lhs tile (its half of the N operand)
// with its own plain TMA tile loads (no multicast), and receives mask columns 128 r .. of the product in its own
// tensor memory: lane = mask column, tensor-memory column = row of lhs.  Against the single-CTA kernel (256 x 128
// tiles, 128 x 128 x 16 MMAs) every SM reads 2/3 of the operand bytes per output from L2 and half as much from
// shared memory per flop, which is what that kernel is bound by.
//
// Sampling.  The V rows of a vector-row are V CONSECUTIVE tensor-memory columns, so after a 32-column load lane c
// holds, for each of the 32 / V vector-rows the load covers, exactly the V outputs of mask entry (vector-row, c) in
// the order they have in memory: a lane that has such an entry writes them with one vector store.  Whether it has,
// and which entry index j it is, comes from a column view of the mask that the plan kernel builds: per (block of 32
// vector-rows, mask column) a 32-bit presence mask and the position of the cell's first entry in a list of entry
// indices ordered by (block, column, vector-row).  No shared-memory boxes, no dynamic register indexing, nothing
// outside the mask is ever stored, so non-finite products elsewhere in the tile cannot leak.  A presence bit holds
// one entry: when the same column appears twice in a vector-row the plan kernel says so and a fix-up kernel copies
// the written entry's outputs to its twins (their values are equal by definition).
//
// Operand traffic.  With both operands streamed every SM takes 32 KiB from L2 per 540 cycles of tensor work.  When the
// rhs of one batch entry fits eight of the CTA's fourteen 16 KiB operand slots (n / 256 x k / 64 <= 8 tiles per CTA) it
// stays in shared memory instead: a pair then takes a contiguous run of work items (batch entry, row tile, column
// tile; column tiles fastest), a tile of rhs is loaded when a batch entry first needs it and is reused by every row
// tile of lhs, and only lhs streams through the remaining slots (0.64 GB instead of 1.07 GB from L2 per call at
// lhs 2048 x 256, rhs 512 x 256, 256 batch entries).  Otherwise both operands stream through rings of seven slots and
// the pairs interleave (items pair, pair + pairs, ...), so that neighbours read the same tiles at the same time.
// Measured on B200 at that shape (ms per call; the single-CTA kernel: 0.174): both modes 0.134-0.139.  With the loads
// switched off (timing experiment) 0.129 -> 0.094 and the SM clock rises from ~1.5-1.7 to 1.97 GHz: the part runs this
// kernel at its power cap, and a good part of what the loads "cost" is clock.  Handing the accumulator back early
// changes nothing.  What did not help: asking tiles into L2 two items ahead, by TMA prefetches from the loader (13 %
// slower) or by plain prefetch instructions from a warp of its own (no change); rings of 4, 6 or 7 stages (within
// 2 %); 128-row lhs tiles shared by two column tiles, which halves the bytes per stage but needs twice the MMA
// instructions (0.154); reading a warp's 64 accumulator columns with one wait instead of two (0.141-0.145, spills).
//
// Organisation per CTA (both CTAs of a pair run the same roles on their own halves):
//   warps 0-15  sampling epilogue: warp (quarter, part) owns accumulator lanes 32 quarter .. (32 mask columns) and
//               tensor-memory columns 64 part .. + 63 (64 rows of lhs); cells are fetched two work items ahead, entry
//               indices one
//   warp 16     one thread issuing the CTA's loads.  They are cta_group::2 loads: the tile lands in the issuing CTA, the
//               bytes are counted on the FIRST CTA's barrier, which that CTA's loader arms with the bytes of both
//   warp 17     first CTA: the MMA-issuing thread of the pair (idle in the second); its commits arrive on the barriers of
//               both CTAs at once, so that no thread has to forward anything
// Every wait is bounded; a wait that runs out raises the abort flag of both CTAs, all roles fall through, a status
// bit is set, both CTAs meet at the final cluster barrier and tensor memory is freed.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "sddmm_dense.cuh"
#include "spmm_pair.cuh"
#include "tc_ptx.cuh"

namespace vs {
namespace pairsddmm {

using densesddmm::kBlockK;
using densesddmm::kStatusTimeout;
using pairspmm::abort_pair;
using pairspmm::wait_or_abort;

constexpr int kTile = 256;                                // mask columns and rows of lhs per work item: 128 + 128 per pair
constexpr int kCtaRows = 128;
constexpr int kSlots = 14;                                // operand slots of 16 KiB per CTA
constexpr int kMaxResident = 8;                           // of them, at most this many hold a resident rhs
constexpr int kEpiWarps = 16;                             // TMEM lane quarter = warp % 4, 64 tensor-memory columns = warp / 4
constexpr int kLoadWarp = kEpiWarps;
constexpr int kMmaWarp = kLoadWarp + 1;
constexpr int kThreads = (kMmaWarp + 1) * 32;             // 576
constexpr int kOperandBytes = kCtaRows * kBlockK * 2;     // 16 KiB: 128 rows of either operand, 64 contraction elements
constexpr int kTmemCols = 2 * kTile;                      // two accumulator buffers
constexpr int kBlockVecRows = 32;                         // vector-rows per presence mask
constexpr int kPlanThreads = 1024;
constexpr int kMaxPlanColumns = 8192;                     // mask widths the plan kernel holds in shared memory
constexpr int kSleepLoad = 32, kSleepMma = 0, kSleepEpilogue = 32;

struct Smem {  // offsets from the 1024-byte aligned base; identical in both CTAs of a pair
    static constexpr int kOperands = 0;                   // kSlots slots: the ring of lhs tiles first, the rhs tiles behind it
    static constexpr int kBarFull = kOperands + kSlots * kOperandBytes;
    static constexpr int kBarDone = kBarFull + kSlots * 8;
    static constexpr int kBarAccFull = kBarDone + kSlots * 8;
    static constexpr int kBarAccEmpty = kBarAccFull + 2 * 8;
    static constexpr int kTmemHolder = kBarAccEmpty + 2 * 8;
    static constexpr int kAbort = kTmemHolder + 8;
    static constexpr int kTotal = kAbort + 8;
};
constexpr int kSmemBytes = Smem::kTotal + 1024;
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");

// The work items of one pair, as (batch entry, row tile of lhs, column tile of the mask).  With a resident rhs: a
// contiguous run of items, column tiles fastest, so that the pair stays with one batch entry as long as it can.
// Otherwise items pair, pair + pairs, ... with row tiles fastest, so that neighbouring pairs read the same rhs tile
// at the same time.  Walked with carries instead of divisions.
struct ItemWalk {
    int x0, x1, b, r0, r1, s0, s1, s2;
    bool nt_fast;
    __device__ __forceinline__ void init(int64_t w, int64_t stride, int m_tiles, int n_tiles, bool nt_fast_) {
        nt_fast = nt_fast_;
        r0 = nt_fast ? n_tiles : m_tiles;
        r1 = nt_fast ? m_tiles : n_tiles;
        x0 = (int)(w % r0);
        const int64_t q = w / r0;
        x1 = (int)(q % r1);
        b = (int)(q / r1);
        s0 = (int)(stride % r0);
        const int64_t sq = stride / r0;
        s1 = (int)(sq % r1);
        s2 = (int)(sq / r1);
    }
    __device__ __forceinline__ void next() {
        x0 += s0; x1 += s1; b += s2;
        if (x0 >= r0) { x0 -= r0; ++x1; }
        if (x1 >= r1) { x1 -= r1; ++b; }
    }
    __device__ __forceinline__ int mt() const { return nt_fast ? x1 : x0; }
    __device__ __forceinline__ int nt() const { return nt_fast ? x0 : x1; }
};

// ---- plan -------------------------------------------------------------------------------------------------
// One CTA per block of 32 vector-rows.  cells[block * n + c] = (presence mask over the block's vector-rows of an
// entry in column c, position in `order` of the cell's first entry); order[] lists entry indices j by (block,
// column, vector-row).  The entries of a block are one contiguous range of j, so a block's cells start at the
// block's first j.  Columns outside [0, n) are dropped: their outputs are not written.  *twins is set when a
// vector-row names a column twice (only one of the two reaches `order`).
__global__ void __launch_bounds__(kPlanThreads)
sddmm_cell_plan_kernel(const int32_t *__restrict__ row_offsets, const int32_t *__restrict__ col_indices, int m_vec, int n, int nnz_vec,
                       uint2 *__restrict__ cells, int32_t *__restrict__ order, int32_t *__restrict__ twins) {
    extern __shared__ uint32_t cell_sh[];   // [n] masks, then [n] positions
    __shared__ int32_t offs[kBlockVecRows + 1];
    __shared__ int32_t part_sum[32];
    pdl_launch_dependents();   // the multiplying kernel may set itself up while the plan is made
    uint32_t *mask = cell_sh, *first = cell_sh + n;
    const int t = threadIdx.x, blk = blockIdx.x, vr0 = blk * kBlockVecRows;
    const int rows = min(kBlockVecRows, m_vec - vr0);
    if (blk == 0 && t == 0) *twins = 0;
    // the scratch holds nnz_vec entries (the caller's count): offsets that claim more are cut there
    if (t <= kBlockVecRows) offs[t] = min(max(__ldg(row_offsets + vr0 + min(t, rows)), 0), nnz_vec);
    for (int c = t; c < n; c += kPlanThreads) mask[c] = 0u;
    __syncthreads();
    const int j0 = offs[0], j1 = max(offs[rows], j0);
    auto row_of = [&](int j) {   // the vector-row (0 .. rows - 1) whose range holds j
        int lo = 0, hi = rows;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (offs[mid] <= j) lo = mid; else hi = mid;
        }
        return lo;
    };
    bool twin = false;
    for (int jb = j0 + t; jb < j1; jb += 4 * kPlanThreads) {   // four entries per thread and trip: their loads fly together
        int c[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) c[u] = jb + u * kPlanThreads < j1 ? __ldg(col_indices + jb + u * kPlanThreads) : -1;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if ((unsigned)c[u] >= (unsigned)n) continue;
            const uint32_t bit = 1u << row_of(jb + u * kPlanThreads);
            twin |= (atomicOr(mask + c[u], bit) & bit) != 0u;
        }
    }
    if (twin) atomicExch(twins, 1);
    __syncthreads();
    // exclusive scan of popc(mask[c]) over the columns: every thread sums a contiguous run, the runs are scanned with
    // shuffles inside each warp and once more across the warps
    const int per = (n + kPlanThreads - 1) / kPlanThreads;
    const int c_lo = min(t * per, n), c_hi = min(c_lo + per, n);
    int sum = 0;
    for (int c = c_lo; c < c_hi; ++c) sum += __popc(mask[c]);
    const int lane = t & 31, warp = t >> 5;
    int incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += up;
    }
    if (lane == 31) part_sum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const int w_sum = lane < kPlanThreads / 32 ? part_sum[lane] : 0;
        int w_incl = w_sum;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, w_incl, d);
            if (lane >= d) w_incl += up;
        }
        if (lane < kPlanThreads / 32) part_sum[lane] = w_incl - w_sum;   // what the warps before this one hold
    }
    __syncthreads();
    int run = j0 + part_sum[warp] + incl - sum;
    uint2 *mine = cells + (int64_t)blk * n;
    for (int c = c_lo; c < c_hi; ++c) {
        first[c] = (uint32_t)run;
        mine[c] = make_uint2(mask[c], (uint32_t)run);
        run += __popc(mask[c]);
    }
    __syncthreads();
    for (int jb = j0 + t; jb < j1; jb += 4 * kPlanThreads) {
        int c[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) c[u] = jb + u * kPlanThreads < j1 ? __ldg(col_indices + jb + u * kPlanThreads) : -1;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if ((unsigned)c[u] >= (unsigned)n) continue;
            const int j = jb + u * kPlanThreads;
            const uint32_t below = (1u << row_of(j)) - 1u;
            order[first[c[u]] + __popc(mask[c[u]] & below)] = j;   // twins write the same place: one of them stays
        }
    }
}

// Runs behind the multiplying kernel; does nothing unless the plan kernel met a column twice in one vector-row.
// Entry j whose place in `order` holds another entry j' is a twin of j': same vector-row, same column, same outputs.
template <typename TOut, int V>
__global__ void __launch_bounds__(kPlanThreads)
sddmm_twin_kernel(const SddmmParams p, const uint2 *__restrict__ cells, const int32_t *__restrict__ order, const int32_t *__restrict__ twins) {
    pdl_wait();
    if (*twins == 0) return;
    const int j = blockIdx.x * kPlanThreads + threadIdx.x;
    if (j >= p.nnz_vec) return;
    const int c = __ldg(p.col_indices + j);
    if ((unsigned)c >= (unsigned)p.n) return;
    int lo = 0, hi = p.m_vec;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(p.row_offsets + mid) <= j) lo = mid; else hi = mid;
    }
    const uint2 cell = __ldg(cells + (int64_t)(lo / kBlockVecRows) * p.n + c);
    const int other = __ldg(order + cell.y + __popc(cell.x & ((1u << (lo % kBlockVecRows)) - 1u)));
    if (other == j) return;
    for (int b = 0; b < p.batch; ++b) {
        TOut *out = static_cast<TOut *>(p.out) + (int64_t)b * p.stride_out;
        for (int v = 0; v < V; ++v) out[(int64_t)j * V + v] = out[(int64_t)other * V + v];
    }
}

// map_lhs: {k, rows of lhs, batch}, map_rhs: {k, n, batch}; both box {64, 128, 1}, K-major with the 128-byte swizzle
// and zero fill outside.  cells / order: see sddmm_cell_plan_kernel; blocks = number of 32-vector-row blocks.
// resident: keep the rhs tiles of the current batch entry in shared memory (the host checks that they fit).
template <typename TOut, int V>
__global__ void __launch_bounds__(kThreads, 1)
sddmm_pair_kernel(const SddmmParams p, const __grid_constant__ CUtensorMap map_lhs, const __grid_constant__ CUtensorMap map_rhs,
                  const uint2 *__restrict__ cells, const int32_t *__restrict__ order, int blocks, int m_tiles, int n_tiles,
                  int resident, uint32_t *status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = tc::smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;   // the same offset in both CTAs: same kernel, same static layout
    uint8_t *sm = smem_raw + (base - raw);

    const int t = threadIdx.x;
    const int warp = t >> 5;
    const int lane = t & 31;
    const uint32_t rank = tc::cluster_ctarank();   // 0: the CTA that issues the MMAs
    const uint32_t peer = rank ^ 1u;
    const uint32_t pair = tc::cluster_id_x(), pairs = tc::cluster_count_x();
    volatile int *abort_flag = reinterpret_cast<volatile int *>(sm + Smem::kAbort);
    const uint32_t abort_addr = base + Smem::kAbort;
    const uint32_t bar_full = base + Smem::kBarFull;
    const uint32_t bar_done = base + Smem::kBarDone;
    const uint32_t bar_acc_full = base + Smem::kBarAccFull;
    const uint32_t bar_acc_empty = base + Smem::kBarAccEmpty;

    if (t == 0) {
        for (int s = 0; s < kSlots; ++s) {
            tc::mbar_init(bar_full + 8 * s, 1);   // first CTA only: its loader's arrival + the bytes of BOTH CTAs' tiles
            tc::mbar_init(bar_done + 8 * s, 1);   // a commit of the MMA-issuing thread, which arrives in both CTAs
        }
        for (int s = 0; s < 2; ++s) {
            tc::mbar_init(bar_acc_full + 8 * s, 1);
            tc::mbar_init(bar_acc_empty + 8 * s, 2 * kEpiWarps);   // one lane per epilogue warp of both CTAs; first CTA only
        }
        *abort_flag = 0;
        tc::fence_mbar_init();
    }
    if (warp == kMmaWarp) {
        tc::tmem_alloc_pair(base + Smem::kTmemHolder, kTmemCols);
        tc::tmem_relinquish_pair();
    }
    tc::fence_proxy_async();
    tc::tc_fence_before_sync();
    tc::cluster_sync();   // barriers and flags of BOTH CTAs exist before anything crosses between them
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(sm + Smem::kTmemHolder);

    pdl_launch_dependents();
    pdl_wait();   // the set-up above may have run beside the plan kernel; its cells are read from here on
    const int k_blocks = p.k / kBlockK;
    const int64_t total_items = (int64_t)p.batch * n_tiles * m_tiles;
    // this pair's items: a contiguous run with a resident rhs, every pairs-th item otherwise
    const int64_t item0 = resident ? total_items * pair / pairs : (int64_t)pair;
    const int64_t item_stride = resident ? 1 : (int64_t)pairs;
    const uint32_t my_items = resident ? (uint32_t)(total_items * (pair + 1) / pairs - item0)
                                       : (total_items > pair ? (uint32_t)((total_items - pair + pairs - 1) / pairs) : 0u);
    const uint32_t total_stages = my_items * (uint32_t)k_blocks;
    // Stage g = (item g / k_blocks, contraction block g % k_blocks).  Its lhs tile goes through ring slot g % ring; its
    // rhs tile sits in slot ring + nt * k_blocks + kb when rhs is resident, in slot ring + g % ring otherwise.
    const uint32_t ring = resident ? (uint32_t)(kSlots - n_tiles * k_blocks) : (uint32_t)(kSlots / 2);
    const uint32_t rhs_slots = base + Smem::kOperands + ring * kOperandBytes;

    if (warp == kLoadWarp) {
        // =========================== loader ==============================================================
        if (lane == 0) {
            bool ok_run = true;
            const uint32_t full_first = tc::map_to_cta(bar_full, 0);
            ItemWalk walk;
            walk.init(item0, item_stride, m_tiles, n_tiles, resident != 0);
            int res_b = -1;                       // the batch entry whose rhs tiles are in the resident slots
            uint32_t valid = 0;                   // which of them have been loaded for it
            uint32_t last_use[kMaxResident];      // the last stage that read each resident slot
#pragma unroll
            for (int i = 0; i < kMaxResident; ++i) last_use[i] = 0u;
            uint32_t used = 0;
            uint32_t g = 0;
            for (uint32_t i = 0; i < my_items && ok_run; ++i, walk.next()) {
                for (int kb = 0; kb < k_blocks && ok_run; ++kb, ++g) {
                    const uint32_t slot = g % ring;
                    if (g >= ring)   // the stage that used this ring slot before must have been multiplied
                        ok_run = wait_or_abort<kSleepLoad>(bar_done + 8 * slot, ((g - ring) / ring) & 1u, abort_flag, abort_addr, peer);
                    if (!ok_run) break;
                    bool need_rhs = true;
                    uint32_t rs = slot;
                    if (resident) {
                        if (walk.b != res_b) { res_b = walk.b; valid = 0u; }
                        rs = (uint32_t)(walk.nt() * k_blocks + kb);
                        need_rhs = ((valid >> rs) & 1u) == 0u;
                        if (need_rhs) {
                            // the previous batch entry's tile in this slot: its last reader may be one of the stages
                            // the ring wait above does not cover yet
                            const uint32_t old = last_use[rs];
                            if (((used >> rs) & 1u) && old + ring > g)
                                ok_run = wait_or_abort<kSleepLoad>(bar_done + 8 * (old % ring), (old / ring) & 1u, abort_flag, abort_addr, peer);
                            if (!ok_run) break;
                            valid |= 1u << rs;
                        }
                        last_use[rs] = g;
                        used |= 1u << rs;
                    }
                    // both CTAs load the same amounts and count them on the FIRST CTA's barrier, which its loader arms
                    const uint32_t bar = full_first + 8 * slot;
                    if (rank == 0) tc::mbar_expect_tx(bar_full + 8 * slot, (uint32_t)((need_rhs ? 4 : 2) * kOperandBytes));
                    tc::tma_load_3d_pair(base + Smem::kOperands + slot * kOperandBytes, &map_lhs, bar, kb * kBlockK,
                                         walk.mt() * kTile + (int)rank * kCtaRows, walk.b);
                    if (need_rhs)
                        tc::tma_load_3d_pair(rhs_slots + rs * kOperandBytes, &map_rhs, bar, kb * kBlockK,
                                             walk.nt() * kTile + (int)rank * kCtaRows, walk.b);
                }
            }
            // the last "multiplied" signals addressed to this CTA must not arrive after it has gone
            const uint32_t tail0 = total_stages > ring ? total_stages - ring : 0u;
            for (uint32_t q = tail0; q < total_stages && ok_run; ++q)
                ok_run = wait_or_abort<kSleepLoad>(bar_done + 8 * (q % ring), (q / ring) & 1u, abort_flag, abort_addr, peer);
        }
    } else if (warp == kMmaWarp) {
        if (lane == 0 && rank == 0) {
            // =========================== MMA issuer of the pair ==========================================
            const uint32_t a_lo0 = tc::smem_desc_lo(rhs_slots, 16);                       // M operand: rows of rhs
            const uint32_t b_lo0 = tc::smem_desc_lo(base + Smem::kOperands, 16);          // N operand: rows of lhs
            const uint32_t hi = tc::smem_desc_hi(1024, (uint32_t)tc::kSwizzle128B);       // K-major: 8-row groups 1 KiB apart
            const uint32_t idesc = tc::make_idesc_f16(kTile, kTile, 0, 0);                // both operands K-major
            uint32_t slot = 0, parity = 0;
            bool ok_run = true;
            ItemWalk walk;
            walk.init(item0, item_stride, m_tiles, n_tiles, resident != 0);
            for (uint32_t i = 0; i < my_items && ok_run; ++i, walk.next()) {
                const uint32_t buf = i & 1u;
                ok_run = wait_or_abort<kSleepMma>(bar_acc_empty + 8 * buf, (i >> 1) & 1u, abort_flag, abort_addr, peer);
                if (!ok_run) break;
                tc::tc_fence_after_sync();
                const uint32_t d = tmem_base + buf * kTile;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    ok_run = wait_or_abort<kSleepMma>(bar_full + 8 * slot, parity, abort_flag, abort_addr, peer);
                    if (!ok_run) break;
                    // no tensor-core fence per stage: the operands were written by TMA, whose completion the barrier carries
                    const uint32_t rs = resident ? (uint32_t)(walk.nt() * k_blocks + kb) : slot;
                    const uint32_t a_lo = a_lo0 + rs * (kOperandBytes >> 4), b_lo = b_lo0 + slot * (kOperandBytes >> 4);
#pragma unroll
                    for (int kk = 0; kk < kBlockK / 16; ++kk)   // 16 contraction elements = 32 bytes along a row
                        tc::mma_f16_ss_pair(d, tc::desc64(a_lo + 2 * kk, hi), tc::desc64(b_lo + 2 * kk, hi), idesc,
                                            (kb > 0 || kk > 0) ? 1u : 0u);
                    tc::mma_commit_pair_both(bar_done + 8 * slot);      // "stage multiplied", to both CTAs' loaders
                    if (++slot == ring) { slot = 0; parity ^= 1u; }
                }
                if (ok_run) tc::mma_commit_pair_both(bar_acc_full + 8 * buf);   // "accumulator complete", to both CTAs' epilogues
            }
        }
    } else {
        // =========================== sampling epilogue ===================================================
        // This lane's mask column is nt * 256 + 128 rank + 32 quarter + lane; the warp's 64 tensor-memory columns are
        // rows 64 part .. + 63 of the lhs tile = 64 / V vector-rows, read by two 32-column loads of 32 / V vector-rows
        // each.  All of them lie in one block of 32 vector-rows, so the lane needs ONE cell per work item.
        constexpr int kPerLoad = 32 / V;                 // vector-rows per 32-column load
        constexpr bool kAheadEntries = 2 * kPerLoad <= 16;   // hold the next item's entry indices as well
        constexpr int kElems = 16 / (int)sizeof(TOut);   // outputs per 16-byte store
        const int quarter = warp & 3, part = warp >> 2;
        const uint32_t lane_taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(part * 64);
        const uint32_t acc_empty_first = tc::map_to_cta(bar_acc_empty, 0);
        if (lane == 0) {
            tc::mbar_arrive_remote(acc_empty_first);        // both accumulator buffers start out free
            tc::mbar_arrive_remote(acc_empty_first + 8);
        }
        auto cell_of = [&](const ItemWalk &w, bool valid, int &bit0) -> uint2 {
            const int c = w.nt() * kTile + (int)rank * kCtaRows + quarter * 32 + lane;
            const int vr = (w.mt() * kTile + part * 64) / V;   // first vector-row this warp samples
            const int blk = vr / kBlockVecRows;
            bit0 = vr % kBlockVecRows;
            return (valid && c < p.n && blk < blocks) ? __ldg(cells + (int64_t)blk * p.n + c) : make_uint2(0u, 0u);
        };
        // the entry indices a lane needs for an item: 2 * kPerLoad bits of its cell, in vector-row order
        auto entries_of = [&](const uint2 cell, int bit0, uint32_t &bits, int (&ent)[2 * kPerLoad]) {
            bits = (cell.x >> bit0) & (uint32_t)((1ull << (2 * kPerLoad)) - 1ull);
            const int pos0 = (int)cell.y + __popc(cell.x & ((1u << bit0) - 1u));
#pragma unroll
            for (int b = 0; b < 2 * kPerLoad; ++b)
                ent[b] = ((bits >> b) & 1u) ? __ldg(order + pos0 + __popc(bits & ((1u << b) - 1u))) : -1;
        };
        ItemWalk walk, ahead;   // `walk`: the item being sampled; `ahead`: two items further on
        walk.init(item0, item_stride, m_tiles, n_tiles, resident != 0);
        ahead = walk;
        int bit0, n_bit0, f_bit0;
        uint32_t bits, n_bits;
        int ent[2 * kPerLoad], n_ent[kAheadEntries ? 2 * kPerLoad : 1];
        uint2 n_cell, f_cell;
        {
            const uint2 c_cell = cell_of(ahead, my_items > 0, bit0);
            ahead.next();
            n_cell = cell_of(ahead, my_items > 1, n_bit0);
            entries_of(c_cell, bit0, bits, ent);
        }
        bool ok_run = true;
        for (uint32_t i = 0; i < my_items && ok_run; ++i, walk.next()) {
            const uint32_t buf = i & 1u;
            // requested now: the cell of item i + 2 and the entry indices of item i + 1 (its cell was requested an item ago);
            // at V = 2 a lane may have 32 entries per item, too many to hold for two items: they are fetched when needed
            ahead.next();
            f_cell = cell_of(ahead, i + 2 < my_items, f_bit0);
            if constexpr (kAheadEntries) entries_of(n_cell, n_bit0, n_bits, n_ent);

            ok_run = __all_sync(0xffffffffu, wait_or_abort<kSleepEpilogue>(bar_acc_full + 8 * buf, (i >> 1) & 1u, abort_flag, abort_addr, peer));
            if (!ok_run) break;
            tc::tc_fence_after_sync();
            TOut *out = static_cast<TOut *>(p.out) + (int64_t)walk.b * p.stride_out;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t sub = (bits >> (h * kPerLoad)) & (uint32_t)((1u << kPerLoad) - 1u);
                if (!__any_sync(0xffffffffu, sub != 0u)) continue;   // warp-uniform: nobody has an entry in these 32 rows
                uint32_t r[32];
                tc::tmem_ld_x32(lane_taddr + buf * kTile + (uint32_t)(h * 32), r);
#pragma unroll
                for (int b = 0; b < kPerLoad; ++b) {
                    const int j = ent[h * kPerLoad + b];
                    if (j < 0) continue;
                    TOut *dst = out + (int64_t)j * V;
                    if constexpr (sizeof(TOut) == 2) {
                        if constexpr (V == 8) {
                            uint4 o;
                            __half2 *hh = reinterpret_cast<__half2 *>(&o);
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                hh[e] = __floats2half2_rn(__uint_as_float(r[b * V + 2 * e]), __uint_as_float(r[b * V + 2 * e + 1]));
                            *reinterpret_cast<uint4 *>(dst) = o;
                        } else if constexpr (V == 4) {
                            uint2 o;
                            __half2 *hh = reinterpret_cast<__half2 *>(&o);
                            hh[0] = __floats2half2_rn(__uint_as_float(r[b * V]), __uint_as_float(r[b * V + 1]));
                            hh[1] = __floats2half2_rn(__uint_as_float(r[b * V + 2]), __uint_as_float(r[b * V + 3]));
                            *reinterpret_cast<uint2 *>(dst) = o;
                        } else {
                            *reinterpret_cast<__half2 *>(dst) = __floats2half2_rn(__uint_as_float(r[b * V]), __uint_as_float(r[b * V + 1]));
                        }
                    } else {
                        if constexpr (V >= 4) {
#pragma unroll
                            for (int e = 0; e < V / kElems; ++e)
                                reinterpret_cast<uint4 *>(dst)[e] = make_uint4(r[b * V + 4 * e], r[b * V + 4 * e + 1], r[b * V + 4 * e + 2], r[b * V + 4 * e + 3]);
                        } else {
                            *reinterpret_cast<uint2 *>(dst) = make_uint2(r[b * V], r[b * V + 1]);
                        }
                    }
                }
            }
            tc::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive_remote(acc_empty_first + 8 * buf);   // sampled: the buffer is free for the pair
            if constexpr (kAheadEntries) {
                bits = n_bits;
#pragma unroll
                for (int b = 0; b < 2 * kPerLoad; ++b) ent[b] = n_ent[b];
            } else {
                entries_of(n_cell, n_bit0, bits, ent);
            }
            n_cell = f_cell; n_bit0 = f_bit0;
        }
    }

    // ---- teardown ---------------------------------------------------------------------------------------
    tc::tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);   // copies that may still be in flight
        if (t == 0) atomicOr(status, kStatusTimeout);
    }
    tc::cluster_sync();   // neither CTA's shared or tensor memory goes away while the other half of an MMA may use it
    if (warp == kMmaWarp) tc::tmem_dealloc_pair(tmem_base, kTmemCols);
}

}  // namespace pairsddmm
}  // namespace vs
