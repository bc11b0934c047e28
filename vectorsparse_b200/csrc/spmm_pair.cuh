// Tensor-core SpMM on densified tiles of the sparse matrix, computed by PAIRS of CTAs (a cluster of two SMs,
// tcgen05 cta_group::2): the `wmmaSpmm` entry point of the reference (src/wmma_spmm.cu:388-409) for dense widths
// that are multiples of 128.  Same formulation, plan and semantics as spmm_dense.cuh next to this file (see there
// for why a zero-filled tile of A beats a row gather on this part); what changes is who multiplies what:
//
//     C[256 rows x tn cols] += A_dense[256 x 64] * B[64 x tn]        per 64-wide block of A's columns, tn = 256 or 128
//
// is ONE stream of 256 x tn x 16 MMAs issued by one thread of the pair's first CTA.  CTA r of the pair densifies
// rows 128 r .. 128 r + 127 of the tile in its own shared memory, loads columns r * tn / 2 .. of the block of B with
// its own plain TMA tile loads (no multicast: each CTA's copies land in its own shared memory only), and
// receives rows 128 r .. of the accumulator in its own tensor memory.  A single-CTA 128 x 128 x 16 MMA reads 8 KB of
// operands in the 64 cycles it takes, all of an SM's shared-memory bandwidth; here each SM reads its 4 KB of A and
// only its own half of B (4 KB at tn = 256) per 128 cycles of tensor work, and A is densified once per row tile for
// all 256 columns.  That leaves the bandwidth the fill, the TMA writes of B and the output staging need.
//
// Organisation per CTA (both CTAs of a pair run the same roles on their own halves):
//   warps 0-7    epilogue: own 128 accumulator lanes -> registers -> swizzled boxes -> TMA stores of whole rows
//   warps 8-19   fill: two warps per A slot (six slots), each owning 128 rows x 32 columns (two plan buckets) of the
//                stage; what a stage needs from global memory is requested right after the previous one was handed over
//   warp 20      one thread issuing the CTA's B loads, six stages ahead: the ring of B tiles is what hides the latency
//                of L2 and HBM (an L2 prefetch warp beside it, as the single-CTA kernel has, made this kernel slower).
//                They are cta_group::2 loads: the tile lands in the issuing CTA, its bytes are counted on the FIRST
//                CTA's barrier, which that CTA's loader arms with the bytes of both halves
//   warp 21      first CTA: the MMA-issuing thread of the pair (idle in the second).  Its commits arrive on the barriers
//                of both CTAs at once (tcgen05.commit with a CTA mask: an arrival, not a copy), so nothing is forwarded
// Barriers, one set per stage in flight.  full[s] (first CTA only): the fill warps of BOTH CTAs, the first CTA's loader
// + the bytes of both CTAs' B tiles.  done[s] and acc_full[b] (both CTAs): a commit of the MMA-issuing thread.
// acc_empty[b] (first CTA): every epilogue thread of both CTAs.  Every wait is bounded; a wait that runs out raises the
// abort flag of both CTAs, all roles fall through, a status bit is set, both CTAs meet at the final cluster barrier and
// tensor memory is freed.
//
// What was measured on the way (B200, 148 SMs, ~1.5 GHz under the power cap while this kernel runs): a pair MMA of
// N = 256 occupies the pipe for ~135 cycles (N = 128: ~71); one thread issues them back to back every ~52 cycles, a
// commit costs it ~105.  A remote mbarrier arrive with cluster-scope release costs ~1100 cycles, the default form a
// few tens; forwarding "stage multiplied" and "B landed" between the CTAs with a thread each (instead of the commit mask
// and the cta_group::2 loads) cost 1-2 %.  Two issuing threads splitting the columns (N = 128 each) read A twice and were slower; walking the
// issue loop with the whole warp was slower; rings of 4 + 8, 5 + 7, 6 + 6 (A + B) stages are within 3 % of each other.
// With the fill, the B loads and the output stores switched off in turn the kernel gains 20, 15 and 23 us of its
// 115; with all three off it takes 77 us, which is the tensor pipe's time for the dense work at that clock.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "spmm_dense.cuh"
#include "tc_ptx.cuh"

namespace vs {
namespace pairspmm {

using densespmm::kBlockK;
using densespmm::kGroupRows;
using densespmm::kPlanCols;
using densespmm::kStatusTimeout;
using densespmm::scatter_vector;
using densespmm::ValueVec;

constexpr int kTileM = 256;                               // rows of A per work item: 128 per CTA of the pair
constexpr int kCtaRows = 128;
constexpr int kMaxTileN = 256;                            // columns of B per work item: 256, or 128 when N % 256 != 0
constexpr int kAStages = 6;                               // ring of densified A tiles
constexpr int kBStages = 6;                               // ring of B tiles: loaded that many stages ahead
constexpr int kFillCols = 32;                             // columns of a stage one fill warp owns: two plan buckets
constexpr int kEpiWarps = 8;                              // TMEM lane quarter = warp % 4, half of the columns = warp / 4
constexpr int kFillWarp0 = kEpiWarps;
constexpr int kFillPerSlot = kBlockK / kFillCols;         // warps per CTA and stage
constexpr int kFillWarps = kAStages * kFillPerSlot;       // 12: warp f fills A slot f % kAStages
constexpr int kOverflowBatches = 4;
constexpr int kLoadWarp = kFillWarp0 + kFillWarps;        // 20
constexpr int kMmaWarp = kLoadWarp + 1;
constexpr int kThreads = (kMmaWarp + 1) * 32;
static_assert(kThreads <= 1024, "too many fill warps for one CTA");
constexpr int kAStageBytes = kCtaRows * kBlockK * 2;      // 16 KiB
constexpr int kBSlabBytes = kBlockK * 64 * 2;             // 8 KiB: 64 rows of B x 64 columns
constexpr int kBStageBytes = (kMaxTileN / 2 / 64) * kBSlabBytes;   // 16 KiB: the CTA's half of 64 x 256
constexpr int kTmemCols = 2 * kMaxTileN;                  // 512: two accumulator buffers of up to 256 columns
constexpr int kStoreCols = 32;
constexpr int kStoreBoxBytes = 32 * 128;
constexpr int kBarStages = kAStages > kBStages ? kAStages : kBStages;   // one set of barriers per stage in flight

struct Smem {  // offsets from the 1024-byte aligned base; identical in both CTAs of a pair
    static constexpr int kA = 0;
    static constexpr int kB = kA + kAStages * kAStageBytes;
    static constexpr int kStaging = kB + kBStages * kBStageBytes;
    static constexpr int kBarFull = kStaging + kEpiWarps * kStoreBoxBytes;
    static constexpr int kBarDone = kBarFull + kBarStages * 8;
    static constexpr int kBarAccFull = kBarDone + kBarStages * 8;
    static constexpr int kBarAccEmpty = kBarAccFull + 2 * 8;
    static constexpr int kTmemHolder = kBarAccEmpty + 2 * 8;
    static constexpr int kAbort = kTmemHolder + 8;
    static constexpr int kTotal = kAbort + 8;
};
constexpr int kSmemBytes = Smem::kTotal + 1024;
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");

// Raises the abort flag of both CTAs of the pair.
__device__ __forceinline__ void abort_pair(volatile int *abort_flag, uint32_t abort_addr, uint32_t peer) {
    *abort_flag = 1;
    tc::st_remote_u32(tc::map_to_cta(abort_addr, peer), 1u);
}

// Bounded mbarrier wait that also gives up when a role of either CTA has raised the abort flag.
template <int kSleepNs>
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int *abort_flag, uint32_t abort_addr, uint32_t peer) {
    if (tc::mbar_try_wait(bar, parity)) return true;
    for (uint32_t i = 0; i < tc::kMaxPolls; ++i) {
        if (kSleepNs > 0) __nanosleep(kSleepNs);
        if (tc::mbar_try_wait(bar, parity)) return true;
        if ((i & 15u) == 15u && *abort_flag) return false;
    }
    abort_pair(abort_flag, abort_addr, peer);
    return false;
}
constexpr int kSleepFill = VS_DENSE_SLEEP, kSleepMma = 0, kSleepEpilogue = VS_DENSE_SLEEP;

// Work items of one pair, c, c + pairs, c + 2 pairs, ...: item w -> (batch entry, column tile, row tile), row tiles
// fastest, so that neighbouring pairs work on the same B.  Walked without divisions per step.
struct Walk {
    int b, nt, mt, kb;
    int d_mt, d_nt, d_b;
    int m_tiles, n_tiles, k_blocks;
    uint32_t g, total;
    __device__ __forceinline__ void init(uint32_t pair, uint32_t pairs, uint32_t g0, uint32_t total_stages, int m_tiles_, int n_tiles_,
                                         int k_blocks_) {
        m_tiles = m_tiles_; n_tiles = n_tiles_; k_blocks = k_blocks_;
        g = g0; total = total_stages;
        d_mt = (int)(pairs % (uint32_t)m_tiles);
        const uint32_t r = pairs / (uint32_t)m_tiles;
        d_nt = (int)(r % (uint32_t)n_tiles);
        d_b = (int)(r / (uint32_t)n_tiles);
        const uint32_t i0 = g0 / (uint32_t)k_blocks;
        kb = (int)(g0 - i0 * (uint32_t)k_blocks);
        const int64_t w = pair + (int64_t)i0 * pairs;
        mt = (int)(w % m_tiles);
        const int64_t rr = w / m_tiles;
        nt = (int)(rr % n_tiles);
        b = (int)(rr / n_tiles);
    }
    __device__ __forceinline__ bool valid() const { return g < total; }
    __device__ __forceinline__ void next_item() {
        mt += d_mt; nt += d_nt; b += d_b;
        if (mt >= m_tiles) { mt -= m_tiles; ++nt; }
        if (nt >= n_tiles) { nt -= n_tiles; ++b; }
    }
    __device__ __forceinline__ void advance(int stages) {
        g += (uint32_t)stages;
        kb += stages;
        while (kb >= k_blocks) { kb -= k_blocks; next_item(); }
    }
};

// map_b: the dense operand as {N, K, batch}, box {64, 64, 1}; map_b2: the same memory as {64, K, N / 64, batch},
// box {64, 64, 2, 1} (both 64-column slabs of a CTA's half of a 256-column tile in one copy); map_out: the output
// as {N, rows, batch}, box {32, 32, 1}.  All with zero fill / clipping outside the matrix; no multicast anywhere.
// tn: columns per work item (256 or 128), N % tn == 0.
template <typename TOut, int V, bool kTransposed>
__global__ void __launch_bounds__(kThreads, 1)
spmm_pair_kernel(const SpmmParams p, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_out,
                 const __grid_constant__ CUtensorMap map_b2, int tn, const int32_t *__restrict__ blk_offsets,
                 const uint2 *__restrict__ blk_entries, int m_tiles, int n_tiles, int k_blocks, uint32_t *status, int32_t *use_dense,
                 int plan_checks) {
    pdl_launch_dependents();
    pdl_wait();
    const bool chosen = plan_dense_chosen(use_dense, plan_checks);
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

    for (int i = t; i < kAStages * kAStageBytes / 16; i += kThreads)   // the A slots start out as zeros
        reinterpret_cast<uint4 *>(sm + Smem::kA)[i] = make_uint4(0, 0, 0, 0);
    if (t == 0) {
        for (int s = 0; s < kBarStages; ++s) {
            // first CTA only: the fill warps of both CTAs, its loader's arrival + the bytes of BOTH CTAs' B tiles
            tc::mbar_init(bar_full + 8 * s, 2 * kFillPerSlot + 1);
            tc::mbar_init(bar_done + 8 * s, 1);   // a commit of the MMA-issuing thread, which arrives in both CTAs
        }
        for (int s = 0; s < 2; ++s) {
            tc::mbar_init(bar_acc_full + 8 * s, 1);
            tc::mbar_init(bar_acc_empty + 8 * s, 2 * kEpiWarps * 32);   // used in the first CTA only
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
    tc::cluster_sync();   // barriers, flags and zeroed slots of BOTH CTAs exist before anything crosses between them
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(sm + Smem::kTmemHolder);

    const int64_t total_items = chosen ? (int64_t)p.batch * n_tiles * m_tiles : 0;
    const uint32_t my_items = (total_items > pair) ? (uint32_t)((total_items - pair + pairs - 1) / pairs) : 0u;
    const uint32_t total_stages = my_items * (uint32_t)k_blocks;
    const int m_rows = kTransposed ? p.m_vec : p.m_vec * V;
    const int half_cols = tn >> 1;              // columns of B this CTA holds per item
    const int slabs = half_cols >> 6;           // 64-column slabs of them: 2 or 1

    // Stage g of the pair (item g / k_blocks, column block g % k_blocks) uses A slot g % kAStages, B slot
    // g % kBStages and barrier set g % kBarStages.  done[g % kBarStages] completing phase g / kBarStages says "stage g
    // has been multiplied": the fill warps of stage g + kAStages and the loader of stage g + kBStages wait for it.
    if (warp >= kFillWarp0 && warp < kLoadWarp) {
        // =========================== fill ================================================================
        // Warp (a_slot, quarter) drops the entries of one plan bucket (this CTA's 128 rows x columns 16 quarter .. + 15
        // of the stage) into the A slot, after taking out what it dropped there for the stage kAStages earlier: a
        // place in the tile is only ever written by the one warp that owns its bucket.  All of them tell the FIRST
        // CTA's barrier.
        // batches of 32 entries a fill warp keeps in flight: a bucket holds 8 / V times as many entries at shorter vectors
        constexpr int kFillBatches = V == 8 ? 2 : 4;
        const int fw = warp - kFillWarp0;
        const uint32_t a_slot = (uint32_t)(fw % kAStages);
        const int quarter_k = fw / kAStages;
        uint8_t *a_part = sm + Smem::kA + a_slot * kAStageBytes;
        const int plan_blocks = (kBlockK / kPlanCols) * k_blocks;
        const uint32_t full_first = tc::map_to_cta(bar_full, 0);
        const int first = lane;                              // this lane's entry of batch 0, from the bucket's start
        constexpr int kStride = 32;                          // from one batch to the next

        struct Pos { int b, mt, kb; bool valid; };
        Walk walk;
        walk.init(pair, pairs, a_slot, total_stages, m_tiles, n_tiles, k_blocks);
        auto locate = [&]() {
            Pos q;
            q.valid = walk.valid(); q.b = walk.b; q.mt = walk.mt; q.kb = walk.kb;
            walk.advance(kAStages);
            return q;
        };
        auto bounds = [&](const Pos &q, int &e0, int &e1) {
            e0 = 0; e1 = 0;
            if (q.valid) {
                const int32_t *o = blk_offsets + ((int64_t)q.mt * (kTileM / kGroupRows) + (int)rank) * (plan_blocks + 1) +
                                   (kBlockK / kPlanCols) * q.kb + (kFillCols / kPlanCols) * quarter_k;
                e0 = __ldg(o) + first;   // this lane's first entry
                e1 = __ldg(o + kFillCols / kPlanCols);
            }
        };
        // Software pipeline over this warp's stages (a_slot, a_slot + kAStages, ...).  Everything a stage needs from
        // global memory — its entries, the values of its first entries, the bucket bounds of the stages after it — is
        // requested right AFTER the previous stage of this warp has been handed over, and is on its way while the
        // warp waits for its slot.  Nothing may still be in flight when the warp reaches the proxy fence: the fence
        // waits for the warp's outstanding loads too, and a value that comes from HBM takes ~2000 cycles, which
        // would then sit between "slot free" and "slot refilled" on the critical path of the ring.
        int c_e0, c_e1, c_b, n_e0, n_e1, n_b, f_e0, f_e1, f_b;
        { const Pos q = locate(); bounds(q, c_e0, c_e1); c_b = q.b; }
        { const Pos q = locate(); bounds(q, n_e0, n_e1); n_b = q.b; }
        { const Pos q = locate(); bounds(q, f_e0, f_e1); f_b = q.b; }
        const __half *values0 = static_cast<const __half *>(p.values);
        uint2 c_ent[kFillBatches], n_ent[kFillBatches];
        ValueVec<V> c_val[kFillBatches];
#pragma unroll
        for (int u = 0; u < kFillBatches; ++u) {
            const int e = c_e0 + kStride * u, en = n_e0 + kStride * u;
            c_ent[u] = e < c_e1 ? __ldg(blk_entries + e) : make_uint2(0u, 0u);
            n_ent[u] = en < n_e1 ? __ldg(blk_entries + en) : make_uint2(0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < kFillBatches; ++u)
            if (c_e0 + kStride * u < c_e1) c_val[u].load(values0 + (int64_t)c_b * p.stride_values + (int64_t)c_ent[u].x * V);
        int p_e0 = 0, p_e1 = 0;
        uint32_t p_pos[kFillBatches] = {};
        bool ok_run = true;
        for (uint32_t g = a_slot; g < total_stages && ok_run; g += kAStages) {
            if (g >= (uint32_t)kAStages) {   // the stage that used this A slot before must have been multiplied
                const uint32_t prev = g - kAStages;
                ok_run = wait_or_abort<kSleepFill>(bar_done + 8 * (prev % kBarStages), (prev / kBarStages) & 1u, abort_flag, abort_addr, peer);
            }
            if (!ok_run) break;
            if (p_e1 - (p_e0 - lane) > kStride * kFillBatches) {   // warp-uniform
                // back to zeros, denser buckets: the positions beyond the ones kept in registers would have to be
                // loaded again; clearing the warp's whole region (its 32 columns are 4 KiB in each 64-row atom) with
                // 16 wide stores per lane is cheaper and waits for nothing
#pragma unroll
                for (int atom = 0; atom < kCtaRows / 64; ++atom)
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        *reinterpret_cast<uint4 *>(a_part + atom * 8192 + quarter_k * 4096 + (i * 32 + lane) * 16) = make_uint4(0, 0, 0, 0);
            } else {   // back to zeros: overwrite exactly the vectors this warp dropped into the slot last time
                typename ValueVec<V>::Raw zero{};
#pragma unroll
                for (int u = 0; u < kFillBatches; ++u)
                    if (p_e0 + kStride * u < p_e1) scatter_vector<V, kTransposed>(a_part, p_pos[u], zero);
            }
            __syncwarp();
#pragma unroll
            for (int u = 0; u < kFillBatches; ++u)
                if (c_e0 + kStride * u < c_e1) scatter_vector<V, kTransposed>(a_part, c_ent[u].y, c_val[u].raw);
            {
                const __half *vals = values0 + (int64_t)c_b * p.stride_values;
                for (int e0 = c_e0 + kStride * kFillBatches; e0 - lane < c_e1; e0 += kStride * kOverflowBatches) {   // denser buckets
                    uint2 en[kOverflowBatches];
                    ValueVec<V> val[kOverflowBatches];
#pragma unroll
                    for (int u = 0; u < kOverflowBatches; ++u) {
                        const int e = e0 + kStride * u;
                        en[u] = e < c_e1 ? __ldg(blk_entries + e) : make_uint2(0u, 0u);
                    }
#pragma unroll
                    for (int u = 0; u < kOverflowBatches; ++u)
                        if (e0 + kStride * u < c_e1) val[u].load(vals + (int64_t)en[u].x * V);
#pragma unroll
                    for (int u = 0; u < kOverflowBatches; ++u)
                        if (e0 + kStride * u < c_e1) scatter_vector<V, kTransposed>(a_part, en[u].y, val[u].raw);
                }
            }
            p_e0 = c_e0; p_e1 = c_e1;
#pragma unroll
            for (int u = 0; u < kFillBatches; ++u) p_pos[u] = c_ent[u].y;
            tc::fence_proxy_async();   // ordinary stores; the MMA reads through the async proxy
            __syncwarp();
            if (lane == 0) tc::mbar_arrive_remote(full_first + 8 * (g % kBarStages));

            // the next stage of this warp: its values, the entries of the one after, the bounds of the one after that
            c_e0 = n_e0; c_e1 = n_e1; c_b = n_b;
#pragma unroll
            for (int u = 0; u < kFillBatches; ++u) c_ent[u] = n_ent[u];
            {
                const __half *vals = values0 + (int64_t)c_b * p.stride_values;
#pragma unroll
                for (int u = 0; u < kFillBatches; ++u)
                    if (c_e0 + kStride * u < c_e1) c_val[u].load(vals + (int64_t)c_ent[u].x * V);
            }
            n_e0 = f_e0; n_e1 = f_e1; n_b = f_b;
#pragma unroll
            for (int u = 0; u < kFillBatches; ++u) {
                const int e = n_e0 + kStride * u;
                n_ent[u] = e < n_e1 ? __ldg(blk_entries + e) : make_uint2(0u, 0u);
            }
            { const Pos q = locate(); bounds(q, f_e0, f_e1); f_b = q.b; }
        }
    } else if (warp == kLoadWarp) {
        // =========================== B loader ============================================================
        // This CTA's half of every B tile, up to kBStages stages ahead, into its own shared memory, completing on its
        // own barrier.  At the end it waits for the last "multiplied" signals addressed to this CTA, so that none of
        // them can arrive after the CTA has gone.
        if (lane == 0) {
            bool ok_run = true;
            const uint32_t full_first = tc::map_to_cta(bar_full, 0);
            Walk walk;
            walk.init(pair, pairs, 0u, total_stages, m_tiles, n_tiles, k_blocks);
            for (uint32_t g = 0; g < total_stages && ok_run; ++g, walk.advance(1)) {
                const uint32_t slot = g % kBStages;
                if (g >= (uint32_t)kBStages) {   // the stage that used this B slot before must have been multiplied
                    const uint32_t prev = g - kBStages;
                    ok_run = wait_or_abort<kSleepFill>(bar_done + 8 * (prev % kBarStages), (prev / kBarStages) & 1u, abort_flag, abort_addr, peer);
                }
                if (!ok_run) break;
                // cta_group::2 loads: the tile lands here, its bytes are counted on the FIRST CTA's barrier, which that
                // CTA's loader arms with the bytes of both halves
                const uint32_t bar = full_first + 8 * (g % kBarStages);
                const int n0 = walk.nt * tn + (int)rank * half_cols;   // first column of this CTA's half
                if (rank == 0) tc::mbar_expect_tx(bar_full + 8 * (g % kBarStages), 2u * (uint32_t)slabs * kBSlabBytes);
                if (slabs == 2) {
                    tc::tma_load_4d_pair(base + Smem::kB + slot * kBStageBytes, &map_b2, bar, 0, walk.kb * kBlockK, n0 >> 6, walk.b);
                } else {
                    tc::tma_load_3d_pair(base + Smem::kB + slot * kBStageBytes, &map_b, bar, n0, walk.kb * kBlockK, walk.b);
                }
            }
            const uint32_t tail0 = total_stages > (uint32_t)kBarStages ? total_stages - kBarStages : 0u;
            for (uint32_t g = tail0; g < total_stages && ok_run; ++g)
                ok_run = wait_or_abort<kSleepFill>(bar_done + 8 * (g % kBarStages), (g / kBarStages) & 1u, abort_flag, abort_addr, peer);
        }
    } else if (warp == kMmaWarp) {
        if (lane == 0 && rank == 0) {
            // =========================== MMA issuer of the pair ==========================================
            const uint32_t a_lo0 = tc::smem_desc_lo(base + Smem::kA, 8192);   // 64-row atoms 8 KiB apart
            const uint32_t a_hi = tc::smem_desc_hi(1024, (uint32_t)tc::kSwizzle128B);
            const uint32_t b_lo0 = tc::smem_desc_lo(base + Smem::kB, kBSlabBytes);   // 64-column slabs 8 KiB apart
            const uint32_t b_hi = tc::smem_desc_hi(1024, (uint32_t)tc::kSwizzle128B);
            const uint32_t idesc = tc::make_idesc_f16(256, tn, 1, 1);   // both operands MN-major
            // Per stage: one barrier poll, four MMAs, one commit.  No tensor-core fence per stage: the operands were
            // written by TMA, or by stores that their writers fenced for the async proxy before arriving.
            uint32_t a_slot = 0, b_slot = 0, bar = 0, parity = 0;
            const int steps_last = ((p.K - 1) & (kBlockK - 1)) / 16 + 1;   // K steps of the last column block of A
            bool ok_run = true;
            for (uint32_t i = 0; i < my_items && ok_run; ++i) {
                const uint32_t buf = i & 1u;
                ok_run = wait_or_abort<kSleepMma>(bar_acc_empty + 8 * buf, (i >> 1) & 1u, abort_flag, abort_addr, peer);
                if (!ok_run) break;
                tc::tc_fence_after_sync();
                const uint32_t d = tmem_base + buf * kMaxTileN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    ok_run = wait_or_abort<kSleepMma>(bar_full + 8 * bar, parity, abort_flag, abort_addr, peer);
                    if (!ok_run) break;
                    const uint32_t a_lo = a_lo0 + a_slot * (kAStageBytes >> 4), b_lo = b_lo0 + b_slot * (kBStageBytes >> 4);
                    // 16 columns of A = 16 rows of B = 2 KiB further on in either operand
                    if (kb + 1 < k_blocks || steps_last == kBlockK / 16) {
                        tc::mma_f16_ss_pair(d, tc::desc64(a_lo, a_hi), tc::desc64(b_lo, b_hi), idesc, kb > 0 ? 1u : 0u);
                        tc::mma_f16_ss_pair(d, tc::desc64(a_lo + 128, a_hi), tc::desc64(b_lo + 128, b_hi), idesc, 1u);
                        tc::mma_f16_ss_pair(d, tc::desc64(a_lo + 256, a_hi), tc::desc64(b_lo + 256, b_hi), idesc, 1u);
                        tc::mma_f16_ss_pair(d, tc::desc64(a_lo + 384, a_hi), tc::desc64(b_lo + 384, b_hi), idesc, 1u);
                    } else {
                        for (int kk = 0; kk < steps_last; ++kk)
                            tc::mma_f16_ss_pair(d, tc::desc64(a_lo + 128 * kk, a_hi), tc::desc64(b_lo + 128 * kk, b_hi), idesc,
                                                (kb > 0 || kk > 0) ? 1u : 0u);
                    }
                    tc::mma_commit_pair_both(bar_done + 8 * bar);   // "stage multiplied", in both CTAs at once
                    if (++a_slot == (uint32_t)kAStages) a_slot = 0;
                    if (++b_slot == (uint32_t)kBStages) b_slot = 0;
                    if (++bar == (uint32_t)kBarStages) { bar = 0; parity ^= 1u; }
                }
                if (ok_run) tc::mma_commit_pair_both(bar_acc_full + 8 * buf);
            }
        }
    } else {
        // =========================== epilogue ============================================================
        // Warp (quarter, half) owns accumulator lanes 32 quarter .. + 31 (rows 128 rank + 32 quarter .. of the tile)
        // and columns half * tn / 2 .. + tn / 2 - 1, moved out 32 columns at a time.
        constexpr int kBoxBytes = 32 * kStoreCols * (int)sizeof(TOut);
        constexpr int kBoxes = kStoreBoxBytes / kBoxBytes;
        constexpr int kRowBytes = kStoreCols * (int)sizeof(TOut);
        constexpr int kChunks = kRowBytes / 16;
        bool ok_run = true;
        float finite_probe[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const int quarter = warp & 3, half = warp >> 2;
        uint8_t *stg = sm + Smem::kStaging + warp * kStoreBoxBytes;
        const uint32_t stg_u32 = base + Smem::kStaging + warp * kStoreBoxBytes;
        const uint32_t lane_taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * half_cols);
        const int swz = (kRowBytes == 128) ? (lane & 7) : ((lane >> 1) & 3);
        const uint32_t acc_empty_first = tc::map_to_cta(bar_acc_empty, 0);
        uint32_t box_count = 0;
        tc::tc_fence_before_sync();
        tc::mbar_arrive_remote(acc_empty_first);        // both accumulator buffers start out free
        tc::mbar_arrive_remote(acc_empty_first + 8);
        Walk walk;
        walk.init(pair, pairs, 0u, my_items, m_tiles, n_tiles, 1);
        for (uint32_t i = 0; i < my_items && ok_run; ++i, walk.advance(1)) {
            const uint32_t buf = i & 1u;
            ok_run = __all_sync(0xffffffffu, wait_or_abort<kSleepEpilogue>(bar_acc_full + 8 * buf, (i >> 1) & 1u, abort_flag, abort_addr, peer));
            if (!ok_run) break;

            tc::tc_fence_after_sync();
            const int row0 = walk.mt * kTileM + (int)rank * kCtaRows + quarter * 32;
            const int col0 = walk.nt * tn + half * half_cols;   // accumulator column c of the item is its output column c
#pragma unroll 1
            for (int c0 = 0; c0 < half_cols; c0 += kStoreCols) {
                uint32_t r[kStoreCols];
                tc::tmem_ld_x32(lane_taddr + buf * kMaxTileN + (uint32_t)c0, r);
                if (row0 < m_rows) {   // warp-uniform
                    if (row0 + lane < m_rows) {
#pragma unroll
                        for (int e = 0; e < kStoreCols; ++e) finite_probe[e & 3] = fmaf(__uint_as_float(r[e]), 0.0f, finite_probe[e & 3]);
                    }
                    const uint32_t box = kBoxes == 2 ? (box_count & 1u) : 0u;
                    if (lane == 0) tc::bulk_wait_group_read<kBoxes - 1>();
                    __syncwarp();
                    uint8_t *dst = stg + box * kBoxBytes + lane * kRowBytes;
#pragma unroll
                    for (int u = 0; u < kChunks; ++u) {
                        uint4 v;
                        if constexpr (sizeof(TOut) == 2) {
                            __half2 *hh = reinterpret_cast<__half2 *>(&v);
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                hh[e] = __floats2half2_rn(__uint_as_float(r[8 * u + 2 * e]), __uint_as_float(r[8 * u + 2 * e + 1]));
                        } else {
                            v = make_uint4(r[4 * u], r[4 * u + 1], r[4 * u + 2], r[4 * u + 3]);
                        }
                        *reinterpret_cast<uint4 *>(dst + ((u ^ swz) << 4)) = v;
                    }
                    tc::fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        tc::tma_store_3d(&map_out, stg_u32 + box * kBoxBytes, col0 + c0, row0, walk.b);
                        tc::bulk_commit_group();
                    }
                    ++box_count;
                }
            }
            tc::tc_fence_before_sync();
            tc::mbar_arrive_remote(acc_empty_first + 8 * buf);   // read out: the buffer is free for the pair

        }
        if (lane == 0) tc::bulk_wait_group<0>();
        const float probe = (finite_probe[0] + finite_probe[1]) + (finite_probe[2] + finite_probe[3]);
        if (__any_sync(0xffffffffu, probe != 0.0f) && lane == 0) atomicExch(use_dense, 0);
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

}  // namespace pairspmm
}  // namespace vs
