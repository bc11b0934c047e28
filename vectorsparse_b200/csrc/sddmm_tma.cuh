// Tensor-core SDDMM for fp16 operands on sm_100a with a TMA row gather: the `wmmaSddmm` entry point of the
// reference (src/wmma_sddmm.cu holds its twelve Volta kernels: V = 8/4/2 times the four `algorithm` variants of
// one function) rebuilt on tcgen05 + TMA.
//
// Formulation.  For one vector-row i and one tile of 128 of its mask entries the kernel computes
//     D[128 entries x 16] (+)= Rg[128 entries x 64] * L_i^T[64 x 16]
// per 64-wide block of the contraction: Rg = rows of rhs selected by col_indices, L_i = the V (<= 8) lhs rows
// of the vector-row, zero-padded to 16.  Both operands are K-major in shared memory with the 128-byte swizzle
// (a row block is 64 fp16 = 128 bytes).  D row e, column v is out[(j0 + e) * V + v]: each epilogue thread owns
// one mask entry and stores its V outputs with one vector store, neighbouring threads writing neighbouring
// addresses.
//
// Both operands arrive by TMA gather4 (four rows x 64 columns per instruction, written swizzled where the MMA
// wants them): lane g of the producing warp fetches mask entries 4g..4g+3 of the tile, lanes 0/1 the lhs rows.
// Entries past the end of a vector-row are not fetched at all (their accumulator rows are never stored); lhs
// rows past V get an out-of-range coordinate and arrive as zeros.
//
// Organisation: as the TMA SpMM.  Two persistent CTAs per SM; warps 0-3 epilogue, warps 4-8 producers (warp w
// takes every 5th stage; a stage is one tile x one 64-wide block of k), warp 9 one MMA-issuing thread.  Work
// items are (batch, vector-row in row_indices order) dealt round-robin; each CTA decodes 128 items at a time.
// Every wait is bounded; a wait that runs out raises the CTA's abort flag, all roles leave through the phase
// barrier, a status bit is set and tensor memory is freed.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace vs {
namespace tmasddmm {

constexpr int kEpiWarps = 4;                             // warps 0..3 (TMEM lane quarter = warp index)
constexpr int kProducerWarp0 = 4;
constexpr int kProducerWarps = 5;                        // warps 4..8: one per ring slot
constexpr int kMmaWarp = kProducerWarp0 + kProducerWarps;  // warp 9
constexpr int kThreads = (kMmaWarp + 1) * 32;            // 320
constexpr int kCtasPerSm = 2;
constexpr int kTileE = 128;                              // mask entries per tile (MMA M)
constexpr int kBlockK = 64;                              // contraction elements per stage (four K=16 MMAs)
constexpr int kStages = 5;
constexpr int kAStageBytes = kTileE * kBlockK * 2;       // 16 KiB gathered rhs rows
constexpr int kBStageBytes = 16 * kBlockK * 2;           // 2 KiB lhs rows (V real, the rest zeros)
constexpr int kAccCols = 16;
constexpr int kTmemCols = 256;
constexpr int kAccSlots = kTmemCols / kAccCols;          // 16
constexpr int kIdxRing = 3;                              // per-warp ring of index blocks (kTileE ints each)
constexpr int kItemsPerPhase = 128;

constexpr uint32_t kStatusTimeout = 32u;

struct Smem {
    static constexpr int kA = 0;
    static constexpr int kB = kA + kStages * kAStageBytes;
    static constexpr int kRow = kB + kStages * kBStageBytes;
    static constexpr int kJ0 = kRow + kItemsPerPhase * 4;
    static constexpr int kEnd = kJ0 + kItemsPerPhase * 4;
    static constexpr int kItemB = kEnd + kItemsPerPhase * 4;
    static constexpr int kIdx = kItemB + kItemsPerPhase * 4;     // [producer warp][ring slot][kTileE]
    static constexpr int kBarFull = kIdx + kProducerWarps * kIdxRing * kTileE * 4;
    static constexpr int kBarEmpty = kBarFull + kStages * 8;
    static constexpr int kBarAccFull = kBarEmpty + kStages * 8;
    static constexpr int kBarAccEmpty = kBarAccFull + kAccSlots * 8;
    static constexpr int kTmemHolder = kBarAccEmpty + kAccSlots * 8;
    static constexpr int kAbort = kTmemHolder + 8;
    static constexpr int kPhaseStages = kAbort + 8;          // two counters, used by alternate phases
    static constexpr int kTotal = kPhaseStages + 8;
};
constexpr int kSmemBytes = Smem::kTotal + 1024;
// a ring slot must always be refilled by the same warp (see the SpMM kernel)
static_assert(kStages % kProducerWarps == 0, "each ring slot needs a fixed owner warp");
static_assert(kCtasPerSm * (kSmemBytes + 1024) <= 227 * 1024, "shared memory budget");

// Stage s of an item: tile s / nkb, k-block s % nkb.  Rows without entries have no stages.
__device__ __forceinline__ int stages_of(int len, int nkb) { return ((len + kTileE - 1) / kTileE) * nkb; }

// Position of one stage inside a phase (item q, stage s of it); advance(k) moves k stages forward across items,
// skipping items that have none.
struct OwnIter {
    const int *j0, *jend;
    int cnt, nkb, q, s, nst, jb, je;
    __device__ __forceinline__ void load() {
        if (q < cnt) { jb = j0[q]; je = jend[q]; nst = stages_of(je - jb, nkb); } else { nst = 1; }
    }
    __device__ __forceinline__ void normalise() {
        while (q < cnt && s >= nst) { s -= nst; ++q; load(); }
    }
    __device__ __forceinline__ void init(const int *j0_, const int *jend_, int cnt_, int nkb_) {
        j0 = j0_; jend = jend_; cnt = cnt_; nkb = nkb_; q = 0; s = 0; jb = 0; je = 0;
        load();
        normalise();
    }
    __device__ __forceinline__ bool valid() const { return q < cnt; }
    __device__ __forceinline__ int tile_j() const { return jb + (s / nkb) * kTileE; }   // first entry of the tile
    __device__ __forceinline__ int kb() const { return s % nkb; }
    __device__ __forceinline__ void advance(int k) { s += k; normalise(); }
};

template <int kSleepNs>
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (tc::mbar_try_wait(bar, parity)) return true;
    for (uint32_t i = 0; i < tc::kMaxPolls; ++i) {
        if (kSleepNs > 0) __nanosleep(kSleepNs);
        if (tc::mbar_try_wait(bar, parity)) return true;
        if ((i & 15u) == 15u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
constexpr int kSleepProducer = 100, kSleepMma = 0, kSleepEpilogue = 100;

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// map_rhs / map_lhs: tensor maps of rhs and lhs seen as ONE row-major fp16 matrix each (all batch entries
// stacked: entry b starts at row b * rows_per_batch), k columns, box 64 columns x 1 row, 128-byte swizzle.
template <typename TOut, int V>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
sddmm_tma_kernel(const SddmmParams p, const __grid_constant__ CUtensorMap map_rhs, const __grid_constant__ CUtensorMap map_lhs,
                 int rhs_rows_per_batch, int rhs_total_rows, int lhs_rows_per_batch, int lhs_total_rows, uint32_t *status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = tc::smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);

    const int t = threadIdx.x;
    const int warp = t >> 5;
    const int lane = t & 31;
    int *l_row = reinterpret_cast<int *>(sm + Smem::kRow);
    int *l_j0 = reinterpret_cast<int *>(sm + Smem::kJ0);
    int *l_end = reinterpret_cast<int *>(sm + Smem::kEnd);
    int *l_b = reinterpret_cast<int *>(sm + Smem::kItemB);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(sm + Smem::kAbort);
    int *phase_tile_count = reinterpret_cast<int *>(sm + Smem::kPhaseStages);
    const uint32_t bar_full = base + Smem::kBarFull;
    const uint32_t bar_empty = base + Smem::kBarEmpty;
    const uint32_t bar_acc_full = base + Smem::kBarAccFull;
    const uint32_t bar_acc_empty = base + Smem::kBarAccEmpty;

    // ---- set-up: zero the lhs stages (rows V..15 stay zero for good), barriers, tensor memory ---------------
    for (int i = t; i < kStages * kBStageBytes / 16; i += kThreads)
        reinterpret_cast<uint4 *>(sm + Smem::kB)[i] = make_uint4(0, 0, 0, 0);
    if (t == 0) {
        for (int s = 0; s < kStages; ++s) {
            tc::mbar_init(bar_full + 8 * s, 1);    // one arrival (with the byte count) by the producing warp
            tc::mbar_init(bar_empty + 8 * s, 1);
        }
        for (int s = 0; s < kAccSlots; ++s) {
            tc::mbar_init(bar_acc_full + 8 * s, 1);
            tc::mbar_init(bar_acc_empty + 8 * s, kEpiWarps * 32);
        }
        *abort_flag = 0;
        phase_tile_count[0] = 0;
        phase_tile_count[1] = 0;
        tc::fence_mbar_init();
    }
    if (warp == kMmaWarp) {
        tc::tmem_alloc(base + Smem::kTmemHolder, kTmemCols);
        tc::tmem_relinquish();
    }
    tc::fence_proxy_async();
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t *>(sm + Smem::kTmemHolder);

    const int nkb = p.k / kBlockK;
    const int64_t total_items = (int64_t)p.batch * p.m_vec;
    const int64_t G = gridDim.x;
    const int64_t my_items = (total_items > blockIdx.x) ? (total_items - blockIdx.x + G - 1) / G : 0;

    uint32_t g_stage = 0;   // stages of earlier phases (ring position and barrier parity), same in every role
    uint32_t g_tile = 0;    // tiles of earlier phases (accumulator slot and parity)

    int phase_parity = 0;
    for (int64_t ph0 = 0; ph0 < my_items; ph0 += kItemsPerPhase, phase_parity ^= 1) {
        const int cnt = (int)((my_items - ph0 < kItemsPerPhase) ? (my_items - ph0) : kItemsPerPhase);
        // ---- phase set-up: decode this CTA's next items in bulk ----------------------------------------------
        if (t < kItemsPerPhase) {
            int tiles = 0;
            if (t < cnt) {
                const int64_t w = blockIdx.x + (ph0 + t) * G;
                const int64_t b = w / p.m_vec;
                const int o = (int)(w - b * p.m_vec);
                const int row = __ldg(p.row_indices + o);
                const int jb = __ldg(p.row_offsets + row), je = __ldg(p.row_offsets + row + 1);
                l_row[t] = row;
                l_j0[t] = jb;
                l_end[t] = je;
                l_b[t] = (int)b;
                tiles = (je - jb + kTileE - 1) / kTileE;
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) tiles += __shfl_xor_sync(0xffffffffu, tiles, off);
            if (lane == 0 && tiles) atomicAdd(phase_tile_count + phase_parity, tiles);
        }
        __syncthreads();
        const uint32_t tiles_here = (uint32_t)phase_tile_count[phase_parity];
        if (t == 0) phase_tile_count[phase_parity ^ 1] = 0;   // next phase's counter; nobody touches it until then

        if (warp >= kProducerWarp0 && warp < kMmaWarp) {
            // =========================== producers =======================================================
            const int pw = warp - kProducerWarp0;
            int *ring = reinterpret_cast<int *>(sm + Smem::kIdx) + pw * kIdxRing * kTileE;
            const uint32_t ring_u32 = base + Smem::kIdx + pw * kIdxRing * kTileE * 4;
            const int s0 = (int)(((uint32_t)pw + kProducerWarps - (g_stage % kProducerWarps)) % kProducerWarps);
            OwnIter cur, fetch;
            cur.init(l_j0, l_end, cnt, nkb);
            cur.advance(s0);
            fetch = cur;
            for (int n = 0; n < 2; ++n) {   // indices of this warp's first two stages: plain loads, once per phase
                if (fetch.valid()) {
#pragma unroll
                    for (int u = 0; u < kTileE / 32; ++u) {
                        const int jj = fetch.tile_j() + lane + 32 * u;
                        ring[n * kTileE + lane + 32 * u] = (jj < fetch.je) ? __ldg(p.col_indices + jj) : 0;
                    }
                    fetch.advance(kProducerWarps);
                }
            }
            __syncwarp();

            uint32_t g = g_stage + (uint32_t)s0;
            int n = 0;
            bool ok_run = true;
            while (cur.valid() && ok_run) {
                const uint32_t slot = g % kStages;
                if (g >= (uint32_t)kStages)
                    ok_run = wait_or_abort<kSleepProducer>(bar_empty + 8 * slot, ((g / kStages) - 1u) & 1u, abort_flag);
                if (!ok_run) break;
                tc::cp_async_wait<1>();   // this stage's indices (fetched two of this warp's stages ago) have landed
                __syncwarp();
                const int q = cur.q;
                const int b = l_b[q];
                const int tj = cur.tile_j();
                const int n_ent = min(kTileE, cur.je - tj);
                const int n_groups = (n_ent + 3) >> 2;
                constexpr int kLhsOps = V > 4 ? 2 : 1;
                const int x = cur.kb() * kBlockK;
                const uint32_t bar = bar_full + 8 * slot;
                if (lane == 0) tc::mbar_expect_tx(bar, (uint32_t)(n_groups + kLhsOps) * 512u);
                __syncwarp();
                if (lane < n_groups) {
                    const int4 c = *reinterpret_cast<const int4 *>(ring + (n % kIdxRing) * kTileE + 4 * lane);
                    const int r0 = b * rhs_rows_per_batch, e = 4 * lane;
                    tc::tma_gather4(base + Smem::kA + slot * kAStageBytes + lane * 512, &map_rhs, bar, x,
                                    r0 + c.x, e + 1 < n_ent ? r0 + c.y : rhs_total_rows,
                                    e + 2 < n_ent ? r0 + c.z : rhs_total_rows, e + 3 < n_ent ? r0 + c.w : rhs_total_rows);
                }
                if (lane < kLhsOps) {
                    const int r0 = b * lhs_rows_per_batch + l_row[q] * V + 4 * lane, e = 4 * lane;
                    tc::tma_gather4(base + Smem::kB + slot * kBStageBytes + lane * 512, &map_lhs, bar, x,
                                    r0, e + 1 < V ? r0 + 1 : lhs_total_rows, e + 2 < V ? r0 + 2 : lhs_total_rows,
                                    e + 3 < V ? r0 + 3 : lhs_total_rows);
                }
                if (fetch.valid()) {   // column indices of this warp's stage n + 2
#pragma unroll
                    for (int u = 0; u < kTileE / 32; ++u) {
                        const int jj = fetch.tile_j() + lane + 32 * u;
                        const bool ok = jj < fetch.je;
                        tc::cp_async_small<4>(ring_u32 + (((n + 2) % kIdxRing) * kTileE + lane + 32 * u) * 4,
                                              ok ? p.col_indices + jj : p.col_indices, ok ? 4u : 0u);
                    }
                    fetch.advance(kProducerWarps);
                }
                tc::cp_async_commit();
                cur.advance(kProducerWarps);
                g += kProducerWarps;
                ++n;
            }
            tc::cp_async_wait<0>();
        } else if (warp == kMmaWarp) {
            // =========================== MMA issuer ========================================================
            // One issuing thread for all stages, in ring order: an mbarrier parity wait is only safe for a
            // consumer that has itself seen the slot's previous use complete.
            if (lane == 0) {
                constexpr uint32_t kIdesc = tc::make_idesc_f16(kTileE, 16, 0, 0);
                const uint32_t a_lo0 = tc::smem_desc_lo(base + Smem::kA, 16);
                const uint32_t b_lo0 = tc::smem_desc_lo(base + Smem::kB, 16);
                const uint32_t hi = tc::smem_desc_hi(1024, (uint32_t)tc::kSwizzle128B);
                uint32_t slot = g_stage % kStages, full_parity = (g_stage / kStages) & 1u;
                uint32_t acc = g_tile % kAccSlots, acc_parity = ((g_tile / kAccSlots) & 1u) ^ 1u;   // parity of the previous use
                bool acc_wait = g_tile >= (uint32_t)kAccSlots;
                bool ok_run = true;
                for (int q = 0; q < cnt && ok_run; ++q) {
                    const int tiles = (l_end[q] - l_j0[q] + kTileE - 1) / kTileE;
                    for (int tl = 0; tl < tiles && ok_run; ++tl) {
                        if (acc_wait) ok_run = wait_or_abort<kSleepMma>(bar_acc_empty + 8 * acc, acc_parity, abort_flag);
                        const uint32_t d = tmem_base + acc * kAccCols;
                        for (int kb = 0; kb < nkb && ok_run; ++kb) {
                            ok_run = wait_or_abort<kSleepMma>(bar_full + 8 * slot, full_parity, abort_flag);
                            if (!ok_run) break;
                            tc::tc_fence_after_sync();
                            const uint32_t a_lo = a_lo0 + slot * (kAStageBytes >> 4);
                            const uint32_t b_lo = b_lo0 + slot * (kBStageBytes >> 4);
#pragma unroll
                            for (int mm = 0; mm < kBlockK / 16; ++mm)
                                tc::mma_f16_ss(d, tc::desc64(a_lo + 2 * mm, hi), tc::desc64(b_lo + 2 * mm, hi), kIdesc,
                                               (kb == 0 && mm == 0) ? 0u : 1u);
                            tc::mma_commit(bar_empty + 8 * slot);
                            if (++slot == (uint32_t)kStages) { slot = 0; full_parity ^= 1u; }
                        }
                        if (ok_run) tc::mma_commit(bar_acc_full + 8 * acc);
                        if (++acc == (uint32_t)kAccSlots) { acc = 0; acc_parity ^= 1u; acc_wait = true; }
                    }
                }
            }
        } else if (warp < kEpiWarps) {
            // =========================== epilogue ==========================================================
            uint32_t ic = g_tile;
            bool ok_run = true;
            for (int q = 0; q < cnt && ok_run; ++q) {
                const int jb = l_j0[q], je = l_end[q];
                TOut *out = static_cast<TOut *>(p.out) + (int64_t)l_b[q] * p.stride_out;
                for (int tj = jb; tj < je && ok_run; tj += kTileE, ++ic) {
                    const uint32_t acc = ic % kAccSlots;
                    // warp-uniform outcome: tcgen05.ld below needs all 32 lanes
                    ok_run = __all_sync(0xffffffffu, wait_or_abort<kSleepEpilogue>(bar_acc_full + 8 * acc, (ic / kAccSlots) & 1u, abort_flag));
                    if (!ok_run) break;
                    tc::tc_fence_after_sync();
                    uint32_t r[8];
                    tc::tmem_ld_x8(tmem_base + ((uint32_t)(warp * 32) << 16) + acc * kAccCols, r);
                    tc::tc_fence_before_sync();
                    mbar_arrive(bar_acc_empty + 8 * acc);     // the accumulator may be overwritten from here on
                    const int jj = tj + t;                    // this thread's mask entry (t = 0..127 here)
                    if (jj < je) {
                        float f[V];
#pragma unroll
                        for (int v = 0; v < V; ++v) f[v] = __uint_as_float(r[v]);
                        TOut *o = out + (int64_t)jj * V;
                        if constexpr (V >= 4) {
                            store_chunk(o, f);
                        } else {
#pragma unroll
                            for (int v = 0; v < V; ++v) store_scalar(o + v, f[v]);
                        }
                    }
                }
            }
        }

        // ---- phase end: everybody is done with the lists; advance the global counters identically ------------
        g_stage += tiles_here * (uint32_t)nkb;
        g_tile += tiles_here;
        tc::tc_fence_before_sync();
        __syncthreads();
        if (*abort_flag) break;
    }

    // ---- teardown ---------------------------------------------------------------------------------------
    if (*abort_flag && t == 0) atomicOr(status, kStatusTimeout);
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == kMmaWarp) tc::tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace tmasddmm
}  // namespace vs
