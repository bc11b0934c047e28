// Tensor-core SpMM for fp16 CVSE matrices on sm_100a with a TMA row gather: the `wmmaSpmm` entry point of the
// reference (src/wmma_spmm.cu:13-314 are its three Volta mma.m8n8k4 kernels) rebuilt on tcgen05 + TMA.
//
// Formulation.  For one vector-row r and one tile of 128 dense columns the kernel computes, transposed,
//     D[128 cols x 16] (+)= Bg^T[128 cols x 16 nnz] * Ar^T[16 nnz x 16]
// Bg = the rows of the dense operand selected by col_indices, Ar = the row's value vectors (V <= 8 of the 16
// columns are real, the rest a constant zero block).  Both operands are MN-major in shared memory: a gathered
// row of B is contiguous along the 128 columns (MMA-M), a value vector along V (MMA-N).  The accumulator lives
// in tensor memory, 16 fp32 columns per work item.
//
// The gather is done by the TMA unit: one cp.async.bulk.tensor ... tile::gather4 instruction fetches four rows
// of B (chosen by four row coordinates) x 64 columns and writes them, 128-byte swizzled, exactly where the MMA
// operand layout wants them; rows past the end of a vector-row are given an out-of-range coordinate and arrive
// as zeros.  A stage (up to 64 nonzero vectors x 128 columns = 16 KiB, up to four K=16 MMAs) is therefore
// ONE warp instruction: lane l issues the gather of rows 4*(l/2).. of column half l%2.  That replaces 32
// cp.async instructions per lane of a software gather and their address arithmetic.
//
// Organisation.  Two persistent CTAs per SM (four MMA-issuing threads per SM), warp-specialised, no CTA-wide
// barrier inside a phase:
//   * warps 0-3, epilogue: wait for `acc_full`, tcgen05.ld their 32 TMEM lanes, release the accumulator
//     (`acc_empty`), transpose through a warp-private staging tile and write C with 16-byte stores.
//   * warps 4-8, producers: warp w takes every 5th stage.  It waits for the stage's ring slot (`empty`), arms
//     the slot's `full` mbarrier with the byte count, issues the gathers, copies the value vectors with
//     cp.async (arriving on `full` when they land), and prefetches the column indices of its stage n+2.
//   * warps 9-10, one thread each (even / odd work items): wait for `full`, issue the MMAs of the stage and
//     commit them to the slot's `empty` mbarrier and, at the end of a row, to `acc_full`.
// Work items are (batch, column tile, vector-row in row_indices order), dealt round-robin to the CTAs so that
// the descending-length order the row swizzle produces becomes a longest-first schedule; each CTA decodes its
// next 128 items in bulk ("phase") so that no role chases row_indices -> row_offsets per item.
// Every wait is bounded; a wait that runs out raises the CTA's abort flag, all roles leave through the phase
// barrier, a status bit is set and tensor memory is freed.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace vs {
namespace tmaspmm {

constexpr int kEpiWarps = 4;                             // warps 0..3 (TMEM lane quarter = warp index)
constexpr int kProducerWarp0 = 4;
constexpr int kProducerWarps = 5;                        // warps 4..8: one per ring slot
constexpr int kMmaWarp = kProducerWarp0 + kProducerWarps;  // warp 9
constexpr int kMmaWarps = 2;                             // two issuing threads (even / odd work items)
constexpr int kThreads = (kMmaWarp + kMmaWarps) * 32;    // 352
constexpr int kCtasPerSm = 2;
constexpr int kTileN = 128;                              // dense columns per work item (MMA M)
constexpr int kStageNnz = 64;                            // nonzero vectors per stage (up to four K=16 MMAs)
constexpr int kMmaPerStage = kStageNnz / 16;
constexpr int kStages = 5;                               // shared-memory ring
constexpr int kAStageBytes = kStageNnz * kTileN * 2;     // 16 KiB
constexpr int kVStageBytes = 2 * kStageNnz * 16;         // 2 KiB: 64 value slots of 16 B, then 1 KiB of zeros
constexpr int kAccCols = 16;                             // TMEM columns per accumulator
constexpr int kTmemCols = 256;
constexpr int kAccSlots = kTmemCols / kAccCols;          // 16
constexpr int kIdxRing = 2;                              // per-warp index blocks (kStageNnz ints each), alternating
constexpr int kItemsPerPhase = 128;
constexpr int kStagingBytes = 8 * 32 * 4;                // per epilogue warp: 8 rows x 32 columns, fp32 worst case

constexpr uint32_t kStatusTimeout = 16u;  // bit raised in the status word when a bounded wait ran out

struct Smem {  // offsets from the 1024-byte aligned base
    static constexpr int kA = 0;
    static constexpr int kV = kA + kStages * kAStageBytes;
    static constexpr int kRow = kV + kStages * kVStageBytes;
    static constexpr int kJ0 = kRow + kItemsPerPhase * 4;
    static constexpr int kEnd = kJ0 + kItemsPerPhase * 4;
    static constexpr int kItemB = kEnd + kItemsPerPhase * 4;
    static constexpr int kItemN0 = kItemB + kItemsPerPhase * 4;
    static constexpr int kIdx = kItemN0 + kItemsPerPhase * 4;    // [producer warp][ring slot][kStageNnz]
    static constexpr int kStaging = kIdx + kProducerWarps * kIdxRing * kStageNnz * 4;
    static constexpr int kBarFull = kStaging + kEpiWarps * kStagingBytes;
    static constexpr int kBarEmpty = kBarFull + kStages * 8;
    static constexpr int kBarAccFull = kBarEmpty + kStages * 8;
    static constexpr int kBarAccEmpty = kBarAccFull + kAccSlots * 8;
    static constexpr int kTmemHolder = kBarAccEmpty + kAccSlots * 8;
    static constexpr int kAbort = kTmemHolder + 8;
    static constexpr int kPhaseStages = kAbort + 8;          // two counters, used by alternate phases
    static constexpr int kMmaDone = kPhaseStages + 8;        // per MMA issuer: stages below this index are waited on
    static constexpr int kTotal = kMmaDone + 8;
};
constexpr int kSmemBytes = Smem::kTotal + 1024;  // + slack for the manual 1024-byte alignment
// A ring slot must always be refilled by the same warp: a producer's parity wait on `empty` is only meaningful
// if that producer has itself seen the slot's previous release (two warps sharing a slot could run a full ring
// apart, pass the wait spuriously and arrive twice in one phase, which traps).
static_assert(kStages % kProducerWarps == 0, "each ring slot needs a fixed owner warp");
static_assert(kCtasPerSm * (kSmemBytes + 1024) <= 227 * 1024, "shared memory budget");

__device__ __forceinline__ int stages_of(int len) { return max(1, (len + kStageNnz - 1) / kStageNnz); }

// Position of one stage inside a phase: item q of the phase's lists and stage s of that item.  advance(k)
// moves k stages forward across item boundaries (every item has at least one stage, empty rows included).
struct OwnIter {
    const int *j0, *jend;
    int cnt, q, s, nst, jb, je;
    __device__ __forceinline__ void load() {
        jb = j0[q]; je = jend[q];
        nst = stages_of(je - jb);
    }
    __device__ __forceinline__ void init(const int *j0_, const int *jend_, int cnt_) {
        j0 = j0_; jend = jend_; cnt = cnt_; q = 0; s = 0; nst = 1; jb = 0; je = 0;
        if (cnt > 0) load();
    }
    __device__ __forceinline__ bool valid() const { return q < cnt; }
    __device__ __forceinline__ int j() const { return jb + s * kStageNnz; }
    __device__ __forceinline__ int nnz() const { return min(kStageNnz, max(0, je - j())); }
    __device__ __forceinline__ void advance(int k) {
        while (q < cnt) {
            if (s + k < nst) { s += k; return; }
            k -= nst - s;
            ++q; s = 0;
            if (q < cnt) load();
            if (k == 0) return;
        }
    }
};

// Bounded mbarrier wait that also gives up when another role of the CTA has raised the abort flag.
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
__device__ __forceinline__ void mbar_expect_tx_only(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Arrives on `bar` once every cp.async this thread has issued so far has completed (no pending-count bump:
// the barrier's expected count already includes this arrival).
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// `map`: tensor map of the dense operand seen as ONE row-major fp16 matrix [total_rows x N] (all batch entries
// stacked: entry b starts at row b * rows_per_batch), box 64 columns x 1 row, 128-byte swizzle, zero fill.
template <typename TOut, int V>
__global__ void __launch_bounds__(kThreads, kCtasPerSm)
spmm_tma_kernel(const SpmmParams p, const __grid_constant__ CUtensorMap map, int rows_per_batch, int total_rows,
                uint32_t *status, const int32_t *plan_hdr, int plan_checks) {
    pdl_launch_dependents();   // the next call's plan kernel may queue up behind this one
    pdl_wait();   // launched behind the dense kernel without waiting for its end: wait here, before its verdict is read
    if (plan_hdr && plan_dense_chosen(plan_hdr, plan_checks)) return;   // the dense kernel has taken this call (decided on the device)
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
    int *l_n0 = reinterpret_cast<int *>(sm + Smem::kItemN0);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(sm + Smem::kAbort);
    int *phase_stage_count = reinterpret_cast<int *>(sm + Smem::kPhaseStages);
    const uint32_t bar_full = base + Smem::kBarFull;
    const uint32_t bar_empty = base + Smem::kBarEmpty;
    const uint32_t bar_acc_full = base + Smem::kBarAccFull;
    const uint32_t bar_acc_empty = base + Smem::kBarAccEmpty;

    // ---- set-up: zero the value slots and their zero halves, barriers, tensor memory ----------------------
    for (int i = t; i < kStages * kVStageBytes / 16; i += kThreads)
        reinterpret_cast<uint4 *>(sm + Smem::kV)[i] = make_uint4(0, 0, 0, 0);
    if (t == 0) {
        for (int s = 0; s < kStages; ++s) {
            tc::mbar_init(bar_full + 8 * s, 32);   // the 32 lanes of the producing warp (value copies landed)
            tc::mbar_init(bar_empty + 8 * s, 1);
        }
        for (int s = 0; s < kAccSlots; ++s) {
            tc::mbar_init(bar_acc_full + 8 * s, 1);
            tc::mbar_init(bar_acc_empty + 8 * s, kEpiWarps * 32);
        }
        *abort_flag = 0;
        phase_stage_count[0] = 0;
        phase_stage_count[1] = 0;
        reinterpret_cast<volatile uint32_t *>(sm + Smem::kMmaDone)[0] = 0;
        reinterpret_cast<volatile uint32_t *>(sm + Smem::kMmaDone)[1] = 0;
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

    const int n_tiles = (p.N + kTileN - 1) / kTileN;
    const int64_t total_items = (int64_t)p.batch * n_tiles * p.m_vec;
    const int64_t G = gridDim.x;
    const int64_t my_items = (total_items > blockIdx.x) ? (total_items - blockIdx.x + G - 1) / G : 0;

    uint32_t g_stage = 0;   // stages of earlier phases (ring position and barrier parity), same in every role
    uint32_t g_item = 0;    // items of earlier phases (accumulator slot and parity)

    int phase_parity = 0;
    for (int64_t ph0 = 0; ph0 < my_items; ph0 += kItemsPerPhase, phase_parity ^= 1) {
        const int cnt = (int)((my_items - ph0 < kItemsPerPhase) ? (my_items - ph0) : kItemsPerPhase);
        // ---- phase set-up: decode this CTA's next items in bulk (one round of global latency) -----------
        if (t < kItemsPerPhase) {
            int nst = 0;
            if (t < cnt) {
                const int64_t w = blockIdx.x + (ph0 + t) * G;
                const int64_t bt = w / p.m_vec;              // (batch, tile) pair
                const int o = (int)(w - bt * p.m_vec);
                const int row = __ldg(p.row_indices + o);
                const int jb = __ldg(p.row_offsets + row), je = __ldg(p.row_offsets + row + 1);
                l_row[t] = row;
                l_j0[t] = jb;
                l_end[t] = je;
                l_b[t] = (int)(bt / n_tiles);
                l_n0[t] = (int)(bt % n_tiles) * kTileN;
                nst = stages_of(je - jb);
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) nst += __shfl_xor_sync(0xffffffffu, nst, off);
            if (lane == 0 && nst) atomicAdd(phase_stage_count + phase_parity, nst);
        }
        __syncthreads();
        const uint32_t stages_here = (uint32_t)phase_stage_count[phase_parity];
        if (t == 0) phase_stage_count[phase_parity ^ 1] = 0;   // next phase's counter; nobody touches it until then

        if (warp >= kProducerWarp0 && warp < kMmaWarp) {
            // =========================== producers =======================================================
            const int pw = warp - kProducerWarp0;
            const int grp = lane >> 1;       // rows 4*grp .. 4*grp+3 of the stage
            const int half = lane & 1;       // columns 64*half .. +63 of the tile
            // destination of this lane's four rows inside a stage: M-atom `half`, k-group grp/2, upper/lower 512 B
            const uint32_t a_off = (uint32_t)(half * (kAStageBytes / 2) + (grp >> 1) * 1024 + (grp & 1) * 512);
            int *ring = reinterpret_cast<int *>(sm + Smem::kIdx) + pw * kIdxRing * kStageNnz;

            // This warp's stages are kProducerWarps apart.  One iterator runs two of them ahead; the positions
            // and column indices of the next two stages wait in registers (indices loaded with plain loads two
            // stages early, so their latency is never seen), and are dropped into shared memory when their stage
            // comes up so that the gathering lanes can read four of them at once.
            const int s0 = (int)(((uint32_t)pw + kProducerWarps - (g_stage % kProducerWarps)) % kProducerWarps);
            OwnIter it;
            it.init(l_j0, l_end, cnt);
            it.advance(s0);
            int pq[2], pj[2], pe[2], pidx[2][kStageNnz / 32];   // [0] = the stage being gathered, [1] = the next one
#pragma unroll
            for (int z = 0; z < 2; ++z) {
                pq[z] = it.valid() ? it.q : cnt;
                pj[z] = it.j();
                pe[z] = it.je;
#pragma unroll
                for (int u = 0; u < kStageNnz / 32; ++u) {
                    const int jj = pj[z] + lane + 32 * u;
                    pidx[z][u] = (pq[z] < cnt && jj < pe[z]) ? __ldg(p.col_indices + jj) : 0;
                }
                it.advance(kProducerWarps);
            }

            uint32_t g = g_stage + (uint32_t)s0;
            int n = 0;
            bool ok_run = true;
            while (pq[0] < cnt && ok_run) {
                const uint32_t slot = g % kStages;
                if (g >= (uint32_t)kStages)
                    ok_run = wait_or_abort<kSleepProducer>(bar_empty + 8 * slot, ((g / kStages) - 1u) & 1u, abort_flag);
                if (!ok_run) break;
                int *my_ring = ring + (n & 1) * kStageNnz;
#pragma unroll
                for (int u = 0; u < kStageNnz / 32; ++u) my_ring[lane + 32 * u] = pidx[0][u];
                const int q = pq[0];
                const int b = l_b[q];
                const int n0 = l_n0[q];
                const int j = pj[0];
                const int nnz = min(kStageNnz, max(0, pe[0] - j));
                const int n_mma = max(1, (nnz + 15) >> 4);
                const bool two_halves = (n0 + 64) < p.N;       // N % 128 == 64: the last tile has one half
                const uint32_t bar = bar_full + 8 * slot;
                const uint32_t v_base = base + Smem::kV + slot * kVStageBytes;
                const __half *vals = static_cast<const __half *>(p.values) + (int64_t)b * p.stride_values;
                constexpr bool kBulkValues = (V == 8);   // a value vector is exactly one 16-byte operand row
                if (lane == 0) {
                    uint32_t bytes = (uint32_t)(4 * n_mma * (two_halves ? 2 : 1)) * 512u;
                    if (kBulkValues) bytes += (uint32_t)nnz * 16u;
                    mbar_expect_tx_only(bar, bytes);
                    if (kBulkValues && nnz > 0) tc::bulk_copy_g2s(v_base, vals + (int64_t)j * V, (uint32_t)nnz * 16u, bar);
                }
                __syncwarp();                                  // indices in shared memory, byte count armed
                if (grp < 4 * n_mma && (half == 0 || two_halves)) {
                    const int4 c = *reinterpret_cast<const int4 *>(my_ring + 4 * grp);
                    const int row0 = b * rows_per_batch;
                    const int e = 4 * grp;
                    // rows past the end of the vector-row get an out-of-range coordinate: they arrive as zeros
                    tc::tma_gather4(base + Smem::kA + slot * kAStageBytes + a_off, &map, bar, n0 + 64 * half,
                                    e + 0 < nnz ? row0 + c.x : total_rows, e + 1 < nnz ? row0 + c.y : total_rows,
                                    e + 2 < nnz ? row0 + c.z : total_rows, e + 3 < nnz ? row0 + c.w : total_rows);
                }
                if constexpr (kBulkValues) {
                    // value slots between the row's end and the end of the last MMA must read as zeros
#pragma unroll
                    for (int u = 0; u < kStageNnz / 32; ++u) {
                        const int e = lane + 32 * u;
                        if (e >= nnz && e < 16 * n_mma) *reinterpret_cast<uint4 *>(sm + Smem::kV + slot * kVStageBytes + e * 16) = make_uint4(0, 0, 0, 0);
                    }
                    mbar_arrive(bar);
                } else {
#pragma unroll
                    for (int u = 0; u < kStageNnz / 32; ++u) {
                        const int e = lane + 32 * u;
                        if (e < 16 * n_mma) {
                            const bool ok = e < nnz;
                            tc::cp_async_small<V * 2>(v_base + e * 16, ok ? vals + (int64_t)(j + e) * V : vals,
                                                      ok ? (uint32_t)(V * 2) : 0u);
                        }
                    }
                    cp_async_arrive_noinc(bar);
                }
                // rotate the look-ahead: the next stage moves up, the one after it is located and its indices loaded
                pq[0] = pq[1]; pj[0] = pj[1]; pe[0] = pe[1];
                pq[1] = it.valid() ? it.q : cnt;
                pj[1] = it.j();
                pe[1] = it.je;
#pragma unroll
                for (int u = 0; u < kStageNnz / 32; ++u) {
                    pidx[0][u] = pidx[1][u];
                    const int jj = pj[1] + lane + 32 * u;
                    pidx[1][u] = (pq[1] < cnt && jj < pe[1]) ? __ldg(p.col_indices + jj) : 0;
                }
                it.advance(kProducerWarps);
                g += kProducerWarps;
                ++n;
            }
            tc::cp_async_wait<0>();
        } else if (warp >= kMmaWarp) {
            // =========================== MMA issuers =======================================================
            // Two issuing threads share the work by item parity (a tcgen05.mma costs its issuing thread ~64
            // cycles and a commit ~59, more than the tensor pipe needs for these small MMAs).  Both walk the
            // whole stage sequence.  An mbarrier parity wait is only meaningful for a consumer that knows the
            // slot's previous use has completed, so before waiting on stage g a thread makes sure the OTHER
            // thread has passed every stage of its own up to g - kStages (`mma_done`, a monotone counter).
            if (lane == 0) {
                const uint32_t mine = (uint32_t)(warp - kMmaWarp);
                volatile uint32_t *mma_done = reinterpret_cast<volatile uint32_t *>(sm + Smem::kMmaDone);
                constexpr uint32_t kIdesc = tc::make_idesc_f16(kTileN, 16, 1, 1);
                const uint32_t a_lo0 = tc::smem_desc_lo(base + Smem::kA, kAStageBytes / 2);
                const uint32_t a_hi = tc::smem_desc_hi(1024, (uint32_t)tc::kSwizzle128B);
                const uint32_t b_lo0 = tc::smem_desc_lo(base + Smem::kV, 128);
                const uint32_t b_hi = tc::smem_desc_hi(kVStageBytes / 2, (uint32_t)tc::kSwizzleNone);
                uint32_t g = g_stage;
                uint32_t slot = g_stage % kStages, full_parity = (g_stage / kStages) & 1u;
                uint32_t acc = g_item % kAccSlots, acc_parity = ((g_item / kAccSlots) & 1u) ^ 1u;   // parity of the PREVIOUS use
                bool acc_wait = g_item >= (uint32_t)kAccSlots;
                uint32_t item_parity = g_item & 1u;
                bool ok_run = true;
                int len = l_end[0] - l_j0[0];
                for (int q = 0; q < cnt && ok_run; ++q, item_parity ^= 1u) {
                    int rem = len;
                    if (q + 1 < cnt) len = l_end[q + 1] - l_j0[q + 1];   // next item's length: off the critical path
                    if (item_parity != mine) {   // the other issuer's item: step over its stages and accumulator
                        const uint32_t nst = (uint32_t)stages_of(rem);
                        g += nst;
                        const uint32_t tmp = slot + nst;
                        full_parity ^= (tmp / kStages) & 1u;
                        slot = tmp % kStages;
                        if (++acc == (uint32_t)kAccSlots) { acc = 0; acc_parity ^= 1u; acc_wait = true; }
                        mma_done[mine] = g;   // every stage of mine below g has been waited on (the skipped ones are not mine)
                        continue;
                    }
                    if (acc_wait) ok_run = wait_or_abort<kSleepMma>(bar_acc_empty + 8 * acc, acc_parity, abort_flag);
                    const uint32_t d = tmem_base + acc * kAccCols;
                    uint32_t accumulate = 0;
                    do {
                        if (ok_run && g >= (uint32_t)kStages) {   // bounded wait for the other issuer (see above)
                            const uint32_t need = g - kStages;
                            uint32_t polls = 0;
                            while ((int32_t)(mma_done[mine ^ 1u] - need) <= 0) {
                                if (++polls > (1u << 24) || *abort_flag) { *abort_flag = 1; ok_run = false; break; }
                            }
                        }
                        if (ok_run) ok_run = wait_or_abort<kSleepMma>(bar_full + 8 * slot, full_parity, abort_flag);
                        if (!ok_run) break;
                        mma_done[mine] = g + 1;
                        tc::fence_proxy_async();   // the value vectors were written by cp.async (generic proxy)
                        tc::tc_fence_after_sync();
                        const int n_mma = rem >= kStageNnz ? kMmaPerStage : max(1, (rem + 15) >> 4);
                        const uint32_t a_lo = a_lo0 + slot * (kAStageBytes >> 4), b_lo = b_lo0 + slot * (kVStageBytes >> 4);
                        tc::mma_f16_ss(d, tc::desc64(a_lo, a_hi), tc::desc64(b_lo, b_hi), kIdesc, accumulate);
                        if (n_mma > 1) tc::mma_f16_ss(d, tc::desc64(a_lo + 128, a_hi), tc::desc64(b_lo + 16, b_hi), kIdesc, 1u);
                        if (kMmaPerStage > 2 && n_mma > 2) tc::mma_f16_ss(d, tc::desc64(a_lo + 256, a_hi), tc::desc64(b_lo + 32, b_hi), kIdesc, 1u);
                        if (kMmaPerStage > 3 && n_mma > 3) tc::mma_f16_ss(d, tc::desc64(a_lo + 384, a_hi), tc::desc64(b_lo + 48, b_hi), kIdesc, 1u);
                        tc::mma_commit(bar_empty + 8 * slot);
                        accumulate = 1;
                        rem -= kStageNnz;
                        ++g;
                        if (++slot == (uint32_t)kStages) { slot = 0; full_parity ^= 1u; }
                    } while (rem > 0);
                    if (ok_run) tc::mma_commit(bar_acc_full + 8 * acc);
                    if (++acc == (uint32_t)kAccSlots) { acc = 0; acc_parity ^= 1u; acc_wait = true; }
                }
                mma_done[mine] = g_stage + stages_here;   // nothing of this phase is left for this thread to wait on
            }
        } else if (warp < kEpiWarps) {
            // =========================== epilogue ==========================================================
            const int quarter = warp;                     // warps 0..3: TMEM lanes 32*warp .. +31
            uint8_t *stg = sm + Smem::kStaging + warp * kStagingBytes;
            bool ok_run = true;
            for (int q = 0; q < cnt && ok_run; ++q) {
                const uint32_t ic = g_item + (uint32_t)q;
                const uint32_t acc = ic % kAccSlots;
                // warp-uniform outcome: tcgen05.ld below needs all 32 lanes
                ok_run = __all_sync(0xffffffffu, wait_or_abort<kSleepEpilogue>(bar_acc_full + 8 * acc, (ic / kAccSlots) & 1u, abort_flag));
                if (!ok_run) break;
                tc::tc_fence_after_sync();
                uint32_t r[8];
                tc::tmem_ld_x8(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kAccCols, r);
                tc::tc_fence_before_sync();
                mbar_arrive(bar_acc_empty + 8 * acc);     // the accumulator may be overwritten from here on

                const int row = l_row[q];
                const int col0 = l_n0[q] + quarter * 32;  // first of this warp's 32 columns
                TOut *out = static_cast<TOut *>(p.out) + (int64_t)l_b[q] * p.stride_out + (int64_t)row * V * p.N + col0;
                TOut *tile = reinterpret_cast<TOut *>(stg);   // [V][32]
                __syncwarp();                                  // previous item's reads of the tile are done
#pragma unroll
                for (int v = 0; v < V; ++v) store_scalar(tile + v * 32 + lane, __uint_as_float(r[v]));
                __syncwarp();
                if (col0 < p.N) {
                    constexpr int kChunksPerRow = 32 * (int)sizeof(TOut) / 16;   // 4 (fp16) or 8 (fp32)
                    constexpr int kChunks = V * kChunksPerRow;
#pragma unroll
                    for (int c0 = 0; c0 < kChunks; c0 += 32) {
                        const int c = c0 + lane;
                        if (c < kChunks) {
                            const int v = c / kChunksPerRow, cc = c % kChunksPerRow;
                            const uint4 val = *reinterpret_cast<const uint4 *>(stg + (v * 32 * sizeof(TOut)) + cc * 16);
                            *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(out + (int64_t)v * p.N) + cc * 16) = val;
                        }
                    }
                }
            }
        }

        // ---- phase end: everybody is done with the lists; advance the global counters identically ------------
        g_stage += stages_here;
        g_item += (uint32_t)cnt;
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

}  // namespace tmaspmm
}  // namespace vs
