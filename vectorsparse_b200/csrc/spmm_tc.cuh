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
// Organisation.  Two persistent CTAs per SM, warp-specialised, no CTA-wide barrier inside a phase:
//   * 10 producer warps, each owning ONE slot of the shared-memory ring and therefore every 10th stage (a stage
//     is up to 32 nonzero vectors of one vector-row = one or two K=16 MMAs).  A warp gathers its whole stage:
//     cp.async 16-byte chunks of B rows straight into the 128-byte-swizzled operand layout (zero-filled past
//     the end of a row) and signals the slot's `full` mbarrier with cp.async.mbarrier.arrive, i.e. when the
//     copies have landed.  Ten stages are therefore being gathered concurrently, and the bookkeeping of a stage
//     is paid by one warp, not by all of them.  The column indices of a warp's stage n+2 are fetched while it
//     gathers stage n, so a gather never waits on an index load.
//   * 1 MMA thread: waits for `full` in ring order, issues the MMAs of the stage and commits them to the slot's
//     `empty` mbarrier (slot reuse) and, at the end of a row, to `acc_full`.
//   * 4 epilogue warps: wait for `acc_full`, tcgen05.ld their 32 lanes, release the
//     accumulator (`acc_empty`), transpose through a warp-private staging tile, write C with 16-byte stores.
// Work items are (batch, column tile, vector-row in row_indices order), dealt round-robin to the CTAs so that
// the descending-length order the row swizzle produces becomes a longest-first schedule; each CTA decodes its
// next 128 items in bulk ("phase") so that no role ever chases row_indices -> row_offsets per item.
// Every wait is bounded; a wait that runs out raises the CTA's abort flag, all roles leave through the phase
// barrier, a status bit is set and tensor memory is freed.
#pragma once
#include "common.cuh"
#include "tc_ptx.cuh"

namespace vs {
namespace tcspmm {

constexpr int kProducerWarps = 10;
constexpr int kMmaWarp0 = kProducerWarps;                // warp 10 issues MMAs; warp 11 keeps the epilogue warps'
constexpr int kEpiWarp0 = kMmaWarp0 + 2;                 // index a multiple of four (TMEM lane quarters): 12..15
constexpr int kEpiWarps = 4;
constexpr int kThreads = (kEpiWarp0 + kEpiWarps) * 32;   // 512
constexpr int kCtasPerSm = 2;                            // two CTAs share an SM: two MMA issuers, 20 gather warps
constexpr int kTileN = 128;                              // dense columns per work item (MMA M)
constexpr int kStageNnz = 32;                            // nonzero vectors per stage (one or two K=16 MMAs)
constexpr int kMmaPerStage = kStageNnz / 16;
constexpr int kStages = kProducerWarps;                  // shared-memory ring: one slot per producer warp
constexpr int kAStageBytes = kStageNnz * kTileN * 2;     // 8 KiB
constexpr int kVStageBytes = 2 * kStageNnz * 16;         // 1 KiB: 32 value slots of 16 B, then 512 B of zeros
constexpr int kAccCols = 16;                             // TMEM columns per accumulator
constexpr int kTmemCols = 256;
constexpr int kAccSlots = kTmemCols / kAccCols;          // 16
constexpr int kIdxRing = 3;                              // per-warp ring of index blocks (kStageNnz ints each)
constexpr int kItemsPerPhase = 128;
constexpr int kStagingBytes = 8 * 32 * 4;                // per epilogue warp: 8 rows x 32 columns, fp32 worst case

constexpr uint32_t kStatusTimeout = 1u;  // bit raised in the status word when a bounded wait ran out

struct Smem {  // offsets from the 1024-byte aligned base
    static constexpr int kA = 0;
    static constexpr int kV = kA + kStages * kAStageBytes;
    static constexpr int kRow = kV + kStages * kVStageBytes;
    static constexpr int kJ0 = kRow + kItemsPerPhase * 4;
    static constexpr int kEnd = kJ0 + kItemsPerPhase * 4;
    static constexpr int kItemB = kEnd + kItemsPerPhase * 4;
    static constexpr int kItemN0 = kItemB + kItemsPerPhase * 4;
    static constexpr int kIdx = kItemN0 + kItemsPerPhase * 4;    // [producer warp][ring slot][64]
    static constexpr int kStaging = kIdx + kProducerWarps * kIdxRing * kStageNnz * 4;
    static constexpr int kBarFull = kStaging + kEpiWarps * kStagingBytes;
    static constexpr int kBarEmpty = kBarFull + kStages * 8;
    static constexpr int kBarAccFull = kBarEmpty + kStages * 8;
    static constexpr int kBarAccEmpty = kBarAccFull + kAccSlots * 8;
    static constexpr int kTmemHolder = kBarAccEmpty + kAccSlots * 8;
    static constexpr int kAbort = kTmemHolder + 8;
    static constexpr int kPhaseStages = kAbort + 8;
    static constexpr int kTotal = kPhaseStages + 8;   // two counters, used by alternate phases
};
constexpr int kSmemBytes = Smem::kTotal + 1024;  // + slack for the manual 1024-byte alignment
static_assert(kCtasPerSm * (kSmemBytes + 1024) <= 227 * 1024, "shared memory budget");
static_assert(kStages == kProducerWarps, "each ring slot is owned by one producer warp");

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

// Bounded mbarrier wait that also gives up when another role of the CTA has raised the abort flag.  Between
// polls the warp sleeps kSleepNs, so that the many warps that are waiting at any moment (a role waits most of
// the time in a balanced pipeline) leave the issue slots to the warps that are working.
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
constexpr int kSleepProducer = 200, kSleepMma = 0, kSleepEpilogue = 200;

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrives on `bar` once every cp.async this thread has issued so far has completed (no pending-count bump:
// the barrier's expected count already includes this arrival).
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

template <typename TOut, int V>
__global__ void __launch_bounds__(kThreads, kCtasPerSm) spmm_tc_kernel(const SpmmParams p, uint32_t *status, const int32_t *plan_hdr, int plan_checks) {
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
            tc::mbar_init(bar_full + 8 * s, 32);
            tc::mbar_init(bar_empty + 8 * s, 1);
        }
        for (int s = 0; s < kAccSlots; ++s) {
            tc::mbar_init(bar_acc_full + 8 * s, 1);
            tc::mbar_init(bar_acc_empty + 8 * s, 128);
        }
        *abort_flag = 0;
        phase_stage_count[0] = 0;
        phase_stage_count[1] = 0;
        tc::fence_mbar_init();
    }
    if (warp == kMmaWarp0) {
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

        if (warp < kProducerWarps) {
            // =========================== producers =======================================================
            const int chunk = lane & 15;     // 16-byte chunk of the 256-byte row segment
            const int h = lane >> 4;         // this lane copies rows h + 2*i, i = 0 .. kStageNnz/2 - 1
            uint32_t x[4];                   // row-in-group dependent part of the destination, for i & 3
#pragma unroll
            for (int m = 0; m < 4; ++m)
                x[m] = (uint32_t)((chunk >> 3) * (kAStageBytes / 2) + (h + 2 * m) * 128 + (((chunk & 7) ^ (h + 2 * m)) << 4));
            const uint32_t slot = (uint32_t)warp;
            const uint32_t a_base = base + Smem::kA + slot * kAStageBytes;
            const uint32_t v_base = base + Smem::kV + slot * kVStageBytes;
            int *ring = reinterpret_cast<int *>(sm + Smem::kIdx) + warp * kIdxRing * kStageNnz;
            const uint32_t ring_u32 = base + Smem::kIdx + warp * kIdxRing * kStageNnz * 4;

            // first stage of this phase that lands in this warp's slot
            const int s0 = (int)(((uint32_t)warp + kStages - (g_stage % kStages)) % kStages);
            OwnIter cur, fetch;
            cur.init(l_j0, l_end, cnt);
            cur.advance(s0);
            fetch = cur;
            // indices of this warp's first two stages: plain loads, once per phase
            for (int n = 0; n < 2; ++n) {
                if (fetch.valid()) {
#pragma unroll
                    for (int u = 0; u < kStageNnz / 32; ++u) {
                        const int jj = fetch.j() + lane + 32 * u;
                        ring[n * kStageNnz + lane + 32 * u] = (jj < fetch.je) ? __ldg(p.col_indices + jj) : 0;
                    }
                    fetch.advance(kStages);
                }
            }
            __syncwarp();

            uint32_t g = g_stage + (uint32_t)s0;
            int n = 0;
            bool ok_run = true;
            while (cur.valid() && ok_run) {
                if (g >= (uint32_t)kStages) ok_run = wait_or_abort<kSleepProducer>(bar_empty + 8 * slot, ((g / kStages) - 1u) & 1u, abort_flag);
                if (!ok_run) break;
                // this stage's indices were fetched two of this warp's stages ago: at most the newest cp.async
                // group may still be pending; the warp barrier publishes the landed indices to all lanes
                tc::cp_async_wait<1>();
                __syncwarp();
                const int q = cur.q;
                const int b = l_b[q];
                const int n0 = l_n0[q];
                const int j = cur.j();
                const int nnz = cur.nnz();
                const int n_mma = max(1, (nnz + 15) >> 4);
                const __half *rhs = static_cast<const __half *>(p.rhs) + (int64_t)b * p.stride_rhs;
                const __half *rhs_t = rhs + n0 + chunk * 8;
                const bool col_ok = (n0 + chunk * 8) < p.N;
                const int *idx = ring + (n % kIdxRing) * kStageNnz + h;
#pragma unroll
                for (int i = 0; i < kStageNnz / 2; ++i) {
                    if (i < 8 * n_mma) {   // rows h + 2i of MMA (i >> 3)
                        const bool ok = col_ok && (h + 2 * i) < nnz;
                        const __half *src = ok ? rhs_t + (int64_t)idx[2 * i] * p.N : rhs;
                        tc::cp_async_16(a_base + x[i & 3] + (i >> 2) * 1024, src, ok ? 16u : 0u);
                    }
                }
                const __half *vals = static_cast<const __half *>(p.values) + (int64_t)b * p.stride_values;
#pragma unroll
                for (int u = 0; u < kStageNnz / 32; ++u) {
                    const int e = lane + 32 * u;
                    if (e < 16 * n_mma) {
                        const bool ok = e < nnz;
                        tc::cp_async_small<V * 2>(v_base + e * 16, ok ? vals + (int64_t)(j + e) * V : vals,
                                                  ok ? (uint32_t)(V * 2) : 0u);
                    }
                }
                // column indices of this warp's stage n + 2
                if (fetch.valid()) {
#pragma unroll
                    for (int u = 0; u < kStageNnz / 32; ++u) {
                        const int jj = fetch.j() + lane + 32 * u;
                        const bool ok = jj < fetch.je;
                        tc::cp_async_small<4>(ring_u32 + (((n + 2) % kIdxRing) * kStageNnz + lane + 32 * u) * 4,
                                              ok ? p.col_indices + jj : p.col_indices, ok ? 4u : 0u);
                    }
                    fetch.advance(kStages);
                }
                cp_async_arrive_noinc(bar_full + 8 * slot);
                tc::cp_async_commit();
                cur.advance(kStages);
                g += kStages;
                ++n;
            }
            tc::cp_async_wait<0>();
        } else if (warp < kEpiWarp0) {
            // =========================== MMA issuers (even / odd items) ====================================
            // One issuing thread for all stages, in ring order: an mbarrier parity wait is only safe for a
            // consumer that has itself seen the slot's previous use complete.
            if (lane == 0 && warp == kMmaWarp0) {
                constexpr uint32_t kIdesc = tc::make_idesc_f16(kTileN, 16, 1, 1);
                const uint32_t a_lo0 = tc::smem_desc_lo(base + Smem::kA, kAStageBytes / 2);
                const uint32_t a_hi = tc::smem_desc_hi(1024, (uint32_t)tc::kSwizzle128B);
                const uint32_t b_lo0 = tc::smem_desc_lo(base + Smem::kV, 128);
                const uint32_t b_hi = tc::smem_desc_hi(kVStageBytes / 2, (uint32_t)tc::kSwizzleNone);
                uint32_t g = g_stage, ic = g_item;
                bool ok_run = true;
                for (int q = 0; q < cnt && ok_run; ++q, ++ic) {
                    int rem = l_end[q] - l_j0[q];
                    const uint32_t acc = ic % kAccSlots;
                    if (ic >= (uint32_t)kAccSlots)
                        ok_run = wait_or_abort<kSleepMma>(bar_acc_empty + 8 * acc, ((ic / kAccSlots) - 1u) & 1u, abort_flag);
                    const uint32_t d = tmem_base + acc * kAccCols;
                    uint32_t accumulate = 0;
                    do {
                        const uint32_t slot = g % kStages;
                        if (ok_run) ok_run = wait_or_abort<kSleepMma>(bar_full + 8 * slot, (g / kStages) & 1u, abort_flag);
                        if (!ok_run) break;
                        tc::fence_proxy_async();
                        tc::tc_fence_after_sync();
                        const int n_mma = rem >= kStageNnz ? kMmaPerStage : max(1, (rem + 15) >> 4);
                        const uint32_t a_lo = a_lo0 + slot * (kAStageBytes >> 4);
                        const uint32_t b_lo = b_lo0 + slot * (kVStageBytes >> 4);
                        tc::mma_f16_ss(d, tc::desc64(a_lo, a_hi), tc::desc64(b_lo, b_hi), kIdesc, accumulate);
                        {
                        if (n_mma > 1) tc::mma_f16_ss(d, tc::desc64(a_lo + 128, a_hi), tc::desc64(b_lo + 16, b_hi), kIdesc, 1u);
                        if (kMmaPerStage > 2 && n_mma > 2) tc::mma_f16_ss(d, tc::desc64(a_lo + 256, a_hi), tc::desc64(b_lo + 32, b_hi), kIdesc, 1u);
                        if (kMmaPerStage > 3 && n_mma > 3) tc::mma_f16_ss(d, tc::desc64(a_lo + 384, a_hi), tc::desc64(b_lo + 48, b_hi), kIdesc, 1u);
                        }
                        tc::mma_commit(bar_empty + 8 * slot);
                        accumulate = 1;
                        rem -= kStageNnz;
                        ++g;
                    } while (rem > 0);
                    if (ok_run) tc::mma_commit(bar_acc_full + 8 * acc);
                }
            }
        } else {
            // =========================== epilogue (even / odd items) ========================================
            const int quarter = warp & 3;                 // TMEM lanes 32*quarter .. +31
            const int ew = warp - kEpiWarp0;              // 0..3
            uint8_t *stg = sm + Smem::kStaging + ew * kStagingBytes;
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
    if (warp == kMmaWarp0) tc::tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace tcspmm
}  // namespace vs
