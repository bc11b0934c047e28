// Tensor-core SDDMM for fp16 operands on sm_100a by multiplying dense tiles and sampling them at the mask: the
// `wmmaSddmm` entry point of the reference (src/wmma_sddmm.cu:3175-3202) for masks that are not extremely sparse
// and contraction lengths of 128 and more.
//
// Why.  The gather kernel next to this file fetches one row of rhs per mask entry (~60 TMA gathers and 16 tiny
// MMAs per vector-row and 256 contraction elements) and is bound by issuing them.  The dense product
//     D[256 rows of lhs x 128 rows of rhs] += lhs[256 x 64] . rhs[128 x 64]^T          per 64 contraction elements
// does 10x the flops at 90 % sparsity with plain TMA tile loads (both operands are already K-major in memory:
// no gather, nothing to build) and 128 x 128 x 16 MMAs; the epilogue keeps only the entries the mask names.
// Nothing outside the mask is ever stored, so non-finite products elsewhere in the tile cannot leak.
//
// Plan.  A small kernel buckets each vector-row's mask entries by 32-column chunk: `chunk_offsets`
// [vector-rows][chunks + 1] and `chunk_entries` (entry index j, column), in any order inside
// a chunk.  It depends on the structure only and is shared by every matrix of a batch.
//
// Organisation: one persistent CTA per SM, work items (batch, 256-row tile of lhs, 128-row tile of rhs).
//   warps 0-7   epilogue: warp (quarter, half) owns 32 rows of the tile.  Per 32 columns: TMEM -> registers ->
//               its row of a swizzled 32 x 32 box of shared memory (already in the output type), then every lane walks the
//               entries of ITS vector-row in that chunk and stores lhs-row x entry values; the V lanes of a
//               vector-row write V consecutive outputs.  The bounds of its entries are loaded one item ahead,
//               the first eight entries of a chunk one chunk ahead, further entries eight at a time.
//   warp 8      one thread issuing the loads: 32 KiB of lhs and 16 KiB of rhs per stage, four stages in a ring
//   warps 9-10  one MMA-issuing thread per 128-row half of the tile
// Accumulators: 2 halves x 128 columns, double buffered (all 512 TMEM columns).  Every wait is bounded; a wait
// that runs out raises the CTA's abort flag, all roles fall through to the end, a status bit is set and tensor
// memory is freed.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace vs {
namespace densesddmm {

constexpr int kTileM = 256;                              // rows of lhs per work item: two MMA operands of 128 rows
constexpr int kTileN = 128;                              // rows of rhs (columns of the mask) per work item (MMA N)
constexpr int kBlockK = 64;                              // contraction elements per stage
constexpr int kChunk = 32;                               // mask columns per plan bucket and per epilogue step
constexpr int kStages = 4;
constexpr int kEpiWarps = 8;                             // warps 0..7: TMEM lane quarter = warp % 4, half of the tile = warp / 4
constexpr int kLoadWarp = kEpiWarps;                     // 8
constexpr int kMmaWarp = kLoadWarp + 1;                  // 9, 10
constexpr int kHalves = kTileM / 128;
constexpr int kThreads = (kMmaWarp + kHalves) * 32;      // 352
constexpr int kAStageBytes = kTileM * kBlockK * 2;       // 32 KiB
constexpr int kBStageBytes = kTileN * kBlockK * 2;       // 16 KiB
constexpr int kAccCols = kHalves * kTileN;               // 256 TMEM columns per accumulator buffer
constexpr int kTmemCols = 2 * kAccCols;                  // 512
constexpr int kBoxBytes = 32 * kChunk * 4;               // 4 KiB per epilogue warp: 32 rows x 32 columns, fp32 at most
constexpr int kAhead = 8;                                // entries of a chunk a lane loads one chunk ahead
constexpr int kPlanThreads = 128;

constexpr uint32_t kStatusTimeout = 128u;  // bit raised in the status word when a bounded wait ran out

struct Smem {  // offsets from the 1024-byte aligned base
    static constexpr int kA = 0;
    static constexpr int kB = kA + kStages * kAStageBytes;
    static constexpr int kStaging = kB + kStages * kBStageBytes;
    static constexpr int kBarFull = kStaging + kEpiWarps * kBoxBytes;
    static constexpr int kBarEmpty = kBarFull + kStages * 8;
    static constexpr int kBarAccFull = kBarEmpty + kStages * 8;
    static constexpr int kBarAccEmpty = kBarAccFull + 2 * 8;
    static constexpr int kTmemHolder = kBarAccEmpty + 2 * 8;
    static constexpr int kAbort = kTmemHolder + 8;
    static constexpr int kTotal = kAbort + 8;
};
constexpr int kSmemBytes = Smem::kTotal + 1024;  // + slack for the manual 1024-byte alignment
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");

// ---- plan -------------------------------------------------------------------------------------------------
// One CTA per vector-row.  chunk_offsets[i * (chunks + 1) + c] .. [.. + c + 1] delimit, inside chunk_entries, the
// mask entries of vector-row i whose column lies in [32 c, 32 c + 32); an entry is (j, column).  Columns
// outside [0, n) are dropped: their outputs are not written (the gather kernels write zeros there; the host
// entry points reject such structures where they can see them).
__global__ void __launch_bounds__(kPlanThreads)
sddmm_plan_kernel(const int32_t *__restrict__ row_offsets, const int32_t *__restrict__ col_indices, int n, int chunks, int nnz_vec,
                  int32_t *__restrict__ chunk_offsets, uint2 *__restrict__ chunk_entries) {
    extern __shared__ int plan_sh[];
    pdl_launch_dependents();   // the multiplying kernel may set itself up while the plan is made
    int *hist = plan_sh;             // [chunks]
    int *cursor = plan_sh + chunks;  // [chunks]
    const int i = blockIdx.x, t = threadIdx.x;
    // the scratch holds nnz_vec entries (the caller's count): offsets that claim more are cut there, so that a
    // count smaller than row_offsets[m_vec] leaves outputs unwritten instead of writing past the scratch
    const int j0 = min(max(__ldg(row_offsets + i), 0), nnz_vec), j1 = min(max(__ldg(row_offsets + i + 1), j0), nnz_vec);
    for (int c = t; c < chunks; c += kPlanThreads) hist[c] = 0;
    __syncthreads();
    for (int j = j0 + t; j < j1; j += kPlanThreads) {
        const int c = __ldg(col_indices + j);
        if ((unsigned)c < (unsigned)n) atomicAdd(hist + c / kChunk, 1);
    }
    __syncthreads();
    if (t == 0) {
        int run = j0;
        int32_t *o = chunk_offsets + (int64_t)i * (chunks + 1);
        for (int c = 0; c < chunks; ++c) {
            cursor[c] = run;
            o[c] = run;
            run += hist[c];
        }
        o[chunks] = run;
    }
    __syncthreads();
    for (int j = j0 + t; j < j1; j += kPlanThreads) {
        const int c = __ldg(col_indices + j);
        if ((unsigned)c >= (unsigned)n) continue;
        const int pos = atomicAdd(cursor + c / kChunk, 1);
        chunk_entries[pos] = make_uint2((uint32_t)j, (uint32_t)c);
    }
}

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
constexpr int kSleepLoad = 32, kSleepMma = 0, kSleepEpilogue = 32;

// The work items of this CTA one after the other (blockIdx.x, + gridDim.x, ...): (batch entry, row tile, column
// tile) with the column tile running fastest, advanced with carries instead of divisions.
struct ItemIter {
    int b, mt, nt;
    int d_nt, d_mt, d_b, m_tiles, n_tiles;
    __device__ __forceinline__ void init(int m_tiles_, int n_tiles_) {
        m_tiles = m_tiles_; n_tiles = n_tiles_;
        const uint32_t G = gridDim.x;
        d_nt = (int)(G % (uint32_t)n_tiles);
        const uint32_t r = G / (uint32_t)n_tiles;
        d_mt = (int)(r % (uint32_t)m_tiles);
        d_b = (int)(r / (uint32_t)m_tiles);
        const uint32_t w = blockIdx.x;
        nt = (int)(w % (uint32_t)n_tiles);
        const uint32_t rr = w / (uint32_t)n_tiles;
        mt = (int)(rr % (uint32_t)m_tiles);
        b = (int)(rr / (uint32_t)m_tiles);
    }
    __device__ __forceinline__ void next() {
        nt += d_nt; mt += d_mt; b += d_b;
        if (nt >= n_tiles) { nt -= n_tiles; ++mt; }
        if (mt >= m_tiles) { mt -= m_tiles; ++b; }
    }
};

// map_lhs: {k, rows of lhs, batch}, box {64, 256, 1}; map_rhs: {k, n, batch}, box {64, 128, 1}; both with the
// 128-byte swizzle and zero fill outside.
template <typename TOut, int V>
__global__ void __launch_bounds__(kThreads, 1)
sddmm_dense_kernel(const SddmmParams p, const __grid_constant__ CUtensorMap map_lhs, const __grid_constant__ CUtensorMap map_rhs,
                   const int32_t *__restrict__ chunk_offsets, const uint2 *__restrict__ chunk_entries, int m_tiles, int n_tiles,
                   int chunks, uint32_t *status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = tc::smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t *sm = smem_raw + (base - raw);

    const int t = threadIdx.x;
    const int warp = t >> 5;
    const int lane = t & 31;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(sm + Smem::kAbort);
    const uint32_t bar_full = base + Smem::kBarFull;
    const uint32_t bar_empty = base + Smem::kBarEmpty;
    const uint32_t bar_acc_full = base + Smem::kBarAccFull;
    const uint32_t bar_acc_empty = base + Smem::kBarAccEmpty;

    if (t == 0) {
        for (int s = 0; s < kStages; ++s) {
            tc::mbar_init(bar_full + 8 * s, 1);         // the loader's arrival (+ the bytes of both operands)
            tc::mbar_init(bar_empty + 8 * s, kHalves);  // one commit per MMA-issuing thread
        }
        for (int s = 0; s < 2; ++s) {
            tc::mbar_init(bar_acc_full + 8 * s, kHalves);
            tc::mbar_init(bar_acc_empty + 8 * s, kEpiWarps * 32);
        }
        *abort_flag = 0;
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

    pdl_wait();   // the set-up above may have run beside the plan kernel; its buckets are read from here on
    const int k_blocks = p.k / kBlockK;
    const int64_t total_items = (int64_t)p.batch * m_tiles * n_tiles;
    const int64_t G = gridDim.x;
    const uint32_t my_items = (total_items > blockIdx.x) ? (uint32_t)((total_items - blockIdx.x + G - 1) / G) : 0u;

    if (warp == kLoadWarp) {
        // =========================== loader ==============================================================
        if (lane == 0) {
            ItemIter it;
            it.init(m_tiles, n_tiles);
            uint32_t slot = 0, use = 0;
            bool ok_run = true;
            for (uint32_t i = 0; i < my_items && ok_run; ++i, it.next()) {
                for (int kb = 0; kb < k_blocks && ok_run; ++kb) {
                    if (use > 0) ok_run = wait_or_abort<kSleepLoad>(bar_empty + 8 * slot, (use - 1u) & 1u, abort_flag);
                    if (!ok_run) break;
                    const uint32_t bar = bar_full + 8 * slot;
                    tc::mbar_expect_tx(bar, (uint32_t)(kAStageBytes + kBStageBytes));   // arrives and arms the byte count
                    tc::tma_load_3d(base + Smem::kA + slot * kAStageBytes, &map_lhs, bar, kb * kBlockK, it.mt * kTileM, it.b);
                    tc::tma_load_3d(base + Smem::kB + slot * kBStageBytes, &map_rhs, bar, kb * kBlockK, it.nt * kTileN, it.b);
                    if (++slot == (uint32_t)kStages) { slot = 0; ++use; }
                }
            }
        }
    } else if (warp >= kMmaWarp) {
        // =========================== MMA issuers =========================================================
        // Thread h multiplies rows 128 h .. 128 h + 127 of the tile.  Both wait on every stage and both commit
        // to its `empty` barrier, so each has seen every earlier use of a slot complete.
        if (lane == 0) {
            const int h = warp - kMmaWarp;
            const uint32_t a_lo0 = tc::smem_desc_lo(base + Smem::kA + h * (128 * kBlockK * 2), 16);
            const uint32_t b_lo0 = tc::smem_desc_lo(base + Smem::kB, 16);
            const uint32_t hi = tc::smem_desc_hi(1024, (uint32_t)tc::kSwizzle128B);   // K-major: 8-row groups 1 KiB apart
            ItemIter it;
            it.init(m_tiles, n_tiles);
            uint32_t slot = 0, parity = 0;
            bool ok_run = true, ready = false;
            for (uint32_t i = 0; i < my_items && ok_run; ++i, it.next()) {
                const int tn = min(kTileN, (p.n - it.nt * kTileN + 15) & ~15);
                const uint32_t idesc = tc::make_idesc_f16(128, tn, 0, 0);   // both operands K-major
                const uint32_t buf = i & 1u;
                if (i >= 2) ok_run = wait_or_abort<kSleepMma>(bar_acc_empty + 8 * buf, ((i >> 1) - 1u) & 1u, abort_flag);
                tc::tc_fence_after_sync();
                const uint32_t d = tmem_base + buf * kAccCols + (uint32_t)h * kTileN;
                for (int kb = 0; kb < k_blocks && ok_run; ++kb) {
                    if (!ready) ok_run = wait_or_abort<kSleepMma>(bar_full + 8 * slot, parity, abort_flag);
                    if (!ok_run) break;
                    tc::tc_fence_after_sync();
                    const uint32_t a_lo = a_lo0 + slot * (kAStageBytes >> 4), b_lo = b_lo0 + slot * (kBStageBytes >> 4);
#pragma unroll
                    for (int kk = 0; kk < kBlockK / 16; ++kk)   // 16 contraction elements = 32 bytes along a row
                        tc::mma_f16_ss(d, tc::desc64(a_lo + 2 * kk, hi), tc::desc64(b_lo + 2 * kk, hi), idesc,
                                       (kb > 0 || kk > 0) ? 1u : 0u);
                    tc::mma_commit(bar_empty + 8 * slot);
                    if (++slot == (uint32_t)kStages) { slot = 0; parity ^= 1u; }
                    // one look at the next stage's barrier while the MMAs above are handed to the pipe
                    ready = (kb + 1 < k_blocks || i + 1 < my_items) && tc::mbar_try_wait(bar_full + 8 * slot, parity);
                }
                if (ok_run) tc::mma_commit(bar_acc_full + 8 * buf);
            }
        }
    } else {
        // =========================== epilogue ============================================================
        const int quarter = warp & 3, half = warp >> 2;   // TMEM lanes 32 quarter ..; rows 128 half .. of the tile
        uint8_t *stg = sm + Smem::kStaging + warp * kBoxBytes;
        const uint32_t lane_taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * kTileN);
        // This lane's row of the box holds its 32 accumulator columns already in the output type (64 or 128
        // bytes); the 16-byte chunks of a row are XOR-swizzled with address bits 7.. so that the row-per-lane
        // stores spread over the banks.
        constexpr int kElem = (int)sizeof(TOut);
        constexpr int kRowBytes = kChunk * kElem;
        constexpr int kPerChunk = 16 / kElem;
        const uint32_t swz = kRowBytes == 128 ? (uint32_t)(lane & 7) : (uint32_t)((lane >> 1) & 3);
        uint8_t *my_row = stg + lane * kRowBytes;
        auto box_write = [&](const uint32_t (&r)[kChunk]) {
#pragma unroll
            for (int u = 0; u < kRowBytes / 16; ++u) {
                uint4 v;
                if constexpr (kElem == 2) {
                    __half2 *hh = reinterpret_cast<__half2 *>(&v);
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        hh[e] = __floats2half2_rn(__uint_as_float(r[8 * u + 2 * e]), __uint_as_float(r[8 * u + 2 * e + 1]));
                } else {
                    v = make_uint4(r[4 * u], r[4 * u + 1], r[4 * u + 2], r[4 * u + 3]);
                }
                *reinterpret_cast<uint4 *>(my_row + (((uint32_t)u ^ swz) << 4)) = v;
            }
        };
        auto box_read = [&](uint32_t cl) -> TOut {
            return *reinterpret_cast<const TOut *>(my_row + (((cl / kPerChunk) ^ swz) << 4) + (cl % kPerChunk) * kElem);
        };
        constexpr int kChunksPerTile = kTileN / kChunk;    // 4
        // What a lane has to know ahead of time: the bounds of its vector-row's entries in the tile's four chunks
        // (loaded one ITEM ahead) and the first kAhead entries of the next chunk it will sample (loaded one CHUNK
        // ahead): the two dependent global loads never sit between the accumulator and the stores.
        auto load_bounds = [&](const ItemIter &w, bool valid, int (&off)[kChunksPerTile + 1]) {
            const int iv = (w.mt * kTileM + half * 128 + quarter * 32 + lane) / V;
            const int c0 = (w.nt * kTileN) / kChunk;
            const bool live = valid && iv < p.m_vec;
            const int32_t *o = chunk_offsets + (int64_t)(live ? iv : 0) * (chunks + 1) + c0;
#pragma unroll
            for (int c = 0; c <= kChunksPerTile; ++c) off[c] = (live && c0 + c <= chunks) ? __ldg(o + c) : 0;
#pragma unroll
            for (int c = 0; c < kChunksPerTile; ++c)
                if (!(live && c0 + c < chunks)) off[c + 1] = off[c];   // no such chunk: empty range
        };
        auto load_entries = [&](int lo, int hi, uint2 (&e)[kAhead]) {
#pragma unroll
            for (int a = 0; a < kAhead; ++a) e[a] = lo + a < hi ? __ldg(chunk_entries + lo + a) : make_uint2(0u, 0u);
        };
        ItemIter it;
        it.init(m_tiles, n_tiles);
        int off[kChunksPerTile + 1], off_next[kChunksPerTile + 1];
        uint2 ent[kAhead];
        load_bounds(it, my_items > 0, off);
        load_entries(off[0], off[1], ent);
        bool ok_run = true;
        for (uint32_t i = 0; i < my_items && ok_run; ++i) {
            const uint32_t buf = i & 1u;
            const int v = (it.mt * kTileM + half * 128 + quarter * 32 + lane) % V;   // this lane's place in its vector-row
            const int tn = min(kTileN, (p.n - it.nt * kTileN + 15) & ~15);
            TOut *out = static_cast<TOut *>(p.out) + (int64_t)it.b * p.stride_out + v;
            it.next();
            load_bounds(it, i + 1 < my_items, off_next);
            // warp-uniform outcome: tcgen05.ld below needs all 32 lanes
            ok_run = __all_sync(0xffffffffu, wait_or_abort<kSleepEpilogue>(bar_acc_full + 8 * buf, (i >> 1) & 1u, abort_flag));
            if (!ok_run) break;
            tc::tc_fence_after_sync();
#pragma unroll
            for (int c = 0; c < kChunksPerTile; ++c) {
                uint2 ent_next[kAhead];   // the chunk after this one: same item, or the first of the next item
                if (c + 1 < kChunksPerTile) load_entries(off[c + 1], off[c + 2], ent_next);
                else load_entries(off_next[0], off_next[1], ent_next);
                if (c * kChunk < tn) {   // warp-uniform
                    uint32_t r[kChunk];
                    __syncwarp();        // together again for the aligned load
                    tc::tmem_ld_x32(lane_taddr + buf * kAccCols + (uint32_t)(c * kChunk), r);
                    if ((c + 1) * kChunk >= tn) {   // the last column this warp needs is in registers
                        tc::tc_fence_before_sync();
                        tc::mbar_arrive(bar_acc_empty + 8 * buf);
                    }
                    // The lane's 32 columns go to its row of the box and come back one entry at a time (no
                    // dynamic register indexing); no lane reads another lane's row, so nothing is synchronised.
                    box_write(r);
#pragma unroll
                    for (int a = 0; a < kAhead; ++a) {
                        if (off[c] + a < off[c + 1]) {
                            out[(int64_t)ent[a].x * V] = box_read(ent[a].y % kChunk);
                        }
                    }
                    // denser rows: the remaining entries eight at a time, so that their loads overlap
                    for (int e = off[c] + kAhead; e < off[c + 1]; e += 8) {
                        uint2 en[8];
#pragma unroll
                        for (int u = 0; u < 8; ++u) en[u] = e + u < off[c + 1] ? __ldg(chunk_entries + e + u) : make_uint2(0u, 0u);
#pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            if (e + u < off[c + 1]) {
                                out[(int64_t)en[u].x * V] = box_read(en[u].y % kChunk);
                            }
                        }
                    }
                }
#pragma unroll
                for (int a = 0; a < kAhead; ++a) ent[a] = ent_next[a];
            }
#pragma unroll
            for (int c = 0; c <= kChunksPerTile; ++c) off[c] = off_next[c];
        }
    }

    // ---- teardown ---------------------------------------------------------------------------------------
    tc::tc_fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        // a bounded wait ran out: give copies that may still be in flight time to land before the CTA ends
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
        if (t == 0) atomicOr(status, kStatusTimeout);
        __syncthreads();
    }
    if (warp == kMmaWarp) tc::tmem_dealloc(tmem_base, kTmemCols);
}

}  // namespace densesddmm
}  // namespace vs
