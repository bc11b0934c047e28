// Tensor-core SpMM for fp16 operands on sm_100a by densifying tiles of the sparse matrix in shared memory: the
// `wmmaSpmm` entry point of the reference (src/wmma_spmm.cu:388-409) for matrices that are not extremely sparse.
//
// Why.  The reference (and the gather kernels next to this file) fetch one row of the dense operand per
// nonzero vector, because on Volta the tensor cores were the scarce resource.  On B200 they are not: a 128 x 128
// x 16 MMA takes ~65 cycles, while gathering the rows a vector-row needs costs hundreds of cycles of TMA / LSU
// issue.  Up to ~97 % sparsity it is cheaper to multiply a zero-filled dense tile of A:
//     C[256 rows x 128 cols] += A_dense[256 x 64] * B[64 x 128]          per 64-wide block of A's columns.
// A_dense is built in shared memory from the CVSE arrays (one store per nonzero vector into a tile of zeros,
// and one to take it out again afterwards: the operand is kept MN-major, rows contiguous, in the
// 128-byte-swizzled layout the MMA reads); B arrives by plain TMA tile loads (two 8 KiB boxes per
// stage, no gather); the products with the zeros are free.  The result is the same sum in another order, except
// when B holds Inf / NaN in rows no nonzero names (0 x Inf = NaN): the epilogue therefore watches for
// non-finite sums and, if it sees one, clears the flag that keeps the gather kernel behind it from running.
//
// Plan.  A small kernel first buckets the nonzero vectors by (128-row group, 16-column block): `blk_offsets`
// [row groups][column blocks + 1] and `blk_entries` (vector index, vector-row within the group, column within
// the block).  The plan depends on the structure only and is shared by every matrix of a batch.
//
// Organisation: one persistent CTA per SM.  Work items are (batch, 128-column tile of B, 256-row tile of A),
// consecutive CTAs taking consecutive row tiles of the same B so that it stays in L2.  A stage is one 64-wide
// block of A's columns: 32 KiB of A (two 128-row MMA operands) + 16 KiB of B, four of each in a ring.
//   warps 0-7    epilogue: TMEM -> registers -> swizzled shared-memory boxes -> TMA stores of whole rows
//   warps 8-23   fill: four warps per A slot, one per 128 rows x 32 columns (two plan buckets) of the stage
//   warp 24      one thread issuing the B loads, up to four stages ahead
//   warp 25      L2 prefetch of the next item's part of B
//   warps 26-27  one MMA-issuing thread per 128-row half of the tile
// Accumulators: 2 halves x 128 columns, double buffered (all 512 TMEM columns), so the epilogue of one item
// overlaps the MMAs of the next.  Every wait is bounded; a wait that runs out raises the CTA's abort flag, all
// roles fall through to the end, a status bit is set and tensor memory is freed.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace vs {
namespace densespmm {

constexpr int kTileM = 256;                              // rows of A per work item: two MMA operands of 128 rows
constexpr int kTileN = 128;                              // columns of B per work item (MMA N)
constexpr int kBlockK = 64;                              // columns of A (rows of B) per stage
constexpr int kGroupRows = 128;                          // rows per plan bucket: one MMA operand
constexpr int kPlanCols = 16;                            // columns per plan bucket: a quarter of a stage
constexpr int kFillCols = 32;                            // columns one fill warp of this kernel owns: two neighbouring buckets
constexpr int kAStages = 4;                              // ring of densified A tiles
constexpr int kBStages = 4;                              // ring of B tiles: deeper, their loads have the latency to hide
constexpr int kEpiWarps = 8;                             // warps 0..7: TMEM lane quarter = warp % 4, half of the tile = warp / 4
constexpr int kFillWarp0 = kEpiWarps;
constexpr int kFillPerSlot = (kTileM / kGroupRows) * (kBlockK / kFillCols);   // 4: one warp per 128 rows x 32 columns of a stage
constexpr int kFillWarps = kAStages * kFillPerSlot;      // 16: warp f fills A slot f % kAStages, bucket f / kAStages
constexpr int kFillBatches = 2;                          // entries a fill warp keeps in flight: 2 x 32
constexpr int kOverflowBatches = 4;                      // batches of 32 loaded together beyond those
constexpr int kLoadWarp = kFillWarp0 + kFillWarps;       // 24: one thread issues the B loads
constexpr int kPrefetchWarp = kLoadWarp + 1;             // 25: asks the next item's rows of B into L2
constexpr int kMmaWarp = kPrefetchWarp + 1;              // 26, 27
constexpr int kHalves = kTileM / 128;                    // 2 MMA operands of 128 rows
#ifndef VS_DENSE_KSPLIT
#define VS_DENSE_KSPLIT 1
#endif
constexpr int kKSplit = VS_DENSE_KSPLIT;                               // issuing threads per half (each takes 4 / kKSplit K steps of a stage)
constexpr int kMmaWarps = kKSplit * kHalves;
constexpr bool kZeroedAcc = kKSplit > 1;                 // accumulators handed back zeroed: MMA order free between threads
constexpr int kThreads = (kMmaWarp + kMmaWarps) * 32;    // 896
constexpr int kAStageBytes = kTileM * kBlockK * 2;       // 32 KiB
constexpr int kBSlabBytes = kBlockK * 64 * 2;            // 8 KiB: 64 rows of B x 64 columns
constexpr int kBStageBytes = (kTileN / 64) * kBSlabBytes;  // 16 KiB
constexpr int kAccCols = kHalves * kTileN;               // 256 TMEM columns per accumulator buffer
constexpr int kTmemCols = 2 * kAccCols;                  // 512
constexpr int kStoreCols = 32;                           // output box of one epilogue warp: 32 rows x 32 columns
constexpr int kStoreBoxBytes = 32 * 128;                 // staging per epilogue warp: two fp16 boxes or one fp32 box
constexpr int kPlanThreads = 1024;
constexpr int kPlanWarps = kPlanThreads / 32;
constexpr int kMaxCheckCtas = 256;                       // CTAs of the plan kernel that look for repeated columns

constexpr uint32_t kStatusTimeout = 64u;  // bit raised in the status word when a bounded wait ran out

struct Smem {  // offsets from the 1024-byte aligned base
    static constexpr int kA = 0;
    static constexpr int kB = kA + kAStages * kAStageBytes;
    static constexpr int kStaging = kB + kBStages * kBStageBytes;   // per epilogue warp: one 32-row x 128-byte box
    static constexpr int kBarFull = kStaging + kEpiWarps * kStoreBoxBytes;   // one pair of barriers per B slot
    static constexpr int kBarEmpty = kBarFull + kBStages * 8;
    static constexpr int kBarAccFull = kBarEmpty + kBStages * 8;
    static constexpr int kBarAccEmpty = kBarAccFull + 2 * 8;
    static constexpr int kTmemHolder = kBarAccEmpty + 2 * 8;
    static constexpr int kAbort = kTmemHolder + 8;
    static constexpr int kLoaderProgress = kAbort + 8;      // stages whose B loads have been issued
    static constexpr int kTotal = kLoaderProgress + 8;
};
constexpr int kSmemBytes = Smem::kTotal + 1024;  // + slack for the manual 1024-byte alignment
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
static_assert(kFillWarps % kAStages == 0, "each ring slot needs fixed owner warps");
static_assert(kBStages == kAStages || kBStages == 2 * kAStages,
              "the stage barriers are shared: a fill warp must see every phase of the barriers it waits on");

// ---- plan -------------------------------------------------------------------------------------------------
// CTAs 0 .. groups-1: one per 128-row group (128 / V vector-rows, whose nonzero vectors are contiguous in the
// CVSE arrays).  blk_offsets[g * (plan_blocks + 1) + c] .. [.. + c + 1] delimit the entries of group g in the
// 16-column block c; entry = (vector index j, (vector-row within the group << 6) | column within the 64-column
// stage).  Columns outside [0, K) are dropped (the gather kernels read zeros for them).
//
// CTAs groups .. gridDim.x-1 look for a column that appears twice in one vector-row (the reference's generator
// pads rows that way, include/bm_test_utils.h:110-124): a dense tile has one place per (row, column), the
// reference's kernels add both values, so such a matrix must go to the gather kernel.  A warp takes a vector-row
// at a time and marks its columns in a bitmap of its own in shared memory; each of these CTAs writes its verdict
// to its own word behind *use_dense (use_dense[4 + i]), so nothing has to be cleared between calls.
//
// The kernel also takes the decision between the densifying and the gather kernels, because the number of
// nonzero vectors is only known here.  Costs in cycles of one SM per 128 columns of B, fitted to measurements
// (2048 x 512, V = 2/4/8, 90-99 % sparse): the dense kernel ~1100 per stage (256 rows x 64 columns of A) whatever
// they hold; the gather kernel ~370 per vector-row plus ~4.7 per nonzero vector.  Dense when cheaper (or forced)
// and the entries fit the scratch (`entry_capacity`).  Every CTA computes the same answer; CTA 0 publishes it
// in *use_dense for the two kernels enqueued behind this one, and nothing is planned when the answer is no.
//
// kTransposed: the plan of A^T for vs_spmm_t, read from the transposed structure of a CVSE matrix with vectors of
// 1 << shift values (vs_cvse_transpose): row_offsets = t_offsets, cols = t_rows, src = t_src.  A row of A^T is a
// column of A; a nonzero vector (i, c) of A lies in row c of A^T, columns i << shift .. (i << shift) + V - 1, which
// never straddle a 16-column block (V divides 16).  The entry keeps the vector's first column and its index in the caller's
// `values` array (t_src), so the multiplying kernel reads the values where the forward operators keep them and
// drops the V of them side by side into one row of its tile.  Groups are 128 rows of A^T.
// Costs: `gather_per_row`, `gather_per_entry` for the kernel that takes the call otherwise, `dense_per_entry` for
// the fill work of the dense kernel where that matters (V stores per vector instead of one).
template <bool kTransposed>
__global__ void __launch_bounds__(kPlanThreads)
dense_plan_kernel(const int32_t *__restrict__ row_offsets, const int32_t *__restrict__ cols, const int32_t *__restrict__ src,
                  int shift, int m_vec, int K, int groups, int rows_per_group, int plan_blocks,
                  int32_t *__restrict__ blk_offsets, uint2 *__restrict__ blk_entries, int64_t entry_capacity, int force_dense,
                  float gather_per_row, float gather_per_entry, float dense_per_entry, int32_t *use_dense) {
    auto offset_of = [&](int i) { return __ldg(row_offsets + i); };
    auto column_of = [&](int j) { return kTransposed ? __ldg(cols + j) << shift : __ldg(cols + j); };
    auto value_of = [&](int j) { return kTransposed ? __ldg(src + j) : j; };
    extern __shared__ int plan_sh[];
    pdl_launch_dependents();   // the multiplying kernel may be scheduled while the plan is made
    pdl_wait();                // this kernel too is launched as a dependent: the call ahead may still be reading the plan scratch
    {
        const int64_t nnz = __ldg(row_offsets + m_vec);
        const float stages = (float)(groups / (kTileM / kGroupRows)) * (float)(plan_blocks / (kBlockK / kPlanCols));
        const float dense_cost = stages * 1100.0f + dense_per_entry * (float)nnz;
        const float gather_cost = (float)m_vec * gather_per_row + gather_per_entry * (float)nnz;
        const bool dense = nnz <= entry_capacity && (force_dense || dense_cost < gather_cost);
        if (blockIdx.x == 0 && threadIdx.x == 0) *use_dense = dense ? 1 : 0;
        if (!dense) return;
    }
    if ((int)blockIdx.x >= groups) {
        const int check = blockIdx.x - groups, checks = gridDim.x - groups;
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        unsigned *seen = reinterpret_cast<unsigned *>(plan_sh) + warp * plan_blocks;   // one bit per column of the row in hand
        int twice = 0;
        for (int r = check * kPlanWarps + warp; r < m_vec; r += checks * kPlanWarps) {
            const int e0 = offset_of(r), e1 = offset_of(r + 1);
            if (e1 - e0 < 2) continue;
            for (int i = lane; i < plan_blocks; i += 32) seen[i] = 0u;
            __syncwarp();
            for (int e = e0 + lane; e < e1; e += 32) {
                const int c = column_of(e);
                if ((unsigned)c >= (unsigned)K) continue;
                const unsigned bit = 1u << (c & 31);
                if (atomicOr(seen + (c >> 5), bit) & bit) twice = 1;   // of two lanes with one column, the later sees the earlier's bit
            }
            __syncwarp();
        }
        twice = __syncthreads_or(twice);
        if (threadIdx.x == 0) use_dense[4 + check] = twice;
        return;
    }
    int *hist = plan_sh;                         // [plan_blocks]
    int *cursor = plan_sh + plan_blocks;         // [plan_blocks]
    int *roff = plan_sh + 2 * plan_blocks;       // [rows_per_group + 1]
    const int g = blockIdx.x, t = threadIdx.x;
    const int r0 = min(m_vec, g * rows_per_group), r1 = min(m_vec, r0 + rows_per_group);
    const int nr = r1 - r0;
    for (int i = t; i < plan_blocks; i += kPlanThreads) hist[i] = 0;
    for (int i = t; i <= nr; i += kPlanThreads) roff[i] = offset_of(r0 + i);
    __syncthreads();
    const int j0 = roff[0], j1 = roff[nr];
    // four entries per thread and trip, so that their loads are in flight together (a group of the transposed matrix
    // is thousands of entries for one CTA)
    for (int jb = j0 + t; jb < j1; jb += 4 * kPlanThreads) {
        int c[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) c[u] = jb + u * kPlanThreads < j1 ? column_of(jb + u * kPlanThreads) : -1;
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if ((unsigned)c[u] < (unsigned)K) atomicAdd(hist + c[u] / kPlanCols, 1);
    }
    __syncthreads();
    if (t < 32) {   // exclusive scan of the histogram by one warp, 32 buckets per trip
        int run = j0;
        int32_t *o = blk_offsets + (int64_t)g * (plan_blocks + 1);
        for (int c0 = 0; c0 < plan_blocks; c0 += 32) {
            const int h = c0 + t < plan_blocks ? hist[c0 + t] : 0;
            int incl = h;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, d);
                if (t >= d) incl += up;
            }
            if (c0 + t < plan_blocks) {
                cursor[c0 + t] = run + incl - h;
                o[c0 + t] = run + incl - h;
            }
            run += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (t == 0) o[plan_blocks] = run;
    }
    __syncthreads();
    for (int jb = j0 + t; jb < j1; jb += 4 * kPlanThreads) {
        int cc[4], vv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int jj = jb + u * kPlanThreads;
            cc[u] = jj < j1 ? column_of(jj) : -1;
            vv[u] = jj < j1 ? value_of(jj) : 0;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
        const int j = jb + u * kPlanThreads;
        const int c = cc[u];
        if ((unsigned)c >= (unsigned)K) continue;
        int lo = 0, hi = nr;   // vector-row of j: the last i with roff[i] <= j (empty rows share an offset)
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (roff[mid] <= j) lo = mid; else hi = mid;
        }
        const int pos = atomicAdd(cursor + c / kPlanCols, 1);
        blk_entries[pos] = make_uint2((uint32_t)vv[u], ((uint32_t)lo << 6) | (uint32_t)(c & (kBlockK - 1)));
        }
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
#ifndef VS_DENSE_SLEEP
#define VS_DENSE_SLEEP 32
#endif
constexpr int kSleepFill = VS_DENSE_SLEEP, kSleepMma = 0, kSleepEpilogue = VS_DENSE_SLEEP;

// Work item w of the launch -> (batch entry, column tile, row tile).
struct Item {
    int b, n0, tn, mt;
};
__device__ __forceinline__ Item decode_item(int64_t w, int m_tiles, int n_tiles, int N) {
    Item it;
    it.mt = (int)(w % m_tiles);
    const int64_t r = w / m_tiles;
    const int nt = (int)(r % n_tiles);
    it.b = (int)(r / n_tiles);
    it.n0 = nt * kTileN;
    it.tn = min(kTileN, (N - it.n0 + 63) & ~63);   // MMA N: whole 64-column boxes of B (zero-filled past N)
    return it;
}

// The same walk without divisions, for the roles that locate a stage every few hundred cycles: position
// (batch entry, column tile, row tile, column block) of stage g, advanced by a fixed number of stages.
struct StageIter {
    int b, nt, mt, kb;
    int d_mt, d_nt, d_b;   // one step of gridDim.x work items, as digits of (b, nt, mt)
    int m_tiles, n_tiles, k_blocks;
    uint32_t g, total;
    __device__ __forceinline__ void init(uint32_t g0, uint32_t total_stages, int m_tiles_, int n_tiles_, int k_blocks_) {
        m_tiles = m_tiles_; n_tiles = n_tiles_; k_blocks = k_blocks_;
        g = g0; total = total_stages;
        const uint32_t G = gridDim.x;
        d_mt = (int)(G % (uint32_t)m_tiles);
        const uint32_t r = G / (uint32_t)m_tiles;
        d_nt = (int)(r % (uint32_t)n_tiles);
        d_b = (int)(r / (uint32_t)n_tiles);
        const uint32_t i0 = g0 / (uint32_t)k_blocks;       // divisions once, here
        kb = (int)(g0 - i0 * (uint32_t)k_blocks);
        const int64_t w = blockIdx.x + (int64_t)i0 * G;
        mt = (int)(w % m_tiles);
        const int64_t rr = w / m_tiles;
        nt = (int)(rr % n_tiles);
        b = (int)(rr / n_tiles);
    }
    __device__ __forceinline__ bool valid() const { return g < total; }
    __device__ __forceinline__ void next_item() {
        mt += d_mt; nt += d_nt; b += d_b;
        if (mt >= m_tiles) { mt -= m_tiles; ++nt; }
        if (nt >= n_tiles) { nt -= n_tiles; ++b; }   // d_nt + carry < 2 n_tiles: one correction is enough
    }
    __device__ __forceinline__ void advance(int stages) {
        g += (uint32_t)stages;
        kb += stages;
        while (kb >= k_blocks) { kb -= k_blocks; next_item(); }
    }
};

// The items of this CTA one after the other (blockIdx.x, + gridDim.x, ...), again without divisions per step.
struct ItemIter {
    StageIter w;
    int N;
    __device__ __forceinline__ void init(int m_tiles, int n_tiles, int N_) {
        w.init(0u, 0xffffffffu, m_tiles, n_tiles, 1);
        N = N_;
    }
    __device__ __forceinline__ Item get() const {
        Item it;
        it.b = w.b; it.mt = w.mt; it.n0 = w.nt * kTileN;
        it.tn = min(kTileN, (N - it.n0 + 63) & ~63);
        return it;
    }
    __device__ __forceinline__ void next() { w.next_item(); }
};

// Drops one nonzero vector (`raw`: its V halves) into the fill warp's 128 rows of the A stage at `a_part`.
// The operand is MN-major (rows of A contiguous) with the 128-byte swizzle: element (row m, column k) of the
// 128 x 64 block lives at (m / 64) * 8 KiB + (k / 8) * 1 KiB + (k % 8) * 128 + (((m % 64) / 8) ^ (k % 8)) * 16 +
// (m % 8) * 2, so the V consecutive rows of a vector (V divides 8) are one contiguous store.
//
// kTransposed (the tile is a piece of A^T): the V values of a vector belong to ONE row, columns k .. k + V - 1
// (k a multiple of V, so they share k / 8): V two-byte stores, 128 bytes apart.
template <int V, bool kTransposed, typename Raw>
__device__ __forceinline__ void scatter_vector(uint8_t *a_part, uint32_t packed, const Raw &raw) {
    const uint32_t k = packed & 63u;
    if constexpr (!kTransposed) {
        const uint32_t m = ((packed >> 6) * V) & (kGroupRows - 1);   // first row of the vector inside the group
        uint8_t *dst = a_part + (m >> 6) * 8192 + (k >> 3) * 1024 + (k & 7u) * 128 + ((((m & 63u) >> 3) ^ (k & 7u)) << 4) + (m & 7u) * 2;
        *reinterpret_cast<Raw *>(dst) = raw;
    } else {
        const uint32_t m = (packed >> 6) & (kGroupRows - 1);         // the row inside the group
        const uint32_t m8 = (m & 63u) >> 3;
        uint8_t *row = a_part + (m >> 6) * 8192 + (k >> 3) * 1024 + (m & 7u) * 2;
        const unsigned short *h = reinterpret_cast<const unsigned short *>(&raw);
#pragma unroll
        for (uint32_t v = 0; v < (uint32_t)V; ++v) {
            const uint32_t kk = (k & 7u) + v;
            *reinterpret_cast<unsigned short *>(row + kk * 128 + ((m8 ^ kk) << 4)) = h[v];
        }
    }
}

template <int V> struct ValueVec;   // the V fp16 values of one nonzero vector, loaded with one instruction
template <> struct ValueVec<8> { typedef uint4 Raw; uint4 raw; __device__ void load(const __half *p) { raw = __ldg(reinterpret_cast<const uint4 *>(p)); } };
template <> struct ValueVec<4> { typedef uint2 Raw; uint2 raw; __device__ void load(const __half *p) { raw = __ldg(reinterpret_cast<const uint2 *>(p)); } };
template <> struct ValueVec<2> { typedef uint32_t Raw; uint32_t raw; __device__ void load(const __half *p) { raw = __ldg(reinterpret_cast<const uint32_t *>(p)); } };
template <> struct ValueVec<1> { typedef unsigned short Raw; unsigned short raw; __device__ void load(const __half *p) { raw = __ldg(reinterpret_cast<const unsigned short *>(p)); } };

// map_b: 3-D tensor map of the dense operand, dimensions {N, K, batch}, box {64, 64, 1}, 128-byte swizzle,
// zero fill outside.  map_b4 (used when N is a multiple of 64): the same memory as {64, K, N / 64, batch} with box
// {64, 64, 2, 1}, i.e. both boxes of a stage in one copy (the TMA unit works through copies one after the
// other, and two 8 KiB copies per stage were what the MMAs waited for).  map_out: the output, dimensions {N, rows, batch}, box {32, 32, 1}, swizzle span =
// the 64 (fp16) or 128 (fp32) bytes of a box row (stores clip at the edges of the matrix).
template <typename TOut, int V, bool kTransposed>
__global__ void __launch_bounds__(kThreads, 1)
spmm_dense_kernel(const SpmmParams p, const __grid_constant__ CUtensorMap map_b,
                  const __grid_constant__ CUtensorMap map_out, const __grid_constant__ CUtensorMap map_b4, int use_b4,
                  const int32_t *__restrict__ blk_offsets,
                  const uint2 *__restrict__ blk_entries, int m_tiles, int n_tiles, int k_blocks, uint32_t *status,
                  int32_t *use_dense, int plan_checks) {
    pdl_launch_dependents();   // the gather kernel behind this one may queue up
    pdl_wait();                // launched while the plan kernel may still be at work: nothing it writes is read before here
    // Not chosen (the gather kernel behind this one takes the call): the CTA still sets itself up and tears itself
    // down, with no work items in between.  (An early return that depends on a barrier's result made the compiler
    // treat the rest of the kernel as possibly divergent: 17 % slower.  Taking the verdict here, ahead of the
    // set-up, is also what the compiler likes best: taken after it — which would let the set-up overlap the plan
    // kernel — the same code ran 14 % slower at 50 % sparsity and 8 % slower at width 64.)
    const bool chosen = plan_dense_chosen(use_dense, plan_checks);
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

    for (int i = t; i < kAStages * kAStageBytes / 16; i += kThreads)   // the A slots start out as zeros
        reinterpret_cast<uint4 *>(sm + Smem::kA)[i] = make_uint4(0, 0, 0, 0);
    if (t == 0) {
        for (int s = 0; s < kBStages; ++s) {
            tc::mbar_init(bar_full + 8 * s, kFillPerSlot + 1);   // the fill warps and the loader (+ the bytes of B)
            tc::mbar_init(bar_empty + 8 * s, kMmaWarps);         // one commit per MMA-issuing thread
        }
        for (int s = 0; s < 2; ++s) {
            tc::mbar_init(bar_acc_full + 8 * s, kMmaWarps);
            tc::mbar_init(bar_acc_empty + 8 * s, kEpiWarps * 32);
        }
        *abort_flag = 0;
        *reinterpret_cast<volatile uint32_t *>(sm + Smem::kLoaderProgress) = 0;
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

    const int64_t total_items = chosen ? (int64_t)p.batch * n_tiles * m_tiles : 0;
    const int64_t G = gridDim.x;
    const uint32_t my_items = (total_items > blockIdx.x) ? (uint32_t)((total_items - blockIdx.x + G - 1) / G) : 0u;
    const uint32_t total_stages = my_items * (uint32_t)k_blocks;
    const int m_rows = kTransposed ? p.m_vec : p.m_vec * V;   // rows of the output (for A^T, p.m_vec counts its rows)

    // Stage g of this CTA (item g / k_blocks, column block g % k_blocks) uses A slot g % kAStages, B slot
    // g % kBStages and the barrier pair of its B slot: `full` collects the four fill warps, the loader's arrival
    // and the bytes of B; `empty` the two MMA threads' commits.  A fill warp waits for the stage kAStages before
    // its own, so it sees every phase of the two barriers it alternates between.
    if (warp >= kFillWarp0 && warp < kLoadWarp) {
        // =========================== fill ================================================================
        const int fw = warp - kFillWarp0;
        const uint32_t a_slot = (uint32_t)(fw % kAStages);
        const int bucket = fw / kAStages;                  // 0..3
        const int half = bucket >> 1;                      // rows 128 * half .. + 127 of the tile
        const int khalf = bucket & 1;                      // columns 32 * khalf .. + 31 of the stage
        uint8_t *a_part = sm + Smem::kA + a_slot * kAStageBytes + half * (kGroupRows * kBlockK * 2);
        const int plan_blocks = (kBlockK / kPlanCols) * k_blocks;

        // Software pipeline over this warp's stages (a_slot, a_slot + 3, ...): bucket bounds two stages ahead,
        // the first 64 entries one stage ahead, their values before the wait for the slot.
        struct Pos { int b, mt, kb; bool valid; };
        StageIter walk;
        walk.init(a_slot, total_stages, m_tiles, n_tiles, k_blocks);
        auto locate = [&]() {   // the walker's position, then kAStages further on
            Pos q;
            q.valid = walk.valid(); q.b = walk.b; q.mt = walk.mt; q.kb = walk.kb;
            walk.advance(kAStages);
            return q;
        };
        auto bounds = [&](const Pos &q, int &e0, int &e1) {
            e0 = 0; e1 = 0;
            if (q.valid) {
                // this warp's two buckets follow one another in the entry list
                const int32_t *o = blk_offsets + ((int64_t)q.mt * (kTileM / kGroupRows) + half) * (plan_blocks + 1) +
                                   (kBlockK / kPlanCols) * q.kb + (kFillCols / kPlanCols) * khalf;
                e0 = __ldg(o);
                e1 = __ldg(o + kFillCols / kPlanCols);
            }
        };
        Pos cur = locate(), nxt = locate();
        int c_e0, c_e1, n_e0, n_e1;
        bounds(cur, c_e0, c_e1);
        bounds(nxt, n_e0, n_e1);
        uint2 c_ent[kFillBatches];
#pragma unroll
        for (int u = 0; u < kFillBatches; ++u) {
            const int e = c_e0 + lane + 32 * u;
            c_ent[u] = e < c_e1 ? __ldg(blk_entries + e) : make_uint2(0u, 0u);
        }
        int p_e0 = 0, p_e1 = 0;            // the bucket this warp dropped into the slot last time
        uint32_t p_pos[kFillBatches] = {};
        bool ok_run = true;
        for (uint32_t g = a_slot; g < total_stages && ok_run; g += kAStages) {
            const __half *vals = static_cast<const __half *>(p.values) + (int64_t)cur.b * p.stride_values;
            // values of the first 64 entries, entries of the next stage, bounds of the one after: all in flight
            // while this warp waits for its slot
            ValueVec<V> c_val[kFillBatches];
#pragma unroll
            for (int u = 0; u < kFillBatches; ++u)
                if (c_e0 + lane + 32 * u < c_e1) c_val[u].load(vals + (int64_t)c_ent[u].x * V);
            uint2 n_ent[kFillBatches];
#pragma unroll
            for (int u = 0; u < kFillBatches; ++u) {
                const int e = n_e0 + lane + 32 * u;
                n_ent[u] = e < n_e1 ? __ldg(blk_entries + e) : make_uint2(0u, 0u);
            }
            const Pos nn = locate();
            int nn_e0, nn_e1;
            bounds(nn, nn_e0, nn_e1);

            if (g >= (uint32_t)kAStages) {   // the stage that used this A slot before must have been multiplied
                const uint32_t prev = g - kAStages;
                ok_run = wait_or_abort<kSleepFill>(bar_empty + 8 * (prev % kBStages), (prev / kBStages) & 1u, abort_flag);
            }
            if (!ok_run) break;
            // The A slots start out as zeros; a slot is brought back to zeros by overwriting exactly the vectors
            // this warp dropped into it for the stage before (kAStages earlier), which costs a few stores
            // instead of 8 KiB of them: shared-memory bandwidth is what bounds this kernel.
            {
                typename ValueVec<V>::Raw zero{};
#pragma unroll
                for (int u = 0; u < kFillBatches; ++u)
                    if (p_e0 + lane + 32 * u < p_e1) scatter_vector<V, kTransposed>(a_part, p_pos[u], zero);
                for (int e0 = p_e0 + 32 * kFillBatches; e0 < p_e1; e0 += 32 * kOverflowBatches) {   // denser buckets
                    uint32_t pos[kOverflowBatches];
#pragma unroll
                    for (int u = 0; u < kOverflowBatches; ++u) {
                        const int e = e0 + 32 * u + lane;
                        pos[u] = e < p_e1 ? __ldg(blk_entries + e).y : 0u;
                    }
#pragma unroll
                    for (int u = 0; u < kOverflowBatches; ++u)
                        if (e0 + 32 * u + lane < p_e1) scatter_vector<V, kTransposed>(a_part, pos[u], zero);
                }
            }
            __syncwarp();
#pragma unroll
            for (int u = 0; u < kFillBatches; ++u)
                if (c_e0 + lane + 32 * u < c_e1) scatter_vector<V, kTransposed>(a_part, c_ent[u].y, c_val[u].raw);
            // buckets with more entries (denser rows): several batches of loads in flight at a time
            for (int e0 = c_e0 + 32 * kFillBatches; e0 < c_e1; e0 += 32 * kOverflowBatches) {
                uint2 en[kOverflowBatches];
                ValueVec<V> val[kOverflowBatches];
#pragma unroll
                for (int u = 0; u < kOverflowBatches; ++u) {
                    const int e = e0 + 32 * u + lane;
                    en[u] = e < c_e1 ? __ldg(blk_entries + e) : make_uint2(0u, 0u);
                }
#pragma unroll
                for (int u = 0; u < kOverflowBatches; ++u)
                    if (e0 + 32 * u + lane < c_e1) val[u].load(vals + (int64_t)en[u].x * V);
#pragma unroll
                for (int u = 0; u < kOverflowBatches; ++u)
                    if (e0 + 32 * u + lane < c_e1) scatter_vector<V, kTransposed>(a_part, en[u].y, val[u].raw);
            }
            p_e0 = c_e0; p_e1 = c_e1;
#pragma unroll
            for (int u = 0; u < kFillBatches; ++u) p_pos[u] = c_ent[u].y;
            tc::fence_proxy_async();   // the tile was written by ordinary stores; the MMA reads through the async proxy
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(bar_full + 8 * (g % kBStages));

            cur = nxt; c_e0 = n_e0; c_e1 = n_e1;
#pragma unroll
            for (int u = 0; u < kFillBatches; ++u) c_ent[u] = n_ent[u];
            nxt = nn; n_e0 = nn_e0; n_e1 = nn_e1;
        }
    } else if (warp == kLoadWarp) {
        // =========================== B loader ============================================================
        // One thread keeps up to kBStages tiles of B in flight: one 64 x 64 box per 64 columns of the item.
        if (lane == 0) {
            volatile uint32_t *progress = reinterpret_cast<volatile uint32_t *>(sm + Smem::kLoaderProgress);
            uint32_t g = 0;
            bool ok_run = true;
            ItemIter items;
            items.init(m_tiles, n_tiles, p.N);
            for (uint32_t i = 0; i < my_items && ok_run; ++i, items.next()) {
                const Item it = items.get();
                const int slabs = (it.tn + 63) >> 6;
                for (int kb = 0; kb < k_blocks && ok_run; ++kb, ++g) {
                    const uint32_t slot = g % kBStages;
                    if (g >= (uint32_t)kBStages)
                        ok_run = wait_or_abort<kSleepFill>(bar_empty + 8 * slot, ((g / kBStages) - 1u) & 1u, abort_flag);
                    if (!ok_run) break;
                    const uint32_t bar = bar_full + 8 * slot;
                    tc::mbar_expect_tx(bar, (uint32_t)slabs * kBSlabBytes);   // arrives and arms the byte count
                    if (use_b4 && slabs == kTileN / 64) {   // both boxes with one instruction
                        tc::tma_load_4d(base + Smem::kB + slot * kBStageBytes, &map_b4, bar, 0, kb * kBlockK, it.n0 >> 6, it.b);
                    } else {
                        for (int s = 0; s < slabs; ++s)
                            tc::tma_load_3d(base + Smem::kB + slot * kBStageBytes + s * kBSlabBytes, &map_b, bar, it.n0 + 64 * s,
                                            kb * kBlockK, it.b);
                    }
                    *progress = g + 1;
                }
            }
        }
    } else if (warp == kPrefetchWarp) {
        // =========================== L2 prefetch =========================================================
        // First touches of B come from DRAM, a latency the ring of six stages does not cover, and prefetches
        // through the TMA queue would hold up the loads queued behind them.  This warp asks each tile into L2
        // with plain prefetches about one work item before the loader wants it, paced by the loader's counter.
        volatile uint32_t *progress = reinterpret_cast<volatile uint32_t *>(sm + Smem::kLoaderProgress);
        const __half *rhs = static_cast<const __half *>(p.rhs);
        uint32_t g = (uint32_t)k_blocks;   // the stage being prefetched
        bool ok_run = true;
        ItemIter items;
        items.init(m_tiles, n_tiles, p.N);
        for (uint32_t i = 1; i < my_items && ok_run; ++i) {
            items.next();
            const Item it = items.get();
            const __half *b_tile = rhs + (int64_t)it.b * p.stride_rhs + it.n0;
            for (int kb = 0; kb < k_blocks && ok_run; ++kb, ++g) {
                const int32_t need = (int32_t)g - k_blocks - 2;   // at most an item and two stages ahead of the loader
                uint32_t polls = 0;
                while ((int32_t)*progress < need) {
                    __nanosleep(200);
                    if (++polls > (1u << 20) || *abort_flag) { ok_run = false; break; }
                }
                if (!ok_run) break;
#pragma unroll
                for (int j = 0; j < 4; ++j) {   // 64 rows x up to two 128-byte lines
                    const int r = kb * kBlockK + lane * 2 + (j >> 1), c = (j & 1) * 64;
                    if (r < p.K && it.n0 + c < p.N) asm volatile("prefetch.global.L2 [%0];" ::"l"(b_tile + (int64_t)r * p.N + c));
                }
            }
        }
    } else if (warp >= kMmaWarp) {
        // =========================== MMA issuers =========================================================
        // Thread (h, j) multiplies rows 128 h .. 128 h + 127 of the tile for its share j of every stage's K
        // steps.  With one thread per half (the shipped configuration) the first MMA of an item overwrites the
        // accumulator.  With more (VS_DENSE_KSPLIT = 2) every MMA accumulates onto accumulators the epilogue
        // hands back zeroed, because the order in which the threads' MMAs reach the pipe is then free; it also
        // varies from run to run, and with it the last bits of the sums.  All threads wait on every stage and
        // commit to its `empty` barrier, so each has seen every earlier use of a slot complete.
        if (lane == 0) {
            constexpr int kSteps = (kBlockK / 16) / kKSplit;   // K steps of a stage per thread
            const int h = (warp - kMmaWarp) / kKSplit, j = (warp - kMmaWarp) % kKSplit;
            const uint32_t a_lo0 = tc::smem_desc_lo(base + Smem::kA + h * (128 * kBlockK * 2), 8192) + 128u * kSteps * j;   // 64-row atoms 8 KiB apart
            const uint32_t a_hi = tc::smem_desc_hi(1024, (uint32_t)tc::kSwizzle128B);
            const uint32_t b_lo0 = tc::smem_desc_lo(base + Smem::kB, kBSlabBytes) + 128u * kSteps * j;   // this thread's first K step
            const uint32_t b_hi = tc::smem_desc_hi(1024, (uint32_t)tc::kSwizzle128B);
            uint32_t a_slot = 0, b_slot = 0, b_parity = 0;
            bool ok_run = true;
            ItemIter items;
            items.init(m_tiles, n_tiles, p.N);
            bool ready = false;   // whether the next stage was already seen full
            for (uint32_t i = 0; i < my_items && ok_run; ++i, items.next()) {
                const Item it = items.get();
                const uint32_t idesc = tc::make_idesc_f16(128, it.tn, 1, 1);   // both operands MN-major
                const uint32_t buf = i & 1u;
                ok_run = wait_or_abort<kSleepMma>(bar_acc_empty + 8 * buf, (i >> 1) & 1u, abort_flag);   // zeroed and free
                tc::tc_fence_after_sync();
                const uint32_t d = tmem_base + buf * kAccCols + (uint32_t)h * kTileN;
                int k_left = p.K - 16 * kSteps * j;   // columns of A from this thread's first K step on
                for (int kb = 0; kb < k_blocks && ok_run; ++kb, k_left -= kBlockK) {
                    if (!ready) ok_run = wait_or_abort<kSleepMma>(bar_full + 8 * b_slot, b_parity, abort_flag);
                    if (!ok_run) break;
                    tc::tc_fence_after_sync();
                    const uint32_t a_lo = a_lo0 + a_slot * (kAStageBytes >> 4), b_lo = b_lo0 + b_slot * (kBStageBytes >> 4);
                    // 16 columns of A = 16 rows of B = 2 KiB further on in either operand
#pragma unroll
                    for (int kk = 0; kk < kSteps; ++kk)
                        if (k_left > 16 * kk)
                            tc::mma_f16_ss(d, tc::desc64(a_lo + 128 * kk, a_hi), tc::desc64(b_lo + 128 * kk, b_hi), idesc,
                                           (kZeroedAcc || kb > 0 || kk > 0) ? 1u : 0u);
                    tc::mma_commit(bar_empty + 8 * b_slot);
                    if (++a_slot == (uint32_t)kAStages) a_slot = 0;
                    if (++b_slot == (uint32_t)kBStages) { b_slot = 0; b_parity ^= 1u; }
                    // one look at the next stage's barrier (this CTA's stages follow one another across items):
                    // its latency passes while the MMAs above are handed to the pipe
                    ready = (kb + 1 < k_blocks || i + 1 < my_items) && tc::mbar_try_wait(bar_full + 8 * b_slot, b_parity);
                }
                if (ok_run) tc::mma_commit(bar_acc_full + 8 * buf);
            }
        }
    } else {
        // =========================== epilogue ============================================================
        // Warp (quarter, half) owns rows 128 half + 32 quarter .. + 31 of every tile: TMEM lanes 32 quarter ..
        // of accumulator columns 128 half ..  It moves them out 32 columns at a time: TMEM -> registers -> a box
        // of shared memory whose 16-byte
        // chunks are XOR-swizzled by row, so that the row-per-thread writes spread over the banks -> one TMA
        // store of 32 whole row segments.  fp16 boxes are 2 KiB and alternate between two buffers.
        constexpr int kBoxBytes = 32 * kStoreCols * (int)sizeof(TOut);       // 2 KiB (fp16) or 4 KiB (fp32)
        constexpr int kBoxes = kStoreBoxBytes / kBoxBytes;                   // 2 or 1 buffers
        constexpr int kRowBytes = kStoreCols * (int)sizeof(TOut);            // 64 or 128: also the swizzle span
        constexpr int kChunks = kRowBytes / 16;                              // 4 or 8 chunks per row
        bool ok_run = true;
        float finite_probe[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const int quarter = warp & 3, half = warp >> 2;
        uint8_t *stg = sm + Smem::kStaging + warp * kStoreBoxBytes;
        const uint32_t stg_u32 = base + Smem::kStaging + warp * kStoreBoxBytes;
        const uint32_t lane_taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(half * kTileN);
        // the swizzle of a 16-byte chunk index: address bits 4.. XOR address bits 7..
        const int swz = (kRowBytes == 128) ? (lane & 7) : ((lane >> 1) & 3);
        uint32_t box_count = 0;
        // both accumulator buffers start out free (and zeroed, if the MMAs rely on that)
        if (kZeroedAcc) {
            for (int c0 = 0; c0 < 2 * kAccCols; c0 += kAccCols)
                for (int c = 0; c < kTileN; c += 32) tc::tmem_st_zero_x32(lane_taddr + (uint32_t)(c0 + c));
            tc::tmem_st_wait();
        }
        tc::tc_fence_before_sync();
        tc::mbar_arrive(bar_acc_empty);
        tc::mbar_arrive(bar_acc_empty + 8);
        ItemIter items;
        items.init(m_tiles, n_tiles, p.N);
        for (uint32_t i = 0; i < my_items && ok_run; ++i, items.next()) {
            const Item it = items.get();
            const uint32_t buf = i & 1u;
            // warp-uniform outcome: tcgen05.ld below needs all 32 lanes
            ok_run = __all_sync(0xffffffffu, wait_or_abort<kSleepEpilogue>(bar_acc_full + 8 * buf, (i >> 1) & 1u, abort_flag));
            if (!ok_run) break;
            tc::tc_fence_after_sync();
            const int row0 = it.mt * kTileM + half * 128 + quarter * 32;   // first row of this warp's boxes
#pragma unroll 1
            for (int c0 = 0; c0 < it.tn; c0 += kStoreCols) {
                uint32_t r[kStoreCols];
                const uint32_t taddr = lane_taddr + buf * kAccCols + (uint32_t)c0;
                tc::tmem_ld_x32(taddr, r);
                if (kZeroedAcc) tc::tmem_st_zero_x32(taddr);
                if (row0 < m_rows && it.n0 + c0 < p.N) {   // warp-uniform
                    // x * 0 is 0 for a finite x and NaN otherwise: one FMA per element finds a non-finite sum
                    // (every column of the box was written by the MMA: columns past N multiply zero-filled B)
                    if (row0 + lane < m_rows) {
#pragma unroll
                        for (int e = 0; e < kStoreCols; ++e) finite_probe[e & 3] = fmaf(__uint_as_float(r[e]), 0.0f, finite_probe[e & 3]);
                    }
                    const uint32_t box = kBoxes == 2 ? (box_count & 1u) : 0u;
                    if (lane == 0) tc::bulk_wait_group_read<kBoxes - 1>();   // the store that used this box before has read it
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
                        tc::tma_store_3d(&map_out, stg_u32 + box * kBoxBytes, it.n0 + c0, row0, it.b);
                        tc::bulk_commit_group();
                    }
                    ++box_count;
                }
            }
            if (kZeroedAcc) tc::tmem_st_wait();
            tc::tc_fence_before_sync();
            tc::mbar_arrive(bar_acc_empty + 8 * buf);   // read out (and zeroed): the buffer is free
        }
        // A zero of the densified tile times an Inf or NaN of B is a NaN that the reference, which only reads
        // the rows of B its nonzeros name, would not produce.  Any non-finite sum hands the call to the gather
        // kernel enqueued behind this one, which then overwrites the output.
        if (lane == 0) tc::bulk_wait_group<0>();   // every store of this warp has reached global memory
        const float probe = (finite_probe[0] + finite_probe[1]) + (finite_probe[2] + finite_probe[3]);
        if (__any_sync(0xffffffffu, probe != 0.0f) && lane == 0) atomicExch(use_dense, 0);
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

}  // namespace densespmm
}  // namespace vs
