// Tensor-core SpMM for fp16 operands on sm_100a by densifying tiles of the sparse matrix in shared memory: the
// `wmmaSpmm` entry point of the reference (src/wmma_spmm.cu:388-409) for matrices that are not extremely sparse.
//
// Why.  The reference (and the gather kernels next to this file) fetch one row of the dense operand per
// nonzero vector, because on Volta the tensor cores were the scarce resource.  On B200 they are not: a 128 x 128
// x 16 MMA takes ~65 cycles, while gathering the rows a vector-row needs costs hundreds of cycles of TMA / LSU
// issue.  Up to ~97 % sparsity it is cheaper to multiply a zero-filled dense tile of A:
//     C[256 rows x 128 cols] += A_dense[256 x 64] * B[64 x 128]          per 64-wide block of A's columns.
// A_dense is built in shared memory from the CVSE arrays (zero fill + one store per nonzero vector: the operand
// is kept MN-major, rows contiguous, in the 128-byte-swizzled layout the MMA reads); B arrives by plain TMA tile loads (two 8 KiB boxes per
// stage, no gather); the products with the zeros are free.  The result is the same sum in another order, except
// when B holds Inf / NaN in rows no nonzero names (0 x Inf = NaN): the epilogue therefore watches for
// non-finite sums and, if it sees one, clears the flag that keeps the gather kernel behind it from running.
//
// Plan.  A small kernel first buckets the nonzero vectors by (128-row group, 64-column block): `blk_offsets`
// [row groups][column blocks + 1] and `blk_entries` (vector index, vector-row within the group, column within
// the block).  The plan depends on the structure only and is shared by every matrix of a batch.
//
// Organisation: one persistent CTA per SM.  Work items are (batch, 128-column tile of B, 256-row tile of A),
// consecutive CTAs taking consecutive row tiles of the same B so that it stays in L2.  A stage is one 64-wide
// block of A's columns: 32 KiB of A (two 128-row MMA operands) + 16 KiB of B, four stages in a ring.
//   warps 0-7    epilogue: TMEM -> registers -> swizzled shared-memory boxes -> TMA stores of whole rows
//   warps 8-15   fill: two warps per ring slot, each owning 128 rows of the A tile; the first of them also
//                issues the stage's B loads
//   warps 16-17  one MMA-issuing thread per 128-row half of the tile
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
constexpr int kGroupRows = 128;                          // rows per plan bucket = rows one fill warp owns = one MMA operand
constexpr int kStages = 4;
constexpr int kEpiWarps = 8;                             // warps 0..7: TMEM lane quarter = warp % 4, half of the tile = warp / 4
constexpr int kFillWarp0 = kEpiWarps;
constexpr int kFillPerSlot = kTileM / kGroupRows;        // 2
constexpr int kFillWarps = kStages * kFillPerSlot;       // 8: warp f fills slot f % kStages, rows 128 * (f / kStages) ..
constexpr int kFillBatches = 4;                          // entries a fill warp keeps in flight: 4 x 32
constexpr int kMmaWarp = kFillWarp0 + kFillWarps;        // 16, 17
constexpr int kMmaWarps = kTileM / 128;                  // 2
constexpr int kThreads = (kMmaWarp + kMmaWarps) * 32;    // 576
constexpr int kAStageBytes = kTileM * kBlockK * 2;       // 32 KiB
constexpr int kBSlabBytes = kBlockK * 64 * 2;            // 8 KiB: 64 rows of B x 64 columns
constexpr int kBStageBytes = (kTileN / 64) * kBSlabBytes;  // 16 KiB
constexpr int kAccCols = kMmaWarps * kTileN;             // 256 TMEM columns per accumulator buffer
constexpr int kTmemCols = 2 * kAccCols;                  // 512
constexpr int kStoreBoxBytes = 32 * 128;                 // output box of one epilogue warp: 32 rows x 128 bytes
constexpr int kPlanThreads = 256;

constexpr uint32_t kStatusTimeout = 64u;  // bit raised in the status word when a bounded wait ran out

struct Smem {  // offsets from the 1024-byte aligned base
    static constexpr int kA = 0;
    static constexpr int kB = kA + kStages * kAStageBytes;
    static constexpr int kStaging = kB + kStages * kBStageBytes;   // per epilogue warp: one 32-row x 128-byte box
    static constexpr int kBarFull = kStaging + kEpiWarps * kStoreBoxBytes;
    static constexpr int kBarEmpty = kBarFull + kStages * 8;
    static constexpr int kBarAccFull = kBarEmpty + kStages * 8;
    static constexpr int kBarAccEmpty = kBarAccFull + 2 * 8;
    static constexpr int kTmemHolder = kBarAccEmpty + 2 * 8;
    static constexpr int kAbort = kTmemHolder + 8;
    static constexpr int kTotal = kAbort + 8;
};
constexpr int kSmemBytes = Smem::kTotal + 1024;  // + slack for the manual 1024-byte alignment
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
static_assert(kFillWarps % kStages == 0, "each ring slot needs fixed owner warps");

// ---- plan -------------------------------------------------------------------------------------------------
// One CTA per 128-row group (128 / V vector-rows, whose nonzero vectors are contiguous in the CVSE arrays).
// blk_offsets[g * (k_blocks + 1) + kb] .. [.. + kb + 1] delimit the entries of group g in column block kb;
// entry = (vector index j, (vector-row within the group << 6) | column within the block).  Columns outside
// [0, K) are dropped (the gather kernels read zeros for them).
//
// The kernel also takes the decision between the densifying and the gather kernels, because the number of
// nonzero vectors is only known here: dense when the density reaches `threshold` and the entries fit the
// scratch (`entry_capacity`).  Every CTA computes the same answer; CTA 0 publishes it in *use_dense for the two
// kernels enqueued behind this one, and nothing is planned when the answer is no.
__global__ void __launch_bounds__(kPlanThreads)
dense_plan_kernel(const int32_t *__restrict__ row_offsets, const int32_t *__restrict__ col_indices, int m_vec, int K,
                  int rows_per_group, int k_blocks, int32_t *__restrict__ blk_offsets, uint2 *__restrict__ blk_entries,
                  int64_t entry_capacity, float threshold, int32_t *use_dense) {
    extern __shared__ int plan_sh[];
    {
        const int64_t nnz = __ldg(row_offsets + m_vec);
        const float density = (float)nnz / ((float)m_vec * (float)K);
        const bool dense = nnz <= entry_capacity && density >= threshold;
        if (blockIdx.x == 0 && threadIdx.x == 0) *use_dense = dense ? 1 : 0;
        if (!dense) return;
    }
    int *hist = plan_sh;                      // [k_blocks]
    int *cursor = plan_sh + k_blocks;         // [k_blocks]
    int *roff = plan_sh + 2 * k_blocks;       // [rows_per_group + 1]
    const int g = blockIdx.x, t = threadIdx.x;
    const int r0 = min(m_vec, g * rows_per_group), r1 = min(m_vec, r0 + rows_per_group);
    const int nr = r1 - r0;
    for (int i = t; i < k_blocks; i += kPlanThreads) hist[i] = 0;
    for (int i = t; i <= nr; i += kPlanThreads) roff[i] = __ldg(row_offsets + r0 + i);
    __syncthreads();
    const int j0 = roff[0], j1 = roff[nr];
    for (int j = j0 + t; j < j1; j += kPlanThreads) {
        const int c = __ldg(col_indices + j);
        if ((unsigned)c < (unsigned)K) atomicAdd(hist + (c >> 6), 1);
    }
    __syncthreads();
    if (t == 0) {
        int run = j0;
        int32_t *o = blk_offsets + (int64_t)g * (k_blocks + 1);
        for (int kb = 0; kb < k_blocks; ++kb) {
            cursor[kb] = run;
            o[kb] = run;
            run += hist[kb];
        }
        o[k_blocks] = run;
    }
    __syncthreads();
    for (int j = j0 + t; j < j1; j += kPlanThreads) {
        const int c = __ldg(col_indices + j);
        if ((unsigned)c >= (unsigned)K) continue;
        int lo = 0, hi = nr;   // vector-row of j: the last i with roff[i] <= j (empty rows share an offset)
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (roff[mid] <= j) lo = mid; else hi = mid;
        }
        const int pos = atomicAdd(cursor + (c >> 6), 1);
        blk_entries[pos] = make_uint2((uint32_t)j, ((uint32_t)lo << 6) | (uint32_t)(c & 63));
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
constexpr int kSleepFill = 100, kSleepMma = 0, kSleepEpilogue = 100;

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

// Drops one nonzero vector (`raw`: its V halves) into the fill warp's 128 rows of the A stage at `a_part`.
// The operand is MN-major (rows of A contiguous) with the 128-byte swizzle: element (row m, column k) of the
// 128 x 64 block lives at (m / 64) * 8 KiB + (k / 8) * 1 KiB + (k % 8) * 128 + (((m % 64) / 8) ^ (k % 8)) * 16 +
// (m % 8) * 2, so the V consecutive rows of a vector (V divides 8) are one contiguous store.
template <int V, typename Raw>
__device__ __forceinline__ void scatter_vector(uint8_t *a_part, uint32_t packed, const Raw &raw) {
    const uint32_t k = packed & 63u;
    const uint32_t m = ((packed >> 6) * V) & (kGroupRows - 1);   // first row of the vector inside the group
    uint8_t *dst = a_part + (m >> 6) * 8192 + (k >> 3) * 1024 + (k & 7u) * 128 + ((((m & 63u) >> 3) ^ (k & 7u)) << 4) + (m & 7u) * 2;
    *reinterpret_cast<Raw *>(dst) = raw;
}

template <int V> struct ValueVec;   // the V fp16 values of one nonzero vector, loaded with one instruction
template <> struct ValueVec<8> { uint4 raw; __device__ void load(const __half *p) { raw = __ldg(reinterpret_cast<const uint4 *>(p)); } };
template <> struct ValueVec<4> { uint2 raw; __device__ void load(const __half *p) { raw = __ldg(reinterpret_cast<const uint2 *>(p)); } };
template <> struct ValueVec<2> { uint32_t raw; __device__ void load(const __half *p) { raw = __ldg(reinterpret_cast<const uint32_t *>(p)); } };
template <> struct ValueVec<1> { unsigned short raw; __device__ void load(const __half *p) { raw = __ldg(reinterpret_cast<const unsigned short *>(p)); } };

// map_b: 3-D tensor map of the dense operand, dimensions {N, K, batch}, box {64, 64, 1}, 128-byte swizzle,
// zero fill outside.  map_out: the output, dimensions {N, rows, batch}, box {128 bytes of columns, 32, 1},
// 128-byte swizzle (stores clip at the edges of the matrix).
template <typename TOut, int V>
__global__ void __launch_bounds__(kThreads, 1)
spmm_dense_kernel(const SpmmParams p, const __grid_constant__ CUtensorMap map_b,
                  const __grid_constant__ CUtensorMap map_out, const int32_t *__restrict__ blk_offsets,
                  const uint2 *__restrict__ blk_entries, int m_tiles, int n_tiles, int k_blocks, uint32_t *status,
                  int32_t *use_dense) {
    if (*use_dense == 0) return;   // the plan kernel chose the gather kernel for this matrix
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
            tc::mbar_init(bar_full + 8 * s, kFillPerSlot);   // one arrival per fill warp (+ the bytes of B)
            tc::mbar_init(bar_empty + 8 * s, kMmaWarps);     // one commit per MMA-issuing thread
        }
        for (int s = 0; s < 2; ++s) {
            tc::mbar_init(bar_acc_full + 8 * s, kMmaWarps);
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

    const int64_t total_items = (int64_t)p.batch * n_tiles * m_tiles;
    const int64_t G = gridDim.x;
    const uint32_t my_items = (total_items > blockIdx.x) ? (uint32_t)((total_items - blockIdx.x + G - 1) / G) : 0u;
    const uint32_t total_stages = my_items * (uint32_t)k_blocks;
    const int m_rows = p.m_vec * V;

    if (warp >= kFillWarp0 && warp < kMmaWarp) {
        // =========================== fill ================================================================
        const int fw = warp - kFillWarp0;
        const uint32_t slot = (uint32_t)(fw % kStages);
        const int part = fw / kStages;                     // rows 128 * part .. + 127 of the tile
        uint8_t *a_part = sm + Smem::kA + slot * kAStageBytes + part * (kGroupRows * kBlockK * 2);
        const uint32_t bar = bar_full + 8 * slot;

        // Software pipeline over this warp's stages (slot, slot + 4, ...): bucket bounds two stages ahead, the
        // first 128 entries one stage ahead, their values before the wait for the slot.
        struct Pos { int b, n0, tn, mt, kb; bool valid; };
        auto locate = [&](uint32_t g) {
            Pos q;
            q.valid = g < total_stages;
            const uint32_t i = q.valid ? g / (uint32_t)k_blocks : 0u;
            q.kb = q.valid ? (int)(g - i * (uint32_t)k_blocks) : 0;
            const Item it = decode_item(blockIdx.x + (int64_t)i * G, m_tiles, n_tiles, p.N);
            q.b = it.b; q.n0 = it.n0; q.tn = it.tn; q.mt = it.mt;
            return q;
        };
        auto bounds = [&](const Pos &q, int &e0, int &e1) {
            e0 = 0; e1 = 0;
            if (q.valid) {
                const int32_t *o = blk_offsets + ((int64_t)q.mt * kFillPerSlot + part) * (k_blocks + 1) + q.kb;
                e0 = __ldg(o);
                e1 = __ldg(o + 1);
            }
        };
        Pos cur = locate(slot), nxt = locate(slot + kStages);
        int c_e0, c_e1, n_e0, n_e1;
        bounds(cur, c_e0, c_e1);
        bounds(nxt, n_e0, n_e1);
        uint2 c_ent[kFillBatches];
#pragma unroll
        for (int u = 0; u < kFillBatches; ++u) {
            const int e = c_e0 + lane + 32 * u;
            c_ent[u] = e < c_e1 ? __ldg(blk_entries + e) : make_uint2(0u, 0u);
        }
        bool ok_run = true;
        VS_PROF_T0();
        for (uint32_t g = slot; g < total_stages && ok_run; g += kStages) {
            const __half *vals = static_cast<const __half *>(p.values) + (int64_t)cur.b * p.stride_values;
            // values of the first 128 entries, entries of the next stage, bounds of the one after: all in flight
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
            const Pos nn = locate(g + 2 * kStages);
            int nn_e0, nn_e1;
            bounds(nn, nn_e0, nn_e1);

            const uint32_t use = g / kStages;
            if (use > 0) ok_run = wait_or_abort<kSleepFill>(bar_empty + 8 * slot, (use - 1u) & 1u, abort_flag);
            if (!ok_run) break;
            VS_PROF_ADD(0);   // fill: prefetch issue + wait for the slot
            if (part == 0 && lane == 0) {   // the stage's rows of B: one 64 x 64 box per 64 columns of the tile
                const int slabs = (cur.tn + 63) >> 6;
                tc::mbar_expect_tx_only(bar, (uint32_t)slabs * kBSlabBytes);
                for (int s = 0; s < slabs; ++s)
                    tc::tma_load_3d(base + Smem::kB + slot * kBStageBytes + s * kBSlabBytes, &map_b, bar, cur.n0 + 64 * s,
                                    cur.kb * kBlockK, cur.b);
            }
            // zero this warp's 16 KiB of the A stage, then drop the nonzeros in
#pragma unroll
            for (int i = 0; i < (kGroupRows * kBlockK * 2) / (32 * 16); ++i)
                reinterpret_cast<uint4 *>(a_part)[i * 32 + lane] = make_uint4(0, 0, 0, 0);
            __syncwarp();
            VS_PROF_ADD(1);   // fill: B loads + zero fill
#pragma unroll
            for (int u = 0; u < kFillBatches; ++u)
                if (c_e0 + lane + 32 * u < c_e1)
                    scatter_vector<V>(a_part, c_ent[u].y, c_val[u].raw);
            for (int e = c_e0 + 32 * kFillBatches + lane; e < c_e1; e += 32) {   // buckets with more entries (denser rows)
                const uint2 ent = __ldg(blk_entries + e);
                ValueVec<V> val;
                val.load(vals + (int64_t)ent.x * V);
                scatter_vector<V>(a_part, ent.y, val.raw);
            }
            tc::fence_proxy_async();   // the tile was written by ordinary stores; the MMA reads through the async proxy
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(bar);

            cur = nxt; c_e0 = n_e0; c_e1 = n_e1;
#pragma unroll
            for (int u = 0; u < kFillBatches; ++u) c_ent[u] = n_ent[u];
            nxt = nn; n_e0 = nn_e0; n_e1 = nn_e1;
            VS_PROF_ADD(2);   // fill: scatter, arrive
        }
        VS_PROF_FLUSH(0);
    } else if (warp >= kMmaWarp) {
        // =========================== MMA issuers =========================================================
        // Thread h multiplies rows 128 h .. 128 h + 127 of the tile.  Both wait on every stage and both commit
        // to its `empty` barrier, so each has seen every earlier use of a slot complete.
        if (lane == 0) {
            const int h = warp - kMmaWarp;
            const uint32_t a_lo0 = tc::smem_desc_lo(base + Smem::kA + h * (128 * kBlockK * 2), 8192);   // 64-row atoms 8 KiB apart
            const uint32_t a_hi = tc::smem_desc_hi(1024, (uint32_t)tc::kSwizzle128B);
            const uint32_t b_lo0 = tc::smem_desc_lo(base + Smem::kB, kBSlabBytes);
            const uint32_t b_hi = tc::smem_desc_hi(1024, (uint32_t)tc::kSwizzle128B);
            uint32_t g = 0;
            bool ok_run = true;
            VS_PROF_T0();
            for (uint32_t i = 0; i < my_items && ok_run; ++i) {
                const Item it = decode_item(blockIdx.x + (int64_t)i * G, m_tiles, n_tiles, p.N);
                const uint32_t idesc = tc::make_idesc_f16(128, it.tn, 1, 1);   // both operands MN-major
                const uint32_t buf = i & 1u;
                if (i >= 2) ok_run = wait_or_abort<kSleepMma>(bar_acc_empty + 8 * buf, ((i >> 1) - 1u) & 1u, abort_flag);
                const uint32_t d = tmem_base + buf * kAccCols + (uint32_t)h * kTileN;
                VS_PROF_ADD(3);   // mma: item decode + wait for the accumulator
                for (int kb = 0; kb < k_blocks && ok_run; ++kb, ++g) {
                    const uint32_t slot = g % kStages;
                    ok_run = wait_or_abort<kSleepMma>(bar_full + 8 * slot, (g / kStages) & 1u, abort_flag);
                    if (!ok_run) break;
                    VS_PROF_ADD(4);   // mma: wait for the stage
                    tc::tc_fence_after_sync();
                    const uint32_t a_lo = a_lo0 + slot * (kAStageBytes >> 4), b_lo = b_lo0 + slot * (kBStageBytes >> 4);
                    const int n_k16 = min(kBlockK / 16, (p.K - kb * kBlockK + 15) >> 4);
#pragma unroll
                    for (int kk = 0; kk < kBlockK / 16; ++kk)
                        if (kk < n_k16)   // 16 columns of A = 16 rows of B = 2 KiB further on in either operand
                            tc::mma_f16_ss(d, tc::desc64(a_lo + 128 * kk, a_hi), tc::desc64(b_lo + 128 * kk, b_hi), idesc,
                                           (kb == 0 && kk == 0) ? 0u : 1u);
                    tc::mma_commit(bar_empty + 8 * slot);
                    VS_PROF_ADD(5);   // mma: issue
                }
                if (ok_run) tc::mma_commit(bar_acc_full + 8 * buf);
            }
            VS_PROF_FLUSH(3);
        }
    } else {
        // =========================== epilogue ============================================================
        bool ok_run = true;
        float finite_probe = 0.0f;
        const int quarter = warp & 3, half = warp >> 2;   // TMEM lanes 32 * quarter .. + 31; rows 128 * half .. of the tile
        uint8_t *stg = sm + Smem::kStaging + warp * kStoreBoxBytes;
        const uint32_t stg_u32 = base + Smem::kStaging + warp * kStoreBoxBytes;
        VS_PROF_T0();
        for (uint32_t i = 0; i < my_items && ok_run; ++i) {
            const Item it = decode_item(blockIdx.x + (int64_t)i * G, m_tiles, n_tiles, p.N);
            const uint32_t buf = i & 1u;
            // warp-uniform outcome: tcgen05.ld below needs all 32 lanes
            ok_run = __all_sync(0xffffffffu, wait_or_abort<kSleepEpilogue>(bar_acc_full + 8 * buf, (i >> 1) & 1u, abort_flag));
            if (!ok_run) break;
            VS_PROF_ADD(6);   // epilogue: wait for the accumulator
            tc::tc_fence_after_sync();
            // Each warp moves its 32 rows, 128 bytes of columns at a time, through a 4 KiB box of shared memory
            // (the 16-byte chunks XOR-swizzled by row so that the row-per-thread writes spread over the banks)
            // and lets TMA write them out as whole rows; the box is refilled once the previous store has read it.
            constexpr int kBoxCols = 128 / (int)sizeof(TOut);   // 64 fp16 or 32 fp32 columns
            const int row0 = it.mt * kTileM + half * 128 + quarter * 32;   // first row of this warp's boxes
#pragma unroll 1
            for (int c0 = 0; c0 < it.tn; c0 += kBoxCols) {
                uint32_t r[kBoxCols];
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * kAccCols + (uint32_t)(half * kTileN + c0);
                if constexpr (kBoxCols == 64) {
                    tc::tmem_ld_x32(taddr, reinterpret_cast<uint32_t(&)[32]>(r[0]));
                    tc::tmem_ld_x32(taddr + 32, reinterpret_cast<uint32_t(&)[32]>(r[32]));
                } else {
                    tc::tmem_ld_x32(taddr, r);
                }
                tc::tmem_ld_wait();
                if (row0 < m_rows && it.n0 + c0 < p.N) {   // warp-uniform
                    // x * 0 is 0 for a finite x and NaN otherwise: one FMA per element finds a non-finite sum
                    // (every column of the box was written by the MMA: columns past N multiply zero-filled B)
                    if (row0 + lane < m_rows) {
#pragma unroll
                        for (int e = 0; e < kBoxCols; ++e) finite_probe = fmaf(__uint_as_float(r[e]), 0.0f, finite_probe);
                    }
                    VS_PROF_ADD(6);
                    if (lane == 0) tc::bulk_wait_group_read<0>();   // the previous store has read the box
                    __syncwarp();
                    VS_PROF_ADD(7);
                    uint8_t *dst = stg + lane * 128;
#pragma unroll
                    for (int u = 0; u < 8; ++u) {   // eight 16-byte chunks per row
                        uint4 v;
                        if constexpr (sizeof(TOut) == 2) {
                            __half2 *hh = reinterpret_cast<__half2 *>(&v);
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                hh[e] = __floats2half2_rn(__uint_as_float(r[8 * u + 2 * e]), __uint_as_float(r[8 * u + 2 * e + 1]));
                        } else {
                            v = make_uint4(r[4 * u], r[4 * u + 1], r[4 * u + 2], r[4 * u + 3]);
                        }
                        *reinterpret_cast<uint4 *>(dst + ((u ^ (lane & 7)) << 4)) = v;
                    }
                    tc::fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        tc::tma_store_3d(&map_out, stg_u32, it.n0 + c0, row0, it.b);
                        tc::bulk_commit_group();
                    }
                    VS_PROF_ADD(8);
                }
            }
            tc::tc_fence_before_sync();
            tc::mbar_arrive(bar_acc_empty + 8 * buf);   // both halves are in registers or stored: the buffer is free
        }
        VS_PROF_FLUSH(6);
        // A zero of the densified tile times an Inf or NaN of B is a NaN that the reference, which only reads
        // the rows of B its nonzeros name, would not produce.  Any non-finite sum hands the call to the gather
        // kernel enqueued behind this one, which then overwrites the output.
        if (lane == 0) tc::bulk_wait_group<0>();   // every store of this warp has reached global memory
        if (__any_sync(0xffffffffu, finite_probe != 0.0f) && lane == 0) atomicExch(use_dense, 0);
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
