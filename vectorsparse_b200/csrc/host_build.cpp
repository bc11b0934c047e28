// Host side of the CVSE format: validator, row swizzle (load balancer), .smtx reader/writer, dense-mask
// converter, magnitude pruning of a dense weight and the seeded pattern / value generators.  Plain C++ on host arrays; no CUDA here.
//
// The reference keeps this logic inline in its drivers and in include/bm_test_utils.h:
//   .smtx parsing               spmm_benchmark.cpp:21-54, sddmm_benchmark.cpp:172-206
//   Identity/SortedRowSwizzle   include/bm_test_utils.h:196-215
//   MakeDenseMatrix             include/bm_test_utils.h:130-142
//   MakeSparseMatrixRandomUniform  include/bm_test_utils.h:70-127
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <numeric>
#include <string>
#include <vector>

#include "vsparse_b200.h"

#define VS_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

// ---- counter-based random numbers: value number `i` of stream `seed` is a pure function of (seed, i) -----
inline uint64_t mix64(uint64_t z) {
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

inline uint64_t stream_key(uint64_t seed, uint64_t stream) { return mix64(mix64(seed) ^ (stream * 0xd1342543de82ef95ull + 1)); }

struct Rng {
    uint64_t key, ctr;
    Rng(uint64_t seed, uint64_t stream) : key(stream_key(seed, stream)), ctr(0) {}
    uint64_t next() { return mix64(key + (ctr++) * 0x9e3779b97f4a7c15ull); }
    double uniform() { return (double)(next() >> 11) * (1.0 / 9007199254740992.0); }  // [0,1)
};

inline double counter_uniform(uint64_t key, uint64_t i) {
    return (double)(mix64(key + i * 0x9e3779b97f4a7c15ull) >> 11) * (1.0 / 9007199254740992.0);
}

// round-to-nearest-even float -> half bits
inline uint16_t f32_to_h16(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u, ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | ((ax > 0x7f800000u) ? 0x200u : 0));
    if (ax >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);
    if (ax < 0x33000001u) return (uint16_t)sign;
    int32_t e = (int32_t)(ax >> 23) - 127;
    uint32_t man = (ax & 0x7fffffu) | 0x800000u;
    if (e < -14) {
        int shift = -14 - e + 13;
        uint32_t q = man >> shift, rem = man & ((1u << shift) - 1u), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (q & 1u))) ++q;
        return (uint16_t)(sign | q);
    }
    uint32_t q = ((uint32_t)(e + 15) << 10) | ((man >> 13) & 0x3ffu), rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) ++q;
    return (uint16_t)(sign | q);
}

// Selection sampling: picks exactly `want` of the integers [0, total) in ascending order, each subset
// equally likely.  `emit(x)` is called for each pick.
template <typename F>
void sample_sorted(Rng &rng, int64_t total, int64_t want, F emit) {
    int64_t need = std::min(want, total);
    for (int64_t x = 0; x < total && need > 0; ++x) {
        if (rng.uniform() * (double)(total - x) < (double)need) {
            emit(x);
            --need;
        }
    }
}

int row_target(int n, double sparsity) {
    long t = std::lround((1.0 - sparsity) * (double)n);
    return (int)std::max(0l, std::min((long)n, t));
}

}  // namespace

VS_EXPORT const char *vs_error_string(int code) {
    switch (code) {
        case VS_OK: return "ok";
        case VS_ERR_VEC_LENGTH: return "Unsupported Vector Length!";
        case VS_ERR_DTYPE: return "unsupported element types for this path";
        case VS_ERR_SHAPE: return "size is negative or cannot be tiled by this path";
        case VS_ERR_NULL: return "null pointer";
        case VS_ERR_ALIGN: return "pointer or stride not 16-byte aligned";
        case VS_ERR_STRUCTURE: return "malformed CVSE structure";
        case VS_ERR_IO: return "file could not be read or written";
        case VS_ERR_ARG: return "invalid argument";
        case VS_ERR_DEVICE: return "a kernel gave up on a bounded wait";
        default: return code > 0 ? "CUDA runtime error" : "unknown error";
    }
}

VS_EXPORT const char *vs_version(void) { return "vsparse_b200 0.1 sm_100a"; }

VS_EXPORT int vs_cvse_validate(int m_vec, int n, int nonzeros_vec, const int32_t *row_offsets,
                               const int32_t *col_indices) {
    if (m_vec < 0 || n < 0 || nonzeros_vec < 0) return VS_ERR_SHAPE;
    if (!row_offsets || (nonzeros_vec > 0 && !col_indices)) return VS_ERR_NULL;
    if (row_offsets[0] != 0) return VS_ERR_STRUCTURE;
    for (int i = 0; i < m_vec; ++i)
        if (row_offsets[i + 1] < row_offsets[i]) return VS_ERR_STRUCTURE;
    if (row_offsets[m_vec] != nonzeros_vec) return VS_ERR_STRUCTURE;
    for (int j = 0; j < nonzeros_vec; ++j)
        if (col_indices[j] < 0 || col_indices[j] >= n) return VS_ERR_STRUCTURE;
    return VS_OK;
}

VS_EXPORT int vs_row_swizzle(int mode, int m_vec, const int32_t *row_offsets, int32_t *row_indices) {
    if (m_vec < 0) return VS_ERR_SHAPE;
    if (!row_indices || (mode == 1 && !row_offsets)) return VS_ERR_NULL;
    std::iota(row_indices, row_indices + m_vec, 0);
    if (mode == 0) return VS_OK;
    if (mode != 1) return VS_ERR_ARG;
    // Longest vector-rows first, so that the tail of a launch is made of short rows.  stable_sort on the
    // identity keeps ties in ascending index order, which makes the permutation reproducible.
    std::stable_sort(row_indices, row_indices + m_vec, [row_offsets](int32_t a, int32_t b) {
        return (row_offsets[a + 1] - row_offsets[a]) > (row_offsets[b + 1] - row_offsets[b]);
    });
    return VS_OK;
}

// ---- .smtx ------------------------------------------------------------------------------------------------

namespace {
// Reads the next integer, skipping spaces, commas and newlines.  Returns false at end of file / bad token.
bool next_int(FILE *f, long *out) {
    int c;
    do { c = std::fgetc(f); } while (c == ' ' || c == ',' || c == '\n' || c == '\r' || c == '\t');
    if (c == EOF) return false;
    bool neg = false;
    if (c == '-') { neg = true; c = std::fgetc(f); }
    if (c < '0' || c > '9') return false;
    long v = 0;
    while (c >= '0' && c <= '9') { v = v * 10 + (c - '0'); c = std::fgetc(f); }
    if (c != EOF) std::ungetc(c, f);
    *out = neg ? -v : v;
    return true;
}
}  // namespace

VS_EXPORT int vs_smtx_read_header(const char *path, int *rows, int *cols, int *nnz) {
    if (!path || !rows || !cols || !nnz) return VS_ERR_NULL;
    FILE *f = std::fopen(path, "r");
    if (!f) return VS_ERR_IO;
    long a, b, c;
    bool ok = next_int(f, &a) && next_int(f, &b) && next_int(f, &c);
    std::fclose(f);
    if (!ok || a < 0 || b < 0 || c < 0) return VS_ERR_IO;
    *rows = (int)a; *cols = (int)b; *nnz = (int)c;
    return VS_OK;
}

VS_EXPORT int vs_smtx_read(const char *path, int rows, int nnz, int32_t *row_offsets, int32_t *col_indices) {
    if (!path || !row_offsets || (nnz > 0 && !col_indices)) return VS_ERR_NULL;
    FILE *f = std::fopen(path, "r");
    if (!f) return VS_ERR_IO;
    long a, b, c, v;
    bool ok = next_int(f, &a) && next_int(f, &b) && next_int(f, &c) && a == rows && c == nnz;
    for (int i = 0; ok && i <= rows; ++i) { ok = next_int(f, &v); row_offsets[i] = (int32_t)v; }
    for (int j = 0; ok && j < nnz; ++j) { ok = next_int(f, &v); col_indices[j] = (int32_t)v; }
    std::fclose(f);
    if (!ok) return VS_ERR_IO;
    return vs_cvse_validate(rows, (int)b, nnz, row_offsets, col_indices);
}

VS_EXPORT int vs_smtx_write(const char *path, int rows, int cols, int nnz, const int32_t *row_offsets,
                            const int32_t *col_indices) {
    if (!path || !row_offsets || (nnz > 0 && !col_indices)) return VS_ERR_NULL;
    FILE *f = std::fopen(path, "w");
    if (!f) return VS_ERR_IO;
    std::fprintf(f, "%d, %d, %d\n", rows, cols, nnz);
    for (int i = 0; i <= rows; ++i) std::fprintf(f, i == rows ? "%d\n" : "%d ", row_offsets[i]);
    for (int j = 0; j < nnz; ++j) std::fprintf(f, j + 1 == nnz ? "%d" : "%d ", col_indices[j]);
    std::fprintf(f, "\n");
    return std::fclose(f) == 0 ? VS_OK : VS_ERR_IO;
}

VS_EXPORT int vs_cvse_from_dense_mask(int m_vec, int n, const uint8_t *mask, int32_t *row_offsets,
                                      int32_t *col_indices) {
    if (m_vec < 0 || n < 0) return VS_ERR_SHAPE;
    if (!mask || !row_offsets) return VS_ERR_NULL;
    int64_t off = 0;
    row_offsets[0] = 0;
    for (int i = 0; i < m_vec; ++i) {
        const uint8_t *row = mask + (size_t)i * n;
        for (int c = 0; c < n; ++c)
            if (row[c]) {
                if (col_indices) col_indices[off] = c;
                ++off;
            }
        if (off > INT32_MAX) return VS_ERR_SHAPE;
        row_offsets[i + 1] = (int32_t)off;
    }
    return (int)off;
}

// ---- structure of the transposed matrix -----------------------------------------------------------------------

VS_EXPORT int vs_cvse_transpose(int m_vec, int n, int nonzeros_vec, const int32_t *row_offsets,
                                const int32_t *col_indices, int32_t *t_offsets, int32_t *t_rows, int32_t *t_src) {
    if (m_vec < 0 || n < 0 || nonzeros_vec < 0) return VS_ERR_SHAPE;
    if (!row_offsets || !t_offsets || (nonzeros_vec > 0 && (!col_indices || !t_rows || !t_src))) return VS_ERR_NULL;
    const int rc = vs_cvse_validate(m_vec, n, nonzeros_vec, row_offsets, col_indices);
    if (rc != VS_OK) return rc;
    // counting sort by column; walking the vector-rows in order keeps each column's entries ascending in i
    std::vector<int32_t> cursor((size_t)n + 1, 0);
    for (int j = 0; j < nonzeros_vec; ++j) ++cursor[(size_t)col_indices[j] + 1];
    t_offsets[0] = 0;
    for (int c = 0; c < n; ++c) {
        cursor[c + 1] += cursor[c];
        t_offsets[c + 1] = cursor[c + 1];
    }
    for (int i = 0; i < m_vec; ++i)
        for (int j = row_offsets[i]; j < row_offsets[i + 1]; ++j) {
            const int32_t at = cursor[col_indices[j]]++;
            t_rows[at] = i;
            t_src[at] = j;
        }
    return VS_OK;
}

// ---- magnitude pruning of a dense weight ----------------------------------------------------------------------

VS_EXPORT int vs_cvse_prune_dense(int m_vec, int n, int vec_length, const float *weight, double sparsity, int scope,
                                  int32_t *row_offsets, int32_t *col_indices, float *values) {
    if (m_vec < 0 || n < 0) return VS_ERR_SHAPE;
    if (!weight || !row_offsets) return VS_ERR_NULL;
    if (!(sparsity >= 0.0 && sparsity <= 1.0) || (scope != 0 && scope != 1)) return VS_ERR_ARG;
    if (vec_length != 1 && vec_length != 2 && vec_length != 4 && vec_length != 8) return VS_ERR_VEC_LENGTH;
    const int V = vec_length;
    const int64_t slots = (int64_t)m_vec * n;
    if (slots > INT32_MAX) return VS_ERR_SHAPE;
    std::vector<double> score((size_t)slots);
    for (int i = 0; i < m_vec; ++i)
        for (int c = 0; c < n; ++c) {
            double s = 0.0;
            for (int v = 0; v < V; ++v) s += std::fabs((double)weight[((size_t)i * V + v) * n + c]);
            score[(size_t)i * n + c] = s;
        }
    std::vector<uint8_t> keep((size_t)slots, 0);
    std::vector<int32_t> order;
    // the `want` best slots of [lo, hi): by score descending, ties by ascending slot number
    auto mark_best = [&](int64_t lo, int64_t hi, int64_t want) {
        order.resize((size_t)(hi - lo));
        std::iota(order.begin(), order.end(), (int32_t)lo);
        want = std::min<int64_t>(want, hi - lo);
        auto better = [&](int32_t a, int32_t b) { return score[a] != score[b] ? score[a] > score[b] : a < b; };
        std::partial_sort(order.begin(), order.begin() + want, order.end(), better);
        for (int64_t q = 0; q < want; ++q) keep[order[q]] = 1;
    };
    if (scope == 0) {
        mark_best(0, slots, (int64_t)std::llround((1.0 - sparsity) * (double)slots));
    } else {
        const int64_t per_row = (int64_t)std::llround((1.0 - sparsity) * (double)n);
        for (int i = 0; i < m_vec; ++i) mark_best((int64_t)i * n, (int64_t)(i + 1) * n, per_row);
    }
    int64_t off = 0;
    row_offsets[0] = 0;
    for (int i = 0; i < m_vec; ++i) {
        for (int c = 0; c < n; ++c) {
            if (!keep[(size_t)i * n + c]) continue;
            if (col_indices) {
                col_indices[off] = c;
                if (values)
                    for (int v = 0; v < V; ++v) values[off * V + v] = weight[((size_t)i * V + v) * n + c];
            }
            ++off;
        }
        row_offsets[i + 1] = (int32_t)off;
    }
    return (int)off;
}

// ---- pattern generators -------------------------------------------------------------------------------------

VS_EXPORT int vs_cvse_generate(int kind, uint64_t seed, int m_vec, int n, int vec_length, double sparsity,
                               int band, int32_t *row_offsets, int32_t *col_indices) {
    if (m_vec < 0 || n < 0) return VS_ERR_SHAPE;
    if (!row_offsets) return VS_ERR_NULL;
    if (!(sparsity >= 0.0 && sparsity <= 1.0)) return VS_ERR_ARG;
    if (vec_length != 1 && vec_length != 2 && vec_length != 4 && vec_length != 8) return VS_ERR_VEC_LENGTH;
    int64_t off = 0;
    row_offsets[0] = 0;
    auto emit = [&](int64_t c) {
        if (col_indices) col_indices[off] = (int32_t)c;
        ++off;
    };

    if (kind == 0 || kind == 1) {
        for (int i = 0; i < m_vec; ++i) {
            Rng rng(seed, (uint64_t)i);
            int want;
            if (kind == 0) {
                want = row_target(n, sparsity);
            } else {
                // Beta(2,2) = the middle one of three uniforms; mean 1/2, so the mean density is 1-sparsity.
                double u[3] = {rng.uniform(), rng.uniform(), rng.uniform()};
                std::sort(u, u + 3);
                double d = std::min(1.0, std::max(0.0, 2.0 * (1.0 - sparsity) * u[1]));
                want = (int)std::lround(d * n);
            }
            sample_sorted(rng, n, want, emit);
            row_offsets[i + 1] = (int32_t)off;
        }
    } else if (kind == 2) {
        int64_t total = (int64_t)m_vec * n;
        int64_t want = std::llround((double)total * (1.0 - sparsity));
        Rng rng(seed, 0);
        int64_t need = std::min(want, total);
        for (int i = 0; i < m_vec; ++i) {
            for (int c = 0; c < n; ++c) {
                int64_t x = (int64_t)i * n + c;
                if (need > 0 && rng.uniform() * (double)(total - x) < (double)need) {
                    emit(c);
                    --need;
                }
            }
            if (off > INT32_MAX) return VS_ERR_SHAPE;
            row_offsets[i + 1] = (int32_t)off;
        }
    } else if (kind == 3) {
        if (band < 0 || band > n) return VS_ERR_ARG;
        const int lattice = 16;
        std::vector<int32_t> row;
        std::vector<uint8_t> taken((size_t)n);
        for (int i = 0; i < m_vec; ++i) {
            Rng rng(seed, (uint64_t)i);
            int want = std::max(row_target(n, sparsity), band);
            std::fill(taken.begin(), taken.end(), 0);
            // the band: `band` columns around the diagonal position of this vector-row, shifted to stay inside
            int64_t centre = (int64_t)i * vec_length + vec_length / 2;
            int64_t lo = centre - band / 2;
            lo = std::max<int64_t>(0, std::min<int64_t>(lo, (int64_t)n - band));
            for (int64_t c = lo; c < lo + band; ++c) taken[(size_t)c] = 1;
            int need = want - band;
            // strided part: a per-row phase on a stride-16 lattice, outside the band
            int phase = (int)(rng.next() % lattice);
            std::vector<int32_t> cand;
            for (int c = phase; c < n; c += lattice)
                if (!taken[(size_t)c]) cand.push_back(c);
            int from_lattice = std::min<int>(need, (int)cand.size());
            sample_sorted(rng, (int64_t)cand.size(), from_lattice, [&](int64_t t) { taken[(size_t)cand[(size_t)t]] = 1; });
            need -= from_lattice;
            if (need > 0) {  // lattice exhausted: fill from every remaining column
                std::vector<int32_t> rest;
                for (int c = 0; c < n; ++c)
                    if (!taken[(size_t)c]) rest.push_back(c);
                sample_sorted(rng, (int64_t)rest.size(), need, [&](int64_t t) { taken[(size_t)rest[(size_t)t]] = 1; });
            }
            for (int c = 0; c < n; ++c)
                if (taken[(size_t)c]) emit(c);
            row_offsets[i + 1] = (int32_t)off;
        }
    } else {
        return VS_ERR_ARG;
    }
    if (off > INT32_MAX) return VS_ERR_SHAPE;
    return (int)off;
}

VS_EXPORT int vs_fill_random(int dtype, int dist, uint64_t seed, double sigma, int64_t count, void *out) {
    if (count < 0) return VS_ERR_SHAPE;
    if (!out && count > 0) return VS_ERR_NULL;
    if (dtype != VS_F16 && dtype != VS_F32) return VS_ERR_DTYPE;
    if (dist != 0 && dist != 1) return VS_ERR_ARG;
    const uint64_t key = stream_key(seed, 0x76616c75ull /* "valu" */);
    float *of = (float *)out;
    uint16_t *oh = (uint16_t *)out;
    for (int64_t i = 0; i < count; ++i) {
        float x;
        if (dist == 0) {
            x = (float)(2.0 * counter_uniform(key, (uint64_t)i) - 1.0);
            if (x >= 1.0f) x = std::nextafterf(1.0f, 0.0f);
        } else {
            // Box-Muller on the counter pair (2p, 2p+1); element i takes the cosine or sine branch
            uint64_t p = (uint64_t)i >> 1;
            double u1 = 1.0 - counter_uniform(key, 2 * p);  // (0,1]
            double u2 = counter_uniform(key, 2 * p + 1);
            double r = std::sqrt(-2.0 * std::log(u1));
            double a = 6.283185307179586476925286766559 * u2;
            x = (float)(sigma * r * ((i & 1) ? std::sin(a) : std::cos(a)));
        }
        if (dtype == VS_F32) of[i] = x;
        else oh[i] = f32_to_h16(x);
    }
    return VS_OK;
}
