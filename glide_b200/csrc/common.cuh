// Shared device primitives: team distance, register bitonic network, visited set.
//
// Semantics follow the reference (file:line relative to its src/ directory); the
// thread mapping does not: the reference runs one CTA per query with one warp per
// candidate row, here one WARP owns a query (or graph point) end to end and splits
// into four 8-lane teams that each stream one row with 128-bit loads.
#pragma once

#include <cfloat>
#include <cstdint>
#include <cuda_runtime.h>

namespace glide {

constexpr uint32_t kInvalid = 0xffffffffu;   // empty slot / no id (utils.cuh:52-55)
constexpr uint32_t kExplored = 0x80000000u;  // id MSB = "already expanded" (utils.cuh:5-8)
constexpr uint32_t kClean = ~kExplored;
constexpr uint32_t kPadClean = kInvalid & kClean;  // an unfilled beam slot after the flag is cleared
constexpr uint32_t kFullMask = 0xffffffffu;
constexpr int kTeam = 8;                     // lanes per team
constexpr int kTeamsPerWarp = 32 / kTeam;

enum Metric : int { kEuclidean = 0, kCosine = 1 };  // params.cuh:5-8

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31u; }

// ---------------------------------------------------------------------------
// Distance. The value is the reference's (distance.cuh:9-27): fp32 sum of squared
// differences, sqrt for Euclidean, raw for Cosine. Two summation orders are used. Centroid
// distances (routing, assignment, k-means) use the TEAM order: team lane t accumulates 4-float chunks t, t+8, ... with fused
// multiply-adds (scalar elements t, t+8, ... when dim % 4 != 0), then a 4,2,1
// shuffle tree folds the team. All lanes of the team return the folded value.
// `q` points to shared memory (16-byte aligned), `row` to global memory.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float team_fold(float acc) {
    acc += __shfl_down_sync(kFullMask, acc, 4, kTeam);
    acc += __shfl_down_sync(kFullMask, acc, 2, kTeam);
    acc += __shfl_down_sync(kFullMask, acc, 1, kTeam);
    return __shfl_sync(kFullMask, acc, 0, kTeam);
}

__device__ __forceinline__ float sq_acc4(const float4 a, const float4 b, float acc) {
    float d;
    d = a.x - b.x; acc = __fmaf_rn(d, d, acc);
    d = a.y - b.y; acc = __fmaf_rn(d, d, acc);
    d = a.z - b.z; acc = __fmaf_rn(d, d, acc);
    d = a.w - b.w; acc = __fmaf_rn(d, d, acc);
    return acc;
}

// Partial sum of one team lane. active == false lanes read nothing.
__device__ __forceinline__ float team_partial(const float *__restrict__ q, const float *__restrict__ row,
                                              uint32_t dim, bool active) {
    const uint32_t t = threadIdx.x & (kTeam - 1);
    float acc = 0.0f;
    if (!active) return acc;
    if ((dim & 3u) == 0) {
        const uint32_t chunks = dim >> 2;
        const float4 *q4 = reinterpret_cast<const float4 *>(q);
        const float4 *r4 = reinterpret_cast<const float4 *>(row);
        uint32_t c = t;
        // four independent 16-byte loads in flight per lane
        for (; c + 3 * kTeam < chunks; c += 4 * kTeam) {
            const float4 b0 = __ldg(r4 + c);
            const float4 b1 = __ldg(r4 + c + kTeam);
            const float4 b2 = __ldg(r4 + c + 2 * kTeam);
            const float4 b3 = __ldg(r4 + c + 3 * kTeam);
            acc = sq_acc4(q4[c], b0, acc);
            acc = sq_acc4(q4[c + kTeam], b1, acc);
            acc = sq_acc4(q4[c + 2 * kTeam], b2, acc);
            acc = sq_acc4(q4[c + 3 * kTeam], b3, acc);
        }
        for (; c < chunks; c += kTeam) acc = sq_acc4(q4[c], __ldg(r4 + c), acc);
    } else {
        for (uint32_t i = t; i < dim; i += kTeam) {
            const float d = q[i] - __ldg(row + i);
            acc = __fmaf_rn(d, d, acc);
        }
    }
    return acc;
}

// ---------------------------------------------------------------------------
// Warp-row distances (candidate scoring and pruning). One data row is read by the whole
// warp: lane l owns the 16-byte chunks l, l+32, ... of the row (for dim 128 exactly one
// 128-bit load per lane and row), accumulates its chunks with fused multiply-adds in
// x,y,z,w order, and the 32 lane sums are folded by a 16,8,4,2,1 xor tree, the reference's
// tree (distance.cuh:18-20). When dim % 4 != 0 lane l owns the scalar elements l, l+32, ...,
// which is exactly the reference's order (distance.cuh:15-17). The query stays in
// registers, R = 8/QR rows are loaded before any is consumed, and the R lane sums are
// folded together: each xor step that still has several rows halves the values per lane
// instead of shuffling all of them (9 shuffles for 8 rows instead of 40). The pairing of
// lanes, hence the rounding, is that of the plain tree.
// ---------------------------------------------------------------------------
template<int R>
__device__ __forceinline__ float fold_rows(float (&p)[R]) {
    const uint32_t lane = lane_id();
    int bit = 16;
#pragma unroll
    for (int half = R / 2; half >= 1; half >>= 1) {
        const bool hi = (lane & bit) != 0;
#pragma unroll
        for (int i = 0; i < half; i++) {
            const float send = hi ? p[i] : p[i + half];
            const float keep = hi ? p[i + half] : p[i];
            p[i] = keep + __shfl_xor_sync(kFullMask, send, bit);
        }
        bit >>= 1;
    }
#pragma unroll
    for (; bit >= 1; bit >>= 1) p[0] += __shfl_xor_sync(kFullMask, p[0], bit);
    return p[0];  // the sum of row (lane >> (5 - log2 R)), replicated over 32/R lanes
}

template<int R> struct Log2 { static constexpr int v = 1 + Log2<R / 2>::v; };
template<> struct Log2<1> { static constexpr int v = 0; };

// id_at(i) -> row id of the i-th row to score (i < n); sink(i, distance) consumes it (called
// by one lane per row). QR = number of 16-byte chunks each lane owns (dim <= 128*QR).
template<int QR, typename IdAt, typename Sink>
__device__ __forceinline__ void warp_rows_v4(const float *q_smem, const float *__restrict__ data, uint32_t dim,
                                             int metric, uint32_t n, IdAt id_at, Sink sink) {
    constexpr int R = 8 / QR;
    const uint32_t lane = lane_id();
    const uint32_t chunks = dim >> 2;
    float4 q[QR];
#pragma unroll
    for (int j = 0; j < QR; j++) {
        const uint32_t c = lane + 32u * j;
        q[j] = (c < chunks) ? reinterpret_cast<const float4 *>(q_smem)[c] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (uint32_t g = 0; g < n; g += R) {
        float4 v[R][QR];
#pragma unroll
        for (int r = 0; r < R; r++) {
            const bool act = g + r < n;
            const uint32_t id = act ? id_at(g + r) : 0u;
            const float4 *row4 = reinterpret_cast<const float4 *>(data + (uint64_t) id * dim);
#pragma unroll
            for (int j = 0; j < QR; j++) {
                const uint32_t c = lane + 32u * j;
                v[r][j] = (act && c < chunks) ? __ldg(row4 + c) : q[j];  // q - q adds exactly nothing
            }
        }
        float p[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < QR; j++) acc = sq_acc4(q[j], v[r][j], acc);
            p[r] = acc;
        }
        const float sum = fold_rows<R>(p);
        const uint32_t my_row = lane >> (5 - Log2<R>::v);
        if ((lane & (32 / R - 1)) == 0 && g + my_row < n) sink(g + my_row, metric == kEuclidean ? sqrtf(sum) : sum);
    }
}

// Lane partial sum of one row for any dim. dim % 4 == 0: the chunk ownership of warp_rows_v4;
// otherwise scalar elements l, l+32, ... (the reference's order).
__device__ __forceinline__ float lane_row_partial(const float *q_smem, const float *__restrict__ row, uint32_t dim) {
    const uint32_t lane = lane_id();
    float acc = 0.0f;
    if ((dim & 3u) == 0) {
        const float4 *q4 = reinterpret_cast<const float4 *>(q_smem);
        const float4 *r4 = reinterpret_cast<const float4 *>(row);
        const uint32_t chunks = dim >> 2;
        // eight 16-byte loads in flight per lane (a 960-dim row is 7.5 of them), accumulated in chunk order
        for (uint32_t c = lane; c < chunks; c += 256) {
            float4 b[8];
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const uint32_t ck = c + 32u * k;
                b[k] = ck < chunks ? __ldg(r4 + ck) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const uint32_t ck = c + 32u * k;
                if (ck < chunks) acc = sq_acc4(q4[ck], b[k], acc);
            }
        }
    } else {
        for (uint32_t i = lane; i < dim; i += 32) {
            const float d = q_smem[i] - __ldg(row + i);
            acc = __fmaf_rn(d, d, acc);
        }
    }
    return acc;
}

// Any dim: one row at a time.
template<typename IdAt, typename Sink>
__device__ __forceinline__ void warp_rows_generic(const float *q_smem, const float *__restrict__ data, uint32_t dim,
                                                  int metric, uint32_t n, IdAt id_at, Sink sink) {
    const uint32_t lane = lane_id();
    for (uint32_t g = 0; g < n; g++) {
        float p[1] = {lane_row_partial(q_smem, data + (uint64_t) id_at(g) * dim, dim)};
        const float sum = fold_rows<1>(p);
        if (lane == 0) sink(g, metric == kEuclidean ? sqrtf(sum) : sum);
    }
}

template<typename IdAt, typename Sink>
__device__ __forceinline__ void warp_rows(const float *q_smem, const float *__restrict__ data, uint32_t dim, int metric,
                                          uint32_t n, IdAt id_at, Sink sink) {
    // register budget (a third variant pushes the search kernels from 64 to 100 registers):
    // the query-in-registers path serves dim <= 128, wider rows stream chunk by chunk against
    // the query in shared memory
    if ((dim & 3u) == 0 && dim <= 128) warp_rows_v4<1>(q_smem, data, dim, metric, n, id_at, sink);
    else warp_rows_generic(q_smem, data, dim, metric, n, id_at, sink);
}

// Lane-resident scoring: lane l holds candidate id `cv` (scored when bit l of `mask` is set) and
// receives its distance; other lanes get FLT_MAX. The ids travel by shuffle, the rows are read by
// the whole warp exactly as in warp_rows (same chunk ownership, same fold), so the distances are
// bit-identical to the shared-memory path; nothing is staged in shared memory.
// Fast path of score_lanes: dim % 4 == 0 and dim <= 128, the query chunk of this lane in `q`
// (zero when the lane owns no chunk).
// ids_smem: 40 words of per-warp scratch, or nullptr. With scratch the ids are first written in rank
// order (one store per lane), so that the batch loop reads each id with one broadcast load instead of
// finding, shuffling and selecting it.
__device__ __forceinline__ float score_lanes_q4(const float4 q, bool own, const float *__restrict__ data, uint32_t dim,
                                                int metric, uint32_t mask, uint32_t cv, uint32_t *ids_smem = nullptr) {
    const uint32_t lane = lane_id();
    float mine = FLT_MAX;
    uint32_t m = mask;
    const uint32_t my_rank = __popc(mask & ((1u << lane) - 1));
    const bool valid = ((mask >> lane) & 1u) != 0;
    const bool all_own = dim == 128;   // every lane owns a chunk: loads need no predicate
    if (ids_smem != nullptr) {
        const uint32_t n = __popc(mask);
        if (valid) ids_smem[my_rank] = cv;
        if (lane < 8) ids_smem[n + lane] = 0u;   // slots past the last row of a ragged batch re-read row 0
        __syncwarp();
        if (all_own) {   // constant row pitch, every lane owns a chunk
            for (uint32_t g = 0; 8u * g < n; g++) {
                float4 v[8];
#pragma unroll
                for (int r = 0; r < 8; r++)
                    v[r] = __ldg(reinterpret_cast<const float4 *>(data + (uint64_t) ids_smem[8u * g + r] * 128u) + lane);
                float p[8];
#pragma unroll
                for (int r = 0; r < 8; r++) p[r] = sq_acc4(q, v[r], 0.0f);
                const float sum = fold_rows<8>(p);  // row r of the batch sits in lanes 4r .. 4r+3
                const float got = __shfl_sync(kFullMask, sum, (my_rank & 7u) * 4u);
                mine = (valid && (my_rank >> 3) == g) ? got : mine;
            }
        } else {
            const uint32_t my_chunk = own ? lane : 0u;   // lanes without a chunk re-read chunk 0 and contribute nothing
            for (uint32_t g = 0; 8u * g < n; g++) {
                float4 v[8];
#pragma unroll
                for (int r = 0; r < 8; r++)
                    v[r] = __ldg(reinterpret_cast<const float4 *>(data + (uint64_t) ids_smem[8u * g + r] * dim) + my_chunk);
                float p[8];
#pragma unroll
                for (int r = 0; r < 8; r++) p[r] = own ? sq_acc4(q, v[r], 0.0f) : 0.0f;
                const float sum = fold_rows<8>(p);
                const float got = __shfl_sync(kFullMask, sum, (my_rank & 7u) * 4u);
                mine = (valid && (my_rank >> 3) == g) ? got : mine;
            }
        }
        __syncwarp();
        if (metric == kEuclidean) mine = valid ? sqrtf(mine) : mine;
        return mine;
    }
    for (uint32_t g = 0; m != 0; g++) {
        float4 v[8];
        if (all_own) {
            // slots past the last row of a ragged batch re-read row 0 (their sums are never delivered):
            // cheaper than predicating eight 128-bit loads and pre-setting their registers
#pragma unroll
            for (int r = 0; r < 8; r++) {
                const bool act = m != 0;
                const uint32_t src = act ? (uint32_t) __ffs(m) - 1u : 0u;
                m &= m - 1u;
                const uint32_t got_id = __shfl_sync(kFullMask, cv, src);
                const uint32_t id = act ? got_id : 0u;
                v[r] = __ldg(reinterpret_cast<const float4 *>(data + (uint64_t) id * 128u) + lane);
            }
        } else {
            // lanes without a chunk of their own re-read chunk 0 and contribute nothing
            const uint32_t my_chunk = own ? lane : 0u;
#pragma unroll
            for (int r = 0; r < 8; r++) {
                const bool act = m != 0;
                const uint32_t src = act ? (uint32_t) __ffs(m) - 1u : 0u;
                m &= m - 1u;
                const uint32_t got_id = __shfl_sync(kFullMask, cv, src);
                const uint32_t id = act ? got_id : 0u;
                v[r] = __ldg(reinterpret_cast<const float4 *>(data + (uint64_t) id * dim) + my_chunk);
            }
        }
        float p[8];
        if (all_own) {
#pragma unroll
            for (int r = 0; r < 8; r++) p[r] = sq_acc4(q, v[r], 0.0f);
        } else {
#pragma unroll
            for (int r = 0; r < 8; r++) p[r] = own ? sq_acc4(q, v[r], 0.0f) : 0.0f;
        }
        const float sum = fold_rows<8>(p);  // row r of the batch sits in lanes 4r .. 4r+3
        const float got = __shfl_sync(kFullMask, sum, (my_rank & 7u) * 4u);
        mine = (valid && (my_rank >> 3) == g) ? got : mine;
    }
    if (metric == kEuclidean) mine = valid ? sqrtf(mine) : mine;  // once per lane, no branch per batch
    return mine;
}

__device__ __forceinline__ bool rows_fit_lanes(uint32_t dim) { return (dim & 3u) == 0 && dim <= 128; }

__device__ __forceinline__ float score_lanes(const float *q_smem, const float *__restrict__ data, uint32_t dim,
                                             int metric, uint32_t mask, uint32_t cv, uint32_t *ids_smem = nullptr) {
    const uint32_t lane = lane_id();
    if (rows_fit_lanes(dim)) {
        const bool own = lane < (dim >> 2);
        const float4 q = own ? reinterpret_cast<const float4 *>(q_smem)[lane] : make_float4(0.f, 0.f, 0.f, 0.f);
        return score_lanes_q4(q, own, data, dim, metric, mask, cv, ids_smem);
    }
    float mine = FLT_MAX;
    uint32_t m = mask;
    while (m != 0) {
        const uint32_t src = (uint32_t) __ffs(m) - 1u;
        m &= m - 1u;
        const uint32_t id = __shfl_sync(kFullMask, cv, src);
        float p[1] = {lane_row_partial(q_smem, data + (uint64_t) id * dim, dim)};
        const float sum = fold_rows<1>(p);
        if (lane == src) mine = metric == kEuclidean ? sqrtf(sum) : sum;
    }
    return mine;
}

__device__ __forceinline__ float finish_metric(float s, int metric) {
    return metric == kEuclidean ? sqrtf(s) : s;
}

// ---------------------------------------------------------------------------
// Register-resident warp bitonic network over 32*N (key,value) pairs; element
// index e = N*lane + i. The comparator never exchanges equal keys, and the
// sequence of comparators is the textbook bitonic sort on e, which is what the
// reference's network computes (bitonic.cuh:24-44, :46-85, :202-212), so equal
// keys end up in the same slots as there.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void cx_regs(float &k0, uint32_t &v0, float &k1, uint32_t &v1, bool asc) {
    // min/max keep equal keys where they are (no exchange on a tie), like the reference's
    // swap_if_needed (bitonic.cuh:24-33); the values follow their keys.
    const float lo = fminf(k0, k1), hi = fmaxf(k0, k1);
    const float n0 = asc ? lo : hi;
    const bool moved = (n0 != k0);
    const uint32_t t0 = moved ? v1 : v0, t1 = moved ? v0 : v1;
    k1 = asc ? hi : lo;
    k0 = n0;
    v0 = t0;
    v1 = t1;
}

template<int N>
__device__ __forceinline__ void cx_lanes(float (&k)[N], uint32_t (&v)[N], uint32_t lane_xor, bool keep_small) {
#pragma unroll
    for (int i = 0; i < N; i++) {
        const float ok = __shfl_xor_sync(kFullMask, k[i], lane_xor);
        const uint32_t ov = __shfl_xor_sync(kFullMask, v[i], lane_xor);
        // keep the smaller (or larger) key; on a tie the own pair stays (bitonic.cuh:35-44)
        const float nk = keep_small ? fminf(k[i], ok) : fmaxf(k[i], ok);
        v[i] = (nk != k[i]) ? ov : v[i];
        k[i] = nk;
    }
}

// One merge phase producing sorted runs of SIZE elements (SIZE >= 2N means cross-lane
// strides). Ascending where (e & SIZE) == 0, or everywhere in the final phase. Every
// bound is a compile-time constant so the whole network unrolls into straight-line code.
template<int N, int SIZE, bool FINAL>
__device__ __forceinline__ void bitonic_phase(float (&k)[N], uint32_t (&v)[N]) {
    const uint32_t lane = lane_id();
    // cross-lane strides: SIZE/2 ... N  (lane stride = stride / N)
#pragma unroll
    for (int stride = SIZE / 2; stride >= N; stride >>= 1) {
        const uint32_t ls = stride / N;
        const bool asc = FINAL || (((N * lane) & SIZE) == 0);
        const bool lower = (lane & ls) == 0;
        cx_lanes<N>(k, v, ls, lower == asc);
    }
    // in-register strides: min(SIZE/2, N/2) ... 1
#pragma unroll
    for (int stride = (SIZE / 2 < N / 2 ? SIZE / 2 : N / 2); stride >= 1; stride >>= 1) {
#pragma unroll
        for (int i = 0; i < N; i++) {
            const int j = i ^ stride;
            if (i < j) {
                const uint32_t e = N * lane + i;
                const bool asc = FINAL || ((e & SIZE) == 0);
                cx_regs(k[i], v[i], k[j], v[j], asc);
            }
        }
    }
}

template<int N, int SIZE>
struct BitonicSortFrom {
    static __device__ __forceinline__ void run(float (&k)[N], uint32_t (&v)[N]) {
        bitonic_phase<N, SIZE, SIZE == 32 * N>(k, v);
        if constexpr (SIZE < 32 * N) BitonicSortFrom<N, SIZE * 2>::run(k, v);
    }
};

template<int N>
__device__ __forceinline__ void warp_sort(float (&k)[N], uint32_t (&v)[N]) {
    BitonicSortFrom<N, 2>::run(k, v);
}

// Last phase only: input must be bitonic over e (bitonic.cuh warp_merge, range 32).
template<int N>
__device__ __forceinline__ void warp_merge_final(float (&k)[N], uint32_t (&v)[N]) {
    bitonic_phase<N, 32 * N, true>(k, v);
}

// Same network on a shared-memory array of 32*n pairs, n a runtime power of two.
// Used where the width is only known at run time (centroid lists).
__device__ inline void warp_sort_smem(float *k, uint32_t *v, uint32_t n_per_lane) {
    const uint32_t total = 32u * n_per_lane, lane = lane_id();
    for (uint32_t size = 2; size <= total; size <<= 1) {
        for (uint32_t stride = size >> 1; stride >= 1; stride >>= 1) {
            for (uint32_t p = lane; p < total / 2; p += 32) {
                const uint32_t lo = ((p / stride) * 2 * stride) + (p % stride);
                const uint32_t hi = lo + stride;
                const bool asc = (size == total) || ((lo & size) == 0);
                const float k0 = k[lo], k1 = k[hi];
                if ((k0 != k1) && ((k0 < k1) != asc)) {
                    k[lo] = k1; k[hi] = k0;
                    const uint32_t t = v[lo]; v[lo] = v[hi]; v[hi] = t;
                }
            }
            __syncwarp();
        }
    }
}

// ---------------------------------------------------------------------------
// Visited set in shared memory, one per warp, in one of two forms chosen by the host:
//   hash    open addressing, linear probing: same slot function and "full table reports seen"
//           rule as hashmap.cuh:33-56. `bits` is the table's size exponent.
//   bitmap  one bit per id, for searches whose ids are partition-local and few enough (the
//           subgraph build). `bits` carries the number of bitmap words above bit 8. The host
//           picks it only when the table of the hash form could never fill up between two
//           resets, so that both forms answer every insert alike; one shared-memory atomic per
//           lane replaces the probe rounds.
// ---------------------------------------------------------------------------
__host__ __device__ inline uint32_t visited_words(uint32_t bits) { return (bits >> 8) ? (bits >> 8) : (1u << bits); }

__device__ __forceinline__ void visited_clear(uint32_t *table, uint32_t bits) {
    const uint32_t words = visited_words(bits), fill = (bits >> 8) ? 0u : kInvalid;
    for (uint32_t i = lane_id(); i < words; i += 32) table[i] = fill;
}

// Called by the whole warp; lanes with want == false only keep the others company. The probe
// loop runs in lockstep (its trip count is the longest probe chain among the lanes), so the warp
// leaves it converged: a per-lane loop with early exits left the lanes split for the code that
// follows, which doubled the row-load instructions of the scoring step.
__device__ __forceinline__ uint32_t visited_insert(uint32_t *table, uint32_t bits, uint32_t key, bool want) {
    if (bits >> 8) {   // bitmap; an id beyond the map (a corrupt adjacency row) is reported as seen
        uint32_t result = 0;
        if (want && (key >> 5) < (bits >> 8)) {
            const uint32_t b = 1u << (key & 31u);
            result = (atomicOr(&table[key >> 5], b) & b) ? 0u : 1u;
        }
        __syncwarp();
        return result;
    }
    const uint32_t size = 1u << bits, mask = size - 1;
    uint32_t index = (key ^ (key >> bits)) & mask;
    uint32_t result = 0, left = size;
    bool pending = want;
    while (__any_sync(kFullMask, pending)) {
        if (pending) {
            const uint32_t old = atomicCAS(&table[index], kInvalid, key);
            result = (old == kInvalid) ? 1u : 0u;
            left--;
            pending = !(old == kInvalid || old == key || left == 0);
            index = (index + 1) & mask;
        }
    }
    return result;
}

typedef unsigned long long u64;

// ---- u64 bitonic network, N keys per lane, position e = N*lane + i -------------
template<int N, int SIZE, bool FINAL>
__device__ __forceinline__ void phase_u64_t(u64 (&k)[N]) {
    const uint32_t lane = lane_id();
#pragma unroll
    for (int stride = SIZE / 2; stride >= N; stride >>= 1) {
        const uint32_t ls = stride / N;
        const bool asc = FINAL || (((N * lane) & SIZE) == 0);
        const bool keep_small = ((lane & ls) == 0) == asc;
#pragma unroll
        for (int i = 0; i < N; i++) {
            const u64 o = __shfl_xor_sync(kFullMask, k[i], ls);
            if (keep_small ? (o < k[i]) : (o > k[i])) k[i] = o;
        }
    }
#pragma unroll
    for (int stride = (SIZE / 2 < N / 2 ? SIZE / 2 : N / 2); stride >= 1; stride >>= 1) {
#pragma unroll
        for (int i = 0; i < N; i++) {
            const int j = i ^ stride;
            if (i < j) {
                const bool asc = FINAL || (((N * lane + i) & SIZE) == 0);
                const u64 a = k[i], b = k[j];
                if ((a > b) == asc && a != b) { k[i] = b; k[j] = a; }
            }
        }
    }
}
template<int N, int SIZE>
struct SortU64From {
    static __device__ __forceinline__ void run(u64 (&k)[N]) {
        phase_u64_t<N, SIZE, SIZE == 32 * N>(k);
        if constexpr (SIZE < 32 * N) SortU64From<N, SIZE * 2>::run(k);
    }
};
template<int N>
__device__ __forceinline__ void sort_u64(u64 (&k)[N]) { SortU64From<N, 2>::run(k); }
// final merge phase of a bitonic sequence of 32*N keys
template<int N>
__device__ __forceinline__ void merge_final_u64(u64 (&k)[N]) { phase_u64_t<N, 32 * N, true>(k); }

__host__ __device__ constexpr uint32_t round_up32(uint32_t x) { return (x + 31u) & ~31u; }

}  // namespace glide
