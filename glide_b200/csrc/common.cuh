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
// differences, sqrt for Euclidean, raw for Cosine. The summation ORDER is this
// repository's own: team lane t accumulates 4-float chunks t, t+8, ... with fused
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

// Two rows at once (same arithmetic per row as team_partial): the loads of both rows are
// issued before either is consumed.
__device__ __forceinline__ void team_partial2(const float *__restrict__ q, const float *__restrict__ row0,
                                              const float *__restrict__ row1, uint32_t dim, bool active0,
                                              bool active1, float &out0, float &out1) {
    const uint32_t t = threadIdx.x & (kTeam - 1);
    float acc0 = 0.0f, acc1 = 0.0f;
    if (active0 && active1 && (dim & 3u) == 0) {
        const uint32_t chunks = dim >> 2;
        const float4 *q4 = reinterpret_cast<const float4 *>(q);
        const float4 *r4 = reinterpret_cast<const float4 *>(row0);
        const float4 *s4 = reinterpret_cast<const float4 *>(row1);
        uint32_t c = t;
        for (; c + kTeam < chunks; c += 2 * kTeam) {
            const float4 b0 = __ldg(r4 + c), b1 = __ldg(r4 + c + kTeam);
            const float4 d0 = __ldg(s4 + c), d1 = __ldg(s4 + c + kTeam);
            const float4 qa = q4[c], qb = q4[c + kTeam];
            acc0 = sq_acc4(qa, b0, acc0); acc1 = sq_acc4(qa, d0, acc1);
            acc0 = sq_acc4(qb, b1, acc0); acc1 = sq_acc4(qb, d1, acc1);
        }
        for (; c < chunks; c += kTeam) {
            const float4 b = __ldg(r4 + c), d = __ldg(s4 + c);
            const float4 qa = q4[c];
            acc0 = sq_acc4(qa, b, acc0);
            acc1 = sq_acc4(qa, d, acc1);
        }
    } else {
        acc0 = team_partial(q, row0, dim, active0);
        acc1 = team_partial(q, row1, dim, active1);
    }
    out0 = acc0;
    out1 = acc1;
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
    if ((k0 != k1) && ((k0 < k1) != asc)) {
        const float tk = k0; k0 = k1; k1 = tk;
        const uint32_t tv = v0; v0 = v1; v1 = tv;
    }
}

template<int N>
__device__ __forceinline__ void cx_lanes(float (&k)[N], uint32_t (&v)[N], uint32_t lane_xor, bool keep_small) {
#pragma unroll
    for (int i = 0; i < N; i++) {
        const float ok = __shfl_xor_sync(kFullMask, k[i], lane_xor);
        const uint32_t ov = __shfl_xor_sync(kFullMask, v[i], lane_xor);
        if ((k[i] != ok) && ((k[i] < ok) != keep_small)) {
            k[i] = ok;
            v[i] = ov;
        }
    }
}

// One merge phase producing sorted runs of `run` = size elements (size >= 2N means
// cross-lane strides). asc decided per element by (e & size) == 0, or always for
// the final phase.
template<int N>
__device__ __forceinline__ void bitonic_phase(float (&k)[N], uint32_t (&v)[N], uint32_t size, bool final_phase) {
    const uint32_t lane = lane_id();
    // cross-lane strides: size/2 ... N  (lane stride = stride / N)
    for (uint32_t stride = size >> 1; stride >= (uint32_t) N; stride >>= 1) {
        const uint32_t ls = stride / N;
        const bool asc = final_phase || (((N * lane) & size) == 0);
        const bool lower = (lane & ls) == 0;
        cx_lanes<N>(k, v, ls, lower == asc);
    }
    // in-register strides: min(size/2, N/2) ... 1
#pragma unroll
    for (int stride = N / 2; stride >= 1; stride >>= 1) {
        if ((uint32_t) stride > (size >> 1)) continue;
#pragma unroll
        for (int i = 0; i < N; i++) {
            const int j = i ^ stride;
            if (i < j) {
                const uint32_t e = N * lane + i;
                const bool asc = final_phase || ((e & size) == 0);
                cx_regs(k[i], v[i], k[j], v[j], asc);
            }
        }
    }
}

template<int N>
__device__ __forceinline__ void warp_sort(float (&k)[N], uint32_t (&v)[N]) {
#pragma unroll
    for (uint32_t size = 2; size <= 32u * N; size <<= 1) bitonic_phase<N>(k, v, size, size == 32u * N);
}

// Last phase only: input must be bitonic over e (bitonic.cuh warp_merge, range 32).
template<int N>
__device__ __forceinline__ void warp_merge_final(float (&k)[N], uint32_t (&v)[N]) {
    bitonic_phase<N>(k, v, 32u * N, true);
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
// Visited set in shared memory: open addressing, linear probing, one table per
// warp. Same slot function and "full table reports seen" rule as hashmap.cuh:33-56.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void visited_clear(uint32_t *table, uint32_t bits) {
    for (uint32_t i = lane_id(); i < (1u << bits); i += 32) table[i] = kInvalid;
}

__device__ __forceinline__ uint32_t visited_insert(uint32_t *table, uint32_t bits, uint32_t key) {
    const uint32_t size = 1u << bits, mask = size - 1;
    uint32_t index = (key ^ (key >> bits)) & mask;
    for (uint32_t i = 0; i < size; i++) {
        const uint32_t old = atomicCAS(&table[index], kInvalid, key);
        if (old == kInvalid) return 1;
        if (old == key) return 0;
        index = (index + 1) & mask;
    }
    return 0;
}

typedef unsigned long long u64;

// ---- u64 bitonic network, N keys per lane, position e = N*lane + i -------------
template<int N>
__device__ __forceinline__ void phase_u64(u64 (&k)[N], uint32_t size, bool final_phase) {
    const uint32_t lane = lane_id();
    for (uint32_t stride = size >> 1; stride >= (uint32_t) N; stride >>= 1) {
        const uint32_t ls = stride / N;
        const bool asc = final_phase || (((N * lane) & size) == 0);
        const bool keep_small = ((lane & ls) == 0) == asc;
#pragma unroll
        for (int i = 0; i < N; i++) {
            const u64 o = __shfl_xor_sync(kFullMask, k[i], ls);
            if (keep_small ? (o < k[i]) : (o > k[i])) k[i] = o;
        }
    }
#pragma unroll
    for (int stride = N / 2; stride >= 1; stride >>= 1) {
        if ((uint32_t) stride > (size >> 1)) continue;
#pragma unroll
        for (int i = 0; i < N; i++) {
            const int j = i ^ stride;
            if (i < j) {
                const bool asc = final_phase || (((N * lane + i) & size) == 0);
                const u64 a = k[i], b = k[j];
                if ((a > b) == asc && a != b) { k[i] = b; k[j] = a; }
            }
        }
    }
}
template<int N>
__device__ __forceinline__ void sort_u64(u64 (&k)[N]) {
#pragma unroll
    for (uint32_t size = 2; size <= 32u * N; size <<= 1) phase_u64<N>(k, size, size == 32u * N);
}

__host__ __device__ constexpr uint32_t round_up32(uint32_t x) { return (x + 31u) & ~31u; }

}  // namespace glide
