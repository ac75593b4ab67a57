// Partition stage kernels: sample gather (reference sample_kernel,
// partition_kernel.cuh:7-20), nearest-centroid assignment with the boundary test
// (define_partition_kernel, :22-66), order-independent slot assignment replacing the
// reference's atomics (:57-60), the permuted copy (reorder_kernel, :68-100) and the
// Lloyd centroid update used in place of cuVS kmeans::fit (partition.cuh:48-54).
#include <algorithm>
#include <cstdlib>
#include "beam_core.cuh"
#include "kernels.h"

namespace glide {

namespace {

__global__ void gather_rows_kernel(const float *__restrict__ data, const uint32_t *__restrict__ ids, uint32_t count,
                                   uint32_t dim, float *__restrict__ out) {
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = lane_id();
    if (warp >= count) return;
    const float *src = data + (uint64_t) ids[warp] * dim;
    float *dst = out + (uint64_t) warp * dim;
    if ((dim & 3u) == 0) {
        for (uint32_t c = lane; c < (dim >> 2); c += 32)
            reinterpret_cast<float4 *>(dst)[c] = __ldg(reinterpret_cast<const float4 *>(src) + c);
    } else {
        for (uint32_t i = lane; i < dim; i += 32) dst[i] = __ldg(src + i);
    }
}

// A warp per point: distances to all centroids, network sort, nearest + boundary flag.
__global__ void __launch_bounds__(256) assign_kernel(const AssignArgs a, uint32_t max_centroid, uint32_t strip_words,
                                                     bool only_flagged) {
    extern __shared__ __align__(16) uint32_t smem[];
    const uint32_t warp = threadIdx.x >> 5, lane = lane_id();
    const uint32_t p = blockIdx.x * (blockDim.x >> 5) + warp;
    if (p >= a.n) return;
    if (only_flagged && a.nearest[p] != kInvalid) return;  // settled by the tiled or tensor-core kernel
    if (only_flagged && a.fallback_counter && lane == 0) atomicAdd(a.fallback_counter, 1ull);
    uint32_t *base = smem + (size_t) warp * strip_words;
    float *query = reinterpret_cast<float *>(base);
    uint32_t *scratch = base + dim_pad4(a.dim);
    load_query(query, a.data + (uint64_t) p * a.dim, a.dim);
    const uint32_t c0 = nearest_centroid(query, a.centroids, a.C, max_centroid, a.dim, a.metric, scratch,
                                         a.is_boundary ? kTopTwo : kNearestOnly);
    if (lane == 0) {
        // A point with a NaN coordinate has NaN distances to every centroid; the network then leaves
        // a padding slot (id 0xffffffff) in front. Such a point goes to partition 0, so that no
        // caller ever indexes start points or segment tables with an id beyond C.
        a.nearest[p] = c0 < a.C ? c0 : 0u;
        if (a.is_boundary) {
            const float *ck = reinterpret_cast<const float *>(scratch);
            // partition_kernel.cuh:58-60
            a.is_boundary[p] = (a.boundary_factor >= 0.0f && a.C > 1 && ck[1] / ck[0] <= a.boundary_factor) ? 0u : kInvalid;
        }
    }
}

// ---------------------------------------------------------------------------
// Tiled assignment: the same distances as assign_kernel, bit for bit, computed as a
// points x centroids contraction. A CTA owns 32 points and walks the centroids in tiles of
// 64; both tiles are staged through shared memory 32 dimensions at a time and each thread
// keeps 2 x 4 (point, centroid) pairs in registers. To reproduce the team summation order
// (lane t of a team owns 16-byte chunks t, t+8, ...; lanes are folded 4-2-1) every pair
// keeps EIGHT partial sums, one per team lane, and folds them in the same tree at the end.
// Each point then needs its smallest and second smallest distance; when the smallest is
// shared by two centroids the point is left to assign_kernel (flag 0xffffffff), whose
// network sort reproduces the reference's tie order.
// ---------------------------------------------------------------------------
constexpr int kAP = 32;          // points per CTA
constexpr int kAC = 64;          // centroids per tile
constexpr int kAK = 32;          // dimensions per stage (8 chunks of 4 = one round of the 8 team lanes)
constexpr int kAPPad = kAP + 2;  // float2 reads stay 8-byte aligned
constexpr int kACPad = kAC + 4;  // float4 reads stay 16-byte aligned

struct NearState {
    float d0, d1;    // smallest and second smallest distance
    uint32_t id;     // centroid of d0
    uint32_t ties;   // how many centroids share d0
};

__device__ __forceinline__ void near_add(NearState &s, float d, uint32_t id) {
    if (d < s.d0) { s.d1 = s.d0; s.d0 = d; s.id = id; s.ties = 1; }
    else if (d == s.d0) { s.d1 = d; s.ties++; }
    else if (d < s.d1) { s.d1 = d; }
}

__device__ __forceinline__ void near_merge(NearState &a, float d0, float d1, uint32_t id, uint32_t ties) {
    if (d0 < a.d0) { a.d1 = fminf(a.d0, d1); a.d0 = d0; a.id = id; a.ties = ties; }
    else if (d0 == a.d0) { a.d1 = d0; a.ties += ties; }
    else { a.d1 = fminf(a.d1, d0); }
}

__global__ void __launch_bounds__(256) assign_tiled_kernel(const AssignArgs a) {
    __shared__ __align__(16) float Ps[kAK * kAPPad];
    __shared__ __align__(16) float Cs[kAK * kACPad];
    const uint32_t tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const uint32_t p0 = blockIdx.x * kAP;
    NearState st[2];
#pragma unroll
    for (int i = 0; i < 2; i++) { st[i].d0 = FLT_MAX; st[i].d1 = FLT_MAX; st[i].id = kInvalid; st[i].ties = 0; }

    for (uint32_t c0 = 0; c0 < a.C; c0 += kAC) {
        float acc[2][4][8];
#pragma unroll
        for (int i = 0; i < 2; i++)
#pragma unroll
            for (int j = 0; j < 4; j++)
#pragma unroll
                for (int t = 0; t < 8; t++) acc[i][j][t] = 0.0f;
        for (uint32_t k0 = 0; k0 < a.dim; k0 += kAK) {
            for (uint32_t e = tid; e < kAP * kAK; e += 256) {
                const uint32_t row = e / kAK, kk = e % kAK;
                const uint32_t p = p0 + row, d = k0 + kk;
                Ps[kk * kAPPad + row] = (p < a.n && d < a.dim) ? __ldg(a.data + (uint64_t) p * a.dim + d) : 0.0f;
            }
            for (uint32_t e = tid; e < kAC * kAK; e += 256) {
                const uint32_t row = e / kAK, kk = e % kAK;
                const uint32_t c = c0 + row, d = k0 + kk;
                Cs[kk * kACPad + row] = (c < a.C && d < a.dim) ? __ldg(a.centroids + (uint64_t) c * a.dim + d) : 0.0f;
            }
            __syncthreads();
#pragma unroll
            for (int t = 0; t < 8; t++) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int kk = 4 * t + e;
                    const float2 pv = *reinterpret_cast<const float2 *>(Ps + kk * kAPPad + 2 * ty);
                    const float4 cv = *reinterpret_cast<const float4 *>(Cs + kk * kACPad + 4 * tx);
                    const float pa[2] = {pv.x, pv.y};
                    const float ca[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
                    for (int i = 0; i < 2; i++)
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const float df = pa[i] - ca[j];
                            acc[i][j][t] = __fmaf_rn(df, df, acc[i][j][t]);
                        }
                }
            }
            __syncthreads();
        }
#pragma unroll
        for (int i = 0; i < 2; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t c = c0 + 4 * tx + j;
                if (c >= a.C) continue;
                const float *s = acc[i][j];
                const float sum = ((s[0] + s[4]) + (s[2] + s[6])) + ((s[1] + s[5]) + (s[3] + s[7]));
                near_add(st[i], a.metric == kEuclidean ? sqrtf(sum) : sum, c);
            }
    }
    // fold the 16 threads (tx) that share a point: they are 16 consecutive lanes
#pragma unroll
    for (int i = 0; i < 2; i++) {
#pragma unroll
        for (int off = 8; off >= 1; off >>= 1) {
            const float d0 = __shfl_xor_sync(kFullMask, st[i].d0, off);
            const float d1 = __shfl_xor_sync(kFullMask, st[i].d1, off);
            const uint32_t id = __shfl_xor_sync(kFullMask, st[i].id, off);
            const uint32_t ties = __shfl_xor_sync(kFullMask, st[i].ties, off);
            near_merge(st[i], d0, d1, id, ties);
        }
        const uint32_t p = p0 + 2 * ty + i;
        if (tx == 0 && p < a.n) {
            const bool unique = st[i].ties == 1;
            a.nearest[p] = unique ? st[i].id : kInvalid;
            if (a.is_boundary && unique)  // partition_kernel.cuh:58-60
                a.is_boundary[p] = (a.boundary_factor >= 0.0f && a.C > 1 && st[i].d1 / st[i].d0 <= a.boundary_factor) ? 0u : kInvalid;
        }
    }
}

constexpr uint32_t kSlotBlock = 256;

// pass 1: per-block histogram of keys
__global__ void __launch_bounds__(kSlotBlock) slot_hist_kernel(const uint32_t *__restrict__ key, uint32_t n, uint32_t K,
                                                                uint32_t *block_hist) {
    extern __shared__ uint32_t hist[];
    for (uint32_t k = threadIdx.x; k < K; k += blockDim.x) hist[k] = 0;
    __syncthreads();
    const uint32_t i = blockIdx.x * kSlotBlock + threadIdx.x;
    if (i < n) {
        const uint32_t k = key[i];
        if (k < K) atomicAdd(&hist[k], 1u);
    }
    __syncthreads();
    for (uint32_t k = threadIdx.x; k < K; k += blockDim.x) block_hist[(uint64_t) blockIdx.x * K + k] = hist[k];
}

// pass 2: per key, exclusive prefix over blocks (in place); totals[k] = count. A CTA owns 32 keys
// (threadIdx.x, coalesced) and splits the blocks into 32 contiguous chunks (threadIdx.y): chunk
// sums, a scan over the chunks in shared memory, then the prefixes.
__global__ void __launch_bounds__(1024) slot_prefix_kernel(uint32_t *block_hist, uint32_t blocks, uint32_t K, uint32_t *totals) {
    __shared__ uint32_t chunk_sum[32][33];
    const uint32_t k = blockIdx.x * 32 + threadIdx.x, y = threadIdx.y;
    const uint32_t per = (blocks + 31) / 32;
    const uint32_t lo = y * per, hi = min(blocks, lo + per);
    uint32_t sum = 0;
    if (k < K)
        for (uint32_t b = lo; b < hi; b++) sum += block_hist[(uint64_t) b * K + k];
    chunk_sum[y][threadIdx.x] = sum;
    __syncthreads();
    if (y == 0) {
        uint32_t run = 0;
        for (uint32_t c = 0; c < 32; c++) {
            const uint32_t v = chunk_sum[c][threadIdx.x];
            chunk_sum[c][threadIdx.x] = run;
            run += v;
        }
        if (k < K) totals[k] = run;
    }
    __syncthreads();
    if (k < K) {
        uint32_t run = chunk_sum[y][threadIdx.x];
        for (uint32_t b = lo; b < hi; b++) {
            const uint32_t v = block_hist[(uint64_t) b * K + k];
            block_hist[(uint64_t) b * K + k] = run;
            run += v;
        }
    }
}

// pass 3: slot = block prefix + rank among earlier points of the block with the same
// key. Warps take turns in ascending order so that ranks follow the point index.
__global__ void __launch_bounds__(kSlotBlock) slot_rank_kernel(const uint32_t *__restrict__ key, uint32_t n, uint32_t K,
                                                                const uint32_t *__restrict__ block_hist,
                                                                uint32_t *slot) {
    extern __shared__ uint32_t run[];
    for (uint32_t k = threadIdx.x; k < K; k += blockDim.x) run[k] = block_hist[(uint64_t) blockIdx.x * K + k];
    __syncthreads();
    const uint32_t i = blockIdx.x * kSlotBlock + threadIdx.x;
    const uint32_t warp = threadIdx.x >> 5, lane = lane_id();
    const uint32_t k = (i < n) ? key[i] : kInvalid;
    const bool valid = k < K;
    for (uint32_t w = 0; w < kSlotBlock / 32; w++) {
        if (warp == w) {
            const uint32_t peers = __match_any_sync(kFullMask, k);
            if (valid) {
                const uint32_t rank = __popc(peers & ((1u << lane) - 1));
                slot[i] = run[k] + rank;
            } else if (i < n) {
                slot[i] = kInvalid;
            }
            __syncwarp();
            if (valid && lane == (uint32_t) (__ffs(peers) - 1)) run[k] += __popc(peers);
        }
        __syncthreads();
    }
}

__global__ void reorder_kernel(const float *__restrict__ data, uint32_t n, uint32_t dim,
                               const uint32_t *__restrict__ seg_index, const uint32_t *__restrict__ seg_start,
                               float *__restrict__ out, uint32_t *__restrict__ map) {
    const uint32_t p = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = lane_id();
    if (p >= n) return;
    const uint32_t r = seg_start[seg_index[3 * (uint64_t) p]] + seg_index[3 * (uint64_t) p + 1];
    const uint32_t b = seg_index[3 * (uint64_t) p + 2];
    const float *src = data + (uint64_t) p * dim;
    float *d0 = out + (uint64_t) r * dim;
    float *d1 = (b != kInvalid) ? out + (uint64_t) (n + b) * dim : nullptr;
    if ((dim & 3u) == 0) {
        for (uint32_t c = lane; c < (dim >> 2); c += 32) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(src) + c);
            reinterpret_cast<float4 *>(d0)[c] = v;
            if (d1) reinterpret_cast<float4 *>(d1)[c] = v;
        }
    } else {
        for (uint32_t i = lane; i < dim; i += 32) {
            const float v = __ldg(src + i);
            d0[i] = v;
            if (d1) d1[i] = v;
        }
    }
    if (lane == 0) {
        map[r] = p;
        if (d1) map[n + b] = p;
    }
}

__global__ void pack_seg_index_kernel(const uint32_t *__restrict__ nearest, const uint32_t *__restrict__ slot,
                                      const uint32_t *__restrict__ bslot, uint32_t n, uint32_t *seg_index) {
    const uint32_t p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= n) return;
    seg_index[3 * (uint64_t) p] = nearest[p];
    seg_index[3 * (uint64_t) p + 1] = slot[p];
    seg_index[3 * (uint64_t) p + 2] = bslot ? bslot[p] : kInvalid;
}

__global__ void scatter_members_kernel(const uint32_t *__restrict__ label, const uint32_t *__restrict__ slot,
                                       const uint32_t *__restrict__ off, uint32_t n, uint32_t *member_ids) {
    const uint32_t p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= n) return;
    member_ids[off[label[p]] + slot[p]] = p;
}

// centroid c = (sum of its members in ascending row order) / count, fp32; an empty
// cluster keeps its centroid.
__global__ void centroid_update_kernel(const float *__restrict__ sample, uint32_t dim,
                                       const uint32_t *__restrict__ member_ids, const uint32_t *__restrict__ off,
                                       const uint32_t *__restrict__ cnt, float *centroids) {
    const uint32_t c = blockIdx.x;
    const uint32_t count = cnt[c];
    if (count == 0) return;
    const uint32_t *members = member_ids + off[c];
    for (uint32_t d = threadIdx.x; d < dim; d += blockDim.x) {
        float acc = 0.0f;
        for (uint32_t m = 0; m < count; m++) acc = acc + __ldg(sample + (uint64_t) members[m] * dim + d);
        centroids[(uint64_t) c * dim + d] = acc / (float) count;
    }
}

__global__ void count_changed_kernel(const uint32_t *__restrict__ a, const uint32_t *__restrict__ b, uint32_t n,
                                     uint32_t *count) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    const bool diff = (i < n) && (a[i] != b[i]);
    const uint32_t m = __ballot_sync(kFullMask, diff);
    if (lane_id() == 0 && m) atomicAdd(count, (uint32_t) __popc(m));
}

// ---- farthest-first traversal (k-means initialisation) ---------------------------------
// Step t: mind2[i] = min(mind2[i], |x_i - c_{t-1}|^2) for every sample row, and the row
// with the largest mind2 (lowest row on ties) becomes c_t. One kernel updates and reduces
// per block, a one-block kernel picks the winner and copies its row.
constexpr uint32_t kFfRowsPerBlock = 256;

__device__ __forceinline__ u64 ff_key(float v, uint32_t row) {
    return ((u64) __float_as_uint(v) << 32) | (u64) (0xffffffffu - row);
}

__global__ void __launch_bounds__(256) ff_update_kernel(const float *__restrict__ sample, uint32_t n, uint32_t dim,
                                                        const float *__restrict__ centre, float *mind2,
                                                        u64 *block_best) {
    extern __shared__ __align__(16) uint32_t smem[];
    __shared__ u64 warp_best[8];
    float *c = reinterpret_cast<float *>(smem);
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) c[i] = centre[i];
    __syncthreads();
    const uint32_t warp = threadIdx.x >> 5, lane = lane_id(), team = lane / kTeam;
    const uint32_t row0 = blockIdx.x * kFfRowsPerBlock;
    u64 best = 0;
    for (uint32_t r = warp * kTeamsPerWarp; r < kFfRowsPerBlock; r += 8 * kTeamsPerWarp) {
        const uint32_t row = row0 + r + team;
        const bool active = row < n;
        const float part = team_partial(c, sample + (uint64_t) (active ? row : 0) * dim, dim, active);
        const float d = team_fold(part);
        if (active) {
            float m = mind2[row];
            if (d < m) m = d;
            if ((lane & (kTeam - 1)) == 0) mind2[row] = m;
            const u64 k = ff_key(m, row);
            if (k > best) best = k;
        }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        const u64 o = __shfl_xor_sync(kFullMask, best, off);
        if (o > best) best = o;
    }
    if (lane == 0) warp_best[warp] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        u64 b = warp_best[0];
        for (int w = 1; w < 8; w++) if (warp_best[w] > b) b = warp_best[w];
        block_best[blockIdx.x] = b;
    }
}

__global__ void __launch_bounds__(256) ff_pick_kernel(const float *__restrict__ sample, uint32_t dim,
                                                      const u64 *__restrict__ block_best, uint32_t blocks,
                                                      float *next_centre) {
    __shared__ u64 warp_best[8];
    __shared__ uint32_t winner;
    u64 best = 0;
    for (uint32_t i = threadIdx.x; i < blocks; i += blockDim.x) if (block_best[i] > best) best = block_best[i];
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        const u64 o = __shfl_xor_sync(kFullMask, best, off);
        if (o > best) best = o;
    }
    if (lane_id() == 0) warp_best[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        u64 b = warp_best[0];
        for (int w = 1; w < 8; w++) if (warp_best[w] > b) b = warp_best[w];
        winner = 0xffffffffu - (uint32_t) b;
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) next_centre[i] = sample[(uint64_t) winner * dim + i];
}

// ---- the same traversal as one launch --------------------------------------------------
// One CTA per SM owns a fixed slice of the sample and keeps it on the chip for the whole
// traversal: as many rows as fit in shared memory, then up to four rows per team of eight lanes
// in registers (dimensions that are multiples of 32 up to 128), the rest re-read from L2. The
// CTAs meet at one grid barrier per centre: update + block maximum, atomic maximum into the
// centre's own slot, barrier, every CTA reads the slot and fetches the winning row as its next
// centre. Same arithmetic and tie rule as the two kernels above, so the centres are the same
// bits. The barrier's wait is bounded: a CTA that waits too long raises the error word, and
// every CTA returns once it sees the word or runs out of patience itself.
constexpr uint32_t kFfThreads = 512;
constexpr uint32_t kFfWarps = kFfThreads / 32;
constexpr uint32_t kFfTeams = kFfThreads / kTeam;
constexpr uint32_t kFfTeamRows = 4;           // rows a team can hold in registers
constexpr uint32_t kFfSpinLimit = 1u << 22;   // around a second of polling
constexpr uint32_t kFfMaxCentres = 4096;

struct FfArgs {
    const float *sample;
    uint32_t n, dim, C;
    float *centroids;
    u64 *step_best;        // one slot per centre, zero at launch
    uint32_t *sync;        // [0] arrivals, [1] error
    uint32_t rows_per_block, shared_rows;
};

__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// team lane's partial sum over a row held in shared memory; the order of team_partial
__device__ __forceinline__ float team_partial_shared(const float *q, const float *row, uint32_t dim) {
    const uint32_t t = threadIdx.x & (kTeam - 1);
    const uint32_t chunks = dim >> 2;
    const float4 *q4 = reinterpret_cast<const float4 *>(q);
    const float4 *r4 = reinterpret_cast<const float4 *>(row);
    float acc = 0.0f;
#pragma unroll 4
    for (uint32_t c = t; c < chunks; c += kTeam) acc = sq_acc4(q4[c], r4[c], acc);
    return acc;
}

__device__ __forceinline__ u64 ff_block_max(u64 best, u64 *warp_best) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        const u64 o = __shfl_xor_sync(kFullMask, best, off);
        if (o > best) best = o;
    }
    if (lane_id() == 0) warp_best[threadIdx.x >> 5] = best;
    __syncthreads();
    u64 b = warp_best[0];
    for (uint32_t w = 1; w < kFfWarps; w++) if (warp_best[w] > b) b = warp_best[w];
    return b;
}

// CH: 16-byte chunks of a row per team lane (dim == 32 * CH) when rows are held in registers, else 0
template<int CH>
__global__ void __launch_bounds__(kFfThreads, 1) ff_persistent_kernel(const FfArgs a) {
    extern __shared__ __align__(16) uint32_t smem[];
    __shared__ u64 warp_best[kFfWarps];
    __shared__ uint32_t gave_up;
    __shared__ u64 step_winner;
    const uint32_t dim = a.dim;
    float *c = reinterpret_cast<float *>(smem);
    float *mind2 = c + dim_pad4(dim);
    float *held = mind2 + ((a.rows_per_block + 3u) & ~3u);
    const uint32_t lo = min(a.n, blockIdx.x * a.rows_per_block), hi = min(a.n, lo + a.rows_per_block);
    const uint32_t mine = hi - lo, in_shared = min(a.shared_rows, mine);
    const uint32_t in_regs = CH > 0 ? min(mine - in_shared, kFfTeams * kFfTeamRows) : 0;
    const uint32_t warp = threadIdx.x >> 5, team = lane_id() / kTeam, t8 = threadIdx.x & (kTeam - 1);
    const uint32_t my_first = in_shared + (threadIdx.x / kTeam) * kFfTeamRows;   // this team's rows in registers
    float4 hr[kFfTeamRows][CH > 0 ? CH : 1];
    {
        const float4 *src = reinterpret_cast<const float4 *>(a.sample + (uint64_t) lo * dim);   // in_shared > 0 only when dim % 4 == 0
        float4 *dst = reinterpret_cast<float4 *>(held);
        const uint32_t chunks = in_shared * (dim >> 2);
        for (uint32_t i = threadIdx.x; i < chunks; i += kFfThreads) dst[i] = __ldg(src + i);
        if (CH > 0) {
#pragma unroll
            for (uint32_t j = 0; j < kFfTeamRows; j++)
#pragma unroll
                for (int k = 0; k < CH; k++)
                    hr[j][k] = my_first + j < in_shared + in_regs ? __ldg(src + (size_t) (my_first + j) * (dim >> 2) + t8 + k * kTeam)
                                                                  : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    for (uint32_t i = threadIdx.x; i < mine; i += kFfThreads) mind2[i] = FLT_MAX;
    for (uint32_t i = threadIdx.x; i < dim; i += kFfThreads) {
        const float v = __ldg(a.sample + i);   // the first centre is the first sample row
        c[i] = v;
        if (blockIdx.x == 0) a.centroids[i] = v;
    }
    if (threadIdx.x == 0) gave_up = 0;
    __syncthreads();
    for (uint32_t t = 0; t + 1 < a.C; t++) {
        u64 best = 0;
        auto settle = [&](uint32_t i, float part, bool active) {
            const float d = team_fold(part);
            if (active) {
                float m = mind2[i];
                if (d < m) m = d;
                if (t8 == 0) mind2[i] = m;
                const u64 k = ff_key(m, lo + i);
                if (k > best) best = k;
            }
        };
        for (uint32_t r = warp * kTeamsPerWarp; r < in_shared; r += kFfWarps * kTeamsPerWarp) {
            const uint32_t i = r + team;
            const bool active = i < in_shared;
            settle(i, active ? team_partial_shared(c, held + (size_t) i * dim, dim) : 0.0f, active);
        }
        if (CH > 0) {
            const float4 *q4 = reinterpret_cast<const float4 *>(c);
#pragma unroll
            for (uint32_t j = 0; j < kFfTeamRows; j++) {
                float acc = 0.0f;
#pragma unroll
                for (int k = 0; k < CH; k++) acc = sq_acc4(q4[t8 + k * kTeam], hr[j][k], acc);
                settle(my_first + j, acc, my_first + j < in_shared + in_regs);
            }
        }
        for (uint32_t r = in_shared + in_regs + warp * kTeamsPerWarp; r < mine; r += kFfWarps * kTeamsPerWarp) {
            const uint32_t i = r + team;
            const bool active = i < mine;
            settle(i, team_partial(c, a.sample + (uint64_t) (lo + (active ? i : 0)) * dim, dim, active), active);
        }
        const u64 block_max = ff_block_max(best, warp_best);
        // arrive with this CTA's maximum and wait for every CTA's
        if (threadIdx.x == 0) {
            atomicMax(reinterpret_cast<unsigned long long *>(a.step_best + t), (unsigned long long) block_max);
            __threadfence();
            atomicAdd(&a.sync[0], 1u);
            const uint32_t target = (t + 1) * gridDim.x;
            uint32_t spins = 0;
            bool ok = true;
            while (ld_acquire_u32(&a.sync[0]) < target) {
                if (++spins > kFfSpinLimit || ((spins & 1023u) == 0 && ld_acquire_u32(&a.sync[1]) != 0)) {
                    atomicExch(&a.sync[1], 1u);
                    ok = false;
                    break;
                }
            }
            if (ok) step_winner = __ldcg(a.step_best + t);
            else gave_up = 1;
        }
        __syncthreads();   // also: nobody reads the old centre or warp_best any more
        if (gave_up) return;
        const uint32_t winner = 0xffffffffu - (uint32_t) step_winner;
        for (uint32_t i = threadIdx.x; i < dim; i += kFfThreads) {
            const float v = __ldg(a.sample + (uint64_t) winner * dim + i);
            c[i] = v;
            if (blockIdx.x == 0) a.centroids[(uint64_t) (t + 1) * dim + i] = v;
        }
        __syncthreads();
    }
}

__global__ void fill_f32_kernel(float *p, uint32_t n, float v) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

uint32_t pow2_at_least(uint32_t x, uint32_t lo) {
    uint32_t m = lo;
    while (m < x) m <<= 1;
    return m;
}

}  // namespace

cudaError_t launch_gather_rows(const float *data, const uint32_t *ids, uint32_t count, uint32_t dim, float *out,
                               cudaStream_t stream) {
    if (count == 0) return cudaSuccess;
    const uint32_t warps = 8;
    gather_rows_kernel<<<(count + warps - 1) / warps, warps * 32, 0, stream>>>(data, ids, count, dim, out);
    return cudaGetLastError();
}

cudaError_t launch_assign(const AssignArgs &a, cudaStream_t stream, uint32_t *launched) {
    if (launched) *launched = 0;
    if (a.n == 0) return cudaSuccess;
    const uint32_t max_centroid = pow2_at_least(a.C, 32);
    const uint32_t strip_words = (dim_pad4(a.dim) + 2 * max_centroid + 3u) & ~3u;
    uint32_t warps = 8;
    while (warps > 1 && (size_t) strip_words * 4 * warps > 96 * 1024) warps >>= 1;
    const size_t smem_bytes = (size_t) strip_words * 4 * warps;
    if (smem_bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(assign_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_bytes);
        if (e != cudaSuccess) return e;
    }
    // the tiled kernel settles every point whose nearest centroid is unique; the warp-per-point
    // kernel then handles the rest (ties at the minimum; all points when dim % 4 != 0)
    // GLIDE_B200_EXACT_ASSIGN=1 keeps the tensor cores out of it (the tests compare both ways)
    static const bool exact_only = [] { const char *e = std::getenv("GLIDE_B200_EXACT_ASSIGN"); return e && e[0] == '1'; }();
    const bool tiled = (a.dim & 3u) == 0 && a.C >= 2;
    if (!exact_only && assign_tc_eligible(a)) {
        cudaError_t e = launch_assign_tc(a, stream);
        if (e != cudaSuccess) return e;
        if (launched) *launched += 2;
    } else if (tiled) {
        assign_tiled_kernel<<<(a.n + kAP - 1) / kAP, 256, 0, stream>>>(a);
        if (launched) *launched += 1;
    }
    if (launched) *launched += 1;
    assign_kernel<<<(a.n + warps - 1) / warps, warps * 32, smem_bytes, stream>>>(a, max_centroid, strip_words, tiled);
    return cudaGetLastError();
}

// Small batches: order[] = the indices 0..n-1 grouped by key, in one CTA (shared-memory histogram, scan,
// scatter). The order inside a group follows the atomics; callers only use the grouping.
__global__ void __launch_bounds__(1024) group_by_key_kernel(const uint32_t *__restrict__ key, uint32_t n, uint32_t K,
                                                            uint32_t *__restrict__ order) {
    extern __shared__ uint32_t sh[];   // K counters, then K cursors
    uint32_t *count = sh, *cursor = sh + K;
    __shared__ uint32_t warp_sums[32];
    for (uint32_t k = threadIdx.x; k < K; k += blockDim.x) count[k] = 0;
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        const uint32_t k = key[i];
        if (k < K) atomicAdd(&count[k], 1u);
    }
    __syncthreads();
    // exclusive scan of count[] into cursor[]: K / blockDim consecutive entries per thread
    const uint32_t per = (K + blockDim.x - 1) / blockDim.x;
    const uint32_t lo = threadIdx.x * per, hi = min(K, lo + per);
    uint32_t local = 0;
    for (uint32_t k = lo; k < hi; k++) local += count[k];
    uint32_t incl = local;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const uint32_t v = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= (uint32_t) off) incl += v;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        uint32_t w = lane < (blockDim.x >> 5) ? warp_sums[lane] : 0;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const uint32_t v = __shfl_up_sync(0xffffffffu, w, off);
            if (lane >= (uint32_t) off) w += v;
        }
        warp_sums[lane] = w;   // inclusive over warps
    }
    __syncthreads();
    uint32_t run = incl - local + (warp ? warp_sums[warp - 1] : 0);
    for (uint32_t k = lo; k < hi; k++) {
        cursor[k] = run;
        run += count[k];
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        const uint32_t k = key[i];
        if (k < K) order[atomicAdd(&cursor[k], 1u)] = i;
    }
}

cudaError_t launch_group_by_key(const uint32_t *key, uint32_t n, uint32_t K, uint32_t *order, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    group_by_key_kernel<<<1, 1024, 2 * (size_t) K * sizeof(uint32_t), stream>>>(key, n, K, order);
    return cudaGetLastError();
}

size_t slot_scratch_words(uint32_t n, uint32_t K) { return (size_t) ((n + kSlotBlock - 1) / kSlotBlock) * K; }

cudaError_t launch_slots(const uint32_t *key, uint32_t n, uint32_t K, uint32_t *slot, uint32_t *totals,
                         uint32_t *scratch, cudaStream_t stream) {
    if (n == 0) return cudaMemsetAsync(totals, 0, K * sizeof(uint32_t), stream);
    const uint32_t blocks = (n + kSlotBlock - 1) / kSlotBlock;
    slot_hist_kernel<<<blocks, kSlotBlock, K * sizeof(uint32_t), stream>>>(key, n, K, scratch);
    slot_prefix_kernel<<<(K + 31) / 32, dim3(32, 32), 0, stream>>>(scratch, blocks, K, totals);
    slot_rank_kernel<<<blocks, kSlotBlock, K * sizeof(uint32_t), stream>>>(key, n, K, scratch, slot);
    return cudaGetLastError();
}

cudaError_t launch_reorder(const float *data, uint32_t n, uint32_t dim, const uint32_t *seg_index,
                           const uint32_t *seg_start_dev, float *reorder_data, uint32_t *map, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    const uint32_t warps = 8;
    reorder_kernel<<<(n + warps - 1) / warps, warps * 32, 0, stream>>>(data, n, dim, seg_index, seg_start_dev,
                                                                       reorder_data, map);
    return cudaGetLastError();
}

cudaError_t launch_pack_seg_index(const uint32_t *nearest, const uint32_t *slot, const uint32_t *bslot, uint32_t n,
                                  uint32_t *seg_index, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    pack_seg_index_kernel<<<(n + 255) / 256, 256, 0, stream>>>(nearest, slot, bslot, n, seg_index);
    return cudaGetLastError();
}

cudaError_t launch_scatter_members(const uint32_t *label, const uint32_t *slot, const uint32_t *off, uint32_t n,
                                   uint32_t *member_ids, cudaStream_t stream) {
    if (n == 0) return cudaSuccess;
    scatter_members_kernel<<<(n + 255) / 256, 256, 0, stream>>>(label, slot, off, n, member_ids);
    return cudaGetLastError();
}

cudaError_t launch_centroid_update(const float *sample, uint32_t dim, const uint32_t *member_ids,
                                   const uint32_t *off, const uint32_t *cnt, uint32_t C, float *centroids,
                                   cudaStream_t stream) {
    const uint32_t threads = dim < 1024 ? ((dim + 31) / 32) * 32 : 1024;
    centroid_update_kernel<<<C, threads, 0, stream>>>(sample, dim, member_ids, off, cnt, centroids);
    return cudaGetLastError();
}

cudaError_t launch_count_changed(const uint32_t *a, const uint32_t *b, uint32_t n, uint32_t *count,
                                 cudaStream_t stream) {
    cudaError_t e = cudaMemsetAsync(count, 0, sizeof(uint32_t), stream);
    if (e != cudaSuccess || n == 0) return e;
    count_changed_kernel<<<(n + 255) / 256, 256, 0, stream>>>(a, b, n, count);
    return cudaGetLastError();
}

size_t farthest_first_scratch_bytes(uint32_t n) {
    // distances, block maxima of the launch-per-centre path, then the per-centre slots and the two
    // barrier words of the one-launch path
    return (size_t) n * 4 + 256 + (size_t) ((n + kFfRowsPerBlock - 1) / kFfRowsPerBlock) * 8 + 256 + kFfMaxCentres * 8 + 256;
}

// One persistent launch when the sample is small enough to stay on the chip and in L2 between
// centres; returns cudaErrorNotSupported when this device or shape cannot take it.
static cudaError_t launch_farthest_first_persistent(const float *sample, uint32_t n, uint32_t dim, uint32_t C,
                                                    float *centroids, char *tail, cudaStream_t stream) {
    int device = 0, sms = 0, coop = 0, smem_max = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&smem_max, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    if (e != cudaSuccess) return e;
    if (!coop || sms <= 0 || C > kFfMaxCentres) return cudaErrorNotSupported;
    const uint32_t G = std::max(1u, std::min<uint32_t>((uint32_t) sms, (n + 63) / 64));
    const uint32_t rows_per_block = (n + G - 1) / G;
    const size_t fixed_bytes = (size_t) dim_pad4(dim) * 4 + (size_t) ((rows_per_block + 3u) & ~3u) * 4;
    const size_t budget = (size_t) smem_max - 1024;
    if (fixed_bytes + 1024 > budget || rows_per_block > 16384) return cudaErrorNotSupported;
    uint32_t shared_rows = 0;
    if ((dim & 3u) == 0) shared_rows = (uint32_t) std::min<size_t>(rows_per_block, (budget - fixed_bytes) / ((size_t) dim * 4));
    const size_t smem = fixed_bytes + (size_t) shared_rows * dim * 4;
    const int ch = (dim % 32 == 0 && dim <= 128) ? (int) (dim / 32) : 0;
    const void *kernel = ch == 1 ? (const void *) ff_persistent_kernel<1> : ch == 2 ? (const void *) ff_persistent_kernel<2>
                       : ch == 3 ? (const void *) ff_persistent_kernel<3> : ch == 4 ? (const void *) ff_persistent_kernel<4>
                                                                                     : (const void *) ff_persistent_kernel<0>;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem);
    int per_sm = 0;
    if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, (int) kFfThreads, smem);
    if (e != cudaSuccess) return e;
    if ((uint64_t) per_sm * (uint64_t) sms < G) return cudaErrorNotSupported;
    FfArgs a{sample, n, dim, C, centroids, reinterpret_cast<u64 *>(tail), reinterpret_cast<uint32_t *>(tail + kFfMaxCentres * 8),
             rows_per_block, shared_rows};
    e = cudaMemsetAsync(tail, 0, kFfMaxCentres * 8 + 8, stream);
    if (e != cudaSuccess) return e;
    void *params[] = {&a};
    e = cudaLaunchCooperativeKernel(kernel, dim3(G), dim3(kFfThreads), params, smem, stream);
    if (e == cudaErrorCooperativeLaunchTooLarge) return cudaErrorNotSupported;   // fewer SMs than the device reports are ours
    if (e != cudaSuccess) return e;
    uint32_t words[2] = {0, 0};
    e = cudaMemcpyAsync(words, a.sync, 8, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return e;
    return words[1] ? cudaErrorLaunchTimeout : cudaSuccess;   // a CTA ran out of patience at the barrier
}

cudaError_t launch_farthest_first(const float *sample, uint32_t n, uint32_t dim, uint32_t C, float *centroids,
                                  void *scratch, cudaStream_t stream) {
    float *mind2 = static_cast<float *>(scratch);
    char *after = static_cast<char *>(scratch) + (((size_t) n * 4 + 255) & ~(size_t) 255);
    u64 *block_best = reinterpret_cast<u64 *>(after);
    const uint32_t blocks = (n + kFfRowsPerBlock - 1) / kFfRowsPerBlock;
    // GLIDE_B200_FF_LAUNCHES=1 keeps the launch-per-centre path (the tests compare both)
    const char *env = std::getenv("GLIDE_B200_FF_LAUNCHES");
    const bool per_centre = env && env[0] == '1';
    if (!per_centre && n > 0 && C > 0 && (uint64_t) n * dim * 4 <= ((uint64_t) 96 << 20)) {
        char *tail = after + (((size_t) blocks * 8 + 255) & ~(size_t) 255);
        const cudaError_t e = launch_farthest_first_persistent(sample, n, dim, C, centroids, tail, stream);
        // a barrier that ran out of patience (the CTAs were not all resident in time, say behind another
        // stream's long kernel) leaves nothing behind that the launches below do not overwrite
        if (e != cudaErrorNotSupported && e != cudaErrorLaunchTimeout) return e;
        (void) cudaGetLastError();
    }
    fill_f32_kernel<<<(n + 255) / 256, 256, 0, stream>>>(mind2, n, FLT_MAX);
    cudaError_t e = cudaMemcpyAsync(centroids, sample, (size_t) dim * 4, cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) return e;
    const size_t smem = (size_t) dim_pad4(dim) * 4;
    for (uint32_t t = 0; t < C; t++) {
        ff_update_kernel<<<blocks, 256, smem, stream>>>(sample, n, dim, centroids + (uint64_t) t * dim, mind2, block_best);
        if (t + 1 < C) ff_pick_kernel<<<1, 256, 0, stream>>>(sample, dim, block_best, blocks, centroids + (uint64_t) (t + 1) * dim);
    }
    return cudaGetLastError();
}

}  // namespace glide
