// Exact brute-force kNN (fp32, squared-difference sums): the ground truth that recall
// is measured against, and the seed/validation tool for the kNN stage. The reference
// has no such kernel (it reads ground truth from a file, small_search.cu:88).
//
// Tiling: a CTA of 256 threads owns 64 queries and walks its slice of the base set in
// tiles of 128 rows; the 64x128 distance tile lives in registers (4x8 per thread) and
// is accumulated over the dimension in steps of 32 staged through shared memory. Rows
// whose distance beats the query's current k-th best are queued and inserted into a
// sorted per-query list by one warp; ties order by ascending id.
#include "common.cuh"
#include "kernels.h"

namespace glide {

namespace {

constexpr int kQT = 64;    // queries per CTA
constexpr int kBT = 128;   // base rows per tile
constexpr int kKT = 32;    // dimension step
constexpr int kQPad = kQT + 4;
constexpr int kBPad = kBT + 4;
constexpr int kMaxK = 128;

struct Cand {
    float d;
    uint32_t id;
};

__device__ __forceinline__ bool cand_less(float d0, uint32_t i0, float d1, uint32_t i1) {
    return (d0 < d1) || (d0 == d1 && i0 < i1);
}

// Insert (d,id) into the ascending list (ld, li) of k entries held in shared memory;
// executed by one whole warp.
__device__ __forceinline__ void list_insert(float *ld, uint32_t *li, uint32_t k, float d, uint32_t id) {
    const uint32_t lane = lane_id();
    if (!cand_less(d, id, ld[k - 1], li[k - 1])) return;
    uint32_t pos = 0;
    for (uint32_t base = 0; base < k; base += 32) {
        const uint32_t i = base + lane;
        const bool before = (i < k) && cand_less(ld[i], li[i], d, id);
        pos += __popc(__ballot_sync(kFullMask, before));
    }
    // shift [pos, k-1) right by one, from the tail
    for (int base = (int) ((k - 1) / 32) * 32; base >= 0; base -= 32) {
        const uint32_t i = base + lane;
        float td = 0.0f;
        uint32_t ti = 0;
        const bool mv = (i >= pos) && (i + 1 < k);
        if (mv) { td = ld[i]; ti = li[i]; }
        __syncwarp();
        if (mv) { ld[i + 1] = td; li[i + 1] = ti; }
        __syncwarp();
    }
    if (lane == 0) { ld[pos] = d; li[pos] = id; }
    __syncwarp();
}

__global__ void __launch_bounds__(256) bruteforce_tile_kernel(const float *__restrict__ base, uint32_t n,
                                                              const float *__restrict__ queries, uint32_t Q,
                                                              uint32_t dim, uint32_t k, uint32_t splits,
                                                              Cand *__restrict__ partial) {
    extern __shared__ __align__(16) uint32_t smem[];
    float *Qs = reinterpret_cast<float *>(smem);                  // [kKT][kQPad]
    float *Bs = Qs + kKT * kQPad;                                 // [kKT][kBPad]
    float *ld = Bs + kKT * kBPad;                                 // [kQT][k]
    uint32_t *li = reinterpret_cast<uint32_t *>(ld + kQT * k);    // [kQT][k]
    Cand *queue = reinterpret_cast<Cand *>(li + kQT * k);         // [kQT][kBT]
    uint32_t *qcount = reinterpret_cast<uint32_t *>(queue + kQT * kBT);  // [kQT]

    const uint32_t tid = threadIdx.x, lane = lane_id(), warp = tid >> 5;
    const uint32_t tx = tid & 15, ty = tid >> 4;
    const uint32_t q0 = blockIdx.x * kQT;
    const uint32_t split = blockIdx.y;
    const uint32_t rows_per_split = (n + splits - 1) / splits;
    const uint32_t r_begin = split * rows_per_split;
    const uint32_t r_end = min(n, r_begin + rows_per_split);

    for (uint32_t i = tid; i < kQT * k; i += 256) { ld[i] = FLT_MAX; li[i] = kInvalid; }
    if (tid < kQT) qcount[tid] = 0;
    __syncthreads();

    for (uint32_t r0 = r_begin; r0 < r_end; r0 += kBT) {
        float acc[4][8];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 8; j++) acc[i][j] = 0.0f;

        for (uint32_t k0 = 0; k0 < dim; k0 += kKT) {
            // stage Q tile (64 rows x 32 dims) and B tile (128 rows x 32 dims), transposed
            for (uint32_t e = tid; e < kQT * kKT; e += 256) {
                const uint32_t row = e / kKT, kk = e % kKT;
                const uint32_t q = q0 + row, d = k0 + kk;
                Qs[kk * kQPad + row] = (q < Q && d < dim) ? __ldg(queries + (uint64_t) q * dim + d) : 0.0f;
            }
            for (uint32_t e = tid; e < kBT * kKT; e += 256) {
                const uint32_t row = e / kKT, kk = e % kKT;
                const uint32_t r = r0 + row, d = k0 + kk;
                Bs[kk * kBPad + row] = (r < r_end && d < dim) ? __ldg(base + (uint64_t) r * dim + d) : 0.0f;
            }
            __syncthreads();
#pragma unroll 8
            for (int kk = 0; kk < kKT; kk++) {
                const float4 qa = *reinterpret_cast<const float4 *>(Qs + kk * kQPad + 4 * ty);
                const float4 b0 = *reinterpret_cast<const float4 *>(Bs + kk * kBPad + 8 * tx);
                const float4 b1 = *reinterpret_cast<const float4 *>(Bs + kk * kBPad + 8 * tx + 4);
                const float qv[4] = {qa.x, qa.y, qa.z, qa.w};
                const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const float df = qv[i] - bv[j];
                        acc[i][j] = __fmaf_rn(df, df, acc[i][j]);
                    }
            }
            __syncthreads();
        }
        // queue rows that can enter a list
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t ql = 4 * ty + i;
            if (q0 + ql >= Q) continue;
            const float thr = ld[ql * k + k - 1];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const uint32_t r = r0 + 8 * tx + j;
                if (r < r_end && acc[i][j] <= thr) {
                    const uint32_t slot = atomicAdd(&qcount[ql], 1u);
                    queue[ql * kBT + slot] = Cand{acc[i][j], r};
                }
            }
        }
        __syncthreads();
        for (uint32_t ql = warp; ql < kQT; ql += 8) {
            const uint32_t m = qcount[ql];
            for (uint32_t c = 0; c < m; c++) {
                const Cand cd = queue[ql * kBT + c];
                list_insert(ld + ql * k, li + ql * k, k, cd.d, cd.id);
            }
            __syncwarp();
            if (lane == 0) qcount[ql] = 0;
        }
        __syncthreads();
    }
    for (uint32_t i = tid; i < kQT * k; i += 256) {
        const uint32_t ql = i / k, j = i % k;
        if (q0 + ql < Q) partial[((uint64_t) (q0 + ql) * splits + split) * k + j] = Cand{ld[i], li[i]};
    }
}

// One warp per query folds the per-split lists.
__global__ void __launch_bounds__(128) bruteforce_merge_kernel(const Cand *__restrict__ partial, uint32_t Q, uint32_t k,
                                                               uint32_t splits, int metric, uint32_t *out_ids,
                                                               float *out_dists) {
    extern __shared__ __align__(16) uint32_t smem[];
    const uint32_t warp = threadIdx.x >> 5, lane = lane_id();
    const uint32_t q = blockIdx.x * (blockDim.x >> 5) + warp;
    if (q >= Q) return;
    float *ld = reinterpret_cast<float *>(smem) + (size_t) warp * 2 * k;
    uint32_t *li = reinterpret_cast<uint32_t *>(ld + k);
    for (uint32_t i = lane; i < k; i += 32) { ld[i] = FLT_MAX; li[i] = kInvalid; }
    __syncwarp();
    const Cand *src = partial + (uint64_t) q * splits * k;
    for (uint32_t c = 0; c < splits * k; c++) {
        const Cand cd = src[c];
        if (cd.id != kInvalid) list_insert(ld, li, k, cd.d, cd.id);
    }
    for (uint32_t i = lane; i < k; i += 32) {
        out_ids[(uint64_t) q * k + i] = li[i];
        if (out_dists) out_dists[(uint64_t) q * k + i] = finish_metric(ld[i], metric);
    }
}

// ---------------------------------------------------------------------------
// Per-partition exact kNN graph: every row against all rows of its own partition. This
// is the kNN stage for partitions small enough that all pairs cost less than NN-descent
// would. A CTA owns up to 64 rows of one partition (tile table built on the host) and
// walks that partition in tiles of 128 rows; rows beating the current k-th best are
// queued as 64-bit keys (distance bits | local id), and after every tile one warp per row
// sorts its queue in registers and folds it into the row's sorted list with one bitonic
// merge. Output: partition-local ids, self excluded, nearest first.
// ---------------------------------------------------------------------------
constexpr u64 kNoKey = ((u64) 0x7f7fffffu << 32) | 0xffffffffull;

struct SegTile {
    uint32_t seg_start, seg_len, first;  // rows [seg_start + first, +64) of the segment
};

template<int NL>  // list width = 32 * NL
__global__ void __launch_bounds__(256, 2) segment_knn_kernel(const float *__restrict__ data, uint32_t dim,
                                                             const SegTile *__restrict__ tiles, int32_t *out,
                                                             uint32_t out_degree, uint32_t row_base) {
    extern __shared__ __align__(16) uint32_t smem[];
    constexpr uint32_t L = 32u * NL;
    float *Qs = reinterpret_cast<float *>(smem);                 // [kKT][kQPad]
    float *Bs = Qs + kKT * kQPad;                                // [kKT][kBPad]
    u64 *lists = reinterpret_cast<u64 *>(Bs + kKT * kBPad);      // [kQT][L]
    u64 *queue = lists + kQT * L;                                // [kQT][kBT]
    uint32_t *qcount = reinterpret_cast<uint32_t *>(queue + kQT * kBT);  // [kQT]

    const SegTile t = tiles[blockIdx.x];
    const uint32_t tid = threadIdx.x, lane = lane_id(), warp = tid >> 5;
    const uint32_t tx = tid & 15, ty = tid >> 4;
    const float *seg = data + (uint64_t) t.seg_start * dim;
    const uint32_t nq = min((uint32_t) kQT, t.seg_len - t.first);

    for (uint32_t i = tid; i < kQT * L; i += 256) lists[i] = kNoKey;
    if (tid < kQT) qcount[tid] = 0;
    __syncthreads();

    for (uint32_t r0 = 0; r0 < t.seg_len; r0 += kBT) {
        float acc[4][8];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 8; j++) acc[i][j] = 0.0f;
        for (uint32_t k0 = 0; k0 < dim; k0 += kKT) {
            for (uint32_t e = tid; e < kQT * kKT; e += 256) {
                const uint32_t row = e / kKT, kk = e % kKT;
                const uint32_t d = k0 + kk;
                Qs[kk * kQPad + row] = (row < nq && d < dim) ? __ldg(seg + (uint64_t) (t.first + row) * dim + d) : 0.0f;
            }
            for (uint32_t e = tid; e < kBT * kKT; e += 256) {
                const uint32_t row = e / kKT, kk = e % kKT;
                const uint32_t r = r0 + row, d = k0 + kk;
                Bs[kk * kBPad + row] = (r < t.seg_len && d < dim) ? __ldg(seg + (uint64_t) r * dim + d) : 0.0f;
            }
            __syncthreads();
#pragma unroll 8
            for (int kk = 0; kk < kKT; kk++) {
                const float4 qa = *reinterpret_cast<const float4 *>(Qs + kk * kQPad + 4 * ty);
                const float4 b0 = *reinterpret_cast<const float4 *>(Bs + kk * kBPad + 8 * tx);
                const float4 b1 = *reinterpret_cast<const float4 *>(Bs + kk * kBPad + 8 * tx + 4);
                const float qv[4] = {qa.x, qa.y, qa.z, qa.w};
                const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const float df = qv[i] - bv[j];
                        acc[i][j] = __fmaf_rn(df, df, acc[i][j]);
                    }
            }
            __syncthreads();
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t ql = 4 * ty + i;
            if (ql >= nq) continue;
            const u64 thr = lists[ql * L + L - 1];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const uint32_t r = r0 + 8 * tx + j;
                if (r >= t.seg_len || r == t.first + ql) continue;
                const u64 key = ((u64) __float_as_uint(acc[i][j]) << 32) | r;
                if (key < thr) queue[ql * kBT + atomicAdd(&qcount[ql], 1u)] = key;
            }
        }
        __syncthreads();
        for (uint32_t ql = warp; ql < nq; ql += 8) {
            const uint32_t m = qcount[ql];
            if (m == 0) continue;
            u64 *q = queue + ql * kBT;
            u64 *list = lists + ql * L;
            // sort the queue (<= 128 keys) ascending, in place
            if (m <= 32) {
                u64 k1[1] = {lane < m ? q[lane] : kNoKey};
                sort_u64<1>(k1);
                __syncwarp();
                q[lane] = k1[0];
                for (uint32_t j = 32 + lane; j < L; j += 32) q[j] = kNoKey;
            } else {
                u64 k4[4];
#pragma unroll
                for (int i = 0; i < 4; i++) k4[i] = (4 * lane + i < m) ? q[4 * lane + i] : kNoKey;
                sort_u64<4>(k4);
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 4; i++) q[4 * lane + i] = k4[i];
            }
            __syncwarp();
            // the L smallest of list and queue: list[j] against queue[L-1-j], then one merge phase
            u64 keys[NL];
#pragma unroll
            for (int i = 0; i < NL; i++) {
                const uint32_t j = NL * lane + i;
                const u64 a = list[j], b = q[L - 1 - j];
                keys[i] = a < b ? a : b;
            }
            merge_final_u64<NL>(keys);
#pragma unroll
            for (int i = 0; i < NL; i++) list[NL * lane + i] = keys[i];
            if (lane == 0) qcount[ql] = 0;
        }
        __syncthreads();
    }
    for (uint32_t i = tid; i < nq * out_degree; i += 256) {
        const uint32_t ql = i / out_degree, j = i % out_degree;
        const uint32_t id = (uint32_t) lists[ql * L + j];
        const uint64_t flat = (uint64_t) (t.seg_start + t.first + ql) * out_degree + j;
        uint32_t u = (uint32_t) (flat + (uint64_t) row_base * out_degree);  // xorshift32, utils.cuh:14-19, as nn_descent.cuh:1384-1391 pads short rows
        u ^= u >> 13; u ^= u << 27; u ^= u >> 5; u *= 0x9E3779B9u;
        out[flat] = (int32_t) (id < t.seg_len ? id : u % t.seg_len);
    }
}

size_t segment_knn_smem_bytes(uint32_t L) {
    return (size_t) (kKT * kQPad + kKT * kBPad) * 4 + (size_t) kQT * L * 8 + (size_t) kQT * kBT * 8 + kQT * 4;
}

size_t tile_smem_bytes(uint32_t k) {
    return (size_t) (kKT * kQPad + kKT * kBPad + 2 * kQT * k + 2 * kQT * kBT + kQT) * 4;
}

}  // namespace

uint32_t bruteforce_default_splits(uint32_t n, uint32_t Q) {
    // enough CTAs for two waves of 148 SMs, slices of at least 8 tiles
    const uint32_t qblocks = (Q + kQT - 1) / kQT;
    uint32_t splits = (2 * 148 + qblocks - 1) / qblocks;
    const uint32_t max_splits = (n + 8 * kBT - 1) / (8 * kBT);
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    if (splits > 64) splits = 64;
    return splits;
}

size_t bruteforce_scratch_bytes(uint32_t Q, uint32_t k, uint32_t splits) {
    return (size_t) Q * splits * k * sizeof(Cand);
}

cudaError_t launch_bruteforce(const float *base, uint32_t n, const float *queries, uint32_t Q, uint32_t dim,
                              uint32_t k, int metric, uint32_t splits, void *scratch, uint32_t *out_ids,
                              float *out_dists, cudaStream_t stream) {
    if (Q == 0) return cudaSuccess;
    if (k == 0 || k > kMaxK || k > n || splits == 0) return cudaErrorInvalidValue;
    const size_t smem_bytes = tile_smem_bytes(k);
    cudaError_t e = cudaFuncSetAttribute(bruteforce_tile_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int) smem_bytes);
    if (e != cudaSuccess) return e;
    const dim3 grid((Q + kQT - 1) / kQT, splits);
    bruteforce_tile_kernel<<<grid, 256, smem_bytes, stream>>>(base, n, queries, Q, dim, k, splits,
                                                             static_cast<Cand *>(scratch));
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const uint32_t warps = 4;
    bruteforce_merge_kernel<<<(Q + warps - 1) / warps, warps * 32, (size_t) warps * 2 * k * 4, stream>>>(
        static_cast<const Cand *>(scratch), Q, k, splits, metric, out_ids, out_dists);
    return cudaGetLastError();
}

uint32_t segment_knn_tile_count(const uint32_t *h_seg_len, uint32_t S, uint32_t max_len) {
    uint32_t tiles = 0;
    for (uint32_t s = 0; s < S; s++)
        if (h_seg_len[s] > 0 && h_seg_len[s] <= max_len) tiles += (h_seg_len[s] + kQT - 1) / kQT;
    return tiles;
}

void segment_knn_fill_tiles(const uint32_t *h_seg_start, const uint32_t *h_seg_len, uint32_t S, uint32_t max_len,
                            uint32_t *h_tiles) {
    SegTile *t = reinterpret_cast<SegTile *>(h_tiles);
    for (uint32_t s = 0; s < S; s++) {
        if (h_seg_len[s] == 0 || h_seg_len[s] > max_len) continue;
        for (uint32_t first = 0; first < h_seg_len[s]; first += kQT) *t++ = SegTile{h_seg_start[s], h_seg_len[s], first};
    }
}

cudaError_t launch_segment_knn(const float *data, uint32_t dim, const uint32_t *d_tiles, uint32_t tile_count,
                               uint32_t out_degree, uint32_t row_base, int32_t *out, cudaStream_t stream) {
    if (tile_count == 0) return cudaSuccess;
    if (out_degree == 0 || out_degree > 64) return cudaErrorInvalidValue;
    const uint32_t L = out_degree <= 32 ? 32 : 64;
    const size_t smem_bytes = segment_knn_smem_bytes(L);
    cudaError_t e;
    if (L == 32) {
        e = cudaFuncSetAttribute(segment_knn_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_bytes);
        if (e != cudaSuccess) return e;
        segment_knn_kernel<1><<<tile_count, 256, smem_bytes, stream>>>(data, dim, reinterpret_cast<const SegTile *>(d_tiles), out, out_degree, row_base);
    } else {
        e = cudaFuncSetAttribute(segment_knn_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_bytes);
        if (e != cudaSuccess) return e;
        segment_knn_kernel<2><<<tile_count, 256, smem_bytes, stream>>>(data, dim, reinterpret_cast<const SegTile *>(d_tiles), out, out_degree, row_base);
    }
    return cudaGetLastError();
}

}  // namespace glide
