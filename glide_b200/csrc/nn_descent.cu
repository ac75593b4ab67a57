// Segmented NN-descent: the kNN graph of every partition, entirely on the GPU.
//
// It produces what the reference's GNND::build produces (nn_descent.cuh:1238-1403): for
// every row of the reordered data set its `out_degree` approximate nearest neighbours
// inside the row's own partition, as partition-local ids. The algorithm is this
// repository's own and is judged by graph recall, not bit parity (the reference's
// result depends on thread timing, nn_descent.cuh:509-579, :1304-1343):
//
//  * lists are K sorted 64-bit keys per row (distance bits | id | "new" flag);
//  * per round: sample (<= S new + <= S old per row, plus hashed reverse samples),
//    local join (one CTA per row: fp32 (a-b)^2 distance tile of new x (new+old) held in
//    registers, staged through shared memory; every participant keeps its best few
//    partners), proposals go to per-row slots with 64-bit atomicMin (order independent),
//    and a warp per row merges its slots into the list with a bitonic network;
//  * no host work inside a round except reading one update counter.
// Every step is a pure function of the previous state, so a run is reproducible.
// Distances inside the lists are squared L2 for both metrics (monotone in the
// reference's values; only ids leave this stage).
#include <vector>

#include "beam_core.cuh"
#include "kernels.h"

namespace glide {

namespace {

constexpr uint32_t kP = 32;             // proposal slots per row
constexpr uint32_t kBestSlots = 4;      // partners kept per participant per join
constexpr uint32_t kMaxS = 32;          // samples per direction
constexpr uint32_t kEmptyId = 0x7fffffffu;
constexpr u64 kEmptyKey = ((u64) 0x7f7fffffu << 32) | 0xffffffffull;  // (FLT_MAX, empty id, flag)

__device__ __forceinline__ u64 make_key(float d, uint32_t id, uint32_t is_new) {
    return ((u64) __float_as_uint(d) << 32) | ((u64) id << 1) | is_new;
}
__device__ __forceinline__ uint32_t key_id(u64 k) { return ((uint32_t) k) >> 1; }
__device__ __forceinline__ uint32_t key_new(u64 k) { return (uint32_t) k & 1u; }
__device__ __forceinline__ float key_dist(u64 k) { return __uint_as_float((uint32_t) (k >> 32)); }

__host__ __device__ __forceinline__ uint32_t hash32(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
    return x;
}

struct NndDev {
    const float *data;
    uint32_t rows, dim;
    const uint32_t *seg_start, *seg_len, *row_segment;
    uint32_t K, S;
    uint32_t seed;
    uint32_t min_len;  // rows of shorter partitions are skipped by every kernel
    uint32_t row_base; // index of row 0 within the whole reordered set
    u64 *lists;       // rows x K, ascending
    u64 *props;       // rows x kP
    uint32_t *new_s;  // rows x 2S  (forward | reverse)
    uint32_t *old_s;  // rows x 2S
    uint32_t *seg_updates;        // S counters: list entries replaced in the current round, per partition
    const uint32_t *seg_active;   // S flags: 0 once a partition has converged (its rows are skipped from then on)
};

__device__ __forceinline__ uint32_t gcd_u32(uint32_t a, uint32_t b) {
    while (b) { const uint32_t t = a % b; a = b; b = t; }
    return a;
}

// Initial lists: K distinct pseudo-random members of the row's partition (an arithmetic
// progression with a row-specific stride coprime to the partition size), with their
// true distances, all flagged new. The reference starts from random ids with distance
// FLT_MAX (nn_descent.cuh:1003-1038). Also clears the row's proposal slots.
template<int NK>
__global__ void __launch_bounds__(256) nnd_init_kernel(const NndDev d) {
    extern __shared__ __align__(16) uint32_t smem[];
    const uint32_t warp = threadIdx.x >> 5, lane = lane_id(), team = lane / kTeam;
    const uint32_t row = blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= d.rows) return;
    constexpr uint32_t K = 32u * NK;
    uint32_t *strip = smem + (size_t) warp * (dim_pad4(d.dim) + 2 * K);
    float *query = reinterpret_cast<float *>(strip);
    uint32_t *ids = strip + dim_pad4(d.dim);
    float *dists = reinterpret_cast<float *>(ids + K);
    const uint32_t seg = d.row_segment[row];
    const uint32_t start = d.seg_start[seg], len = d.seg_len[seg], self = row - start;
    if (len < d.min_len) return;
    load_query(query, d.data + (uint64_t) row * d.dim, d.dim);
    uint32_t stride = 1;
    if (len > 2) {
        stride = 1 + hash32((row + d.row_base) ^ d.seed) % (len - 1);
        for (int tries = 0; tries < 64 && gcd_u32(stride, len) != 1; tries++) stride = stride % (len - 1) + 1;
        if (gcd_u32(stride, len) != 1) stride = 1;
    }
    for (uint32_t j = lane; j < K; j += 32)
        ids[j] = (j + 1 < len) ? (uint32_t) ((self + (u64) (j + 1) * stride) % len) : kEmptyId;
    __syncwarp();
    for (uint32_t j0 = 0; j0 < K; j0 += kTeamsPerWarp) {
        const uint32_t j = j0 + team;
        const uint32_t id = ids[j];
        const bool active = id != kEmptyId;
        const float part = team_partial(query, d.data + (uint64_t) (start + (active ? id : 0)) * d.dim, d.dim, active);
        const float sum = team_fold(part);
        if ((lane & (kTeam - 1)) == 0) dists[j] = sum;
    }
    __syncwarp();
    u64 keys[NK];
#pragma unroll
    for (int i = 0; i < NK; i++) {
        const uint32_t j = NK * lane + i;
        keys[i] = (ids[j] != kEmptyId) ? make_key(dists[j], ids[j], 1) : kEmptyKey;
    }
    sort_u64<NK>(keys);
#pragma unroll
    for (int i = 0; i < NK; i++) d.lists[(uint64_t) row * K + NK * lane + i] = keys[i];
    for (uint32_t j = lane; j < kP; j += 32) d.props[(uint64_t) row * kP + j] = kEmptyKey;
}

// Sampling (the reference samples on the host, nn_descent.cuh:1040-1104): the S nearest
// entries still flagged new become this round's "new" sample and lose the flag; the S
// nearest unflagged entries are the "old" sample. Every sampled edge row->v is also
// offered to v's reverse sample, slot hash(row) % S, smallest id wins.
__global__ void __launch_bounds__(256) nnd_sample_kernel(const NndDev d) {
    const uint32_t warp = threadIdx.x >> 5, lane = lane_id();
    const uint32_t row = blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= d.rows) return;
    const uint32_t K = d.K, S = d.S;
    const uint32_t seg = d.row_segment[row];
    if (d.seg_len[seg] < d.min_len || !d.seg_active[seg]) return;
    const uint32_t start = d.seg_start[seg], self = row - start;
    u64 *list = d.lists + (uint64_t) row * K;
    uint32_t *fnew = d.new_s + (uint64_t) row * 2 * S;
    uint32_t *fold = d.old_s + (uint64_t) row * 2 * S;
    const uint32_t rslot = S + hash32(self) % S;
    uint32_t n_new = 0, n_old = 0;
    for (uint32_t base = 0; base < K; base += 32) {
        const uint32_t e = base + lane;
        const u64 key = list[e];
        const uint32_t id = key_id(key);
        const bool valid = id != kEmptyId;
        const bool is_new = valid && key_new(key);
        const bool is_old = valid && !key_new(key);
        const uint32_t m_new = __ballot_sync(kFullMask, is_new);
        const uint32_t m_old = __ballot_sync(kFullMask, is_old);
        const uint32_t lt = (1u << lane) - 1;
        if (is_new) {
            const uint32_t r = n_new + __popc(m_new & lt);
            if (r < S) {
                fnew[r] = id;
                list[e] = key & ~1ull;
                atomicMin(d.new_s + (uint64_t) (start + id) * 2 * S + rslot, self);
            }
        }
        if (is_old) {
            const uint32_t r = n_old + __popc(m_old & lt);
            if (r < S) {
                fold[r] = id;
                atomicMin(d.old_s + (uint64_t) (start + id) * 2 * S + rslot, self);
            }
        }
        n_new += __popc(m_new);
        n_old += __popc(m_old);
    }
}

constexpr int kJT = 32;                  // dimension step of the join tile
constexpr int kJM = 4 * kMaxS;           // participants per join (new fwd+rev, old fwd+rev)
constexpr int kJPad = kJM + 4;

// Local join, one CTA (256 threads) per row. Participants: de-duplicated new ids
// (<= 2S) then old ids (<= 2S). Pairs: new x new (upper triangle) and new x old, the
// pairs of nn_descent.cuh:783-796, :862-875. Each participant keeps, per group of
// partner columns, the nearest partner that beats its current worst list entry, and
// those few are proposed to its row.
__global__ void __launch_bounds__(256) nnd_join_kernel(const NndDev d) {
    __shared__ __align__(16) float tile[kJT * kJPad];
    __shared__ uint32_t raw[kJM];
    __shared__ uint32_t ids[kJM];
    __shared__ float worst[kJM];
    __shared__ u64 best[kJM * kBestSlots];
    __shared__ uint32_t warp_cnt[4];

    const uint32_t row = blockIdx.x;
    const uint32_t tid = threadIdx.x, lane = lane_id(), warp = tid >> 5;
    const uint32_t S = d.S, K = d.K;
    const uint32_t seg = d.row_segment[row];
    if (d.seg_len[seg] < d.min_len || !d.seg_active[seg]) return;
    const uint32_t start = d.seg_start[seg];

    // raw ids: [0,2S) new, [2S,4S) old
    if (tid < 4 * S) {
        const uint32_t half = tid / (2 * S), off = tid % (2 * S);
        raw[tid] = (half == 0 ? d.new_s : d.old_s)[(uint64_t) row * 2 * S + off];
    }
    for (uint32_t i = tid; i < kJM * kBestSlots; i += 256) best[i] = kEmptyKey;
    __syncthreads();
    bool keep = false;
    uint32_t my_id = kInvalid;
    if (tid < 4 * S) {
        my_id = raw[tid];
        keep = my_id != kInvalid;
        if (keep) {
            const bool is_old = tid >= 2 * S;
            const uint32_t lo = is_old ? 0 : 0, hi = tid;  // everything before me (new before old)
            for (uint32_t j = lo; j < hi; j++)
                if (raw[j] == my_id) { keep = false; break; }
        }
    }
    // stable compaction: new first, then old. 2S is a multiple of 32 only when S >= 16;
    // handle the general case with two ballots per warp.
    const bool is_new_slot = tid < 2 * S;
    const uint32_t m_new = __ballot_sync(kFullMask, keep && is_new_slot);
    const uint32_t m_old = __ballot_sync(kFullMask, keep && !is_new_slot);
    if (warp < 4 && lane == 0) warp_cnt[warp] = (uint32_t) __popc(m_new) | ((uint32_t) __popc(m_old) << 16);
    __syncthreads();
    uint32_t nnew = 0, nold = 0, new_before = 0, old_before = 0;
    for (uint32_t w = 0; w < 4; w++) {
        const uint32_t c = warp_cnt[w];
        if (w < warp) { new_before += c & 0xffff; old_before += c >> 16; }
        nnew += c & 0xffff;
        nold += c >> 16;
    }
    if (nnew == 0) return;
    const uint32_t M = nnew + nold;
    if (keep) {
        const uint32_t lt = (1u << lane) - 1;
        const uint32_t pos = is_new_slot ? new_before + __popc(m_new & lt) : nnew + old_before + __popc(m_old & lt);
        ids[pos] = my_id;
        worst[pos] = key_dist(d.lists[(uint64_t) (start + my_id) * K + K - 1]);
    }
    __syncthreads();

    const uint32_t tx = tid & 15, ty = tid >> 4;
    const bool tile_active = (4 * ty < nnew) && (8 * tx < M);
    float acc[4][8];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.0f;

    for (uint32_t k0 = 0; k0 < d.dim; k0 += kJT) {
        for (uint32_t e = tid; e < M * kJT; e += 256) {
            const uint32_t m = e / kJT, kk = e % kJT;
            const uint32_t dd = k0 + kk;
            tile[kk * kJPad + m] = (dd < d.dim) ? __ldg(d.data + (uint64_t) (start + ids[m]) * d.dim + dd) : 0.0f;
        }
        __syncthreads();
        if (tile_active) {
#pragma unroll 8
            for (int kk = 0; kk < kJT; kk++) {
                const float4 a = *reinterpret_cast<const float4 *>(tile + kk * kJPad + 4 * ty);
                const float4 b0 = *reinterpret_cast<const float4 *>(tile + kk * kJPad + 8 * tx);
                const float4 b1 = *reinterpret_cast<const float4 *>(tile + kk * kJPad + 8 * tx + 4);
                const float av[4] = {a.x, a.y, a.z, a.w};
                const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const float df = av[i] - bv[j];
                        acc[i][j] = __fmaf_rn(df, df, acc[i][j]);
                    }
            }
        }
        __syncthreads();
    }

    if (tile_active) {
        u64 rbest[4], cbest[8];
#pragma unroll
        for (int i = 0; i < 4; i++) rbest[i] = kEmptyKey;
#pragma unroll
        for (int j = 0; j < 8; j++) cbest[j] = kEmptyKey;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t r = 4 * ty + i;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const uint32_t c = 8 * tx + j;
                const bool valid = (r < nnew) && (c < M) && (c >= nnew || c > r);
                if (!valid) continue;
                const float dist = acc[i][j];
                if (dist < worst[r]) {
                    const u64 k = make_key(dist, ids[c], 1);
                    if (k < rbest[i]) rbest[i] = k;
                }
                if (dist < worst[c]) {
                    const u64 k = make_key(dist, ids[r], 1);
                    if (k < cbest[j]) cbest[j] = k;
                }
            }
        }
#pragma unroll
        for (int i = 0; i < 4; i++)
            if (rbest[i] != kEmptyKey) atomicMin(&best[(4 * ty + i) * kBestSlots + (tx % kBestSlots)], rbest[i]);
#pragma unroll
        for (int j = 0; j < 8; j++)
            if (cbest[j] != kEmptyKey) atomicMin(&best[(8 * tx + j) * kBestSlots + (ty % kBestSlots)], cbest[j]);
    }
    __syncthreads();
    for (uint32_t t = tid; t < M * kBestSlots; t += 256) {
        const u64 k = best[t];
        if (k == kEmptyKey) continue;
        const uint32_t target = start + ids[t / kBestSlots];
        atomicMin(d.props + (uint64_t) target * kP + hash32(key_id(k)) % kP, k);
    }
}

// Merge a row's proposal slots into its list: drop proposals already listed, sort the
// rest, take the K smallest of list and proposals with one bitonic merge, count how many
// proposals made it, and clear the slots for the next round.
template<int NK>
__global__ void __launch_bounds__(256) nnd_merge_kernel(const NndDev d) {
    const uint32_t warp = threadIdx.x >> 5, lane = lane_id();
    const uint32_t row = blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= d.rows) return;
    const uint32_t seg = d.row_segment[row];
    if (d.seg_len[seg] < d.min_len || !d.seg_active[seg]) return;
    constexpr uint32_t K = 32u * NK;
    u64 *list = d.lists + (uint64_t) row * K;
    u64 keys[NK];
#pragma unroll
    for (int i = 0; i < NK; i++) keys[i] = list[NK * lane + i];
    u64 prop[1] = {d.props[(uint64_t) row * kP + lane]};
    const uint32_t any = __ballot_sync(kFullMask, prop[0] != kEmptyKey);
    if (any == 0) return;
    d.props[(uint64_t) row * kP + lane] = kEmptyKey;
    // drop proposals whose id is already in the list
    const uint32_t pid = key_id(prop[0]);
#pragma unroll
    for (int i = 0; i < NK; i++) {
        for (uint32_t l = 0; l < 32; l++) {
            const u64 o = __shfl_sync(kFullMask, keys[i], l);
            if (key_id(o) == pid) prop[0] = kEmptyKey;
        }
    }
    sort_u64<1>(prop);
    // position j = NK*lane + i of the list pairs with proposal K-1-j (ascending list against
    // descending proposals gives a bitonic sequence holding the K smallest)
    uint32_t inserted = 0;
#pragma unroll
    for (int i = 0; i < NK; i++) {
        const uint32_t j = NK * lane + i;
        const uint32_t pj = K - 1 - j;
        const u64 cand = __shfl_sync(kFullMask, prop[0], pj & 31u);
        const bool take = (pj < 32) && (cand < keys[i]);
        if (take) keys[i] = cand;
        inserted += __popc(__ballot_sync(kFullMask, take));
    }
    merge_final_u64<NK>(keys);
#pragma unroll
    for (int i = 0; i < NK; i++) list[NK * lane + i] = keys[i];
    if (lane == 0 && inserted) atomicAdd(d.seg_updates + seg, inserted);
}

// Final shrink (nn_descent.cuh:1376-1392): the first out_degree ids per row; an empty
// slot is replaced by xorshift32(flat index) % partition size as there.
__device__ __forceinline__ uint32_t xorshift32(uint32_t u) {  // utils.cuh:14-19
    u ^= u >> 13; u ^= u << 27; u ^= u >> 5;
    return u * 0x9E3779B9u;
}
__global__ void nnd_output_kernel(const NndDev d, int32_t *out, uint32_t out_degree) {
    const uint64_t t = (uint64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (uint64_t) d.rows * out_degree) return;
    const uint32_t row = (uint32_t) (t / out_degree), j = (uint32_t) (t % out_degree);
    const uint32_t len = d.seg_len[d.row_segment[row]];
    if (len < d.min_len) return;
    const uint32_t id = key_id(d.lists[(uint64_t) row * d.K + j]);
    out[t] = (int32_t) ((id < len) ? id : xorshift32((uint32_t) (t + (uint64_t) d.row_base * out_degree)) % len);
}

__global__ void row_segment_kernel(const uint32_t *seg_start, const uint32_t *seg_len, uint32_t S, uint32_t rows,
                                   uint32_t *row_segment) {
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    uint32_t s = 0;
    while (s + 1 < S && r >= seg_start[s] + seg_len[s]) s++;
    row_segment[r] = s;
}

size_t align256(size_t x) { return (x + 255) & ~(size_t) 255; }

}  // namespace

size_t nnd_workspace_bytes(uint32_t rows, uint32_t K, uint32_t sample, uint32_t S) {
    return align256((size_t) rows * K * 8) + align256((size_t) rows * kP * 8) +
           2 * align256((size_t) rows * 2 * sample * 4) + align256((size_t) rows * 4) + 2 * align256((size_t) S * 4) + 256;
}

cudaError_t run_nn_descent(const NndArgs &a, cudaStream_t stream) {
    if (a.rows == 0) return cudaSuccess;
    if ((a.K != 32 && a.K != 64) || a.sample == 0 || a.sample > kMaxS || a.out_degree > a.K)
        return cudaErrorInvalidValue;
    if (a.workspace_bytes < nnd_workspace_bytes(a.rows, a.K, a.sample, a.S)) return cudaErrorInvalidValue;
    NndDev d;
    d.data = a.data; d.rows = a.rows; d.dim = a.dim;
    d.seg_start = a.seg_start; d.seg_len = a.seg_len;
    d.K = a.K; d.S = a.sample; d.seed = (uint32_t) (a.seed * 0x9E3779B97F4A7C15ull >> 32);
    d.min_len = a.min_seg_len;
    d.row_base = a.row_base;
    char *w = static_cast<char *>(a.workspace);
    d.lists = reinterpret_cast<u64 *>(w); w += align256((size_t) a.rows * a.K * 8);
    d.props = reinterpret_cast<u64 *>(w); w += align256((size_t) a.rows * kP * 8);
    d.new_s = reinterpret_cast<uint32_t *>(w); w += align256((size_t) a.rows * 2 * a.sample * 4);
    d.old_s = reinterpret_cast<uint32_t *>(w); w += align256((size_t) a.rows * 2 * a.sample * 4);
    uint32_t *row_segment = reinterpret_cast<uint32_t *>(w); w += align256((size_t) a.rows * 4);
    d.seg_updates = reinterpret_cast<uint32_t *>(w); w += align256((size_t) a.S * 4);
    uint32_t *seg_active = reinterpret_cast<uint32_t *>(w);
    d.seg_active = seg_active;
    d.row_segment = row_segment;
    // Convergence is judged per partition (as the reference does, nn_descent.cuh:1280-1283): which
    // partitions share a call does not change any partition's result.
    std::vector<uint32_t> h_len(a.S), h_active(a.S), h_updates(a.S);
    cudaError_t e0 = cudaMemcpyAsync(h_len.data(), a.seg_len, (size_t) a.S * 4, cudaMemcpyDeviceToHost, stream);
    if (e0 == cudaSuccess) e0 = cudaStreamSynchronize(stream);
    if (e0 != cudaSuccess) return e0;
    uint32_t live = 0;
    for (uint32_t s2 = 0; s2 < a.S; s2++) { h_active[s2] = h_len[s2] >= a.min_seg_len ? 1u : 0u; live += h_active[s2]; }
    if ((e0 = cudaMemcpyAsync(seg_active, h_active.data(), (size_t) a.S * 4, cudaMemcpyHostToDevice, stream)) != cudaSuccess) return e0;

    cudaError_t e;
    row_segment_kernel<<<(a.rows + 255) / 256, 256, 0, stream>>>(a.seg_start, a.seg_len, a.S, a.rows, row_segment);
    const uint32_t warps = 8;
    const uint32_t wgrid = (a.rows + warps - 1) / warps;
    const size_t init_smem = (size_t) warps * (dim_pad4(a.dim) + 2 * a.K) * 4;
    if (a.K == 32) {
        if (init_smem > 48 * 1024) cudaFuncSetAttribute(nnd_init_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) init_smem);
        nnd_init_kernel<1><<<wgrid, warps * 32, init_smem, stream>>>(d);
    } else {
        if (init_smem > 48 * 1024) cudaFuncSetAttribute(nnd_init_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) init_smem);
        nnd_init_kernel<2><<<wgrid, warps * 32, init_smem, stream>>>(d);
    }
    if ((e = cudaGetLastError()) != cudaSuccess) return e;

    cudaEvent_t ev[5];
    const bool timing = a.stage_ms != nullptr;
    if (timing) {
        for (auto &x : ev) cudaEventCreate(&x);
        for (int i = 0; i < 4; i++) a.stage_ms[i] = 0.0f;
    }
    uint32_t it = 0;
    const size_t sample_bytes = (size_t) a.rows * 2 * a.sample * 4;
    for (; it < a.max_iterations; it++) {
        if (timing) cudaEventRecord(ev[0], stream);
        if ((e = cudaMemsetAsync(d.new_s, 0xff, sample_bytes, stream)) != cudaSuccess) return e;
        if ((e = cudaMemsetAsync(d.old_s, 0xff, sample_bytes, stream)) != cudaSuccess) return e;
        if ((e = cudaMemsetAsync(d.seg_updates, 0, (size_t) a.S * 4, stream)) != cudaSuccess) return e;
        nnd_sample_kernel<<<wgrid, warps * 32, 0, stream>>>(d);
        if (timing) cudaEventRecord(ev[1], stream);
        nnd_join_kernel<<<a.rows, 256, 0, stream>>>(d);
        if (timing) cudaEventRecord(ev[2], stream);
        if (a.K == 32) nnd_merge_kernel<1><<<wgrid, warps * 32, 0, stream>>>(d);
        else nnd_merge_kernel<2><<<wgrid, warps * 32, 0, stream>>>(d);
        if (timing) cudaEventRecord(ev[3], stream);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
        if ((e = cudaMemcpyAsync(h_updates.data(), d.seg_updates, (size_t) a.S * 4, cudaMemcpyDeviceToHost, stream)) != cudaSuccess) return e;
        if ((e = cudaStreamSynchronize(stream)) != cudaSuccess) return e;
        if (timing) {
            float ms;
            cudaEventElapsedTime(&ms, ev[0], ev[1]); a.stage_ms[0] += ms;
            cudaEventElapsedTime(&ms, ev[1], ev[2]); a.stage_ms[1] += ms;
            cudaEventElapsedTime(&ms, ev[2], ev[3]); a.stage_ms[2] += ms;
        }
        // the reference stops a partition when a sampled update count falls below
        // threshold * rows * dim / 100 (nn_descent.cuh:1280-1283); here: when fewer than
        // threshold * rows * K of its list entries changed in the round.
        bool changed = false;
        for (uint32_t s2 = 0; s2 < a.S; s2++) {
            if (!h_active[s2]) continue;
            if ((double) h_updates[s2] < (double) a.termination_threshold * h_len[s2] * a.K) {
                h_active[s2] = 0;
                live--;
                changed = true;
            }
        }
        if (changed && (e = cudaMemcpyAsync(seg_active, h_active.data(), (size_t) a.S * 4, cudaMemcpyHostToDevice, stream)) != cudaSuccess) return e;
        if (live == 0) { it++; break; }
    }
    if (timing) for (auto &x : ev) cudaEventDestroy(x);
    if (a.iterations_run) *a.iterations_run = it;
    const uint64_t total = (uint64_t) a.rows * a.out_degree;
    nnd_output_kernel<<<(uint32_t) ((total + 255) / 256), 256, 0, stream>>>(d, a.out_knn, a.out_degree);
    return cudaGetLastError();
}

}  // namespace glide
