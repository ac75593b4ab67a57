// Graph construction kernels: per-point beam search over the kNN subgraph +
// occlusion pruning (reference build_kernel, graph_kernel.cuh:249-316), boundary
// partition build + merge (:160-247, :318-376), reverse-edge insertion (:378-453) and
// refinement of rows that still have holes (:455-673). Large-path variants
// (:675-821) are the same kernels with one segment and no id map.
//
// One warp owns one point from search to row write; the beam stays in registers and
// is spilled to the warp's shared strip only for pruning.
#include <cstdlib>

#include "beam_core.cuh"
#include "kernels.h"
#include "scan.cuh"

namespace glide {

namespace {

struct BuildDev {
    BuildArgs a;
    uint32_t max_centroid;
    uint32_t strip_words;
    uint32_t max_beam;    // 32*NB
    uint32_t max_degree;  // round_up32(out_degree)
};

// Extra strip layout (words): picks[max_degree] row[max_degree] bits[max_degree/32].
struct PruneStrip {
    uint32_t *picks;
    uint32_t *row;
    uint32_t *bits;
};

__host__ __device__ inline uint32_t prune_strip_words(uint32_t max_degree) { return 2 * max_degree + max_degree / 32; }

__device__ __forceinline__ PruneStrip make_prune_strip(uint32_t *extra, uint32_t max_degree) {
    PruneStrip ps;
    ps.picks = extra;
    ps.row = ps.picks + max_degree;
    ps.bits = ps.row + max_degree;
    return ps;
}

// ---------------------------------------------------------------------------
// Register-resident pruning: sync_prune (graph_kernel.cuh:70-143) and its refine variant
// (:455-578) on the beam as it sits in registers (entry j = NB*lane + i), without a pool in
// shared memory. The reference compacts the pool after every pick; here an entry is a bit in
// alive[i] (bit l = lane l, register i), "first pool entry" is the alive entry with the smallest
// j, and dropping an entry clears its bit, which visits the same centres in the same order and
// tests the same pairs. build: the centre is pool[0], every other entry e is dropped when
// alpha * d(centre, e) < d(point, e). refine: the centre is the first entry that is neither the
// point nor already in its row, entries before it are dropped, and the centre itself goes through
// the test with the others (d = 0, so it stays only at distance 0 from the point).
// picks[0..limit) receives pool-relative ids, unused slots kInvalid. Returns rows read;
// *pool_size = entries that were filled.
// ---------------------------------------------------------------------------
template<int NB>
__device__ __forceinline__ uint32_t prune_lanes(const float (&bk)[NB], const uint32_t (&bv)[NB], uint32_t beam,
                                                const PruneStrip &ps, float *q_smem, uint32_t *ids_smem,
                                                const float *__restrict__ data,
                                                uint32_t dim, uint32_t degree, uint32_t max_degree, uint32_t limit,
                                                float alpha, int metric, bool refine, uint32_t point_id,
                                                uint32_t *pool_size) {
    const uint32_t lane = lane_id();
    for (uint32_t i = lane; i < max_degree; i += 32) ps.picks[i] = kInvalid;
    uint32_t id[NB], alive[NB], eligible[NB];
    uint32_t P = 0;
#pragma unroll
    for (int i = 0; i < NB; i++) {
        const uint32_t j = NB * lane + i;
        id[i] = bv[i] & kClean;
        const bool filled = (j < beam) && (id[i] != kPadClean);
        alive[i] = __ballot_sync(kFullMask, filled);
        P += __popc(alive[i]);
        bool ok = filled;
        if (refine && filled) {  // select_point (:455-492): not the point, not in its row
            ok = id[i] != point_id;
            for (uint32_t r = 0; r < degree && ok; r++) ok = ps.row[r] != id[i];
        }
        eligible[i] = __ballot_sync(kFullMask, ok);
    }
    *pool_size = P;
    __syncwarp();
    const bool fast = rows_fit_lanes(dim);
    const bool own = lane < (dim >> 2);
    uint32_t nsize = 0, rows = 0;
    while (nsize < limit) {
        uint32_t best = kInvalid;
#pragma unroll
        for (int i = 0; i < NB; i++) {
            const uint32_t m = alive[i] & eligible[i];
            if (m) best = min(best, (uint32_t) NB * ((uint32_t) __ffs(m) - 1u) + (uint32_t) i);
        }
        if (best == kInvalid) break;
        const uint32_t cl = best / NB, ci = best % NB;
        uint32_t mine = id[0];
#pragma unroll
        for (int i = 1; i < NB; i++) mine = ((uint32_t) i == ci) ? id[i] : mine;
        const uint32_t center = __shfl_sync(kFullMask, mine, cl);
        if (lane == 0) ps.picks[nsize] = center;
        nsize++;
#pragma unroll
        for (int i = 0; i < NB; i++) {
            if (refine) {  // entries before the centre leave the pool
                const uint32_t upto = ((uint32_t) i < ci) ? cl + 1 : cl;   // lanes 0 .. upto-1
                alive[i] &= ~(upto >= 32 ? 0xffffffffu : ((1u << upto) - 1u));
            } else if ((uint32_t) i == ci) {
                alive[i] &= ~(1u << cl);
            }
        }
        float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
        if (fast) {
            if (own) q = __ldg(reinterpret_cast<const float4 *>(data + (uint64_t) center * dim) + lane);
        } else {
            __syncwarp();
            load_query(q_smem, data + (uint64_t) center * dim, dim);
        }
#pragma unroll
        for (int i = 0; i < NB; i++) {
            if (alive[i] == 0) continue;
            rows += __popc(alive[i]);
            const float d = fast ? score_lanes_q4(q, own, data, dim, metric, alive[i], id[i], ids_smem)
                                 : score_lanes(q_smem, data, dim, metric, alive[i], id[i]);
            const bool occluded = ((alive[i] >> lane) & 1u) && (alpha * d < bk[i]);   // graph_kernel.cuh:103-114
            alive[i] &= ~__ballot_sync(kFullMask, occluded);
        }
    }
    __syncwarp();
    return rows;
}

// map_to_graph_boundary, graph_kernel.cuh:160-247. ps.picks holds the pruned result
// in reorder ids, ps.row the existing row. Writes the merged row to `out`.
__device__ __forceinline__ void boundary_merge(const PruneStrip &ps, const uint32_t *__restrict__ map,
                                               uint32_t degree, uint32_t max_degree, uint32_t *out) {
    const uint32_t lane = lane_id();
    for (uint32_t i = lane; i < max_degree / 32; i += 32) ps.bits[i] = 0;
    __syncwarp();
    uint32_t valid_num = 0, rep_num = 0;
    for (uint32_t base = 0; base < max_degree; base += 32) {
        const uint32_t i = base + lane;
        const bool valid = (i < degree) && (ps.picks[i] != kInvalid);
        const uint32_t index = valid ? __ldg(map + ps.picks[i]) : kInvalid;
        bool non_rep = true;
        uint32_t j = 0;
        if (valid) {
            for (j = 0; j < degree; j++) {
                const uint32_t e = ps.row[j];
                if (e == kInvalid) break;
                if (e == index) { non_rep = false; break; }
            }
        }
        const uint32_t m1 = __ballot_sync(kFullMask, valid && non_rep);
        const uint32_t m2 = __ballot_sync(kFullMask, valid && !non_rep);
        __syncwarp();
        if (valid && non_rep) ps.picks[valid_num + __popc(m1 & ((1u << lane) - 1))] = index;
        if (valid && !non_rep) atomicOr(&ps.bits[j / 32], 1u << (j % 32));
        valid_num += __popc(m1);
        rep_num += __popc(m2);
        __syncwarp();
    }
    if (rep_num >= degree / 2) {
        uint32_t pos_num = 0;
        for (uint32_t base = 0; base < max_degree && pos_num < valid_num; base += 32) {
            const uint32_t i = base + lane;
            const bool empty = (i < degree) && (ps.row[i] == kInvalid);
            const uint32_t mask = __ballot_sync(kFullMask, empty);
            if (empty) {
                const uint32_t pos = pos_num + __popc(mask & ((1u << lane) - 1));
                if (pos < valid_num) out[i] = ps.picks[pos];
            }
            pos_num += __popc(mask);
        }
    } else {
        const uint32_t max_need = degree / 2 - rep_num;
        const uint32_t need = valid_num < max_need ? valid_num : max_need;
        uint32_t pos_num = 0;
        for (uint32_t base = 0; base < max_degree && pos_num < need; base += 32) {
            const uint32_t gi = max_degree - 1 - (base + lane);
            const bool in_range = gi < degree;
            const bool rep = in_range && ((ps.bits[gi / 32] >> (gi % 32)) & 1u);
            const bool empty = in_range && (ps.row[gi] == kInvalid);
            const bool ok = in_range && (empty || !rep);
            const uint32_t mask = __ballot_sync(kFullMask, ok);
            if (ok) {
                const uint32_t pos = pos_num + __popc(mask & ((1u << lane) - 1));
                if (pos < need) out[gi] = ps.picks[pos];
            }
            pos_num += __popc(mask);
        }
    }
}

// LANES: adjacency rows searched have at most 32 entries; candidates stay in registers
// (beam_loop_lanes) and the strip holds no candidate arrays.
template<int NB, int NC, bool LANES>
__global__ void __launch_bounds__(256, NB <= 4 ? 4 : 2) build_kernel(const BuildDev d) {
    extern __shared__ __align__(16) uint32_t smem[];
    const BuildArgs &a = d.a;
    const uint32_t warps_per_cta = blockDim.x >> 5;
    const uint32_t warp = threadIdx.x >> 5, lane = lane_id();
    const uint32_t t = blockIdx.x * warps_per_cta + warp;
    if (t >= (a.count_dev ? __ldg(a.count_dev) : a.count)) return;
    const uint32_t point = a.first + (a.order ? a.order[t] : t);
    const BeamParams p{a.p.beam, a.p.max_iterations, a.p.min_iterations, a.p.hash_bit, a.p.hash_reset_interval};
    WarpStrip s = make_strip(smem + (size_t) warp * d.strip_words, a.dim, LANES ? kLaneScratch : 32u * NC, p.hash_bit);
    if constexpr (NB == 16) s.tail = smem + (size_t) (warp + 1) * d.strip_words - kTwoWarpScratch;
    PruneStrip ps = make_prune_strip(s.extra, d.max_degree);
    const uint32_t degree = a.out_degree;

    uint32_t rows = 0, prune_rows = 0, iters = 0;
    bool short_pool = false;
    float bk[NB];
    uint32_t bv[NB];

    if (a.mode == kModeBuild || a.mode == kModeBoundary) {
        uint32_t seg = a.fixed_segment;
        if (a.mode == kModeBuild) {  // graph_kernel.cuh:276-282
            // first partition that ends beyond the point; partitions lie one after another, so
            // their ends never decrease and a bisection finds what the reference's scan finds
            uint32_t lo = 0, hi = a.S;
            while (lo < hi) {
                const uint32_t mid = (lo + hi) >> 1;
                if (point < __ldg(a.seg_start + mid) + __ldg(a.seg_len + mid)) hi = mid; else lo = mid + 1;
            }
            seg = lo;
            if (seg == a.S) return;
        }
        const uint32_t seg_start = a.seg_start[seg];
        const float *pdata = a.data + (uint64_t) seg_start * a.dim;
        const uint32_t *pknn = a.graph_in + (uint64_t) seg_start * a.in_degree;
        load_query(s.query, a.data + (uint64_t) point * a.dim, a.dim);
        visited_clear(s.visited, p.hash_bit);
        __syncwarp();
        // The seed step compares the row's partition-local ids with the point's reorder
        // id, as the reference does (graph_kernel.cuh:295-298).
        bool wide = false;
        if constexpr (LANES) {
            float ck;
            uint32_t cv;
            rows += seed_lanes(s, a.start_points[seg], point, pknn, a.in_degree, p.hash_bit, pdata, a.dim, a.metric, ck, cv,
                               &wide);
            iters = beam_loop_lanes<NB>(bk, bv, s, p, point - seg_start, pknn, a.in_degree, pdata, a.dim, a.metric, &rows,
                                        ck, cv, wide);
        } else {
            rows += seed_from_row(s, a.start_points[seg], point, pknn, a.in_degree, p.hash_bit, pdata, a.dim, a.metric, &wide);
            iters = beam_loop<NB, NC, true>(bk, bv, s, p, point - seg_start, pknn, a.in_degree, pdata, a.dim, a.metric, &rows,
                                            wide);
        }
        uint32_t P;
        prune_rows = prune_lanes<NB>(bk, bv, p.beam, ps, s.query, LANES ? s.cand_id : nullptr, pdata, a.dim, degree, d.max_degree, degree, a.alpha, a.metric,
                                     false, kInvalid, &P);
        short_pool = P < p.beam;
        const uint32_t orig = a.map ? a.map[point] : point;
        uint32_t *out = a.graph_out + (uint64_t) (a.rows_by_point ? point - a.out_first : orig) * degree;
        if (a.mode == kModeBuild) {  // map_to_graph_sub / map_to_graph (:145-158)
            for (uint32_t i = lane; i < degree; i += 32) {
                const uint32_t id = ps.picks[i];
                out[i] = (id == kInvalid) ? kInvalid : (a.map ? a.map[id + seg_start] : id + seg_start);
            }
        } else {
            for (uint32_t i = lane; i < d.max_degree; i += 32) {
                ps.row[i] = (i < degree) ? out[i] : kInvalid;
                if (ps.picks[i] != kInvalid) ps.picks[i] += seg_start;
            }
            __syncwarp();
            boundary_merge(ps, a.map, degree, d.max_degree, out);
        }
    } else {
        // refine (graph_kernel.cuh:580-673, :730-821). Searches read graph_in, rows are
        // written to graph_out; the caller passes a snapshot as graph_in so that results
        // do not depend on the order in which points finish.
        const uint32_t *in_row = a.graph_in + (uint64_t) point * degree;
        uint32_t *out = a.graph_out + (uint64_t) (point - a.out_first) * degree;
        uint32_t need = 0;
        for (uint32_t base = 0; base < d.max_degree; base += 32) {
            const uint32_t i = base + lane;
            const uint32_t e = (i < degree) ? __ldg(in_row + i) : kInvalid;
            ps.row[i] = e;
            need += __popc(__ballot_sync(kFullMask, (i < degree) && (e == kInvalid)));
        }
        __syncwarp();
        if (need == 0) {
            if (out != in_row)
                for (uint32_t i = lane; i < degree; i += 32) out[i] = ps.row[i];
            return;
        }
        load_query(s.query, a.data + (uint64_t) point * a.dim, a.dim);
        visited_clear(s.visited, p.hash_bit);
        __syncwarp();
        bool wide = false;
        // kModeRefine: routed by the pre-pass (search_kernel.cuh:258-269 via graph_kernel.cuh:638-642)
        uint32_t routed = 0;
        if (a.mode == kModeRefine) {
            routed = a.route[point - a.route_first];
            if (routed >= a.C) routed = 0;   // the routing kernels never write an id beyond C; checked all the same
        }
        const uint32_t start = a.start_points[routed];
        const uint32_t exclude = a.mode == kModeRefine ? kInvalid : point;
        if constexpr (LANES) {
            float ck;
            uint32_t cv;
            rows += seed_lanes(s, start, exclude, a.graph_in, degree, p.hash_bit, a.data, a.dim, a.metric, ck, cv, &wide);
            iters = beam_loop_lanes<NB>(bk, bv, s, p, point, a.graph_in, degree, a.data, a.dim, a.metric, &rows, ck, cv, wide);
        } else {
            rows += seed_from_row(s, start, exclude, a.graph_in, degree, p.hash_bit, a.data, a.dim, a.metric, &wide);
            iters = beam_loop<NB, NC, true>(bk, bv, s, p, point, a.graph_in, degree, a.data, a.dim, a.metric, &rows, wide);
        }
        uint32_t P;
        prune_rows = prune_lanes<NB>(bk, bv, p.beam, ps, s.query, LANES ? s.cand_id : nullptr, a.data, a.dim, degree, d.max_degree, need, a.alpha, a.metric,
                                     true, point, &P);
        short_pool = P < p.beam;
        uint32_t pos_num = 0;  // :660-671: holes, front to back
        for (uint32_t base = 0; base < d.max_degree; base += 32) {
            const uint32_t i = base + lane;
            const bool hole = (i < degree) && (ps.row[i] == kInvalid);
            const uint32_t mask = __ballot_sync(kFullMask, hole);
            if (i < degree) out[i] = hole ? ps.picks[pos_num + __popc(mask & ((1u << lane) - 1))] : ps.row[i];
            pos_num += __popc(mask);
        }
    }
    if (a.counters && lane == 0) {
        atomicAdd(a.counters + 0, (unsigned long long) rows);
        atomicAdd(a.counters + 1, (unsigned long long) iters);
        atomicAdd(a.counters + 2, (unsigned long long) prune_rows);
        if (short_pool) atomicAdd(a.counters + 3, 1ull);
    }
}

uint32_t pow2_at_least(uint32_t x, uint32_t lo) {
    uint32_t m = lo;
    while (m < x) m <<= 1;
    return m;
}

template<int NB, int NC, bool LANES = false>
cudaError_t launch_build_t(const BuildDev &d, uint32_t warps_per_cta, size_t smem_bytes, cudaStream_t stream) {
    auto kernel = build_kernel<NB, NC, LANES>;
    if (smem_bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_bytes);
        if (e != cudaSuccess) return e;
    }
    const uint32_t grid = (d.a.count + warps_per_cta - 1) / warps_per_cta;
    kernel<<<grid, warps_per_cta * 32, smem_bytes, stream>>>(d);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Reverse edges (graph_kernel.cuh:378-453). The reference appends with atomics from
// `degree` concurrent launches, so which sources a crowded node keeps is arbitrary.
// Here every node keeps the `degree` smallest (rank, source) pairs, i.e. the outcome of
// the reference when its launches run one after another in ascending thread order:
// edges are bucketed by destination (count, scan, fill) and each bucket is reduced by
// one warp with a bitonic selection, so the result does not depend on arrival order.
// ---------------------------------------------------------------------------
__global__ void reverse_count_kernel(const uint32_t *__restrict__ graph, uint32_t num, uint32_t degree,
                                     uint32_t *counts) {
    const uint64_t e = (uint64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= (uint64_t) num * degree) return;
    const uint32_t dst = graph[e];
    if (dst < num) atomicAdd(counts + dst, 1u);
}

__global__ void reverse_fill_kernel(const uint32_t *__restrict__ graph, uint32_t num, uint32_t degree,
                                    const uint32_t *__restrict__ offsets, uint32_t *cursor,
                                    unsigned long long *edges) {
    const uint64_t e = (uint64_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= (uint64_t) num * degree) return;
    const uint32_t dst = graph[e];
    if (dst >= num) return;
    const uint32_t src = (uint32_t) (e / degree), rank = (uint32_t) (e % degree);
    const uint32_t slot = atomicAdd(cursor + dst, 1u);
    edges[offsets[dst] + slot] = ((unsigned long long) rank << 32) | src;
}

// 64-bit compare-exchange network over the 32 lanes of a warp (one key per lane).
__device__ __forceinline__ unsigned long long warp_sort_u64(unsigned long long key) {
    const uint32_t lane = lane_id();
#pragma unroll
    for (uint32_t size = 2; size <= 32; size <<= 1) {
#pragma unroll
        for (uint32_t stride = size >> 1; stride >= 1; stride >>= 1) {
            const unsigned long long other = __shfl_xor_sync(kFullMask, key, stride);
            const bool asc = (size == 32) || ((lane & size) == 0);
            const bool lower = (lane & stride) == 0;
            const bool keep_small = (lower == asc);
            if (keep_small ? (other < key) : (other > key)) key = other;
        }
    }
    return key;
}

__device__ __forceinline__ uint32_t lower_bound_u64(const unsigned long long *a, uint32_t n, unsigned long long key) {
    uint32_t lo = 0, hi = n;
    while (lo < hi) {
        const uint32_t mid = (lo + hi) >> 1;
        if (a[mid] < key) lo = mid + 1; else hi = mid;
    }
    return lo;
}

// One warp per node: keep the smallest (rank, src) keys among incoming edges whose
// source is not already in the node's row ("have" test, :395-405), as many as the row
// has holes, then fill the holes front to back in that order (insert_reverse_kernel,
// :416-453). Chunks of 32 incoming keys are sorted in registers and merged into a
// sorted shared list by rank counting, so no step depends on arrival order.
__global__ void __launch_bounds__(256) reverse_insert_kernel(uint32_t *graph, uint32_t num, uint32_t degree,
                                                             const uint32_t *__restrict__ offsets,
                                                             const unsigned long long *__restrict__ edges,
                                                             uint32_t max_degree) {
    extern __shared__ __align__(16) uint32_t smem[];
    const uint32_t warp = threadIdx.x >> 5, lane = lane_id();
    const uint32_t node = blockIdx.x * (blockDim.x >> 5) + warp;
    if (node >= num) return;
    // strip (words): keepA[2*max_degree] keepB[2*max_degree] chunk[64] row[max_degree]
    uint32_t *strip = smem + (size_t) warp * (5 * max_degree + 64);
    unsigned long long *cur = reinterpret_cast<unsigned long long *>(strip);
    unsigned long long *nxt = cur + max_degree;
    unsigned long long *chunk = nxt + max_degree;
    uint32_t *row = strip + 4 * max_degree + 64;
    uint32_t holes = 0;
    for (uint32_t base = 0; base < max_degree; base += 32) {
        const uint32_t i = base + lane;
        const uint32_t e = (i < degree) ? graph[(uint64_t) node * degree + i] : kInvalid;
        row[i] = e;
        holes += __popc(__ballot_sync(kFullMask, (i < degree) && (e == kInvalid)));
    }
    __syncwarp();
    const uint32_t begin = offsets[node], cnt = offsets[node + 1] - begin;
    if (holes == 0 || cnt == 0) return;
    const unsigned long long *in = edges + begin;
    const uint32_t cap = holes;  // holes <= degree, the reference's list capacity
    uint32_t kept = 0;
    for (uint32_t base = 0; base < cnt; base += 32) {
        const uint32_t i = base + lane;
        unsigned long long key = ~0ull;
        if (i < cnt) {
            key = in[i];
            const uint32_t src = (uint32_t) key;
            for (uint32_t j = 0; j < degree; j++)
                if (row[j] == src) { key = ~0ull; break; }
            if (kept == cap && key != ~0ull && key > cur[cap - 1]) key = ~0ull;  // cannot enter
        }
        const uint32_t any = __ballot_sync(kFullMask, key != ~0ull);
        if (any == 0) continue;
        const uint32_t n_valid = __popc(any);
        key = warp_sort_u64(key);  // valid keys first, ascending
        chunk[lane] = key;
        __syncwarp();
        if (lane < n_valid) {
            const uint32_t pos = lane + lower_bound_u64(cur, kept, key);
            if (pos < cap) nxt[pos] = key;
        }
        for (uint32_t k = lane; k < kept; k += 32) {
            const unsigned long long kk = cur[k];
            const uint32_t pos = k + lower_bound_u64(chunk, n_valid, kk);
            if (pos < cap) nxt[pos] = kk;
        }
        __syncwarp();
        kept = (kept + n_valid < cap) ? kept + n_valid : cap;
        unsigned long long *t = cur; cur = nxt; nxt = t;
    }
    uint32_t pos_num = 0;
    for (uint32_t base = 0; base < max_degree && pos_num < kept; base += 32) {
        const uint32_t i = base + lane;
        const bool hole = (i < degree) && (row[i] == kInvalid);
        const uint32_t mask = __ballot_sync(kFullMask, hole);
        if (hole) {
            const uint32_t pos = pos_num + __popc(mask & ((1u << lane) - 1));
            if (pos < kept) graph[(uint64_t) node * degree + i] = (uint32_t) cur[pos];
        }
        pos_num += __popc(mask);
    }
}

}  // namespace

namespace {
// flags[r] = 1 when row first + r has an empty slot: a warp per row, one coalesced read
__global__ void hole_flags_kernel(const uint32_t *__restrict__ graph, uint32_t first, uint32_t count, uint32_t degree, uint32_t *flags) {
    const uint32_t r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = lane_id();
    if (r >= count) return;
    const uint32_t *row = graph + (uint64_t) (first + r) * degree;
    bool hole = false;
    for (uint32_t i = lane; i < degree; i += 32) hole = hole || (__ldg(row + i) == kInvalid);
    const uint32_t any = __ballot_sync(kFullMask, hole);
    if (lane == 0) flags[r] = any != 0 ? 1u : 0u;
}

// Ordered compaction by one CTA: order_out = the entries of order_in (or 0, 1, 2, ...) whose flag is set.
// Every warp owns one contiguous run of the list and walks it 32 entries at a time, once to count its
// kept entries and, after the 32 counts are scanned, once more to write them; the reads of a pass do
// not depend on one another, so their latencies overlap.
__global__ void __launch_bounds__(1024) compact_flagged_kernel(const uint32_t *__restrict__ flags, const uint32_t *__restrict__ order_in,
                                                               uint32_t count, uint32_t *order_out, uint32_t *count_out) {
    __shared__ uint32_t warp_sums[32];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t per_warp = ((count + 1023u) / 1024u) * 32u;   // a multiple of 32 entries per warp
    const uint32_t lo = min(count, warp * per_warp), hi = min(count, lo + per_warp);
    uint32_t kept = 0;
#pragma unroll 8
    for (uint32_t i0 = lo; i0 < hi; i0 += 32) {
        const uint32_t i = i0 + lane;
        const uint32_t r = i < hi ? (order_in ? __ldg(order_in + i) : i) : 0u;
        kept += __popc(__ballot_sync(kFullMask, i < hi && flags[r] != 0));
    }
    if (lane == 0) warp_sums[warp] = kept;
    __syncthreads();
    uint32_t at = 0, total = 0;
    for (uint32_t w = 0; w < 32; w++) {
        const uint32_t c = warp_sums[w];
        if (w < warp) at += c;
        total += c;
    }
#pragma unroll 8
    for (uint32_t i0 = lo; i0 < hi; i0 += 32) {
        const uint32_t i = i0 + lane;
        const uint32_t r = i < hi ? (order_in ? __ldg(order_in + i) : i) : 0u;
        const bool keep = i < hi && flags[r] != 0;
        const uint32_t m = __ballot_sync(kFullMask, keep);
        if (keep) order_out[at + __popc(m & ((1u << lane) - 1u))] = r;
        at += __popc(m);
    }
    if (tid == 0) *count_out = total;
}
}  // namespace

cudaError_t launch_rows_with_holes(const uint32_t *graph, uint32_t first, uint32_t count, uint32_t degree,
                                   const uint32_t *order_in, uint32_t *flags, uint32_t *order_out, uint32_t *count_out,
                                   cudaStream_t stream) {
    if (count == 0) return cudaMemsetAsync(count_out, 0, 4, stream);
    hole_flags_kernel<<<(unsigned) (((uint64_t) count * 32 + 255) / 256), 256, 0, stream>>>(graph, first, count, degree, flags);
    compact_flagged_kernel<<<1, 1024, 0, stream>>>(flags, order_in, count, order_out, count_out);
    return cudaGetLastError();
}

cudaError_t launch_build(const BuildArgs &a, cudaStream_t stream) {
    if (a.count == 0) return cudaSuccess;
    BuildDev d;
    d.a = a;
    d.max_centroid = pow2_at_least(a.C ? a.C : 1, 32);
    const uint32_t max_beam = a.p.beam <= 64 ? 64 : (a.p.beam <= 128 ? 128 : (a.p.beam <= 256 ? 256 : 512));
    const uint32_t max_cand = a.in_degree <= 64 ? 64 : (a.in_degree <= 128 ? 128 : 256);
    d.max_beam = max_beam;
    d.max_degree = round_up32(a.out_degree);
    uint32_t extra = prune_strip_words(d.max_degree);
    const bool lanes = a.in_degree <= 32;
    // Partition-local searches may keep their visited set as a bitmap: when it is no larger than
    // the hash table (or 4 KB), and when the hash table could not fill up between two resets
    // (beam entries put back at a reset, one adjacency row per expansion, the seed row), the only
    // case in which the two forms would answer differently.
    if ((a.mode == kModeBuild || a.mode == kModeBoundary) && a.max_seg_rows && a.p.hash_bit < 32 && !getenv("GLIDE_B200_NO_BITMAP")) {
        const uint64_t cap = 1ull << a.p.hash_bit, words = ((uint64_t) a.max_seg_rows + 31) / 32;
        const uint64_t inserts = (uint64_t) a.p.beam + (uint64_t) a.in_degree * (a.p.hash_reset_interval + 2ull) + 2;
        if (words <= (cap > 1024 ? cap : 1024) && inserts <= cap) d.a.p.hash_bit = a.p.hash_bit | ((uint32_t) words << 8);
    }
    d.strip_words = (strip_words_base(a.dim, lanes ? kLaneScratch : max_cand, d.a.p.hash_bit) + extra + two_warp_scratch_words(max_beam) + 3u) & ~3u;
    const size_t strip_bytes = (size_t) d.strip_words * 4;
    uint32_t warps = 8;
    while (warps > 1 && strip_bytes * warps > 96 * 1024) warps >>= 1;
    if (strip_bytes * warps > 200 * 1024) return cudaErrorInvalidValue;
    const int nb = max_beam / 32, nc = max_cand / 32;
    if (lanes) {
        const size_t bytes = strip_bytes * warps;
        if (nb == 2) return launch_build_t<2, 2, true>(d, warps, bytes, stream);
        if (nb == 4) return launch_build_t<4, 2, true>(d, warps, bytes, stream);
        if (nb == 8) return launch_build_t<8, 2, true>(d, warps, bytes, stream);
        return launch_build_t<16, 2, true>(d, warps, bytes, stream);
    }
    GLIDE_DISPATCH_NB_NC(launch_build_t, nb, nc, d, warps, strip_bytes * warps, stream);
}

// First launches pay for loading the kernel and for growing the device's local-memory
// reservation (tens of milliseconds); a context pays them once, at creation, with launches that
// find no work (count = 0: every warp returns at once).
cudaError_t preload_build_kernels(cudaStream_t stream) {
    BuildDev d{};
    build_kernel<2, 2, true><<<1, 32, 0, stream>>>(d);
    build_kernel<4, 2, true><<<1, 32, 0, stream>>>(d);
    build_kernel<2, 2, false><<<1, 32, 0, stream>>>(d);
    build_kernel<4, 2, false><<<1, 32, 0, stream>>>(d);
    return cudaGetLastError();
}

}  // namespace glide

namespace glide {

size_t reverse_scan_tmp_bytes(uint32_t num) { return scan_tmp_bytes(num); }

cudaError_t launch_reverse(const ReverseArgs &a, cudaStream_t stream) {
    if (a.num == 0) return cudaSuccess;
    const uint64_t edges = (uint64_t) a.num * a.degree;
    const uint32_t threads = 256;
    const uint32_t blocks = (uint32_t) ((edges + threads - 1) / threads);
    cudaError_t e = cudaMemsetAsync(a.counts, 0, (size_t) (a.num + 1) * sizeof(uint32_t), stream);
    if (e != cudaSuccess) return e;
    reverse_count_kernel<<<blocks, threads, 0, stream>>>(a.graph, a.num, a.degree, a.counts);
    e = exclusive_scan_u32(a.counts, a.num, a.offsets, a.scan_tmp, stream);
    if (e != cudaSuccess) return e;
    e = cudaMemsetAsync(a.counts, 0, (size_t) (a.num + 1) * sizeof(uint32_t), stream);  // reused as fill cursor
    if (e != cudaSuccess) return e;
    reverse_fill_kernel<<<blocks, threads, 0, stream>>>(a.graph, a.num, a.degree, a.offsets, a.counts, a.edges);
    const uint32_t max_degree = round_up32(a.degree);
    const uint32_t warps = 8;
    const size_t smem_bytes = (size_t) warps * (5 * max_degree + 64) * 4;
    if (smem_bytes > 48 * 1024) {
        e = cudaFuncSetAttribute(reverse_insert_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_bytes);
        if (e != cudaSuccess) return e;
    }
    reverse_insert_kernel<<<(a.num + warps - 1) / warps, warps * 32, smem_bytes, stream>>>(
        a.graph, a.num, a.degree, a.offsets, a.edges, max_degree);
    return cudaGetLastError();
}

}  // namespace glide
