// Query search kernels: the small path's routed search (reference search_kernel,
// search_kernel.cuh:393-490), the large path's query routing (select_segment_kernel,
// :546-607) and per-partition search with running top-k merge (search_on_sub_kernel +
// result_merge, :609-765).
#include <cstdlib>

#include "beam_core.cuh"
#include "kernels.h"

namespace glide {

namespace {

struct SearchDev {
    SearchArgs a;
    uint32_t max_centroid;
    uint32_t max_topk;
    uint32_t strip_words;
};

// Last bitonic phase on a shared array of 32*n pairs (the input must be bitonic).
__device__ inline void warp_merge_final_smem(float *k, uint32_t *v, uint32_t n_per_lane) {
    const uint32_t total = 32u * n_per_lane, lane = lane_id();
    for (uint32_t stride = total >> 1; stride >= 1; stride >>= 1) {
        for (uint32_t p = lane; p < total / 2; p += 32) {
            const uint32_t lo = ((p / stride) * 2 * stride) + (p % stride);
            const uint32_t hi = lo + stride;
            const float k0 = k[lo], k1 = k[hi];
            if ((k0 != k1) && !(k0 < k1)) {
                k[lo] = k1; k[hi] = k0;
                const uint32_t t = v[lo]; v[lo] = v[hi]; v[hi] = t;
            }
        }
        __syncwarp();
    }
}

// LANES: adjacency rows of at most 32 entries, candidates stay in registers (beam_loop_lanes);
// the strip then holds only the query and the visited set.
// The partition a large-path search runs in.
struct PartView {
    const float *data;
    const uint32_t *graph, *map;
    uint32_t start_point;
};

template<int NB, int NC, bool LANES, bool PARTS = false>
__device__ __forceinline__ void search_one(const SearchDev &d, const WarpStrip &s, const BeamParams &p, uint32_t q,
                                           const PartView &given, bool check_routed) {
    const SearchArgs &a = d.a;
    const uint32_t lane = lane_id();
    // outside the multi-partition kernel the partition is the launch's own (kernel parameters, no registers)
    const PartView view = PARTS ? given : PartView{a.data, a.graph, a.map, a.start_point};

    const bool sub = (a.segment_ids != nullptr);
    if (sub && check_routed) {  // search_kernel.cuh:676-692: skip queries not routed to this partition
        bool routed = false;
        if (lane == 0) {
            for (uint32_t i = 0; i < a.segment_num; i++) {
                const uint32_t sid = a.segment_ids[(uint64_t) q * a.segment_num + i];
                if (sid == a.segment_id) { routed = true; break; }
                if (sid == kInvalid) break;
            }
        }
        routed = __shfl_sync(kFullMask, routed ? 1 : 0, 0) != 0;
        if (!routed) return;
    }

    load_query(s.query, a.queries + (uint64_t) q * a.dim, a.dim);
    visited_clear(s.visited, p.hash_bit);
    __syncwarp();

    uint32_t rows = 0;
    uint32_t start_node;
    if (!sub) {
        // the nearest centroid was found by the routing pre-pass (search_kernel.cuh:258-269)
        const uint32_t r = a.route[q];
        start_node = a.start_points[r < a.C ? r : 0u];   // the routing kernels never write an id beyond C; checked all the same
    } else {
        start_node = view.start_point;
    }
    float bk[NB];
    uint32_t bv[NB];
    uint32_t iters;
    if constexpr (LANES) {
        float ck;
        uint32_t cv;
        rows += seed_lanes(s, start_node, kInvalid, view.graph, a.degree, p.hash_bit, view.data, a.dim, a.metric, ck, cv);
        iters = beam_loop_lanes<NB>(bk, bv, s, p, kInvalid, view.graph, a.degree, view.data, a.dim, a.metric, &rows, ck, cv);
    } else {
        rows += seed_from_row(s, start_node, kInvalid, view.graph, a.degree, p.hash_bit, view.data, a.dim, a.metric);
        iters = beam_loop<NB, NC>(bk, bv, s, p, kInvalid, view.graph, a.degree, view.data, a.dim, a.metric, &rows);
    }

    if (!sub) {
#pragma unroll
        for (int i = 0; i < NB; i++) {
            const uint32_t j = NB * lane + i;
            if (j < a.top_k) {
                a.out_ids[(uint64_t) q * a.top_k + j] = bv[i] & kClean;
                a.out_dists[(uint64_t) q * a.top_k + j] = bk[i];
            }
        }
    } else {
        // result_merge (search_kernel.cuh:609-651): fold the first top_k beam entries
        // into the running result with a network of width max_topk.
        const uint32_t M = d.max_topk, n = M / 32;
        float *mk = reinterpret_cast<float *>(s.extra);
        uint32_t *mv = s.extra + M;
        float *rk = reinterpret_cast<float *>(s.extra + 2 * M);  // this partition's result, by beam position
        uint32_t *rv = s.extra + 3 * M;
#pragma unroll
        for (int i = 0; i < NB; i++) {
            const uint32_t j = NB * lane + i;
            if (j < a.top_k) {
                rk[j] = bk[i];
                const uint32_t id = bv[i] & kClean;
                rv[j] = (id == kPadClean) ? kInvalid : view.map[id];  // an unfilled slot has no global id
            }
        }
        float *fd = a.out_dists + (uint64_t) q * a.top_k;
        uint32_t *fi = a.out_ids + (uint64_t) q * a.top_k;
        for (uint32_t j = lane; j < M; j += 32) {
            mk[j] = (j < a.top_k) ? fd[j] : FLT_MAX;
            mv[j] = (j < a.top_k) ? fi[j] : kInvalid;
        }
        __syncwarp();
        for (uint32_t j = lane; j < M; j += 32) {
            const uint32_t k = M - 1 - j;
            if (k < a.top_k && mk[j] > rk[k]) {
                mk[j] = rk[k];
                mv[j] = rv[k];
            }
        }
        __syncwarp();
        warp_merge_final_smem(mk, mv, n);
        for (uint32_t j = lane; j < a.top_k; j += 32) {
            fd[j] = mk[j];
            fi[j] = mv[j];
        }
    }
    if (a.counters && lane == 0) {
        atomicAdd(a.counters + 0, (unsigned long long) rows);
        atomicAdd(a.counters + 1, (unsigned long long) iters);
    }
}

// A warp per query. With a ticket counter the grid is sized to what the device holds at once and
// every warp draws its next query as soon as it finishes one, so a slow query delays neither the
// other warps of its CTA nor a whole wave of CTAs.
template<int NB, int NC, bool LANES, bool PARTS = false>
__device__ __forceinline__ void search_body(const SearchDev &d) {
    extern __shared__ __align__(16) uint32_t smem[];
    const SearchArgs &a = d.a;
    const uint32_t warps_per_cta = blockDim.x >> 5;
    const uint32_t warp = threadIdx.x >> 5, lane = lane_id();
    const BeamParams p{a.p.beam, a.p.max_iterations, a.p.min_iterations, a.p.hash_bit, a.p.hash_reset_interval};
    WarpStrip s = make_strip(smem + (size_t) warp * d.strip_words, a.dim, LANES ? kLaneScratch : 32u * NC, p.hash_bit);
    if constexpr (NB == 16) s.tail = smem + (size_t) (warp + 1) * d.strip_words - kTwoWarpScratch;
    const PartView whole{a.data, a.graph, a.map, a.start_point};
    if (a.ticket == nullptr) {
        const uint32_t q = blockIdx.x * warps_per_cta + warp;
        if (q < a.Q) search_one<NB, NC, LANES>(d, s, p, q, whole, true);
        return;
    }
    while (true) {
        uint32_t q = 0;
        if (lane == 0) q = atomicAdd(a.ticket, 1u);
        q = __shfl_sync(kFullMask, q, 0);
        if (q >= a.Q) break;
        if (a.order) q = a.order[q];
        if constexpr (!PARTS) {
            search_one<NB, NC, LANES>(d, s, p, q, whole, true);
        } else {
            // Every partition the query is routed to, in ascending partition order: the order in which
            // the reference's loop over partitions (glide_large_impl.cuh:424-493) folds them into the
            // running result. The routed list is a prefix of the query's row of segment_ids.
            const uint32_t *ids = a.segment_ids + (uint64_t) q * a.segment_num;
            const uint32_t r0 = lane < a.segment_num ? ids[lane] : kInvalid;
            const uint32_t r1 = lane + 32u < a.segment_num ? ids[lane + 32u] : kInvalid;
            const bool longer = a.segment_num > 64u && ids[64] != kInvalid;   // rare: more than 64 partitions routed
            uint32_t prev = kInvalid;
            while (true) {
                uint32_t best = kInvalid;
                if (r0 != kInvalid && (prev == kInvalid || r0 > prev)) best = r0;
                if (r1 != kInvalid && (prev == kInvalid || r1 > prev) && r1 < best) best = r1;
                if (longer)
                    for (uint32_t i = 64u + lane; i < a.segment_num; i += 32u) {
                        const uint32_t sid = ids[i];
                        if (sid != kInvalid && (prev == kInvalid || sid > prev) && sid < best) best = sid;
                    }
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) best = min(best, __shfl_xor_sync(kFullMask, best, off));
                if (best == kInvalid) break;
                prev = best;
                const PartitionRef ref = a.parts[best];
                if (ref.data != nullptr) search_one<NB, NC, LANES, true>(d, s, p, q, PartView{ref.data, ref.graph, ref.map, ref.start_point}, false);
                __syncwarp();
            }
        }
        __syncwarp();
    }
}

// Register targets per beam class (measured): 64 registers for beams up to 64 slots (4 CTAs per
// SM), 80 up to 128, 128 beyond. The 32-slot instance does best with the compiler's own choice.
template<int NB, int NC, bool LANES>
__global__ void __launch_bounds__(256, NB == 2 ? 4 : (NB == 4 ? 3 : 2)) search_kernel(const SearchDev d) {
    search_body<NB, NC, LANES>(d);
}

// 32-slot beams: nine warps per CTA and four CTAs per SM (56 registers) hold 36 queries per SM at
// once, 5,328 on 148 SMs, so that a batch of 10,000 queries is two full rounds; with eight warps
// (4,736 at once) the same batch is two rounds and a third with a tenth of the warps busy.
template<int NC, bool LANES>
__global__ void __launch_bounds__(288, 4) search_kernel_32(const SearchDev d) {
    search_body<1, NC, LANES>(d);
}

// select_segment_kernel (search_kernel.cuh:546-607): a warp per query.
__global__ void __launch_bounds__(128) select_segment_kernel(const SelectSegmentArgs a, uint32_t max_centroid,
                                                             uint32_t strip_words) {
    extern __shared__ __align__(16) uint32_t smem[];
    const uint32_t warp = threadIdx.x >> 5, lane = lane_id();
    const uint32_t q = blockIdx.x * (blockDim.x >> 5) + warp;
    if (q >= a.Q) return;
    uint32_t *base = smem + (size_t) warp * strip_words;
    float *query = reinterpret_cast<float *>(base);
    uint32_t *scratch = base + dim_pad4(a.dim);
    load_query(query, a.queries + (uint64_t) q * a.dim, a.dim);
    nearest_centroid(query, a.centroids, a.C, max_centroid, a.dim, a.metric, scratch, kSorted);
    const float *ck = reinterpret_cast<const float *>(scratch);
    const uint32_t *cv = scratch + max_centroid;
    uint32_t *out = a.out + (uint64_t) q * a.C;
    const float d0 = ck[0];
    uint32_t allow_num = 0;
    for (uint32_t base_i = 0; base_i < a.C; base_i += 32) {
        const uint32_t i = base_i + lane;
        const bool allow = (i < a.C) && (ck[i] / d0 <= a.boundary_factor);
        if (i < a.C) out[i] = allow ? cv[i] : kInvalid;
        allow_num += __popc(__ballot_sync(kFullMask, allow));
    }
    __syncwarp();
    if (allow_num < a.min_segment_num) {
        const uint32_t need = a.min_segment_num - allow_num;
        for (uint32_t i = lane; i < need; i += 32)
            if (allow_num + i < a.C) out[allow_num + i] = cv[allow_num + i];
    }
}

uint32_t pow2_at_least(uint32_t x, uint32_t lo) {
    uint32_t m = lo;
    while (m < x) m <<= 1;
    return m;
}

// Large path with every partition in device memory: a warp walks all the partitions its query is routed to.
template<int NB, int NC, bool LANES>
__global__ void __launch_bounds__(256, NB <= 4 ? 3 : 2) search_parts_kernel(const SearchDev d) {
    search_body<NB, NC, LANES, true>(d);
}

template<int NB, int NC, bool LANES = false>
cudaError_t launch_search_t(const SearchDev &d, uint32_t warps_per_cta, size_t smem_bytes, cudaStream_t stream) {
    void (*kernel)(const SearchDev) = search_kernel<NB, NC, LANES>;
    if constexpr (NB == 1) kernel = search_kernel_32<NC, LANES>;
    if constexpr (NB > 1) {
        if (d.a.parts != nullptr) kernel = search_parts_kernel<NB, NC, LANES>;
    }
    if (smem_bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_bytes);
        if (e != cudaSuccess) return e;
    }
    uint32_t grid = (d.a.Q + warps_per_cta - 1) / warps_per_cta;
    if (d.a.ticket) {
        int per_sm = 0, dev = 0, sms = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, (int) (warps_per_cta * 32), smem_bytes);
        if (e != cudaSuccess) return e;
        if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
        if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
        const uint32_t resident = (uint32_t) (per_sm > 0 ? per_sm : 1) * (uint32_t) sms;
        if (grid > resident) grid = resident;
        if ((e = cudaMemsetAsync(d.a.ticket, 0, sizeof(uint32_t), stream)) != cudaSuccess) return e;
    }
    kernel<<<grid, warps_per_cta * 32, smem_bytes, stream>>>(d);
    return cudaGetLastError();
}

}  // namespace

// See preload_build_kernels: launches without work (Q = 0, no ticket) that load the common instances.
cudaError_t preload_search_kernels(cudaStream_t stream) {
    SearchDev d{};
    search_kernel_32<2, true><<<1, 32, 0, stream>>>(d);
    search_kernel<2, 2, true><<<1, 32, 0, stream>>>(d);
    search_kernel<4, 2, true><<<1, 32, 0, stream>>>(d);
    search_kernel<2, 2, false><<<1, 32, 0, stream>>>(d);
    return cudaGetLastError();
}

cudaError_t launch_search(const SearchArgs &a, cudaStream_t stream) {
    if (a.Q == 0) return cudaSuccess;
    SearchDev d;
    d.a = a;
    d.max_centroid = pow2_at_least(a.C, 32);
    d.max_topk = a.top_k <= 32 ? 32 : (a.top_k <= 64 ? 64 : 128);  // kernel_config.cuh:309-319
    // same size ladders as kernel_config.cuh:190-204 so that ties fall identically
    const uint32_t max_beam = a.p.beam <= 64 ? 64 : (a.p.beam <= 128 ? 128 : (a.p.beam <= 256 ? 256 : 512));
    const uint32_t max_cand = a.degree <= 64 ? 64 : (a.degree <= 128 ? 128 : 256);
    const uint32_t extra = a.segment_ids ? 4 * d.max_topk : 0;
    const bool lanes = a.degree <= 32;
    d.strip_words = (strip_words_base(a.dim, lanes ? kLaneScratch : max_cand, a.p.hash_bit) + extra + two_warp_scratch_words(max_beam) + 3u) & ~3u;
    const size_t strip_bytes = (size_t) d.strip_words * 4;
    uint32_t warps = 8;
    while (warps > 1 && strip_bytes * warps > 96 * 1024) warps >>= 1;
    if (strip_bytes * warps > 200 * 1024) return cudaErrorInvalidValue;
    const int nb = max_beam / 32, nc = max_cand / 32;
    if (lanes) {
        if (a.p.beam <= 32 && warps == 8 && strip_bytes * 9 * 4 <= 200 * 1024 && a.parts == nullptr) {
            static const uint32_t w32 = [] {   // experiments: GLIDE_B200_SEARCH_WARPS=8 restores eight warps per CTA
                const char *e = std::getenv("GLIDE_B200_SEARCH_WARPS");
                const uint32_t v = e ? (uint32_t) std::strtoul(e, nullptr, 10) : 9u;
                return (v >= 1 && v <= 9) ? v : 9u;
            }();
            warps = w32;
        }
        const size_t bytes = strip_bytes * warps;
        if (a.p.beam <= 32 && a.parts == nullptr) return launch_search_t<1, 2, true>(d, warps, bytes, stream);   // (the 64-slot kernel gives the same beam)
        if (nb == 2) return launch_search_t<2, 2, true>(d, warps, bytes, stream);
        if (nb == 4) return launch_search_t<4, 2, true>(d, warps, bytes, stream);
        if (nb == 8) return launch_search_t<8, 2, true>(d, warps, bytes, stream);
        return launch_search_t<16, 2, true>(d, warps, bytes, stream);
    }
    GLIDE_DISPATCH_NB_NC(launch_search_t, nb, nc, d, warps, strip_bytes * warps, stream);
}

cudaError_t launch_select_segments(const SelectSegmentArgs &a, cudaStream_t stream) {
    if (a.Q == 0) return cudaSuccess;
    const uint32_t max_centroid = pow2_at_least(a.C, 32);
    const uint32_t strip_words = (dim_pad4(a.dim) + 2 * max_centroid + 3u) & ~3u;
    const uint32_t warps = 4;
    const size_t smem_bytes = (size_t) strip_words * 4 * warps;
    if (smem_bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(select_segment_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int) smem_bytes);
        if (e != cudaSuccess) return e;
    }
    select_segment_kernel<<<(a.Q + warps - 1) / warps, warps * 32, smem_bytes, stream>>>(a, max_centroid, strip_words);
    return cudaGetLastError();
}

}  // namespace glide
