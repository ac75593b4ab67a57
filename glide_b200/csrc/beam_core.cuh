// Warp-per-query greedy beam search core, shared by query search, subgraph build,
// boundary build, refinement and the large-path per-partition search.
//
// Behaviour (what is computed, in which order ties fall) follows the reference's
// search loop, search_kernel.cuh:393-490 and graph_kernel.cuh:5-68. Layout does not:
// the beam lives in registers for the whole search (NB pairs per lane, position
// j = NB*lane + i), candidates pass through a small per-warp shared-memory strip,
// and several warps (= several independent queries) share a CTA with no CTA-wide
// barrier inside the loop.
#pragma once

#include "common.cuh"

namespace glide {

// Lane-resident kernels keep no candidate arrays in the strip, only 2 x this many words at cand_id
// (the cand_id and cand_dist slots of the layout below) for the ids of a scoring call in rank
// order: up to 32 ids plus 8 of padding.
constexpr uint32_t kLaneScratch = 20;

struct BeamParams {
    uint32_t beam;            // multiple of 32, <= 32*NB
    uint32_t max_iterations;
    uint32_t min_iterations;
    uint32_t hash_bit;
    uint32_t hash_reset_interval;
};

// Per-warp shared memory strip. All offsets in 4-byte words; query first so that it
// is 16-byte aligned.
struct WarpStrip {
    float *query;        // dim_pad floats
    uint32_t *cand_id;   // 32*NC
    float *cand_dist;    // 32*NC
    uint32_t *visited;   // visited_words(hash_bit)
    uint32_t *work;      // 32*NC: slots of the candidates to score
    uint32_t *work_id;   // 32*NC: their ids
    uint32_t *extra;     // mode-specific scratch (pool, rows, merge buffers)
    uint32_t *tail;      // the last kTwoWarpScratch words of the strip: present (and set by the kernel) only for beams
                         // above 256 slots, whose merge runs on shared arrays (merge_beam_two_warps)
};

// beam keys [512], beam ids [512], one sorted candidate row of the lane-resident kernels: keys [32], ids [32]
constexpr uint32_t kTwoWarpScratch = 2 * 512 + 64;
__host__ __device__ inline uint32_t two_warp_scratch_words(uint32_t max_beam) { return max_beam > 256 ? kTwoWarpScratch : 0u; }

__host__ __device__ inline uint32_t dim_pad4(uint32_t dim) { return (dim + 3u) & ~3u; }

__host__ __device__ inline uint32_t strip_words_base(uint32_t dim, uint32_t max_cand, uint32_t hash_bit) {
    return dim_pad4(dim) + 4 * max_cand + visited_words(hash_bit);
}

__device__ __forceinline__ WarpStrip make_strip(uint32_t *base, uint32_t dim, uint32_t max_cand, uint32_t hash_bit) {
    WarpStrip s;
    s.query = reinterpret_cast<float *>(base);
    s.cand_id = base + dim_pad4(dim);
    s.cand_dist = reinterpret_cast<float *>(s.cand_id + max_cand);
    s.visited = s.cand_id + 2 * max_cand;
    s.work = s.visited + visited_words(hash_bit);
    s.work_id = s.work + max_cand;
    s.extra = s.work_id + max_cand;
    s.tail = nullptr;
    return s;
}

__device__ __forceinline__ void load_query(float *q_smem, const float *q_global, uint32_t dim) {
    const uint32_t lane = lane_id();
    if ((dim & 3u) == 0) {
        const float4 *src = reinterpret_cast<const float4 *>(q_global);
        float4 *dst = reinterpret_cast<float4 *>(q_smem);
        for (uint32_t c = lane; c < (dim >> 2); c += 32) dst[c] = __ldg(src + c);
    } else {
        for (uint32_t i = lane; i < dim; i += 32) q_smem[i] = __ldg(q_global + i);
    }
    __syncwarp();
}

// Distances of the query to every valid candidate (cand_id[i] != kInvalid, and
// != skip_id), written to cand_dist[i]; other slots get FLT_MAX. Candidates keep
// their slot, which decides how ties fall in the sort that follows. Valid slots are
// compacted into the strip's work list and scored by warp_rows (whole-warp row loads,
// several rows in flight). Returns the number of rows read by this warp
// (for the traffic counters).
__device__ __forceinline__ uint32_t score_candidates(const WarpStrip &s, uint32_t count, uint32_t skip_id,
                                                     const float *__restrict__ data, uint32_t dim, int metric) {
    const uint32_t lane = lane_id();
    uint32_t n = 0;
    for (uint32_t base = 0; base < count; base += 32) {
        const uint32_t i = base + lane;
        const uint32_t id = (i < count) ? s.cand_id[i] : kInvalid;
        const bool valid = (id != kInvalid) && (id != skip_id);
        if (i < count && !valid) s.cand_dist[i] = FLT_MAX;
        const uint32_t mask = __ballot_sync(kFullMask, valid);
        if (valid) {
            const uint32_t k = n + __popc(mask & ((1u << lane) - 1));
            s.work[k] = i;
            s.work_id[k] = id;
        }
        n += __popc(mask);
    }
    __syncwarp();
    warp_rows(s.query, data, dim, metric, n,
              [&](uint32_t i) { return s.work_id[i]; },
              [&](uint32_t i, float d) { s.cand_dist[s.work[i]] = d; });
    __syncwarp();
    return n;
}

// search_kernel.cuh:362-391: read the parent's adjacency row, keep ids that are new
// to the visited set (and are not own_id), then score them.
__device__ __forceinline__ uint32_t expand_parent(const WarpStrip &s, uint32_t parent, uint32_t own_id,
                                                  const uint32_t *__restrict__ graph, uint32_t degree,
                                                  uint32_t hash_bit, const float *__restrict__ data,
                                                  uint32_t dim, int metric) {
    for (uint32_t base = 0; base < degree; base += 32) {
        const uint32_t i = base + lane_id();
        uint32_t nb = kInvalid;
        if (i < degree && parent != kInvalid) nb = __ldg(graph + (uint64_t) parent * degree + i);
        const uint32_t flag = visited_insert(s.visited, hash_bit, nb, nb != kInvalid && nb != own_id);
        if (i < degree) s.cand_id[i] = flag ? nb : kInvalid;
    }
    __syncwarp();
    return score_candidates(s, degree, kInvalid, data, dim, metric);
}

// search_kernel.cuh:336-360: seed from a start point's row. exclude_id keeps its
// slot but gets distance FLT_MAX.
// *excluded_kept is set when the excluded id occurs: that slot then holds a valid id with distance
// FLT_MAX, the one input the narrow candidate sort of beam_loop cannot take.
__device__ __forceinline__ uint32_t seed_from_row(const WarpStrip &s, uint32_t start_point, uint32_t exclude_id,
                                                  const uint32_t *__restrict__ graph, uint32_t degree,
                                                  uint32_t hash_bit, const float *__restrict__ data,
                                                  uint32_t dim, int metric, bool *excluded_kept = nullptr) {
    bool kept = false;
    for (uint32_t base = 0; base < degree; base += 32) {
        const uint32_t i = base + lane_id();
        uint32_t index = kInvalid;
        if (i < degree) index = __ldg(graph + (uint64_t) start_point * degree + i);
        const uint32_t flag = visited_insert(s.visited, hash_bit, index, index != kInvalid);
        if (i < degree) s.cand_id[i] = flag ? index : kInvalid;
        kept = kept || (__ballot_sync(kFullMask, flag && index == exclude_id) != 0);
    }
    if (excluded_kept) *excluded_kept = kept;
    __syncwarp();
    return score_candidates(s, degree, exclude_id, data, dim, metric);
}

// search_kernel.cuh:258-269: distances to all centroids, ordered as the reference's
// network of width max_centroid (power of two >= C, >= 32) orders them; returns the nearest
// centroid's id. scratch: 2 * max_centroid words (keys then ids). What is valid afterwards
// depends on `need`: kNearestOnly - nothing else; kTopTwo - keys[0], keys[1], ids[0];
// kSorted - both arrays fully sorted. When the smallest distance is unique the first two
// need no sort (position 0 of the sorted list is the minimum whatever the network does);
// a tie at the minimum falls back to the full network so that the reference's tie order
// is reproduced.
enum CentroidNeed : int { kNearestOnly = 0, kTopTwo = 1, kSorted = 2 };

__device__ __forceinline__ uint32_t nearest_centroid(const float *q_smem, const float *__restrict__ centroids,
                                                     uint32_t C, uint32_t max_centroid, uint32_t dim, int metric,
                                                     uint32_t *scratch, int need) {
    const uint32_t lane = lane_id(), team = lane / kTeam;
    const uint32_t n = max_centroid / 32;
    float *ck = reinterpret_cast<float *>(scratch);
    uint32_t *cv = scratch + max_centroid;
    // element j starts in lane j%32, register j/32, i.e. network position n*(j%32) + j/32
    for (uint32_t j = lane; j < max_centroid; j += 32) {
        const uint32_t e = n * (j % 32) + j / 32;
        ck[e] = FLT_MAX;
        cv[e] = kInvalid;
    }
    __syncwarp();
    for (uint32_t c0 = 0; c0 < C; c0 += kTeamsPerWarp) {
        const uint32_t c = c0 + team;
        const bool active = c < C;
        const float part = team_partial(q_smem, centroids + (uint64_t) (active ? c : 0) * dim, dim, active);
        const float sum = team_fold(part);
        if (active && (lane & (kTeam - 1)) == 0) {
            const uint32_t e = n * (c % 32) + c / 32;
            ck[e] = finish_metric(sum, metric);
            cv[e] = c;
        }
    }
    __syncwarp();
    if (need != kSorted) {
        float m0 = FLT_MAX;
        for (uint32_t e = lane; e < max_centroid; e += 32)
            if (cv[e] != kInvalid && ck[e] < m0) m0 = ck[e];
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) m0 = fminf(m0, __shfl_xor_sync(kFullMask, m0, off));
        uint32_t cnt = 0, pos = 0;
        for (uint32_t e = lane; e < max_centroid; e += 32)
            if (cv[e] != kInvalid && ck[e] == m0) { cnt++; pos = e; }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            cnt += __shfl_xor_sync(kFullMask, cnt, off);
            pos = max(pos, __shfl_xor_sync(kFullMask, pos, off));
        }
        if (cnt == 1) {
            const uint32_t id = cv[pos];
            if (need == kTopTwo) {
                float m1 = FLT_MAX;
                for (uint32_t e = lane; e < max_centroid; e += 32)
                    if (e != pos && cv[e] != kInvalid && ck[e] < m1) m1 = ck[e];
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) m1 = fminf(m1, __shfl_xor_sync(kFullMask, m1, off));
                __syncwarp();
                if (lane == 0) { ck[0] = m0; ck[1] = m1; cv[0] = id; }
                __syncwarp();
            }
            return id;
        }
    }
    warp_sort_smem(ck, cv, n);
    return cv[0];
}

// search_kernel.cuh:148-233: for MAX_BEAM = 512 the reference merges with two warps and ends up with
// its own order among equal distances. One warp replays both here on shared arrays: candidates
// (ascending, cand_k / cand_v, the first min(degree, beam) valid) replace mirrored beam slots where
// they are strictly smaller, the two halves of the beam exchange pairwise, and each half is merged
// after being loaded around its turning point (the first slot that changed), which makes the loaded
// sequence bitonic. sk / sv: 512 words each. The beam comes in and leaves in registers (position
// j = 16 * lane + i).
__device__ __forceinline__ void merge_beam_two_warps(float (&bk)[16], uint32_t (&bv)[16], uint32_t beam, uint32_t degree,
                                                     const float *cand_k, const uint32_t *cand_v, float *sk, uint32_t *sv) {
    const uint32_t lane = lane_id(), half = beam >> 1;
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const uint32_t j = 16u * lane + i;
        if (j < beam) { sk[j] = bk[i]; sv[j] = bv[i]; }
    }
    __syncwarp();
    uint32_t t0 = half, t1 = half, t2 = half;
    const uint32_t lim = degree < beam ? degree : beam;
    for (uint32_t k = lane; k < lim; k += 32) {
        const uint32_t j = beam - 1u - k;
        const float c = cand_k[k];
        if (sk[j] > c) {
            sk[j] = c;
            sv[j] = cand_v[k];
            if (j < half) t2 = min(t2, j); else t1 = min(t1, j - half);
        }
    }
    __syncwarp();
    for (uint32_t j = lane; j < half; j += 32) {
        const uint32_t k = j + half;
        const float a = sk[j], b = sk[k];
        if (a > b) {
            sk[j] = b; sk[k] = a;
            const uint32_t t = sv[j]; sv[j] = sv[k]; sv[k] = t;
            t0 = min(t0, j);
        }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        t0 = min(t0, __shfl_xor_sync(kFullMask, t0, off));
        t1 = min(t1, __shfl_xor_sync(kFullMask, t1, off));
        t2 = min(t2, __shfl_xor_sync(kFullMask, t2, off));
    }
    if (t2 < half) t1 = t2;
    __syncwarp();
#pragma unroll 1
    for (uint32_t w = 0; w < 2; w++) {
        const uint32_t turning = w == 0 ? t0 : t1;
        float k8[8];
        uint32_t v8[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            uint32_t k = beam, j = 8u * lane + i;
            if (j < turning) {
                k = j + half * w;
            } else if (j >= 256u - half) {
                j -= 256u - half;
                if (turning <= j && j < half) k = j + half * w;
            }
            k8[i] = k < beam ? sk[k] : FLT_MAX;
            v8[i] = k < beam ? sv[k] : kInvalid;
        }
        __syncwarp();
        warp_merge_final<8>(k8, v8);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t j = 8u * lane + i;
            if (j < half) { sk[j + half * w] = k8[i]; sv[j + half * w] = v8[i]; }
        }
        __syncwarp();
    }
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const uint32_t j = 16u * lane + i;
        bk[i] = j < beam ? sk[j] : FLT_MAX;
        bv[i] = j < beam ? sv[j] : kInvalid;
    }
    __syncwarp();
}

// search_kernel.cuh:38-95: for MAX_CANDIDATE = 256 the reference sorts the candidates with two warps:
// each sorts its half of 128, the halves exchange mirrored elements (equal keys stay, the first half
// keeps the smaller), and each merges its half again. Replayed by one warp with two register sets on
// the candidate arrays in shared memory.
__device__ __forceinline__ void sort_candidates_two_warps(float *cand_k, uint32_t *cand_v, uint32_t degree, uint32_t beam) {
    const uint32_t lane = lane_id();
    constexpr uint32_t per = 128;
    float ka[2][4];
    uint32_t va[2][4];
#pragma unroll
    for (int w = 0; w < 2; w++) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t j = lane + 32u * i + per * w;
            ka[w][i] = j < degree ? cand_k[j] : FLT_MAX;
            va[w][i] = j < degree ? cand_v[j] : kInvalid;
        }
    }
    __syncwarp();
#pragma unroll
    for (int w = 0; w < 2; w++) {
        warp_sort<4>(ka[w], va[w]);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t jl = 4u * lane + i, j = jl + per * w;
            if (j < degree && jl < beam) { cand_k[j] = ka[w][i]; cand_v[j] = va[w][i]; }
        }
    }
    __syncwarp();
    const uint32_t used = (beam + per - 1) / per;
#pragma unroll
    for (int w = 0; w < 2; w++) {
        if ((uint32_t) w >= used) continue;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t jl = 4u * lane + i, kl = per - 1u - jl, j = jl + per * w, k = 256u - 1u - j;
            if (j >= degree || k >= degree || kl >= beam) continue;
            const float other = cand_k[k];
            if (ka[w][i] == other) continue;
            if ((w == 0) == (ka[w][i] > other)) { ka[w][i] = other; va[w][i] = cand_v[k]; }
        }
    }
    __syncwarp();
#pragma unroll
    for (int w = 0; w < 2; w++) {
        if ((uint32_t) w >= used) continue;
        warp_merge_final<4>(ka[w], va[w]);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t j = 4u * lane + i + per * w;
            if (j < degree && j < beam) { cand_k[j] = ka[w][i]; cand_v[j] = va[w][i]; }
        }
    }
    __syncwarp();
}

// The search loop proper. On return bk/bv hold the beam (ascending, position
// j = NB*lane + i, ids still carrying the explored flag). Returns the number of
// expansions; *rows_read accumulates data rows fetched.
template<int NB, int NC, bool NARROW_SORT = false>
__device__ __forceinline__ uint32_t beam_loop(float (&bk)[NB], uint32_t (&bv)[NB], const WarpStrip &s,
                                              const BeamParams &p, uint32_t own_id,
                                              const uint32_t *__restrict__ graph, uint32_t degree,
                                              const float *__restrict__ data, uint32_t dim, int metric,
                                              uint32_t *rows_read, bool wide_first_sort = false) {
    const uint32_t lane = lane_id();
    constexpr uint32_t MAXB = 32u * NB;
    uint32_t iter = 0;
    bool terminate = false;
    uint32_t rows = 0;
    while (true) {
        // -- sort the candidates (search_kernel.cuh:9-37) --
        // The reference sorts MAX_CANDIDATE = 64 slots even for degree <= 32, the upper half being
        // padding (FLT_MAX, 0xffffffff). As long as every FLT_MAX slot carries the padding id, the
        // first `degree` outputs of that network equal those of the 32-slot network on the real
        // slots alone, ties included (checked exhaustively-at-random in
        // tests/test_oracle_primitives.py); the only input that breaks this is the seed row's
        // excluded id (valid id, FLT_MAX), flagged by wide_first_sort. Used by the build kernels
        // (instruction bound); the query search kernel is bound by row gathers and measured
        // slower with it.
        if (NARROW_SORT && NC == 2 && degree <= 32 && !(wide_first_sort && iter == 0)) {
            float ck[1] = {lane < degree ? s.cand_dist[lane] : FLT_MAX};
            uint32_t cv[1] = {lane < degree ? s.cand_id[lane] : kInvalid};
            warp_sort<1>(ck, cv);
            __syncwarp();
            if (lane < degree && lane < p.beam) {
                s.cand_dist[lane] = ck[0];
                s.cand_id[lane] = cv[0];
            }
            __syncwarp();
        } else if constexpr (NC == 8) {
            sort_candidates_two_warps(s.cand_dist, s.cand_id, degree, p.beam);
        } else {
            float ck[NC];
            uint32_t cv[NC];
#pragma unroll
            for (int i = 0; i < NC; i++) {
                const uint32_t j = lane + 32u * i;
                ck[i] = (j < degree) ? s.cand_dist[j] : FLT_MAX;
                cv[i] = (j < degree) ? s.cand_id[j] : kInvalid;
            }
            warp_sort<NC>(ck, cv);
            __syncwarp();
#pragma unroll
            for (int i = 0; i < NC; i++) {
                const uint32_t j = NC * lane + i;
                if (j < degree && j < p.beam) {
                    s.cand_dist[j] = ck[i];
                    s.cand_id[j] = cv[i];
                }
            }
            __syncwarp();
        }
        // -- merge into the beam (search_kernel.cuh:97-147) --
        if (iter == 0) {
#pragma unroll
            for (int i = 0; i < NB; i++) {
                const uint32_t j = NB * lane + i;
                const bool take = (j < p.beam) && (j < degree);
                bk[i] = take ? s.cand_dist[j] : FLT_MAX;
                bv[i] = take ? s.cand_id[j] : kInvalid;
            }
        } else if constexpr (NB == 16) {
            merge_beam_two_warps(bk, bv, p.beam, degree, s.cand_dist, s.cand_id, reinterpret_cast<float *>(s.tail), s.tail + 512);
        } else {
#pragma unroll
            for (int i = 0; i < NB; i++) {
                const uint32_t j = NB * lane + i;
                const uint32_t k = MAXB - 1 - j;
                if (k < p.beam && k < degree) {
                    const float c = s.cand_dist[k];
                    if (bk[i] > c) {
                        bk[i] = c;
                        bv[i] = s.cand_id[k];
                    }
                }
            }
            warp_merge_final<NB>(bk, bv);
#pragma unroll
            for (int i = 0; i < NB; i++) {
                const uint32_t j = NB * lane + i;
                if (j >= p.beam) {  // the reference keeps only `beam` slots between iterations
                    bk[i] = FLT_MAX;
                    bv[i] = kInvalid;
                }
            }
        }
        __syncwarp();
        const bool reset = ((iter + 1) % p.hash_reset_interval) == 0;
        if (reset) {
            visited_clear(s.visited, p.hash_bit);
            __syncwarp();
        }
        if (iter + 1 == p.max_iterations) break;
        // -- first beam slot not yet expanded (search_kernel.cuh:292-325) --
        uint32_t parent = kInvalid;
        {
            int first = -1;
#pragma unroll
            for (int i = NB - 1; i >= 0; i--)
                if ((bv[i] & kExplored) == 0) first = i;
            const uint32_t has = __ballot_sync(kFullMask, first >= 0);
            if (has == 0) {
                terminate = true;
            } else {
                const uint32_t src = __ffs(has) - 1;
                uint32_t mine = kInvalid;
                if (lane == src) {
#pragma unroll
                    for (int i = 0; i < NB; i++)
                        if (i == first) {
                            mine = bv[i];
                            bv[i] |= kExplored;
                        }
                }
                parent = __shfl_sync(kFullMask, mine, src);
            }
        }
        if (reset) {  // search_kernel.cuh:327-334
#pragma unroll
            for (int i = 0; i < NB; i++) {
                const uint32_t j = NB * lane + i;
                visited_insert(s.visited, p.hash_bit, bv[i] & kClean, j < p.beam);
            }
            __syncwarp();
        }
        if (terminate && iter >= p.min_iterations) break;
        rows += expand_parent(s, parent, own_id, graph, degree, p.hash_bit, data, dim, metric);
        iter++;
    }
    if (rows_read) *rows_read += rows;
    return iter;
}

// ---------------------------------------------------------------------------
// Lane-resident variant for adjacency rows of at most 32 entries: candidate slot l lives in
// lane l's registers from the adjacency read to the merge, so the loop touches shared memory
// only for the visited set. Same networks, same tie order:
//  * the reference sorts MAX_CANDIDATE = 64 slots, the upper 32 being padding (FLT_MAX,
//    0xffffffff); the first 32 outputs of that network equal those of the 32-slot network on the
//    real slots alone as long as every FLT_MAX slot carries the padding id (checked at random in
//    tests/test_oracle_primitives.py). The one input that breaks this is the seed row's excluded
//    id (a valid id with FLT_MAX), which takes the 64-slot network once (wide_first_sort);
//  * for beam <= 32 the 64-position merge network splits, after its first stride-32 step, into
//    two independent halves of which only the lower one is kept, so NB = 1 gives the same beam.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t seed_lanes(const WarpStrip &s, uint32_t start_point, uint32_t exclude_id,
                                               const uint32_t *__restrict__ graph, uint32_t degree, uint32_t hash_bit,
                                               const float *__restrict__ data, uint32_t dim, int metric, float &ck,
                                               uint32_t &cv, bool *excluded_kept = nullptr) {
    const uint32_t lane = lane_id();
    uint32_t index = kInvalid;
    if (lane < degree) index = __ldg(graph + (uint64_t) start_point * degree + lane);
    const uint32_t flag = visited_insert(s.visited, hash_bit, index, index != kInvalid);
    cv = flag ? index : kInvalid;
    if (excluded_kept) *excluded_kept = __ballot_sync(kFullMask, flag && index == exclude_id) != 0;
    const uint32_t mask = __ballot_sync(kFullMask, cv != kInvalid && cv != exclude_id);
    __syncwarp();
    ck = score_lanes(s.query, data, dim, metric, mask, cv, s.cand_id);
    return __popc(mask);
}

__device__ __forceinline__ uint32_t expand_lanes(const WarpStrip &s, uint32_t parent, uint32_t own_id,
                                                 const uint32_t *__restrict__ graph, uint32_t degree, uint32_t hash_bit,
                                                 const float *__restrict__ data, uint32_t dim, int metric, float &ck,
                                                 uint32_t &cv) {
    const uint32_t lane = lane_id();
    uint32_t nb = kInvalid;
    if (lane < degree && parent != kInvalid) nb = __ldg(graph + (uint64_t) parent * degree + lane);
    const uint32_t flag = visited_insert(s.visited, hash_bit, nb, nb != kInvalid && nb != own_id);
    cv = flag ? nb : kInvalid;
    const uint32_t mask = __ballot_sync(kFullMask, flag != 0);
    __syncwarp();
    ck = score_lanes(s.query, data, dim, metric, mask, cv, s.cand_id);
    return __popc(mask);
}

// (ck, cv): the seed step's candidates, slot = lane. Otherwise as beam_loop.
template<int NB>
__device__ __forceinline__ uint32_t beam_loop_lanes(float (&bk)[NB], uint32_t (&bv)[NB], const WarpStrip &s,
                                                    const BeamParams &p, uint32_t own_id,
                                                    const uint32_t *__restrict__ graph, uint32_t degree,
                                                    const float *__restrict__ data, uint32_t dim, int metric,
                                                    uint32_t *rows_read, float ck, uint32_t cv,
                                                    bool wide_first_sort = false) {
    const uint32_t lane = lane_id();
    constexpr uint32_t MAXB = 32u * NB;
    uint32_t iter = 0;
    bool terminate = false;
    uint32_t rows = 0;
    while (true) {
        // -- sort the candidates (search_kernel.cuh:9-37): afterwards lane j holds the j-th --
        if (wide_first_sort && iter == 0) {
            float k2[2] = {ck, FLT_MAX};          // slot j = lane + 32*i
            uint32_t v2[2] = {cv, kInvalid};
            warp_sort<2>(k2, v2);                 // sorted position e = 2*lane + i
            const float a = __shfl_sync(kFullMask, k2[0], lane >> 1), b = __shfl_sync(kFullMask, k2[1], lane >> 1);
            const uint32_t c = __shfl_sync(kFullMask, v2[0], lane >> 1), d = __shfl_sync(kFullMask, v2[1], lane >> 1);
            ck = (lane & 1u) ? b : a;
            cv = (lane & 1u) ? d : c;
        } else {
            float k1[1] = {ck};
            uint32_t v1[1] = {cv};
            warp_sort<1>(k1, v1);
            ck = k1[0];
            cv = v1[0];
        }
        // -- merge into the beam (search_kernel.cuh:97-147) --
        if (iter == 0) {
#pragma unroll
            for (int i = 0; i < NB; i++) {
                const uint32_t j = NB * lane + i;
                const float c = __shfl_sync(kFullMask, ck, j & 31u);
                const uint32_t id = __shfl_sync(kFullMask, cv, j & 31u);
                const bool take = (j < p.beam) && (j < degree);
                bk[i] = take ? c : FLT_MAX;
                bv[i] = take ? id : kInvalid;
            }
        } else if constexpr (NB == 16) {
            float *row_k = reinterpret_cast<float *>(s.tail + 1024);
            uint32_t *row_v = s.tail + 1024 + 32;
            row_k[lane] = ck;          // the sorted candidate row, slot = lane
            row_v[lane] = cv;
            __syncwarp();
            merge_beam_two_warps(bk, bv, p.beam, degree, row_k, row_v, reinterpret_cast<float *>(s.tail), s.tail + 512);
        } else {
#pragma unroll
            for (int i = 0; i < NB; i++) {
                const uint32_t j = NB * lane + i;
                const uint32_t k = MAXB - 1 - j;
                const float c = __shfl_sync(kFullMask, ck, k & 31u);
                const uint32_t id = __shfl_sync(kFullMask, cv, k & 31u);
                if (k < p.beam && k < degree && bk[i] > c) {
                    bk[i] = c;
                    bv[i] = id;
                }
            }
            warp_merge_final<NB>(bk, bv);
#pragma unroll
            for (int i = 0; i < NB; i++) {
                const uint32_t j = NB * lane + i;
                if (j >= p.beam) {  // the reference keeps only `beam` slots between iterations
                    bk[i] = FLT_MAX;
                    bv[i] = kInvalid;
                }
            }
        }
        const bool reset = ((iter + 1) % p.hash_reset_interval) == 0;
        if (reset) {
            __syncwarp();
            visited_clear(s.visited, p.hash_bit);
            __syncwarp();
        }
        if (iter + 1 == p.max_iterations) break;
        // -- first beam slot not yet expanded (search_kernel.cuh:292-325) --
        uint32_t parent = kInvalid;
        {
            int first = -1;
#pragma unroll
            for (int i = NB - 1; i >= 0; i--)
                if ((bv[i] & kExplored) == 0) first = i;
            const uint32_t has = __ballot_sync(kFullMask, first >= 0);
            if (has == 0) {
                terminate = true;
            } else {
                const uint32_t src = __ffs(has) - 1;
                uint32_t mine = kInvalid;
                if (lane == src) {
#pragma unroll
                    for (int i = 0; i < NB; i++)
                        if (i == first) {
                            mine = bv[i];
                            bv[i] |= kExplored;
                        }
                }
                parent = __shfl_sync(kFullMask, mine, src);
            }
        }
        if (reset) {  // search_kernel.cuh:327-334
#pragma unroll
            for (int i = 0; i < NB; i++) {
                const uint32_t j = NB * lane + i;
                visited_insert(s.visited, p.hash_bit, bv[i] & kClean, j < p.beam);
            }
            __syncwarp();
        }
        if (terminate && iter >= p.min_iterations) break;
        rows += expand_lanes(s, parent, own_id, graph, degree, p.hash_bit, data, dim, metric, ck, cv);
        iter++;
    }
    if (rows_read) *rows_read += rows;
    return iter;
}

}  // namespace glide

// Binds run-time (beam, degree) size classes to template instances; the classes are the
// reference's ladders (kernel_config.cuh:36-61): beam <=64/128/256/512, degree <=64/128/256.
#define GLIDE_DISPATCH_NB_NC(FN, nb, nc, ...)                                              \
    do {                                                                                   \
        if (nc == 2) {                                                                     \
            if (nb == 2) return FN<2, 2>(__VA_ARGS__);                                     \
            if (nb == 4) return FN<4, 2>(__VA_ARGS__);                                     \
            if (nb == 8) return FN<8, 2>(__VA_ARGS__);                                     \
            return FN<16, 2>(__VA_ARGS__);                                                 \
        } else if (nc == 4) {                                                              \
            if (nb == 2) return FN<2, 4>(__VA_ARGS__);                                     \
            if (nb == 4) return FN<4, 4>(__VA_ARGS__);                                     \
            if (nb == 8) return FN<8, 4>(__VA_ARGS__);                                     \
            return FN<16, 4>(__VA_ARGS__);                                                 \
        } else {                                                                           \
            if (nb == 2) return FN<2, 8>(__VA_ARGS__);                                     \
            if (nb == 4) return FN<4, 8>(__VA_ARGS__);                                     \
            if (nb == 8) return FN<8, 8>(__VA_ARGS__);                                     \
            return FN<16, 8>(__VA_ARGS__);                                                 \
        }                                                                                  \
    } while (0)
