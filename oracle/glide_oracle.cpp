// CPU oracle for the GLIDE hot path.
//
// THIS FILE IS TEST INFRASTRUCTURE. It is a sequential restatement, written from
// scratch, of what the reference's CUDA kernels compute, so that the CUDA path of
// this repository can be checked against it. Nothing in the product path may link
// or call it; only tests, the smoke check and the CPU-baseline leg of the benchmark
// do.
//
// PINNING. The reference ships no golden vectors, known-answer tests or fixtures for any
// stage, has no CPU code path, and its programs cannot be built without RAFT/cuVS (fetched
// at configure time, absent here). Its kernel headers, however, compile on their own:
// ref_harness.cu launches the reference's search, build, boundary, reverse, refine and
// partition kernels, and the GPU tests (tests/test_gpu_reference.py) compare them with this
// restatement in the reference's summation order: search, build, boundary merge and
// assignment bit for bit; reverse edges as one of the arrival orders allowed here; refine up
// to the reference's in-place race. Outputs of those reference kernels on small seeded inputs are
// stored under tests/golden/ (made by tests/golden/make_reference_goldens.py) and compared
// with this restatement by the CPU-only tests. PARITY UNPINNED for what has no reference arithmetic in
// the tree: k-means and NN-descent (cuVS calls), which restate this repository's own
// algorithms.
//
// Each function cites the reference file:line it follows (paths relative to the
// reference's src/ directory).
//
// Arithmetic notes that matter for bit-exactness:
//  * nvcc contracts `acc += d*d` into one fused multiply-add (default -fmad=true),
//    so every accumulation here uses fmaf(). This file must be compiled with
//    -ffp-contract=off so that nothing else is fused.
//  * sqrtf and the fp32 division are IEEE-correct on both sides (nvcc defaults
//    -prec-sqrt=true, -prec-div=true).
#include <algorithm>
#include <cfloat>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

constexpr uint32_t kInvalid = 0xffffffffu;   // utils.cuh:52-55 (get_max_value<uint32_t>)
constexpr uint32_t kExplored = 0x80000000u;  // utils.cuh:5-8 (index_mask::explored)
constexpr uint32_t kClean = ~kExplored;
constexpr float kMaxF = FLT_MAX;             // utils.cuh:47-50

enum Metric : int { kEuclidean = 0, kCosine = 1 };  // params.cuh:5-8

// Summation orders. kOrderRef is the reference's: lane l of a 32-lane warp adds
// elements l, l+32, ... and a shuffle-down tree (16,8,4,2,1) folds the lanes
// (distance.cuh:13-21). The other two are the orders of this repository's CUDA kernels.
// kOrderTeam (centroid distances: routing, assignment, k-means): a team of 8 lanes, lane t
// owning 4-float chunks t, t+8, ... (scalar elements t, t+8, ... when dim is not a multiple
// of 4), folded by a 4,2,1 tree. kOrderWarp (candidate scoring and pruning): the 32 lanes
// of a warp, lane l owning 4-float chunks l, l+32, ..., folded by the reference's
// 16,8,4,2,1 tree; when dim is not a multiple of 4 it is exactly kOrderRef.
enum Order : int { kOrderRef = 0, kOrderTeam = 1, kOrderWarp = 2 };

inline float sq_sum(const float *a, const float *b, uint32_t dim, int order) {
    float lane[32];
    uint32_t T, V;
    if (order == kOrderRef) {
        T = 32;
        V = 1;
    } else if (order == kOrderWarp) {
        T = 32;
        V = (dim % 4 == 0) ? 4 : 1;
    } else {
        T = 8;
        V = (dim % 4 == 0) ? 4 : 1;
    }
    const uint32_t chunks = dim / V;
    for (uint32_t t = 0; t < T; t++) {
        float acc = 0.0f;
        for (uint32_t c = t; c < chunks; c += T) {
            for (uint32_t e = 0; e < V; e++) {
                const float diff = a[c * V + e] - b[c * V + e];
                acc = fmaf(diff, diff, acc);
            }
        }
        lane[t] = acc;
    }
    for (uint32_t off = T / 2; off > 0; off >>= 1) {
        for (uint32_t t = 0; t < off; t++) lane[t] = lane[t] + lane[t + off];
    }
    return lane[0];
}

// distance.cuh:9-27: sqrt of the sum for Euclidean, the raw sum for Cosine
// (vectors are normalised by the caller).
inline float distance(const float *a, const float *b, uint32_t dim, int metric, int order) {
    const float s = sq_sum(a, b, dim, order);
    return metric == kEuclidean ? sqrtf(s) : s;
}

// ---------------------------------------------------------------------------
// Register-resident warp bitonic network, emulated as 32 lanes x N registers.
// bitonic.cuh:24-44 (compare-exchange never swaps equal keys), :46-85 (generic
// merge step), :202-212 (sort = merges of range 1,2,...,32). Only power-of-two N
// occurs (N = MAX/32 with MAX in {32,64,128,256,512}).
// ---------------------------------------------------------------------------
struct WarpRegs {
    uint32_t N;
    std::vector<float> k;     // [lane * N + i]
    std::vector<uint32_t> v;  // [lane * N + i]
    explicit WarpRegs(uint32_t n) : N(n), k(32 * n), v(32 * n) {}
    float &K(uint32_t lane, uint32_t i) { return k[lane * N + i]; }
    uint32_t &V(uint32_t lane, uint32_t i) { return v[lane * N + i]; }
};

inline void cx_local(float &k0, uint32_t &v0, float &k1, uint32_t &v1, bool asc) {
    if ((k0 != k1) && ((k0 < k1) != asc)) {
        std::swap(k0, k1);
        std::swap(v0, v1);
    }
}

void warp_merge(WarpRegs &r, uint32_t range) {
    const uint32_t N = r.N;
    if (range == 1) {
        for (uint32_t lane = 0; lane < 32; lane++) {
            for (uint32_t b = 2; b <= N; b <<= 1) {
                for (uint32_t c = b / 2; c >= 1; c >>= 1) {
                    for (uint32_t i = 0; i < N; i++) {
                        const uint32_t j = i ^ c;
                        if (i >= j) continue;
                        const uint32_t line = i + N * lane;
                        const bool p = ((line & b) != 0) == ((line & c) != 0);
                        cx_local(r.K(lane, i), r.V(lane, i), r.K(lane, j), r.V(lane, j), p);
                    }
                }
            }
        }
        return;
    }
    const uint32_t b = range;
    std::vector<float> nk(32 * N);
    std::vector<uint32_t> nv(32 * N);
    for (uint32_t c = b / 2; c >= 1; c >>= 1) {
        for (uint32_t lane = 0; lane < 32; lane++) {
            const bool p = ((lane & b) != 0) == ((lane & c) != 0);
            const uint32_t other = lane ^ c;
            for (uint32_t i = 0; i < N; i++) {
                const float k0 = r.K(lane, i), k1 = r.K(other, i);
                if ((k0 != k1) && ((k0 < k1) != p)) {
                    nk[lane * N + i] = k1;
                    nv[lane * N + i] = r.V(other, i);
                } else {
                    nk[lane * N + i] = k0;
                    nv[lane * N + i] = r.V(lane, i);
                }
            }
        }
        r.k = nk;
        r.v = nv;
    }
    for (uint32_t lane = 0; lane < 32; lane++) {
        const bool p = ((lane & b) == 0);
        for (uint32_t c = N / 2; c >= 1; c >>= 1) {
            for (uint32_t i = 0; i < N; i++) {
                const uint32_t j = i ^ c;
                if (i >= j) continue;
                cx_local(r.K(lane, i), r.V(lane, i), r.K(lane, j), r.V(lane, j), p);
            }
        }
    }
}

void warp_sort(WarpRegs &r) {
    for (uint32_t range = 1; range <= 32; range <<= 1) warp_merge(r, range);
}

// distance.cuh:29-59. Element j is loaded into lane j%32, register j/32; results
// are read back lane-major (position N*lane+i).
void sort_with_key_value(uint32_t max_number, uint32_t number, uint32_t *vals, float *keys) {
    const uint32_t N = (max_number + 31) / 32;
    WarpRegs r(N);
    for (uint32_t lane = 0; lane < 32; lane++)
        for (uint32_t i = 0; i < N; i++) {
            const uint32_t j = lane + 32 * i;
            r.K(lane, i) = (j < number) ? keys[j] : kMaxF;
            r.V(lane, i) = (j < number) ? vals[j] : kInvalid;
        }
    warp_sort(r);
    for (uint32_t lane = 0; lane < 32; lane++)
        for (uint32_t i = 0; i < N; i++) {
            const uint32_t j = N * lane + i;
            if (j < number) {
                keys[j] = r.K(lane, i);
                vals[j] = r.V(lane, i);
            }
        }
}

// ---------------------------------------------------------------------------
// Visited set: open addressing, linear probing. hashmap.cuh:21-56. A full table
// reports "already seen".
// ---------------------------------------------------------------------------
struct VisitedSet {
    uint32_t bits;
    std::vector<uint32_t> table;
    explicit VisitedSet(uint32_t b) : bits(b), table(1u << b, kInvalid) {}
    void clear() { std::fill(table.begin(), table.end(), kInvalid); }
    uint32_t insert(uint32_t key) {
        const uint32_t size = 1u << bits, mask = size - 1;
        uint32_t index = (key ^ (key >> bits)) & mask;
        for (uint32_t i = 0; i < size; i++) {
            if (table[index] == kInvalid) {
                table[index] = key;
                return 1;
            }
            if (table[index] == key) return 0;
            index = (index + 1) & mask;
        }
        return 0;
    }
};

uint32_t ladder_beam(uint32_t beam) {  // kernel_config.cuh:40-48
    if (beam <= 64) return 64;
    if (beam <= 128) return 128;
    if (beam <= 256) return 256;
    return 512;
}
uint32_t ladder_cand(uint32_t degree) {  // kernel_config.cuh:52-60
    if (degree <= 64) return 64;
    if (degree <= 128) return 128;
    return 256;
}
// The reference picks MAX_CENTROID from 32/64/128/256 (kernel_config.cuh:206-216,
// 223-235); its >32 branch keys on graph_degree and silently ignores centroids
// beyond the template size. Here: the smallest power of two >= C, at least 32.
uint32_t ladder_centroid(uint32_t c) {
    uint32_t m = 32;
    while (m < c) m <<= 1;
    return m;
}

// Tests switch the two-warp sort and merge off to check them against the single-warp network
// (same keys in the same order; only ids of equal keys may differ).
bool g_two_warps = true;

struct SearchCfg {
    uint32_t beam;            // already rounded to a multiple of 32 (params.cuh:94-98)
    uint32_t max_iterations;  // params.cuh:85-93
    uint32_t min_iterations;
    uint32_t hash_bit;             // params.cuh:49-66
    uint32_t hash_reset_interval;  // params.cuh:68-80
};

// One beam-search state: search_kernel.cuh:393-490 / graph_kernel.cuh:5-68.
struct BeamState {
    uint32_t beam, max_beam, deg, max_cand;
    std::vector<float> beam_dist, cand_dist;
    std::vector<uint32_t> beam_id, cand_id;
    VisitedSet visited;
    uint64_t n_dist = 0;  // distance evaluations against data rows
    uint32_t n_iter = 0;  // expansions
    bool two_warps = g_two_warps;   // the reference's kernels run with at least 64 threads (two warps) per query or point
    BeamState(const SearchCfg &c, uint32_t degree)
        : beam(c.beam), max_beam(ladder_beam(c.beam)), deg(degree), max_cand(ladder_cand(degree)),
          beam_dist(c.beam, kMaxF), cand_dist(degree, kMaxF), beam_id(c.beam, kInvalid),
          cand_id(degree, kInvalid), visited(c.hash_bit) {}

    // search_kernel.cuh:38-95: MAX_CANDIDATE > 128 splits the candidates over two warps. Each sorts its
    // half of 128, the halves exchange mirrored elements (equal keys stay where they are, warp 0
    // keeps the smaller), and each merges its half again. Restated as the reference's kernels run it:
    // two register files, one candidate buffer.
    void sort_candidates_two_warps() {
        const uint32_t per = (max_cand + 1) / 2, N = (per + 31) / 32;
        WarpRegs regs[2] = {WarpRegs(N), WarpRegs(N)};
        for (uint32_t w = 0; w < 2; w++) {
            WarpRegs &r = regs[w];
            for (uint32_t lane = 0; lane < 32; lane++)
                for (uint32_t i = 0; i < N; i++) {
                    const uint32_t j = lane + 32 * i + per * w;
                    r.K(lane, i) = (j < deg) ? cand_dist[j] : kMaxF;
                    r.V(lane, i) = (j < deg) ? cand_id[j] : kInvalid;
                }
        }
        for (uint32_t w = 0; w < 2; w++) {   // both warps have read before either writes (reads and writes touch its own half only)
            WarpRegs &r = regs[w];
            warp_sort(r);
            for (uint32_t lane = 0; lane < 32; lane++)
                for (uint32_t i = 0; i < N; i++) {
                    const uint32_t jl = N * lane + i, j = jl + per * w;
                    if (j < deg && jl < beam) {
                        cand_dist[j] = r.K(lane, i);
                        cand_id[j] = r.V(lane, i);
                    }
                }
        }
        const uint32_t used = (beam + per - 1) / per;
        for (uint32_t w = 0; w < used && w < 2; w++) {   // reads of the buffer only: no order between the warps
            WarpRegs &r = regs[w];
            for (uint32_t lane = 0; lane < 32; lane++)
                for (uint32_t i = 0; i < N; i++) {
                    const uint32_t jl = N * lane + i, kl = per - 1 - jl, j = jl + per * w, k = max_cand - 1 - j;
                    if (j >= deg || k >= deg || kl >= beam) continue;
                    const float other = cand_dist[k];
                    if (r.K(lane, i) == other) continue;
                    if ((w == 0) == (r.K(lane, i) > other)) {
                        r.K(lane, i) = other;
                        r.V(lane, i) = cand_id[k];
                    }
                }
        }
        for (uint32_t w = 0; w < used && w < 2; w++) {
            WarpRegs &r = regs[w];
            warp_merge(r, 32);
            for (uint32_t lane = 0; lane < 32; lane++)
                for (uint32_t i = 0; i < N; i++) {
                    const uint32_t j = N * lane + i + per * w;
                    if (j < deg && j < beam) {
                        cand_dist[j] = r.K(lane, i);
                        cand_id[j] = r.V(lane, i);
                    }
                }
        }
    }
    // search_kernel.cuh:148-233: MAX_BEAM > 256 merges with two warps. Candidates replace mirrored beam
    // slots, the two halves of the beam exchange pairwise, and each warp merges its half, which it
    // loads around a "turning point" (the first slot the exchange touched) so that the sequence is
    // bitonic. The three minima the reference takes with atomics do not depend on thread order.
    void merge_into_beam_two_warps() {
        const uint32_t half = beam / 2, per = (max_beam + 1) / 2, N = (per + 31) / 32;
        uint32_t ws[3] = {half, half, half};
        const uint32_t lim = std::min(deg, beam);
        for (uint32_t k = 0; k < lim; k++) {
            const uint32_t j = beam - 1 - k;
            if (beam_dist[j] > cand_dist[k]) {
                beam_dist[j] = cand_dist[k];
                beam_id[j] = cand_id[k];
                if (j < half) ws[2] = std::min(ws[2], j);
                else ws[1] = std::min(ws[1], j - half);
            }
        }
        for (uint32_t j = 0; j < half; j++) {
            const uint32_t k = j + half;
            if (beam_dist[j] > beam_dist[k]) {
                std::swap(beam_dist[j], beam_dist[k]);
                std::swap(beam_id[j], beam_id[k]);
                ws[0] = std::min(ws[0], j);
            }
        }
        if (ws[2] < half) ws[1] = ws[2];
        for (uint32_t w = 0; w < 2; w++) {
            const uint32_t turning = ws[w];
            WarpRegs r(N);
            for (uint32_t lane = 0; lane < 32; lane++)
                for (uint32_t i = 0; i < N; i++) {
                    uint32_t k = beam, j = N * lane + i;
                    if (j < turning) {
                        k = j + half * w;
                    } else if (j >= max_beam / 2 - half) {
                        j -= max_beam / 2 - half;
                        if (turning <= j && j < half) k = j + half * w;
                    }
                    r.K(lane, i) = (k < beam) ? beam_dist[k] : kMaxF;
                    r.V(lane, i) = (k < beam) ? beam_id[k] : kInvalid;
                }
            warp_merge(r, 32);
            for (uint32_t lane = 0; lane < 32; lane++)
                for (uint32_t i = 0; i < N; i++) {
                    const uint32_t j = N * lane + i;
                    if (j < half) {
                        beam_dist[j + half * w] = r.K(lane, i);
                        beam_id[j + half * w] = r.V(lane, i);
                    }
                }
        }
    }
    // search_kernel.cuh:9-37 (single-warp branch).
    void sort_candidates() {
        if (max_cand > 128 && two_warps) return sort_candidates_two_warps();
        const uint32_t N = max_cand / 32;
        WarpRegs r(N);
        for (uint32_t lane = 0; lane < 32; lane++)
            for (uint32_t i = 0; i < N; i++) {
                const uint32_t j = lane + 32 * i;
                r.K(lane, i) = (j < deg) ? cand_dist[j] : kMaxF;
                r.V(lane, i) = (j < deg) ? cand_id[j] : kInvalid;
            }
        warp_sort(r);
        for (uint32_t lane = 0; lane < 32; lane++)
            for (uint32_t i = 0; i < N; i++) {
                const uint32_t j = N * lane + i;
                if (j < deg && j < beam) {
                    cand_dist[j] = r.K(lane, i);
                    cand_id[j] = r.V(lane, i);
                }
            }
    }
    // search_kernel.cuh:97-147 (single-warp branch).
    void merge_into_beam(bool first) {
        if (first) {
            for (uint32_t i = 0; i < beam; i++) {
                beam_dist[i] = (i < deg) ? cand_dist[i] : kMaxF;
                beam_id[i] = (i < deg) ? cand_id[i] : kInvalid;
            }
            return;
        }
        if (max_beam > 256 && two_warps) return merge_into_beam_two_warps();
        const uint32_t N = max_beam / 32;
        WarpRegs r(N);
        for (uint32_t lane = 0; lane < 32; lane++)
            for (uint32_t i = 0; i < N; i++) {
                const uint32_t j = N * lane + i;
                r.K(lane, i) = (j < beam) ? beam_dist[j] : kMaxF;
                r.V(lane, i) = (j < beam) ? beam_id[j] : kInvalid;
            }
        for (uint32_t lane = 0; lane < 32; lane++)
            for (uint32_t i = 0; i < N; i++) {
                const uint32_t j = N * lane + i;
                const uint32_t k = max_beam - 1 - j;
                if (k >= beam || k >= deg) continue;
                if (r.K(lane, i) > cand_dist[k]) {
                    r.K(lane, i) = cand_dist[k];
                    r.V(lane, i) = cand_id[k];
                }
            }
        warp_merge(r, 32);
        for (uint32_t lane = 0; lane < 32; lane++)
            for (uint32_t i = 0; i < N; i++) {
                const uint32_t j = N * lane + i;
                if (j < beam) {
                    beam_dist[j] = r.K(lane, i);
                    beam_id[j] = r.V(lane, i);
                }
            }
    }
    // search_kernel.cuh:292-325: first beam slot not yet expanded.
    uint32_t select_parent(bool &terminate) {
        for (uint32_t j = 0; j < beam; j++) {
            if ((beam_id[j] & kExplored) == 0) {
                const uint32_t id = beam_id[j];
                beam_id[j] |= kExplored;
                return id;
            }
        }
        terminate = true;
        return kInvalid;
    }
    // search_kernel.cuh:327-334.
    void restore_visited() {
        for (uint32_t i = 0; i < beam; i++) visited.insert(beam_id[i] & kClean);
    }
    // search_kernel.cuh:362-391. own_id = 0xffffffff for query search.
    void expand(uint32_t parent, uint32_t own_id, const uint32_t *graph, const float *query,
                const float *data, uint32_t dim, int metric, int order) {
        for (uint32_t i = 0; i < deg; i++) {
            uint32_t nb = kInvalid;
            if (parent != kInvalid) nb = graph[(uint64_t) parent * deg + i];
            const uint32_t flag = (nb != kInvalid && nb != own_id) ? visited.insert(nb) : 0;
            cand_id[i] = flag ? nb : kInvalid;
        }
        for (uint32_t i = 0; i < deg; i++) {
            const uint32_t id = cand_id[i];
            if (id != kInvalid) {
                cand_dist[i] = distance(query, data + (uint64_t) id * dim, dim, metric, order);
                n_dist++;
            } else {
                cand_dist[i] = kMaxF;
            }
        }
    }
    // The loop of search_kernel.cuh:433-482 == graph_kernel.cuh:16-63.
    void run(const SearchCfg &c, uint32_t own_id, const uint32_t *graph, const float *query,
             const float *data, uint32_t dim, int metric, int order) {
        uint32_t iter = 0;
        bool terminate = false;
        while (true) {
            sort_candidates();
            merge_into_beam(iter == 0);
            const bool reset = ((iter + 1) % c.hash_reset_interval == 0);
            if (reset) visited.clear();
            if (iter + 1 == c.max_iterations) break;
            const uint32_t parent = select_parent(terminate);
            if (reset) restore_visited();
            if (terminate && iter >= c.min_iterations) break;
            expand(parent, own_id, graph, query, data, dim, metric, order);
            iter++;
        }
        n_iter = iter;
    }
    // search_kernel.cuh:248-290: route to the nearest centroid, seed with the
    // adjacency row of that partition's start point.
    void seed_by_centroid(const float *query, const float *data, const uint32_t *graph,
                          const uint32_t *start_points, const float *centroids, uint32_t C,
                          uint32_t dim, int metric, int order, int route_order) {
        std::vector<uint32_t> cid(C);
        std::vector<float> cd(C);
        for (uint32_t i = 0; i < C; i++) {
            cid[i] = i;
            cd[i] = distance(query, centroids + (uint64_t) i * dim, dim, metric, route_order);
        }
        sort_with_key_value(ladder_centroid(C), C, cid.data(), cd.data());
        const uint32_t node = start_points[cid[0]];
        for (uint32_t i = 0; i < deg; i++) {
            const uint32_t index = graph[(uint64_t) node * deg + i];
            const uint32_t flag = (index != kInvalid) ? visited.insert(index) : 0;
            cand_id[i] = flag ? index : kInvalid;
        }
        for (uint32_t i = 0; i < deg; i++) {
            const uint32_t id = cand_id[i];
            if (id != kInvalid) {
                cand_dist[i] = distance(query, data + (uint64_t) id * dim, dim, metric, order);
                n_dist++;
            } else {
                cand_dist[i] = kMaxF;
            }
        }
    }
    // search_kernel.cuh:336-360: seed with a given start point's row. exclude_id is
    // compared with the row's ids as the reference does; note build_kernel passes the
    // point's REORDER id here although the row holds partition-local ids
    // (graph_kernel.cuh:295-298), and the excluded id keeps its slot with distance
    // FLT_MAX.
    void seed_by_row(const float *query, uint32_t exclude_id, const float *data,
                     const uint32_t *graph, uint32_t start_point, uint32_t dim, int metric,
                     int order) {
        for (uint32_t i = 0; i < deg; i++) {
            const uint32_t index = graph[(uint64_t) start_point * deg + i];
            const uint32_t flag = (index != kInvalid) ? visited.insert(index) : 0;
            cand_id[i] = flag ? index : kInvalid;
        }
        for (uint32_t i = 0; i < deg; i++) {
            const uint32_t id = cand_id[i];
            if (id != kInvalid && id != exclude_id) {
                cand_dist[i] = distance(query, data + (uint64_t) id * dim, dim, metric, order);
                n_dist++;
            } else {
                cand_dist[i] = kMaxF;
            }
        }
    }
    // graph_kernel.cuh:65-67, plus a guard the reference lacks: unfilled beam slots
    // (id 0xffffffff, 0x7fffffff once the flag is cleared) would be dereferenced as
    // data rows by the pruning code (graph_kernel.cuh:92,104); they are dropped here,
    // order preserved. With a full beam this is the identity.
    void finish_pool(std::vector<uint32_t> &ids, std::vector<float> &dists) const {
        ids.clear();
        dists.clear();
        for (uint32_t i = 0; i < beam; i++) {
            const uint32_t id = beam_id[i] & kClean;
            if (id == (kInvalid & kClean)) continue;
            ids.push_back(id);
            dists.push_back(beam_dist[i]);
        }
    }
};

// graph_kernel.cuh:70-143. ids are relative to `data` (caller pre-offsets the
// partition); out has `degree` slots, unused ones 0xffffffff.
void sync_prune(const float *data, uint32_t dim, std::vector<uint32_t> &pid,
                std::vector<float> &pdist, uint32_t degree, float alpha, int metric, int order,
                uint32_t *out, uint64_t *n_pairs) {
    for (uint32_t i = 0; i < degree; i++) out[i] = kInvalid;
    uint32_t nsize = 0;
    size_t P = pid.size();
    while (nsize < degree && P > 0) {
        const uint32_t id = pid[0];
        out[nsize++] = id;
        size_t next = 0;
        for (size_t i = 1; i < P; i++) {
            const float d = distance(data + (uint64_t) id * dim, data + (uint64_t) pid[i] * dim, dim,
                                     metric, order);
            if (n_pairs) (*n_pairs)++;
            const bool allow = !(alpha * d < pdist[i]);
            if (allow) {
                pid[next] = pid[i];
                pdist[next] = pdist[i];
                next++;
            }
        }
        P = next;
    }
}

// graph_kernel.cuh:160-247. row: existing graph row (degree), res: pruned result in
// REORDER ids (degree slots), map: reorder id -> original id.
void boundary_merge(uint32_t *row, const uint32_t *res, const uint32_t *map, uint32_t degree) {
    const uint32_t maxdeg = (degree + 31) & ~31u;
    std::vector<uint32_t> E(maxdeg, kInvalid), R;
    std::vector<uint8_t> shared(maxdeg, 0);
    for (uint32_t i = 0; i < degree; i++) E[i] = row[i];
    uint32_t rep = 0;
    for (uint32_t i = 0; i < degree; i++) {
        if (res[i] == kInvalid) continue;
        const uint32_t index = map[res[i]];
        bool non_rep = true;
        uint32_t j;
        for (j = 0; j < degree; j++) {
            if (E[j] == kInvalid) break;
            if (E[j] == index) {
                non_rep = false;
                break;
            }
        }
        if (non_rep) {
            R.push_back(index);
        } else {
            shared[j] = 1;
            rep++;
        }
    }
    const uint32_t valid = (uint32_t) R.size();
    if (rep >= degree / 2) {
        uint32_t pos = 0;
        for (uint32_t i = 0; i < degree && pos < valid; i++)
            if (E[i] == kInvalid) row[i] = R[pos++];
    } else {
        const uint32_t max_need = degree / 2 - rep;
        const uint32_t need = std::min(valid, max_need);
        uint32_t pos = 0;
        for (uint32_t i = 0; i < maxdeg && pos < need; i++) {
            const uint32_t gi = maxdeg - 1 - i;
            if (gi >= degree) continue;
            if (E[gi] == kInvalid || !shared[gi]) row[gi] = R[pos++];
        }
    }
}

// graph_kernel.cuh:455-578 (+ :660-671 for the fill). Works on one row.
void prune_refine(const float *data, uint32_t dim, uint32_t point_id, std::vector<uint32_t> &pid,
                  std::vector<float> &pdist, const uint32_t *row_in, uint32_t degree, float alpha,
                  int metric, int order, uint32_t *row_out, uint64_t *n_pairs) {
    uint32_t need = 0;
    for (uint32_t i = 0; i < degree; i++) need += (row_in[i] == kInvalid);
    std::vector<uint32_t> picks(degree, kInvalid);
    uint32_t nsize = 0;
    size_t P = pid.size();
    while (nsize < need && P > 0) {
        size_t pos = P;
        for (size_t i = 0; i < P; i++) {
            const uint32_t id = pid[i];
            if (id == kInvalid || id == point_id) continue;
            bool present = false;
            for (uint32_t j = 0; j < degree; j++)
                if (row_in[j] == id) {
                    present = true;
                    break;
                }
            if (!present) {
                pos = i;
                break;
            }
        }
        if (pos == P) break;
        const uint32_t id = pid[pos];
        picks[nsize++] = id;
        size_t next = 0;
        for (size_t i = pos; i < P; i++) {
            const float d = distance(data + (uint64_t) id * dim, data + (uint64_t) pid[i] * dim, dim,
                                     metric, order);
            if (n_pairs) (*n_pairs)++;
            const bool allow = !(alpha * d < pdist[i]);
            if (allow) {
                pid[next] = pid[i];
                pdist[next] = pdist[i];
                next++;
            }
        }
        P = next;
    }
    uint32_t pos = 0;
    for (uint32_t i = 0; i < degree; i++) {
        if (row_in[i] == kInvalid) {
            row_out[i] = picks[pos++];
        } else {
            row_out[i] = row_in[i];
        }
    }
}

template<typename F>
void parallel_for(int64_t n, int threads, F f) {
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_max_threads();
#pragma omp parallel for schedule(dynamic, 16) num_threads(threads)
#endif
    for (int64_t i = 0; i < n; i++) f(i);
}

}  // namespace

extern "C" {

int orc_max_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

float orc_distance(const float *a, const float *b, uint32_t dim, int metric, int order) {
    return distance(a, b, dim, metric, order);
}

// params.cuh:49-66
uint32_t orc_hash_bitlen(uint32_t beam, uint32_t graph_degree, float max_fill, uint32_t min_bitlen) {
    uint32_t bitlen;
    const uint32_t max_visited = beam + graph_degree;
    uint32_t lo = 8;
    const uint32_t hi = 13;
    if (lo < min_bitlen) lo = min_bitlen;
    bitlen = lo;
    while (max_visited > (float) (1u << bitlen) * max_fill) bitlen += 1;
    if (bitlen > hi) bitlen = hi;
    return bitlen;
}

// params.cuh:68-80
uint32_t orc_hash_reset_interval(uint32_t beam, uint32_t graph_degree, float max_fill, uint32_t bitlen) {
    uint32_t interval = 1;
    while (true) {
        const uint32_t max_visited = beam + graph_degree * (interval + 1);
        if (max_visited > (float) (1u << bitlen) * max_fill) break;
        interval += 1;
    }
    return interval;
}

// params.cuh:82-99
void orc_adjust_search_params(uint32_t min_iterations, uint32_t *max_iterations, uint32_t *beam) {
    uint32_t m = *max_iterations;
    if (*max_iterations == 0) m = (uint32_t) (1 + std::min(*beam * 1.1, *beam + 10.0));
    if (*max_iterations < min_iterations) m = min_iterations;
    if (*max_iterations < m) *max_iterations = m;
    if (*beam % 32) *beam += 32 - (*beam % 32);
}

// Exposed for unit tests of the network: arrays are [lane*N + i].
void orc_warp_sort(float *keys, uint32_t *vals, uint32_t N) {
    WarpRegs r(N);
    std::copy(keys, keys + 32 * N, r.k.begin());
    std::copy(vals, vals + 32 * N, r.v.begin());
    warp_sort(r);
    std::copy(r.k.begin(), r.k.end(), keys);
    std::copy(r.v.begin(), r.v.end(), vals);
}

void orc_sort_with_key_value(uint32_t max_number, uint32_t number, uint32_t *vals, float *keys) {
    sort_with_key_value(max_number, number, vals, keys);
}

// search_kernel.cuh:393-490 for Q queries. counters (optional) = Q x 2 u64:
// distance evaluations against data rows, expansions.
int orc_search(const float *data, uint32_t dim, const uint32_t *graph, uint32_t degree,
               const float *centroids, uint32_t C, const uint32_t *start_points, const float *queries,
               uint32_t Q, uint32_t top_k, uint32_t beam, uint32_t max_iterations,
               uint32_t min_iterations, uint32_t hash_bit, uint32_t hash_reset_interval, int metric,
               int order, int route_order, uint32_t *out_ids, float *out_dists, uint64_t *counters,
               int threads) {
    if (beam % 32 || beam == 0 || beam > 512 || degree > 256 || top_k > beam) return -1;
    const SearchCfg cfg{beam, max_iterations, min_iterations, hash_bit, hash_reset_interval};
    parallel_for(Q, threads, [&](int64_t q) {
        BeamState s(cfg, degree);
        const float *query = queries + (uint64_t) q * dim;
        s.seed_by_centroid(query, data, graph, start_points, centroids, C, dim, metric, order, route_order);
        s.run(cfg, kInvalid, graph, query, data, dim, metric, order);
        for (uint32_t i = 0; i < top_k; i++) {
            out_ids[(uint64_t) q * top_k + i] = s.beam_id[i] & kClean;
            out_dists[(uint64_t) q * top_k + i] = s.beam_dist[i];
        }
        if (counters) {
            counters[2 * q] = s.n_dist;
            counters[2 * q + 1] = s.n_iter;
        }
    });
    return 0;
}

// build_kernel, graph_kernel.cuh:249-316, for reorder ids [first, first+count):
// beam search over the partition's kNN subgraph (local ids), occlusion pruning, row
// written at the ORIGINAL id through map. seg arrays have S entries (C main
// partitions + the boundary partition); start_points are partition-local ids.
int orc_build_rows(const float *reorder_data, uint32_t dim, const uint32_t *knn, uint32_t knn_degree,
                   const uint32_t *seg_start, const uint32_t *seg_len, uint32_t S,
                   const uint32_t *start_points, const uint32_t *map, uint32_t first, uint32_t count,
                   uint32_t graph_degree, uint32_t beam, uint32_t max_iterations,
                   uint32_t min_iterations, uint32_t hash_bit, uint32_t hash_reset_interval,
                   float alpha, int metric, int order, uint32_t *graph, uint64_t *counters,
                   int threads) {
    if (beam % 32 || beam == 0 || beam > 512 || knn_degree > 256) return -1;
    const SearchCfg cfg{beam, max_iterations, min_iterations, hash_bit, hash_reset_interval};
    parallel_for(count, threads, [&](int64_t t) {
        const uint32_t r = first + (uint32_t) t;
        uint32_t s;
        for (s = 0; s < S; s++)
            if (r < seg_start[s] + seg_len[s]) break;  // graph_kernel.cuh:276-282
        if (s == S) return;
        const float *pdata = reorder_data + (uint64_t) seg_start[s] * dim;
        const uint32_t *pknn = knn + (uint64_t) seg_start[s] * knn_degree;
        const float *query = reorder_data + (uint64_t) r * dim;
        BeamState st(cfg, knn_degree);
        st.seed_by_row(query, r, pdata, pknn, start_points[s], dim, metric, order);
        st.run(cfg, r - seg_start[s], pknn, query, pdata, dim, metric, order);
        std::vector<uint32_t> pid;
        std::vector<float> pdist;
        st.finish_pool(pid, pdist);
        const uint64_t pool_size = pid.size();
        std::vector<uint32_t> out(graph_degree);
        uint64_t pairs = 0;
        sync_prune(pdata, dim, pid, pdist, graph_degree, alpha, metric, order, out.data(), &pairs);
        uint32_t *row = graph + (uint64_t) map[r] * graph_degree;
        for (uint32_t i = 0; i < graph_degree; i++)  // graph_kernel.cuh:152-158 (+segment_start :92)
            row[i] = (out[i] == kInvalid) ? kInvalid : map[out[i] + seg_start[s]];
        if (counters) {
            counters[4 * t] = st.n_dist;
            counters[4 * t + 1] = st.n_iter;
            counters[4 * t + 2] = pairs;
            counters[4 * t + 3] = pool_size;  // == beam when no beam slot stayed unfilled
        }
    });
    return 0;
}

// build_boundary_kernel, graph_kernel.cuh:318-376, for all copies in the boundary
// partition (segment S-1, reorder ids [num, num+B)); merges into existing rows.
int orc_build_boundary(const float *reorder_data, uint32_t dim, const uint32_t *knn,
                       uint32_t knn_degree, uint32_t num, uint32_t boundary_num,
                       uint32_t start_point_local, const uint32_t *map, uint32_t graph_degree,
                       uint32_t beam, uint32_t max_iterations, uint32_t min_iterations,
                       uint32_t hash_bit, uint32_t hash_reset_interval, float alpha, int metric,
                       int order, uint32_t *graph, uint64_t *pool_sizes, int threads) {
    if (beam % 32 || beam == 0 || beam > 512 || knn_degree > 256) return -1;
    const SearchCfg cfg{beam, max_iterations, min_iterations, hash_bit, hash_reset_interval};
    const float *pdata = reorder_data + (uint64_t) num * dim;
    const uint32_t *pknn = knn + (uint64_t) num * knn_degree;
    parallel_for(boundary_num, threads, [&](int64_t t) {
        const uint32_t r = num + (uint32_t) t;
        const float *query = reorder_data + (uint64_t) r * dim;
        BeamState st(cfg, knn_degree);
        st.seed_by_row(query, r, pdata, pknn, start_point_local, dim, metric, order);
        st.run(cfg, r - num, pknn, query, pdata, dim, metric, order);
        std::vector<uint32_t> pid;
        std::vector<float> pdist;
        st.finish_pool(pid, pdist);
        if (pool_sizes) pool_sizes[t] = pid.size();
        std::vector<uint32_t> out(graph_degree);
        sync_prune(pdata, dim, pid, pdist, graph_degree, alpha, metric, order, out.data(), nullptr);
        for (uint32_t i = 0; i < graph_degree; i++)
            if (out[i] != kInvalid) out[i] += num;  // sync_prune adds segment_start (:92)
        // every original point has at most one boundary copy, so rows are disjoint
        boundary_merge(graph + (uint64_t) map[r] * graph_degree, out.data(), map, graph_degree);
    });
    return 0;
}

// reverse_graph_kernel + insert_reverse_kernel, graph_kernel.cuh:378-453. The
// reference's arrival order (atomics, `degree` concurrent launches) is arbitrary;
// this fixes the order rank-major then ascending source id, which is one of the
// orders the reference can produce.
int orc_reverse_graph(uint32_t *graph, uint32_t num, uint32_t degree) {
    std::vector<uint32_t> rev((uint64_t) num * degree, kInvalid), cnt(num, 0);
    for (uint32_t k = 0; k < degree; k++) {
        for (uint32_t src = 0; src < num; src++) {
            const uint32_t dst = graph[(uint64_t) src * degree + k];
            if (dst >= num) continue;
            bool have = false;
            for (uint32_t i = 0; i < degree; i++)
                if (graph[(uint64_t) dst * degree + i] == src) {
                    have = true;
                    break;
                }
            if (have) continue;
            const uint32_t idx = cnt[dst]++;
            if (idx < degree) rev[(uint64_t) dst * degree + idx] = src;
        }
    }
    for (uint32_t p = 0; p < num; p++) {
        const uint32_t nrev = std::min(cnt[p], degree);
        uint32_t pos = 0;
        for (uint32_t i = 0; i < degree && pos < nrev; i++) {
            uint32_t &slot = graph[(uint64_t) p * degree + i];
            if (slot == kInvalid) slot = rev[(uint64_t) p * degree + pos++];
        }
    }
    return 0;
}

// refine_kernel, graph_kernel.cuh:580-673, and refine_for_large_kernel, :730-821 (row_mode: no
// centroids, the search is seeded from start_points[0]'s row with the point itself excluded,
// graph_kernel.cuh:790-792). The reference updates rows in place while other CTAs traverse them,
// so its result depends on the schedule. Here the points are taken in waves of wave_rows
// consecutive ids: every search of a wave reads the graph as the waves before it left it, and the
// wave's rows are written when the whole wave is done. This is the outcome of the reference when
// its CTAs run wave by wave in id order with all reads of a wave preceding its writes.
// wave_rows == 0: one wave (every search reads the graph as it was before refinement).
int orc_refine(const float *data, uint32_t num, uint32_t dim, const uint32_t *graph_in,
               uint32_t *graph_out, uint32_t degree, const float *centroids, uint32_t C,
               const uint32_t *start_points, uint32_t beam, uint32_t max_iterations,
               uint32_t min_iterations, uint32_t hash_bit, uint32_t hash_reset_interval, float alpha,
               int metric, int order, int route_order, uint64_t *pool_sizes, int threads,
               uint32_t wave_rows, int row_mode) {
    if (beam % 32 || beam == 0 || beam > 512 || degree > 256) return -1;
    const SearchCfg cfg{beam, max_iterations, min_iterations, hash_bit, hash_reset_interval};
    if (wave_rows == 0 || wave_rows > num) wave_rows = num;
    std::vector<uint32_t> cur(graph_in, graph_in + (uint64_t) num * degree);   // what searches read
    for (uint32_t lo = 0; lo < num; lo += wave_rows) {
        const uint32_t hi = std::min<uint64_t>(num, (uint64_t) lo + wave_rows);
        parallel_for(hi - lo, threads, [&](int64_t t) {
            const uint32_t p = lo + (uint32_t) t;
            const uint32_t *row = cur.data() + (uint64_t) p * degree;
            uint32_t *out = graph_out + (uint64_t) p * degree;
            uint32_t need = 0;
            for (uint32_t i = 0; i < degree; i++) need += (row[i] == kInvalid);
            if (pool_sizes) pool_sizes[p] = beam;  // rows without holes are not searched
            if (need == 0) {
                for (uint32_t i = 0; i < degree; i++) out[i] = row[i];
                return;
            }
            const float *query = data + (uint64_t) p * dim;
            BeamState st(cfg, degree);
            if (row_mode) st.seed_by_row(query, p, data, cur.data(), start_points[0], dim, metric, order);
            else st.seed_by_centroid(query, data, cur.data(), start_points, centroids, C, dim, metric, order, route_order);
            st.run(cfg, p, cur.data(), query, data, dim, metric, order);
            std::vector<uint32_t> pid;
            std::vector<float> pdist;
            st.finish_pool(pid, pdist);
            if (pool_sizes) pool_sizes[p] = pid.size();
            prune_refine(data, dim, p, pid, pdist, row, degree, alpha, metric, order, out, nullptr);
        });
        std::memcpy(cur.data() + (uint64_t) lo * degree, graph_out + (uint64_t) lo * degree, (uint64_t) (hi - lo) * degree * 4);
    }
    return 0;
}

// define_partition_kernel, partition_kernel.cuh:22-66. seg_index = n x 3
// (segment, slot in segment, slot in boundary segment or 0xffffffff); seg_len has
// C+1 entries. Slots are handed out in ascending original id (the reference's come
// from atomics and are arbitrary within a segment).
int orc_define_partition(const float *data, uint32_t n, uint32_t dim, const float *centroids,
                         uint32_t C, float boundary_factor, int metric, int order,
                         uint32_t *seg_index, uint32_t *seg_len, float *ratio_out) {
    std::vector<uint32_t> nearest(n);
    std::vector<uint8_t> is_boundary(n);
    parallel_for(n, 0, [&](int64_t p) {
        std::vector<uint32_t> cid(C);
        std::vector<float> cd(C);
        for (uint32_t i = 0; i < C; i++) {
            cid[i] = i;
            cd[i] = distance(data + (uint64_t) p * dim, centroids + (uint64_t) i * dim, dim, metric, order);
        }
        sort_with_key_value(ladder_centroid(C), C, cid.data(), cd.data());
        nearest[p] = cid[0];
        is_boundary[p] = (C > 1 && cd[1] / cd[0] <= boundary_factor) ? 1 : 0;
        if (ratio_out) ratio_out[p] = (C > 1) ? cd[1] / cd[0] : INFINITY;
    });
    for (uint32_t i = 0; i <= C; i++) seg_len[i] = 0;
    for (uint32_t p = 0; p < n; p++) {
        seg_index[3 * (uint64_t) p] = nearest[p];
        seg_index[3 * (uint64_t) p + 1] = seg_len[nearest[p]]++;
        seg_index[3 * (uint64_t) p + 2] = is_boundary[p] ? seg_len[C]++ : kInvalid;
    }
    return 0;
}

// reorder_kernel, partition_kernel.cuh:68-100.
int orc_reorder(const float *data, uint32_t n, uint32_t dim, const uint32_t *seg_index,
                const uint32_t *seg_start, float *reorder_data, uint32_t *map) {
    for (uint32_t p = 0; p < n; p++) {
        const uint32_t s = seg_index[3 * (uint64_t) p];
        const uint32_t r = seg_start[s] + seg_index[3 * (uint64_t) p + 1];
        std::memcpy(reorder_data + (uint64_t) r * dim, data + (uint64_t) p * dim, dim * sizeof(float));
        map[r] = p;
        const uint32_t b = seg_index[3 * (uint64_t) p + 2];
        if (b != kInvalid) {
            std::memcpy(reorder_data + (uint64_t) (n + b) * dim, data + (uint64_t) p * dim,
                        dim * sizeof(float));
            map[n + b] = p;
        }
    }
    return 0;
}

// select_segment_kernel, search_kernel.cuh:546-607 (large path query routing).
// out = Q x C ids, 0xffffffff padded.
int orc_select_segments(const float *queries, uint32_t Q, uint32_t dim, const float *centroids,
                        uint32_t C, uint32_t min_segment_num, float boundary_factor, int metric,
                        int order, uint32_t *out) {
    parallel_for(Q, 0, [&](int64_t q) {
        std::vector<uint32_t> cid(C);
        std::vector<float> cd(C);
        for (uint32_t i = 0; i < C; i++) {
            cid[i] = i;
            cd[i] = distance(queries + (uint64_t) q * dim, centroids + (uint64_t) i * dim, dim, metric, order);
        }
        sort_with_key_value(ladder_centroid(C), C, cid.data(), cd.data());
        uint32_t *o = out + (uint64_t) q * C;
        for (uint32_t i = 0; i < C; i++) o[i] = kInvalid;
        uint32_t allow = 0;
        for (uint32_t i = 0; i < C; i++)
            if (cd[i] / cd[0] <= boundary_factor) {
                o[i] = cid[i];
                allow++;
            }
        if (allow < min_segment_num)
            for (uint32_t i = 0; i < min_segment_num - allow && allow + i < C; i++) o[allow + i] = cid[allow + i];
    });
    return 0;
}

// search_on_sub_kernel + result_merge, search_kernel.cuh:609-765: one partition of
// the large path. final_* (Q x top_k) carry the running result across partitions
// and must start as (FLT_MAX, 0xffffffff). data/graph are the partition's (local
// ids), map = local id -> global id.
int orc_search_on_sub(const float *data, uint32_t dim, const uint32_t *graph, uint32_t degree,
                      const uint32_t *map, uint32_t start_point, const float *queries, uint32_t Q,
                      const uint32_t *segment_ids, uint32_t segment_num, uint32_t segment_id,
                      uint32_t top_k, uint32_t beam, uint32_t max_iterations, uint32_t min_iterations,
                      uint32_t hash_bit, uint32_t hash_reset_interval, int metric, int order,
                      uint32_t *final_ids, float *final_dists, int threads) {
    if (beam % 32 || beam == 0 || beam > 512 || degree > 256 || top_k > 128 || top_k > beam) return -1;
    const SearchCfg cfg{beam, max_iterations, min_iterations, hash_bit, hash_reset_interval};
    const uint32_t max_topk = top_k <= 32 ? 32 : (top_k <= 64 ? 64 : 128);  // kernel_config.cuh:309-319
    parallel_for(Q, threads, [&](int64_t q) {
        bool routed = false;
        for (uint32_t i = 0; i < segment_num; i++) {  // search_kernel.cuh:676-688
            const uint32_t s = segment_ids[(uint64_t) q * segment_num + i];
            if (s == segment_id) {
                routed = true;
                break;
            }
            if (s == kInvalid) break;
        }
        if (!routed) return;
        BeamState st(cfg, degree);
        const float *query = queries + (uint64_t) q * dim;
        st.seed_by_row(query, kInvalid, data, graph, start_point, dim, metric, order);
        st.run(cfg, kInvalid, graph, query, data, dim, metric, order);
        // result_merge
        const uint32_t N = max_topk / 32;
        WarpRegs r(N);
        float *fd = final_dists + (uint64_t) q * top_k;
        uint32_t *fi = final_ids + (uint64_t) q * top_k;
        for (uint32_t lane = 0; lane < 32; lane++)
            for (uint32_t i = 0; i < N; i++) {
                const uint32_t j = N * lane + i;
                r.K(lane, i) = (j < top_k) ? fd[j] : kMaxF;
                r.V(lane, i) = (j < top_k) ? fi[j] : kInvalid;
            }
        for (uint32_t lane = 0; lane < 32; lane++)
            for (uint32_t i = 0; i < N; i++) {
                const uint32_t j = N * lane + i;
                const uint32_t k = max_topk - 1 - j;
                if (k >= top_k) continue;
                if (r.K(lane, i) > st.beam_dist[k]) {
                    r.K(lane, i) = st.beam_dist[k];
                    const uint32_t id = st.beam_id[k] & kClean;
                    // guard: an unfilled beam slot has no global id
                    r.V(lane, i) = (id == (kInvalid & kClean)) ? kInvalid : map[id];
                }
            }
        warp_merge(r, 32);
        for (uint32_t lane = 0; lane < 32; lane++)
            for (uint32_t i = 0; i < N; i++) {
                const uint32_t j = N * lane + i;
                if (j < top_k) {
                    fd[j] = r.K(lane, i);
                    fi[j] = r.V(lane, i);
                }
            }
    });
    return 0;
}

// result_merge (search_kernel.cuh:609-651) over whole result sets: set 0 is the running result, sets
// 1 .. G-1 are folded into it in order, as search_on_sub_kernel folds one partition after another.
// ids/dists: G x Q x top_k; out: Q x top_k.
int orc_merge_results(const uint32_t *ids, const float *dists, uint32_t G, uint32_t Q, uint32_t top_k,
                      uint32_t *out_ids, float *out_dists) {
    if (top_k == 0 || top_k > 128 || G == 0) return -1;
    const uint32_t max_topk = top_k <= 32 ? 32 : (top_k <= 64 ? 64 : 128);  // kernel_config.cuh:309-319
    const uint32_t N = max_topk / 32;
    const uint64_t set = (uint64_t) Q * top_k;
    parallel_for(Q, 0, [&](int64_t q) {
        std::vector<float> fd(dists + q * top_k, dists + (q + 1) * top_k);
        std::vector<uint32_t> fi(ids + q * top_k, ids + (q + 1) * top_k);
        for (uint32_t g = 1; g < G; g++) {
            const float *rd = dists + g * set + (uint64_t) q * top_k;
            const uint32_t *ri = ids + g * set + (uint64_t) q * top_k;
            WarpRegs r(N);
            for (uint32_t lane = 0; lane < 32; lane++)
                for (uint32_t i = 0; i < N; i++) {
                    const uint32_t j = N * lane + i;
                    r.K(lane, i) = (j < top_k) ? fd[j] : kMaxF;
                    r.V(lane, i) = (j < top_k) ? fi[j] : kInvalid;
                }
            for (uint32_t lane = 0; lane < 32; lane++)
                for (uint32_t i = 0; i < N; i++) {
                    const uint32_t j = N * lane + i;
                    const uint32_t k = max_topk - 1 - j;
                    if (k >= top_k) continue;
                    if (r.K(lane, i) > rd[k]) {
                        r.K(lane, i) = rd[k];
                        r.V(lane, i) = ri[k];
                    }
                }
            warp_merge(r, 32);
            for (uint32_t lane = 0; lane < 32; lane++)
                for (uint32_t i = 0; i < N; i++) {
                    const uint32_t j = N * lane + i;
                    if (j < top_k) {
                        fd[j] = r.K(lane, i);
                        fi[j] = r.V(lane, i);
                    }
                }
        }
        for (uint32_t j = 0; j < top_k; j++) {
            out_dists[(uint64_t) q * top_k + j] = fd[j];
            out_ids[(uint64_t) q * top_k + j] = fi[j];
        }
    });
    return 0;
}

// load.cuh:10-30: the matrix file read the reference's way, one ifstream::read per row into
// pageable memory. `out` holds rows x dim elements of elem_bytes each. Returns 0, or -5 when the
// file cannot be opened or ends early.
int orc_load_matrix_rowwise(const char *path, uint32_t elem_bytes, void *out, uint32_t *rows_out, uint32_t *dim_out) {
    std::ifstream file(path, std::ios::binary);
    if (!file) return -5;
    uint32_t num = 0, dim = 0;
    file.read(reinterpret_cast<char *>(&num), sizeof(uint32_t));
    file.read(reinterpret_cast<char *>(&dim), sizeof(uint32_t));
    if (!file) return -5;
    if (rows_out) *rows_out = num;
    if (dim_out) *dim_out = dim;
    if (!out) return 0;
    char *dst = static_cast<char *>(out);
    const uint64_t row_bytes = (uint64_t) dim * elem_bytes;
    for (uint32_t i = 0; i < num; i++) {
        file.read(dst + (uint64_t) i * row_bytes, (std::streamsize) row_bytes);
        if (!file) return -5;
    }
    return 0;
}

void orc_set_two_warps(int on) { g_two_warps = on != 0; }

// small_search.cu:14-36
float orc_recall(const uint32_t *neighbors, uint32_t nb_stride, const uint32_t *truth,
                 uint32_t truth_stride, uint32_t Q, uint32_t top_k) {
    float total = 0.0f;
    for (uint32_t q = 0; q < Q; q++) {
        uint32_t correct = 0;
        for (uint32_t k = 0; k < top_k; k++) {
            const uint32_t id = neighbors[(uint64_t) q * nb_stride + k];
            for (uint32_t t = 0; t < top_k; t++)
                if (truth[(uint64_t) q * truth_stride + t] == id) {
                    correct++;
                    break;
                }
        }
        total += (float) correct / top_k;
    }
    return total / Q;
}

// ---------------------------------------------------------------------------
// Exact brute-force kNN: the ground truth for recall and the host-core baseline.
// Not a restatement of reference code (the reference reads ground truth from a
// file, small_search.cu:88); distances are plain fp32 (a-b)^2 sums, ties broken
// by ascending id. sqrt applied for Euclidean so values compare with the kernels'.
// ---------------------------------------------------------------------------
#if defined(__x86_64__)
__attribute__((target("avx2,fma"))) static void l2_block_avx2(const float *q, const float *base,
                                                                uint32_t rows, uint32_t dim, float *out);
#endif
static void l2_block_generic(const float *q, const float *base, uint32_t rows, uint32_t dim, float *out) {
    for (uint32_t r = 0; r < rows; r++) {
        const float *b = base + (uint64_t) r * dim;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        uint32_t i = 0;
        for (; i + 8 <= dim; i += 8)
            for (uint32_t e = 0; e < 8; e++) {
                const float d = q[i + e] - b[i + e];
                acc[e] = fmaf(d, d, acc[e]);
            }
        float s = ((acc[0] + acc[4]) + (acc[2] + acc[6])) + ((acc[1] + acc[5]) + (acc[3] + acc[7]));
        for (; i < dim; i++) {
            const float d = q[i] - b[i];
            s = fmaf(d, d, s);
        }
        out[r] = s;
    }
}
#if defined(__x86_64__)
#include <immintrin.h>
__attribute__((target("avx2,fma"))) static void l2_block_avx2(const float *q, const float *base,
                                                                uint32_t rows, uint32_t dim, float *out) {
    for (uint32_t r = 0; r < rows; r++) {
        const float *b = base + (uint64_t) r * dim;
        __m256 acc = _mm256_setzero_ps();
        uint32_t i = 0;
        for (; i + 8 <= dim; i += 8) {
            const __m256 d = _mm256_sub_ps(_mm256_loadu_ps(q + i), _mm256_loadu_ps(b + i));
            acc = _mm256_fmadd_ps(d, d, acc);
        }
        // same fold as the generic version: (a0+a4),(a1+a5),(a2+a6),(a3+a7) ...
        __m128 lo = _mm256_castps256_ps128(acc), hi = _mm256_extractf128_ps(acc, 1);
        __m128 s4 = _mm_add_ps(lo, hi);                    // a0+a4, a1+a5, a2+a6, a3+a7
        __m128 s2 = _mm_add_ps(s4, _mm_movehl_ps(s4, s4));  // (a0+a4)+(a2+a6), (a1+a5)+(a3+a7)
        float s = _mm_cvtss_f32(_mm_add_ss(s2, _mm_shuffle_ps(s2, s2, 1)));
        for (; i < dim; i++) {
            const float d = q[i] - b[i];
            s = fmaf(d, d, s);
        }
        out[r] = s;
    }
}
#endif

int orc_bruteforce_knn(const float *base, uint32_t n, const float *queries, uint32_t Q, uint32_t dim,
                       uint32_t k, int metric, uint32_t *out_ids, float *out_dists, int threads) {
    if (k == 0 || k > n) return -1;
    bool avx2 = false;
#if defined(__x86_64__)
    avx2 = __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
#endif
    const uint32_t kBlock = 1024;
    parallel_for(Q, threads, [&](int64_t q) {
        const float *qv = queries + (uint64_t) q * dim;
        std::vector<std::pair<float, uint32_t>> heap;  // max-heap on (dist,id)
        heap.reserve(k + 1);
        std::vector<float> d(kBlock);
        for (uint32_t r0 = 0; r0 < n; r0 += kBlock) {
            const uint32_t rows = std::min(kBlock, n - r0);
#if defined(__x86_64__)
            if (avx2) l2_block_avx2(qv, base + (uint64_t) r0 * dim, rows, dim, d.data());
            else
#endif
                l2_block_generic(qv, base + (uint64_t) r0 * dim, rows, dim, d.data());
            for (uint32_t r = 0; r < rows; r++) {
                const std::pair<float, uint32_t> e(d[r], r0 + r);
                if (heap.size() < k) {
                    heap.push_back(e);
                    std::push_heap(heap.begin(), heap.end());
                } else if (e < heap.front()) {
                    std::pop_heap(heap.begin(), heap.end());
                    heap.back() = e;
                    std::push_heap(heap.begin(), heap.end());
                }
            }
        }
        std::sort_heap(heap.begin(), heap.end());
        for (uint32_t i = 0; i < k; i++) {
            out_ids[(uint64_t) q * k + i] = heap[i].second;
            if (out_dists) out_dists[(uint64_t) q * k + i] = metric == kEuclidean ? sqrtf(heap[i].first) : heap[i].first;
        }
    });
    return 0;
}

// ---------------------------------------------------------------------------
// Lloyd k-means. The reference calls cuvs::cluster::kmeans::fit (cuVS branch-24.08,
// partition.cpp call site partition.cuh:48-54) whose arithmetic is not in the
// reference tree: PARITY UNPINNED. This restates this repository's own
// deterministic variant: centroids start as the first C sample rows (init 0) or as a
// farthest-first traversal of the sample (init 1); each round
// assigns every row to its nearest centroid (the partition stage's rule: distances
// in `metric`/`order`, sorted with the warp network), then recomputes each centroid as the fp32 sum of its members in
// ascending row order divided by the count (an empty cluster keeps its centroid);
// stops after max_iter rounds or when no assignment changes. Returns rounds run.
// ---------------------------------------------------------------------------
int orc_kmeans(const float *sample, uint32_t n, uint32_t dim, uint32_t C, uint32_t max_iter, int metric,
               int order, int init, float *centroids, uint32_t *labels_out) {
    if (n < C) return -1;
    if (init == 0) {
        std::memcpy(centroids, sample, (uint64_t) C * dim * sizeof(float));
    } else {
        // farthest-first traversal: start from row 0, then repeatedly take the row whose
        // squared distance to its nearest chosen centroid is largest (lowest row on ties)
        std::vector<float> mind2(n, kMaxF);
        uint32_t next = 0;
        for (uint32_t t = 0; t < C; t++) {
            std::memcpy(centroids + (uint64_t) t * dim, sample + (uint64_t) next * dim, dim * sizeof(float));
            const float *c = centroids + (uint64_t) t * dim;
            parallel_for(n, 0, [&](int64_t p) {
                const float d = sq_sum(sample + (uint64_t) p * dim, c, dim, order);
                if (d < mind2[p]) mind2[p] = d;
            });
            float best = -1.0f;
            for (uint32_t p = 0; p < n; p++)
                if (mind2[p] > best) {
                    best = mind2[p];
                    next = p;
                }
        }
    }
    std::vector<uint32_t> labels(n, kInvalid);
    int rounds = 0;
    for (uint32_t it = 0; it < max_iter; it++) {
        std::vector<uint32_t> nl(n);
        parallel_for(n, 0, [&](int64_t p) {
            std::vector<uint32_t> cid(C);
            std::vector<float> cd(C);
            for (uint32_t c = 0; c < C; c++) {
                cid[c] = c;
                cd[c] = distance(sample + (uint64_t) p * dim, centroids + (uint64_t) c * dim, dim, metric, order);
            }
            sort_with_key_value(ladder_centroid(C), C, cid.data(), cd.data());
            nl[p] = cid[0];
        });
        rounds++;
        const bool changed = (nl != labels);
        labels = nl;
        if (!changed) break;
        std::vector<float> sum((uint64_t) C * dim, 0.0f);
        std::vector<uint32_t> cnt(C, 0);
        for (uint32_t p = 0; p < n; p++) {
            const uint32_t c = labels[p];
            cnt[c]++;
            float *s = sum.data() + (uint64_t) c * dim;
            const float *x = sample + (uint64_t) p * dim;
            for (uint32_t i = 0; i < dim; i++) s[i] = s[i] + x[i];
        }
        for (uint32_t c = 0; c < C; c++) {
            if (cnt[c] == 0) continue;
            for (uint32_t i = 0; i < dim; i++)
                centroids[(uint64_t) c * dim + i] = sum[(uint64_t) c * dim + i] / (float) cnt[c];
        }
    }
    if (labels_out) std::memcpy(labels_out, labels.data(), n * sizeof(uint32_t));
    return rounds;
}

}  // extern "C"
