// Exact per-partition kNN graph on the tensor cores: the kNN stage's brute-force seeding.
//
// The product is the one of the reference's kNN stage (build_nnd, nn_descent.cuh:1405-1467): for
// every row of the reordered set its nearest rows inside its own partition, partition-local ids,
// nearest first. The reference gets there by NN-descent whose distance tiles are fp16 wmma Gram
// tiles (nn_descent.cuh:783-811); here every row meets every row of its partition:
//
//   norms    |x|^2 of every row, exact fp32.
//   contract a CTA owns 128 rows of one partition (the M of a 128 x 128 x 8 TF32 MMA) and walks the
//            partition in tiles of 128 rows. The CTA's own rows are written into tensor memory once
//            (tcgen05.st) and are the MMA's A operand from there; the partition's tiles arrive by TMA
//            (one 2-D tensor map over the whole reordered matrix, boxes of 32 floats x 128 rows,
//            128-byte swizzle, no multicast) into three stages of shared memory; tcgen05.mma
//            kind::tf32 accumulates the 128 x 128 dot products in tensor memory (two buffers), and
//            sixteen epilogue warps read them back (tcgen05.ld): thread (row, part)
//            turns 32 dot products of a tile into |a|^2 + |b|^2 - 2 a.b (four threads per row; with
//            two, the tile loop was bound by the latency of eight warps' dependent instruction chains:
//            31 % of the issue slots and 26 % of the tensor pipe busy).
//   select   two passes over the partition: the first finds per row a threshold that at least L
//            columns meet (from minima over groups of columns), the second stores every column at or
//            below it in a buffer private to the storing thread: no sorting, no atomics and no
//            barrier between warps inside the tile loop.
//   re-rank  the exact fp32 distance of the L approximately nearest candidates, sorted by
//            (distance, id): the first out_degree are the row.
//
// kind::tf32 keeps 10 mantissa bits per operand, so integer-valued rows below 1024 give exact dot
// products and the result is the exact kNN graph with ties by ascending id; elsewhere the approximate
// order only has to bring the true neighbours into the L = 2 x list-width candidates, and the
// re-rank orders them exactly. One thread issues the copies and another the MMAs; every mbarrier wait is
// bounded, and a CTA whose wait runs out raises a flag that makes the host redo the rows with the
// SIMT kernels.
#include <cstdlib>
#include <vector>

#include "beam_core.cuh"
#include "kernels.h"
#include "umma.cuh"

namespace glide {

namespace {

using namespace umma;

constexpr uint32_t kRows = 128;            // rows per CTA = columns per tile
constexpr uint32_t kTmemCols = 512;        // two accumulator buffers of 128 columns, then the CTA's own rows (up to 128 columns)
constexpr uint32_t kTmemA = 2 * kRows;     // first column of the CTA's own rows
constexpr uint32_t kStages = 3;            // tiles of the partition in flight in shared memory
constexpr uint32_t kSplit = 4;             // epilogue threads per row: each owns kCols columns of every tile
constexpr uint32_t kCols = kRows / kSplit;
constexpr uint32_t kEpiWarps = 4 * kSplit; // a warp reads the 32 tensor-memory lanes of its quadrant (warp % 4)
constexpr uint32_t kThreads = (kEpiWarps + 2) * 32;   // + the MMA warp and the copy warp (one thread of each works)
static_assert(kCols == 32 || kCols == 64, "the epilogue reads 32 columns per tcgen05.ld");
constexpr u64 kNoKey = ~0ull;

struct KnnTile {
    uint32_t seg_start, seg_len, first;    // rows [first, first + 128) of the segment
};

struct KnnTcArgs {
    const float *data;
    uint32_t dim;
    uint64_t rows_total;       // rows of data
    const float *norms;        // per row of data
    const KnnTile *tiles;      // one per CTA
    u64 *cand;                 // launch rows x cap
    uint32_t *cand_count;      // launch rows x kSplit (written when a CTA is done)
    float *gmin;               // launch rows x 2 x groups (kSplit threads x part_groups each): group minima of pass 1
    uint32_t *fail_flag;
};

__global__ void row_norms_kernel(const float *__restrict__ data, uint64_t rows, uint32_t dim, float *norms) {
    const uint64_t r = ((uint64_t) blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = lane_id();
    if (r >= rows) return;
    const float4 *row = reinterpret_cast<const float4 *>(data + r * dim);
    float s = 0.0f;
    for (uint32_t k = lane; k < (dim >> 2); k += 32) {
        const float4 v = __ldg(row + k);
        s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) s += __shfl_xor_sync(kFullMask, s, off);
    if (lane == 0) norms[r] = s;
}

// Selection without sorting inside the tile loop. The partition is walked TWICE:
//
//   pass 1  every thread (row, part: kCols of the 128 columns of each tile) splits the columns it
//           sees into `part_groups` consecutive groups and keeps the minimum distance of each. The row's
//           threshold is the `keep`-th smallest of its group minima: at least `keep` columns lie at
//           or below it (the minima themselves), and for rows in no particular order 1.15 to 1.4 x
//           keep do, whatever the partition's size.
//   pass 2  the same tiles again; every column at or below the threshold is stored in the thread's
//           private candidate buffer (a plain store at the thread's own counter: no atomics, no
//           compaction, no barrier between warps).
//
// The second pass costs a second round of MMAs, which are a small part of a tile's time; in exchange
// the epilogue is a few instructions per column in both passes. NL = 1: lists of 32 (out_degree <=
// 32), keep = 64 candidates re-ranked exactly; NL = 2: lists of 64, keep = 128. A thread's buffer
// holds part_cap keys; a row that would need more (hundreds of rows at exactly the threshold
// distance, or near neighbours stored next to one another so that few groups hold them all) raises
// the overflow flag and the host recomputes with the fp32 kernels.
template<int NL> struct Sizes {
    // 2 x groups = 4 x keep group slots per row: the group size is rounded up to a power of two, so
    // a row ends up with between 2 x keep and 4 x keep groups, and the keep-th smallest minimum then
    // lets 1.15 to 1.4 x keep columns through. (With only 2 x keep slots a partition of nine tiles
    // had 72 groups for keep = 64; its threshold sat near the largest minimum and let 150 to 200
    // columns through, more than the buffers hold.)
    static constexpr uint32_t keep = 64u * NL, groups = 128u * NL, cap = 256u * NL;
    static constexpr uint32_t part_cap = cap / kSplit, part_groups = 2u * groups / kSplit;
    static constexpr int sort_n = 8 * NL;    // keys per lane when a warp sorts a row's candidates (32 * sort_n = cap)
    static constexpr int thr_n = 8 * NL;     // values per lane when a warp sorts a row's 2 x groups minima
};

__host__ __device__ inline uint32_t pow2_ceil(uint32_t x) {
    uint32_t p = 1;
    while (p < x) p <<= 1;
    return p;
}

// Pass 1 over 32 columns: minima of consecutive runs of GS columns go to out[0], out[1], ...; the
// running minimum of an unfinished run is carried in m (GS <= 32 here, so every run ends inside).
template<int GS>
__device__ __forceinline__ float group_minima(const float (&e)[32], float m, float *out, bool active) {
#pragma unroll
    for (int j = 0; j < 32; j++) {
        m = fminf(m, e[j]);
        if ((j + 1) % GS == 0) {
            if (active) out[j / GS] = m;
            m = FLT_MAX;
        }
    }
    return m;
}

template<int NL>
__global__ void __launch_bounds__(kThreads) knn_umma_kernel(const KnnTcArgs a, const __grid_constant__ CUtensorMap tm_rows) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);
    const uint32_t dim = a.dim, kblocks = dim >> 5, ksteps = dim >> 3;
    const uint32_t sub_bytes = kRows * 128u;                  // one 32-float column block of a tile
    const uint32_t tile_bytes = kblocks * sub_bytes;
    uint8_t *Bs = base;                                       // kStages tiles of the partition; the CTA's own rows live in tensor memory
    float *cn_w = reinterpret_cast<float *>(Bs + kStages * tile_bytes); // a warp's column norms of the current tile
    float *thr_s = cn_w + kEpiWarps * kCols;                            // 128 row thresholds
    uint64_t *bars = reinterpret_cast<uint64_t *>(thr_s + kRows);       // a_full, b_full[3], stage_free[3], mma_done[2], tmem_free[2]
    uint64_t *a_full = bars, *b_full = bars + 1, *stage_free = b_full + kStages, *mma_done = stage_free + kStages, *tmem_free = mma_done + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(tmem_free + 2);
    volatile uint32_t *failed = tmem_slot + 1;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const KnnTile tile = a.tiles[blockIdx.x];
    const uint32_t tiles = (tile.seg_len + kRows - 1) / kRows, total = 2 * tiles;
    const uint64_t launch_row0 = (uint64_t) blockIdx.x * kRows;

    if (tid == 0) {
        mbar_init(a_full, 4 * kblocks);   // the warps that write the CTA's rows into tensor memory
        for (uint32_t s = 0; s < kStages; s++) { mbar_init(b_full + s, 1); mbar_init(stage_free + s, 1); }
        for (int c = 0; c < 2; c++) { mbar_init(mma_done + c, 1); mbar_init(tmem_free + c, kEpiWarps); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        *failed = 0;
    }
    if (warp == kEpiWarps) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == kEpiWarps + 1) {
        // ================= copy warp: operand tiles by TMA, one thread =================
        // Stage s takes tile t + 2 as soon as the MMAs of tile t have read it; the MMA thread does not
        // wait for that, so the MMAs of tile t + 1 are already queued behind those of tile t.
        if (lane == 0) {
            auto load_tile = [&](uint8_t *dst, uint32_t row0, uint64_t *bar) {
                mbar_expect_tx(bar, tile_bytes);
                for (uint32_t kb = 0; kb < kblocks; kb++) tma_load_2d(dst + kb * sub_bytes, &tm_rows, kb * 32u, row0, bar);
            };
            for (uint32_t i = 0; i < kStages && i < total; i++) load_tile(Bs + i * tile_bytes, tile.seg_start + (i % tiles) * kRows, b_full + i);
            for (uint32_t t = 0; t + kStages < total; t++) {
                const uint32_t s = t % kStages, use = t / kStages;
                if (!mbar_wait(stage_free + s, use & 1u, failed)) break;
                load_tile(Bs + s * tile_bytes, tile.seg_start + ((t + kStages) % tiles) * kRows, b_full + s);
            }
        }
    } else if (warp == kEpiWarps) {
        // ================= MMA warp: one thread issues =================
        if (lane == 0) {
            // instruction descriptor: D fp32, A and B TF32, both K-major, N = 128, M = 128
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((kRows >> 3) << 17) | ((kRows >> 4) << 24);
            const uint32_t b_addr = smem_u32(Bs);
            bool ok = mbar_wait(a_full, 0, failed);
            for (uint32_t t = 0; t < total && ok; t++) {   // t counts tiles over both passes
                const uint32_t s = t % kStages, use = t / kStages, acc = t & 1u, acc_use = t >> 1;
                ok = mbar_wait(b_full + s, use & 1u, failed);
                if (ok && t >= 2) ok = mbar_wait(tmem_free + acc, (acc_use - 1) & 1u, failed);
                if (!ok) break;
                fence_after();
                for (uint32_t ks = 0; ks < ksteps; ks++) {   // eight TF32 values of every row per step: eight columns of A
                    const uint32_t off = (ks >> 2) * sub_bytes + (ks & 3u) * 32u;
                    mma_tf32_ts(tmem_base + acc * kRows, tmem_base + kTmemA + ks * 8u, desc_sw128(b_addr + s * tile_bytes + off), idesc,
                                ks > 0 ? 1u : 0u);
                }
                commit_to(stage_free + s);   // the stage may be refilled
                commit_to(mma_done + acc);   // the accumulator may be read
            }
        }
    } else {
        // ================= epilogue warps: thread (row, part) owns kCols columns of every tile =================
        const uint32_t quad = warp & 3u, part = warp >> 2;
        const uint32_t row = quad * 32u + lane;
        const uint32_t rl = tile.first + row;                      // the row's partition-local id
        const bool active = rl < tile.seg_len;
        const float pnr = active ? __ldg(a.norms + tile.seg_start + rl) : 0.0f;
        // The CTA's own rows go into tensor memory once: warp (quad, part) writes columns part * 32 ... of the 32
        // rows of its quadrant (lane = row), read straight from global memory; rows beyond the matrix are zeros.
        if (part < kblocks) {
            uint32_t v[32];
            const uint64_t grow = (uint64_t) tile.seg_start + rl;
            const float4 *src = reinterpret_cast<const float4 *>(a.data + grow * dim + part * 32u);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float4 x = grow < a.rows_total ? __ldg(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                v[4 * i] = __float_as_uint(x.x); v[4 * i + 1] = __float_as_uint(x.y);
                v[4 * i + 2] = __float_as_uint(x.z); v[4 * i + 3] = __float_as_uint(x.w);
            }
            tmem_store32(tmem_base + ((quad * 32u) << 16) + kTmemA + part * 32u, v);
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(a_full);
        }
        float *cn = cn_w + warp * kCols;                           // this warp's column norms of the current tile
        constexpr uint32_t G = Sizes<NL>::part_groups;
        float *my_gmin = a.gmin + ((launch_row0 + row) * kSplit + part) * G;
        u64 *my_cand = a.cand + (launch_row0 + row) * Sizes<NL>::cap + part * Sizes<NL>::part_cap;
        // groups: whole tiles when the partition has more tiles than groups, else runs of gs columns
        // inside a tile (gs a power of two, at least tiles * kCols / G, so that at most G groups arise)
        const bool by_tile = tiles > G;
        const uint32_t gs = by_tile ? 2u * kCols : min(kCols, pow2_ceil((tiles * kCols + G - 1) / G));
        const uint32_t gs_shift = 31u - (uint32_t) __clz(gs), per_tile = by_tile ? 0u : kCols / gs;
        if (active)
            for (uint32_t g = 0; g < G; g++) my_gmin[g] = FLT_MAX;
        float m = FLT_MAX, thr = 0.0f;
        uint32_t mine = 0, grp = 0, grp_rem = 0;
        float cn_ahead[kCols / 32u];
#pragma unroll
        for (uint32_t h = 0; h < kCols / 32u; h++) {
            const uint32_t c = part * kCols + lane + 32u * h;
            cn_ahead[h] = c < tile.seg_len ? __ldg(a.norms + tile.seg_start + c) : 0.0f;
        }
        for (uint32_t t = 0; t < total; t++) {
            const uint32_t s = t & 1u, use = t >> 1;   // the accumulator buffer and its turn
            const bool second = t >= tiles;
            const uint32_t tt = second ? t - tiles : t;
            if (t == tiles) {
                // ---- between the passes: every row's threshold from its group minima ----
                named_barrier_sync(1, kEpiWarps * 32);
                constexpr uint32_t kRowsPerWarp = kRows / kEpiWarps;
                for (uint32_t r = warp * kRowsPerWarp; r < (warp + 1) * kRowsPerWarp; r++) {
                    constexpr int N = Sizes<NL>::thr_n;
                    const float *g = a.gmin + (launch_row0 + r) * 2 * Sizes<NL>::groups;
                    float k[N];
                    uint32_t v[N];
#pragma unroll
                    for (int i = 0; i < N; i++) { k[i] = g[lane + 32u * i]; v[i] = 0u; }
                    warp_sort<N>(k, v);                              // ascending over e = N * lane + i
                    const float kth = __shfl_sync(kFullMask, k[N - 1], 7);    // e = 8 N - 1 = keep - 1
                    if (lane == 0) thr_s[r] = kth;
                }
                named_barrier_sync(1, kEpiWarps * 32);
                thr = thr_s[row];
            }
            __syncwarp();
            // the column norms of this tile were requested a tile ago; those of the next are requested now,
            // so their trip to L2 runs under this tile's work instead of in front of the next one's
#pragma unroll
            for (uint32_t h = 0; h < kCols / 32u; h++) cn[lane + 32u * h] = cn_ahead[h];
            if (t + 1 < total) {
                const uint32_t tn = (t + 1 == tiles) ? 0u : tt + 1;
#pragma unroll
                for (uint32_t h = 0; h < kCols / 32u; h++) {
                    const uint32_t c = tn * kRows + part * kCols + lane + 32u * h;
                    cn_ahead[h] = c < tile.seg_len ? __ldg(a.norms + tile.seg_start + c) : 0.0f;
                }
            }
            __syncwarp();
            bool ok = !*failed && mbar_wait(mma_done + s, use & 1u, failed);
            ok = __all_sync(kFullMask, ok);   // tcgen05.ld is a warp-wide instruction
            if (!ok) continue;
            fence_after();
            const uint32_t c0 = tt * kRows + part * kCols;
            // A tile needs the per-column checks only when it holds a column beyond the partition's end
            // or the row itself; the 32 rows of a warp are consecutive, so that is the same for all lanes
            // up to a tile or two.
            const bool checks = __any_sync(kFullMask, c0 + kCols > tile.seg_len || (rl >= c0 && rl < c0 + kCols));
            for (uint32_t cb = 0; cb < kCols; cb += 32) {
                uint32_t r[32];
                tmem_load32(tmem_base + ((quad * 32u) << 16) + s * kRows + part * kCols + cb, r);
                float e[32];   // |b|^2 - 2 a.b: the distance without the row's own |a|^2, which shifts a row's values alike
#pragma unroll
                for (int j4 = 0; j4 < 32; j4 += 4) {
                    const float4 cn4 = *reinterpret_cast<const float4 *>(cn + cb + j4);  // broadcast
                    e[j4] = __fmaf_rn(-2.0f, __uint_as_float(r[j4]), cn4.x);
                    e[j4 + 1] = __fmaf_rn(-2.0f, __uint_as_float(r[j4 + 1]), cn4.y);
                    e[j4 + 2] = __fmaf_rn(-2.0f, __uint_as_float(r[j4 + 2]), cn4.z);
                    e[j4 + 3] = __fmaf_rn(-2.0f, __uint_as_float(r[j4 + 3]), cn4.w);
                }
                if (checks) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const uint32_t cid = c0 + cb + j;
                        if (cid >= tile.seg_len || cid == rl) e[j] = __int_as_float(0x7f800000);   // +inf: above every threshold
                    }
                }
                if (!second) {
                    switch (gs_shift) {   // the group size is a power of two: resolved at compile time inside each case
                        case 0: m = group_minima<1>(e, m, my_gmin + tt * per_tile + (cb >> 0), active); break;
                        case 1: m = group_minima<2>(e, m, my_gmin + tt * per_tile + (cb >> 1), active); break;
                        case 2: m = group_minima<4>(e, m, my_gmin + tt * per_tile + (cb >> 2), active); break;
                        case 3: m = group_minima<8>(e, m, my_gmin + tt * per_tile + (cb >> 3), active); break;
                        case 4: m = group_minima<16>(e, m, my_gmin + tt * per_tile + (cb >> 4), active); break;
                        case 5: m = group_minima<32>(e, m, my_gmin + tt * per_tile + (cb >> 5), active); break;
                        default: {   // a thread's whole share of the tile (when that is 64 columns), or whole tiles: the run ends later
#pragma unroll
                            for (int j = 0; j < 32; j++) m = fminf(m, e[j]);
                            if (!by_tile && cb + 32u == kCols) {
                                if (active) my_gmin[tt] = m;
                                m = FLT_MAX;
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        if (e[j] <= thr && active) {
                            // the key carries the full distance, clamped at zero (rounding can leave it just below)
                            if (mine < Sizes<NL>::part_cap)
                                my_cand[mine] = ((u64) __float_as_uint(fmaxf(e[j] + pnr, 0.0f)) << 32) | (c0 + cb + j);
                            mine++;
                        }
                    }
                }
            }
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tmem_free + s);
            if (!second && by_tile) {   // a group of whole tiles ends with this tile
                // tile tt belongs to group floor(tt * G / tiles); stepped without dividing: tt * G = grp * tiles + grp_rem,
                // and G < tiles here, so the group number grows by at most one per tile
                grp_rem += G;
                const bool last_of_group = grp_rem >= tiles;
                if (tt + 1 == tiles || last_of_group) {
                    if (active) my_gmin[grp] = m;
                    m = FLT_MAX;
                }
                if (last_of_group) { grp_rem -= tiles; grp++; }
            }
        }
        if (active) a.cand_count[kSplit * (launch_row0 + row) + part] = min(mine, Sizes<NL>::part_cap);
        if (mine > Sizes<NL>::part_cap) atomicExch(a.fail_flag, 2u);    // more candidates than a buffer holds
        if (*failed && lane == 0) atomicExch(a.fail_flag, 1u);          // a bounded wait ran out
    }
    fence_before();
    __syncthreads();
    if (warp == kEpiWarps) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
}

// Exact re-rank: a warp per row. The `keep` approximately nearest candidates get their exact fp32
// distance (whole-warp row loads, the summation order of the search kernels), are sorted by
// (distance, id), and the first out_degree ids are written; a row with fewer candidates than
// out_degree (a partition of fewer rows) is padded with xorshift32(flat index) % partition size, as
// nn_descent.cuh:1384-1391 pads.
template<int NL>
__global__ void __launch_bounds__(256) knn_rerank_kernel(const KnnTcArgs a, uint32_t launch_rows, uint32_t out_degree,
                                                         uint32_t row_base, int32_t *out) {
    extern __shared__ __align__(16) uint32_t smem[];
    constexpr int N = Sizes<NL>::sort_n;
    constexpr uint32_t keep = Sizes<NL>::keep;
    const uint32_t warp = threadIdx.x >> 5, lane = lane_id();
    const uint32_t lr = blockIdx.x * (blockDim.x >> 5) + warp;
    if (lr >= launch_rows) return;
    const KnnTile tile = a.tiles[lr / kRows];
    const uint32_t rl = tile.first + lr % kRows;
    if (rl >= tile.seg_len) return;
    uint32_t *strip = smem + (size_t) warp * (dim_pad4(a.dim) + 2 * keep);
    float *query = reinterpret_cast<float *>(strip);
    uint32_t *ids = strip + dim_pad4(a.dim);
    float *dist = reinterpret_cast<float *>(ids + keep);
    const float *seg = a.data + (uint64_t) tile.seg_start * a.dim;
    // the row's candidates: kSplit buffers of part_cap keys, the first count[p] of each valid
    const u64 *buf = a.cand + (uint64_t) lr * Sizes<NL>::cap;
    uint32_t count[kSplit], cnt = 0;
#pragma unroll
    for (uint32_t p = 0; p < kSplit; p++) {
        count[p] = min(a.cand_count[kSplit * (uint64_t) lr + p], Sizes<NL>::part_cap);
        cnt += count[p];
    }
    u64 k[N];
#pragma unroll
    for (int i = 0; i < N; i++) {
        const uint32_t e = lane + 32u * i;            // slot e of the row's cap = 32 N slots
        const uint32_t p = e / Sizes<NL>::part_cap, off = e % Sizes<NL>::part_cap;
        k[i] = off < count[p] ? buf[e] : kNoKey;
    }
    sort_u64<N>(k);
    const uint32_t n = min(cnt, keep);
#pragma unroll
    for (int i = 0; i < N; i++) {
        const uint32_t e = (uint32_t) N * lane + i;
        if (e < keep) ids[e] = e < n ? (uint32_t) k[i] : 0u;
    }
    load_query(query, seg + (uint64_t) rl * a.dim, a.dim);
    __syncwarp();
    warp_rows(query, seg, a.dim, kCosine /* squared sums: order only */, n,
              [&](uint32_t i) { return ids[i]; }, [&](uint32_t i, float d) { dist[i] = d; });
    __syncwarp();
    u64 ek[2 * NL];
#pragma unroll
    for (int i = 0; i < 2 * NL; i++) {
        const uint32_t e = lane + 32u * i;
        ek[i] = e < n ? (((u64) __float_as_uint(dist[e]) << 32) | ids[e]) : kNoKey;
    }
    sort_u64<2 * NL>(ek);
#pragma unroll
    for (int i = 0; i < 2 * NL; i++) {
        const uint32_t e = (uint32_t) (2 * NL) * lane + i;
        if (e < out_degree) {
            const uint64_t flat = (uint64_t) (tile.seg_start + rl) * out_degree + e;
            uint32_t u = (uint32_t) (flat + (uint64_t) row_base * out_degree);  // xorshift32, utils.cuh:14-19
            u ^= u >> 13; u ^= u << 27; u ^= u >> 5; u *= 0x9E3779B9u;
            const uint32_t id = (uint32_t) ek[i];
            out[flat] = (int32_t) (e < n ? id : u % tile.seg_len);
        }
    }
}

size_t align256(size_t x) { return (x + 255) & ~(size_t) 255; }

constexpr uint32_t kMaxCtasPerLaunch = 2368;   // sixteen waves of 148 CTAs; 303,104 rows at 2.5 KB (5 KB for lists of 64) of scratch a row

template<int NL>
cudaError_t run(const float *data, uint64_t rows_total, uint32_t dim, const std::vector<KnnTile> &tiles, uint32_t out_degree,
                uint32_t row_base, char *scratch, int32_t *out, uint32_t *h_failed, cudaStream_t stream) {
    float *norms = reinterpret_cast<float *>(scratch); scratch += align256(rows_total * 4);
    uint32_t *fail_flag = reinterpret_cast<uint32_t *>(scratch); scratch += 256;
    KnnTile *d_tiles = reinterpret_cast<KnnTile *>(scratch); scratch += align256((size_t) kMaxCtasPerLaunch * sizeof(KnnTile));
    uint32_t *cand_count = reinterpret_cast<uint32_t *>(scratch); scratch += align256((size_t) kMaxCtasPerLaunch * kRows * kSplit * 4);
    float *gmin = reinterpret_cast<float *>(scratch); scratch += align256((size_t) kMaxCtasPerLaunch * kRows * 2 * Sizes<NL>::groups * 4);
    u64 *cand = reinterpret_cast<u64 *>(scratch);
    CUtensorMap tm;
    if (!make_row_map(&tm, data, rows_total, dim, kRows)) return cudaErrorNotSupported;
    cudaError_t e = cudaMemsetAsync(fail_flag, 0, 4, stream);
    if (e != cudaSuccess) return e;
    row_norms_kernel<<<(unsigned) ((rows_total * 32 + 255) / 256), 256, 0, stream>>>(data, rows_total, dim, norms);
    const size_t smem_main = 1024 + (size_t) 3 * kRows * dim * 4 + (kEpiWarps * kCols + kRows) * 4 + (1 + 2 * kStages + 4) * 8 + 16;
    if ((e = cudaFuncSetAttribute(knn_umma_kernel<NL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_main)) != cudaSuccess) return e;
    const uint32_t rr_warps = 8;
    const size_t smem_rr = (size_t) rr_warps * (dim_pad4(dim) + 2 * Sizes<NL>::keep) * 4;
    if (smem_rr > 48 * 1024 &&
        (e = cudaFuncSetAttribute(knn_rerank_kernel<NL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_rr)) != cudaSuccess) return e;
    KnnTcArgs a{data, dim, rows_total, norms, d_tiles, cand, cand_count, gmin, fail_flag};
    for (size_t first = 0; first < tiles.size(); first += kMaxCtasPerLaunch) {
        const uint32_t n = (uint32_t) std::min<size_t>(kMaxCtasPerLaunch, tiles.size() - first);
        // the table is pageable host memory: the copy has read it when the call returns
        if ((e = cudaMemcpyAsync(d_tiles, tiles.data() + first, (size_t) n * sizeof(KnnTile), cudaMemcpyHostToDevice, stream)) != cudaSuccess) return e;
        knn_umma_kernel<NL><<<n, kThreads, smem_main, stream>>>(a, tm);
        knn_rerank_kernel<NL><<<(n * kRows + rr_warps - 1) / rr_warps, rr_warps * 32, smem_rr, stream>>>(a, n * kRows, out_degree, row_base, out);
        if ((e = cudaGetLastError()) != cudaSuccess) return e;
    }
    if ((e = cudaMemcpyAsync(h_failed, fail_flag, 4, cudaMemcpyDeviceToHost, stream)) != cudaSuccess) return e;
    return cudaStreamSynchronize(stream);
}

}  // namespace

bool knn_tc_eligible(const float *data, uint32_t dim, uint32_t out_degree) {
    static const bool off = [] { const char *v = std::getenv("GLIDE_B200_NO_TC_KNN"); return v && v[0] == '1'; }();
    return !off && dim >= 32 && (dim & 31u) == 0 && dim <= 128 && out_degree >= 1 && out_degree <= 64 &&
           (reinterpret_cast<uintptr_t>(data) & 15u) == 0 && encode_tiled_fn() != nullptr;
}

size_t knn_tc_scratch_bytes(uint64_t rows_total, uint32_t out_degree) {
    const size_t nl = out_degree <= 32 ? 1 : 2;
    const size_t per_row = 4 * kSplit /* counts */ + 2 * 128 * nl * 4 /* group minima */ + 256 * nl * 8 /* candidates */;
    return align256(rows_total * 4) + 256 + align256((size_t) kMaxCtasPerLaunch * sizeof(KnnTile)) +
           (size_t) kMaxCtasPerLaunch * kRows * per_row + 4 * 256;
}

// Exact kNN rows of every listed partition with 2 <= length <= max_len (rows of `data`, partition s =
// rows [h_seg_start[s], +h_seg_len[s])). *h_failed != 0 afterwards: a bounded wait ran out somewhere and
// the rows must be recomputed by another kernel. Synchronises the stream.
cudaError_t launch_knn_tc(const float *data, uint64_t rows_total, uint32_t dim, const uint32_t *h_seg_start,
                          const uint32_t *h_seg_len, uint32_t S, uint32_t max_len, uint32_t out_degree, uint32_t row_base,
                          void *scratch, int32_t *out, uint32_t *h_failed, cudaStream_t stream) {
    std::vector<KnnTile> tiles;
    for (uint32_t s = 0; s < S; s++) {
        if (h_seg_len[s] < 1 || h_seg_len[s] > max_len) continue;
        for (uint32_t first = 0; first < h_seg_len[s]; first += kRows) tiles.push_back(KnnTile{h_seg_start[s], h_seg_len[s], first});
    }
    *h_failed = 0;
    if (tiles.empty()) return cudaSuccess;
    if (out_degree <= 32) return run<1>(data, rows_total, dim, tiles, out_degree, row_base, static_cast<char *>(scratch), out, h_failed, stream);
    return run<2>(data, rows_total, dim, tiles, out_degree, row_base, static_cast<char *>(scratch), out, h_failed, stream);
}

}  // namespace glide
