// Nearest-centroid assignment with a tensor-core prefilter and an exact re-rank.
//
// The reference computes, for every point (or query), the fp32 distance to every centroid and
// sorts them (partition_kernel.cuh:21-61, search_kernel.cuh:258-269); only the nearest and, for
// the boundary test, the second nearest matter. That is a points x centroids contraction, so the
// bulk of it runs on the tensor cores:
//
//   pass 1  approximate squared distances |p|^2 + |c|^2 - 2 p.c with the dot products from TF32
//           MMAs (fp32 accumulate, exact fp32 norms); per point the smallest and second smallest.
//   pass 2  the same tiles again; every centroid whose approximate distance is within a rigorous
//           error margin of that minimum becomes a candidate (at most kCand per point).
//   re-rank the exact fp32 distance of every candidate in the reference's summation order (the
//           8-lane team order of common.cuh), then nearest / second nearest / boundary flag.
//
// The margin bounds |approx - exact|: kind::tf32 keeps 10 explicit mantissa bits of each fp32
// operand (relative error below 2^-10), so the dot product is off by at most ~2^-9 |p||c|
// (Cauchy-Schwarz) and the distance by twice that, 2^-8 |p||c|; the kernel allows 2^-7 |p||c| plus
// the rounding of the norms and of the reference's own sum, and compares against the minimum plus
// twice that. A point with more candidates than fit, or whose two best exact distances are equal,
// is left with the flag 0xffffffff for the warp-per-point kernel, whose full network sort
// reproduces the reference's tie order. The results are therefore those of the exact path, bit for
// bit.
//
// The contraction runs on the 5th-generation tensor cores: tcgen05.mma kind::tf32, 128 x 128 x 8
// per instruction, operands in shared memory, accumulator in tensor memory.
#include <cstdlib>
#include <cuda.h>
#include "beam_core.cuh"
#include "kernels.h"
#include "umma.cuh"

namespace glide {

namespace {

constexpr int kCand = 16;       // candidates kept per point
constexpr uint32_t kUmmaRows = 128;   // points per CTA = centroids per tile
constexpr uint32_t kMaxDim = 128;

__device__ __forceinline__ void min2_add(float &m1, float &m2, float d) {
    m2 = fminf(m2, fmaxf(m1, d));
    m1 = fminf(m1, d);
}

struct ExactNear {
    float d0, d1;
    uint32_t id, ties;
};

__device__ __forceinline__ void exact_add(ExactNear &s, float d, uint32_t id) {
    if (d < s.d0) { s.d1 = s.d0; s.d0 = d; s.id = id; s.ties = 1; }
    else if (d == s.d0) { s.d1 = d; s.ties++; }
    else if (d < s.d1) { s.d1 = d; }
}

// Exact re-rank of one CTA's 128 points in the reference's team order: an 8-lane team per point
// (four points per warp at a time), the team walks the point's candidates. count[row]: number of
// candidates (> kCand: overflow), bit 31: the second nearest is known to be too far for the
// boundary test. Point rows are re-read from global memory.
__device__ __forceinline__ void rerank_rows(const AssignArgs &a, uint32_t p0, const uint32_t *count, const uint32_t *cand,
                                            uint32_t warp, uint32_t warps) {
    const uint32_t lane = lane_id(), team = lane >> 3;
    for (uint32_t row0 = warp * 4; row0 < kUmmaRows; row0 += warps * 4) {
        const uint32_t row = row0 + team;
        const uint32_t p = p0 + row;
        const bool live = p < a.n;
        const uint32_t n_c = live ? (count[row] & 0x7fffffffu) : 0u;
        const bool far_second = (count[row] >> 31) != 0;
        const bool overflow = n_c > (uint32_t) kCand;
        const uint32_t mine = overflow ? 0u : n_c;
        uint32_t longest = mine;
#pragma unroll
        for (int off = 16; off >= 8; off >>= 1) longest = max(longest, __shfl_xor_sync(kFullMask, longest, off));
        ExactNear st{FLT_MAX, FLT_MAX, kInvalid, 0u};
        for (uint32_t j = 0; j < longest; j++) {
            const bool active = j < mine;
            const uint32_t cid = active ? cand[row * kCand + j] : 0u;
            const float part = team_partial(a.data + (uint64_t) (live ? p : 0) * a.dim, a.centroids + (uint64_t) cid * a.dim, a.dim, active);
            const float sum = team_fold(part);
            if (active) exact_add(st, finish_metric(sum, a.metric), cid);  // every lane of the team holds the same state
        }
        if (live && (lane & 7u) == 0) {
            const bool unique = !overflow && st.ties == 1;
            a.nearest[p] = unique ? st.id : kInvalid;
            if (a.is_boundary && unique)  // partition_kernel.cuh:58-60
                a.is_boundary[p] = (!far_second && a.boundary_factor >= 0.0f && a.C > 1 && st.d1 / st.d0 <= a.boundary_factor) ? 0u : kInvalid;
        }
    }
}

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gmem_src, bool valid) {
    const uint32_t dst = (uint32_t) __cvta_generic_to_shared(smem_dst);
    const uint32_t bytes = valid ? 16u : 0u;  // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template<int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Squared norms of the centroids (exact inputs, fp32 sum) and their maximum in norms[C].
__global__ void centroid_norms_kernel(const float *__restrict__ centroids, uint32_t C, uint32_t dim, float *norms) {
    const uint32_t c = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = lane_id();
    if (c >= C) return;
    const float4 *row = reinterpret_cast<const float4 *>(centroids + (uint64_t) c * dim);
    float s = 0.0f;
    for (uint32_t k = lane; k < (dim >> 2); k += 32) {
        const float4 v = __ldg(row + k);
        s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) s += __shfl_xor_sync(kFullMask, s, off);
    if (lane == 0) {
        norms[c] = s;
        atomicMax(reinterpret_cast<int *>(norms + C), __float_as_int(s));  // non-negative floats order as ints
    }
}

// ---------------------------------------------------------------------------
// One CTA owns 128 points
// (the M of a 128 x 128 x 8 TF32 MMA), walks the centroids in tiles of 128 and keeps the
// 128 x 128 fp32 accumulator of a tile in tensor memory, double buffered (256 columns), so the
// MMAs of tile t+1 run while the threads read tile t out with tcgen05.ld. Row i of the
// accumulator lives in tensor-memory lane i and is read by thread i alone: the running minimum,
// the threshold and the candidate list of a point never leave its thread.
//
// Operands are staged by cp.async straight into the K-major "no swizzle" canonical layout the
// MMA's shared-memory descriptor names: 8 rows x 16 bytes form a contiguous 128-byte core
// matrix; the next 16-byte K chunk follows at +128 bytes (leading byte offset), the next 8-row
// group at +chunks*128 bytes (stride byte offset). kind::tf32 reads fp32 words and drops the low
// 13 mantissa bits, a relative error of 2^-10 per operand; the margin below allows twice the
// resulting bound. Every wait on an mbarrier is bounded; a CTA whose wait runs out flags all of
// its points for the exact kernel instead of trusting the accumulator.
// ---------------------------------------------------------------------------
constexpr uint32_t kTmemCols = 256;   // two accumulator buffers of 128 columns
using namespace umma;   // smem_u32, mma_tf32, tmem_load32, mbarriers with bounded waits, TMA loads (umma.cuh)

__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    // start address, leading byte offset, stride byte offset (all without their 4 LSBs), descriptor
    // version 1, no swizzle
    return (uint64_t) ((smem_addr >> 4) & 0x3fffu) | ((uint64_t) ((lbo_bytes >> 4) & 0x3fffu) << 16) |
           ((uint64_t) ((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46);
}

__global__ void __launch_bounds__(128) assign_umma_kernel(const AssignArgs a) {
    extern __shared__ __align__(128) uint8_t smem_u[];
    const uint32_t dim = a.dim, chunks = dim >> 2, ksteps = dim >> 3;
    const uint32_t tile_bytes = kUmmaRows * dim * 4;
    const uint32_t sbo = chunks * 128u, lbo = 128u;
    uint8_t *As = smem_u;
    uint8_t *Bs = As + tile_bytes;                                          // two tiles
    float *cn_s = reinterpret_cast<float *>(Bs + 2 * tile_bytes);           // 2 x 128 centroid norms
    uint32_t *cand = reinterpret_cast<uint32_t *>(cn_s + 2 * kUmmaRows);    // 128 x kCand
    uint64_t *mbar = reinterpret_cast<uint64_t *>(cand + kUmmaRows * kCand);  // 2
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(mbar + 2);
    const float *norms = a.tc_norms;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t p0 = blockIdx.x * kUmmaRows;
    const uint32_t tiles = (a.C + kUmmaRows - 1) / kUmmaRows, total = 2 * tiles;

    // 128 rows x chunks 16-byte pieces; a warp instruction moves 8 rows x 4 chunks: 64 contiguous
    // bytes per row on the global side, 512 contiguous bytes on the shared side
    auto stage_rows = [&](uint8_t *dst, const float *src, uint32_t first_row, uint32_t row_limit) {
        const uint32_t cgroups = chunks >> 2;
        for (uint32_t g = warp; g < 16 * cgroups; g += 4) {
            const uint32_t r = (g / cgroups) * 8 + (lane & 7), c = (g % cgroups) * 4 + (lane >> 3);
            const bool valid = first_row + r < row_limit;
            cp_async16(dst + (r >> 3) * sbo + c * lbo + (r & 7) * 16,
                       src + (uint64_t) (valid ? first_row + r : 0) * dim + 4 * c, valid);
        }
    };
    auto stage_tile = [&](uint32_t t) {  // t counts tiles over both passes
        const uint32_t c0 = (t % tiles) * kUmmaRows;
        stage_rows(Bs + (t & 1u) * tile_bytes, a.centroids, c0, a.C);
        cn_s[(t & 1u) * kUmmaRows + tid] = c0 + tid < a.C ? __ldg(norms + c0 + tid) : 0.0f;
        cp_async_commit();
    };

    if (tid == 0) {
        const uint32_t b0 = smem_u32(mbar), b1 = smem_u32(mbar + 1);
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(b0) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(b1) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    stage_rows(As, a.data, p0, a.n);
    stage_tile(0);
    cp_async_wait<0>();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    // squared norm of this thread's point, from the staged copy
    float pnr = 0.0f;
    for (uint32_t c = 0; c < chunks; c++) {
        const float4 v = *reinterpret_cast<const float4 *>(As + (tid >> 3) * sbo + c * lbo + (tid & 7) * 16);
        pnr += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    const float cm = __ldg(norms + a.C);
    const float err = 0.0078125f * sqrtf(pnr) * sqrtf(cm) + 1.52587890625e-5f * (pnr + cm);

    // instruction descriptor: D fp32, A and B TF32, both K-major, N = 128, M = 128
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((kUmmaRows >> 3) << 17) | ((kUmmaRows >> 4) << 24);
    const uint32_t a_addr = smem_u32(As), b_addr = smem_u32(Bs);
    const uint32_t lane_base = (warp & 3u) * 32u;

    float m1 = FLT_MAX, m2 = FLT_MAX, thr = 0.0f;
    uint32_t n_c = 0;
    bool ok = true, need_second = false;
    for (uint32_t t = 0; t < total; t++) {
        const uint32_t buf = t & 1u;
        if (tid == 0) {
            for (uint32_t ks = 0; ks < ksteps; ks++)
                mma_tf32(tmem_base + buf * kUmmaRows, umma_desc(a_addr + ks * 2 * lbo, lbo, sbo),
                          umma_desc(b_addr + buf * tile_bytes + ks * 2 * lbo, lbo, sbo), idesc, ks > 0 ? 1u : 0u);
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(mbar + buf))
                         : "memory");
        }
        if (t + 1 < total) stage_tile(t + 1);   // overlaps the MMAs of tile t
        {   // wait for the MMAs of tile t: phase parity of this buffer's barrier
            const uint32_t bar = smem_u32(mbar + buf), parity = (t >> 1) & 1u;
            uint32_t done = 0;
            for (uint32_t spin = 0; spin < kSpinLimit && !done; spin++) {
                asm volatile(
                    "{\n\t"
                    ".reg .pred p;\n\t"
                    "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                    "selp.u32 %0, 1, 0, p;\n\t"
                    "}\n"
                    : "=r"(done)
                    : "r"(bar), "r"(parity)
                    : "memory");
            }
            // every thread takes the same branch below (tcgen05.ld is a warp-wide instruction)
            ok = __syncthreads_and(done != 0) != 0;
        }
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t c0 = (t % tiles) * kUmmaRows;
        const float *cn = cn_s + buf * kUmmaRows;
        const bool second = t >= tiles;
        for (uint32_t cb = 0; cb < kUmmaRows; cb += 32) {
            uint32_t r[32];
            tmem_load32(tmem_base + (lane_base << 16) + buf * kUmmaRows + cb, r);
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const uint32_t cid = c0 + cb + j;
                const float d = (cid < a.C) ? (pnr + cn[cb + j]) - 2.0f * __uint_as_float(r[j]) : FLT_MAX;
                if (!second) {
                    min2_add(m1, m2, d);
                } else if (d <= thr) {
                    if (n_c < (uint32_t) kCand) cand[tid * kCand + n_c] = cid;
                    n_c++;
                }
            }
        }
        if (t + 1 == tiles) {
            // Routing and k-means need the nearest centroid only. The boundary test d1 / d0 <= factor
            // (partition_kernel.cuh:58-60) needs the exact second nearest distance only when the ratio
            // can come near the factor at all: if even the most favourable reading of the two
            // approximate minima leaves it clearly above, the point is not a boundary point and the
            // dense crowd of centroids around the second minimum never has to be re-ranked.
            const bool boundary_test = a.is_boundary && a.boundary_factor >= 0.0f && a.C > 1;
            if (boundary_test) {
                const float lo2 = fmaxf(m2 - err, 0.0f), hi1 = m1 + err;
                const float f = a.metric == kEuclidean ? a.boundary_factor * a.boundary_factor : a.boundary_factor;
                need_second = !(lo2 > f * hi1 * 1.001f);
            }
            const float base = need_second ? m2 : m1;
            thr = base + 2.0f * err + 6.103515625e-5f * fabsf(base);
        }
        cp_async_wait<0>();
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    cp_async_wait<0>();
    __shared__ uint32_t cnt_s[kUmmaRows];
    // a CTA whose wait ran out leaves every point to the exact kernel; bit 31: second nearest not needed
    cnt_s[tid] = (ok ? n_c : (uint32_t) kCand + 1) | (need_second ? 0u : 0x80000000u);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");

    rerank_rows(a, p0, cnt_s, cand, warp, 4);
}

cudaError_t launch_umma(const AssignArgs &a, cudaStream_t stream) {
    const size_t smem_bytes = (size_t) 3 * kUmmaRows * a.dim * 4 + 2 * kUmmaRows * 4 + kUmmaRows * kCand * 4 + 2 * 8 + 16;
    cudaError_t e = cudaFuncSetAttribute(assign_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_bytes);
    if (e != cudaSuccess) return e;
    assign_umma_kernel<<<(a.n + kUmmaRows - 1) / kUmmaRows, 128, smem_bytes, stream>>>(a);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Warp-specialised variant for dim % 32 == 0: operand tiles arrive by TMA (2-D tensor maps over
// the row-major matrices, boxes of 32 floats x 128 rows, 128-byte swizzle), one producer thread
// issues the copies and the MMAs, eight epilogue warps read the accumulators (warp w: tensor-memory
// lanes 32*(w%4).., columns 64*(w/4)..). A tile then costs max(copy, MMA, epilogue), not their sum.
//
// Barriers (mbarriers in shared memory; every wait is bounded and a wait that runs out raises
// `failed`, after which nobody waits any more and every point of the CTA is flagged):
//   a_full        the point tile has landed              (TMA complete_tx)
//   b_full[s]     centroid tile in stage s has landed    (TMA complete_tx)
//   mma_done[s]   MMAs of the tile in stage s / TMEM buffer s have completed (tcgen05.commit);
//                 frees stage s for the next copy and hands buffer s to the epilogue
//   tmem_free[s]  all eight epilogue warps have read buffer s (8 arrivals)
// ---------------------------------------------------------------------------
constexpr uint32_t kEpilogueWarps = 8;
constexpr uint32_t kTmaThreads = (kEpilogueWarps + 1) * 32;

__global__ void __launch_bounds__(kTmaThreads) assign_umma_tma_kernel(const AssignArgs a, const __grid_constant__ CUtensorMap tm_points,
                                                                       const __grid_constant__ CUtensorMap tm_centroids) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t) 1023);
    const uint32_t dim = a.dim, kblocks = dim >> 5, ksteps = dim >> 3;
    const uint32_t sub_bytes = kUmmaRows * 128u;              // one 32-float column block of a tile
    const uint32_t tile_bytes = kblocks * sub_bytes;
    uint8_t *As = base;
    uint8_t *Bs = As + tile_bytes;                            // two stages
    // Norms of the centroid tiles, FOUR buffers (tile t uses t & 3): the copy for tile t+2 is issued as
    // soon as the MMAs of tile t are done, while the epilogue may still be reading tile t's norms; the
    // copy for tile t+4 is only issued after the MMAs of tile t+2, which waited for that epilogue.
    float *cn_s = reinterpret_cast<float *>(Bs + 2 * tile_bytes);
    float *rowmin = cn_s + 4 * kUmmaRows;                                 // 2 halves x 128 rows x 2
    uint32_t *cand = reinterpret_cast<uint32_t *>(rowmin + 4 * kUmmaRows);  // 128 x kCand
    uint32_t *cnt = cand + kUmmaRows * kCand;                 // 128 counters; later bit 31: far second
    uint64_t *bars = reinterpret_cast<uint64_t *>(cnt + kUmmaRows);       // a_full, b_full[2], mma_done[2], tmem_free[2]
    uint64_t *a_full = bars, *b_full = bars + 1, *mma_done = bars + 3, *tmem_free = bars + 5;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 7);
    volatile uint32_t *failed = tmem_slot + 1;
    const float *norms = a.tc_norms;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t p0 = blockIdx.x * kUmmaRows;
    const uint32_t tiles = (a.C + kUmmaRows - 1) / kUmmaRows, total = 2 * tiles;

    if (tid == 0) {
        mbar_init(a_full, 1);
        for (int s = 0; s < 2; s++) { mbar_init(b_full + s, 1); mbar_init(mma_done + s, 1); mbar_init(tmem_free + s, kEpilogueWarps); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        *failed = 0;
    }
    if (tid < kUmmaRows) cnt[tid] = 0;
    if (warp == kEpilogueWarps) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == kEpilogueWarps) {
        // ================= producer: TMA copies and MMA issue, one thread =================
        if (lane == 0) {
            // a centroid tile travels with the 128 norms of its rows (a plain bulk copy; the norms
            // array is padded to a whole tile)
            auto load_tile = [&](uint8_t *dst, const CUtensorMap *tm, uint32_t row0, uint64_t *bar, float *norm_dst) {
                mbar_expect_tx(bar, tile_bytes + (norm_dst ? kUmmaRows * 4u : 0u));
                for (uint32_t kb = 0; kb < kblocks; kb++) tma_load_2d(dst + kb * sub_bytes, tm, kb * 32u, row0, bar);
                if (norm_dst)
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                     smem_u32(norm_dst)),
                                 "l"(reinterpret_cast<uint64_t>(norms + row0)), "r"(kUmmaRows * 4u), "r"(smem_u32(bar))
                                 : "memory");
            };
            load_tile(As, &tm_points, p0, a_full, nullptr);
            load_tile(Bs, &tm_centroids, 0, b_full + 0, cn_s);
            if (total > 1) load_tile(Bs + tile_bytes, &tm_centroids, (1u % tiles) * kUmmaRows, b_full + 1, cn_s + kUmmaRows);
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((kUmmaRows >> 3) << 17) | ((kUmmaRows >> 4) << 24);
            const uint32_t a_addr = smem_u32(As), b_addr = smem_u32(Bs);
            bool ok = mbar_wait(a_full, 0, failed);
            for (uint32_t t = 0; t < total && ok; t++) {
                const uint32_t s = t & 1u, use = t >> 1;
                ok = mbar_wait(b_full + s, use & 1u, failed);
                if (ok && t >= 2) ok = mbar_wait(tmem_free + s, (use - 1) & 1u, failed);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (uint32_t ks = 0; ks < ksteps; ks++) {
                    const uint32_t off = (ks >> 2) * sub_bytes + (ks & 3u) * 32u;
                    mma_tf32(tmem_base + s * kUmmaRows, desc_sw128(a_addr + off),
                              desc_sw128(b_addr + s * tile_bytes + off), idesc, ks > 0 ? 1u : 0u);
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(mma_done + s))
                             : "memory");
                if (t + 2 < total) {   // stage s is free once these MMAs have read it
                    ok = mbar_wait(mma_done + s, use & 1u, failed);
                    if (ok) load_tile(Bs + s * tile_bytes, &tm_centroids, ((t + 2) % tiles) * kUmmaRows, b_full + s, cn_s + ((t + 2) & 3u) * kUmmaRows);
                }
            }
        }
    } else {
        // ================= epilogue warps =================
        const uint32_t quad = warp & 3u, half = warp >> 2;
        const uint32_t row = quad * 32u + lane;
        const uint32_t p = p0 + row;
        float pnr = 0.0f;
        if (p < a.n) {
            const float4 *src = reinterpret_cast<const float4 *>(a.data + (uint64_t) p * dim);
            for (uint32_t c = 0; c < (dim >> 2); c++) {
                const float4 v = __ldg(src + c);
                pnr += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
        }
        const float cm = __ldg(norms + a.C);
        const float err = 0.0078125f * sqrtf(pnr) * sqrtf(cm) + 1.52587890625e-5f * (pnr + cm);
        float m1 = FLT_MAX, m2 = FLT_MAX, thr = 0.0f;
        bool need_second = false;
        for (uint32_t t = 0; t < total; t++) {
            const uint32_t s = t & 1u, use = t >> 1;
            bool ok = !*failed && mbar_wait(mma_done + s, use & 1u, failed);
            ok = __all_sync(kFullMask, ok);   // tcgen05.ld is a warp-wide instruction
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t c0 = (t % tiles) * kUmmaRows + half * 64u;
                const bool second = t >= tiles;
                for (uint32_t cb = 0; cb < 64; cb += 32) {
                    uint32_t r[32];
                    tmem_load32(tmem_base + ((quad * 32u) << 16) + s * kUmmaRows + half * 64u + cb, r);
#pragma unroll
                    for (int j4 = 0; j4 < 32; j4 += 4) {
                        const uint32_t cid = c0 + cb + j4;
                        const float4 cn4 = *reinterpret_cast<const float4 *>(cn_s + (t & 3u) * kUmmaRows + half * 64u + cb + j4);  // broadcast
                        const float cn[4] = {cn4.x, cn4.y, cn4.z, cn4.w};
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const float d = (cid + j < a.C) ? (pnr + cn[j]) - 2.0f * __uint_as_float(r[j4 + j]) : FLT_MAX;
                            if (!second) {
                                min2_add(m1, m2, d);
                            } else if (d <= thr) {
                                const uint32_t k = atomicAdd(&cnt[row], 1u);
                                if (k < (uint32_t) kCand) cand[row * kCand + k] = cid + j;
                            }
                        }
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(tmem_free + s);
            }
            if (t + 1 == tiles) {
                // both column halves of a row meet here
                rowmin[(half * kUmmaRows + row) * 2] = m1;
                rowmin[(half * kUmmaRows + row) * 2 + 1] = m2;
                named_barrier_sync(1, kEpilogueWarps * 32);
                const float o1 = rowmin[((half ^ 1u) * kUmmaRows + row) * 2], o2 = rowmin[((half ^ 1u) * kUmmaRows + row) * 2 + 1];
                m2 = fminf(fminf(m2, o2), fmaxf(m1, o1));
                m1 = fminf(m1, o1);
                const bool boundary_test = a.is_boundary && a.boundary_factor >= 0.0f && a.C > 1;
                if (boundary_test) {
                    const float lo2 = fmaxf(m2 - err, 0.0f), hi1 = m1 + err;
                    const float f = a.metric == kEuclidean ? a.boundary_factor * a.boundary_factor : a.boundary_factor;
                    need_second = !(lo2 > f * hi1 * 1.001f);
                }
                const float basev = need_second ? m2 : m1;
                thr = basev + 2.0f * err + 6.103515625e-5f * fabsf(basev);
            }
        }
        named_barrier_sync(1, kEpilogueWarps * 32);
        if (half == 0) {
            const uint32_t n_c = *failed ? (uint32_t) kCand + 1 : cnt[row];
            cnt[row] = (n_c > (uint32_t) kCand ? (uint32_t) kCand + 1 : n_c) | (need_second ? 0u : 0x80000000u);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kEpilogueWarps) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
        return;
    }

    rerank_rows(a, p0, cnt, cand, warp, kEpilogueWarps);
}

// Returns cudaErrorNotSupported when the tensor maps cannot be made (the caller then takes the cp.async kernel).
cudaError_t launch_umma_tma(const AssignArgs &a, cudaStream_t stream) {
    if ((reinterpret_cast<uintptr_t>(a.data) & 15u) || (reinterpret_cast<uintptr_t>(a.centroids) & 15u)) return cudaErrorNotSupported;
    CUtensorMap tm_points, tm_centroids;
    if (!make_row_map(&tm_points, a.data, a.n, a.dim, kUmmaRows) || !make_row_map(&tm_centroids, a.centroids, a.C, a.dim, kUmmaRows)) return cudaErrorNotSupported;
    const size_t smem_bytes = 1024 + (size_t) 3 * kUmmaRows * a.dim * 4 + 8 * kUmmaRows * 4 + kUmmaRows * kCand * 4 + kUmmaRows * 4 + 7 * 8 + 16;
    cudaError_t e = cudaFuncSetAttribute(assign_umma_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_bytes);
    if (e != cudaSuccess) return e;
    assign_umma_tma_kernel<<<(a.n + kUmmaRows - 1) / kUmmaRows, kTmaThreads, smem_bytes, stream>>>(a, tm_points, tm_centroids);
    return cudaGetLastError();
}

}  // namespace

bool assign_tc_eligible(const AssignArgs &a) {
    return a.tc_norms != nullptr && (a.dim & 15u) == 0 && a.dim <= kMaxDim && a.C >= 2;
}

cudaError_t launch_assign_tc(const AssignArgs &a, cudaStream_t stream) {
    cudaError_t e = cudaMemsetAsync(a.tc_norms + a.C, 0, sizeof(float), stream);
    if (e != cudaSuccess) return e;
    centroid_norms_kernel<<<(a.C + 7) / 8, 256, 0, stream>>>(a.centroids, a.C, a.dim, a.tc_norms);
    static const bool no_tma = [] { const char *v = std::getenv("GLIDE_B200_NO_TMA"); return v && v[0] == '1'; }();
    if ((a.dim & 31u) == 0 && !no_tma) {
        e = launch_umma_tma(a, stream);
        if (e != cudaErrorNotSupported) return e;
    }
    return launch_umma(a, stream);
}

}  // namespace glide
