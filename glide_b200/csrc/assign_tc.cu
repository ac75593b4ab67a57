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
// The margin bounds |approx - exact|: TF32 operands carry a relative rounding error of 2^-11
// each, so the dot product is off by at most ~2^-10 |p||c| (Cauchy-Schwarz), the distance by
// twice that; the margin is twice THAT again plus the rounding of the norms and of the
// reference's own sum. A point with more candidates than fit, or whose two best exact distances
// are equal, is left with the flag 0xffffffff for the warp-per-point kernel, whose full network
// sort reproduces the reference's tie order. The results are therefore those of the exact path,
// bit for bit.
//
// The contraction is issued as mma.sync m16n8k8 TF32: at 2 x Q x C x dim flops (2.6 GFLOP for
// 10,000 queries x 1,024 centroids x 128) it is latency bound, not tensor-throughput bound.
#include "beam_core.cuh"
#include "kernels.h"

namespace glide {

namespace {

constexpr int kCand = 8;        // candidates kept per point
constexpr int kTile = 64;       // centroids per tile
constexpr int kMaxKSteps = 16;  // dim <= 128

__device__ __forceinline__ uint32_t to_tf32(float x) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return u;
}

__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void min2_add(float &m1, float &m2, float d) {
    m2 = fminf(m2, fmaxf(m1, d));
    m1 = fminf(m1, d);
}

__device__ __forceinline__ void min2_merge(float &m1, float &m2, float o1, float o2) {
    m2 = fminf(fminf(m2, o2), fmaxf(m1, o1));
    m1 = fminf(m1, o1);
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

__device__ __forceinline__ void exact_merge(ExactNear &a, float d0, float d1, uint32_t id, uint32_t ties) {
    if (d0 < a.d0) { a.d1 = fminf(a.d0, d1); a.d0 = d0; a.id = id; a.ties = ties; }
    else if (d0 == a.d0) { a.d1 = d0; a.ties += ties; }
    else { a.d1 = fminf(a.d1, d0); }
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

// PT points per CTA (32 or 64), PT/16 m-tiles, two warps per m-tile (each takes four of the
// eight n8 tiles of a 64-centroid tile): PT/8 warps. Centroid tiles arrive through a two-stage
// cp.async pipeline (exact fp32 in shared memory, rounded to TF32 as the fragments are read).
template<int PT>
__global__ void __launch_bounds__(PT * 4) assign_tc_kernel(const AssignArgs a) {
    extern __shared__ __align__(16) float smem_f[];
    constexpr int MT = PT / 16;
    constexpr int WARPS = MT * 2;
    constexpr int THREADS = WARPS * 32;
    const uint32_t dim = a.dim, dimp = dim + 4, ksteps = dim >> 3, chunks = dim >> 2;
    float *Praw = smem_f;                              // PT x dimp, exact fp32 rows of the points
    float *Cs = Praw + PT * dimp;                      // 2 x kTile x dimp, exact fp32 centroid tiles
    float *pn = Cs + 2 * kTile * dimp;                 // PT norms
    float *thr = pn + PT;                              // PT thresholds
    float *rowmin = thr + PT;                          // 2 x PT x 2 (n-half, row, min1/min2)
    uint32_t *cnt = reinterpret_cast<uint32_t *>(rowmin + 4 * PT);   // PT
    uint32_t *cand = cnt + PT;                         // PT x kCand
    const float *norms = a.tc_norms;

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t gid = lane >> 2, tig = lane & 3;
    const uint32_t mt = warp % MT, nh = warp / MT;
    const uint32_t p0 = blockIdx.x * PT;
    const uint32_t tiles = (a.C + kTile - 1) / kTile;

    auto issue_tile = [&](uint32_t t) {  // t counts tiles over both passes
        const uint32_t c0 = (t % tiles) * kTile;
        float *buf = Cs + (t & 1u) * kTile * dimp;
        for (uint32_t e = tid; e < kTile * chunks; e += THREADS) {
            const uint32_t row = e / chunks, c = e % chunks;
            const uint32_t cid = c0 + row;
            const bool valid = cid < a.C;
            cp_async16(buf + row * dimp + 4 * c, a.centroids + (uint64_t) (valid ? cid : 0) * dim + 4 * c, valid);
        }
        cp_async_commit();
    };
    issue_tile(0);

    // ---- stage the points (exact), their norms, and this warp's A fragments ----
    for (uint32_t e = tid; e < PT * 32; e += THREADS) {
        const uint32_t row = e >> 5, c = e & 31;
        const uint32_t p = p0 + row;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (p < a.n && c < chunks) v = __ldg(reinterpret_cast<const float4 *>(a.data + (uint64_t) p * dim) + c);
        float s = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) s += __shfl_xor_sync(kFullMask, s, off);
        if (c < chunks) *reinterpret_cast<float4 *>(Praw + row * dimp + 4 * c) = v;
        if (c == 0) pn[row] = s;
    }
    if (tid < PT) cnt[tid] = 0;
    __syncthreads();
    uint32_t af[kMaxKSteps][4];
#pragma unroll
    for (int ks = 0; ks < kMaxKSteps; ks++) {
        if ((uint32_t) ks < ksteps) {
            const float *r0 = Praw + (mt * 16 + gid) * dimp + ks * 8, *r1 = r0 + 8 * dimp;
            af[ks][0] = to_tf32(r0[tig]);
            af[ks][1] = to_tf32(r1[tig]);
            af[ks][2] = to_tf32(r0[tig + 4]);
            af[ks][3] = to_tf32(r1[tig + 4]);
        } else {
            af[ks][0] = af[ks][1] = af[ks][2] = af[ks][3] = 0u;
        }
    }
    const uint32_t row0 = mt * 16 + gid, row1 = row0 + 8;
    const float pn0 = pn[row0], pn1 = pn[row1];

    float m1[2] = {FLT_MAX, FLT_MAX}, m2[2] = {FLT_MAX, FLT_MAX};
    float t0 = 0.f, t1 = 0.f;
    for (uint32_t t = 0; t < 2 * tiles; t++) {
        const int pass = t >= tiles;
        const uint32_t c0 = (t % tiles) * kTile;
        if (t + 1 < 2 * tiles) {
            issue_tile(t + 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();  // tile t has landed for every thread
        const float *buf = Cs + (t & 1u) * kTile * dimp;
        float2 cn2[4];
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
            const uint32_t cid = c0 + (nh * 4 + nt) * 8 + 2 * tig;   // even, so cid + 1 <= C when cid < C and C is even
            cn2[nt].x = cid < a.C ? __ldg(norms + cid) : 0.0f;
            cn2[nt].y = cid + 1 < a.C ? __ldg(norms + cid + 1) : 0.0f;
        }
        float acc[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; nt++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[nt][i] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < kMaxKSteps; ks++) {
            if ((uint32_t) ks < ksteps) {
#pragma unroll
                for (int nt = 0; nt < 4; nt++) {
                    const float *b = buf + ((nh * 4 + nt) * 8 + gid) * dimp + ks * 8 + tig;
                    mma_tf32(acc[nt], af[ks], to_tf32(b[0]), to_tf32(b[4]));
                }
            }
        }
#pragma unroll
        for (int nt = 0; nt < 4; nt++) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t cid = c0 + (nh * 4 + nt) * 8 + 2 * tig + (i & 1);
                if (cid >= a.C) continue;
                const int r = i >> 1;
                const float d = (r ? pn1 : pn0) + ((i & 1) ? cn2[nt].y : cn2[nt].x) - 2.0f * acc[nt][i];
                if (pass == 0) {
                    min2_add(m1[r], m2[r], d);
                } else if (d <= (r ? t1 : t0)) {
                    const uint32_t row = r ? row1 : row0;
                    const uint32_t k = atomicAdd(&cnt[row], 1u);
                    if (k < (uint32_t) kCand) cand[row * kCand + k] = cid;
                }
            }
        }
        if (t + 1 == tiles) {
            // smallest / second smallest per row: over the quad, then over the two n-halves
#pragma unroll
            for (int r = 0; r < 2; r++) {
#pragma unroll
                for (int off = 1; off <= 2; off <<= 1) {
                    const float o1 = __shfl_xor_sync(kFullMask, m1[r], off), o2 = __shfl_xor_sync(kFullMask, m2[r], off);
                    min2_merge(m1[r], m2[r], o1, o2);
                }
            }
            if (tig == 0) {
                rowmin[(nh * PT + row0) * 2 + 0] = m1[0];
                rowmin[(nh * PT + row0) * 2 + 1] = m2[0];
                rowmin[(nh * PT + row1) * 2 + 0] = m1[1];
                rowmin[(nh * PT + row1) * 2 + 1] = m2[1];
            }
            __syncthreads();
            if (tid < PT) {
                float a1 = rowmin[tid * 2], a2 = rowmin[tid * 2 + 1];
                min2_merge(a1, a2, rowmin[(PT + tid) * 2], rowmin[(PT + tid) * 2 + 1]);
                // the boundary test needs the second nearest too; routing and k-means only the nearest
                const float base = (a.is_boundary && a.C > 1) ? a2 : a1;
                const float pnr = pn[tid], cm = __ldg(norms + a.C);
                const float err = 0.00390625f * sqrtf(pnr) * sqrtf(cm) + 1.52587890625e-5f * (pnr + cm);
                thr[tid] = base + 2.0f * err + 6.103515625e-5f * fabsf(base);
            }
            __syncthreads();
            t0 = thr[row0];
            t1 = thr[row1];
        }
        __syncthreads();  // buffer t & 1 is free for tile t + 2
    }

    // ---- exact re-rank in the reference's team order ----
    const uint32_t team = lane >> 3;
    for (uint32_t row = warp; row < (uint32_t) PT; row += WARPS) {
        const uint32_t p = p0 + row;
        if (p >= a.n) continue;
        const uint32_t n_c = cnt[row];
        ExactNear st{FLT_MAX, FLT_MAX, kInvalid, 0u};
        const bool overflow = n_c > (uint32_t) kCand;
        if (!overflow) {
            for (uint32_t g = 0; g < n_c; g += 4) {
                const uint32_t j = g + team;
                const bool active = j < n_c;
                const uint32_t cid = active ? cand[row * kCand + j] : 0u;
                const float part = team_partial(Praw + row * dimp, a.centroids + (uint64_t) cid * dim, dim, active);
                const float sum = team_fold(part);
                if (active) exact_add(st, finish_metric(sum, a.metric), cid);  // every lane of the team holds the same state
            }
            // fold the four teams (lanes 0, 8, 16, 24 are representative)
#pragma unroll
            for (int off = 16; off >= 8; off >>= 1) {
                const float d0 = __shfl_xor_sync(kFullMask, st.d0, off), d1 = __shfl_xor_sync(kFullMask, st.d1, off);
                const uint32_t id = __shfl_xor_sync(kFullMask, st.id, off), ties = __shfl_xor_sync(kFullMask, st.ties, off);
                exact_merge(st, d0, d1, id, ties);
            }
        }
        if (lane == 0) {
            const bool unique = !overflow && st.ties == 1;
            a.nearest[p] = unique ? st.id : kInvalid;
            if (a.is_boundary && unique)  // partition_kernel.cuh:58-60
                a.is_boundary[p] = (a.boundary_factor >= 0.0f && a.C > 1 && st.d1 / st.d0 <= a.boundary_factor) ? 0u : kInvalid;
        }
    }
}

template<int PT>
cudaError_t launch_tc(const AssignArgs &a, cudaStream_t stream) {
    const uint32_t dimp = a.dim + 4;
    const size_t smem_bytes = ((size_t) (PT + 2 * kTile) * dimp + PT + PT + 4 * PT + PT + PT * kCand) * 4;
    auto kernel = assign_tc_kernel<PT>;
    if (smem_bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem_bytes);
        if (e != cudaSuccess) return e;
    }
    kernel<<<(a.n + PT - 1) / PT, PT * 4, smem_bytes, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace

bool assign_tc_eligible(const AssignArgs &a) {
    return a.tc_norms != nullptr && (a.dim & 7u) == 0 && a.dim <= 8 * kMaxKSteps && a.C >= 2;
}

cudaError_t launch_assign_tc(const AssignArgs &a, cudaStream_t stream) {
    cudaError_t e = cudaMemsetAsync(a.tc_norms + a.C, 0, sizeof(float), stream);
    if (e != cudaSuccess) return e;
    centroid_norms_kernel<<<(a.C + 7) / 8, 256, 0, stream>>>(a.centroids, a.C, a.dim, a.tc_norms);
    // small batches: more, smaller CTAs
    if (a.n <= 65536) return launch_tc<32>(a, stream);
    return launch_tc<64>(a, stream);
}

}  // namespace glide
