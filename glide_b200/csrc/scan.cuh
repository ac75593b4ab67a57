// Exclusive prefix sum over u32 arrays (three small kernels, no library). Used to turn
// per-destination / per-segment counts into offsets.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

namespace glide {

constexpr uint32_t kScanBlock = 1024;

__device__ __forceinline__ uint32_t block_exclusive_scan(uint32_t v, uint32_t *warp_sums, uint32_t *total) {
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    uint32_t incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const uint32_t o = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= (uint32_t) off) incl += o;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        uint32_t w = (lane < (blockDim.x >> 5)) ? warp_sums[lane] : 0;
        uint32_t wi = w;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const uint32_t o = __shfl_up_sync(0xffffffffu, wi, off);
            if (lane >= (uint32_t) off) wi += o;
        }
        warp_sums[lane] = wi - w;
        if (lane == 31) *total = wi;
    }
    __syncthreads();
    return incl - v + warp_sums[warp];
}

// pass 1: per-block exclusive scan, block totals to block_sums
static __global__ void __launch_bounds__(kScanBlock) scan_blocks_kernel(const uint32_t *__restrict__ in, uint32_t n,
                                                                  uint32_t *out, uint32_t *block_sums) {
    __shared__ uint32_t warp_sums[32];
    __shared__ uint32_t total;
    const uint32_t i = blockIdx.x * kScanBlock + threadIdx.x;
    const uint32_t v = (i < n) ? in[i] : 0;
    const uint32_t ex = block_exclusive_scan(v, warp_sums, &total);
    if (i < n) out[i] = ex;
    if (threadIdx.x == 0) block_sums[blockIdx.x] = total;
}

// pass 2: one block scans the block totals in place (chunks of 1024 with a carry);
// writes the grand total to block_sums[num_blocks].
static __global__ void __launch_bounds__(kScanBlock) scan_sums_kernel(uint32_t *block_sums, uint32_t num_blocks) {
    __shared__ uint32_t warp_sums[32];
    __shared__ uint32_t total;
    uint32_t carry = 0;
    for (uint32_t base = 0; base < num_blocks; base += kScanBlock) {
        const uint32_t i = base + threadIdx.x;
        const uint32_t v = (i < num_blocks) ? block_sums[i] : 0;
        const uint32_t ex = block_exclusive_scan(v, warp_sums, &total);
        if (i < num_blocks) block_sums[i] = ex + carry;
        carry += total;
        __syncthreads();
    }
    if (threadIdx.x == 0) block_sums[num_blocks] = carry;
}

// pass 3: add block offsets; out[n] = grand total
static __global__ void __launch_bounds__(kScanBlock) scan_add_kernel(uint32_t *out, uint32_t n,
                                                               const uint32_t *__restrict__ block_sums,
                                                               uint32_t num_blocks) {
    const uint32_t i = blockIdx.x * kScanBlock + threadIdx.x;
    if (i < n) out[i] += block_sums[blockIdx.x];
    if (i == 0) out[n] = block_sums[num_blocks];
}

inline size_t scan_tmp_bytes(uint32_t n) { return ((size_t) (n + kScanBlock - 1) / kScanBlock + 1) * sizeof(uint32_t); }

// out must have n+1 entries (out[n] = total). in and out may alias.
inline cudaError_t exclusive_scan_u32(const uint32_t *in, uint32_t n, uint32_t *out, void *tmp, cudaStream_t stream) {
    const uint32_t blocks = (n + kScanBlock - 1) / kScanBlock;
    uint32_t *sums = static_cast<uint32_t *>(tmp);
    if (blocks == 0) return cudaMemsetAsync(out, 0, sizeof(uint32_t), stream);
    scan_blocks_kernel<<<blocks, kScanBlock, 0, stream>>>(in, n, out, sums);
    scan_sums_kernel<<<1, kScanBlock, 0, stream>>>(sums, blocks);
    scan_add_kernel<<<blocks, kScanBlock, 0, stream>>>(out, n, sums, blocks);
    return cudaGetLastError();
}

}  // namespace glide
