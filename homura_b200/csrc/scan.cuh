// Ordered compaction in three steps, shared by the kernels that keep "the k-th element that qualifies, in row-major
// order": a count per tile (one thread block of 256 candidates), the tiles' starting positions by a running sum
// in two launches, and a placement pass that recomputes the candidates and ranks them inside the tile.
// Workspace layout, in 64-bit words: counts[tiles], starts[tiles], total.
#pragma once

#include "common.cuh"

namespace hmc {

constexpr int kScanThreads = 256;

// The number of set flags among the threads of a block that come before this one, and (total) in the whole block.
// All kScanThreads threads call it.
__device__ __forceinline__ uint32_t block_rank(bool flag, uint32_t &total) {
    __shared__ uint32_t warp_sum[kScanThreads / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t ballot = __ballot_sync(0xFFFFFFFFu, flag);
    if (lane == 0) warp_sum[warp] = __popc(ballot);
    __syncthreads();
    uint32_t before = 0, all = 0;
#pragma unroll
    for (int w = 0; w < kScanThreads / 32; ++w) {
        const uint32_t s = warp_sum[w];
        if (w < warp) before += s;
        all += s;
    }
    __syncthreads();
    total = all;
    return before + __popc(ballot & ((1u << lane) - 1u));
}

// starts[t] = counts[0] + ... + counts[t - 1]; *total = the sum of all: two launches of ceil(n / 1024) blocks. The
// first gives every block of 1024 counts its own running sum and leaves the block's total in the first of its counts
// (which nothing reads afterwards); the second adds the totals of the blocks before. `counts` is overwritten.
constexpr int kStartsBlock = 1024;

__device__ __forceinline__ uint64_t warp_inclusive_sum(uint64_t v, int lane) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint64_t up = __shfl_up_sync(0xFFFFFFFFu, v, d);
        if (lane >= d) v += up;
    }
    return v;
}

static __global__ void __launch_bounds__(kStartsBlock) local_starts_kernel(uint64_t *counts, uint64_t *starts, uint64_t n) {
    __shared__ uint64_t warp_sum[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint64_t t = static_cast<uint64_t>(blockIdx.x) * kStartsBlock + threadIdx.x;
    const uint64_t mine = t < n ? counts[t] : 0;
    const uint64_t inclusive = warp_inclusive_sum(mine, lane);
    if (lane == 31) warp_sum[warp] = inclusive;
    __syncthreads();
    if (warp == 0) warp_sum[lane] = warp_inclusive_sum(warp_sum[lane], lane);
    __syncthreads();
    const uint64_t before = warp > 0 ? warp_sum[warp - 1] : 0;
    if (t < n) starts[t] = before + inclusive - mine;
    if (threadIdx.x == 0) counts[static_cast<uint64_t>(blockIdx.x) * kStartsBlock] = warp_sum[31];
}

static __global__ void __launch_bounds__(kStartsBlock) add_base_kernel(const uint64_t *counts, uint64_t *starts, uint64_t *total,
                                                                       uint64_t n) {
    __shared__ uint64_t warp_sum[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint64_t part = 0;
    for (uint64_t b = threadIdx.x; b < blockIdx.x; b += kStartsBlock) part += counts[b * kStartsBlock];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) part += __shfl_xor_sync(0xFFFFFFFFu, part, d);
    if (lane == 0) warp_sum[warp] = part;
    __syncthreads();
    uint64_t base = 0;
#pragma unroll
    for (int w = 0; w < 32; ++w) base += warp_sum[w];
    const uint64_t t = static_cast<uint64_t>(blockIdx.x) * kStartsBlock + threadIdx.x;
    if (t < n && blockIdx.x > 0) starts[t] += base;
    if (blockIdx.x == gridDim.x - 1 && threadIdx.x == 0) *total = base + counts[static_cast<uint64_t>(blockIdx.x) * kStartsBlock];
}

// n > 0 counts.
inline void launch_tile_starts(cudaStream_t stream, uint64_t *counts, uint64_t *starts, uint64_t *total, uint64_t n) {
    const unsigned grid = static_cast<unsigned>((n + kStartsBlock - 1) / kStartsBlock);
    local_starts_kernel<<<grid, kStartsBlock, 0, stream>>>(counts, starts, n);
    add_base_kernel<<<grid, kStartsBlock, 0, stream>>>(counts, starts, total, n);
}

inline uint64_t scan_tiles(uint64_t n) { return (n + kScanThreads - 1) / kScanThreads; }
inline int64_t scan_workspace_words(uint64_t n) { return static_cast<int64_t>(2 * scan_tiles(n) + 1); }

}  // namespace hmc
