// Ordered compaction in three steps, shared by the kernels that keep "the k-th element that qualifies, in row-major
// order": a count per tile (one thread block of 256 candidates), the tiles' starting positions by a one-block
// running sum, and a placement pass that recomputes the candidates and ranks them inside the tile.
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

// starts[t] = counts[0] + ... + counts[t - 1]; *total = the sum of all. One block of 1024 threads.
static __global__ void __launch_bounds__(1024) tile_starts_kernel(const uint64_t *counts, uint64_t *starts, uint64_t *total,
                                                                  uint64_t tiles) {
    __shared__ uint64_t warp_sum[32];
    __shared__ uint64_t carry_shared;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint64_t carry = 0;
    for (uint64_t t0 = 0; t0 < tiles; t0 += 1024) {
        const uint64_t t = t0 + threadIdx.x;
        const uint64_t mine = t < tiles ? counts[t] : 0;
        uint64_t inclusive = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint64_t up = __shfl_up_sync(0xFFFFFFFFu, inclusive, d);
            if (lane >= d) inclusive += up;
        }
        if (lane == 31) warp_sum[warp] = inclusive;
        __syncthreads();
        uint64_t before = 0;
        for (int w = 0; w < warp; ++w) before += warp_sum[w];
        if (t < tiles) starts[t] = carry + before + inclusive - mine;
        if (threadIdx.x == 1023) carry_shared = carry + before + inclusive;
        __syncthreads();
        carry = carry_shared;
    }
    if (threadIdx.x == 0) *total = carry;
}

inline uint64_t scan_tiles(uint64_t n) { return (n + kScanThreads - 1) / kScanThreads; }
inline int64_t scan_workspace_words(uint64_t n) { return static_cast<int64_t>(2 * scan_tiles(n) + 1); }

}  // namespace hmc
