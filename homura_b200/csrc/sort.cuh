// A stable least-significant-digit radix sort of (key, value) pairs, eight bits per pass, for the kernels that must
// add contributions to one target in the order the CPU adds them (index_add, scatter_add). Each pass is four
// launches: a histogram of the digit per tile of 1024 keys (digit-major, so that one running sum over the table gives
// every (digit, tile) its first destination), that running sum, and a placement that ranks equal digits inside the
// tile in their order of arrival. The first pass takes the values to be 0, 1, 2, ... when none are given.
#pragma once

#include "common.cuh"
#include "scan.cuh"

namespace hmc {

constexpr int kSortRounds = 4;                              // a tile is walked in rounds of one key per thread
constexpr int kSortTile = kScanThreads * kSortRounds;

inline uint64_t sort_tiles(uint64_t n) { return (n + kSortTile - 1) / kSortTile; }

// Bytes of workspace for n pairs with keys of up to 8 bytes: two key arrays, two value arrays, the digit table twice
// and the total, every part on an 8-byte boundary.
inline int64_t sort_workspace_bytes(uint64_t n) {
    const uint64_t even = (n + 1) & ~uint64_t{1};
    return static_cast<int64_t>(2 * n * 8 + 2 * even * 4 + (2 * 256 * sort_tiles(n) + 1) * 8);
}

template <class K> struct SortSpace {
    K *keys[2];
    uint32_t *vals[2];
    uint64_t *counts, *starts, *total;
};

template <class K> inline SortSpace<K> sort_space(void *workspace, uint64_t n) {
    const uint64_t even = (n + 1) & ~uint64_t{1};
    char *p = static_cast<char *>(workspace);
    SortSpace<K> s;
    s.keys[0] = reinterpret_cast<K *>(p);
    s.keys[1] = reinterpret_cast<K *>(p + n * 8);
    p += 2 * n * 8;
    s.vals[0] = reinterpret_cast<uint32_t *>(p);
    s.vals[1] = reinterpret_cast<uint32_t *>(p + even * 4);
    p += 2 * even * 4;
    s.counts = reinterpret_cast<uint64_t *>(p);
    s.starts = s.counts + 256 * sort_tiles(n);
    s.total = s.starts + 256 * sort_tiles(n);
    return s;
}

template <class K>
__global__ void __launch_bounds__(kScanThreads) sort_count_kernel(const K *keys, uint64_t n, int shift, uint64_t *counts,
                                                                  uint64_t tiles) {
    __shared__ uint32_t hist[256];
    for (uint64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
        hist[threadIdx.x] = 0;
        __syncthreads();
#pragma unroll
        for (int r = 0; r < kSortRounds; ++r) {
            const uint64_t i = t * kSortTile + r * kScanThreads + threadIdx.x;
            if (i < n) atomicAdd(&hist[(keys[i] >> shift) & 255], 1u);
        }
        __syncthreads();
        counts[threadIdx.x * tiles + t] = hist[threadIdx.x];
        __syncthreads();
    }
}

template <class K>
__global__ void __launch_bounds__(kScanThreads) sort_place_kernel(const K *keys, const uint32_t *vals, K *keys_out, uint32_t *vals_out,
                                                                  uint64_t n, int shift, const uint64_t *starts, uint64_t tiles) {
    __shared__ uint64_t cursor[256];
    __shared__ uint32_t warp_count[kScanThreads / 32][256];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
        cursor[threadIdx.x] = starts[threadIdx.x * tiles + t];
#pragma unroll
        for (int w = 0; w < kScanThreads / 32; ++w) warp_count[w][threadIdx.x] = 0;
        __syncthreads();
#pragma unroll
        for (int r = 0; r < kSortRounds; ++r) {
            const uint64_t i = t * kSortTile + r * kScanThreads + threadIdx.x;
            const bool live = i < n;
            const K key = live ? keys[i] : K{0};
            // the threads past the end take a digit of their own, so that they rank among themselves only
            const unsigned digit = live ? static_cast<unsigned>((key >> shift) & 255) : 256u;
            const unsigned peers = __match_any_sync(0xFFFFFFFFu, digit);
            const unsigned rank = __popc(peers & ((1u << lane) - 1u));
            if (live && rank == 0) warp_count[warp][digit] = __popc(peers);
            __syncthreads();
            if (live) {
                uint64_t dest = cursor[digit] + rank;
                for (int w = 0; w < warp; ++w) dest += warp_count[w][digit];
                keys_out[dest] = key;
                vals_out[dest] = vals != nullptr ? vals[i] : static_cast<uint32_t>(i);
            }
            __syncthreads();
            uint32_t seen = 0;
#pragma unroll
            for (int w = 0; w < kScanThreads / 32; ++w) {
                seen += warp_count[w][threadIdx.x];
                warp_count[w][threadIdx.x] = 0;
            }
            cursor[threadIdx.x] += seen;
            __syncthreads();
        }
    }
}

// Sorts the n pairs whose keys lie in s.keys[0] (values 0..n-1) by key, keys below 2^bits; returns in `result` the
// index (0 or 1) of the arrays that hold the sorted pairs.
template <class K> inline hmc_status sort_pairs(cudaStream_t stream, const SortSpace<K> &s, uint64_t n, int bits, int *result) {
    const uint64_t tiles = sort_tiles(n);
    const unsigned grid = static_cast<unsigned>(tiles < (uint64_t{1} << 16) ? tiles : (uint64_t{1} << 16));
    int from = 0;
    bool first = true;
    for (int shift = 0; shift < bits || first; shift += 8) {
        sort_count_kernel<K><<<grid, kScanThreads, 0, stream>>>(s.keys[from], n, shift, s.counts, tiles);
        launch_tile_starts(stream, s.counts, s.starts, s.total, 256 * tiles);
        sort_place_kernel<K><<<grid, kScanThreads, 0, stream>>>(s.keys[from], first ? nullptr : s.vals[from], s.keys[1 - from],
                                                                s.vals[1 - from], n, shift, s.starts, tiles);
        hmc_status st = launch_status("sort kernel launch");
        if (st != HMC_OK) return st;
        from = 1 - from;
        first = false;
    }
    *result = from;
    return HMC_OK;
}

}  // namespace hmc
