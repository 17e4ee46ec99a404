// index_overwrite (the overwriting index_put: the last of repeated positions wins) and mask_coordinates (nonzero).
// Stand in for hmr_index_overwrite and hmr_mask_count / hmr_mask_coordinates of csrc/index.hip; semantics of
// cpu::index_overwrite and cpu::mask_coordinates (src/backend/cpu/misc.rs:105-151).
//
// Both are deterministic without a sort. The winner of an output slice is the largest i whose position names it
// (an atomic maximum, whose result does not depend on the order of arrival), then every named slice is copied
// from its winner. The coordinates of the true elements are an ordered compaction: counts per tile, the tiles'
// starting positions, placement by rank inside the tile.
#include "common.cuh"
#include "elem.cuh"
#include "map.cuh"
#include "scan.cuh"

namespace hmc {
namespace {

constexpr int kWriteThreads = 256;

// (The caller has checked the positions; one outside the dimension names no slice rather than a word beyond the table.)
__global__ void __launch_bounds__(kWriteThreads) winners_kernel(long long *winner, const int64_t *positions, int64_t m, int64_t size) {
    for (int64_t i = blockIdx.x * static_cast<int64_t>(kWriteThreads) + threadIdx.x; i < m;
         i += static_cast<int64_t>(gridDim.x) * kWriteThreads) {
        const int64_t p = positions[i];
        if (p >= 0 && p < size) atomicMax(winner + p, static_cast<long long>(i));
    }
}

struct OverwriteArgs {
    hmc_tensor_desc out;   // with its own size along `at`
    hmc_tensor_desc src;
    const long long *winner;
    int32_t at;
    int64_t items;         // elements of out
};

template <class W>
__global__ void __launch_bounds__(kWriteThreads) overwrite_kernel(const __grid_constant__ OverwriteArgs a) {
    W *out = static_cast<W *>(a.out.data) + a.out.offset;
    const W *src = static_cast<const W *>(a.src.data) + a.src.offset;
    for (int64_t item = blockIdx.x * static_cast<int64_t>(kWriteThreads) + threadIdx.x; item < a.items;
         item += static_cast<int64_t>(gridDim.x) * kWriteThreads) {
        int64_t rest = item, oo = 0, so = 0;
        bool named = true;
        for (int d = a.out.ndim - 1; d >= 0; --d) {
            const int64_t q = d == 0 ? 0 : rest / a.out.sizes[d];
            const int64_t c = rest - q * a.out.sizes[d];
            rest = q;
            oo += c * a.out.strides[d];
            if (d == a.at) {
                const long long w = a.winner[c];
                named = w >= 0;
                so += (named ? w : 0) * a.src.strides[d];
            } else {
                so += c * a.src.strides[d];
            }
        }
        if (named) out[oo] = src[so];
    }
}

struct MaskArgs {
    hmc_tensor_desc mask;
    int64_t n;
    uint64_t tiles;
    uint64_t *counts, *starts, *total;
    int64_t *out;      // coordinates (placement only)
    int64_t columns;   // of out: the number of true elements the caller read back
};

__device__ __forceinline__ bool mask_at(const MaskArgs &a, int64_t item, int64_t (&coord)[HMC_MAX_DIMS]) {
    int64_t off = a.mask.offset;
    for (int k = a.mask.ndim - 1; k >= 0; --k) {
        const int64_t q = k == 0 ? 0 : item / a.mask.sizes[k];
        coord[k] = item - q * a.mask.sizes[k];
        off += coord[k] * a.mask.strides[k];
        item = q;
    }
    return static_cast<const uint8_t *>(a.mask.data)[off] != 0;
}

template <bool PLACE>
__global__ void __launch_bounds__(kScanThreads) mask_kernel(const __grid_constant__ MaskArgs a) {
    for (uint64_t tile = blockIdx.x; tile < a.tiles; tile += gridDim.x) {
        const int64_t item = static_cast<int64_t>(tile) * kScanThreads + threadIdx.x;
        int64_t coord[HMC_MAX_DIMS];
        const bool set = item < a.n && mask_at(a, item, coord);
        uint32_t total;
        const uint32_t rank = block_rank(set, total);
        if constexpr (PLACE) {
            if (set) {
                // (a caller that passes fewer columns than the count it was given loses the rest, not other memory)
                const int64_t k = static_cast<int64_t>(a.starts[tile]) + rank;
                if (k < a.columns) {
                    for (int d = 0; d < a.mask.ndim; ++d) a.out[d * a.columns + k] = coord[d];
                }
            }
        } else {
            if (threadIdx.x == 0) a.counts[tile] = total;
        }
    }
}

template <class F> hmc_status by_size(int dtype, F &&f) {
    switch (element_size(dtype)) {
        case 1: return f(uint8_t{});
        case 2: return f(uint16_t{});
        case 4: return f(uint32_t{});
        default: return f(uint64_t{});
    }
}

unsigned write_grid(int64_t items, int threads) {
    const int64_t blocks = ceil_div(items, threads);
    return static_cast<unsigned>(blocks < 1 ? 1 : (blocks < (int64_t{1} << 20) ? blocks : (int64_t{1} << 20)));
}

hmc_status mask_args(const hmc_tensor_desc *mask, void *workspace, int64_t workspace_bytes, MaskArgs &a) {
    hmc_status s = check_desc(mask, "the mask");
    if (s != HMC_OK) return s;
    if (mask->dtype != HMC_BOOL) return fail(HMC_INVALID, "the mask is a Bool tensor");
    int64_t n = 1;
    for (int k = 0; k < mask->ndim; ++k) {
        if (__builtin_mul_overflow(n, mask->sizes[k], &n)) return fail(HMC_INVALID, "the number of elements overflows 63 bits");
    }
    if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 7) != 0) {
        return fail(HMC_INVALID, "the mask workspace is missing or not 8-byte aligned");
    }
    if (workspace_bytes < scan_workspace_words(static_cast<uint64_t>(n)) * 8) return fail(HMC_INVALID, "the mask workspace is too small");
    if (n > 0 && mask->data == nullptr) return fail(HMC_INVALID, "null data pointer");
    a = MaskArgs{};
    a.mask = *mask;
    a.n = n;
    a.tiles = scan_tiles(static_cast<uint64_t>(n));
    a.counts = static_cast<uint64_t *>(workspace);
    a.starts = a.counts + a.tiles;
    a.total = a.counts + 2 * a.tiles;
    return HMC_OK;
}

}  // namespace
}  // namespace hmc

using namespace hmc;

HMC_API hmc_status hmc_index_overwrite_workspace(int64_t size, int64_t *bytes) {
    return guarded([&]() -> hmc_status {
        if (bytes == nullptr) return fail(HMC_INVALID, "null output");
        if (size < 0) return fail(HMC_INVALID, "negative size");
        *bytes = size * 8;
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_index_overwrite(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *src,
                                       const hmc_tensor_desc *positions, int32_t dim, void *workspace, int64_t workspace_bytes) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        hmc_status s = check_desc(out, "the output");
        if (s == HMC_OK) s = check_desc(src, "the input");
        if (s == HMC_OK) s = check_desc(positions, "the positions");
        if (s != HMC_OK) return s;
        if (out->dtype != src->dtype) return fail(HMC_INVALID, "index_overwrite writes its input's dtype");
        if (out->ndim != src->ndim || out->ndim < 1) return fail(HMC_INVALID, "index_overwrite takes operands of the same rank, at least 1");
        if (dim < 0 || dim >= out->ndim) return fail(HMC_INVALID, "the indexed dimension is out of range");
        if (positions->dtype != HMC_I64 || positions->ndim != 1 || (positions->sizes[0] > 1 && positions->strides[0] != 1)) {
            return fail(HMC_INVALID, "the positions are a contiguous 1-D I64 tensor");
        }
        const int64_t m = positions->sizes[0], size = out->sizes[dim];
        if (src->sizes[dim] != m) return fail(HMC_INVALID, "the input's size along the indexed dimension is the number of positions");
        int64_t n = 1, moved = 1;
        for (int k = 0; k < out->ndim; ++k) {
            if (k != dim && out->sizes[k] != src->sizes[k]) return fail(HMC_INVALID, "operands differ in their sizes");
            if (__builtin_mul_overflow(n, out->sizes[k], &n) || __builtin_mul_overflow(moved, src->sizes[k], &moved)) {
                return fail(HMC_INVALID, "the number of elements overflows 63 bits");
            }
        }
        if (moved == 0 || n == 0) return HMC_OK;
        if (workspace == nullptr || workspace_bytes < size * 8 || (reinterpret_cast<uintptr_t>(workspace) & 7) != 0) {
            return fail(HMC_INVALID, "the workspace of index_overwrite is missing, too small or not 8-byte aligned");
        }
        if (out->data == nullptr || src->data == nullptr || positions->data == nullptr) return fail(HMC_INVALID, "null data pointer");
        long long *winner = static_cast<long long *>(workspace);
        HMC_CUDA(cudaMemsetAsync(winner, 0xFF, static_cast<size_t>(size) * 8, ctx->stream), "cudaMemsetAsync");  // every slot -1
        winners_kernel<<<write_grid(m, kWriteThreads), kWriteThreads, 0, ctx->stream>>>(
            winner, static_cast<const int64_t *>(positions->data) + positions->offset, m, size);
        s = launch_status("index_overwrite (winners) kernel launch");
        if (s != HMC_OK) return s;
        OverwriteArgs a{*out, *src, winner, dim, n};
        const unsigned grid = write_grid(n, kWriteThreads);
        return by_size(src->dtype, [&](auto w) -> hmc_status {
            overwrite_kernel<decltype(w)><<<grid, kWriteThreads, 0, ctx->stream>>>(a);
            return launch_status("index_overwrite kernel launch");
        });
    });
}

HMC_API hmc_status hmc_mask_workspace(int64_t n, int64_t *bytes, int64_t *total_word) {
    return guarded([&]() -> hmc_status {
        if (bytes == nullptr || total_word == nullptr) return fail(HMC_INVALID, "null output");
        if (n < 0) return fail(HMC_INVALID, "negative size");
        *bytes = scan_workspace_words(static_cast<uint64_t>(n)) * 8;
        *total_word = static_cast<int64_t>(2 * scan_tiles(static_cast<uint64_t>(n)));
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_mask_count(hmc_context_t ctx, const hmc_tensor_desc *mask, void *workspace, int64_t workspace_bytes) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        MaskArgs a;
        hmc_status s = mask_args(mask, workspace, workspace_bytes, a);
        if (s != HMC_OK) return s;
        if (a.tiles == 0) {
            HMC_CUDA(cudaMemsetAsync(a.total, 0, 8, ctx->stream), "cudaMemsetAsync");
            return HMC_OK;
        }
        const unsigned grid = static_cast<unsigned>(a.tiles < (uint64_t{1} << 20) ? a.tiles : (uint64_t{1} << 20));
        mask_kernel<false><<<grid, kScanThreads, 0, ctx->stream>>>(a);
        s = launch_status("mask count kernel launch");
        if (s != HMC_OK) return s;
        launch_tile_starts(ctx->stream, a.counts, a.starts, a.total, a.tiles);
        return launch_status("mask positions kernel launch");
    });
}

HMC_API hmc_status hmc_mask_coordinates(hmc_context_t ctx, const hmc_tensor_desc *mask, void *workspace, int64_t workspace_bytes,
                                        const hmc_tensor_desc *out) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        MaskArgs a;
        hmc_status s = mask_args(mask, workspace, workspace_bytes, a);
        if (s != HMC_OK) return s;
        s = check_desc(out, "the coordinates");
        if (s != HMC_OK) return s;
        if (out->dtype != HMC_I64) return fail(HMC_INVALID, "the coordinates are an I64 tensor");
        if (out->ndim != 2 || out->sizes[0] != mask->ndim) return fail(HMC_INVALID, "the coordinates are [the mask's rank, the number of true elements]");
        int64_t expect = 1;
        for (int k = out->ndim - 1; k >= 0; --k) {
            if (out->sizes[k] != 1 && out->strides[k] != expect) return fail(HMC_INVALID, "the coordinates are contiguous");
            expect *= out->sizes[k];
        }
        if (a.tiles == 0 || expect == 0) return HMC_OK;
        if (out->data == nullptr) return fail(HMC_INVALID, "null data pointer");
        a.out = static_cast<int64_t *>(out->data) + out->offset;
        a.columns = out->sizes[1];
        const unsigned grid = static_cast<unsigned>(a.tiles < (uint64_t{1} << 20) ? a.tiles : (uint64_t{1} << 20));
        mask_kernel<true><<<grid, kScanThreads, 0, ctx->stream>>>(a);
        return launch_status("mask coordinates kernel launch");
    });
}
