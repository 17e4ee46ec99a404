// Random sampling on the device with the Philox4x32-10 counter of homura's generator (src/ops/random.rs): the
// same counter, key, word order and conversions as the CPU's sample_float and sample_int, so that uniform
// samples and integers carry the CPU's bits; normal samples go through this library's log, cos and sin.
// Stands in for csrc/random.hip (hmr_random_uniform, hmr_random_normal, hmr_random_int).
//
// One thread computes one Philox block (four 32-bit words) and writes the block's values with one store: four
// values of F16, BF16 or F32, two of F64, two normals, or two integers. The kernels are bound by the integer
// pipe (ten rounds of two wide multiplications) and by the write bandwidth, in that order.
//
// Integer sampling rejects words below a threshold, so where a word lands depends on how many words before
// it were rejected. A batch is cut into tiles of HMC_RANDOM_INT_TILE blocks: a first kernel counts the accepted
// words of each tile, a running sum (two launches) turns the counts into starting positions, and a last kernel
// recomputes the words and writes the accepted ones at their positions, in the CPU's word order.
#include <math_constants.h>

#include "common.cuh"
#include "elem.cuh"
#include "map.cuh"
#include "scan.cuh"

namespace hmc {
namespace {

constexpr int kSampleThreads = 256;
constexpr int kBlocksPerThread = 4;  // Philox blocks a thread of the uniform and the unrejected integer sampler takes

struct Words4 {
    uint32_t w[4];
};

// Block n under the key [seed, seed >> 32]. src/ops/random.rs:29-51, 75-83.
__device__ __forceinline__ Words4 philox_block(uint64_t n, uint64_t seed) {
    constexpr uint32_t kM0 = 0xD2511F53u, kM1 = 0xCD9E8D57u;
    constexpr uint32_t kW0 = 0x9E3779B9u, kW1 = 0xBB67AE85u;
    uint32_t c0 = static_cast<uint32_t>(n), c1 = static_cast<uint32_t>(n >> 32), c2 = 0, c3 = 0;
    uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
#pragma unroll
    for (int round = 0; round < 10; ++round) {
        if (round > 0) {
            k0 += kW0;
            k1 += kW1;
        }
        const uint64_t p0 = static_cast<uint64_t>(kM0) * c0;  // one wide multiplication each
        const uint64_t p1 = static_cast<uint64_t>(kM1) * c2;
        c0 = static_cast<uint32_t>(p1 >> 32) ^ c1 ^ k0;
        c1 = static_cast<uint32_t>(p1);
        c2 = static_cast<uint32_t>(p0 >> 32) ^ c3 ^ k1;
        c3 = static_cast<uint32_t>(p0);
    }
    return Words4{{c0, c1, c2, c3}};
}

// A uniform f64 in [0, 1) from 53 bits; exact. src/ops/random.rs:86-90.
__device__ __forceinline__ double unit_f64(uint32_t hi, uint32_t lo) {
    const uint64_t bits = (static_cast<uint64_t>(hi) << 21) ^ (static_cast<uint64_t>(lo) >> 11);
    return static_cast<double>(bits) * (1.0 / 9007199254740992.0);
}

template <class T> constexpr int significand_bits() {
    return std::is_same_v<T, F16> ? 11 : (std::is_same_v<T, BF16> ? 8 : (std::is_same_v<T, float> ? 24 : 53));
}

// from + u * (to - from) rounded to T; a result that reaches `to` becomes `from`. src/ops/random.rs:268-277.
template <class T>
__device__ __forceinline__ T uniform_value(double u, double from, double width, double to, T first) {
    const T v = from_f64<T>(from + u * width);
    return (from < to && to_f64(v) >= to) ? first : v;
}

// UNIT: from = 0 and to = 1 in a dtype narrower than f64. The sample k * 2^-BITS (k below 2^BITS) is then a value
// of T itself, so the f64 scaling, the rounding and the comparison with `to` change nothing and are left out.
template <class T, bool UNIT>
__global__ void __launch_bounds__(kSampleThreads) uniform_kernel(T *out, int64_t n, uint64_t seed, uint64_t offset, double from,
                                                                  double to) {
    constexpr int PER = std::is_same_v<T, double> ? 2 : 4;
    constexpr int BITS = significand_bits<T>();
    const int64_t blocks = (n + PER - 1) / PER;
    const double width = to - from;
    const T first = from_f64<T>(from);
    const bool aligned = (reinterpret_cast<uintptr_t>(out) & (sizeof(T) * PER - 1)) == 0;
    // (a thread takes kBlocksPerThread blocks a grid stride apart: their rounds interleave)
#pragma unroll 4
    for (int64_t b = static_cast<int64_t>(blockIdx.x) * kSampleThreads + threadIdx.x; b < blocks;
         b += static_cast<int64_t>(gridDim.x) * kSampleThreads) {
        const Words4 r = philox_block(offset + static_cast<uint64_t>(b), seed);
        Pack<T, PER> v;
#pragma unroll
        for (int j = 0; j < PER; ++j) {
            if constexpr (UNIT && PER == 4) {
                v.v[j] = down<T>(__uint2float_rn(r.w[j] >> (32 - BITS)) * (1.0f / static_cast<float>(1u << BITS)));  // exact
            } else {
                double u;
                if constexpr (PER == 2) u = unit_f64(r.w[2 * j], r.w[2 * j + 1]);
                else u = static_cast<double>(r.w[j] >> (32 - BITS)) * (1.0 / static_cast<double>(1u << BITS));  // exact, as the division
                v.v[j] = uniform_value<T>(u, from, width, to, first);
            }
        }
        const int64_t i0 = b * PER;
        if (aligned && i0 + PER <= n) {
            *reinterpret_cast<Pack<T, PER> *>(out + i0) = v;
        } else {
#pragma unroll
            for (int j = 0; j < PER; ++j)
                if (i0 + j < n) out[i0 + j] = v.v[j];
        }
    }
}

// Box-Muller, two values per block. src/ops/random.rs:184-197.
template <class T>
__global__ void __launch_bounds__(kSampleThreads) normal_kernel(T *out, int64_t n, uint64_t seed, uint64_t offset, double mean,
                                                                 double std) {
    const int64_t blocks = (n + 1) / 2;
    const bool aligned = (reinterpret_cast<uintptr_t>(out) & (sizeof(T) * 2 - 1)) == 0;
    for (int64_t b = static_cast<int64_t>(blockIdx.x) * kSampleThreads + threadIdx.x; b < blocks;
         b += static_cast<int64_t>(gridDim.x) * kSampleThreads) {
        const Words4 w = philox_block(offset + static_cast<uint64_t>(b), seed);
        const double u1 = 1.0 - unit_f64(w.w[0], w.w[1]);
        const double u2 = unit_f64(w.w[2], w.w[3]);
        const double r = sqrt(-2.0 * log(u1));
        const double theta = 2.0 * 3.14159265358979323846 * u2;
        double s, c;
        sincos(theta, &s, &c);
        Pack<T, 2> v;
        v.v[0] = from_f64<T>(mean + std * r * c);
        v.v[1] = from_f64<T>(mean + std * r * s);
        const int64_t i0 = b * 2;
        if (aligned && i0 + 2 <= n) {
            *reinterpret_cast<Pack<T, 2> *>(out + i0) = v;
        } else {
            out[i0] = v.v[0];
            if (i0 + 1 < n) out[i0 + 1] = v.v[1];
        }
    }
}

// The two 64-bit words of a block in the order the CPU takes them. src/ops/random.rs:226-229.
__device__ __forceinline__ void block_words(uint64_t n, uint64_t seed, uint64_t &first, uint64_t &second) {
    const Words4 r = philox_block(n, seed);
    first = (static_cast<uint64_t>(r.w[0]) << 32) | r.w[1];
    second = (static_cast<uint64_t>(r.w[2]) << 32) | r.w[3];
}

// w % range without the general 64-bit division where the range allows: a mask for a power of two; for a range of
// at most 2^21, two steps through inv = 1 / range in f64: the high half h (below 2^32, exact as an f64) gives
// h * inv truncated, the quotient or one beside it, so one correction leaves h % range; then x = that * 2^32 + the
// low half is below 2^53, exact again, and the same step gives the remainder. The branches are the same for every
// thread of a launch.
struct Modulus {
    uint64_t range;
    double inv;     // 1 / range, for kind 1
    int32_t kind;   // 0: power of two, 1: at most 2^21, 2: any
};

inline Modulus modulus_of(uint64_t range) {
    Modulus m;
    m.range = range;
    m.inv = 1.0 / static_cast<double>(range);
    m.kind = (range & (range - 1)) == 0 ? 0 : (range <= (1u << 21) ? 1 : 2);
    return m;
}

__device__ __forceinline__ uint64_t word_mod(uint64_t w, const Modulus &m) {
    if (m.kind == 0) return w & (m.range - 1);
    if (m.kind == 1) {
        const int64_t r = static_cast<int64_t>(m.range);
        const int64_t hi = static_cast<int64_t>(w >> 32);
        int64_t h = hi - __double2ll_rz(__ll2double_rn(hi) * m.inv) * r;
        if (h < 0) h += r;
        if (h >= r) h -= r;
        const int64_t x = (h << 32) | static_cast<int64_t>(static_cast<uint32_t>(w));
        int64_t rem = x - __double2ll_rz(__ll2double_rn(x) * m.inv) * r;
        if (rem < 0) rem += r;
        if (rem >= r) rem -= r;
        return static_cast<uint64_t>(rem);
    }
    return w % m.range;
}

// threshold == 0: word k of the batch is value k.
__global__ void __launch_bounds__(kSampleThreads) int_all_kernel(int64_t *out, int64_t n, uint64_t seed, uint64_t offset,
                                                                  uint64_t blocks, int64_t low, const Modulus range) {
    const bool aligned = (reinterpret_cast<uintptr_t>(out) & 15) == 0;
#pragma unroll 4
    for (uint64_t b = static_cast<uint64_t>(blockIdx.x) * kSampleThreads + threadIdx.x; b < blocks;
         b += static_cast<uint64_t>(gridDim.x) * kSampleThreads) {
        uint64_t w0, w1;
        block_words(offset + b, seed, w0, w1);
        Pack<int64_t, 2> v;
        v.v[0] = static_cast<int64_t>(static_cast<uint64_t>(low) + word_mod(w0, range));
        v.v[1] = static_cast<int64_t>(static_cast<uint64_t>(low) + word_mod(w1, range));
        const int64_t i0 = static_cast<int64_t>(b) * 2;
        if (aligned && i0 + 2 <= n) {
            *reinterpret_cast<Pack<int64_t, 2> *>(out + i0) = v;
        } else {
            if (i0 < n) out[i0] = v.v[0];
            if (i0 + 1 < n) out[i0 + 1] = v.v[1];
        }
    }
}

// The number of accepted words among the threads of a block that come before this one, and (total) in all.
__device__ __forceinline__ uint32_t block_exclusive_count(uint32_t mine, uint32_t &total) {
    __shared__ uint32_t warp_sum[kSampleThreads / 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t inclusive = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t up = __shfl_up_sync(0xFFFFFFFFu, inclusive, d);
        if (lane >= d) inclusive += up;
    }
    if (lane == 31) warp_sum[warp] = inclusive;
    __syncthreads();
    uint32_t before = 0, all = 0;
#pragma unroll
    for (int w = 0; w < kSampleThreads / 32; ++w) {
        const uint32_t s = warp_sum[w];
        if (w < warp) before += s;
        all += s;
    }
    __syncthreads();
    total = all;
    return before + inclusive - mine;
}

// A tile is HMC_RANDOM_INT_TILE blocks: one block of threads, one Philox block per thread.
static_assert(HMC_RANDOM_INT_TILE == kSampleThreads, "a tile is one thread block");

// Counts the accepted words of every tile and, while it has the words, writes them where they belong if no word
// of an earlier tile was rejected (position of the tile's first word: two per block before it). For the ranges of
// practice a rejection has a probability near 2^-48, so that is nearly always the final place.
__global__ void __launch_bounds__(kSampleThreads) int_count_kernel(uint64_t *counts, uint64_t tiles, uint64_t seed, uint64_t offset,
                                                                    uint64_t blocks, uint64_t threshold, int64_t *out, int64_t n,
                                                                    int64_t low, const Modulus range) {
    for (uint64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const uint64_t b = tile * HMC_RANDOM_INT_TILE + threadIdx.x;
        uint64_t w0 = 0, w1 = 0;
        bool take0 = false, take1 = false;
        if (b < blocks) {
            block_words(offset + b, seed, w0, w1);
            take0 = w0 >= threshold;
            take1 = w1 >= threshold;
        }
        if (__syncthreads_and(take0 && take1)) {  // a whole tile, nothing rejected: no ranks to find
            if (threadIdx.x == 0) counts[tile] = 2 * HMC_RANDOM_INT_TILE;
            const uint64_t first = 2 * b;
            Pack<int64_t, 2> v;
            v.v[0] = static_cast<int64_t>(static_cast<uint64_t>(low) + word_mod(w0, range));
            v.v[1] = static_cast<int64_t>(static_cast<uint64_t>(low) + word_mod(w1, range));
            if (first + 2 <= static_cast<uint64_t>(n) && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
                *reinterpret_cast<Pack<int64_t, 2> *>(out + first) = v;
            } else {
                if (first < static_cast<uint64_t>(n)) out[first] = v.v[0];
                if (first + 1 < static_cast<uint64_t>(n)) out[first + 1] = v.v[1];
            }
            continue;
        }
        uint32_t total;
        uint64_t at = tile * (2 * HMC_RANDOM_INT_TILE) + block_exclusive_count((take0 ? 1u : 0u) + (take1 ? 1u : 0u), total);
        if (threadIdx.x == 0) counts[tile] = total;
        if (take0) {
            if (at < static_cast<uint64_t>(n)) out[at] = static_cast<int64_t>(static_cast<uint64_t>(low) + word_mod(w0, range));
            at += 1;
        }
        if (take1 && at < static_cast<uint64_t>(n)) out[at] = static_cast<int64_t>(static_cast<uint64_t>(low) + word_mod(w1, range));
    }
}

// The tiles after the first rejected word: their words are recomputed and written at their final places. (Positions at
// and beyond the number of accepted words may hold words of the first attempt; a later batch overwrites them.)
constexpr int kPlaceSpan = 32;

__global__ void __launch_bounds__(kSampleThreads) int_place_kernel(int64_t *out, int64_t n, const uint64_t *starts, uint64_t tiles,
                                                                    uint64_t seed, uint64_t offset, uint64_t blocks, int64_t low,
                                                                    const Modulus range, uint64_t threshold) {
    // A block takes spans of kPlaceSpan tiles; its first threads look at one tile's start each, and a span without
    // work (the usual case: every tile already in place) costs one barrier instead of a block per tile.
    for (uint64_t span = blockIdx.x; span * kPlaceSpan < tiles; span += gridDim.x) {
        const uint64_t t0 = span * kPlaceSpan;
        bool work = false;
        if (threadIdx.x < kPlaceSpan && t0 + threadIdx.x < tiles) {
            const uint64_t st = starts[t0 + threadIdx.x];
            work = st < static_cast<uint64_t>(n) && st != (t0 + threadIdx.x) * (2 * HMC_RANDOM_INT_TILE);
        }
        if (!__syncthreads_or(work)) continue;
        const uint64_t t1 = t0 + kPlaceSpan < tiles ? t0 + kPlaceSpan : tiles;
        for (uint64_t tile = t0; tile < t1; ++tile) {
            const uint64_t start = starts[tile];
            // (both the same for the whole block) everything here is dropped, or already in place
            if (start >= static_cast<uint64_t>(n) || start == tile * (2 * HMC_RANDOM_INT_TILE)) continue;
            const uint64_t b = tile * HMC_RANDOM_INT_TILE + threadIdx.x;
            uint64_t w0 = 0, w1 = 0;
            bool take0 = false, take1 = false;
            if (b < blocks) {
                block_words(offset + b, seed, w0, w1);
                take0 = w0 >= threshold;
                take1 = w1 >= threshold;
            }
            uint32_t total;
            uint64_t at = start + block_exclusive_count((take0 ? 1u : 0u) + (take1 ? 1u : 0u), total);
            if (take0) {
                if (at < static_cast<uint64_t>(n)) out[at] = static_cast<int64_t>(static_cast<uint64_t>(low) + word_mod(w0, range));
                at += 1;
            }
            if (take1 && at < static_cast<uint64_t>(n)) out[at] = static_cast<int64_t>(static_cast<uint64_t>(low) + word_mod(w1, range));
        }
    }
}

// `out` must be flat and contiguous; returns its element count and first element.
hmc_status check_flat(const hmc_tensor_desc *out, int64_t *n) {
    hmc_status s = check_desc(out, "the output");
    if (s != HMC_OK) return s;
    if (out->ndim > 1) return fail(HMC_INVALID, "the output of a sampler is flat (at most one dimension)");
    *n = out->ndim == 0 ? 1 : out->sizes[0];
    if (out->ndim == 1 && *n > 1 && out->strides[0] != 1) return fail(HMC_INVALID, "the output of a sampler is contiguous");
    if (*n > 0 && out->data == nullptr) return fail(HMC_INVALID, "null data pointer");
    return HMC_OK;
}

unsigned sample_grid(int64_t work_items) {
    const int64_t blocks = ceil_div(work_items, kSampleThreads);
    const int64_t cap = int64_t{1} << 22;
    return static_cast<unsigned>(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

}  // namespace
}  // namespace hmc

using namespace hmc;

HMC_API hmc_status hmc_random_uniform(hmc_context_t ctx, const hmc_tensor_desc *out, uint64_t seed, uint64_t offset, double from,
                                      double to) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        int64_t n = 0;
        hmc_status s = check_flat(out, &n);
        if (s != HMC_OK) return s;
        if (!dtype_is_float(out->dtype)) return fail(HMC_INVALID, "uniform sampling needs a floating point tensor");
        if (n == 0) return HMC_OK;
        return dispatch_float(out->dtype, [&](auto t) -> hmc_status {
            using T = decltype(t);
            constexpr int per = std::is_same_v<T, double> ? 2 : 4;
            T *p = static_cast<T *>(out->data) + out->offset;
            if (per == 4 && from == 0.0 && to == 1.0 && !std::signbit(from)) {
                uniform_kernel<T, true><<<sample_grid(ceil_div(n, per * kBlocksPerThread)), kSampleThreads, 0, ctx->stream>>>(p, n, seed, offset, from, to);
            } else {
                uniform_kernel<T, false><<<sample_grid(ceil_div(n, per * kBlocksPerThread)), kSampleThreads, 0, ctx->stream>>>(p, n, seed, offset, from, to);
            }
            return launch_status("uniform sampling kernel launch");
        });
    });
}

HMC_API hmc_status hmc_random_normal(hmc_context_t ctx, const hmc_tensor_desc *out, uint64_t seed, uint64_t offset, double mean,
                                     double std) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        int64_t n = 0;
        hmc_status s = check_flat(out, &n);
        if (s != HMC_OK) return s;
        if (!dtype_is_float(out->dtype)) return fail(HMC_INVALID, "normal sampling needs a floating point tensor");
        if (n == 0) return HMC_OK;
        return dispatch_float(out->dtype, [&](auto t) -> hmc_status {
            using T = decltype(t);
            T *p = static_cast<T *>(out->data) + out->offset;
            normal_kernel<T><<<sample_grid(ceil_div(n, 2)), kSampleThreads, 0, ctx->stream>>>(p, n, seed, offset, mean, std);
            return launch_status("normal sampling kernel launch");
        });
    });
}

HMC_API hmc_status hmc_random_int(hmc_context_t ctx, const hmc_tensor_desc *out, uint64_t seed, uint64_t offset, uint64_t blocks,
                                  int64_t low, uint64_t range, uint64_t threshold, void *workspace) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        int64_t n = 0;
        hmc_status s = check_flat(out, &n);
        if (s != HMC_OK) return s;
        if (out->dtype != HMC_I64) return fail(HMC_INVALID, "integer sampling writes an I64 tensor");
        if (range == 0) return fail(HMC_INVALID, "integer sampling needs a nonempty range");
        if (threshold >= range) return fail(HMC_INVALID, "the rejection threshold is below the range");
        if (blocks > (uint64_t{1} << 62)) return fail(HMC_INVALID, "too many blocks");
        int64_t *p = static_cast<int64_t *>(out->data) + out->offset;
        if (threshold == 0) {
            if (n == 0 || blocks == 0) return HMC_OK;
            int_all_kernel<<<sample_grid(ceil_div(static_cast<int64_t>(blocks), kBlocksPerThread)), kSampleThreads, 0, ctx->stream>>>(p, n, seed, offset, blocks, low,
                                                                                                       modulus_of(range));
            return launch_status("integer sampling kernel launch");
        }
        if (workspace == nullptr) return fail(HMC_INVALID, "integer sampling with rejection needs its workspace");
        if ((reinterpret_cast<uintptr_t>(workspace) & 7) != 0) return fail(HMC_INVALID, "the workspace is not 8-byte aligned");
        const uint64_t tiles = (blocks + HMC_RANDOM_INT_TILE - 1) / HMC_RANDOM_INT_TILE;
        uint64_t *counts = static_cast<uint64_t *>(workspace);
        uint64_t *starts = counts + tiles;
        uint64_t *total = counts + 2 * tiles;
        if (tiles == 0) {
            HMC_CUDA(cudaMemsetAsync(total, 0, sizeof(uint64_t), ctx->stream), "cudaMemsetAsync");
            return HMC_OK;
        }
        const unsigned grid = static_cast<unsigned>(tiles < (uint64_t{1} << 22) ? tiles : (uint64_t{1} << 22));
        int_count_kernel<<<grid, kSampleThreads, 0, ctx->stream>>>(counts, tiles, seed, offset, blocks, threshold, p, n, low, modulus_of(range));
        s = launch_status("integer sampling (count) kernel launch");
        if (s != HMC_OK) return s;
        launch_tile_starts(ctx->stream, counts, starts, total, tiles);
        s = launch_status("integer sampling (positions) kernel launch");
        if (s != HMC_OK) return s;
        if (n == 0) return HMC_OK;
        const uint64_t spans = (tiles + kPlaceSpan - 1) / kPlaceSpan;
        const unsigned place_grid = static_cast<unsigned>(spans < (uint64_t{1} << 22) ? spans : (uint64_t{1} << 22));
        int_place_kernel<<<place_grid, kSampleThreads, 0, ctx->stream>>>(p, n, starts, tiles, seed, offset, blocks, low, modulus_of(range), threshold);
        return launch_status("integer sampling (placement) kernel launch");
    });
}
