// Elementwise functions of a transposed tensor of 2-byte elements (silu of x.t(), x.t().contiguous(), a cast of
// x.t() between the half types): out[.., a, b] = f(in[.., b, a]) where the input has its unit stride along a and
// the output along b.
//
// The general tiled kernel of map.cuh reads the tile against the grain with 32-bit shared-memory loads and
// repacks pairs, about six instructions an element more than a contiguous kernel has. For 2-byte elements the
// hardware has the whole transposition in two instructions:
//
//   * the tensor memory accelerator fetches a 64 x 64 tile (8 KB) of the input into shared memory with one
//     cp.async.bulk.tensor instruction issued by one thread, in the 128-byte swizzled layout, completing on an
//     mbarrier; it clips tiles at the tensor's edge by itself (loads beyond the edge read zeros, stores beyond it
//     are dropped), so ragged shapes need no code;
//   * ldmatrix.trans hands each lane of a warp pairs of elements that are adjacent along b out of 8 x 8 blocks
//     stored along a: the transposition happens in the load. The function is applied to the registers (it is
//     elementwise, so it does not matter which lane holds what), and stmatrix writes the same registers as rows
//     of the output tile, again swizzled, which one cp.async.bulk.tensor store sends to global memory in whole
//     128-byte rows.
//
// A block of 128 threads keeps two input tiles in flight (the copy of the next tile runs while one is computed) and
// one output tile. No thread issues a global load or store. Every wait
// on an mbarrier is bounded: when one runs out the block stops taking tiles and sets the context's status word,
// which hmc_context_synchronize reports.
//
// Tensor maps describe this GPU's own allocation only; the copies are plain (one destination CTA).
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "elem.cuh"

namespace hmc {

constexpr int kT16Tile = 64;                              // elements along either edge of a tile
constexpr int kT16TileBytes = kT16Tile * kT16Tile * 2;    // 8 KB
constexpr int kT16Stages = 2;                             // input tiles in flight per block
constexpr int kT16Threads = 128;
constexpr int kT16Warps = kT16Threads / 32;
constexpr int kT16BlocksPerSm = 8;
constexpr int kT16Strip = 8;                              // tiles along a that consecutive tile numbers share
constexpr int kT16WaitLimit = 1 << 22;                    // polls of an mbarrier before a wait gives up
constexpr size_t kT16SharedBytes = static_cast<size_t>(kT16Stages + 1) * kT16TileBytes + 1024;  // + room to align

struct Transpose16Args {
    uint32_t tiles_a, tiles_b, tiles;  // tiles along a, along b, in all (outer * tiles_a * tiles_b < 2^31)
};

// Encodes the tensor map of a [outer][rows][cols] view of 2-byte elements with cols contiguous: boxes of
// 64 x 64 x 1 in the 128-byte swizzle. False when the layout does not qualify (alignment) or the driver refuses.
bool t16_encode_map(CUtensorMap *map, const void *base, int64_t cols, int64_t rows, int64_t outer, int64_t row_stride_elems,
                    int64_t outer_stride_elems);

__device__ __forceinline__ uint32_t t16_shared(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void t16_barrier_init(uint64_t *bar) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(t16_shared(bar)) : "memory");
}
__device__ __forceinline__ void t16_barrier_expect(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(t16_shared(bar)), "r"(bytes) : "memory");
}
// Waits for the phase with the given parity, for a bounded number of polls. False: gave up.
__device__ __forceinline__ bool t16_barrier_wait(uint64_t *bar, uint32_t parity) {
    for (int i = 0; i < kT16WaitLimit; ++i) {
        uint32_t done;
        asm volatile(
            "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
            : "=r"(done)
            : "r"(t16_shared(bar)), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
// One tile from global to shared memory; the bytes count towards `bar`.
__device__ __forceinline__ void t16_fetch(void *tile, const CUtensorMap *map, int x, int y, int z, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
            t16_shared(tile)),
        "l"(map), "r"(x), "r"(y), "r"(z), "r"(t16_shared(bar))
        : "memory");
}
// One tile from shared to global memory, as a bulk group of the issuing thread.
__device__ __forceinline__ void t16_store(const CUtensorMap *map, int x, int y, int z, const void *tile) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(map), "r"(x), "r"(y),
                 "r"(z), "r"(t16_shared(tile))
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Until at most `N` of this thread's stores still read their shared-memory source.
template <int N>
__device__ __forceinline__ void t16_stores_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void t16_stores_done() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// f on the two elements of a register.
template <class F>
__device__ __forceinline__ uint32_t t16_apply(const F &f, uint32_t w) {
    using TA = typename F::A;
    using TO = typename F::Out;
    static_assert(sizeof(TA) == 2 && sizeof(TO) == 2, "2-byte elements");
    const uint16_t lo = static_cast<uint16_t>(w & 0xFFFFu), hi = static_cast<uint16_t>(w >> 16);
    TA x0, x1;
    memcpy(&x0, &lo, 2);
    memcpy(&x1, &hi, 2);
    TO y0, y1;
    if constexpr (has_compute<F>::value && (std::is_same_v<TO, F16> || std::is_same_v<TO, BF16>)) {
        down2(y0, y1, f.compute(x0), f.compute(x1));
    } else if constexpr (has_compute<F>::value) {
        y0 = down<TO>(f.compute(x0));
        y1 = down<TO>(f.compute(x1));
    } else {
        y0 = f(x0);
        y1 = f(x1);
    }
    uint16_t r0, r1;
    memcpy(&r0, &y0, 2);
    memcpy(&r1, &y1, 2);
    return static_cast<uint32_t>(r0) | (static_cast<uint32_t>(r1) << 16);
}

// The input map's dimensions are (a, b, outer), the output map's (b, a, outer). Grid: resident blocks; block i
// takes tiles i, i + grid, ... Tile numbers run through strips of kT16Strip tiles along a: within a strip along a
// first, then along b, so that the tiles in flight at any time cover runs of a kilobyte and more on both sides
// (the input's rows run along a, the output's along b): numbered along b alone, every 128-byte row of an input tile
// would be the only piece of its DRAM page in flight.
//
// A block is small (four warps, two input tiles and one output tile, 25 KB) so that eight of them share an SM: while
// one block is between tiles (its two barriers, thread 0's store and next fetch) the others keep the special
// function unit and the copy engine busy. Measured on B200 for silu of bf16 [8192, 8192].t(): 49 us with this
// shape against 51 us with four blocks of four input and two output tiles, 52 us with blocks of 256 threads, and
// 51-61 us with one pipeline per warp or a warp set aside to fetch; the same kernel without arithmetic takes 43 us.
template <class F>
__global__ void __launch_bounds__(kT16Threads) transpose16_kernel(const __grid_constant__ CUtensorMap in_map,
                                                                   const __grid_constant__ CUtensorMap out_map,
                                                                   const Transpose16Args args, const F f, int *status) {
    extern __shared__ unsigned char t16_memory[];
    __shared__ __align__(8) uint64_t full[kT16Stages];
    __shared__ int gave_up;
    // the swizzled layout repeats every 1024 bytes: tiles start on such a boundary
    unsigned char *tiles = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(t16_memory) + 1023) & ~uintptr_t{1023});
    unsigned char *out_tile = tiles + kT16Stages * kT16TileBytes;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kT16Stages; ++s) t16_barrier_init(&full[s]);
        gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    auto coordinates = [&](uint32_t t, int &ta, int &tb, int &outer) {
        const uint32_t per_outer = args.tiles_a * args.tiles_b;
        const uint32_t o = t / per_outer, rest = t - o * per_outer;
        const uint32_t per_strip = kT16Strip * args.tiles_b;
        const uint32_t strip = rest / per_strip, in_strip = rest - strip * per_strip;
        const uint32_t left = args.tiles_a - strip * kT16Strip;
        const uint32_t width = left < kT16Strip ? left : kT16Strip;  // the last strip may be narrower
        const uint32_t b = in_strip / width;
        outer = static_cast<int>(o);
        tb = static_cast<int>(b);
        ta = static_cast<int>(strip * kT16Strip + (in_strip - b * width));
    };
    auto fetch = [&](uint32_t t, int stage) {
        int ta, tb, outer;
        coordinates(t, ta, tb, outer);
        t16_barrier_expect(&full[stage], kT16TileBytes);
        t16_fetch(tiles + stage * kT16TileBytes, &in_map, ta * kT16Tile, tb * kT16Tile, outer, &full[stage]);
    };
    if (threadIdx.x == 0) {
        uint32_t t = blockIdx.x;
        for (int s = 0; s < kT16Stages && t < args.tiles; ++s, t += gridDim.x) fetch(t, s);
    }
    int stage = 0;
    uint32_t parity = 0;
    for (uint32_t t = blockIdx.x; t < args.tiles; t += gridDim.x) {
        if (!t16_barrier_wait(&full[stage], parity)) gave_up = 1;
        // the previous tile's store has finished reading the output tile
        if (threadIdx.x == 0) t16_stores_read<0>();
        __syncthreads();
        if (gave_up) {  // (every thread sees the same value: nobody writes it between this barrier and the next)
            if (threadIdx.x == 0) atomicExch(status, 1);
            break;
        }
        const unsigned char *in_tile = tiles + stage * kT16TileBytes;
        // a warp takes the 8 x 32 pieces (a-block ia, b-group jb) number warp, warp + 4, ... of the sixteen
#pragma unroll
        for (int piece = 0; piece < 16 / kT16Warps; ++piece) {
            const int id = piece * kT16Warps + warp;
            const int ia = id >> 1, jb = id & 1;
            // lane l names row b = jb * 32 + l of the input tile, the 16-byte chunk ia of it (swizzled by the row)
            const int row_in = jb * 32 + lane;
            const uint32_t from = t16_shared(in_tile + row_in * 128 + ((ia ^ (row_in & 7)) << 4));
            uint32_t d0, d1, d2, d3;
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                         : "=r"(d0), "=r"(d1), "=r"(d2), "=r"(d3)
                         : "r"(from)
                         : "memory");
            d0 = t16_apply(f, d0);
            d1 = t16_apply(f, d1);
            d2 = t16_apply(f, d2);
            d3 = t16_apply(f, d3);
            // lane l names row a = ia * 8 + (l % 8) of the output tile, chunk jb * 4 + l / 8 of it
            const int row_out = ia * 8 + (lane & 7);
            const uint32_t to = t16_shared(out_tile + row_out * 128 + (((jb * 4 + (lane >> 3)) ^ (row_out & 7)) << 4));
            asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};" ::"r"(to), "r"(d0), "r"(d1), "r"(d2), "r"(d3)
                         : "memory");
        }
        // the output tile is complete and visible to the copy engine; the input stage is free
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        if (threadIdx.x == 0) {
            int ta, tb, outer;
            coordinates(t, ta, tb, outer);
            t16_store(&out_map, tb * kT16Tile, ta * kT16Tile, outer, out_tile);
            const uint64_t next = t + static_cast<uint64_t>(kT16Stages) * gridDim.x;
            if (next < args.tiles) fetch(static_cast<uint32_t>(next), stage);
        }
        if (++stage == kT16Stages) {
            stage = 0;
            parity ^= 1;
        }
    }
    if (threadIdx.x == 0) t16_stores_done();
}

// ---- the same for functions of three operands of which the first is the transposed one ----
// out[.., a, b] = f(x[.., b, a], B[.., a, b], C[.., a, b]) for a 2-byte x that has its unit stride along a; B and C are
// addressed by their strides in the output's orientation (a bias per row, a scale per column, whole tensors), the
// output may be of any size (the fused chain's f32 result). The input side is the kernel above; the output side
// needs no tile: after ldmatrix.trans a lane holds pairs of elements that are neighbours along b, which it combines with
// its B and C values and stores straight to global memory, eight lanes filling a 32-byte sector of a 4-byte output.
struct Transpose16Operand {
    const void *base;
    int64_t stride_a, stride_b, stride_outer;  // elements
};
struct Transpose16Args3 {
    uint32_t tiles_a, tiles_b, tiles;
    int64_t size_a, size_b;
    void *out;
    int64_t out_stride_a, out_stride_outer;    // elements; the output has unit stride along b
    Transpose16Operand b, c;
};

template <class F>
__global__ void __launch_bounds__(kT16Threads) transpose16_three_kernel(const __grid_constant__ CUtensorMap in_map,
                                                                         const __grid_constant__ Transpose16Args3 args, const F f,
                                                                         int *status) {
    using TX = typename F::A;
    using TB = typename F::B;
    using TC = typename F::C;
    using TO = typename F::Out;
    static_assert(sizeof(TX) == 2, "a 2-byte first operand");
    extern __shared__ unsigned char t16_memory[];
    __shared__ __align__(8) uint64_t full[kT16Stages];
    __shared__ int gave_up;
    unsigned char *tiles = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(t16_memory) + 1023) & ~uintptr_t{1023});
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kT16Stages; ++s) t16_barrier_init(&full[s]);
        gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    auto coordinates = [&](uint32_t t, int &ta, int &tb, int &outer) {
        const uint32_t per_outer = args.tiles_a * args.tiles_b;
        const uint32_t o = t / per_outer, rest = t - o * per_outer;
        const uint32_t per_strip = kT16Strip * args.tiles_b;
        const uint32_t strip = rest / per_strip, in_strip = rest - strip * per_strip;
        const uint32_t left = args.tiles_a - strip * kT16Strip;
        const uint32_t width = left < kT16Strip ? left : kT16Strip;
        const uint32_t b = in_strip / width;
        outer = static_cast<int>(o);
        tb = static_cast<int>(b);
        ta = static_cast<int>(strip * kT16Strip + (in_strip - b * width));
    };
    auto fetch = [&](uint32_t t, int stage) {
        int ta, tb, outer;
        coordinates(t, ta, tb, outer);
        t16_barrier_expect(&full[stage], kT16TileBytes);
        t16_fetch(tiles + stage * kT16TileBytes, &in_map, ta * kT16Tile, tb * kT16Tile, outer, &full[stage]);
    };
    if (threadIdx.x == 0) {
        uint32_t t = blockIdx.x;
        for (int s = 0; s < kT16Stages && t < args.tiles; ++s, t += gridDim.x) fetch(t, s);
    }
    const TB *pb = static_cast<const TB *>(args.b.base);
    const TC *pc = static_cast<const TC *>(args.c.base);
    TO *po = static_cast<TO *>(args.out);
    const bool pairs_aligned = (reinterpret_cast<uintptr_t>(po) % (2 * sizeof(TO))) == 0 && args.out_stride_a % 2 == 0 &&
                               args.out_stride_outer % 2 == 0;
    int stage = 0;
    uint32_t parity = 0;
    for (uint32_t t = blockIdx.x; t < args.tiles; t += gridDim.x) {
        if (!t16_barrier_wait(&full[stage], parity)) gave_up = 1;
        __syncthreads();
        if (gave_up) {
            if (threadIdx.x == 0) atomicExch(status, 1);
            break;
        }
        int ta, tb, outer;
        coordinates(t, ta, tb, outer);
        const unsigned char *in_tile = tiles + stage * kT16TileBytes;
#pragma unroll
        for (int piece = 0; piece < 16 / kT16Warps; ++piece) {
            const int id = piece * kT16Warps + warp;
            const int ia = id >> 1, jb = id & 1;
            const int row_in = jb * 32 + lane;
            const uint32_t from = t16_shared(in_tile + row_in * 128 + ((ia ^ (row_in & 7)) << 4));
            uint32_t d[4];
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                         : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                         : "r"(from)
                         : "memory");
            // this lane's output row, and the first of its two columns in each of the four 8 x 8 blocks; positions
            // beyond the edges are clamped for the loads (which then need no branches and all go out together)
            // and skipped by the stores
            // (sizes are below 2^31 here: the tiles are counted in 32 bits)
            const int ra = ta * kT16Tile + ia * 8 + (lane >> 2);
            const int cb = tb * kT16Tile + jb * 32 + 2 * (lane & 3);
            const int size_a = static_cast<int>(args.size_a), size_b = static_cast<int>(args.size_b);
            const int ra_safe = ra < size_a ? ra : size_a - 1;
            const TB *b_row = pb + outer * args.b.stride_outer + ra_safe * args.b.stride_a;
            const TC *c_row = pc + outer * args.c.stride_outer + ra_safe * args.c.stride_a;
            TB bv[4][2];
            TC cv[4][2];
            // an operand that does not change along b (a value per output row) is read once
            if (args.b.stride_b == 0) {
                const TB v = b_row[0];
#pragma unroll
                for (int m = 0; m < 4; ++m) bv[m][0] = bv[m][1] = v;
            } else {
#pragma unroll
                for (int m = 0; m < 4; ++m) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int col = cb + 8 * m + e;
                        bv[m][e] = b_row[static_cast<int64_t>(col < size_b ? col : size_b - 1) * args.b.stride_b];
                    }
                }
            }
            if (args.c.stride_b == 0) {
                const TC v = c_row[0];
#pragma unroll
                for (int m = 0; m < 4; ++m) cv[m][0] = cv[m][1] = v;
            } else {
#pragma unroll
                for (int m = 0; m < 4; ++m) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int col = cb + 8 * m + e;
                        cv[m][e] = c_row[static_cast<int64_t>(col < size_b ? col : size_b - 1) * args.c.stride_b];
                    }
                }
            }
            TO *out_row = po + outer * args.out_stride_outer + ra_safe * args.out_stride_a;
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                const int col = cb + 8 * m;
                const uint16_t lo = static_cast<uint16_t>(d[m] & 0xFFFFu), hi = static_cast<uint16_t>(d[m] >> 16);
                TX x0, x1;
                memcpy(&x0, &lo, 2);
                memcpy(&x1, &hi, 2);
                TO y0, y1;
                if constexpr (std::is_same_v<TO, F16> || std::is_same_v<TO, BF16>) {
                    down2(y0, y1, f.compute(x0, bv[m][0], cv[m][0]), f.compute(x1, bv[m][1], cv[m][1]));
                } else {
                    y0 = down<TO>(f.compute(x0, bv[m][0], cv[m][0]));
                    y1 = down<TO>(f.compute(x1, bv[m][1], cv[m][1]));
                }
                if (ra < size_a && col < size_b) {
                    const bool second = col + 1 < size_b;
                    if (second && pairs_aligned) {
                        Pack<TO, 2> pair;
                        pair.v[0] = y0;
                        pair.v[1] = y1;
                        *reinterpret_cast<Pack<TO, 2> *>(out_row + col) = pair;
                    } else {
                        out_row[col] = y0;
                        if (second) out_row[col + 1] = y1;
                    }
                }
            }
        }
        __syncthreads();  // everybody has read the input tile
        if (threadIdx.x == 0) {
            const uint64_t next = t + static_cast<uint64_t>(kT16Stages) * gridDim.x;
            if (next < args.tiles) fetch(static_cast<uint32_t>(next), stage);
        }
        if (++stage == kT16Stages) {
            stage = 0;
            parity ^= 1;
        }
    }
}

}  // namespace hmc
