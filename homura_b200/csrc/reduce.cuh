// The reduction engine: plans, kernels and launch helpers shared by sum, prod, mean, max, min,
// all, any, var/std and the arg reductions.
//
// A reduction is given as `kept` (kept dimensions with the source's strides, data, offset, dtype)
// and `red` (reduced dimensions with the source's strides); output o (row-major over the kept
// sizes) folds the reduced elements j = 0..nred-1 (row-major over the reduced sizes).
//
// Two kernels cover every layout, chosen from sizes and strides alone (never from the device or
// the data's address), so a given reduction always folds in the same order:
//
//  * rows (kind 0): the reduced elements of an output are a sequence of runs along the last reduced
//    dimension. An output (or one chunk of its reduced range) belongs to a team of G = 1, 32 or 256
//    lanes; a run is cut into pieces of 32 bytes, piece w goes to lane w mod G, and a lane folds its
//    pieces in order, run after run. Unit-stride runs that start on a 32-byte boundary are read with
//    256-bit loads, four in flight per lane; any other run is read element by element under the same
//    assignment, hence with the same result bits. The lanes of a team are folded by shuffles in lane
//    order and, for 256 lanes, the warps through shared memory in warp order. The grid is one block
//    per 256 / G outputs and chunk, all launched at once: on B200 a read-only sweep by many short
//    blocks measured 5 % faster than the same sweep by a resident grid that loops.
//  * columns (kind 1): the outputs are adjacent in memory (the last kept dimension has stride 1)
//    and the reduced elements are strided. A block is 32 x 8 threads; a thread owns VC adjacent
//    outputs (one 16-byte load per reduced index), the 8 warps take reduced indices j, j+8, ...,
//    and are combined in warp order through shared memory. Global loads are fully coalesced.
//
// When the outputs alone cannot fill the GPU, the reduced range is cut into `splits` chunks; each
// chunk writes a partial per output into the caller's workspace (slots of 16 bytes are reserved) and the
// partials of an output are folded in an order that depends on the plan alone. Who folds them: the block
// that finishes last among those sharing blockIdx.x (each takes a ticket from a counter of the context
// when its partials are written; the one that draws the last ticket resets the counter and folds), so that
// no second launch is paid; or, when a block would have too many partials to fold by itself or there are
// more blocks along x than counters, a second kernel. Both fold in the same order.
//
// Accumulators follow homura's CPU fold (src/backend/cpu/reduce.rs:42-131): floats in f64,
// integers wrapping in i64, extremes as (value, index) with "first NaN, then first of equals".
#pragma once

#include "common.cuh"
#include "elem.cuh"

namespace hmc {

constexpr int kRThreads = 256;
constexpr int64_t kTargetLanes = 148 * 2048;  // fixed, so that plans do not depend on the device
// The column kernel's blocks: enough of them for every SM several times over (blocks that read a few hundred KB
// each and all start at once measured a third faster than one resident wave), each reading at least this much.
constexpr int64_t kTargetColumnBlocks = 148 * 8;
constexpr int64_t kColumnBlockBytes = 256 * 1024;
constexpr int64_t kMaxSplits = 4096;
constexpr int64_t kWarpRowOutputs = 148 * 32;  // outputs from which a long row is folded by a warp
constexpr int64_t kWarpRowLength = 1 << 16;    // and the longest such row
constexpr int64_t kPartialBytes = 16;

struct ReducePlan {
    int32_t kind;    // 0 rows, 1 columns
    int32_t group;   // lanes per team (kind 0)
    int32_t vec;     // elements per 32-byte piece of the source dtype (kind 0)
    int32_t vc;      // outputs per thread (kind 1)
    int64_t nout, nred;
    int64_t row, step;  // last reduced dimension: size and source stride
    int64_t splits, chunk;
    int64_t ncols, kouter, xtiles;  // kind 1: last kept size, product of the others, column tiles
    // kind 0, no chunks, and every output folds one unit-stride run of whole 32-byte pieces (nred < 2^31): what the
    // one-pass variance kernel for rows requires.
    int32_t simple;
};

struct ReduceArgs {
    hmc_tensor_desc kept;
    hmc_tensor_desc red;
    ReducePlan plan;
    void *partials;
    unsigned *tickets;  // the context's counters (kTickets of them, all zero between kernels), or null
};

inline int64_t desc_count(const hmc_tensor_desc &d) {
    int64_t n = 1;
    for (int k = 0; k < d.ndim; ++k) n *= d.sizes[k];
    return n;
}

ReducePlan make_reduce_plan(const hmc_tensor_desc &kept, const hmc_tensor_desc &red);
// Validation shared by every reduction entry point: both descriptions are well formed, agree in dtype, and neither
// the number of outputs nor the number of reduced elements overflows 64 bits.
hmc_status check_reduction(const hmc_tensor_desc *kept, const hmc_tensor_desc *red);
// `out` is a contiguous description of `nout` elements with a data pointer.
hmc_status check_output(const hmc_tensor_desc *out, const hmc_tensor_desc *kept, const char *what, int64_t nout);

inline int64_t plan_partial_bytes(const ReducePlan &p) { return p.splits > 1 ? p.splits * p.nout * kPartialBytes : 0; }

// ---- device helpers ----
__device__ __forceinline__ int64_t decompose(const hmc_tensor_desc &d, int64_t idx, int ndim) {
    int64_t off = 0;
    for (int k = ndim - 1; k > 0; --k) {
        int64_t size = d.sizes[k];
        int64_t q = idx / size;
        off += (idx - q * size) * d.strides[k];
        idx = q;
    }
    if (ndim > 0) off += idx * d.strides[0];
    return off;
}

template <class Acc>
__device__ __forceinline__ Acc shuffle_down(Acc v, int delta) {
    static_assert(sizeof(Acc) == 4 || sizeof(Acc) == 8 || sizeof(Acc) == 16, "accumulator size");
    if constexpr (sizeof(Acc) == 4) {
        uint32_t w;
        memcpy(&w, &v, 4);
        w = __shfl_down_sync(0xFFFFFFFFu, w, delta);
        memcpy(&v, &w, 4);
    } else if constexpr (sizeof(Acc) == 8) {
        uint64_t w;
        memcpy(&w, &v, 8);
        w = __shfl_down_sync(0xFFFFFFFFu, w, delta);
        memcpy(&v, &w, 8);
    } else {
        uint64_t w[2];
        memcpy(w, &v, 16);
        w[0] = __shfl_down_sync(0xFFFFFFFFu, w[0], delta);
        w[1] = __shfl_down_sync(0xFFFFFFFFu, w[1], delta);
        memcpy(&v, w, 16);
    }
    return v;
}

// ---- a thread's own ring of 16-byte slots in shared memory, filled by asynchronous copies ----
// A thread only reads the slots it copied itself, so waiting for its own copy groups is all the synchronisation
// there is; the data in flight occupies no registers.
__device__ __forceinline__ void ring_copy_16(void *shared_dst, const void *global_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(shared_dst))),
                 "l"(global_src)
                 : "memory");
}
__device__ __forceinline__ void ring_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Until at most N of this thread's copy groups are still in flight.
template <int N>
__device__ __forceinline__ void ring_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ---- partials ----
// A partial that another block wrote, read past this SM's L1.
template <class Acc>
__device__ __forceinline__ Acc load_partial(const Acc *p) {
    static_assert(sizeof(Acc) == 4 || sizeof(Acc) == 8 || sizeof(Acc) == 16, "accumulator size");
    Acc v;
    if constexpr (sizeof(Acc) == 4) {
        const unsigned w = __ldcg(reinterpret_cast<const unsigned *>(p));
        memcpy(&v, &w, 4);
    } else if constexpr (sizeof(Acc) == 8) {
        const unsigned long long w = __ldcg(reinterpret_cast<const unsigned long long *>(p));
        memcpy(&v, &w, 8);
    } else {
        const ulonglong2 w = __ldcg(reinterpret_cast<const ulonglong2 *>(p));
        memcpy(&v, &w, 16);
    }
    return v;
}

// Called by every thread of a block once the block's partials are stored: true in the block that is the last of
// the gridDim.y blocks sharing blockIdx.x to get here, which may then read all their partials. (No block waits
// for another: a block that is not the last simply leaves.)
__device__ __forceinline__ bool drew_last_ticket(unsigned *tickets) {
    __shared__ bool last;
    __threadfence();  // this thread's partials are visible to the device ...
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();  // ... and so are the whole block's, before its ticket is drawn
        const unsigned mine = atomicAdd(&tickets[blockIdx.x], 1u);
        last = mine + 1 == gridDim.y;
        if (last) tickets[blockIdx.x] = 0;  // everybody has drawn: ready for the next kernel
    }
    __syncthreads();
    const bool result = last;
    if (result) __threadfence();
    return result;
}

// The partials of output o folded in chunk order by one thread, eight loads in flight.
template <class Op>
__device__ __forceinline__ typename Op::Acc fold_partials_in_order(const Op &op, const typename Op::Acc *partials, int64_t o,
                                                                   int64_t nout, int64_t splits) {
    using Acc = typename Op::Acc;
    Acc acc = op.init();
    for (int64_t c0 = 0; c0 < splits; c0 += 8) {
        Acc x[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (c0 + u < splits) x[u] = load_partial(partials + (c0 + u) * nout + o);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (c0 + u < splits) acc = op.combine(acc, x[u]);
        }
    }
    return acc;
}

// ---- teams ----
// The accumulators of a team's G lanes folded in lane order; the result is valid in the team's lane 0. Every
// thread of the block calls it (256-lane teams meet at block barriers).
template <int G, class Op>
__device__ __forceinline__ typename Op::Acc fold_team(const Op &op, typename Op::Acc acc) {
    using Acc = typename Op::Acc;
    if constexpr (G == 1) {
        return acc;
    } else {
        // lane l takes lane l + d: after the last step the team's lane 0 holds its lanes in order (teams of
        // fewer than 32 lanes are aligned groups of a warp's lanes)
#pragma unroll
        for (int d = 1; d < (G < 32 ? G : 32); d <<= 1) {
            const Acc later = shuffle_down(acc, d);
            acc = op.combine(acc, later);
        }
        if constexpr (G == 256) {
            __shared__ Acc of_warp[kRThreads / 32];
            const int warp = threadIdx.x >> 5;
            if ((threadIdx.x & 31) == 0) of_warp[warp] = acc;
            __syncthreads();
            if (threadIdx.x == 0) {
#pragma unroll
                for (int w = 1; w < kRThreads / 32; ++w) acc = op.combine(acc, of_warp[w]);
            }
            __syncthreads();
        }
        return acc;
    }
}

// (value, index); index < 0 marks the empty fold. src/backend/cpu/reduce.rs:75-86.
template <class TT>
struct alignas(16) Best {
    TT v;
    int64_t i;
};

template <class T> __device__ __forceinline__ auto order_key(T x) {
    if constexpr (std::is_same_v<T, F16> || std::is_same_v<T, BF16>) return up(x);
    else if constexpr (std::is_same_v<T, Bool>) return x.b;
    else return x;
}

template <class TT, bool MAX> struct Extreme;
template <class Op> struct is_extreme : std::false_type {};
template <class TT, bool MAX> struct is_extreme<Extreme<TT, MAX>> : std::true_type {};
template <class Op> struct extreme_is_max : std::false_type {};
template <class TT> struct extreme_is_max<Extreme<TT, true>> : std::true_type {};

// acc folded with element x (index j of output o), where j is larger than every index already in acc: what a
// lane does element by element. Ops may give a cheaper form of it than combine(acc, load(x)).
template <class Op, class = void> struct has_step : std::false_type {};
template <class Op> struct has_step<Op, std::void_t<decltype(&Op::step)>> : std::true_type {};
template <class Op>
__device__ __forceinline__ typename Op::Acc fold_step(const Op &op, typename Op::Acc acc, typename Op::T x, int64_t o, int64_t j) {
    if constexpr (has_step<Op>::value) return op.step(acc, x, j);
    else return op.combine(acc, op.load(x, o, j));
}

// An op with what it needs of output o already in registers; ops without per-output state are returned as is.
template <class Op, class = void> struct has_bound : std::false_type {};
template <class Op> struct has_bound<Op, std::void_t<decltype(&Op::bound)>> : std::true_type {};
template <class Op>
__device__ __forceinline__ Op bind_output(const Op &op, int64_t o) {
    if constexpr (has_bound<Op>::value) return op.bound(o);
    else return op;
}

template <class T, int VEC>
struct alignas(sizeof(T) * VEC >= 16 ? 16 : sizeof(T) * VEC) RVec {
    T v[VEC];
};

// ---- rows ----
// A piece: 32 bytes of a run, read with one 256-bit load.
template <class T>
struct alignas(32) Piece {
    static constexpr int N = 32 / static_cast<int>(sizeof(T));
    T v[N];
};
template <class T>
__device__ __forceinline__ Piece<T> load_piece(const T *p) {
    uint32_t w[8];
    // (not volatile: the compiler may schedule it like any other load)
    asm("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
        : "=r"(w[0]), "=r"(w[1]), "=r"(w[2]), "=r"(w[3]), "=r"(w[4]), "=r"(w[5]), "=r"(w[6]), "=r"(w[7])
        : "l"(p));
    Piece<T> out;
    memcpy(&out, w, 32);
    return out;
}

// A batch of pieces folded into `acc`; `at[u]` is the reduced index of piece u's first element.
template <int U, class Op>
__device__ __forceinline__ void fold_batch(const Op &op, typename Op::Acc &acc, const Piece<typename Op::T> (&x)[U],
                                           const int64_t (&at)[U], int64_t o) {
    constexpr int N = Piece<typename Op::T>::N;
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
        for (int e = 0; e < N; ++e) acc = fold_step(op, acc, x[u].v[e], o, at[u] + e);
    }
}

// One lane's share of the elements [lo, hi) of a run: the run's element i lies at p[i * step] and has the reduced
// index first + i; piece w = elements [w N, (w + 1) N) belongs to lane w mod G.
template <int G, class Op>
__device__ __forceinline__ void fold_run(const Op &op, typename Op::Acc &acc, const typename Op::T *p, int64_t step, int64_t lo,
                                         int64_t hi, int64_t first, int lane, int64_t o) {
    using T = typename Op::T;
    constexpr int N = Piece<T>::N;
    constexpr int U = 4;
    const int64_t w_lo = lo / N, w_whole = hi / N, w_end = (hi + N - 1) / N;
    // the lane's first piece at or after w_lo
    int64_t w = w_lo + ((lane - w_lo % G) + G) % G;
    auto ragged = [&](int64_t piece) {
        for (int e = 0; e < N; ++e) {
            const int64_t i = piece * N + e;
            if (i >= lo && i < hi) acc = fold_step(op, acc, p[i * step], o, first + i);
        }
    };
    if (w == w_lo && w * N < lo && w < w_end) {  // the range starts inside this piece
        ragged(w);
        w += G;
    }
    if (step == 1 && (reinterpret_cast<uintptr_t>(p) & 31) == 0) {
        if constexpr (is_extreme<Op>::value) {
            // max / min: the general step (first NaN, then first of equals, a 64-bit index) costs about forty
            // instructions an element. Here the lane keeps the best key, its value and place by plain comparisons over
            // all its whole pieces of the run (a later element wins only if strictly better, so the first of equals
            // stays) and folds that once. NaNs are not handled but detected (the sum of the keys is NaN if one of
            // them is; an infinity minus infinity raises a false alarm, which is harmless): the lane then folds the
            // same pieces again with the general step.
            if (w < w_whole) {
                constexpr bool kMax = extreme_is_max<Op>::value;
                const int64_t w_first = w;
                T best = p[w * N];
                auto best_key = order_key(best);
                uint32_t best_at = 0;  // the element's place among those this lane takes: piece count * N + e
                uint32_t count = 0;
                float alarm = 0.0f;
                auto take = [&](const Piece<T> &x) {
                    if constexpr (Tr<T>::kind == kFloat) {
                        float sum = static_cast<float>(order_key(x.v[0]));
#pragma unroll
                        for (int e = 1; e < N; ++e) sum += static_cast<float>(order_key(x.v[e]));
                        alarm += sum;
                    }
#pragma unroll
                    for (int e = 0; e < N; ++e) {
                        const auto k = order_key(x.v[e]);
                        const bool better = kMax ? k > best_key : k < best_key;
                        best_key = better ? k : best_key;
                        best = better ? x.v[e] : best;
                        best_at = better ? count + e : best_at;
                    }
                    count += N;
                };
                // (a lane takes fewer than 2^32 elements of a run: longer runs fall back to the general step below)
                if ((w_whole - w_first) / G < (int64_t{1} << 31) / N) {
                    for (; w + (U - 1) * G < w_whole; w += U * G) {
                        Piece<T> x[U];
#pragma unroll
                        for (int u = 0; u < U; ++u) x[u] = load_piece(p + (w + u * G) * N);
#pragma unroll
                        for (int u = 0; u < U; ++u) take(x[u]);
                    }
                    for (; w < w_whole; w += G) take(load_piece(p + w * N));
                    if (alarm == alarm) {
                        const int64_t piece = w_first + static_cast<int64_t>(best_at / N) * G;
                        acc = op.combine(acc, typename Op::Acc{best, first + piece * N + best_at % N});
                    } else {
                        for (int64_t v = w_first; v < w_whole; v += G) {
                            const Piece<T> x = load_piece(p + v * N);
#pragma unroll
                            for (int e = 0; e < N; ++e) acc = fold_step(op, acc, x.v[e], o, first + v * N + e);
                        }
                    }
                }
            }
        }
        for (; w + (U - 1) * G < w_whole; w += U * G) {
            Piece<T> x[U];
            int64_t at[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                at[u] = first + (w + u * G) * N;
                x[u] = load_piece(p + (w + u * G) * N);
            }
            fold_batch<U>(op, acc, x, at, o);
        }
        for (; w < w_whole; w += G) {
            const Piece<T> x[1] = {load_piece(p + w * N)};
            const int64_t at[1] = {first + w * N};
            fold_batch<1>(op, acc, x, at, o);
        }
    } else {
        for (; w < w_whole; w += G) {
#pragma unroll
            for (int e = 0; e < N; ++e) acc = fold_step(op, acc, p[(w * N + e) * step], o, first + w * N + e);
        }
    }
    if (w < w_end) ragged(w);  // the range ends inside this piece (w == w_whole)
}

// One lane's share of the reduced elements [j0, j1) of output o, whose first element lies at `base`: the runs
// that the range touches, in order.
template <int G, class Op>
__device__ __forceinline__ typename Op::Acc fold_span(const Op &op, const ReduceArgs &a, int64_t o, int64_t base, int64_t j0,
                                                      int64_t j1, int lane) {
    using T = typename Op::T;
    typename Op::Acc acc = op.init();
    if (j1 <= j0) return acc;
    const T *src = static_cast<const T *>(a.kept.data) + base;
    const int64_t row = a.plan.row, step = a.plan.step;
    if (a.red.ndim <= 1) {
        fold_run<G>(op, acc, src, step, j0, j1, 0, lane, o);
        return acc;
    }
    const int64_t q_first = j0 / row, q_last = (j1 - 1) / row;
    for (int64_t q = q_first; q <= q_last; ++q) {
        const int64_t first = q * row;
        const int64_t lo = q == q_first ? j0 - first : 0;
        const int64_t hi = q == q_last ? j1 - first : row;
        fold_run<G>(op, acc, src + decompose(a.red, q, a.red.ndim - 1), step, lo, hi, first, lane, o);
    }
    return acc;
}

// A lane's share of the partials of output o: chunks lane, lane + G, ... in order (a single lane: all, in order).
template <int G, class Op>
__device__ __forceinline__ typename Op::Acc team_partials(const Op &op, const typename Op::Acc *partials, int64_t o, bool live,
                                                          int lane, const ReducePlan &p) {
    using Acc = typename Op::Acc;
    if constexpr (G == 1) {
        return live ? fold_partials_in_order(op, partials, o, p.nout, p.splits) : op.init();
    } else {
        Acc acc = op.init();
        if (live) {
            int64_t c = lane;
            for (; c + 3 * G < p.splits; c += 4 * G) {
                Acc x[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) x[u] = load_partial(partials + (c + u * G) * p.nout + o);
#pragma unroll
                for (int u = 0; u < 4; ++u) acc = op.combine(acc, x[u]);
            }
            for (; c < p.splits; c += G) acc = op.combine(acc, load_partial(partials + c * p.nout + o));
        }
        return acc;
    }
}

// kind 0. Grid: (teams of outputs, chunks), every block launched at once: block (x, y) folds chunk y of the
// 256 / G outputs x * (256 / G) ... (Four blocks share an SM; max / min, whose lanes carry a candidate beside
// the loads in flight, get the registers of two.)
template <int G, class Op, class Sink>
__global__ void __launch_bounds__(kRThreads, is_extreme<Op>::value ? 3 : 4) reduce_rows_kernel(const __grid_constant__ ReduceArgs a, const Op op, const Sink sink) {
    using Acc = typename Op::Acc;
    constexpr int kTeams = kRThreads / G;
    const ReducePlan &p = a.plan;
    const int lane = threadIdx.x % G;
    const int64_t o = static_cast<int64_t>(blockIdx.x) * kTeams + threadIdx.x / G;
    const int64_t chunk = blockIdx.y;
    const bool live = o < p.nout;
    Acc acc = op.init();
    if (live) {
        const int64_t j0 = chunk * p.chunk;
        const int64_t j1 = j0 + p.chunk < p.nred ? j0 + p.chunk : p.nred;
        acc = fold_span<G>(op, a, o, a.kept.offset + decompose(a.kept, o, a.kept.ndim), j0, j1, lane);
    }
    acc = fold_team<G>(op, acc);
    if (p.splits == 1) {
        if (lane == 0 && live) sink.put(o, acc, p.nred);
        return;
    }
    Acc *partials = static_cast<Acc *>(a.partials);
    if (lane == 0 && live) partials[chunk * p.nout + o] = acc;
    if (a.tickets == nullptr || !drew_last_ticket(a.tickets)) return;
    acc = fold_team<G>(op, team_partials<G>(op, partials, o, live, lane, p));
    if (lane == 0 && live) sink.put(o, acc, p.nred);
}

// The partials of a strip of W outputs (W = 64, 128 or 256) folded by one block: thread t takes output t % W and, of
// its chunks, every (256 / W)-th starting with chunk t / W, in order, with all its loads (or sixteen at a time)
// in flight at once; the threads of an output are then folded in that order. A warp reads 32 neighbouring outputs
// of one chunk, whole sectors. (A block that walked through its outputs a few at a time, one round trip to the L2
// after another, took 7 us for 128 outputs of 32 chunks; this takes under 2.)
template <int W, class Op>
__device__ __forceinline__ typename Op::Acc strip_share(const Op &op, const typename Op::Acc *partials, int64_t o, bool live,
                                                        int h, const ReducePlan &p) {
    using Acc = typename Op::Acc;
    constexpr int H = kRThreads / W;
    constexpr int B = sizeof(Acc) > 8 ? 8 : 16;
    Acc acc = op.init();
    if (live) {
        for (int64_t c0 = h; c0 < p.splits; c0 += static_cast<int64_t>(B) * H) {
            Acc x[B];
#pragma unroll
            for (int u = 0; u < B; ++u) {
                if (c0 + u * H < p.splits) x[u] = load_partial(partials + (c0 + u * H) * p.nout + o);
            }
#pragma unroll
            for (int u = 0; u < B; ++u) {
                if (c0 + u * H < p.splits) acc = op.combine(acc, x[u]);
            }
        }
    }
    return acc;
}

// kind 1. Grid: (kouter * xtiles, splits), every block launched at once; block 32 x 8: thread (tx, ty) owns the VC
// adjacent outputs tx * VC .. of its strip of 32 * VC outputs and folds the reduced indices j0 + ty, j0 + ty + 8, ...
// of its chunk; the eight warps are then folded in warp order through shared memory.
template <class Op, class Sink>
__global__ void __launch_bounds__(kRThreads, is_extreme<Op>::value ? 2 : 4) reduce_columns_kernel(const __grid_constant__ ReduceArgs a, const Op op,
                                                                   const Sink sink) {
    using T = typename Op::T;
    using Acc = typename Op::Acc;
    constexpr int VC = (16 / sizeof(T)) > 8 ? 8 : (16 / sizeof(T));
    constexpr int UNR = 8;  // loads in flight per thread
    const ReducePlan &p = a.plan;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t chunk = blockIdx.y;
    const int64_t j0 = chunk * p.chunk;
    const int64_t j1 = j0 + p.chunk < p.nred ? j0 + p.chunk : p.nred;
    const int last = a.kept.ndim - 1;
    __shared__ Acc stage[7][32 * VC];
    const int64_t outer = blockIdx.x / p.xtiles;
    const int64_t tile = blockIdx.x - outer * p.xtiles;
    const int64_t c0 = tile * (32 * VC) + static_cast<int64_t>(tx) * VC;
    // Offset of the outer kept index; the column index adds c (stride 1).
    const int64_t base = a.kept.offset + (last > 0 ? decompose(a.kept, outer, last) : 0);
    const int64_t o0 = outer * p.ncols + c0;
    const T *src = static_cast<const T *>(a.kept.data) + base + c0;
    Acc acc[VC];
#pragma unroll
    for (int e = 0; e < VC; ++e) acc[e] = op.init();
    // what the op needs to know about an output (its mean, for the squared deviations) is fetched once
    Op ops[VC];
#pragma unroll
    for (int e = 0; e < VC; ++e) ops[e] = bind_output(op, c0 + e < p.ncols ? o0 + e : 0);
    const bool in_range = c0 < p.ncols;
    const bool whole = c0 + VC <= p.ncols;
    if (in_range) {
        const int64_t stride = a.red.strides[0];
        const bool walk = a.red.ndim == 1 && whole && (reinterpret_cast<uintptr_t>(src) & (alignof(RVec<T, VC>) - 1)) == 0 &&
                          (stride * static_cast<int64_t>(sizeof(T))) % static_cast<int64_t>(alignof(RVec<T, VC>)) == 0;
        if (walk) {
            // one reduced dimension, whole aligned vectors: a pointer that steps by eight rows
            const T *q = src + (j0 + ty) * stride;
            const int64_t step = 8 * stride;
            int64_t j = j0 + ty;
            for (; j + (UNR - 1) * 8 < j1; j += UNR * 8, q += UNR * step) {
                RVec<T, VC> x[UNR];
#pragma unroll
                for (int u = 0; u < UNR; ++u) x[u] = *reinterpret_cast<const RVec<T, VC> *>(q + u * step);
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
#pragma unroll
                    for (int e = 0; e < VC; ++e) acc[e] = fold_step(ops[e], acc[e], x[u].v[e], o0 + e, j + u * 8);
                }
            }
            for (; j < j1; j += 8, q += step) {
                const RVec<T, VC> x = *reinterpret_cast<const RVec<T, VC> *>(q);
#pragma unroll
                for (int e = 0; e < VC; ++e) acc[e] = fold_step(ops[e], acc[e], x.v[e], o0 + e, j);
            }
        } else {
            const bool single = a.red.ndim == 1;
            for (int64_t j = j0 + ty; j < j1; j += 8) {
                const T *q = src + (single ? j * stride : decompose(a.red, j, a.red.ndim));
#pragma unroll
                for (int e = 0; e < VC; ++e) {
                    if (c0 + e < p.ncols) acc[e] = fold_step(ops[e], acc[e], q[e], o0 + e, j);
                }
            }
        }
    }
    if (ty > 0) {
#pragma unroll
        for (int e = 0; e < VC; ++e) stage[ty - 1][tx * VC + e] = acc[e];
    }
    __syncthreads();
    Acc *partials = static_cast<Acc *>(a.partials);
    if (ty == 0 && in_range) {
#pragma unroll
        for (int e = 0; e < VC; ++e) {
            if (c0 + e >= p.ncols) continue;
            Acc r = acc[e];
            for (int w = 0; w < 7; ++w) r = op.combine(r, stage[w][tx * VC + e]);
            if (p.splits == 1) sink.put(o0 + e, r, p.nred);
            else partials[chunk * p.nout + o0 + e] = r;
        }
    }
    if (p.splits == 1 || a.tickets == nullptr || !drew_last_ticket(a.tickets)) return;
    // the strip's outputs (the warps' staging area is free again: every thread passed the ticket's barriers)
    constexpr int W = 32 * VC, H = kRThreads / W;
    const int w = threadIdx.x % W, h = threadIdx.x / W;
    const int64_t c = tile * W + w;
    const bool live = c < p.ncols;
    const int64_t o = outer * p.ncols + c;
    Acc r = strip_share<W>(op, partials, live ? o : 0, live, h, p);
    if constexpr (H > 1) {
        if (h > 0) stage[h - 1][w] = r;
        __syncthreads();
        if (h == 0) {
#pragma unroll
            for (int k = 1; k < H; ++k) r = op.combine(r, stage[k - 1][w]);
        }
    }
    if (h == 0 && live) sink.put(o, r, p.nred);
}

// The same fold as a kernel of its own, for launches whose blocks cannot take tickets. Grid: one block per strip.
template <class Op, class Sink>
__global__ void __launch_bounds__(kRThreads) reduce_strip_combine_kernel(const __grid_constant__ ReduceArgs a, const Op op,
                                                                         const Sink sink) {
    using T = typename Op::T;
    using Acc = typename Op::Acc;
    constexpr int VC = (16 / sizeof(T)) > 8 ? 8 : (16 / sizeof(T));
    constexpr int W = 32 * VC, H = kRThreads / W;
    const ReducePlan &p = a.plan;
    __shared__ Acc stage[H > 1 ? H - 1 : 1][W];
    const int64_t outer = blockIdx.x / p.xtiles;
    const int64_t tile = blockIdx.x - outer * p.xtiles;
    const int w = threadIdx.x % W, h = threadIdx.x / W;
    const int64_t c = tile * W + w;
    const bool live = c < p.ncols;
    const int64_t o = outer * p.ncols + c;
    Acc r = strip_share<W>(op, static_cast<const Acc *>(a.partials), live ? o : 0, live, h, p);
    if constexpr (H > 1) {
        if (h > 0) stage[h - 1][w] = r;
        __syncthreads();
        if (h == 0) {
#pragma unroll
            for (int k = 1; k < H; ++k) r = op.combine(r, stage[k - 1][w]);
        }
    }
    if (h == 0 && live) sink.put(o, r, p.nred);
}

// The partials of an output folded in chunk order by a team of L lanes (1, 32 or 256): lane l takes chunks
// l, l + L, ... and the team folds in lane order. Grid: one block per 256 / L outputs.
template <int L, class Op, class Sink>
__global__ void __launch_bounds__(kRThreads) reduce_combine_kernel(const __grid_constant__ ReduceArgs a, const Op op,
                                                                   const Sink sink) {
    using Acc = typename Op::Acc;
    const ReducePlan &p = a.plan;
    const Acc *partials = static_cast<const Acc *>(a.partials);
    const int lane = threadIdx.x % L;
    const int64_t o = static_cast<int64_t>(blockIdx.x) * (kRThreads / L) + threadIdx.x / L;
    const bool live = o < p.nout;
    const Acc acc = fold_team<L>(op, team_partials<L>(op, partials, o, live, lane, p));
    if (lane == 0 && live) sink.put(o, acc, p.nred);
}

// The number of partials up to which the block that finishes last folds them itself where few threads share an
// output's partials (columns: one to four; single-lane rows: one); teams of 32 and 256 lanes always do.
constexpr int64_t kSelfFoldSplits = 64;

inline unsigned clamp_grid(int64_t n, int64_t cap) { return static_cast<unsigned>(n < cap ? (n < 1 ? 1 : n) : cap); }

// Queues the reduction on `stream`. a.plan is set; a.partials holds plan_partial_bytes(a.plan).
template <class Op, class Sink>
hmc_status launch_reduce(const ReduceArgs &a, const Op &op, const Sink &sink, cudaStream_t stream) {
    static_assert(sizeof(typename Op::Acc) <= kPartialBytes, "accumulator too large for a partial");
    const ReducePlan &p = a.plan;
    if (p.nout == 0) return HMC_OK;
    // the lanes that share an output's partials (part of the fold order, so a function of the plan alone)
    const int lanes = p.kind == 0 ? p.group : (p.splits > kSelfFoldSplits ? 32 : 0);  // (0: the strip's block folds)
    ReduceArgs args = a;
    const int64_t blocks_x = p.kind == 1 ? p.kouter * p.xtiles : (p.nout + kRThreads / p.group - 1) / (kRThreads / p.group);
    const bool self_fold = p.splits > 1 && a.tickets != nullptr && blocks_x <= kTickets &&
                           (p.kind == 0 ? (p.group > 1 || p.splits <= kSelfFoldSplits) : lanes == 0);
    if (!self_fold) args.tickets = nullptr;
    if (p.kind == 1) {
        if (blocks_x > 0x7FFFFFFF) return fail(HMC_INVALID, "a reduction with more than 2^31 strips of outputs");
        dim3 grid(static_cast<unsigned>(blocks_x), static_cast<unsigned>(p.splits));
        reduce_columns_kernel<Op, Sink><<<grid, kRThreads, 0, stream>>>(args, op, sink);
    } else {
        if (blocks_x > 0x7FFFFFFF) return fail(HMC_INVALID, "a reduction with more than 2^31 blocks of outputs");
        dim3 grid(static_cast<unsigned>(blocks_x), static_cast<unsigned>(p.splits));
        if (p.group == 256) reduce_rows_kernel<256, Op, Sink><<<grid, kRThreads, 0, stream>>>(args, op, sink);
        else if (p.group == 32) reduce_rows_kernel<32, Op, Sink><<<grid, kRThreads, 0, stream>>>(args, op, sink);
        else reduce_rows_kernel<1, Op, Sink><<<grid, kRThreads, 0, stream>>>(args, op, sink);
    }
    hmc_status s = launch_status("reduction kernel launch");
    if (s != HMC_OK) return s;
    if (p.splits > 1 && !self_fold) {
        if (lanes == 0) {
            reduce_strip_combine_kernel<Op, Sink><<<static_cast<unsigned>(blocks_x), kRThreads, 0, stream>>>(a, op, sink);
        } else {
            const int64_t blocks = (p.nout + kRThreads / lanes - 1) / (kRThreads / lanes);
            if (blocks > 0x7FFFFFFF) return fail(HMC_INVALID, "a reduction with more than 2^31 blocks of outputs");
            const unsigned grid = static_cast<unsigned>(blocks);
            if (lanes == 256) reduce_combine_kernel<256, Op, Sink><<<grid, kRThreads, 0, stream>>>(a, op, sink);
            else if (lanes == 32) reduce_combine_kernel<32, Op, Sink><<<grid, kRThreads, 0, stream>>>(a, op, sink);
            else reduce_combine_kernel<1, Op, Sink><<<grid, kRThreads, 0, stream>>>(a, op, sink);
        }
        s = launch_status("reduction combine kernel launch");
    }
    return s;
}

// ---- accumulator ops ----
template <class T> __device__ __forceinline__ double widen(T x) { return to_f64(x); }

template <class TT, bool PROD>
struct FloatFold {
    using T = TT;
    using Acc = double;
    __device__ __forceinline__ Acc init() const { return PROD ? 1.0 : 0.0; }
    __device__ __forceinline__ Acc load(T x, int64_t, int64_t) const { return widen(x); }
    __device__ __forceinline__ Acc combine(Acc a, Acc b) const { return PROD ? a * b : a + b; }
};

template <class TT, bool PROD>
struct IntFold {
    using T = TT;
    using Acc = int64_t;
    __device__ __forceinline__ Acc init() const { return PROD ? 1 : 0; }
    __device__ __forceinline__ Acc load(T x, int64_t, int64_t) const { return to_i64(x); }
    __device__ __forceinline__ Acc combine(Acc a, Acc b) const {
        uint64_t ua = static_cast<uint64_t>(a), ub = static_cast<uint64_t>(b);
        return static_cast<int64_t>(PROD ? ua * ub : ua + ub);
    }
};

template <class TT, bool ALL>
struct Truth {
    using T = TT;
    using Acc = uint32_t;
    __device__ __forceinline__ Acc init() const { return ALL ? 1u : 0u; }
    __device__ __forceinline__ Acc load(T x, int64_t, int64_t) const { return to_bool(x) ? 1u : 0u; }
    __device__ __forceinline__ Acc combine(Acc a, Acc b) const { return ALL ? (a & b) : (a | b); }
};

template <class TT, bool MAX>
struct Extreme {
    using T = TT;
    using Acc = Best<TT>;
    __device__ __forceinline__ Acc init() const { return Acc{TT{}, -1}; }
    __device__ __forceinline__ Acc load(T x, int64_t, int64_t j) const { return Acc{x, j}; }
    // x comes after everything in acc: it wins only by being the first NaN or strictly better
    // (`replaces`, src/backend/cpu/reduce.rs:75-86).
    __device__ __forceinline__ Acc step(Acc acc, T x, int64_t j) const {
        const auto kx = order_key(x), ka = order_key(acc.v);
        bool take;
        if constexpr (Tr<TT>::kind == kFloat) take = (ka == ka) && (kx != kx || (MAX ? kx > ka : kx < ka));
        else take = MAX ? kx > ka : kx < ka;
        take = take || acc.i < 0;
        return take ? Acc{x, j} : acc;
    }
    __device__ __forceinline__ Acc combine(Acc a, Acc b) const {
        if (a.i < 0) return b;
        if (b.i < 0) return a;
        auto ka = order_key(a.v), kb = order_key(b.v);
        if constexpr (Tr<TT>::kind == kFloat) {
            const bool an = ka != ka, bn = kb != kb;
            if (an || bn) return (an && (!bn || a.i < b.i)) ? a : b;
        }
        if (MAX ? kb > ka : kb < ka) return b;
        if (MAX ? ka > kb : ka < kb) return a;
        return a.i < b.i ? a : b;
    }
};

// (x - mean)^2 in f64 with the mean of the element's output. src/backend/cpu/reduce.rs:153-160.
template <class TT>
struct SquaredDeviation {
    using T = TT;
    using Acc = double;
    const double *means;
    double mean;
    __device__ __forceinline__ Acc init() const { return 0.0; }
    __device__ __forceinline__ Acc load(T x, int64_t o, int64_t) const {
        const double d = widen(x) - (means != nullptr ? means[o] : mean);
        return d * d;
    }
    __device__ __forceinline__ SquaredDeviation bound(int64_t o) const {
        return SquaredDeviation{nullptr, means != nullptr ? means[o] : mean};
    }
    __device__ __forceinline__ Acc combine(Acc a, Acc b) const { return a + b; }
};

// ---- sinks ----
// Float sum / prod / mean: mode 0 rounds the f64 to T, mode 1 divides by the count first, mode 2
// stores the f64 mean into `means` (first pass of var), mode 3 stores the f64 accumulator itself (the
// partial of one shard).
template <class T>
struct FloatSink {
    T *out;
    double *means;
    int mode;
    __device__ __forceinline__ void put(int64_t o, double a, int64_t count) const {
        if (mode == 0) out[o] = from_f64<T>(a);
        else if (mode == 1) out[o] = from_f64<T>(a / static_cast<double>(count));
        else if (mode == 2) means[o] = a / static_cast<double>(count);
        else means[o] = a;
    }
};
struct Int64Sink {
    int64_t *out;
    __device__ __forceinline__ void put(int64_t o, int64_t a, int64_t) const { out[o] = a; }
};
struct TruthSink {
    uint8_t *out;
    __device__ __forceinline__ void put(int64_t o, uint32_t a, int64_t) const { out[o] = static_cast<uint8_t>(a != 0); }
};
template <class T>
struct ExtremeSink {
    T *values;        // may be null
    int64_t *indices; // may be null
    __device__ __forceinline__ void put(int64_t o, Best<T> a, int64_t) const {
        if (values != nullptr) values[o] = a.v;
        if (indices != nullptr) indices[o] = a.i;
    }
};
// var / std: sum of squares / divisor, NaN for an empty reduction.
template <class T>
struct VarSink {
    T *out;
    double divisor;
    int take_sqrt;
    __device__ __forceinline__ void put(int64_t o, double sq, int64_t count) const {
        double v = count == 0 ? __longlong_as_double(0x7FF8000000000000ll) : sq / divisor;
        out[o] = from_f64<T>(take_sqrt ? sqrt(v) : v);
    }
};

// Internal launchers, one translation unit each.
hmc_status reduce_float(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, ReduceArgs &a);
hmc_status reduce_float_partial(hmc_context_t ctx, int32_t op, double *partial, ReduceArgs &a);
hmc_status reduce_var_partial(hmc_context_t ctx, double *partial, ReduceArgs &a, const double *means);
hmc_status reduce_var(hmc_context_t ctx, const hmc_tensor_desc *out, ReduceArgs &a, double correction, int take_sqrt,
                      double *means);
hmc_status reduce_int(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, ReduceArgs &a);
hmc_status reduce_truth(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, ReduceArgs &a);
hmc_status reduce_extreme(hmc_context_t ctx, bool is_max, void *values, int64_t *indices, ReduceArgs &a);

}  // namespace hmc
