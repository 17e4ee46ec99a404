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
//  * group (kind 0): an output is folded by G = 1, 32 or 256 lanes. The last reduced dimension is
//    the "row"; it is cut into vectors of VEC elements (16 bytes), vector v of a row goes to lane
//    v mod G, and a lane folds its vectors in order. Rows with unit stride whose start is 16-byte
//    aligned are read with 128-bit loads, four in flight per lane; any other row is read element
//    by element with the same assignment, hence the same result bits. Lanes are combined by warp
//    shuffles and, for G = 256, through shared memory in warp order.
//  * columns (kind 1): the outputs are adjacent in memory (the last kept dimension has stride 1)
//    and the reduced elements are strided. A block is 32 x 8 threads; a thread owns VC adjacent
//    outputs (one 16-byte load per reduced index), the 8 warps take reduced indices j, j+8, ...,
//    and are combined in warp order through shared memory. Global loads are fully coalesced.
//
// When the outputs alone cannot fill the GPU, the reduced range is cut into `splits` chunks; each
// chunk writes a 16-byte partial per output into the caller's workspace and a second kernel folds
// the partials of an output in chunk order.
//
// Accumulators follow homura's CPU fold (src/backend/cpu/reduce.rs:42-131): floats in f64,
// integers wrapping in i64, extremes as (value, index) with "first NaN, then first of equals".
#pragma once

#include "common.cuh"
#include "elem.cuh"

namespace hmc {

constexpr int kRThreads = 256;
constexpr int64_t kTargetLanes = 148 * 2048;  // fixed, so that plans do not depend on the device
constexpr int64_t kTargetColumnBlocks = 148 * 3;  // one wave of the column kernel's blocks (three are resident per SM)
constexpr int64_t kMaxSplits = 4096;
constexpr int64_t kWarpRowOutputs = 148 * 32;  // outputs from which a long row is folded by a warp
constexpr int64_t kWarpRowLength = 1 << 16;    // and the longest such row
constexpr int64_t kPartialBytes = 16;

struct ReducePlan {
    int32_t kind;    // 0 group, 1 columns
    int32_t group;   // lanes per output (kind 0)
    int32_t vec;     // elements per 16-byte vector of the source dtype
    int32_t vc;      // outputs per thread (kind 1)
    int64_t nout, nred;
    int64_t row, step;  // last reduced dimension: size and source stride
    int64_t splits, chunk;
    int64_t ncols, kouter, xtiles;  // kind 1: last kept size, product of the others, column tiles
    // kind 0, no chunks, and every output folds one unit-stride row of whole vectors (nred < 2^31): rows that
    // start on a 16-byte boundary take a loop without the bookkeeping of ranges, dimensions and ragged ends.
    int32_t simple;
};

struct ReduceArgs {
    hmc_tensor_desc kept;
    hmc_tensor_desc red;
    ReducePlan plan;
    void *partials;
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

// The result of the G lanes of a group, valid in its lane 0. All threads of the block call it.
template <int G, class Op>
__device__ __forceinline__ typename Op::Acc group_combine(const Op &op, typename Op::Acc acc) {
    using Acc = typename Op::Acc;
    if constexpr (G == 1) {
        return acc;
    } else {
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            Acc other = shuffle_down(acc, d);
            acc = op.combine(acc, other);
        }
        if constexpr (G == 256) {
            __shared__ Acc warp_acc[kRThreads / 32];
            const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
            if (lane == 0) warp_acc[warp] = acc;
            __syncthreads();
            if (threadIdx.x == 0) {
                for (int w = 1; w < kRThreads / 32; ++w) acc = op.combine(acc, warp_acc[w]);
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

// Folds the reduced elements [j0, j1) of output o, whose kept offset is `base`, for one lane.
template <int G, class Op>
__device__ __forceinline__ typename Op::Acc fold_range(const Op &op, const ReduceArgs &a, int64_t o, int64_t base,
                                                       int64_t j0, int64_t j1, int lane) {
    using T = typename Op::T;
    using Acc = typename Op::Acc;
    constexpr int VEC = 16 / sizeof(T);
    constexpr int UNR = 4;
    const T *src = static_cast<const T *>(a.kept.data);
    const int64_t row = a.plan.row, step = a.plan.step;
    Acc acc = op.init();
    if (j1 <= j0) return acc;
    for (int64_t q = j0 / row; q * row < j1; ++q) {
        const int64_t first = q * row;
        const int64_t lo = j0 > first ? j0 - first : 0;
        const int64_t hi = j1 - first < row ? j1 - first : row;
        const int64_t r = base + (a.red.ndim > 1 ? decompose(a.red, q, a.red.ndim - 1) : 0);
        const T *p = src + r;
        const int64_t v_end = (hi + VEC - 1) / VEC;
        int64_t v = lo / VEC + lane;
        const bool fast = step == 1 && (reinterpret_cast<uintptr_t>(p) & 15) == 0;
        if (fast) {
            // A range that starts inside a vector: its lane takes the leading elements one by one.
            if (v < v_end && v * VEC < lo) {
                for (int e = 0; e < VEC; ++e) {
                    const int64_t i = v * VEC + e;
                    if (i >= lo && i < hi) acc = fold_step(op, acc, p[i], o, first + i);
                }
                v += G;
            }
            // Whole, aligned vectors, UNR of them in flight.
            while (v + (UNR - 1) * G < v_end && (v + (UNR - 1) * G) * VEC + VEC <= hi) {
                RVec<T, VEC> x[UNR];
#pragma unroll
                for (int u = 0; u < UNR; ++u) x[u] = *reinterpret_cast<const RVec<T, VEC> *>(p + (v + u * G) * VEC);
                bool general = true;
                if constexpr (is_extreme<Op>::value) {
                    // The best of the batch by plain comparisons (a later element wins only if strictly better), then
                    // one general combination with what came before; a NaN in the batch (seen in the sum of the
                    // keys) sends the batch through the general step instead.
                    constexpr bool kMax = extreme_is_max<Op>::value;
                    auto best_key = order_key(x[0].v[0]);
                    T best = x[0].v[0];
                    int code = 0;
                    float alarm = 0.0f;
#pragma unroll
                    for (int u = 0; u < UNR; ++u) {
#pragma unroll
                        for (int e = 0; e < VEC; ++e) {
                            const auto k = order_key(x[u].v[e]);
                            if constexpr (Tr<T>::kind == kFloat) alarm += static_cast<float>(k);
                            const bool better = kMax ? k > best_key : k < best_key;
                            best_key = better ? k : best_key;
                            best = better ? x[u].v[e] : best;
                            code = better ? u * VEC + e : code;
                        }
                    }
                    if (alarm == alarm) {
                        const int64_t at = first + (v + (code / VEC) * G) * VEC + code % VEC;
                        acc = op.combine(acc, Acc{best, at});
                        general = false;
                    }
                }
                if (general) {
#pragma unroll
                    for (int u = 0; u < UNR; ++u) {
#pragma unroll
                        for (int e = 0; e < VEC; ++e) acc = fold_step(op, acc, x[u].v[e], o, first + (v + u * G) * VEC + e);
                    }
                }
                v += UNR * G;
            }
            for (; v < v_end; v += G) {
                const int64_t i0 = v * VEC;
                if (i0 + VEC <= hi) {
                    RVec<T, VEC> x = *reinterpret_cast<const RVec<T, VEC> *>(p + i0);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) acc = fold_step(op, acc, x.v[e], o, first + i0 + e);
                } else {
                    for (int e = 0; e < VEC; ++e) {
                        const int64_t i = i0 + e;
                        if (i < hi) acc = fold_step(op, acc, p[i], o, first + i);
                    }
                }
            }
        } else {
            for (; v < v_end; v += G) {
                const int64_t i0 = v * VEC;
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    const int64_t i = i0 + e;
                    if (i >= lo && i < hi) acc = fold_step(op, acc, p[i * step], o, first + i);
                }
            }
        }
    }
    return acc;
}

// One lane's share of a simple row (plan.simple): vectors lane, lane + G, ... of the nvec vectors at p, in
// the order and with the element indices fold_range gives them, hence the same bits.
template <int G, class Op>
__device__ __forceinline__ typename Op::Acc fold_simple_row(const Op &op, const typename Op::T *p, uint32_t nvec, int lane,
                                                            int64_t o) {
    using T = typename Op::T;
    using Acc = typename Op::Acc;
    constexpr int VEC = 16 / sizeof(T);
    constexpr int UNR = 4;
    Acc acc = op.init();
    uint32_t v = lane;
    for (; v + (UNR - 1) * G < nvec; v += UNR * G) {
        RVec<T, VEC> x[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) x[u] = *reinterpret_cast<const RVec<T, VEC> *>(p + static_cast<size_t>(v + u * G) * VEC);
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc = fold_step(op, acc, x[u].v[e], o, static_cast<int64_t>(v + u * G) * VEC + e);
        }
    }
    for (; v < nvec; v += G) {
        const RVec<T, VEC> x = *reinterpret_cast<const RVec<T, VEC> *>(p + static_cast<size_t>(v) * VEC);
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc = fold_step(op, acc, x.v[e], o, static_cast<int64_t>(v) * VEC + e);
    }
    return acc;
}


// The same for max / min / argmax / argmin, where the general step (first NaN, then first of equals, a 64-bit
// index) costs about forty instructions per element. Here a lane keeps the best key, its raw value and a
// 32-bit index, and takes a later element only if it is strictly better: "first of equals" as in the general
// step. NaNs are not handled but detected (the sum of a vector's keys is NaN if one of them is; an
// infinity minus infinity there raises a false alarm, which is harmless): `redo` tells the caller to fold the
// row again with the general step.
template <int G, class TT, bool MAX>
__device__ __forceinline__ typename Extreme<TT, MAX>::Acc fold_simple_row_extreme(const TT *p, uint32_t nvec, int lane, bool &redo) {
    using Acc = typename Extreme<TT, MAX>::Acc;
    constexpr int VEC = 16 / sizeof(TT);
    constexpr int UNR = 4;
    constexpr bool kFloating = Tr<TT>::kind == kFloat;
    redo = false;
    if (static_cast<uint32_t>(lane) >= nvec) return Acc{TT{}, -1};
    TT best = p[static_cast<size_t>(lane) * VEC];
    auto best_key = order_key(best);
    uint32_t best_at = lane * VEC;
    float alarm = 0.0f;
    auto take_vector = [&](const RVec<TT, VEC> &x, uint32_t at) {
        if constexpr (kFloating) {
            float s = static_cast<float>(order_key(x.v[0]));
#pragma unroll
            for (int e = 1; e < VEC; ++e) s += static_cast<float>(order_key(x.v[e]));
            alarm += s;
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            const auto k = order_key(x.v[e]);
            const bool better = MAX ? k > best_key : k < best_key;
            best_key = better ? k : best_key;
            best = better ? x.v[e] : best;
            best_at = better ? at + e : best_at;
        }
    };
    uint32_t v = lane;
    for (; v + (UNR - 1) * G < nvec; v += UNR * G) {
        RVec<TT, VEC> x[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) x[u] = *reinterpret_cast<const RVec<TT, VEC> *>(p + static_cast<size_t>(v + u * G) * VEC);
#pragma unroll
        for (int u = 0; u < UNR; ++u) take_vector(x[u], (v + u * G) * VEC);
    }
    for (; v < nvec; v += G) take_vector(*reinterpret_cast<const RVec<TT, VEC> *>(p + static_cast<size_t>(v) * VEC), v * VEC);
    if constexpr (kFloating) redo = alarm != alarm;
    return Acc{best, static_cast<int64_t>(best_at)};
}

// kind 0. Grid: (tiles of 256 / G outputs, splits).
template <int G, class Op, class Sink>
__global__ void __launch_bounds__(kRThreads) reduce_group_kernel(const __grid_constant__ ReduceArgs a, const Op op,
                                                                 const Sink sink) {
    using Acc = typename Op::Acc;
    constexpr int P = kRThreads / G;
    const ReducePlan &p = a.plan;
    const int lane = threadIdx.x % G;
    const int slot = threadIdx.x / G;
    const int64_t c = blockIdx.y;
    const int64_t j0 = c * p.chunk;
    const int64_t j1 = j0 + p.chunk < p.nred ? j0 + p.chunk : p.nred;
    const int64_t tiles = (p.nout + P - 1) / P;
    for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int64_t o = tile * P + slot;
        Acc acc = op.init();
        if (o < p.nout) {
            using T = typename Op::T;
            const int64_t base = a.kept.offset + decompose(a.kept, o, a.kept.ndim);
            const T *row = static_cast<const T *>(a.kept.data) + base;
            bool general = true;
            if constexpr (G > 1) {
                if (p.simple && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
                    const uint32_t nvec = static_cast<uint32_t>(p.nred) / (16 / sizeof(T));
                    if constexpr (is_extreme<Op>::value) {
                        bool redo;
                        acc = fold_simple_row_extreme<G, T, std::is_same_v<Op, Extreme<T, true>>>(row, nvec, lane, redo);
                        // the lanes of an output agree on folding again (an output's lanes are a warp, or the block)
                        if constexpr (G == 32) general = __any_sync(0xFFFFFFFFu, redo);
                        else general = __syncthreads_or(redo);
                    } else {
                        acc = fold_simple_row<G>(op, row, nvec, lane, o);
                        general = false;
                    }
                }
            }
            if (general) acc = fold_range<G>(op, a, o, base, j0, j1, lane);
        }
        acc = group_combine<G>(op, acc);
        if (lane == 0 && o < p.nout) {
            if (p.splits == 1) sink.put(o, acc, p.nred);
            else static_cast<Acc *>(a.partials)[c * p.nout + o] = acc;
        }
    }
}

// kind 1. Grid: (kouter * xtiles, splits); block 32 x 8.
template <class Op, class Sink>
__global__ void __launch_bounds__(kRThreads) reduce_columns_kernel(const __grid_constant__ ReduceArgs a, const Op op,
                                                                   const Sink sink) {
    using T = typename Op::T;
    using Acc = typename Op::Acc;
    constexpr int VC = (16 / sizeof(T)) > 8 ? 8 : (16 / sizeof(T));
    constexpr int UNR = 8;  // loads in flight per thread: 8 measured 6 % faster than 4 on B200 (three blocks per SM)
    const ReducePlan &p = a.plan;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t chunk = blockIdx.y;
    const int64_t j0 = chunk * p.chunk;
    const int64_t j1 = j0 + p.chunk < p.nred ? j0 + p.chunk : p.nred;
    const int last = a.kept.ndim - 1;
    const bool single = a.red.ndim == 1;
    auto red_off = [&](int64_t j) { return single ? j * a.red.strides[0] : decompose(a.red, j, a.red.ndim); };
    __shared__ Acc stage[7][32 * VC];
    const int64_t xblocks = p.kouter * p.xtiles;
    for (int64_t bx = blockIdx.x; bx < xblocks; bx += gridDim.x) {
        const int64_t outer = bx / p.xtiles;
        const int64_t tile = bx - outer * p.xtiles;
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
            int64_t j = j0 + ty;
            for (; j + (UNR - 1) * 8 < j1; j += UNR * 8) {
                RVec<T, VC> x[UNR];
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
                    const T *q = src + red_off(j + u * 8);
                    if (whole && (reinterpret_cast<uintptr_t>(q) & (alignof(RVec<T, VC>) - 1)) == 0) {
                        x[u] = *reinterpret_cast<const RVec<T, VC> *>(q);
                    } else {
#pragma unroll
                        for (int e = 0; e < VC; ++e) x[u].v[e] = c0 + e < p.ncols ? q[e] : T{};
                    }
                }
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
#pragma unroll
                    for (int e = 0; e < VC; ++e) {
                        if (whole || c0 + e < p.ncols) acc[e] = fold_step(ops[e], acc[e], x[u].v[e], o0 + e, j + u * 8);
                    }
                }
            }
            for (; j < j1; j += 8) {
                const T *q = src + red_off(j);
#pragma unroll
                for (int e = 0; e < VC; ++e) {
                    if (c0 + e < p.ncols) acc[e] = fold_step(ops[e], acc[e], q[e], o0 + e, j);
                }
            }
        }
        if (ty > 0) {
#pragma unroll
            for (int e = 0; e < VC; ++e) stage[ty - 1][tx * VC + e] = acc[e];
        }
        __syncthreads();
        if (ty == 0 && in_range) {
#pragma unroll
            for (int e = 0; e < VC; ++e) {
                if (c0 + e >= p.ncols) continue;
                Acc r = acc[e];
                for (int w = 0; w < 7; ++w) r = op.combine(r, stage[w][tx * VC + e]);
                if (p.splits == 1) sink.put(o0 + e, r, p.nred);
                else static_cast<Acc *>(a.partials)[chunk * p.nout + o0 + e] = r;
            }
        }
        __syncthreads();
    }
}

// Folds the partials of each output in chunk order. L lanes per output (1, 32 or 256): lane l folds chunks
// l, l + L, ... and the lanes are combined in lane order (shuffles, and shared memory for 256).
template <int L, class Op, class Sink>
__global__ void __launch_bounds__(kRThreads) reduce_combine_kernel(const __grid_constant__ ReduceArgs a, const Op op,
                                                                   const Sink sink) {
    using Acc = typename Op::Acc;
    const ReducePlan &p = a.plan;
    const Acc *partials = static_cast<const Acc *>(a.partials);
    const int lane = threadIdx.x % L;
    const int64_t per_block = kRThreads / L;
    const int64_t rounds = (p.nout + per_block - 1) / per_block;
    for (int64_t t = blockIdx.x; t < rounds; t += gridDim.x) {
        const int64_t o = t * per_block + threadIdx.x / L;
        Acc acc = op.init();
        if (o < p.nout) {
#pragma unroll 4
            for (int64_t c = lane; c < p.splits; c += L) acc = op.combine(acc, partials[c * p.nout + o]);
        }
        if constexpr (L == 32) {
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) acc = op.combine(acc, shuffle_down(acc, d));
        } else if constexpr (L == 256) {
            acc = group_combine<256>(op, acc);
        }
        if (lane == 0 && o < p.nout) sink.put(o, acc, p.nred);
    }
}

inline unsigned clamp_grid(int64_t n, int64_t cap) { return static_cast<unsigned>(n < cap ? (n < 1 ? 1 : n) : cap); }

// Queues the reduction on `stream`. a.plan is set; a.partials holds plan_partial_bytes(a.plan).
template <class Op, class Sink>
hmc_status launch_reduce(const ReduceArgs &a, const Op &op, const Sink &sink, cudaStream_t stream) {
    static_assert(sizeof(typename Op::Acc) <= kPartialBytes, "accumulator too large for a partial");
    const ReducePlan &p = a.plan;
    if (p.nout == 0) return HMC_OK;
    if (p.kind == 1) {
        dim3 grid(clamp_grid(p.kouter * p.xtiles, 1 << 20), static_cast<unsigned>(p.splits));
        reduce_columns_kernel<Op, Sink><<<grid, kRThreads, 0, stream>>>(a, op, sink);
    } else {
        const int64_t per_block = kRThreads / p.group;
        const int64_t tiles = (p.nout + per_block - 1) / per_block;
        dim3 grid(clamp_grid(tiles, 1 << 20), static_cast<unsigned>(p.splits));
        if (p.group == 256) reduce_group_kernel<256, Op, Sink><<<grid, kRThreads, 0, stream>>>(a, op, sink);
        else if (p.group == 32) reduce_group_kernel<32, Op, Sink><<<grid, kRThreads, 0, stream>>>(a, op, sink);
        else reduce_group_kernel<1, Op, Sink><<<grid, kRThreads, 0, stream>>>(a, op, sink);
    }
    hmc_status s = launch_status("reduction kernel launch");
    if (s != HMC_OK) return s;
    if (p.splits > 1) {
        if (p.splits >= 512 && p.nout <= 64) {
            // a few outputs with very many partials each (a full reduction): a block per output
            reduce_combine_kernel<256, Op, Sink><<<clamp_grid(p.nout, 1 << 16), kRThreads, 0, stream>>>(a, op, sink);
        } else if (p.splits >= 64) {
            const int64_t rounds = (p.nout + 7) / 8;
            reduce_combine_kernel<32, Op, Sink><<<clamp_grid(rounds, 1 << 16), kRThreads, 0, stream>>>(a, op, sink);
        } else {
            const int64_t rounds = (p.nout + kRThreads - 1) / kRThreads;
            reduce_combine_kernel<1, Op, Sink><<<clamp_grid(rounds, 1 << 16), kRThreads, 0, stream>>>(a, op, sink);
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
