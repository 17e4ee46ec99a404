// The elementwise engine: one kernel template that walks up to four strided operands (operand 0 is
// the output) and applies a functor to every element.
//
// Layout handling. The caller has merged dimensions, so a contiguous tensor is one dimension. The
// innermost dimension is the unit of work: a row of n0 elements is cut into segments, a thread owns
// VEC consecutive inner elements (16 bytes of the narrowest operand), and per operand the access is
// chosen by its inner stride: 1 -> one 128-bit (or narrower) vector access when the address is
// aligned, scalar accesses otherwise; 0 -> one load broadcast to the lanes (row bias); other ->
// strided scalar accesses. The outer dimensions are decomposed once per thread and row, not per
// element, and a plain 2-D operand (row or column broadcast, narrowed view) needs no division at
// all. Short rows share a block (threads-per-row is the power of two covering n0 / VEC).
//
// Each thread issues UNR independent vector loads per input before it computes and stores, so a
// resident SM has tens of KB in flight, which HBM3e needs to reach its bandwidth.
#pragma once

#include "common.cuh"
#include "elem.cuh"

namespace hmc {

constexpr int kThreads = 256;
#ifndef HMC_MAP_ITEMS_PER_BLOCK
#define HMC_MAP_ITEMS_PER_BLOCK 4
#endif
#ifndef HMC_MAP_MIN_BLOCKS
#define HMC_MAP_MIN_BLOCKS 4
#endif
constexpr int kOperands = 4;

struct Unused {};

struct MapArgs {
    int32_t ndim;          // >= 1
    int32_t tpr_log2;      // threads per row = 1 << tpr_log2
    int64_t n0;            // inner size
    int64_t rows;          // product of the outer sizes
    int64_t segs;          // segments per row
    int64_t items;         // row groups * segs
    int32_t rows_fit32;    // rows < 2^31: 32-bit index arithmetic for the row decomposition
    // item / segs without a division, for items < 2^31: (item * segs_magic) >> segs_shift
    int32_t segs_shift;    // 0: not available (use the 64-bit division)
    uint64_t segs_magic;
    uint32_t constant_mask;  // bit k: operand k is a constant held in constant[k]
    uint64_t constant[kOperands];
    // The tiled kernel (operands read against the grain through shared memory):
    uint32_t tile_mask;     // bit k: input k has unit stride along the second-to-last dimension
    int64_t tiles_a, tiles_b, ntiles;
    char *base[kOperands];  // data + offset, as bytes
    int64_t sizes[HMC_MAX_DIMS];
    int64_t strides[kOperands][HMC_MAX_DIMS];
};

template <class T, int VEC>
struct alignas((sizeof(T) * VEC) >= 16 ? 16 : sizeof(T) * VEC) Pack {
    T v[VEC];
};
template <int VEC>
struct Pack<Unused, VEC> {};

template <class T> constexpr int size_or(int fallback) { return sizeof(T); }
template <> constexpr int size_or<Unused>(int fallback) { return fallback; }

template <class F> constexpr int vec_of() {
    constexpr int so = sizeof(typename F::Out);
    constexpr int sa = size_or<typename F::A>(so), sb = size_or<typename F::B>(so), sc = size_or<typename F::C>(so);
    constexpr int mn = so < sa ? (so < sb ? (so < sc ? so : sc) : (sb < sc ? sb : sc)) : (sa < sb ? (sa < sc ? sa : sc) : (sb < sc ? sb : sc));
    constexpr int mx = so > sa ? (so > sb ? (so > sc ? so : sc) : (sb > sc ? sb : sc)) : (sa > sb ? (sa > sc ? sa : sc) : (sb > sc ? sb : sc));
    constexpr int a = 16 / mn, b = 64 / mx;
    return a < b ? a : b;
}
template <class T> constexpr int size_or_zero() { return sizeof(T); }
template <> constexpr int size_or_zero<Unused>() { return 0; }

template <class F> constexpr int unroll_of() {
    // About 64 bytes of inputs in flight per thread and iteration (the loads of all inputs are issued before
    // the first store), and never more than 64 bytes of output held at once.
    constexpr int in_bytes = (size_or_zero<typename F::A>() + size_or_zero<typename F::B>() + size_or_zero<typename F::C>()) *
                             vec_of<F>();
    constexpr int out_bytes = static_cast<int>(sizeof(typename F::Out)) * vec_of<F>();
    constexpr int by_in = in_bytes == 0 ? 4 : (in_bytes >= 64 ? 1 : (in_bytes >= 32 ? 2 : 4));
    constexpr int by_out = out_bytes >= 64 ? 1 : (out_bytes >= 32 ? 2 : 4);
    return by_in < by_out ? by_in : by_out;
}

// How an operand is walked along the inner dimension.
enum : int { kModeUnit = 0, kModeBroadcast = 1, kModeStrided = 2, kModeConstant = 3 };

__device__ __forceinline__ int operand_mode(const MapArgs &a, int k) {
    if (a.constant_mask & (1u << k)) return kModeConstant;
    const int64_t s0 = a.strides[k][a.ndim - 1];
    return s0 == 1 ? kModeUnit : (s0 == 0 ? kModeBroadcast : kModeStrided);
}

// VEC elements of operand k starting at inner index idx; `row` points to the row's first element.
template <class T, int VEC>
__device__ __forceinline__ void load_operand(Pack<T, VEC> &dst, const MapArgs &a, int k, int mode, const T *row,
                                             int64_t idx) {
    if constexpr (!std::is_same_v<T, Unused>) {
        if (mode == kModeUnit) {
            const T *p = row + idx;
            if (idx + VEC <= a.n0 && (reinterpret_cast<uintptr_t>(p) & (alignof(Pack<T, VEC>) - 1)) == 0) {
                dst = *reinterpret_cast<const Pack<T, VEC> *>(p);
            } else {
#pragma unroll
                for (int j = 0; j < VEC; ++j)
                    if (idx + j < a.n0) dst.v[j] = p[j];
            }
        } else if (mode == kModeBroadcast) {
            const T c = *row;
#pragma unroll
            for (int j = 0; j < VEC; ++j) dst.v[j] = c;
        } else if (mode == kModeConstant) {
            T c;
            uint64_t bits = a.constant[k];
            memcpy(&c, &bits, sizeof(T));
#pragma unroll
            for (int j = 0; j < VEC; ++j) dst.v[j] = c;
        } else {
            const int64_t s0 = a.strides[k][a.ndim - 1];
#pragma unroll
            for (int j = 0; j < VEC; ++j)
                if (idx + j < a.n0) dst.v[j] = row[(idx + j) * s0];
        }
    }
}

template <class T, int VEC>
__device__ __forceinline__ void store_operand(const Pack<T, VEC> &src, const MapArgs &a, int k, int mode, T *row,
                                              int64_t idx) {
    if (mode == kModeUnit) {
        T *p = row + idx;
        if (idx + VEC <= a.n0 && (reinterpret_cast<uintptr_t>(p) & (alignof(Pack<T, VEC>) - 1)) == 0) {
            *reinterpret_cast<Pack<T, VEC> *>(p) = src;
        } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j)
                if (idx + j < a.n0) p[j] = src.v[j];
        }
    } else {
        const int64_t s0 = a.strides[k][a.ndim - 1];
#pragma unroll
        for (int j = 0; j < VEC; ++j)
            if (idx + j < a.n0) row[(idx + j) * s0] = src.v[j];
    }
}

// The offsets of the operands at outer index `row` (all dimensions but the last), in elements.
__device__ __forceinline__ void row_offsets(const MapArgs &a, int64_t row, int64_t off[kOperands]) {
    const int last = a.ndim - 1;
#pragma unroll
    for (int k = 0; k < kOperands; ++k) off[k] = 0;
    if (last <= 0) return;
    if (a.rows_fit32) {
        uint32_t r = static_cast<uint32_t>(row);
        for (int d = last - 1; d > 0; --d) {
            const uint32_t size = static_cast<uint32_t>(a.sizes[d]);
            const uint32_t q = r / size;
            const uint32_t i = r - q * size;
#pragma unroll
            for (int k = 0; k < kOperands; ++k) off[k] += static_cast<int64_t>(i) * a.strides[k][d];
            r = q;
        }
#pragma unroll
        for (int k = 0; k < kOperands; ++k) off[k] += static_cast<int64_t>(r) * a.strides[k][0];
    } else {
        int64_t r = row;
        for (int d = last - 1; d > 0; --d) {
            const int64_t size = a.sizes[d];
            const int64_t q = r / size;
            const int64_t i = r - q * size;
#pragma unroll
            for (int k = 0; k < kOperands; ++k) off[k] += i * a.strides[k][d];
            r = q;
        }
#pragma unroll
        for (int k = 0; k < kOperands; ++k) off[k] += r * a.strides[k][0];
    }
}

template <class T, int VEC> __device__ __forceinline__ bool vector_aligned(const T *p) {
    if constexpr (std::is_same_v<T, Unused>) return true;
    else return (reinterpret_cast<uintptr_t>(p) & (alignof(Pack<T, VEC>) - 1)) == 0;
}

// The one value of a broadcast or constant operand for a row (unused for unit-stride operands).
template <class T>
__device__ __forceinline__ Pack<T, 1> splat_value(const MapArgs &a, int k, int mode, const T *row) {
    Pack<T, 1> out;
    if constexpr (!std::is_same_v<T, Unused>) {
        if (mode == kModeBroadcast) {
            out.v[0] = *row;
        } else if (mode == kModeConstant) {
            uint64_t bits = a.constant[k];
            memcpy(&out.v[0], &bits, sizeof(T));
        } else {
            out.v[0] = T{};
        }
    }
    return out;
}

template <class T, int VEC>
__device__ __forceinline__ void fast_load(Pack<T, VEC> &dst, int mode, const T *row, int64_t idx, const Pack<T, 1> &c) {
    if constexpr (!std::is_same_v<T, Unused>) {
        if (mode == kModeUnit) {
            dst = *reinterpret_cast<const Pack<T, VEC> *>(row + idx);
        } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j) dst.v[j] = c.v[0];
        }
    }
}

template <class T> __device__ __forceinline__ T *operand_row(const MapArgs &a, int k, int64_t off) {
    if constexpr (std::is_same_v<T, Unused>) return nullptr;
    else return reinterpret_cast<T *>(a.base[k]) + off;
}

template <class F, class = void> struct has_compute : std::false_type {};
template <class F> struct has_compute<F, std::void_t<typename F::Compute>> : std::true_type {};

template <class F, class A, class B, class C>
__device__ __forceinline__ auto apply(const F &f, const A &a, const B &b, const C &c, int j) {
    if constexpr (has_compute<F>::value) {
        if constexpr (std::is_same_v<typename F::B, Unused>) return f.compute(a.v[j]);
        else if constexpr (std::is_same_v<typename F::C, Unused>) return f.compute(a.v[j], b.v[j]);
        else return f.compute(a.v[j], b.v[j], c.v[j]);
    } else {
        if constexpr (std::is_same_v<typename F::A, Unused>) return f();
        else if constexpr (std::is_same_v<typename F::B, Unused>) return f(a.v[j]);
        else if constexpr (std::is_same_v<typename F::C, Unused>) return f(a.v[j], b.v[j]);
        else return f(a.v[j], b.v[j], c.v[j]);
    }
}

// The outputs of N elements: functors with compute() give results in the computation type, which are
// rounded to the output dtype here, two per conversion for the half types.
template <class F, int N, class A, class B, class C>
__device__ __forceinline__ void apply_all(Pack<typename F::Out, N> &out, const F &f, const A &a, const B &b, const C &c) {
    using TO = typename F::Out;
    if constexpr (has_compute<F>::value && (std::is_same_v<TO, F16> || std::is_same_v<TO, BF16>) && N % 2 == 0) {
#pragma unroll
        for (int j = 0; j < N; j += 2) {
            const float r0 = apply<F>(f, a, b, c, j), r1 = apply<F>(f, a, b, c, j + 1);
            down2(out.v[j], out.v[j + 1], r0, r1);
        }
    } else if constexpr (has_compute<F>::value) {
#pragma unroll
        for (int j = 0; j < N; ++j) out.v[j] = down<TO>(apply<F>(f, a, b, c, j));
    } else {
#pragma unroll
        for (int j = 0; j < N; ++j) out.v[j] = apply<F>(f, a, b, c, j);
    }
}

template <class F>
__global__ void __launch_bounds__(kThreads, HMC_MAP_MIN_BLOCKS) map_kernel(const __grid_constant__ MapArgs a, const F f) {
    using TO = typename F::Out;
    using TA = typename F::A;
    using TB = typename F::B;
    using TC = typename F::C;
    constexpr int VEC = vec_of<F>();
    constexpr int UNR = unroll_of<F>();
    const int tpr = 1 << a.tpr_log2;
    const int lane = threadIdx.x & (tpr - 1);
    const int rib = threadIdx.x >> a.tpr_log2;
    const int rpb = kThreads >> a.tpr_log2;
    const int mo = operand_mode(a, 0), ma = operand_mode(a, 1), mb = operand_mode(a, 2), mc = operand_mode(a, 3);
    const int64_t step = static_cast<int64_t>(tpr) * VEC;
    const bool modes_fast = mo == kModeUnit && ma != kModeStrided && mb != kModeStrided && mc != kModeStrided;

    for (int64_t item = blockIdx.x; item < a.items; item += gridDim.x) {
        int64_t rg, seg;
        if (a.rows == 1) {
            rg = 0;
            seg = item;
        } else if (a.segs == 1) {
            rg = item;
            seg = 0;
        } else if (a.segs_shift != 0) {
            rg = static_cast<int64_t>((static_cast<uint64_t>(item) * a.segs_magic) >> a.segs_shift);
            seg = item - rg * a.segs;
        } else {
            rg = item / a.segs;
            seg = item - rg * a.segs;
        }
        const int64_t row = rg * rpb + rib;
        if (row >= a.rows) continue;
        TO *po;
        const TA *pa;
        const TB *pb;
        const TC *pc;
        {
            int64_t off[kOperands];
            row_offsets(a, row, off);
            po = operand_row<TO>(a, 0, off[0]);
            pa = operand_row<TA>(a, 1, off[1]);
            pb = operand_row<TB>(a, 2, off[2]);
            pc = operand_row<TC>(a, 3, off[3]);
        }
        const int64_t i0 = seg * (step * UNR) + static_cast<int64_t>(lane) * VEC;
        Pack<TA, VEC> va[UNR];
        Pack<TB, VEC> vb[UNR];
        Pack<TC, VEC> vc[UNR];
        // The common case, decided once per row segment: every vector of this thread is whole, the output and
        // the unit-stride inputs are aligned for vector accesses, the other inputs are one value per row.
        const bool fast = modes_fast && i0 + (UNR - 1) * step + VEC <= a.n0 && vector_aligned<TO, VEC>(po) &&
                          (ma != kModeUnit || vector_aligned<TA, VEC>(pa)) && (mb != kModeUnit || vector_aligned<TB, VEC>(pb)) &&
                          (mc != kModeUnit || vector_aligned<TC, VEC>(pc));
        if (fast) {
            const Pack<TA, 1> ca = splat_value<TA>(a, 1, ma, pa);
            const Pack<TB, 1> cb = splat_value<TB>(a, 2, mb, pb);
            const Pack<TC, 1> cc = splat_value<TC>(a, 3, mc, pc);
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                const int64_t idx = i0 + u * step;
                fast_load<TA, VEC>(va[u], ma, pa, idx, ca);
                fast_load<TB, VEC>(vb[u], mb, pb, idx, cb);
                fast_load<TC, VEC>(vc[u], mc, pc, idx, cc);
            }
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                const int64_t idx = i0 + u * step;
                Pack<TO, VEC> vo;
                apply_all<F, VEC>(vo, f, va[u], vb[u], vc[u]);
                *reinterpret_cast<Pack<TO, VEC> *>(po + idx) = vo;
            }
            continue;
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int64_t idx = i0 + u * step;
            if (idx < a.n0) {
                load_operand<TA, VEC>(va[u], a, 1, ma, pa, idx);
                load_operand<TB, VEC>(vb[u], a, 2, mb, pb, idx);
                load_operand<TC, VEC>(vc[u], a, 3, mc, pc, idx);
            }
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int64_t idx = i0 + u * step;
            if (idx < a.n0) {
                Pack<TO, VEC> vo;
                apply_all<F, VEC>(vo, f, va[u], vb[u], vc[u]);
                store_operand<TO, VEC>(vo, a, 0, mo, po, idx);
            }
        }
    }
}

// ---- the lean kernel ----
// The layouts that carry almost all of the traffic: one or two dimensions, every operand either unit-stride
// along the inner dimension with rows that start on a vector boundary, or one value per row (a column
// broadcast such as a bias [N, 1]), or a constant; a row-broadcast operand (a scale [1, N]) is the first kind
// with a row stride of 0. Such launches need none of the general kernel's bookkeeping: a thread's vectors are
// found with a handful of integer operations, which matters for 1- and 2-byte elements, where a kernel at HBM
// speed has an instruction budget of about fifteen per element.
struct LeanArgs {
    char *base[kOperands];
    int64_t row_stride[kOperands];  // elements
    uint32_t inner[kOperands];      // 1: unit stride, 0: one value per row
    uint64_t constant[kOperands];
    uint32_t constant_mask;
    uint32_t n0;                    // inner size (< 2^31)
    int64_t rows;
};

template <class T, int VEC>
__device__ __forceinline__ void lean_load(Pack<T, VEC> &dst, const T *row, uint32_t inner, uint32_t col, const Pack<T, 1> &c) {
    if constexpr (!std::is_same_v<T, Unused>) {
        if (inner) {
            dst = *reinterpret_cast<const Pack<T, VEC> *>(row + col);
        } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j) dst.v[j] = c.v[0];
        }
    }
}

template <class F>
__global__ void __launch_bounds__(kThreads, 4) map_lean_kernel(const __grid_constant__ LeanArgs a, const F f) {
    using TO = typename F::Out;
    using TA = typename F::A;
    using TB = typename F::B;
    using TC = typename F::C;
    constexpr int VEC = vec_of<F>();
    constexpr int UNR = unroll_of<F>();
    constexpr uint32_t kStep = kThreads * VEC;
    const uint32_t col0 = blockIdx.x * (kStep * UNR) + threadIdx.x * VEC;
    const bool ka = a.constant_mask & 2u, kb = a.constant_mask & 4u, kc = a.constant_mask & 8u;
    for (int64_t row = blockIdx.y; row < a.rows; row += gridDim.y) {
        TO *po = reinterpret_cast<TO *>(a.base[0]) + row * a.row_stride[0];
        const TA *pa = nullptr;
        const TB *pb = nullptr;
        const TC *pc = nullptr;
        Pack<TA, 1> ca;
        Pack<TB, 1> cb;
        Pack<TC, 1> cc;
        if constexpr (!std::is_same_v<TA, Unused>) {
            pa = reinterpret_cast<const TA *>(a.base[1]) + row * a.row_stride[1];
            if (ka) memcpy(&ca.v[0], &a.constant[1], sizeof(TA));
            else if (!a.inner[1]) ca.v[0] = *pa;
        }
        if constexpr (!std::is_same_v<TB, Unused>) {
            pb = reinterpret_cast<const TB *>(a.base[2]) + row * a.row_stride[2];
            if (kb) memcpy(&cb.v[0], &a.constant[2], sizeof(TB));
            else if (!a.inner[2]) cb.v[0] = *pb;
        }
        if constexpr (!std::is_same_v<TC, Unused>) {
            pc = reinterpret_cast<const TC *>(a.base[3]) + row * a.row_stride[3];
            if (kc) memcpy(&cc.v[0], &a.constant[3], sizeof(TC));
            else if (!a.inner[3]) cc.v[0] = *pc;
        }
        Pack<TA, VEC> va[UNR];
        Pack<TB, VEC> vb[UNR];
        Pack<TC, VEC> vc[UNR];
        if (col0 + (UNR - 1) * kStep + VEC <= a.n0) {
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                const uint32_t col = col0 + u * kStep;
                lean_load<TA, VEC>(va[u], pa, a.inner[1] && !ka, col, ca);
                lean_load<TB, VEC>(vb[u], pb, a.inner[2] && !kb, col, cb);
                lean_load<TC, VEC>(vc[u], pc, a.inner[3] && !kc, col, cc);
            }
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                const uint32_t col = col0 + u * kStep;
                Pack<TO, VEC> vo;
                apply_all<F, VEC>(vo, f, va[u], vb[u], vc[u]);
                *reinterpret_cast<Pack<TO, VEC> *>(po + col) = vo;
            }
        } else {
            // the ragged end of a row: whole vectors while they fit, then single elements
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                const uint32_t col = col0 + u * kStep;
                if (col + VEC <= a.n0) {
                    lean_load<TA, VEC>(va[0], pa, a.inner[1] && !ka, col, ca);
                    lean_load<TB, VEC>(vb[0], pb, a.inner[2] && !kb, col, cb);
                    lean_load<TC, VEC>(vc[0], pc, a.inner[3] && !kc, col, cc);
                    Pack<TO, VEC> vo;
                    apply_all<F, VEC>(vo, f, va[0], vb[0], vc[0]);
                    *reinterpret_cast<Pack<TO, VEC> *>(po + col) = vo;
                } else if (col < a.n0) {
                    for (uint32_t e = col; e < a.n0; ++e) {
                        Pack<TA, 1> xa;
                        Pack<TB, 1> xb;
                        Pack<TC, 1> xc;
                        if constexpr (!std::is_same_v<TA, Unused>) xa.v[0] = (a.inner[1] && !ka) ? pa[e] : ca.v[0];
                        if constexpr (!std::is_same_v<TB, Unused>) xb.v[0] = (a.inner[2] && !kb) ? pb[e] : cb.v[0];
                        if constexpr (!std::is_same_v<TC, Unused>) xc.v[0] = (a.inner[3] && !kc) ? pc[e] : cc.v[0];
                        Pack<TO, 1> one;
                        apply_all<F, 1>(one, f, xa, xb, xc);
                        po[e] = one.v[0];
                    }
                }
            }
        }
    }
}

// Fills `lean` if the launch described by `a` (built by build_map_args) qualifies for the lean kernel.
bool build_lean_args(LeanArgs &lean, const MapArgs &a, const int *elem_size, int vec);

// ---- the tiled kernel ----
// For operands whose unit stride runs along the second-to-last dimension A while the output's runs
// along the last dimension B (a transposed view). Work is cut into 64 x 64 tiles. A tile of each such
// operand is read with 16-byte loads along A (its grain), parked in shared memory as rows of A with
// a 16-byte padded pitch, and read back along B: a thread produces one 32-byte sector of the output
// (EB consecutive elements along B at one A), the lanes of a warp sit on consecutive A, so every
// shared-memory gather is conflict free and every global access moves whole sectors. Tiles on the
// boundary, and operands that are not 16-byte aligned, take an element-wise path through the same
// shared-memory tile.
constexpr int kTile = 64;

template <class T> constexpr int tile_pitch() {  // elements per shared-memory row (one B index, 64 A's)
    if constexpr (std::is_same_v<T, Unused>) return 0;
    else return kTile + 16 / static_cast<int>(sizeof(T));
}
template <class T> constexpr size_t tile_bytes() {
    if constexpr (std::is_same_v<T, Unused>) return 0;
    else return static_cast<size_t>(kTile) * tile_pitch<T>() * sizeof(T);
}
template <class TO> constexpr int tile_eb() {  // output elements per thread along B: a 32-byte sector
    return sizeof(TO) >= 8 ? 4 : (sizeof(TO) == 4 ? 8 : 16);
}

// Fills tile[b][a] (b, a in 0..63) with operand k's elements (a0 + a, b0 + b); `p` points at (a0, b0).
template <class T>
__device__ __forceinline__ void tile_fill(T *tile, const T *p, int64_t sb, bool vector_ok, int na, int nb) {
    if constexpr (!std::is_same_v<T, Unused>) {
        constexpr int P = tile_pitch<T>();
        constexpr int VA = 16 / sizeof(T);
        constexpr int CH = kTile / VA;  // 16-byte chunks per row
        if (vector_ok) {
            constexpr int N = kTile * CH / kThreads;
            Pack<T, VA> v[N];
#pragma unroll
            for (int i = 0; i < N; ++i) {
                const int idx = threadIdx.x + kThreads * i;
                const int b = idx / CH, ac = idx % CH;
                v[i] = *reinterpret_cast<const Pack<T, VA> *>(p + b * sb + ac * VA);
            }
#pragma unroll
            for (int i = 0; i < N; ++i) {
                const int idx = threadIdx.x + kThreads * i;
                const int b = idx / CH, ac = idx % CH;
                *reinterpret_cast<Pack<T, VA> *>(tile + b * P + ac * VA) = v[i];
            }
        } else {
            const int tx = threadIdx.x & (kTile - 1), ty = threadIdx.x >> 6;
            for (int b = ty; b < nb; b += kThreads / kTile) {
                if (tx < na) tile[b * P + tx] = p[b * sb + tx];
            }
        }
    }
}

// EB elements of input k for output position (a, b .. b + EB): from the tile, a constant, or memory.
template <class T, int EB>
__device__ __forceinline__ void tile_gather(Pack<T, EB> &dst, const T *tile, bool tiled, const MapArgs &arg, int k,
                                            const T *p, int64_t sa, int64_t sb, int a, int b, int nvalid) {
    if constexpr (!std::is_same_v<T, Unused>) {
        constexpr int P = tile_pitch<T>();
        if (tiled) {
#pragma unroll
            for (int j = 0; j < EB; ++j) dst.v[j] = tile[(b + j) * P + a];
        } else if (arg.constant_mask & (1u << k)) {
            T c;
            uint64_t bits = arg.constant[k];
            memcpy(&c, &bits, sizeof(T));
#pragma unroll
            for (int j = 0; j < EB; ++j) dst.v[j] = c;
        } else {
            const T *q = p + a * sa + b * sb;
            if (sb == 0) {
                const T c = *q;
#pragma unroll
                for (int j = 0; j < EB; ++j) dst.v[j] = c;
            } else if (sb == 1 && nvalid == EB && (reinterpret_cast<uintptr_t>(q) & 15) == 0) {
                constexpr int V = 16 / sizeof(T);
#pragma unroll
                for (int j = 0; j < EB; j += V) {
                    const Pack<T, V> x = *reinterpret_cast<const Pack<T, V> *>(q + j);
#pragma unroll
                    for (int e = 0; e < V; ++e) dst.v[j + e] = x.v[e];
                }
            } else {
#pragma unroll
                for (int j = 0; j < EB; ++j)
                    if (j < nvalid) dst.v[j] = q[j * sb];
            }
        }
    }
}

template <class F>
__global__ void __launch_bounds__(kThreads) map_tile_kernel(const __grid_constant__ MapArgs a, const F f) {
    using TO = typename F::Out;
    using TA = typename F::A;
    using TB = typename F::B;
    using TC = typename F::C;
    constexpr int EB = tile_eb<TO>();
    constexpr int BC = kTile / EB;                 // sectors per tile row
    constexpr int ITEMS = kTile * BC / kThreads;   // sectors per thread
    extern __shared__ __align__(16) unsigned char tile_memory[];
    TA *tile_a = reinterpret_cast<TA *>(tile_memory);
    TB *tile_b = reinterpret_cast<TB *>(tile_memory + tile_bytes<TA>());
    TC *tile_c = reinterpret_cast<TC *>(tile_memory + tile_bytes<TA>() + tile_bytes<TB>());
    const bool ta = a.tile_mask & 2u, tb = a.tile_mask & 4u, tc = a.tile_mask & 8u;
    const int da = a.ndim - 2, db = a.ndim - 1;
    const int64_t size_a = a.sizes[da], size_b = a.sizes[db];
    const int64_t sao = a.strides[0][da];
    const int64_t saa = a.strides[1][da], sab = a.strides[1][db];
    const int64_t sba = a.strides[2][da], sbb = a.strides[2][db];
    const int64_t sca = a.strides[3][da], scb = a.strides[3][db];
    // A fixed number of resident blocks walk the tiles (B fastest): measured faster on B200 than one block per
    // tile, in either grid order.
    for (int64_t t = blockIdx.x; t < a.ntiles; t += gridDim.x) {
        int64_t jb, ja, outer;
        if (a.ntiles < (int64_t{1} << 31)) {
            const uint32_t t32 = static_cast<uint32_t>(t), nb32 = static_cast<uint32_t>(a.tiles_b), na32 = static_cast<uint32_t>(a.tiles_a);
            const uint32_t t2 = t32 / nb32;
            jb = t32 - t2 * nb32;
            const uint32_t o = t2 / na32;
            ja = t2 - o * na32;
            outer = o;
        } else {
            jb = t % a.tiles_b;
            const int64_t t2 = t / a.tiles_b;
            ja = t2 % a.tiles_a;
            outer = t2 / a.tiles_a;
        }
        int64_t off[kOperands] = {0, 0, 0, 0};
        for (int d = da - 1; d >= 0; --d) {
            const int64_t size = a.sizes[d];
            const int64_t q = outer / size;
            const int64_t i = outer - q * size;
#pragma unroll
            for (int k = 0; k < kOperands; ++k) off[k] += i * a.strides[k][d];
            outer = q;
        }
        const int64_t a0 = ja * kTile, b0 = jb * kTile;
        const int na = static_cast<int>(size_a - a0 < kTile ? size_a - a0 : kTile);
        const int nb = static_cast<int>(size_b - b0 < kTile ? size_b - b0 : kTile);
        const bool whole = na == kTile && nb == kTile;
        // pointers at the tile's corner (a0, b0)
        TO *po = operand_row<TO>(a, 0, off[0] + a0 * sao + b0);
        const TA *pa = operand_row<TA>(a, 1, off[1] + a0 * saa + b0 * sab);
        const TB *pb = operand_row<TB>(a, 2, off[2] + a0 * sba + b0 * sbb);
        const TC *pc = operand_row<TC>(a, 3, off[3] + a0 * sca + b0 * scb);
        if (ta) tile_fill<TA>(tile_a, pa, sab, whole && vector_aligned<TA, 16 / size_or<TA>(1)>(pa) && (sab * size_or<TA>(1)) % 16 == 0, na, nb);
        if (tb) tile_fill<TB>(tile_b, pb, sbb, whole && vector_aligned<TB, 16 / size_or<TB>(1)>(pb) && (sbb * size_or<TB>(1)) % 16 == 0, na, nb);
        if (tc) tile_fill<TC>(tile_c, pc, scb, whole && vector_aligned<TC, 16 / size_or<TC>(1)>(pc) && (scb * size_or<TC>(1)) % 16 == 0, na, nb);
        __syncthreads();
        const bool out_vector = whole && (reinterpret_cast<uintptr_t>(po) & 15) == 0 && (sao * sizeof(TO)) % 16 == 0;
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
            const int idx = threadIdx.x + kThreads * it;
            const int aa = idx % kTile, bb = (idx / kTile) * EB;
            if (aa < na && bb < nb) {
                const int nvalid = nb - bb < EB ? nb - bb : EB;
                Pack<TA, EB> va;
                Pack<TB, EB> vb;
                Pack<TC, EB> vc;
                tile_gather<TA, EB>(va, tile_a, ta, a, 1, pa, saa, sab, aa, bb, nvalid);
                tile_gather<TB, EB>(vb, tile_b, tb, a, 2, pb, sba, sbb, aa, bb, nvalid);
                tile_gather<TC, EB>(vc, tile_c, tc, a, 3, pc, sca, scb, aa, bb, nvalid);
                Pack<TO, EB> vo;
                apply_all<F, EB>(vo, f, va, vb, vc);
                TO *q = po + aa * sao + bb;
                if (out_vector) {
                    constexpr int V = 16 / sizeof(TO);
#pragma unroll
                    for (int j = 0; j < EB; j += V) {
                        Pack<TO, V> x;
#pragma unroll
                        for (int e = 0; e < V; ++e) x.v[e] = vo.v[j + e];
                        *reinterpret_cast<Pack<TO, V> *>(q + j) = x;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < EB; ++j)
                        if (j < nvalid) q[j] = vo.v[j];
                }
            }
        }
        __syncthreads();
    }
}

// One operand of a launch: a description, or (for inputs) a constant given by its bits.
struct MapOperand {
    const hmc_tensor_desc *desc = nullptr;
    uint64_t bits = 0;
    bool constant = false;
};

inline MapOperand tensor_operand(const hmc_tensor_desc *d) { return MapOperand{d, 0, false}; }
inline MapOperand constant_operand(uint64_t bits) { return MapOperand{nullptr, bits, true}; }

// Checks one description; `what` names the operand in the message.
hmc_status check_desc(const hmc_tensor_desc *d, const char *what);
// Checks that all descriptions are valid and agree in ndim and sizes; `count` = number of elements.
hmc_status check_operands(const hmc_tensor_desc *const *descs, int n, int64_t *count);

// Fills `a` for `out` and up to three inputs (absent ones: default MapOperand with desc null and
// constant false). `vec` and `unr` are those of the functor.
void build_map_args(MapArgs &a, const hmc_tensor_desc *out, const MapOperand *inputs, int ninputs, int vec, int unr);

template <class F>
hmc_status launch_map(hmc_context_t ctx, const F &f, const hmc_tensor_desc *out, const MapOperand *inputs, int ninputs) {
    MapArgs a;
    build_map_args(a, out, inputs, ninputs, vec_of<F>(), unroll_of<F>());
    if (a.items == 0) return HMC_OK;
    {
        LeanArgs lean;
        const int sizes[kOperands] = {static_cast<int>(sizeof(typename F::Out)), size_or_zero<typename F::A>(),
                                      size_or_zero<typename F::B>(), size_or_zero<typename F::C>()};
        if (a.tile_mask == 0 && build_lean_args(lean, a, sizes, vec_of<F>())) {
            const int64_t chunk = static_cast<int64_t>(kThreads) * vec_of<F>() * unroll_of<F>();
            dim3 grid(static_cast<unsigned>(ceil_div(lean.n0, chunk)), static_cast<unsigned>(lean.rows < 65535 ? lean.rows : 65535));
            map_lean_kernel<F><<<grid, kThreads, 0, ctx->stream>>>(lean, f);
            return launch_status("elementwise kernel launch");
        }
    }
    if (a.tile_mask != 0) {
        const size_t smem = tile_bytes<typename F::A>() + tile_bytes<typename F::B>() + tile_bytes<typename F::C>();
        if (smem > 48 * 1024) {
            static bool raised = false;  // per instantiation; the attribute is sticky for the function
            if (!raised) {
                cudaError_t err = cudaFuncSetAttribute(map_tile_kernel<F>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                       static_cast<int>(smem));
                if (err != cudaSuccess) return cuda_fail(err, "cudaFuncSetAttribute");
                raised = true;
            }
        }
        const int64_t tcap = static_cast<int64_t>(ctx->sm_count) * 32;
        const unsigned tgrid = static_cast<unsigned>(a.ntiles < tcap ? a.ntiles : tcap);
        map_tile_kernel<F><<<tgrid, kThreads, smem, ctx->stream>>>(a, f);
        return launch_status("tiled elementwise kernel launch");
    }
    // A few items per block: enough blocks for the hardware scheduler to balance them over the SMs (many
    // more than are resident at once), while a thread's set-up (operand modes, row offsets) is paid once
    // per several vectors rather than once per vector.
    const int64_t cap = int64_t{1} << 30;
    const int64_t per_block = a.items >= static_cast<int64_t>(ctx->sm_count) * 32 ? HMC_MAP_ITEMS_PER_BLOCK : 1;
    const int64_t blocks = ceil_div(a.items, per_block);
    unsigned grid = static_cast<unsigned>(blocks < cap ? blocks : cap);
    map_kernel<F><<<grid, kThreads, 0, ctx->stream>>>(a, f);
    return launch_status("elementwise kernel launch");
}

}  // namespace hmc
