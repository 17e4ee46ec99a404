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
    int32_t tile_stages;              // shared-memory stages of the tile ring
    uint32_t stage_bytes;             // bytes of one stage: the tiles of the transposed inputs
    uint32_t tile_off[kOperands];     // where input k's tile lies within a stage
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

// A functor may state its own unrolling as a member kUnroll (one whose operands are mostly broadcasts, which the
// rule below counts as traffic, knows better how many bytes it really has in flight).
template <class F, class = void> struct has_unroll : std::false_type {};
template <class F> struct has_unroll<F, std::void_t<decltype(F::kUnroll)>> : std::true_type {};

template <class F> constexpr int unroll_of() {
    if constexpr (has_unroll<F>::value) return F::kUnroll;
    // About 64 bytes of inputs in flight per thread and iteration (the loads of all inputs are issued before
    // the first store), and never more than 64 bytes of output held at once.
    constexpr int in_bytes = (size_or_zero<typename F::A>() + size_or_zero<typename F::B>() + size_or_zero<typename F::C>()) *
                             vec_of<F>();
    constexpr int out_bytes = static_cast<int>(sizeof(typename F::Out)) * vec_of<F>();
    constexpr int by_in = in_bytes == 0 ? 4 : (in_bytes >= 64 ? 1 : (in_bytes >= 32 ? 2 : 4));
    constexpr int by_out = out_bytes >= 64 ? 1 : (out_bytes >= 32 ? 2 : 4);
    return by_in < by_out ? by_in : by_out;
}

// 32 bytes in one instruction (sm_100's 256-bit global accesses): a lane then moves a whole sector, where two
// 16-byte accesses leave half of every sector to the second instruction. The address is 32-byte aligned.
struct alignas(32) Bytes32 {
    uint32_t w[8];
};
__device__ __forceinline__ Bytes32 load_32_bytes(const void *p) {
    Bytes32 v;
    // not volatile: the compiler may schedule it like any other load (measurably faster than a fixed order)
    asm("ld.global.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]), "=r"(v.w[6]), "=r"(v.w[7])
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void store_32_bytes(void *p, const Bytes32 &v) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(v.w[0]), "r"(v.w[1]), "r"(v.w[2]), "r"(v.w[3]),
                 "r"(v.w[4]), "r"(v.w[5]), "r"(v.w[6]), "r"(v.w[7])
                 : "memory");
}
// A vector of a row; `wide`: the vector's address is a multiple of 32 (it matters for vectors of 32 and 64 bytes).
template <class T, int VEC>
__device__ __forceinline__ void vector_load(Pack<T, VEC> &dst, const T *p, bool wide) {
    constexpr int kBytes = static_cast<int>(sizeof(T)) * VEC;
    if constexpr (kBytes % 32 == 0) {
        if (wide) {
#pragma unroll
            for (int i = 0; i < kBytes / 32; ++i) {
                const Bytes32 v = load_32_bytes(reinterpret_cast<const char *>(p) + 32 * i);
                memcpy(reinterpret_cast<char *>(&dst) + 32 * i, &v, 32);
            }
            return;
        }
    }
    dst = *reinterpret_cast<const Pack<T, VEC> *>(p);
}
template <class T, int VEC>
__device__ __forceinline__ void vector_store(T *p, const Pack<T, VEC> &src, bool wide) {
    constexpr int kBytes = static_cast<int>(sizeof(T)) * VEC;
    if constexpr (kBytes % 32 == 0) {
        if (wide) {
#pragma unroll
            for (int i = 0; i < kBytes / 32; ++i) {
                Bytes32 v;
                memcpy(&v, reinterpret_cast<const char *>(&src) + 32 * i, 32);
                store_32_bytes(reinterpret_cast<char *>(p) + 32 * i, v);
            }
            return;
        }
    }
    *reinterpret_cast<Pack<T, VEC> *>(p) = src;
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
            vector_store<T, VEC>(p, src, (reinterpret_cast<uintptr_t>(p) & 31) == 0);
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
                vector_store<TO, VEC>(po + idx, vo, (reinterpret_cast<uintptr_t>(po + idx) & 31) == 0);
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
// Resident blocks per SM the lean kernel is compiled for: 4 (64 registers) by default; functors that need few
// registers can ask for more by specialising this, which puts more loads in flight for latency-bound layouts.
template <class F> struct LeanMinBlocks { static constexpr int value = 4; };
constexpr int64_t kLeanBlocksWanted = 148 * 16;  // blocks below which a launch keeps one row per block
struct LeanArgs {
    char *base[kOperands];
    int64_t row_stride[kOperands];  // elements
    uint32_t inner[kOperands];      // 1: unit stride, 0: one value per row
    uint64_t constant[kOperands];
    uint32_t constant_mask;
    uint32_t n0;                    // inner size (< 2^31)
    uint32_t wide_mask;             // bit k: operand k's rows start on 32-byte boundaries
    int64_t rows;
};

template <class T, int VEC>
__device__ __forceinline__ void lean_load(Pack<T, VEC> &dst, const T *row, uint32_t inner, uint32_t col, const Pack<T, 1> &c, bool wide) {
    if constexpr (!std::is_same_v<T, Unused>) {
        if (inner) {
            vector_load<T, VEC>(dst, row + col, wide);
        } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j) dst.v[j] = c.v[0];
        }
    }
}

template <class F>
__global__ void __launch_bounds__(kThreads, LeanMinBlocks<F>::value) map_lean_kernel(const __grid_constant__ LeanArgs a, const F f) {
    using TO = typename F::Out;
    using TA = typename F::A;
    using TB = typename F::B;
    using TC = typename F::C;
    constexpr int VEC = vec_of<F>();
    constexpr int UNR = unroll_of<F>();
    constexpr uint32_t kStep = kThreads * VEC;
    const uint32_t col0 = blockIdx.x * (kStep * UNR) + threadIdx.x * VEC;
    const bool ka = a.constant_mask & 2u, kb = a.constant_mask & 4u, kc = a.constant_mask & 8u;
    const bool wo = a.wide_mask & 1u, wa = a.wide_mask & 2u, wb = a.wide_mask & 4u, wc = a.wide_mask & 8u;
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
                lean_load<TA, VEC>(va[u], pa, a.inner[1] && !ka, col, ca, wa);
                lean_load<TB, VEC>(vb[u], pb, a.inner[2] && !kb, col, cb, wb);
                lean_load<TC, VEC>(vc[u], pc, a.inner[3] && !kc, col, cc, wc);
            }
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                const uint32_t col = col0 + u * kStep;
                Pack<TO, VEC> vo;
                apply_all<F, VEC>(vo, f, va[u], vb[u], vc[u]);
                vector_store<TO, VEC>(po + col, vo, wo);
            }
        } else {
            // the ragged end of a row: whole vectors while they fit, then single elements
#pragma unroll
            for (int u = 0; u < UNR; ++u) {
                const uint32_t col = col0 + u * kStep;
                if (col + VEC <= a.n0) {
                    lean_load<TA, VEC>(va[0], pa, a.inner[1] && !ka, col, ca, wa);
                    lean_load<TB, VEC>(vb[0], pb, a.inner[2] && !kb, col, cb, wb);
                    lean_load<TC, VEC>(vc[0], pc, a.inner[3] && !kc, col, cc, wc);
                    Pack<TO, VEC> vo;
                    apply_all<F, VEC>(vo, f, va[0], vb[0], vc[0]);
                    vector_store<TO, VEC>(po + col, vo, wo);
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
// along the last dimension B (a transposed view). Work is cut into square tiles of (A, B): 128 x 128
// elements when every operand has 1- or 2-byte elements, 64 x 64 otherwise, so that the runs a tile reads
// and writes are 128 to 512 bytes long and the bookkeeping per tile is spread over at least four 16-byte
// outputs per thread. A tile of a transposed operand comes into shared memory as rows along A (16-byte
// asynchronous copies straight from global to shared memory), and is read back against the grain: a thread
// produces one 16-byte piece of an output row (NB consecutive B at GA consecutive A), eight neighbouring
// lanes produce 128 consecutive bytes of that row, so global loads and stores both move whole lines. The
// 16-byte chunks of a shared-memory row are permuted by the row's output-chunk number (XOR), which makes
// the against-the-grain reads conflict free when input and output elements have the same size. A block
// keeps the copies of its next tiles in flight in a ring of stages while it computes the current one.
// Tiles on the boundary, and operands that are not 16-byte aligned, are filled element by element into the
// same layout.
#ifndef HMC_TILE_MIN_BLOCKS
#define HMC_TILE_MIN_BLOCKS 3
#endif
#ifndef HMC_TILE_RING_KB
#define HMC_TILE_RING_KB 40
#endif
constexpr int kTileStagesMax = 4;
constexpr int kTileKnownDevices = 64;                        // GPUs whose launch limits are remembered
constexpr size_t kTileRingBytes = HMC_TILE_RING_KB * 1024;   // shared memory a block's ring aims for

// The tile edge, in elements, of a functor's launches.
template <class F> constexpr int tile_dim() {
    constexpr int so = sizeof(typename F::Out);
    constexpr int sa = size_or_zero<typename F::A>(), sb = size_or_zero<typename F::B>(), sc = size_or_zero<typename F::C>();
    constexpr int m1 = so > sa ? so : sa, m2 = sb > sc ? sb : sc;
    return (m1 > m2 ? m1 : m2) <= 2 ? 128 : 64;
}
template <class T, int TD> constexpr size_t tile_bytes() {
    if constexpr (std::is_same_v<T, Unused>) return 0;
    else return static_cast<size_t>(TD) * TD * sizeof(T);
}
template <class TO> constexpr int tile_nb() { return 16 / static_cast<int>(sizeof(TO)); }  // B's per thread: 16 bytes of output
template <class TO> constexpr int tile_ga() { return sizeof(TO) <= 2 ? 2 : 1; }            // A's per thread

// Byte offset of element (row r along B, a along A) of a tile whose rows are cut into tasks of NB rows.
template <class T, int NB, int TD>
__device__ __forceinline__ uint32_t tile_offset(int r, int a) {
    constexpr int E = sizeof(T);
    constexpr int kChunks = TD * E / 16;
    constexpr int kMask = (kChunks < 8 ? kChunks : 8) - 1;
    const uint32_t byte = static_cast<uint32_t>(a) * E;
    return static_cast<uint32_t>(r) * (TD * E) + (((byte >> 4) ^ (static_cast<uint32_t>(r / NB) & kMask)) << 4) + (byte & 15u);
}

__device__ __forceinline__ void async_copy_16(void *shared_dst, const void *global_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(shared_dst))),
                 "l"(global_src)
                 : "memory");
}
__device__ __forceinline__ void async_copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// Waits until at most `pending` of this thread's committed groups are still in flight.
__device__ __forceinline__ void async_copy_wait(int pending) {
    switch (pending) {
        case 0: asm volatile("cp.async.wait_group 0;" ::: "memory"); break;
        case 1: asm volatile("cp.async.wait_group 1;" ::: "memory"); break;
        case 2: asm volatile("cp.async.wait_group 2;" ::: "memory"); break;
        default: asm volatile("cp.async.wait_group 3;" ::: "memory"); break;
    }
}

// Starts the copies of a whole, aligned tile: row r of the tile is the TD elements at p + r * sb.
template <class T, int NB, int TD>
__device__ __forceinline__ void tile_fetch(unsigned char *tile, const T *p, int64_t sb) {
    if constexpr (!std::is_same_v<T, Unused>) {
        constexpr int E = sizeof(T);
        constexpr int CH = TD * E / 16;  // 16-byte chunks per row
        constexpr int N = (TD * CH + kThreads - 1) / kThreads;
        constexpr int kMask = (CH < 8 ? CH : 8) - 1;
        const char *src = reinterpret_cast<const char *>(p);
        const int64_t row_bytes = sb * E;
#pragma unroll
        for (int i = 0; i < N; ++i) {
            const int x = threadIdx.x + kThreads * i;
            const int r = x / CH, c = x % CH;
            if (TD * CH % kThreads == 0 || r < TD)
                async_copy_16(tile + r * (TD * E) + ((c ^ ((r / NB) & kMask)) << 4), src + r * row_bytes + c * 16);
        }
    }
}

// The same tile element by element, for tiles on the boundary and rows that are not 16-byte aligned.
template <class T, int NB, int TD>
__device__ __forceinline__ void tile_fill(unsigned char *tile, const T *p, int64_t sb, int na, int nb) {
    if constexpr (!std::is_same_v<T, Unused>) {
        const int tx = threadIdx.x % TD;
        for (int r = threadIdx.x / TD; r < nb; r += kThreads / TD) {
            if (tx < na) *reinterpret_cast<T *>(tile + tile_offset<T, NB, TD>(r, tx)) = p[r * sb + tx];
        }
    }
}

// Input k at output positions (a0 + g, b0 + j), g < GA, j < NB, into dst.v[g * NB + j]: from the tile, a
// constant, or memory.
template <class T, int GA, int NB, int TD>
__device__ __forceinline__ void tile_gather(Pack<T, GA * NB> &dst, const unsigned char *tile, bool tiled, const MapArgs &arg, int k,
                                            const T *p, int64_t sa, int64_t sb, int a0, int b0, int na, int nvalid) {
    if constexpr (!std::is_same_v<T, Unused>) {
        if (tiled) {
            // b0 is a multiple of NB, so the NB rows of a task share one chunk permutation: one address, then
            // constant row steps
            const unsigned char *first = tile + tile_offset<T, NB, TD>(b0, a0);
#pragma unroll
            for (int j = 0; j < NB; ++j) {
                const Pack<T, GA> w = *reinterpret_cast<const Pack<T, GA> *>(first + j * (TD * static_cast<int>(sizeof(T))));
#pragma unroll
                for (int g = 0; g < GA; ++g) dst.v[g * NB + j] = w.v[g];
            }
        } else if (arg.constant_mask & (1u << k)) {
            T c;
            uint64_t bits = arg.constant[k];
            memcpy(&c, &bits, sizeof(T));
#pragma unroll
            for (int j = 0; j < GA * NB; ++j) dst.v[j] = c;
        } else {
#pragma unroll
            for (int g = 0; g < GA; ++g) {
                if (a0 + g >= na) continue;
                const T *q = p + (a0 + g) * sa + b0 * sb;
                constexpr int V = NB * sizeof(T) >= 16 ? 16 / static_cast<int>(sizeof(T)) : NB;  // elements per vector load
                if (sb == 0) {
                    const T c = *q;
#pragma unroll
                    for (int j = 0; j < NB; ++j) dst.v[g * NB + j] = c;
                } else if (sb == 1 && nvalid == NB && (reinterpret_cast<uintptr_t>(q) & (V * sizeof(T) - 1)) == 0) {
#pragma unroll
                    for (int j = 0; j < NB; j += V) {
                        const Pack<T, V> x = *reinterpret_cast<const Pack<T, V> *>(q + j);
#pragma unroll
                        for (int e = 0; e < V; ++e) dst.v[g * NB + j + e] = x.v[e];
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < NB; ++j)
                        if (j < nvalid) dst.v[g * NB + j] = q[j * sb];
                }
            }
        }
    }
}

// A tile number as coordinates: the tile index along the dimension that neighbouring tile numbers walk
// first, along the other one, and the index over the outer dimensions. A block's tile numbers advance by
// the grid size; the coordinates follow by carries instead of divisions.
struct TileCursor {
    int64_t jf, js, outer;
};
__device__ __forceinline__ TileCursor tile_cursor(int64_t t, int64_t fast, int64_t slow) {
    TileCursor c;
    if (t < (int64_t{1} << 31) && fast < (int64_t{1} << 31) && slow < (int64_t{1} << 31)) {
        const uint32_t t32 = static_cast<uint32_t>(t), nf = static_cast<uint32_t>(fast), ns = static_cast<uint32_t>(slow);
        const uint32_t t2 = t32 / nf, o = t2 / ns;
        c.jf = t32 - t2 * nf;
        c.js = t2 - o * ns;
        c.outer = o;
    } else {
        c.jf = t % fast;
        const int64_t t2 = t / fast;
        c.js = t2 % slow;
        c.outer = t2 / slow;
    }
    return c;
}
__device__ __forceinline__ void tile_advance(TileCursor &c, const TileCursor &step, int64_t fast, int64_t slow) {
    c.jf += step.jf;
    const int64_t c1 = c.jf >= fast;
    c.jf -= c1 ? fast : 0;
    c.js += step.js + c1;
    const int64_t c2 = c.js >= slow;
    c.js -= c2 ? slow : 0;
    c.outer += step.outer + c2;
}

// Where a tile lies: pointers at its corner, its extent, and whether its transposed operands can all be
// fetched by 16-byte asynchronous copies.
template <class F>
struct TileGeom {
    typename F::Out *po;
    const typename F::A *pa;
    const typename F::B *pb;
    const typename F::C *pc;
    int na, nb;
    bool whole, async;
};

template <class T>
__device__ __forceinline__ bool tile_rows_aligned(const T *p, int64_t sb) {
    if constexpr (std::is_same_v<T, Unused>) return true;
    else return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && (sb * static_cast<int64_t>(sizeof(T))) % 16 == 0;
}

template <class F>
__device__ __forceinline__ TileGeom<F> tile_geometry(const MapArgs &a, const TileCursor &c) {
    using TO = typename F::Out;
    using TA = typename F::A;
    using TB = typename F::B;
    using TC = typename F::C;
    constexpr int TD = tile_dim<F>();
    const int da = a.ndim - 2, db = a.ndim - 1;
    const int64_t jb = c.jf, ja = c.js;  // neighbouring tile numbers walk B first (either order measured the same)
    int64_t off[kOperands] = {0, 0, 0, 0};
    int64_t outer = c.outer;
    for (int d = da - 1; d >= 0; --d) {
        const int64_t size = a.sizes[d];
        const int64_t q = outer / size;
        const int64_t i = outer - q * size;
#pragma unroll
        for (int k = 0; k < kOperands; ++k) off[k] += i * a.strides[k][d];
        outer = q;
    }
    const int64_t a0 = ja * TD, b0 = jb * TD;
    const int64_t size_a = a.sizes[da], size_b = a.sizes[db];
    TileGeom<F> g;
    g.na = static_cast<int>(size_a - a0 < TD ? size_a - a0 : TD);
    g.nb = static_cast<int>(size_b - b0 < TD ? size_b - b0 : TD);
    g.whole = g.na == TD && g.nb == TD;
    g.po = operand_row<TO>(a, 0, off[0] + a0 * a.strides[0][da] + b0);
    g.pa = operand_row<TA>(a, 1, off[1] + a0 * a.strides[1][da] + b0 * a.strides[1][db]);
    g.pb = operand_row<TB>(a, 2, off[2] + a0 * a.strides[2][da] + b0 * a.strides[2][db]);
    g.pc = operand_row<TC>(a, 3, off[3] + a0 * a.strides[3][da] + b0 * a.strides[3][db]);
    g.async = g.whole && (!(a.tile_mask & 2u) || tile_rows_aligned<TA>(g.pa, a.strides[1][db])) &&
              (!(a.tile_mask & 4u) || tile_rows_aligned<TB>(g.pb, a.strides[2][db])) &&
              (!(a.tile_mask & 8u) || tile_rows_aligned<TC>(g.pc, a.strides[3][db]));
    return g;
}

template <class F>
__global__ void __launch_bounds__(kThreads, HMC_TILE_MIN_BLOCKS) map_tile_kernel(const __grid_constant__ MapArgs a, const F f) {
    using TO = typename F::Out;
    using TA = typename F::A;
    using TB = typename F::B;
    using TC = typename F::C;
    constexpr int TD = tile_dim<F>();
    constexpr int NB = tile_nb<TO>();
    constexpr int GA = tile_ga<TO>();
    constexpr int CB = TD / NB;                     // 16-byte pieces per output row of the tile
    constexpr int LB = CB < 8 ? CB : 8;             // neighbouring lanes along B
    constexpr int AG = TD / GA;                     // groups of A
    constexpr int TASKS = AG * CB;
    constexpr int ITEMS = (TASKS + kThreads - 1) / kThreads;
    extern __shared__ __align__(128) unsigned char tile_memory[];
    const bool ta = a.tile_mask & 2u, tb = a.tile_mask & 4u, tc = a.tile_mask & 8u;
    const int da = a.ndim - 2, db = a.ndim - 1;
    const int64_t sao = a.strides[0][da];
    const int64_t saa = a.strides[1][da], sab = a.strides[1][db];
    const int64_t sba = a.strides[2][da], sbb = a.strides[2][db];
    const int64_t sca = a.strides[3][da], scb = a.strides[3][db];
    const int stages = a.tile_stages;
    // A fixed number of resident blocks walk the tiles: block i takes tiles i, i + grid, i + 2 grid, ...
    const int64_t fast = a.tiles_b, slow = a.tiles_a;
    const TileCursor step = tile_cursor(gridDim.x, fast, slow);
    TileCursor ahead = tile_cursor(blockIdx.x, fast, slow);  // the tile whose copies are started next
    TileCursor here = ahead;                                 // the tile computed next
    int64_t t_ahead = blockIdx.x;
    // Starts the copies of the tile `ahead` into stage s when the tile qualifies, and closes a group either
    // way, so that every thread's groups count tiles.
    auto prefetch = [&](int s) {
        if (t_ahead < a.ntiles) {
            const TileGeom<F> g = tile_geometry<F>(a, ahead);
            if (g.async) {
                unsigned char *stage = tile_memory + s * a.stage_bytes;
                if (ta) tile_fetch<TA, NB, TD>(stage + a.tile_off[1], g.pa, sab);
                if (tb) tile_fetch<TB, NB, TD>(stage + a.tile_off[2], g.pb, sbb);
                if (tc) tile_fetch<TC, NB, TD>(stage + a.tile_off[3], g.pc, scb);
            }
        }
        async_copy_commit();
        t_ahead += gridDim.x;
        tile_advance(ahead, step, fast, slow);
    };
    for (int s = 0; s < stages - 1; ++s) prefetch(s);
    int s = 0;
    for (int64_t t = blockIdx.x; t < a.ntiles; t += gridDim.x) {
        async_copy_wait(stages - 2);  // this thread's copies of tile t have landed
        __syncthreads();              // and everybody's; and everybody is done with the stage refilled next
        prefetch(s == 0 ? stages - 1 : s - 1);
        const TileGeom<F> g = tile_geometry<F>(a, here);
        tile_advance(here, step, fast, slow);
        unsigned char *stage = tile_memory + s * a.stage_bytes;
        const unsigned char *tile_a = stage + a.tile_off[1], *tile_b = stage + a.tile_off[2], *tile_c = stage + a.tile_off[3];
        if (!g.async) {
            if (ta) tile_fill<TA, NB, TD>(stage + a.tile_off[1], g.pa, sab, g.na, g.nb);
            if (tb) tile_fill<TB, NB, TD>(stage + a.tile_off[2], g.pb, sbb, g.na, g.nb);
            if (tc) tile_fill<TC, NB, TD>(stage + a.tile_off[3], g.pc, scb, g.na, g.nb);
            __syncthreads();
        }
        const bool out_vector = g.whole && (reinterpret_cast<uintptr_t>(g.po) & 15) == 0 && (sao * sizeof(TO)) % 16 == 0;
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
            const int q = threadIdx.x + kThreads * it;
            const int rest = q / LB;
            const int a0 = (rest % AG) * GA, b0 = ((rest / AG) * LB + q % LB) * NB;
            if ((TASKS % kThreads == 0 || q < TASKS) && a0 < g.na && b0 < g.nb) {
                const int nvalid = g.nb - b0 < NB ? g.nb - b0 : NB;
                Pack<TA, GA * NB> va;
                Pack<TB, GA * NB> vb;
                Pack<TC, GA * NB> vc;
                tile_gather<TA, GA, NB, TD>(va, tile_a, ta, a, 1, g.pa, saa, sab, a0, b0, g.na, nvalid);
                tile_gather<TB, GA, NB, TD>(vb, tile_b, tb, a, 2, g.pb, sba, sbb, a0, b0, g.na, nvalid);
                tile_gather<TC, GA, NB, TD>(vc, tile_c, tc, a, 3, g.pc, sca, scb, a0, b0, g.na, nvalid);
                Pack<TO, GA * NB> vo;
                apply_all<F, GA * NB>(vo, f, va, vb, vc);
#pragma unroll
                for (int gg = 0; gg < GA; ++gg) {
                    if (a0 + gg >= g.na) continue;
                    TO *out = g.po + (a0 + gg) * sao + b0;
                    if (out_vector) {
                        Pack<TO, NB> x;
#pragma unroll
                        for (int e = 0; e < NB; ++e) x.v[e] = vo.v[gg * NB + e];
                        *reinterpret_cast<Pack<TO, NB> *>(out) = x;
                    } else {
#pragma unroll
                        for (int j = 0; j < NB; ++j)
                            if (j < nvalid) out[j] = vo.v[gg * NB + j];
                    }
                }
            }
        }
        s = s + 1 == stages ? 0 : s + 1;
    }
    async_copy_wait(0);
}

}  // namespace hmc

#include "transpose16.cuh"

namespace hmc {

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

// Queues transpose16_kernel for the layout in `a` when it qualifies (alignment of both sides); false: not taken.
template <class F>
bool launch_transpose16(hmc_context_t ctx, const MapArgs &a, const F &f, hmc_status &status) {
    if (ctx->status == nullptr) return false;
    const int da = a.ndim - 2, db = a.ndim - 1;
    const int64_t size_a = a.sizes[da], size_b = a.sizes[db], outer = a.ndim == 3 ? a.sizes[0] : 1;
    CUtensorMap in_map, out_map;
    if (!t16_encode_map(&in_map, a.base[1], size_a, size_b, outer, a.strides[1][db], a.ndim == 3 ? a.strides[1][0] : 0)) return false;
    if (!t16_encode_map(&out_map, a.base[0], size_b, size_a, outer, a.strides[0][da], a.ndim == 3 ? a.strides[0][0] : 0)) return false;
    const int64_t tiles_a = ceil_div(size_a, kT16Tile), tiles_b = ceil_div(size_b, kT16Tile);
    if (tiles_a * tiles_b >= (int64_t{1} << 31) / (outer > 0 ? outer : 1)) return false;  // the kernel counts tiles in 32 bits
    Transpose16Args args;
    args.tiles_a = static_cast<uint32_t>(tiles_a);
    args.tiles_b = static_cast<uint32_t>(tiles_b);
    args.tiles = static_cast<uint32_t>(outer * tiles_a * tiles_b);
    static bool raised[kTileKnownDevices] = {};
    if (ctx->device >= kTileKnownDevices || !raised[ctx->device]) {
        cudaError_t err = cudaFuncSetAttribute(transpose16_kernel<F>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(kT16SharedBytes));
        if (err != cudaSuccess) {
            status = cuda_fail(err, "cudaFuncSetAttribute");
            return true;
        }
        if (ctx->device < kTileKnownDevices) raised[ctx->device] = true;
    }
    const int64_t resident = static_cast<int64_t>(ctx->sm_count) * kT16BlocksPerSm;
    const unsigned grid = static_cast<unsigned>(static_cast<int64_t>(args.tiles) < resident ? args.tiles : resident);
    transpose16_kernel<F><<<grid, kT16Threads, kT16SharedBytes, ctx->stream>>>(in_map, out_map, args, f, ctx->status);
    status = launch_status("transposing kernel launch");
    return true;
}

// Queues transpose16_three_kernel for the layout in `a` when it qualifies: the first input transposed and of 2-byte
// elements, the output with unit stride along the last dimension, the other two inputs tensors of any strides.
template <class F>
bool launch_transpose16_three(hmc_context_t ctx, const MapArgs &a, const F &f, hmc_status &status) {
    if (ctx->status == nullptr) return false;
    const int da = a.ndim - 2, db = a.ndim - 1;
    if (a.strides[0][db] != 1) return false;
    const int64_t size_a = a.sizes[da], size_b = a.sizes[db], outer = a.ndim == 3 ? a.sizes[0] : 1;
    CUtensorMap in_map;
    if (!t16_encode_map(&in_map, a.base[1], size_a, size_b, outer, a.strides[1][db], a.ndim == 3 ? a.strides[1][0] : 0)) return false;
    const int64_t tiles_a = ceil_div(size_a, kT16Tile), tiles_b = ceil_div(size_b, kT16Tile);
    if (tiles_a * tiles_b >= (int64_t{1} << 31) / (outer > 0 ? outer : 1) || size_a >= (int64_t{1} << 31) - kT16Tile ||
        size_b >= (int64_t{1} << 31) - kT16Tile) {
        return false;  // the kernel counts tiles, rows and columns in 32 bits
    }
    Transpose16Args3 args;
    args.tiles_a = static_cast<uint32_t>(tiles_a);
    args.tiles_b = static_cast<uint32_t>(tiles_b);
    args.tiles = static_cast<uint32_t>(outer * tiles_a * tiles_b);
    args.size_a = size_a;
    args.size_b = size_b;
    args.out = a.base[0];
    args.out_stride_a = a.strides[0][da];
    args.out_stride_outer = a.ndim == 3 ? a.strides[0][0] : 0;
    args.b = Transpose16Operand{a.base[2], a.strides[2][da], a.strides[2][db], a.ndim == 3 ? a.strides[2][0] : 0};
    args.c = Transpose16Operand{a.base[3], a.strides[3][da], a.strides[3][db], a.ndim == 3 ? a.strides[3][0] : 0};
    constexpr size_t kShared = static_cast<size_t>(kT16Stages) * kT16TileBytes + 1024;
    const int64_t resident = static_cast<int64_t>(ctx->sm_count) * kT16BlocksPerSm;
    const unsigned grid = static_cast<unsigned>(static_cast<int64_t>(args.tiles) < resident ? args.tiles : resident);
    transpose16_three_kernel<F><<<grid, kT16Threads, kShared, ctx->stream>>>(in_map, args, f, ctx->status);
    status = launch_status("transposing kernel launch");
    return true;
}

// Functors of three inputs that want the kernel above when only their first input is transposed say so with a member
// kTransposedFirst.
template <class F, class = void> struct wants_transposed_first : std::false_type {};
template <class F> struct wants_transposed_first<F, std::void_t<decltype(F::kTransposedFirst)>> : std::bool_constant<F::kTransposedFirst> {};

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
            // A block takes up to four rows (row y, y + grid.y, ...) while that leaves enough blocks to fill the GPU
            // several times over: a thread's set-up is paid once, and a quarter of the blocks are scheduled.
            // Measured on B200 for bf16 [8192, 8192] times a row-broadcast scale: 47.1 us with one row a block, 43.4
            // with two, 43.0 with four, 45.0 with eight. (Cutting a long single row into such rows as well measured
            // 4 % slower for a bf16 silu and 2 % slower for an f32 product of 2^29 elements.)
            const int64_t gx = ceil_div(lean.n0, chunk);
            int64_t per_block = 1;
            while (per_block < 4 && gx * ceil_div(lean.rows, per_block * 2) >= kLeanBlocksWanted) per_block *= 2;
            const int64_t gy = ceil_div(lean.rows, per_block);
            dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy < 65535 ? gy : 65535));
            map_lean_kernel<F><<<grid, kThreads, 0, ctx->stream>>>(lean, f);
            return launch_status("elementwise kernel launch");
        }
    }
    if constexpr (sizeof(typename F::Out) == 2 && size_or_zero<typename F::A>() == 2 && std::is_same_v<typename F::B, Unused> &&
                  std::is_same_v<typename F::C, Unused>) {
        // one transposed input of 2-byte elements, two or three dimensions: the copy engine and the matrix
        // load / store instructions do the transposition
        if (a.tile_mask == 2u && a.constant_mask == 0 && (a.ndim == 2 || a.ndim == 3)) {
            hmc_status done = HMC_OK;
            if (launch_transpose16<F>(ctx, a, f, done)) return done;
        }
    }
    if constexpr (wants_transposed_first<F>::value && size_or_zero<typename F::A>() == 2) {
        if (a.tile_mask == 2u && a.constant_mask == 0 && (a.ndim == 2 || a.ndim == 3)) {
            hmc_status done = HMC_OK;
            if (launch_transpose16_three<F>(ctx, a, f, done)) return done;
        }
    }
    if (a.tile_mask != 0) {
        constexpr int TD = tile_dim<F>();
        const size_t tb[kOperands] = {0, tile_bytes<typename F::A, TD>(), tile_bytes<typename F::B, TD>(), tile_bytes<typename F::C, TD>()};
        {
            const int da = a.ndim - 2, db = a.ndim - 1;
            a.tiles_a = ceil_div(a.sizes[da], TD);
            a.tiles_b = ceil_div(a.sizes[db], TD);
            int64_t outer = 1;
            for (int d = 0; d < da; ++d) outer *= a.sizes[d];
            a.ntiles = outer * a.tiles_a * a.tiles_b;
        }
        a.stage_bytes = 0;
        for (int k = 1; k < kOperands; ++k) {
            a.tile_off[k] = a.stage_bytes;
            if (a.tile_mask & (1u << k)) a.stage_bytes += static_cast<uint32_t>(tb[k]);
        }
        const int fit = static_cast<int>(kTileRingBytes / a.stage_bytes);
        a.tile_stages = fit < 2 ? 2 : (fit > kTileStagesMax ? kTileStagesMax : fit);
        const size_t smem = static_cast<size_t>(a.stage_bytes) * a.tile_stages;
        // The shared-memory limit and the number of resident blocks, per instantiation, GPU and ring size.
        struct Known { size_t raised = 0, smem = 0; int blocks = 0; };
        static Known known_on[kTileKnownDevices];
        Known local;
        Known &known = ctx->device < kTileKnownDevices ? known_on[ctx->device] : local;
        if (smem > 48 * 1024 && smem > known.raised) {
            cudaError_t err = cudaFuncSetAttribute(map_tile_kernel<F>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   static_cast<int>(smem));
            if (err != cudaSuccess) return cuda_fail(err, "cudaFuncSetAttribute");
            known.raised = smem;
        }
        if (known.smem != smem) {
            int blocks = 0;
            cudaError_t err = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, map_tile_kernel<F>, kThreads, smem);
            if (err != cudaSuccess) return cuda_fail(err, "cudaOccupancyMaxActiveBlocksPerMultiprocessor");
            if (blocks < 1) return fail(HMC_INTERNAL_ERROR, "the tiled kernel does not fit on this GPU");
            known.blocks = blocks;
            known.smem = smem;
        }
        const int known_blocks = known.blocks;
        const int64_t tcap = static_cast<int64_t>(ctx->sm_count) * known_blocks;
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
