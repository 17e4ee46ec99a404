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
template <class F> constexpr int unroll_of() {
    // 64 bytes of the widest operand per thread and iteration.
    constexpr int so = sizeof(typename F::Out);
    constexpr int sa = size_or<typename F::A>(so), sb = size_or<typename F::B>(so), sc = size_or<typename F::C>(so);
    constexpr int mx = so > sa ? (so > sb ? (so > sc ? so : sc) : (sb > sc ? sb : sc)) : (sa > sb ? (sa > sc ? sa : sc) : (sb > sc ? sb : sc));
    constexpr int bytes = mx * vec_of<F>();
    return bytes >= 64 ? 1 : (bytes >= 32 ? 2 : 4);
}

template <class T, int VEC>
__device__ __forceinline__ void load_operand(Pack<T, VEC> &dst, const MapArgs &a, int k, int64_t row_off, int64_t idx,
                                             int64_t s0) {
    if constexpr (!std::is_same_v<T, Unused>) {
        if (a.constant_mask & (1u << k)) {
            T c;
            uint64_t bits = a.constant[k];
            memcpy(&c, &bits, sizeof(T));
#pragma unroll
            for (int j = 0; j < VEC; ++j) dst.v[j] = c;
            return;
        }
        const T *p = reinterpret_cast<const T *>(a.base[k]) + row_off;
        if (s0 == 1) {
            p += idx;
            if (idx + VEC <= a.n0 && (reinterpret_cast<uintptr_t>(p) & (alignof(Pack<T, VEC>) - 1)) == 0) {
                dst = *reinterpret_cast<const Pack<T, VEC> *>(p);
            } else {
#pragma unroll
                for (int j = 0; j < VEC; ++j)
                    if (idx + j < a.n0) dst.v[j] = p[j];
            }
        } else if (s0 == 0) {
            T c = *p;
#pragma unroll
            for (int j = 0; j < VEC; ++j) dst.v[j] = c;
        } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j)
                if (idx + j < a.n0) dst.v[j] = p[(idx + j) * s0];
        }
    }
}

template <class T, int VEC>
__device__ __forceinline__ void store_operand(const Pack<T, VEC> &src, const MapArgs &a, int64_t row_off, int64_t idx,
                                              int64_t s0, int k = 0) {
    T *p = reinterpret_cast<T *>(a.base[k]) + row_off;
    if (s0 == 1) {
        p += idx;
        if (idx + VEC <= a.n0 && (reinterpret_cast<uintptr_t>(p) & (alignof(Pack<T, VEC>) - 1)) == 0) {
            *reinterpret_cast<Pack<T, VEC> *>(p) = src;
        } else {
#pragma unroll
            for (int j = 0; j < VEC; ++j)
                if (idx + j < a.n0) p[j] = src.v[j];
        }
    } else {
#pragma unroll
        for (int j = 0; j < VEC; ++j)
            if (idx + j < a.n0) p[(idx + j) * s0] = src.v[j];
    }
}

template <class F, class A, class B, class C>
__device__ __forceinline__ typename F::Out apply(const F &f, const A &a, const B &b, const C &c, int j) {
    if constexpr (std::is_same_v<typename F::A, Unused>) return f();
    else if constexpr (std::is_same_v<typename F::B, Unused>) return f(a.v[j]);
    else if constexpr (std::is_same_v<typename F::C, Unused>) return f(a.v[j], b.v[j]);
    else return f(a.v[j], b.v[j], c.v[j]);
}

template <class F>
__global__ void __launch_bounds__(kThreads) map_kernel(const __grid_constant__ MapArgs a, const F f) {
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
    const int last = a.ndim - 1;
    const int64_t s0o = a.strides[0][last], s0a = a.strides[1][last], s0b = a.strides[2][last], s0c = a.strides[3][last];
    const int64_t step = static_cast<int64_t>(tpr) * VEC;

    for (int64_t item = blockIdx.x; item < a.items; item += gridDim.x) {
        int64_t rg, seg;
        if (a.rows == 1) {
            rg = 0;
            seg = item;
        } else if (a.segs == 1) {
            rg = item;
            seg = 0;
        } else {
            rg = item / a.segs;
            seg = item - rg * a.segs;
        }
        const int64_t row = rg * rpb + rib;
        if (row >= a.rows) continue;
        int64_t off[kOperands] = {0, 0, 0, 0};
        if (last > 0) {
            if (a.rows_fit32) {
                uint32_t r = static_cast<uint32_t>(row);
                for (int d = last - 1; d > 0; --d) {
                    uint32_t size = static_cast<uint32_t>(a.sizes[d]);
                    uint32_t q = r / size;
                    uint32_t i = r - q * size;
#pragma unroll
                    for (int k = 0; k < kOperands; ++k) off[k] += static_cast<int64_t>(i) * a.strides[k][d];
                    r = q;
                }
#pragma unroll
                for (int k = 0; k < kOperands; ++k) off[k] += static_cast<int64_t>(r) * a.strides[k][0];
            } else {
                int64_t r = row;
                for (int d = last - 1; d > 0; --d) {
                    int64_t size = a.sizes[d];
                    int64_t q = r / size;
                    int64_t i = r - q * size;
#pragma unroll
                    for (int k = 0; k < kOperands; ++k) off[k] += i * a.strides[k][d];
                    r = q;
                }
#pragma unroll
                for (int k = 0; k < kOperands; ++k) off[k] += r * a.strides[k][0];
            }
        }
        const int64_t i0 = seg * (step * UNR) + static_cast<int64_t>(lane) * VEC;
        Pack<TA, VEC> va[UNR];
        Pack<TB, VEC> vb[UNR];
        Pack<TC, VEC> vc[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int64_t idx = i0 + u * step;
            if (idx < a.n0) {
                load_operand<TA, VEC>(va[u], a, 1, off[1], idx, s0a);
                load_operand<TB, VEC>(vb[u], a, 2, off[2], idx, s0b);
                load_operand<TC, VEC>(vc[u], a, 3, off[3], idx, s0c);
            }
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int64_t idx = i0 + u * step;
            if (idx < a.n0) {
                Pack<TO, VEC> vo;
#pragma unroll
                for (int j = 0; j < VEC; ++j) vo.v[j] = apply<F>(f, va[u], vb[u], vc[u], j);
                store_operand<TO, VEC>(vo, a, off[0], idx, s0o);
            }
        }
    }
}

// ---- the tiled kernel ----
// For operands whose unit stride runs along the second-to-last dimension A while the output's runs
// along the last dimension B (a transposed view): a 64 x 64 tile of each such operand is read with
// the threads consecutive along A (full 32-byte sectors), parked in shared memory, and read back with
// the threads consecutive along B, so that both the loads and the stores are coalesced. The tile's
// row pitch is padded so that both passes are free of bank conflicts for every element size.
constexpr int kTile = 64;

template <class T> constexpr int tile_pitch() {
    if constexpr (std::is_same_v<T, Unused>) return 0;
    else return kTile + (sizeof(T) <= 4 ? 4 / static_cast<int>(sizeof(T)) : 1);
}
template <class T> constexpr size_t tile_bytes() {
    if constexpr (std::is_same_v<T, Unused>) return 0;
    else return (static_cast<size_t>(kTile) * tile_pitch<T>() * sizeof(T) + 15) / 16 * 16;
}

template <class T>
__device__ __forceinline__ void tile_fill(T *tile, const MapArgs &a, int k, int64_t off, int64_t a0, int64_t b0,
                                          int64_t size_a, int64_t size_b, int64_t sb) {
    if constexpr (!std::is_same_v<T, Unused>) {
        constexpr int P = tile_pitch<T>();
        const int tx = threadIdx.x & (kTile - 1), ty = threadIdx.x >> 6;
        const T *p = reinterpret_cast<const T *>(a.base[k]) + off + (a0 + tx);
        T v[kTile / 4];
#pragma unroll
        for (int i = 0; i < kTile / 4; ++i) {
            const int b = ty + 4 * i;
            if (a0 + tx < size_a && b0 + b < size_b) v[i] = p[(b0 + b) * sb];
        }
#pragma unroll
        for (int i = 0; i < kTile / 4; ++i) tile[(ty + 4 * i) * P + tx] = v[i];
    }
}

template <class T>
__device__ __forceinline__ T tile_or_direct(const T *tile, bool tiled, const MapArgs &a, int k, int64_t off, int aa,
                                            int bb, int64_t a0, int64_t b0, int64_t sa, int64_t sb) {
    if (tiled) return tile[bb * tile_pitch<T>() + aa];
    if (a.constant_mask & (1u << k)) {
        T c;
        uint64_t bits = a.constant[k];
        memcpy(&c, &bits, sizeof(T));
        return c;
    }
    return reinterpret_cast<const T *>(a.base[k])[off + (a0 + aa) * sa + (b0 + bb) * sb];
}

template <class F>
__global__ void __launch_bounds__(kThreads) map_tile_kernel(const __grid_constant__ MapArgs a, const F f) {
    using TO = typename F::Out;
    using TA = typename F::A;
    using TB = typename F::B;
    using TC = typename F::C;
    extern __shared__ __align__(16) unsigned char tile_memory[];
    TA *tile_a = reinterpret_cast<TA *>(tile_memory);
    TB *tile_b = reinterpret_cast<TB *>(tile_memory + tile_bytes<TA>());
    TC *tile_c = reinterpret_cast<TC *>(tile_memory + tile_bytes<TA>() + tile_bytes<TB>());
    const bool ta = a.tile_mask & 2u, tb = a.tile_mask & 4u, tc = a.tile_mask & 8u;
    const int da = a.ndim - 2, db = a.ndim - 1;
    const int64_t size_a = a.sizes[da], size_b = a.sizes[db];
    const int tx = threadIdx.x & (kTile - 1), ty = threadIdx.x >> 6;
    constexpr int R = kTile / 4;
    for (int64_t t = blockIdx.x; t < a.ntiles; t += gridDim.x) {
        const int64_t jb = t % a.tiles_b;
        const int64_t t2 = t / a.tiles_b;
        const int64_t ja = t2 % a.tiles_a;
        int64_t outer = t2 / a.tiles_a;
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
        if (ta) tile_fill<TA>(tile_a, a, 1, off[1], a0, b0, size_a, size_b, a.strides[1][db]);
        if (tb) tile_fill<TB>(tile_b, a, 2, off[2], a0, b0, size_a, size_b, a.strides[2][db]);
        if (tc) tile_fill<TC>(tile_c, a, 3, off[3], a0, b0, size_a, size_b, a.strides[3][db]);
        __syncthreads();
        Pack<TA, R> va;
        Pack<TB, R> vb;
        Pack<TC, R> vc;
        const bool col_ok = b0 + tx < size_b;
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int aa = ty + 4 * i;
            if (col_ok && a0 + aa < size_a) {
                if constexpr (!std::is_same_v<TA, Unused>)
                    va.v[i] = tile_or_direct<TA>(tile_a, ta, a, 1, off[1], aa, tx, a0, b0, a.strides[1][da], a.strides[1][db]);
                if constexpr (!std::is_same_v<TB, Unused>)
                    vb.v[i] = tile_or_direct<TB>(tile_b, tb, a, 2, off[2], aa, tx, a0, b0, a.strides[2][da], a.strides[2][db]);
                if constexpr (!std::is_same_v<TC, Unused>)
                    vc.v[i] = tile_or_direct<TC>(tile_c, tc, a, 3, off[3], aa, tx, a0, b0, a.strides[3][da], a.strides[3][db]);
            }
        }
        TO *po = reinterpret_cast<TO *>(a.base[0]) + off[0];
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int aa = ty + 4 * i;
            if (col_ok && a0 + aa < size_a) {
                po[(a0 + aa) * a.strides[0][da] + (b0 + tx) * a.strides[0][db]] = apply<F>(f, va, vb, vc, i);
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
    int64_t cap = static_cast<int64_t>(ctx->sm_count) * 16;
    unsigned grid = static_cast<unsigned>(a.items < cap ? a.items : cap);
    map_kernel<F><<<grid, kThreads, 0, ctx->stream>>>(a, f);
    return launch_status("elementwise kernel launch");
}

}  // namespace hmc
