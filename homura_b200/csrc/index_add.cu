// index_add, scatter_add and index_positions. Stand in for hmr_index_add, hmr_scatter_add and hmr_index_positions of
// csrc/index.hip; semantics of cpu::index_add, cpu::scatter_add (through add_at) and cpu::index_positions
// (src/backend/cpu/misc.rs:154-317).
//
// The CPU sums every output element in f64 (floats) or wrapping i64 (integers; a Bool is the or), starting from the
// element's own value, in the order of the contributions, and rounds once. To give the same bits whatever the
// scheduling, the contributions are sorted by target with a stable sort (sort.cuh), so that equal targets keep their
// order; the first entry of each run of equal targets then adds the whole run, in that order. Targets that nothing
// names are not touched.
#include "common.cuh"
#include "elem.cuh"
#include "map.cuh"
#include "sort.cuh"

namespace hmc {
namespace {

constexpr int kAddThreads = 256;

__device__ __forceinline__ int64_t position_at(const void *data, int dtype, int64_t at) {
    return dtype == HMC_I32 ? static_cast<int64_t>(static_cast<const int32_t *>(data)[at]) : static_cast<const int64_t *>(data)[at];
}

template <class T> struct Sum {
    static constexpr bool kIsFloat = Tr<T>::kind == hmc::kFloat;
    using A = typename std::conditional<kIsFloat, double, int64_t>::type;
    static __device__ __forceinline__ A load(T v) {
        if constexpr (kIsFloat) return to_f64(v);
        else return to_i64(v);
    }
    static __device__ __forceinline__ A add(A a, T v) {
        if constexpr (kIsFloat) return a + to_f64(v);
        else return static_cast<int64_t>(static_cast<uint64_t>(a) + static_cast<uint64_t>(to_i64(v)));
    }
    static __device__ __forceinline__ T store(A a) {
        if constexpr (kIsFloat) return from_f64<T>(a);
        else return from_i64<T>(a);
    }
};

// ---- index_add ----

template <class K>
__global__ void __launch_bounds__(kAddThreads) index_add_keys_kernel(K *keys, const void *index, int index_dtype, int64_t index_stride,
                                                                     int64_t m, int64_t size) {
    for (int64_t i = blockIdx.x * static_cast<int64_t>(kAddThreads) + threadIdx.x; i < m;
         i += static_cast<int64_t>(gridDim.x) * kAddThreads) {
        int64_t j = position_at(index, index_dtype, i * index_stride);
        if (j < 0) j += size;
        // a position outside the dimension sorts behind all others and is skipped
        keys[i] = static_cast<K>(j >= 0 && j < size ? j : size);
    }
}

template <class K> struct IndexAddArgs {
    hmc_tensor_desc out;   // with its own size along `at`
    hmc_tensor_desc src;   // with the number of positions along `at`
    const K *keys;         // the sorted positions
    const uint32_t *vals;  // and the slice of src each came from
    int32_t at;
    int64_t m, size;
    int64_t rest;          // elements of a slice
    int64_t work;          // m * rest
};

// One thread per (sorted position, VEC adjacent elements of its slice); only the first position of a run of equal
// targets works, and adds the run in order. With VEC > 1 the innermost dimension is contiguous in both tensors and is
// walked in 16-byte vectors (its size in `sizes` is then counted in vectors).
template <class T, class K, int VEC>
__global__ void __launch_bounds__(kAddThreads) index_add_kernel(const __grid_constant__ IndexAddArgs<K> a) {
    using S = Sum<T>;
    T *out = static_cast<T *>(a.out.data) + a.out.offset;
    const T *src = static_cast<const T *>(a.src.data) + a.src.offset;
    const bool narrow = a.work <= 0xFFFFFFFFll;  // 32-bit divisions
    const int last = a.out.ndim - 1;
    for (int64_t w = blockIdx.x * static_cast<int64_t>(kAddThreads) + threadIdx.x; w < a.work;
         w += static_cast<int64_t>(gridDim.x) * kAddThreads) {
        const int64_t k = a.rest == 1 ? w : (narrow ? static_cast<int64_t>(static_cast<uint32_t>(w) / static_cast<uint32_t>(a.rest)) : w / a.rest);
        const K key = a.keys[k];
        if (static_cast<int64_t>(key) >= a.size || (k > 0 && a.keys[k - 1] == key)) continue;  // not the first of its run
        int64_t item = w - k * a.rest, oo = 0, so = 0;
        for (int d = last; d >= 0; --d) {
            if (d == a.at) continue;
            const int64_t q = narrow ? static_cast<int64_t>(static_cast<uint32_t>(item) / static_cast<uint32_t>(a.out.sizes[d])) : item / a.out.sizes[d];
            const int64_t c = (item - q * a.out.sizes[d]) * (d == last ? VEC : 1);
            item = q;
            oo += c * a.out.strides[d];
            so += c * a.src.strides[d];
        }
        oo += static_cast<int64_t>(key) * a.out.strides[a.at];
        const int64_t step = a.src.strides[a.at];
        Pack<T, VEC> x;
        vector_load<T, VEC>(x, out + oo, true);  // (vectors of 32 bytes are chosen for 32-byte aligned slices only)
        typename S::A acc[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[e] = S::load(x.v[e]);
        for (int64_t kk = k; kk < a.m && a.keys[kk] == key; ++kk) {
            vector_load<T, VEC>(x, src + so + static_cast<int64_t>(a.vals[kk]) * step, true);
#pragma unroll
            for (int e = 0; e < VEC; ++e) acc[e] = S::add(acc[e], x.v[e]);
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) x.v[e] = S::store(acc[e]);
        vector_store<T, VEC>(out + oo, x, true);
    }
}

// ---- scatter_add ----

template <class K> struct ScatterArgs {
    hmc_tensor_desc index;  // the walked shape
    hmc_tensor_desc out;    // with its own size along `at`
    hmc_tensor_desc src;
    K *keys;
    const K *sorted;
    const uint32_t *vals;
    int32_t at;
    int64_t n;              // elements of the index
    int64_t size;           // out's size along `at`
    uint64_t bound;         // one more than the largest offset into out
};

template <class K>
__global__ void __launch_bounds__(kAddThreads) scatter_keys_kernel(const __grid_constant__ ScatterArgs<K> a) {
    for (int64_t p = blockIdx.x * static_cast<int64_t>(kAddThreads) + threadIdx.x; p < a.n;
         p += static_cast<int64_t>(gridDim.x) * kAddThreads) {
        int64_t rest = p, io = a.index.offset, oo = 0;
        for (int d = a.index.ndim - 1; d >= 0; --d) {
            const int64_t q = rest / a.index.sizes[d];
            const int64_t c = rest - q * a.index.sizes[d];
            rest = q;
            io += c * a.index.strides[d];
            if (d != a.at) oo += c * a.out.strides[d];
        }
        const int64_t j = position_at(a.index.data, a.index.dtype, io);
        a.keys[p] = static_cast<K>(j >= 0 && j < a.size ? static_cast<uint64_t>(oo + j * a.out.strides[a.at]) : a.bound);
    }
}

template <class T, class K>
__global__ void __launch_bounds__(kAddThreads) scatter_add_kernel(const __grid_constant__ ScatterArgs<K> a) {
    using S = Sum<T>;
    T *out = static_cast<T *>(a.out.data) + a.out.offset;
    const T *src = static_cast<const T *>(a.src.data) + a.src.offset;
    for (int64_t k = blockIdx.x * static_cast<int64_t>(kAddThreads) + threadIdx.x; k < a.n;
         k += static_cast<int64_t>(gridDim.x) * kAddThreads) {
        const K key = a.sorted[k];
        if (static_cast<uint64_t>(key) >= a.bound || (k > 0 && a.sorted[k - 1] == key)) continue;
        typename S::A acc = S::load(out[key]);
        for (int64_t kk = k; kk < a.n && a.sorted[kk] == key; ++kk) {
            int64_t rest = a.vals[kk], so = 0;
            for (int d = a.index.ndim - 1; d >= 0; --d) {
                const int64_t q = rest / a.index.sizes[d];
                so += (rest - q * a.index.sizes[d]) * a.src.strides[d];
                rest = q;
            }
            acc = S::add(acc, src[so]);
        }
        out[key] = S::store(acc);
    }
}

// ---- index_positions ----

struct PositionsArgs {
    hmc_tensor_desc out, coord;
    int64_t size, stride, items;
    int32_t first;
};

__global__ void __launch_bounds__(kAddThreads) index_positions_kernel(const __grid_constant__ PositionsArgs a) {
    int64_t *out = static_cast<int64_t *>(a.out.data) + a.out.offset;
    for (int64_t item = blockIdx.x * static_cast<int64_t>(kAddThreads) + threadIdx.x; item < a.items;
         item += static_cast<int64_t>(gridDim.x) * kAddThreads) {
        int64_t rest = item, oo = 0, co = a.coord.offset;
        for (int d = a.out.ndim - 1; d >= 0; --d) {
            const int64_t q = rest / a.out.sizes[d];
            const int64_t c = rest - q * a.out.sizes[d];
            rest = q;
            oo += c * a.out.strides[d];
            co += c * a.coord.strides[d];
        }
        int64_t v = position_at(a.coord.data, a.coord.dtype, co);
        if (v < 0) v += a.size;
        const int64_t term = static_cast<int64_t>(static_cast<uint64_t>(v) * static_cast<uint64_t>(a.stride));
        out[oo] = a.first ? term : static_cast<int64_t>(static_cast<uint64_t>(out[oo]) + static_cast<uint64_t>(term));
    }
}

unsigned add_grid(int64_t items) {
    const int64_t blocks = ceil_div(items, static_cast<int64_t>(kAddThreads));
    return static_cast<unsigned>(blocks < 1 ? 1 : (blocks < (int64_t{1} << 20) ? blocks : (int64_t{1} << 20)));
}

int bits_of(uint64_t v) {
    int b = 0;
    while (v != 0) {
        ++b;
        v >>= 1;
    }
    return b;
}

hmc_status check_workspace(void *workspace, int64_t workspace_bytes, int64_t n, const char *what) {
    if (workspace == nullptr || workspace_bytes < sort_workspace_bytes(static_cast<uint64_t>(n)) ||
        (reinterpret_cast<uintptr_t>(workspace) & 7) != 0) {
        return fail(HMC_INVALID, what);
    }
    return HMC_OK;
}

}  // namespace
}  // namespace hmc

using namespace hmc;

HMC_API hmc_status hmc_index_add_workspace(int64_t m, int64_t size, int64_t *bytes) {
    return guarded([&]() -> hmc_status {
        if (bytes == nullptr) return fail(HMC_INVALID, "null output");
        if (m < 0 || size < 0) return fail(HMC_INVALID, "negative size");
        if (m > 0xFFFFFFFFll) return fail(HMC_INVALID, "index_add takes fewer than 2^32 positions");
        *bytes = sort_workspace_bytes(static_cast<uint64_t>(m));
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_index_add(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *src, const hmc_tensor_desc *index,
                                 int32_t dim, void *workspace, int64_t workspace_bytes) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        hmc_status s = check_desc(out, "the output");
        if (s == HMC_OK) s = check_desc(src, "the input");
        if (s == HMC_OK) s = check_desc(index, "the index");
        if (s != HMC_OK) return s;
        if (out->dtype != src->dtype) return fail(HMC_INVALID, "index_add writes its input's dtype");
        if (out->ndim != src->ndim || out->ndim < 1) return fail(HMC_INVALID, "index_add takes operands of the same rank, at least 1");
        if (dim < 0 || dim >= out->ndim) return fail(HMC_INVALID, "the indexed dimension is out of range");
        if ((index->dtype != HMC_I64 && index->dtype != HMC_I32) || index->ndim != 1) return fail(HMC_INVALID, "the index is a 1-D I32 or I64 tensor");
        const int64_t m = index->sizes[0], size = out->sizes[dim];
        if (src->sizes[dim] != m) return fail(HMC_INVALID, "the input's size along the indexed dimension is the number of positions");
        if (m > 0xFFFFFFFFll) return fail(HMC_INVALID, "index_add takes fewer than 2^32 positions");
        int64_t rest = 1, n = 1;
        for (int k = 0; k < out->ndim; ++k) {
            if (k != dim && out->sizes[k] != src->sizes[k]) return fail(HMC_INVALID, "operands differ in their sizes");
            if (k != dim && __builtin_mul_overflow(rest, out->sizes[k], &rest)) return fail(HMC_INVALID, "the number of elements overflows 63 bits");
            if (__builtin_mul_overflow(n, out->sizes[k], &n)) return fail(HMC_INVALID, "the number of elements overflows 63 bits");
        }
        int64_t work = 0;
        if (__builtin_mul_overflow(rest, m, &work)) return fail(HMC_INVALID, "the number of elements overflows 63 bits");
        if (work == 0 || n == 0) return HMC_OK;
        s = check_workspace(workspace, workspace_bytes, m, "the workspace of index_add is missing, too small or not 8-byte aligned");
        if (s != HMC_OK) return s;
        if (out->data == nullptr || src->data == nullptr || index->data == nullptr) return fail(HMC_INVALID, "null data pointer");
        const void *first = static_cast<const char *>(index->data) + index->offset * element_size(index->dtype);
        auto run = [&](auto key_tag) -> hmc_status {
            using K = decltype(key_tag);
            SortSpace<K> space = sort_space<K>(workspace, static_cast<uint64_t>(m));
            index_add_keys_kernel<K><<<add_grid(m), kAddThreads, 0, ctx->stream>>>(space.keys[0], first, index->dtype, index->strides[0], m, size);
            hmc_status st = launch_status("index_add keys kernel launch");
            if (st != HMC_OK) return st;
            int sorted = 0;
            st = sort_pairs<K>(ctx->stream, space, static_cast<uint64_t>(m), bits_of(static_cast<uint64_t>(size)), &sorted);
            if (st != HMC_OK) return st;
            IndexAddArgs<K> a{*out, *src, space.keys[sorted], space.vals[sorted], dim, m, size, rest, work};
            return dispatch_all(out->dtype, [&](auto t) -> hmc_status {
                using T = decltype(t);
                // vectors of 32 bytes (one 256-bit access), else of 16, along the innermost dimension where both tensors allow them
                const int last = out->ndim - 1;
                auto aligned_to = [&](int bytes) {
                    const int per = bytes / static_cast<int>(sizeof(T));
                    bool ok = per > 1 && dim != last && out->strides[last] == 1 && src->strides[last] == 1 && out->sizes[last] % per == 0 &&
                              ((reinterpret_cast<uintptr_t>(out->data) + out->offset * sizeof(T)) % bytes) == 0 &&
                              ((reinterpret_cast<uintptr_t>(src->data) + src->offset * sizeof(T)) % bytes) == 0;
                    for (int k = 0; k < last && ok; ++k) ok = out->strides[k] % per == 0 && src->strides[k] % per == 0;
                    return ok;
                };
                auto run_vectors = [&](auto vec_tag) {
                    constexpr int VEC = decltype(vec_tag)::value;
                    IndexAddArgs<K> v = a;
                    v.out.sizes[last] /= VEC;
                    v.rest /= VEC;
                    v.work /= VEC;
                    index_add_kernel<T, K, VEC><<<add_grid(v.work), kAddThreads, 0, ctx->stream>>>(v);
                };
                if (aligned_to(32)) run_vectors(std::integral_constant<int, 32 / static_cast<int>(sizeof(T))>{});
                else if (aligned_to(16)) run_vectors(std::integral_constant<int, (16 / static_cast<int>(sizeof(T)) > 1 ? 16 / static_cast<int>(sizeof(T)) : 2)>{});
                else index_add_kernel<T, K, 1><<<add_grid(work), kAddThreads, 0, ctx->stream>>>(a);
                return launch_status("index_add kernel launch");
            });
        };
        return size < 0xFFFFFFFFll ? run(uint32_t{}) : run(uint64_t{});
    });
}

HMC_API hmc_status hmc_scatter_add_workspace(int64_t n, int64_t *bytes) {
    return guarded([&]() -> hmc_status {
        if (bytes == nullptr) return fail(HMC_INVALID, "null output");
        if (n < 0) return fail(HMC_INVALID, "negative size");
        if (n > 0xFFFFFFFFll) return fail(HMC_INVALID, "scatter_add takes an index of fewer than 2^32 elements");
        *bytes = sort_workspace_bytes(static_cast<uint64_t>(n));
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_scatter_add(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *src, const hmc_tensor_desc *index,
                                   int32_t dim, void *workspace, int64_t workspace_bytes) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        hmc_status s = check_desc(out, "the output");
        if (s == HMC_OK) s = check_desc(src, "the input");
        if (s == HMC_OK) s = check_desc(index, "the index");
        if (s != HMC_OK) return s;
        if (out->dtype != src->dtype) return fail(HMC_INVALID, "scatter_add writes its input's dtype");
        if (out->ndim != src->ndim || out->ndim != index->ndim || out->ndim < 1) {
            return fail(HMC_INVALID, "scatter_add takes operands of the same rank, at least 1");
        }
        if (dim < 0 || dim >= out->ndim) return fail(HMC_INVALID, "the scattered dimension is out of range");
        if (index->dtype != HMC_I64 && index->dtype != HMC_I32) return fail(HMC_INVALID, "an index tensor is I32 or I64");
        int64_t n = 1;
        uint64_t bound = 1;
        for (int k = 0; k < out->ndim; ++k) {
            if (index->sizes[k] > src->sizes[k]) return fail(HMC_INVALID, "the index reaches beyond the input");
            if (k != dim && index->sizes[k] > out->sizes[k]) return fail(HMC_INVALID, "the index reaches beyond the output");
            if (__builtin_mul_overflow(n, index->sizes[k], &n)) return fail(HMC_INVALID, "the number of elements overflows 63 bits");
            if (out->sizes[k] == 0) return n == 0 ? HMC_OK : fail(HMC_INVALID, "an empty output takes no contributions");
            bound += static_cast<uint64_t>(out->sizes[k] - 1) * static_cast<uint64_t>(out->strides[k]);
        }
        if (n == 0) return HMC_OK;
        if (n > 0xFFFFFFFFll) return fail(HMC_INVALID, "scatter_add takes an index of fewer than 2^32 elements");
        s = check_workspace(workspace, workspace_bytes, n, "the workspace of scatter_add is missing, too small or not 8-byte aligned");
        if (s != HMC_OK) return s;
        if (out->data == nullptr || src->data == nullptr || index->data == nullptr) return fail(HMC_INVALID, "null data pointer");
        auto run = [&](auto key_tag) -> hmc_status {
            using K = decltype(key_tag);
            SortSpace<K> space = sort_space<K>(workspace, static_cast<uint64_t>(n));
            ScatterArgs<K> a{*index, *out, *src, space.keys[0], nullptr, nullptr, dim, n, out->sizes[dim], bound};
            scatter_keys_kernel<K><<<add_grid(n), kAddThreads, 0, ctx->stream>>>(a);
            hmc_status st = launch_status("scatter_add keys kernel launch");
            if (st != HMC_OK) return st;
            int sorted = 0;
            st = sort_pairs<K>(ctx->stream, space, static_cast<uint64_t>(n), bits_of(bound), &sorted);
            if (st != HMC_OK) return st;
            a.sorted = space.keys[sorted];
            a.vals = space.vals[sorted];
            return dispatch_all(out->dtype, [&](auto t) -> hmc_status {
                scatter_add_kernel<decltype(t), K><<<add_grid(n), kAddThreads, 0, ctx->stream>>>(a);
                return launch_status("scatter_add kernel launch");
            });
        };
        return bound < 0xFFFFFFFFull ? run(uint32_t{}) : run(uint64_t{});
    });
}

HMC_API hmc_status hmc_index_positions(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *coord, int64_t size,
                                       int64_t stride, int32_t first) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        const hmc_tensor_desc *d[2] = {out, coord};
        int64_t n = 0;
        hmc_status s = check_operands(d, 2, &n);
        if (s != HMC_OK) return s;
        if (out->dtype != HMC_I64) return fail(HMC_INVALID, "the positions are an I64 tensor");
        if (coord->dtype != HMC_I64 && coord->dtype != HMC_I32) return fail(HMC_INVALID, "an index tensor is I32 or I64");
        if (n == 0) return HMC_OK;
        if (out->data == nullptr || coord->data == nullptr) return fail(HMC_INVALID, "null data pointer");
        PositionsArgs a{*out, *coord, size, stride, n, first};
        index_positions_kernel<<<add_grid(n), kAddThreads, 0, ctx->stream>>>(a);
        return launch_status("index_positions kernel launch");
    });
}
