// The read side of homura's indexing family: the check of index values, index_select (an embedding lookup is
// index_select along dimension 0) and gather. Stand in for hmr_index_check, hmr_index_select and hmr_gather of
// csrc/index.hip; semantics of cpu::index_select and cpu::gather (src/backend/cpu/misc.rs:77-103, 319-342).
//
// Gathers move bytes: one instantiation per element size. index_select copies whole slices, so when the innermost
// dimension is not the indexed one and both tensors have unit stride along it, a thread moves a 16-byte vector
// and a slice is read and written in full lines; everything else moves single elements with the same addressing.
#include "common.cuh"
#include "elem.cuh"
#include "map.cuh"

namespace hmc {
namespace {

constexpr int kIndexThreads = 256;

__device__ __forceinline__ int64_t index_at(const void *data, int dtype, int64_t at) {
    return dtype == HMC_I32 ? static_cast<int64_t>(static_cast<const int32_t *>(data)[at]) : static_cast<const int64_t *>(data)[at];
}

struct SelectArgs {
    hmc_tensor_desc out;
    hmc_tensor_desc src;
    const void *index;      // the 1-D index, at its first element
    int64_t index_stride;
    int32_t index_dtype;
    int32_t at;             // the indexed dimension
    int32_t wrap_negative;
    int32_t vector;         // the innermost dimension is walked in 16-byte vectors
    int64_t size;           // src's size along `at`
    int64_t inner;          // out's innermost size in work items (vectors or elements)
    int64_t items;          // work items in all
};

// Where work item `item` lies: the offsets of its output and source elements.
template <int VEC>
__device__ __forceinline__ void select_offsets(const SelectArgs &a, int64_t item, int64_t &oo, int64_t &so) {
    const int last = a.out.ndim - 1;
    // (32-bit division where the item number allows: a 64-bit one costs several times as much, per 16 bytes)
    int64_t rest = a.items < (int64_t{1} << 31) ? static_cast<int64_t>(static_cast<uint32_t>(item) / static_cast<uint32_t>(a.inner))
                                                : item / a.inner;
    const int64_t c_last = (item - rest * a.inner) * VEC;
    oo = c_last * a.out.strides[last];
    if (last == a.at) {
        int64_t j = index_at(a.index, a.index_dtype, c_last * a.index_stride);
        if (a.wrap_negative && j < 0) j += a.size;
        so = j * a.src.strides[last];
    } else {
        so = c_last * a.src.strides[last];
    }
    for (int d = last - 1; d >= 0; --d) {
        const int64_t q = d == 0 ? 0 : rest / a.out.sizes[d];  // the outermost coordinate is what is left
        const int64_t c = rest - q * a.out.sizes[d];
        rest = q;
        oo += c * a.out.strides[d];
        if (d == a.at) {
            int64_t j = index_at(a.index, a.index_dtype, c * a.index_stride);
            if (a.wrap_negative && j < 0) j += a.size;
            so += j * a.src.strides[d];
        } else {
            so += c * a.src.strides[d];
        }
    }
}

// Work item -> coordinates of out (the innermost one in units of VEC elements); the source offset takes the index
// element in place of the coordinate along `at`. Four items per thread and round, their loads in flight together:
// the rows of a lookup are scattered over the table, so a thread waits for memory, not for its neighbours.
template <class W, int VEC>
__global__ void __launch_bounds__(kIndexThreads) index_select_kernel(const __grid_constant__ SelectArgs a) {
    constexpr int UNR = 4;
    W *out = static_cast<W *>(a.out.data) + a.out.offset;
    const W *src = static_cast<const W *>(a.src.data) + a.src.offset;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kIndexThreads;
    for (int64_t item = blockIdx.x * static_cast<int64_t>(kIndexThreads) + threadIdx.x; item < a.items; item += UNR * stride) {
        int64_t oo[UNR], so[UNR];
        Pack<W, VEC> x[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            if (item + u * stride < a.items) {
                select_offsets<VEC>(a, item + u * stride, oo[u], so[u]);
                vector_load<W, VEC>(x[u], src + so[u], true);  // (vectors of 32 bytes are chosen for 32-byte aligned slices only)
            }
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            if (item + u * stride < a.items) vector_store<W, VEC>(out + oo[u], x[u], true);
        }
    }
}

struct GatherArgs {
    hmc_tensor_desc out;
    hmc_tensor_desc src;
    hmc_tensor_desc index;
    int32_t at;
    int64_t items;
};

template <class W>
__global__ void __launch_bounds__(kIndexThreads) gather_kernel(const __grid_constant__ GatherArgs a) {
    W *out = static_cast<W *>(a.out.data) + a.out.offset;
    const W *src = static_cast<const W *>(a.src.data) + a.src.offset;
    for (int64_t item = blockIdx.x * static_cast<int64_t>(kIndexThreads) + threadIdx.x; item < a.items;
         item += static_cast<int64_t>(gridDim.x) * kIndexThreads) {
        int64_t rest = item, oo = 0, so = 0, io = a.index.offset;
        for (int d = a.out.ndim - 1; d >= 0; --d) {
            const int64_t q = rest / a.out.sizes[d];
            const int64_t c = rest - q * a.out.sizes[d];
            rest = q;
            oo += c * a.out.strides[d];
            io += c * a.index.strides[d];
            if (d != a.at) so += c * a.src.strides[d];
        }
        so += index_at(a.index.data, a.index.dtype, io) * a.src.strides[a.at];
        out[oo] = src[so];
    }
}

struct CheckArgs {
    hmc_tensor_desc index;
    int64_t low, high, exempt;
    int32_t has_exempt;
    int64_t items;
    unsigned long long *slot;
};

__global__ void index_check_reset_kernel(unsigned long long *slot) {
    slot[0] = ~0ull;
    slot[1] = 0;
}

__device__ __forceinline__ int64_t check_offset(const hmc_tensor_desc &d, int64_t item) {
    int64_t off = d.offset;
    for (int k = d.ndim - 1; k >= 0; --k) {
        const int64_t q = item / d.sizes[k];
        off += (item - q * d.sizes[k]) * d.strides[k];
        item = q;
    }
    return off;
}

// The smallest row-major position of an element outside the range: an atomic minimum over the offenders.
__global__ void __launch_bounds__(kIndexThreads) index_check_kernel(const __grid_constant__ CheckArgs a) {
    unsigned long long first = ~0ull;
    for (int64_t item = blockIdx.x * static_cast<int64_t>(kIndexThreads) + threadIdx.x; item < a.items;
         item += static_cast<int64_t>(gridDim.x) * kIndexThreads) {
        const int64_t v = index_at(a.index.data, a.index.dtype, check_offset(a.index, item));
        const bool bad = (v < a.low || v >= a.high) && !(a.has_exempt && v == a.exempt);
        if (bad && static_cast<unsigned long long>(item) < first) first = static_cast<unsigned long long>(item);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xFFFFFFFFu, first, d);
        first = other < first ? other : first;
    }
    if ((threadIdx.x & 31) == 0 && first != ~0ull) atomicMin(a.slot, first);
}

// The value at the position found (one thread, after the minimum is final).
__global__ void index_check_value_kernel(const __grid_constant__ CheckArgs a) {
    const unsigned long long at = a.slot[0];
    if (at == ~0ull) return;
    a.slot[1] = static_cast<unsigned long long>(index_at(a.index.data, a.index.dtype, check_offset(a.index, static_cast<int64_t>(at))));
}

template <class F> hmc_status by_size(int dtype, F &&f) {
    switch (element_size(dtype)) {
        case 1: return f(uint8_t{});
        case 2: return f(uint16_t{});
        case 4: return f(uint32_t{});
        default: return f(uint64_t{});
    }
}

unsigned index_grid(int64_t items) {
    const int64_t blocks = ceil_div(items, kIndexThreads);
    return static_cast<unsigned>(blocks < 1 ? 1 : (blocks < (int64_t{1} << 20) ? blocks : (int64_t{1} << 20)));
}

hmc_status check_index_desc(const hmc_tensor_desc *index) {
    hmc_status s = check_desc(index, "the index");
    if (s != HMC_OK) return s;
    if (index->dtype != HMC_I32 && index->dtype != HMC_I64) return fail(HMC_INVALID, "an index tensor is I32 or I64");
    return HMC_OK;
}

}  // namespace
}  // namespace hmc

using namespace hmc;

HMC_API hmc_status hmc_index_check(hmc_context_t ctx, const hmc_tensor_desc *index, int64_t low, int64_t high, int32_t has_exempt,
                                   int64_t exempt, uint64_t *slot) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        hmc_status s = check_index_desc(index);
        if (s != HMC_OK) return s;
        if (slot == nullptr) return fail(HMC_INVALID, "null status slot");
        if ((reinterpret_cast<uintptr_t>(slot) & 7) != 0) return fail(HMC_INVALID, "the status slot is not 8-byte aligned");
        int64_t n = 1;
        for (int k = 0; k < index->ndim; ++k) {
            if (__builtin_mul_overflow(n, index->sizes[k], &n)) return fail(HMC_INVALID, "the number of elements overflows 63 bits");
        }
        unsigned long long *words = reinterpret_cast<unsigned long long *>(slot);
        index_check_reset_kernel<<<1, 1, 0, ctx->stream>>>(words);
        s = launch_status("index check (reset) kernel launch");
        if (s != HMC_OK || n == 0) return s;
        if (index->data == nullptr) return fail(HMC_INVALID, "null data pointer");
        CheckArgs a{*index, low, high, exempt, has_exempt != 0, n, words};
        index_check_kernel<<<index_grid(n), kIndexThreads, 0, ctx->stream>>>(a);
        s = launch_status("index check kernel launch");
        if (s != HMC_OK) return s;
        index_check_value_kernel<<<1, 1, 0, ctx->stream>>>(a);
        return launch_status("index check (value) kernel launch");
    });
}

HMC_API hmc_status hmc_test_index_value(hmc_context_t ctx, const hmc_tensor_desc *index, uint64_t *slot) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        hmc_status s = check_index_desc(index);
        if (s != HMC_OK) return s;
        if (slot == nullptr || (reinterpret_cast<uintptr_t>(slot) & 7) != 0) return fail(HMC_INVALID, "the status slot is missing or not 8-byte aligned");
        if (index->data == nullptr) return fail(HMC_INVALID, "null data pointer");
        CheckArgs a{*index, 0, 0, 0, 0, 0, reinterpret_cast<unsigned long long *>(slot)};
        index_check_value_kernel<<<1, 1, 0, ctx->stream>>>(a);
        return launch_status("index check (value) kernel launch");
    });
}

HMC_API hmc_status hmc_index_select(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *src,
                                    const hmc_tensor_desc *index, int32_t dim, int32_t wrap_negative) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        hmc_status s = check_desc(out, "the output");
        if (s == HMC_OK) s = check_desc(src, "the input");
        if (s == HMC_OK) s = check_index_desc(index);
        if (s != HMC_OK) return s;
        if (out->dtype != src->dtype) return fail(HMC_INVALID, "index_select writes its input's dtype");
        if (out->ndim != src->ndim || out->ndim < 1) return fail(HMC_INVALID, "index_select takes operands of the same rank, at least 1");
        if (dim < 0 || dim >= out->ndim) return fail(HMC_INVALID, "the indexed dimension is out of range");
        if (index->ndim > 1) return fail(HMC_INVALID, "the index of index_select has one dimension");
        const int64_t m = index->ndim == 0 ? 1 : index->sizes[0];
        int64_t n = 1;
        for (int k = 0; k < out->ndim; ++k) {
            if (k != dim && out->sizes[k] != src->sizes[k]) return fail(HMC_INVALID, "operands differ in their sizes");
            if (__builtin_mul_overflow(n, out->sizes[k], &n)) return fail(HMC_INVALID, "the number of elements overflows 63 bits");
        }
        if (out->sizes[dim] != m) return fail(HMC_INVALID, "the output's size along the indexed dimension is the index's length");
        if (n == 0) return HMC_OK;
        if (out->data == nullptr || src->data == nullptr || index->data == nullptr) return fail(HMC_INVALID, "null data pointer");
        const int es = element_size(src->dtype);
        const int last = out->ndim - 1;
        const int vec = 16 / es;
        SelectArgs a{};
        a.out = *out;
        a.src = *src;
        a.index = static_cast<const char *>(index->data) + index->offset * (index->dtype == HMC_I32 ? 4 : 8);
        a.index_stride = index->ndim == 0 ? 0 : index->strides[0];
        a.index_dtype = index->dtype;
        a.at = dim;
        a.wrap_negative = wrap_negative != 0;
        a.size = src->sizes[dim];
        // Vectors along the innermost dimension when it is not the indexed one, both tensors walk it with unit stride,
        // its length is whole vectors, and every other stride and both first elements keep the alignment: of 32 bytes
        // (one 256-bit access each) where all of that holds for 32, else of 16
        auto aligned_to = [&](int bytes) {
            const int per = bytes / es;
            bool ok = dim != last && out->strides[last] == 1 && src->strides[last] == 1 && out->sizes[last] % per == 0;
            ok = ok && (reinterpret_cast<uintptr_t>(out->data) + static_cast<uintptr_t>(out->offset) * es) % bytes == 0 &&
                 (reinterpret_cast<uintptr_t>(src->data) + static_cast<uintptr_t>(src->offset) * es) % bytes == 0;
            for (int k = 0; k < last && ok; ++k) ok = (out->strides[k] * es) % bytes == 0 && (src->strides[k] * es) % bytes == 0;
            return ok;
        };
        const bool wide = aligned_to(32);
        const bool vector = wide || aligned_to(16);
        const int per = wide ? 2 * vec : vec;
        a.vector = vector;
        a.inner = vector ? out->sizes[last] / per : out->sizes[last];
        a.items = n / (vector ? per : 1);
        const unsigned grid = index_grid(ceil_div(a.items, 4));  // four items per thread
        return by_size(src->dtype, [&](auto w) -> hmc_status {
            using W = decltype(w);
            if (wide) index_select_kernel<W, 32 / sizeof(W)><<<grid, kIndexThreads, 0, ctx->stream>>>(a);
            else if (vector) index_select_kernel<W, 16 / sizeof(W)><<<grid, kIndexThreads, 0, ctx->stream>>>(a);
            else index_select_kernel<W, 1><<<grid, kIndexThreads, 0, ctx->stream>>>(a);
            return launch_status("index_select kernel launch");
        });
    });
}

HMC_API hmc_status hmc_gather(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *src, const hmc_tensor_desc *index,
                              int32_t dim) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        hmc_status s = check_desc(out, "the output");
        if (s == HMC_OK) s = check_desc(src, "the input");
        if (s == HMC_OK) s = check_index_desc(index);
        if (s != HMC_OK) return s;
        if (out->dtype != src->dtype) return fail(HMC_INVALID, "gather writes its input's dtype");
        if (out->ndim != src->ndim || out->ndim != index->ndim || out->ndim < 1) {
            return fail(HMC_INVALID, "gather takes operands of the same rank, at least 1");
        }
        if (dim < 0 || dim >= out->ndim) return fail(HMC_INVALID, "the gathered dimension is out of range");
        int64_t n = 1;
        for (int k = 0; k < out->ndim; ++k) {
            if (out->sizes[k] != index->sizes[k]) return fail(HMC_INVALID, "the output has the index's sizes");
            if (k != dim && out->sizes[k] > src->sizes[k]) return fail(HMC_INVALID, "the index reaches beyond the input");
            if (__builtin_mul_overflow(n, out->sizes[k], &n)) return fail(HMC_INVALID, "the number of elements overflows 63 bits");
        }
        if (n == 0) return HMC_OK;
        if (out->data == nullptr || src->data == nullptr || index->data == nullptr) return fail(HMC_INVALID, "null data pointer");
        GatherArgs a{*out, *src, *index, dim, n};
        const unsigned grid = index_grid(n);
        return by_size(src->dtype, [&](auto w) -> hmc_status {
            gather_kernel<decltype(w)><<<grid, kIndexThreads, 0, ctx->stream>>>(a);
            return launch_status("gather kernel launch");
        });
    });
}
