// triangle (tril / triu, the causal mask in front of a softmax) and flip: the two elementwise neighbours of the
// copy kernels whose result depends on an element's position. Stand in for hmr_triangle and hmr_flip of
// csrc/elementwise.hip; semantics of cpu::triangle and cpu::flip (src/backend/cpu/misc.rs:347-411).
#include "functors.cuh"
#include "ops.cuh"

namespace hmc {
namespace {

constexpr int kTriThreads = 256;

struct TriangleArgs {
    char *out;
    const char *src;
    int32_t nbatch;                 // batch dimensions (all but the last two)
    int32_t upper;
    int64_t diagonal;
    int64_t rows, cols, lines;      // lines = batch * rows
    int64_t out_row, out_col, src_row, src_col;  // strides of the last two dimensions, in elements
    int64_t batch_sizes[HMC_MAX_DIMS];
    int64_t out_batch[HMC_MAX_DIMS];
    int64_t src_batch[HMC_MAX_DIMS];
};

// A block walks lines (one matrix row each); its threads walk the columns, VEC adjacent ones at a time where
// both rows are contiguous and aligned. Elements outside the triangle are written as zero without reading
// the source, so a causal mask costs half the reads.
template <class W>
__global__ void __launch_bounds__(kTriThreads) triangle_kernel(const __grid_constant__ TriangleArgs a) {
    constexpr int VEC = 16 / sizeof(W);
    W *out = reinterpret_cast<W *>(a.out);
    const W *src = reinterpret_cast<const W *>(a.src);
    for (int64_t line = blockIdx.y; line < a.lines; line += gridDim.y) {
        // (32-bit division where the line number allows: a 64-bit one costs several times as much, per thread)
        int64_t batch = a.lines < (int64_t{1} << 31) ? static_cast<int64_t>(static_cast<uint32_t>(line) / static_cast<uint32_t>(a.rows))
                                                      : line / a.rows;
        const int64_t r = line - batch * a.rows;
        int64_t oo = r * a.out_row, so = r * a.src_row;
        for (int d = a.nbatch - 1; d > 0; --d) {
            const int64_t q = batch / a.batch_sizes[d];
            const int64_t i = batch - q * a.batch_sizes[d];
            oo += i * a.out_batch[d];
            so += i * a.src_batch[d];
            batch = q;
        }
        if (a.nbatch > 0) {
            oo += batch * a.out_batch[0];
            so += batch * a.src_batch[0];
        }
        // kept columns: c - r >= diagonal (upper) or c - r <= diagonal (lower)
        const int64_t edge = r + a.diagonal;  // upper keeps c >= edge, lower keeps c <= edge
        W *po = out + oo;
        const W *ps = src + so;
        const bool vector = a.out_col == 1 && a.src_col == 1 && (reinterpret_cast<uintptr_t>(po) & 15) == 0 &&
                            (reinterpret_cast<uintptr_t>(ps) & 15) == 0;
        if (vector) {
            const int64_t nvec = a.cols / VEC;
            for (int64_t v = static_cast<int64_t>(blockIdx.x) * kTriThreads + threadIdx.x; v < nvec;
                 v += static_cast<int64_t>(gridDim.x) * kTriThreads) {
                const int64_t c0 = v * VEC;
                const bool all_kept = a.upper ? c0 >= edge : c0 + VEC - 1 <= edge;
                const bool none_kept = a.upper ? c0 + VEC - 1 < edge : c0 > edge;
                Pack<W, VEC> x;
                if (none_kept) {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) x.v[e] = W{0};
                } else {
                    x = *reinterpret_cast<const Pack<W, VEC> *>(ps + c0);
                    if (!all_kept) {
#pragma unroll
                        for (int e = 0; e < VEC; ++e) {
                            const bool keep = a.upper ? c0 + e >= edge : c0 + e <= edge;
                            if (!keep) x.v[e] = W{0};
                        }
                    }
                }
                *reinterpret_cast<Pack<W, VEC> *>(po + c0) = x;
            }
            // the columns after the last whole vector
            const int64_t c = nvec * VEC + static_cast<int64_t>(blockIdx.x) * kTriThreads + threadIdx.x;
            if (c < a.cols) {
                const bool keep = a.upper ? c >= edge : c <= edge;
                po[c] = keep ? ps[c] : W{0};
            }
        } else {
            for (int64_t c = static_cast<int64_t>(blockIdx.x) * kTriThreads + threadIdx.x; c < a.cols;
                 c += static_cast<int64_t>(gridDim.x) * kTriThreads) {
                const bool keep = a.upper ? c >= edge : c <= edge;
                po[c * a.out_col] = keep ? ps[c * a.src_col] : W{0};
            }
        }
    }
}

// Both tensors contiguous, rows a whole number of 32-byte groups, both 32-byte aligned: a thread takes groups of
// 32 bytes by their flat number (two in flight), finds (row, first column) with 32-bit divisions, and moves the group
// with one 256-bit load and store; groups outside the triangle are stored as zeros without the load.
struct FlatTriangleArgs {
    char *out;
    const char *src;
    uint32_t rows, groups_per_row;   // groups of 32 bytes
    int32_t upper;
    int64_t diagonal;
    int64_t groups;                  // below 2^32
};

template <class W>
__global__ void __launch_bounds__(kTriThreads) triangle_flat_kernel(const __grid_constant__ FlatTriangleArgs a) {
    constexpr int PER = 32 / sizeof(W);
    constexpr int UNR = 2;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kTriThreads;
    for (int64_t g0 = blockIdx.x * static_cast<int64_t>(kTriThreads) + threadIdx.x; g0 < a.groups; g0 += UNR * stride) {
        Bytes32 x[UNR];
        int64_t c0[UNR], edge[UNR];
        bool live[UNR], none[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int64_t g = g0 + u * stride;
            live[u] = g < a.groups;
            if (!live[u]) continue;
            const uint32_t line = static_cast<uint32_t>(g) / a.groups_per_row;
            const uint32_t r = line % a.rows;
            c0[u] = static_cast<int64_t>(static_cast<uint32_t>(g) - line * a.groups_per_row) * PER;
            edge[u] = static_cast<int64_t>(r) + a.diagonal;  // upper keeps c >= edge, lower keeps c <= edge
            none[u] = a.upper ? c0[u] + PER - 1 < edge[u] : c0[u] > edge[u];
            if (none[u]) {
#pragma unroll
                for (int e = 0; e < 8; ++e) x[u].w[e] = 0;
            } else {
                x[u] = load_32_bytes(a.src + g * 32);
            }
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            if (!live[u]) continue;
            const bool all = a.upper ? c0[u] >= edge[u] : c0[u] + PER - 1 <= edge[u];
            if (!none[u] && !all) {
                W v[PER];
                memcpy(v, &x[u], 32);
#pragma unroll
                for (int e = 0; e < PER; ++e) {
                    const bool keep = a.upper ? c0[u] + e >= edge[u] : c0[u] + e <= edge[u];
                    if (!keep) v[e] = W{0};
                }
                memcpy(&x[u], v, 32);
            }
            store_32_bytes(a.out + (g0 + u * stride) * 32, x[u]);
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

}  // namespace
}  // namespace hmc

using namespace hmc;

HMC_API hmc_status hmc_triangle(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *src, int64_t diagonal,
                                int32_t upper) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        const hmc_tensor_desc *d[2] = {out, src};
        int64_t n = 0;
        hmc_status s = check_operands(d, 2, &n);
        if (s != HMC_OK) return s;
        if (out->dtype != src->dtype) return fail(HMC_INVALID, "triangle writes its input's dtype");
        if (src->ndim < 2) return fail(HMC_INVALID, "triangle needs at least two dimensions");
        if (n == 0) return HMC_OK;
        if (out->data == nullptr || src->data == nullptr) return fail(HMC_INVALID, "null data pointer");
        const int nd = src->ndim;
        const int es = element_size(src->dtype);
        TriangleArgs a{};
        a.out = static_cast<char *>(out->data) + out->offset * es;
        a.src = static_cast<const char *>(src->data) + src->offset * es;
        a.nbatch = nd - 2;
        a.upper = upper != 0;
        a.diagonal = diagonal;
        a.rows = src->sizes[nd - 2];
        a.cols = src->sizes[nd - 1];
        a.out_row = out->strides[nd - 2];
        a.out_col = out->strides[nd - 1];
        a.src_row = src->strides[nd - 2];
        a.src_col = src->strides[nd - 1];
        int64_t batch = 1;
        for (int k = 0; k < nd - 2; ++k) {
            a.batch_sizes[k] = src->sizes[k];
            a.out_batch[k] = out->strides[k];
            a.src_batch[k] = src->strides[k];
            batch *= src->sizes[k];
        }
        a.lines = batch * a.rows;
        // r + diagonal must not overflow: clamp the diagonal to the matrix (beyond it nothing changes)
        const int64_t reach = a.rows + a.cols + 1;
        if (a.diagonal > reach) a.diagonal = reach;
        if (a.diagonal < -reach) a.diagonal = -reach;
        // the flat kernel where both tensors are contiguous and cut into whole, aligned groups of 32 bytes
        {
            bool flat = (a.cols * es) % 32 == 0 && ((reinterpret_cast<uintptr_t>(a.out) | reinterpret_cast<uintptr_t>(a.src)) & 31) == 0 &&
                        a.rows < (int64_t{1} << 31);
            int64_t expect = 1;
            for (int k = nd - 1; k >= 0 && flat; --k) {
                flat = (src->sizes[k] == 1 || (src->strides[k] == expect && out->strides[k] == expect));
                expect *= src->sizes[k];
            }
            const int64_t groups = n / (32 / es);
            if (flat && groups < (int64_t{1} << 32)) {
                FlatTriangleArgs f{a.out, const_cast<const char *>(a.src), static_cast<uint32_t>(a.rows),
                                   static_cast<uint32_t>(a.cols * es / 32), a.upper, a.diagonal, groups};
                const int64_t blocks = ceil_div(groups, static_cast<int64_t>(2 * kTriThreads));
                const unsigned g = static_cast<unsigned>(blocks < (int64_t{1} << 20) ? blocks : (int64_t{1} << 20));
                return by_size(src->dtype, [&](auto w) -> hmc_status {
                    triangle_flat_kernel<decltype(w)><<<g, kTriThreads, 0, ctx->stream>>>(f);
                    return launch_status("triangle kernel launch");
                });
            }
        }
        // up to four vectors per thread, so that a thread's share of finding its line is spread over 64 bytes
        const int64_t per_line = ceil_div(a.cols, 4 * kTriThreads * (16 / es));
        dim3 grid(static_cast<unsigned>(per_line < 1 ? 1 : (per_line < 65535 ? per_line : 65535)),
                  static_cast<unsigned>(a.lines < 65535 ? a.lines : 65535));
        return by_size(src->dtype, [&](auto w) -> hmc_status {
            triangle_kernel<decltype(w)><<<grid, kTriThreads, 0, ctx->stream>>>(a);
            return launch_status("triangle kernel launch");
        });
    });
}

HMC_API hmc_status hmc_flip(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *src) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        // src is checked here rather than by check_operands: its strides may be negative
        hmc_status s = check_desc(out, "the output");
        if (s != HMC_OK) return s;
        if (src == nullptr) return fail(HMC_INVALID, "null description of the input");
        if (!dtype_valid(src->dtype) || src->dtype != out->dtype) return fail(HMC_INVALID, "flip writes its input's dtype");
        if (src->ndim != out->ndim) return fail(HMC_INVALID, "operands differ in their number of dimensions");
        if (src->offset < 0) return fail(HMC_INVALID, "negative offset of the input");
        int64_t n = 1;
        for (int k = 0; k < out->ndim; ++k) {
            if (src->sizes[k] != out->sizes[k]) return fail(HMC_INVALID, "operands differ in their sizes");
            if (__builtin_mul_overflow(n, out->sizes[k], &n)) return fail(HMC_INVALID, "the number of elements overflows 63 bits");
        }
        if (n == 0) return HMC_OK;
        if (out->data == nullptr || src->data == nullptr) return fail(HMC_INVALID, "null data pointer");
        // every element the walk reaches must lie at or after the start of the storage
        int64_t lowest = src->offset;
        for (int k = 0; k < src->ndim; ++k) {
            if (src->strides[k] < 0) lowest += (src->sizes[k] - 1) * src->strides[k];
        }
        if (lowest < 0) return fail(HMC_INVALID, "the flipped view reaches before its storage");
        return launch_move(ctx, out, src);
    });
}
