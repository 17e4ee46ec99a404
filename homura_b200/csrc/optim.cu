// The decoupled-weight-decay Adam update of one parameter in a single kernel.
//
// homura's optimizer (src/optim/adam.rs:125-171) issues about fourteen elementwise kernels and six
// temporaries per parameter: p *= 1 - lr*wd; exp_avg = lerp(exp_avg, g, 1 - beta1);
// exp_avg_sq *= beta2; exp_avg_sq = addcmul(exp_avg_sq, g, g, 1 - beta2);
// denom = sqrt(exp_avg_sq) / sqrt(bias2) + eps; p = addcdiv(p, exp_avg, denom, -step_size).
// Every one of those kernels rounds its result to the parameter's dtype. This kernel performs the
// same operations in the same order on registers and rounds at the same points, so the three
// updated tensors carry the bits of the op-by-op path while reading and writing each of them once
// (28 bytes per f32 element instead of ~130).
#include <string>
#include <vector>

#include "functors.cuh"

namespace hmc {
namespace {

template <class T>
struct AdamW {
    using C = typename Comp<T>::C;
    C decay, lerp_coeff, beta2, one_minus_beta2, bias2_sqrt, eps, neg_step_size;
    bool has_decay, lerp_small;

    // Rounds to the dtype and widens again: the store and reload between two of homura's kernels.
    __device__ __forceinline__ static C rt(C c) { return up(down<T>(c)); }

    __device__ __forceinline__ void operator()(T &p, T g0, T &m0, T &v0) const {
        C x = up(p);
        const C g = up(g0);
        const C m = up(m0);
        const C v = up(v0);
        if (has_decay) x = rt(x * decay);
        const C m1 = rt(m_fma(lerp_coeff, g - m, lerp_small ? m : g));
        const C v1 = rt(v * beta2);
        const C v2 = rt(m_fma(one_minus_beta2 * g, g, v1));
        const C s = rt(m_sqrt(v2));
        const C d = rt(s / bias2_sqrt);
        const C d2 = rt(d + eps);
        const C x1 = x + neg_step_size * m1 / d2;
        p = down<T>(x1);
        m0 = down<T>(m1);
        v0 = down<T>(v2);
    }
};

// Same walk as map_kernel (operand 0 param, 1 grad, 2 exp_avg, 3 exp_avg_sq), three of them written.
template <class T>
__global__ void __launch_bounds__(kThreads) adamw_kernel(const __grid_constant__ MapArgs a, const AdamW<T> f) {
    constexpr int VEC = 16 / sizeof(T);
    constexpr int UNR = 2;
    const int tpr = 1 << a.tpr_log2;
    const int lane = threadIdx.x & (tpr - 1);
    const int rib = threadIdx.x >> a.tpr_log2;
    const int rpb = kThreads >> a.tpr_log2;
    const int64_t step = static_cast<int64_t>(tpr) * VEC;
    int mode[kOperands];
#pragma unroll
    for (int k = 0; k < kOperands; ++k) mode[k] = operand_mode(a, k);
    for (int64_t item = blockIdx.x; item < a.items; item += gridDim.x) {
        int64_t rg, seg;
        if (a.rows == 1) { rg = 0; seg = item; }
        else if (a.segs == 1) { rg = item; seg = 0; }
        else if (a.segs_shift != 0) {
            rg = static_cast<int64_t>((static_cast<uint64_t>(item) * a.segs_magic) >> a.segs_shift);
            seg = item - rg * a.segs;
        } else { rg = item / a.segs; seg = item - rg * a.segs; }
        const int64_t row = rg * rpb + rib;
        if (row >= a.rows) continue;
        int64_t off[kOperands];
        row_offsets(a, row, off);
        T *pp = operand_row<T>(a, 0, off[0]);
        const T *pg = operand_row<T>(a, 1, off[1]);
        T *pm = operand_row<T>(a, 2, off[2]);
        T *pv = operand_row<T>(a, 3, off[3]);
        const int64_t i0 = seg * (step * UNR) + static_cast<int64_t>(lane) * VEC;
        Pack<T, VEC> vp[UNR], vg[UNR], vm[UNR], vv[UNR];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int64_t idx = i0 + u * step;
            if (idx < a.n0) {
                load_operand<T, VEC>(vp[u], a, 0, mode[0], pp, idx);
                load_operand<T, VEC>(vg[u], a, 1, mode[1], pg, idx);
                load_operand<T, VEC>(vm[u], a, 2, mode[2], pm, idx);
                load_operand<T, VEC>(vv[u], a, 3, mode[3], pv, idx);
            }
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const int64_t idx = i0 + u * step;
            if (idx < a.n0) {
#pragma unroll
                for (int j = 0; j < VEC; ++j) f(vp[u].v[j], vg[u].v[j], vm[u].v[j], vv[u].v[j]);
                store_operand<T, VEC>(vp[u], a, 0, mode[0], pp, idx);
                store_operand<T, VEC>(vm[u], a, 2, mode[2], pm, idx);
                store_operand<T, VEC>(vv[u], a, 3, mode[3], pv, idx);
            }
        }
    }
}


// ---- many parameters in one launch ----
//
// An optimizer step over a model is hundreds of tensors, some of a few hundred elements (norm weights): a launch
// per tensor makes the small ones cost as much as a launch each and leaves the GPU draining between the large
// ones. Here the tensors of one parameter group (same scalars) are described by a table in device memory; the
// work is cut into chunks of kManyChunk elements that never span two tensors, a persistent grid takes the
// chunks in turn, and a chunk finds its tensor by a binary search over the running chunk counts. The
// arithmetic is AdamW<T> above, so every element has the bits of hmc_adamw_step and of the op-by-op path.
//
// The squares of the gradient (what `g.mul(&g).sum()` adds up for a gradient norm) can be summed on the way,
// since the gradient is in registers anyway: each product is rounded to the dtype as the elementwise kernel
// would round it, accumulated in f64 per thread in element order, folded over the block in lane order into one
// partial per chunk, and a second small kernel folds each tensor's partials in chunk order: the same bits on
// every run and for every grid size.
struct ManyTensor {
    char *param;
    const char *grad;
    char *exp_avg;
    char *exp_avg_sq;
    int64_t n;
};

constexpr int kManyUnroll = 2;
template <class T> constexpr int many_vec() { return 32 / static_cast<int>(sizeof(T)); }
template <class T> constexpr int many_chunk() { return kThreads * many_vec<T>() * kManyUnroll; }

template <class T, int VEC>
__device__ __forceinline__ void load_wide(Pack<T, VEC> &dst, const T *p) {
    const Bytes32 v = load_32_bytes(p);
    memcpy(&dst, &v, 32);
}
template <class T, int VEC>
__device__ __forceinline__ void store_wide(T *p, const Pack<T, VEC> &src) {
    Bytes32 v;
    memcpy(&v, &src, 32);
    store_32_bytes(p, v);
}

template <class T, bool NORM>
__global__ void __launch_bounds__(kThreads) adamw_many_kernel(const ManyTensor *__restrict__ tensors,
                                                              const int64_t *__restrict__ first_chunk, int count,
                                                              int64_t chunks, const AdamW<T> f,
                                                              double *__restrict__ partials) {
    using C = typename Comp<T>::C;
    constexpr int VEC = many_vec<T>();
    constexpr int CHUNK = many_chunk<T>();
    __shared__ double warp_sums[kThreads / 32];
    for (int64_t chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x) {
        // the last tensor whose first chunk is not after this one (first_chunk has count + 1 entries)
        int lo = 0, hi = count;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (first_chunk[mid] <= chunk) lo = mid; else hi = mid;
        }
        const ManyTensor t = tensors[lo];
        const int64_t base = (chunk - first_chunk[lo]) * CHUNK;
        const int64_t left = t.n - base;
        T *pp = reinterpret_cast<T *>(t.param) + base;
        const T *pg = reinterpret_cast<const T *>(t.grad) + base;
        T *pm = reinterpret_cast<T *>(t.exp_avg) + base;
        T *pv = reinterpret_cast<T *>(t.exp_avg_sq) + base;
        const bool wide = ((reinterpret_cast<uintptr_t>(pp) | reinterpret_cast<uintptr_t>(pg) | reinterpret_cast<uintptr_t>(pm) |
                            reinterpret_cast<uintptr_t>(pv)) & 31) == 0;
        double acc = 0.0;
        if (left >= CHUNK && wide) {
            Pack<T, VEC> vp[kManyUnroll], vg[kManyUnroll], vm[kManyUnroll], vv[kManyUnroll];
#pragma unroll
            for (int u = 0; u < kManyUnroll; ++u) {
                const int i = (u * kThreads + static_cast<int>(threadIdx.x)) * VEC;
                load_wide<T, VEC>(vp[u], pp + i);
                load_wide<T, VEC>(vg[u], pg + i);
                load_wide<T, VEC>(vm[u], pm + i);
                load_wide<T, VEC>(vv[u], pv + i);
            }
#pragma unroll
            for (int u = 0; u < kManyUnroll; ++u) {
                const int i = (u * kThreads + static_cast<int>(threadIdx.x)) * VEC;
#pragma unroll
                for (int j = 0; j < VEC; ++j) {
                    if constexpr (NORM) {
                        const C g = up(vg[u].v[j]);
                        acc += static_cast<double>(AdamW<T>::rt(g * g));
                    }
                    f(vp[u].v[j], vg[u].v[j], vm[u].v[j], vv[u].v[j]);
                }
                store_wide<T, VEC>(pp + i, vp[u]);
                store_wide<T, VEC>(pm + i, vm[u]);
                store_wide<T, VEC>(pv + i, vv[u]);
            }
        } else {
            // a tensor's last chunk, or tensors that do not start on a 32-byte boundary: element by element,
            // each thread the same elements it owns in the fast path, so the sums fold in the same order
            const int64_t n = left < CHUNK ? left : CHUNK;
#pragma unroll
            for (int u = 0; u < kManyUnroll; ++u) {
                const int64_t i0 = (u * kThreads + static_cast<int>(threadIdx.x)) * VEC;
                for (int j = 0; j < VEC; ++j) {
                    const int64_t i = i0 + j;
                    if (i >= n) break;
                    T p = pp[i], m = pm[i], v = pv[i];
                    const T g = pg[i];
                    if constexpr (NORM) {
                        const C gc = up(g);
                        acc += static_cast<double>(AdamW<T>::rt(gc * gc));
                    }
                    f(p, g, m, v);
                    pp[i] = p;
                    pm[i] = m;
                    pv[i] = v;
                }
            }
        }
        if constexpr (NORM) {
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, d);
            if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = acc;
            __syncthreads();
            if (threadIdx.x == 0) {
                double s = warp_sums[0];
#pragma unroll
                for (int w = 1; w < kThreads / 32; ++w) s += warp_sums[w];
                partials[chunk] = s;
            }
            __syncthreads();
        }
    }
}

// grad_sq[t] = the partials of tensor t added in chunk order: a warp per tensor, lane l takes partials
// l, l + 32, ..., then the lanes fold in a fixed tree.
__global__ void __launch_bounds__(kThreads) adamw_many_fold_kernel(const int64_t *__restrict__ first_chunk, int count,
                                                                   const double *__restrict__ partials,
                                                                   double *__restrict__ grad_sq) {
    const int t = static_cast<int>((static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5);
    if (t >= count) return;
    const int lane = threadIdx.x & 31;
    double s = 0.0;
    for (int64_t c = first_chunk[t] + lane; c < first_chunk[t + 1]; c += 32) s += partials[c];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) s += __shfl_down_sync(0xffffffffu, s, d);
    if (lane == 0) grad_sq[t] = s;
}

inline int64_t align256(int64_t n) { return (n + 255) / 256 * 256; }

// Chunk counts and the workspace layout: [tensor table][first_chunk, count + 1][partials, one per chunk].
struct ManyLayout {
    int64_t chunks = 0, table_bytes = 0, prefix_bytes = 0, partial_bytes = 0;
    int64_t total() const { return table_bytes + prefix_bytes + partial_bytes; }
};
hmc_status many_layout(int32_t dtype, const hmc_adamw_tensor *tensors, int64_t count, bool norm, ManyLayout &l,
                       std::vector<int64_t> *first_chunk) {
    if (!dtype_is_float(dtype)) return fail(HMC_INVALID, "an AdamW step takes floating point tensors");
    if (count < 0 || count > (1 << 24)) return fail(HMC_INVALID, "tensor count out of range");
    if (count > 0 && tensors == nullptr) return fail(HMC_INVALID, "null tensor table");
    const int64_t chunk = kThreads * (32 / static_cast<int64_t>(element_size(dtype))) * kManyUnroll;
    if (first_chunk != nullptr) first_chunk->assign(static_cast<size_t>(count) + 1, 0);
    int64_t chunks = 0;
    for (int64_t t = 0; t < count; ++t) {
        const hmc_adamw_tensor &x = tensors[t];
        if (x.n < 0) return fail(HMC_INVALID, "negative element count");
        if (x.n > 0 && (x.param == nullptr || x.grad == nullptr || x.exp_avg == nullptr || x.exp_avg_sq == nullptr)) {
            return fail(HMC_INVALID, "null tensor in the table");
        }
        if (first_chunk != nullptr) (*first_chunk)[static_cast<size_t>(t)] = chunks;
        chunks += ceil_div(x.n, chunk);
    }
    if (first_chunk != nullptr) (*first_chunk)[static_cast<size_t>(count)] = chunks;
    l.chunks = chunks;
    l.table_bytes = align256(count * static_cast<int64_t>(sizeof(ManyTensor)));
    l.prefix_bytes = align256((count + 1) * 8);
    l.partial_bytes = norm ? align256(chunks * 8) : 0;
    return HMC_OK;
}

}  // namespace
}  // namespace hmc

using namespace hmc;

HMC_API hmc_status hmc_adamw_step(hmc_context_t ctx, const hmc_tensor_desc *param, const hmc_tensor_desc *grad,
                                  const hmc_tensor_desc *exp_avg, const hmc_tensor_desc *exp_avg_sq,
                                  const hmc_adamw_scalars *scalars) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        if (scalars == nullptr) return fail(HMC_INVALID, "null scalars");
        const hmc_tensor_desc *d[4] = {param, grad, exp_avg, exp_avg_sq};
        for (int k = 0; k < 4; ++k) {
            if (d[k] == nullptr) return fail(HMC_INVALID, "null description");
        }
        int64_t n = 0;
        hmc_status s = check_operands(d, 4, &n);
        if (s != HMC_OK) return s;
        const int dt = param->dtype;
        if (!dtype_is_float(dt) || grad->dtype != dt || exp_avg->dtype != dt || exp_avg_sq->dtype != dt) {
            return fail(HMC_INVALID, "an AdamW step takes floating point tensors of one dtype");
        }
        if (n == 0) return HMC_OK;
        return dispatch_float(dt, [&](auto t) -> hmc_status {
            using T = decltype(t);
            using C = typename Comp<T>::C;
            AdamW<T> f;
            f.decay = static_cast<C>(scalars->decay);
            f.lerp_coeff = static_cast<C>(scalars->lerp_coeff);
            f.beta2 = static_cast<C>(scalars->beta2);
            f.one_minus_beta2 = static_cast<C>(scalars->one_minus_beta2);
            f.bias2_sqrt = static_cast<C>(scalars->bias2_sqrt);
            f.eps = static_cast<C>(scalars->eps);
            f.neg_step_size = static_cast<C>(scalars->neg_step_size);
            f.has_decay = scalars->has_decay != 0;
            f.lerp_small = scalars->lerp_small != 0;
            MapOperand in[3] = {tensor_operand(grad), tensor_operand(exp_avg), tensor_operand(exp_avg_sq)};
            MapArgs a;
            build_map_args(a, param, in, 3, 16 / static_cast<int>(sizeof(T)), 2);
            const int64_t cap = static_cast<int64_t>(ctx->sm_count) * 16;
            const unsigned grid = static_cast<unsigned>(a.items < cap ? a.items : cap);
            adamw_kernel<T><<<grid, kThreads, 0, ctx->stream>>>(a, f);
            return launch_status("adamw kernel launch");
        });
    });
}

HMC_API hmc_status hmc_adamw_step_many_workspace(int32_t dtype, const hmc_adamw_tensor *tensors, int64_t count,
                                                 int32_t with_grad_sq, int64_t *bytes) {
    return guarded([&]() -> hmc_status {
        if (bytes == nullptr) return fail(HMC_INVALID, "null result");
        ManyLayout l;
        hmc_status s = many_layout(dtype, tensors, count, with_grad_sq != 0, l, nullptr);
        if (s != HMC_OK) return s;
        *bytes = l.total();
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_adamw_step_many(hmc_context_t ctx, int32_t dtype, const hmc_adamw_tensor *tensors, int64_t count,
                                       const hmc_adamw_scalars *scalars, double *grad_sq, void *workspace,
                                       int64_t workspace_bytes) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        if (scalars == nullptr) return fail(HMC_INVALID, "null scalars");
        ManyLayout l;
        std::vector<int64_t> first_chunk;
        hmc_status s = many_layout(dtype, tensors, count, grad_sq != nullptr, l, &first_chunk);
        if (s != HMC_OK) return s;
        if (count == 0) return HMC_OK;
        if (workspace == nullptr || workspace_bytes < l.total()) {
            return fail(HMC_INVALID, "the workspace of an AdamW step over many tensors is too small: " +
                                         std::to_string(workspace_bytes) + " bytes given, " + std::to_string(l.total()) + " needed");
        }
        if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0) return fail(HMC_INVALID, "the workspace is not 256-byte aligned");
        std::vector<ManyTensor> table(static_cast<size_t>(count));
        for (int64_t t = 0; t < count; ++t) {
            table[static_cast<size_t>(t)] = ManyTensor{static_cast<char *>(tensors[t].param), static_cast<const char *>(tensors[t].grad),
                                                       static_cast<char *>(tensors[t].exp_avg),
                                                       static_cast<char *>(tensors[t].exp_avg_sq), tensors[t].n};
        }
        char *ws = static_cast<char *>(workspace);
        ManyTensor *d_table = reinterpret_cast<ManyTensor *>(ws);
        int64_t *d_first = reinterpret_cast<int64_t *>(ws + l.table_bytes);
        double *d_partials = reinterpret_cast<double *>(ws + l.table_bytes + l.prefix_bytes);
        // pageable host memory: the runtime has staged the bytes when these calls return, so the vectors may go
        HMC_CUDA(cudaMemcpyAsync(d_table, table.data(), table.size() * sizeof(ManyTensor), cudaMemcpyHostToDevice, ctx->stream),
                 "copy of the tensor table");
        HMC_CUDA(cudaMemcpyAsync(d_first, first_chunk.data(), first_chunk.size() * 8, cudaMemcpyHostToDevice, ctx->stream),
                 "copy of the chunk table");
        if (l.chunks == 0) {
            if (grad_sq != nullptr) HMC_CUDA(cudaMemsetAsync(grad_sq, 0, static_cast<size_t>(count) * 8, ctx->stream), "memset");
            return HMC_OK;
        }
        return dispatch_float(dtype, [&](auto tt) -> hmc_status {
            using T = decltype(tt);
            using C = typename Comp<T>::C;
            AdamW<T> f;
            f.decay = static_cast<C>(scalars->decay);
            f.lerp_coeff = static_cast<C>(scalars->lerp_coeff);
            f.beta2 = static_cast<C>(scalars->beta2);
            f.one_minus_beta2 = static_cast<C>(scalars->one_minus_beta2);
            f.bias2_sqrt = static_cast<C>(scalars->bias2_sqrt);
            f.eps = static_cast<C>(scalars->eps);
            f.neg_step_size = static_cast<C>(scalars->neg_step_size);
            f.has_decay = scalars->has_decay != 0;
            f.lerp_small = scalars->lerp_small != 0;
            const int64_t cap = static_cast<int64_t>(ctx->sm_count) * 4;
            const unsigned grid = static_cast<unsigned>(l.chunks < cap ? l.chunks : cap);
            if (grad_sq != nullptr) {
                adamw_many_kernel<T, true><<<grid, kThreads, 0, ctx->stream>>>(d_table, d_first, static_cast<int>(count), l.chunks, f, d_partials);
                hmc_status ls = launch_status("adamw kernel launch");
                if (ls != HMC_OK) return ls;
                const unsigned fold_grid = static_cast<unsigned>(ceil_div(count * 32, kThreads));
                adamw_many_fold_kernel<<<fold_grid, kThreads, 0, ctx->stream>>>(d_first, static_cast<int>(count), d_partials, grad_sq);
                return launch_status("gradient square fold launch");
            }
            adamw_many_kernel<T, false><<<grid, kThreads, 0, ctx->stream>>>(d_table, d_first, static_cast<int>(count), l.chunks, f, nullptr);
            return launch_status("adamw kernel launch");
        });
    });
}
