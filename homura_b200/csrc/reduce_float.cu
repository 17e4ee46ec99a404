// Float sum / prod / mean and var / std.
#include "reduce.cuh"

namespace hmc {

hmc_status reduce_float(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, ReduceArgs &a) {
    return dispatch_float(a.kept.dtype, [&](auto t) {
        using T = decltype(t);
        T *o = static_cast<T *>(out->data) + out->offset;
        if (op == HMC_REDUCE_PROD) return launch_reduce(a, FloatFold<T, true>{}, FloatSink<T>{o, nullptr, 0}, ctx->stream);
        return launch_reduce(a, FloatFold<T, false>{}, FloatSink<T>{o, nullptr, op == HMC_REDUCE_MEAN ? 1 : 0}, ctx->stream);
    });
}

hmc_status reduce_float_partial(hmc_context_t ctx, int32_t op, double *partial, ReduceArgs &a) {
    return dispatch_float(a.kept.dtype, [&](auto t) {
        using T = decltype(t);
        if (op == HMC_REDUCE_PROD) return launch_reduce(a, FloatFold<T, true>{}, FloatSink<T>{nullptr, partial, 3}, ctx->stream);
        return launch_reduce(a, FloatFold<T, false>{}, FloatSink<T>{nullptr, partial, 3}, ctx->stream);
    });
}

// The f64 sums of squared deviations from given f64 means, one per output (a shard's share of a variance).
hmc_status reduce_var_partial(hmc_context_t ctx, double *partial, ReduceArgs &a, const double *means) {
    return dispatch_float(a.kept.dtype, [&](auto t) {
        using T = decltype(t);
        return launch_reduce(a, SquaredDeviation<T>{means, 0.0}, FloatSink<T>{nullptr, partial, 3}, ctx->stream);
    });
}

namespace {

// Sum, mean and squared deviations of each output in one kernel, for plans without chunks: the
// second walk over the row finds it in cache. The folds and the lane tree are those of the two
// separate reductions, so both routes give the same bits.
template <int G, class T>
__global__ void __launch_bounds__(kRThreads) deviations_kernel(const __grid_constant__ ReduceArgs a, const VarSink<T> sink) {
    constexpr int P = kRThreads / G;
    const ReducePlan &p = a.plan;
    const int lane = threadIdx.x % G;
    const int slot = threadIdx.x / G;
    __shared__ double mean_of[P];
    FloatFold<T, false> fold;
    const int64_t tiles = (p.nout + P - 1) / P;
    for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int64_t o = tile * P + slot;
        const bool valid = o < p.nout;
        const int64_t base = valid ? a.kept.offset + decompose(a.kept, o, a.kept.ndim) : 0;
        const T *row = static_cast<const T *>(a.kept.data) + base;
        const bool simple = G > 1 && p.simple && (reinterpret_cast<uintptr_t>(row) & 15) == 0;
        const uint32_t nvec = static_cast<uint32_t>(p.nred) / (16 / sizeof(T));
        double sum = !valid ? 0.0 : (simple ? fold_simple_row<G>(fold, row, nvec, lane, o) : fold_range<G>(fold, a, o, base, 0, p.nred, lane));
        sum = group_combine<G>(fold, sum);
        if (lane == 0) mean_of[slot] = sum / static_cast<double>(p.nred);
        if constexpr (G > 1) {
            if constexpr (G == 32) __syncwarp(); else __syncthreads();
        }
        SquaredDeviation<T> dev{nullptr, mean_of[slot]};
        double sq = !valid ? 0.0 : (simple ? fold_simple_row<G>(dev, row, nvec, lane, o) : fold_range<G>(dev, a, o, base, 0, p.nred, lane));
        sq = group_combine<G>(dev, sq);
        if (lane == 0 && valid) sink.put(o, sq, p.nred);
        if constexpr (G == 256) __syncthreads();
    }
}

}  // namespace

hmc_status reduce_var(hmc_context_t ctx, const hmc_tensor_desc *out, ReduceArgs &a, double correction, int take_sqrt,
                      double *means) {
    return dispatch_float(a.kept.dtype, [&](auto t) -> hmc_status {
        using T = decltype(t);
        const ReducePlan &p = a.plan;
        T *o = static_cast<T *>(out->data) + out->offset;
        double divisor = static_cast<double>(p.nred) - correction;
        if (!(divisor > 0.0)) divisor = 0.0;
        VarSink<T> sink{o, divisor, take_sqrt};
        if (p.kind == 0 && p.splits == 1) {
            const int64_t per_block = kRThreads / p.group;
            const int64_t tiles = (p.nout + per_block - 1) / per_block;
            unsigned grid = clamp_grid(tiles, 1 << 20);
            if (p.group == 256) deviations_kernel<256, T><<<grid, kRThreads, 0, ctx->stream>>>(a, sink);
            else if (p.group == 32) deviations_kernel<32, T><<<grid, kRThreads, 0, ctx->stream>>>(a, sink);
            else deviations_kernel<1, T><<<grid, kRThreads, 0, ctx->stream>>>(a, sink);
            return launch_status("var kernel launch");
        }
        hmc_status s = launch_reduce(a, FloatFold<T, false>{}, FloatSink<T>{nullptr, means, 2}, ctx->stream);
        if (s != HMC_OK) return s;
        return launch_reduce(a, SquaredDeviation<T>{means, 0.0}, sink, ctx->stream);
    });
}

}  // namespace hmc
