// Float sum / prod / mean and var / std.
#include "math.cuh"
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
// second walk over the row finds it in cache. The folds and the team's order are those of the two
// separate reductions, so both routes give the same bits. Grid: one block per 256 / G outputs.
template <int G, class T>
__global__ void __launch_bounds__(kRThreads) deviations_kernel(const __grid_constant__ ReduceArgs a, const VarSink<T> sink) {
    constexpr int kTeams = kRThreads / G;
    const ReducePlan &p = a.plan;
    const int lane = threadIdx.x % G;
    const int team = threadIdx.x / G;
    __shared__ double mean_of[kTeams];
    const FloatFold<T, false> fold;
    const int64_t o = static_cast<int64_t>(blockIdx.x) * kTeams + team;
    const bool live = o < p.nout;
    const int64_t base = live ? a.kept.offset + decompose(a.kept, o, a.kept.ndim) : 0;
    double sum = live ? fold_span<G>(fold, a, o, base, 0, p.nred, lane) : 0.0;
    sum = fold_team<G>(fold, sum);
    if (lane == 0) mean_of[team] = sum / static_cast<double>(p.nred);
    if constexpr (G == 32) __syncwarp();
    else __syncthreads();
    const SquaredDeviation<T> dev{nullptr, mean_of[team]};
    double sq = live ? fold_span<G>(dev, a, o, base, 0, p.nred, lane) : 0.0;
    sq = fold_team<G>(dev, sq);
    if (lane == 0 && live) sink.put(o, sq, p.nred);
}


// ---- variance over columns in one pass ----
// The layout of reduce_columns_kernel (a thread owns VC adjacent outputs, the 8 warps of a block take the reduced
// indices j, j + 8, ...), but instead of a pass for the means and a pass for the deviations a thread keeps
// (count, mean, M2 = sum of squared deviations from that mean) per output and merges batches of four rows into
// them with the pairwise update of Chan, Golub and LeVeque: the batch's own mean and M2 first (exact two-pass
// on its B values), then mean += d * B / n, M2 += M2_batch + d * d * (n - B) * B / n with d = batch mean - mean.
// All in f64: the result differs from the two-pass value by a few f64 ulps, far below the rounding to F16,
// BF16 or F32 (F64 tensors keep the two passes). One read of the source instead of two.
struct Moments {
    double mean, m2;
};
static_assert(sizeof(Moments) == kPartialBytes, "the moments of a chunk are one partial");

__device__ __forceinline__ void merge_moments(double &n, double &mean, double &m2, double nb, double mean_b, double m2_b) {
    if (nb == 0.0) return;
    const double total = n + nb;
    const double d = mean_b - mean;
    const double w = nb * reciprocal_short(total);  // counts are small whole numbers: an ulp or two off nb / total
    mean = n == 0.0 ? mean_b : mean + d * w;
    m2 = n == 0.0 ? m2_b : m2 + m2_b + d * d * n * w;
    n = total;
}

template <class T>
__global__ void __launch_bounds__(kRThreads) var_columns_kernel(const __grid_constant__ ReduceArgs a, const VarSink<T> sink) {
    constexpr int VC = (16 / sizeof(T)) > 8 ? 8 : (16 / sizeof(T));
    constexpr int UNR = 4;  // rows of a batch, all in flight at once (8 measured slower: registers)
    const ReducePlan &p = a.plan;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t chunk = blockIdx.y;
    const int64_t j0 = chunk * p.chunk;
    const int64_t j1 = j0 + p.chunk < p.nred ? j0 + p.chunk : p.nred;
    const int last = a.kept.ndim - 1;
    __shared__ double stage_mean[7][32 * VC];
    __shared__ double stage_m2[7][32 * VC];
    __shared__ double stage_n[8];
    // Grid: (kouter * xtiles, splits), one block per strip of 32 * VC outputs and chunk.
    const int64_t outer = blockIdx.x / p.xtiles;
    const int64_t tile = blockIdx.x - outer * p.xtiles;
    const int64_t c0 = tile * (32 * VC) + static_cast<int64_t>(tx) * VC;
    const int64_t base = a.kept.offset + (last > 0 ? decompose(a.kept, outer, last) : 0);
    const int64_t o0 = outer * p.ncols + c0;
    const T *src = static_cast<const T *>(a.kept.data) + base + c0;
    double n = 0.0, mean[VC], m2[VC];
#pragma unroll
    for (int e = 0; e < VC; ++e) mean[e] = m2[e] = 0.0;
    const bool in_range = c0 < p.ncols;
    const bool whole = c0 + VC <= p.ncols;
    if (in_range) {
        const int64_t stride = a.red.strides[0];
        const bool single = a.red.ndim == 1;
        const bool walk = single && whole && (reinterpret_cast<uintptr_t>(src) & (alignof(RVec<T, VC>) - 1)) == 0 &&
                          (stride * static_cast<int64_t>(sizeof(T))) % static_cast<int64_t>(alignof(RVec<T, VC>)) == 0;
        auto red_off = [&](int64_t j) { return single ? j * stride : decompose(a.red, j, a.red.ndim); };
        int64_t j = j0 + ty;
        if (walk) {
            // whole aligned vectors along one reduced dimension: batches of four rows, a pointer that steps by eight
            const T *q = src + j * stride;
            const int64_t step = 8 * stride;
            for (; j + (UNR - 1) * 8 < j1; j += UNR * 8, q += UNR * step) {
                RVec<T, VC> x[UNR];
#pragma unroll
                for (int u = 0; u < UNR; ++u) x[u] = *reinterpret_cast<const RVec<T, VC> *>(q + u * step);
                const double total = n + UNR;
                const double w = UNR / total;
#pragma unroll
                for (int e = 0; e < VC; ++e) {
                    double v[UNR];
#pragma unroll
                    for (int u = 0; u < UNR; ++u) v[u] = to_f64(x[u].v[e]);
                    double sum = 0.0;
#pragma unroll
                    for (int u = 0; u < UNR; ++u) sum += v[u];
                    const double mb = sum * (1.0 / UNR);
                    double sq = 0.0;
#pragma unroll
                    for (int u = 0; u < UNR; ++u) sq += (v[u] - mb) * (v[u] - mb);
                    const double d = mb - mean[e];
                    mean[e] = n == 0.0 ? mb : mean[e] + d * w;
                    m2[e] = n == 0.0 ? sq : m2[e] + sq + d * d * n * w;
                }
                n = total;
            }
        }
        for (; j < j1; j += 8) {
            const T *q = src + red_off(j);
            const double total = n + 1.0;
            const double w = 1.0 / total;
#pragma unroll
            for (int e = 0; e < VC; ++e) {
                if (c0 + e < p.ncols) {
                    const double v = to_f64(q[e]);
                    const double d = v - mean[e];
                    mean[e] = n == 0.0 ? v : mean[e] + d * w;
                    m2[e] = n == 0.0 ? 0.0 : m2[e] + d * d * n * w;
                }
            }
            n = total;
        }
    }
    if (ty > 0) {
#pragma unroll
        for (int e = 0; e < VC; ++e) {
            stage_mean[ty - 1][tx * VC + e] = mean[e];
            stage_m2[ty - 1][tx * VC + e] = m2[e];
        }
    }
    if (tx == 0) stage_n[ty] = n;
    __syncthreads();
    if (ty == 0 && in_range) {
#pragma unroll
        for (int e = 0; e < VC; ++e) {
            if (c0 + e >= p.ncols) continue;
            double cn = n, cm = mean[e], c2 = m2[e];
            for (int w = 0; w < 7; ++w) merge_moments(cn, cm, c2, stage_n[w + 1], stage_mean[w][tx * VC + e], stage_m2[w][tx * VC + e]);
            if (p.splits == 1) sink.put(o0 + e, c2, p.nred);
            else static_cast<Moments *>(a.partials)[chunk * p.nout + o0 + e] = Moments{cm, c2};
        }
    }
}

// The chunks' moments of each output merged in chunk order (a chunk's count follows from the plan).
template <class T>
__global__ void __launch_bounds__(kRThreads) var_combine_kernel(const __grid_constant__ ReduceArgs a, const VarSink<T> sink) {
    const ReducePlan &p = a.plan;
    const Moments *partials = static_cast<const Moments *>(a.partials);
    for (int64_t o = blockIdx.x * static_cast<int64_t>(kRThreads) + threadIdx.x; o < p.nout;
         o += static_cast<int64_t>(gridDim.x) * kRThreads) {
        double n = 0.0, mean = 0.0, m2 = 0.0;
        for (int64_t c = 0; c < p.splits; ++c) {
            const int64_t j0 = c * p.chunk;
            const int64_t j1 = j0 + p.chunk < p.nred ? j0 + p.chunk : p.nred;
            const Moments m = partials[c * p.nout + o];
            merge_moments(n, mean, m2, static_cast<double>(j1 - j0), m.mean, m.m2);
        }
        sink.put(o, m2, p.nred);
    }
}

// ---- variance over rows in one pass ----
// The same moments for rows that are one unit-stride run of whole, aligned vectors (plan.simple): a lane merges
// batches of up to four vectors (exact two-pass moments of the 16 or 32 values in registers) into its
// (count, mean, M2), the lanes of a row are merged in lane order by shuffles and, for 256 lanes, the warps in
// warp order through shared memory. The row is read once; the two-pass kernel above reads it twice and misses
// the caches for part of the second walk.
template <class T, int N>
__device__ __forceinline__ void batch_moments(const double (&v)[N], double &mean_b, double &m2_b) {
    double s = 0.0;
#pragma unroll
    for (int i = 0; i < N; ++i) s += v[i];
    mean_b = s * (1.0 / N);
    double sq = 0.0;
#pragma unroll
    for (int i = 0; i < N; ++i) sq += (v[i] - mean_b) * (v[i] - mean_b);
    m2_b = sq;
}

template <int G, class T>
__global__ void __launch_bounds__(kRThreads) var_rows_kernel(const __grid_constant__ ReduceArgs a, const VarSink<T> sink) {
    constexpr int P = kRThreads / G;
    constexpr int VEC = 16 / sizeof(T);
    constexpr int UNR = 4;
    const ReducePlan &p = a.plan;
    const int lane = threadIdx.x % G;
    const int slot = threadIdx.x / G;
    __shared__ double warp_n[8], warp_mean[8], warp_m2[8];
    const uint32_t nvec = static_cast<uint32_t>(p.nred) / VEC;
    const int64_t tiles = (p.nout + P - 1) / P;
    for (int64_t tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const int64_t o = tile * P + slot;
        const bool valid = o < p.nout;
        double n = 0.0, mean = 0.0, m2 = 0.0;
        if (valid) {
            const T *row = static_cast<const T *>(a.kept.data) + a.kept.offset + decompose(a.kept, o, a.kept.ndim);
            uint32_t v = lane;
            for (; v + (UNR - 1) * G < nvec; v += UNR * G) {
                RVec<T, VEC> x[UNR];
#pragma unroll
                for (int u = 0; u < UNR; ++u) x[u] = *reinterpret_cast<const RVec<T, VEC> *>(row + static_cast<size_t>(v + u * G) * VEC);
                double w[UNR * VEC];
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
#pragma unroll
                    for (int e = 0; e < VEC; ++e) w[u * VEC + e] = to_f64(x[u].v[e]);
                }
                double mb, sq;
                batch_moments<T, UNR * VEC>(w, mb, sq);
                merge_moments(n, mean, m2, static_cast<double>(UNR * VEC), mb, sq);
            }
            for (; v < nvec; v += G) {
                const RVec<T, VEC> x = *reinterpret_cast<const RVec<T, VEC> *>(row + static_cast<size_t>(v) * VEC);
                double w[VEC];
#pragma unroll
                for (int e = 0; e < VEC; ++e) w[e] = to_f64(x.v[e]);
                double mb, sq;
                batch_moments<T, VEC>(w, mb, sq);
                merge_moments(n, mean, m2, static_cast<double>(VEC), mb, sq);
            }
        }
        if constexpr (G > 1) {
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) {
                const double on = __shfl_down_sync(0xFFFFFFFFu, n, d);
                const double om = __shfl_down_sync(0xFFFFFFFFu, mean, d);
                const double o2 = __shfl_down_sync(0xFFFFFFFFu, m2, d);
                merge_moments(n, mean, m2, on, om, o2);
            }
        }
        if constexpr (G == 256) {
            const int warp = threadIdx.x >> 5;
            if ((threadIdx.x & 31) == 0) {
                warp_n[warp] = n;
                warp_mean[warp] = mean;
                warp_m2[warp] = m2;
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                for (int w = 1; w < 8; ++w) merge_moments(n, mean, m2, warp_n[w], warp_mean[w], warp_m2[w]);
            }
            __syncthreads();
        }
        if (lane == 0 && valid) sink.put(o, m2, p.nred);
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
            if constexpr (!std::is_same_v<T, double>) {
                // every row one aligned run of whole vectors: the one-pass kernel
                bool aligned = p.simple && p.group > 1 &&
                               (reinterpret_cast<uintptr_t>(a.kept.data) + static_cast<uintptr_t>(a.kept.offset) * sizeof(T)) % 16 == 0;
                for (int k = 0; k < a.kept.ndim; ++k) aligned = aligned && (a.kept.strides[k] * static_cast<int64_t>(sizeof(T))) % 16 == 0;
                if (aligned) {
                    const int64_t per = kRThreads / p.group;
                    const unsigned g = clamp_grid((p.nout + per - 1) / per, 1 << 20);
                    if (p.group == 256) var_rows_kernel<256, T><<<g, kRThreads, 0, ctx->stream>>>(a, sink);
                    else var_rows_kernel<32, T><<<g, kRThreads, 0, ctx->stream>>>(a, sink);
                    return launch_status("var kernel launch");
                }
            }
            const int64_t per_block = kRThreads / p.group;
            const int64_t blocks = (p.nout + per_block - 1) / per_block;
            if (blocks > 0x7FFFFFFF) return fail(HMC_INVALID, "a reduction with more than 2^31 blocks of outputs");
            const unsigned grid = static_cast<unsigned>(blocks);
            if (p.group == 256) deviations_kernel<256, T><<<grid, kRThreads, 0, ctx->stream>>>(a, sink);
            else if (p.group == 32) deviations_kernel<32, T><<<grid, kRThreads, 0, ctx->stream>>>(a, sink);
            else deviations_kernel<1, T><<<grid, kRThreads, 0, ctx->stream>>>(a, sink);
            return launch_status("var kernel launch");
        }
        if constexpr (!std::is_same_v<T, double>) {
            if (p.kind == 1) {
                if (p.kouter * p.xtiles > 0x7FFFFFFF) return fail(HMC_INVALID, "a reduction with more than 2^31 strips of outputs");
                dim3 grid(static_cast<unsigned>(p.kouter * p.xtiles), static_cast<unsigned>(p.splits));
                var_columns_kernel<T><<<grid, kRThreads, 0, ctx->stream>>>(a, sink);
                hmc_status s1 = launch_status("var kernel launch");
                if (s1 != HMC_OK || p.splits == 1) return s1;
                var_combine_kernel<T><<<clamp_grid((p.nout + kRThreads - 1) / kRThreads, 1 << 16), kRThreads, 0, ctx->stream>>>(a, sink);
                return launch_status("var combine kernel launch");
            }
        }
        hmc_status s = launch_reduce(a, FloatFold<T, false>{}, FloatSink<T>{nullptr, means, 2}, ctx->stream);
        if (s != HMC_OK) return s;
        return launch_reduce(a, SquaredDeviation<T>{means, 0.0}, sink, ctx->stream);
    });
}

}  // namespace hmc
