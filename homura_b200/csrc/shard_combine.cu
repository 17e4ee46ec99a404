// The per-shard partial reduction and the rank-ordered combine of gathered partials (no NCCL in here).
#include "../../include/homura_cuda_shard.h"
#include "map.cuh"
#include "reduce.cuh"

namespace hmc {
namespace {

template <class T>
__global__ void combine_float_kernel(T *out, const double *gathered, int ranks, int64_t nout, int op, double count) {
    for (int64_t o = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; o < nout;
         o += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        double acc = op == HMC_REDUCE_PROD ? 1.0 : 0.0;
        for (int r = 0; r < ranks; ++r) {
            const double p = gathered[r * nout + o];
            acc = op == HMC_REDUCE_PROD ? acc * p : acc + p;
        }
        out[o] = from_f64<T>(op == HMC_REDUCE_MEAN ? acc / count : acc);
    }
}

__global__ void combine_means_kernel(double *means, const double *gathered, int ranks, int64_t nout, double count) {
    for (int64_t o = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; o < nout;
         o += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        double acc = 0.0;
        for (int r = 0; r < ranks; ++r) acc += gathered[r * nout + o];
        means[o] = acc / count;
    }
}

template <class T>
__global__ void combine_var_kernel(VarSink<T> sink, const double *gathered, int ranks, int64_t nout, int64_t count) {
    for (int64_t o = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; o < nout;
         o += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        double acc = 0.0;
        for (int r = 0; r < ranks; ++r) acc += gathered[r * nout + o];
        sink.put(o, acc, count);
    }
}

__global__ void combine_int_kernel(int64_t *out, const int64_t *gathered, int ranks, int64_t nout, int prod) {
    for (int64_t o = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; o < nout;
         o += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        uint64_t acc = prod ? 1 : 0;
        for (int r = 0; r < ranks; ++r) {
            const uint64_t p = static_cast<uint64_t>(gathered[r * nout + o]);
            acc = prod ? acc * p : acc + p;
        }
        out[o] = static_cast<int64_t>(acc);
    }
}

constexpr int kMaxRanks = 64;
struct Offsets {
    int64_t v[kMaxRanks];
};

template <class T, bool MAX>
__global__ void combine_extreme_kernel(T *values, int64_t *indices, const T *gv, const int64_t *gi, Offsets offsets,
                                       int ranks, int64_t nout) {
    Extreme<T, MAX> op;
    for (int64_t o = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; o < nout;
         o += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        Best<T> acc = op.init();
        for (int r = 0; r < ranks; ++r) {
            // Ranks hold consecutive blocks of the sharded dimension, so ordering by (rank, local index) is the
            // global order; without indices the rank alone orders equal values.
            const int64_t local = gi != nullptr ? gi[r * nout + o] : 0;
            const int64_t global = gi != nullptr ? local + offsets.v[r] : r;
            acc = op.combine(acc, Best<T>{gv[r * nout + o], global});
        }
        if (values != nullptr) values[o] = acc.v;
        if (indices != nullptr) indices[o] = acc.i;
    }
}

hmc_status check_flat_output(const hmc_tensor_desc *out, int64_t nout, const char *what) {
    hmc_status s = check_desc(out, what);
    if (s != HMC_OK) return s;
    if (desc_count(*out) != nout) return fail(HMC_INVALID, std::string(what) + " does not have one element per output");
    int64_t expect = 1;
    for (int k = out->ndim - 1; k >= 0; --k) {
        if (out->sizes[k] != 1 && out->strides[k] != expect) return fail(HMC_INVALID, std::string(what) + " is not contiguous");
        expect *= out->sizes[k];
    }
    if (nout > 0 && out->data == nullptr) return fail(HMC_INVALID, "null data pointer");
    return HMC_OK;
}

unsigned blocks_for(int64_t n) { return static_cast<unsigned>(std::min<int64_t>(std::max<int64_t>((n + 255) / 256, 1), 4096)); }

}  // namespace
}  // namespace hmc

using namespace hmc;

HMC_API hmc_status hmc_reduce_partial(hmc_context_t ctx, int32_t op, double *partial, const hmc_tensor_desc *kept,
                                      const hmc_tensor_desc *red, void *workspace, int64_t workspace_bytes) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        hmc_status s = check_desc(kept, "the kept dimensions");
        if (s != HMC_OK) return s;
        s = check_desc(red, "the reduced dimensions");
        if (s != HMC_OK) return s;
        if (op != HMC_REDUCE_SUM && op != HMC_REDUCE_PROD && op != HMC_REDUCE_MEAN) {
            return fail(HMC_INVALID, "hmc_reduce_partial takes SUM, PROD or MEAN");
        }
        if (!dtype_is_float(kept->dtype) || red->dtype != kept->dtype) {
            return fail(HMC_INVALID, "hmc_reduce_partial takes a floating point tensor");
        }
        ReduceArgs a{*kept, *red, make_reduce_plan(*kept, *red), nullptr, ctx->tickets};
        if (a.plan.nout == 0) return HMC_OK;
        if (partial == nullptr) return fail(HMC_INVALID, "null partials");
        if (a.plan.nred > 0 && kept->data == nullptr) return fail(HMC_INVALID, "null data pointer");
        const int64_t need = plan_partial_bytes(a.plan);
        if (need > 0 && (workspace == nullptr || workspace_bytes < need)) {
            return fail(HMC_INVALID, "the workspace of a reduction is too small: " + std::to_string(need) + " bytes needed");
        }
        a.partials = need > 0 ? workspace : nullptr;
        return reduce_float_partial(ctx, op, partial, a);
    });
}

HMC_API hmc_status hmc_shard_combine_float(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out,
                                           const double *gathered, int32_t ranks, int64_t nout, int64_t total_count) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        if (op != HMC_REDUCE_SUM && op != HMC_REDUCE_PROD && op != HMC_REDUCE_MEAN) {
            return fail(HMC_INVALID, "hmc_shard_combine_float takes SUM, PROD or MEAN");
        }
        if (ranks < 1 || nout < 0) return fail(HMC_INVALID, "bad rank or output count");
        hmc_status s = check_flat_output(out, nout, "the output");
        if (s != HMC_OK) return s;
        if (!dtype_is_float(out->dtype)) return fail(HMC_INVALID, "the output is a floating point tensor");
        if (nout == 0) return HMC_OK;
        if (gathered == nullptr) return fail(HMC_INVALID, "null partials");
        return dispatch_float(out->dtype, [&](auto t) -> hmc_status {
            using T = decltype(t);
            combine_float_kernel<T><<<blocks_for(nout), 256, 0, ctx->stream>>>(static_cast<T *>(out->data) + out->offset, gathered,
                                                                               ranks, nout, op, static_cast<double>(total_count));
            return launch_status("shard combine launch");
        });
    });
}

HMC_API hmc_status hmc_shard_combine_int(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out,
                                         const int64_t *gathered, int32_t ranks, int64_t nout) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        if (op != HMC_REDUCE_SUM && op != HMC_REDUCE_PROD) return fail(HMC_INVALID, "hmc_shard_combine_int takes SUM or PROD");
        if (ranks < 1 || nout < 0) return fail(HMC_INVALID, "bad rank or output count");
        hmc_status s = check_flat_output(out, nout, "the output");
        if (s != HMC_OK) return s;
        if (out->dtype != HMC_I64) return fail(HMC_INVALID, "the output is an I64 tensor");
        if (nout == 0) return HMC_OK;
        if (gathered == nullptr) return fail(HMC_INVALID, "null partials");
        combine_int_kernel<<<blocks_for(nout), 256, 0, ctx->stream>>>(static_cast<int64_t *>(out->data) + out->offset, gathered,
                                                                      ranks, nout, op == HMC_REDUCE_PROD);
        return launch_status("shard combine launch");
    });
}

HMC_API hmc_status hmc_shard_combine_extreme(hmc_context_t ctx, int32_t is_max, const hmc_tensor_desc *out_values,
                                             const hmc_tensor_desc *out_indices, const void *gathered_values,
                                             int32_t dtype, const int64_t *gathered_indices,
                                             const int64_t *index_offsets, int32_t ranks, int64_t nout) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        if (ranks < 1 || ranks > kMaxRanks || nout < 0) return fail(HMC_INVALID, "bad rank or output count");
        if (!dtype_valid(dtype)) return fail(HMC_INVALID, "unknown dtype code");
        if (out_values != nullptr) {
            hmc_status s = check_flat_output(out_values, nout, "the values");
            if (s != HMC_OK) return s;
            if (out_values->dtype != dtype) return fail(HMC_INVALID, "the values have the partials' dtype");
        }
        if (out_indices != nullptr) {
            hmc_status s = check_flat_output(out_indices, nout, "the indices");
            if (s != HMC_OK) return s;
            if (out_indices->dtype != HMC_I64) return fail(HMC_INVALID, "the indices are an I64 tensor");
            if (gathered_indices == nullptr || index_offsets == nullptr) return fail(HMC_INVALID, "indices need the ranks' indices and offsets");
        }
        if (nout == 0) return HMC_OK;
        if (gathered_values == nullptr) return fail(HMC_INVALID, "null partials");
        Offsets offsets{};
        for (int r = 0; r < ranks; ++r) offsets.v[r] = index_offsets != nullptr ? index_offsets[r] : 0;
        return dispatch_all(dtype, [&](auto t) -> hmc_status {
            using T = decltype(t);
            T *v = out_values != nullptr ? static_cast<T *>(out_values->data) + out_values->offset : nullptr;
            int64_t *i = out_indices != nullptr ? static_cast<int64_t *>(out_indices->data) + out_indices->offset : nullptr;
            const T *gv = static_cast<const T *>(gathered_values);
            if (is_max) combine_extreme_kernel<T, true><<<blocks_for(nout), 256, 0, ctx->stream>>>(v, i, gv, gathered_indices, offsets, ranks, nout);
            else combine_extreme_kernel<T, false><<<blocks_for(nout), 256, 0, ctx->stream>>>(v, i, gv, gathered_indices, offsets, ranks, nout);
            return launch_status("shard combine launch");
        });
    });
}

HMC_API hmc_status hmc_shard_combine_means(hmc_context_t ctx, double *means, const double *gathered, int32_t ranks, int64_t nout,
                                           int64_t total_count) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        if (ranks < 1 || nout < 0 || total_count < 0) return fail(HMC_INVALID, "bad rank, output or element count");
        if (nout == 0) return HMC_OK;
        if (means == nullptr || gathered == nullptr) return fail(HMC_INVALID, "null means or partials");
        combine_means_kernel<<<blocks_for(nout), 256, 0, ctx->stream>>>(means, gathered, ranks, nout, static_cast<double>(total_count));
        return launch_status("shard combine launch");
    });
}

HMC_API hmc_status hmc_var_partial(hmc_context_t ctx, double *partial, const hmc_tensor_desc *kept, const hmc_tensor_desc *red,
                                   const double *means, void *workspace, int64_t workspace_bytes) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        hmc_status s = check_desc(kept, "the kept dimensions");
        if (s != HMC_OK) return s;
        s = check_desc(red, "the reduced dimensions");
        if (s != HMC_OK) return s;
        if (!dtype_is_float(kept->dtype) || red->dtype != kept->dtype) return fail(HMC_INVALID, "hmc_var_partial takes a floating point tensor");
        ReduceArgs a{*kept, *red, make_reduce_plan(*kept, *red), nullptr, ctx->tickets};
        if (a.plan.nout == 0) return HMC_OK;
        if (partial == nullptr || means == nullptr) return fail(HMC_INVALID, "null partials or means");
        if (a.plan.nred > 0 && kept->data == nullptr) return fail(HMC_INVALID, "null data pointer");
        const int64_t need = plan_partial_bytes(a.plan);
        if (need > 0 && (workspace == nullptr || workspace_bytes < need)) {
            return fail(HMC_INVALID, "the workspace of a reduction is too small: " + std::to_string(need) + " bytes needed");
        }
        a.partials = need > 0 ? workspace : nullptr;
        return reduce_var_partial(ctx, partial, a, means);
    });
}

HMC_API hmc_status hmc_shard_combine_var(hmc_context_t ctx, const hmc_tensor_desc *out, const double *gathered, int32_t ranks,
                                         int64_t nout, int64_t total_count, double correction, int32_t take_sqrt) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        if (ranks < 1 || nout < 0 || total_count < 0) return fail(HMC_INVALID, "bad rank, output or element count");
        hmc_status s = check_flat_output(out, nout, "the output");
        if (s != HMC_OK) return s;
        if (!dtype_is_float(out->dtype)) return fail(HMC_INVALID, "the output is a floating point tensor");
        if (nout == 0) return HMC_OK;
        if (gathered == nullptr) return fail(HMC_INVALID, "null partials");
        double divisor = static_cast<double>(total_count) - correction;
        if (!(divisor > 0.0)) divisor = 0.0;
        return dispatch_float(out->dtype, [&](auto t) -> hmc_status {
            using T = decltype(t);
            VarSink<T> sink{static_cast<T *>(out->data) + out->offset, divisor, take_sqrt};
            combine_var_kernel<T><<<blocks_for(nout), 256, 0, ctx->stream>>>(sink, gathered, ranks, nout, total_count);
            return launch_status("shard combine launch");
        });
    });
}
