// Plans and C entry points of the reductions. Stands in for the entry points of homura's
// csrc/reduce.hip (hmr_reduce, hmr_var, hmr_arg_reduce, hmr_reduce_workspace).
#include "map.cuh"
#include "reduce.cuh"

#include <algorithm>

namespace hmc {

ReducePlan make_reduce_plan(const hmc_tensor_desc &kept, const hmc_tensor_desc &red) {
    ReducePlan p{};
    const int es = element_size(kept.dtype);
    p.vec = 32 / es;
    p.vc = 16 / es > 8 ? 8 : 16 / es;
    p.nout = desc_count(kept);
    p.nred = desc_count(red);
    p.row = red.ndim > 0 ? red.sizes[red.ndim - 1] : 1;
    p.step = red.ndim > 0 ? red.strides[red.ndim - 1] : 1;
    if (p.row <= 1) {
        // Nothing, or single elements, to walk along: any step is as good as 1.
        if (p.row == 0) p.row = 1;
        p.step = 1;
    }
    p.kind = 0;
    p.group = 1;
    p.splits = 1;
    p.chunk = p.nred;
    if (p.nout == 0 || p.nred == 0) return p;
    const bool rows_contiguous = p.step == 1 && p.row >= 32;
    const bool outputs_adjacent = kept.ndim > 0 && kept.strides[kept.ndim - 1] == 1 && kept.sizes[kept.ndim - 1] >= 32;
    if (outputs_adjacent && !rows_contiguous) {
        p.kind = 1;
        p.ncols = kept.sizes[kept.ndim - 1];
        p.kouter = p.nout / p.ncols;
        p.xtiles = ceil_div(p.ncols, 32 * p.vc);
        const int64_t blocks = p.kouter * p.xtiles;
        if (blocks < kTargetColumnBlocks) {
            // chunks until there are enough blocks, as long as a block still reads a worthwhile amount
            const int64_t want = ceil_div(kTargetColumnBlocks, blocks);
            const int64_t strip_bytes = 32 * static_cast<int64_t>(p.vc) * es;
            const int64_t worth = std::min(p.nred / 64, p.nred * strip_bytes / kColumnBlockBytes);
            p.splits = std::max<int64_t>(1, std::min({want, worth, kMaxSplits}));
        }
        p.chunk = ceil_div(p.nred, p.splits);
        p.splits = ceil_div(p.nred, p.chunk);
        return p;
    }
    // A block of 256 lanes per output for long rows, a warp for short ones; and a warp also for long rows when
    // there are enough outputs to give every warp of the GPU one (a lane's set-up and the group's combination
    // are then paid once per 1/32 of a row instead of once per 1/256).
    p.group = p.nred >= 1024 ? 256 : (p.nred >= 64 ? 32 : 1);
    if (p.group == 256 && p.nout >= kWarpRowOutputs && p.nred <= kWarpRowLength) p.group = 32;
    const int64_t lanes = p.nout * p.group;
    if (lanes < kTargetLanes) {
        const int64_t want = ceil_div(kTargetLanes, lanes);
        const int64_t worth = p.nred / (static_cast<int64_t>(p.group) * p.vec * 16);
        p.splits = std::max<int64_t>(1, std::min({want, worth, kMaxSplits}));
    }
    p.simple = p.splits == 1 && p.group > 1 && red.ndim == 1 && p.step == 1 && p.nred % (32 / es) == 0 && p.nred < (int64_t{1} << 31);
    if (p.splits > 1) {
        // Whole pieces per lane and chunk, so that only a range's two ends can be ragged.
        const int64_t unit = static_cast<int64_t>(p.group) * p.vec;
        p.chunk = ceil_div(ceil_div(p.nred, p.splits), unit) * unit;
        p.splits = ceil_div(p.nred, p.chunk);
    }
    return p;
}

hmc_status check_reduction(const hmc_tensor_desc *kept, const hmc_tensor_desc *red) {
    hmc_status s = check_desc(kept, "the kept dimensions");
    if (s != HMC_OK) return s;
    s = check_desc(red, "the reduced dimensions");
    if (s != HMC_OK) return s;
    if (red->dtype != kept->dtype) return fail(HMC_INVALID, "kept and reduced descriptions differ in dtype");
    int64_t n = 1;
    for (int k = 0; k < kept->ndim; ++k) {
        if (__builtin_mul_overflow(n, std::max<int64_t>(kept->sizes[k], 1), &n)) return fail(HMC_INVALID, "too many outputs");
    }
    n = 1;
    for (int k = 0; k < red->ndim; ++k) {
        if (__builtin_mul_overflow(n, std::max<int64_t>(red->sizes[k], 1), &n)) return fail(HMC_INVALID, "too many reduced elements");
    }
    return HMC_OK;
}

// Checks a contiguous output description against the kept sizes; returns its first element.
hmc_status check_output(const hmc_tensor_desc *out, const hmc_tensor_desc *kept, const char *what, int64_t nout) {
    hmc_status s = check_desc(out, what);
    if (s != HMC_OK) return s;
    if (desc_count(*out) != nout) return fail(HMC_INVALID, std::string(what) + " does not have one element per kept position");
    int64_t expect = 1;
    for (int k = out->ndim - 1; k >= 0; --k) {
        if (out->sizes[k] != 1 && out->strides[k] != expect) return fail(HMC_INVALID, std::string(what) + " is not contiguous");
        expect *= out->sizes[k];
    }
    if (nout > 0 && out->data == nullptr) return fail(HMC_INVALID, "null data pointer");
    return HMC_OK;
}

namespace {

// The 16-byte aligned size of the f64 means var keeps between its two passes when it cannot do
// both in one kernel.
int64_t means_bytes(const ReducePlan &p, bool var) {
    const bool one_kernel = p.kind == 0 && p.splits == 1;
    return var && !one_kernel ? (p.nout * 8 + 15) / 16 * 16 : 0;
}

hmc_status take_workspace(ReduceArgs &a, bool var, void *workspace, int64_t bytes, double **means) {
    const int64_t mb = means_bytes(a.plan, var);
    const int64_t need = mb + plan_partial_bytes(a.plan);
    if (need > 0 && (workspace == nullptr || bytes < need)) {
        return fail(HMC_INVALID, "the workspace of a reduction is too small: " + std::to_string(need) + " bytes needed");
    }
    if (need > 0 && (reinterpret_cast<uintptr_t>(workspace) & 15) != 0) {
        return fail(HMC_INVALID, "the workspace of a reduction must be 16-byte aligned");
    }
    if (means != nullptr) *means = mb > 0 ? static_cast<double *>(workspace) : nullptr;
    a.partials = plan_partial_bytes(a.plan) > 0 ? static_cast<char *>(workspace) + mb : nullptr;
    return HMC_OK;
}

void *first_element(const hmc_tensor_desc *d) {
    return static_cast<char *>(d->data) + d->offset * element_size(d->dtype);
}

}  // namespace
}  // namespace hmc

using namespace hmc;

HMC_API hmc_status hmc_reduce_workspace(const hmc_tensor_desc *kept, const hmc_tensor_desc *red, int32_t var,
                                        int64_t *bytes) {
    return guarded([&]() -> hmc_status {
        if (bytes == nullptr) return fail(HMC_INVALID, "null output");
        hmc_status s = check_reduction(kept, red);
        if (s != HMC_OK) return s;
        ReducePlan p = make_reduce_plan(*kept, *red);
        *bytes = means_bytes(p, var != 0) + plan_partial_bytes(p);
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_test_reduce_plan(const hmc_tensor_desc *kept, const hmc_tensor_desc *red, int64_t *kind,
                                        int64_t *splits, int64_t *chunk) {
    return guarded([&]() -> hmc_status {
        if (kind == nullptr || splits == nullptr || chunk == nullptr) return fail(HMC_INVALID, "null output");
        hmc_status s = check_reduction(kept, red);
        if (s != HMC_OK) return s;
        ReducePlan p = make_reduce_plan(*kept, *red);
        // kind: 1 for columns, else the lanes per output (1, 32, 256) negated... kept simple:
        // 0/32/256-lane groups are reported as 1000 + lanes.
        *kind = p.kind == 1 ? 1 : 1000 + p.group;
        *splits = p.splits;
        *chunk = p.chunk;
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_reduce(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, const hmc_tensor_desc *kept,
                              const hmc_tensor_desc *red, void *workspace, int64_t workspace_bytes) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        hmc_status s = check_reduction(kept, red);
        if (s != HMC_OK) return s;
        if (op < HMC_REDUCE_SUM || op > HMC_REDUCE_ANY) return fail(HMC_INVALID, "unknown reduction");
        ReduceArgs a{*kept, *red, make_reduce_plan(*kept, *red), nullptr, ctx->tickets};
        s = check_output(out, kept, "the output", a.plan.nout);
        if (s != HMC_OK) return s;
        const int dt = kept->dtype;
        const bool is_float = dtype_is_float(dt);
        int expect;
        switch (op) {
            case HMC_REDUCE_SUM: case HMC_REDUCE_PROD: expect = is_float ? dt : HMC_I64; break;
            case HMC_REDUCE_MEAN:
                if (!is_float) return fail(HMC_INVALID, "mean needs a floating point tensor");
                expect = dt;
                break;
            case HMC_REDUCE_MAX: case HMC_REDUCE_MIN: expect = dt; break;
            default: expect = dt == HMC_U8 ? HMC_U8 : HMC_BOOL; break;
        }
        if (out->dtype != expect) return fail(HMC_INVALID, "the output of the reduction has the wrong dtype");
        if ((op == HMC_REDUCE_MAX || op == HMC_REDUCE_MIN) && a.plan.nred == 0 && a.plan.nout > 0) {
            return fail(HMC_INVALID, "max and min need a nonempty reduction");
        }
        if (a.plan.nout == 0) return HMC_OK;
        if (a.plan.nout > 0 && a.plan.nred > 0 && kept->data == nullptr) return fail(HMC_INVALID, "null data pointer");
        s = take_workspace(a, false, workspace, workspace_bytes, nullptr);
        if (s != HMC_OK) return s;
        switch (op) {
            case HMC_REDUCE_SUM: case HMC_REDUCE_PROD:
                return is_float ? reduce_float(ctx, op, out, a) : reduce_int(ctx, op, out, a);
            case HMC_REDUCE_MEAN: return reduce_float(ctx, op, out, a);
            case HMC_REDUCE_MAX: case HMC_REDUCE_MIN:
                return reduce_extreme(ctx, op == HMC_REDUCE_MAX, first_element(out), nullptr, a);
            default: return reduce_truth(ctx, op, out, a);
        }
    });
}

HMC_API hmc_status hmc_var(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *kept,
                           const hmc_tensor_desc *red, double correction, int32_t take_sqrt, void *workspace,
                           int64_t workspace_bytes) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        hmc_status s = check_reduction(kept, red);
        if (s != HMC_OK) return s;
        if (!dtype_is_float(kept->dtype)) return fail(HMC_INVALID, "var and std need a floating point tensor");
        ReduceArgs a{*kept, *red, make_reduce_plan(*kept, *red), nullptr, ctx->tickets};
        s = check_output(out, kept, "the output", a.plan.nout);
        if (s != HMC_OK) return s;
        if (out->dtype != kept->dtype) return fail(HMC_INVALID, "the output of var has the source's dtype");
        if (a.plan.nout == 0) return HMC_OK;
        if (a.plan.nred > 0 && kept->data == nullptr) return fail(HMC_INVALID, "null data pointer");
        double *means = nullptr;
        s = take_workspace(a, true, workspace, workspace_bytes, &means);
        if (s != HMC_OK) return s;
        return reduce_var(ctx, out, a, correction, take_sqrt, means);
    });
}

HMC_API hmc_status hmc_arg_reduce(hmc_context_t ctx, const hmc_tensor_desc *values, const hmc_tensor_desc *indices,
                                  const hmc_tensor_desc *kept, const hmc_tensor_desc *red, int32_t is_max,
                                  void *workspace, int64_t workspace_bytes) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        hmc_status s = check_reduction(kept, red);
        if (s != HMC_OK) return s;
        if (red->ndim > 1) return fail(HMC_INVALID, "an arg reduction folds one dimension");
        ReduceArgs a{*kept, *red, make_reduce_plan(*kept, *red), nullptr, ctx->tickets};
        s = check_output(indices, kept, "the indices", a.plan.nout);
        if (s != HMC_OK) return s;
        if (indices->dtype != HMC_I64) return fail(HMC_INVALID, "the indices are an I64 tensor");
        if (values != nullptr) {
            s = check_output(values, kept, "the values", a.plan.nout);
            if (s != HMC_OK) return s;
            if (values->dtype != kept->dtype) return fail(HMC_INVALID, "the values have the source's dtype");
        }
        if (a.plan.nout == 0) return HMC_OK;
        if (a.plan.nred == 0) return fail(HMC_INVALID, "cannot compute the arg reduction of an empty dimension");
        if (kept->data == nullptr) return fail(HMC_INVALID, "null data pointer");
        s = take_workspace(a, false, workspace, workspace_bytes, nullptr);
        if (s != HMC_OK) return s;
        return reduce_extreme(ctx, is_max != 0, values != nullptr ? first_element(values) : nullptr,
                              static_cast<int64_t *>(first_element(indices)), a);
    });
}
