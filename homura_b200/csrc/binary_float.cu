// Float binary arithmetic, the scalar forms, the optimizers' fused steps and the promoting add.
#include "functors.cuh"
#include "ops.cuh"

namespace hmc {

hmc_status launch_binary_float(hmc_context_t ctx, int32_t op, int32_t dtype, const hmc_tensor_desc *out,
                               const MapOperand &a, const MapOperand &b) {
    MapOperand in[2] = {a, b};
    return dispatch_float(dtype, [&](auto t) {
        using T = decltype(t);
        switch (op) {
#define HMC_CASE(OP) \
    case OP: return launch_map(ctx, BinaryFloat<T, OP>{}, out, in, 2);
            HMC_CASE(HMC_BINARY_ADD)
            HMC_CASE(HMC_BINARY_SUB)
            HMC_CASE(HMC_BINARY_MUL)
            HMC_CASE(HMC_BINARY_DIV)
            HMC_CASE(HMC_BINARY_POW)
            HMC_CASE(HMC_BINARY_MAXIMUM)
            HMC_CASE(HMC_BINARY_MINIMUM)
#undef HMC_CASE
        }
        return fail(HMC_INVALID, "this binary op is not an arithmetic op of floating point tensors");
    });
}

hmc_status launch_scalar(hmc_context_t ctx, int32_t mode, const hmc_tensor_desc *out, const hmc_tensor_desc *a,
                         double s) {
    MapOperand in[1] = {tensor_operand(a)};
    return dispatch_float(a->dtype, [&](auto t) {
        using T = decltype(t);
        using C = typename Comp<T>::C;
        const C sc = static_cast<C>(s);
        switch (mode) {
            case 0: return launch_map(ctx, ScalarOp<T, 0>{sc}, out, in, 1);
            case 1: return launch_map(ctx, ScalarOp<T, 1>{sc}, out, in, 1);
            default: return launch_map(ctx, ScalarOp<T, 2>{sc}, out, in, 1);
        }
    });
}

hmc_status launch_fused(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, const hmc_tensor_desc *a,
                        const hmc_tensor_desc *b, const hmc_tensor_desc *c, double k, bool small) {
    return dispatch_float(out->dtype, [&](auto t) {
        using T = decltype(t);
        using C = typename Comp<T>::C;
        const C kc = static_cast<C>(k);
        MapOperand in[3] = {tensor_operand(a), tensor_operand(b), tensor_operand(c)};
        switch (op) {
            case HMC_FUSED_SCALED_ADD: return launch_map(ctx, Fused2<T, HMC_FUSED_SCALED_ADD>{kc, small}, out, in, 2);
            case HMC_FUSED_LERP: return launch_map(ctx, Fused2<T, HMC_FUSED_LERP>{kc, small}, out, in, 2);
            case HMC_FUSED_ADDCMUL: return launch_map(ctx, Fused3<T, HMC_FUSED_ADDCMUL>{kc}, out, in, 3);
            case HMC_FUSED_ADDCDIV: return launch_map(ctx, Fused3<T, HMC_FUSED_ADDCDIV>{kc}, out, in, 3);
        }
        return fail(HMC_INVALID, "unknown fused op");
    });
}

namespace {
template <class P, class TA, class TB>
hmc_status promoted(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, const MapOperand *in) {
    switch (op) {
        case HMC_BINARY_ADD: return launch_map(ctx, BinaryPromoted<P, TA, TB, HMC_BINARY_ADD>{}, out, in, 2);
        case HMC_BINARY_SUB: return launch_map(ctx, BinaryPromoted<P, TA, TB, HMC_BINARY_SUB>{}, out, in, 2);
        case HMC_BINARY_MUL: return launch_map(ctx, BinaryPromoted<P, TA, TB, HMC_BINARY_MUL>{}, out, in, 2);
    }
    return fail(HMC_INVALID, "hmc_binary_promoted supports ADD, SUB and MUL");
}
}  // namespace

hmc_status launch_binary_promoted(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out,
                                  const hmc_tensor_desc *a, const hmc_tensor_desc *b) {
    MapOperand in[2] = {tensor_operand(a), tensor_operand(b)};
    const int da = a->dtype, db = b->dtype, dp = out->dtype;
    if (dp == HMC_F32) {
        if (da == HMC_BF16 && db == HMC_F32) return promoted<float, BF16, float>(ctx, op, out, in);
        if (da == HMC_F32 && db == HMC_BF16) return promoted<float, float, BF16>(ctx, op, out, in);
        if (da == HMC_F16 && db == HMC_F32) return promoted<float, F16, float>(ctx, op, out, in);
        if (da == HMC_F32 && db == HMC_F16) return promoted<float, float, F16>(ctx, op, out, in);
        if (da == HMC_F16 && db == HMC_BF16) return promoted<float, F16, BF16>(ctx, op, out, in);
        if (da == HMC_BF16 && db == HMC_F16) return promoted<float, BF16, F16>(ctx, op, out, in);
    }
    return fail(HMC_INVALID, "hmc_binary_promoted: unsupported dtype combination");
}

}  // namespace hmc
