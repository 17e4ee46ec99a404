// Integer Neg/Abs/Relu/Sign, Sign of Bool (identity) and LogicalNot of every dtype.
#include "functors.cuh"
#include "ops.cuh"

namespace hmc {

hmc_status launch_unary_other(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, const hmc_tensor_desc *src) {
    MapOperand in[1] = {tensor_operand(src)};
    if (op == HMC_UNARY_LOGICAL_NOT) {
        return dispatch_all(src->dtype, [&](auto t) {
            using T = decltype(t);
            return launch_map(ctx, LogicalNot<T>{}, out, in, 1);
        });
    }
    if (src->dtype == HMC_BOOL) {
        if (op == HMC_UNARY_SIGN) return launch_map(ctx, Move<uint8_t>{}, out, in, 1);
        return fail(HMC_INVALID, "this unary op is not supported for bool tensors");
    }
    return dispatch_int(src->dtype, [&](auto t) {
        using T = decltype(t);
        switch (op) {
            case HMC_UNARY_NEG: return launch_map(ctx, UnaryInt<T, HMC_UNARY_NEG>{}, out, in, 1);
            case HMC_UNARY_ABS: return launch_map(ctx, UnaryInt<T, HMC_UNARY_ABS>{}, out, in, 1);
            case HMC_UNARY_RELU: return launch_map(ctx, UnaryInt<T, HMC_UNARY_RELU>{}, out, in, 1);
            case HMC_UNARY_SIGN: return launch_map(ctx, UnaryInt<T, HMC_UNARY_SIGN>{}, out, in, 1);
        }
        return fail(HMC_INVALID, "this unary op needs a floating point tensor");
    });
}

}  // namespace hmc
