// Integer binary arithmetic (wrapping) and the Bool forms of Add/Mul/Maximum/Minimum and the
// logical ops.
#include "functors.cuh"
#include "ops.cuh"

namespace hmc {

hmc_status launch_binary_int(hmc_context_t ctx, int32_t op, int32_t dtype, const hmc_tensor_desc *out,
                             const MapOperand &a, const MapOperand &b) {
    MapOperand in[2] = {a, b};
    if (dtype == HMC_BOOL) {
        switch (op) {
            case HMC_BINARY_ADD: case HMC_BINARY_MAXIMUM: case HMC_BINARY_LOGICAL_OR:
                return launch_map(ctx, BoolLogic<false>{}, out, in, 2);
            case HMC_BINARY_MUL: case HMC_BINARY_MINIMUM: case HMC_BINARY_LOGICAL_AND:
                return launch_map(ctx, BoolLogic<true>{}, out, in, 2);
        }
        return fail(HMC_INVALID, "this binary op is not supported for bool tensors");
    }
    return dispatch_int(dtype, [&](auto t) {
        using T = decltype(t);
        switch (op) {
#define HMC_CASE(OP) \
    case OP: return launch_map(ctx, BinaryInt<T, OP>{}, out, in, 2);
            HMC_CASE(HMC_BINARY_ADD)
            HMC_CASE(HMC_BINARY_SUB)
            HMC_CASE(HMC_BINARY_MUL)
            HMC_CASE(HMC_BINARY_POW)
            HMC_CASE(HMC_BINARY_MAXIMUM)
            HMC_CASE(HMC_BINARY_MINIMUM)
#undef HMC_CASE
        }
        return fail(HMC_INVALID, "this binary op is not supported for integer tensors");
    });
}

}  // namespace hmc
