// The six comparisons of every dtype, writing Bool.
#include "functors.cuh"
#include "ops.cuh"

namespace hmc {

hmc_status launch_compare(hmc_context_t ctx, int32_t op, int32_t dtype, const hmc_tensor_desc *out,
                          const MapOperand &a, const MapOperand &b) {
    MapOperand in[2] = {a, b};
    return dispatch_all(dtype, [&](auto t) {
        using T = decltype(t);
        switch (op) {
#define HMC_CASE(OP) \
    case OP: return launch_map(ctx, Compare<T, OP>{}, out, in, 2);
            HMC_CASE(HMC_BINARY_GREATER)
            HMC_CASE(HMC_BINARY_GREATER_EQUAL)
            HMC_CASE(HMC_BINARY_LESS)
            HMC_CASE(HMC_BINARY_LESS_EQUAL)
            HMC_CASE(HMC_BINARY_EQUAL)
            HMC_CASE(HMC_BINARY_NOT_EQUAL)
#undef HMC_CASE
        }
        return fail(HMC_INVALID, "not a comparison");
    });
}

}  // namespace hmc
