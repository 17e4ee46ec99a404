// Body of cast_a.cu / cast_b.cu: dst = cast(src) for every destination dtype of some source dtypes.
#pragma once

#include "functors.cuh"
#include "ops.cuh"

namespace hmc {

template <class S>
hmc_status launch_cast_from(hmc_context_t ctx, const hmc_tensor_desc *dst, const hmc_tensor_desc *src) {
    MapOperand in[1] = {tensor_operand(src)};
    return dispatch_all(dst->dtype, [&](auto d) {
        using D = decltype(d);
        if constexpr (std::is_same_v<D, S>) {
            return launch_move(ctx, dst, src);
        } else {
            return launch_map(ctx, Cast<D, S>{}, dst, in, 1);
        }
    });
}

}  // namespace hmc
