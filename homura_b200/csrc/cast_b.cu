// Casts whose source is I64, F16, BF16, F32 or F64.
#include "cast.cuh"

namespace hmc {
hmc_status launch_cast_b(hmc_context_t ctx, const hmc_tensor_desc *dst, const hmc_tensor_desc *src) {
    switch (src->dtype) {
        case HMC_I64: return launch_cast_from<int64_t>(ctx, dst, src);
        case HMC_F16: return launch_cast_from<F16>(ctx, dst, src);
        case HMC_BF16: return launch_cast_from<BF16>(ctx, dst, src);
        case HMC_F32: return launch_cast_from<float>(ctx, dst, src);
        case HMC_F64: return launch_cast_from<double>(ctx, dst, src);
    }
    return fail(HMC_INVALID, "unknown source dtype");
}
}  // namespace hmc
