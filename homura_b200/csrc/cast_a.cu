// Casts whose source is Bool, U8, I8, I16 or I32.
#include "cast.cuh"

namespace hmc {
hmc_status launch_cast_a(hmc_context_t ctx, const hmc_tensor_desc *dst, const hmc_tensor_desc *src) {
    switch (src->dtype) {
        case HMC_BOOL: return launch_cast_from<Bool>(ctx, dst, src);
        case HMC_U8: return launch_cast_from<uint8_t>(ctx, dst, src);
        case HMC_I8: return launch_cast_from<int8_t>(ctx, dst, src);
        case HMC_I16: return launch_cast_from<int16_t>(ctx, dst, src);
        case HMC_I32: return launch_cast_from<int32_t>(ctx, dst, src);
    }
    return fail(HMC_INVALID, "unknown source dtype");
}
}  // namespace hmc
