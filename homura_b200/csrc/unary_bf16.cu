// Float unary kernels of one dtype (see unary_float.cuh).
#include "unary_float.cuh"

namespace hmc {
hmc_status launch_unary_bf16(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, const hmc_tensor_desc *src) {
    return launch_unary_float<BF16>(ctx, op, out, src);
}
}  // namespace hmc
