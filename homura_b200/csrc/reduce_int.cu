// Integer and bool sum / prod (wrapping, into I64) and all / any.
#include "reduce.cuh"

namespace hmc {

hmc_status reduce_int(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, ReduceArgs &a) {
    int64_t *o = static_cast<int64_t *>(out->data) + out->offset;
    return dispatch_all(a.kept.dtype, [&](auto t) -> hmc_status {
        using T = decltype(t);
        if constexpr (Tr<T>::kind == kFloat) {
            return fail(HMC_INVALID, "internal error: integer fold of a float tensor");
        } else {
            if (op == HMC_REDUCE_PROD) return launch_reduce(a, IntFold<T, true>{}, Int64Sink{o}, ctx->stream);
            return launch_reduce(a, IntFold<T, false>{}, Int64Sink{o}, ctx->stream);
        }
    });
}

hmc_status reduce_truth(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, ReduceArgs &a) {
    uint8_t *o = static_cast<uint8_t *>(out->data) + out->offset;
    return dispatch_all(a.kept.dtype, [&](auto t) -> hmc_status {
        using T = decltype(t);
        if (op == HMC_REDUCE_ALL) return launch_reduce(a, Truth<T, true>{}, TruthSink{o}, ctx->stream);
        return launch_reduce(a, Truth<T, false>{}, TruthSink{o}, ctx->stream);
    });
}

}  // namespace hmc
