// max / min and argmax / argmin of every dtype.
#include "reduce.cuh"

namespace hmc {

hmc_status reduce_extreme(hmc_context_t ctx, bool is_max, void *values, int64_t *indices, ReduceArgs &a) {
    return dispatch_all(a.kept.dtype, [&](auto t) -> hmc_status {
        using T = decltype(t);
        ExtremeSink<T> sink{static_cast<T *>(values), indices};
        if (is_max) return launch_reduce(a, Extreme<T, true>{}, sink, ctx->stream);
        return launch_reduce(a, Extreme<T, false>{}, sink, ctx->stream);
    });
}

}  // namespace hmc
