// Same-dtype strided copy, fill, and where: byte movers instantiated per element size.
#include "functors.cuh"
#include "ops.cuh"

namespace hmc {

template <class F> static hmc_status by_size(int dtype, F &&f) {
    switch (element_size(dtype)) {
        case 1: return f(uint8_t{});
        case 2: return f(uint16_t{});
        case 4: return f(uint32_t{});
        default: return f(uint64_t{});
    }
}

hmc_status launch_move(hmc_context_t ctx, const hmc_tensor_desc *dst, const hmc_tensor_desc *src) {
    MapOperand in[1] = {tensor_operand(src)};
    return by_size(dst->dtype, [&](auto w) { return launch_map(ctx, Move<decltype(w)>{}, dst, in, 1); });
}

hmc_status launch_fill(hmc_context_t ctx, const hmc_tensor_desc *dst, uint64_t bits) {
    return by_size(dst->dtype, [&](auto w) {
        using W = decltype(w);
        return launch_map(ctx, Fill<W>{static_cast<W>(bits)}, dst, nullptr, 0);
    });
}

hmc_status launch_select(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *cond,
                         const MapOperand &x, const MapOperand &y) {
    MapOperand in[3] = {tensor_operand(cond), x, y};
    return by_size(out->dtype, [&](auto w) { return launch_map(ctx, Select<decltype(w)>{}, out, in, 3); });
}

}  // namespace hmc
