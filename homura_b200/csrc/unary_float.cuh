// Body of the four unary_<dtype>.cu files: the float unary ops of one dtype.
#pragma once

#include "functors.cuh"
#include "ops.cuh"

namespace hmc {

template <class T>
hmc_status launch_unary_float(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, const hmc_tensor_desc *src) {
    MapOperand in[1] = {tensor_operand(src)};
    switch (op) {
#define HMC_CASE(OP) \
    case OP: return launch_map(ctx, UnaryFloat<T, OP>{}, out, in, 1);
        HMC_CASE(HMC_UNARY_NEG)
        HMC_CASE(HMC_UNARY_ABS)
        HMC_CASE(HMC_UNARY_SIGN)
        HMC_CASE(HMC_UNARY_RELU)
        HMC_CASE(HMC_UNARY_EXP)
        HMC_CASE(HMC_UNARY_LOG)
        HMC_CASE(HMC_UNARY_SQRT)
        HMC_CASE(HMC_UNARY_RSQRT)
        HMC_CASE(HMC_UNARY_RECIPROCAL)
        HMC_CASE(HMC_UNARY_SIN)
        HMC_CASE(HMC_UNARY_COS)
        HMC_CASE(HMC_UNARY_ERF)
        HMC_CASE(HMC_UNARY_TANH)
        HMC_CASE(HMC_UNARY_SIGMOID)
        HMC_CASE(HMC_UNARY_LOG_SIGMOID)
        HMC_CASE(HMC_UNARY_SILU)
        HMC_CASE(HMC_UNARY_GELU)
        HMC_CASE(HMC_UNARY_GELU_TANH)
#undef HMC_CASE
    }
    return fail(HMC_INVALID, "unknown unary op");
}

}  // namespace hmc
