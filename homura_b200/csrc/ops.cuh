// Internal launchers of the elementwise families. Each lives in its own translation unit so that
// the many kernel instantiations compile in parallel; the C entry points (entries.cu) validate the
// call and pick one of these. All return HMC_INVALID (with a message) for an op the dtype lacks.
#pragma once

#include "map.cuh"

namespace hmc {

hmc_status launch_unary_f16(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, const hmc_tensor_desc *src);
hmc_status launch_unary_bf16(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, const hmc_tensor_desc *src);
hmc_status launch_unary_f32(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, const hmc_tensor_desc *src);
hmc_status launch_unary_f64(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, const hmc_tensor_desc *src);
// Integer Neg/Abs/Relu/Sign, Sign of Bool, LogicalNot of every dtype.
hmc_status launch_unary_other(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, const hmc_tensor_desc *src);

// dst = cast(src) for two different dtypes, split by the source dtype.
hmc_status launch_cast_a(hmc_context_t ctx, const hmc_tensor_desc *dst, const hmc_tensor_desc *src);  // Bool..I32
hmc_status launch_cast_b(hmc_context_t ctx, const hmc_tensor_desc *dst, const hmc_tensor_desc *src);  // I64..F64
// Same-dtype copy and fill, by element size.
hmc_status launch_move(hmc_context_t ctx, const hmc_tensor_desc *dst, const hmc_tensor_desc *src);
hmc_status launch_fill(hmc_context_t ctx, const hmc_tensor_desc *dst, uint64_t bits);

// a and b: a description or a constant of the operands' dtype `dtype`.
hmc_status launch_binary_float(hmc_context_t ctx, int32_t op, int32_t dtype, const hmc_tensor_desc *out,
                               const MapOperand &a, const MapOperand &b);
hmc_status launch_binary_int(hmc_context_t ctx, int32_t op, int32_t dtype, const hmc_tensor_desc *out,
                             const MapOperand &a, const MapOperand &b);
hmc_status launch_compare(hmc_context_t ctx, int32_t op, int32_t dtype, const hmc_tensor_desc *out,
                          const MapOperand &a, const MapOperand &b);
hmc_status launch_binary_promoted(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out,
                                  const hmc_tensor_desc *a, const hmc_tensor_desc *b);
hmc_status launch_scalar(hmc_context_t ctx, int32_t mode, const hmc_tensor_desc *out, const hmc_tensor_desc *a,
                         double s);
hmc_status launch_fused(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, const hmc_tensor_desc *a,
                        const hmc_tensor_desc *b, const hmc_tensor_desc *c, double k, bool small);
hmc_status launch_select(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *cond,
                         const MapOperand &x, const MapOperand &y);

}  // namespace hmc
