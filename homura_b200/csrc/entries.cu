// The C entry points of the elementwise families: argument checks, then one of the launchers of
// ops.cuh. Stands in for the entry points of homura's csrc/elementwise.hip and csrc/copy.hip.
#include "ops.cuh"

using namespace hmc;

namespace {

bool is_comparison(int32_t op) { return op >= HMC_BINARY_GREATER && op <= HMC_BINARY_NOT_EQUAL; }
bool is_logical(int32_t op) { return op == HMC_BINARY_LOGICAL_AND || op == HMC_BINARY_LOGICAL_OR; }

// Shared tail of hmc_binary and hmc_binary_constant: `dtype` is the operands' dtype.
hmc_status binary_dispatch(hmc_context_t ctx, int32_t op, int32_t dtype, const hmc_tensor_desc *out,
                           const MapOperand &a, const MapOperand &b) {
    if (op < 0 || op >= HMC_BINARY_COUNT) return fail(HMC_INVALID, "unknown binary op");
    if (is_comparison(op)) {
        if (out->dtype != HMC_BOOL) return fail(HMC_INVALID, "a comparison writes a Bool tensor");
        return launch_compare(ctx, op, dtype, out, a, b);
    }
    if (is_logical(op)) {
        if (dtype != HMC_BOOL || out->dtype != HMC_BOOL) return fail(HMC_INVALID, "logical ops take and write Bool tensors");
        return launch_binary_int(ctx, op, dtype, out, a, b);
    }
    if (out->dtype != dtype) return fail(HMC_INVALID, "the output of an arithmetic op has the operands' dtype");
    if (dtype_is_float(dtype)) return launch_binary_float(ctx, op, dtype, out, a, b);
    if (op == HMC_BINARY_DIV) return fail(HMC_INVALID, "division needs floating point operands");
    return launch_binary_int(ctx, op, dtype, out, a, b);
}

}  // namespace

HMC_API hmc_status hmc_copy(hmc_context_t ctx, const hmc_tensor_desc *dst, const hmc_tensor_desc *src) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        const hmc_tensor_desc *d[2] = {dst, src};
        int64_t n = 0;
        hmc_status s = check_operands(d, 2, &n);
        if (s != HMC_OK) return s;
        if (n == 0) return HMC_OK;
        if (dst->dtype == src->dtype) return launch_move(ctx, dst, src);
        return src->dtype <= HMC_I32 ? launch_cast_a(ctx, dst, src) : launch_cast_b(ctx, dst, src);
    });
}

HMC_API hmc_status hmc_fill(hmc_context_t ctx, const hmc_tensor_desc *dst, uint64_t bits) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        const hmc_tensor_desc *d[1] = {dst};
        int64_t n = 0;
        hmc_status s = check_operands(d, 1, &n);
        if (s != HMC_OK) return s;
        if (n == 0) return HMC_OK;
        return launch_fill(ctx, dst, bits);
    });
}

HMC_API hmc_status hmc_unary(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, const hmc_tensor_desc *src) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        const hmc_tensor_desc *d[2] = {out, src};
        int64_t n = 0;
        hmc_status s = check_operands(d, 2, &n);
        if (s != HMC_OK) return s;
        if (op < 0 || op >= HMC_UNARY_COUNT) return fail(HMC_INVALID, "unknown unary op");
        if (op == HMC_UNARY_LOGICAL_NOT) {
            if (out->dtype != HMC_BOOL) return fail(HMC_INVALID, "logical_not writes a Bool tensor");
        } else if (out->dtype != src->dtype) {
            return fail(HMC_INVALID, "a unary op writes its input's dtype");
        }
        const bool plain = op == HMC_UNARY_NEG || op == HMC_UNARY_ABS || op == HMC_UNARY_RELU || op == HMC_UNARY_SIGN;
        if (op != HMC_UNARY_LOGICAL_NOT && !plain && !dtype_is_float(src->dtype)) {
            return fail(HMC_INVALID, "this unary op needs a floating point tensor");
        }
        if (op != HMC_UNARY_LOGICAL_NOT && src->dtype == HMC_BOOL && op != HMC_UNARY_SIGN) {
            return fail(HMC_INVALID, "this unary op is not supported for bool tensors");
        }
        if (n == 0) return HMC_OK;
        if (op == HMC_UNARY_LOGICAL_NOT || !dtype_is_float(src->dtype)) return launch_unary_other(ctx, op, out, src);
        switch (src->dtype) {
            case HMC_F16: return launch_unary_f16(ctx, op, out, src);
            case HMC_BF16: return launch_unary_bf16(ctx, op, out, src);
            case HMC_F32: return launch_unary_f32(ctx, op, out, src);
            default: return launch_unary_f64(ctx, op, out, src);
        }
    });
}

HMC_API hmc_status hmc_binary(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, const hmc_tensor_desc *a,
                              const hmc_tensor_desc *b) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        const hmc_tensor_desc *d[3] = {out, a, b};
        int64_t n = 0;
        hmc_status s = check_operands(d, 3, &n);
        if (s != HMC_OK) return s;
        if (a->dtype != b->dtype) return fail(HMC_INVALID, "the operands of a binary op have one dtype");
        if (n == 0) {
            // Still refuse what the dtypes don't support, as a launch would.
            if (op < 0 || op >= HMC_BINARY_COUNT) return fail(HMC_INVALID, "unknown binary op");
            return HMC_OK;
        }
        return binary_dispatch(ctx, op, a->dtype, out, tensor_operand(a), tensor_operand(b));
    });
}

HMC_API hmc_status hmc_binary_constant(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out,
                                       const hmc_tensor_desc *a, uint64_t bits, int32_t constant_first) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        const hmc_tensor_desc *d[2] = {out, a};
        int64_t n = 0;
        hmc_status s = check_operands(d, 2, &n);
        if (s != HMC_OK) return s;
        if (n == 0) {
            if (op < 0 || op >= HMC_BINARY_COUNT) return fail(HMC_INVALID, "unknown binary op");
            return HMC_OK;
        }
        MapOperand t = tensor_operand(a), c = constant_operand(bits);
        // x ** 2 (the square in a norm or a variance) is x * x, as the power kernel itself evaluates it: the product
        // kernel gives the same bits without carrying the general power's code and registers.
        // (F16, BF16 and F32, whose power is evaluated in f32; an F64 power stays with the f64 library)
        if (op == HMC_BINARY_POW && !constant_first && dtype_is_float(a->dtype) && a->dtype != HMC_F64 && out->dtype == a->dtype) {
            const uint64_t two = a->dtype == HMC_F32 ? 0x40000000ull : 0x4000ull;
            const uint64_t mask = a->dtype == HMC_F32 ? 0xFFFFFFFFull : 0xFFFFull;
            if ((bits & mask) == two) return binary_dispatch(ctx, HMC_BINARY_MUL, a->dtype, out, t, t);
        }
        return constant_first ? binary_dispatch(ctx, op, a->dtype, out, c, t) : binary_dispatch(ctx, op, a->dtype, out, t, c);
    });
}

HMC_API hmc_status hmc_binary_scalar(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out,
                                     const hmc_tensor_desc *a, double s, int32_t scalar_first) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        const hmc_tensor_desc *d[2] = {out, a};
        int64_t n = 0;
        hmc_status st = check_operands(d, 2, &n);
        if (st != HMC_OK) return st;
        if (op != HMC_BINARY_MUL && op != HMC_BINARY_DIV) return fail(HMC_INVALID, "hmc_binary_scalar takes MUL or DIV");
        if (!dtype_is_float(a->dtype) || out->dtype != a->dtype) {
            return fail(HMC_INVALID, "hmc_binary_scalar takes a floating point tensor and writes its dtype");
        }
        if (n == 0) return HMC_OK;
        int mode = op == HMC_BINARY_MUL ? 0 : (scalar_first ? 2 : 1);
        return launch_scalar(ctx, mode, out, a, s);
    });
}

HMC_API hmc_status hmc_fused(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out, const hmc_tensor_desc *a,
                             const hmc_tensor_desc *b, const hmc_tensor_desc *c, double coefficient, int32_t small) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        const bool three = op == HMC_FUSED_ADDCMUL || op == HMC_FUSED_ADDCDIV;
        if (op < HMC_FUSED_SCALED_ADD || op > HMC_FUSED_ADDCDIV) return fail(HMC_INVALID, "unknown fused op");
        if (three && c == nullptr) return fail(HMC_INVALID, "addcmul and addcdiv have three operands");
        if (!three && c != nullptr) return fail(HMC_INVALID, "scaled add and lerp have two operands");
        const hmc_tensor_desc *d[4] = {out, a, b, c};
        int64_t n = 0;
        hmc_status s = check_operands(d, three ? 4 : 3, &n);
        if (s != HMC_OK) return s;
        if (!dtype_is_float(out->dtype) || a->dtype != out->dtype || b->dtype != out->dtype ||
            (three && c->dtype != out->dtype)) {
            return fail(HMC_INVALID, "the fused steps take floating point operands of one dtype");
        }
        if (n == 0) return HMC_OK;
        return launch_fused(ctx, op, out, a, b, c, coefficient, small != 0);
    });
}

HMC_API hmc_status hmc_where(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *cond,
                             const hmc_tensor_desc *x, const hmc_tensor_desc *y) {
    return guarded([&]() -> hmc_status {
        if (x == nullptr || y == nullptr) return fail(HMC_INVALID, "null description of a branch");
        return hmc_where_constant(ctx, out, cond, x, 0, y, 0);
    });
}

HMC_API hmc_status hmc_where_constant(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *cond,
                                      const hmc_tensor_desc *x, uint64_t x_bits, const hmc_tensor_desc *y,
                                      uint64_t y_bits) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        if (out == nullptr || cond == nullptr) return fail(HMC_INVALID, "null description");
        const hmc_tensor_desc *d[4] = {out, cond, x, y};
        int64_t n = 0;
        hmc_status s = check_operands(d, 4, &n);
        if (s != HMC_OK) return s;
        if (cond->dtype != HMC_BOOL) return fail(HMC_INVALID, "the condition of where is a Bool tensor");
        if ((x != nullptr && x->dtype != out->dtype) || (y != nullptr && y->dtype != out->dtype)) {
            return fail(HMC_INVALID, "the branches of where have the output's dtype");
        }
        if (n == 0) return HMC_OK;
        MapOperand xo = x != nullptr ? tensor_operand(x) : constant_operand(x_bits);
        MapOperand yo = y != nullptr ? tensor_operand(y) : constant_operand(y_bits);
        return launch_select(ctx, out, cond, xo, yo);
    });
}

HMC_API hmc_status hmc_binary_promoted(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out,
                                       const hmc_tensor_desc *a, const hmc_tensor_desc *b) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        const hmc_tensor_desc *d[3] = {out, a, b};
        int64_t n = 0;
        hmc_status s = check_operands(d, 3, &n);
        if (s != HMC_OK) return s;
        if (a->dtype == b->dtype) {
            if (n == 0) return HMC_OK;
            return binary_dispatch(ctx, op, a->dtype, out, tensor_operand(a), tensor_operand(b));
        }
        if (n == 0) return HMC_OK;
        return launch_binary_promoted(ctx, op, out, a, b);
    });
}
