// out = (unary(x) op1 b) op2 c in one pass, with the roundings of the three kernels it replaces.
//
// homura's front end evaluates an expression such as silu(x) * scale + bias as three elementwise kernels, each
// of which rounds its result to the tensor's dtype and writes it to memory for the next to read back: for
// bf16 x with an f32 bias that is 14 bytes of traffic per element where the expression needs 6 (read x, write
// the f32 result). This kernel keeps the two intermediates in registers and rounds them at the same points to
// the same dtypes (unary result to T, first binary result to T, then both operands of the second binary op
// converted to the promoted dtype as homura's cast kernels convert them), so its output carries the bits of the
// three-kernel sequence. x and b have one dtype T (F16, BF16 or F32), c any of those, the output their promotion.
#include "functors.cuh"
#include "ops.cuh"

namespace hmc {
namespace {

// x op y for op in {ADD, SUB, MUL} chosen at run time: a sum or difference is x + sign * y as one fused operation
// (the product with +-1 is exact, so the single rounding is that of x +- y), and one select picks it or the product:
// three instructions where computing all three results and selecting twice takes five.
template <class Cc>
__device__ __forceinline__ Cc chain_arith(bool is_mul, Cc sign, Cc x, Cc y) {
    Cc sum;
    if constexpr (std::is_same_v<Cc, float>) sum = __fmaf_rn(y, sign, x);
    else sum = __fma_rn(y, sign, x);
    return is_mul ? x * y : sum;
}

template <class T, class TC, class P, int UOP>
struct Chain {
    using Out = P; using A = T; using B = T; using C = TC;
    using Compute = typename Comp<P>::C;
    using Ct = typename Comp<T>::C;
    bool first_is_mul, second_is_mul;
    Ct first_sign;
    Compute second_sign;
    Chain(int first, int second)
        : first_is_mul(first == HMC_BINARY_MUL), second_is_mul(second == HMC_BINARY_MUL),
          first_sign(first == HMC_BINARY_SUB ? Ct(-1) : Ct(1)), second_sign(second == HMC_BINARY_SUB ? Compute(-1) : Compute(1)) {}
    static constexpr bool kFast = std::is_same_v<T, F16> || std::is_same_v<T, BF16>;
    // b and c are broadcasts in the expressions this is for (a scale per column, a bias per row): what is in flight
    // per thread is x, 16 bytes a vector
    static constexpr int kUnroll = 2;
    // with a transposed x (and b, c in the output's orientation) the copy engine and ldmatrix do the transposition
    static constexpr bool kTransposedFirst = true;
    __device__ __forceinline__ Compute compute(T x, T b, TC c) const {
        const T t1 = down<T>(unary_math<UOP, Ct, kFast>(up(x)));
        const T t2 = down<T>(chain_arith<Ct>(first_is_mul, first_sign, up(t1), up(b)));
        return chain_arith<Compute>(second_is_mul, second_sign, up(convert<P, T>(t2)), up(convert<P, TC>(c)));
    }
};

template <class T, class TC, class P>
hmc_status chain_unary(hmc_context_t ctx, int32_t unary_op, int first, int second, const hmc_tensor_desc *out, const MapOperand *in) {
    switch (unary_op) {
#define HMC_CASE(OP) \
    case OP: return launch_map(ctx, Chain<T, TC, P, OP>(first, second), out, in, 3);
        HMC_CASE(HMC_UNARY_RELU)
        HMC_CASE(HMC_UNARY_EXP)
        HMC_CASE(HMC_UNARY_TANH)
        HMC_CASE(HMC_UNARY_SIGMOID)
        HMC_CASE(HMC_UNARY_SILU)
        HMC_CASE(HMC_UNARY_GELU)
        HMC_CASE(HMC_UNARY_GELU_TANH)
#undef HMC_CASE
    }
    return fail(HMC_INVALID, "hmc_unary_binary_binary: the unary op is not one of relu, exp, tanh, sigmoid, silu, gelu, gelu_tanh");
}

}  // namespace
}  // namespace hmc

using namespace hmc;

HMC_API hmc_status hmc_unary_binary_binary(hmc_context_t ctx, int32_t unary_op, int32_t first_op, int32_t second_op,
                                           const hmc_tensor_desc *out, const hmc_tensor_desc *x, const hmc_tensor_desc *b,
                                           const hmc_tensor_desc *c) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        const hmc_tensor_desc *d[4] = {out, x, b, c};
        int64_t n = 0;
        hmc_status s = check_operands(d, 4, &n);
        if (s != HMC_OK) return s;
        for (int op : {first_op, second_op}) {
            if (op != HMC_BINARY_ADD && op != HMC_BINARY_SUB && op != HMC_BINARY_MUL) {
                return fail(HMC_INVALID, "hmc_unary_binary_binary: the binary ops are ADD, SUB or MUL");
            }
        }
        const int t = x->dtype, tc = c->dtype, p = out->dtype;
        if (b->dtype != t) return fail(HMC_INVALID, "hmc_unary_binary_binary: x and b must have one dtype");
        if (n == 0) return HMC_OK;
        MapOperand in[3] = {tensor_operand(x), tensor_operand(b), tensor_operand(c)};
        if (t == HMC_BF16 && tc == HMC_F32 && p == HMC_F32) return chain_unary<BF16, float, float>(ctx, unary_op, first_op, second_op, out, in);
        if (t == HMC_F16 && tc == HMC_F32 && p == HMC_F32) return chain_unary<F16, float, float>(ctx, unary_op, first_op, second_op, out, in);
        if (t == HMC_BF16 && tc == HMC_BF16 && p == HMC_BF16) return chain_unary<BF16, BF16, BF16>(ctx, unary_op, first_op, second_op, out, in);
        if (t == HMC_F16 && tc == HMC_F16 && p == HMC_F16) return chain_unary<F16, F16, F16>(ctx, unary_op, first_op, second_op, out, in);
        if (t == HMC_F32 && tc == HMC_F32 && p == HMC_F32) return chain_unary<float, float, float>(ctx, unary_op, first_op, second_op, out, in);
        return fail(HMC_INVALID, "hmc_unary_binary_binary: unsupported dtype combination");
    });
}
