// addr (the rank-one update out = beta * input + alpha * v1 v2^T) and exclusive_cumprod: the remaining position-free
// neighbours of the elementwise and reduction kernels. Stand in for hmr_addr (csrc/elementwise.hip) and
// hmr_exclusive_cumprod (csrc/reduce.hip); semantics of cpu::addr (src/backend/cpu/linalg.rs:227-410) and
// cpu::exclusive_cumprod (src/backend/cpu/reduce.rs:228-329).
//
// addr is an elementwise map over [n, m] whose first two inputs are broadcast views of the vectors (v1 constant
// along a row, v2 along a column), so it runs on the elementwise engine with its own functors: every step of the
// CPU kernel is rounded to the dtype in the same place. exclusive_cumprod multiplies along a line one element at a
// time in the accumulation type, as the CPU does (a product in another order would round differently): one thread
// per line, lines side by side in a warp.
#include "functors.cuh"
#include "ops.cuh"
#include "reduce.cuh"

namespace hmc {
namespace {

// FloatOuter (src/backend/cpu/linalg.rs:262-310). MODE 0: beta == 0 (no input), 1: beta == 1, 2: any other beta.
template <class T, int MODE>
struct AddrFloat {
    using Out = T; using A = T; using B = T; using C = std::conditional_t<MODE == 0, Unused, T>;
    using Cm = typename Comp<T>::C;
    Cm alpha, beta;
    bool scale_row;
    __device__ __forceinline__ T product(T x, T y) const {
        const T a = scale_row ? down<T>(up(x) * alpha) : x;
        return down<T>(up(a) * up(y));
    }
    __device__ __forceinline__ T operator()(T x, T y) const { return product(x, y); }
    __device__ __forceinline__ T operator()(T x, T y, T c) const {
        const T p = product(x, y);
        const T cc = MODE == 1 ? c : down<T>(up(c) * beta);
        return down<T>(up(cc) + up(p));
    }
};

// IntOuter (src/backend/cpu/linalg.rs:312-334): wrapping i64 arithmetic, truncated to the dtype once.
template <class T, bool INPUT>
struct AddrInt {
    using Out = T; using A = T; using B = T; using C = std::conditional_t<INPUT, T, Unused>;
    int64_t alpha, beta;
    __device__ __forceinline__ uint64_t product(T x, T y) const {
        return static_cast<uint64_t>(to_i64(x)) * static_cast<uint64_t>(to_i64(y)) * static_cast<uint64_t>(alpha);
    }
    __device__ __forceinline__ T operator()(T x, T y) const { return wrap_int<T>(static_cast<int64_t>(product(x, y))); }
    __device__ __forceinline__ T operator()(T x, T y, T c) const {
        return wrap_int<T>(static_cast<int64_t>(static_cast<uint64_t>(to_i64(c)) * static_cast<uint64_t>(beta) + product(x, y)));
    }
};

// BoolOuter (src/backend/cpu/linalg.rs:336-363).
template <bool INPUT>
struct AddrBool {
    using Out = Bool; using A = Bool; using B = Bool; using C = std::conditional_t<INPUT, Bool, Unused>;
    bool alpha;
    __device__ __forceinline__ Bool operator()(Bool x, Bool y) const { return Bool{static_cast<uint8_t>(x.b && alpha && y.b)}; }
    __device__ __forceinline__ Bool operator()(Bool x, Bool y, Bool c) const {
        return Bool{static_cast<uint8_t>(c.b || (x.b && alpha && y.b))};
    }
};

template <class T> struct Accumulator { using type = double; };
template <> struct Accumulator<F16> { using type = float; };
template <> struct Accumulator<BF16> { using type = float; };

struct ScanArgs {
    hmc_tensor_desc out_lines;
    hmc_tensor_desc src_lines;
    int64_t nlines, n, so, si;
    int32_t reverse;
};

template <class T>
__global__ void __launch_bounds__(256) exclusive_cumprod_kernel(const __grid_constant__ ScanArgs a) {
    using Acc = typename Accumulator<T>::type;
    const T *src = static_cast<const T *>(a.src_lines.data);
    T *dst = static_cast<T *>(a.out_lines.data);
    for (int64_t line = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; line < a.nlines;
         line += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const T *ps = src + a.src_lines.offset + decompose(a.src_lines, line, a.src_lines.ndim);
        T *po = dst + a.out_lines.offset + decompose(a.out_lines, line, a.out_lines.ndim);
        Acc acc = 1;
        for (int64_t k = 0; k < a.n; ++k) {
            const int64_t at = a.reverse ? a.n - 1 - k : k;
            // the source element is read before the output is written: in place is allowed
            const T x = ps[at * a.si];
            if constexpr (std::is_same_v<Acc, float>) {
                po[at * a.so] = down<T>(acc);
                acc = acc * up(x);
            } else {
                po[at * a.so] = from_f64<T>(acc);
                acc = acc * to_f64(x);
            }
        }
    }
}

}  // namespace
}  // namespace hmc

using namespace hmc;

HMC_API hmc_status hmc_addr(hmc_context_t ctx, const hmc_tensor_desc *out, const hmc_tensor_desc *v1, const hmc_tensor_desc *v2,
                            const hmc_tensor_desc *input, double alpha, double beta, int64_t alpha_int, int64_t beta_int) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        const hmc_tensor_desc *d[4] = {out, v1, v2, input};
        int64_t n = 0;
        hmc_status s = check_operands(d, input != nullptr ? 4 : 3, &n);
        if (s != HMC_OK) return s;
        if (v1 == nullptr || v2 == nullptr) return fail(HMC_INVALID, "null description of a vector");
        if (v1->dtype != out->dtype || v2->dtype != out->dtype || (input != nullptr && input->dtype != out->dtype)) {
            return fail(HMC_INVALID, "addr takes operands of one dtype");
        }
        if (n == 0) return HMC_OK;
        const int dt = out->dtype;
        MapOperand in[3] = {tensor_operand(v1), tensor_operand(v2), tensor_operand(input)};
        if (dtype_is_float(dt)) {
            const bool reads = beta != 0.0;
            if (reads && input == nullptr) return fail(HMC_INVALID, "addr with a nonzero beta needs its input");
            return dispatch_float(dt, [&](auto t) -> hmc_status {
                using T = decltype(t);
                using Cm = typename Comp<T>::C;
                const Cm a = static_cast<Cm>(alpha), b = static_cast<Cm>(beta);
                const bool scale_row = !(a == Cm{1});
                if (!reads) return launch_map(ctx, AddrFloat<T, 0>{a, b, scale_row}, out, in, 2);
                if (b == Cm{1}) return launch_map(ctx, AddrFloat<T, 1>{a, b, scale_row}, out, in, 3);
                return launch_map(ctx, AddrFloat<T, 2>{a, b, scale_row}, out, in, 3);
            });
        }
        const bool reads = beta_int != 0;
        if (reads && input == nullptr) return fail(HMC_INVALID, "addr with a nonzero beta needs its input");
        if (dt == HMC_BOOL) {
            if (!reads) return launch_map(ctx, AddrBool<false>{alpha_int != 0}, out, in, 2);
            return launch_map(ctx, AddrBool<true>{alpha_int != 0}, out, in, 3);
        }
        return dispatch_int(dt, [&](auto t) -> hmc_status {
            using T = decltype(t);
            if (!reads) return launch_map(ctx, AddrInt<T, false>{alpha_int, beta_int}, out, in, 2);
            return launch_map(ctx, AddrInt<T, true>{alpha_int, beta_int}, out, in, 3);
        });
    });
}

HMC_API hmc_status hmc_exclusive_cumprod(hmc_context_t ctx, const hmc_tensor_desc *out_lines, const hmc_tensor_desc *src_lines,
                                         int64_t n, int64_t out_stride, int64_t src_stride, int32_t reverse) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        const hmc_tensor_desc *d[2] = {out_lines, src_lines};
        int64_t nlines = 0;
        hmc_status s = check_operands(d, 2, &nlines);
        if (s != HMC_OK) return s;
        if (n < 0 || out_stride < 0 || src_stride < 0) return fail(HMC_INVALID, "negative line length or stride");
        if (out_lines->dtype != src_lines->dtype) return fail(HMC_INVALID, "exclusive_cumprod writes its input's dtype");
        if (!dtype_is_float(src_lines->dtype)) return fail(HMC_INVALID, "exclusive_cumprod needs a floating point tensor");
        if (nlines == 0 || n == 0) return HMC_OK;
        if (out_lines->data == nullptr || src_lines->data == nullptr) return fail(HMC_INVALID, "null data pointer");
        ScanArgs a{*out_lines, *src_lines, nlines, n, out_stride, src_stride, reverse != 0};
        const int64_t blocks = ceil_div(nlines, 256);
        const unsigned grid = static_cast<unsigned>(blocks < (int64_t{1} << 20) ? blocks : (int64_t{1} << 20));
        return dispatch_float(src_lines->dtype, [&](auto t) -> hmc_status {
            exclusive_cumprod_kernel<decltype(t)><<<grid, 256, 0, ctx->stream>>>(a);
            return launch_status("exclusive_cumprod kernel launch");
        });
    });
}
