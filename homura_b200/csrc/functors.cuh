// The functors the elementwise engine is instantiated with. A functor names the element types of
// its output and of up to three inputs (Unused for absent ones) and maps input elements to an
// output element; what it computes follows homura's CPU kernels (src/backend/cpu/mod.rs).
#pragma once

#include "map.cuh"
#include "math.cuh"

namespace hmc {

// ---- unary (cpu::unary, src/backend/cpu/mod.rs:334-407) ----
// Float functors give their result in the computation type through compute(); the engine rounds the
// results of a whole vector to the dtype (two per conversion for the half types).
template <class T, int OP>
struct UnaryFloat {
    using Out = T; using A = T; using B = Unused; using C = Unused;
    using Compute = typename Comp<T>::C;
    static constexpr bool kFast = std::is_same_v<T, F16> || std::is_same_v<T, BF16>;
    __device__ __forceinline__ Compute compute(T v) const { return unary_math<OP, Compute, kFast>(up(v)); }
};

template <class T, int OP>
struct UnaryInt {
    using Out = T; using A = T; using B = Unused; using C = Unused;
    __device__ __forceinline__ T operator()(T x) const {
        if constexpr (OP == HMC_UNARY_NEG) return wneg(x);
        else if constexpr (OP == HMC_UNARY_ABS) {
            if constexpr (std::is_unsigned_v<T>) return x; else return x < 0 ? wneg(x) : x;
        } else if constexpr (OP == HMC_UNARY_RELU) return x > 0 ? x : T{0};
        else {
            static_assert(OP == HMC_UNARY_SIGN, "unknown integer unary op");
            if constexpr (std::is_unsigned_v<T>) return x > 0 ? T{1} : T{0};
            else return x > 0 ? T{1} : (x < 0 ? static_cast<T>(-1) : T{0});
        }
    }
};

template <class T>
struct LogicalNot {
    using Out = Bool; using A = T; using B = Unused; using C = Unused;
    __device__ __forceinline__ Bool operator()(T x) const { return Bool{static_cast<uint8_t>(!to_bool(x))}; }
};

// ---- copy / cast / fill (cpu::copy, cpu::fill, src/backend/cpu/mod.rs:314-332) ----
template <class D, class S>
struct Cast {
    using Out = D; using A = S; using B = Unused; using C = Unused;
    __device__ __forceinline__ D operator()(S x) const { return convert<D, S>(x); }
};

// Same-dtype copies and fills move bytes; one instantiation per element size.
template <class W>
struct Move {
    using Out = W; using A = W; using B = Unused; using C = Unused;
    __device__ __forceinline__ W operator()(W x) const { return x; }
};
template <class W>
struct Fill {
    using Out = W; using A = Unused; using B = Unused; using C = Unused;
    W value;
    __device__ __forceinline__ W operator()() const { return value; }
};

// ---- binary (cpu::binary, src/backend/cpu/mod.rs:409-466) ----
template <class T, int OP>
struct BinaryFloat {
    using Out = T; using A = T; using B = T; using C = Unused;
    using Compute = typename Comp<T>::C;
    __device__ __forceinline__ Compute compute(T x, T y) const { return binary_math<OP, Compute>(up(x), up(y)); }
};

// Two 2-byte inputs and a 2-byte output: 40 registers are enough, and six resident blocks instead of four measured
// 5 % faster on B200 for a bf16 product with a row-broadcast operand (latency bound).
template <class T, int OP>
struct LeanMinBlocks<BinaryFloat<T, OP>> {
    static constexpr int value = sizeof(T) <= 2 && OP != HMC_BINARY_POW && OP != HMC_BINARY_DIV ? 6 : 4;
};

// out = op(cast(a), cast(b)) in the promoted float dtype P: the bits of homura's separate cast
// kernels followed by the binary kernel.
template <class P, class TA, class TB, int OP>
struct BinaryPromoted {
    using Out = P; using A = TA; using B = TB; using C = Unused;
    using Compute = typename Comp<P>::C;
    __device__ __forceinline__ Compute compute(TA x, TB y) const {
        return binary_math<OP, Compute>(up(convert<P, TA>(x)), up(convert<P, TB>(y)));
    }
};

template <class T, int OP>
struct BinaryInt {
    using Out = T; using A = T; using B = T; using C = Unused;
    __device__ __forceinline__ T operator()(T x, T y) const {
        if constexpr (OP == HMC_BINARY_ADD) return wadd(x, y);
        else if constexpr (OP == HMC_BINARY_SUB) return wsub(x, y);
        else if constexpr (OP == HMC_BINARY_MUL) return wmul(x, y);
        else if constexpr (OP == HMC_BINARY_POW) return int_pow(x, y);
        else if constexpr (OP == HMC_BINARY_MAXIMUM) return x > y ? x : y;
        else {
            static_assert(OP == HMC_BINARY_MINIMUM, "unknown integer binary op");
            return x < y ? x : y;
        }
    }
};

template <bool AND>
struct BoolLogic {
    using Out = Bool; using A = Bool; using B = Bool; using C = Unused;
    __device__ __forceinline__ Bool operator()(Bool x, Bool y) const {
        return Bool{static_cast<uint8_t>(AND ? (x.b && y.b) : (x.b || y.b))};
    }
};

template <class T> __device__ __forceinline__ auto compare_key(T x) {
    if constexpr (std::is_same_v<T, F16> || std::is_same_v<T, BF16>) return up(x);
    else if constexpr (std::is_same_v<T, Bool>) return x.b;
    else return x;
}

template <class T, int OP>
struct Compare {
    using Out = Bool; using A = T; using B = T; using C = Unused;
    __device__ __forceinline__ Bool operator()(T p, T q) const {
        auto x = compare_key(p);
        auto y = compare_key(q);
        bool r;
        if constexpr (OP == HMC_BINARY_GREATER) r = x > y;
        else if constexpr (OP == HMC_BINARY_GREATER_EQUAL) r = x >= y;
        else if constexpr (OP == HMC_BINARY_LESS) r = x < y;
        else if constexpr (OP == HMC_BINARY_LESS_EQUAL) r = x <= y;
        else if constexpr (OP == HMC_BINARY_EQUAL) r = x == y;
        else r = x != y;
        return Bool{static_cast<uint8_t>(r)};
    }
};

// cpu::binary_scalar (src/backend/cpu/mod.rs:487-507): MODE 0 a*s, 1 a/s, 2 s/a.
template <class T, int MODE>
struct ScalarOp {
    using Out = T; using A = T; using B = Unused; using C = Unused;
    using Compute = typename Comp<T>::C;
    Compute s;
    __device__ __forceinline__ Compute compute(T x) const {
        if constexpr (MODE == 0) return up(x) * s;
        else if constexpr (MODE == 1) return up(x) / s;
        else return s / up(x);
    }
};

// cpu::fused (src/backend/cpu/mod.rs:509-569).
template <class T, int OP>
struct Fused2 {
    using Out = T; using A = T; using B = T; using C = Unused;
    using Compute = typename Comp<T>::C;
    Compute k;
    bool small;
    __device__ __forceinline__ Compute compute(T a, T b) const {
        auto x = up(a), y = up(b);
        if constexpr (OP == HMC_FUSED_SCALED_ADD) return m_fma(y, k, x);
        else return m_fma(k, y - x, small ? x : y);
    }
};
template <class T, int OP>
struct Fused3 {
    using Out = T; using A = T; using B = T; using C = T;
    using Compute = typename Comp<T>::C;
    Compute k;
    __device__ __forceinline__ Compute compute(T a, T b, T c) const {
        auto x = up(a), y = up(b), z = up(c);
        if constexpr (OP == HMC_FUSED_ADDCMUL) return m_fma(k * y, z, x);
        else return x + k * y / z;
    }
};

// cpu::where_ (src/backend/cpu/mod.rs:571-577) on the raw bits of an element size.
template <class W>
struct Select {
    using Out = W; using A = Bool; using B = W; using C = W;
    __device__ __forceinline__ W operator()(Bool c, W x, W y) const { return c.b ? x : y; }
};

// The unsigned word of an element size.
template <int BYTES> struct Word;
template <> struct Word<1> { using T = uint8_t; };
template <> struct Word<2> { using T = uint16_t; };
template <> struct Word<4> { using T = uint32_t; };
template <> struct Word<8> { using T = uint64_t; };

}  // namespace hmc
