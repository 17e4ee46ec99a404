// Device maths of the elementwise functors, in the computation type C of the dtype (float for
// F16/BF16/F32, double for F64), formula for formula as homura's CPU backend writes them
// (src/backend/cpu/mod.rs:362-403). The library is compiled with -fmad=false, so a*b+c is two
// roundings unless fma() is spelled out, which is where the CPU calls mul_add.
//
// exp, log, log1p, tanh and pow of the float computation type restate the host C library's algorithms and
// return its bits (libm32.cuh); so do exp, log1p and tanh of the double computation type (libm64.cuh), and with
// them sigmoid, silu, log_sigmoid, erf, gelu and gelu_tanh of F64 tensors; log, sin, cos and pow of F64 tensors are
// the CUDA library's (within an ulp or two of the C library's). sin, cos and erf of the float computation type are evaluated in double and
// rounded once: the correctly rounded f32 value except within ~1e-9 ulp of a tie, hence within one ulp of
// the C library's sinf / cosf (whose own error is below one ulp) and of the CPU's f64 erf rounded to f32.
#pragma once

#include "elem.cuh"
#include "libm32.cuh"
#include "libm64.cuh"

namespace hmc {

// e^d for an f64 argument to a relative error below 2^-40 (not the last bits of an f64): 2^k * 2^r with
// t = d * log2(e), k = round(t), r = t - k in [-1/2, 1/2], 2^r by its Taylor polynomial of degree 10, the
// scaling through the exponent field. Results below 2^-1022 come out as 2^-1022-ish tiny values instead of
// subnormals, which is all a sum of exponentials or an f32 result needs.
__device__ __forceinline__ double exp_lite(double d) {
    double t = d * 1.4426950408889634074;
    t = fmin(fmax(t, -1100.0), 1100.0);
    const double magic = 6755399441055744.0;  // 1.5 * 2^52: adding it leaves round(t) in the low word
    const double z = t + magic;
    const double r = t - (z - magic);
    int k = __double2loint(z);
    double p = 0x1.e4cf5158b8ecap-28;
    p = __fma_rn(p, r, 0x1.b5253d395e7c4p-24);
    p = __fma_rn(p, r, 0x1.62c0223a5c824p-20);
    p = __fma_rn(p, r, 0x1.ffcbfc588b0c7p-17);
    p = __fma_rn(p, r, 0x1.430912f86c787p-13);
    p = __fma_rn(p, r, 0x1.5d87fe78a6731p-10);
    p = __fma_rn(p, r, 0x1.3b2ab6fba4e77p-7);
    p = __fma_rn(p, r, 0x1.c6b08d704a0c0p-5);
    p = __fma_rn(p, r, 0x1.ebfbdff82c58fp-3);
    p = __fma_rn(p, r, 0x1.62e42fefa39efp-1);
    p = __fma_rn(p, r, 1.0);
    k = max(-1022, min(1023, k));
    const double y = p * __hiloint2double((k + 1023) << 20, 0);
    return d != d ? d : y;
}

// exp(d) for -1000 < d <= 0 or NaN, to a relative error below 2^-36: what a softmax row needs whose results
// are rounded to 24 bits or fewer. No range checks (the caller keeps d in range), a polynomial of degree 9,
// and a NaN passes through the arithmetic by itself. 14 f64 operations.
__device__ __forceinline__ double exp_short(double d) {
    const double t = d * 1.4426950408889634074;
    const double magic = 6755399441055744.0;  // 1.5 * 2^52: adding it leaves round(t) in the low word
    const double z = t + magic;
    const double r = t - (z - magic);
    const int k = __double2loint(z);
    double p = 0x1.b5253d395e7c4p-24;
    p = __fma_rn(p, r, 0x1.62c0223a5c824p-20);
    p = __fma_rn(p, r, 0x1.ffcbfc588b0c7p-17);
    p = __fma_rn(p, r, 0x1.430912f86c787p-13);
    p = __fma_rn(p, r, 0x1.5d87fe78a6731p-10);
    p = __fma_rn(p, r, 0x1.3b2ab6fba4e77p-7);
    p = __fma_rn(p, r, 0x1.c6b08d704a0c0p-5);
    p = __fma_rn(p, r, 0x1.ebfbdff82c58fp-3);
    p = __fma_rn(p, r, 0x1.62e42fefa39efp-1);
    p = __fma_rn(p, r, 1.0);
    return p * __hiloint2double((k + 1023) << 20, 0);
}

// 1 / s for a finite s >= 1 (or NaN) to within an f64 ulp or two: the hardware's 20-bit estimate and two Newton
// steps, a quarter of the instructions of the IEEE division. For results that are rounded to 24 bits or fewer.
__device__ __forceinline__ double reciprocal_short(double s) {
    double r;
    asm("rcp.approx.ftz.f64 %0, %1;" : "=d"(r) : "d"(s));
    r = __fma_rn(r, __fma_rn(-s, r, 1.0), r);
    r = __fma_rn(r, __fma_rn(-s, r, 1.0), r);
    return r;
}

// The f32 exponential, logarithm, log1p, tanh and power return the host C library's bits (libm32.cuh), so
// that formulas built on them (sigmoid, silu, log_sigmoid, gelu_tanh) are the CPU's bit for bit as well.
__device__ __forceinline__ float m_exp(float x) { return lm::expf(x); }
__device__ __forceinline__ double m_exp(double x) { return lm64::exp(x); }
__device__ __forceinline__ float m_log(float x) { return lm::logf(x); }
__device__ __forceinline__ double m_log(double x) { return log(x); }
__device__ __forceinline__ float m_log1p(float x) { return lm::log1pf(x); }
__device__ __forceinline__ double m_log1p(double x) { return lm64::log1p(x); }
__device__ __forceinline__ float m_sqrt(float x) { return sqrtf(x); }
__device__ __forceinline__ double m_sqrt(double x) { return sqrt(x); }
__device__ __forceinline__ float m_sin(float x) { return static_cast<float>(sin(static_cast<double>(x))); }
__device__ __forceinline__ double m_sin(double x) { return sin(x); }
__device__ __forceinline__ float m_cos(float x) { return static_cast<float>(cos(static_cast<double>(x))); }
__device__ __forceinline__ double m_cos(double x) { return cos(x); }
__device__ __forceinline__ float m_tanh(float x) { return lm::tanhf(x); }
__device__ __forceinline__ double m_tanh(double x) { return lm64::tanh(x); }
__device__ __forceinline__ float m_pow(float x, float y) {
    // x^2 (homura's `x.pow(2)`, e.g. in its rms_norm) is x * x rounded once. The C library's powf(x, 2) is within
    // 0.82 ulp of x^2 but not always the nearest value, so this differs from the CPU's result by one ulp for about
    // one argument in a thousand (an exact product with few bits, such as the square of a bf16 or f16 value, is
    // the same on both sides); every other exponent takes the library's algorithm and returns its bits.
    if (y == 2.0f) return x * x;
    return lm::powf(x, y);
}
__device__ __forceinline__ double m_pow(double x, double y) { return pow(x, y); }
__device__ __forceinline__ float m_abs(float x) { return fabsf(x); }
__device__ __forceinline__ double m_abs(double x) { return fabs(x); }
__device__ __forceinline__ float m_fma(float a, float b, float c) { return __fmaf_rn(a, b, c); }
__device__ __forceinline__ double m_fma(double a, double b, double c) { return __fma_rn(a, b, c); }

// homura's own erf in f64 (src/backend/cpu/num.rs:189-219): a series of positive terms below 1.5,
// the continued fraction of erfc up to 6, then 1. Used for F64 tensors, where the result is not
// rounded to a narrower type afterwards and the formula itself decides the last bits.
__device__ inline double erf_series(double x) {
    if (x != x) return x;
    const double ax = fabs(x);
    double r;
    if (ax < 1.5) {
        const double x2 = ax * ax;
        double term = ax, sum = ax, n = 0.0;
        while (term > 1e-17 * sum) {
            n += 1.0;
            term *= 2.0 * x2 / (2.0 * n + 1.0);
            sum += term;
        }
        r = 1.12837916709551257390 * lm64::exp(-x2) * sum;
    } else if (ax < 6.0) {
        double f = ax;
        for (int k = 80; k >= 1; --k) f = ax + (static_cast<double>(k) * 0.5) / f;
        r = 1.0 - lm64::exp(-ax * ax) / (1.7724538509055159 * f);
    } else {
        r = 1.0;
    }
    return copysign(r, x);
}
// For the float computation type the f64 value is rounded to f32 afterwards, so any f64 erf that is
// good to a few ulp gives the same f32 bits; the runtime's is far cheaper than 80 divisions.
__device__ __forceinline__ float m_erf(float x) { return static_cast<float>(erf(static_cast<double>(x))); }
__device__ __forceinline__ double m_erf(double x) { return erf_series(x); }

// For F16 and BF16 tensors the exponential family is evaluated with the special function unit in f32
// (ex2.approx, rcp.approx: relative error about 2^-21): the result is rounded to 11 or 8 significand bits
// afterwards, so it equals the correctly rounded one except within 2^-10 (F16) or 2^-13 (BF16) of a
// rounding tie, and then it is the neighbouring value: inside the one-ulp bar for transcendentals, at a
// handful of instructions per element, which is what a 2-byte element leaves room for at HBM speed.
__device__ __forceinline__ float fast_exp2(float t) {
    float y;
    asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(t));
    return y;
}
__device__ __forceinline__ float fast_exp(float x) { return fast_exp2(x * 1.44269504088896341f); }
// 1 / (1 + exp(-x)) with one special-function instruction each for the exponential and the reciprocal, both
// in their flush-to-zero forms, which need no fix-up code. That is safe here: an exponential small enough to
// be flushed vanishes in 1 + e anyway, and the reciprocal is taken of (1 + e) / 4, which keeps its result a
// normal number for every finite 1 + e; the final scaling by 1/4 is an ordinary multiplication, which keeps
// subnormal results. An overflowing exponential gives 0 like the CPU's f32 evaluation.
__device__ __forceinline__ float fast_sigmoid(float x) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -1.44269504088896341f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(__fmaf_rn(e, 0.25f, 0.25f)));
    return r * 0.25f;
}

template <int OP, class C, bool FAST = false>
__device__ __forceinline__ C unary_math(C x) {
    const C one = 1, zero = 0, half = static_cast<C>(0.5);
    if constexpr (FAST && std::is_same_v<C, float>) {
        if constexpr (OP == HMC_UNARY_EXP) return fast_exp(x);
        else if constexpr (OP == HMC_UNARY_SIGMOID) return fast_sigmoid(x);
        else if constexpr (OP == HMC_UNARY_SILU) return x * fast_sigmoid(x);
    }
    if constexpr (OP == HMC_UNARY_NEG) return -x;
    else if constexpr (OP == HMC_UNARY_ABS) return m_abs(x);
    else if constexpr (OP == HMC_UNARY_RELU) return (x != x || x > zero) ? x : zero;
    else if constexpr (OP == HMC_UNARY_SIGN) return x > zero ? one : (x < zero ? -one : zero);
    else if constexpr (OP == HMC_UNARY_EXP) return m_exp(x);
    else if constexpr (OP == HMC_UNARY_LOG) return m_log(x);
    else if constexpr (OP == HMC_UNARY_SQRT) return m_sqrt(x);
    else if constexpr (OP == HMC_UNARY_RSQRT) return one / m_sqrt(x);
    else if constexpr (OP == HMC_UNARY_RECIPROCAL) return one / x;
    else if constexpr (OP == HMC_UNARY_SIN) return m_sin(x);
    else if constexpr (OP == HMC_UNARY_COS) return m_cos(x);
    else if constexpr (OP == HMC_UNARY_ERF) return m_erf(x);
    else if constexpr (OP == HMC_UNARY_TANH) return m_tanh(x);
    else if constexpr (OP == HMC_UNARY_SIGMOID) return one / (one + m_exp(-x));
    else if constexpr (OP == HMC_UNARY_LOG_SIGMOID) {
        const C mn = (x != x || x < zero) ? x : zero;
        return mn - m_log1p(m_exp(-m_abs(x)));
    } else if constexpr (OP == HMC_UNARY_SILU) return x / (one + m_exp(-x));
    else if constexpr (OP == HMC_UNARY_GELU) {
        const C k = static_cast<C>(0.70710678118654752440);
        return half * x * (one + m_erf(x * k));
    } else {
        static_assert(OP == HMC_UNARY_GELU_TANH, "unknown unary op");
        // sqrt(2/pi) evaluated in f64, then converted, as the CPU does.
        const C k = static_cast<C>(0.79788456080286535588);
        const C c = static_cast<C>(0.044715);
        return half * x * (one + m_tanh(k * (x + c * x * x * x)));
    }
}

template <int OP, class C>
__device__ __forceinline__ C binary_math(C x, C y) {
    if constexpr (OP == HMC_BINARY_ADD) return x + y;
    else if constexpr (OP == HMC_BINARY_SUB) return x - y;
    else if constexpr (OP == HMC_BINARY_MUL) return x * y;
    else if constexpr (OP == HMC_BINARY_DIV) return x / y;
    else if constexpr (OP == HMC_BINARY_POW) return m_pow(x, y);
    else if constexpr (OP == HMC_BINARY_MAXIMUM) return (x != x || x > y) ? x : y;
    else {
        static_assert(OP == HMC_BINARY_MINIMUM, "unknown binary op");
        return (x != x || x < y) ? x : y;
    }
}

// Wrapping integer arithmetic (src/backend/cpu/num.rs:109-187).
template <class T> __device__ __forceinline__ T wadd(T a, T b) {
    using U = std::make_unsigned_t<T>;
    return static_cast<T>(static_cast<U>(static_cast<U>(a) + static_cast<U>(b)));
}
template <class T> __device__ __forceinline__ T wsub(T a, T b) {
    using U = std::make_unsigned_t<T>;
    return static_cast<T>(static_cast<U>(static_cast<U>(a) - static_cast<U>(b)));
}
template <class T> __device__ __forceinline__ T wmul(T a, T b) {
    using U = std::make_unsigned_t<T>;
    return static_cast<T>(static_cast<U>(static_cast<uint64_t>(static_cast<U>(a)) * static_cast<uint64_t>(static_cast<U>(b))));
}
template <class T> __device__ __forceinline__ T wneg(T a) {
    using U = std::make_unsigned_t<T>;
    return static_cast<T>(static_cast<U>(U{0} - static_cast<U>(a)));
}
template <class T> __device__ __forceinline__ T int_pow(T base, T exp) {
    int64_t e = static_cast<int64_t>(exp);
    if (e < 0) {
        int64_t b = static_cast<int64_t>(base);
        if (b == 1) return T{1};
        if (b == -1) return (e % 2 == 0) ? T{1} : base;
        return T{0};
    }
    T result = 1, b = base;
    uint64_t ue = static_cast<uint64_t>(e);
    while (ue > 0) {
        if (ue & 1) result = wmul(result, b);
        b = wmul(b, b);
        ue >>= 1;
    }
    return result;
}

}  // namespace hmc
