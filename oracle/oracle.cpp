// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// A single-threaded CPU restatement of the arithmetic of homura's CPU reference backend for the
// elementwise / reduction hot path, used only as the checker of the CUDA kernels (tests, the smoke
// check, and the timed CPU baseline of the benchmark). Nothing that ships may call into it.
//
// Parity status: the original is Rust and cannot be built where this was written (no rustc), so
// this restatement is pinned indirectly: against homura's golden fixtures (PyTorch results, at
// homura's tolerances; AdamW fixtures bit for bit) and against the known-answer tests that live in
// homura's sources. Transcendental functions call the host libm, exactly what Rust's f32::exp and
// friends resolve to on Linux; homura's own tests do not pin those bit for bit either.
//
// Each function names the part of homura it follows (paths inside homura's repository).
//
// Interface: the tensor description of include/homura_cuda.h with `data` pointing to host memory.
// Every entry returns 0, or 2 where homura's CPU kernel would panic.

#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <type_traits>
#include <vector>

#include "../include/homura_cuda.h"

namespace {

// ---------------------------------------------------------------------------------------------
// Element types. src/dtype.rs:9-30. F16/BF16 are carried as tagged 16-bit patterns.
// ---------------------------------------------------------------------------------------------
struct F16 { uint16_t b; };
struct BF16 { uint16_t b; };
struct Bool { uint8_t b; };

inline uint32_t f32_bits(float f) { uint32_t u; std::memcpy(&u, &f, 4); return u; }
inline float bits_f32(uint32_t u) { float f; std::memcpy(&f, &u, 4); return f; }
inline uint64_t f64_bits(double f) { uint64_t u; std::memcpy(&u, &f, 8); return u; }
inline double bits_f64(uint64_t u) { double f; std::memcpy(&f, &u, 8); return f; }

// `half` 2.7 f16 -> f32 (software path; equal to F16C on every input): exact, NaN made quiet with
// its payload shifted up. Called by homura at src/backend/cpu/num.rs:85-95.
inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0x1F) {
        if (man == 0) return bits_f32(sign | 0x7F800000u);
        return bits_f32(sign | 0x7FC00000u | (man << 13));
    }
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        // subnormal: man * 2^-24, exact in f32
        float v = (float)man * 5.9604644775390625e-08f;
        return bits_f32(f32_bits(v) | sign);
    }
    return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

// `half` 2.7 f32 -> f16: round to nearest even, overflow to infinity, NaN keeps its top payload bits
// and is made quiet. Restated by homura in csrc/elem.hpp:131-160.
inline uint16_t f32_to_f16(float f) {
    uint32_t x = f32_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t exp = (x >> 23) & 0xFFu;
    uint32_t man = x & 0x7FFFFFu;
    if (exp == 0xFF) {
        return (uint16_t)(sign | 0x7C00u | (man ? 0x0200u : 0u) | (man >> 13));
    }
    int32_t e = (int32_t)exp - 127 + 15;
    if (e >= 0x1F) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (14 - e > 24) return (uint16_t)sign;
        uint32_t m = man | 0x800000u;
        uint32_t shift = (uint32_t)(14 - e);
        uint32_t hm = m >> shift;
        uint32_t round = 1u << (shift - 1);
        if ((m & round) && (m & (3 * round - 1))) hm += 1;
        return (uint16_t)(sign | hm);
    }
    uint32_t h = sign | ((uint32_t)e << 10) | (man >> 13);
    if ((man & 0x1000u) && (man & 0x2FFFu)) h += 1;
    return (uint16_t)h;
}

// `half` 2.7 bf16 <-> f32. csrc/elem.hpp:162-172 restates the rounding.
inline float bf16_to_f32(uint16_t h) {
    if ((h & 0x7FFFu) > 0x7F80u) return bits_f32(((uint32_t)h | 0x0040u) << 16);
    return bits_f32((uint32_t)h << 16);
}
inline uint16_t f32_to_bf16(float f) {
    uint32_t x = f32_bits(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x0040u);
    if ((x & 0x8000u) && (x & 0x17FFFu)) return (uint16_t)((x >> 16) + 1);
    return (uint16_t)(x >> 16);
}

// Rust's `v as i64` for floats: toward zero, saturating, NaN -> 0. src/dtype.rs:195-204.
inline int64_t f64_as_i64(double v) {
    if (v != v) return 0;
    if (v >= 9223372036854775808.0) return INT64_MAX;
    if (v <= -9223372036854775808.0) return INT64_MIN;
    return (int64_t)v;
}
inline int64_t f32_as_i64(float v) { return f64_as_i64((double)v); }

template <class T> struct Tr;  // traits: code, kind
enum Kind { kBool, kInt, kFloat };
#define TRAIT(T, CODE, KIND) template <> struct Tr<T> { static constexpr int code = CODE; static constexpr Kind kind = KIND; };
TRAIT(Bool, HMC_BOOL, kBool)
TRAIT(uint8_t, HMC_U8, kInt)
TRAIT(int8_t, HMC_I8, kInt)
TRAIT(int16_t, HMC_I16, kInt)
TRAIT(int32_t, HMC_I32, kInt)
TRAIT(int64_t, HMC_I64, kInt)
TRAIT(F16, HMC_F16, kFloat)
TRAIT(BF16, HMC_BF16, kFloat)
TRAIT(float, HMC_F32, kFloat)
TRAIT(double, HMC_F64, kFloat)

// Sealed::{to_f64,to_i64,to_bool,from_f64,from_i64,from_bool}. src/dtype.rs:144-273.
template <class T> inline double to_f64(T v) { return (double)v; }
template <> inline double to_f64(F16 v) { return (double)f16_to_f32(v.b); }
template <> inline double to_f64(BF16 v) { return (double)bf16_to_f32(v.b); }
template <> inline double to_f64(Bool v) { return v.b ? 1.0 : 0.0; }

template <class T> inline int64_t to_i64(T v) { return (int64_t)v; }
template <> inline int64_t to_i64(float v) { return f32_as_i64(v); }
template <> inline int64_t to_i64(double v) { return f64_as_i64(v); }
template <> inline int64_t to_i64(F16 v) { return f32_as_i64(f16_to_f32(v.b)); }
template <> inline int64_t to_i64(BF16 v) { return f32_as_i64(bf16_to_f32(v.b)); }
template <> inline int64_t to_i64(Bool v) { return v.b ? 1 : 0; }

template <class T> inline bool to_bool(T v) { return v != 0; }
template <> inline bool to_bool(F16 v) { return f16_to_f32(v.b) != 0.0f; }
template <> inline bool to_bool(BF16 v) { return bf16_to_f32(v.b) != 0.0f; }
template <> inline bool to_bool(Bool v) { return v.b != 0; }

template <class T> inline T wrap_int(int64_t v) {
    using U = std::make_unsigned_t<T>;
    U u = (U)(uint64_t)v;
    T t; std::memcpy(&t, &u, sizeof t); return t;
}

template <class T> inline T from_f64(double v) { return wrap_int<T>(f64_as_i64(v)); }
template <> inline float from_f64(double v) { return (float)v; }
template <> inline double from_f64(double v) { return v; }
template <> inline F16 from_f64(double v) { return F16{f32_to_f16((float)v)}; }
template <> inline BF16 from_f64(double v) { return BF16{f32_to_bf16((float)v)}; }
template <> inline Bool from_f64(double v) { return Bool{(uint8_t)(v != 0.0)}; }

template <class T> inline T from_i64(int64_t v) { return wrap_int<T>(v); }
template <> inline float from_i64(int64_t v) { return (float)v; }
template <> inline double from_i64(int64_t v) { return (double)v; }
template <> inline F16 from_i64(int64_t v) { return F16{f32_to_f16((float)v)}; }
template <> inline BF16 from_i64(int64_t v) { return BF16{f32_to_bf16((float)v)}; }
template <> inline Bool from_i64(int64_t v) { return Bool{(uint8_t)(v != 0)}; }

template <class T> inline T from_bool(bool v) { return (T)(v ? 1 : 0); }
template <> inline F16 from_bool(bool v) { return F16{(uint16_t)(v ? 0x3C00 : 0)}; }
template <> inline BF16 from_bool(bool v) { return BF16{(uint16_t)(v ? 0x3F80 : 0)}; }
template <> inline Bool from_bool(bool v) { return Bool{(uint8_t)v}; }

// Element::to_element. src/dtype.rs:185-192.
template <class D, class S> inline D to_element(S x) {
    if constexpr (Tr<S>::kind == kFloat) return from_f64<D>(to_f64(x));
    else if constexpr (Tr<S>::kind == kInt) return from_i64<D>(to_i64(x));
    else return from_bool<D>(to_bool(x));
}

// FloatElement: computation type, up and down. src/backend/cpu/num.rs:55-107.
template <class T> struct Comp { using C = float; };
template <> struct Comp<double> { using C = double; };
inline float up(float v) { return v; }
inline double up(double v) { return v; }
inline float up(F16 v) { return f16_to_f32(v.b); }
inline float up(BF16 v) { return bf16_to_f32(v.b); }
template <class T> inline T down(typename Comp<T>::C c);
template <> inline float down<float>(float c) { return c; }
template <> inline double down<double>(double c) { return c; }
template <> inline F16 down<F16>(float c) { return F16{f32_to_f16(c)}; }
template <> inline BF16 down<BF16>(float c) { return BF16{f32_to_bf16(c)}; }

// ---------------------------------------------------------------------------------------------
// Strided walk over N operands in row-major order. src/backend/cpu/iter.rs:21-94 (the merging of
// dimensions there changes the loop nest, not the order of visits).
// ---------------------------------------------------------------------------------------------
template <int N, class F>
void walk(int ndim, const int64_t *sizes, const int64_t *const strides[N], const int64_t base[N], F &&f) {
    for (int d = 0; d < ndim; ++d) if (sizes[d] == 0) return;
    int64_t off[N];
    for (int k = 0; k < N; ++k) off[k] = base[k];
    if (ndim == 0) { f(off); return; }
    int64_t idx[HMC_MAX_DIMS] = {0};
    const int last = ndim - 1;
    for (;;) {
        int64_t o[N];
        for (int k = 0; k < N; ++k) o[k] = off[k];
        for (int64_t i = 0; i < sizes[last]; ++i) {
            f(o);
            for (int k = 0; k < N; ++k) o[k] += strides[k][last];
        }
        int d = last - 1;
        for (; d >= 0; --d) {
            idx[d] += 1;
            for (int k = 0; k < N; ++k) off[k] += strides[k][d];
            if (idx[d] < sizes[d]) break;
            for (int k = 0; k < N; ++k) off[k] -= strides[k][d] * sizes[d];
            idx[d] = 0;
        }
        if (d < 0) return;
    }
}

inline bool same_shape(const hmc_tensor_desc *a, const hmc_tensor_desc *b) {
    if (a->ndim != b->ndim) return false;
    for (int d = 0; d < a->ndim; ++d) if (a->sizes[d] != b->sizes[d]) return false;
    return true;
}

// map1 / map2 / map3. src/backend/cpu/mod.rs:196-261.
template <class O, class A, class F>
int map1(const hmc_tensor_desc *out, const hmc_tensor_desc *a, F f) {
    if (!same_shape(out, a)) return 2;
    O *po = (O *)out->data; const A *pa = (const A *)a->data;
    const int64_t *st[2] = {out->strides, a->strides};
    int64_t base[2] = {out->offset, a->offset};
    walk<2>(out->ndim, out->sizes, st, base, [&](const int64_t *o) { po[o[0]] = f(pa[o[1]]); });
    return 0;
}
template <class O, class A, class B, class F>
int map2(const hmc_tensor_desc *out, const hmc_tensor_desc *a, const hmc_tensor_desc *b, F f) {
    if (!same_shape(out, a) || !same_shape(out, b)) return 2;
    O *po = (O *)out->data; const A *pa = (const A *)a->data; const B *pb = (const B *)b->data;
    const int64_t *st[3] = {out->strides, a->strides, b->strides};
    int64_t base[3] = {out->offset, a->offset, b->offset};
    walk<3>(out->ndim, out->sizes, st, base, [&](const int64_t *o) { po[o[0]] = f(pa[o[1]], pb[o[2]]); });
    return 0;
}
template <class O, class A, class B, class C, class F>
int map3(const hmc_tensor_desc *out, const hmc_tensor_desc *a, const hmc_tensor_desc *b,
         const hmc_tensor_desc *c, F f) {
    if (!same_shape(out, a) || !same_shape(out, b) || !same_shape(out, c)) return 2;
    O *po = (O *)out->data; const A *pa = (const A *)a->data; const B *pb = (const B *)b->data;
    const C *pc = (const C *)c->data;
    const int64_t *st[4] = {out->strides, a->strides, b->strides, c->strides};
    int64_t base[4] = {out->offset, a->offset, b->offset, c->offset};
    walk<4>(out->ndim, out->sizes, st, base,
            [&](const int64_t *o) { po[o[0]] = f(pa[o[1]], pb[o[2]], pc[o[3]]); });
    return 0;
}

// dispatch over dtypes (dispatch_all / dispatch_float / dispatch_int, src/backend/cpu/mod.rs:66-166)
template <class F> int dispatch_all(int dtype, F &&f) {
    switch (dtype) {
        case HMC_BOOL: return f(Bool{});
        case HMC_U8: return f(uint8_t{});
        case HMC_I8: return f(int8_t{});
        case HMC_I16: return f(int16_t{});
        case HMC_I32: return f(int32_t{});
        case HMC_I64: return f(int64_t{});
        case HMC_F16: return f(F16{});
        case HMC_BF16: return f(BF16{});
        case HMC_F32: return f(float{});
        case HMC_F64: return f(double{});
    }
    return 2;
}
template <class F> int dispatch_float(int dtype, F &&f) {
    switch (dtype) {
        case HMC_F16: return f(F16{});
        case HMC_BF16: return f(BF16{});
        case HMC_F32: return f(float{});
        case HMC_F64: return f(double{});
    }
    return 2;
}
template <class F> int dispatch_int(int dtype, F &&f) {
    switch (dtype) {
        case HMC_U8: return f(uint8_t{});
        case HMC_I8: return f(int8_t{});
        case HMC_I16: return f(int16_t{});
        case HMC_I32: return f(int32_t{});
        case HMC_I64: return f(int64_t{});
    }
    return 2;
}
inline bool is_float(int dt) { return dt >= HMC_F16 && dt <= HMC_F64; }
inline bool is_int(int dt) { return dt >= HMC_U8 && dt <= HMC_I64; }

// wrapping integer helpers. src/backend/cpu/num.rs:109-158.
template <class T> inline T wadd(T a, T b) { using U = std::make_unsigned_t<T>; return (T)(U)((U)a + (U)b); }
template <class T> inline T wsub(T a, T b) { using U = std::make_unsigned_t<T>; return (T)(U)((U)a - (U)b); }
template <class T> inline T wmul(T a, T b) {
    using U = std::make_unsigned_t<T>;
    return (T)(U)((uint64_t)(U)a * (uint64_t)(U)b);
}
template <class T> inline T wneg(T a) { using U = std::make_unsigned_t<T>; return (T)(U)((U)0 - (U)a); }
template <class T> inline T wabs(T a) {
    if constexpr (std::is_unsigned_v<T>) return a; else return a < 0 ? wneg(a) : a;
}

// int_pow. src/backend/cpu/num.rs:160-187.
template <class T> inline T int_pow(T base, T exp) {
    int64_t e = (int64_t)exp;
    if (e < 0) {
        int64_t b = (int64_t)base;
        if (b == 1) return (T)1;
        if (b == -1) return (e % 2 == 0) ? (T)1 : base;
        return (T)0;
    }
    T result = 1, b = base;
    uint64_t ue = (uint64_t)e;
    while (ue > 0) {
        if (ue & 1) result = wmul(result, b);
        b = wmul(b, b);
        ue >>= 1;
    }
    return result;
}

// erf: homura's own evaluation in f64 (positive-term series below 1.5, continued fraction of erfc
// up to 6, then 1). src/backend/cpu/num.rs:189-219.
double erf_f64(double x) {
    if (x != x) return x;
    double ax = std::fabs(x);
    double r;
    if (ax < 1.5) {
        double x2 = ax * ax, term = ax, sum = ax, n = 0.0;
        while (term > 1e-17 * sum) {
            n += 1.0;
            term *= 2.0 * x2 / (2.0 * n + 1.0);
            sum += term;
        }
        r = 1.1283791670955126 /* 2/sqrt(pi) */ * std::exp(-x2) * sum;
    } else if (ax < 6.0) {
        double f = ax;
        for (int k = 80; k >= 1; --k) f = ax + ((double)k * 0.5) / f;
        r = 1.0 - std::exp(-ax * ax) / (std::sqrt(3.141592653589793) * f);
    } else {
        r = 1.0;
    }
    return std::copysign(r, x);
}
inline float erf_c(float x) { return (float)erf_f64((double)x); }
inline double erf_c(double x) { return erf_f64(x); }

// Float maths of the computation type: the libm entry Rust's methods lower to.
inline float m_exp(float x) { return expf(x); }     inline double m_exp(double x) { return exp(x); }
inline float m_log(float x) { return logf(x); }     inline double m_log(double x) { return log(x); }
inline float m_log1p(float x) { return log1pf(x); } inline double m_log1p(double x) { return log1p(x); }
inline float m_sqrt(float x) { return sqrtf(x); }   inline double m_sqrt(double x) { return sqrt(x); }
inline float m_sin(float x) { return sinf(x); }     inline double m_sin(double x) { return sin(x); }
inline float m_cos(float x) { return cosf(x); }     inline double m_cos(double x) { return cos(x); }
inline float m_tanh(float x) { return tanhf(x); }   inline double m_tanh(double x) { return tanh(x); }
inline float m_pow(float x, float y) { return powf(x, y); } inline double m_pow(double x, double y) { return pow(x, y); }
inline float m_fma(float a, float b, float c) { return fmaf(a, b, c); }
inline double m_fma(double a, double b, double c) { return fma(a, b, c); }
inline float m_abs(float x) { return fabsf(x); }    inline double m_abs(double x) { return fabs(x); }

}  // namespace

extern "C" {

// cpu::copy. src/backend/cpu/mod.rs:314-324.
int orc_copy(const hmc_tensor_desc *dst, const hmc_tensor_desc *src) {
    return dispatch_all(src->dtype, [&](auto s) {
        using S = decltype(s);
        return dispatch_all(dst->dtype, [&](auto d) {
            using D = decltype(d);
            if constexpr (std::is_same_v<S, D>) return map1<D, S>(dst, src, [](S x) { return x; });
            else return map1<D, S>(dst, src, [](S x) { return to_element<D, S>(x); });
        });
    });
}

// cpu::fill with the value already converted to the element (`bits`), as the GPU boundary takes
// it. src/backend/cpu/mod.rs:326-332, src/backend/rocm/copy.rs:256-270.
int orc_fill(const hmc_tensor_desc *dst, uint64_t bits) {
    return dispatch_all(dst->dtype, [&](auto d) {
        using D = decltype(d);
        D v; std::memcpy(&v, &bits, sizeof v);
        D *p = (D *)dst->data;
        const int64_t *st[1] = {dst->strides};
        int64_t base[1] = {dst->offset};
        walk<1>(dst->ndim, dst->sizes, st, base, [&](const int64_t *o) { p[o[0]] = v; });
        return 0;
    });
}

// cpu::unary. src/backend/cpu/mod.rs:334-407.
int orc_unary(int32_t op, const hmc_tensor_desc *out, const hmc_tensor_desc *src) {
    const int dt = src->dtype;
    if (op == HMC_UNARY_LOGICAL_NOT) {
        if (out->dtype != HMC_BOOL) return 2;
        return dispatch_all(dt, [&](auto t) {
            using T = decltype(t);
            return map1<Bool, T>(out, src, [](T x) { return Bool{(uint8_t)!to_bool(x)}; });
        });
    }
    if (out->dtype != dt) return 2;
    if (op == HMC_UNARY_SIGN && dt == HMC_BOOL) return map1<Bool, Bool>(out, src, [](Bool x) { return x; });
    if ((op == HMC_UNARY_NEG || op == HMC_UNARY_ABS || op == HMC_UNARY_RELU || op == HMC_UNARY_SIGN) && is_int(dt)) {
        return dispatch_int(dt, [&](auto t) {
            using T = decltype(t);
            switch (op) {
                case HMC_UNARY_NEG: return map1<T, T>(out, src, [](T x) { return wneg(x); });
                case HMC_UNARY_ABS: return map1<T, T>(out, src, [](T x) { return wabs(x); });
                case HMC_UNARY_RELU: return map1<T, T>(out, src, [](T x) { return x > 0 ? x : (T)0; });
                default: return map1<T, T>(out, src, [](T x) { return x > 0 ? (T)1 : (x < 0 ? wneg((T)1) : (T)0); });
            }
        });
    }
    return dispatch_float(dt, [&](auto t) {
        using T = decltype(t);
        using C = typename Comp<T>::C;
        const C one = 1, zero = 0, half = (C)0.5;
        auto fm = [&](auto g) { return map1<T, T>(out, src, [g](T v) { C x = up(v); return down<T>(g(x)); }); };
        switch (op) {
            case HMC_UNARY_NEG: return fm([](C x) { return -x; });
            case HMC_UNARY_ABS: return fm([](C x) { return m_abs(x); });
            case HMC_UNARY_RELU: return fm([=](C x) { return (x != x || x > zero) ? x : zero; });
            case HMC_UNARY_SIGN: return fm([=](C x) { return x > zero ? one : (x < zero ? -one : zero); });
            case HMC_UNARY_EXP: return fm([](C x) { return m_exp(x); });
            case HMC_UNARY_LOG: return fm([](C x) { return m_log(x); });
            case HMC_UNARY_SQRT: return fm([](C x) { return m_sqrt(x); });
            case HMC_UNARY_RSQRT: return fm([=](C x) { return one / m_sqrt(x); });
            case HMC_UNARY_RECIPROCAL: return fm([=](C x) { return one / x; });
            case HMC_UNARY_SIN: return fm([](C x) { return m_sin(x); });
            case HMC_UNARY_COS: return fm([](C x) { return m_cos(x); });
            case HMC_UNARY_ERF: return fm([](C x) { return erf_c(x); });
            case HMC_UNARY_TANH: return fm([](C x) { return m_tanh(x); });
            case HMC_UNARY_SIGMOID: return fm([=](C x) { return one / (one + m_exp(-x)); });
            case HMC_UNARY_LOG_SIGMOID:
                return fm([=](C x) {
                    C mn = (x != x || x < zero) ? x : zero;
                    return mn - m_log1p(m_exp(-m_abs(x)));
                });
            case HMC_UNARY_SILU: return fm([=](C x) { return x / (one + m_exp(-x)); });
            case HMC_UNARY_GELU: {
                const C k = (C)0.70710678118654752440;  // FRAC_1_SQRT_2
                return fm([=](C x) { return half * x * (one + erf_c(x * k)); });
            }
            case HMC_UNARY_GELU_TANH: {
                const C k = (C)std::sqrt(2.0 / 3.14159265358979323846);
                const C c = (C)0.044715;
                return fm([=](C x) { return half * x * (one + m_tanh(k * (x + c * x * x * x))); });
            }
        }
        return 2;
    });
}

// cpu::binary. src/backend/cpu/mod.rs:409-466.
int orc_binary(int32_t op, const hmc_tensor_desc *out, const hmc_tensor_desc *a, const hmc_tensor_desc *b) {
    const int dt = a->dtype;
    if (b->dtype != dt) return 2;
    if (op >= HMC_BINARY_GREATER && op <= HMC_BINARY_NOT_EQUAL) {
        if (out->dtype != HMC_BOOL) return 2;
        return dispatch_all(dt, [&](auto t) {
            using T = decltype(t);
            auto cmp = [&](auto g) {
                return map2<Bool, T, T>(out, a, b, [g](T x, T y) {
                    if constexpr (std::is_same_v<T, F16> || std::is_same_v<T, BF16>) return Bool{(uint8_t)g(up(x), up(y))};
                    else if constexpr (std::is_same_v<T, Bool>) return Bool{(uint8_t)g(x.b, y.b)};
                    else return Bool{(uint8_t)g(x, y)};
                });
            };
            switch (op) {
                case HMC_BINARY_GREATER: return cmp([](auto x, auto y) { return x > y; });
                case HMC_BINARY_GREATER_EQUAL: return cmp([](auto x, auto y) { return x >= y; });
                case HMC_BINARY_LESS: return cmp([](auto x, auto y) { return x < y; });
                case HMC_BINARY_LESS_EQUAL: return cmp([](auto x, auto y) { return x <= y; });
                case HMC_BINARY_EQUAL: return cmp([](auto x, auto y) { return x == y; });
                default: return cmp([](auto x, auto y) { return x != y; });
            }
        });
    }
    if (op == HMC_BINARY_LOGICAL_AND || op == HMC_BINARY_LOGICAL_OR) {
        if (dt != HMC_BOOL || out->dtype != HMC_BOOL) return 2;
        const bool is_and = op == HMC_BINARY_LOGICAL_AND;
        return map2<Bool, Bool, Bool>(out, a, b, [=](Bool x, Bool y) {
            return Bool{(uint8_t)(is_and ? (x.b && y.b) : (x.b || y.b))};
        });
    }
    if (out->dtype != dt) return 2;
    if (dt == HMC_BOOL) {
        if (op == HMC_BINARY_ADD || op == HMC_BINARY_MAXIMUM)
            return map2<Bool, Bool, Bool>(out, a, b, [](Bool x, Bool y) { return Bool{(uint8_t)(x.b || y.b)}; });
        if (op == HMC_BINARY_MUL || op == HMC_BINARY_MINIMUM)
            return map2<Bool, Bool, Bool>(out, a, b, [](Bool x, Bool y) { return Bool{(uint8_t)(x.b && y.b)}; });
        return 2;
    }
    if (is_int(dt)) {
        return dispatch_int(dt, [&](auto t) {
            using T = decltype(t);
            switch (op) {
                case HMC_BINARY_ADD: return map2<T, T, T>(out, a, b, [](T x, T y) { return wadd(x, y); });
                case HMC_BINARY_SUB: return map2<T, T, T>(out, a, b, [](T x, T y) { return wsub(x, y); });
                case HMC_BINARY_MUL: return map2<T, T, T>(out, a, b, [](T x, T y) { return wmul(x, y); });
                case HMC_BINARY_POW: return map2<T, T, T>(out, a, b, [](T x, T y) { return int_pow(x, y); });
                case HMC_BINARY_MAXIMUM: return map2<T, T, T>(out, a, b, [](T x, T y) { return x > y ? x : y; });
                case HMC_BINARY_MINIMUM: return map2<T, T, T>(out, a, b, [](T x, T y) { return x < y ? x : y; });
            }
            return 2;
        });
    }
    return dispatch_float(dt, [&](auto t) {
        using T = decltype(t);
        using C = typename Comp<T>::C;
        auto fm = [&](auto g) {
            return map2<T, T, T>(out, a, b, [g](T u, T v) { C x = up(u), y = up(v); return down<T>(g(x, y)); });
        };
        switch (op) {
            case HMC_BINARY_ADD: return fm([](C x, C y) { return x + y; });
            case HMC_BINARY_SUB: return fm([](C x, C y) { return x - y; });
            case HMC_BINARY_MUL: return fm([](C x, C y) { return x * y; });
            case HMC_BINARY_DIV: return fm([](C x, C y) { return x / y; });
            case HMC_BINARY_POW: return fm([](C x, C y) { return m_pow(x, y); });
            case HMC_BINARY_MAXIMUM: return fm([](C x, C y) { return (x != x || x > y) ? x : y; });
            case HMC_BINARY_MINIMUM: return fm([](C x, C y) { return (x != x || x < y) ? x : y; });
        }
        return 2;
    });
}

// cpu::binary_constant: binary with a one-element tensor of the constant broadcast to a's shape.
// src/backend/cpu/mod.rs:468-485.
int orc_binary_constant(int32_t op, const hmc_tensor_desc *out, const hmc_tensor_desc *a, uint64_t bits,
                        int32_t constant_first) {
    uint64_t cell = bits;
    hmc_tensor_desc c = *a;
    c.data = &cell;
    c.offset = 0;
    for (int d = 0; d < c.ndim; ++d) c.strides[d] = 0;
    return constant_first ? orc_binary(op, out, &c, a) : orc_binary(op, out, a, &c);
}

// cpu::binary_scalar. src/backend/cpu/mod.rs:487-507.
int orc_binary_scalar(int32_t op, const hmc_tensor_desc *out, const hmc_tensor_desc *a, double s,
                      int32_t scalar_first) {
    if (out->dtype != a->dtype) return 2;
    return dispatch_float(a->dtype, [&](auto t) {
        using T = decltype(t);
        using C = typename Comp<T>::C;
        const C sc = (C)s;
        if (op == HMC_BINARY_MUL) return map1<T, T>(out, a, [=](T x) { return down<T>(up(x) * sc); });
        if (op == HMC_BINARY_DIV && !scalar_first) return map1<T, T>(out, a, [=](T x) { return down<T>(up(x) / sc); });
        if (op == HMC_BINARY_DIV) return map1<T, T>(out, a, [=](T x) { return down<T>(sc / up(x)); });
        return 2;
    });
}

// cpu::fused with the scalar as homura's Fused carries it (alpha, weight or value as f64); the
// coefficient is derived here the way the CPU kernel derives it. src/backend/cpu/mod.rs:509-569.
int orc_fused(int32_t op, const hmc_tensor_desc *out, const hmc_tensor_desc *a, const hmc_tensor_desc *b,
              const hmc_tensor_desc *c, double value) {
    if (a->dtype != out->dtype || b->dtype != out->dtype || (c && c->dtype != out->dtype)) return 2;
    return dispatch_float(out->dtype, [&](auto t) {
        using T = decltype(t);
        using C = typename Comp<T>::C;
        switch (op) {
            case HMC_FUSED_SCALED_ADD: {
                const C alpha = up(down<T>((C)value));
                return map2<T, T, T>(out, a, b, [=](T x, T y) { return down<T>(m_fma(up(y), alpha, up(x))); });
            }
            case HMC_FUSED_LERP: {
                const C w = (C)value;
                const bool small = m_abs(w) < (C)0.5;
                const C coeff = small ? w : w - (C)1.0;
                return map2<T, T, T>(out, a, b, [=](T x0, T y0) {
                    C x = up(x0), y = up(y0);
                    return down<T>(m_fma(coeff, y - x, small ? x : y));
                });
            }
            case HMC_FUSED_ADDCMUL: {
                if (!c) return 2;
                const C v = (C)value;
                return map3<T, T, T, T>(out, a, b, c, [=](T x, T y, T z) { return down<T>(m_fma(v * up(y), up(z), up(x))); });
            }
            case HMC_FUSED_ADDCDIV: {
                if (!c) return 2;
                const C v = (C)value;
                return map3<T, T, T, T>(out, a, b, c, [=](T x, T y, T z) { return down<T>(up(x) + v * up(y) / up(z)); });
            }
        }
        return 2;
    });
}

// cpu::where_. src/backend/cpu/mod.rs:571-577.
int orc_where(const hmc_tensor_desc *out, const hmc_tensor_desc *cond, const hmc_tensor_desc *x,
              const hmc_tensor_desc *y) {
    if (cond->dtype != HMC_BOOL || x->dtype != out->dtype || y->dtype != out->dtype) return 2;
    return dispatch_all(out->dtype, [&](auto t) {
        using T = decltype(t);
        return map3<T, Bool, T, T>(out, cond, x, y, [](Bool c, T p, T q) { return c.b ? p : q; });
    });
}

// cpu::where_constant. src/backend/cpu/mod.rs:579-600.
int orc_where_constant(const hmc_tensor_desc *out, const hmc_tensor_desc *cond, const hmc_tensor_desc *x,
                       uint64_t x_bits, const hmc_tensor_desc *y, uint64_t y_bits) {
    uint64_t xc = x_bits, yc = y_bits;
    hmc_tensor_desc xd, yd;
    auto constant = [&](hmc_tensor_desc &d, uint64_t *cell) {
        d = *out;
        d.data = cell;
        d.offset = 0;
        for (int k = 0; k < d.ndim; ++k) d.strides[k] = 0;
    };
    if (!x) constant(xd, &xc);
    if (!y) constant(yd, &yc);
    return orc_where(out, cond, x ? x : &xd, y ? y : &yd);
}

}  // extern "C"

namespace {

// fold. src/backend/cpu/reduce.rs:42-73: for every kept position (row-major), the reduced elements
// in row-major order.
template <class S, class O, class A, class Step, class Finish>
int fold(const hmc_tensor_desc *out, const hmc_tensor_desc *kept, const hmc_tensor_desc *red, A init,
         Step step, Finish finish) {
    int64_t count = 1;
    for (int d = 0; d < red->ndim; ++d) count *= red->sizes[d];
    const S *ps = (const S *)kept->data;
    O *po = (O *)out->data;
    const int64_t *kst[1] = {kept->strides};
    const int64_t *rst[1] = {red->strides};
    int64_t o = out->offset;
    int64_t kbase[1] = {kept->offset};
    walk<1>(kept->ndim, kept->sizes, kst, kbase, [&](const int64_t *i) {
        A acc = init;
        int64_t rbase[1] = {i[0]};
        walk<1>(red->ndim, red->sizes, rst, rbase, [&](const int64_t *j) { acc = step(acc, ps[j[0]]); });
        po[o++] = finish(acc, count);
    });
    return 0;
}

// `replaces`. src/backend/cpu/reduce.rs:75-86.
template <class T> struct Opt { bool has; T v; };
template <class T> inline bool elem_is_nan(T x) {
    if constexpr (std::is_same_v<T, F16> || std::is_same_v<T, BF16>) { float f = up(x); return f != f; }
    else if constexpr (std::is_floating_point_v<T>) return x != x;
    else return false;
}
template <class T> inline bool elem_gt(T x, T y) {
    if constexpr (std::is_same_v<T, F16> || std::is_same_v<T, BF16>) return up(x) > up(y);
    else if constexpr (std::is_same_v<T, Bool>) return x.b > y.b;
    else return x > y;
}
template <class T> inline bool replaces(Opt<T> acc, T x, bool is_max) {
    if (!acc.has) return true;
    if (elem_is_nan(acc.v)) return false;
    return elem_is_nan(x) || (is_max ? elem_gt(x, acc.v) : elem_gt(acc.v, x));
}

}  // namespace

extern "C" {

// cpu::reduce. src/backend/cpu/reduce.rs:88-131.
int orc_reduce(int32_t op, const hmc_tensor_desc *out, const hmc_tensor_desc *kept, const hmc_tensor_desc *red) {
    const int dt = kept->dtype;
    if ((op == HMC_REDUCE_SUM || op == HMC_REDUCE_PROD || op == HMC_REDUCE_MEAN) && is_float(dt)) {
        if (out->dtype != dt) return 2;
        return dispatch_float(dt, [&](auto t) {
            using T = decltype(t);
            if (op == HMC_REDUCE_SUM)
                return fold<T, T, double>(out, kept, red, 0.0, [](double a, T x) { return a + to_f64(x); },
                                          [](double a, int64_t) { return from_f64<T>(a); });
            if (op == HMC_REDUCE_PROD)
                return fold<T, T, double>(out, kept, red, 1.0, [](double a, T x) { return a * to_f64(x); },
                                          [](double a, int64_t) { return from_f64<T>(a); });
            return fold<T, T, double>(out, kept, red, 0.0, [](double a, T x) { return a + to_f64(x); },
                                      [](double a, int64_t n) { return from_f64<T>(a / (double)n); });
        });
    }
    if (op == HMC_REDUCE_SUM || op == HMC_REDUCE_PROD) {
        if (out->dtype != HMC_I64) return 2;
        return dispatch_all(dt, [&](auto t) {
            using T = decltype(t);
            if (op == HMC_REDUCE_SUM)
                return fold<T, int64_t, int64_t>(out, kept, red, 0, [](int64_t a, T x) { return wadd(a, to_i64(x)); },
                                                 [](int64_t a, int64_t) { return a; });
            return fold<T, int64_t, int64_t>(out, kept, red, 1, [](int64_t a, T x) { return wmul(a, to_i64(x)); },
                                             [](int64_t a, int64_t) { return a; });
        });
    }
    if (op == HMC_REDUCE_MEAN) return 2;
    if (op == HMC_REDUCE_MAX || op == HMC_REDUCE_MIN) {
        if (out->dtype != dt) return 2;
        int64_t count = 1;
        for (int d = 0; d < red->ndim; ++d) count *= red->sizes[d];
        int64_t nout = 1;
        for (int d = 0; d < kept->ndim; ++d) nout *= kept->sizes[d];
        if (count == 0 && nout > 0) return 2;  // "reduction over an empty dimension"
        const bool is_max = op == HMC_REDUCE_MAX;
        return dispatch_all(dt, [&](auto t) {
            using T = decltype(t);
            return fold<T, T, Opt<T>>(out, kept, red, Opt<T>{false, T{}},
                                      [=](Opt<T> a, T x) { return replaces(a, x, is_max) ? Opt<T>{true, x} : a; },
                                      [](Opt<T> a, int64_t) { return a.v; });
        });
    }
    if (op == HMC_REDUCE_ALL || op == HMC_REDUCE_ANY) {
        const bool all = op == HMC_REDUCE_ALL;
        return dispatch_all(dt, [&](auto t) {
            using T = decltype(t);
            auto step = [=](bool a, T x) { return all ? (a && to_bool(x)) : (a || to_bool(x)); };
            if (out->dtype == HMC_U8)
                return fold<T, uint8_t, bool>(out, kept, red, all, step, [](bool a, int64_t) { return (uint8_t)a; });
            if (out->dtype != HMC_BOOL) return 2;
            return fold<T, Bool, bool>(out, kept, red, all, step, [](bool a, int64_t) { return Bool{(uint8_t)a}; });
        });
    }
    return 2;
}

// cpu::var. src/backend/cpu/reduce.rs:133-170.
int orc_var(const hmc_tensor_desc *out, const hmc_tensor_desc *kept, const hmc_tensor_desc *red,
            double correction, int32_t take_sqrt) {
    if (out->dtype != kept->dtype) return 2;
    return dispatch_float(kept->dtype, [&](auto t) {
        using T = decltype(t);
        int64_t count = 1;
        for (int d = 0; d < red->ndim; ++d) count *= red->sizes[d];
        const double divisor = std::fmax((double)count - correction, 0.0);
        const T *ps = (const T *)kept->data;
        T *po = (T *)out->data;
        const int64_t *kst[1] = {kept->strides};
        const int64_t *rst[1] = {red->strides};
        int64_t o = out->offset;
        int64_t kbase[1] = {kept->offset};
        walk<1>(kept->ndim, kept->sizes, kst, kbase, [&](const int64_t *i) {
            double sum = 0.0;
            int64_t rbase[1] = {i[0]};
            walk<1>(red->ndim, red->sizes, rst, rbase, [&](const int64_t *j) { sum += to_f64(ps[j[0]]); });
            double mean = sum / (double)count;
            double sq = 0.0;
            walk<1>(red->ndim, red->sizes, rst, rbase, [&](const int64_t *j) {
                double d = to_f64(ps[j[0]]) - mean;
                sq += d * d;
            });
            double v = count == 0 ? std::numeric_limits<double>::quiet_NaN() : sq / divisor;
            po[o++] = from_f64<T>(take_sqrt ? std::sqrt(v) : v);
        });
        return 0;
    });
}

// cpu::arg_reduce. src/backend/cpu/reduce.rs:172-225. `red` has the one reduced dimension (ndim 0
// stands for a 0-dim source: one element, index 0).
int orc_arg_reduce(const hmc_tensor_desc *values, const hmc_tensor_desc *indices, const hmc_tensor_desc *kept,
                   const hmc_tensor_desc *red, int32_t is_max) {
    if (red->ndim > 1 || indices->dtype != HMC_I64 || (values && values->dtype != kept->dtype)) return 2;
    const int64_t n = red->ndim == 0 ? 1 : red->sizes[0];
    const int64_t stride = red->ndim == 0 ? 0 : red->strides[0];
    if (n <= 0) return 2;
    return dispatch_all(kept->dtype, [&](auto t) {
        using T = decltype(t);
        const T *ps = (const T *)kept->data;
        int64_t *pi = (int64_t *)indices->data;
        T *pv = values ? (T *)values->data : nullptr;
        const int64_t *kst[1] = {kept->strides};
        int64_t kbase[1] = {kept->offset};
        int64_t o = 0;
        walk<1>(kept->ndim, kept->sizes, kst, kbase, [&](const int64_t *i) {
            Opt<T> best{false, T{}};
            int64_t best_index = 0;
            for (int64_t k = 0; k < n; ++k) {
                T x = ps[i[0] + k * stride];
                if (replaces(best, x, is_max != 0)) { best = Opt<T>{true, x}; best_index = k; }
            }
            pi[indices->offset + o] = best_index;
            if (pv) pv[values->offset + o] = best.v;
            ++o;
        });
        return 0;
    });
}

// cpu::softmax. src/backend/cpu/misc.rs:13-51.
int orc_softmax(const hmc_tensor_desc *out_rows, const hmc_tensor_desc *src_rows, int64_t n, int64_t so,
                int64_t si, int32_t log) {
    if (out_rows->dtype != src_rows->dtype || !same_shape(out_rows, src_rows)) return 2;
    return dispatch_float(src_rows->dtype, [&](auto t) {
        using T = decltype(t);
        const T *ps = (const T *)src_rows->data;
        T *po = (T *)out_rows->data;
        const int64_t *st[2] = {out_rows->strides, src_rows->strides};
        int64_t base[2] = {out_rows->offset, src_rows->offset};
        walk<2>(out_rows->ndim, out_rows->sizes, st, base, [&](const int64_t *oi) {
            const int64_t o = oi[0], i = oi[1];
            auto x = [&](int64_t k) { return to_f64(ps[i + k * si]); };
            double mx = -std::numeric_limits<double>::infinity();
            for (int64_t k = 0; k < n; ++k) { double v = x(k); if (v > mx) mx = v; }
            double sum = 0.0;
            for (int64_t k = 0; k < n; ++k) sum += std::exp(x(k) - mx);
            double log_sum = std::log(sum);
            for (int64_t k = 0; k < n; ++k) {
                double v = log ? x(k) - mx - log_sum : std::exp(x(k) - mx) / sum;
                po[o + k * so] = from_f64<T>(v);
            }
        });
        return 0;
    });
}

// One AdamW step on one parameter as the sequence of CPU kernels homura's optimizer issues
// (decoupled weight decay, no amsgrad, no maximize). src/optim/adam.rs:125-171; the in-place
// writes are "compute, then copy into the target" (src/ops/binary.rs:568-587), which leaves the
// same bits as writing directly. `step` is the step count after the increment (1, 2, ...).
// All tensors are contiguous of n elements here; layouts are exercised through the single ops.
int orc_adamw_step(int32_t dtype, int64_t n, void *param, const void *grad, void *exp_avg, void *exp_avg_sq,
                   double lr, double beta1, double beta2, double eps, double weight_decay, double step) {
    auto desc = [&](void *p) {
        hmc_tensor_desc d{};
        d.data = p; d.dtype = dtype; d.ndim = 1; d.sizes[0] = n; d.strides[0] = 1;
        return d;
    };
    const size_t es = dtype == HMC_F64 ? 8 : dtype == HMC_F32 ? 4 : 2;
    std::vector<uint8_t> t1(n * es + 8), t2(n * es + 8);
    hmc_tensor_desc p = desc(param), g = desc((void *)grad), m = desc(exp_avg), v = desc(exp_avg_sq);
    hmc_tensor_desc tmp = desc(t1.data()), tmp2 = desc(t2.data());
    int rc = 0;
    auto bits_of = [&](double s) {  // Scalar::Float -> element bits, as cpu::fill converts.
        uint64_t b = 0;
        switch (dtype) {
            case HMC_F64: { b = f64_bits(s); break; }
            case HMC_F32: { b = f32_bits((float)s); break; }
            case HMC_F16: { b = f32_to_f16((float)s); break; }
            default: { b = f32_to_bf16((float)s); break; }
        }
        return b;
    };
    const bool half = dtype == HMC_F16 || dtype == HMC_BF16;
    // Mul/Div by a scalar: f16/bf16 keep the scalar in f32 (binary_scalar), others round it to
    // the dtype (binary_constant). src/ops/binary.rs:118-133.
    auto mul_scalar = [&](hmc_tensor_desc *o, hmc_tensor_desc *a, double s) {
        return half ? orc_binary_scalar(HMC_BINARY_MUL, o, a, s, 0) : orc_binary_constant(HMC_BINARY_MUL, o, a, bits_of(s), 0);
    };
    auto div_scalar = [&](hmc_tensor_desc *o, hmc_tensor_desc *a, double s) {
        return half ? orc_binary_scalar(HMC_BINARY_DIV, o, a, s, 0) : orc_binary_constant(HMC_BINARY_DIV, o, a, bits_of(s), 0);
    };
    if (weight_decay != 0.0) rc |= mul_scalar(&p, &p, 1.0 - lr * weight_decay);
    rc |= orc_fused(HMC_FUSED_LERP, &tmp, &m, &g, nullptr, 1.0 - beta1);
    rc |= orc_copy(&m, &tmp);
    rc |= mul_scalar(&v, &v, beta2);
    rc |= orc_fused(HMC_FUSED_ADDCMUL, &tmp, &v, &g, &g, 1.0 - beta2);
    rc |= orc_copy(&v, &tmp);
    const double bias_correction2 = 1.0 - std::pow(beta2, step);
    const double step_size = lr / (1.0 - std::pow(beta1, step));
    const double bias_correction2_sqrt = std::pow(bias_correction2, 0.5);
    rc |= orc_unary(HMC_UNARY_SQRT, &tmp, &v);
    rc |= div_scalar(&tmp2, &tmp, bias_correction2_sqrt);
    rc |= orc_binary_constant(HMC_BINARY_ADD, &tmp2, &tmp2, bits_of(eps), 0);
    rc |= orc_fused(HMC_FUSED_ADDCDIV, &tmp, &p, &m, &tmp2, -step_size);
    rc |= orc_copy(&p, &tmp);
    return rc;
}

// ---- random sampling (src/ops/random.rs) ----

// One Philox4x32-10 block. src/ops/random.rs:29-51.
void orc_philox(const uint32_t counter[4], const uint32_t key[2], uint32_t out[4]) {
    const uint64_t M0 = 0xD2511F53ull, M1 = 0xCD9E8D57ull;
    const uint32_t W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
    uint32_t c[4] = {counter[0], counter[1], counter[2], counter[3]};
    uint32_t k[2] = {key[0], key[1]};
    for (int round = 0; round < 10; ++round) {
        if (round > 0) { k[0] += W0; k[1] += W1; }
        const uint64_t p0 = M0 * c[0], p1 = M1 * c[2];
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k[0], n1 = (uint32_t)p1;
        const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k[1], n3 = (uint32_t)p0;
        c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    }
    for (int i = 0; i < 4; ++i) out[i] = c[i];
}

}  // extern "C"

namespace {
// Block n of a generator seeded with `seed` (reserve, src/ops/random.rs:75-83).
void block_of(uint64_t seed, uint64_t n, uint32_t out[4]) {
    const uint32_t counter[4] = {(uint32_t)n, (uint32_t)(n >> 32), 0, 0};
    const uint32_t key[2] = {(uint32_t)seed, (uint32_t)(seed >> 32)};
    orc_philox(counter, key, out);
}
// src/ops/random.rs:86-95.
double unit_f64(uint32_t hi, uint32_t lo) {
    const uint64_t bits = ((uint64_t)hi << 21) ^ ((uint64_t)lo >> 11);
    return (double)bits * (1.0 / 9007199254740992.0);
}
double unit_bits(uint32_t x, int bits) { return (double)(x >> (32 - bits)) / (double)(1ull << bits); }
int float_digits(int dtype) { return dtype == HMC_F16 ? 11 : dtype == HMC_BF16 ? 8 : dtype == HMC_F32 ? 24 : 53; }
}  // namespace

extern "C" {

// sample_float's Uniform arm and the conversion of random_tensor: n values of a float dtype into the flat
// `out`, from block `offset` on. src/ops/random.rs:162-183, 262-281.
int orc_random_uniform(int32_t dtype, void *out, int64_t n, uint64_t seed, uint64_t offset, double from, double to) {
    return dispatch_float(dtype, [&](auto t) {
        using T = decltype(t);
        T *po = (T *)out;
        const int per_block = dtype == HMC_F64 ? 2 : 4;
        const int bits = float_digits(dtype);
        for (int64_t i = 0; i < n; ++i) {
            uint32_t b[4];
            block_of(seed, offset + (uint64_t)(i / per_block), b);
            const int j = (int)(i % per_block);
            const double u = per_block == 2 ? unit_f64(b[2 * j], b[2 * j + 1]) : unit_bits(b[j], bits);
            const double x = from + u * (to - from);
            T v = from_f64<T>(x);
            if (from < to && to_f64(v) >= to) v = from_f64<T>(from);
            po[i] = v;
        }
        return 0;
    });
}

// sample_float's Normal arm. src/ops/random.rs:184-197.
int orc_random_normal(int32_t dtype, void *out, int64_t n, uint64_t seed, uint64_t offset, double mean, double std_) {
    return dispatch_float(dtype, [&](auto t) {
        using T = decltype(t);
        T *po = (T *)out;
        for (int64_t i = 0; i < n; i += 2) {
            uint32_t b[4];
            block_of(seed, offset + (uint64_t)(i / 2), b);
            const double u1 = 1.0 - unit_f64(b[0], b[1]);
            const double u2 = unit_f64(b[2], b[3]);
            const double r = std::sqrt(-2.0 * std::log(u1));
            const double theta = 2.0 * 3.14159265358979323846 * u2;
            po[i] = from_f64<T>(mean + std_ * r * std::cos(theta));
            if (i + 1 < n) po[i + 1] = from_f64<T>(mean + std_ * r * std::sin(theta));
        }
        return 0;
    });
}

// One batch of sample_int (src/ops/random.rs:213-238): the words of `blocks` blocks from `offset` on, in the
// order the CPU pops them ([w0 w1], then [w2 w3] of each block); words >= threshold become
// low + word % range and fill out[0 .. nout); returns how many words of the batch were >= threshold.
int64_t orc_random_int_batch(int64_t *out, int64_t nout, uint64_t seed, uint64_t offset, uint64_t blocks, int64_t low,
                             uint64_t range, uint64_t threshold) {
    int64_t accepted = 0;
    for (uint64_t i = 0; i < blocks; ++i) {
        uint32_t b[4];
        block_of(seed, offset + i, b);
        const uint64_t w[2] = {((uint64_t)b[0] << 32) | b[1], ((uint64_t)b[2] << 32) | b[3]};
        for (int j = 0; j < 2; ++j) {
            if (w[j] >= threshold) {
                if (accepted < nout) out[accepted] = (int64_t)((uint64_t)low + w[j] % range);
                accepted += 1;
            }
        }
    }
    return accepted;
}

// The whole of sample_int: batches until n values are there; *blocks_used gets the blocks reserved.
// src/ops/random.rs:213-238 (and int_range, :201-207, for range and threshold).
int orc_random_int(int64_t *out, int64_t n, uint64_t seed, uint64_t offset, int64_t low, int64_t high, uint64_t *blocks_used) {
    const uint64_t range = (uint64_t)high - (uint64_t)low;
    const uint64_t threshold = (0 - range) % range;
    int64_t done = 0;
    uint64_t used = 0;
    while (done < n) {
        const int64_t needed = n - done;
        const uint64_t blocks = (uint64_t)((needed + 1) / 2);
        const int64_t got = orc_random_int_batch(out + done, needed, seed, offset + used, blocks, low, range, threshold);
        used += blocks;
        done += got < needed ? got : needed;
    }
    if (blocks_used) *blocks_used = used;
    return 0;
}

// cpu::triangle. src/backend/cpu/misc.rs:347-381.
int orc_triangle(const hmc_tensor_desc *out, const hmc_tensor_desc *src, int64_t diagonal, int32_t upper) {
    if (out->dtype != src->dtype || !same_shape(out, src) || src->ndim < 2) return 2;
    const int nd = src->ndim;
    const int64_t rows = src->sizes[nd - 2], cols = src->sizes[nd - 1];
    return dispatch_all(src->dtype, [&](auto t) {
        using T = decltype(t);
        const T *ps = (const T *)src->data;
        T *po = (T *)out->data;
        const int64_t *st[2] = {out->strides, src->strides};
        int64_t base[2] = {out->offset, src->offset};
        walk<2>(nd - 2, src->sizes, st, base, [&](const int64_t *oi) {
            for (int64_t r = 0; r < rows; ++r) {
                for (int64_t c = 0; c < cols; ++c) {
                    const int64_t d = c - r;
                    const bool keep = upper ? d >= diagonal : d <= diagonal;
                    T zero{};
                    po[oi[0] + r * out->strides[nd - 2] + c * out->strides[nd - 1]] =
                        keep ? ps[oi[1] + r * src->strides[nd - 2] + c * src->strides[nd - 1]] : zero;
                }
            }
        });
        return 0;
    });
}

// cpu::flip, given like the device entry point: src's strides are negative along the flipped dimensions and
// its offset is at the element that comes first. src/backend/cpu/misc.rs:384-411.
int orc_flip(const hmc_tensor_desc *out, const hmc_tensor_desc *src) {
    if (out->dtype != src->dtype || !same_shape(out, src)) return 2;
    return dispatch_all(src->dtype, [&](auto t) {
        using T = decltype(t);
        const T *ps = (const T *)src->data;
        T *po = (T *)out->data;
        const int64_t *st[2] = {out->strides, src->strides};
        int64_t base[2] = {out->offset, src->offset};
        walk<2>(src->ndim, src->sizes, st, base, [&](const int64_t *oi) { po[oi[0]] = ps[oi[1]]; });
        return 0;
    });
}

// cpu::addr with the steps of FloatOuter / IntOuter / BoolOuter; the operands are given like the device entry point
// (all four as [n, m] views, v1 and v2 broadcast). src/backend/cpu/linalg.rs:227-410.
int orc_addr(const hmc_tensor_desc *out, const hmc_tensor_desc *v1, const hmc_tensor_desc *v2, const hmc_tensor_desc *input,
             double alpha, double beta, int64_t alpha_int, int64_t beta_int) {
    const int dt = out->dtype;
    if (v1->dtype != dt || v2->dtype != dt || (input && input->dtype != dt)) return 2;
    if (is_float(dt)) {
        return dispatch_float(dt, [&](auto t) {
            using T = decltype(t);
            using C = typename Comp<T>::C;
            const C a = (C)alpha, b = (C)beta;
            auto row = [=](T x) { return a == (C)1 ? x : down<T>(up(x) * a); };
            if (b == (C)0) return map2<T, T, T>(out, v1, v2, [=](T x, T y) { return down<T>(up(row(x)) * up(y)); });
            if (!input) return 2;
            return map3<T, T, T, T>(out, v1, v2, input, [=](T x, T y, T c) {
                const T p = down<T>(up(row(x)) * up(y));
                const T cc = b == (C)1 ? c : down<T>(up(c) * b);
                return down<T>(up(cc) + up(p));
            });
        });
    }
    if (dt == HMC_BOOL) {
        const bool a = alpha_int != 0;
        if (beta_int == 0) return map2<Bool, Bool, Bool>(out, v1, v2, [=](Bool x, Bool y) { return Bool{(uint8_t)(x.b && a && y.b)}; });
        if (!input) return 2;
        return map3<Bool, Bool, Bool, Bool>(out, v1, v2, input,
                                            [=](Bool x, Bool y, Bool c) { return Bool{(uint8_t)(c.b || (x.b && a && y.b))}; });
    }
    return dispatch_int(dt, [&](auto t) {
        using T = decltype(t);
        auto product = [=](T x, T y) {
            uint64_t p = (uint64_t)(int64_t)x * (uint64_t)(int64_t)y;
            return alpha_int == 1 ? p : p * (uint64_t)alpha_int;
        };
        if (beta_int == 0) return map2<T, T, T>(out, v1, v2, [=](T x, T y) { return (T)(int64_t)product(x, y); });
        if (!input) return 2;
        return map3<T, T, T, T>(out, v1, v2, input, [=](T x, T y, T c) {
            const uint64_t cc = beta_int == 1 ? (uint64_t)(int64_t)c : (uint64_t)(int64_t)c * (uint64_t)beta_int;
            return (T)(int64_t)(cc + product(x, y));
        });
    });
}

// cpu::exclusive_cumprod on lines given as for orc_softmax. src/backend/cpu/reduce.rs:228-329.
int orc_exclusive_cumprod(const hmc_tensor_desc *out_lines, const hmc_tensor_desc *src_lines, int64_t n, int64_t so, int64_t si,
                          int32_t reverse) {
    if (out_lines->dtype != src_lines->dtype || !same_shape(out_lines, src_lines)) return 2;
    return dispatch_float(src_lines->dtype, [&](auto t) {
        using T = decltype(t);
        const T *ps = (const T *)src_lines->data;
        T *po = (T *)out_lines->data;
        const int64_t *st[2] = {out_lines->strides, src_lines->strides};
        int64_t base[2] = {out_lines->offset, src_lines->offset};
        walk<2>(out_lines->ndim, out_lines->sizes, st, base, [&](const int64_t *oi) {
            if constexpr (std::is_same_v<T, F16> || std::is_same_v<T, BF16>) {
                float acc = 1.0f;
                for (int64_t k = 0; k < n; ++k) {
                    const int64_t at = reverse ? n - 1 - k : k;
                    const T x = ps[oi[1] + at * si];
                    po[oi[0] + at * so] = down<T>(acc);
                    acc = acc * up(x);
                }
            } else {
                double acc = 1.0;
                for (int64_t k = 0; k < n; ++k) {
                    const int64_t at = reverse ? n - 1 - k : k;
                    const T x = ps[oi[1] + at * si];
                    po[oi[0] + at * so] = from_f64<T>(acc);
                    acc = acc * to_f64(x);
                }
            }
        });
        return 0;
    });
}

// ---- gathers (src/backend/cpu/misc.rs) ----
static inline int64_t index_value(const hmc_tensor_desc *index, int64_t at) {
    return index->dtype == HMC_I32 ? (int64_t)((const int32_t *)index->data)[at] : ((const int64_t *)index->data)[at];
}

// The first index element, in row-major order, outside [low, high) and not the exempt value: slot[0] its position
// (UINT64_MAX for none), slot[1] its value. What `positions` (src/backend/cpu/misc.rs:30-75) reports in its panic.
int orc_index_check(const hmc_tensor_desc *index, int64_t low, int64_t high, int32_t has_exempt, int64_t exempt, uint64_t *slot) {
    if (index->dtype != HMC_I32 && index->dtype != HMC_I64) return 2;
    slot[0] = ~0ull;
    slot[1] = 0;
    const int64_t *st[1] = {index->strides};
    int64_t base[1] = {index->offset};
    uint64_t position = 0;
    walk<1>(index->ndim, index->sizes, st, base, [&](const int64_t *o) {
        const int64_t v = index_value(index, o[0]);
        const bool bad = (v < low || v >= high) && !(has_exempt && v == exempt);
        if (bad && slot[0] == ~0ull) { slot[0] = position; slot[1] = (uint64_t)v; }
        position += 1;
    });
    return 0;
}

// cpu::index_select, operands given like the device entry point. src/backend/cpu/misc.rs:77-103.
int orc_index_select(const hmc_tensor_desc *out, const hmc_tensor_desc *src, const hmc_tensor_desc *index, int32_t dim,
                     int32_t wrap_negative) {
    if (out->dtype != src->dtype || out->ndim != src->ndim || dim < 0 || dim >= out->ndim) return 2;
    const int64_t size = src->sizes[dim];
    const int64_t istride = index->ndim == 0 ? 0 : index->strides[0];
    return dispatch_all(src->dtype, [&](auto t) {
        using T = decltype(t);
        const T *ps = (const T *)src->data;
        T *po = (T *)out->data;
        // walk out with src's strides, the stride along dim set to 0, and a counter along dim for the index
        hmc_tensor_desc walk_src = *src, counter = *out;
        walk_src.strides[dim] = 0;
        for (int k = 0; k < out->ndim; ++k) counter.strides[k] = k == dim ? 1 : 0;
        const int64_t *st[3] = {out->strides, walk_src.strides, counter.strides};
        int64_t base[3] = {out->offset, src->offset, 0};
        walk<3>(out->ndim, out->sizes, st, base, [&](const int64_t *o) {
            int64_t j = index_value(index, index->offset + o[2] * istride);
            if (wrap_negative && j < 0) j += size;
            po[o[0]] = ps[o[1] + j * src->strides[dim]];
        });
        return 0;
    });
}

// cpu::gather. src/backend/cpu/misc.rs:319-342.
int orc_gather(const hmc_tensor_desc *out, const hmc_tensor_desc *src, const hmc_tensor_desc *index, int32_t dim) {
    if (out->dtype != src->dtype || out->ndim != src->ndim || out->ndim != index->ndim || dim < 0 || dim >= out->ndim) return 2;
    return dispatch_all(src->dtype, [&](auto t) {
        using T = decltype(t);
        const T *ps = (const T *)src->data;
        T *po = (T *)out->data;
        hmc_tensor_desc walk_src = *src;
        walk_src.strides[dim] = 0;
        const int64_t *st[3] = {out->strides, walk_src.strides, index->strides};
        int64_t base[3] = {out->offset, src->offset, index->offset};
        walk<3>(out->ndim, out->sizes, st, base, [&](const int64_t *o) {
            po[o[0]] = ps[o[1] + index_value(index, o[2]) * src->strides[dim]];
        });
        return 0;
    });
}

// cpu::index_overwrite: slice i of src goes to slice positions[i] of out, in order (the last of repeated positions
// wins). src/backend/cpu/misc.rs:105-125.
int orc_index_overwrite(const hmc_tensor_desc *out, const hmc_tensor_desc *src, const hmc_tensor_desc *positions, int32_t dim) {
    if (out->dtype != src->dtype || out->ndim != src->ndim || dim < 0 || dim >= out->ndim || positions->dtype != HMC_I64) return 2;
    return dispatch_all(src->dtype, [&](auto t) {
        using T = decltype(t);
        const T *ps = (const T *)src->data;
        T *po = (T *)out->data;
        const int64_t *pp = (const int64_t *)positions->data + positions->offset;
        // walk src in row-major order (slices in order of i); out's stride along dim is applied through the position
        hmc_tensor_desc walk_out = *out, counter = *src;
        walk_out.strides[dim] = 0;
        for (int k = 0; k < src->ndim; ++k) counter.strides[k] = k == dim ? 1 : 0;
        const int64_t *st[3] = {src->strides, walk_out.strides, counter.strides};
        int64_t base[3] = {src->offset, out->offset, 0};
        // row-major order visits, for every outer coordinate, the slices in order of i: a later i overwrites an earlier one
        walk<3>(src->ndim, src->sizes, st, base, [&](const int64_t *o) { po[o[1] + pp[o[2]] * out->strides[dim]] = ps[o[0]]; });
        return 0;
    });
}

}  // extern "C"

// add_at (src/backend/cpu/misc.rs:219-256): every element of the contiguous out goes to f64 (floats) or i64 (integers,
// wrapping; a Bool is the or), takes its contributions in order, and is rounded once. `each` calls back with
// (offset into out counted from its first element, storage offset of src) per contribution, in the CPU's order.
template <class T, class Each> static void add_at(T *po, int64_t n, const T *ps, Each &&each) {
    if constexpr (Tr<T>::kind == kFloat) {
        std::vector<double> acc(n);
        for (int64_t k = 0; k < n; ++k) acc[k] = to_f64(po[k]);
        each([&](int64_t o, int64_t s) { acc[o] += to_f64(ps[s]); });
        for (int64_t k = 0; k < n; ++k) po[k] = from_f64<T>(acc[k]);
    } else {
        std::vector<int64_t> acc(n);
        for (int64_t k = 0; k < n; ++k) acc[k] = to_i64(po[k]);
        each([&](int64_t o, int64_t s) { acc[o] = (int64_t)((uint64_t)acc[o] + (uint64_t)to_i64(ps[s])); });
        for (int64_t k = 0; k < n; ++k) po[k] = from_i64<T>(acc[k]);
    }
}

static int64_t span_of(const hmc_tensor_desc *d) {
    int64_t n = 1;
    for (int k = 0; k < d->ndim; ++k) {
        if (d->sizes[k] == 0) return 0;
        n += (d->sizes[k] - 1) * d->strides[k];
    }
    return n;
}

extern "C" {

// cpu::index_add: slice i of src along dim is added into slice index[i] of out (negative positions count from the
// end). src/backend/cpu/misc.rs:258-293.
int orc_index_add(const hmc_tensor_desc *out, const hmc_tensor_desc *src, const hmc_tensor_desc *index, int32_t dim) {
    if (out->dtype != src->dtype || out->ndim != src->ndim || dim < 0 || dim >= out->ndim || index->dtype != HMC_I64) return 2;
    const int64_t size = out->sizes[dim];
    return dispatch_all(src->dtype, [&](auto t) {
        using T = decltype(t);
        const int64_t *pi = (const int64_t *)index->data + index->offset;
        hmc_tensor_desc walk_out = *out, counter = *src;
        walk_out.strides[dim] = 0;
        for (int k = 0; k < src->ndim; ++k) counter.strides[k] = k == dim ? 1 : 0;
        const int64_t *st[3] = {src->strides, walk_out.strides, counter.strides};
        int64_t base[3] = {src->offset, 0, 0};
        // row-major order over src visits, for every other coordinate, the slices in order of i
        add_at<T>((T *)out->data + out->offset, span_of(out), (const T *)src->data, [&](auto add) {
            walk<3>(src->ndim, src->sizes, st, base, [&](const int64_t *o) {
                int64_t j = pi[o[2] * index->strides[0]];
                if (j < 0) j += size;
                add(o[1] + j * out->strides[dim], o[0]);
            });
        });
        return 0;
    });
}

// cpu::scatter_add: out[.., index[p], ..] += src[p] for every position p of the index, in row-major order.
// src/backend/cpu/misc.rs:295-317.
int orc_scatter_add(const hmc_tensor_desc *out, const hmc_tensor_desc *src, const hmc_tensor_desc *index, int32_t dim) {
    if (out->dtype != src->dtype || out->ndim != src->ndim || out->ndim != index->ndim || dim < 0 || dim >= out->ndim ||
        index->dtype != HMC_I64) {
        return 2;
    }
    return dispatch_all(src->dtype, [&](auto t) {
        using T = decltype(t);
        const int64_t *pi = (const int64_t *)index->data;
        hmc_tensor_desc walk_out = *out;
        walk_out.strides[dim] = 0;
        const int64_t *st[3] = {index->strides, walk_out.strides, src->strides};
        int64_t base[3] = {index->offset, 0, src->offset};
        add_at<T>((T *)out->data + out->offset, span_of(out), (const T *)src->data, [&](auto add) {
            walk<3>(index->ndim, index->sizes, st, base, [&](const int64_t *o) { add(o[1] + pi[o[0]] * out->strides[dim], o[2]); });
        });
        return 0;
    });
}

// One indexed dimension of cpu::index_positions: out = (first) or += wrapped coordinate * stride.
// src/backend/cpu/misc.rs:154-204.
int orc_index_positions(const hmc_tensor_desc *out, const hmc_tensor_desc *coord, int64_t size, int64_t stride, int32_t first) {
    if (out->dtype != HMC_I64 || coord->dtype != HMC_I64 || out->ndim != coord->ndim) return 2;
    int64_t *po = (int64_t *)out->data;
    const int64_t *pc = (const int64_t *)coord->data;
    const int64_t *st[2] = {out->strides, coord->strides};
    int64_t base[2] = {out->offset, coord->offset};
    walk<2>(out->ndim, out->sizes, st, base, [&](const int64_t *o) {
        const int64_t v = pc[o[1]] < 0 ? pc[o[1]] + size : pc[o[1]];
        po[o[0]] = (first ? 0 : po[o[0]]) + v * stride;
    });
    return 0;
}

// cpu::mask_coordinates: the number of true elements, and coordinate d of the k-th one (row-major) in out[d * count + k].
// src/backend/cpu/misc.rs:127-151.
int64_t orc_mask_count(const hmc_tensor_desc *mask) {
    if (mask->dtype != HMC_BOOL) return -1;
    int64_t count = 0;
    const int64_t *st[1] = {mask->strides};
    int64_t base[1] = {mask->offset};
    walk<1>(mask->ndim, mask->sizes, st, base, [&](const int64_t *o) { count += ((const uint8_t *)mask->data)[o[0]] != 0; });
    return count;
}
int orc_mask_coordinates(const hmc_tensor_desc *mask, int64_t *out, int64_t count) {
    if (mask->dtype != HMC_BOOL) return 2;
    int64_t index[HMC_MAX_DIMS] = {0};
    int64_t k = 0;
    const int64_t *st[1] = {mask->strides};
    int64_t base[1] = {mask->offset};
    walk<1>(mask->ndim, mask->sizes, st, base, [&](const int64_t *o) {
        if (((const uint8_t *)mask->data)[o[0]] != 0) {
            for (int d = 0; d < mask->ndim; ++d) out[d * count + k] = index[d];
            k += 1;
        }
        for (int d = mask->ndim - 1; d >= 0; --d) {
            index[d] += 1;
            if (index[d] < mask->sizes[d]) break;
            index[d] = 0;
        }
    });
    return 0;
}

// Scalar conversions exposed for the tests of the cast tables (src/dtype.rs:543-665).
uint16_t orc_f32_to_f16(float f) { return f32_to_f16(f); }
uint16_t orc_f32_to_bf16(float f) { return f32_to_bf16(f); }
float orc_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
float orc_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }
double orc_erf(double x) { return erf_f64(x); }

}  // extern "C"
