// Element types of the ten dtypes and the conversions between them, bit for bit those of homura's
// Element::to_element (src/dtype.rs:144-273): a float source goes through f64, an integer source
// through i64, a bool source is 0/1; half types are always rounded through f32 to nearest even;
// float -> integer truncates toward zero, saturates to i64 (NaN is 0) and then wraps; a NaN that
// is narrowed keeps the top of its payload and is made quiet.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdint>
#include <type_traits>

#include "../../include/homura_cuda.h"

namespace hmc {

struct Bool { uint8_t b; };
struct F16 { uint16_t b; };
struct BF16 { uint16_t b; };

enum Kind { kBool, kInt, kFloat };

template <class T> struct Tr;
#define HMC_TRAIT(T, CODE, KIND) \
    template <> struct Tr<T> { static constexpr int code = CODE; static constexpr Kind kind = KIND; };
HMC_TRAIT(Bool, HMC_BOOL, kBool)
HMC_TRAIT(uint8_t, HMC_U8, kInt)
HMC_TRAIT(int8_t, HMC_I8, kInt)
HMC_TRAIT(int16_t, HMC_I16, kInt)
HMC_TRAIT(int32_t, HMC_I32, kInt)
HMC_TRAIT(int64_t, HMC_I64, kInt)
HMC_TRAIT(F16, HMC_F16, kFloat)
HMC_TRAIT(BF16, HMC_BF16, kFloat)
HMC_TRAIT(float, HMC_F32, kFloat)
HMC_TRAIT(double, HMC_F64, kFloat)
#undef HMC_TRAIT

__host__ __device__ inline int element_size(int dtype) {
    switch (dtype) {
        case HMC_BOOL: case HMC_U8: case HMC_I8: return 1;
        case HMC_I16: case HMC_F16: case HMC_BF16: return 2;
        case HMC_I32: case HMC_F32: return 4;
        default: return 8;
    }
}
inline bool dtype_valid(int dtype) { return dtype >= HMC_BOOL && dtype <= HMC_F64; }
inline bool dtype_is_float(int dtype) { return dtype >= HMC_F16 && dtype <= HMC_F64; }
inline bool dtype_is_int(int dtype) { return dtype >= HMC_U8 && dtype <= HMC_I64; }

// ---- f32 <-> half types ----
__device__ __forceinline__ float f16_to_f32(uint16_t h) {
    // Exact. The hardware conversion turns every NaN into the canonical one, `half` keeps the sign and
    // payload and sets the quiet bit, so NaNs are widened by hand.
    if ((h & 0x7FFFu) > 0x7C00u) {
        return __uint_as_float((static_cast<uint32_t>(h & 0x8000u) << 16) | 0x7FC00000u |
                               (static_cast<uint32_t>(h & 0x03FFu) << 13));
    }
    return __half2float(__ushort_as_half(h));
}
__device__ __forceinline__ uint16_t f32_to_f16(float f) {
    uint32_t x = __float_as_uint(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) {
        // NaN: sign, all-ones exponent, quiet bit, top ten payload bits.
        return static_cast<uint16_t>(((x >> 16) & 0x8000u) | 0x7E00u | ((x >> 13) & 0x03FFu));
    }
    return __half_as_ushort(__float2half_rn(f));
}
__device__ __forceinline__ float bf16_to_f32(uint16_t h) { return __uint_as_float(static_cast<uint32_t>(h) << 16); }
// The widening used by casts: a NaN comes out quiet, as it does from `half`'s to_f32.
__device__ __forceinline__ float bf16_to_f32_quiet(uint16_t h) {
    uint32_t x = static_cast<uint32_t>(h) << 16;
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) x |= 0x00400000u;
    return __uint_as_float(x);
}
__device__ __forceinline__ uint16_t f32_to_bf16(float f) {
    uint32_t x = __float_as_uint(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return static_cast<uint16_t>((x >> 16) | 0x0040u);
    // Round to nearest even on the 16 dropped bits.
    return static_cast<uint16_t>((x + 0x7FFFu + ((x >> 16) & 1u)) >> 16);
}

// ---- to f64 / i64 / bool ----
template <class T> __device__ __forceinline__ double to_f64(T v) { return static_cast<double>(v); }
template <> __device__ __forceinline__ double to_f64(F16 v) { return static_cast<double>(f16_to_f32(v.b)); }
template <> __device__ __forceinline__ double to_f64(BF16 v) { return static_cast<double>(bf16_to_f32_quiet(v.b)); }
template <> __device__ __forceinline__ double to_f64(Bool v) { return v.b ? 1.0 : 0.0; }

// Rust's `as i64`: toward zero, saturating, NaN -> 0. The hardware conversion saturates the same way but
// turns a NaN into i64::MIN.
__device__ __forceinline__ int64_t f64_as_i64(double v) { return v != v ? 0 : __double2ll_rz(v); }
__device__ __forceinline__ int64_t f32_as_i64(float v) { return v != v ? 0 : __float2ll_rz(v); }

template <class T> __device__ __forceinline__ int64_t to_i64(T v) { return static_cast<int64_t>(v); }
template <> __device__ __forceinline__ int64_t to_i64(float v) { return f32_as_i64(v); }
template <> __device__ __forceinline__ int64_t to_i64(double v) { return f64_as_i64(v); }
template <> __device__ __forceinline__ int64_t to_i64(F16 v) { return f32_as_i64(f16_to_f32(v.b)); }
template <> __device__ __forceinline__ int64_t to_i64(BF16 v) { return f32_as_i64(bf16_to_f32(v.b)); }
template <> __device__ __forceinline__ int64_t to_i64(Bool v) { return v.b ? 1 : 0; }

template <class T> __device__ __forceinline__ bool to_bool(T v) { return v != 0; }
template <> __device__ __forceinline__ bool to_bool(F16 v) { return (v.b & 0x7FFFu) != 0; }
template <> __device__ __forceinline__ bool to_bool(BF16 v) { return (v.b & 0x7FFFu) != 0; }
template <> __device__ __forceinline__ bool to_bool(Bool v) { return v.b != 0; }

// ---- from f64 / i64 / bool ----
template <class T> __device__ __forceinline__ T wrap_int(int64_t v) {
    return static_cast<T>(static_cast<std::make_unsigned_t<T>>(static_cast<uint64_t>(v)));
}
// f64 -> f32, round to nearest even; a NaN keeps the top 23 payload bits and the sign and becomes
// quiet (what x86's cvtsd2ss gives homura's CPU backend).
__device__ __forceinline__ float f64_to_f32(double v) {
    if (v != v) {
        uint64_t b = static_cast<uint64_t>(__double_as_longlong(v));
        uint32_t x = static_cast<uint32_t>((b >> 32) & 0x80000000u) | 0x7FC00000u |
                     static_cast<uint32_t>((b >> 29) & 0x003FFFFFu);
        return __uint_as_float(x);
    }
    return __double2float_rn(v);
}

template <class T> __device__ __forceinline__ T from_f64(double v) { return wrap_int<T>(f64_as_i64(v)); }
template <> __device__ __forceinline__ float from_f64(double v) { return f64_to_f32(v); }
template <> __device__ __forceinline__ double from_f64(double v) { return v; }
template <> __device__ __forceinline__ F16 from_f64(double v) { return F16{f32_to_f16(f64_to_f32(v))}; }
template <> __device__ __forceinline__ BF16 from_f64(double v) { return BF16{f32_to_bf16(f64_to_f32(v))}; }
template <> __device__ __forceinline__ Bool from_f64(double v) { return Bool{static_cast<uint8_t>(v != 0.0)}; }

template <class T> __device__ __forceinline__ T from_i64(int64_t v) { return wrap_int<T>(v); }
template <> __device__ __forceinline__ float from_i64(int64_t v) { return __ll2float_rn(v); }
template <> __device__ __forceinline__ double from_i64(int64_t v) { return __ll2double_rn(v); }
template <> __device__ __forceinline__ F16 from_i64(int64_t v) { return F16{f32_to_f16(__ll2float_rn(v))}; }
template <> __device__ __forceinline__ BF16 from_i64(int64_t v) { return BF16{f32_to_bf16(__ll2float_rn(v))}; }
template <> __device__ __forceinline__ Bool from_i64(int64_t v) { return Bool{static_cast<uint8_t>(v != 0)}; }

template <class T> __device__ __forceinline__ T from_bool(bool v) { return static_cast<T>(v ? 1 : 0); }
template <> __device__ __forceinline__ F16 from_bool(bool v) { return F16{static_cast<uint16_t>(v ? 0x3C00 : 0)}; }
template <> __device__ __forceinline__ BF16 from_bool(bool v) { return BF16{static_cast<uint16_t>(v ? 0x3F80 : 0)}; }
template <> __device__ __forceinline__ Bool from_bool(bool v) { return Bool{static_cast<uint8_t>(v)}; }

// Element::to_element.
template <class D, class S> __device__ __forceinline__ D convert(S x) {
    if constexpr (std::is_same_v<D, S>) {
        return x;
    } else if constexpr (Tr<S>::kind == kFloat) {
        // The fast lanes below give the bits of the f64 route: widening is exact, and a value that
        // is already an f32 is rounded to a half type exactly once either way.
        if constexpr (std::is_same_v<D, float> && std::is_same_v<S, F16>) return f16_to_f32(x.b);
        else if constexpr (std::is_same_v<D, float> && std::is_same_v<S, BF16>) return bf16_to_f32_quiet(x.b);
        else if constexpr (std::is_same_v<D, F16> && std::is_same_v<S, float>) return F16{f32_to_f16(x)};
        else if constexpr (std::is_same_v<D, BF16> && std::is_same_v<S, float>) return BF16{f32_to_bf16(x)};
        else if constexpr (std::is_same_v<D, F16> && std::is_same_v<S, BF16>) return F16{f32_to_f16(bf16_to_f32_quiet(x.b))};
        else if constexpr (std::is_same_v<D, BF16> && std::is_same_v<S, F16>) return BF16{f32_to_bf16(f16_to_f32(x.b))};
        else return from_f64<D>(to_f64(x));
    } else if constexpr (Tr<S>::kind == kInt) {
        return from_i64<D>(to_i64(x));
    } else {
        return from_bool<D>(to_bool(x));
    }
}

// The computation type of a float dtype (FloatElement::C, src/backend/cpu/num.rs:55-107).
template <class T> struct Comp { using C = float; };
template <> struct Comp<double> { using C = double; };

// Widening and rounding around arithmetic use the hardware conversions: exact widening, round to nearest
// even. They differ from the cast routines above only in the sign and payload of a NaN (the hardware
// produces its canonical NaN), which no arithmetic result is compared on.
__device__ __forceinline__ float up(float v) { return v; }
__device__ __forceinline__ double up(double v) { return v; }
__device__ __forceinline__ float up(F16 v) { return __half2float(__ushort_as_half(v.b)); }
__device__ __forceinline__ float up(BF16 v) { return bf16_to_f32(v.b); }

template <class T> __device__ __forceinline__ T down(typename Comp<T>::C c);
template <> __device__ __forceinline__ float down<float>(float c) { return c; }
template <> __device__ __forceinline__ double down<double>(double c) { return c; }
template <> __device__ __forceinline__ F16 down<F16>(float c) { return F16{__half_as_ushort(__float2half_rn(c))}; }
template <> __device__ __forceinline__ BF16 down<BF16>(float c) {
    return BF16{__bfloat16_as_ushort(__float2bfloat16_rn(c))};
}

// Two results rounded with one packed conversion.
__device__ __forceinline__ void down2(F16 &lo, F16 &hi, float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    lo.b = __half_as_ushort(__low2half(h));
    hi.b = __half_as_ushort(__high2half(h));
}
__device__ __forceinline__ void down2(BF16 &lo, BF16 &hi, float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    lo.b = __bfloat16_as_ushort(__low2bfloat16(h));
    hi.b = __bfloat16_as_ushort(__high2bfloat16(h));
}

// Host-side dispatch of a dtype code to a type tag.
template <class F> inline hmc_status dispatch_all(int dtype, F &&f) {
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
    return HMC_INVALID;
}
template <class F> inline hmc_status dispatch_float(int dtype, F &&f) {
    switch (dtype) {
        case HMC_F16: return f(F16{});
        case HMC_BF16: return f(BF16{});
        case HMC_F32: return f(float{});
        case HMC_F64: return f(double{});
    }
    return HMC_INVALID;
}
template <class F> inline hmc_status dispatch_int(int dtype, F &&f) {
    switch (dtype) {
        case HMC_U8: return f(uint8_t{});
        case HMC_I8: return f(int8_t{});
        case HMC_I16: return f(int16_t{});
        case HMC_I32: return f(int32_t{});
        case HMC_I64: return f(int64_t{});
    }
    return HMC_INVALID;
}

}  // namespace hmc
