// Single-precision transcendentals with the bits of the host C library.
//
// homura's CPU backend evaluates F16/BF16/F32 tensors in f32 and calls Rust's f32::exp, ln, ln_1p, tanh and
// powf, which are the C library's expf, logf, log1pf, tanhf and powf (src/backend/cpu/mod.rs:378-402, 459).
// On the hosts this backend is built for that library is glibc 2.39 on x86-64 with FMA, whose functions are
// not correctly rounded: a device function that is merely accurate differs from them in the last place now
// and then, and formulas that cancel (1 + tanh(..) in gelu_tanh, min(x, 0) - log1p(e^-|x|) in log_sigmoid)
// turn that into many places. The functions below therefore restate the library's published algorithms
// operation for operation, so that the device returns the same bits:
//
//   expf, logf, powf   the table-driven double-precision algorithms of the ARM optimized routines (2017),
//                      which glibc has carried since 2.27 (sysdeps/ieee754/flt-32/e_{expf,logf,powf}.c); its
//                      x86-64 build runs the variant compiled with fused multiply-adds on FMA hosts, so the
//                      products feeding a sum are fused here the way that compilation fuses them;
//   expm1f, tanhf, log1pf   the FreeBSD msun / fdlibm single-precision algorithms glibc 2.39 still carries
//                      (sysdeps/ieee754/flt-32/s_{expm1f,tanhf,log1pf}.c), plain f32 arithmetic without
//                      fused operations.
//
// The header compiles for the host too (with g++; under nvcc the functions are device functions), where
// tests/native/libm32_check.cpp compares every function with the host's own library over all 2^32 arguments
// (expf, logf, expm1f, tanhf, log1pf, powf with the exponent 2) and over random pairs and every special pair
// (powf). The 2^(i/32) table is 2^(i/32) rounded to nearest with the index folded into the exponent field; the
// other constants are the algorithms' published ones.
#pragma once

#include <cstdint>
#include <cstring>

#if defined(__CUDACC__)
#define LM_HD __device__ __forceinline__
#define LM_TABLE __device__ const
#else
#define LM_HD static inline
#define LM_TABLE static const
#endif

namespace hmc {
namespace lm {

LM_HD uint32_t f2u(float x) {
#if defined(__CUDA_ARCH__)
    return __float_as_uint(x);
#else
    uint32_t u;
    memcpy(&u, &x, 4);
    return u;
#endif
}
LM_HD float u2f(uint32_t u) {
#if defined(__CUDA_ARCH__)
    return __uint_as_float(u);
#else
    float x;
    memcpy(&x, &u, 4);
    return x;
#endif
}
LM_HD uint64_t d2u(double x) {
#if defined(__CUDA_ARCH__)
    return static_cast<uint64_t>(__double_as_longlong(x));
#else
    uint64_t u;
    memcpy(&u, &x, 8);
    return u;
#endif
}
LM_HD double u2d(uint64_t u) {
#if defined(__CUDA_ARCH__)
    return __longlong_as_double(static_cast<long long>(u));
#else
    double x;
    memcpy(&x, &u, 8);
    return x;
#endif
}
// One rounding of a * b + c.
LM_HD double fmad(double a, double b, double c) {
#if defined(__CUDA_ARCH__)
    return __fma_rn(a, b, c);
#else
    return __builtin_fma(a, b, c);
#endif
}
LM_HD float absf(float x) { return u2f(f2u(x) & 0x7fffffffu); }

// bits(2^(i/32) rounded to nearest) - (i << 47): adding k << 47 to entry k % 32 gives the bits of 2^(k/32).
LM_TABLE uint64_t kExp2Table[32] = {
    0x3ff0000000000000ull, 0x3fefd9b0d3158574ull, 0x3fefb5586cf9890full, 0x3fef9301d0125b51ull,
    0x3fef72b83c7d517bull, 0x3fef54873168b9aaull, 0x3fef387a6e756238ull, 0x3fef1e9df51fdee1ull,
    0x3fef06fe0a31b715ull, 0x3feef1a7373aa9cbull, 0x3feedea64c123422ull, 0x3feece086061892dull,
    0x3feebfdad5362a27ull, 0x3feeb42b569d4f82ull, 0x3feeab07dd485429ull, 0x3feea47eb03a5585ull,
    0x3feea09e667f3bcdull, 0x3fee9f75e8ec5f74ull, 0x3feea11473eb0187ull, 0x3feea589994cce13ull,
    0x3feeace5422aa0dbull, 0x3feeb737b0cdc5e5ull, 0x3feec49182a3f090ull, 0x3feed503b23e255dull,
    0x3feee89f995ad3adull, 0x3feeff76f2fb5e47ull, 0x3fef199bdd85529cull, 0x3fef3720dcef9069ull,
    0x3fef5818dcfba487ull, 0x3fef7c97337b9b5full, 0x3fefa4afa2a490daull, 0x3fefd0765b6e4540ull,
};

// 16 intervals of the significand starting at 0x3f330000 (about 0.6992): 1/c for a point c near the middle
// of the interval, ln(c) and log2(c).
struct LogEntry {
    double invc, lnc, log2c;
};
LM_TABLE LogEntry kLogTable[16] = {
    {0x1.661ec79f8f3bep+0, -0x1.57bf7808caadep-2, -0x1.efec65b963019p-2},
    {0x1.571ed4aaf883dp+0, -0x1.2bef0a7c06ddbp-2, -0x1.b0b6832d4fca4p-2},
    {0x1.49539f0f010bp+0, -0x1.01eae7f513a67p-2, -0x1.7418b0a1fb77bp-2},
    {0x1.3c995b0b80385p+0, -0x1.b31d8a68224e9p-3, -0x1.39de91a6dcf7bp-2},
    {0x1.30d190c8864a5p+0, -0x1.6574f0ac07758p-3, -0x1.01d9bf3f2b631p-2},
    {0x1.25e227b0b8eap+0, -0x1.1aa2bc79c81p-3, -0x1.97c1d1b3b7afp-3},
    {0x1.1bb4a4a1a343fp+0, -0x1.a4e76ce8c0e5ep-4, -0x1.2f9e393af3c9fp-3},
    {0x1.12358f08ae5bap+0, -0x1.1973c5a611cccp-4, -0x1.960cbbf788d5cp-4},
    {0x1.0953f419900a7p+0, -0x1.252f438e10c1ep-5, -0x1.a6f9db6475fcep-5},
    {0x1p+0, 0x0p+0, 0x0p+0},
    {0x1.e608cfd9a47acp-1, 0x1.aa5aa5df25984p-5, 0x1.338ca9f24f53dp-4},
    {0x1.ca4b31f026aap-1, 0x1.c5e53aa362eb4p-4, 0x1.476a9543891bap-3},
    {0x1.b2036576afce6p-1, 0x1.526e57720db08p-3, 0x1.e840b4ac4e4d2p-3},
    {0x1.9c2d163a1aa2dp-1, 0x1.bc2860d22477p-3, 0x1.40645f0c6651cp-2},
    {0x1.886e6037841edp-1, 0x1.1058bc8a07ee1p-2, 0x1.88e9c2c1b9ff8p-2},
    {0x1.767dcf5534862p-1, 0x1.4043057b6ee09p-2, 0x1.ce0a44eb17bccp-2},
};

// e^x. x * 32/ln2 = k + r with |r| <= 1/2; e^x = 2^(k/32) * 2^(r/32), the first factor from the table, the
// second a cubic in r; everything in double, one rounding to float at the end (which also produces
// subnormal results).
LM_HD float expf(float x) {
    const uint32_t ux = f2u(x);
    const uint32_t abstop = (ux >> 20) & 0x7ffu;
    if (abstop >= 0x42bu) {  // |x| >= 88, infinite or NaN
        if (ux == 0xff800000u) return 0.0f;
        if (abstop >= 0x7f8u) return x + x;
        if (x > 0x1.62e42ep6f) return u2f(0x7f800000u);
        if (x < -0x1.9fe368p6f) return 0.0f;
    }
    const double xd = static_cast<double>(x);
    const double inv = 0x1.71547652b82fep+0 * 32.0;
    const double shift = 0x1.8p+52;
    // the product x * 32/ln2 is never rounded by itself: it is fused into both sums that use it
    double kd = fmad(inv, xd, shift);
    const uint64_t ki = d2u(kd);
    kd -= shift;
    const double r = fmad(inv, xd, -kd);
    const uint64_t t = kExp2Table[ki & 31u] + (ki << 47);
    const double s = u2d(t);
    const double c0 = 0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0;
    const double c1 = 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0;
    const double c2 = 0x1.62e42ff0c52d6p-1 / 32.0;
    const double q = fmad(c0, r, c1);
    const double r2 = r * r;
    double y = fmad(c2, r, 1.0);
    y = fmad(q, r2, y);
    y = y * s;
    return static_cast<float>(y);
}

// ln x. x = 2^k * z with z in [0x3f330000, 2 * 0x3f330000) as floats; ln x = ln(z / c) + ln c + k ln 2 with c
// from the table, ln(1 + r) for r = z / c - 1 by a cubic.
LM_HD float logf(float x) {
    uint32_t ix = f2u(x);
    if (ix == 0x3f800000u) return 0.0f;
    if (ix - 0x00800000u >= 0x7f800000u - 0x00800000u) {  // below 2^-126, negative, infinite or NaN
        if (ix * 2u == 0u) return u2f(0xff800000u);
        if (ix == 0x7f800000u) return x;
        if ((ix & 0x80000000u) || ix * 2u >= 0xff000000u) return u2f(0x7fc00000u);
        ix = f2u(x * 0x1p23f);
        ix -= 23u << 23;
    }
    const uint32_t tmp = ix - 0x3f330000u;
    const int i = static_cast<int>((tmp >> 19) & 15u);
    const int k = static_cast<int32_t>(tmp) >> 23;
    const uint32_t iz = ix - (tmp & 0xff800000u);
    const double invc = kLogTable[i].invc;
    const double lnc = kLogTable[i].lnc;
    const double z = static_cast<double>(u2f(iz));
    const double r = fmad(z, invc, -1.0);
    const double y0 = fmad(static_cast<double>(k), 0x1.62e42fefa39efp-1, lnc);
    const double r2 = r * r;
    double y = fmad(0x1.5575b0be00b6ap-2, r, -0x1.ffffef20a4123p-2);
    y = fmad(-0x1.00ea348b88334p-2, r2, y);
    y = fmad(y, r2, y0 + r);
    return static_cast<float>(y);
}

// 0 when y is not an integer, 1 when it is an odd one, 2 when it is an even one.
LM_HD int pow_integer_class(uint32_t iy) {
    const int e = static_cast<int>((iy >> 23) & 0xffu);
    if (e < 0x7f) return 0;
    if (e > 0x7f + 23) return 2;
    if (iy & ((1u << (0x7f + 23 - e)) - 1u)) return 0;
    if (iy & (1u << (0x7f + 23 - e))) return 1;
    return 2;
}
LM_HD bool pow_zero_inf_nan(uint32_t i) { return 2u * i - 1u >= 2u * 0x7f800000u - 1u; }
LM_HD bool pow_signalling(uint32_t i) { return 2u * (i ^ 0x00400000u) > 2u * 0x7fc00000u; }

// x^y = 2^(y log2 x): log2 x in double to about 2^-68 relative (table + quartic), the product in double,
// then 2^t as in expf (with the sign of the result carried into the exponent field's top bit).
LM_HD float powf(float x, float y) {
    uint32_t sign_bias = 0;
    uint32_t ix = f2u(x);
    const uint32_t iy = f2u(y);
    if (ix - 0x00800000u >= 0x7f800000u - 0x00800000u || pow_zero_inf_nan(iy)) {
        if (pow_zero_inf_nan(iy)) {
            if (2u * iy == 0u) return pow_signalling(ix) ? x + y : 1.0f;
            if (ix == 0x3f800000u) return pow_signalling(iy) ? x + y : 1.0f;
            if (2u * ix > 2u * 0x7f800000u || 2u * iy > 2u * 0x7f800000u) return x + y;
            if (2u * ix == 2u * 0x3f800000u) return 1.0f;
            if ((2u * ix < 2u * 0x3f800000u) == !(iy & 0x80000000u)) return 0.0f;
            return y * y;
        }
        if (pow_zero_inf_nan(ix)) {
            float x2 = x * x;
            if ((ix & 0x80000000u) && pow_integer_class(iy) == 1) {
                x2 = -x2;
                sign_bias = 1;
            }
            if (2u * ix == 0u && (iy & 0x80000000u)) return u2f(sign_bias ? 0xff800000u : 0x7f800000u);
            return (iy & 0x80000000u) ? 1.0f / x2 : x2;
        }
        if (ix & 0x80000000u) {  // finite negative base
            const int yint = pow_integer_class(iy);
            if (yint == 0) return u2f(0x7fc00000u);
            if (yint == 1) sign_bias = 1u << (5 + 11);
            ix &= 0x7fffffffu;
        }
        if (ix < 0x00800000u) {  // subnormal base
            ix = f2u(x * 0x1p23f);
            ix &= 0x7fffffffu;
            ix -= 23u << 23;
        }
    }
    // log2 of the (now positive, normal) base
    const uint32_t tmp = ix - 0x3f330000u;
    const int i = static_cast<int>((tmp >> 19) & 15u);
    const uint32_t top = tmp & 0xff800000u;
    const uint32_t iz = ix - top;
    const int k = static_cast<int32_t>(top) >> 23;
    const double invc = kLogTable[i].invc;
    const double log2c = kLogTable[i].log2c;
    const double z = static_cast<double>(u2f(iz));
    const double r = fmad(z, invc, -1.0);
    const double y0 = log2c + static_cast<double>(k);
    const double r2 = r * r;
    double yy = fmad(0x1.27616c9496e0bp-2, r, -0x1.71969a075c67ap-2);
    const double p = fmad(0x1.ec70a6ca7baddp-2, r, -0x1.7154748bef6c8p-1);
    const double r4 = r2 * r2;
    double q = fmad(0x1.71547652ab82bp0, r, y0);
    q = fmad(p, r2, q);
    yy = fmad(yy, r4, q);
    const double ylogx = static_cast<double>(y) * yy;
    if (((d2u(ylogx) >> 47) & 0xffffu) >= (d2u(126.0) >> 47)) {  // |y log2 x| >= 126
        if (ylogx > 0x1.fffffffd1d571p+6) return u2f(sign_bias ? 0xff800000u : 0x7f800000u);
        if (ylogx <= -150.0) return u2f(sign_bias ? 0x80000000u : 0u);
    }
    // 2^ylogx
    const double shift = 0x1.8p+52 / 32.0;
    double kd = ylogx + shift;
    const uint64_t ki = d2u(kd);
    kd -= shift;
    const double rr = ylogx - kd;
    const uint64_t t = kExp2Table[ki & 31u] + ((ki + sign_bias) << 47);
    const double s = u2d(t);
    const double e = fmad(0x1.c6af84b912394p-5, rr, 0x1.ebfce50fac4f3p-3);
    const double rr2 = rr * rr;
    double w = fmad(0x1.62e42ff0c52d6p-1, rr, 1.0);
    w = fmad(e, rr2, w);
    w = w * s;
    return static_cast<float>(w);
}

// e^x - 1 in f32 arithmetic: x = k ln2 + r with |r| <= ln2 / 2 (ln2 in two pieces, c the rounding error of
// r), e^r - 1 = r + r^2/2 * (..) through the rational form r - r * (R - T) / (6 - r T) * .., then the scaling
// by 2^k case by case so that nothing cancels.
LM_HD float expm1f(float x) {
    const float ln2_hi = 6.9313812256e-01f, ln2_lo = 9.0580006145e-06f, invln2 = 1.4426950216e+00f;
    const float Q1 = -3.3333335072e-02f, Q2 = 1.5873016091e-03f, Q3 = -7.9365076090e-05f,
                Q4 = 4.0082177293e-06f, Q5 = -2.0109921195e-07f;
    uint32_t hx = f2u(x);
    const bool negative = (hx & 0x80000000u) != 0;
    hx &= 0x7fffffffu;
    if (hx >= 0x4195b844u) {  // |x| >= 27 ln2
        if (hx >= 0x42b17218u) {  // |x| >= 88.72..
            if (hx > 0x7f800000u) return x + x;
            if (hx == 0x7f800000u) return negative ? -1.0f : x;
            if (x > 8.8721679688e+01f) return u2f(0x7f800000u);
        }
        if (negative) return -1.0f;
    }
    float hi, lo, c = 0.0f;
    int k;
    if (hx > 0x3eb17218u) {  // |x| > ln2 / 2
        if (hx < 0x3F851592u) {  // |x| < 1.5 ln2
            if (!negative) {
                hi = x - ln2_hi;
                lo = ln2_lo;
                k = 1;
            } else {
                hi = x + ln2_hi;
                lo = -ln2_lo;
                k = -1;
            }
        } else {
            k = static_cast<int>(invln2 * x + (negative ? -0.5f : 0.5f));
            const float t = static_cast<float>(k);
            hi = x - t * ln2_hi;
            lo = t * ln2_lo;
        }
        x = hi - lo;
        c = (hi - x) - lo;
    } else if (hx < 0x33000000u) {  // |x| < 2^-25
        return x;
    } else {
        k = 0;
    }
    const float hfx = 0.5f * x;
    const float hxs = x * hfx;
    const float r1 = 1.0f + hxs * (Q1 + hxs * (Q2 + hxs * (Q3 + hxs * (Q4 + hxs * Q5))));
    float t = 3.0f - r1 * hfx;
    float e = hxs * ((r1 - t) / (6.0f - x * t));
    if (k == 0) return x - (x * e - hxs);
    e = (x * (e - c) - c);
    e -= hxs;
    if (k == -1) return 0.5f * (x - e) - 0.5f;
    if (k == 1) {
        if (x < -0.25f) return -2.0f * (e - (x + 0.5f));
        return 1.0f + 2.0f * (x - e);
    }
    float y;
    if (k <= -2 || k > 56) {
        y = 1.0f - (e - x);
        y = u2f(f2u(y) + (static_cast<uint32_t>(k) << 23));
        return y - 1.0f;
    }
    if (k < 23) {
        t = u2f(0x3f800000u - (0x1000000u >> k));  // 1 - 2^-k
        y = t - (e - x);
        y = u2f(f2u(y) + (static_cast<uint32_t>(k) << 23));
    } else {
        t = u2f(static_cast<uint32_t>(0x7f - k) << 23);  // 2^-k
        y = x - (e + t);
        y += 1.0f;
        y = u2f(f2u(y) + (static_cast<uint32_t>(k) << 23));
    }
    return y;
}

// tanh x from e^(2|x|) - 1 (|x| >= 1) or e^(-2|x|) - 1 (|x| < 1), 1 beyond 22.
LM_HD float tanhf(float x) {
    const uint32_t jx = f2u(x);
    const uint32_t ix = jx & 0x7fffffffu;
    const bool negative = (jx & 0x80000000u) != 0;
    if (ix >= 0x7f800000u) return negative ? 1.0f / x - 1.0f : 1.0f / x + 1.0f;
    float z;
    if (ix < 0x41b00000u) {  // |x| < 22
        if (ix == 0u) return x;
        if (ix < 0x24000000u) return x * (1.0f + x);  // |x| < 2^-55
        if (ix >= 0x3f800000u) {
            const float t = expm1f(2.0f * absf(x));
            z = 1.0f - 2.0f / (t + 2.0f);
        } else {
            const float t = expm1f(-2.0f * absf(x));
            z = -t / (t + 2.0f);
        }
    } else {
        z = 1.0f;  // 1 - 1e-30 rounds to 1
    }
    return negative ? -z : z;
}

// ln(1 + x) in f32 arithmetic: 1 + x = 2^k * (1 + f) with sqrt(2)/2 < 1 + f < sqrt(2) and a correction c for
// the rounding of 1 + x, ln(1 + f) = f - f^2/2 + s (f^2/2 + R(s^2)) with s = f / (2 + f).
LM_HD float log1pf(float x) {
    const float ln2_hi = 6.9313812256e-01f, ln2_lo = 9.0580006145e-06f;
    const float Lp1 = 6.6666668653e-01f, Lp2 = 4.0000000596e-01f, Lp3 = 2.8571429849e-01f, Lp4 = 2.2222198546e-01f,
                Lp5 = 1.8183572590e-01f, Lp6 = 1.5313838422e-01f, Lp7 = 1.4798198640e-01f;
    const int32_t hx = static_cast<int32_t>(f2u(x));
    const int32_t ax = hx & 0x7fffffff;
    int32_t k = 1, hu = 0;
    float f = 0.0f, c = 0.0f;
    if (hx < 0x3ed413d7) {  // x < sqrt(2) - 1
        if (ax >= 0x3f800000) {  // x <= -1
            if (x == -1.0f) return u2f(0xff800000u);
            return u2f(0x7fc00000u);
        }
        if (ax < 0x31000000) {  // |x| < 2^-29
            if (ax < 0x24800000) return x;  // |x| < 2^-54
            return x - x * x * 0.5f;
        }
        if (hx > 0 || hx <= static_cast<int32_t>(0xbe95f61fu)) {  // -0.2929 < x < 0.41422
            k = 0;
            f = x;
            hu = 1;
        }
    }
    if (hx >= 0x7f800000) return x + x;
    if (k != 0) {
        float u;
        if (hx < 0x5a000000) {
            u = 1.0f + x;
            hu = static_cast<int32_t>(f2u(u));
            k = (hu >> 23) - 127;
            c = (k > 0) ? 1.0f - (u - x) : x - (u - 1.0f);
            c /= u;
        } else {
            u = x;
            hu = static_cast<int32_t>(f2u(u));
            k = (hu >> 23) - 127;
            c = 0.0f;
        }
        hu &= 0x007fffff;
        if (hu < 0x3504f7) {
            u = u2f(static_cast<uint32_t>(hu) | 0x3f800000u);
        } else {
            k += 1;
            u = u2f(static_cast<uint32_t>(hu) | 0x3f000000u);
            hu = (0x00800000 - hu) >> 2;
        }
        f = u - 1.0f;
    }
    const float hfsq = 0.5f * f * f;
    const float fk = static_cast<float>(k);
    if (hu == 0) {  // |f| < 2^-20
        if (f == 0.0f) {
            if (k == 0) return 0.0f;
            c += fk * ln2_lo;
            return fk * ln2_hi + c;
        }
        const float R = hfsq * (1.0f - 0.66666666666666666f * f);
        if (k == 0) return f - R;
        return fk * ln2_hi - ((R - (fk * ln2_lo + c)) - f);
    }
    const float s = f / (2.0f + f);
    const float z = s * s;
    const float R = z * (Lp1 + z * (Lp2 + z * (Lp3 + z * (Lp4 + z * (Lp5 + z * (Lp6 + z * Lp7))))));
    if (k == 0) return f - (hfsq - s * (hfsq + R));
    return fk * ln2_hi - ((hfsq - (s * (hfsq + R) + (fk * ln2_lo + c))) - f);
}

}  // namespace lm
}  // namespace hmc
