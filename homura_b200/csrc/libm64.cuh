// Double-precision exp, expm1, tanh and log1p with the bits of the host C library.
//
// homura's CPU backend evaluates F64 tensors with Rust's f64::exp, tanh and ln_1p, which are the C
// library's exp, tanh and log1p (src/backend/cpu/mod.rs:378-402). On the hosts this backend is built for that
// library is glibc 2.39 on x86-64 with FMA; none of these functions is correctly rounded there, and formulas that
// cancel (1 + tanh(..) in gelu_tanh) turn a last-place difference into dozens of places. The functions below restate
// the library's published algorithms operation for operation:
//
//   exp      the table-driven algorithm of the ARM optimized routines (sysdeps/ieee754/dbl-64/e_exp.c since glibc
//            2.28): 2^(k/128) from a table, a degree-5 polynomial in the remainder;
//   expm1, tanh, log1p   the fdlibm algorithms (sysdeps/ieee754/dbl-64/s_{expm1,tanh,log1p}.c), whose x86-64 builds
//            for FMA hosts contract a product into the sum that follows it where the compiler finds both in one basic
//            block; the fused operations below are placed where that build has them (a product that is shared by
//            two branches is computed once, rounded).
//
// The header compiles for the host too, where tests/native/libm64_check.cpp compares every function with the host's
// own library over hundreds of millions of arguments (random bit patterns, the whole finite range, and the small
// arguments where the polynomials work). The table holds 2^(k/128) rounded to nearest with k folded into the exponent
// field, and the relative remainder of that rounding: regenerated from first principles, not copied.
#pragma once

#include <cstdint>
#include <cstring>

#if defined(__CUDACC__)
#define LM64_HD __device__ __forceinline__
#define LM64_TABLE __device__ const
#else
#include <cmath>
#define LM64_HD static inline
#define LM64_TABLE static const
#endif

namespace hmc {
namespace lm64 {

LM64_HD uint64_t d2u(double x) {
#if defined(__CUDA_ARCH__)
    return static_cast<uint64_t>(__double_as_longlong(x));
#else
    uint64_t u;
    memcpy(&u, &x, 8);
    return u;
#endif
}
LM64_HD double u2d(uint64_t u) {
#if defined(__CUDA_ARCH__)
    return __longlong_as_double(static_cast<long long>(u));
#else
    double x;
    memcpy(&x, &u, 8);
    return x;
#endif
}
LM64_HD double fmad(double a, double b, double c) {
#if defined(__CUDA_ARCH__)
    return __fma_rn(a, b, c);
#else
    return std::fma(a, b, c);
#endif
}
LM64_HD uint32_t hi32(double x) { return static_cast<uint32_t>(d2u(x) >> 32); }
LM64_HD uint32_t lo32(double x) { return static_cast<uint32_t>(d2u(x)); }
LM64_HD double with_hi(double x, uint32_t h) { return u2d((static_cast<uint64_t>(h) << 32) | lo32(x)); }
LM64_HD double infinity() { return u2d(0x7ff0000000000000ull); }

// {relative remainder T[k], bits of H[k] = RN(2^(k/128)) minus k * 2^45}: 2^(k/128) = H[k] (1 + T[k]).
LM64_TABLE uint64_t kExpTable[256] = {
    0x0000000000000000ull, 0x3ff0000000000000ull, 0x3c9b3b4f1a88bf6eull, 0x3feff63da9fb3335ull,
    0xbc7160139cd8dc5dull, 0x3fefec9a3e778061ull, 0xbc905e7a108766d1ull, 0x3fefe315e86e7f85ull,
    0x3c8cd2523567f613ull, 0x3fefd9b0d3158574ull, 0xbc8bce8023f98efaull, 0x3fefd06b29ddf6deull,
    0x3c60f74e61e6c861ull, 0x3fefc74518759bc8ull, 0x3c90a3e45b33d399ull, 0x3fefbe3ecac6f383ull,
    0x3c979aa65d837b6dull, 0x3fefb5586cf9890full, 0x3c8eb51a92fdeffcull, 0x3fefac922b7247f7ull,
    0x3c3ebe3d702f9cd1ull, 0x3fefa3ec32d3d1a2ull, 0xbc6a033489906e0bull, 0x3fef9b66affed31bull,
    0xbc9556522a2fbd0eull, 0x3fef9301d0125b51ull, 0xbc5080ef8c4eea55ull, 0x3fef8abdc06c31ccull,
    0xbc91c923b9d5f416ull, 0x3fef829aaea92de0ull, 0x3c80d3e3e95c55afull, 0x3fef7a98c8a58e51ull,
    0xbc801b15eaa59348ull, 0x3fef72b83c7d517bull, 0xbc8f1ff055de323dull, 0x3fef6af9388c8deaull,
    0x3c8b898c3f1353bfull, 0x3fef635beb6fcb75ull, 0xbc96d99c7611eb26ull, 0x3fef5be084045cd4ull,
    0x3c9aecf73e3a2f60ull, 0x3fef54873168b9aaull, 0xbc8fe782cb86389dull, 0x3fef4d5022fcd91dull,
    0x3c8a6f4144a6c38dull, 0x3fef463b88628cd6ull, 0x3c807a05b0e4047dull, 0x3fef3f49917ddc96ull,
    0x3c968efde3a8a894ull, 0x3fef387a6e756238ull, 0x3c875e18f274487dull, 0x3fef31ce4fb2a63full,
    0x3c80472b981fe7f2ull, 0x3fef2b4565e27cddull, 0xbc96b87b3f71085eull, 0x3fef24dfe1f56381ull,
    0x3c82f7e16d09ab31ull, 0x3fef1e9df51fdee1ull, 0xbc3d219b1a6fbffaull, 0x3fef187fd0dad990ull,
    0x3c8b3782720c0ab4ull, 0x3fef1285a6e4030bull, 0x3c6e149289cecb8full, 0x3fef0cafa93e2f56ull,
    0x3c834d754db0abb6ull, 0x3fef06fe0a31b715ull, 0x3c864201e2ac744cull, 0x3fef0170fc4cd831ull,
    0x3c8fdd395dd3f84aull, 0x3feefc08b26416ffull, 0xbc86a3803b8e5b04ull, 0x3feef6c55f929ff1ull,
    0xbc924aedcc4b5068ull, 0x3feef1a7373aa9cbull, 0xbc9907f81b512d8eull, 0x3feeecae6d05d866ull,
    0xbc71d1e83e9436d2ull, 0x3feee7db34e59ff7ull, 0xbc991919b3ce1b15ull, 0x3feee32dc313a8e5ull,
    0x3c859f48a72a4c6dull, 0x3feedea64c123422ull, 0xbc9312607a28698aull, 0x3feeda4504ac801cull,
    0xbc58a78f4817895bull, 0x3feed60a21f72e2aull, 0xbc7c2c9b67499a1bull, 0x3feed1f5d950a897ull,
    0x3c4363ed60c2ac11ull, 0x3feece086061892dull, 0x3c9666093b0664efull, 0x3feeca41ed1d0057ull,
    0x3c6ecce1daa10379ull, 0x3feec6a2b5c13cd0ull, 0x3c93ff8e3f0f1230ull, 0x3feec32af0d7d3deull,
    0x3c7690cebb7aafb0ull, 0x3feebfdad5362a27ull, 0x3c931dbdeb54e077ull, 0x3feebcb299fddd0dull,
    0xbc8f94340071a38eull, 0x3feeb9b2769d2ca7ull, 0xbc87deccdc93a349ull, 0x3feeb6daa2cf6642ull,
    0xbc78dec6bd0f385full, 0x3feeb42b569d4f82ull, 0xbc861246ec7b5cf6ull, 0x3feeb1a4ca5d920full,
    0x3c93350518fdd78eull, 0x3feeaf4736b527daull, 0x3c7b98b72f8a9b05ull, 0x3feead12d497c7fdull,
    0x3c9063e1e21c5409ull, 0x3feeab07dd485429ull, 0x3c34c7855019c6eaull, 0x3feea9268a5946b7ull,
    0x3c9432e62b64c035ull, 0x3feea76f15ad2148ull, 0xbc8ce44a6199769full, 0x3feea5e1b976dc09ull,
    0xbc8c33c53bef4da8ull, 0x3feea47eb03a5585ull, 0xbc845378892be9aeull, 0x3feea34634ccc320ull,
    0xbc93cedd78565858ull, 0x3feea23882552225ull, 0x3c5710aa807e1964ull, 0x3feea155d44ca973ull,
    0xbc93b3efbf5e2228ull, 0x3feea09e667f3bcdull, 0xbc6a12ad8734b982ull, 0x3feea012750bdabfull,
    0xbc6367efb86da9eeull, 0x3fee9fb23c651a2full, 0xbc80dc3d54e08851ull, 0x3fee9f7df9519484ull,
    0xbc781f647e5a3ecfull, 0x3fee9f75e8ec5f74ull, 0xbc86ee4ac08b7db0ull, 0x3fee9f9a48a58174ull,
    0xbc8619321e55e68aull, 0x3fee9feb564267c9ull, 0x3c909ccb5e09d4d3ull, 0x3feea0694fde5d3full,
    0xbc7b32dcb94da51dull, 0x3feea11473eb0187ull, 0x3c94ecfd5467c06bull, 0x3feea1ed0130c132ull,
    0x3c65ebe1abd66c55ull, 0x3feea2f336cf4e62ull, 0xbc88a1c52fb3cf42ull, 0x3feea427543e1a12ull,
    0xbc9369b6f13b3734ull, 0x3feea589994cce13ull, 0xbc805e843a19ff1eull, 0x3feea71a4623c7adull,
    0xbc94d450d872576eull, 0x3feea8d99b4492edull, 0x3c90ad675b0e8a00ull, 0x3feeaac7d98a6699ull,
    0x3c8db72fc1f0eab4ull, 0x3feeace5422aa0dbull, 0xbc65b6609cc5e7ffull, 0x3feeaf3216b5448cull,
    0x3c7bf68359f35f44ull, 0x3feeb1ae99157736ull, 0xbc93091fa71e3d83ull, 0x3feeb45b0b91ffc6ull,
    0xbc5da9b88b6c1e29ull, 0x3feeb737b0cdc5e5ull, 0xbc6c23f97c90b959ull, 0x3feeba44cbc8520full,
    0xbc92434322f4f9aaull, 0x3feebd829fde4e50ull, 0xbc85ca6cd7668e4bull, 0x3feec0f170ca07baull,
    0x3c71affc2b91ce27ull, 0x3feec49182a3f090ull, 0x3c6dd235e10a73bbull, 0x3feec86319e32323ull,
    0xbc87c50422622263ull, 0x3feecc667b5de565ull, 0x3c8b1c86e3e231d5ull, 0x3feed09bec4a2d33ull,
    0xbc91bbd1d3bcbb15ull, 0x3feed503b23e255dull, 0x3c90cc319cee31d2ull, 0x3feed99e1330b358ull,
    0x3c8469846e735ab3ull, 0x3feede6b5579fdbfull, 0xbc82dfcd978e9db4ull, 0x3feee36bbfd3f37aull,
    0x3c8c1a7792cb3387ull, 0x3feee89f995ad3adull, 0xbc907b8f4ad1d9faull, 0x3feeee07298db666ull,
    0xbc55c3d956dcaebaull, 0x3feef3a2b84f15fbull, 0xbc90a40e3da6f640ull, 0x3feef9728de5593aull,
    0xbc68d6f438ad9334ull, 0x3feeff76f2fb5e47ull, 0xbc91eee26b588a35ull, 0x3fef05b030a1064aull,
    0x3c74ffd70a5fddcdull, 0x3fef0c1e904bc1d2ull, 0xbc91bdfbfa9298acull, 0x3fef12c25bd71e09ull,
    0x3c736eae30af0cb3ull, 0x3fef199bdd85529cull, 0x3c8ee3325c9ffd94ull, 0x3fef20ab5fffd07aull,
    0x3c84e08fd10959acull, 0x3fef27f12e57d14bull, 0x3c63cdaf384e1a67ull, 0x3fef2f6d9406e7b5ull,
    0x3c676b2c6c921968ull, 0x3fef3720dcef9069ull, 0xbc808a1883ccb5d2ull, 0x3fef3f0b555dc3faull,
    0xbc8fad5d3ffffa6full, 0x3fef472d4a07897cull, 0xbc900dae3875a949ull, 0x3fef4f87080d89f2ull,
    0x3c74a385a63d07a7ull, 0x3fef5818dcfba487ull, 0xbc82919e2040220full, 0x3fef60e316c98398ull,
    0x3c8e5a50d5c192acull, 0x3fef69e603db3285ull, 0x3c843a59ac016b4bull, 0x3fef7321f301b460ull,
    0xbc82d52107b43e1full, 0x3fef7c97337b9b5full, 0xbc892ab93b470dc9ull, 0x3fef864614f5a129ull,
    0x3c74b604603a88d3ull, 0x3fef902ee78b3ff6ull, 0x3c83c5ec519d7271ull, 0x3fef9a51fbc74c83ull,
    0xbc8ff7128fd391f0ull, 0x3fefa4afa2a490daull, 0xbc8dae98e223747dull, 0x3fefaf482d8e67f1ull,
    0x3c8ec3bc41aa2008ull, 0x3fefba1bee615a27ull, 0x3c842b94c3a9eb32ull, 0x3fefc52b376bba97ull,
    0x3c8a64a931d185eeull, 0x3fefd0765b6e4540ull, 0xbc8e37bae43be3edull, 0x3fefdbfdad9cbe14ull,
    0x3c77893b4d91cd9dull, 0x3fefe7c1819e90d8ull, 0x3c5305c14160cc89ull, 0x3feff3c22b8f71f1ull,
};

// A result that overflows, underflows or is subnormal: the scale factor is split so that the last multiplication
// rounds once.
LM64_HD double exp_special(double tmp, uint64_t sbits, uint64_t ki) {
    if ((ki & 0x80000000u) == 0) {  // k > 0: the exponent of scale may have overflowed
        sbits -= 1009ull << 52;
        const double scale = u2d(sbits);
        return 0x1p1009 * fmad(scale, tmp, scale);
    }
    sbits += 1022ull << 52;
    const double scale = u2d(sbits);
    const double p = scale * tmp;  // (used twice in the library's build: one rounded product)
    double y = scale + p;
    if (y < 1.0) {
        // round y to the precision of the subnormal result before the final scaling
        double lo = scale - y + p;
        const double hi = 1.0 + y;
        lo = 1.0 - hi + y + lo;
        y = (hi + lo) - 1.0;
        if (y == 0.0) y = 0.0;  // (-0.0 becomes 0.0)
    }
    return 0x1p-1022 * y;
}

LM64_HD double exp(double x) {
    uint32_t abstop = static_cast<uint32_t>(d2u(x) >> 52) & 0x7ffu;
    if (abstop - 0x3c9u >= 0x408u - 0x3c9u) {       // |x| < 2^-54, |x| >= 512, or not finite
        if (abstop - 0x3c9u >= 0x80000000u) return 1.0 + x;  // tiny
        if (abstop >= 0x409u) {                     // |x| >= 1024
            if (d2u(x) == 0xfff0000000000000ull) return 0.0;
            if (abstop >= 0x7ffu) return 1.0 + x;
            return (d2u(x) >> 63) ? 0.0 : infinity();
        }
        abstop = 0;  // large |x|: the result is put together by exp_special
    }
    const double inv = 0x1.71547652b82fep0 * 128.0, shift = 0x1.8p52;
    double kd = fmad(inv, x, shift);
    const uint64_t ki = d2u(kd);
    kd -= shift;
    const double r = fmad(kd, -0x1.cf79abc9e3b3ap-47, fmad(kd, -0x1.62e42fefa0000p-8, x));
    const uint64_t idx = 2 * (ki % 128), top = ki << (52 - 7);
    const double tail = u2d(kExpTable[idx]);
    const uint64_t sbits = kExpTable[idx + 1] + top;
    const double r2 = r * r;
    const double tmp = fmad(r2 * r2, fmad(r, 0x1.1111167a4d017p-7, 0x1.55555cf172b91p-5),
                            fmad(r2, fmad(r, 0x1.555555555543cp-3, 0x1.ffffffffffdbdp-2), tail + r));
    if (abstop == 0) return exp_special(tmp, sbits, ki);
    const double scale = u2d(sbits);
    return fmad(scale, tmp, scale);
}

LM64_HD double expm1(double x) {
    const double one = 1.0, huge = 1.0e+300, tiny = 1.0e-300, o_threshold = 7.09782712893383973096e+02,
                 ln2_hi = 6.93147180369123816490e-01, ln2_lo = 1.90821492927058770002e-10, invln2 = 1.44269504088896338700e+00;
    const double Q1 = -3.33333333333331316428e-02, Q2 = 1.58730158725481460165e-03, Q3 = -7.93650757867487942473e-05,
                 Q4 = 4.00821782732936239552e-06, Q5 = -2.01099218183624371326e-07;
    double y, hi, lo, c = 0.0, t, e;
    int32_t k;
    uint32_t hx = hi32(x);
    const uint32_t xsb = hx & 0x80000000u;
    hx &= 0x7fffffffu;
    if (hx >= 0x4043687Au) {  // |x| >= 56 ln2
        if (hx >= 0x40862E42u) {
            if (hx >= 0x7ff00000u) {
                if (((hx & 0xfffffu) | lo32(x)) != 0) return x + x;
                return xsb == 0 ? x : -1.0;
            }
            if (x > o_threshold) return huge * huge;
        }
        if (xsb != 0) return tiny - one;
    }
    if (hx > 0x3fd62e42u) {  // |x| > 0.5 ln2
        if (hx < 0x3FF0A2B2u) {
            if (xsb == 0) { hi = x - ln2_hi; lo = ln2_lo; k = 1; }
            else { hi = x + ln2_hi; lo = -ln2_lo; k = -1; }
        } else {
            k = static_cast<int32_t>(fmad(invln2, x, xsb == 0 ? 0.5 : -0.5));
            t = k;
            hi = fmad(-t, ln2_hi, x);
            lo = t * ln2_lo;
        }
        x = hi - lo;
        c = (hi - x) - lo;
    } else if (hx < 0x3c900000u) {
        t = huge + x;
        return x - (t - (huge + x));
    } else {
        k = 0;
    }
    const double hfx = 0.5 * x;
    const double hxs = x * hfx;
    const double R1 = fmad(hxs, Q1, one), h2 = hxs * hxs;
    const double R2 = fmad(hxs, Q3, Q2), h4 = h2 * h2;
    const double R3 = fmad(hxs, Q5, Q4);
    const double r1 = fmad(h4, R3, fmad(h2, R2, R1));
    t = fmad(-r1, hfx, 3.0);
    e = hxs * ((r1 - t) / fmad(-x, t, 6.0));
    if (k == 0) return x - fmad(x, e, -hxs);
    e = fmad(x, e - c, -c);
    e -= hxs;
    if (k == -1) return fmad(0.5, x - e, -0.5);
    if (k == 1) {
        if (x < -0.25) return -2.0 * (e - (x + 0.5));
        return fmad(2.0, x - e, one);
    }
    if (k <= -2 || k > 56) {
        y = one - (e - x);
        y = with_hi(y, hi32(y) + (static_cast<uint32_t>(k) << 20));
        return y - one;
    }
    t = one;
    if (k < 20) {
        t = with_hi(t, 0x3ff00000u - (0x200000u >> k));
        y = t - (e - x);
        y = with_hi(y, hi32(y) + (static_cast<uint32_t>(k) << 20));
    } else {
        t = with_hi(t, static_cast<uint32_t>(0x3ff - k) << 20);
        y = x - (e + t);
        y += one;
        y = with_hi(y, hi32(y) + (static_cast<uint32_t>(k) << 20));
    }
    return y;
}

LM64_HD double tanh(double x) {
    const double one = 1.0, two = 2.0, tiny = 1.0e-300;
    const int32_t jx = static_cast<int32_t>(hi32(x)), ix = jx & 0x7fffffff;
    double z;
    if (ix >= 0x7ff00000) return jx >= 0 ? one / x + one : one / x - one;
    if (ix < 0x40360000) {  // |x| < 22
        if ((static_cast<uint32_t>(ix) | lo32(x)) == 0) return x;
        if (ix < 0x3c800000) return x * (one + x);
        const double ax = u2d(d2u(x) & 0x7fffffffffffffffull);
        if (ix >= 0x3ff00000) {
            const double t = expm1(two * ax);
            z = one - two / (t + two);
        } else {
            const double t = expm1(-two * ax);
            z = -t / (t + two);
        }
    } else {
        z = one - tiny;
    }
    return jx >= 0 ? z : -z;
}

LM64_HD double log1p(double x) {
    const double ln2_hi = 6.93147180369123816490e-01, ln2_lo = 1.90821492927058770002e-10, two54 = 1.80143985094819840000e+16;
    const double Lp1 = 6.666666666666735130e-01, Lp2 = 3.999999999940941908e-01, Lp3 = 2.857142874366239149e-01,
                 Lp4 = 2.222219843214978396e-01, Lp5 = 1.818357216161805012e-01, Lp6 = 1.531383769920937332e-01,
                 Lp7 = 1.479819860511658591e-01;
    double f = 0.0, c = 0.0, u;
    int32_t k = 1, hu = 0;
    const int32_t hx = static_cast<int32_t>(hi32(x)), ax = hx & 0x7fffffff;
    if (hx < 0x3FDA827A) {  // x < 0.41422
        if (ax >= 0x3ff00000) {  // x <= -1
            if (x == -1.0) return -two54 / 0.0;
            return (x - x) / (x - x);
        }
        if (ax < 0x3e200000) {  // |x| < 2^-29
            if (ax < 0x3c900000) return x;
            return fmad(-(x * x), 0.5, x);
        }
        if (hx > 0 || hx <= static_cast<int32_t>(0xbfd2bec3u)) {  // -0.2929 < x < 0.41422
            k = 0;
            f = x;
            hu = 1;
        }
    } else if (hx >= 0x7ff00000) {
        return x + x;
    }
    if (k != 0) {
        if (hx < 0x43400000) {
            u = 1.0 + x;
            hu = static_cast<int32_t>(hi32(u));
            k = (hu >> 20) - 1023;
            c = k > 0 ? 1.0 - (u - x) : x - (u - 1.0);  // the rounding error of 1 + x
            c /= u;
        } else {
            u = x;
            hu = static_cast<int32_t>(hi32(u));
            k = (hu >> 20) - 1023;
            c = 0.0;
        }
        hu &= 0x000fffff;
        if (hu < 0x6a09e) {
            u = with_hi(u, static_cast<uint32_t>(hu) | 0x3ff00000u);
        } else {
            k += 1;
            u = with_hi(u, static_cast<uint32_t>(hu) | 0x3fe00000u);
            hu = (0x00100000 - hu) >> 2;
        }
        f = u - 1.0;
    }
    const double kd = static_cast<double>(k);
    const double hfsq = 0.5 * f * f;
    if (hu == 0) {  // |f| < 2^-20
        if (f == 0.0) {
            if (k == 0) return 0.0;
            c = fmad(kd, ln2_lo, c);
            return fmad(kd, ln2_hi, c);
        }
        const double R = hfsq * fmad(-0.66666666666666666, f, 1.0);
        if (k == 0) return f - R;
        return fmad(kd, ln2_hi, -((R - fmad(kd, ln2_lo, c)) - f));
    }
    const double s = f / (2.0 + f);
    const double z = s * s;
    const double z2 = z * z;
    const double R2 = fmad(z, Lp3, Lp2), z4 = z2 * z2;
    const double R3 = fmad(z, Lp5, Lp4), z6 = z4 * z2;
    const double R4 = fmad(z, Lp7, Lp6);
    const double R = fmad(z6, R4, fmad(z4, R3, fmad(z, Lp1, z2 * R2)));
    const double shared = s * (hfsq + R);  // (common to both branches: one rounded product)
    if (k == 0) return f - (hfsq - shared);
    return fmad(kd, ln2_hi, -((hfsq - (shared + fmad(kd, ln2_lo, c))) - f));
}

}  // namespace lm64
}  // namespace hmc
