// TEST INFRASTRUCTURE. A stand-in for the HIP runtime header, just enough to compile homura's cast header
// (csrc/elem.hpp) for the host: the device qualifier disappears and the five bit-cast / conversion
// intrinsics it uses become their host equivalents.
#pragma once
#include <cstdint>
#include <cstring>

#define __device__
#define __host__

inline long long __double_as_longlong(double v) { long long b; std::memcpy(&b, &v, 8); return b; }
inline double __longlong_as_double(long long b) { double v; std::memcpy(&v, &b, 8); return v; }
inline uint32_t __float_as_uint(float v) { uint32_t b; std::memcpy(&b, &v, 4); return b; }
inline float __uint_as_float(uint32_t b) { float v; std::memcpy(&v, &b, 4); return v; }
// round to nearest even; x86's cvtsd2ss keeps a NaN's top payload bits and makes it quiet
inline float __double2float_rn(double v) { return static_cast<float>(v); }
