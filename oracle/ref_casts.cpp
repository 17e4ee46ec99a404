// TEST INFRASTRUCTURE. Compiles homura's own C++ restatement of its casts (csrc/elem.hpp, included from where
// homura's sources are mounted; nothing of it is copied here) for the host and exposes it as one function,
// so that the oracle's conversions can be checked against the reference's code on any bit patterns.
#include <cstdint>

#include "elem.hpp"

namespace {
template <int D, int S>
void run(const void *in, void *out, int64_t n) {
    using TS = typename hmr::Elem<S>::T;
    using TD = typename hmr::Elem<D>::T;
    const TS *p = static_cast<const TS *>(in);
    TD *q = static_cast<TD *>(out);
    for (int64_t i = 0; i < n; ++i) q[i] = hmr::convert<D, S>(p[i]);
}
template <int S>
int from(int dst, const void *in, void *out, int64_t n) {
    switch (dst) {
        case 0: run<0, S>(in, out, n); return 0;
        case 1: run<1, S>(in, out, n); return 0;
        case 2: run<2, S>(in, out, n); return 0;
        case 3: run<3, S>(in, out, n); return 0;
        case 4: run<4, S>(in, out, n); return 0;
        case 5: run<5, S>(in, out, n); return 0;
        case 6: run<6, S>(in, out, n); return 0;
        case 7: run<7, S>(in, out, n); return 0;
        case 8: run<8, S>(in, out, n); return 0;
        case 9: run<9, S>(in, out, n); return 0;
    }
    return 2;
}
}  // namespace

extern "C" int ref_convert(int dst, int src, const void *in, void *out, int64_t n) {
    switch (src) {
        case 0: return from<0>(dst, in, out, n);
        case 1: return from<1>(dst, in, out, n);
        case 2: return from<2>(dst, in, out, n);
        case 3: return from<3>(dst, in, out, n);
        case 4: return from<4>(dst, in, out, n);
        case 5: return from<5>(dst, in, out, n);
        case 6: return from<6>(dst, in, out, n);
        case 7: return from<7>(dst, in, out, n);
        case 8: return from<8>(dst, in, out, n);
        case 9: return from<9>(dst, in, out, n);
    }
    return 2;
}
