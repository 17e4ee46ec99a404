// Compares the restated double-precision functions of homura_b200/csrc/libm64.cuh, compiled for the host, with the
// host C library's own on seeded arguments: a quarter random bit patterns, a quarter uniform over the function's whole
// finite range, a quarter uniform in (-2, 2) and a quarter in (-0.25, 0.25), plus a list of special values. Prints
// "<function> <arguments compared> <mismatches>" per function and exits non-zero when any differ. A NaN only has
// to meet a NaN.
//
//   g++ -O2 -std=c++17 -ffp-contract=off -mfma -fopenmp libm64_check.cpp -o libm64_check
//   ./libm64_check [arguments per function = 2^28]
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "../../homura_b200/csrc/libm64.cuh"

namespace lm = hmc::lm64;

static inline bool same(double a, double b) {
    if (a != a && b != b) return true;
    return lm::d2u(a) == lm::d2u(b);
}

static inline uint64_t mix(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

static inline double argument(long long i, double span, uint64_t seed) {
    const uint64_t w = mix(static_cast<uint64_t>(i) * 0x2545F4914F6CDD1Dull + seed);
    const double u = static_cast<double>(static_cast<int64_t>(w >> 11)) * 0x1p-53 - 0.5;
    switch (i & 3) {
        case 0: return lm::u2d(w);
        case 1: return u * 2.0 * span;
        case 2: return u * 4.0;
        default: return u * 0.5;
    }
}

template <class Mine, class Theirs>
static long long sweep(const char *name, Mine mine, Theirs theirs, long long count, double span, uint64_t seed) {
    const double special[] = {0.0, -0.0, 1.0, -1.0, 0.5, -0.5, 2.0, -2.0, 22.0, -22.0, 1e-300, -1e-300, 5e-324, -5e-324, 0x1p-54,
                              -0x1p-54, 0x1p-29, 708.0, 709.78, 709.79, 710.0, -708.0, -745.0, -745.2, -746.0, 1e308, -1e308,
                              INFINITY, -INFINITY, NAN, 0.41421, 0.41422, -0.2929, -0.29291, 0.34657, 1.0397, 38.8, -38.8};
    long long bad = 0, compared = 0;
    double first = 0.0;
    bool have = false;
    for (double x : special) {
        ++compared;
        if (!same(mine(x), theirs(x))) {
            ++bad;
            if (!have) { first = x; have = true; }
        }
    }
#pragma omp parallel for schedule(static) reduction(+ : bad, compared)
    for (long long i = 0; i < count; ++i) {
        const double x = argument(i, span, seed);
        ++compared;
        if (!same(mine(x), theirs(x))) {
            ++bad;
#pragma omp critical
            if (!have) { first = x; have = true; }
        }
    }
    printf("%s %lld %lld", name, compared, bad);
    if (have) printf("  first %a: mine %a theirs %a", first, mine(first), theirs(first));
    printf("\n");
    return bad;
}

int main(int argc, char **argv) {
    const long long count = argc > 1 ? atoll(argv[1]) : (1ll << 28);
    long long bad = 0;
    bad += sweep("exp", [](double x) { return lm::exp(x); }, [](double x) { return std::exp(x); }, count, 750.0, 1);
    bad += sweep("expm1", [](double x) { return lm::expm1(x); }, [](double x) { return std::expm1(x); }, count, 720.0, 2);
    bad += sweep("tanh", [](double x) { return lm::tanh(x); }, [](double x) { return std::tanh(x); }, count, 25.0, 3);
    bad += sweep("log1p", [](double x) { return lm::log1p(x); }, [](double x) { return std::log1p(x); }, count, 1e6, 4);
    return bad != 0;
}
