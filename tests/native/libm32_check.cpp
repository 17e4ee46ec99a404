// Compares the restated single-precision functions of homura_b200/csrc/libm32.cuh, compiled for the host,
// with the host C library's own: every float argument (or every stride-th one) for the unary functions,
// random and special pairs for powf. Prints "<function> <arguments compared> <mismatches>" per function and
// exits non-zero when any differ. A NaN only has to meet a NaN.
//
//   g++ -O2 -std=c++17 -ffp-contract=off -mfma -fopenmp libm32_check.cpp -o libm32_check
//   ./libm32_check [stride=1] [pairs=2^28] [function ...]
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../../homura_b200/csrc/libm32.cuh"

namespace lm = hmc::lm;

static inline bool same(float a, float b) {
    if (a != a && b != b) return true;
    return lm::f2u(a) == lm::f2u(b);
}

template <class Mine, class Theirs>
static long long sweep(const char *name, Mine mine, Theirs theirs, unsigned long long stride) {
    long long bad = 0;
    unsigned first = 0;
    bool have = false;
#pragma omp parallel for schedule(static) reduction(+ : bad)
    for (long long b = 0; b < (1ll << 32); b += (long long)stride) {
        const float x = lm::u2f((uint32_t)b);
        const float m = mine(x), t = theirs(x);
        if (!same(m, t)) {
            ++bad;
#pragma omp critical
            if (!have || (uint32_t)b < first) {
                first = (uint32_t)b;
                have = true;
            }
        }
    }
    printf("%s %lld %lld", name, (long long)(((1ull << 32) + stride - 1) / stride), bad);
    if (have) {
        const float x = lm::u2f(first);
        printf("  first %#x (%a): mine %a theirs %a", first, x, mine(x), theirs(x));
    }
    printf("\n");
    return bad;
}

static inline uint64_t mix(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

static long long pow_pairs(long long pairs) {
    const float special[] = {0.0f, -0.0f, 1.0f, -1.0f, 2.0f, -2.0f, 0.5f, -0.5f, 3.0f, -3.0f, 1.5f, -1.5f, 1e-45f, -1e-45f,
                             1e-40f, 1.1754944e-38f, 3.4028235e38f, -3.4028235e38f, INFINITY, -INFINITY, NAN, 1e10f, -1e10f,
                             16777216.0f, 16777217.0f, -16777216.0f, 8388607.5f, 127.0f, 128.0f, -149.0f, -150.0f, 0.99999994f,
                             1.0000001f, 88.0f, -104.0f, 2147483648.0f, 4294967296.0f, 0.1f, 10.0f, 1e-3f, 7.0f, -7.0f};
    const int ns = sizeof(special) / sizeof(special[0]);
    long long bad = 0, total = 0;
    for (int i = 0; i < ns; ++i)
        for (int j = 0; j < ns; ++j) {
            ++total;
            if (!same(lm::powf(special[i], special[j]), ::powf(special[i], special[j]))) {
                if (bad < 5)
                    printf("  powf(%a, %a): mine %a theirs %a\n", special[i], special[j], lm::powf(special[i], special[j]),
                           ::powf(special[i], special[j]));
                ++bad;
            }
        }
    long long rb = 0;
#pragma omp parallel for schedule(static) reduction(+ : rb)
    for (long long n = 0; n < pairs; ++n) {
        const uint64_t w = mix((uint64_t)n);
        float x, y;
        switch (n & 3) {
            case 0:  // any two bit patterns
                x = lm::u2f((uint32_t)w);
                y = lm::u2f((uint32_t)(w >> 32));
                break;
            case 1:  // positive base near 1, large exponents: results spread over the whole range
                x = lm::u2f(0x3f000000u + (uint32_t)(w & 0xffffffu));
                y = (float)((double)(int64_t)(w >> 40) / 4096.0 - 2048.0);
                break;
            case 2:  // moderate base and exponent
                x = (float)((double)(w & 0xffffffu) / 65536.0 + 1e-3);
                y = (float)((double)((w >> 24) & 0xffffffu) / 1048576.0 - 8.0);
                break;
            default:  // negative bases with integer exponents, subnormal bases
                x = (w & 1) ? -(float)((double)((w >> 1) & 0xffffu) / 256.0) : lm::u2f((uint32_t)(w >> 1) & 0x7fffffu);
                y = (float)(int)((w >> 40) % 41) - 20.0f;
                break;
        }
        if (!same(lm::powf(x, y), ::powf(x, y))) {
            ++rb;
            if (rb < 3) printf("  powf(%a, %a): mine %a theirs %a\n", x, y, lm::powf(x, y), ::powf(x, y));
        }
    }
    printf("powf %lld %lld\n", total + pairs, bad + rb);
    return bad + rb;
}

int main(int argc, char **argv) {
    const unsigned long long stride = argc > 1 ? strtoull(argv[1], nullptr, 10) : 1;
    const long long pairs = argc > 2 ? atoll(argv[2]) : (1ll << 28);
    std::vector<std::string> which;
    for (int i = 3; i < argc; ++i) which.push_back(argv[i]);
    auto wanted = [&](const char *n) {
        if (which.empty()) return true;
        for (auto &w : which)
            if (w == n) return true;
        return false;
    };
    long long bad = 0;
    if (wanted("expf")) bad += sweep("expf", [](float x) { return lm::expf(x); }, [](float x) { return ::expf(x); }, stride);
    if (wanted("logf")) bad += sweep("logf", [](float x) { return lm::logf(x); }, [](float x) { return ::logf(x); }, stride);
    if (wanted("expm1f")) bad += sweep("expm1f", [](float x) { return lm::expm1f(x); }, [](float x) { return ::expm1f(x); }, stride);
    if (wanted("tanhf")) bad += sweep("tanhf", [](float x) { return lm::tanhf(x); }, [](float x) { return ::tanhf(x); }, stride);
    if (wanted("log1pf")) bad += sweep("log1pf", [](float x) { return lm::log1pf(x); }, [](float x) { return ::log1pf(x); }, stride);
    // powf with the exponent 2, through a variable the compiler cannot see through (it would turn powf(x, 2.0f)
    // into x * x, which the library's powf does not always return: it is within 0.82 ulp, not correctly rounded)
    if (wanted("powf2")) {
        static volatile float two = 2.0f;
        bad += sweep("powf2", [](float x) { return lm::powf(x, two); }, [](float x) { return ::powf(x, two); }, stride);
    }
    if (wanted("powf")) bad += pow_pairs(pairs);
    return bad ? 1 : 0;
}
