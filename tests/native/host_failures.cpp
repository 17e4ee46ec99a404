// Failure paths of the library's host code that a real GPU cannot be made to produce on demand: CUDA calls that
// fail during clean-up or for lack of device memory, what such failures leave as the thread's last CUDA error, a
// host heap that stays exhausted, and the caching allocator's release-and-retry over a device that refuses
// segments. runtime.cu, memory.cu and caching.cu are compiled with g++ against the stand-in runtime of
// tests/fake_cuda, and operator new is replaced so that a mode can make every host allocation fail. Each mode
// runs in its own process (tests/test_host_failures.py), so that an abort (an exception escaping a noexcept
// function) fails only that mode. After homura's csrc/tests/host_failures.cpp; not part of the library.
//
//   g++ -std=c++17 -DHMC_FAKE_CUDA -I tests/fake_cuda -x c++ tests/native/host_failures.cpp -o host_failures
//   ./host_failures --list | ./host_failures <mode>
#if defined(__GNUC__) && !defined(__clang__)
#pragma GCC diagnostic ignored "-Wmismatched-new-delete"
#endif

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <stdexcept>

#include "../../homura_b200/csrc/runtime.cu"
#include "../../homura_b200/csrc/memory.cu"
#include "../../homura_b200/csrc/caching.cu"

void *operator new(std::size_t n) {
    if (fake::deny_new) throw std::bad_alloc();
    if (void *p = std::malloc(n ? n : 1)) return p;
    throw std::bad_alloc();
}
void *operator new[](std::size_t n) { return operator new(n); }
void *operator new(std::size_t n, const std::nothrow_t &) noexcept { return fake::deny_new ? nullptr : std::malloc(n ? n : 1); }
void *operator new[](std::size_t n, const std::nothrow_t &) noexcept { return fake::deny_new ? nullptr : std::malloc(n ? n : 1); }
void operator delete(void *p) noexcept { std::free(p); }
void operator delete[](void *p) noexcept { std::free(p); }
void operator delete(void *p, std::size_t) noexcept { std::free(p); }
void operator delete[](void *p, std::size_t) noexcept { std::free(p); }

// The device part of hmc_reduce_noalloc is not in this build: its address look-up always succeeds.
namespace hmc {
hmc_status noalloc_scratch_on(int, void **out) {
    if (out != nullptr) *out = nullptr;
    return HMC_OK;
}
}  // namespace hmc

namespace {

int failures = 0;

// (checks allocate nothing: some run while operator new throws)
#define CHECK(cond)                                                                        \
    do {                                                                                   \
        if (!(cond)) {                                                                     \
            std::fprintf(stderr, "%s:%d: check failed: %s\n", __FILE__, __LINE__, #cond); \
            ++failures;                                                                    \
        }                                                                                  \
    } while (0)
#define CHECK_ERROR(expected)                                                                                   \
    do {                                                                                                        \
        const char *actual_ = hmc_last_error();                                                                 \
        if (std::strcmp(actual_, expected) != 0) {                                                              \
            std::fprintf(stderr, "%s:%d: last error is \"%s\", expected \"%s\"\n", __FILE__, __LINE__, actual_, expected); \
            ++failures;                                                                                         \
        }                                                                                                       \
    } while (0)
#define CHECK_ERROR_HAS(piece)                                                                                   \
    do {                                                                                                         \
        const char *actual_ = hmc_last_error();                                                                  \
        if (std::strstr(actual_, piece) == nullptr) {                                                            \
            std::fprintf(stderr, "%s:%d: last error \"%s\" lacks \"%s\"\n", __FILE__, __LINE__, actual_, piece); \
            ++failures;                                                                                          \
        }                                                                                                        \
    } while (0)
// The streams the runtime holds agree with what the library counts for this thread.
#define CHECK_STREAMS(n)                          \
    do {                                          \
        CHECK(fake::live_streams == (n));         \
        CHECK(hmc_test_live_streams() == (n));    \
    } while (0)

// After a failure: nothing of it is left as the thread's last CUDA error, and a context can still be created
// and destroyed, leaving the thread on its own device.
void create_and_destroy() {
    CHECK(fake::last_error == cudaSuccess);
    fake::launch_error = cudaSuccess;
    fake::destroy_error = cudaSuccess;
    const int before = fake::live_streams;
    hmc_context_t ctx = nullptr;
    CHECK(hmc_context_create(0, &ctx) == HMC_OK);
    CHECK(ctx != nullptr);
    CHECK_STREAMS(before + 1);
    CHECK(hmc_context_destroy(ctx) == HMC_OK);
    CHECK_STREAMS(before);
    CHECK(fake::current_device == 1);
}

// Context creation fails after the stream exists: the stream is destroyed on device 0, before the thread is put
// back on device 1.
void late_failure() {
    hmc_test_fail_after_probe(1);
    hmc_context_t ctx = reinterpret_cast<hmc_context_t>(1);
    CHECK(hmc_context_create(0, &ctx) == HMC_OUT_OF_MEMORY);
    CHECK(ctx == nullptr);
    CHECK_ERROR("out of host memory");
    CHECK_STREAMS(0);
    CHECK(fake::destroyed_on == 0);
    CHECK(fake::current_device == 1);
    create_and_destroy();
}

void probe_failure() {
    fake::launch_error = cudaErrorMemoryAllocation;
    hmc_context_t ctx = nullptr;
    CHECK(hmc_context_create(0, &ctx) == HMC_OUT_OF_MEMORY);
    CHECK(ctx == nullptr);
    CHECK_ERROR("probe kernel: out of memory");
    CHECK_STREAMS(0);
    CHECK(fake::destroyed_on == 0);
    CHECK(fake::current_device == 1);
    create_and_destroy();
}

// The probe fails and so does destroying the stream: the probe's error is the one reported, and the stream the
// runtime still holds stays counted.
void probe_then_destroy_failure() {
    fake::launch_error = cudaErrorMemoryAllocation;
    fake::destroy_error = cudaErrorInvalidResourceHandle;
    hmc_context_t ctx = nullptr;
    CHECK(hmc_context_create(0, &ctx) == HMC_OUT_OF_MEMORY);
    CHECK(ctx == nullptr);
    CHECK_ERROR("probe kernel: out of memory");
    CHECK_STREAMS(1);
    CHECK(fake::current_device == 1);
    create_and_destroy();
}

// Destroying the stream fails while no host memory is left: nothing escapes the clean-up, the first error stands.
void destroy_failure_without_memory() {
    hmc_test_fail_after_probe(1);
    fake::destroy_error = cudaErrorInvalidResourceHandle;
    fake::deny_new_after_destroy = true;
    hmc_context_t ctx = nullptr;
    CHECK(hmc_context_create(0, &ctx) == HMC_OUT_OF_MEMORY);
    CHECK(ctx == nullptr);
    CHECK_ERROR("out of host memory");
    CHECK_STREAMS(1);
    CHECK(fake::current_device == 1);
    fake::deny_new_after_destroy = false;
    fake::deny_new = false;
    create_and_destroy();
}

// The explicit destroy reports its own failure and counts the stream the runtime kept.
void destroy_failure() {
    hmc_context_t ctx = nullptr;
    CHECK(hmc_context_create(0, &ctx) == HMC_OK);
    fake::destroy_error = cudaErrorInvalidResourceHandle;
    CHECK(hmc_context_destroy(ctx) == HMC_CUDA_ERROR);
    CHECK_ERROR("cudaStreamDestroy: invalid resource handle");
    CHECK_STREAMS(1);
    CHECK(fake::current_device == 1);
    create_and_destroy();
}

// The same while no host memory is left: status and text are still the CUDA error's (recording a message needs
// no allocation).
void destroy_failure_without_memory_explicit() {
    hmc_context_t ctx = nullptr;
    CHECK(hmc_context_create(0, &ctx) == HMC_OK);
    fake::destroy_error = cudaErrorInvalidResourceHandle;
    fake::deny_new_after_destroy = true;
    CHECK(hmc_context_destroy(ctx) == HMC_CUDA_ERROR);
    CHECK_ERROR("cudaStreamDestroy: invalid resource handle");
    CHECK_STREAMS(1);
    CHECK(fake::current_device == 1);
    fake::deny_new_after_destroy = false;
    fake::deny_new = false;
    create_and_destroy();
}

// The probe fails and host memory runs out from then on: the probe's error is still reported in full.
void probe_failure_without_memory() {
    fake::launch_error = cudaErrorInvalidResourceHandle;
    fake::deny_new_after_launch = true;
    hmc_context_t ctx = nullptr;
    CHECK(hmc_context_create(0, &ctx) == HMC_CUDA_ERROR);
    CHECK(ctx == nullptr);
    CHECK_ERROR("probe kernel: invalid resource handle");
    CHECK_STREAMS(0);
    CHECK(fake::current_device == 1);
    fake::deny_new_after_launch = false;
    fake::deny_new = false;
    create_and_destroy();
}

// Host memory runs out for good: entry points return HMC_OUT_OF_MEMORY instead of aborting, messages are still
// recorded (they need no allocation), and everything works again once memory is back.
void persistent_oom() {
    fake::deny_new = true;
    hmc_context_t ctx = nullptr;
    CHECK(hmc_context_create(0, &ctx) == HMC_OUT_OF_MEMORY);
    CHECK(ctx == nullptr);
    CHECK_ERROR("out of host memory");
    CHECK(hmc_test_fail("a message longer than any small-string buffer, recorded without the heap") == HMC_INVALID);
    CHECK_ERROR("a message longer than any small-string buffer, recorded without the heap");
    CHECK(hmc_context_create(7, &ctx) == HMC_OUT_OF_MEMORY);  // (its message is built on the heap)
    CHECK_ERROR("out of host memory");
    hmc_allocator_t alloc = nullptr;
    hmc_memory_ops ops{nullptr, [](void *, uint64_t, uint64_t *) { return HMC_MEM_OUT_OF_MEMORY; },
                       [](void *, uint64_t) { return HMC_MEM_OK; }, [](void *) { return HMC_MEM_OK; }};
    CHECK(hmc_allocator_create(&ops, &alloc) == HMC_OUT_OF_MEMORY);
    CHECK_STREAMS(0);
    fake::deny_new = false;
    CHECK(hmc_test_fail("a message recorded once memory is back") == HMC_INVALID);
    CHECK_ERROR("a message recorded once memory is back");
    create_and_destroy();
}

// Another exception from an entry point's body, with and without host memory.
void exception_without_memory() {
    const std::runtime_error error("the body's error");
    auto body = [&]() -> hmc_status { throw error; };
    CHECK(hmc::guarded(body) == HMC_INTERNAL_ERROR);
    CHECK_ERROR("internal error: the body's error");
    fake::deny_new = true;
    CHECK(hmc_test_fail("") == HMC_INVALID);
    CHECK(hmc::guarded(body) == HMC_INTERNAL_ERROR);
    CHECK_ERROR("internal error: the body's error");
    auto odd = [&]() -> hmc_status { throw 42; };
    CHECK(hmc::guarded(odd) == HMC_INTERNAL_ERROR);
    CHECK_ERROR("internal error");
    fake::deny_new = false;
}

// The probe's own cudaMalloc fails: out of memory, and the retry right after it on this thread succeeds, since
// the failure does not stay as the last error that the next probe's launch check reads.
void probe_malloc_failure_then_retry() {
    fake::malloc_failures = 1;
    hmc_context_t ctx = nullptr;
    CHECK(hmc_context_create(0, &ctx) == HMC_OUT_OF_MEMORY);
    CHECK(ctx == nullptr);
    CHECK_ERROR("probe: cudaMalloc: out of memory");
    CHECK_STREAMS(0);
    create_and_destroy();
}

// An error that the caller's own CUDA calls left on this thread does not fail the probe's launch check, nor the
// submission of a later operation.
void earlier_error_before_the_probe() {
    fake::last_error = cudaErrorInvalidResourceHandle;
    hmc_context_t ctx = nullptr;
    CHECK(hmc_context_create(0, &ctx) == HMC_OK);
    void *p = nullptr;
    CHECK(hmc_malloc(0, 64, &p) == HMC_OK);
    fake::last_error = cudaErrorInvalidValue;
    CHECK(hmc_memset(ctx, p, 1, 64) == HMC_OK);
    CHECK(fake::last_error == cudaSuccess);
    CHECK(hmc_free(0, p) == HMC_OK);
    CHECK(hmc_context_destroy(ctx) == HMC_OK);
    create_and_destroy();
}

void malloc_failure() {
    fake::malloc_failures = 1;
    void *p = reinterpret_cast<void *>(1);
    CHECK(hmc_malloc(0, 4096, &p) == HMC_OUT_OF_MEMORY);
    CHECK(p == nullptr);
    CHECK_ERROR("cudaMalloc: out of memory");
    CHECK(fake::current_device == 1);
    CHECK(fake::last_error == cudaSuccess);
    CHECK(hmc_malloc(0, 4096, &p) == HMC_OK);
    CHECK(p != nullptr);
    CHECK(hmc_free(0, p) == HMC_OK);
    create_and_destroy();
}

// Queuing a fill fails for lack of memory: HMC_OUT_OF_MEMORY, nothing left as the last error, and the next
// submission works; the byte is the one asked for.
void memset_failure() {
    hmc_context_t ctx = nullptr;
    CHECK(hmc_context_create(0, &ctx) == HMC_OK);
    void *p = nullptr;
    CHECK(hmc_malloc(0, 64, &p) == HMC_OK);
    std::memset(p, 0xab, 64);
    fake::memset_error = cudaErrorMemoryAllocation;
    CHECK(hmc_memset(ctx, p, 0, 64) == HMC_OUT_OF_MEMORY);
    CHECK_ERROR("cudaMemsetAsync: out of memory");
    CHECK(fake::last_error == cudaSuccess);
    CHECK(fake::current_device == 1);
    fake::memset_error = cudaSuccess;
    CHECK(hmc_memset(ctx, p, 0, 64) == HMC_OK);
    const unsigned char zeros[64] = {};
    CHECK(std::memcmp(p, zeros, 64) == 0);
    CHECK(hmc_memset(ctx, p, 0xff, 64) == HMC_OK);
    unsigned char ones[64];
    std::memset(ones, 0xff, 64);
    CHECK(std::memcmp(p, ones, 64) == 0);
    CHECK(hmc_free(0, p) == HMC_OK);
    CHECK(hmc_context_destroy(ctx) == HMC_OK);
    create_and_destroy();
}

// The caching allocator over the (stand-in) device: a refused segment makes it wait for the stream, give its
// wholly free segments back and try exactly once more; when that fails too the message is the out-of-memory
// report with the device's numbers, the counters are unchanged, and the next request works.
void allocator_release_and_retry() {
    hmc_context_t ctx = nullptr;
    CHECK(hmc_context_create(0, &ctx) == HMC_OK);
    hmc_allocator_t a = nullptr;
    CHECK(hmc_allocator_create_cuda(ctx, &a) == HMC_OK);
    uint64_t big = 0, size = 0;
    CHECK(hmc_allocator_allocate(a, 8u << 20, &big, &size) == HMC_OK);
    CHECK(size == (8u << 20));
    CHECK(hmc_allocator_release(a, big) == HMC_OK);  // cached: an 8 MiB segment, wholly free
    hmc_memory_stats st{};
    CHECK(hmc_allocator_stats(a, &st) == HMC_OK);
    CHECK(st.allocated == 0 && st.reserved == (8u << 20));
    // a larger request: the device refuses once; the cached segment goes back (after a wait), the retry succeeds
    const int frees = fake::frees, syncs = fake::synchronizes, mallocs = fake::mallocs;
    fake::malloc_failures = 1;
    uint64_t other = 0;
    CHECK(hmc_allocator_allocate(a, 16u << 20, &other, &size) == HMC_OK);
    CHECK(fake::frees == frees + 1 && fake::synchronizes > syncs && fake::mallocs == mallocs + 2);
    CHECK(hmc_allocator_stats(a, &st) == HMC_OK);
    CHECK(st.allocated == (16u << 20) && st.reserved == (16u << 20));
    CHECK(fake::last_error == cudaSuccess);
    // the device refuses for good: one retry, then the report
    fake::malloc_always_fails = true;
    const int before = fake::mallocs;
    uint64_t none = 1;
    CHECK(hmc_allocator_allocate(a, 32u << 20, &none, &size) == HMC_OUT_OF_MEMORY);
    CHECK(fake::mallocs == before + 2);
    CHECK_ERROR_HAS("CUDA out of memory. Tried to allocate 32.00 MiB. cuda:0 has a total capacity of 32.00 GiB");
    CHECK_ERROR_HAS("16.00 MiB is allocated by homura");
    CHECK(hmc_allocator_stats(a, &st) == HMC_OK);
    CHECK(st.allocated == (16u << 20) && st.reserved == (16u << 20));
    CHECK(fake::last_error == cudaSuccess);
    fake::malloc_always_fails = false;
    CHECK(hmc_allocator_allocate(a, 32u << 20, &none, &size) == HMC_OK);
    CHECK(hmc_allocator_release(a, none) == HMC_OK);
    CHECK(hmc_allocator_release(a, other) == HMC_OK);
    CHECK(hmc_allocator_release(a, other) == HMC_INVALID);
    CHECK_ERROR("freeing a block twice");
    CHECK(hmc_allocator_destroy(a) == HMC_OK);
    CHECK(hmc_context_destroy(ctx) == HMC_OK);
    create_and_destroy();
}

// The wait before segments go back fails: the allocation reports that failure, keeps its cache, and works again
// once the stream answers.
void allocator_synchronize_failure() {
    hmc_context_t ctx = nullptr;
    CHECK(hmc_context_create(0, &ctx) == HMC_OK);
    hmc_allocator_t a = nullptr;
    CHECK(hmc_allocator_create_cuda(ctx, &a) == HMC_OK);
    uint64_t big = 0, size = 0;
    CHECK(hmc_allocator_allocate(a, 8u << 20, &big, &size) == HMC_OK);
    CHECK(hmc_allocator_release(a, big) == HMC_OK);
    fake::malloc_failures = 1;
    fake::synchronize_error = cudaErrorInvalidResourceHandle;
    uint64_t other = 0;
    const hmc_status s = hmc_allocator_allocate(a, 16u << 20, &other, &size);
    CHECK(s == HMC_CUDA_ERROR);
    CHECK_ERROR_HAS("cudaStreamSynchronize: invalid resource handle");
    CHECK(fake::last_error == cudaSuccess);
    fake::synchronize_error = cudaSuccess;
    hmc_memory_stats st{};
    CHECK(hmc_allocator_stats(a, &st) == HMC_OK);
    CHECK(st.allocated == 0 && st.reserved == (8u << 20));
    CHECK(hmc_allocator_allocate(a, 16u << 20, &other, &size) == HMC_OK);
    CHECK(hmc_allocator_release(a, other) == HMC_OK);
    CHECK(hmc_allocator_destroy(a) == HMC_OK);
    CHECK(hmc_context_destroy(ctx) == HMC_OK);
    create_and_destroy();
}

struct Mode {
    const char *name;
    void (*run)();
};

const Mode modes[] = {
    {"late-failure", late_failure},
    {"probe-failure", probe_failure},
    {"probe-then-destroy-failure", probe_then_destroy_failure},
    {"destroy-failure-without-memory", destroy_failure_without_memory},
    {"destroy-failure", destroy_failure},
    {"destroy-failure-without-memory-explicit", destroy_failure_without_memory_explicit},
    {"probe-failure-without-memory", probe_failure_without_memory},
    {"persistent-oom", persistent_oom},
    {"exception-without-memory", exception_without_memory},
    {"probe-malloc-failure-then-retry", probe_malloc_failure_then_retry},
    {"earlier-error-before-the-probe", earlier_error_before_the_probe},
    {"malloc-failure", malloc_failure},
    {"memset-failure", memset_failure},
    {"allocator-release-and-retry", allocator_release_and_retry},
    {"allocator-synchronize-failure", allocator_synchronize_failure},
};

}  // namespace

int main(int argc, char **argv) {
    if (argc == 2 && std::strcmp(argv[1], "--list") == 0) {
        for (const Mode &m : modes) std::printf("%s\n", m.name);
        return 0;
    }
    if (argc != 2) {
        std::fprintf(stderr, "usage: host_failures --list | <mode>\n");
        return 2;
    }
    for (const Mode &m : modes) {
        if (std::strcmp(argv[1], m.name) == 0) {
            m.run();
            return failures == 0 ? 0 : 1;
        }
    }
    std::fprintf(stderr, "unknown mode %s\n", argv[1]);
    return 2;
}
