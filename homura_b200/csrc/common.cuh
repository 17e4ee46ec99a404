// Shared host-side plumbing of the library: status and per-thread error text, the exception
// barrier every entry point runs behind, device switching, the context object and the hooks that
// let tests inject failures without touching a GPU.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <exception>
#include <new>
#include <string>

#include "../../include/homura_cuda.h"

#define HMC_API extern "C" __attribute__((visibility("default")))

namespace hmc {
struct TraceState;
constexpr int kTickets = 1024;       // counters per context
constexpr int kTicketsOffset = 64;   // words between the status word and the first counter (same allocation)
}
struct hmc_context {
    int32_t device;
    cudaStream_t stream;
    int32_t sm_count;
    hmc::TraceState *trace;  // per-call timing records, when the timing log is on (else null)
    int *status;             // a word in device memory that a kernel sets when one of its bounded waits runs out
    unsigned *tickets;       // hmc::kTickets counters in device memory, zero between kernels: the blocks of a reduction that
                             // share partials count themselves off on one, and the last resets it
};

struct hmc_event {
    int32_t device;
    cudaEvent_t event;
};

namespace hmc {

// The calling thread's last error text, in storage that exists from the thread's first call: recording a
// message never allocates, so it also works when the host heap is exhausted (texts beyond the capacity are cut).
class Message {
  public:
    void assign(const char *text) noexcept { std::snprintf(text_, sizeof text_, "%s", text != nullptr ? text : ""); }
    void clear() noexcept { text_[0] = '\0'; }
    const char *c_str() const noexcept { return text_; }

  private:
    char text_[1024] = {};
};

// ---- per-thread state ----
struct ThreadState {
    Message message;
    int fail_stream_create = 0;
    int fail_after_probe = 0;
    int fail_properties = 0;
    int fail_data = 0;
    bool fail_data_oom = false;
    int live_streams = 0;
};
ThreadState &thread_state();

// Records `message` for the calling thread and returns `status`. The form taking a C string allocates nothing.
hmc_status fail(hmc_status status, const char *message) noexcept;
hmc_status fail(hmc_status status, const std::string &message) noexcept;

// Turns a CUDA error into a status (out of memory is its own status), records "<what>: <text>" and
// clears the runtime's sticky last-error so that the failure does not resurface in a later,
// unrelated call of the user's program.
hmc_status cuda_fail(cudaError_t err, const char *what);

#define HMC_CUDA(call, what)                                      \
    do {                                                          \
        cudaError_t hmc_err_ = (call);                            \
        if (hmc_err_ != cudaSuccess) return ::hmc::cuda_fail(hmc_err_, what); \
    } while (0)

// Runs `body` (returning hmc_status) so that no C++ exception reaches the caller. The handlers allocate nothing
// (the message store is fixed storage), so they cannot throw in turn when the host heap is exhausted.
template <class Body>
hmc_status guarded(Body &&body) noexcept {
    try {
        return body();
    } catch (const std::bad_alloc &) {
        return fail(HMC_OUT_OF_MEMORY, "out of host memory");
    } catch (const std::exception &e) {
        char text[512];
        std::snprintf(text, sizeof text, "internal error: %s", e.what());
        return fail(HMC_INTERNAL_ERROR, text);
    } catch (...) {
        return fail(HMC_INTERNAL_ERROR, "internal error");
    }
}

// Makes `device` current for its lifetime and restores whatever was current before.
class DeviceGuard {
  public:
    explicit DeviceGuard(int device);
    ~DeviceGuard();
    DeviceGuard(const DeviceGuard &) = delete;
    DeviceGuard &operator=(const DeviceGuard &) = delete;
    hmc_status status() const { return status_; }

  private:
    int previous_ = -1;
    bool switched_ = false;
    hmc_status status_ = HMC_OK;
};

// The injected failure of a data operation, if one is armed for this thread: returns true and sets
// `status`. Called before anything is queued.
bool injected_data_failure(hmc_status &status);

// Checks the context pointer, arms the device guard, consumes an injected failure. Expands in an
// entry point body (which returns hmc_status).
#define HMC_ENTER(ctx)                                                              \
    if ((ctx) == nullptr) return ::hmc::fail(HMC_INVALID, "null context");         \
    {                                                                               \
        hmc_status hmc_inj_;                                                        \
        if (::hmc::injected_data_failure(hmc_inj_)) return hmc_inj_;               \
    }                                                                               \
    ::hmc::DeviceGuard hmc_guard_((ctx)->device);                                   \
    if (hmc_guard_.status() != HMC_OK) return hmc_guard_.status();                  \
    ::hmc::forget_earlier_error();                                                  \
    ::hmc::EntryTrace hmc_trace_((ctx), __PRETTY_FUNCTION__)

// Opt-in tracing of the entry points that queue work, read from the environment once per process:
//   HMC_TIMING_LOG=<file>  every such call is bracketed by two events on the context's stream; the elapsed device
//                          times are appended to the file as "<entry>\t<ms>" lines when the context is next
//                          synchronised or destroyed (nothing waits inside the calls themselves);
//   HMC_NVTX=1             every such call is an NVTX range named after the entry, for timeline tools.
// With neither set an entry pays one predictable branch.
class EntryTrace {
  public:
    EntryTrace(hmc_context *ctx, const char *pretty_function) {
        if (enabled()) begin(ctx, pretty_function);
    }
    ~EntryTrace() {
        if (active_) end();
    }
    EntryTrace(const EntryTrace &) = delete;
    EntryTrace &operator=(const EntryTrace &) = delete;
    static bool enabled();

  private:
    void begin(hmc_context *ctx, const char *pretty_function);
    void end();
    hmc_context *ctx_ = nullptr;
    bool active_ = false, range_ = false;
    int record_ = -1;
};
// Writes out what the timing log holds for `ctx` (the stream must have been synchronised).
void flush_trace(hmc_context *ctx);
void destroy_trace(hmc_context *ctx);

// An error that the caller's own CUDA calls left as the thread's last error must not be taken for a failure of
// the launch this entry is about to check: reading it clears it.
inline void forget_earlier_error() { (void)cudaGetLastError(); }

// A kernel launch. Host-only builds of the runtime files (the failure harness, which compiles them with g++
// against a stand-in CUDA runtime) route it through that runtime instead of the <<<>>> syntax.
#if defined(HMC_FAKE_CUDA)
#define HMC_LAUNCH(kernel, grid, block, shared, stream, ...) ::fake::launch([&] { kernel(__VA_ARGS__); })
#else
#define HMC_LAUNCH(kernel, grid, block, shared, stream, ...) kernel<<<(grid), (block), (shared), (stream)>>>(__VA_ARGS__)
#endif

// Looks up, once per device, the device address of the scratch array hmc_reduce_noalloc uses, which also makes the
// runtime load the module that holds it. `device` is the calling thread's current device.
hmc_status noalloc_scratch_on(int device, void **out);

// After a kernel launch: picks up a launch failure (and clears it).
hmc_status launch_status(const char *what);

inline int64_t ceil_div(int64_t n, int64_t d) { return n / d + (n % d != 0); }

}  // namespace hmc
