// Device discovery, contexts, error state and the ABI self-description.
// Stands in for homura's csrc/runtime.hip on NVIDIA hardware.
#include <cctype>
#include <cstddef>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#if !defined(HMC_FAKE_CUDA)
#include <nvtx3/nvToolsExt.h>
#endif

#include "common.cuh"

namespace hmc {

ThreadState &thread_state() {
    thread_local ThreadState state;
    return state;
}

hmc_status fail(hmc_status status, const char *message) noexcept {
    thread_state().message.assign(message);
    return status;
}
hmc_status fail(hmc_status status, const std::string &message) noexcept { return fail(status, message.c_str()); }

hmc_status cuda_fail(cudaError_t err, const char *what) {
    // Reading the error clears the runtime's per-thread record of it.
    cudaGetLastError();
    char text[512];
    std::snprintf(text, sizeof text, "%s: %s", what, cudaGetErrorString(err));
    bool oom = err == cudaErrorMemoryAllocation;
    return fail(oom ? HMC_OUT_OF_MEMORY : HMC_CUDA_ERROR, text);
}

hmc_status launch_status(const char *what) {
    cudaError_t err = cudaGetLastError();
    if (err == cudaSuccess) return HMC_OK;
    return cuda_fail(err, what);
}

DeviceGuard::DeviceGuard(int device) {
    cudaError_t err = cudaGetDevice(&previous_);
    if (err != cudaSuccess) {
        status_ = cuda_fail(err, "cudaGetDevice");
        return;
    }
    if (previous_ != device) {
        err = cudaSetDevice(device);
        if (err != cudaSuccess) {
            status_ = cuda_fail(err, "cudaSetDevice");
            return;
        }
        switched_ = true;
    }
}

DeviceGuard::~DeviceGuard() {
    if (switched_) {
        if (cudaSetDevice(previous_) != cudaSuccess) cudaGetLastError();
    }
}

// ---- tracing ----
struct TraceRecord {
    char name[48];
    cudaEvent_t start, stop;
};
struct TraceState {
    std::vector<TraceRecord> records;
    std::vector<cudaEvent_t> spare;
};

namespace {
struct TraceConfig {
    bool nvtx = false;
    std::string log_path;
    std::mutex log_mutex;
};
TraceConfig &trace_config() {
    static TraceConfig config;
    static std::once_flag once;
    std::call_once(once, [] {
        if (const char *p = std::getenv("HMC_TIMING_LOG")) config.log_path = p;
        if (const char *n = std::getenv("HMC_NVTX")) config.nvtx = n[0] != '\0' && n[0] != '0';
    });
    return config;
}
// "hmc_status hmc_unary(...)::<lambda()>" -> "hmc_unary"
void entry_name(const char *pretty, char (&out)[48]) {
    const char *p = std::strstr(pretty, "hmc_");
    while (p != nullptr && std::strncmp(p, "hmc_status", 10) == 0) p = std::strstr(p + 10, "hmc_");
    size_t n = 0;
    if (p != nullptr) {
        while (n + 1 < sizeof out && (std::isalnum(static_cast<unsigned char>(p[n])) || p[n] == '_')) {
            out[n] = p[n];
            ++n;
        }
    }
    out[n] = '\0';
}
cudaEvent_t trace_event(TraceState *t) {
    if (!t->spare.empty()) {
        cudaEvent_t e = t->spare.back();
        t->spare.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    if (cudaEventCreate(&e) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return e;
}
}  // namespace

bool EntryTrace::enabled() {
    static const bool on = trace_config().nvtx || !trace_config().log_path.empty();
    return on;
}

void EntryTrace::begin(hmc_context *ctx, const char *pretty_function) {
    // (tracing is an aid: a failure inside it switches the record off and never fails the entry)
    try {
        ctx_ = ctx;
        active_ = true;
        TraceRecord r{};
        entry_name(pretty_function, r.name);
#if !defined(HMC_FAKE_CUDA)
        if (trace_config().nvtx) {
            nvtxRangePushA(r.name);
            range_ = true;
        }
#endif
        if (!trace_config().log_path.empty()) {
            if (ctx->trace == nullptr) ctx->trace = new TraceState();
            r.start = trace_event(ctx->trace);
            r.stop = trace_event(ctx->trace);
            if (r.start != nullptr && r.stop != nullptr && cudaEventRecord(r.start, ctx->stream) == cudaSuccess) {
                ctx->trace->records.push_back(r);
                record_ = static_cast<int>(ctx->trace->records.size()) - 1;
            } else {
                cudaGetLastError();
            }
        }
    } catch (...) {
        record_ = -1;
    }
}

void EntryTrace::end() {
    if (record_ >= 0) {
        if (cudaEventRecord(ctx_->trace->records[static_cast<size_t>(record_)].stop, ctx_->stream) != cudaSuccess) cudaGetLastError();
    }
#if !defined(HMC_FAKE_CUDA)
    if (range_) nvtxRangePop();
#endif
}

void flush_trace(hmc_context *ctx) {
    if (ctx == nullptr || ctx->trace == nullptr || ctx->trace->records.empty()) return;
    try {
        TraceConfig &config = trace_config();
        std::lock_guard<std::mutex> lock(config.log_mutex);
        std::FILE *f = std::fopen(config.log_path.c_str(), "a");
        for (TraceRecord &r : ctx->trace->records) {
            float ms = 0.0f;
            if (cudaEventElapsedTime(&ms, r.start, r.stop) != cudaSuccess) {
                cudaGetLastError();
                ms = -1.0f;  // (an entry that failed before its closing event was recorded)
            }
            if (f != nullptr) std::fprintf(f, "%s\t%.6f\n", r.name, static_cast<double>(ms));
            ctx->trace->spare.push_back(r.start);
            ctx->trace->spare.push_back(r.stop);
        }
        if (f != nullptr) std::fclose(f);
        ctx->trace->records.clear();
    } catch (...) {
    }
}

void destroy_trace(hmc_context *ctx) {
    if (ctx == nullptr || ctx->trace == nullptr) return;
    for (TraceRecord &r : ctx->trace->records) {
        cudaEventDestroy(r.start);
        cudaEventDestroy(r.stop);
    }
    for (cudaEvent_t e : ctx->trace->spare) cudaEventDestroy(e);
    cudaGetLastError();
    delete ctx->trace;
    ctx->trace = nullptr;
}

bool injected_data_failure(hmc_status &status) {
    ThreadState &t = thread_state();
    if (t.fail_data <= 0) return false;
    t.fail_data -= 1;
    status = t.fail_data_oom ? fail(HMC_OUT_OF_MEMORY, "injected failure: out of memory")
                             : fail(HMC_CUDA_ERROR, "injected failure: invalid resource handle");
    return true;
}

namespace {

constexpr uint32_t kProbeWord = 0x484D4332u;  // "HMC2"

__global__ void probe_kernel(uint32_t *slot) { *slot = kProbeWord; }

hmc_status check_device(int32_t device) {
    int count = 0;
    cudaError_t err = cudaGetDeviceCount(&count);
    if (err != cudaSuccess) {
        cudaGetLastError();
        count = 0;
    }
    if (device < 0 || device >= count) {
        return fail(HMC_INVALID, "device index " + std::to_string(device) + " is out of range (" +
                                     std::to_string(count) + " CUDA devices)");
    }
    return HMC_OK;
}

// The architectures compiled into this library. sm_100a code runs on compute capability 10.0 only.
constexpr const char *kBuiltArchs = "sm_100a";

bool arch_supported(int major, int minor) { return major == 10 && minor == 0; }

}  // namespace
}  // namespace hmc

using namespace hmc;

HMC_API const char *hmc_last_error(void) { return thread_state().message.c_str(); }

HMC_API hmc_status hmc_device_count(int32_t *count) {
    return guarded([&]() -> hmc_status {
        if (count == nullptr) return fail(HMC_INVALID, "null count");
        int n = 0;
        cudaError_t err = cudaGetDeviceCount(&n);
        if (err != cudaSuccess) {
            // No driver, or no device: not an error for the caller, there is just nothing to use.
            cudaGetLastError();
            n = 0;
        }
        *count = n;
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_device_properties_get(int32_t device, hmc_device_properties *out) {
    return guarded([&]() -> hmc_status {
        if (out == nullptr) return fail(HMC_INVALID, "null properties");
        ThreadState &t = thread_state();
        if (t.fail_properties > 0) {
            t.fail_properties -= 1;
            return fail(HMC_CUDA_ERROR, "injected failure: device properties");
        }
        hmc_status s = check_device(device);
        if (s != HMC_OK) return s;
        cudaDeviceProp prop;
        HMC_CUDA(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
        std::memset(out, 0, sizeof *out);
        std::snprintf(out->name, HMC_NAME_LEN, "%s", prop.name);
        std::snprintf(out->arch, HMC_ARCH_LEN, "sm_%d%d", prop.major, prop.minor);
        out->multiprocessor_count = prop.multiProcessorCount;
        out->warp_size = prop.warpSize;
        out->total_memory = prop.totalGlobalMem;
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_mem_get_info(int32_t device, uint64_t *free_bytes, uint64_t *total_bytes) {
    return guarded([&]() -> hmc_status {
        if (free_bytes == nullptr || total_bytes == nullptr) return fail(HMC_INVALID, "null output");
        hmc_status s = check_device(device);
        if (s != HMC_OK) return s;
        DeviceGuard guard(device);
        if (guard.status() != HMC_OK) return guard.status();
        size_t f = 0, t = 0;
        HMC_CUDA(cudaMemGetInfo(&f, &t), "cudaMemGetInfo");
        *free_bytes = f;
        *total_bytes = t;
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_context_create(int32_t device, hmc_context_t *out) {
    return guarded([&]() -> hmc_status {
        if (out == nullptr) return fail(HMC_INVALID, "null context output");
        *out = nullptr;
        hmc_status s = check_device(device);
        if (s != HMC_OK) return s;
        cudaDeviceProp prop;
        HMC_CUDA(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
        if (!arch_supported(prop.major, prop.minor)) {
            return fail(HMC_INVALID, std::string("GPU ") + prop.name + " (sm_" + std::to_string(prop.major) +
                                         std::to_string(prop.minor) + ") is not supported: this library was built for " +
                                         kBuiltArchs);
        }
        DeviceGuard guard(device);
        if (guard.status() != HMC_OK) return guard.status();
        ThreadState &t = thread_state();
        if (t.fail_stream_create > 0) {
            t.fail_stream_create -= 1;
            return fail(HMC_OUT_OF_MEMORY, "injected failure: stream creation");
        }
        cudaStream_t stream = nullptr;
        HMC_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "cudaStreamCreateWithFlags");
        t.live_streams += 1;
        // Everything below must destroy the stream before failing.
        // (the failure's message is already recorded and survives: the clean-up records nothing. A stream the
        // runtime refuses to destroy stays counted.)
        auto abandon = [&](hmc_status status) {
            if (cudaStreamDestroy(stream) == cudaSuccess) t.live_streams -= 1;
            else cudaGetLastError();
            return status;
        };
        uint32_t *slot = nullptr;
        // one allocation: the probe's word, which stays as the status word, and the reductions' counters after it
        constexpr size_t kSlotBytes = (kTicketsOffset + kTickets) * sizeof(uint32_t);
        cudaError_t err = cudaMalloc(&slot, kSlotBytes);
        if (err != cudaSuccess) return abandon(cuda_fail(err, "probe: cudaMalloc"));
        uint32_t answer = 0;
        forget_earlier_error();
        HMC_LAUNCH(probe_kernel, 1, 1, 0, stream, slot);
        err = cudaGetLastError();
        if (err == cudaSuccess) err = cudaMemcpyAsync(&answer, slot, sizeof answer, cudaMemcpyDeviceToHost, stream);
        if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
        // The probe's word stays with the context as its status word (zero: nothing to report).
        if (err == cudaSuccess) err = cudaMemsetAsync(slot, 0, kSlotBytes, stream);
        if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
        auto abandon_slot = [&](hmc_status status) {
            if (cudaFree(slot) != cudaSuccess) cudaGetLastError();
            return abandon(status);
        };
        if (err != cudaSuccess) return abandon_slot(cuda_fail(err, "probe kernel"));
        if (answer != kProbeWord) return abandon_slot(fail(HMC_CUDA_ERROR, "probe kernel wrote the wrong value"));
        // The scratch array of hmc_reduce_noalloc: looking up its address now makes the runtime load the module
        // that holds it while this call is allocating anyway. A failure here is not the context's: the entry point
        // looks the address up again when it is first used.
        if (noalloc_scratch_on(device, nullptr) != HMC_OK) t.message.clear();
        hmc_context *ctx = nullptr;
        if (t.fail_after_probe > 0) {
            t.fail_after_probe -= 1;
            return abandon_slot(fail(HMC_OUT_OF_MEMORY, "out of host memory"));
        }
        ctx = new (std::nothrow) hmc_context{device, stream, prop.multiProcessorCount, nullptr, reinterpret_cast<int *>(slot), slot + kTicketsOffset};
        if (ctx == nullptr) return abandon_slot(fail(HMC_OUT_OF_MEMORY, "out of host memory"));
        *out = ctx;
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_context_destroy(hmc_context_t ctx) {
    return guarded([&]() -> hmc_status {
        if (ctx == nullptr) return HMC_OK;
        DeviceGuard guard(ctx->device);
        if (guard.status() != HMC_OK) return guard.status();
        if (ctx->trace != nullptr) {
            if (cudaStreamSynchronize(ctx->stream) == cudaSuccess) flush_trace(ctx);
            else cudaGetLastError();
            destroy_trace(ctx);
        }
        if (ctx->status != nullptr && cudaFree(ctx->status) != cudaSuccess) cudaGetLastError();
        cudaError_t err = cudaStreamDestroy(ctx->stream);
        if (err == cudaSuccess) thread_state().live_streams -= 1;
        delete ctx;
        if (err != cudaSuccess) return cuda_fail(err, "cudaStreamDestroy");
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_context_synchronize(hmc_context_t ctx) {
    return guarded([&]() -> hmc_status {
        if (ctx == nullptr) return fail(HMC_INVALID, "null context");
        DeviceGuard guard(ctx->device);
        if (guard.status() != HMC_OK) return guard.status();
        HMC_CUDA(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
        flush_trace(ctx);
        if (ctx->status != nullptr) {
            // kernels that wait on barriers give up after a bounded number of polls and say so here
            int word = 0;
            HMC_CUDA(cudaMemcpyAsync(&word, ctx->status, sizeof word, cudaMemcpyDeviceToHost, ctx->stream), "cudaMemcpyAsync (status)");
            HMC_CUDA(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
            if (word != 0) {
                HMC_CUDA(cudaMemsetAsync(ctx->status, 0, sizeof word, ctx->stream), "cudaMemsetAsync (status)");
                return fail(HMC_CUDA_ERROR, "a kernel gave up a bounded wait on the device: results queued before this call are incomplete");
            }
        }
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_context_stream(hmc_context_t ctx, void **stream) {
    return guarded([&]() -> hmc_status {
        if (ctx == nullptr || stream == nullptr) return fail(HMC_INVALID, "null argument");
        *stream = static_cast<void *>(ctx->stream);
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_event_create(hmc_context_t ctx, hmc_event_t *out) {
    return guarded([&]() -> hmc_status {
        if (ctx == nullptr || out == nullptr) return fail(HMC_INVALID, "null argument");
        DeviceGuard guard(ctx->device);
        if (guard.status() != HMC_OK) return guard.status();
        cudaEvent_t ev;
        HMC_CUDA(cudaEventCreate(&ev), "cudaEventCreate");
        hmc_event *e = new (std::nothrow) hmc_event{ctx->device, ev};
        if (e == nullptr) {
            cudaEventDestroy(ev);
            return fail(HMC_OUT_OF_MEMORY, "out of host memory");
        }
        *out = e;
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_event_record(hmc_context_t ctx, hmc_event_t ev) {
    return guarded([&]() -> hmc_status {
        if (ctx == nullptr || ev == nullptr) return fail(HMC_INVALID, "null argument");
        DeviceGuard guard(ctx->device);
        if (guard.status() != HMC_OK) return guard.status();
        HMC_CUDA(cudaEventRecord(ev->event, ctx->stream), "cudaEventRecord");
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_event_elapsed_ms(hmc_event_t start, hmc_event_t stop, float *ms) {
    return guarded([&]() -> hmc_status {
        if (start == nullptr || stop == nullptr || ms == nullptr) return fail(HMC_INVALID, "null argument");
        DeviceGuard guard(stop->device);
        if (guard.status() != HMC_OK) return guard.status();
        HMC_CUDA(cudaEventSynchronize(stop->event), "cudaEventSynchronize");
        HMC_CUDA(cudaEventElapsedTime(ms, start->event, stop->event), "cudaEventElapsedTime");
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_event_destroy(hmc_event_t ev) {
    return guarded([&]() -> hmc_status {
        if (ev == nullptr) return HMC_OK;
        DeviceGuard guard(ev->device);
        if (guard.status() != HMC_OK) return guard.status();
        cudaError_t err = cudaEventDestroy(ev->event);
        delete ev;
        if (err != cudaSuccess) return cuda_fail(err, "cudaEventDestroy");
        return HMC_OK;
    });
}

HMC_API const char *hmc_built_archs(void) { return kBuiltArchs; }

HMC_API void hmc_abi_check(hmc_abi_info *out) {
    if (out == nullptr) return;
    std::memset(out, 0, sizeof *out);
    out->abi_info_size = sizeof(hmc_abi_info);
    out->properties_size = sizeof(hmc_device_properties);
    out->properties_align = alignof(hmc_device_properties);
    out->properties_offsets[0] = offsetof(hmc_device_properties, name);
    out->properties_offsets[1] = offsetof(hmc_device_properties, arch);
    out->properties_offsets[2] = offsetof(hmc_device_properties, multiprocessor_count);
    out->properties_offsets[3] = offsetof(hmc_device_properties, warp_size);
    out->properties_offsets[4] = offsetof(hmc_device_properties, total_memory);
    const int32_t statuses[5] = {HMC_OK, HMC_OUT_OF_MEMORY, HMC_INVALID, HMC_CUDA_ERROR, HMC_INTERNAL_ERROR};
    std::memcpy(out->status_values, statuses, sizeof statuses);
    out->name_len = HMC_NAME_LEN;
    out->arch_len = HMC_ARCH_LEN;
    out->desc_size = sizeof(hmc_tensor_desc);
    out->desc_align = alignof(hmc_tensor_desc);
    out->desc_offsets[0] = offsetof(hmc_tensor_desc, data);
    out->desc_offsets[1] = offsetof(hmc_tensor_desc, offset);
    out->desc_offsets[2] = offsetof(hmc_tensor_desc, dtype);
    out->desc_offsets[3] = offsetof(hmc_tensor_desc, ndim);
    out->desc_offsets[4] = offsetof(hmc_tensor_desc, sizes);
    out->desc_offsets[5] = offsetof(hmc_tensor_desc, strides);
    const int32_t dtypes[10] = {HMC_BOOL, HMC_U8, HMC_I8, HMC_I16, HMC_I32, HMC_I64, HMC_F16, HMC_BF16, HMC_F32, HMC_F64};
    std::memcpy(out->dtype_values, dtypes, sizeof dtypes);
    out->max_dims = HMC_MAX_DIMS;
    out->adamw_scalars_size = sizeof(hmc_adamw_scalars);
    out->adamw_scalars_align = alignof(hmc_adamw_scalars);
}

// ---- testing hooks ----
HMC_API void hmc_test_fail_stream_create(int32_t n) { thread_state().fail_stream_create = n; }
HMC_API void hmc_test_fail_after_probe(int32_t n) { thread_state().fail_after_probe = n; }
HMC_API void hmc_test_fail_properties(int32_t n) { thread_state().fail_properties = n; }
HMC_API void hmc_test_fail_data(int32_t n, int32_t out_of_memory) {
    thread_state().fail_data = n;
    thread_state().fail_data_oom = out_of_memory != 0;
}
HMC_API int32_t hmc_test_live_streams(void) { return thread_state().live_streams; }
HMC_API hmc_status hmc_test_current_device(int32_t *device) {
    return guarded([&]() -> hmc_status {
        if (device == nullptr) return fail(HMC_INVALID, "null device");
        int d = 0;
        HMC_CUDA(cudaGetDevice(&d), "cudaGetDevice");
        *device = d;
        return HMC_OK;
    });
}
HMC_API hmc_status hmc_test_set_current_device(int32_t device) {
    return guarded([&]() -> hmc_status {
        HMC_CUDA(cudaSetDevice(device), "cudaSetDevice");
        return HMC_OK;
    });
}
HMC_API hmc_status hmc_test_fail(const char *message) {
    return guarded([&]() -> hmc_status { return fail(HMC_INVALID, message ? message : ""); });
}
