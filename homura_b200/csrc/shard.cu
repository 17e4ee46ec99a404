// NCCL plumbing of the sharded reductions: communicator and all-gather on the context's stream.
//
// The communicator is created non-blocking, so that no call into the library can hold a rank for ever: a call
// that the library has not finished queuing is polled with a deadline, hmc_comm_wait waits for the stream with
// the same deadline, and when a deadline passes or the library reports an asynchronous error the communicator
// is aborted (kernels of it that are still waiting for a peer stop; the context's stream stays usable) and the
// call returns HMC_CUDA_ERROR. A caller that wants the bound calls hmc_comm_wait where it would otherwise
// synchronise the context after a collective.
#include <nccl.h>

#include <chrono>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>

#include "../../include/homura_cuda_shard.h"
#include "common.cuh"

struct hmc_comm {
    hmc_context_t ctx;
    ncclComm_t comm;
    int ranks;
    int64_t timeout_ms;  // how long a call may wait for the library, and hmc_comm_wait for the stream
    bool aborted;        // the communicator was torn down after an error or an expired wait
};

// This file is linked into its own library and reaches the core library through its C ABI only, so that
// the core keeps exporting nothing but hmc_* symbols.
namespace {

// Leaves `message` as the calling thread's hmc_last_error() and returns `status`.
hmc_status fail(hmc_status status, const std::string &message) {
    hmc_test_fail(message.c_str());
    return status;
}
hmc_status nccl_fail(ncclResult_t r, const char *what) {
    return fail(HMC_CUDA_ERROR, std::string(what) + ": " + ncclGetErrorString(r));
}
static_assert(sizeof(ncclUniqueId) <= HMC_COMM_ID_BYTES, "communicator id does not fit");

template <class Body>
hmc_status guarded(Body &&body) noexcept {
    try {
        return body();
    } catch (...) {
        return HMC_INTERNAL_ERROR;
    }
}

// Makes the context's device current for a scope.
class DeviceScope {
  public:
    explicit DeviceScope(int device) {
        if (cudaGetDevice(&previous_) != cudaSuccess) {
            cudaGetLastError();
            ok_ = false;
            return;
        }
        if (previous_ != device) {
            ok_ = cudaSetDevice(device) == cudaSuccess;
            switched_ = ok_;
            if (!ok_) cudaGetLastError();
        }
    }
    ~DeviceScope() {
        if (switched_ && cudaSetDevice(previous_) != cudaSuccess) cudaGetLastError();
    }
    hmc_status status() const { return ok_ ? HMC_OK : fail(HMC_CUDA_ERROR, "cannot switch the CUDA device"); }

  private:
    int previous_ = -1;
    bool switched_ = false, ok_ = true;
};

}  // namespace

HMC_API hmc_status hmc_comm_unique_id(uint8_t *id) {
    return guarded([&]() -> hmc_status {
        if (id == nullptr) return fail(HMC_INVALID, "null id");
        ncclUniqueId u;
        ncclResult_t r = ncclGetUniqueId(&u);
        if (r != ncclSuccess) return nccl_fail(r, "ncclGetUniqueId");
        std::memset(id, 0, HMC_COMM_ID_BYTES);
        std::memcpy(id, &u, sizeof u);
        return HMC_OK;
    });
}

namespace {

constexpr int64_t kDefaultTimeoutMs = 60 * 1000;

int64_t now_ms() {
    return std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// Tears the communicator down after a failure: kernels of it that are still waiting for a peer stop, and the
// context's stream runs on. Every later call on the communicator is refused.
void abort_comm(hmc_comm *c) {
    if (!c->aborted) {
        c->aborted = true;
        ncclCommAbort(c->comm);
    }
}

// The communicator is non-blocking: a call may return ncclInProgress while the library still works on it in
// the background. Polls until the library is done with it, reports an asynchronous error, and gives up (aborting
// the communicator) when the deadline passes: a rank that never joins must not block its peers for ever.
hmc_status settle(hmc_comm *c, ncclResult_t r, const char *what) {
    const int64_t deadline = now_ms() + c->timeout_ms;
    while (r == ncclInProgress) {
        ncclResult_t q = ncclCommGetAsyncError(c->comm, &r);
        if (q != ncclSuccess) {
            r = q;
            break;
        }
        if (r != ncclInProgress) break;
        if (now_ms() > deadline) {
            abort_comm(c);
            return fail(HMC_CUDA_ERROR, std::string(what) + ": no progress within " + std::to_string(c->timeout_ms) +
                                            " ms (a rank is missing or stalled); the communicator was aborted");
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    if (r != ncclSuccess) {
        hmc_status s = nccl_fail(r, what);
        abort_comm(c);
        return s;
    }
    return HMC_OK;
}

}  // namespace

HMC_API hmc_status hmc_comm_create(hmc_context_t ctx, int32_t ranks, int32_t rank, const uint8_t *id, hmc_comm_t *out) {
    return guarded([&]() -> hmc_status {
        if (ctx == nullptr || id == nullptr || out == nullptr) return fail(HMC_INVALID, "null argument");
        *out = nullptr;
        if (ranks < 1 || rank < 0 || rank >= ranks) return fail(HMC_INVALID, "rank out of range");
        DeviceScope guard(ctx->device);
        if (guard.status() != HMC_OK) return guard.status();
        ncclUniqueId u;
        std::memcpy(&u, id, sizeof u);
        hmc_comm *c = new (std::nothrow) hmc_comm{ctx, nullptr, ranks, kDefaultTimeoutMs, false};
        if (c == nullptr) return fail(HMC_OUT_OF_MEMORY, "out of host memory");
        if (const char *e = std::getenv("HMC_COMM_TIMEOUT_MS")) {
            const long long v = std::atoll(e);
            if (v > 0) c->timeout_ms = v;
        }
        ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
        config.blocking = 0;
        ncclResult_t r = ncclCommInitRankConfig(&c->comm, ranks, u, rank, &config);
        if (r != ncclSuccess && r != ncclInProgress) {
            hmc_status s = nccl_fail(r, "ncclCommInitRankConfig");
            delete c;
            return s;
        }
        hmc_status s = settle(c, ncclInProgress, "ncclCommInitRankConfig");
        if (s != HMC_OK) {
            delete c;
            return s;
        }
        *out = c;
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_comm_set_timeout(hmc_comm_t comm, int64_t milliseconds) {
    return guarded([&]() -> hmc_status {
        if (comm == nullptr) return fail(HMC_INVALID, "null communicator");
        if (milliseconds <= 0) return fail(HMC_INVALID, "the timeout must be positive");
        comm->timeout_ms = milliseconds;
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_comm_destroy(hmc_comm_t comm) {
    return guarded([&]() -> hmc_status {
        if (comm == nullptr) return HMC_OK;
        DeviceScope guard(comm->ctx->device);
        if (guard.status() != HMC_OK) return guard.status();
        hmc_status s = HMC_OK;
        if (!comm->aborted) {
            // finalize flushes what is queued; it may itself be in progress for a while
            s = settle(comm, ncclCommFinalize(comm->comm), "ncclCommFinalize");
            if (s == HMC_OK) {
                ncclResult_t r = ncclCommDestroy(comm->comm);
                if (r != ncclSuccess) s = nccl_fail(r, "ncclCommDestroy");
            }
        }
        delete comm;
        return s;
    });
}

HMC_API hmc_status hmc_comm_allgather(hmc_comm_t comm, const void *send, void *recv, uint64_t bytes) {
    return guarded([&]() -> hmc_status {
        if (comm == nullptr) return fail(HMC_INVALID, "null communicator");
        if (comm->aborted) return fail(HMC_INVALID, "the communicator was aborted after an earlier failure");
        if (bytes == 0) return HMC_OK;
        if (send == nullptr || recv == nullptr) return fail(HMC_INVALID, "null buffer");
        DeviceScope guard(comm->ctx->device);
        if (guard.status() != HMC_OK) return guard.status();
        // (the kernel is in the stream once the library reports the call settled; work queued after this entry
        // returns is ordered behind it)
        return settle(comm, ncclAllGather(send, recv, bytes, ncclUint8, comm->comm, comm->ctx->stream), "ncclAllGather");
    });
}

HMC_API hmc_status hmc_comm_abort(hmc_comm_t comm) {
    return guarded([&]() -> hmc_status {
        if (comm == nullptr) return fail(HMC_INVALID, "null communicator");
        DeviceScope guard(comm->ctx->device);
        if (guard.status() != HMC_OK) return guard.status();
        abort_comm(comm);
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_comm_wait(hmc_comm_t comm) {
    return guarded([&]() -> hmc_status {
        if (comm == nullptr) return fail(HMC_INVALID, "null communicator");
        if (comm->aborted) return fail(HMC_INVALID, "the communicator was aborted after an earlier failure");
        DeviceScope guard(comm->ctx->device);
        if (guard.status() != HMC_OK) return guard.status();
        const int64_t deadline = now_ms() + comm->timeout_ms;
        for (;;) {
            cudaError_t q = cudaStreamQuery(comm->ctx->stream);
            if (q == cudaSuccess) return HMC_OK;
            if (q != cudaErrorNotReady) {
                cudaGetLastError();
                abort_comm(comm);
                return fail(HMC_CUDA_ERROR, std::string("cudaStreamQuery: ") + cudaGetErrorString(q));
            }
            ncclResult_t state = ncclSuccess;
            ncclResult_t r = ncclCommGetAsyncError(comm->comm, &state);
            if (r != ncclSuccess || (state != ncclSuccess && state != ncclInProgress)) {
                hmc_status s = nccl_fail(r != ncclSuccess ? r : state, "a collective failed");
                abort_comm(comm);
                return s;
            }
            if (now_ms() > deadline) {
                abort_comm(comm);
                return fail(HMC_CUDA_ERROR, "the collectives queued on the stream did not finish within " +
                                                std::to_string(comm->timeout_ms) +
                                                " ms (a rank is missing or stalled); the communicator was aborted");
            }
            std::this_thread::sleep_for(std::chrono::microseconds(100));
        }
    });
}
