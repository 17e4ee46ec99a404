// NCCL plumbing of the sharded reductions: communicator and all-gather on the context's stream.
#include <nccl.h>

#include <cstring>

#include "../../include/homura_cuda_shard.h"
#include "common.cuh"

struct hmc_comm {
    hmc_context_t ctx;
    ncclComm_t comm;
    int ranks;
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

HMC_API hmc_status hmc_comm_create(hmc_context_t ctx, int32_t ranks, int32_t rank, const uint8_t *id, hmc_comm_t *out) {
    return guarded([&]() -> hmc_status {
        if (ctx == nullptr || id == nullptr || out == nullptr) return fail(HMC_INVALID, "null argument");
        *out = nullptr;
        if (ranks < 1 || rank < 0 || rank >= ranks) return fail(HMC_INVALID, "rank out of range");
        DeviceScope guard(ctx->device);
        if (guard.status() != HMC_OK) return guard.status();
        ncclUniqueId u;
        std::memcpy(&u, id, sizeof u);
        ncclComm_t comm;
        ncclResult_t r = ncclCommInitRank(&comm, ranks, u, rank);
        if (r != ncclSuccess) return nccl_fail(r, "ncclCommInitRank");
        hmc_comm *c = new (std::nothrow) hmc_comm{ctx, comm, ranks};
        if (c == nullptr) {
            ncclCommDestroy(comm);
            return fail(HMC_OUT_OF_MEMORY, "out of host memory");
        }
        *out = c;
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_comm_destroy(hmc_comm_t comm) {
    return guarded([&]() -> hmc_status {
        if (comm == nullptr) return HMC_OK;
        DeviceScope guard(comm->ctx->device);
        if (guard.status() != HMC_OK) return guard.status();
        ncclResult_t r = ncclCommDestroy(comm->comm);
        delete comm;
        if (r != ncclSuccess) return nccl_fail(r, "ncclCommDestroy");
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_comm_allgather(hmc_comm_t comm, const void *send, void *recv, uint64_t bytes) {
    return guarded([&]() -> hmc_status {
        if (comm == nullptr) return fail(HMC_INVALID, "null communicator");
        if (bytes == 0) return HMC_OK;
        if (send == nullptr || recv == nullptr) return fail(HMC_INVALID, "null buffer");
        DeviceScope guard(comm->ctx->device);
        if (guard.status() != HMC_OK) return guard.status();
        ncclResult_t r = ncclAllGather(send, recv, bytes, ncclUint8, comm->comm, comm->ctx->stream);
        if (r != ncclSuccess) return nccl_fail(r, "ncclAllGather");
        return HMC_OK;
    });
}
