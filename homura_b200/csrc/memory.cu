// Raw device segments for the caller's caching allocator, memset and the host <-> device copies.
// Stands in for homura's csrc/memory.hip.
#include "common.cuh"

using namespace hmc;

namespace {
hmc_status check_device_index(int32_t device) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess) {
        cudaGetLastError();
        count = 0;
    }
    if (device < 0 || device >= count) return fail(HMC_INVALID, "device index out of range");
    return HMC_OK;
}
}  // namespace

HMC_API hmc_status hmc_malloc(int32_t device, uint64_t nbytes, void **out) {
    return guarded([&]() -> hmc_status {
        if (out == nullptr) return fail(HMC_INVALID, "null output pointer");
        *out = nullptr;
        hmc_status s = check_device_index(device);
        if (s != HMC_OK) return s;
        hmc_status inj;
        if (injected_data_failure(inj)) return inj;
        if (nbytes == 0) return HMC_OK;
        DeviceGuard guard(device);
        if (guard.status() != HMC_OK) return guard.status();
        void *p = nullptr;
        HMC_CUDA(cudaMalloc(&p, nbytes), "cudaMalloc");
        *out = p;
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_free(int32_t device, void *ptr) {
    return guarded([&]() -> hmc_status {
        if (ptr == nullptr) return HMC_OK;
        hmc_status s = check_device_index(device);
        if (s != HMC_OK) return s;
        DeviceGuard guard(device);
        if (guard.status() != HMC_OK) return guard.status();
        HMC_CUDA(cudaFree(ptr), "cudaFree");
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_host_alloc(uint64_t nbytes, void **out) {
    return guarded([&]() -> hmc_status {
        if (out == nullptr) return fail(HMC_INVALID, "null output pointer");
        *out = nullptr;
        if (nbytes == 0) return HMC_OK;
        void *p = nullptr;
        HMC_CUDA(cudaHostAlloc(&p, nbytes, cudaHostAllocPortable), "cudaHostAlloc");
        *out = p;
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_host_free(void *ptr) {
    return guarded([&]() -> hmc_status {
        if (ptr == nullptr) return HMC_OK;
        HMC_CUDA(cudaFreeHost(ptr), "cudaFreeHost");
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_memset(hmc_context_t ctx, void *ptr, uint8_t value, uint64_t nbytes) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        if (nbytes == 0) return HMC_OK;
        if (ptr == nullptr) return fail(HMC_INVALID, "null pointer");
        HMC_CUDA(cudaMemsetAsync(ptr, value, nbytes, ctx->stream), "cudaMemsetAsync");
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_copy_to_host(hmc_context_t ctx, void *dst, const void *src, uint64_t nbytes) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        if (nbytes == 0) return HMC_OK;
        if (dst == nullptr || src == nullptr) return fail(HMC_INVALID, "null pointer");
        HMC_CUDA(cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToHost, ctx->stream), "cudaMemcpyAsync (to host)");
        HMC_CUDA(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_copy_from_host(hmc_context_t ctx, void *dst, const void *src, uint64_t nbytes) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        if (nbytes == 0) return HMC_OK;
        if (dst == nullptr || src == nullptr) return fail(HMC_INVALID, "null pointer");
        HMC_CUDA(cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyHostToDevice, ctx->stream), "cudaMemcpyAsync (from host)");
        HMC_CUDA(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_copy_device(hmc_context_t ctx, void *dst, const void *src, uint64_t nbytes) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        if (nbytes == 0) return HMC_OK;
        if (dst == nullptr || src == nullptr) return fail(HMC_INVALID, "null pointer");
        HMC_CUDA(cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToDevice, ctx->stream), "cudaMemcpyAsync (device)");
        return HMC_OK;
    });
}
