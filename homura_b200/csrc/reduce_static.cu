// hmc_reduce_noalloc: hmc_reduce for callers that cannot obtain a workspace.
//
// A reduction whose plan cuts the reduced range into chunks parks one 16-byte partial per (chunk, output)
// in scratch memory before a second kernel folds them. hmc_reduce takes that scratch from the caller, who
// normally gets it from a device allocator. Some callers cannot ask an allocator at the moment they need
// the reduction: a handler that runs *because* the device pool is exhausted and still wants a checksum or
// a norm of what it holds; a latency-critical loop that must not take the allocator's lock or pay for a
// driver allocation, which synchronises the whole device; a host that has handed every byte of device
// memory to an arena of its own. For them this entry point keeps the scratch inside the library: a fixed
// array in the device image, HMC_NOALLOC_SCRATCH_BYTES long, present on every GPU that loads the library
// for as long as the process lives. The entry point calls no cudaMalloc, cudaFree, or any routine that
// allocates on the device or the host heap on its way to the launch.
//
// What follows from one shared array:
//  * a plan that needs more than the array holds is refused with HMC_INVALID and a message that states
//    both sizes; nothing is launched;
//  * two calls that overlap on the GPU (different streams or contexts of one device) race on the array;
//    calls on one context are ordered by its stream and are safe back to back;
//  * the array keeps whatever the previous call left. That is harmless: every partial slot a plan reads
//    is written by the same call's first kernel before the second kernel reads it, so nothing has to
//    start at zero and nothing is cleared.
//
// The device address of the array is looked up once per device, with that device current: when a context is
// created on the device (hmc_context_create does it, so that the runtime loads the module holding the array
// while memory is still plentiful), or else by the first call of this entry point there, which should then be
// made before a stream capture is begun on that device. "Allocates nothing" describes a call whose code is
// already resident: unless the process runs with CUDA_MODULE_LOADING=EAGER the runtime loads each kernel the
// first time it is launched, which takes device memory, so a caller that must not allocate later makes one
// call per (op, dtype, layout class) it will need at start-up.
#include <mutex>

#include "map.cuh"
#include "reduce.cuh"

namespace {

constexpr int64_t kScratchBytes = HMC_NOALLOC_SCRATCH_BYTES;
constexpr int kMaxDevices = 64;

// In device code this is the array; in host code the name is only a handle for cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char noalloc_scratch[kScratchBytes];

std::mutex address_mutex;
void *scratch_address[kMaxDevices] = {};

}  // namespace

namespace hmc {

hmc_status noalloc_scratch_on(int device, void **out) {
    if (device < 0 || device >= kMaxDevices) return fail(HMC_INVALID, "device index beyond the scratch table");
    std::lock_guard<std::mutex> lock(address_mutex);
    if (scratch_address[device] == nullptr) {
        void *ptr = nullptr;
        cudaError_t err = cudaGetSymbolAddress(&ptr, noalloc_scratch);
        if (err != cudaSuccess) return cuda_fail(err, "cudaGetSymbolAddress");
        if (ptr == nullptr || (reinterpret_cast<uintptr_t>(ptr) & 255) != 0) {
            return fail(HMC_INTERNAL_ERROR, "the scratch array has no usable device address");
        }
        scratch_address[device] = ptr;
    }
    if (out != nullptr) *out = scratch_address[device];
    return HMC_OK;
}

}  // namespace hmc

using namespace hmc;

HMC_API hmc_status hmc_reduce_noalloc(hmc_context_t ctx, int32_t op, const hmc_tensor_desc *out,
                                      const hmc_tensor_desc *kept, const hmc_tensor_desc *red) {
    return guarded([&]() -> hmc_status {
        HMC_ENTER(ctx);
        hmc_status s = check_reduction(kept, red);
        if (s != HMC_OK) return s;
        if (op < HMC_REDUCE_SUM || op > HMC_REDUCE_ANY) return fail(HMC_INVALID, "unknown reduction");
        ReduceArgs a{*kept, *red, make_reduce_plan(*kept, *red), nullptr, ctx->tickets};
        s = check_output(out, kept, "the output", a.plan.nout);
        if (s != HMC_OK) return s;
        const int dt = kept->dtype;
        const bool is_float = dtype_is_float(dt);
        int expect = dt;
        if (op == HMC_REDUCE_SUM || op == HMC_REDUCE_PROD) expect = is_float ? dt : HMC_I64;
        else if (op == HMC_REDUCE_MEAN && !is_float) return fail(HMC_INVALID, "mean needs a floating point tensor");
        else if (op == HMC_REDUCE_ALL || op == HMC_REDUCE_ANY) expect = dt == HMC_U8 ? HMC_U8 : HMC_BOOL;
        if (out->dtype != expect) return fail(HMC_INVALID, "the output of the reduction has the wrong dtype");
        if ((op == HMC_REDUCE_MAX || op == HMC_REDUCE_MIN) && a.plan.nred == 0 && a.plan.nout > 0) {
            return fail(HMC_INVALID, "max and min need a nonempty reduction");
        }
        if (a.plan.nout == 0) return HMC_OK;
        if (a.plan.nred > 0 && kept->data == nullptr) return fail(HMC_INVALID, "null data pointer");
        const int64_t need = plan_partial_bytes(a.plan);
        if (need > kScratchBytes) {
            return fail(HMC_INVALID, "hmc_reduce_noalloc: this reduction needs " + std::to_string(need) +
                                         " bytes of scratch, the built-in array holds " + std::to_string(kScratchBytes) +
                                         "; use hmc_reduce with a workspace");
        }
        if (need > 0) {
            void *scratch = nullptr;
            s = noalloc_scratch_on(ctx->device, &scratch);
            if (s != HMC_OK) return s;
            a.partials = scratch;
        }
        switch (op) {
            case HMC_REDUCE_SUM: case HMC_REDUCE_PROD:
                return is_float ? reduce_float(ctx, op, out, a) : reduce_int(ctx, op, out, a);
            case HMC_REDUCE_MEAN: return reduce_float(ctx, op, out, a);
            case HMC_REDUCE_MAX: case HMC_REDUCE_MIN:
                return reduce_extreme(ctx, op == HMC_REDUCE_MAX,
                                      static_cast<char *>(out->data) + out->offset * element_size(out->dtype), nullptr, a);
            default: return reduce_truth(ctx, op, out, a);
        }
    });
}
