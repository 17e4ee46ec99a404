/*
 * homura_cuda_alloc.h: a native caching allocator with the semantics of homura's own
 * (src/backend/caching.rs), for hosts that do not bring one.
 *
 * homura's Rust side keeps its allocator in Rust and only needs hmc_malloc / hmc_free from
 * homura_cuda.h; nothing in homura_cuda.h depends on this header. It exists so that a host written
 * in another language (this repository's own test and benchmark drivers) gets the same behaviour:
 *  - requests of up to 1 MiB are rounded to 512 bytes and cut from 2 MiB segments; larger ones are
 *    rounded to 2 MiB and get a segment of their own (src/backend/caching.rs:22-28, 113-118);
 *  - a freed block is cached, merged with free neighbours of its segment, and reused best fit by
 *    (size, address), split when larger than needed (caching.rs:159-263);
 *  - when the device refuses a segment, the segments that are entirely free are released (after a
 *    wait for the stream) and the request is tried exactly once more (caching.rs:174-204, 266-292);
 *  - allocated / reserved / peak counters change together (src/storage.rs:89-167).
 * Blocks are reusable as soon as they are released: with one stream per device, work that still
 * uses a block was queued before the work that reuses it (caching.rs:9-13).
 */
#ifndef HOMURA_CUDA_ALLOC_H
#define HOMURA_CUDA_ALLOC_H

#include "homura_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Results of the memory callbacks below. */
#define HMC_MEM_OK 0
#define HMC_MEM_OUT_OF_MEMORY 1
#define HMC_MEM_FAILED 2

/* The device memory behind an allocator (homura's `trait Memory`, caching.rs:31-38). A callback
 * that returns HMC_MEM_FAILED may leave a message with hmc_allocator_set_callback_error. */
typedef struct hmc_memory_ops {
    void *user;
    int32_t (*malloc_fn)(void *user, uint64_t size, uint64_t *addr);
    int32_t (*free_fn)(void *user, uint64_t addr);
    int32_t (*synchronize_fn)(void *user);
} hmc_memory_ops;

typedef struct hmc_allocator *hmc_allocator_t;

typedef struct hmc_memory_stats {
    uint64_t allocated; /* bytes in blocks handed out (rounded sizes) */
    uint64_t reserved;  /* bytes in segments held from the device */
    uint64_t peak;      /* highest `allocated` since the last reset */
} hmc_memory_stats;

/* An allocator over caller-supplied memory (tests use a fake device with a capacity). */
hmc_status hmc_allocator_create(const hmc_memory_ops *ops, hmc_allocator_t *out);
/* An allocator over hmc_malloc / hmc_free of the context's device, waiting on its stream before
 * segments go back to the device. The context must outlive the allocator. */
hmc_status hmc_allocator_create_cuda(hmc_context_t ctx, hmc_allocator_t *out);
/* Releases every segment (blocks still handed out become invalid) and destroys the allocator. */
hmc_status hmc_allocator_destroy(hmc_allocator_t a);

/* A block of at least nbytes (> 0): its address and rounded size. HMC_OUT_OF_MEMORY when the
 * device has nothing left even after the cache was released; for a CUDA allocator the message is
 * "CUDA out of memory. Tried to allocate ... MiB. cuda:N has a total capacity of ..." in the style
 * of src/backend/rocm/memory.rs:203-218. */
hmc_status hmc_allocator_allocate(hmc_allocator_t a, uint64_t nbytes, uint64_t *addr, uint64_t *size);
/* Returns a block to the cache. HMC_INVALID for an address that is not a handed-out block. */
hmc_status hmc_allocator_release(hmc_allocator_t a, uint64_t addr);
/* Frees the cached segments that are entirely free (Device::empty_cache, src/device.rs:121-166). */
hmc_status hmc_allocator_empty_cache(hmc_allocator_t a);
hmc_status hmc_allocator_stats(hmc_allocator_t a, hmc_memory_stats *out);
hmc_status hmc_allocator_reset_peak(hmc_allocator_t a);
/* The rounded size of a request and whether it is served from the small pool; HMC_INVALID when
 * rounding overflows. */
hmc_status hmc_allocator_rounded(uint64_t nbytes, uint64_t *size, int32_t *is_small);
void hmc_allocator_set_callback_error(const char *message);

#ifdef __cplusplus
}
#endif

#endif /* HOMURA_CUDA_ALLOC_H */
