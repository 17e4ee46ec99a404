// A caching allocator with the bookkeeping of homura's src/backend/caching.rs, in C++ (host only).
#include <map>
#include <mutex>
#include <set>
#include <unordered_map>
#include <vector>

#include "../../include/homura_cuda_alloc.h"
#include "common.cuh"

namespace {

constexpr uint64_t kSmallMax = 1ull << 20;
constexpr uint64_t kSmallRound = 512;
constexpr uint64_t kSmallSegment = 2ull << 20;
constexpr uint64_t kLargeRound = 2ull << 20;

thread_local std::string callback_error;

bool rounded(uint64_t nbytes, uint64_t &size, bool &small) {
    small = nbytes <= kSmallMax;
    const uint64_t unit = small ? kSmallRound : kLargeRound;
    const uint64_t n = nbytes == 0 ? 1 : nbytes;
    const uint64_t units = n / unit + (n % unit != 0);
    if (units > UINT64_MAX / unit) return false;
    size = units * unit;
    return true;
}

struct BlockInfo {
    uint64_t size;
    bool free;
    bool small;
    bool has_prev, has_next;
    uint64_t prev, next;
};

}  // namespace

struct hmc_allocator {
    hmc_memory_ops ops{};
    hmc_context_t ctx = nullptr;  // set for a CUDA allocator
    std::mutex pool_mutex;
    std::unordered_map<uint64_t, BlockInfo> blocks;
    std::set<std::pair<uint64_t, uint64_t>> free_small, free_large;  // (size, address)
    std::map<uint64_t, uint64_t> segments;                           // address -> size
    std::mutex counter_mutex;
    hmc_memory_stats stats{0, 0, 0};

    std::set<std::pair<uint64_t, uint64_t>> &free_set(bool small) { return small ? free_small : free_large; }

    void count(int64_t allocated, int64_t reserved) {
        std::lock_guard<std::mutex> lock(counter_mutex);
        stats.allocated += allocated;
        stats.reserved += reserved;
        if (stats.allocated > stats.peak) stats.peak = stats.allocated;
    }

    hmc_status callback_failed(const char *what) {
        std::string m = callback_error.empty() ? std::string(what) + " failed" : callback_error;
        callback_error.clear();
        return hmc::fail(HMC_CUDA_ERROR, m);
    }

    // Frees the segments that consist of one free block, after waiting for queued work.
    hmc_status release_cached() {
        std::vector<std::pair<uint64_t, uint64_t>> unused;
        for (const auto &seg : segments) {
            const BlockInfo &b = blocks.at(seg.first);
            if (b.free && b.size == seg.second) unused.push_back(seg);
        }
        if (unused.empty()) return HMC_OK;
        if (ops.synchronize_fn(ops.user) != HMC_MEM_OK) return callback_failed("synchronize");
        for (const auto &seg : unused) {
            if (ops.free_fn(ops.user, seg.first) != HMC_MEM_OK) return callback_failed("free");
            const BlockInfo b = blocks.at(seg.first);
            blocks.erase(seg.first);
            free_set(b.small).erase({seg.second, seg.first});
            segments.erase(seg.first);
            count(0, -static_cast<int64_t>(seg.second));
        }
        return HMC_OK;
    }

    hmc_status new_segment(uint64_t size, bool small, uint64_t &addr) {
        int32_t r = ops.malloc_fn(ops.user, size, &addr);
        if (r == HMC_MEM_OUT_OF_MEMORY) {
            hmc_status s = release_cached();
            if (s != HMC_OK) return s;
            r = ops.malloc_fn(ops.user, size, &addr);
            if (r == HMC_MEM_OUT_OF_MEMORY) return HMC_OUT_OF_MEMORY;  // message set by allocate()
        }
        if (r != HMC_MEM_OK) return callback_failed("malloc");
        blocks[addr] = BlockInfo{size, true, small, false, false, 0, 0};
        free_set(small).insert({size, addr});
        segments[addr] = size;
        count(0, static_cast<int64_t>(size));
        return HMC_OK;
    }

    // Marks the free block at `addr` used and splits off what lies beyond `size`.
    void take(uint64_t addr, uint64_t size) {
        BlockInfo &b = blocks.at(addr);
        const uint64_t old = b.size;
        const bool small = b.small;
        free_set(small).erase({old, addr});
        if (old > size) {
            const uint64_t rest = addr + size;
            BlockInfo tail{old - size, true, small, true, b.has_next, addr, b.next};
            if (b.has_next) blocks.at(b.next).prev = rest;
            b.size = size;
            b.has_next = true;
            b.next = rest;
            blocks[rest] = tail;
            free_set(small).insert({old - size, rest});
        }
        blocks.at(addr).free = false;
    }

    // Folds the free block `second` into its free predecessor `first`.
    void merge(uint64_t first, uint64_t second) {
        const BlockInfo s = blocks.at(second);
        blocks.erase(second);
        free_set(s.small).erase({s.size, second});
        BlockInfo &f = blocks.at(first);
        free_set(f.small).erase({f.size, first});
        f.size += s.size;
        f.has_next = s.has_next;
        f.next = s.next;
        if (s.has_next) blocks.at(s.next).prev = first;
    }
};

namespace {

int32_t cuda_malloc_cb(void *user, uint64_t size, uint64_t *addr) {
    hmc_allocator *a = static_cast<hmc_allocator *>(user);
    void *p = nullptr;
    hmc_status s = hmc_malloc(a->ctx->device, size, &p);
    if (s == HMC_OUT_OF_MEMORY) return HMC_MEM_OUT_OF_MEMORY;
    if (s != HMC_OK) {
        callback_error = hmc_last_error();
        return HMC_MEM_FAILED;
    }
    *addr = reinterpret_cast<uint64_t>(p);
    return HMC_MEM_OK;
}
int32_t cuda_free_cb(void *user, uint64_t addr) {
    hmc_allocator *a = static_cast<hmc_allocator *>(user);
    if (hmc_free(a->ctx->device, reinterpret_cast<void *>(addr)) != HMC_OK) {
        callback_error = hmc_last_error();
        return HMC_MEM_FAILED;
    }
    return HMC_MEM_OK;
}
int32_t cuda_sync_cb(void *user) {
    hmc_allocator *a = static_cast<hmc_allocator *>(user);
    if (hmc_context_synchronize(a->ctx) != HMC_OK) {
        callback_error = hmc_last_error();
        return HMC_MEM_FAILED;
    }
    return HMC_MEM_OK;
}

std::string oom_message(hmc_allocator *a, uint64_t requested) {
    char text[512];
    const double mib = 1048576.0, gib = 1073741824.0;
    hmc_memory_stats st;
    {
        std::lock_guard<std::mutex> lock(a->counter_mutex);
        st = a->stats;
    }
    if (a->ctx == nullptr) {
        std::snprintf(text, sizeof text, "out of memory. Tried to allocate %.2f MiB.", requested / mib);
        return text;
    }
    uint64_t free_b = 0, total_b = 0;
    hmc_mem_get_info(a->ctx->device, &free_b, &total_b);
    const uint64_t unallocated = st.reserved > st.allocated ? st.reserved - st.allocated : 0;
    std::snprintf(text, sizeof text,
                  "CUDA out of memory. Tried to allocate %.2f MiB. cuda:%d has a total capacity of %.2f GiB of which "
                  "%.2f MiB is free. Of the allocated memory %.2f MiB is allocated by homura, and %.2f MiB is reserved "
                  "but unallocated.",
                  requested / mib, a->ctx->device, total_b / gib, free_b / mib, st.allocated / mib, unallocated / mib);
    return text;
}

}  // namespace

using hmc::fail;
using hmc::guarded;

HMC_API void hmc_allocator_set_callback_error(const char *message) { callback_error = message ? message : ""; }

HMC_API hmc_status hmc_allocator_rounded(uint64_t nbytes, uint64_t *size, int32_t *is_small) {
    return guarded([&]() -> hmc_status {
        if (size == nullptr || is_small == nullptr) return fail(HMC_INVALID, "null output");
        bool small = false;
        if (!rounded(nbytes, *size, small)) return fail(HMC_INVALID, "the rounded size overflows");
        *is_small = small ? 1 : 0;
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_allocator_create(const hmc_memory_ops *ops, hmc_allocator_t *out) {
    return guarded([&]() -> hmc_status {
        if (ops == nullptr || out == nullptr || ops->malloc_fn == nullptr || ops->free_fn == nullptr ||
            ops->synchronize_fn == nullptr) {
            return fail(HMC_INVALID, "null memory callbacks");
        }
        hmc_allocator *a = new hmc_allocator();
        a->ops = *ops;
        *out = a;
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_allocator_create_cuda(hmc_context_t ctx, hmc_allocator_t *out) {
    return guarded([&]() -> hmc_status {
        if (ctx == nullptr || out == nullptr) return fail(HMC_INVALID, "null argument");
        hmc_allocator *a = new hmc_allocator();
        a->ctx = ctx;
        a->ops = hmc_memory_ops{a, cuda_malloc_cb, cuda_free_cb, cuda_sync_cb};
        *out = a;
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_allocator_destroy(hmc_allocator_t a) {
    return guarded([&]() -> hmc_status {
        if (a == nullptr) return HMC_OK;
        hmc_status result = HMC_OK;
        {
            std::lock_guard<std::mutex> lock(a->pool_mutex);
            if (!a->segments.empty()) {
                if (a->ops.synchronize_fn(a->ops.user) != HMC_MEM_OK) result = a->callback_failed("synchronize");
                for (const auto &seg : a->segments) {
                    if (a->ops.free_fn(a->ops.user, seg.first) != HMC_MEM_OK) result = a->callback_failed("free");
                }
            }
        }
        delete a;
        return result;
    });
}

HMC_API hmc_status hmc_allocator_allocate(hmc_allocator_t a, uint64_t nbytes, uint64_t *addr, uint64_t *size) {
    return guarded([&]() -> hmc_status {
        if (a == nullptr || addr == nullptr || size == nullptr) return fail(HMC_INVALID, "null argument");
        if (nbytes == 0) return fail(HMC_INVALID, "a block has at least one byte");
        uint64_t want = 0;
        bool small = false;
        if (!rounded(nbytes, want, small)) return fail(HMC_OUT_OF_MEMORY, oom_message(a, nbytes));
        std::lock_guard<std::mutex> lock(a->pool_mutex);
        auto &set = a->free_set(small);
        auto fit = set.lower_bound({want, 0});
        uint64_t at = 0;
        if (fit != set.end()) {
            at = fit->second;
        } else {
            hmc_status s = a->new_segment(small ? kSmallSegment : want, small, at);
            if (s == HMC_OUT_OF_MEMORY) return fail(HMC_OUT_OF_MEMORY, oom_message(a, nbytes));
            if (s != HMC_OK) return s;
        }
        a->take(at, want);
        a->count(static_cast<int64_t>(want), 0);
        *addr = at;
        *size = want;
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_allocator_release(hmc_allocator_t a, uint64_t addr) {
    return guarded([&]() -> hmc_status {
        if (a == nullptr) return fail(HMC_INVALID, "null allocator");
        std::lock_guard<std::mutex> lock(a->pool_mutex);
        auto it = a->blocks.find(addr);
        if (it == a->blocks.end()) return fail(HMC_INVALID, "freeing a block the allocator doesn't know");
        if (it->second.free) return fail(HMC_INVALID, "freeing a block twice");
        it->second.free = true;
        const bool small = it->second.small;
        a->count(-static_cast<int64_t>(it->second.size), 0);
        uint64_t at = addr;
        {
            const BlockInfo &b = a->blocks.at(at);
            if (b.has_next && a->blocks.at(b.next).free) a->merge(at, b.next);
        }
        {
            const BlockInfo &b = a->blocks.at(at);
            if (b.has_prev && a->blocks.at(b.prev).free) {
                const uint64_t prev = b.prev;
                a->merge(prev, at);
                at = prev;
            }
        }
        a->free_set(small).insert({a->blocks.at(at).size, at});
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_allocator_empty_cache(hmc_allocator_t a) {
    return guarded([&]() -> hmc_status {
        if (a == nullptr) return fail(HMC_INVALID, "null allocator");
        std::lock_guard<std::mutex> lock(a->pool_mutex);
        return a->release_cached();
    });
}

HMC_API hmc_status hmc_allocator_stats(hmc_allocator_t a, hmc_memory_stats *out) {
    return guarded([&]() -> hmc_status {
        if (a == nullptr || out == nullptr) return fail(HMC_INVALID, "null argument");
        std::lock_guard<std::mutex> lock(a->counter_mutex);
        *out = a->stats;
        return HMC_OK;
    });
}

HMC_API hmc_status hmc_allocator_reset_peak(hmc_allocator_t a) {
    return guarded([&]() -> hmc_status {
        if (a == nullptr) return fail(HMC_INVALID, "null allocator");
        std::lock_guard<std::mutex> lock(a->counter_mutex);
        a->stats.peak = a->stats.allocated;
        return HMC_OK;
    });
}
