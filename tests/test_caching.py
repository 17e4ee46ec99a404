"""The native caching allocator over a fake device with a capacity and an operation log, without a GPU: the
scenarios of homura's own allocator tests (src/backend/caching.rs:295-572), here driven through the C ABI
of include/homura_cuda_alloc.h."""
import threading

import pytest

from homura_b200 import caching
from homura_b200.caching import CachingAllocator, MallocOutOfMemory, OutOfMemory, PoolFailed

MIB = 1 << 20
SEGMENT = 2 * MIB


class FakeMemory:
    """Memory with a capacity, handing out increasing addresses and recording what it did."""

    def __init__(self, capacity):
        self.capacity, self.used, self.next = capacity, 0, 1 << 40
        self.live, self.log = {}, []
        self.fail_mallocs, self.fail_free = 0, False

    def malloc(self, size):
        if self.fail_mallocs > 0:
            self.fail_mallocs -= 1
            raise RuntimeError("injected")
        if self.used + size > self.capacity:
            self.log.append(f"oom {size}")
            raise MallocOutOfMemory()
        addr = self.next
        self.next += size + 4096
        self.used += size
        self.live[addr] = size
        self.log.append(f"malloc {size}")
        return addr

    def free(self, addr):
        if self.fail_free:
            raise RuntimeError("free failed")
        size = self.live.pop(addr)
        self.used -= size
        self.log.append(f"free {size}")

    def synchronize(self):
        self.log.append("sync")


def allocator(capacity):
    mem = FakeMemory(capacity)
    return CachingAllocator(mem), mem


def take_log(mem):
    out, mem.log = mem.log, []
    return out


def stats(a):
    s = a.memory_stats()
    return s["allocated"], s["reserved"], s["peak"]


def alloc(a, n):
    b = a.allocate(n)
    b.live = False  # the tests release by address, explicitly
    return b


def test_requests_are_rounded():
    assert caching.rounded(1) == (512, True)
    assert caching.rounded(512) == (512, True)
    assert caching.rounded(513) == (1024, True)
    assert caching.rounded(MIB) == (MIB, True)
    assert caching.rounded(MIB + 1) == (2 * MIB, False)
    assert caching.rounded(5 * MIB) == (6 * MIB, False)
    assert caching.rounded(2**64 - 1) is None
    a, _ = allocator(64 * MIB)
    with pytest.raises(OutOfMemory):
        a.allocate(2**64 - 1)


def test_small_requests_share_a_segment():
    a, mem = allocator(64 * MIB)
    b1, b2, b3 = alloc(a, 100), alloc(a, 1000), alloc(a, MIB)
    assert (b1.size, b2.size, b3.size) == (512, 1024, MIB)
    assert b2.ptr == b1.ptr + 512 and b3.ptr == b2.ptr + 1024
    assert take_log(mem) == ["malloc 2097152"]
    assert stats(a) == (512 + 1024 + MIB, 2 * MIB, 512 + 1024 + MIB)
    b4 = alloc(a, MIB)
    assert take_log(mem) == ["malloc 2097152"]
    assert b4.ptr >= b1.ptr + SEGMENT
    assert stats(a)[1] == 4 * MIB


def test_large_requests_get_their_own_segment():
    a, mem = allocator(64 * MIB)
    b = alloc(a, 3 * MIB)
    assert b.size == 4 * MIB and take_log(mem) == ["malloc 4194304"]
    a.release(b.ptr)
    c = alloc(a, 2 * MIB)
    assert (c.ptr, c.size) == (b.ptr, 2 * MIB)
    d = alloc(a, 2 * MIB)
    assert d.ptr == b.ptr + 2 * MIB and take_log(mem) == []
    e = alloc(a, 512)
    assert take_log(mem) == ["malloc 2097152"]
    assert e.ptr < b.ptr or e.ptr >= b.ptr + 4 * MIB


def test_freed_blocks_are_reused_best_fit():
    a, mem = allocator(64 * MIB)
    blocks = [alloc(a, n) for n in (4096, 512, 1024, 512, 8192)]
    a.release(blocks[0].ptr)
    a.release(blocks[2].ptr)
    got = alloc(a, 600)
    assert (got.ptr, got.size) == (blocks[2].ptr, 1024)
    c = alloc(a, 2048)
    assert (c.ptr, c.size) == (blocks[0].ptr, 2048)
    assert alloc(a, 2048).ptr == blocks[0].ptr + 2048
    assert take_log(mem) == ["malloc 2097152"]


def test_freed_neighbours_merge_and_whole_segments_are_released():
    a, mem = allocator(64 * MIB)
    small = [alloc(a, 512) for _ in range(4)]
    large = alloc(a, 2 * MIB)
    assert take_log(mem) == ["malloc 2097152", "malloc 2097152"]
    for i in (1, 3, 0):
        a.release(small[i].ptr)
    a.empty_cache()
    assert take_log(mem) == []
    a.release(small[2].ptr)
    whole = alloc(a, MIB)
    assert whole.ptr == small[0].ptr
    a.release(whole.ptr)
    a.empty_cache()
    assert take_log(mem) == ["sync", "free 2097152"]
    assert stats(a) == (2 * MIB, 2 * MIB, 3 * MIB)
    a.release(large.ptr)
    a.empty_cache()
    assert take_log(mem) == ["sync", "free 2097152"]
    assert stats(a)[:2] == (0, 0)
    a.empty_cache()
    assert take_log(mem) == []


def test_out_of_memory_releases_the_cache_and_retries_once():
    a, mem = allocator(8 * MIB)
    x, y = alloc(a, 4 * MIB), alloc(a, 512)
    a.release(x.ptr)
    take_log(mem)
    z = alloc(a, 6 * MIB)
    assert z.size == 6 * MIB
    assert take_log(mem) == ["oom 6291456", "sync", "free 4194304", "malloc 6291456"]
    assert stats(a)[1] == 8 * MIB
    before = stats(a)
    with pytest.raises(OutOfMemory) as e:
        a.allocate(4 * MIB)
    assert "Tried to allocate 4.00 MiB" in str(e.value)
    assert take_log(mem) == ["oom 4194304", "oom 4194304"]
    assert stats(a) == before
    a.release(y.ptr)
    a.release(z.ptr)
    assert alloc(a, 4 * MIB).ptr == z.ptr


def test_device_failures_are_reported():
    a, mem = allocator(8 * MIB)
    mem.fail_mallocs = 1
    with pytest.raises(PoolFailed, match="injected"):
        a.allocate(512)
    assert stats(a) == (0, 0, 0)
    b = alloc(a, 512)
    a.release(b.ptr)
    mem.fail_free = True
    with pytest.raises(PoolFailed, match="free failed"):
        a.empty_cache()


def test_the_peak_follows_allocations_and_resets_to_the_current_value():
    a, _ = allocator(64 * MIB)
    x, y = alloc(a, 3 * MIB), alloc(a, MIB)
    a.release(x.ptr)
    assert stats(a) == (MIB, 6 * MIB, 5 * MIB)
    a.reset_peak_memory_stats()
    assert stats(a)[2] == MIB
    a.release(y.ptr)
    assert stats(a) == (0, 6 * MIB, MIB)


def test_a_double_free_is_refused():
    a, _ = allocator(8 * MIB)
    b = alloc(a, 512)
    a.release(b.ptr)
    with pytest.raises(PoolFailed, match="freeing a block twice"):
        a.release(b.ptr)
    with pytest.raises(PoolFailed, match="doesn't know"):
        a.release(12345)


def test_zero_bytes_take_no_block():
    a, mem = allocator(8 * MIB)
    b = a.allocate(0)
    assert b.ptr == 0 and b.size == 0 and take_log(mem) == [] and stats(a) == (0, 0, 0)


def test_blocks_are_freed_from_many_threads():
    a, mem = allocator(256 * MIB)
    errors = []

    def work(t):
        try:
            for i in range(200):
                b = alloc(a, 1 + (t * 7919 + i * 104729) % (3 * MIB))
                a.release(b.ptr)
        except Exception as e:  # pragma: no cover
            errors.append(e)

    threads = [threading.Thread(target=work, args=(t,)) for t in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors
    assert stats(a)[0] == 0
    a.empty_cache()
    assert stats(a)[1] == 0 and not mem.live


def test_blocks_release_themselves_when_dropped():
    a, _ = allocator(8 * MIB)
    b = a.allocate(1000)
    assert stats(a)[0] == 1024
    del b
    assert stats(a)[0] == 0
