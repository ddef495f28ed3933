"""Native allocator logic on host memory (no GPU): the cases of crates/rmlx-alloc/tests and the
inline tests of bfc.rs / cache.rs / allocator.rs (split/coalesce, best-fit window, LRU eviction,
limits, double-free and foreign-free detection, leak counters)."""
import zlib

import pytest

from rmlx_b200.runtime.alloc import AllocError, BfcArena, CachingAllocator, crc32


def test_bfc_split_coalesce_and_best_fit():
    a = BfcArena(1 << 20, alignment=256)
    x = a.alloc(1000)        # rounded to 1024
    y = a.alloc(4096)
    z = a.alloc(256)
    assert (x, y, z) == (0, 1024, 5120)
    assert a.in_use() == 1024 + 4096 + 256
    a.free(y)
    assert a.num_blocks() == 4                      # x | hole | z | tail
    w = a.alloc(2048)                                # best fit takes the hole, not the tail
    assert w == 1024
    a.free(w); a.free(x); a.free(z)
    assert a.num_blocks() == 1 and a.in_use() == 0 and a.largest_free() == 1 << 20
    assert a.peak() == 1024 + 4096 + 256
    with pytest.raises(AllocError):
        a.free(z)                                    # double free
    with pytest.raises(AllocError):
        a.alloc(2 << 20)


def test_bfc_is_deterministic_across_instances():
    # two "ranks" doing the same sequence get the same offsets: the symmetric-heap property
    seq = [300, 70000, 4096, 12, 999999]
    outs = []
    for _ in range(2):
        a = BfcArena(8 << 20)
        offs = [a.alloc(n) for n in seq]
        a.free(offs[1])
        offs.append(a.alloc(65536))
        outs.append(offs)
    assert outs[0] == outs[1]


def test_caching_allocator_cache_hit_and_stats():
    al = CachingAllocator()
    with pytest.raises(AllocError):
        al.alloc(0)
    p, sz = al.alloc(10000)
    assert sz == 12288                                # page-rounded
    al.free(p)
    q, sz2 = al.alloc(9000)                           # within the best-fit window -> same buffer
    assert q == p and sz2 == 12288
    st = al.stats()
    assert st.cache_hits == 1 and st.backing_allocs == 1 and st.allocs == 2 and st.frees == 1
    al.free(q)
    r, _ = al.alloc(4096)                             # 12288 > min(2*4096, 4096+8192): no reuse
    assert r != p
    al.free(r)
    assert not al.leak_detector().has_leaks()
    al.clear_cache()
    assert al.stats().cached_bytes == 0 and al.stats().backing_bytes == 0


def test_small_pool_and_ownership_checks():
    al = CachingAllocator()
    ptrs = [al.alloc(17)[0] for _ in range(10)]
    assert len(set(ptrs)) == 10
    assert all(abs(a - b) % 256 == 0 for a, b in zip(ptrs, ptrs[1:]))
    assert al.stats().small_allocs == 10 and al.stats().backing_allocs == 1
    for p in ptrs:
        al.free(p)
    with pytest.raises(AllocError, match="double free"):
        al.free(ptrs[0])
    with pytest.raises(AllocError, match="does not own"):
        al.free(0xDEAD000)
    st = al.stats()
    assert st.errors_double_free == 1 and st.errors_foreign_free == 1


def test_limits_and_gc():
    al = CachingAllocator(memory_limit=1 << 20, cache_limit=256 << 10)
    a, _ = al.alloc(512 << 10)
    b, _ = al.alloc(400 << 10)
    with pytest.raises(AllocError):
        al.alloc(512 << 10)                           # over the memory limit
    al.free(a)                                        # 512K cached > 256K cache limit -> evicted
    assert al.stats().cached_bytes == 0
    c, _ = al.alloc(512 << 10)                        # fits again
    al.free(b); al.free(c)
    assert al.stats().gc_runs >= 1
    assert al.leak_detector().outstanding() == 0
    al.reset_peak_memory()
    assert al.stats().peak == 0


def test_crc32_matches_zlib():
    for data in (b"", b"a", b"hello world" * 100):
        assert crc32(data) == zlib.crc32(data)
