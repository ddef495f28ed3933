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


def _run_ops(arena_alloc, arena_free, ops, align):
    """Replay (kind, value) operations; returns the live {offset: size} map after checking that no
    two live blocks overlap and that every offset is aligned."""
    live = {}
    order = []
    for kind, v in ops:
        if kind == "a":
            off = arena_alloc(v)
            if off is None:
                continue
            assert off % align == 0
            for o, n in live.items():
                assert off + v <= o or o + n <= off, "overlapping blocks"
            live[off] = v
            order.append(off)
        elif order:
            off = order.pop(v % len(order))
            arena_free(off, live.pop(off))
    return live, order


def test_arenas_never_overlap_and_coalesce_back_to_one_block():
    """Random allocate / free sequences (hypothesis) on the native BFC arena and on the symmetric
    heap's offset arena: blocks never overlap, offsets are aligned, two arenas fed the same sequence
    agree (ranks must derive the same offsets), and after freeing everything the whole range is one
    free block again."""
    from hypothesis import given, settings, strategies as st
    from rmlx_b200.parallel.symm_heap import OffsetArena
    from rmlx_b200.runtime.alloc import AllocError, BfcArena

    ops_st = st.lists(st.one_of(st.tuples(st.just("a"), st.integers(1, 5000)),
                                st.tuples(st.just("f"), st.integers(0, 1000))), max_size=60)

    @settings(max_examples=60, deadline=None, derandomize=True)
    @given(ops_st)
    def bfc(ops):
        size = 64 * 1024
        arenas = [BfcArena(size, alignment=256), BfcArena(size, alignment=256)]

        def alloc_on(a):
            def f(n):
                try:
                    return a.alloc(n)
                except AllocError:
                    return None
            return f
        results = [_run_ops(alloc_on(a), lambda off, _n, a=a: a.free(off), ops, 256) for a in arenas]
        assert results[0] == results[1]                      # deterministic across instances
        live, order = results[0]
        a = arenas[0]
        for off in list(order):
            a.free(off)
        assert a.in_use() == 0 and a.largest_free() == size  # everything coalesced
        for x in arenas:
            x.close()

    @settings(max_examples=60, deadline=None, derandomize=True)
    @given(ops_st)
    def offsets(ops):
        def fresh():
            a = OffsetArena()
            a.grow(32 * 1024)
            return a
        arenas = [fresh(), fresh()]
        results = [_run_ops(lambda n, a=a: a.take((n + 255) // 256 * 256),
                            lambda off, n, a=a: a.give(off, (n + 255) // 256 * 256), ops, 256) for a in arenas]
        assert results[0] == results[1]
        live, order = results[0]
        a = arenas[0]
        for off in list(order):
            a.give(off, (live[off] + 255) // 256 * 256)
        assert a.free == [(0, 32 * 1024)] and a.free_bytes() == 32 * 1024
        a.grow(1024)                                          # growth extends the last free range
        assert a.free == [(0, 33 * 1024)]

    bfc()
    offsets()
