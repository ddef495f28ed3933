// Host-side memory management for device buffers: a best-fit-with-coalescing arena, a size-binned
// reuse cache, a fixed-slot pool for tiny buffers, and the caching allocator that ties them
// together with limits, ownership checks and leak statistics.
//
// The backing store is a pair of function pointers (alloc/free), so the same code manages plain
// cudaMalloc memory, a symmetric peer-mapped region (every rank performs the same allocation
// sequence and therefore gets the same offsets), or host memory in CPU tests.
//
// Capabilities follow the reference's allocator crate: MetalAllocator (zero-size reject, small
// pool for <= 256 B, limits, cache-first, GC at a threshold, double-free / foreign-free detection;
// crates/rmlx-alloc/src/allocator.rs:178-478), BufferCache (page-aligned size bins, best fit within
// min(2x, +2 pages), LRU eviction; crates/rmlx-alloc/src/cache.rs:18-140), BfcAllocator
// (crates/rmlx-alloc/src/bfc.rs:111-390), SmallBufferPool (crates/rmlx-alloc/src/small_alloc.rs:54-160),
// AllocStats / LeakDetector (crates/rmlx-alloc/src/stats.rs, leak_detector.rs).
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <list>
#include <map>
#include <mutex>
#include <set>
#include <unordered_map>
#include <vector>

namespace {

constexpr uint64_t kPage = 4096;
inline uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

// ------------------------------------------------------------------------------------------------
// Best-fit with coalescing over one contiguous region addressed by offsets.
// ------------------------------------------------------------------------------------------------
class Bfc {
 public:
  Bfc(uint64_t size, uint64_t alignment) : size_(size), align_(alignment ? alignment : 256) {
    blocks_[0] = Block{size, true};
    free_.insert({size, 0});
  }
  // Returns offset or UINT64_MAX.
  uint64_t alloc(uint64_t bytes) {
    if (bytes == 0) return UINT64_MAX;
    bytes = align_up(bytes, align_);
    auto it = free_.lower_bound({bytes, 0});
    if (it == free_.end()) return UINT64_MAX;
    const uint64_t off = it->second, have = it->first;
    free_.erase(it);
    Block& b = blocks_[off];
    b.free = false;
    if (have > bytes) {  // split
      b.size = bytes;
      blocks_[off + bytes] = Block{have - bytes, true};
      free_.insert({have - bytes, off + bytes});
    }
    in_use_ += bytes;
    if (in_use_ > peak_) peak_ = in_use_;
    return off;
  }
  // 0 ok, -1 unknown offset, -2 double free
  int release(uint64_t off) {
    auto it = blocks_.find(off);
    if (it == blocks_.end()) return -1;
    if (it->second.free) return -2;
    in_use_ -= it->second.size;
    it->second.free = true;
    // coalesce with next
    auto nx = std::next(it);
    if (nx != blocks_.end() && nx->second.free) {
      free_.erase({nx->second.size, nx->first});
      it->second.size += nx->second.size;
      blocks_.erase(nx);
    }
    // coalesce with previous
    if (it != blocks_.begin()) {
      auto pv = std::prev(it);
      if (pv->second.free) {
        free_.erase({pv->second.size, pv->first});
        pv->second.size += it->second.size;
        blocks_.erase(it);
        it = pv;
      }
    }
    free_.insert({it->second.size, it->first});
    return 0;
  }
  uint64_t in_use() const { return in_use_; }
  uint64_t peak() const { return peak_; }
  uint64_t largest_free() const { return free_.empty() ? 0 : free_.rbegin()->first; }
  uint64_t num_blocks() const { return blocks_.size(); }
  uint64_t size() const { return size_; }
  uint64_t block_size(uint64_t off) const {
    auto it = blocks_.find(off);
    return it == blocks_.end() ? 0 : it->second.size;
  }

 private:
  struct Block { uint64_t size; bool free; };
  uint64_t size_, align_, in_use_ = 0, peak_ = 0;
  std::map<uint64_t, Block> blocks_;                  // offset -> block
  std::set<std::pair<uint64_t, uint64_t>> free_;      // (size, offset)
};

// ------------------------------------------------------------------------------------------------
// Size-binned cache of released buffers.
// ------------------------------------------------------------------------------------------------
class BufferCache {
 public:
  explicit BufferCache(uint64_t max_bytes) : max_(max_bytes) {}
  // Best fit: smallest cached buffer with size in [want, min(2*want, want + 2 pages)].
  bool take(uint64_t want, uint64_t* addr, uint64_t* size) {
    want = align_up(want, kPage);
    auto it = bins_.lower_bound(want);
    const uint64_t hi = std::min(2 * want, want + 2 * kPage);
    if (it == bins_.end() || it->first > hi || it->second.empty()) { ++miss_; return false; }
    auto lit = it->second.back();
    it->second.pop_back();
    *addr = lit->addr; *size = lit->size;
    lru_.erase(lit);
    if (it->second.empty()) bins_.erase(it);
    bytes_ -= *size;
    ++hit_;
    return true;
  }
  void put(uint64_t addr, uint64_t size) {
    lru_.push_front(Entry{addr, size});
    bins_[size].push_back(lru_.begin());
    bytes_ += size;
  }
  // Evict least-recently-released entries until at most `target` bytes remain.
  template <class F>
  uint64_t evict_to(uint64_t target, F&& free_fn) {
    uint64_t freed = 0;
    while (bytes_ > target && !lru_.empty()) {
      auto last = std::prev(lru_.end());
      auto& v = bins_[last->size];
      for (size_t i = 0; i < v.size(); ++i)
        if (v[i] == last) { v.erase(v.begin() + i); break; }
      if (v.empty()) bins_.erase(last->size);
      bytes_ -= last->size;
      freed += last->size;
      free_fn(last->addr, last->size);
      lru_.erase(last);
    }
    return freed;
  }
  uint64_t bytes() const { return bytes_; }
  uint64_t max_bytes() const { return max_; }
  void set_max(uint64_t m) { max_ = m; }
  uint64_t hits() const { return hit_; }
  uint64_t misses() const { return miss_; }

 private:
  struct Entry { uint64_t addr, size; };
  std::list<Entry> lru_;
  std::map<uint64_t, std::vector<std::list<Entry>::iterator>> bins_;
  uint64_t bytes_ = 0, max_, hit_ = 0, miss_ = 0;
};

typedef uint64_t (*BackAlloc)(uint64_t bytes, void* ctx);   // returns address or 0
typedef void (*BackFree)(uint64_t addr, uint64_t bytes, void* ctx);

uint64_t host_alloc(uint64_t bytes, void*) {
  void* p = nullptr;
  if (posix_memalign(&p, 256, bytes) != 0) return 0;
  return reinterpret_cast<uint64_t>(p);
}
void host_free(uint64_t addr, uint64_t, void*) { free(reinterpret_cast<void*>(addr)); }

struct Stats {
  uint64_t allocs = 0, frees = 0, bytes_in_use = 0, peak = 0, backing_allocs = 0, backing_bytes = 0,
           cache_hits = 0, cache_misses = 0, small_allocs = 0, errors_double_free = 0,
           errors_foreign_free = 0, gc_runs = 0, cached_bytes = 0;
};

// ------------------------------------------------------------------------------------------------
// Caching allocator.
// ------------------------------------------------------------------------------------------------
class CachingAllocator {
 public:
  CachingAllocator(BackAlloc a, BackFree f, void* ctx, uint64_t memory_limit, uint64_t cache_limit,
                   uint64_t gc_limit)
      : alloc_(a ? a : host_alloc), free_(f ? f : host_free), ctx_(ctx), memory_limit_(memory_limit),
        gc_limit_(gc_limit), cache_(cache_limit) {}
  ~CachingAllocator() {
    cache_.evict_to(0, [&](uint64_t addr, uint64_t sz) { free_(addr, sz, ctx_); });
    for (auto s : small_slabs_) free_(s, kSmallSlab, ctx_);
  }

  // 0 = failure (zero size, over limit, backing failure). *out_size receives the usable size.
  uint64_t allocate(uint64_t bytes, uint64_t* out_size) {
    std::lock_guard<std::mutex> g(mu_);
    if (bytes == 0) return 0;
    if (bytes <= kSmallSlot) {
      const uint64_t a = small_alloc();
      if (a) {
        owned_[a] = Owned{kSmallSlot, true};
        note_alloc(kSmallSlot);
        ++st_.small_allocs;
        if (out_size) *out_size = kSmallSlot;
        return a;
      }
    }
    const uint64_t want = align_up(bytes, kPage);
    uint64_t addr = 0, size = 0;
    if (cache_.take(want, &addr, &size)) {
      ++st_.cache_hits;
    } else {
      ++st_.cache_misses;
      if (memory_limit_ && st_.backing_bytes + want > memory_limit_) {
        // try to make room by dropping cached buffers before giving up
        run_gc(0);
        if (st_.backing_bytes + want > memory_limit_) return 0;
      }
      addr = alloc_(want, ctx_);
      if (!addr) {
        run_gc(0);
        addr = alloc_(want, ctx_);
        if (!addr) return 0;
      }
      size = want;
      ++st_.backing_allocs;
      st_.backing_bytes += want;
    }
    owned_[addr] = Owned{size, false};
    released_.erase(addr);
    note_alloc(size);
    if (out_size) *out_size = size;
    return addr;
  }

  // 0 ok, -1 foreign pointer, -2 double free
  int release(uint64_t addr) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = owned_.find(addr);
    if (it == owned_.end()) {
      if (released_.count(addr)) { ++st_.errors_double_free; return -2; }
      ++st_.errors_foreign_free;
      return -1;
    }
    const Owned o = it->second;
    owned_.erase(it);
    released_.insert(addr);
    if (released_.size() > 65536) released_.clear();
    ++st_.frees;
    st_.bytes_in_use -= o.size;
    if (o.small) { small_free_.push_back(addr); return 0; }
    cache_.put(addr, o.size);
    if (cache_.bytes() > cache_.max_bytes()) run_gc(cache_.max_bytes());
    else if (gc_limit_ && cache_.bytes() > gc_limit_) run_gc(gc_limit_ / 2);
    return 0;
  }

  void clear_cache() { std::lock_guard<std::mutex> g(mu_); run_gc(0); }
  void set_limits(uint64_t mem, uint64_t cache, uint64_t gc) {
    std::lock_guard<std::mutex> g(mu_);
    memory_limit_ = mem; cache_.set_max(cache); gc_limit_ = gc;
  }
  void reset_peak() { std::lock_guard<std::mutex> g(mu_); st_.peak = st_.bytes_in_use; }
  Stats stats() {
    std::lock_guard<std::mutex> g(mu_);
    Stats s = st_;
    s.cached_bytes = cache_.bytes();
    return s;
  }
  uint64_t outstanding() { std::lock_guard<std::mutex> g(mu_); return owned_.size(); }

 private:
  static constexpr uint64_t kSmallSlot = 256, kSmallSlab = 64 * 1024;
  struct Owned { uint64_t size; bool small; };
  void note_alloc(uint64_t size) {
    ++st_.allocs;
    st_.bytes_in_use += size;
    if (st_.bytes_in_use > st_.peak) st_.peak = st_.bytes_in_use;
  }
  uint64_t small_alloc() {
    if (small_free_.empty()) {
      const uint64_t slab = alloc_(kSmallSlab, ctx_);
      if (!slab) return 0;
      small_slabs_.push_back(slab);
      st_.backing_bytes += kSmallSlab;
      ++st_.backing_allocs;
      for (uint64_t o = 0; o < kSmallSlab; o += kSmallSlot) small_free_.push_back(slab + o);
    }
    const uint64_t a = small_free_.back();
    small_free_.pop_back();
    released_.erase(a);
    return a;
  }
  void run_gc(uint64_t target) {
    ++st_.gc_runs;
    const uint64_t freed = cache_.evict_to(target, [&](uint64_t addr, uint64_t sz) {
      free_(addr, sz, ctx_);
      released_.erase(addr);
    });
    st_.backing_bytes -= freed;
  }

  BackAlloc alloc_;
  BackFree free_;
  void* ctx_;
  uint64_t memory_limit_, gc_limit_;
  BufferCache cache_;
  std::unordered_map<uint64_t, Owned> owned_;
  std::set<uint64_t> released_;
  std::vector<uint64_t> small_free_, small_slabs_;
  Stats st_;
  std::mutex mu_;
};

}  // namespace

extern "C" {

// ---- BFC arena -----------------------------------------------------------------------------------
void* rmlx_bfc_create(uint64_t size, uint64_t alignment) { return new Bfc(size, alignment); }
void rmlx_bfc_destroy(void* h) { delete static_cast<Bfc*>(h); }
uint64_t rmlx_bfc_alloc(void* h, uint64_t bytes) { return static_cast<Bfc*>(h)->alloc(bytes); }
int rmlx_bfc_free(void* h, uint64_t off) { return static_cast<Bfc*>(h)->release(off); }
uint64_t rmlx_bfc_in_use(void* h) { return static_cast<Bfc*>(h)->in_use(); }
uint64_t rmlx_bfc_peak(void* h) { return static_cast<Bfc*>(h)->peak(); }
uint64_t rmlx_bfc_largest_free(void* h) { return static_cast<Bfc*>(h)->largest_free(); }
uint64_t rmlx_bfc_num_blocks(void* h) { return static_cast<Bfc*>(h)->num_blocks(); }
uint64_t rmlx_bfc_block_size(void* h, uint64_t off) { return static_cast<Bfc*>(h)->block_size(off); }

// ---- caching allocator ---------------------------------------------------------------------------
// alloc_fn / free_fn may be null (host memory). Limits of 0 mean "none".
void* rmlx_alloc_create(void* alloc_fn, void* free_fn, void* ctx, uint64_t memory_limit,
                        uint64_t cache_limit, uint64_t gc_limit) {
  return new CachingAllocator(reinterpret_cast<BackAlloc>(alloc_fn),
                              reinterpret_cast<BackFree>(free_fn), ctx, memory_limit,
                              cache_limit ? cache_limit : UINT64_MAX, gc_limit);
}
void rmlx_alloc_destroy(void* h) { delete static_cast<CachingAllocator*>(h); }
uint64_t rmlx_alloc_malloc(void* h, uint64_t bytes, uint64_t* out_size) {
  return static_cast<CachingAllocator*>(h)->allocate(bytes, out_size);
}
int rmlx_alloc_free(void* h, uint64_t addr) { return static_cast<CachingAllocator*>(h)->release(addr); }
void rmlx_alloc_clear_cache(void* h) { static_cast<CachingAllocator*>(h)->clear_cache(); }
void rmlx_alloc_set_limits(void* h, uint64_t mem, uint64_t cache, uint64_t gc) {
  static_cast<CachingAllocator*>(h)->set_limits(mem, cache ? cache : UINT64_MAX, gc);
}
void rmlx_alloc_reset_peak(void* h) { static_cast<CachingAllocator*>(h)->reset_peak(); }
uint64_t rmlx_alloc_outstanding(void* h) { return static_cast<CachingAllocator*>(h)->outstanding(); }
// out: 13 uint64 in the order of struct Stats
void rmlx_alloc_stats(void* h, uint64_t* out) {
  const Stats s = static_cast<CachingAllocator*>(h)->stats();
  const uint64_t v[13] = {s.allocs, s.frees, s.bytes_in_use, s.peak, s.backing_allocs,
                          s.backing_bytes, s.cache_hits, s.cache_misses, s.small_allocs,
                          s.errors_double_free, s.errors_foreign_free, s.gc_runs, s.cached_bytes};
  memcpy(out, v, sizeof(v));
}

// ---- CRC32 (IEEE) for framed host-side messages ----------------------------------------------------
uint32_t rmlx_crc32(const uint8_t* data, uint64_t n, uint32_t seed) {
  static uint32_t table[256];
  static bool init = false;
  if (!init) {
    for (uint32_t i = 0; i < 256; ++i) {
      uint32_t c = i;
      for (int k = 0; k < 8; ++k) c = (c & 1) ? 0xEDB88320u ^ (c >> 1) : c >> 1;
      table[i] = c;
    }
    init = true;
  }
  uint32_t c = ~seed;
  for (uint64_t i = 0; i < n; ++i) c = table[(c ^ data[i]) & 0xff] ^ (c >> 8);
  return ~c;
}

}  // extern "C"
