// Native execution runtime: a keyed store of instantiated CUDA graphs (capture, replay, LRU
// eviction, counters) and events with deadline-bounded, cancellable host waits.
//
// The store is what the reference's ExecGraph + IcbCache are to Metal command buffers
// (crates/rmlx-metal/src/exec_graph.rs:110-401, crates/rmlx-metal/src/icb.rs:320-420): a decode
// step is recorded once per batch bucket and replayed with no per-kernel host work. Capture is
// "thread local": other threads may keep using the device while this thread records. Anything
// recorded must be allocation-free (a graph replays the addresses it was recorded with), which is
// for the caller to guarantee; the store only records, instantiates, launches and evicts.
//
// Events follow GpuEvent / GpuFence (crates/rmlx-metal/src/event.rs:15-117, fence.rs:24-130): a
// host wait polls with spin -> yield -> sleep, gives up at a deadline, and can be cancelled
// through a flag another thread sets.
#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <cstdint>
#include <list>
#include <mutex>
#include <thread>
#include <unordered_map>

namespace {

struct Entry {
  uint64_t key;
  cudaGraph_t graph;
  cudaGraphExec_t exec;
  size_t nodes;
};

struct Store {
  std::mutex mu;
  size_t max_entries;
  cudaStream_t stream = nullptr;   // the store's own recording stream (created on first request)
  std::list<Entry> lru;                                          // front = most recently used
  std::unordered_map<uint64_t, std::list<Entry>::iterator> by_key;
  uint64_t hits = 0, misses = 0, captures = 0, evictions = 0, launches = 0;
  bool capturing = false;

  void drop(std::list<Entry>::iterator it) {
    cudaGraphExecDestroy(it->exec);
    cudaGraphDestroy(it->graph);
    by_key.erase(it->key);
    lru.erase(it);
  }
};

}  // namespace

extern "C" void* rmlx_graphs_create(int max_entries) {
  Store* s = new Store();
  s->max_entries = max_entries > 0 ? size_t(max_entries) : 1;
  return s;
}

extern "C" void rmlx_graphs_destroy(void* h) {
  Store* s = static_cast<Store*>(h);
  if (!s) return;
  {
    std::lock_guard<std::mutex> g(s->mu);
    while (!s->lru.empty()) s->drop(s->lru.begin());
    if (s->stream) cudaStreamDestroy(s->stream);
  }
  delete s;
}

// The store's own non-blocking stream for recording (null when it cannot be created). Recording on
// a stream that nothing else uses keeps the recording's mode and dependencies away from streams
// that other capture mechanisms pick from a shared pool.
extern "C" void* rmlx_graphs_stream(void* h) {
  Store* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  if (!s->stream && cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking) != cudaSuccess) {
    cudaGetLastError();
    s->stream = nullptr;
  }
  return s->stream;
}

// 1 when a graph is stored under `key` (counts a hit or a miss).
extern "C" int rmlx_graphs_has(void* h, uint64_t key) {
  Store* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  const bool has = s->by_key.count(key) != 0;
  (has ? s->hits : s->misses)++;
  return has ? 1 : 0;
}

// Starts recording everything this thread submits to `st` (not the legacy default stream).
extern "C" int rmlx_graphs_begin(void* h, cudaStream_t st) {
  Store* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  if (s->capturing || st == nullptr) return -2;
  if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) != cudaSuccess) return -1;
  s->capturing = true;
  return 0;
}

// Ends the recording and stores the instantiated graph under `key` (replacing an older one and
// evicting the least recently used entry beyond the bound). Returns the number of nodes, < 0 on error.
extern "C" int rmlx_graphs_end(void* h, uint64_t key, cudaStream_t st) {
  Store* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  if (!s->capturing) return -2;
  s->capturing = false;
  cudaGraph_t graph = nullptr;
  if (cudaStreamEndCapture(st, &graph) != cudaSuccess || graph == nullptr) {
    cudaGetLastError();
    return -1;
  }
  cudaGraphExec_t exec = nullptr;
  if (cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess) {
    cudaGetLastError();
    cudaGraphDestroy(graph);
    return -1;
  }
  size_t nodes = 0;
  cudaGraphGetNodes(graph, nullptr, &nodes);
  auto old = s->by_key.find(key);
  if (old != s->by_key.end()) s->drop(old->second);
  s->lru.push_front(Entry{key, graph, exec, nodes});
  s->by_key[key] = s->lru.begin();
  s->captures++;
  while (s->lru.size() > s->max_entries) {
    s->drop(std::prev(s->lru.end()));
    s->evictions++;
  }
  return int(nodes);
}

// Ends a recording whose body failed and throws the result away.
extern "C" int rmlx_graphs_abort(void* h, cudaStream_t st) {
  Store* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  if (!s->capturing) return 0;
  s->capturing = false;
  cudaGraph_t graph = nullptr;
  cudaStreamEndCapture(st, &graph);
  cudaGetLastError();
  if (graph) cudaGraphDestroy(graph);
  return 0;
}

// Replays the graph stored under `key` on `st`. -3: nothing stored under that key.
extern "C" int rmlx_graphs_launch(void* h, uint64_t key, cudaStream_t st) {
  Store* s = static_cast<Store*>(h);
  cudaGraphExec_t exec;
  {
    std::lock_guard<std::mutex> g(s->mu);
    auto it = s->by_key.find(key);
    if (it == s->by_key.end()) return -3;
    s->lru.splice(s->lru.begin(), s->lru, it->second);
    exec = it->second->exec;
    s->launches++;
  }
  return cudaGraphLaunch(exec, st) == cudaSuccess ? 0 : -1;
}

// Drops one entry (or all with all != 0). Returns how many were dropped.
extern "C" int rmlx_graphs_invalidate(void* h, uint64_t key, int all) {
  Store* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  int n = 0;
  if (all) {
    while (!s->lru.empty()) { s->drop(s->lru.begin()); ++n; }
  } else {
    auto it = s->by_key.find(key);
    if (it != s->by_key.end()) { s->drop(it->second); n = 1; }
  }
  return n;
}

// out[0..6] = entries, hits, misses, captures, evictions, launches, nodes of the most recent entry.
extern "C" void rmlx_graphs_stats(void* h, uint64_t* out) {
  Store* s = static_cast<Store*>(h);
  std::lock_guard<std::mutex> g(s->mu);
  out[0] = s->lru.size(); out[1] = s->hits; out[2] = s->misses; out[3] = s->captures;
  out[4] = s->evictions; out[5] = s->launches;
  out[6] = s->lru.empty() ? 0 : s->lru.front().nodes;
}

// ------------------------------------------------------------------------------------------------
// Events with bounded host waits
// ------------------------------------------------------------------------------------------------
extern "C" void* rmlx_event_create(int timing) {
  cudaEvent_t ev = nullptr;
  if (cudaEventCreateWithFlags(&ev, timing ? cudaEventDefault : cudaEventDisableTiming) != cudaSuccess) return nullptr;
  return ev;
}

extern "C" void rmlx_event_destroy(void* ev) {
  if (ev) cudaEventDestroy(static_cast<cudaEvent_t>(ev));
}

extern "C" int rmlx_event_record(void* ev, cudaStream_t st) {
  return cudaEventRecord(static_cast<cudaEvent_t>(ev), st) == cudaSuccess ? 0 : -1;
}

// Makes `st` wait (on the device) for the work recorded before `ev`.
extern "C" int rmlx_event_stream_wait(void* ev, cudaStream_t st) {
  return cudaStreamWaitEvent(st, static_cast<cudaEvent_t>(ev), 0) == cudaSuccess ? 0 : -1;
}

// Host wait: 0 = complete, 1 = the deadline passed, 2 = cancelled (*cancel became non-zero),
// -1 = the event reports an error. Polls: 2000 spins, then yields, then 50 us sleeps.
extern "C" int rmlx_event_wait_host(void* ev, long long timeout_us, const volatile int* cancel) {
  const auto t0 = std::chrono::steady_clock::now();
  for (uint64_t i = 0;; ++i) {
    const cudaError_t e = cudaEventQuery(static_cast<cudaEvent_t>(ev));
    if (e == cudaSuccess) return 0;
    if (e != cudaErrorNotReady) { cudaGetLastError(); return -1; }
    if (cancel && *cancel) return 2;
    if (timeout_us >= 0) {
      const auto dt = std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
      if (dt >= timeout_us) return 1;
    }
    if (i < 2000) continue;
    if (i < 4000) std::this_thread::yield();
    else std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

extern "C" float rmlx_event_elapsed_ms(void* a, void* b) {
  float ms = -1.f;
  if (cudaEventElapsedTime(&ms, static_cast<cudaEvent_t>(a), static_cast<cudaEvent_t>(b)) != cudaSuccess) {
    cudaGetLastError();
    return -1.f;
  }
  return ms;
}
