// Stand-alone collectives over peer-mapped memory (NVLink): all-gather, all-to-all, reduce-scatter,
// two-shot all-reduce (reduce-scatter + all-gather in one kernel) and broadcast. The one-shot
// all-reduce for decode-sized messages, the barrier and the arg-max exchange live in tp_decode.cu.
//
// One kernel per call, the same on every rank: every CTA pushes its slice of this rank's data into
// the peers' receive areas (16-byte stores, data is never pulled), publishes one count per CTA to
// every peer (release), waits until every CTA of every rank has published (acquire, bounded), and
// then finishes locally (copy out, or sum the world's chunks in fp32). The two-shot all-reduce
// pushes the reduced chunk to every peer and waits once more. Receive areas are double-buffered by
// the parity of a per-communicator call counter kept on the device, and counters only grow, so a
// rank that runs ahead can neither overwrite data a slower rank still reads nor race a reset.
//
// Replaces the CPU-executed ring / mesh / tree algorithms of the reference
// (crates/rmlx-distributed/src/group.rs:877-1393, 1690-1830).
#include "../common/ptx.cuh"
#include "../common/launch.cuh"

namespace rb {

constexpr int kCollMaxRanks = 8;
constexpr int kCollThreads = 512;
enum CollOp { kAllGather = 0, kAllToAll = 1, kReduceScatter = 2, kAllReduce = 3, kBroadcast = 4 };

// control block (uint32): [0] calls completed, [1] exit ticket, [2] phase-1 arrivals (every call),
// [3] phase-2 arrivals (all-reduce calls only), [4] all-reduce calls completed, [5],[6] this rank's
// CTAs counting themselves before the last one publishes
struct CollPeers {
  char* buf[kCollMaxRanks];       // 2 parities x (recv area [world x chunk_cap] + result area [world x chunk_cap])
  uint32_t* ctl[kCollMaxRanks];
  int rank, world;
};

__device__ __forceinline__ void coll_copy(char* __restrict__ dst, const char* __restrict__ src, size_t bytes,
                                          size_t tid, size_t nthreads, bool volatile_src) {
  const size_t nvec = bytes / 16;
  const uint4* s = reinterpret_cast<const uint4*>(src);
  uint4* d = reinterpret_cast<uint4*>(dst);
  for (size_t i = tid; i < nvec; i += 4 * nthreads) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i + u * nthreads < nvec) v[u] = volatile_src ? __ldcg(s + i + u * nthreads) : s[i + u * nthreads];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i + u * nthreads < nvec) d[i + u * nthreads] = v[u];
  }
}

template <bool BF16>
__device__ __forceinline__ void coll_reduce(char* __restrict__ dst, const char* __restrict__ recv,
                                            size_t chunk_cap, size_t bytes, int world, size_t tid,
                                            size_t nthreads) {
  const size_t nvec = bytes / 16;
  for (size_t i = tid; i < nvec; i += nthreads) {
    float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < world; ++s) {
      const uint4 v = __ldcg(reinterpret_cast<const uint4*>(recv + size_t(s) * chunk_cap) + i);
      if (BF16) {
        f[0] += bf16lo(v.x); f[1] += bf16hi(v.x); f[2] += bf16lo(v.y); f[3] += bf16hi(v.y);
        f[4] += bf16lo(v.z); f[5] += bf16hi(v.z); f[6] += bf16lo(v.w); f[7] += bf16hi(v.w);
      } else {
        f[0] += __uint_as_float(v.x); f[1] += __uint_as_float(v.y);
        f[2] += __uint_as_float(v.z); f[3] += __uint_as_float(v.w);
      }
    }
    uint4 o;
    if (BF16) {
      o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]);
      o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
    } else {
      o.x = __float_as_uint(f[0]); o.y = __float_as_uint(f[1]);
      o.z = __float_as_uint(f[2]); o.w = __float_as_uint(f[3]);
    }
    reinterpret_cast<uint4*>(dst)[i] = o;
  }
}

// The CTAs of a rank first count themselves on a local word; the last one publishes a single
// arrival per peer (so a peer's counter sees ``world`` remote atomics per phase, not world x grid),
// then everyone waits for all ranks. Returns false after the wait budget.
__device__ __forceinline__ bool coll_rendezvous(const CollPeers& pp, int word, uint32_t target, int* s_ok,
                                                int* status) {
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* local = pp.ctl[pp.rank] + word + 3;        // words 5 and 6
    __threadfence_system();                              // this CTA's stores are visible everywhere
    if (atomicAdd(local, 1u) == gridDim.x - 1) {
      *local = 0u;
      __threadfence_system();
      for (int p = 0; p < pp.world; ++p) red_release_sys_add(pp.ctl[p] + word, 1u);
    }
    *s_ok = wait_flag_ge(pp.ctl[pp.rank] + word, target) ? 1 : 0;
    if (!*s_ok && status) atomicExch(status, int(kStatusPeerTimeout));
  }
  __syncthreads();
  return *s_ok != 0;
}

// chunk: bytes of one rank's piece (a multiple of 16); chunk_cap: bytes reserved per piece in the areas.
__global__ void __launch_bounds__(kCollThreads)
coll_kernel(CollPeers pp, int op, int bf16, const char* __restrict__ src, char* __restrict__ dst,
            size_t chunk, size_t chunk_cap, int root, int* __restrict__ status) {
  __shared__ int s_ok;
  const int rank = pp.rank, world = pp.world;
  uint32_t* ctl = pp.ctl[rank];
  const uint32_t e1 = ctl[0] + 1u;
  const uint32_t a1 = ctl[4] + 1u;          // the second rendezvous is counted per all-reduce call
  const size_t parity_off = (e1 & 1u) ? 0 : size_t(2) * world * chunk_cap;
  const size_t result_off = parity_off + size_t(world) * chunk_cap;
  const size_t tid = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t nthreads = size_t(gridDim.x) * blockDim.x;

  // phase 1: push
  for (int pi = 0; pi < world; ++pi) {
    int p = rank + pi; if (p >= world) p -= world;
    char* recv = pp.buf[p] + parity_off + size_t(rank) * chunk_cap;
    if (op == kAllGather) coll_copy(recv, src, chunk, tid, nthreads, false);
    else if (op == kBroadcast) { if (rank == root) coll_copy(pp.buf[p] + parity_off, src, chunk, tid, nthreads, false); }
    else coll_copy(recv, src + size_t(p) * chunk, chunk, tid, nthreads, false);
  }
  bool ok = coll_rendezvous(pp, 2, e1 * uint32_t(world), &s_ok, status);

  // phase 2: finish locally
  const char* mine = pp.buf[rank] + parity_off;
  if (ok) {
    if (op == kAllGather || op == kAllToAll) {
      for (int s = 0; s < world; ++s)
        coll_copy(dst + size_t(s) * chunk, mine + size_t(s) * chunk_cap, chunk, tid, nthreads, true);
    } else if (op == kBroadcast) {
      coll_copy(dst, mine, chunk, tid, nthreads, true);
    } else if (op == kReduceScatter) {
      if (bf16) coll_reduce<true>(dst, mine, chunk_cap, chunk, world, tid, nthreads);
      else coll_reduce<false>(dst, mine, chunk_cap, chunk, world, tid, nthreads);
    } else {   // all-reduce: reduce my chunk into my own result slot, then hand it to everyone
      char* red = pp.buf[rank] + result_off + size_t(rank) * chunk_cap;
      if (bf16) coll_reduce<true>(red, mine, chunk_cap, chunk, world, tid, nthreads);
      else coll_reduce<false>(red, mine, chunk_cap, chunk, world, tid, nthreads);
      // each thread forwards exactly the vectors it reduced, so no block-wide barrier is needed first
      const size_t nvec = chunk / 16;
      for (size_t i = tid; i < nvec; i += nthreads) {
        const uint4 v = reinterpret_cast<const uint4*>(red)[i];
        for (int pi = 1; pi < world; ++pi) {
          int p = rank + pi; if (p >= world) p -= world;
          reinterpret_cast<uint4*>(pp.buf[p] + result_off + size_t(rank) * chunk_cap)[i] = v;
        }
      }
      ok = coll_rendezvous(pp, 3, a1 * uint32_t(world), &s_ok, status);
      if (ok)
        for (int s = 0; s < world; ++s)
          coll_copy(dst + size_t(s) * chunk, pp.buf[rank] + result_off + size_t(s) * chunk_cap, chunk, tid,
                    nthreads, true);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(ctl + 1, 1u) == gridDim.x - 1) {
      ctl[1] = 0u;
      if (op == kAllReduce) ctl[4] = a1;
      __threadfence();
      ctl[0] = e1;
    }
  }
}

}  // namespace rb

using namespace rb;

// buf[r], ctl[r]: rank r's data and control areas as mapped in this process. ``chunk`` bytes per rank
// piece (multiple of 16, <= chunk_cap). Input/outputs by operation, n = chunk:
//   all-gather      src [n]           -> dst [world*n]
//   all-to-all      src [world*n]     -> dst [world*n]   (piece p goes to rank p)
//   reduce-scatter  src [world*n]     -> dst [n]         (sum over ranks of piece ``rank``)
//   all-reduce      src [world*n]     -> dst [world*n]   (sum over ranks)
//   broadcast       src [n] on root   -> dst [n]
// dtype: 0 raw bytes / fp32 sums, 1 bf16 sums (fp32 accumulation). Ranks may use different
// ``blocks`` (arrivals are published once per rank).
extern "C" int rmlx_coll(void* const* buf, void* const* ctl, int rank, int world, int op, int bf16,
                         const void* src, void* dst, unsigned long long chunk,
                         unsigned long long chunk_cap, int root, int blocks, int* status,
                         cudaStream_t st) {
  if (world < 1 || world > kCollMaxRanks || rank < 0 || rank >= world) return -2;
  if (op < 0 || op > kBroadcast || chunk == 0 || chunk % 16 || chunk > chunk_cap || chunk_cap % 16) return -2;
  if (root < 0 || root >= world) return -2;
  CollPeers pp;
  pp.rank = rank; pp.world = world;
  for (int p = 0; p < world; ++p) {
    pp.buf[p] = static_cast<char*>(buf[p]);
    pp.ctl[p] = static_cast<uint32_t*>(ctl[p]);
  }
  if (blocks < 1) blocks = 32;
  return launch(coll_kernel, dim3(blocks), dim3(kCollThreads), 0, st, false, pp, op, bf16,
                static_cast<const char*>(src), static_cast<char*>(dst), size_t(chunk), size_t(chunk_cap),
                root, status);
}

// bytes of a rank's data area for a given per-piece capacity
extern "C" unsigned long long rmlx_coll_area_bytes(int world, unsigned long long chunk_cap) {
  return 4ull * world * chunk_cap;
}
