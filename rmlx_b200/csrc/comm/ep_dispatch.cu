// Expert-parallel dispatch and combine over peer-mapped memory (NVLink), one kernel each.
//
// Dispatch: every rank has routed its T tokens to top-k experts (global ids) and knows how many
// pairs go to each expert (the router's counts). The kernel
//   1. all-gathers the count vectors by storing them into every peer's table,
//   2. derives from the full [world][E] table where each (expert, source rank) block starts in the
//      destination rank's slab — rows are laid out grouped by local expert, then by source rank,
//      which is exactly the layout the grouped expert GEMM consumes, so nothing is permuted on
//      arrival,
//   3. copies each token row straight into its slot of the destination slab (8 KB peer stores per
//      row, a warp per row) together with a return address (source rank, pair index),
//   4. counts arrivals and returns when every inbound row has landed.
// Nothing is dropped and there is no capacity factor: the only limit is the slab size, checked
// before any store (an overflow sets the status word and skips the call's stores on every rank,
// because every rank sees the same table).
//
// Combine: the owner of each expert row stores the expert output back to the source rank's return
// buffer at the pair index; when all k x T rows are back, the source computes
// out[t] = residual[t] + sum_s w[t,s] * ret[t*k+s].
//
// Counters only grow (per-call epoch kept on the device), waits are bounded, peers are only written,
// never read. Replaces route_rdma / combine_rdma with their blocking exchanges and CPU packing
// (crates/rmlx-distributed/src/moe_exchange.rs:519-581, 1102-1195, 2288-2330).
#include "../common/ptx.cuh"
#include "../common/launch.cuh"

namespace rb {

constexpr int kEpMaxRanks = 8;
constexpr int kEpMaxExperts = 512;
constexpr int kEpThreads = 256;
constexpr uint32_t kEpStatusOverflow = 0x4f56464cu;   // 'OVFL'

// Layout of a rank's control block (uint32 words), identical on every rank.
//   [0] epoch  [1] exit ticket  [2] counts-arrived  [3] rows-arrived  [4] returns-arrived
//   [5] this rank's blocks counting themselves before the last one publishes an arrival
//   [8 .. 8+E)            cursors (per global expert, this rank's pairs placed so far)
//   [8+E .. 8+E+world*E)  table of everyone's counts, row = source rank
struct EpPeers {
  uint32_t* ctl[kEpMaxRanks];
  __nv_bfloat16* slab[kEpMaxRanks];     // [capacity_rows, D]
  uint32_t* meta[kEpMaxRanks];          // [capacity_rows]   (src rank << 24 | pair)
  __nv_bfloat16* ret[kEpMaxRanks];      // [max_pairs, D]
  int rank, world;
};

__device__ __forceinline__ void ep_fail(int* status, uint32_t code) {
  if (status) atomicExch(status, int(code));
}

// One warp copies a row of nvec 16-byte vectors with eight loads in flight per lane.
__device__ __forceinline__ void ep_copy_row(uint4* __restrict__ dst, const uint4* __restrict__ src,
                                            int nvec, int lane) {
  for (int i = lane; i < nvec; i += 256) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) if (i + u * 32 < nvec) v[u] = src[i + u * 32];
#pragma unroll
    for (int u = 0; u < 8; ++u) if (i + u * 32 < nvec) dst[i + u * 32] = v[u];
  }
}

// -------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kEpThreads)
ep_dispatch_kernel(EpPeers pp, const __nv_bfloat16* __restrict__ x, int x_stride,
                   const int* __restrict__ idx, const int* __restrict__ counts, int T, int top_k, int D,
                   int E, int capacity_rows, int* __restrict__ recv_offsets,
                   int* __restrict__ recv_rows, int* __restrict__ status) {
  __shared__ int s_myoff[kEpMaxExperts];     // where this rank's block of expert e starts (dest slab)
  __shared__ int s_table[kEpMaxRanks * kEpMaxExperts];   // everyone's counts, row = source rank
  __shared__ int s_total[kEpMaxExperts];     // pairs per expert over all ranks
  __shared__ int s_ok;
  const int rank = pp.rank, world = pp.world, e_local = E / world;
  uint32_t* ctl = pp.ctl[rank];
  const uint32_t e1 = ctl[0] + 1u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // 1. publish this rank's counts to everyone (block 0), then everyone waits for the full table
  if (blockIdx.x == 0) {
    for (int p = 0; p < world; ++p) {
      uint32_t* dst = pp.ctl[p] + 8 + E + rank * E;
      for (int e = threadIdx.x; e < E; e += blockDim.x) dst[e] = uint32_t(counts[e]);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      for (int p = 0; p < world; ++p) red_release_sys_add(pp.ctl[p] + 2, 1u);
    }
  }
  if (threadIdx.x == 0) {
    s_ok = wait_flag_ge(ctl + 2, e1 * uint32_t(world)) ? 1 : 0;
    if (!s_ok) ep_fail(status, kStatusPeerTimeout);
  }
  __syncthreads();
  bool ok = s_ok != 0;

  // 2. block starts. The table goes to shared memory in one coalesced pass (it is read many
  // times); then thread e handles global expert e.
  int* table = s_table;
  if (ok) {
    const volatile uint32_t* gt = ctl + 8 + E;
    for (int i = threadIdx.x; i < world * E; i += blockDim.x) s_table[i] = int(gt[i]);
  }
  __syncthreads();
  if (ok) {
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      int tot = 0;
      for (int s = 0; s < world; ++s) tot += table[s * E + e];
      s_total[e] = tot;
    }
  }
  __syncthreads();
  if (ok) {
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      const int first = (e / e_local) * e_local;
      int base = 0;
      for (int e2 = first; e2 < e; ++e2) base += s_total[e2];
      int before = 0;
      for (int s = 0; s < rank; ++s) before += table[s * E + e];
      s_myoff[e] = base + before;
    }
    // every rank sees the same table, so every rank takes the same decision on overflow
    if (threadIdx.x < world) {
      int total = 0;
      for (int e = threadIdx.x * e_local; e < (threadIdx.x + 1) * e_local; ++e) total += s_total[e];
      if (total > capacity_rows) { s_ok = 0; ep_fail(status, kEpStatusOverflow); }
    }
  }
  __syncthreads();
  ok = s_ok != 0;
  if (ok && blockIdx.x == 0) {
    // offsets of this rank's local experts for the grouped GEMM
    if (threadIdx.x <= e_local) {
      int acc = 0;
      for (int e = rank * e_local; e < rank * e_local + threadIdx.x; ++e) acc += s_total[e];
      recv_offsets[threadIdx.x] = acc;
      if (threadIdx.x == e_local && recv_rows) *recv_rows = acc;
    }
  }

  // 3. rows: a warp per (token, slot) pair
  if (ok) {
    uint32_t* cursors = ctl + 8;
    const int pairs = T * top_k;
    const int warps_total = gridDim.x * (kEpThreads / 32);
    for (int p = blockIdx.x * (kEpThreads / 32) + warp; p < pairs; p += warps_total) {
      int e = 0, pos = 0;
      if (lane == 0) {
        e = idx[p];
        // an expert id outside the table, or a row beyond the slab (ids that do not match the
        // counts), is reported and skipped: nothing is written through a bad index
        if (e < 0 || e >= E) {
          e = -1;
          ep_fail(status, kStatusBadArgument);
        } else {
          pos = s_myoff[e] + int(atomicAdd(cursors + e, 1u));
          if (pos < 0 || pos >= capacity_rows) { e = -1; ep_fail(status, kEpStatusOverflow); }
        }
      }
      e = __shfl_sync(0xffffffffu, e, 0);
      pos = __shfl_sync(0xffffffffu, pos, 0);
      if (e < 0) continue;
      const int dest = e / e_local;
      ep_copy_row(reinterpret_cast<uint4*>(pp.slab[dest] + size_t(pos) * D),
                  reinterpret_cast<const uint4*>(x + size_t(p / top_k) * x_stride), D / 8, lane);
      if (lane == 0) pp.meta[dest][pos] = (uint32_t(rank) << 24) | uint32_t(p);
    }
  }
  __syncthreads();

  // 4. tell everyone this block is done; wait until every block of every rank is
  if (threadIdx.x == 0) {
    // blocks count themselves locally; the last one publishes one arrival per peer
    __threadfence_system();
    if (atomicAdd(ctl + 5, 1u) == gridDim.x - 1) {
      ctl[5] = 0u;
      __threadfence_system();
      for (int p = 0; p < world; ++p) red_release_sys_add(pp.ctl[p] + 3, 1u);
    }
    if (!wait_flag_ge(ctl + 3, e1 * uint32_t(world))) ep_fail(status, kStatusPeerTimeout);
    // the last block to leave zeroes the cursors and advances the epoch
    __threadfence();
    if (atomicAdd(ctl + 1, 1u) == gridDim.x - 1) {
      for (int e = 0; e < E; ++e) ctl[8 + e] = 0u;
      ctl[1] = 0u;
      __threadfence();
      ctl[0] = e1;
    }
  }
}

// -------------------------------------------------------------------------------------------------
// The combine's counters live in a second control block (same layout, words 0..4 used) so that a
// dispatch and a combine never share an epoch.
__global__ void __launch_bounds__(kEpThreads)
ep_combine_kernel(EpPeers pp, uint32_t* __restrict__ ctl, const __nv_bfloat16* __restrict__ y,
                  const int* __restrict__ recv_rows, const float* __restrict__ wts,
                  const __nv_bfloat16* __restrict__ residual, int res_stride,
                  __nv_bfloat16* __restrict__ out, int out_stride, int T, int top_k, int D,
                  int* __restrict__ status) {
  __shared__ int s_ok;
  const int rank = pp.rank, world = pp.world;
  const uint32_t e1 = ctl[0] + 1u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps_total = gridDim.x * (kEpThreads / 32);
  const int gw = blockIdx.x * (kEpThreads / 32) + warp;

  // 1. expert outputs go home: row i of y belongs to (src, pair) = meta[i]
  const int rows = *recv_rows;
  for (int i = gw; i < rows; i += warps_total) {
    const uint32_t m = pp.meta[rank][i];
    const int src = int(m >> 24), pair = int(m & 0xffffffu);
    ep_copy_row(reinterpret_cast<uint4*>(pp.ret[src] + size_t(pair) * D),
                reinterpret_cast<const uint4*>(y + size_t(i) * D), D / 8, lane);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(ctl + 5, 1u) == gridDim.x - 1) {
      ctl[5] = 0u;
      __threadfence_system();
      // the remote control blocks sit at the same offset from each rank's base as the local one
      const size_t off = size_t(ctl - pp.ctl[rank]);
      for (int p = 0; p < world; ++p) red_release_sys_add(pp.ctl[p] + off + 4, 1u);
    }
    s_ok = wait_flag_ge(ctl + 4, e1 * uint32_t(world)) ? 1 : 0;
    if (!s_ok) ep_fail(status, kStatusPeerTimeout);
  }
  __syncthreads();

  // 2. weighted sum of the k returned rows of each local token (+ residual)
  if (s_ok) {
    const __nv_bfloat16* ret = pp.ret[rank];
    for (int t = gw; t < T; t += warps_total) {
      for (int c = lane; c < D / 8; c += 32) {
        float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (residual) {
          const uint4 rv = *reinterpret_cast<const uint4*>(residual + size_t(t) * res_stride + c * 8);
          f[0] = bf16lo(rv.x); f[1] = bf16hi(rv.x); f[2] = bf16lo(rv.y); f[3] = bf16hi(rv.y);
          f[4] = bf16lo(rv.z); f[5] = bf16hi(rv.z); f[6] = bf16lo(rv.w); f[7] = bf16hi(rv.w);
        }
        for (int s = 0; s < top_k; ++s) {
          const float w = wts[t * top_k + s];
          const uint4 v = __ldcg(reinterpret_cast<const uint4*>(ret + (size_t(t) * top_k + s) * D + c * 8));
          f[0] += w * bf16lo(v.x); f[1] += w * bf16hi(v.x); f[2] += w * bf16lo(v.y); f[3] += w * bf16hi(v.y);
          f[4] += w * bf16lo(v.z); f[5] += w * bf16hi(v.z); f[6] += w * bf16lo(v.w); f[7] += w * bf16hi(v.w);
        }
        uint4 o;
        o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]);
        o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
        *reinterpret_cast<uint4*>(out + size_t(t) * out_stride + c * 8) = o;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(ctl + 1, 1u) == gridDim.x - 1) { ctl[1] = 0u; __threadfence(); ctl[0] = e1; }
  }
}

}  // namespace rb

using namespace rb;

static int ep_fill(EpPeers* pp, void* const* ctl, void* const* slab, void* const* meta, void* const* ret,
                   int rank, int world) {
  if (world < 1 || world > kEpMaxRanks || rank < 0 || rank >= world) return -2;
  pp->rank = rank; pp->world = world;
  for (int p = 0; p < world; ++p) {
    pp->ctl[p] = static_cast<uint32_t*>(ctl[p]);
    pp->slab[p] = static_cast<__nv_bfloat16*>(slab[p]);
    pp->meta[p] = static_cast<uint32_t*>(meta[p]);
    pp->ret[p] = static_cast<__nv_bfloat16*>(ret[p]);
  }
  return 0;
}

// words a control block needs
extern "C" int rmlx_ep_ctl_words(int world, int E) { return 8 + E + world * E; }

// x [T, D] bf16; idx [T, k] int32 global expert ids; counts [E] int32 (pairs per expert, this rank).
// Outputs (device): recv_offsets [E/world + 1], recv_rows [1]. Rows land in slab[rank].
extern "C" int rmlx_ep_dispatch(void* const* ctl, void* const* slab, void* const* meta, void* const* ret,
                                int rank, int world, const void* x, int x_stride, const int* idx,
                                const int* counts, int T, int top_k, int D, int E, int capacity_rows,
                                int* recv_offsets, int* recv_rows, int blocks, int* status,
                                cudaStream_t st) {
  EpPeers pp;
  if (ep_fill(&pp, ctl, slab, meta, ret, rank, world)) return -2;
  if (E < world || E % world || E > kEpMaxExperts || D % 8 || x_stride % 8 || T < 0 || top_k < 1) return -2;
  if (size_t(T) * top_k >= (1u << 24)) return -2;
  if (blocks < 1) blocks = 32;
  return launch(ep_dispatch_kernel, dim3(blocks), dim3(kEpThreads), 0, st, false, pp,
                static_cast<const __nv_bfloat16*>(x), x_stride, idx, counts, T, top_k, D, E,
                capacity_rows, recv_offsets, recv_rows, status);
}

// y [rows, D] bf16 in slab order (the grouped GEMM's output); ctl2: this rank's combine control block
// (every rank passes the block at the same offset of its region). out [T, D] bf16.
extern "C" int rmlx_ep_combine(void* const* ctl, void* const* slab, void* const* meta, void* const* ret,
                               int rank, int world, void* ctl2, const void* y, const int* recv_rows,
                               const float* wts, const void* residual, int res_stride, void* out,
                               int out_stride, int T, int top_k, int D, int blocks, int* status,
                               cudaStream_t st) {
  EpPeers pp;
  if (ep_fill(&pp, ctl, slab, meta, ret, rank, world)) return -2;
  if (D % 8 || out_stride % 8 || (residual && res_stride % 8)) return -2;
  if (blocks < 1) blocks = 32;
  return launch(ep_combine_kernel, dim3(blocks), dim3(kEpThreads), 0, st, false, pp,
                static_cast<uint32_t*>(ctl2), static_cast<const __nv_bfloat16*>(y), recv_rows, wts,
                static_cast<const __nv_bfloat16*>(residual), res_stride,
                static_cast<__nv_bfloat16*>(out), out_stride, T, top_k, D, status);
}
