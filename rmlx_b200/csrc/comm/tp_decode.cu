// Tensor-parallel decode kernels that fuse the row-parallel projection with its all-reduce over
// NVLink peer memory: ONE launch computes the local partial product, pushes it into every rank's
// receive buffer with plain peer stores that carry their own arrival tag, and every block then
// collects its own rows from all ranks (bounded waits), sums the partials in rank order, adds the
// residual and writes the result. No host, no NCCL, no extra launch.
//
//   SgDenseTp             O projection (or dense down projection) + all-reduce + residual, on the
//   SgMoeDownTp           weight-streaming mat-vec (stream_gemv.cuh): expert down projection +
//                         routing-weighted combine + all-reduce + residual
//   gemv_allreduce        the same two on the per-row kernels (shapes the streaming kernel does
//   moe_down_allreduce    not take)
//   argmax_allreduce      vocabulary-parallel greedy sampling: local arg-max, 8-byte key exchange
//   allreduce_oneshot     stand-alone one-shot all-reduce of a small fp32 vector (+ residual)
//   barrier               epoch barrier on the peers' flag words
//
// This replaces the reference's host-driven split: command buffer -> CPU ring/tree all-reduce over
// RDMA -> next command buffer (crates/rmlx-nn/src/transformer.rs:4543-4597,
// crates/rmlx-distributed/src/group.rs:348-504, crates/rmlx-nn/src/parallel.rs:619-693).
//
// Receive-buffer protocol (per rank, in symmetric memory; every rank has the same layout):
//   recv[slot][src_rank][Bmax][N] 8-byte words (fp32 value, 32-bit tag). A value and its arrival
//   flag travel in one 8-byte store, so the exchange costs one NVLink crossing: no fence, no
//   counter, no reducer blocks. Tag and slot come from ONE device-side sequence number per
//   communicator, ctr[0] = all-reduces completed so far (every kind of call advances it: the last
//   block of a kernel to finish bumps it): tag = seq + 1, slot = seq & 1. Every call kind uses the
//   same layout of the receive area, so a word left by an earlier call can never carry the tag a
//   later call waits for. A rank can run at most one all-reduce ahead of a peer (finishing one
//   needs the peer's contribution to it), so two slots suffice, and because the slot is derived on
//   the device the alternation holds for any mix of captured and eager calls. All waits are
//   bounded; a wait that gives up sets a status word the host reads, and the kernel still
//   terminates.
//
// Remote data is only ever read with plain loads from this GPU's own memory (peers push); nothing
// here uses TMA on peer memory.
#include <cstring>
#include "../common/gemv_core.cuh"
#include "../common/launch.cuh"
#include "../kernels/stream_problems.cuh"

namespace rb {

constexpr int kMaxWorld = 8;
constexpr int kTpRowsPerWarp = 2;
constexpr int kTpRowsPerCta = kGemvWarps * kTpRowsPerWarp;  // 16

__device__ int g_tp_status = 0;

struct TpPeers {
  float* recv[kMaxWorld];        // each rank's receive area of 8-byte (value, tag) words (peer-mapped)
  uint32_t* ctr[kMaxWorld];      // each rank's counters: [0] all-reduces completed, [1] exit ticket of the running one
  int rank, world, bmax;         // bmax: batch rows the receive area is laid out for
};

// 8-byte (value, tag) words: a peer's store of such a word is a single transaction, so the tag is
// the arrival flag of its value and no fence or separate counter is needed (the low-latency
// protocol of collective libraries). Tags are the sequence number + 1; memory starts zeroed.
__device__ __forceinline__ void st_ll(uint2* p, float v, uint32_t tag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(tag) : "memory");
}
__device__ __forceinline__ bool ld_ll(const uint2* p, uint32_t tag, float& v) {
  for (uint32_t i = 0; i < kPeerPollLimit; ++i) {
    uint32_t a, b;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(a), "=r"(b) : "l"(p) : "memory");
    if (b == tag) { v = __uint_as_float(a); return true; }
    if (i > 256) __nanosleep(i > 8192 ? 128 : 20);
  }
  v = 0.f;
  return false;
}

// Exchange this block's partial values and finish its own rows.
//   vals: shared memory [B][kTpRowsPerCta] fp32 partial sums for rows n0 .. n0+15
//   recv layout per rank (8-byte words): slot_off + (src*bmax + b)*N + n
// Thread (b, i) stores its value, tagged, into every peer's receive area, then collects the same
// element from every peer out of its own receive area (all peers polled in one loop) and sums in
// rank order (so every rank gets bit-identical results), adds the residual and writes the output.
// Blocks never wait for other blocks: the same block index owns the same rows on every rank.
// ctr[0] is the communicator's sequence number, ctr[1] the exit ticket that advances it (both
// local).
// `b0` is the batch row of vals[0] (the expert kernel launches one token per grid row); the
// counters are read after the kernel's dependency wait, so they reflect every earlier all-reduce.
template <int B>
__device__ __forceinline__ void tp_push_reduce(const TpPeers& P, const float* vals, int n0, int N,
                                               int b0, const __nv_bfloat16* residual, int res_stride,
                                               __nv_bfloat16* out, int out_stride) {
  const int tid = threadIdx.x;
  uint32_t* ctr = P.ctr[P.rank];
  const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(ctr);
  const uint32_t tag = seq + 1u;
  const size_t slot_off = size_t(seq & 1u) * P.world * P.bmax * N;
  if (tid < B * kTpRowsPerCta) {
    const int b = tid / kTpRowsPerCta, i = tid % kTpRowsPerCta;
    if (n0 + i < N) {
      const float v = vals[tid];
      const size_t mine = slot_off + (size_t(P.rank) * P.bmax + b0 + b) * N + n0 + i;
      for (int pi = 1; pi < P.world; ++pi) {
        int p = P.rank + pi; if (p >= P.world) p -= P.world;
        st_ll(reinterpret_cast<uint2*>(P.recv[p]) + mine, v, tag);
      }
      const uint2* rb = reinterpret_cast<const uint2*>(P.recv[P.rank]) + slot_off;
      float s = 0.f;
      bool ok = true;
      // all peers' words are polled together: one NVLink latency, not world - 1
      float u[kMaxWorld];
      uint32_t pending = 0;
      for (int src = 0; src < P.world; ++src) { u[src] = v; if (src != P.rank) pending |= 1u << src; }
      for (uint32_t it = 0; pending && it < kPeerPollLimit; ++it) {
        for (int src = 0; src < P.world; ++src) {
          if (!((pending >> src) & 1u)) continue;
          uint32_t a, t2;
          asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(a), "=r"(t2)
                       : "l"(rb + (size_t(src) * P.bmax + b0 + b) * N + n0 + i) : "memory");
          if (t2 == tag) { u[src] = __uint_as_float(a); pending &= ~(1u << src); }
        }
        if (pending && it > 256) __nanosleep(it > 8192 ? 128 : 20);
      }
      if (pending) { ok = false; for (int src = 0; src < P.world; ++src) if ((pending >> src) & 1u) u[src] = 0.f; }
      for (int src = 0; src < P.world; ++src) s += u[src];
      if (!ok) atomicExch(&g_tp_status, kStatusPeerTimeout);
      if (residual) s += __bfloat162float(residual[size_t(b) * res_stride + n0 + i]);
      out[size_t(b) * out_stride + n0 + i] = __float2bfloat16_rn(s);
    }
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(ctr + 1, 1u) == gridDim.x * gridDim.y - 1) { ctr[1] = 0u; __threadfence(); *reinterpret_cast<volatile uint32_t*>(ctr) = tag; }
  }
}

// ------------------------------------------------------------------------------------------------
// out[b, n] = residual[b, n] + sum_ranks W_r[n, :] . x_r[b, :]      (x_r: this rank's K shard)
// ------------------------------------------------------------------------------------------------
template <class WT, int B>
__global__ void __launch_bounds__(kGemvThreads)
gemv_allreduce_kernel(Matrix<WT> W, const __nv_bfloat16* __restrict__ x, int x_stride,
                      const __nv_bfloat16* __restrict__ residual, int res_stride,
                      __nv_bfloat16* __restrict__ out, int out_stride, int N, TpPeers P) {
  extern __shared__ __align__(16) char smem[];
  __shared__ float vals[B * kTpRowsPerCta];
  const int K = W.K;
  const size_t bstride = (XStage<WT>::bytes(K) + 15) & ~size_t(15);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  using Row = typename Matrix<WT>::Row;
  const int n0 = blockIdx.x * kTpRowsPerCta;
  const int nw = n0 + warp * kTpRowsPerWarp;
  Row rows[kTpRowsPerWarp];
  Tile<Row, kTpRowsPerWarp> t0;
#pragma unroll
  for (int r = 0; r < kTpRowsPerWarp; ++r) rows[r] = W.row(min(nw + r, N - 1));
  load_tile<kTpRowsPerWarp>(rows, K, 0, t0);
  pdl_launch_dependents();   // let the next kernel start its weight prefetch now; its own wait covers our completion
  pdl_wait();
#pragma unroll
  for (int b = 0; b < B; ++b)
    XStage<WT>::stage(smem + b * bstride, x + size_t(b) * x_stride, nullptr, K, nullptr, false);
  __syncthreads();
  float acc[kTpRowsPerWarp][B];
#pragma unroll
  for (int r = 0; r < kTpRowsPerWarp; ++r)
#pragma unroll
    for (int b = 0; b < B; ++b) acc[r][b] = 0.f;
  warp_dot<kTpRowsPerWarp, B, Row>(rows, smem, bstride, K, acc, t0);
#pragma unroll
  for (int r = 0; r < kTpRowsPerWarp; ++r)
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const float v = warp_sum(acc[r][b]);
      if (lane == 0) vals[b * kTpRowsPerCta + warp * kTpRowsPerWarp + r] = v;
    }
  __syncthreads();
  tp_push_reduce<B>(P, vals, n0, N, 0, residual, res_stride, out, out_stride);
  pdl_launch_dependents();
}

// ------------------------------------------------------------------------------------------------
// MoE down + combine + all-reduce + residual for one token per grid.y.
// ------------------------------------------------------------------------------------------------
template <class WT>
struct ExpertMat;
template <>
struct ExpertMat<WBf16> {
  using Row = RowBf16;
  const __nv_bfloat16* w; int rows, K;
  __device__ Row row(int e, size_t n) const { return Row{w + (size_t(e) * rows + n) * size_t(K)}; }
};
template <>
struct ExpertMat<WQ4> {
  using Row = RowQ4;
  const uint32_t* w; const __nv_bfloat16* scales; const __nv_bfloat16* biases; int rows, K;
  __device__ Row row(int e, size_t n) const {
    const size_t r = size_t(e) * rows + n;
    return Row{w + r * size_t(K >> 3), scales + r * size_t(K >> 6), biases + r * size_t(K >> 6)};
  }
};

constexpr int kTpMaxTopK = 8;

// One token (B = 1) per launch row; the batch is the grid's y dimension. All rows share the
// communicator's sequence number (the last block of the whole grid bumps it).
template <class WT>
__global__ void __launch_bounds__(kGemvThreads)
moe_down_allreduce_kernel(ExpertMat<WT> W, const __nv_bfloat16* __restrict__ act, int act_stride,
                          const int* __restrict__ topk_idx, const float* __restrict__ topk_w,
                          const __nv_bfloat16* __restrict__ residual, int res_stride,
                          __nv_bfloat16* __restrict__ out, int out_stride, int N, int top_k,
                          int expert_base, int experts_local, TpPeers P) {
  extern __shared__ __align__(16) char smem[];
  __shared__ int s_e[kTpMaxTopK];
  __shared__ float s_w[kTpMaxTopK];
  __shared__ float vals[kTpRowsPerCta];
  const int I = W.K;
  const size_t bstride = (XStage<WT>::bytes(I) + 15) & ~size_t(15);
  const int b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  using Row = typename ExpertMat<WT>::Row;
  pdl_launch_dependents();   // let the next kernel start its weight prefetch now; its own wait covers our completion
  pdl_wait();
  if (threadIdx.x < top_k) {
    const int e = topk_idx[b * top_k + threadIdx.x] - expert_base;
    const bool local = e >= 0 && e < experts_local;
    s_e[threadIdx.x] = local ? e : -1;
    s_w[threadIdx.x] = local ? topk_w[b * top_k + threadIdx.x] : 0.f;
  }
  __syncthreads();
  for (int s = 0; s < top_k; ++s)
    if (s_e[s] >= 0)
      XStage<WT>::stage(smem + s * bstride, act + size_t(b * top_k + s) * act_stride, nullptr, I,
                        nullptr, false);
  __syncthreads();
  const int n0 = blockIdx.x * kTpRowsPerCta;
  const int nw = n0 + warp * kTpRowsPerWarp;
  float tot[kTpRowsPerWarp];
#pragma unroll
  for (int r = 0; r < kTpRowsPerWarp; ++r) tot[r] = 0.f;
  for (int s = 0; s < top_k; ++s) {
    const int e = s_e[s];
    if (e < 0) continue;
    Row rows[kTpRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kTpRowsPerWarp; ++r) rows[r] = W.row(e, min(nw + r, N - 1));
    float acc[kTpRowsPerWarp][1];
#pragma unroll
    for (int r = 0; r < kTpRowsPerWarp; ++r) acc[r][0] = 0.f;
    warp_dot<kTpRowsPerWarp, 1, Row>(rows, smem + s * bstride, 0, I, acc);
#pragma unroll
    for (int r = 0; r < kTpRowsPerWarp; ++r) tot[r] = fmaf(s_w[s], acc[r][0], tot[r]);
  }
#pragma unroll
  for (int r = 0; r < kTpRowsPerWarp; ++r) {
    const float v = warp_sum(tot[r]);
    if (lane == 0) vals[warp * kTpRowsPerWarp + r] = v;
  }
  __syncthreads();
  tp_push_reduce<1>(P, vals, n0, N, b, residual ? residual + size_t(b) * res_stride : nullptr, 0,
                    out + size_t(b) * out_stride, 0);
  pdl_launch_dependents();
}

// ------------------------------------------------------------------------------------------------
// Stand-alone one-shot all-reduce: out = residual + sum_ranks in_r  (fp32 in, bf16 or fp32 out).
// grid.x blocks each own a contiguous slice; the same push / count / wait protocol.
// ------------------------------------------------------------------------------------------------
template <bool OUT_F32>
__global__ void __launch_bounds__(256)
allreduce_oneshot_kernel(const float* __restrict__ in, const __nv_bfloat16* __restrict__ residual,
                         void* __restrict__ out, int n, TpPeers P, size_t slot_floats) {
  pdl_launch_dependents();   // let the next kernel start its weight prefetch now; its own wait covers our completion
  pdl_wait();
  uint32_t* ctr = P.ctr[P.rank];
  const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(ctr);
  const uint32_t tag = seq + 1u;
  const size_t slot_off = size_t(seq & 1u) * slot_floats;
  const int per = (n + gridDim.x - 1) / gridDim.x;
  const int lo = blockIdx.x * per, hi = min(n, lo + per);
  const uint2* rb = reinterpret_cast<const uint2*>(P.recv[P.rank]) + slot_off;
  // all stores first, so that a thread's several elements cross the link together
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = in[i];
    const size_t mine = slot_off + size_t(P.rank) * n + i;
    for (int pi = 1; pi < P.world; ++pi) {
      int p = P.rank + pi; if (p >= P.world) p -= P.world;
      st_ll(reinterpret_cast<uint2*>(P.recv[p]) + mine, v, tag);
    }
  }
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = in[i];
    float s = 0.f;
    bool ok = true;
    for (int src = 0; src < P.world; ++src) {
      float u = v;
      if (src != P.rank) ok = ld_ll(rb + size_t(src) * n + i, tag, u) && ok;
      s += u;
    }
    if (!ok) atomicExch(&g_tp_status, kStatusPeerTimeout);
    if (residual) s += __bfloat162float(residual[i]);
    if (OUT_F32) reinterpret_cast<float*>(out)[i] = s;
    else reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(s);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(ctr + 1, 1u) == gridDim.x - 1) { ctr[1] = 0u; __threadfence(); *reinterpret_cast<volatile uint32_t*>(ctr) = tag; }
  }
  pdl_launch_dependents();
}

// Vocabulary-parallel greedy sampling. Each rank has fp32 logits for its vocabulary slice; the
// winner key (order-preserving value bits, inverted global index) of every rank is pushed to all
// ranks and the maximum taken, so every rank ends with the same token. One block.
__global__ void __launch_bounds__(1024)
argmax_allreduce_kernel(const float* __restrict__ logits, int V_local, int stride, int vocab_base,
                        int B, int* __restrict__ out, unsigned long long* const* __restrict__ keys_peer,
                        TpPeers P, int slot) {
  // keys layout per rank: [slot][B][world] u64
  __shared__ float sv[32];
  __shared__ int si[32];
  pdl_launch_dependents();   // let the next kernel start its weight prefetch now; its own wait covers our completion
  pdl_wait();
  for (int b = 0; b < B; ++b) {
    const float* row = logits + size_t(b) * stride;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V_local; i += 1024) {
      const float v = row[i];
      if (v > best) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
      best = sv[threadIdx.x]; bi = si[threadIdx.x];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      uint32_t u = __float_as_uint(best);
      u ^= (u >> 31) ? 0xffffffffu : 0x80000000u;
      const unsigned long long key = (static_cast<unsigned long long>(u) << 32) |
                                     (0xffffffffu - static_cast<uint32_t>(bi + vocab_base));
      if (threadIdx.x < P.world)
        keys_peer[threadIdx.x][(size_t(slot) * B + b) * P.world + P.rank] = key;
    }
    __syncthreads();
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < P.world) red_release_sys_add(P.ctr[threadIdx.x] + slot * 2, 1u);
  uint32_t* ctr = P.ctr[P.rank] + slot * 2;
  if (threadIdx.x == 0) {
    if (!wait_flag_ge(ctr, uint32_t(P.world))) atomicExch(&g_tp_status, kStatusPeerTimeout);
  }
  __syncthreads();
  if (threadIdx.x < B) {
    const unsigned long long* k = keys_peer[P.rank] + (size_t(slot) * B + threadIdx.x) * P.world;
    unsigned long long m = 0ull;
    for (int r = 0; r < P.world; ++r) {
      const unsigned long long v = __ldcg(k + r);
      m = v > m ? v : m;
    }
    out[threadIdx.x] = static_cast<int>(0xffffffffu - static_cast<uint32_t>(m & 0xffffffffull));
  }
  __syncthreads();
  if (threadIdx.x == 0) { __threadfence(); ctr[0] = 0u; }
  pdl_launch_dependents();
}

// Epoch barrier: every rank adds 1 to every rank's word, then waits for world * epoch.
__global__ void barrier_kernel(TpPeers P, int word, uint32_t epoch) {
  if (threadIdx.x < P.world) {
    __threadfence_system();
    red_release_sys_add(P.ctr[threadIdx.x] + word, 1u);
  }
  if (threadIdx.x == 0) {
    if (!wait_flag_ge(P.ctr[P.rank] + word, uint32_t(P.world) * epoch))
      atomicExch(&g_tp_status, kStatusPeerTimeout);
  }
}


// ------------------------------------------------------------------------------------------------
// The same two fused kernels on the weight-streaming mat-vec. A finished quad (four consecutive
// output rows) is pushed at once, as two 16-byte stores of two (value, tag) words per rank, this
// rank's own receive area included; when the block has pushed all of its quads its consumer
// threads collect the block's rows from every rank, so the wait for the peers overlaps the rest of
// the block's own weight stream.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void st_ll2(uint2* p, float v0, float v1, uint32_t tag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(__float_as_uint(v0)),
               "r"(tag), "r"(__float_as_uint(v1)), "r"(tag) : "memory");
}

struct SgTpTail {
  TpPeers P;
  const __nv_bfloat16* residual; int res_stride;
  __nv_bfloat16* out; int out_stride;
  int N;                          // multiple of 4
  uint32_t tag; size_t slot_off;  // of the running all-reduce (begin())
  int q0, q1;                     // this block's quads

  __device__ __forceinline__ void begin() {
    const uint32_t seq = *reinterpret_cast<volatile uint32_t*>(P.ctr[P.rank]);
    tag = seq + 1u;
    slot_off = size_t(seq & 1u) * P.world * P.bmax * N;
  }
  // one lane per quad; v: the quad's four partial sums for B batch rows starting at row b0
  template <int B>
  __device__ __forceinline__ void push(int quad, const float (&v)[4][B], int b0) const {
    const int n = quad * 4;
    if (n >= N) return;
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const size_t idx = slot_off + (size_t(P.rank) * P.bmax + b0 + b) * N + n;
      for (int pi = 0; pi < P.world; ++pi) {
        int p = P.rank + pi; if (p >= P.world) p -= P.world;
        uint2* d = reinterpret_cast<uint2*>(P.recv[p]) + idx;
        st_ll2(d, v[0][b], v[1][b], tag);
        st_ll2(d + 2, v[2][b], v[3][b], tag);
      }
    }
  }
  // all consumer threads, once per block, after its last push
  template <int B>
  __device__ __forceinline__ void finish(int b0) const {
    const int r0 = q0 * 4, rows = max(min(q1 * 4, N) - r0, 0);
    const uint2* rb = reinterpret_cast<const uint2*>(P.recv[P.rank]) + slot_off;
    for (int e = threadIdx.x; e < rows * B; e += kSgConsumers) {
      const int b = e / rows, n = r0 + e - b * rows;
      float u[kMaxWorld];
      uint32_t pending = (1u << P.world) - 1u;
#pragma unroll
      for (int src = 0; src < kMaxWorld; ++src) u[src] = 0.f;
      for (uint32_t it = 0; pending && it < kPeerPollLimit; ++it) {
#pragma unroll
        for (int src = 0; src < kMaxWorld; ++src) {
          if (!((pending >> src) & 1u)) continue;
          uint32_t a, t2;
          asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(a), "=r"(t2)
                       : "l"(rb + (size_t(src) * P.bmax + b0 + b) * N + n) : "memory");
          if (t2 == tag) { u[src] = __uint_as_float(a); pending &= ~(1u << src); }
        }
        if (pending && it > 256) __nanosleep(it > 8192 ? 128 : 20);
      }
      if (pending) atomicExch(&g_tp_status, kStatusPeerTimeout);
      float s = 0.f;
#pragma unroll
      for (int src = 0; src < kMaxWorld; ++src) s += u[src];   // rank order: bit-identical on every rank
      if (residual) s += bf16lo(__ldcg(reinterpret_cast<const uint16_t*>(residual + size_t(b) * res_stride + n)));
      out[size_t(b) * out_stride + n] = __float2bfloat16_rn(s);
    }
    sg_consumer_sync();
    if (threadIdx.x == 0) {
      uint32_t* ctr = P.ctr[P.rank];
      __threadfence();
      if (atomicAdd(ctr + 1, 1u) == gridDim.x * gridDim.y - 1) { ctr[1] = 0u; __threadfence(); *reinterpret_cast<volatile uint32_t*>(ctr) = tag; }
    }
  }
};

template <int WK, int B>
struct SgDenseTp : SgDense<WK, B, false> {
  SgTpTail T;
  __device__ void cta_range(const SgPlan& pl, int& q0, int& q1) {
    SgDense<WK, B, false>::cta_range(pl, q0, q1);
    T.q0 = q0; T.q1 = q1;
  }
  __device__ void init(bool producer) { if (!producer) T.begin(); }
  __device__ void epilogue(int quad, float (&v)[4][B], SgSmem& sm) {
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const float inv = sm.c->misc[b];
#pragma unroll
      for (int r = 0; r < 4; ++r) v[r][b] *= inv;
    }
    T.template push<B>(quad, v, 0);
  }
  __device__ void cta_done(SgSmem&) { T.template finish<B>(0); }
};

// One token per grid partition (B = 1); `residual` / `out` of the tail point at the token's row.
template <int WK>
struct SgMoeDownTp : SgMoeDownBase<WK> {
  SgTpTail T;
  __device__ void cta_range(const SgPlan& pl, int& q0, int& q1) {
    SgMoeDownBase<WK>::cta_range(pl, q0, q1);
    T.q0 = q0; T.q1 = q1;
  }
  __device__ void init(bool producer) {
    this->load_routing();
    if (!producer) {
      T.begin();
      if (T.residual) T.residual += size_t(this->token) * T.res_stride;
      T.out += size_t(this->token) * T.out_stride;
    }
  }
  __device__ void stage_x(SgSmem& sm, const SgPlan&) { this->stage_moe_x(sm); }
  __device__ void epilogue(int quad, float (&v)[4][1], SgSmem&) { T.template push<1>(quad, v, this->token); }
  __device__ void cta_done(SgSmem&) { T.template finish<1>(this->token); }
};

static bool& tp_stream_on() { static bool v = true; return v; }
static long long& tp_stream_launches() { static long long v = 0; return v; }

static int* tp_status_ptr() {
  static int* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!cached[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_tp_status) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
    cached[dev] = static_cast<int*>(p);
  }
  return cached[dev];
}

static SgTpTail make_tail(const TpPeers& P, const void* residual, int res_stride, void* out,
                          int out_stride, int N) {
  SgTpTail T;
  T.P = P;
  T.residual = static_cast<const __nv_bfloat16*>(residual); T.res_stride = res_stride;
  T.out = static_cast<__nv_bfloat16*>(out); T.out_stride = out_stride;
  T.N = N; T.tag = 0u; T.slot_off = 0; T.q0 = T.q1 = 0;
  return T;
}

template <int WK, int B>
static int run_dense_tp(int kind_bits, const void* w, const void* sc, const void* bi, const void* x,
                        int x_stride, const SgTpTail& T, int N, int K, int pdl, cudaStream_t st) {
  SgDenseTp<WK, B> P;
  P.W = sg_weights(WK, w, sc, bi, K);
  P.N = N; P.K = K;
  P.x = static_cast<const __nv_bfloat16*>(x); P.x_stride = x_stride;
  P.norm_w = nullptr; P.eps = 0.f;
  P.residual = nullptr; P.res_stride = 0; P.out = nullptr; P.out_stride = 0;
  P.T = T;
  const SgPlan pl = sg_make_plan(kind_bits, P.W.units, 1, false, N / 4, sm_count(), 1 << 20,
                                 sg_x_bytes(WK, K, B), 0, B);
  return sg_launch(P, pl, pl.grid, tp_status_ptr(), pdl, st);
}

template <int WK>
static int run_moe_down_tp(int kind_bits, const void* w, const void* sc, const void* bi,
                           const void* act, int act_stride, const int* topk_idx,
                           const float* topk_w, const SgTpTail& T, int B, int top_k, int N, int I,
                           int expert_base, int experts_local, int pdl, cudaStream_t st) {
  SgMoeDownTp<WK> P;
  P.W = sg_weights(WK, w, sc, bi, I);
  P.N = N; P.I = I;
  P.act = static_cast<const __nv_bfloat16*>(act); P.act_stride = act_stride;
  P.R = SgRouting{topk_idx, topk_w, top_k, expert_base, experts_local};
  P.token = 0; P.ntok = B; P.nloc = 0; P.packed = 0ull;
  P.T = T;
  const int per_token = sm_count() / B > 0 ? sm_count() / B : 1;
  const SgPlan pl = sg_make_plan(kind_bits, P.W.units, top_k, false, N / 4, per_token, 1 << 20,
                                 sg_x_bytes(WK, top_k * I, 1), 64, 1);
  return sg_launch(P, pl, pl.grid * B, tp_status_ptr(), pdl, st);
}

template <class WT>
static Matrix<WT> mk_matrix(const void* w, const void* s, const void* b, int K);
template <>
Matrix<WBf16> mk_matrix<WBf16>(const void* w, const void*, const void*, int K) {
  return Matrix<WBf16>{static_cast<const __nv_bfloat16*>(w), K};
}
template <>
Matrix<WQ4> mk_matrix<WQ4>(const void* w, const void* s, const void* b, int K) {
  return Matrix<WQ4>{static_cast<const uint32_t*>(w), static_cast<const __nv_bfloat16*>(s),
                     static_cast<const __nv_bfloat16*>(b), K};
}

static TpPeers make_peers(void* const* recv, void* const* ctr, int rank, int world, int bmax = 1) {
  TpPeers P;
  for (int i = 0; i < kMaxWorld; ++i) {
    P.recv[i] = i < world ? static_cast<float*>(recv[i]) : nullptr;
    P.ctr[i] = i < world ? static_cast<uint32_t*>(ctr[i]) : nullptr;
  }
  P.rank = rank; P.world = world; P.bmax = bmax;
  return P;
}

}  // namespace rb

using namespace rb;

// The fused projections take the weight-streaming kernel when the shape fits (default), else the
// per-row kernels; off: always the per-row kernels.
extern "C" int rmlx_tp_set_stream(int on) { tp_stream_on() = on != 0; return 0; }
// Launches (captures included) of this process that took the weight-streaming form.
extern "C" long long rmlx_tp_stream_launches() { return tp_stream_launches(); }

extern "C" int rmlx_tp_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_tp_status, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_tp_status, &zero, sizeof(int));
  return v;
}

// recv / ctr: host arrays of `world` device pointers (peer-mapped bases, index = rank).
// bmax: batch rows the receive area is laid out for (2 slots x world x bmax x N words); the slot
// and the tag are derived on the device from the communicator's sequence number.
extern "C" int rmlx_tp_gemv_allreduce(int w_kind, const void* w, const void* scales,
                                      const void* biases, const void* x, int x_stride,
                                      const void* residual, int res_stride, void* out,
                                      int out_stride, int B, int N, int K, void* const* recv,
                                      void* const* ctr, int rank, int world, int bmax, int pdl,
                                      cudaStream_t st) {
  const int kind_bits = w_kind;      // bit 8: fp16 scales and biases (streaming kernel only)
  w_kind &= 0xff;
  if (K % 8 || (w_kind != 0 && K % 64) || B < 1 || B > 4 || B > bmax || N < 1 || world < 1 ||
      world > kMaxWorld)
    return -2;
  const TpPeers P = make_peers(recv, ctr, rank, world, bmax);
  // 8-bit weights and fp16 scales exist only in the streaming kernels
  const bool stream_only = w_kind == 2 || (kind_bits & 0x100);
  if ((tp_stream_on() || stream_only) && N % 4 == 0 && w_kind >= 0 && w_kind <= 2 &&
      sg_weights_ok(w_kind, w, scales, biases, K)) {
    const SgTpTail T = make_tail(P, residual, res_stride, out, out_stride, N);
    int rc = -2;
#define RB_TPS(KIND_)                                                                              \
    if (w_kind == KIND_) switch (B) {                                                                \
      case 1: rc = run_dense_tp<KIND_, 1>(kind_bits, w, scales, biases, x, x_stride, T, N, K, pdl, st); break; \
      case 2: rc = run_dense_tp<KIND_, 2>(kind_bits, w, scales, biases, x, x_stride, T, N, K, pdl, st); break; \
      case 3: rc = run_dense_tp<KIND_, 3>(kind_bits, w, scales, biases, x, x_stride, T, N, K, pdl, st); break; \
      default: rc = run_dense_tp<KIND_, 4>(kind_bits, w, scales, biases, x, x_stride, T, N, K, pdl, st); break; \
    }
    RB_TPS(0) RB_TPS(1) RB_TPS(2)
#undef RB_TPS
    if (rc != -2) { tp_stream_launches() += rc == 0; return rc; }
  }
  if (stream_only) return -2;
  const int grid = (N + kTpRowsPerCta - 1) / kTpRowsPerCta;
#define RB_TPG(WT, BB)                                                                            \
  {                                                                                               \
    const size_t smem = ((XStage<WT>::bytes(K) + 15) & ~size_t(15)) * BB;                         \
    auto kern = gemv_allreduce_kernel<WT, BB>;                                                    \
    RB_CHECK(set_max_smem(kern, smem));                                                           \
    return launch(kern, dim3(grid), dim3(kGemvThreads), smem, st, pdl != 0,                       \
                  mk_matrix<WT>(w, scales, biases, K), static_cast<const __nv_bfloat16*>(x),      \
                  x_stride, static_cast<const __nv_bfloat16*>(residual), res_stride,              \
                  static_cast<__nv_bfloat16*>(out), out_stride, N, P);                         \
  }
#define RB_TPG_B(WT)                                            \
  switch (B) {                                                  \
    case 1: RB_TPG(WT, 1) case 2: RB_TPG(WT, 2)                 \
    case 3: RB_TPG(WT, 3) default: RB_TPG(WT, 4)                \
  }
  if (w_kind == 0) { RB_TPG_B(WBf16) } else if (w_kind == 1) { RB_TPG_B(WQ4) }
#undef RB_TPG_B
#undef RB_TPG
  return -2;
}

extern "C" int rmlx_tp_moe_down_allreduce(int w_kind, const void* w, const void* scales,
                                          const void* biases, const void* act, int act_stride,
                                          const int* topk_idx, const float* topk_w,
                                          const void* residual, int res_stride, void* out,
                                          int out_stride, int B, int top_k, int N, int I,
                                          int expert_base, int experts_local, void* const* recv,
                                          void* const* ctr, int rank, int world, int bmax, int pdl,
                                          cudaStream_t st) {
  const int kind_bits = w_kind;      // bit 8: fp16 scales and biases (streaming kernel only)
  w_kind &= 0xff;
  if (I % 8 || (w_kind != 0 && I % 64) || B < 1 || B > bmax || top_k < 1 || top_k > kTpMaxTopK ||
      world < 1 || world > kMaxWorld)
    return -2;
  const TpPeers P = make_peers(recv, ctr, rank, world, bmax);
  const bool stream_only = w_kind == 2 || (kind_bits & 0x100);
  if ((tp_stream_on() || stream_only) && N % 4 == 0 && w_kind >= 0 && w_kind <= 2 && experts_local <= 256 &&
      sg_weights_ok(w_kind, w, scales, biases, I) && !(w_kind == 0 && I % 32)) {
    const SgTpTail T = make_tail(P, residual, res_stride, out, out_stride, N);
    int rc = -2;
#define RB_TPS(KIND_)                                                                              \
    if (w_kind == KIND_)                                                                           \
      rc = run_moe_down_tp<KIND_>(kind_bits, w, scales, biases, act, act_stride, topk_idx, topk_w, \
                                  T, B, top_k, N, I, expert_base, experts_local, pdl, st);
    RB_TPS(0) RB_TPS(1) RB_TPS(2)
#undef RB_TPS
    if (rc != -2) { tp_stream_launches() += rc == 0; return rc; }
  }
  if (stream_only) return -2;
  const int gx = (N + kTpRowsPerCta - 1) / kTpRowsPerCta;
#define RB_TPD(WT, MK)                                                                            \
  {                                                                                               \
    const size_t smem = ((XStage<WT>::bytes(I) + 15) & ~size_t(15)) * top_k;                      \
    auto kern = moe_down_allreduce_kernel<WT>;                                                    \
    RB_CHECK(set_max_smem(kern, smem));                                                           \
    return launch(kern, dim3(gx, B), dim3(kGemvThreads), smem, st, pdl != 0, MK,                  \
                  static_cast<const __nv_bfloat16*>(act), act_stride, topk_idx, topk_w,           \
                  static_cast<const __nv_bfloat16*>(residual), res_stride,                        \
                  static_cast<__nv_bfloat16*>(out), out_stride, N, top_k, expert_base,            \
                  experts_local, P);                                                              \
  }
  if (w_kind == 0)
    RB_TPD(WBf16, (ExpertMat<WBf16>{static_cast<const __nv_bfloat16*>(w), N, I}))
  if (w_kind == 1)
    RB_TPD(WQ4, (ExpertMat<WQ4>{static_cast<const uint32_t*>(w),
                                static_cast<const __nv_bfloat16*>(scales),
                                static_cast<const __nv_bfloat16*>(biases), N, I}))
#undef RB_TPD
  return -2;
}

// slot_floats: words of one slot of the receive area (world x bmax x N); n <= bmax x N.
extern "C" int rmlx_tp_allreduce(const float* in, const void* residual, void* out, int out_f32,
                                 int n, void* const* recv, void* const* ctr, int rank, int world,
                                 long long slot_floats, int pdl, cudaStream_t st) {
  if (n < 1 || world < 1 || world > kMaxWorld || 1LL * world * n > slot_floats) return -2;
  const TpPeers P = make_peers(recv, ctr, rank, world);
  int grid = (n + 2047) / 2048;
  if (grid > 32) grid = 32;
  if (out_f32)
    return launch(allreduce_oneshot_kernel<true>, dim3(grid), dim3(256), 0, st, pdl != 0, in,
                  static_cast<const __nv_bfloat16*>(residual), out, n, P, size_t(slot_floats));
  return launch(allreduce_oneshot_kernel<false>, dim3(grid), dim3(256), 0, st, pdl != 0, in,
                static_cast<const __nv_bfloat16*>(residual), out, n, P, size_t(slot_floats));
}

// keys_peer_dev: DEVICE array of `world` pointers to each rank's key area.
extern "C" int rmlx_tp_argmax(const float* logits, int V_local, int stride, int vocab_base, int B,
                              int* out, void* keys_peer_dev, void* const* recv, void* const* ctr,
                              int rank, int world, int slot, int pdl, cudaStream_t st) {
  if (B < 1 || B > 1024 || world < 1 || world > kMaxWorld) return -2;
  const TpPeers P = make_peers(recv, ctr, rank, world);
  return launch(argmax_allreduce_kernel, dim3(1), dim3(1024), 0, st, pdl != 0, logits, V_local,
                stride, vocab_base, B, out,
                static_cast<unsigned long long* const*>(keys_peer_dev), P, slot);
}

extern "C" int rmlx_tp_barrier(void* const* recv, void* const* ctr, int rank, int world, int word,
                               unsigned int epoch, cudaStream_t st) {
  const TpPeers P = make_peers(recv, ctr, rank, world);
  barrier_kernel<<<1, 32, 0, st>>>(P, word, epoch);
  return static_cast<int>(cudaGetLastError());
}

// ---- symmetric memory plumbing (CUDA IPC) --------------------------------------------------------
extern "C" int rmlx_symm_malloc(void** ptr, unsigned long long bytes) {
  RB_CHECK(cudaMalloc(ptr, bytes));
  return static_cast<int>(cudaMemset(*ptr, 0, bytes));
}
extern "C" int rmlx_symm_free(void* ptr) { return static_cast<int>(cudaFree(ptr)); }
extern "C" int rmlx_symm_get_handle(void* ptr, void* handle64) {
  cudaIpcMemHandle_t h;
  RB_CHECK(cudaIpcGetMemHandle(&h, ptr));
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
extern "C" int rmlx_symm_open_handle(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return static_cast<int>(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}
extern "C" int rmlx_symm_close_handle(void* ptr) { return static_cast<int>(cudaIpcCloseMemHandle(ptr)); }
