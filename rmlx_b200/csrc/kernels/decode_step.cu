// One decode step of a mixture-of-experts decoder as ONE persistent kernel (batch 1).
//
// Every SM runs one block for the whole token: a producer warp streams weights (and KV pages)
// through a shared-memory ring with bulk asynchronous copies, sixteen consumer warps multiply, and
// the phases of a layer are separated by grid-wide barriers instead of kernel boundaries:
//
//   A  RMSNorm + QKV projection + RoPE + paged K/V append            | barrier
//   B  paged flash decode: every block takes one (kv-head tile, KV split) and leaves a partial
//      (the KV pages come through the same ring as the weights)      | barrier
//   B2 merge of the split partials into the attention output         | barrier
//   C  O projection + residual                                       | barrier
//   D  router logits (RMSNorm folded in)                             | barrier
//   D2 softmax + top-k, computed redundantly in every block (no barrier)
//   E  routed experts' gate/up + SwiGLU                              | barrier
//   F  routed experts' down projection + weighted combine + residual | barrier
//
// and after the last layer the final RMSNorm + LM head. The producer runs ahead of the consumers
// across phase boundaries: while the blocks are in a latency-bound phase (attention, routing) the
// next projection's weights are already arriving, so HBM does not go idle at the boundaries the
// way it does between kernels. Weights that depend on the routing result (E, F) and pages that
// depend on this token's K/V (B) are gated by a block-local sequence word.
//
// Activations that cross blocks go through global memory and are read with L2 loads. The grid
// barrier is a monotonic counter (zeroed by the host before the launch) with a bounded spin; the
// kernel is launched cooperatively so all blocks are resident. An expired wait raises the block's
// abort flag: every later wait returns at once, the kernel finishes (with a wrong result) and the
// status word says so.
//
// This is the B200 form of the reference's single-command-buffer decode: its fused 7-dispatch
// layer and CachedDecode (crates/rmlx-nn/src/transformer.rs:2306-2555,3613-4050) remove host
// round trips between dispatches; here the dispatch boundaries themselves are gone.
#include <cooperative_groups.h>
#include "stream_problems.cuh"

namespace rb {

constexpr int kStPage = 16;
constexpr int kStFdWarps = 8;            // consumer warps that take a KV page per stage
constexpr int kStMaxExperts = 256;

struct StepLayer {
  SgWeights wqkv, wo, wgu, wdn;
  const __nv_bfloat16* norm1;
  const __nv_bfloat16* norm2;
  const __nv_bfloat16* router;           // [E, D] bf16
  const float* expert_bias;              // [E] or null
  __nv_bfloat16* k_cache;                // [blocks, Hkv, 16, HD]
  __nv_bfloat16* v_cache;
  int expert_base, experts_local;
  SgPlan p_qkv, p_o, p_router, p_gu, p_dn;
};

struct StepParams {
  const StepLayer* layers;
  int num_layers;
  int D, Hq, Hkv, HD, I, E, top_k, V;
  int q4;                                // weight kind of the projections: 0 bf16, 1 Q4, 2 Q8 (the router is bf16)
  float eps, scale_log2;
  int max_blocks, window, traditional;
  const int* tokens;                     // [1]
  const int* positions;                  // [1]
  const int* seq_lens;                   // [1] context length including this token
  const int* block_table;                // [1, max_blocks]
  const float* cos_t;
  const float* sin_t;
  const __nv_bfloat16* embed;            // [vocab, D]
  const __nv_bfloat16* final_norm;
  SgWeights lm_head;
  SgPlan p_lm;
  // activations (global, one token)
  __nv_bfloat16* h;                      // [D] residual stream between layers
  __nv_bfloat16* h2;                     // [D]
  __nv_bfloat16* q;                      // [Hq, HD]
  __nv_bfloat16* attn;                   // [Hq, HD]
  __nv_bfloat16* act;                    // [top_k, I]
  float* router_logits;                  // [E]
  int* topk_idx;                         // [top_k] (written by block 0, for inspection)
  float* topk_w;
  float* fd_part_o;                      // [tiles, S, 16, HD]
  float* fd_part_ml;                     // [tiles, S, 16, 2]
  float* logits;                         // [V] fp32
  unsigned int* grid_bar;                // zero on entry
  unsigned long long* trace;             // optional: block 0 stamps the global timer at phase ends [layers][32]
  int* status;
  // shared-memory layout
  int ns, slot_bytes, x_bytes, part_floats, extra_bytes;
};

static __device__ int g_step_status = 0;

struct StepSmem {
  SgSmem sm;
  float* fdbuf;                          // attention phase: the Q tile, then the merge buffer
};

__host__ __device__ inline int step_fdbuf_bytes(int HD) {
  // merge buffer [4 page slots][2 halves][32 lanes][NT/2 * 4 + 4] floats; the Q tile (16 padded rows) fits in it
  return 4 * 2 * 32 * (HD / 16 * 4 + 4) * 4;
}

__device__ __forceinline__ StepSmem step_carve(char* smem, const StepParams& p) {
  StepSmem t;
  char* base = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem) + 127) & ~uintptr_t(127));
  SgSmem& s = t.sm;
  s.c = reinterpret_cast<SgCtl*>(base);
  s.ring = base + sg_ctl_bytes();
  s.xs = s.ring + size_t(p.ns) * p.slot_bytes;
  s.part = reinterpret_cast<float*>(s.xs + p.x_bytes);
  s.extra = reinterpret_cast<char*>(s.part + p.part_floats);
  t.fdbuf = reinterpret_cast<float*>(s.extra + p.extra_bytes);
  return t;
}

__host__ inline size_t step_smem_bytes(const StepParams& p, int HD) {
  return size_t(sg_ctl_bytes()) + size_t(p.ns) * p.slot_bytes + p.x_bytes + size_t(p.part_floats) * 4 +
         p.extra_bytes + step_fdbuf_bytes(HD) + 256;
}

__device__ __forceinline__ void step_stamp(const StepParams& p, int layer, int k) {
  if (p.trace && blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned long long tm;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tm));
    p.trace[layer * 32 + k] = tm;
  }
}

// ---- grid barrier: monotonic counter, bounded spin, consumer warps only ------------------------
__device__ __forceinline__ void step_grid_sync(const StepParams& p, StepSmem& t, unsigned int& target) {
  target += gridDim.x;
  sg_consumer_sync();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(p.grid_bar, 1u);
    if (!*t.sm.c->abortf) {
      bool ok = false;
      for (uint32_t i = 0; i < kPeerPollLimit; ++i) {
        if (static_cast<int32_t>(ld_acquire_sys(p.grid_bar) - target) >= 0) { ok = true; break; }
        if (i > 32) __nanosleep(i > 4096 ? 128 : 20);
      }
      if (!ok) { *t.sm.c->abortf = 1u; atomicCAS(const_cast<uint32_t*>(t.sm.c->abortf) + 1, 0u, target & 0xffffu | 0x50000u); }
    }
    __threadfence();
  }
  sg_consumer_sync();
}

// consumers -> producer: one more gated event has happened
__device__ __forceinline__ void step_signal(StepSmem& t) {
  if (threadIdx.x == 0) {
    asm volatile("fence.proxy.async;" ::: "memory");   // our generic writes before the producer's bulk reads
    __threadfence_block();
    t.sm.c->go = t.sm.c->go + 1u;
  }
}
__device__ __forceinline__ bool step_wait_go(StepSmem& t, uint32_t want) {
  // the longest budget of all: when something upstream is stuck, that wait should be the one that reports
  for (uint32_t i = 0; i < (kPeerPollLimit << 4); ++i) {
    if (t.sm.c->go >= want) { __threadfence_block(); return true; }
    if (*t.sm.c->abortf) return false;
    if (i > 16) __nanosleep(40);
  }
  *t.sm.c->abortf = 1u;
  atomicCAS(const_cast<uint32_t*>(t.sm.c->abortf) + 1, 0u, want | 0x40000u);
  return false;
}

// ---- attention phase ------------------------------------------------------------------------------
struct FdSplit { int tile, split, S, kvh, gt, pg0, pg1, len, first; bool on; };

__device__ __forceinline__ FdSplit step_fd_split(const StepParams& p) {
  FdSplit f;
  const int G = p.Hq / p.Hkv, gtiles = (G + 15) / 16, tiles = p.Hkv * gtiles;
  f.S = int(gridDim.x) / tiles;
  f.tile = int(blockIdx.x) % tiles;
  f.split = int(blockIdx.x) / tiles;
  f.on = f.S > 0 && f.split < f.S;
  f.kvh = f.tile / gtiles; f.gt = f.tile % gtiles;
  f.len = __ldcg(p.seq_lens);
  f.first = (p.window > 0 && f.len > p.window) ? f.len - p.window : 0;
  const int pg_begin = f.first / kStPage;
  const int pg_total = (f.len + kStPage - 1) / kStPage - pg_begin;
  const int per = f.S > 0 ? (pg_total + f.S - 1) / f.S : 0;
  f.pg0 = pg_begin + f.split * per;
  f.pg1 = min(f.pg0 + per, pg_begin + pg_total);
  if (!f.on) { f.pg0 = f.pg1 = 0; }
  return f;
}

// Producer: the split's pages, eight (K, V) pairs per ring slot, 16 lanes issue one page each.
__device__ __forceinline__ bool step_fd_produce(const StepParams& p, const StepLayer& L, StepSmem& t,
                                                SgRingPos& rp, const FdSplit& f) {
  const int lane = threadIdx.x & 31;
  const uint32_t page_bytes = uint32_t(kStPage) * p.HD * 2;
  for (int pg = f.pg0; pg < f.pg1; pg += kStFdWarps) {
    const int s = rp.s;
    if (rp.round > 0 && !sg_wait(t.sm.c->empty + s, (rp.round - 1) & 1, t.sm.c->abortf, 0x71)) return false;
    char* stage = t.sm.ring + size_t(s) * rp.slot_bytes;
    uint32_t bytes = 0;
    const int j = lane >> 1, kv = lane & 1;
    if (lane < 2 * kStFdWarps && pg + j < f.pg1) {
      const int blk = RB_BOUNDS(pg + j, p.max_blocks) ? __ldcg(p.block_table + pg + j) : 0;   // page 0 is reserved
      const char* src = reinterpret_cast<const char*>(kv ? L.v_cache : L.k_cache) +
                        (size_t(blk) * p.Hkv + f.kvh) * page_bytes;
      bulk_g2s(stage + (size_t(j) * 2 + kv) * page_bytes, src, page_bytes, t.sm.c->full + s);
      bytes = page_bytes;
    }
    bytes = __reduce_add_sync(0xffffffffu, bytes);
    if (lane == 0) mbar_arrive_expect_tx(t.sm.c->full + s, bytes);
    if (++rp.s == rp.ns) { rp.s = 0; ++rp.round; }
  }
  return true;
}

__device__ __forceinline__ void st_ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void st_ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void st_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
      "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Consumers: a KV page of a stage is shared by two warps; both form the 16 x 16 score tile, each
// accumulates one half of the head dimension (a warp's state then fits the kernel's 96 registers;
// the query tile stays in shared memory and is re-read per k-step). After the split's pages the
// eight page slots are merged pairwise through a small buffer and slot 0's warps write the split's
// partial. The pages sit in the ring unswizzled (bulk copies): the ldmatrix bank conflicts are
// accepted, a warp handles one or two pages per step.
template <int HD>
__device__ __forceinline__ void step_fd_consume(const StepParams& p, StepSmem& t, SgRingPos& rp,
                                                const FdSplit& f) {
  constexpr int KS = HD / 16, NTH = HD / 16;          // k-steps; n-tiles of this warp's half
  constexpr int PAGE_BYTES = kStPage * HD * 2;
  constexpr int QROW = HD * 2 + 16;                   // padded row of the Q tile (conflict-free ldmatrix)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int slot = warp >> 1, half = warp & 1;        // page slot of a stage, half of the head dimension
  const int G = p.Hq / p.Hkv;
  // ---- Q tile -> shared memory (rows beyond the group are zero)
  char* qs = reinterpret_cast<char*>(t.fdbuf);
  for (int i = threadIdx.x; i < 16 * (HD / 8); i += kSgConsumers) {
    const int row = i / (HD / 8), c = i - row * (HD / 8);
    const int h = f.gt * 16 + row;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (f.on && h < G) v = __ldcg(reinterpret_cast<const uint4*>(p.q + (size_t(f.kvh) * G + h) * HD) + c);
    *reinterpret_cast<uint4*>(qs + row * QROW + c * 16) = v;
  }
  sg_consumer_sync();
  float o[NTH][4];
#pragma unroll
  for (int j = 0; j < NTH; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const uint32_t qbase = smem_u32(qs) + (lane & 15) * QROW + (lane >> 4) * 16;
  for (int pg = f.pg0; pg < f.pg1; pg += kStFdWarps) {
    const int s = rp.s;
    const bool ok = sg_wait(t.sm.c->full + s, rp.round & 1u, t.sm.c->abortf, 0x72);
    const int mypg = pg + slot;
    if (ok && mypg < f.pg1) {
      const uint32_t kbase = smem_u32(t.sm.ring + size_t(s) * rp.slot_bytes + size_t(slot) * 2 * PAGE_BYTES);
      const uint32_t vbase = kbase + PAGE_BYTES;
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const int mi = lane >> 3, r = lane & 7;
        const int tok = (mi >> 1) * 8 + r, c = 2 * ks + (mi & 1);
        uint32_t qa[4], kb[4];
        st_ldmatrix_x4(qa, qbase + ks * 32);
        st_ldmatrix_x4(kb, kbase + tok * (HD * 2) + (c << 4));
        st_mma(s0, qa, kb[0], kb[1]);
        st_mma(s1, qa, kb[2], kb[3]);
      }
      const int tok0 = mypg * kStPage + tq * 2;
      float sv[8] = {s0[0], s0[1], s1[0], s1[1], s0[2], s0[3], s1[2], s1[3]};
      const int tk[4] = {tok0, tok0 + 1, tok0 + 8, tok0 + 9};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const bool in = tk[i] < f.len && tk[i] >= f.first;
        sv[i] = in ? sv[i] * p.scale_log2 : -INFINITY;
        sv[4 + i] = in ? sv[4 + i] * p.scale_log2 : -INFINITY;
      }
      float mx0 = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
      float mx1 = fmaxf(fmaxf(sv[4], sv[5]), fmaxf(sv[6], sv[7]));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float nm0 = fmaxf(m0, mx0), nm1 = fmaxf(m1, mx1);
      const float c0 = exp2f(m0 - nm0), c1 = exp2f(m1 - nm1);   // a page holds a visible token: nm finite
      m0 = nm0; m1 = nm1;
      float pr[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) { pr[i] = exp2f(sv[i] - m0); pr[4 + i] = exp2f(sv[4 + i] - m1); }
      l0 = l0 * c0 + (pr[0] + pr[1] + pr[2] + pr[3]);
      l1 = l1 * c1 + (pr[4] + pr[5] + pr[6] + pr[7]);
      uint32_t pa[4] = {pack_bf16(pr[0], pr[1]), pack_bf16(pr[4], pr[5]), pack_bf16(pr[2], pr[3]),
                        pack_bf16(pr[6], pr[7])};
#pragma unroll
      for (int j = 0; j < NTH; ++j) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
#pragma unroll
      for (int j = 0; j < NTH; j += 2) {
        const int mi = lane >> 3, r = lane & 7;
        const int tok = (mi & 1) * 8 + r, c = half * NTH + j + (mi >> 1);
        uint32_t vb[4];
        st_ldmatrix_x4_trans(vb, vbase + tok * (HD * 2) + (c << 4));
        st_mma(o[j], pa, vb[0], vb[1]);
        st_mma(o[j + 1], pa, vb[2], vb[3]);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(t.sm.c->empty + s);
    if (++rp.s == rp.ns) { rp.s = 0; ++rp.round; }
  }
  // quad totals of the row sums (the four lanes of a quad hold different key columns)
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  // ---- pairwise merge of the page slots: (4..7 -> 0..3), (2,3 -> 0,1), (1 -> 0); the Q tile is no
  //      longer needed, its memory is the merge buffer
  constexpr int LSTRIDE = NTH * 4 + 4;                // floats per lane in the buffer
  sg_consumer_sync();
  for (int stride = kStFdWarps / 2; stride >= 1; stride >>= 1) {
    if (slot >= stride && slot < 2 * stride) {
      float* b = t.fdbuf + ((size_t(slot - stride) * 2 + half) * 32 + lane) * LSTRIDE;
#pragma unroll
      for (int j = 0; j < NTH; ++j) *reinterpret_cast<float4*>(b + j * 4) = make_float4(o[j][0], o[j][1], o[j][2], o[j][3]);
      *reinterpret_cast<float4*>(b + NTH * 4) = make_float4(m0, m1, l0, l1);
    }
    sg_consumer_sync();
    if (slot < stride) {
      const float* b = t.fdbuf + ((size_t(slot) * 2 + half) * 32 + lane) * LSTRIDE;
      const float4 ml = *reinterpret_cast<const float4*>(b + NTH * 4);
      const float nm0 = fmaxf(m0, ml.x), nm1 = fmaxf(m1, ml.y);
      const float a0 = m0 == -INFINITY ? 0.f : exp2f(m0 - nm0), a1 = m1 == -INFINITY ? 0.f : exp2f(m1 - nm1);
      const float b0 = ml.x == -INFINITY ? 0.f : exp2f(ml.x - nm0), b1 = ml.y == -INFINITY ? 0.f : exp2f(ml.y - nm1);
      m0 = nm0; m1 = nm1;
      l0 = l0 * a0 + ml.z * b0; l1 = l1 * a1 + ml.w * b1;
#pragma unroll
      for (int j = 0; j < NTH; ++j) {
        const float4 v = *reinterpret_cast<const float4*>(b + j * 4);
        o[j][0] = o[j][0] * a0 + v.x * b0; o[j][1] = o[j][1] * a0 + v.y * b0;
        o[j][2] = o[j][2] * a1 + v.z * b1; o[j][3] = o[j][3] * a1 + v.w * b1;
      }
    }
    sg_consumer_sync();
  }
  if (slot == 0 && f.on) {
    float* po = p.fd_part_o + (size_t(f.tile) * f.S + f.split) * 16 * HD;
    float* pm = p.fd_part_ml + (size_t(f.tile) * f.S + f.split) * 32;
#pragma unroll
    for (int j = 0; j < NTH; ++j) {
      const int d = (half * NTH + j) * 8 + tq * 2;
      *reinterpret_cast<float2*>(po + g * HD + d) = make_float2(o[j][0], o[j][1]);
      *reinterpret_cast<float2*>(po + (g + 8) * HD + d) = make_float2(o[j][2], o[j][3]);
    }
    if (half == 0 && tq == 0) { pm[g * 2] = m0; pm[g * 2 + 1] = l0; pm[(g + 8) * 2] = m1; pm[(g + 8) * 2 + 1] = l1; }
  }
}

// Merge of the split partials: block c takes query heads c, c + grid, ...
__device__ __forceinline__ void step_fd_merge(const StepParams& p, StepSmem& t) {
  const int G = p.Hq / p.Hkv, gtiles = (G + 15) / 16, tiles = p.Hkv * gtiles, S = int(gridDim.x) / tiles;
  float* wgt = t.fdbuf;                              // [S] weights, then [1] 1/L
  const int tid = threadIdx.x;
  for (int h = blockIdx.x; h < p.Hq; h += gridDim.x) {
    const int kvh = h / G, hr = h - kvh * G, gt = hr / 16, row = hr - gt * 16;
    const int tile = kvh * gtiles + gt;
    const float* ml = p.fd_part_ml + size_t(tile) * S * 32;
    if (tid < 32) {
      float M = -INFINITY;
      for (int s = tid; s < S; s += 32) M = fmaxf(M, __ldcg(ml + s * 32 + row * 2));
      M = warp_max(M);
      float L = 0.f;
      for (int s = tid; s < S; s += 32) {
        const float ms = __ldcg(ml + s * 32 + row * 2);
        const float w = ms == -INFINITY ? 0.f : exp2f(ms - M);
        wgt[s] = w;
        L += __ldcg(ml + s * 32 + row * 2 + 1) * w;
      }
      L = warp_sum(L);
      if (tid == 0) wgt[S] = L > 0.f ? 1.f / L : 0.f;
    }
    sg_consumer_sync();
    if (tid < p.HD) {
      const float* po = p.fd_part_o + (size_t(tile) * S * 16 + row) * p.HD + tid;
      float acc = 0.f;
      for (int s = 0; s < S; ++s) acc = fmaf(__ldcg(po + size_t(s) * 16 * p.HD), wgt[s], acc);
      p.attn[size_t(h) * p.HD + tid] = __float2bfloat16_rn(acc * wgt[S]);
    }
    sg_consumer_sync();
  }
}

// Softmax over E router logits + top-k + renormalise, one warp; ties go to the lowest index
// (same selection as moe_topk_route, crates/rmlx-core/src/ops/topk_route.rs:212).
__device__ __forceinline__ void step_topk(const StepParams& p, const StepLayer& L, StepSmem& t) {
  const int lane = threadIdx.x & 31;
  float v[kStMaxExperts / 32];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < kStMaxExperts / 32; ++i) {
    const int e = i * 32 + lane;
    v[i] = e < p.E ? __ldcg(p.router_logits + e) + (L.expert_bias ? L.expert_bias[e] : 0.f) : -INFINITY;
    m = fmaxf(m, v[i]);
  }
  m = warp_max(m);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kStMaxExperts / 32; ++i) {
    v[i] = (i * 32 + lane < p.E) ? __expf(v[i] - m) : -1.f;
    s += fmaxf(v[i], 0.f);
  }
  s = warp_sum(s);
  const float inv = 1.f / s;
  float sel_w = 0.f, wsum = 0.f;
  int sel_e = 0;
  for (int r = 0; r < p.top_k; ++r) {
    float best = -2.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kStMaxExperts / 32; ++i)
      if (v[i] > best) { best = v[i]; best_e = i * 32 + lane; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
#pragma unroll
    for (int i = 0; i < kStMaxExperts / 32; ++i)
      if (i * 32 + lane == best_e) v[i] = -1.f;
    const float pw = best * inv;
    wsum += pw;
    if (lane == r) { sel_w = pw; sel_e = best_e; }
  }
  if (lane < p.top_k) {
    t.sm.c->r_idx[lane] = sel_e;
    t.sm.c->r_w[lane] = sel_w / wsum;
    if (blockIdx.x == 0) { p.topk_idx[lane] = sel_e; p.topk_w[lane] = sel_w / wsum; }
  }
}

// Runs one streaming problem's consumer side (activations staged first) with the lane width its
// plan chose.
template <class P>
__device__ __forceinline__ void step_consume(const StepParams& p, int layer, P& prob, const SgPlan& pl, StepSmem& t, SgRingPos& rp, uint32_t tag) {
  rp.tag = tag;
  int q0, q1;
  prob.cta_range(pl, q0, q1);
  prob.init(false);
  prob.stage_x(t.sm, pl);
  step_stamp(p, layer, 16 + int(tag));
  if (pl.LW == 32) sg_consume<P, 32>(prob, pl, t.sm, rp, q0, q1);
  else if (pl.LW == 16) sg_consume<P, 16>(prob, pl, t.sm, rp, q0, q1);
  else sg_consume<P, 8>(prob, pl, t.sm, rp, q0, q1);
}
template <class P>
__device__ __forceinline__ bool step_produce(P& prob, const SgPlan& pl, StepSmem& t, SgRingPos& rp, uint32_t tag) {
  rp.tag = tag;
  int q0, q1;
  prob.cta_range(pl, q0, q1);
  prob.init(true);
  if (pl.LW == 32) return sg_produce<P, 32>(prob, pl, t.sm, rp, q0, q1);
  if (pl.LW == 16) return sg_produce<P, 16>(prob, pl, t.sm, rp, q0, q1);
  return sg_produce<P, 8>(prob, pl, t.sm, rp, q0, q1);
}

template <int WK>
struct StepProblems {
  using Qkv = SgQkvRope<WK, 1>;
  using Oproj = SgDense<WK, 1, false>;
  using Router = SgDense<0, 1, true>;
  using GateUp = SgMoeGateUp<WK>;
  using Down = SgMoeDown<WK, false>;
  using LmHead = SgDense<WK, 1, true>;

  static __device__ Qkv qkv(const StepParams& p, const StepLayer& L, const __nv_bfloat16* x) {
    Qkv P;
    P.W = L.wqkv; P.K = p.D; P.x = x; P.x_stride = 0; P.norm_w = L.norm1; P.eps = p.eps;
    P.a = SgRopeArgs{p.q, L.k_cache, L.v_cache, p.block_table, p.positions, nullptr, p.cos_t, p.sin_t,
                     p.Hq, p.Hkv, p.HD, p.max_blocks, kStPage, p.traditional};
    return P;
  }
  static __device__ Oproj oproj(const StepParams& p, const StepLayer& L, const __nv_bfloat16* res) {
    Oproj P;
    P.W = L.wo; P.N = p.D; P.K = p.Hq * p.HD; P.x = p.attn; P.x_stride = 0; P.norm_w = nullptr; P.eps = p.eps;
    P.residual = res; P.res_stride = 0; P.out = p.h2; P.out_stride = 0;
    return P;
  }
  static __device__ Router router(const StepParams& p, const StepLayer& L) {
    Router P;
    P.W = SgWeights{reinterpret_cast<const char*>(L.router), nullptr, nullptr, p.D >> 3, 0};
    P.N = p.E; P.K = p.D; P.x = p.h2; P.x_stride = 0; P.norm_w = L.norm2; P.eps = p.eps;
    P.residual = nullptr; P.res_stride = 0; P.out = p.router_logits; P.out_stride = 0;
    return P;
  }
  static __device__ GateUp gate_up(const StepParams& p, const StepLayer& L, const StepSmem& t) {
    GateUp P;
    P.W = L.wgu; P.I = p.I; P.K = p.D; P.x = p.h2; P.x_stride = 0; P.norm_w = L.norm2; P.eps = p.eps;
    P.act = p.act; P.act_stride = p.I;
    P.R = SgRouting{t.sm.c->r_idx, t.sm.c->r_w, p.top_k, L.expert_base, L.experts_local};
    P.token = 0; P.ntok = 1; P.packed = 0; P.mask = 0;
    return P;
  }
  static __device__ Down down(const StepParams& p, const StepLayer& L, const StepSmem& t) {
    Down P;
    P.W = L.wdn; P.N = p.D; P.I = p.I; P.act = p.act; P.act_stride = p.I;
    P.R = SgRouting{t.sm.c->r_idx, t.sm.c->r_w, p.top_k, L.expert_base, L.experts_local};
    P.token = 0; P.ntok = 1; P.nloc = 0; P.packed = 0;
    P.residual = p.h2; P.res_stride = 0; P.out = p.h; P.out_stride = 0;
    return P;
  }
  static __device__ LmHead lm_head(const StepParams& p) {
    LmHead P;
    P.W = p.lm_head; P.N = p.V; P.K = p.D; P.x = p.h; P.x_stride = 0; P.norm_w = p.final_norm; P.eps = p.eps;
    P.residual = nullptr; P.res_stride = 0; P.out = p.logits; P.out_stride = 0;
    return P;
  }
};

template <int WK, int HD>
__global__ void __launch_bounds__(kSgThreads, 1) decode_step_kernel(StepParams p) {
  extern __shared__ char smem_raw[];
  using SP = StepProblems<WK>;
  StepSmem t = step_carve(smem_raw, p);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.ns; ++s) {
      mbar_init(t.sm.c->full + s, 1);
      mbar_init(t.sm.c->empty + s, kSgConsumerWarps);
    }
    sg_init_handover(t.sm, p.ns);
    t.sm.c->abortf[0] = 0u; t.sm.c->abortf[1] = 0u;
    t.sm.c->go = 0u;
    fence_mbar_init();
  }
  __syncthreads();
  SgRingPos rp{0, 0u, 0u, p.ns, p.slot_bytes, 0u};
  const __nv_bfloat16* x0 = p.embed + size_t(__ldcg(p.tokens)) * p.D;

  if (warp == kSgConsumerWarps) {
    // ------------------------------------------------------------------ producer warp
    bool ok = true;
    uint32_t gate = 0;
    for (int l = 0; l < p.num_layers && ok; ++l) {
      const StepLayer& L = p.layers[l];
      { auto P = SP::qkv(p, L, l == 0 ? x0 : p.h); ok = step_produce(P, L.p_qkv, t, rp, 1); }
      ok = ok && step_wait_go(t, ++gate);            // this token's K/V are in their pages
      if (ok) { const FdSplit f = step_fd_split(p); ok = step_fd_produce(p, L, t, rp, f); }
      if (ok) { auto P = SP::oproj(p, L, nullptr); ok = step_produce(P, L.p_o, t, rp, 2); }
      if (ok) { auto P = SP::router(p, L); ok = step_produce(P, L.p_router, t, rp, 3); }
      ok = ok && step_wait_go(t, ++gate);            // the routing result is in shared memory
      if (ok) { auto P = SP::gate_up(p, L, t); ok = step_produce(P, L.p_gu, t, rp, 4); }
      if (ok) { auto P = SP::down(p, L, t); ok = step_produce(P, L.p_dn, t, rp, 5); }
    }
    if (ok) { auto P = SP::lm_head(p); ok = step_produce(P, p.p_lm, t, rp, 6); }
    if (!ok) {
      sg_drain(t.sm, rp);
      if (lane == 0) atomicExch(p.status, sg_abort_status(t.sm.c->abortf, kStatusMbarTimeout));
    }
    return;
  }

  // -------------------------------------------------------------------- consumer warps
  unsigned int bar_target = 0;
  for (int l = 0; l < p.num_layers; ++l) {
    const StepLayer& L = p.layers[l];
    const __nv_bfloat16* h_in = l == 0 ? x0 : p.h;
    step_stamp(p, l, 0);
    { auto P = SP::qkv(p, L, h_in); step_consume(p, l, P, L.p_qkv, t, rp, 1); }
    step_stamp(p, l, 1);
    step_grid_sync(p, t, bar_target);
    step_signal(t);
    step_stamp(p, l, 2);
    { const FdSplit f = step_fd_split(p); step_fd_consume<HD>(p, t, rp, f); }
    step_stamp(p, l, 3);
    step_grid_sync(p, t, bar_target);
    step_stamp(p, l, 4);
    step_fd_merge(p, t);
    step_grid_sync(p, t, bar_target);
    step_stamp(p, l, 5);
    { auto P = SP::oproj(p, L, h_in); step_consume(p, l, P, L.p_o, t, rp, 2); }
    step_stamp(p, l, 6);
    step_grid_sync(p, t, bar_target);
    step_stamp(p, l, 7);
    { auto P = SP::router(p, L); step_consume(p, l, P, L.p_router, t, rp, 3); }
    step_stamp(p, l, 8);
    step_grid_sync(p, t, bar_target);
    step_stamp(p, l, 9);
    if (warp == 0) step_topk(p, L, t);
    sg_consumer_sync();
    step_signal(t);
    step_stamp(p, l, 10);
    { auto P = SP::gate_up(p, L, t); step_consume(p, l, P, L.p_gu, t, rp, 4); }
    step_stamp(p, l, 11);
    step_grid_sync(p, t, bar_target);
    step_stamp(p, l, 12);
    { auto P = SP::down(p, L, t); step_consume(p, l, P, L.p_dn, t, rp, 5); }
    step_stamp(p, l, 13);
    step_grid_sync(p, t, bar_target);
    step_stamp(p, l, 14);
  }
  { auto P = SP::lm_head(p); step_consume(p, p.num_layers - 1, P, p.p_lm, t, rp, 6); }
  if (*t.sm.c->abortf && threadIdx.x == 0) atomicExch(p.status, sg_abort_status(t.sm.c->abortf, kStatusMbarTimeout));
}

}  // namespace rb

using namespace rb;
RB_BOUNDS_REGISTER("decode_step.cu")


// ---- host interface -----------------------------------------------------------------------------
// The caller fills a plain-int description of the model and the per-layer pointers; the plans and
// the shared-memory layout are computed here.
struct RmlxStepLayerDesc {
  const void *wqkv, *wqkv_s, *wqkv_b;
  const void *wo, *wo_s, *wo_b;
  const void *wgu, *wgu_s, *wgu_b;       // [E_local, 2I, D]
  const void *wdn, *wdn_s, *wdn_b;       // [E_local, D, I]
  const void *norm1, *norm2, *router, *expert_bias;
  void *k_cache, *v_cache;
  int expert_base, experts_local;
};

struct RmlxStepDesc {
  int num_layers, D, Hq, Hkv, HD, I, E, top_k, V, q4;
  float eps, scale;
  int max_blocks, window, traditional;
  const void *tokens, *positions, *seq_lens, *block_table, *cos_t, *sin_t, *embed, *final_norm;
  const void *lm, *lm_s, *lm_b;
  void *h, *h2, *q, *attn, *act, *router_logits, *topk_idx, *topk_w, *fd_part_o, *fd_part_ml, *logits;
  void *grid_bar;
  void *trace;                           // optional [num_layers * 32] u64 phase stamps of block 0
  void *layers_dev;                      // device buffer of num_layers * rmlx_decode_step_layer_bytes()
};

extern "C" int rmlx_decode_step_layer_bytes() { return int(sizeof(StepLayer)); }
extern "C" int rmlx_decode_step_desc_bytes() { return int(sizeof(RmlxStepDesc)); }
extern "C" int rmlx_decode_step_layer_desc_bytes() { return int(sizeof(RmlxStepLayerDesc)); }

// Scratch sizes (floats) of the attention phase for a grid of `grid` blocks.
extern "C" long long rmlx_decode_step_fd_part_o_elems(int grid, int Hq, int Hkv, int HD) {
  const int G = Hq / Hkv, tiles = Hkv * ((G + 15) / 16);
  return 1LL * tiles * (grid / tiles > 0 ? grid / tiles : 1) * 16 * HD;
}
extern "C" long long rmlx_decode_step_fd_part_ml_elems(int grid, int Hq, int Hkv) {
  const int G = Hq / Hkv, tiles = Hkv * ((G + 15) / 16);
  return 1LL * tiles * (grid / tiles > 0 ? grid / tiles : 1) * 32;
}
extern "C" int rmlx_decode_step_grid() { return sm_count(); }

extern "C" int rmlx_decode_step_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_step_status, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_step_status, &zero, sizeof(int));
  return v;
}

static int step_fill(const RmlxStepDesc& d, const RmlxStepLayerDesc* ld, StepParams& p,
                     StepLayer* host_layers, int grid) {
  const int q4 = d.q4;               // weight kind
  if (q4 < 0 || q4 > 2) return -2;
  if (d.HD != 64 && d.HD != 128) return -2;
  if (d.E > kStMaxExperts || d.top_k > kSgMaxTopK || d.I % 2 || d.Hq % d.Hkv) return -2;
  const int G = d.Hq / d.Hkv, tiles = d.Hkv * ((G + 15) / 16);
  if (tiles > grid || d.Hq * d.HD % 8) return -2;
  p = StepParams{};
  p.num_layers = d.num_layers; p.D = d.D; p.Hq = d.Hq; p.Hkv = d.Hkv; p.HD = d.HD; p.I = d.I; p.E = d.E;
  p.top_k = d.top_k; p.V = d.V; p.q4 = d.q4; p.eps = d.eps; p.scale_log2 = d.scale * 1.4426950408889634f;
  p.max_blocks = d.max_blocks; p.window = d.window; p.traditional = d.traditional;
  p.tokens = static_cast<const int*>(d.tokens); p.positions = static_cast<const int*>(d.positions);
  p.seq_lens = static_cast<const int*>(d.seq_lens); p.block_table = static_cast<const int*>(d.block_table);
  p.cos_t = static_cast<const float*>(d.cos_t); p.sin_t = static_cast<const float*>(d.sin_t);
  p.embed = static_cast<const __nv_bfloat16*>(d.embed);
  p.final_norm = static_cast<const __nv_bfloat16*>(d.final_norm);
  p.h = static_cast<__nv_bfloat16*>(d.h); p.h2 = static_cast<__nv_bfloat16*>(d.h2);
  p.q = static_cast<__nv_bfloat16*>(d.q); p.attn = static_cast<__nv_bfloat16*>(d.attn);
  p.act = static_cast<__nv_bfloat16*>(d.act); p.router_logits = static_cast<float*>(d.router_logits);
  p.topk_idx = static_cast<int*>(d.topk_idx); p.topk_w = static_cast<float*>(d.topk_w);
  p.fd_part_o = static_cast<float*>(d.fd_part_o); p.fd_part_ml = static_cast<float*>(d.fd_part_ml);
  p.logits = static_cast<float*>(d.logits); p.grid_bar = static_cast<unsigned int*>(d.grid_bar);
  p.trace = static_cast<unsigned long long*>(d.trace);
  p.layers = static_cast<const StepLayer*>(d.layers_dev);

  int slot = kStFdWarps * 2 * kStPage * d.HD * 2;      // a stage of KV pages
  int xb = 0, extra = 64, qpt = 1;
  auto take = [&](const SgPlan& pl) -> bool {
    if (pl.grid < 1 || pl.grid > grid) return false;
    if (pl.stage_bytes > slot) slot = pl.stage_bytes;
    if (pl.x_bytes > xb) xb = pl.x_bytes;
    if (pl.extra_bytes > extra) extra = pl.extra_bytes;
    if (pl.qpt > qpt) qpt = pl.qpt;
    return true;
  };
  const int Kq = d.Hq * d.HD, hq2 = d.I / 2;
  for (int l = 0; l < d.num_layers; ++l) {
    const RmlxStepLayerDesc& s = ld[l];
    StepLayer& L = host_layers[l];
    if (!sg_weights_ok(q4, s.wqkv, s.wqkv_s, s.wqkv_b, d.D) || !sg_weights_ok(q4, s.wo, s.wo_s, s.wo_b, Kq) ||
        !sg_weights_ok(q4, s.wgu, s.wgu_s, s.wgu_b, d.D) || !sg_weights_ok(q4, s.wdn, s.wdn_s, s.wdn_b, d.I) ||
        !sg_aligned16(s.router) || d.D % 64 || (q4 == 0 && d.I % 32) || s.experts_local > 256)
      return -2;
    L.wqkv = sg_weights(q4, s.wqkv, s.wqkv_s, s.wqkv_b, d.D);
    L.wo = sg_weights(q4, s.wo, s.wo_s, s.wo_b, Kq);
    L.wgu = sg_weights(q4, s.wgu, s.wgu_s, s.wgu_b, d.D);
    L.wdn = sg_weights(q4, s.wdn, s.wdn_s, s.wdn_b, d.I);
    L.norm1 = static_cast<const __nv_bfloat16*>(s.norm1); L.norm2 = static_cast<const __nv_bfloat16*>(s.norm2);
    L.router = static_cast<const __nv_bfloat16*>(s.router);
    L.expert_bias = static_cast<const float*>(s.expert_bias);
    L.k_cache = static_cast<__nv_bfloat16*>(s.k_cache); L.v_cache = static_cast<__nv_bfloat16*>(s.v_cache);
    L.expert_base = s.expert_base; L.experts_local = s.experts_local;
    L.p_qkv = sg_make_plan(q4, L.wqkv.units, 1, !d.traditional, (d.Hq + 2 * d.Hkv) * (d.HD / 4), grid,
                           d.HD / 4, sg_x_bytes(q4, d.D, 1), SgQkvRope<1, 1>::extra_bytes(d.HD, 1), 1);
    L.p_o = sg_make_plan(q4, L.wo.units, 1, false, (d.D + 3) / 4, grid, 1 << 20, sg_x_bytes(q4, Kq, 1), 0, 1);
    L.p_router = sg_make_plan(0, d.D >> 3, 1, false, (d.E + 3) / 4, grid, 1 << 20, sg_x_bytes(0, d.D, 1), 0, 1);
    L.p_gu = sg_make_plan(q4, L.wgu.units, 1, true, d.top_k * hq2, grid, hq2 & -hq2, sg_x_bytes(q4, d.D, 1), 0, 1);
    L.p_dn = sg_make_plan(q4, L.wdn.units, d.top_k, false, (d.D + 3) / 4, grid, 1 << 20,
                          sg_x_bytes(q4, d.top_k * d.I, 1), 64, 1);
    if (!take(L.p_qkv) || !take(L.p_o) || !take(L.p_router) || !take(L.p_gu) || !take(L.p_dn)) return -2;
  }
  if (!sg_weights_ok(q4, d.lm, d.lm_s, d.lm_b, d.D)) return -2;
  p.lm_head = sg_weights(q4, d.lm, d.lm_s, d.lm_b, d.D);
  p.p_lm = sg_make_plan(q4, p.lm_head.units, 1, false, (d.V + 3) / 4, grid, 1 << 20, sg_x_bytes(q4, d.D, 1), 0, 1);
  if (!take(p.p_lm)) return -2;
  p.ns = 2;
  p.slot_bytes = (slot + 127) & ~127;
  p.x_bytes = xb;
  p.part_floats = sg_part_floats(p.ns, qpt, 1);
  p.extra_bytes = (extra + 15) & ~15;
  if (step_smem_bytes(p, d.HD) > 220 * 1024) return -2;
  return 0;
}

// Builds the device-side layer table (a synchronous copy: call once, outside stream capture).
// `layer_descs`: host array of num_layers RmlxStepLayerDesc. Returns 0, or -2 when the model does
// not fit this kernel (the caller then runs the step as separate kernels).
extern "C" int rmlx_decode_step_prepare(const void* desc, const void* layer_descs) {
  const RmlxStepDesc& d = *static_cast<const RmlxStepDesc*>(desc);
  if (d.num_layers < 1 || d.num_layers > 4096) return -2;
  StepLayer* host_layers = new StepLayer[d.num_layers];
  StepParams p;
  int rc = step_fill(d, static_cast<const RmlxStepLayerDesc*>(layer_descs), p, host_layers, sm_count());
  if (rc == 0)
    rc = static_cast<int>(cudaMemcpy(d.layers_dev, host_layers, sizeof(StepLayer) * d.num_layers, cudaMemcpyHostToDevice));
  delete[] host_layers;
  return rc;
}

// Launches the step (grid_bar must be zero: the caller clears it on the same stream first).
extern "C" int rmlx_decode_step_launch(const void* desc, const void* layer_descs, cudaStream_t st) {
  const RmlxStepDesc& d = *static_cast<const RmlxStepDesc*>(desc);
  const int grid = sm_count();
  StepLayer* host_layers = new StepLayer[d.num_layers];
  StepParams p;
  int rc = step_fill(d, static_cast<const RmlxStepLayerDesc*>(layer_descs), p, host_layers, grid);
  delete[] host_layers;
  if (rc != 0) return rc;
  void* sp = nullptr;
  RB_CHECK(cudaGetSymbolAddress(&sp, g_step_status));
  p.status = static_cast<int*>(sp);
  const size_t smem = step_smem_bytes(p, d.HD);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kSgThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
#define RB_STEP(Q4_, HD_)                                                                          \
  {                                                                                                \
    auto kern = decode_step_kernel<Q4_, HD_>;                                                      \
    RB_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem))); \
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);                                             \
    if (e != cudaSuccess) (void)cudaGetLastError();                                                \
    return static_cast<int>(e);                                                                    \
  }
  if (d.q4 == 1 && d.HD == 128) RB_STEP(1, 128)
  if (d.q4 == 1 && d.HD == 64) RB_STEP(1, 64)
  if (d.q4 == 2 && d.HD == 128) RB_STEP(2, 128)
  if (d.q4 == 2 && d.HD == 64) RB_STEP(2, 64)
  if (d.q4 == 0 && d.HD == 128) RB_STEP(0, 128)
  if (d.q4 == 0 && d.HD == 64) RB_STEP(0, 64)
#undef RB_STEP
  return -2;
}
