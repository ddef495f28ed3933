// Persistent weight-streaming mat-vec for decode (a handful of activation vectors against a large
// weight matrix): ONE block per SM, a producer warp that keeps a ring of shared-memory stages full
// with large bulk asynchronous copies (cp.async.bulk + mbarrier transaction counts), and sixteen
// consumer warps that multiply out of shared memory.
//
// Shape of the ring, from measurements on B200 (148 blocks, one producer each, HBM -> shared):
//   * a bulk copy costs ~55 cycles of the copy engine whatever its size, so 512-byte copies reach
//     1.8 TB/s, 2 KB 4.6 TB/s and >= 8 KB 6.5 TB/s: rows are therefore fetched as whole contiguous
//     runs of rows ("segments"), one copy per segment and stage, never row by row;
//   * with one block per SM the stream delivers 4.0 TB/s with 16 KB stages and 6.2-6.7 TB/s with
//     32 KB stages;
//   * the 4-bit inner loop is bound by instruction latency, not by a pipe (half-precision FMA and
//     integer logic both issue at half rate on this part): eight consumer warps reach 37 % issue
//     utilisation, so there are sixteen, each with two tasks per stage in flight.
// Stages are ~64 KB and the ring holds ~170 KB: the decode projections are short (a
// block of the QKV projection owns 148 KB of weights), so a block has most or all of its weights in
// flight before its first multiply. In a programmatic-dependent-launch chain a block of the next
// kernel takes over an SM as soon as this kernel's block leaves it, and fills its ring while the
// other SMs finish and the activations are staged. Activations are staged once per SM; four weight rows
// share every activation read from shared memory (the 4-bit path is bound by instruction issue
// and shared-memory bandwidth, not by HBM).
//
// Work decomposition. A "quad" is four output rows that one lane group accumulates together (a
// problem decides which four rows: consecutive ones, or the two row pairs that RoPE / SwiGLU
// combine). A row is cut into K slices of LW 16-byte units (LW = 32, 16 or 8 lanes; a unit is 32
// four-bit weights or 8 bf16 weights); a task is (32 / LW) quads x one slice. A stage holds QS
// quads with ALL their slices (or, for very long rows, one of KP column parts); its sixteen warps
// are arranged TR x SQ: TR task rows, SQ warps striding over the slices of a task row. When SQ > 1
// the warps of a task row hand their partial sums to the row's first warp through shared memory
// and a per-row mbarrier (the last warp to hand over signals); that warp adds them in a fixed
// order (deterministic results) and runs the problem's epilogue. There is no block-wide barrier in the main loop.
//
// Scales and biases of the 4-bit format (bf16 per 64 weights: one byte of each per unit) travel
// through the same ring, one copy per segment. Their rows need not start on 16-byte boundaries, so
// the producer copies the enclosing aligned span and posts the remainder in the stage's meta data.
//
// Every wait is bounded: an expired mbarrier wait raises a block-wide abort flag, the block keeps
// its control flow (no barrier is skipped), waits for its own copies in flight and reports through
// a status word.
//
// The reference's decode mat-vecs are its gemv / affine_qmv_fast / fused_rms_gemv Metal kernels
// (crates/rmlx-core/src/ops/gemv.rs:488, quantized.rs:407, fused.rs:1530); none of them stages
// weights through an asynchronous ring.
#pragma once
#include "../common/gemv_core.cuh"
#include "../common/launch.cuh"

namespace rb {

constexpr int kSgConsumerWarps = 16;
constexpr int kSgConsumers = kSgConsumerWarps * 32;        // 512
constexpr int kSgThreads = kSgConsumers + 32;              // + producer warp
constexpr int kSgMaxStages = 4;
constexpr int kSgMaxSeg = 8;                               // segments per stage
constexpr int kSgStageTarget = 64 * 1024;                  // weight bytes per stage

struct SgPlan {
  int LW;            // lanes (16-byte units) per K slice: 32, 16 or 8
  int qpt;           // quads per task = 32 / LW
  int TR, SQ;        // warps of a stage: TR task rows x SQ slice strides (TR * SQ == 16)
  int QS;            // quads per stage = TR * qpt
  int units;         // 16-byte units per row (per routed slot for the expert down projection)
  int spl;           // slices per (slot) row = ceil(units / LW)
  int KP;            // column parts per row block (1 unless a single task row exceeds the stage)
  int spp;           // slices per part
  int pairs;         // rows of a quad come as two pairs from two segments (else 4 consecutive rows)
  int nseg;          // segments per stage (1, 2, or the number of routed slots)
  int seg_rows;      // rows per segment and stage
  int w_row_bytes;   // bytes per row inside a stage (one part)
  int w_seg_bytes;   // seg_rows * w_row_bytes
  int aux_seg_bytes; // reserved per segment for the scale span (same again for the bias span)
  int aux_off;       // offset of the aux area inside a stage
  int stage_bytes;
  int qpc;           // quads per block (multiple of QS)
  int quads;         // quads in the problem (per token for the per-token problems)
  int ns;            // ring stages
  int x_bytes;       // staged activations (all vectors)
  int extra_bytes;   // problem-specific shared memory
  int grid;          // blocks (per token for the per-token problems); 0 = shape not supported
  int drop_stage;    // test hook: block 0's producer withholds this stage (-1: none)
  int srow;          // quantised weights: bytes of scales (and of biases) per row
  int scale_f16;     // scales and biases are fp16 (MLX checkpoints in half precision), else bf16
};

__host__ __device__ inline int sg_part_floats(int ns, int qpt, int B) { return ns * kSgConsumerWarps * qpt * 4 * B; }

__host__ inline size_t sg_smem_bytes(const SgPlan& p, int B);

// Chooses the task shape and the block partition. `units`: 16-byte weight units per row (per slot);
// `nslots`: how many such rows are chained along K (1, or top-k for the expert down projection);
// `pairs`: quads are two row pairs from two segments; `quads`: quads to spread over at most
// `max_ctas` blocks; `qs_cap`: upper bound on quads per stage (a stage must not straddle a head or
// an expert). Returns grid == 0 when the shape does not fit.
// `kind`: 0 bf16 weights, 1 4-bit affine, 2 8-bit affine (group 64, bf16 scale and bias).
__host__ inline SgPlan sg_make_plan(int kind, int units, int nslots, bool pairs, int quads, int max_ctas,
                                    int qs_cap, int x_bytes, int extra_bytes, int B) {
  SgPlan p{};
  const int base_kind = kind & 0xff;    // bit 8 of `kind`: fp16 scales and biases
  const bool q4 = base_kind != 0;       // quantised: scales and biases travel with the weights
  p.srow = base_kind == 1 ? units : base_kind == 2 ? units / 2 : 0;
  int best_lw = 32, best_pad = 1 << 30;
  const int lws[3] = {32, 16, 8};
  for (int i = 0; i < 3; ++i) {
    const int lw = lws[i];
    const int pad = (units + lw - 1) / lw * lw;
    if (pad < best_pad) { best_pad = pad; best_lw = lw; }
  }
  p.LW = best_lw;
  p.qpt = 32 / p.LW;
  p.units = units;
  p.spl = (units + p.LW - 1) / p.LW;
  p.pairs = pairs ? 1 : 0;
  p.nseg = pairs ? 2 : nslots;
  p.quads = quads;
  if (p.nseg > kSgMaxSeg || quads < 1 || units < 1 || (pairs && nslots != 1)) return p;
  const int row_bytes = units * 16 * nslots;          // one output row, all slots
  // quads per stage: as many as fit the stage target, a power of two times qpt
  int tr = kSgConsumerWarps;
  while (tr > 1 && (tr * p.qpt * 4 * row_bytes > kSgStageTarget || tr * p.qpt > qs_cap)) tr >>= 1;
  if (tr * p.qpt > qs_cap) return p;                  // cap smaller than one task
  if (max_ctas < 1) max_ctas = 1;
  int qpc = (quads + max_ctas - 1) / max_ctas;
  while (tr > 1 && tr * p.qpt >= 2 * qpc) tr >>= 1;   // never more task rows than a block has work for
  p.TR = tr; p.SQ = kSgConsumerWarps / tr; p.QS = tr * p.qpt;
  qpc = (qpc + p.QS - 1) / p.QS * p.QS;
  p.qpc = qpc;
  p.KP = 1;
  if (p.QS * 4 * row_bytes > kSgStageTarget + kSgStageTarget / 2) {   // a single task row is too long
    if (nslots != 1 || q4) return p;
    p.KP = (p.QS * 4 * row_bytes + kSgStageTarget - 1) / kSgStageTarget;
  }
  p.spp = (p.spl + p.KP - 1) / p.KP;
  p.KP = (p.spl + p.spp - 1) / p.spp;
  p.seg_rows = (pairs ? 2 : 4) * p.QS;
  p.w_row_bytes = (p.KP == 1 ? units : p.spp * p.LW) * 16;
  p.w_seg_bytes = p.seg_rows * p.w_row_bytes;
  p.aux_seg_bytes = q4 ? ((p.seg_rows * p.srow + 32 + 15) & ~15) : 0;
  p.aux_off = (p.nseg * p.w_seg_bytes + 127) & ~127;
  p.stage_bytes = (p.aux_off + 2 * p.nseg * p.aux_seg_bytes + 127) & ~127;
  p.x_bytes = (x_bytes + 127) & ~127;
  p.extra_bytes = (extra_bytes + 15) & ~15;
  // ring depth: as deep as ~150 KB allows (a short kernel then has all of its weights in flight
  // before its first multiply), never deeper than the block has stages
  {
    const int stages = ((qpc + p.QS - 1) / p.QS) * p.KP;
    int ns = (170 * 1024) / p.stage_bytes;
    if (ns > kSgMaxStages) ns = kSgMaxStages;
    if (ns > stages) ns = stages;
    if (ns < 2) ns = 2;
    p.ns = ns;
  }
  p.grid = (quads + qpc - 1) / qpc;
  p.drop_stage = -1;
  p.scale_f16 = kind >> 8 & 1;
  (void)B;
  return p;
}

// ------------------------------------------------------------------------------------------------
// device helpers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void sg_consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kSgConsumers) : "memory"); }

__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes,
                                         uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// mbarrier wait that looks at the abort flag first, so a block that has given up once never burns
// another budget.
// `where` names the waiting site; the first site whose wait expires is kept beside the abort flag
// and ends up in the status word (bits 8 and up), so a failure can be located from the host.
__device__ __forceinline__ bool sg_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abortf,
                                        uint32_t where = 0) {
  if (*abortf) return false;
  const bool ok = mbar_wait(bar, parity, abortf, 1u << 19);
  if (!ok) atomicCAS(const_cast<uint32_t*>(abortf) + 1, 0u, where);
  return ok;
}
__device__ __forceinline__ int sg_abort_status(volatile uint32_t* abortf, int code) {
  return code | int(abortf[1] << 8);
}

// Sum over the consumer threads. `red` has one float per consumer warp; two consumer barriers.
__device__ __forceinline__ float sg_consumer_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  sg_consumer_sync();
  float t = (lane < kSgConsumerWarps) ? red[lane] : 0.f;
  t = warp_sum(t);
  sg_consumer_sync();
  return t;
}

// One task of the 4-bit path: rows w0..w3 (16-byte unit each) against the staged activations. The
// four (scale, bias) pairs are read from the stage only when the dot products are done (they would
// otherwise sit in eight registers through the whole inner loop): `alo` / `ahi` address the scales
// of rows 0 / 2, the next row's is `units` bytes on, the biases `bias_off` bytes on.
template <int B>
__device__ __forceinline__ void sg_task_q4(const uint4 (&w)[4], uint32_t alo, uint32_t ahi, uint32_t units,
                                           uint32_t bias_off, bool sf16, const char* xs, size_t xstride,
                                           int NHG, int xunit, float (&acc)[4][B]) {
  auto lds16 = [sf16](uint32_t addr) -> float {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return sf16 ? __half2float(__ushort_as_half(v)) : bf16lo(v);
  };
#pragma unroll
  for (int b = 0; b < B; ++b) {
    const uint4* xh = reinterpret_cast<const uint4*>(xs + b * xstride);
    const float* aux = reinterpret_cast<const float*>(xs + b * xstride + size_t(NHG) * 64);
    const float xsum = aux[xunit], qmul = aux[NHG + xunit];
    __half2 a0[4], a1[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) a0[r] = a1[r] = __float2half2_rn(0.f);
    {
      const uint4 x0 = xh[xunit];
#pragma unroll
      for (int r = 0; r < 4; ++r) q4_word_fma(w[r].x, x0, a0[r], a1[r]);
      const uint4 x1 = xh[NHG + xunit];
#pragma unroll
      for (int r = 0; r < 4; ++r) q4_word_fma(w[r].y, x1, a0[r], a1[r]);
      const uint4 x2 = xh[2 * NHG + xunit];
#pragma unroll
      for (int r = 0; r < 4; ++r) q4_word_fma(w[r].z, x2, a0[r], a1[r]);
      const uint4 x3 = xh[3 * NHG + xunit];
#pragma unroll
      for (int r = 0; r < 4; ++r) q4_word_fma(w[r].w, x3, a0[r], a1[r]);
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const uint32_t a = ((r >> 1) ? ahi : alo) + ((r & 1) ? units : 0u);
      const float sc = lds16(a), bi = lds16(a + bias_off);
      const float2 f0 = __half22float2(a0[r]), f1 = __half22float2(a1[r]);
      const float qx = ((f0.x + f0.y) + (f1.x + f1.y)) * qmul;
      acc[r][b] = fmaf(sc, qx, fmaf(bi, xsum, acc[r][b]));
    }
  }
}

// One task of the 8-bit path: rows w0..w3 (16 weights each) against the staged activations.
template <int B>
__device__ __forceinline__ void sg_task_q8(const uint4 (&w)[4], uint32_t alo, uint32_t ahi, uint32_t srow,
                                           uint32_t bias_off, bool sf16, const char* xs, size_t xstride,
                                           int NU, int xunit, float (&acc)[4][B]) {
  auto lds16 = [sf16](uint32_t addr) -> float {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return sf16 ? __half2float(__ushort_as_half(v)) : bf16lo(v);
  };
#pragma unroll
  for (int b = 0; b < B; ++b) {
    const uint4* xh = reinterpret_cast<const uint4*>(xs + b * xstride);
    const float* aux = reinterpret_cast<const float*>(xs + b * xstride + size_t(NU) * 32);
    const float xsum = aux[xunit], qmul = aux[NU + xunit];
    const uint4 x0 = xh[xunit], x1 = xh[NU + xunit];
    const __half2* h0 = reinterpret_cast<const __half2*>(&x0);
    const __half2* h1 = reinterpret_cast<const __half2*>(&x1);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      __half2 a0 = __float2half2_rn(0.f), a1 = a0;
      q8_word_fma(w[r].x, h0[0], h0[1], a0, a1);
      q8_word_fma(w[r].y, h0[2], h0[3], a0, a1);
      q8_word_fma(w[r].z, h1[0], h1[1], a0, a1);
      q8_word_fma(w[r].w, h1[2], h1[3], a0, a1);
      const uint32_t a = ((r >> 1) ? ahi : alo) + ((r & 1) ? srow : 0u);
      const float sc = lds16(a), bi = lds16(a + bias_off);
      const float2 f0 = __half22float2(a0), f1 = __half22float2(a1);
      const float qx = ((f0.x + f0.y) + (f1.x + f1.y)) * qmul;
      acc[r][b] = fmaf(sc, qx, fmaf(bi, xsum, acc[r][b]));
    }
  }
}

template <int B>
__device__ __forceinline__ void sg_task_bf16(const uint4 (&w)[4], const char* xs, size_t xstride,
                                             int NCH, int xunit, float (&acc)[4][B]) {
#pragma unroll
  for (int b = 0; b < B; ++b) {
    const float4* x4 = reinterpret_cast<const float4*>(xs + b * xstride);
    const float4 x0 = x4[xunit], x1 = x4[NCH + xunit];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      float a = acc[r][b];
      a = fmaf(bf16lo(w[r].x), x0.x, a); a = fmaf(bf16hi(w[r].x), x0.y, a);
      a = fmaf(bf16lo(w[r].y), x0.z, a); a = fmaf(bf16hi(w[r].y), x0.w, a);
      a = fmaf(bf16lo(w[r].z), x1.x, a); a = fmaf(bf16hi(w[r].z), x1.y, a);
      a = fmaf(bf16lo(w[r].w), x1.z, a); a = fmaf(bf16hi(w[r].w), x1.w, a);
      acc[r][b] = a;
    }
  }
}

// One task's operands in registers.
struct SgTask { uint4 w[4]; uint32_t alo, ahi; int xunit; bool on; };   // alo/ahi: shared-memory addresses of the scale pairs

// Per stage and segment, posted by the producer: how far the scale / bias spans start past a
// 16-byte boundary, and how many rows the segment holds (0 = segment absent).
struct SgSegMeta { uint16_t mis_sc, mis_bi, rows, pad; };

// Fixed-layout control block at the start of a block's shared memory. Everything small lives here
// so that one pointer reaches it (sixteen separate pointers cost thirty-two registers per thread).
struct SgCtl {
  uint64_t full[kSgMaxStages];
  uint64_t empty[kSgMaxStages];
  uint64_t partbar[kSgMaxStages * kSgConsumerWarps];   // one arrival each: the last warp to hand over signals
  uint32_t pcnt[kSgMaxStages * kSgConsumerWarps];      // hand-overs counted so far
  uint32_t ppar[kSgMaxStages * kSgConsumerWarps];      // parity each hand-over barrier completes next
  SgSegMeta meta[kSgMaxStages * kSgMaxSeg];
  volatile uint32_t abortf[2];                         // abort flag, first expired wait site
  volatile uint32_t go;                                // multi-problem kernels: events passed by the consumers
  uint32_t pad0;
  float misc[64];                                      // inv_rms[4], red[16], free use
  int r_idx[8];                                        // multi-problem kernels: routing result
  float r_w[8];
};

// Shared-memory map of one block: the control block, then the ring, the staged activations, the
// partial sums [ns][warps][qpt][4][B] and the problem's own area.
struct SgSmem {
  SgCtl* c;
  char* ring;
  char* xs;
  float* part;
  char* extra;
};

__host__ __device__ inline int sg_ctl_bytes() { return (int(sizeof(SgCtl)) + 127) & ~127; }

__device__ __forceinline__ SgSmem sg_carve(char* smem, const SgPlan& pl, int B) {
  SgSmem s;
  char* base = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem) + 127) & ~uintptr_t(127));
  s.c = reinterpret_cast<SgCtl*>(base);
  s.ring = base + sg_ctl_bytes();
  s.xs = s.ring + size_t(pl.ns) * pl.stage_bytes;
  s.part = reinterpret_cast<float*>(s.xs + pl.x_bytes);
  s.extra = reinterpret_cast<char*>(s.part + sg_part_floats(pl.ns, pl.qpt, B));
  return s;
}

__host__ inline size_t sg_smem_bytes(const SgPlan& p, int B) {
  return size_t(sg_ctl_bytes()) + size_t(p.ns) * p.stage_bytes + p.x_bytes +
         size_t(sg_part_floats(p.ns, p.qpt, B)) * 4 + p.extra_bytes + 256;
}

// Source of one segment of a stage.
struct SgSegSrc {
  const char* w;    // first row of the segment (first unit)
  const char* sc;   // its scales (one byte per unit), Q4 only
  const char* bi;
  int rows;         // valid rows (0: nothing to fetch)
};

// A problem P provides:
//   static constexpr int kKind (0 bf16, 1 Q4, 2 Q8); static constexpr int kB;
//   static constexpr bool kWeightsNeedWait;
//   static constexpr bool kMultiSlot                     rows chained along K over several segments
//   void cta_range(const SgPlan&, int& q0, int& q1)      this block's quads
//   void init(bool producer)                             every thread; consumers call it after
//                                                        pdl_wait, the producer too when
//                                                        kWeightsNeedWait
//   int nslots()                                         rows chained along K (<= plan.nseg)
//   SgSegSrc seg(const SgPlan&, int stage_q0, int nq, int g)   segment g of the stage that starts
//                                                        at quad stage_q0 and holds nq quads
//   int xunits()                                         units in one staged vector
//   void stage_x(SgSmem&, const SgPlan&)                 all consumer threads; ends in a barrier
//   void epilogue(int quad, float (&v)[4][kB], SgSmem&)  one lane per finished quad
//   void cta_done(SgSmem&)                               all consumer threads, once
// Position in the ring; it survives from one problem to the next when several run in one kernel.
struct SgRingPos {
  int s;              // slot of the next stage
  uint32_t round;     // how often the ring has wrapped
  uint32_t spare;
  int ns;             // slots
  int slot_bytes;     // distance between slots
  uint32_t tag;       // names the running problem in wait-site codes
};

// Producer side of one problem: issues the bulk copies of this block's stages, in order. Runs in
// one warp. Returns false when a wait expired.
template <class P, int LW>
__device__ __forceinline__ bool sg_produce(P& prob, const SgPlan& pl, SgSmem& sm, SgRingPos& rp, int q0, int q1) {
  const int lane = threadIdx.x & 31;
  const int myq = q1 > q0 ? q1 - q0 : 0;
  const int nrb = (myq + pl.QS - 1) / pl.QS;       // row blocks of this block
  const int nst = nrb * pl.KP;
  const int nseg = pl.pairs ? 2 : prob.nslots();
  for (int i = 0; i < nst; ++i) {
    const int s = rp.s;
    if (rp.round > 0 && !sg_wait(sm.c->empty + s, (rp.round - 1) & 1, sm.c->abortf, rp.tag * 16 + 1)) return false;
    if (i == pl.drop_stage && blockIdx.x == 0) {
      // test hook (a message that is never sent): the consumers' wait for this stage runs out
      if (++rp.s == rp.ns) { rp.s = 0; ++rp.round; }
      continue;
    }
    const int rb = i / pl.KP, kp = i - rb * pl.KP;
    const int sq0 = q0 + rb * pl.QS, nq = min(pl.QS, q1 - sq0);
    char* stage = sm.ring + size_t(s) * rp.slot_bytes;
    uint32_t bytes = 0;
    if (lane < nseg) {
      const SgSegSrc src = prob.seg(pl, sq0, nq, lane);
      SgSegMeta m{0, 0, uint16_t(src.rows), 0};
      if (src.rows > 0) {
        char* dst = stage + size_t(lane) * pl.w_seg_bytes;
        if (pl.KP == 1) {
          const uint32_t n = uint32_t(src.rows) * uint32_t(pl.units) * 16u;
          bulk_g2s(dst, src.w, n, sm.c->full + s);
          bytes += n;
        } else {
          const int u0 = kp * pl.spp * LW;
          const uint32_t n = uint32_t(min(pl.spp * LW, pl.units - u0)) * 16u;
          for (int r = 0; r < src.rows; ++r)
            bulk_g2s(dst + size_t(r) * pl.w_row_bytes, src.w + (size_t(r) * pl.units + u0) * 16, n, sm.c->full + s);
          bytes += n * uint32_t(src.rows);
        }
        if (P::kKind != 0) {
          const uintptr_t a = reinterpret_cast<uintptr_t>(src.sc), b2 = reinterpret_cast<uintptr_t>(src.bi);
          const uint32_t span = uint32_t(src.rows) * uint32_t(pl.srow);
          const uintptr_t alo = a & ~uintptr_t(15), ahi = (a + span + 15) & ~uintptr_t(15);
          const uintptr_t blo = b2 & ~uintptr_t(15), bhi = (b2 + span + 15) & ~uintptr_t(15);
          char* ax = stage + pl.aux_off + size_t(lane) * 2 * pl.aux_seg_bytes;
          bulk_g2s(ax, reinterpret_cast<const void*>(alo), uint32_t(ahi - alo), sm.c->full + s);
          bulk_g2s(ax + pl.aux_seg_bytes, reinterpret_cast<const void*>(blo), uint32_t(bhi - blo), sm.c->full + s);
          bytes += uint32_t(ahi - alo) + uint32_t(bhi - blo);
          m.mis_sc = uint16_t(a & 15u); m.mis_bi = uint16_t(b2 & 15u);
        }
      }
      sm.c->meta[s * kSgMaxSeg + lane] = m;
    }
    bytes = __reduce_add_sync(0xffffffffu, bytes);
    __syncwarp();
    if (lane == 0) mbar_arrive_expect_tx(sm.c->full + s, bytes);
    if (++rp.s == rp.ns) { rp.s = 0; ++rp.round; }
  }
  return true;
}

// After a wait has expired: the copies of the last `ns` stages may still be in flight towards this
// block's shared memory; wait for them (bounded) before the block leaves.
__device__ __forceinline__ void sg_drain(SgSmem& sm, const SgRingPos& rp) {
  for (int k = 0; k < rp.ns; ++k) {
    // slot k was last armed in round rp.round (k < rp.s) or rp.round - 1
    const int r = int(rp.round) - (k < rp.s ? 0 : 1);
    if (r >= 0) mbar_wait(sm.c->full + k, uint32_t(r) & 1u, sm.c->abortf, 1u << 16);
  }
}

// Hand-over barriers and counters of a block: one thread, once, before any use.
__device__ __forceinline__ void sg_init_handover(SgSmem& sm, int ns) {
  for (int i = 0; i < ns * kSgConsumerWarps; ++i) {
    mbar_init(sm.c->partbar + i, 1);
    sm.c->pcnt[i] = 0u;
    sm.c->ppar[i] = 0u;
  }
}

// Consumer side of one problem: all consumer warps. The activations are already staged.
template <class P, int LW>
__device__ __forceinline__ void sg_consume(P& prob, const SgPlan& pl, SgSmem& sm, SgRingPos& rp, int q0, int q1) {
  constexpr int B = P::kB;
  constexpr int QPT = 32 / LW;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int myq = q1 > q0 ? q1 - q0 : 0;
  const int nrb = (myq + pl.QS - 1) / pl.QS;
  const int nslots = prob.nslots();
  const int tr = warp / pl.SQ, sq = warp - tr * pl.SQ;
  const int sub = lane / LW, l = lane - sub * LW;
  const int xunits = prob.xunits();
  const size_t xstride = P::kKind == 1 ? (size_t(xunits) * 72 + 15) & ~size_t(15)
                         : P::kKind == 2 ? size_t(xunits) * 40 : size_t(xunits) * 32;
  const int qi = tr * QPT + sub;                    // this lane group's quad inside a stage
  const int nsl = pl.spl * nslots;                  // slices per output row (all slots)
  // rows of the quad inside a stage: pairs come from segments 0 and 1, consecutive rows from one
  const int row_lo = pl.pairs ? 2 * qi : 4 * qi, row_hi = pl.pairs ? 2 * qi : 4 * qi + 2;
  const uint32_t rowb = uint32_t(pl.w_row_bytes), units = uint32_t(pl.srow);   // `units`: bytes between rows' scales
  const uint32_t w_lo_off = uint32_t(row_lo) * rowb, w_hi_off = (pl.pairs ? uint32_t(pl.w_seg_bytes) : 0u) + uint32_t(row_hi) * rowb;
  const uint32_t a_lo_off = uint32_t(pl.aux_off) + uint32_t(row_lo) * units;
  const uint32_t a_hi_off = uint32_t(pl.aux_off) + (pl.pairs ? 2u * uint32_t(pl.aux_seg_bytes) : 0u) + uint32_t(row_hi) * units;

  for (int rb = 0; rb < nrb; ++rb) {
    float acc[4][B];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int b = 0; b < B; ++b) acc[r][b] = 0.f;
    const int sq0 = q0 + rb * pl.QS;
    const bool qvalid = sq0 + qi < q1;
    int s_used = 0;
    for (int kp = 0; kp < pl.KP; ++kp) {
      const int s = rp.s;
      s_used = s;
      const bool ok = sg_wait(sm.c->full + s, rp.round & 1u, sm.c->abortf, rp.tag * 16 + 2);
      if (ok && qvalid) {
        const char* stage = sm.ring + uint32_t(s) * uint32_t(rp.slot_bytes);
        const int s_lo = pl.KP == 1 ? 0 : kp * pl.spp, s_hi = pl.KP == 1 ? nsl : min(pl.spl, s_lo + pl.spp);
        // two slices per trip: the second one's shared-memory loads overlap the first one's math
        auto load = [&](int sl, SgTask& t) {
          int slot = 0, u = sl * LW + l;
          if (P::kMultiSlot) { slot = sl / pl.spl; u = (sl - slot * pl.spl) * LW + l; }
          const int segm = P::kMultiSlot ? slot : 0;
          const SgSegMeta mlo = sm.c->meta[s * kSgMaxSeg + segm];
          const SgSegMeta mhi = pl.pairs ? sm.c->meta[s * kSgMaxSeg + 1] : mlo;
          t.on = u < pl.units && row_lo < mlo.rows;      // a segment that was not fetched has rows == 0
          u = min(u, pl.units - 1);
          const uint32_t ucol = uint32_t(pl.KP == 1 ? u : u - s_lo * LW) * 16u;
          const char* sbase = stage + (P::kMultiSlot ? uint32_t(slot) * uint32_t(pl.w_seg_bytes) : 0u);
          t.w[0] = *reinterpret_cast<const uint4*>(sbase + w_lo_off + ucol);
          t.w[1] = *reinterpret_cast<const uint4*>(sbase + w_lo_off + rowb + ucol);
          t.w[2] = *reinterpret_cast<const uint4*>(sbase + w_hi_off + ucol);
          t.w[3] = *reinterpret_cast<const uint4*>(sbase + w_hi_off + rowb + ucol);
          t.xunit = slot * pl.units + u;
          if (P::kKind != 0) {
            const char* abase = stage + (P::kMultiSlot ? uint32_t(slot) * 2u * uint32_t(pl.aux_seg_bytes) : 0u) +
                                (P::kKind == 1 ? (u & ~1) : ((u >> 2) << 1));
            // the biases sit aux_seg_bytes after the scales (the launcher checks that both arrays start at
            // the same remainder modulo 16, so one remainder serves both)
            t.alo = smem_u32(abase + a_lo_off + mlo.mis_sc);
            t.ahi = smem_u32(abase + a_hi_off + mhi.mis_sc);
          }
        };
        for (int sl = s_lo + sq; sl < s_hi; sl += 2 * pl.SQ) {
          SgTask t0, t1;
          const bool two = sl + pl.SQ < s_hi;
          load(sl, t0);
          load(two ? sl + pl.SQ : sl, t1);
          t1.on = t1.on && two;
          if (t0.on) {
            if (P::kKind == 1) sg_task_q4<B>(t0.w, t0.alo, t0.ahi, units, uint32_t(pl.aux_seg_bytes), pl.scale_f16 != 0, sm.xs, xstride, xunits, t0.xunit, acc);
            else if (P::kKind == 2) sg_task_q8<B>(t0.w, t0.alo, t0.ahi, units, uint32_t(pl.aux_seg_bytes), pl.scale_f16 != 0, sm.xs, xstride, xunits, t0.xunit, acc);
            else sg_task_bf16<B>(t0.w, sm.xs, xstride, xunits, t0.xunit, acc);
          }
          if (t1.on) {
            if (P::kKind == 1) sg_task_q4<B>(t1.w, t1.alo, t1.ahi, units, uint32_t(pl.aux_seg_bytes), pl.scale_f16 != 0, sm.xs, xstride, xunits, t1.xunit, acc);
            else if (P::kKind == 2) sg_task_q8<B>(t1.w, t1.alo, t1.ahi, units, uint32_t(pl.aux_seg_bytes), pl.scale_f16 != 0, sm.xs, xstride, xunits, t1.xunit, acc);
            else sg_task_bf16<B>(t1.w, sm.xs, xstride, xunits, t1.xunit, acc);
          }
        }
      }
      __syncwarp();
      if (kp + 1 < pl.KP && lane == 0) mbar_arrive(sm.c->empty + s);   // the last part is released after the hand-over
      if (++rp.s == rp.ns) { rp.s = 0; ++rp.round; }
    }
    // ---- lane-group totals, hand-over to the task row's first warp, epilogue
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int b = 0; b < B; ++b) {
        float v = acc[r][b];
#pragma unroll
        for (int o = LW >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        acc[r][b] = v;
      }
    const int sh = s_used;
    if (pl.SQ > 1) {
      float* part = sm.part + size_t(sh) * (kSgConsumerWarps * QPT * 4 * B);
      if (sq != 0) {
        if (l == 0) {
          float* pp = part + ((warp * QPT + sub) * 4) * B;
#pragma unroll
          for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int b = 0; b < B; ++b) pp[r * B + b] = acc[r][b];
        }
        __syncwarp();
        if (lane == 0) {
          // the last of the SQ - 1 warps to hand over signals the task row's first warp
          __threadfence_block();
          uint32_t* cnt = sm.c->pcnt + sh * kSgConsumerWarps + tr;
          if (atomicAdd(cnt, 1u) == uint32_t(pl.SQ - 2)) {
            *cnt = 0u;
            __threadfence_block();
            mbar_arrive(sm.c->partbar + sh * kSgConsumerWarps + tr);
          }
        }
      } else {
        // the barrier's parity lives in shared memory: which warp owns a task row changes from
        // one problem to the next
        uint32_t* ppar = sm.c->ppar + sh * kSgConsumerWarps + tr;
        const uint32_t par = *ppar;
        sg_wait(sm.c->partbar + sh * kSgConsumerWarps + tr, par & 1u, sm.c->abortf, rp.tag * 16 + 3);
        __syncwarp();
        if (lane == 0) *ppar = par ^ 1u;
        for (int k = 1; k < pl.SQ; ++k) {
          const float* pp = part + (((warp + k) * QPT + sub) * 4) * B;
#pragma unroll
          for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int b = 0; b < B; ++b) acc[r][b] += pp[r * B + b];
        }
      }
    }
    if (sq == 0 && qvalid && l == 0) prob.epilogue(sq0 + qi, acc, sm);
    __syncwarp();
    if (lane == 0) mbar_arrive(sm.c->empty + sh);
  }
}

template <class P, int LW>
__global__ void __launch_bounds__(kSgThreads, 1) sg_kernel(P prob, SgPlan pl, int* status) {
  extern __shared__ char smem_raw[];
  SgSmem sm = sg_carve(smem_raw, pl, P::kB);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < pl.ns; ++s) {
      mbar_init(sm.c->full + s, 1);
      mbar_init(sm.c->empty + s, kSgConsumerWarps);
    }
    sg_init_handover(sm, pl.ns);
    sm.c->abortf[0] = 0u; sm.c->abortf[1] = 0u;
    fence_mbar_init();
  }
  __syncthreads();
  pdl_launch_dependents();
  int q0, q1;
  prob.cta_range(pl, q0, q1);
  SgRingPos rp{0, 0u, 0u, pl.ns, pl.stage_bytes, 0u};
  if (warp == kSgConsumerWarps) {
    if (P::kWeightsNeedWait) pdl_wait();
    prob.init(true);
    if (!sg_produce<P, LW>(prob, pl, sm, rp, q0, q1)) {
      sg_drain(sm, rp);
      if (lane == 0) atomicExch(status, sg_abort_status(sm.c->abortf, kStatusMbarTimeout));
    }
    return;
  }
  pdl_wait();
  prob.init(false);
  prob.stage_x(sm, pl);
  sg_consume<P, LW>(prob, pl, sm, rp, q0, q1);
  prob.cta_done(sm);
  if (*sm.c->abortf && threadIdx.x == 0) atomicExch(status, sg_abort_status(sm.c->abortf, kStatusMbarTimeout));
}

// ------------------------------------------------------------------------------------------------
// Weight addressing shared by the problems.
// ------------------------------------------------------------------------------------------------
struct SgWeights {
  const char* w;    // rows of units*16 bytes
  const char* sc;   // quantised: rows of `srow` bytes (one bf16 per 64 weights); else unused
  const char* bi;
  int units;
  int srow;
  __device__ __forceinline__ SgSegSrc rows(size_t n, int count) const {
    return SgSegSrc{w + n * size_t(units) * 16, sc + n * size_t(srow), bi + n * size_t(srow), count};
  }
};

// Test hook: the next launch withholds one stage in block 0 (see SgPlan::drop_stage).
__host__ inline int& sg_debug_drop() { static int v = -1; return v; }

__host__ inline bool sg_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Activation staging for up to B vectors of K values: x (bf16, global) times an optional
// per-channel norm weight; writes inv_rms[b] to misc[b] (1 when there is no norm).
template <int WK, int B>
__device__ __forceinline__ void sg_stage_plain(SgSmem& sm, const __nv_bfloat16* x, int x_stride,
                                               const __nv_bfloat16* norm_w, float eps, int K) {
  const int tid = threadIdx.x;
  const size_t xstride = WK == 1 ? (size_t(K >> 5) * 72 + 15) & ~size_t(15)
                         : WK == 2 ? size_t(K >> 4) * 40 : size_t(K >> 3) * 32;
#pragma unroll
  for (int b = 0; b < B; ++b) {
    XLoadBf16 ld{x + size_t(b) * x_stride, norm_w, 0.f};
    if (WK == 1) XStage<WQ4>::stage_part(sm.xs + b * xstride, K, ld, tid, kSgConsumers);
    else if (WK == 2) XStage<WQ8>::stage_part(sm.xs + b * xstride, K, ld, tid, kSgConsumers);
    else XStage<WBf16>::stage_part(sm.xs + b * xstride, K, ld, tid, kSgConsumers);
    if (norm_w) {
      const float ssq = sg_consumer_sum(ld.ssq, sm.c->misc + 4);
      if (tid == 0) sm.c->misc[b] = rsqrtf(ssq / float(K) + eps);
    } else if (tid == 0) {
      sm.c->misc[b] = 1.f;
    }
  }
  sg_consumer_sync();
}

}  // namespace rb
