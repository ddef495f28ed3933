// The decode projections expressed as problems of the weight-streaming mat-vec (stream_gemv.cuh):
// which four rows form a quad, how the activations are staged, and what happens to a quad's four
// dot products.
//
//   SgDense       out = residual + inv_rms * W (x * g)        QKV (unfused), O projection, LM head
//   SgQkvRope     RMSNorm + merged QKV + RoPE(Q, K) + paged K/V append
//   SgGateUp      RMSNorm + dense gate/up + SwiGLU
//   SgMoeGateUp   per routed slot: RMSNorm + expert gate/up + SwiGLU
//   SgMoeDown     expert down projections chained along K with the routing weights folded into
//                 the staged activations, + residual
//
// Reference counterparts: fused_rms_gemv / fused_swiglu_down (crates/rmlx-core/src/ops/fused.rs:
// 967,1530), rope + kv copy (ops/rope.rs:500-870, ops/copy.rs:554), gather_qmv
// (ops/quantized.rs:9634) and ExpertGroup::grouped_forward (crates/rmlx-nn/src/expert_group.rs:308).
#pragma once
#include "stream_gemv.cuh"

namespace rb {

constexpr int kSgMaxTopK = 8;

__device__ __forceinline__ float sg_silu_mul(float g, float u) { return g / (1.f + __expf(-g)) * u; }

// ------------------------------------------------------------------------------------------------
template <int WK, int B, bool OUT_F32>
struct SgDense {
  static constexpr int kKind = WK;
  static constexpr int kB = B;
  static constexpr bool kWeightsNeedWait = false;
  static constexpr bool kMultiSlot = false;
  SgWeights W;
  int N, K;
  const __nv_bfloat16* x; int x_stride;
  const __nv_bfloat16* norm_w; float eps;
  const __nv_bfloat16* residual; int res_stride;
  void* out; int out_stride;

  __device__ void cta_range(const SgPlan& pl, int& q0, int& q1) const {
    q0 = blockIdx.x * pl.qpc; q1 = min(pl.quads, q0 + pl.qpc);
  }
  __device__ void init(bool) {}
  __device__ int nslots() const { return 1; }
  __device__ int xunits() const { return WK == 1 ? K >> 5 : WK == 2 ? K >> 4 : K >> 3; }
  __device__ SgSegSrc seg(const SgPlan&, int sq0, int nq, int) const {
    return W.rows(size_t(sq0) * 4, min(4 * nq, N - 4 * sq0));
  }
  __device__ void stage_x(SgSmem& sm, const SgPlan&) { sg_stage_plain<WK, B>(sm, x, x_stride, norm_w, eps, K); }
  __device__ void epilogue(int quad, float (&v)[4][B], SgSmem& sm) {
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const float inv = sm.c->misc[b];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int n = quad * 4 + r;
        if (n < N) {
          float o = v[r][b] * inv;
          if (residual) o += bf16lo(__ldcg(reinterpret_cast<const uint16_t*>(residual + size_t(b) * res_stride + n)));
          if (OUT_F32) static_cast<float*>(out)[size_t(b) * out_stride + n] = o;
          else static_cast<__nv_bfloat16*>(out)[size_t(b) * out_stride + n] = __float2bfloat16_rn(o);
        }
      }
    }
  }
  __device__ void cta_done(SgSmem&) {}
};

// ------------------------------------------------------------------------------------------------
struct SgRopeArgs {
  __nv_bfloat16* q_out;          // [B, Hq, HD]
  __nv_bfloat16* k_cache;        // [blocks, Hkv, page, HD]
  __nv_bfloat16* v_cache;
  const int* block_table;        // [seqs, max_blocks]
  const int* positions;          // [B]
  const int* row_seq;            // [B] or nullptr (row b belongs to sequence b)
  const float* cos_t;            // [max_pos, HD/2]
  const float* sin_t;
  int Hq, Hkv, HD, max_blocks, page, traditional;
};

// A quad is the two rotation pairs (2p, 2p+1) of one head: rows {2p, 2p+1, HD/2+2p, HD/2+2p+1}
// (or four consecutive rows in the interleaved "traditional" layout), so the rotation happens on
// the fp32 dot products and the un-rotated projection never reaches memory.
template <int WK, int B>
struct SgQkvRope {
  static constexpr int kKind = WK;
  static constexpr int kB = B;
  static constexpr bool kWeightsNeedWait = false;
  static constexpr bool kMultiSlot = false;
  SgWeights W;
  int K;
  const __nv_bfloat16* x; int x_stride;
  const __nv_bfloat16* norm_w; float eps;
  SgRopeArgs a;

  __device__ void cta_range(const SgPlan& pl, int& q0, int& q1) const {
    q0 = blockIdx.x * pl.qpc; q1 = min(pl.quads, q0 + pl.qpc);
  }
  __device__ void init(bool) {}
  __device__ int nslots() const { return 1; }
  __device__ int xunits() const { return WK == 1 ? K >> 5 : WK == 2 ? K >> 4 : K >> 3; }
  __device__ SgSegSrc seg(const SgPlan&, int sq0, int nq, int g) const {
    if (a.traditional) return W.rows(size_t(sq0) * 4, 4 * nq);
    const int qph = a.HD >> 2, head = sq0 / qph, p0 = sq0 - head * qph;
    return W.rows(size_t(head) * a.HD + (g ? (a.HD >> 1) : 0) + 2 * p0, 2 * nq);
  }
  // extra shared memory per batch row: cos[HD/2], sin[HD/2] of the row's position, then the
  // position and the page it appends to, so the epilogue touches no global memory but its stores
  static __host__ __device__ int extra_bytes(int HD, int Bn) { return Bn * (HD * 4 + 16); }
  __device__ void stage_x(SgSmem& sm, const SgPlan&) {
    const int half = a.HD >> 1;
    for (int t = threadIdx.x; t < B * half; t += kSgConsumers) {
      const int b = t / half, i = t - b * half;
      const int pos = a.positions[b];
      float* cs = reinterpret_cast<float*>(sm.extra + b * (a.HD * 4 + 16));
      cs[i] = a.cos_t[size_t(pos) * half + i];
      cs[half + i] = a.sin_t[size_t(pos) * half + i];
      if (i == 0) {
        int* pi = reinterpret_cast<int*>(cs + a.HD);
        const int seq = a.row_seq ? a.row_seq[b] : b;
        pi[0] = pos;
        pi[1] = RB_BOUNDS(pos / a.page, a.max_blocks)
                    ? a.block_table[size_t(seq) * a.max_blocks + pos / a.page] : -1;
      }
    }
    sg_stage_plain<WK, B>(sm, x, x_stride, norm_w, eps, K);
  }
  __device__ void epilogue(int quad, float (&v)[4][B], SgSmem& sm) {
    const int half = a.HD >> 1, qph = a.HD >> 2, head = quad / qph, p = quad - head * qph;
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const float inv = sm.c->misc[b];
      const float* cs = reinterpret_cast<const float*>(sm.extra + b * (a.HD * 4 + 16));
      const int* pi = reinterpret_cast<const int*>(cs + a.HD);
      const int pos = pi[0];
      // pair j in {0,1}: rotation index i = 2p + j. Quad rows are {lo0, lo1, hi0, hi1} in the
      // half-split layout and {lo0, hi0, lo1, hi1} in the interleaved one.
      float lo[2], hi[2];
      if (a.traditional) { lo[0] = v[0][b]; hi[0] = v[1][b]; lo[1] = v[2][b]; hi[1] = v[3][b]; }
      else { lo[0] = v[0][b]; lo[1] = v[1][b]; hi[0] = v[2][b]; hi[1] = v[3][b]; }
#pragma unroll
      for (int j = 0; j < 2; ++j) { lo[j] *= inv; hi[j] *= inv; }
      if (head < a.Hq + a.Hkv) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int i = 2 * p + j;
          const float c = cs[i], s = cs[half + i];
          const float r0 = lo[j] * c - hi[j] * s, r1 = hi[j] * c + lo[j] * s;
          lo[j] = r0; hi[j] = r1;
        }
      }
      __nv_bfloat16* dst;
      if (head < a.Hq) {
        dst = a.q_out + (size_t(b) * a.Hq + head) * a.HD;
      } else {
        const int blk = pi[1];
        if (blk < 0) continue;              // bounds-checked build: position beyond the block table
        const bool is_k = head < a.Hq + a.Hkv;
        const int kvh = is_k ? head - a.Hq : head - a.Hq - a.Hkv;
        dst = (is_k ? a.k_cache : a.v_cache) + ((size_t(blk) * a.Hkv + kvh) * a.page + pos % a.page) * a.HD;
      }
      if (a.traditional) {
        uint2 o;
        o.x = pack_bf16(lo[0], hi[0]); o.y = pack_bf16(lo[1], hi[1]);
        *reinterpret_cast<uint2*>(dst + 4 * p) = o;
      } else {
        *reinterpret_cast<uint32_t*>(dst + 2 * p) = pack_bf16(lo[0], lo[1]);
        *reinterpret_cast<uint32_t*>(dst + half + 2 * p) = pack_bf16(hi[0], hi[1]);
      }
    }
  }
  __device__ void cta_done(SgSmem&) {}
};

// ------------------------------------------------------------------------------------------------
// Dense SwiGLU first half: W holds the gate rows [0, I) then the up rows [I, 2I); a quad is
// {gate 2q, gate 2q+1, up 2q, up 2q+1}.
template <int WK, int B>
struct SgGateUp {
  static constexpr int kKind = WK;
  static constexpr int kB = B;
  static constexpr bool kWeightsNeedWait = false;
  static constexpr bool kMultiSlot = false;
  SgWeights W;
  int I, K;
  const __nv_bfloat16* x; int x_stride;
  const __nv_bfloat16* norm_w; float eps;
  __nv_bfloat16* act; int act_stride;

  __device__ void cta_range(const SgPlan& pl, int& q0, int& q1) const {
    q0 = blockIdx.x * pl.qpc; q1 = min(pl.quads, q0 + pl.qpc);
  }
  __device__ void init(bool) {}
  __device__ int nslots() const { return 1; }
  __device__ int xunits() const { return WK == 1 ? K >> 5 : WK == 2 ? K >> 4 : K >> 3; }
  __device__ SgSegSrc seg(const SgPlan&, int sq0, int nq, int g) const {
    return W.rows(size_t(g ? I : 0) + 2 * size_t(sq0), 2 * nq);
  }
  __device__ void stage_x(SgSmem& sm, const SgPlan&) { sg_stage_plain<WK, B>(sm, x, x_stride, norm_w, eps, K); }
  __device__ void epilogue(int quad, float (&v)[4][B], SgSmem& sm) {
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const float inv = sm.c->misc[b];
      const float a0 = sg_silu_mul(v[0][b] * inv, v[2][b] * inv), a1 = sg_silu_mul(v[1][b] * inv, v[3][b] * inv);
      *reinterpret_cast<uint32_t*>(act + size_t(b) * act_stride + 2 * quad) = pack_bf16(a0, a1);
    }
  }
  __device__ void cta_done(SgSmem&) {}
};

// ------------------------------------------------------------------------------------------------
// Routed experts. The grid is cut per token (blockIdx.x / pl.grid); the expert of every routed
// slot is kept as one byte of a 64-bit register (local index, at most 256 local experts).
struct SgRouting {
  const int* topk_idx;     // [tokens, top_k] global expert ids
  const float* topk_w;     // [tokens, top_k]
  int top_k, expert_base, experts_local;
  __device__ void load(int token, unsigned long long& packed, uint32_t& mask) const {
    packed = 0ull; mask = 0u;
    for (int s = 0; s < top_k; ++s) {
      const int e = topk_idx[token * top_k + s] - expert_base;
      if (e >= 0 && e < experts_local) { packed |= static_cast<unsigned long long>(e) << (8 * s); mask |= 1u << s; }
    }
  }
};

template <int WK>
struct SgMoeGateUp {
  static constexpr int kKind = WK;
  static constexpr int kB = 1;
  static constexpr bool kWeightsNeedWait = true;
  static constexpr bool kMultiSlot = false;
  SgWeights W;             // rows: [E_local][2I]
  int I, K;
  const __nv_bfloat16* x; int x_stride;
  const __nv_bfloat16* norm_w; float eps;
  __nv_bfloat16* act; int act_stride;   // [tokens*top_k, I]
  SgRouting R;
  int token, ntok;
  unsigned long long packed; uint32_t mask;

  __device__ void cta_range(const SgPlan& pl, int& q0, int& q1) {
    token = blockIdx.x / pl.grid;
    const int c = blockIdx.x - token * pl.grid;
    q0 = c * pl.qpc; q1 = min(pl.quads, q0 + pl.qpc);
    if (token >= ntok) { token = 0; q0 = q1 = 0; }
  }
  __device__ void init(bool) { R.load(token, packed, mask); }
  __device__ int nslots() const { return 1; }
  __device__ int xunits() const { return WK == 1 ? K >> 5 : WK == 2 ? K >> 4 : K >> 3; }
  __device__ SgSegSrc seg(const SgPlan&, int sq0, int nq, int g) const {
    const int hq = I >> 1, s = sq0 / hq, i2 = sq0 - s * hq;
    if (!((mask >> s) & 1u)) return SgSegSrc{nullptr, nullptr, nullptr, 0};
    const int e = int((packed >> (8 * s)) & 0xffull);
    return W.rows(size_t(e) * 2 * I + (g ? I : 0) + 2 * size_t(i2), 2 * nq);
  }
  __device__ void stage_x(SgSmem& sm, const SgPlan&) {
    sg_stage_plain<WK, 1>(sm, x + size_t(token) * x_stride, 0, norm_w, eps, K);
  }
  __device__ void epilogue(int quad, float (&v)[4][1], SgSmem& sm) {
    const int hq = I >> 1, s = quad / hq, i2 = quad - s * hq;
    if (!((mask >> s) & 1u)) return;
    const float inv = sm.c->misc[0];
    const float a0 = sg_silu_mul(v[0][0] * inv, v[2][0] * inv), a1 = sg_silu_mul(v[1][0] * inv, v[3][0] * inv);
    *reinterpret_cast<uint32_t*>(act + size_t(token * R.top_k + s) * act_stride + 2 * i2) = pack_bf16(a0, a1);
  }
  __device__ void cta_done(SgSmem&) {}
};

// Activation source for the chained expert down projection: chunk c of the virtual vector that
// concatenates the local slots' activations, each scaled by its routing weight.
struct XLoadMoeAct {
  const __nv_bfloat16* act;   // token's first slot row
  int act_stride, cps;        // chunks (of 8) per slot
  const int* slot_of;         // shared memory: virtual slot -> routing slot
  const float* w_of;          // shared memory: virtual slot -> routing weight
  __device__ __forceinline__ void operator()(int c, float (&f)[8]) {
    const int vs = c / cps, cc = c - vs * cps;
    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(act + size_t(slot_of[vs]) * act_stride + (cc << 3)));
    const float w = w_of[vs];
    f[0] = bf16lo(v.x) * w; f[1] = bf16hi(v.x) * w; f[2] = bf16lo(v.y) * w; f[3] = bf16hi(v.y) * w;
    f[4] = bf16lo(v.z) * w; f[5] = bf16hi(v.z) * w; f[6] = bf16lo(v.w) * w; f[7] = bf16hi(v.w) * w;
  }
};

// Shared by the single-GPU and the tensor-parallel form of the expert down projection.
template <int WK>
struct SgMoeDownBase {
  static constexpr int kKind = WK;
  static constexpr int kB = 1;
  static constexpr bool kWeightsNeedWait = true;
  static constexpr bool kMultiSlot = true;
  SgWeights W;             // rows: [E_local][N], I columns
  int N, I;
  const __nv_bfloat16* act; int act_stride;   // [tokens*top_k, I]
  SgRouting R;
  int token, ntok, nloc;
  unsigned long long packed;                   // local expert of virtual slot v in byte v

  __device__ void cta_range(const SgPlan& pl, int& q0, int& q1) {
    token = blockIdx.x / pl.grid;
    const int c = blockIdx.x - token * pl.grid;
    q0 = c * pl.qpc; q1 = min(pl.quads, q0 + pl.qpc);
    if (token >= ntok) { token = 0; q0 = q1 = 0; }
  }
  __device__ void load_routing() {
    packed = 0ull; nloc = 0;
    for (int s = 0; s < R.top_k; ++s) {
      const int e = R.topk_idx[token * R.top_k + s] - R.expert_base;
      if (e >= 0 && e < R.experts_local) { packed |= static_cast<unsigned long long>(e) << (8 * nloc); ++nloc; }
    }
  }
  __device__ int nslots() const { return nloc; }
  __device__ int xunits() const { return nloc * (WK == 1 ? I >> 5 : WK == 2 ? I >> 4 : I >> 3); }
  __device__ SgSegSrc seg(const SgPlan&, int sq0, int nq, int g) const {
    const int e = int((packed >> (8 * g)) & 0xffull);
    return W.rows(size_t(e) * N + 4 * size_t(sq0), min(4 * nq, N - 4 * sq0));
  }
  // extra shared memory: int slot_of[8]; float w_of[8]
  __device__ void stage_moe_x(SgSmem& sm) {
    int* slot_of = reinterpret_cast<int*>(sm.extra);
    float* w_of = reinterpret_cast<float*>(sm.extra + 32);
    if (threadIdx.x == 0) {
      int n = 0;
      for (int s = 0; s < R.top_k; ++s) {
        const int e = R.topk_idx[token * R.top_k + s] - R.expert_base;
        if (e >= 0 && e < R.experts_local) { slot_of[n] = s; w_of[n] = R.topk_w[token * R.top_k + s]; ++n; }
      }
    }
    sg_consumer_sync();
    if (nloc > 0) {
      XLoadMoeAct ld{act + size_t(token) * R.top_k * act_stride, act_stride, I >> 3, slot_of, w_of};
      if (WK == 1) XStage<WQ4>::stage_part(sm.xs, nloc * I, ld, threadIdx.x, kSgConsumers);
      else if (WK == 2) XStage<WQ8>::stage_part(sm.xs, nloc * I, ld, threadIdx.x, kSgConsumers);
      else XStage<WBf16>::stage_part(sm.xs, nloc * I, ld, threadIdx.x, kSgConsumers);
    }
    sg_consumer_sync();
  }
};

template <int WK, bool OUT_F32>
struct SgMoeDown : SgMoeDownBase<WK> {
  const __nv_bfloat16* residual; int res_stride;
  void* out; int out_stride;
  __device__ void init(bool) { this->load_routing(); }
  __device__ void stage_x(SgSmem& sm, const SgPlan&) { this->stage_moe_x(sm); }
  __device__ void epilogue(int quad, float (&v)[4][1], SgSmem&) {
    const int b = this->token;
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int n = quad * 4 + r;
      if (n < this->N) {
        float o = v[r][0];
        if (residual) o += bf16lo(__ldcg(reinterpret_cast<const uint16_t*>(residual + size_t(b) * res_stride + n)));
        if (OUT_F32) static_cast<float*>(out)[size_t(b) * out_stride + n] = o;
        else static_cast<__nv_bfloat16*>(out)[size_t(b) * out_stride + n] = __float2bfloat16_rn(o);
      }
    }
  }
  __device__ void cta_done(SgSmem&) {}
};

// ------------------------------------------------------------------------------------------------
// Host-side helpers shared by the launchers.
// ------------------------------------------------------------------------------------------------
inline SgWeights sg_weights(int kind, const void* w, const void* sc, const void* bi, int K) {
  SgWeights W;
  W.w = static_cast<const char*>(w);
  W.sc = static_cast<const char*>(sc);
  W.bi = static_cast<const char*>(bi);
  W.units = kind == 1 ? K >> 5 : kind == 2 ? K >> 4 : K >> 3;
  W.srow = kind != 0 ? K >> 5 : 0;        // one bf16 per 64 weights
  return W;
}
inline bool sg_weights_ok(int kind, const void* w, const void* sc, const void* bi, int K) {
  if (kind != 0)
    return K % 64 == 0 && sg_aligned16(w) && sc && bi && (reinterpret_cast<uintptr_t>(sc) & 1u) == 0 &&
           ((reinterpret_cast<uintptr_t>(sc) ^ reinterpret_cast<uintptr_t>(bi)) & 15u) == 0;
  return K % 8 == 0 && sg_aligned16(w);
}
inline int sg_x_bytes(int kind, int K, int B) {
  const size_t one = kind == 1 ? (size_t(K >> 5) * 72 + 15) & ~size_t(15)
                     : kind == 2 ? size_t(K >> 4) * 40 : size_t(K >> 3) * 32;
  return int(one * B);
}

template <class P>
inline int sg_launch(const P& prob, const SgPlan& plan, int grid, int* status, int pdl, cudaStream_t st) {
  if (plan.grid < 1) return -2;
  SgPlan pl = plan;
  pl.drop_stage = sg_debug_drop();
  sg_debug_drop() = -1;
  const size_t smem = sg_smem_bytes(pl, P::kB);
  if (smem > 200 * 1024) return -2;
#define SG_LAUNCH_LW(LW_)                                                                         \
  {                                                                                               \
    auto kern = sg_kernel<P, LW_>;                                                                \
    RB_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem))); \
    return launch(kern, dim3(grid), dim3(kSgThreads), smem, st, pdl != 0, prob, pl, status);      \
  }
  if (pl.LW == 32) SG_LAUNCH_LW(32)
  if (pl.LW == 16) SG_LAUNCH_LW(16)
  if (pl.LW == 8) SG_LAUNCH_LW(8)
#undef SG_LAUNCH_LW
  return -2;
}

}  // namespace rb
