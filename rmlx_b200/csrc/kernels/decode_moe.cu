// Decode-time mixture-of-experts kernels. Routing, offsets and expert selection never leave the
// device (the reference reads the routing result back to the host on every forward,
// crates/rmlx-nn/src/moe.rs:600-601).
//
//   moe_router        RMSNorm + gate projection + softmax + top-k + renormalise, one launch; the
//                     last block to finish its logits does the selection
//                     (reference: moe_topk_route_f32, crates/rmlx-core/src/ops/topk_route.rs:212)
//   topk_route        the same selection over precomputed logits for many tokens, with the
//                     per-expert histogram; prefix offsets by moe_prefix_offsets
//                     (reference: moe_prefix_scan_u32, topk_route.rs:373)
//   moe_gate_up       per (token, slot): act = silu(Wg[e]·xn) * (Wu[e]·xn), RMSNorm folded in
//   moe_down          per token: out = residual + sum_slot w_slot * Wd[e_slot]·act[slot]
//                     (reference: gather_qmv_fast_*, crates/rmlx-core/src/ops/quantized.rs:9634 and
//                     ExpertGroup::grouped_forward, crates/rmlx-nn/src/expert_group.rs:308)
#include <cstdlib>
#include "../common/gemv_core.cuh"
#include "../common/launch.cuh"

namespace rb {

constexpr int kMaxExperts = 256;
constexpr int kMaxTopK = 8;

// Softmax over E logits held 8-per-lane, then k rounds of warp arg-max (ties: lowest index wins),
// weights renormalised to sum 1. Executed by one full warp for one token.
__device__ __forceinline__ void warp_topk(const float* logits, const float* bias, int E, int k,
                                          int* out_idx, float* out_w, int* counts) {
  const int lane = threadIdx.x & 31;
  float v[kMaxExperts / 32];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < kMaxExperts / 32; ++i) {
    const int e = i * 32 + lane;
    v[i] = (e < E) ? logits[e] + (bias ? bias[e] : 0.f) : -INFINITY;
    m = fmaxf(m, v[i]);
  }
  m = warp_max(m);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxExperts / 32; ++i) {
    v[i] = (i * 32 + lane < E) ? __expf(v[i] - m) : -1.f;  // probabilities are >= 0; -1 = absent
    s += fmaxf(v[i], 0.f);
  }
  s = warp_sum(s);
  const float inv = 1.f / s;
  float sel_w = 0.f;
  int sel_e = 0;
  float wsum = 0.f;
  for (int r = 0; r < k; ++r) {
    float best = -2.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxExperts / 32; ++i) {
      if (v[i] > best) { best = v[i]; best_e = i * 32 + lane; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
#pragma unroll
    for (int i = 0; i < kMaxExperts / 32; ++i)
      if (i * 32 + lane == best_e) v[i] = -1.f;
    const float p = best * inv;
    wsum += p;
    if (lane == r) { sel_w = p; sel_e = best_e; }
  }
  if (lane < k) {
    out_idx[lane] = sel_e;
    out_w[lane] = sel_w / wsum;
    if (counts) atomicAdd(counts + sel_e, 1);
  }
}

template <int B>
__global__ void __launch_bounds__(kGemvThreads)
moe_router_kernel(const __nv_bfloat16* __restrict__ gate_w, const __nv_bfloat16* __restrict__ x,
                  int x_stride, const __nv_bfloat16* __restrict__ norm_w, float eps,
                  const float* __restrict__ expert_bias, float* __restrict__ logits,
                  int* __restrict__ topk_idx, float* __restrict__ topk_w, int* __restrict__ counts,
                  unsigned int* __restrict__ ticket, int E, int K, int k) {
  // One block per expert row; the eight warps split K, so every lane has all of its weight bytes
  // in flight at once (a 4096-wide row is 2 x 16 bytes per lane) and the whole machine takes part.
  extern __shared__ __align__(16) char smem[];
  __shared__ float red[kGemvWarps];
  __shared__ float inv_rms[B];
  __shared__ float part[kGemvWarps][B];
  __shared__ unsigned int last;
  const size_t bstride = (XStage<WBf16>::bytes(K) + 15) & ~size_t(15);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nchunk = K >> 3;
  const int per_warp = (nchunk + kGemvWarps - 1) / kGemvWarps;
  for (int e = blockIdx.x; e < E; e += gridDim.x) {
    const __nv_bfloat16* wrow = gate_w + size_t(e) * K;
    // this warp's slice of the row: chunks [c_lo, c_hi)
    const int c_lo = warp * per_warp, c_hi = min(nchunk, c_lo + per_warp);
    uint4 wv[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = c_lo + u * 32 + lane;
      wv[u] = (c < c_hi) ? ldg_stream(wrow + (size_t(c) << 3)) : make_uint4(0, 0, 0, 0);
    }
    if (e == blockIdx.x) {
      pdl_launch_dependents();   // let the next kernel start its weight prefetch now; its own wait covers our completion
      pdl_wait();
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const float ssq = XStage<WBf16>::stage(smem + b * bstride, x + size_t(b) * x_stride, norm_w,
                                               K, red, norm_w != nullptr);
        if (threadIdx.x == 0) inv_rms[b] = norm_w ? rsqrtf(ssq / float(K) + eps) : 1.f;
      }
      __syncthreads();
    }
    float acc[B];
#pragma unroll
    for (int b = 0; b < B; ++b) acc[b] = 0.f;
    for (int c0 = c_lo; c0 < c_hi; c0 += 128) {
      if (c0 != c_lo) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int c = c0 + u * 32 + lane;
          wv[u] = (c < c_hi) ? ldg_stream(wrow + (size_t(c) << 3)) : make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = c0 + u * 32 + lane;
        if (c < c_hi) {
#pragma unroll
          for (int b = 0; b < B; ++b) {
            const float4* xs = reinterpret_cast<const float4*>(smem + b * bstride);
            const float4 x0 = xs[c], x1 = xs[nchunk + c];
            float a = acc[b];
            a = fmaf(bf16lo(wv[u].x), x0.x, a); a = fmaf(bf16hi(wv[u].x), x0.y, a);
            a = fmaf(bf16lo(wv[u].y), x0.z, a); a = fmaf(bf16hi(wv[u].y), x0.w, a);
            a = fmaf(bf16lo(wv[u].z), x1.x, a); a = fmaf(bf16hi(wv[u].z), x1.y, a);
            a = fmaf(bf16lo(wv[u].w), x1.z, a); a = fmaf(bf16hi(wv[u].w), x1.w, a);
            acc[b] = a;
          }
        }
      }
    }
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const float v = warp_sum(acc[b]);
      if (lane == 0) part[warp][b] = v;
    }
    __syncthreads();
    if (threadIdx.x < B) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < kGemvWarps; ++w) v += part[w][threadIdx.x];
      logits[size_t(threadIdx.x) * E + e] = v * inv_rms[threadIdx.x];
    }
    __syncthreads();
  }
  // Last block to arrive selects the experts for every token of this launch.
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last = (atomicAdd(ticket, 1u) == gridDim.x - 1) ? 1u : 0u;
  __syncthreads();
  if (last) {
    __threadfence();
    for (int b = warp; b < B; b += kGemvWarps)
      warp_topk(logits + size_t(b) * E, expert_bias, E, k, topk_idx + size_t(b) * k,
                topk_w + size_t(b) * k, counts);
    if (threadIdx.x == 0) *ticket = 0u;  // ready for the next launch (graph replay included)
  }
  pdl_launch_dependents();
}

__global__ void __launch_bounds__(256)
topk_route_kernel(const float* __restrict__ logits, const float* __restrict__ expert_bias,
                  int* __restrict__ topk_idx, float* __restrict__ topk_w, int* __restrict__ counts,
                  int T, int E, int k) {
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t < T)
    warp_topk(logits + size_t(t) * E, expert_bias, E, k, topk_idx + size_t(t) * k,
              topk_w + size_t(t) * k, counts);
}

// offsets[e] = sum_{j<e} counts[j], offsets[E] = total. One warp.
__global__ void moe_prefix_offsets_kernel(const int* __restrict__ counts, int* __restrict__ offsets,
                                          int E) {
  const int lane = threadIdx.x;
  int carry = 0;
  for (int base = 0; base < E; base += 32) {
    const int e = base + lane;
    const int c = (e < E) ? counts[e] : 0;
    int inc = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += n;
    }
    if (e < E) offsets[e] = carry + inc - c;
    carry += __shfl_sync(0xffffffffu, inc, 31);
  }
  if (lane == 0) offsets[E] = carry;
}

// Stacked expert matrices [E, rows, K].
template <class WT>
struct ExpertMatrix;
template <>
struct ExpertMatrix<WBf16> {
  using Row = RowBf16;
  const __nv_bfloat16* w;
  int rows, K;
  __device__ Row row(int e, size_t n) const { return Row{w + (size_t(e) * rows + n) * size_t(K)}; }
};
template <>
struct ExpertMatrix<WQ4> {
  using Row = RowQ4;
  const uint32_t* w;
  const __nv_bfloat16* scales;
  const __nv_bfloat16* biases;
  int rows, K;
  __device__ Row row(int e, size_t n) const {
    const size_t r = size_t(e) * rows + n;
    return Row{w + r * size_t(K >> 3), scales + r * size_t(K >> 6), biases + r * size_t(K >> 6)};
  }
};

constexpr int kRowsPerWarpDown = 2;
constexpr int kGuPairsPerWarp = 2;  // (gate, up) row pairs in flight per warp

// grid = (row blocks, token*slot pairs). `i_begin`/`i_count` select a slice of the intermediate
// dimension (tensor-parallel shards own a slice of every expert).
template <class WT>
__global__ void __launch_bounds__(kGemvThreads, 2)
moe_gate_up_kernel(ExpertMatrix<WT> W /*rows = 2*I_full: gate then up*/,
                   const __nv_bfloat16* __restrict__ x, int x_stride,
                   const __nv_bfloat16* __restrict__ norm_w, float eps,
                   const int* __restrict__ topk_idx, __nv_bfloat16* __restrict__ act,
                   int act_stride, int I, int top_k, int expert_base, int experts_local) {
  extern __shared__ __align__(16) char smem[];
  __shared__ float red[kGemvWarps];
  __shared__ float inv_rms_s;
  const int K = W.K;
  const int pair = blockIdx.y, b = pair / top_k;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();   // let the next kernel start its weight prefetch now; its own wait covers our completion
  pdl_wait();
  const int e = topk_idx[pair] - expert_base;
  if (e < 0 || e >= experts_local) return;  // expert lives on another rank
  using Row = typename ExpertMatrix<WT>::Row;
  constexpr int R = 2 * kGuPairsPerWarp;
  int i0 = (blockIdx.x * kGemvWarps + warp) * kGuPairsPerWarp;
  Row rows[R];
  Tile<Row, R> t0;
  auto set_rows = [&](int base) {
#pragma unroll
    for (int j = 0; j < kGuPairsPerWarp; ++j) {
      const int i = min(base + j, I - 1);
      rows[2 * j] = W.row(e, i);
      rows[2 * j + 1] = W.row(e, size_t(I) + i);
    }
  };
  if (i0 < I) { set_rows(i0); load_tile<R>(rows, K, 0, t0); }  // in flight during the staging
  const float ssq = XStage<WT>::stage(smem, x + size_t(b) * x_stride, norm_w, K, red,
                                      norm_w != nullptr);
  if (threadIdx.x == 0) inv_rms_s = norm_w ? rsqrtf(ssq / float(K) + eps) : 1.f;
  __syncthreads();
  const float inv_rms = inv_rms_s;
  for (bool first = true; i0 < I; i0 += gridDim.x * kGemvWarps * kGuPairsPerWarp, first = false) {
    if (!first) { set_rows(i0); load_tile<R>(rows, K, 0, t0); }
    float acc[R][1];
#pragma unroll
    for (int j = 0; j < R; ++j) acc[j][0] = 0.f;
    warp_dot<R, 1, Row>(rows, smem, 0, K, acc, t0);
#pragma unroll
    for (int j = 0; j < kGuPairsPerWarp; ++j) {
      const float g = warp_sum(acc[2 * j][0]) * inv_rms;
      const float u = warp_sum(acc[2 * j + 1][0]) * inv_rms;
      if (lane == j && i0 + j < I)
        act[size_t(pair) * act_stride + i0 + j] = __float2bfloat16_rn(g / (1.f + __expf(-g)) * u);
    }
  }
  pdl_launch_dependents();
}

// grid = (row blocks, tokens). Stages the token's top_k activation vectors, then every output row
// accumulates over the slots with the routing weight applied per slot. Slots whose expert is not
// local contribute nothing (the cross-rank sum happens in the caller's all-reduce).
template <class WT, bool OUT_F32>
__global__ void __launch_bounds__(kGemvThreads, 2)     // two blocks per SM: keeps more weight loads in flight
moe_down_kernel(ExpertMatrix<WT> W /*rows = N, K = I*/, const __nv_bfloat16* __restrict__ act,
                int act_stride, const int* __restrict__ topk_idx, const float* __restrict__ topk_w,
                const __nv_bfloat16* __restrict__ residual, int res_stride, void* __restrict__ out,
                int out_stride, int N, int top_k, int expert_base, int experts_local) {
  extern __shared__ __align__(16) char smem[];
  __shared__ int s_e[kMaxTopK];
  __shared__ float s_w[kMaxTopK];
  const int I = W.K;
  const size_t bstride = (XStage<WT>::bytes(I) + 15) & ~size_t(15);
  const int b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();   // let the next kernel start its weight prefetch now; its own wait covers our completion
  pdl_wait();
  if (threadIdx.x < top_k) {
    const int e = topk_idx[b * top_k + threadIdx.x] - expert_base;
    const bool local = e >= 0 && e < experts_local;
    s_e[threadIdx.x] = local ? e : -1;
    s_w[threadIdx.x] = local ? topk_w[b * top_k + threadIdx.x] : 0.f;
  }
  __syncthreads();
  using Row = typename ExpertMatrix<WT>::Row;
  constexpr int R = kRowsPerWarpDown;
  auto next_local = [&](int s) { while (s < top_k && s_e[s] < 0) ++s; return s; };
  int n0 = (blockIdx.x * kGemvWarps + warp) * R;
  const int s_first = next_local(0);
  Row rows[R];
  Tile<Row, R> cur;
  if (n0 < N && s_first < top_k) {  // first slot's weights fly while the activations are staged
#pragma unroll
    for (int r = 0; r < R; ++r) rows[r] = W.row(s_e[s_first], min(n0 + r, N - 1));
    load_tile<R>(rows, I, 0, cur);
  }
  for (int s = 0; s < top_k; ++s) {
    if (s_e[s] >= 0)
      XStage<WT>::stage(smem + s * bstride, act + size_t(b * top_k + s) * act_stride, nullptr, I,
                        nullptr, false);
  }
  __syncthreads();
  const int units = row_units(rows[0], I);
  for (bool first = true; n0 < N; n0 += gridDim.x * kGemvWarps * R, first = false) {
    float tot[R];
#pragma unroll
    for (int r = 0; r < R; ++r) tot[r] = 0.f;
    int s = s_first;
    if (!first && s < top_k) {
#pragma unroll
      for (int r = 0; r < R; ++r) rows[r] = W.row(s_e[s], min(n0 + r, N - 1));
      load_tile<R>(rows, I, 0, cur);
    }
    while (s < top_k) {
      // software pipeline over the slots: the next expert's first tile is requested before the
      // current one is consumed
      const int sn = next_local(s + 1);
      Row rows_n[R];
      Tile<Row, R> nxt;
      if (sn < top_k) {
#pragma unroll
        for (int r = 0; r < R; ++r) rows_n[r] = W.row(s_e[sn], min(n0 + r, N - 1));
        load_tile<R>(rows_n, I, 0, nxt);
      }
      float acc[R][1];
#pragma unroll
      for (int r = 0; r < R; ++r) acc[r][0] = 0.f;
      if (units <= 64) fma_tile<R, 1>(cur, 0, smem + s * bstride, 0, I, acc);
      else warp_dot<R, 1, Row>(rows, smem + s * bstride, 0, I, acc, cur);
      const float w = s_w[s];
#pragma unroll
      for (int r = 0; r < R; ++r) tot[r] = fmaf(w, acc[r][0], tot[r]);
      if (sn < top_k) {
        cur = nxt;
#pragma unroll
        for (int r = 0; r < R; ++r) rows[r] = rows_n[r];
      }
      s = sn;
    }
#pragma unroll
    for (int r = 0; r < kRowsPerWarpDown; ++r) {
      const float v = warp_sum(tot[r]);
      if (lane == r && n0 + r < N) {
        float o = v;
        if (residual) o += __bfloat162float(residual[size_t(b) * res_stride + n0 + r]);
        if (OUT_F32) reinterpret_cast<float*>(out)[size_t(b) * out_stride + n0 + r] = o;
        else reinterpret_cast<__nv_bfloat16*>(out)[size_t(b) * out_stride + n0 + r] =
                 __float2bfloat16_rn(o);
      }
    }
  }
  pdl_launch_dependents();
}

// Slot-parallel form of the expert down projection: warp s of a block takes routing slot s (its own
// expert), stages that slot's activation by itself and multiplies the block's kDownRows output rows;
// the block then adds the weighted partial sums of its warps. All experts' weight loads of a row
// set are in flight at once (the sequential form above walks the slots one after the other, which
// is the better shape only when a row is long enough to keep a warp busy).
constexpr int kDownRows = 4;

template <class WT, bool OUT_F32>
__global__ void __launch_bounds__(kGemvThreads, 2)
moe_down_par_kernel(ExpertMatrix<WT> W /*rows = N, K = I*/, const __nv_bfloat16* __restrict__ act,
                    int act_stride, const int* __restrict__ topk_idx, const float* __restrict__ topk_w,
                    const __nv_bfloat16* __restrict__ residual, int res_stride, void* __restrict__ out,
                    int out_stride, int N, int top_k, int expert_base, int experts_local) {
  extern __shared__ __align__(16) char smem[];
  __shared__ float s_part[kGemvWarps][kDownRows];
  const int I = W.K;
  const size_t bstride = (XStage<WT>::bytes(I) + 15) & ~size_t(15);
  const int b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  using Row = typename ExpertMatrix<WT>::Row;
  pdl_launch_dependents();
  pdl_wait();
  float tot[kDownRows];
#pragma unroll
  for (int r = 0; r < kDownRows; ++r) tot[r] = 0.f;
  const int n0 = blockIdx.x * kDownRows;
  for (int s = warp; s < top_k; s += kGemvWarps) {      // top_k <= 8: one slot per warp
    const int e = topk_idx[b * top_k + s] - expert_base;
    if (e < 0 || e >= experts_local) continue;
    Row rows[kDownRows];
    Tile<Row, kDownRows> t0;
#pragma unroll
    for (int r = 0; r < kDownRows; ++r) rows[r] = W.row(e, min(n0 + r, N - 1));
    load_tile<kDownRows>(rows, I, 0, t0);               // in flight while the activation is staged
    XLoadBf16 ld{act + size_t(b * top_k + s) * act_stride, nullptr, 0.f};
    char* xs = smem + warp * bstride;
    XStage<WT>::stage_warp(xs, I, ld);
    float acc[kDownRows][1];
#pragma unroll
    for (int r = 0; r < kDownRows; ++r) acc[r][0] = 0.f;
    warp_dot<kDownRows, 1, Row>(rows, xs, 0, I, acc, t0);
    const float w = topk_w[b * top_k + s];
#pragma unroll
    for (int r = 0; r < kDownRows; ++r) tot[r] = fmaf(w, acc[r][0], tot[r]);
    __syncwarp();                                       // the staged vector is reused by the next slot
  }
#pragma unroll
  for (int r = 0; r < kDownRows; ++r) {
    const float v = warp_sum(tot[r]);
    if (lane == 0) s_part[warp][r] = v;
  }
  __syncthreads();
  if (threadIdx.x < kDownRows && n0 + threadIdx.x < N) {
    const int r = threadIdx.x;
    float o = 0.f;
#pragma unroll
    for (int w = 0; w < kGemvWarps; ++w) o += s_part[w][r];
    if (residual) o += __bfloat162float(residual[size_t(b) * res_stride + n0 + r]);
    if (OUT_F32) reinterpret_cast<float*>(out)[size_t(b) * out_stride + n0 + r] = o;
    else reinterpret_cast<__nv_bfloat16*>(out)[size_t(b) * out_stride + n0 + r] = __float2bfloat16_rn(o);
  }
}

template <class WT>
static ExpertMatrix<WT> make_expert_matrix(const void* w, const void* s, const void* b, int rows,
                                           int K);
template <>
ExpertMatrix<WBf16> make_expert_matrix<WBf16>(const void* w, const void*, const void*, int rows,
                                              int K) {
  return ExpertMatrix<WBf16>{static_cast<const __nv_bfloat16*>(w), rows, K};
}
template <>
ExpertMatrix<WQ4> make_expert_matrix<WQ4>(const void* w, const void* s, const void* b, int rows,
                                          int K) {
  return ExpertMatrix<WQ4>{static_cast<const uint32_t*>(w), static_cast<const __nv_bfloat16*>(s),
                           static_cast<const __nv_bfloat16*>(b), rows, K};
}

template <class WT>
static int launch_moe_gate_up(const void* w, const void* sc, const void* bi, const void* x,
                              int x_stride, const void* norm_w, float eps, const int* idx, void* act,
                              int act_stride, int B, int top_k, int I, int K, int expert_base,
                              int experts_local, int pdl, cudaStream_t st) {
  const size_t smem = (XStage<WT>::bytes(K) + 15) & ~size_t(15);
  auto kern = moe_gate_up_kernel<WT>;
  RB_CHECK(set_max_smem(kern, smem));
  int gx = (I + kGemvWarps * kGuPairsPerWarp - 1) / (kGemvWarps * kGuPairsPerWarp);
  if (gx < 1) gx = 1;
  return launch(kern, dim3(gx, B * top_k), dim3(kGemvThreads), smem, st, pdl != 0,
                make_expert_matrix<WT>(w, sc, bi, 2 * I, K), static_cast<const __nv_bfloat16*>(x),
                x_stride, static_cast<const __nv_bfloat16*>(norm_w), eps, idx,
                static_cast<__nv_bfloat16*>(act), act_stride, I, top_k, expert_base, experts_local);
}

// RMLX_MOE_DOWN=par selects the slot-parallel kernel. Default is the sequential-slot kernel: with
// its one-expert-ahead prefetch it measures the same or slightly better at full-width rows.
static bool moe_down_parallel_slots() {
  static const bool v = [] {
    const char* e = getenv("RMLX_MOE_DOWN");
    return e && e[0] == 'p';
  }();
  return v;
}

template <class WT, bool OUT_F32>
static int launch_moe_down(const void* w, const void* sc, const void* bi, const void* act,
                           int act_stride, const int* idx, const float* tw, const void* res,
                           int res_stride, void* out, int out_stride, int B, int top_k, int N, int I,
                           int expert_base, int experts_local, int pdl, cudaStream_t st) {
  if (moe_down_parallel_slots()) {
    const size_t psmem = ((XStage<WT>::bytes(I) + 15) & ~size_t(15)) * kGemvWarps;
    auto pk = moe_down_par_kernel<WT, OUT_F32>;
    RB_CHECK(set_max_smem(pk, psmem));
    return launch(pk, dim3((N + kDownRows - 1) / kDownRows, B), dim3(kGemvThreads), psmem, st, pdl != 0,
                  make_expert_matrix<WT>(w, sc, bi, N, I), static_cast<const __nv_bfloat16*>(act),
                  act_stride, idx, tw, static_cast<const __nv_bfloat16*>(res), res_stride, out,
                  out_stride, N, top_k, expert_base, experts_local);
  }
  const size_t smem = ((XStage<WT>::bytes(I) + 15) & ~size_t(15)) * top_k;
  auto kern = moe_down_kernel<WT, OUT_F32>;
  RB_CHECK(set_max_smem(kern, smem));
  int gx = (N + kGemvWarps * kRowsPerWarpDown - 1) / (kGemvWarps * kRowsPerWarpDown);
  const int cap = sm_count() * 4;
  if (gx > cap) gx = cap;
  return launch(kern, dim3(gx, B), dim3(kGemvThreads), smem, st, pdl != 0,
                make_expert_matrix<WT>(w, sc, bi, N, I), static_cast<const __nv_bfloat16*>(act),
                act_stride, idx, tw, static_cast<const __nv_bfloat16*>(res), res_stride, out,
                out_stride, N, top_k, expert_base, experts_local);
}

}  // namespace rb

using namespace rb;

// Scratch: `logits` fp32 [B, E] and `ticket` one zero-initialised uint32 (left at zero on return).
// counts may be null; when given it must be zeroed by the caller and receives the histogram.
extern "C" int rmlx_moe_router(const void* gate_w, const void* x, int x_stride, const void* norm_w,
                               float eps, const float* expert_bias, float* logits, int* topk_idx,
                               float* topk_w, int* counts, unsigned int* ticket, int B, int E, int K,
                               int k, int pdl, cudaStream_t st) {
  if (E > kMaxExperts || k > kMaxTopK || k > E || K % 8 || B < 1 || B > 4) return -2;
  const size_t bstride = (XStage<WBf16>::bytes(K) + 15) & ~size_t(15);
  int grid = E;
#define RB_ROUTER(BB)                                                                            \
  {                                                                                              \
    auto kern = moe_router_kernel<BB>;                                                           \
    RB_CHECK(set_max_smem(kern, bstride * BB));                                                  \
    return launch(kern, dim3(grid), dim3(kGemvThreads), bstride * BB, st, pdl != 0,              \
                  static_cast<const __nv_bfloat16*>(gate_w), static_cast<const __nv_bfloat16*>(x), \
                  x_stride, static_cast<const __nv_bfloat16*>(norm_w), eps, expert_bias, logits, \
                  topk_idx, topk_w, counts, ticket, E, K, k);                                    \
  }
  switch (B) {
    case 1: RB_ROUTER(1)
    case 2: RB_ROUTER(2)
    case 3: RB_ROUTER(3)
    default: RB_ROUTER(4)
  }
#undef RB_ROUTER
}

extern "C" int rmlx_topk_route(const float* logits, const float* expert_bias, int* topk_idx,
                               float* topk_w, int* counts, int* offsets, int T, int E, int k,
                               cudaStream_t st) {
  if (E > kMaxExperts || k > kMaxTopK || k > E || T < 1) return -2;
  if (counts) RB_CHECK(cudaMemsetAsync(counts, 0, sizeof(int) * E, st));
  topk_route_kernel<<<(T + 7) / 8, 256, 0, st>>>(logits, expert_bias, topk_idx, topk_w, counts, T, E, k);
  if (counts && offsets) moe_prefix_offsets_kernel<<<1, 32, 0, st>>>(counts, offsets, E);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int rmlx_moe_gate_up(int w_kind, const void* w, const void* scales, const void* biases,
                                const void* x, int x_stride, const void* norm_w, float eps,
                                const int* topk_idx, void* act, int act_stride, int B, int top_k,
                                int I, int K, int expert_base, int experts_local, int pdl,
                                cudaStream_t st) {
  if (K % 8 || (w_kind == 1 && K % 64) || B < 1 || top_k < 1 || top_k > kMaxTopK) return -2;
  if (w_kind == 0)
    return launch_moe_gate_up<WBf16>(w, scales, biases, x, x_stride, norm_w, eps, topk_idx, act,
                                     act_stride, B, top_k, I, K, expert_base, experts_local, pdl, st);
  if (w_kind == 1)
    return launch_moe_gate_up<WQ4>(w, scales, biases, x, x_stride, norm_w, eps, topk_idx, act,
                                   act_stride, B, top_k, I, K, expert_base, experts_local, pdl, st);
  return -2;
}

extern "C" int rmlx_moe_down(int w_kind, const void* w, const void* scales, const void* biases,
                             const void* act, int act_stride, const int* topk_idx,
                             const float* topk_w, const void* residual, int res_stride, void* out,
                             int out_stride, int out_f32, int B, int top_k, int N, int I,
                             int expert_base, int experts_local, int pdl, cudaStream_t st) {
  if (I % 8 || (w_kind == 1 && I % 64) || B < 1 || top_k < 1 || top_k > kMaxTopK) return -2;
#define RB_DOWN(WT, F32)                                                                         \
  return launch_moe_down<WT, F32>(w, scales, biases, act, act_stride, topk_idx, topk_w, residual, \
                                  res_stride, out, out_stride, B, top_k, N, I, expert_base,      \
                                  experts_local, pdl, st)
  if (w_kind == 0) { if (out_f32) RB_DOWN(WBf16, true); else RB_DOWN(WBf16, false); }
  if (w_kind == 1) { if (out_f32) RB_DOWN(WQ4, true); else RB_DOWN(WQ4, false); }
#undef RB_DOWN
  return -2;
}
