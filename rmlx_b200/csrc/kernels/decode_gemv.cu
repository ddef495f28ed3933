// Decode-time dense projections: out[b, n] = residual[b, n] + inv_rms[b] * sum_k W[n, k] * (x[b, k] * g[k])
//
// One kernel covers the three dense decode projections of a transformer layer and the LM head:
//   * RMSNorm + QKV projection            (norm weight given, no residual)
//   * O projection + residual              (no norm, residual given)
//   * final RMSNorm + LM head              (norm weight given, fp32 logits)
//   * RMSNorm + gate/up projection with SwiGLU epilogue, and SwiGLU + down projection + residual
//     for dense feed-forward blocks (see swiglu kernels below).
// RMSNorm is folded in algebraically: the activation is staged as x*g and the accumulated dot
// product is scaled by inv_rms afterwards, so the input is read once.
//
// Counterpart in the reference: fused_rms_gemv_* and gemv_bias_* (crates/rmlx-core/src/ops/fused.rs:1530,
// crates/rmlx-core/src/ops/gemv.rs:488) and fused_swiglu_down_* (fused.rs:967); Q4 rows follow
// affine_qmv_fast_* (crates/rmlx-core/src/ops/quantized.rs:407).
#include "../common/gemv_core.cuh"
#include "../common/launch.cuh"

namespace rb {

constexpr int kRowsPerWarp = 2;

template <class WT, int B, bool OUT_F32>
__global__ void __launch_bounds__(kGemvThreads)
rms_gemv_kernel(Matrix<WT> W, const __nv_bfloat16* __restrict__ x, int x_stride,
                const __nv_bfloat16* __restrict__ norm_w, float eps,
                const __nv_bfloat16* __restrict__ residual, int res_stride, void* __restrict__ out,
                int out_stride, int N) {
  extern __shared__ __align__(16) char smem[];
  __shared__ float red[kGemvWarps];
  __shared__ float inv_rms[B];
  const int K = W.K;
  const size_t bstride = (XStage<WT>::bytes(K) + 15) & ~size_t(15);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // Weights depend neither on the previous kernel nor on the activations: issue the first tile's
  // loads now, so their latency overlaps the wait and the staging below.
  using Row = typename Matrix<WT>::Row;
  int n0 = (blockIdx.x * kGemvWarps + warp) * kRowsPerWarp;
  Row rows[kRowsPerWarp];
  Tile<Row, kRowsPerWarp> t0;
  if (n0 < N) {
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) rows[r] = W.row(min(n0 + r, N - 1));
    load_tile<kRowsPerWarp>(rows, K, 0, t0);
  }
  pdl_launch_dependents();   // let the next kernel start its weight prefetch now; its own wait covers our completion
  pdl_wait();

#pragma unroll
  for (int b = 0; b < B; ++b) {
    const float ssq = XStage<WT>::stage(smem + b * bstride, x + size_t(b) * x_stride, norm_w, K,
                                        red, norm_w != nullptr);
    if (threadIdx.x == 0) inv_rms[b] = norm_w ? rsqrtf(ssq / float(K) + eps) : 1.f;
  }
  __syncthreads();

  for (bool first = true; n0 < N; n0 += gridDim.x * kGemvWarps * kRowsPerWarp, first = false) {
    if (!first) {
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) rows[r] = W.row(min(n0 + r, N - 1));
      load_tile<kRowsPerWarp>(rows, K, 0, t0);
    }
    float acc[kRowsPerWarp][B];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
      for (int b = 0; b < B; ++b) acc[r][b] = 0.f;
    warp_dot<kRowsPerWarp, B, Row>(rows, smem, bstride, K, acc, t0);
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const float v = warp_sum(acc[r][b]);
        if (lane == r * B + b && n0 + r < N) {
          float o = v * inv_rms[b];
          if (residual) o += __bfloat162float(residual[size_t(b) * res_stride + n0 + r]);
          if (OUT_F32) reinterpret_cast<float*>(out)[size_t(b) * out_stride + n0 + r] = o;
          else reinterpret_cast<__nv_bfloat16*>(out)[size_t(b) * out_stride + n0 + r] =
                   __float2bfloat16_rn(o);
        }
      }
  }
  pdl_launch_dependents();
}

// Dense SwiGLU feed-forward, first half: act[b, i] = silu(Wg[i]·xn[b]) * (Wu[i]·xn[b]) where the
// merged weight holds the gate rows [0, I) followed by the up rows [I, 2I).
template <class WT, int B>
__global__ void __launch_bounds__(kGemvThreads)
rms_gate_up_swiglu_kernel(Matrix<WT> W, const __nv_bfloat16* __restrict__ x, int x_stride,
                          const __nv_bfloat16* __restrict__ norm_w, float eps,
                          __nv_bfloat16* __restrict__ act, int act_stride, int I) {
  extern __shared__ __align__(16) char smem[];
  __shared__ float red[kGemvWarps];
  __shared__ float inv_rms[B];
  const int K = W.K;
  const size_t bstride = (XStage<WT>::bytes(K) + 15) & ~size_t(15);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  using Row = typename Matrix<WT>::Row;
  int i = blockIdx.x * kGemvWarps + warp;
  Row rows[2];
  Tile<Row, 2> t0;
  if (i < I) {
    rows[0] = W.row(i); rows[1] = W.row(size_t(I) + i);
    load_tile<2>(rows, K, 0, t0);
  }
  pdl_launch_dependents();   // let the next kernel start its weight prefetch now; its own wait covers our completion
  pdl_wait();
#pragma unroll
  for (int b = 0; b < B; ++b) {
    const float ssq = XStage<WT>::stage(smem + b * bstride, x + size_t(b) * x_stride, norm_w, K,
                                        red, norm_w != nullptr);
    if (threadIdx.x == 0) inv_rms[b] = norm_w ? rsqrtf(ssq / float(K) + eps) : 1.f;
  }
  __syncthreads();
  for (bool first = true; i < I; i += gridDim.x * kGemvWarps, first = false) {
    if (!first) {
      rows[0] = W.row(i); rows[1] = W.row(size_t(I) + i);
      load_tile<2>(rows, K, 0, t0);
    }
    float acc[2][B];
#pragma unroll
    for (int b = 0; b < B; ++b) acc[0][b] = acc[1][b] = 0.f;
    warp_dot<2, B, Row>(rows, smem, bstride, K, acc, t0);
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const float g = warp_sum(acc[0][b]) * inv_rms[b];
      const float u = warp_sum(acc[1][b]) * inv_rms[b];
      if (lane == b) act[size_t(b) * act_stride + i] = __float2bfloat16_rn(g / (1.f + __expf(-g)) * u);
    }
  }
  pdl_launch_dependents();
}

// Dense SwiGLU feed-forward, second half, in the reference's form: the input is the raw merged
// gate_up vector [2I]; silu(gate)*up is computed while staging, then down projection + residual.
template <class WT, int B>
__global__ void __launch_bounds__(kGemvThreads)
swiglu_down_kernel(Matrix<WT> W /*[N, I]*/, const __nv_bfloat16* __restrict__ gate_up,
                   int gu_stride, const __nv_bfloat16* __restrict__ residual, int res_stride,
                   __nv_bfloat16* __restrict__ out, int out_stride, int N) {
  extern __shared__ __align__(16) char smem[];
  const int I = W.K;
  const size_t bstride = (XStage<WT>::bytes(I) + 15) & ~size_t(15);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  using Row = typename Matrix<WT>::Row;
  int n0 = (blockIdx.x * kGemvWarps + warp) * kRowsPerWarp;
  Row rows[kRowsPerWarp];
  Tile<Row, kRowsPerWarp> t0;
  if (n0 < N) {
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) rows[r] = W.row(min(n0 + r, N - 1));
    load_tile<kRowsPerWarp>(rows, I, 0, t0);
  }
  pdl_launch_dependents();   // let the next kernel start its weight prefetch now; its own wait covers our completion
  pdl_wait();
#pragma unroll
  for (int b = 0; b < B; ++b) {
    XLoadSwiglu ld{gate_up + size_t(b) * gu_stride, I};
    XStage<WT>::stage_with(smem + b * bstride, I, ld);
  }
  for (bool first = true; n0 < N; n0 += gridDim.x * kGemvWarps * kRowsPerWarp, first = false) {
    if (!first) {
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) rows[r] = W.row(min(n0 + r, N - 1));
      load_tile<kRowsPerWarp>(rows, I, 0, t0);
    }
    float acc[kRowsPerWarp][B];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
      for (int b = 0; b < B; ++b) acc[r][b] = 0.f;
    warp_dot<kRowsPerWarp, B, Row>(rows, smem, bstride, I, acc, t0);
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const float v = warp_sum(acc[r][b]);
        if (lane == r * B + b && n0 + r < N) {
          float o = v;
          if (residual) o += __bfloat162float(residual[size_t(b) * res_stride + n0 + r]);
          out[size_t(b) * out_stride + n0 + r] = __float2bfloat16_rn(o);
        }
      }
  }
  pdl_launch_dependents();
}

template <class WT>
static Matrix<WT> make_matrix(const void* w, const void* s, const void* b, int K);
template <>
Matrix<WBf16> make_matrix<WBf16>(const void* w, const void*, const void*, int K) {
  return Matrix<WBf16>{static_cast<const __nv_bfloat16*>(w), K};
}
template <>
Matrix<WQ4> make_matrix<WQ4>(const void* w, const void* s, const void* b, int K) {
  return Matrix<WQ4>{static_cast<const uint32_t*>(w), static_cast<const __nv_bfloat16*>(s),
                     static_cast<const __nv_bfloat16*>(b), K};
}

static int grid_for_rows(int rows_total, int rows_per_cta) {
  const int want = (rows_total + rows_per_cta - 1) / rows_per_cta;
  const int cap = sm_count() * 8;
  return want < cap ? (want > 0 ? want : 1) : cap;
}

template <class WT, int B, bool OUT_F32>
static int launch_rms_gemv(const void* w, const void* sc, const void* bi, const void* x,
                           int x_stride, const void* norm_w, float eps, const void* res,
                           int res_stride, void* out, int out_stride, int N, int K, int pdl,
                           cudaStream_t st) {
  const size_t bstride = (XStage<WT>::bytes(K) + 15) & ~size_t(15);
  const size_t smem = bstride * B;
  auto kern = rms_gemv_kernel<WT, B, OUT_F32>;
  RB_CHECK(set_max_smem(kern, smem));
  const int grid = grid_for_rows(N, kGemvWarps * kRowsPerWarp);
  return launch(kern, dim3(grid), dim3(kGemvThreads), smem, st, pdl != 0, make_matrix<WT>(w, sc, bi, K),
                static_cast<const __nv_bfloat16*>(x), x_stride,
                static_cast<const __nv_bfloat16*>(norm_w), eps,
                static_cast<const __nv_bfloat16*>(res), res_stride, out, out_stride, N);
}

template <class WT, int B>
static int launch_gate_up(const void* w, const void* sc, const void* bi, const void* x, int x_stride,
                          const void* norm_w, float eps, void* act, int act_stride, int I, int K,
                          int pdl, cudaStream_t st) {
  const size_t bstride = (XStage<WT>::bytes(K) + 15) & ~size_t(15);
  const size_t smem = bstride * B;
  auto kern = rms_gate_up_swiglu_kernel<WT, B>;
  RB_CHECK(set_max_smem(kern, smem));
  const int grid = grid_for_rows(I, kGemvWarps);
  return launch(kern, dim3(grid), dim3(kGemvThreads), smem, st, pdl != 0, make_matrix<WT>(w, sc, bi, K),
                static_cast<const __nv_bfloat16*>(x), x_stride,
                static_cast<const __nv_bfloat16*>(norm_w), eps, static_cast<__nv_bfloat16*>(act),
                act_stride, I);
}

template <class WT, int B>
static int launch_swiglu_down(const void* w, const void* sc, const void* bi, const void* gu,
                              int gu_stride, const void* res, int res_stride, void* out,
                              int out_stride, int N, int I, int pdl, cudaStream_t st) {
  const size_t bstride = (XStage<WT>::bytes(I) + 15) & ~size_t(15);
  const size_t smem = bstride * B;
  auto kern = swiglu_down_kernel<WT, B>;
  RB_CHECK(set_max_smem(kern, smem));
  const int grid = grid_for_rows(N, kGemvWarps * kRowsPerWarp);
  return launch(kern, dim3(grid), dim3(kGemvThreads), smem, st, pdl != 0, make_matrix<WT>(w, sc, bi, I),
                static_cast<const __nv_bfloat16*>(gu), gu_stride,
                static_cast<const __nv_bfloat16*>(res), res_stride,
                static_cast<__nv_bfloat16*>(out), out_stride, N);
}

}  // namespace rb

using namespace rb;

#define RB_DISPATCH_B(B_, ...)                       \
  switch (B_) {                                      \
    case 1: { constexpr int kB = 1; __VA_ARGS__; }   \
    case 2: { constexpr int kB = 2; __VA_ARGS__; }   \
    case 3: { constexpr int kB = 3; __VA_ARGS__; }   \
    case 4: { constexpr int kB = 4; __VA_ARGS__; }   \
    default: return -2;                              \
  }

// Largest number of activation vectors one launch handles; larger batches are chunked by the
// caller (or go to the tensor-core GEMM).
extern "C" int rmlx_gemv_max_batch() { return 4; }

// w_kind: 0 = bf16 [N,K]; 1 = MLX-affine Q4 (w uint32 [N,K/8], scales/biases bf16 [N,K/64]).
// K must be a multiple of 64 (bf16: of 8). Strides are in elements. out_f32 selects fp32 output.
extern "C" int rmlx_rms_gemv(int w_kind, const void* w, const void* scales, const void* biases,
                             const void* x, int x_stride, const void* norm_w, float eps,
                             const void* residual, int res_stride, void* out, int out_stride,
                             int out_f32, int B, int N, int K, int pdl, cudaStream_t st) {
  if (K % 8 || (w_kind == 1 && K % 64) || B < 1 || N < 1) return -2;
  if (w_kind == 0) {
    if (out_f32) { RB_DISPATCH_B(B, return (launch_rms_gemv<WBf16, kB, true>(w, scales, biases, x, x_stride, norm_w, eps, residual, res_stride, out, out_stride, N, K, pdl, st))) }
    else { RB_DISPATCH_B(B, return (launch_rms_gemv<WBf16, kB, false>(w, scales, biases, x, x_stride, norm_w, eps, residual, res_stride, out, out_stride, N, K, pdl, st))) }
  } else if (w_kind == 1) {
    if (out_f32) { RB_DISPATCH_B(B, return (launch_rms_gemv<WQ4, kB, true>(w, scales, biases, x, x_stride, norm_w, eps, residual, res_stride, out, out_stride, N, K, pdl, st))) }
    else { RB_DISPATCH_B(B, return (launch_rms_gemv<WQ4, kB, false>(w, scales, biases, x, x_stride, norm_w, eps, residual, res_stride, out, out_stride, N, K, pdl, st))) }
  }
  return -2;
}

extern "C" int rmlx_rms_gate_up_swiglu(int w_kind, const void* w, const void* scales,
                                       const void* biases, const void* x, int x_stride,
                                       const void* norm_w, float eps, void* act, int act_stride,
                                       int B, int I, int K, int pdl, cudaStream_t st) {
  if (K % 8 || (w_kind == 1 && K % 64) || B < 1 || I < 1) return -2;
  if (w_kind == 0) { RB_DISPATCH_B(B, return (launch_gate_up<WBf16, kB>(w, scales, biases, x, x_stride, norm_w, eps, act, act_stride, I, K, pdl, st))) }
  else if (w_kind == 1) { RB_DISPATCH_B(B, return (launch_gate_up<WQ4, kB>(w, scales, biases, x, x_stride, norm_w, eps, act, act_stride, I, K, pdl, st))) }
  return -2;
}

extern "C" int rmlx_swiglu_down(int w_kind, const void* w, const void* scales, const void* biases,
                                const void* gate_up, int gu_stride, const void* residual,
                                int res_stride, void* out, int out_stride, int B, int N, int I,
                                int pdl, cudaStream_t st) {
  if (I % 8 || (w_kind == 1 && I % 64) || B < 1 || N < 1) return -2;
  if (w_kind == 0) { RB_DISPATCH_B(B, return (launch_swiglu_down<WBf16, kB>(w, scales, biases, gate_up, gu_stride, residual, res_stride, out, out_stride, N, I, pdl, st))) }
  else if (w_kind == 1) { RB_DISPATCH_B(B, return (launch_swiglu_down<WQ4, kB>(w, scales, biases, gate_up, gu_stride, residual, res_stride, out, out_stride, N, I, pdl, st))) }
  return -2;
}
