// Launchers of the weight-streaming decode projections (stream_gemv.cuh, stream_problems.cuh) for
// one GPU. Every entry point returns -2 for shapes the streaming kernel does not take (the caller
// then uses the per-row kernels of decode_gemv.cu / decode_moe.cu).
#include "stream_problems.cuh"

namespace rb {

static __device__ int g_sg_status = 0;

// Set by the entry points for the launch they are about to make: scales / biases are fp16.
static thread_local int t_scale_f16 = 0;

static int* sg_status_ptr() {
  static int* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!cached[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_sg_status) != cudaSuccess) { (void)cudaGetLastError(); return nullptr; }
    cached[dev] = static_cast<int*>(p);
  }
  return cached[dev];
}

template <int WK, int B, bool F32>
static int run_dense(const void* w, const void* sc, const void* bi, const void* x, int x_stride,
                     const void* norm_w, float eps, const void* res, int res_stride, void* out,
                     int out_stride, int N, int K, int pdl, cudaStream_t st) {
  SgDense<WK, B, F32> P;
  P.W = sg_weights(WK, w, sc, bi, K);
  P.N = N; P.K = K;
  P.x = static_cast<const __nv_bfloat16*>(x); P.x_stride = x_stride;
  P.norm_w = static_cast<const __nv_bfloat16*>(norm_w); P.eps = eps;
  P.residual = static_cast<const __nv_bfloat16*>(res); P.res_stride = res_stride;
  P.out = out; P.out_stride = out_stride;
  const SgPlan pl = sg_make_plan(WK | (t_scale_f16 << 8), P.W.units, 1, false, (N + 3) / 4, sm_count(), 1 << 20, sg_x_bytes(WK, K, B), 0, B);
  return sg_launch(P, pl, pl.grid, sg_status_ptr(), pdl, st);
}

template <int WK, int B>
static int run_qkv(const void* w, const void* sc, const void* bi, const void* x, int x_stride,
                   const void* norm_w, float eps, const SgRopeArgs& a, int K, int pdl, cudaStream_t st) {
  SgQkvRope<WK, B> P;
  P.W = sg_weights(WK, w, sc, bi, K);
  P.K = K;
  P.x = static_cast<const __nv_bfloat16*>(x); P.x_stride = x_stride;
  P.norm_w = static_cast<const __nv_bfloat16*>(norm_w); P.eps = eps;
  P.a = a;
  const int quads = (a.Hq + 2 * a.Hkv) * (a.HD / 4);
  const SgPlan pl = sg_make_plan(WK | (t_scale_f16 << 8), P.W.units, 1, !a.traditional, quads, sm_count(), a.HD / 4, sg_x_bytes(WK, K, B),
                                 SgQkvRope<WK, B>::extra_bytes(a.HD, B), B);
  return sg_launch(P, pl, pl.grid, sg_status_ptr(), pdl, st);
}

template <int WK, int B>
static int run_gate_up(const void* w, const void* sc, const void* bi, const void* x, int x_stride,
                       const void* norm_w, float eps, void* act, int act_stride, int I, int K, int pdl,
                       cudaStream_t st) {
  SgGateUp<WK, B> P;
  P.W = sg_weights(WK, w, sc, bi, K);
  P.I = I; P.K = K;
  P.x = static_cast<const __nv_bfloat16*>(x); P.x_stride = x_stride;
  P.norm_w = static_cast<const __nv_bfloat16*>(norm_w); P.eps = eps;
  P.act = static_cast<__nv_bfloat16*>(act); P.act_stride = act_stride;
  const SgPlan pl = sg_make_plan(WK | (t_scale_f16 << 8), P.W.units, 1, true, I / 2, sm_count(), 1 << 20, sg_x_bytes(WK, K, B), 0, B);
  return sg_launch(P, pl, pl.grid, sg_status_ptr(), pdl, st);
}

template <int WK>
static int run_moe_gate_up(const void* w, const void* sc, const void* bi, const void* x, int x_stride,
                           const void* norm_w, float eps, const int* idx, void* act, int act_stride,
                           int B, int top_k, int I, int K, int expert_base, int experts_local, int pdl,
                           cudaStream_t st) {
  SgMoeGateUp<WK> P;
  P.W = sg_weights(WK, w, sc, bi, K);
  P.I = I; P.K = K;
  P.x = static_cast<const __nv_bfloat16*>(x); P.x_stride = x_stride;
  P.norm_w = static_cast<const __nv_bfloat16*>(norm_w); P.eps = eps;
  P.act = static_cast<__nv_bfloat16*>(act); P.act_stride = act_stride;
  P.R = SgRouting{idx, nullptr, top_k, expert_base, experts_local};
  P.token = 0; P.ntok = B; P.packed = 0; P.mask = 0;
  const int per_token = sm_count() / B > 0 ? sm_count() / B : 1;
  const int hq = I / 2;
  const SgPlan pl = sg_make_plan(WK | (t_scale_f16 << 8), P.W.units, 1, true, top_k * hq, per_token, hq & -hq, sg_x_bytes(WK, K, 1), 0, 1);
  return sg_launch(P, pl, pl.grid * B, sg_status_ptr(), pdl, st);
}

template <int WK, bool F32>
static int run_moe_down(const void* w, const void* sc, const void* bi, const void* act, int act_stride,
                        const int* idx, const float* tw, const void* res, int res_stride, void* out,
                        int out_stride, int B, int top_k, int N, int I, int expert_base,
                        int experts_local, int pdl, cudaStream_t st) {
  SgMoeDown<WK, F32> P;
  P.W = sg_weights(WK, w, sc, bi, I);
  P.N = N; P.I = I;
  P.act = static_cast<const __nv_bfloat16*>(act); P.act_stride = act_stride;
  P.R = SgRouting{idx, tw, top_k, expert_base, experts_local};
  P.token = 0; P.ntok = B; P.nloc = 0; P.packed = 0;
  P.residual = static_cast<const __nv_bfloat16*>(res); P.res_stride = res_stride;
  P.out = out; P.out_stride = out_stride;
  const int per_token = sm_count() / B > 0 ? sm_count() / B : 1;
  const SgPlan pl = sg_make_plan(WK | (t_scale_f16 << 8), P.W.units, top_k, false, (N + 3) / 4, per_token, 1 << 20,
                                 sg_x_bytes(WK, top_k * I, 1), 64, 1);
  return sg_launch(P, pl, pl.grid * B, sg_status_ptr(), pdl, st);
}

}  // namespace rb

using namespace rb;
RB_BOUNDS_REGISTER("decode_stream.cu")


#define SG_DISPATCH_B(B_, ...)                       \
  switch (B_) {                                      \
    case 1: { constexpr int kB = 1; __VA_ARGS__; }   \
    case 2: { constexpr int kB = 2; __VA_ARGS__; }   \
    case 3: { constexpr int kB = 3; __VA_ARGS__; }   \
    case 4: { constexpr int kB = 4; __VA_ARGS__; }   \
    default: return -2;                              \
  }

// 0, or the code of a bounded wait that expired in a streaming kernel since the last call.
extern "C" int rmlx_sg_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_sg_status, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_sg_status, &zero, sizeof(int));
  return v;
}

// Test hook for the bounded-wait path: block 0 of the NEXT streaming launch never sends stage
// `stage`; its consumers' wait expires, the block aborts cleanly and rmlx_sg_status() reports it.
extern "C" void rmlx_sg_debug_drop_stage(int stage) { sg_debug_drop() = stage; }

// Same contract as rmlx_rms_gemv (decode_gemv.cu).
extern "C" int rmlx_sg_rms_gemv(int w_kind, const void* w, const void* scales, const void* biases,
                                const void* x, int x_stride, const void* norm_w, float eps,
                                const void* residual, int res_stride, void* out, int out_stride,
                                int out_f32, int B, int N, int K, int pdl, cudaStream_t st) {
  t_scale_f16 = (w_kind >> 8) & 1;   // bit 8: fp16 scales and biases
  w_kind &= 0xff;
  if (B < 1 || N < 1 || w_kind < 0 || w_kind > 2 || !sg_weights_ok(w_kind, w, scales, biases, K))
    return -2;
#define SG_ARGS w, scales, biases, x, x_stride, norm_w, eps, residual, res_stride, out, out_stride, N, K, pdl, st
#define SG_KIND(KIND_)                                                                  \
  if (w_kind == KIND_) {                                                                \
    if (out_f32) { SG_DISPATCH_B(B, return (run_dense<KIND_, kB, true>(SG_ARGS))) }     \
    else { SG_DISPATCH_B(B, return (run_dense<KIND_, kB, false>(SG_ARGS))) }            \
  }
  SG_KIND(0) SG_KIND(1) SG_KIND(2)
#undef SG_KIND
#undef SG_ARGS
  return -2;
}

// Same contract as rmlx_rms_qkv_rope (decode_qkv_rope.cu); head_dim must be a multiple of 4.
extern "C" int rmlx_sg_rms_qkv_rope(int w_kind, const void* w, const void* scales, const void* biases,
                                    const void* x, int x_stride, const void* norm_w, float eps,
                                    void* q_out, void* k_cache, void* v_cache, const int* block_table,
                                    const int* positions, const int* row_seq, const float* cos_t,
                                    const float* sin_t, int B, int K, int Hq, int Hkv, int HD,
                                    int max_blocks, int page, int traditional, int pdl,
                                    cudaStream_t st) {
  t_scale_f16 = (w_kind >> 8) & 1;   // bit 8: fp16 scales and biases
  w_kind &= 0xff;
  if (B < 1 || HD % 4 || Hq < 1 || Hkv < 1 || w_kind < 0 || w_kind > 2 ||
      !sg_weights_ok(w_kind, w, scales, biases, K))
    return -2;
  SgRopeArgs a{static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache),
               static_cast<__nv_bfloat16*>(v_cache), block_table, positions, row_seq, cos_t, sin_t,
               Hq, Hkv, HD, max_blocks, page, traditional};
  if (w_kind == 1) { SG_DISPATCH_B(B, return (run_qkv<1, kB>(w, scales, biases, x, x_stride, norm_w, eps, a, K, pdl, st))) }
  else if (w_kind == 2) { SG_DISPATCH_B(B, return (run_qkv<2, kB>(w, scales, biases, x, x_stride, norm_w, eps, a, K, pdl, st))) }
  else { SG_DISPATCH_B(B, return (run_qkv<0, kB>(w, scales, biases, x, x_stride, norm_w, eps, a, K, pdl, st))) }
  return -2;
}

// Same contract as rmlx_rms_gate_up_swiglu; I must be even.
extern "C" int rmlx_sg_gate_up(int w_kind, const void* w, const void* scales, const void* biases,
                               const void* x, int x_stride, const void* norm_w, float eps, void* act,
                               int act_stride, int B, int I, int K, int pdl, cudaStream_t st) {
  t_scale_f16 = (w_kind >> 8) & 1;   // bit 8: fp16 scales and biases
  w_kind &= 0xff;
  if (B < 1 || I < 2 || I % 2 || w_kind < 0 || w_kind > 2 || !sg_weights_ok(w_kind, w, scales, biases, K))
    return -2;
  if (w_kind == 1) { SG_DISPATCH_B(B, return (run_gate_up<1, kB>(w, scales, biases, x, x_stride, norm_w, eps, act, act_stride, I, K, pdl, st))) }
  else if (w_kind == 2) { SG_DISPATCH_B(B, return (run_gate_up<2, kB>(w, scales, biases, x, x_stride, norm_w, eps, act, act_stride, I, K, pdl, st))) }
  else { SG_DISPATCH_B(B, return (run_gate_up<0, kB>(w, scales, biases, x, x_stride, norm_w, eps, act, act_stride, I, K, pdl, st))) }
  return -2;
}

// Same contract as rmlx_moe_gate_up; I must be even, at most 256 local experts.
extern "C" int rmlx_sg_moe_gate_up(int w_kind, const void* w, const void* scales, const void* biases,
                                   const void* x, int x_stride, const void* norm_w, float eps,
                                   const int* topk_idx, void* act, int act_stride, int B, int top_k,
                                   int I, int K, int expert_base, int experts_local, int pdl,
                                   cudaStream_t st) {
  t_scale_f16 = (w_kind >> 8) & 1;   // bit 8: fp16 scales and biases
  w_kind &= 0xff;
  if (B < 1 || top_k < 1 || top_k > kSgMaxTopK || I % 2 || experts_local > 256 || w_kind < 0 ||
      w_kind > 2 || !sg_weights_ok(w_kind, w, scales, biases, K))
    return -2;
#define SG_MGU(KIND_)                                                                                   \
  if (w_kind == KIND_)                                                                                  \
    return run_moe_gate_up<KIND_>(w, scales, biases, x, x_stride, norm_w, eps, topk_idx, act, act_stride, \
                                  B, top_k, I, K, expert_base, experts_local, pdl, st);
  SG_MGU(0) SG_MGU(1) SG_MGU(2)
#undef SG_MGU
  return -2;
}

// Same contract as rmlx_moe_down; at most 256 local experts.
extern "C" int rmlx_sg_moe_down(int w_kind, const void* w, const void* scales, const void* biases,
                                const void* act, int act_stride, const int* topk_idx,
                                const float* topk_w, const void* residual, int res_stride, void* out,
                                int out_stride, int out_f32, int B, int top_k, int N, int I,
                                int expert_base, int experts_local, int pdl, cudaStream_t st) {
  t_scale_f16 = (w_kind >> 8) & 1;   // bit 8: fp16 scales and biases
  w_kind &= 0xff;
  if (B < 1 || top_k < 1 || top_k > kSgMaxTopK || experts_local > 256 || w_kind < 0 || w_kind > 2 ||
      !sg_weights_ok(w_kind, w, scales, biases, I) || (w_kind == 0 && I % 32))
    return -2;
#define SG_DOWN(Q4_, F32_)                                                                         \
  return run_moe_down<Q4_, F32_>(w, scales, biases, act, act_stride, topk_idx, topk_w, residual,  \
                                 res_stride, out, out_stride, B, top_k, N, I, expert_base,       \
                                 experts_local, pdl, st)
  if (w_kind == 1) { if (out_f32) SG_DOWN(1, true); else SG_DOWN(1, false); }
  else if (w_kind == 2) { if (out_f32) SG_DOWN(2, true); else SG_DOWN(2, false); }
  else { if (out_f32) SG_DOWN(0, true); else SG_DOWN(0, false); }
#undef SG_DOWN
  return -2;
}

// The plan the streaming kernels would run a projection with (host arithmetic only: no launch, no
// device needed), for tests of the planner and for tools. `op`: 0 dense mat-vec of N rows, 1 gate/up
// with SwiGLU (N = intermediate size: quads are two row pairs), 2 expert down projection (rows
// chained over `top_k` routed slots of K weights each). `ctas`: blocks to spread over (0: the
// device's SM count). out[0..15] = LW, qpt, TR, SQ, QS, units, spl, KP, nseg, seg_rows, stage_bytes,
// ns, qpc, grid, shared memory of a block, supported (grid > 0 and the block fits the launch helper's bound).
extern "C" int rmlx_sg_plan_query(int w_kind, int op, int B, int N, int K, int top_k, int ctas, int* out) {
  if (w_kind < 0 || w_kind > 2 || op < 0 || op > 2 || B < 1 || N < 1 || K < 8 || !out) return -2;
  const int units = w_kind == 1 ? K >> 5 : w_kind == 2 ? K >> 4 : K >> 3;
  if (ctas <= 0) ctas = sm_count();
  SgPlan p;
  if (op == 0) {
    p = sg_make_plan(w_kind, units, 1, false, (N + 3) / 4, ctas, 1 << 20, sg_x_bytes(w_kind, K, B), 0, B);
  } else if (op == 1) {
    p = sg_make_plan(w_kind, units, 1, true, N / 2, ctas, 1 << 20, sg_x_bytes(w_kind, K, B), 0, B);
  } else {
    if (top_k < 1 || top_k > kSgMaxTopK) return -2;
    const int per_token = ctas / B > 0 ? ctas / B : 1;            // as the launcher: the blocks are shared out over the tokens
    p = sg_make_plan(w_kind, units, top_k, false, (N + 3) / 4, per_token, 1 << 20, sg_x_bytes(w_kind, K * top_k, 1), 64, 1);
  }
  const size_t smem = p.grid > 0 ? sg_smem_bytes(p, op == 2 ? 1 : B) : 0;
  const int v[16] = {p.LW, p.qpt, p.TR, p.SQ, p.QS, p.units, p.spl, p.KP, p.nseg, p.seg_rows, p.stage_bytes,
                     p.ns, p.qpc, p.grid, int(smem), p.grid > 0 && smem <= 200 * 1024 ? 1 : 0};   // the launch helper's own bound
  for (int i = 0; i < 16; ++i) out[i] = v[i];
  return 0;
}
