// Row movement around the grouped expert GEMMs (many tokens): scatter token rows into
// expert-sorted order at offsets claimed with per-expert cursors, and the routing-weighted
// combine of the expert outputs back into token order with the residual.
//
// Replaces index_gather_* / scatter_weighted_add_* (crates/rmlx-core/src/ops/moe_kernels.rs:46-180)
// and moe_permute_tokens / moe_combine (crates/rmlx-distributed/src/moe_kernels.rs:93,
// crates/rmlx-distributed/src/moe_exchange.rs:2362). The combine reads each token's k rows in slot
// order, so the result does not depend on the order in which rows were claimed.
#include "../common/ptx.cuh"
#include "../common/launch.cuh"

namespace rb {

// One warp per (token, slot) pair. cursors[E] must be zero on entry.
__global__ void __launch_bounds__(256)
moe_scatter_rows_kernel(const __nv_bfloat16* __restrict__ x, int x_stride,
                        const int* __restrict__ topk_idx, const int* __restrict__ offsets,
                        int* __restrict__ cursors, __nv_bfloat16* __restrict__ xs,
                        int* __restrict__ row_of_pair, int pairs, int top_k, int D) {
  const int p = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (p >= pairs) return;
  int pos = 0;
  if (lane == 0) {
    const int e = topk_idx[p];
    pos = offsets[e] + atomicAdd(cursors + e, 1);
    row_of_pair[p] = pos;
  }
  pos = __shfl_sync(0xffffffffu, pos, 0);
  const uint4* src = reinterpret_cast<const uint4*>(x + size_t(p / top_k) * x_stride);
  uint4* dst = reinterpret_cast<uint4*>(xs + size_t(pos) * D);
  for (int i = lane; i < D / 8; i += 32) dst[i] = src[i];
}

// out[t] = residual[t] + sum_s w[t,s] * y[row_of_pair[t*k+s]]
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ row_of_pair,
                   const float* __restrict__ topk_w, const __nv_bfloat16* __restrict__ residual,
                   int res_stride, __nv_bfloat16* __restrict__ out, int out_stride, int top_k, int D) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < D / 8; c += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (residual) {
      const uint4 r = *reinterpret_cast<const uint4*>(residual + size_t(t) * res_stride + c * 8);
      acc[0] = bf16lo(r.x); acc[1] = bf16hi(r.x); acc[2] = bf16lo(r.y); acc[3] = bf16hi(r.y);
      acc[4] = bf16lo(r.z); acc[5] = bf16hi(r.z); acc[6] = bf16lo(r.w); acc[7] = bf16hi(r.w);
    }
    for (int s = 0; s < top_k; ++s) {
      const int row = row_of_pair[t * top_k + s];
      if (row < 0) continue;       // dropped / non-local pair
      const float w = topk_w[t * top_k + s];
      const uint4 v = *reinterpret_cast<const uint4*>(y + size_t(row) * D + c * 8);
      acc[0] = fmaf(w, bf16lo(v.x), acc[0]); acc[1] = fmaf(w, bf16hi(v.x), acc[1]);
      acc[2] = fmaf(w, bf16lo(v.y), acc[2]); acc[3] = fmaf(w, bf16hi(v.y), acc[3]);
      acc[4] = fmaf(w, bf16lo(v.z), acc[4]); acc[5] = fmaf(w, bf16hi(v.z), acc[5]);
      acc[6] = fmaf(w, bf16lo(v.w), acc[6]); acc[7] = fmaf(w, bf16hi(v.w), acc[7]);
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + size_t(t) * out_stride + c * 8) = o;
  }
}

}  // namespace rb

using namespace rb;

extern "C" int rmlx_moe_scatter_rows(const void* x, int x_stride, const int* topk_idx,
                                     const int* offsets, int* cursors, void* xs, int* row_of_pair,
                                     int T, int top_k, int D, int E, cudaStream_t st) {
  if (T < 1 || D % 8) return -2;
  RB_CHECK(cudaMemsetAsync(cursors, 0, sizeof(int) * E, st));
  const int pairs = T * top_k;
  moe_scatter_rows_kernel<<<(pairs + 7) / 8, 256, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), x_stride, topk_idx, offsets, cursors,
      static_cast<__nv_bfloat16*>(xs), row_of_pair, pairs, top_k, D);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int rmlx_moe_combine(const void* y, const int* row_of_pair, const float* topk_w,
                                const void* residual, int res_stride, void* out, int out_stride,
                                int T, int top_k, int D, cudaStream_t st) {
  if (T < 1 || D % 8) return -2;
  moe_combine_kernel<<<T, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(y), row_of_pair, topk_w,
                                        static_cast<const __nv_bfloat16*>(residual), res_stride,
                                        static_cast<__nv_bfloat16*>(out), out_stride, top_k, D);
  return static_cast<int>(cudaGetLastError());
}
