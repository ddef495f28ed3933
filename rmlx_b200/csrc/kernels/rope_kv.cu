// RoPE on Q and K plus the paged KV-cache append, one launch for every head of every token.
//
// Input is the merged QKV projection output [T, (Hq + 2*Hkv) * HD]. Q heads are rotated and
// written to q_out; K heads are rotated and written straight into their page slot; V heads are
// copied into theirs. Positions, block tables and the token->sequence map are device buffers, so
// the launch is shape-stable under CUDA graph replay while the cache grows.
//
// Replaces rope_qk(v)_batch_* + kv_cache_copy_batched_* (crates/rmlx-core/src/ops/rope.rs:500-870,
// crates/rmlx-core/src/ops/copy.rs:554) and PagedKvCache::append's host memcpy
// (crates/rmlx-nn/src/paged_kv_cache.rs:413-458).
// Rotation layouts: split-half (pairs i, i+HD/2; default) or traditional (pairs 2i, 2i+1), with
// cos/sin tables [max_pos, HD/2] as in crates/rmlx-core/src/ops/rope.rs:15-60.
#include "../common/ptx.cuh"
#include "../common/launch.cuh"

namespace rb {

__global__ void rope_kv_write_kernel(const __nv_bfloat16* __restrict__ qkv,
                                     __nv_bfloat16* __restrict__ q_out,
                                     __nv_bfloat16* __restrict__ k_cache,
                                     __nv_bfloat16* __restrict__ v_cache,
                                     const int* __restrict__ block_table,
                                     const int* __restrict__ positions,
                                     const int* __restrict__ token_seq,
                                     const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                     int Hq, int Hkv, int HD, int max_blocks, int page,
                                     int traditional) {
  const int tkn = blockIdx.x, i = threadIdx.x;  // i in [0, HD/2)
  const int half = HD >> 1;
  pdl_launch_dependents();   // let the next kernel start its weight prefetch now; its own wait covers our completion
  pdl_wait();
  const int pos = positions[tkn];
  const int ia = traditional ? 2 * i : i, ib = traditional ? 2 * i + 1 : i + half;
  const float c = cos_t[size_t(pos) * half + i], s = sin_t[size_t(pos) * half + i];
  // a block takes every gridDim.y-th head of its token (one head each for decode-sized launches,
  // a strip of heads for prompts, where one block per head would be mostly launch overhead)
  for (int head = blockIdx.y; head < Hq + 2 * Hkv; head += gridDim.y) {
    const __nv_bfloat16* src = qkv + (size_t(tkn) * (Hq + 2 * Hkv) + head) * HD;
    const float a = __bfloat162float(src[ia]), b = __bfloat162float(src[ib]);
    __nv_bfloat16* dst;
    if (head < Hq) {
      dst = q_out + (size_t(tkn) * Hq + head) * HD;
    } else {
      const int seq = token_seq ? token_seq[tkn] : tkn;
      if (!RB_BOUNDS(pos / page, max_blocks)) continue;
      const int blk = block_table[size_t(seq) * max_blocks + pos / page];
      const bool is_k = head < Hq + Hkv;
      const int kvh = is_k ? head - Hq : head - Hq - Hkv;
      dst = (is_k ? k_cache : v_cache) + ((size_t(blk) * Hkv + kvh) * page + pos % page) * HD;
      if (!is_k) { dst[ia] = src[ia]; dst[ib] = src[ib]; continue; }
    }
    dst[ia] = __float2bfloat16_rn(a * c - b * s);
    dst[ib] = __float2bfloat16_rn(b * c + a * s);
  }
}

// Stand-alone RoPE over [T, H, HD] (used by tests and by attention variants that keep their own
// cache layout, e.g. latent attention's decoupled rope key).
__global__ void rope_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                            const int* __restrict__ positions, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, int H, int HD, int traditional,
                            int inverse) {
  const int tkn = blockIdx.x, head = blockIdx.y, i = threadIdx.x;
  const int half = HD >> 1;
  const int pos = positions[tkn];
  const size_t base = (size_t(tkn) * H + head) * HD;
  const int ia = traditional ? 2 * i : i, ib = traditional ? 2 * i + 1 : i + half;
  const float a = __bfloat162float(x[base + ia]), b = __bfloat162float(x[base + ib]);
  const float c = cos_t[size_t(pos) * half + i];
  const float s = inverse ? -sin_t[size_t(pos) * half + i] : sin_t[size_t(pos) * half + i];
  out[base + ia] = __float2bfloat16_rn(a * c - b * s);
  out[base + ib] = __float2bfloat16_rn(b * c + a * s);
}

}  // namespace rb

using namespace rb;
RB_BOUNDS_REGISTER("rope_kv.cu")


extern "C" int rmlx_rope_kv_write(const void* qkv, void* q_out, void* k_cache, void* v_cache,
                                  const int* block_table, const int* positions, const int* token_seq,
                                  const float* cos_t, const float* sin_t, int T, int Hq, int Hkv,
                                  int HD, int max_blocks, int page, int traditional, int pdl,
                                  cudaStream_t st) {
  if (T < 1 || HD % 2 || HD / 2 > 1024) return -2;
  const int H = Hq + 2 * Hkv;
  const int gy = T >= 128 ? (H + 17) / 18 : H;     // prompts: ~18 heads per block
  return launch(rope_kv_write_kernel, dim3(T, gy), dim3(HD / 2), 0, st, pdl != 0,
                static_cast<const __nv_bfloat16*>(qkv), static_cast<__nv_bfloat16*>(q_out),
                static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache),
                block_table, positions, token_seq, cos_t, sin_t, Hq, Hkv, HD, max_blocks, page,
                traditional);
}

extern "C" int rmlx_rope(const void* x, void* out, const int* positions, const float* cos_t,
                         const float* sin_t, int T, int H, int HD, int traditional, int inverse,
                         cudaStream_t st) {
  if (T < 1 || HD % 2 || HD / 2 > 1024) return -2;
  rope_kernel<<<dim3(T, H), HD / 2, 0, st>>>(static_cast<const __nv_bfloat16*>(x),
                                             static_cast<__nv_bfloat16*>(out), positions, cos_t,
                                             sin_t, H, HD, traditional, inverse);
  return static_cast<int>(cudaGetLastError());
}
