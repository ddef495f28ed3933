// 8-bit paged KV cache: RoPE + quantising append, and page expansion.
//
// Format (per layer): data uint8 [blocks, Hkv, 16, HD]; sb bf16 [blocks, Hkv, 16, HD/64, 2]
// holding (scale, bias) per token and group of 64 along the head dimension, x = q * scale + bias
// with q in 0..255: the affine group format of the reference's QuantizedKvCache
// (crates/rmlx-nn/src/attention.rs:4438-4680, bits = 8, group 64), which the reference keeps on
// the host and re-quantises on every append; here a new token's rows are quantised once, on the
// device, inside the kernel that rotates them, and the attention kernel (flash_decode.cu) expands
// pages in shared memory. Half the cache bytes per token at decode.
//
//   rope_kv_write_q8    merged QKV rows -> rotated Q (bf16), rotated K and V quantised into pages
//   kv_dequant_pages    the pages of one sequence -> contiguous bf16 pages (prompt attention over
//                       an 8-bit cache, tests)
#include "../common/ptx.cuh"
#include "../common/launch.cuh"

namespace rb {

constexpr int kKq8Warps = 4;

template <int J>   // J = HD / 32 values per lane: lane l owns elements l + 32 j
__global__ void __launch_bounds__(kKq8Warps * 32)
rope_kv_write_q8_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                        uint8_t* __restrict__ k_q, __nv_bfloat16* __restrict__ k_sb,
                        uint8_t* __restrict__ v_q, __nv_bfloat16* __restrict__ v_sb,
                        const int* __restrict__ block_table, const int* __restrict__ positions,
                        const int* __restrict__ token_seq, const float* __restrict__ cos_t,
                        const float* __restrict__ sin_t, int Hq, int Hkv, int max_blocks, int page,
                        int traditional) {
  constexpr int HD = J * 32, G64 = HD / 64, half = HD / 2;
  const int tkn = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  pdl_wait();
  const int pos = positions[tkn];
  const int H = Hq + 2 * Hkv;
  for (int head = blockIdx.y * kKq8Warps + warp; head < H; head += gridDim.y * kKq8Warps) {
    const __nv_bfloat16* src = qkv + (size_t(tkn) * H + head) * HD;
    float x[J];
#pragma unroll
    for (int j = 0; j < J; ++j) x[j] = __bfloat162float(src[lane + 32 * j]);
    if (head < Hq + Hkv) {                      // rotate Q and K
      if (!traditional) {
#pragma unroll
        for (int j = 0; j < J / 2; ++j) {
          const int i = lane + 32 * j;
          const float c = cos_t[size_t(pos) * half + i], s = sin_t[size_t(pos) * half + i];
          const float a = x[j], b = x[j + J / 2];
          x[j] = a * c - b * s;
          x[j + J / 2] = b * c + a * s;
        }
      } else {
#pragma unroll
        for (int j = 0; j < J; ++j) {
          const int e = lane + 32 * j, i = e >> 1;
          const float c = cos_t[size_t(pos) * half + i], s = sin_t[size_t(pos) * half + i];
          const float other = __shfl_xor_sync(0xffffffffu, x[j], 1);
          x[j] = (e & 1) ? x[j] * c + other * s : x[j] * c - other * s;
        }
      }
    }
    if (head < Hq) {
      __nv_bfloat16* dst = q_out + (size_t(tkn) * Hq + head) * HD;
#pragma unroll
      for (int j = 0; j < J; ++j) dst[lane + 32 * j] = __float2bfloat16_rn(x[j]);
      continue;
    }
    if (!RB_BOUNDS(pos / page, max_blocks)) continue;
    const int seq = token_seq ? token_seq[tkn] : tkn;
    const int blk = block_table[size_t(seq) * max_blocks + pos / page];
    const bool is_k = head < Hq + Hkv;
    const int kvh = is_k ? head - Hq : head - Hq - Hkv;
    const size_t row = (size_t(blk) * Hkv + kvh) * page + pos % page;
    uint8_t* dq = (is_k ? k_q : v_q) + row * HD;
    __nv_bfloat16* dsb = (is_k ? k_sb : v_sb) + row * G64 * 2;
#pragma unroll
    for (int g = 0; g < G64; ++g) {
      float mn = fminf(x[2 * g], x[2 * g + 1]), mx = fmaxf(x[2 * g], x[2 * g + 1]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      }
      // bias: the minimum rounded DOWN to bf16; scale: (max - stored bias) / 255 rounded UP to
      // bf16, so neither end of the range clips; the codes are computed against the stored pair
      const uint32_t mnb = __float_as_uint(mn);
      const float bi = __uint_as_float(mn >= 0.f ? (mnb & 0xFFFF0000u) : ((mnb + 0xFFFFu) & 0xFFFF0000u));
      const __nv_bfloat16 bb16 = __float2bfloat16_rn(bi);     // exact: bi is a bf16 value
      float span = fmaxf(mx - bi, 0.f) / 255.f;
      if (!(span > 0.f)) span = 1.f;
      const float sc = __uint_as_float((__float_as_uint(span) + 0xFFFFu) & 0xFFFF0000u);
      const __nv_bfloat16 sb16 = __float2bfloat16_rn(sc);     // exact: sc is a bf16 value
      const float inv = 1.f / sc;
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        const float q = rintf((x[2 * g + jj] - bi) * inv);
        dq[lane + 32 * (2 * g + jj)] = static_cast<uint8_t>(fminf(fmaxf(q, 0.f), 255.f));
      }
      if (lane == 0) { dsb[2 * g] = sb16; dsb[2 * g + 1] = bb16; }
    }
  }
}

// out [n_pages, Hkv, 16, HD] bf16: page i of the output is page table[i] of the cache.
__global__ void __launch_bounds__(256)
kv_dequant_pages_kernel(const uint8_t* __restrict__ q, const __nv_bfloat16* __restrict__ sb,
                        const int* __restrict__ table, __nv_bfloat16* __restrict__ out, int Hkv,
                        int page, int HD) {
  const int G64 = HD / 64;
  const size_t src_page = size_t(table[blockIdx.x]) * Hkv + blockIdx.y;
  const size_t dst_page = size_t(blockIdx.x) * Hkv + blockIdx.y;
  const int n = page * HD;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int r = i / HD, e = i - r * HD;
    const __nv_bfloat16* s = sb + ((src_page * page + r) * G64 + (e >> 6)) * 2;
    const float v = float(q[src_page * n + i]) * __bfloat162float(s[0]) + __bfloat162float(s[1]);
    out[dst_page * n + i] = __float2bfloat16_rn(v);
  }
}

}  // namespace rb

using namespace rb;
RB_BOUNDS_REGISTER("kv_q8.cu")

// Same contract as rmlx_rope_kv_write with the cache in the 8-bit format; head_dim 64, 128 or 256.
extern "C" int rmlx_rope_kv_write_q8(const void* qkv, void* q_out, void* k_q, void* k_sb, void* v_q,
                                     void* v_sb, const int* block_table, const int* positions,
                                     const int* token_seq, const float* cos_t, const float* sin_t,
                                     int T, int Hq, int Hkv, int HD, int max_blocks, int page,
                                     int traditional, int pdl, cudaStream_t st) {
  if (T < 1 || (HD != 64 && HD != 128 && HD != 256)) return -2;
  const int H = Hq + 2 * Hkv;
  const int per = T >= 128 ? 16 : kKq8Warps;       // heads per block: prompts take a strip of heads
  const dim3 grid(T, (H + per - 1) / per);
#define RB_KQ8(J_)                                                                                 \
  return launch(rope_kv_write_q8_kernel<J_>, grid, dim3(kKq8Warps * 32), 0, st, pdl != 0,          \
                static_cast<const __nv_bfloat16*>(qkv), static_cast<__nv_bfloat16*>(q_out),        \
                static_cast<uint8_t*>(k_q), static_cast<__nv_bfloat16*>(k_sb),                     \
                static_cast<uint8_t*>(v_q), static_cast<__nv_bfloat16*>(v_sb), block_table,        \
                positions, token_seq, cos_t, sin_t, Hq, Hkv, max_blocks, page, traditional);
  if (HD == 64) { RB_KQ8(2) }
  if (HD == 128) { RB_KQ8(4) }
  RB_KQ8(8)
#undef RB_KQ8
}

extern "C" int rmlx_kv_dequant_pages(const void* q, const void* sb, const int* table, void* out,
                                     int n_pages, int Hkv, int page, int HD, cudaStream_t st) {
  if (n_pages < 1 || HD % 64) return -2;
  kv_dequant_pages_kernel<<<dim3(n_pages, Hkv), 256, 0, st>>>(
      static_cast<const uint8_t*>(q), static_cast<const __nv_bfloat16*>(sb), table,
      static_cast<__nv_bfloat16*>(out), Hkv, page, HD);
  return static_cast<int>(cudaGetLastError());
}
