// Building blocks for the bandwidth-bound decode kernels (matrix-vector products with a handful of
// activation vectors): activation staging into shared memory, and per-warp dot products against
// bf16 rows or MLX-affine 4-bit rows (packed uint32, group 64, bf16 scale and bias: w = s*q + b).
//
// Weights are streamed with 16-byte no-allocate loads, one contiguous 512-byte span per warp
// instruction; activations sit in shared memory in a layout that makes every 16-byte shared load
// conflict-free. Accumulation is fp32 (the 4-bit path accumulates 16 products in fp16 pairs before
// flushing to fp32; its activations are block-scaled per 32 values so that this stays accurate).
#pragma once
#include "ptx.cuh"

namespace rb {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;

struct WBf16 {};  // weights: bf16 [N, K] row-major
struct WQ4 {};    // weights: uint32 [N, K/8], scales/biases bf16 [N, K/64]
struct WQ8 {};    // weights: uint32 [N, K/4] (bytes), scales/biases bf16 [N, K/64]

// One weight row as seen by a dot product.
struct RowBf16 {
  const __nv_bfloat16* w;
};
struct RowQ4 {
  const uint32_t* w;            // K/8 words
  const __nv_bfloat16* scales;  // K/64
  const __nv_bfloat16* biases;  // K/64
};

__device__ __forceinline__ float block_sum_256(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < kGemvWarps) ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// ------------------------------------------------------------------------------------------------
// Activation staging.
//
// bf16-weight path: fp32, "split-chunk" layout. A chunk is 8 consecutive k. Its first four values
// live in float4 unit c, its last four in unit K/8 + c, so the 32 lanes of a warp, which own 32
// consecutive chunks, read 32 consecutive float4 units each time.
//
// 4-bit path: fp16, one 16-byte unit per packed word (8 k). Unit (hg, j) for half-group hg = k/32
// and word j = (k%32)/8 sits at index j*(K/32) + hg. Inside a unit the order is x0,x4,x1,x5,x2,x6,
// x3,x7 so that half2 p pairs with nibbles p and p+4 of the word, which one mask extracts together.
// The nibbles are used as they sit in the word, as fp16 *subnormals* (a nibble at bits 0-3 of a
// half is q * 2^-24, at bits 4-7 it is 16q * 2^-24), so no subtraction of a magic constant is
// needed. To keep the products in fp16's normal range every half-group of 32 activations is scaled
// by a power of two S chosen from its own largest magnitude (the largest scaled value lies in
// [2^14, 2^15)); the halves that meet the bits-4-7 nibbles carry S/16 instead. All of that is
// exact. Beside the units sit, per half-group, the fp32 sum of the (rounded, unscaled) activations
// for the affine bias term and the factor 2^24 / S that brings a partial sum back to real units.
// ------------------------------------------------------------------------------------------------
// Sources of activation values for the staging routines: fill f[0..7] with chunk c (k = 8c .. 8c+7).
struct XLoadBf16 {          // x (global, bf16), optionally times a per-channel weight; tracks sum x^2
  const __nv_bfloat16* x;
  const __nv_bfloat16* scale_w;
  float ssq;
  __device__ __forceinline__ void operator()(int c, float (&f)[8]) {
    // L2 load: in a kernel that runs several projections back to back, x was written by other
    // blocks of the same kernel and must not come from this SM's L1
    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(x + (c << 3)));
    f[0] = bf16lo(v.x); f[1] = bf16hi(v.x); f[2] = bf16lo(v.y); f[3] = bf16hi(v.y);
    f[4] = bf16lo(v.z); f[5] = bf16hi(v.z); f[6] = bf16lo(v.w); f[7] = bf16hi(v.w);
#pragma unroll
    for (int i = 0; i < 8; ++i) ssq += f[i] * f[i];
    if (scale_w) {
      const uint4 s = *reinterpret_cast<const uint4*>(scale_w + (c << 3));
      f[0] *= bf16lo(s.x); f[1] *= bf16hi(s.x); f[2] *= bf16lo(s.y); f[3] *= bf16hi(s.y);
      f[4] *= bf16lo(s.z); f[5] *= bf16hi(s.z); f[6] *= bf16lo(s.w); f[7] *= bf16hi(s.w);
    }
  }
};
struct XLoadSwiglu {        // silu(gate) * up from a [gate | up] row of 2*I bf16
  const __nv_bfloat16* gu;
  int I;
  __device__ __forceinline__ void operator()(int c, float (&f)[8]) {
    const uint4 gv = *reinterpret_cast<const uint4*>(gu + (c << 3));
    const uint4 uv = *reinterpret_cast<const uint4*>(gu + I + (c << 3));
    const float g[8] = {bf16lo(gv.x), bf16hi(gv.x), bf16lo(gv.y), bf16hi(gv.y),
                        bf16lo(gv.z), bf16hi(gv.z), bf16lo(gv.w), bf16hi(gv.w)};
    const float u[8] = {bf16lo(uv.x), bf16hi(uv.x), bf16lo(uv.y), bf16hi(uv.y),
                        bf16lo(uv.z), bf16hi(uv.z), bf16lo(uv.w), bf16hi(uv.w)};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      // stable sigmoid: never exponentiates a positive number
      const float e = __expf(-fabsf(g[i]));
      const float sig = g[i] >= 0.f ? 1.f / (1.f + e) : e / (1.f + e);
      f[i] = g[i] * sig * u[i];
    }
  }
};
// ------------------------------------------------------------------------------------------------
template <class WT>
struct XStage;

template <>
struct XStage<WBf16> {
  static __host__ __device__ size_t bytes(int K) { return size_t(K) * 4; }
  // x: K bf16 (global), scale_w: K bf16 or nullptr. Returns sum of squares of x (block-wide).
  // Stage K values produced chunk by chunk by ``load``. Ends with a block barrier.
  template <class F>
  static __device__ void stage_with(char* smem, int K, F& load) {
    stage_part(smem, K, load, threadIdx.x, kGemvThreads);
    __syncthreads();
  }
  // One warp stages a whole vector by itself (ends with a warp barrier): lets the warps of a block
  // stage different vectors at the same time.
  template <class F>
  static __device__ void stage_warp(char* smem, int K, F& load) {
    stage_part(smem, K, load, threadIdx.x & 31, 32);
    __syncwarp();
  }
  template <class F>
  static __device__ void stage_part(char* smem, int K, F& load, int t, int nt) {
    float4* xs = reinterpret_cast<float4*>(smem);
    const int nchunk = K >> 3;
    for (int c = t; c < nchunk; c += nt) {
      float f[8];
      load(c, f);
      xs[c] = make_float4(f[0], f[1], f[2], f[3]);
      xs[nchunk + c] = make_float4(f[4], f[5], f[6], f[7]);
    }
  }
  static __device__ float stage(char* smem, const __nv_bfloat16* x, const __nv_bfloat16* scale_w,
                                int K, float* red, bool want_ssq) {
    XLoadBf16 ld{x, scale_w, 0.f};
    stage_with(smem, K, ld);
    return want_ssq ? block_sum_256(ld.ssq, red) : 0.f;
  }
};

template <>
struct XStage<WQ4> {
  // fp16 units, then per half-group: fp32 sum of the activations, fp32 factor 2^24 / S.
  static __host__ __device__ size_t bytes(int K) { return size_t(K) * 2 + size_t(K >> 5) * 8; }
  static __device__ const float* xsum(const char* smem, int K) {
    return reinterpret_cast<const float*>(smem + size_t(K) * 2);
  }
  // Stage K values produced chunk by chunk by ``load``. Every thread runs every trip of the loop
  // (the four lanes that share a half-group exchange their maxima and sums by shuffle). Ends with a
  // block barrier.
  template <class F>
  static __device__ void stage_with(char* smem, int K, F& load) {
    stage_part(smem, K, load, threadIdx.x, kGemvThreads);
    __syncthreads();
  }
  // One warp stages a whole vector by itself (ends with a warp barrier).
  template <class F>
  static __device__ void stage_warp(char* smem, int K, F& load) {
    stage_part(smem, K, load, threadIdx.x & 31, 32);
    __syncwarp();
  }
  template <class F>
  static __device__ void stage_part(char* smem, int K, F& load, int t, int nt) {
    uint4* xh = reinterpret_cast<uint4*>(smem);
    const int nchunk = K >> 3, nhg = K >> 5;
    float* xs = reinterpret_cast<float*>(smem + size_t(K) * 2);
    float* qm = xs + nhg;
    for (int c0 = 0; c0 < nchunk; c0 += nt) {
      const int c = c0 + t;
      const bool valid = c < nchunk;               // nchunk is a multiple of 4: groups are all-in or all-out
      float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (valid) load(c, f);
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      // amax < 2^(ex-126); S = 2^e puts the largest value into [2^14, 2^15). Zero or tiny groups
      // and infinities are clamped so that S and 2^24 / S stay finite.
      const int ex = (__float_as_int(amax) >> 23) & 0xff;
      const int e = max(-60, min(141 - ex, 40));
      const float S = __int_as_float((127 + e) << 23), S16 = S * 0.0625f;
      const float inv = __int_as_float((127 - e) << 23);
      const __half2 p0 = __floats2half2_rn(f[0] * S, f[4] * S), p1 = __floats2half2_rn(f[1] * S16, f[5] * S16);
      const __half2 p2 = __floats2half2_rn(f[2] * S, f[6] * S), p3 = __floats2half2_rn(f[3] * S16, f[7] * S16);
      const float2 a = __half22float2(p0), b = __half22float2(p1), cc = __half22float2(p2), d = __half22float2(p3);
      float sum = ((a.x + a.y) + (cc.x + cc.y)) * inv + ((b.x + b.y) + (d.x + d.y)) * (inv * 16.f);
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      if (valid) {
        uint4 o;
        o.x = *reinterpret_cast<const uint32_t*>(&p0); o.y = *reinterpret_cast<const uint32_t*>(&p1);
        o.z = *reinterpret_cast<const uint32_t*>(&p2); o.w = *reinterpret_cast<const uint32_t*>(&p3);
        xh[(c & 3) * nhg + (c >> 2)] = o;
        if ((c & 3) == 0) { xs[c >> 2] = sum; qm[c >> 2] = inv * 16777216.f; }
      }
    }
  }
  static __device__ float stage(char* smem, const __nv_bfloat16* x, const __nv_bfloat16* scale_w,
                                int K, float* red, bool want_ssq) {
    XLoadBf16 ld{x, scale_w, 0.f};
    stage_with(smem, K, ld);
    return want_ssq ? block_sum_256(ld.ssq, red) : 0.f;
  }
};

// 8-bit affine weights (w = s*q + b, q an unsigned byte, four per word): the bytes are used in
// place as fp16 subnormals exactly like the nibbles above (a byte at bits 0-7 of a half is
// q * 2^-24), two masks per word: t0 = w & 0x00ff00ff pairs bytes (0, 2), t1 = (w >> 8) & 0x00ff00ff
// pairs bytes (1, 3). A unit is 16 weights (one uint4); its activations are two 16-byte pieces,
// piece h at index h*(K/16) + unit, holding (x0,x2),(x1,x3) of words 2h and 2h+1. Every 16
// activations carry their own power-of-two scale; beside the pieces sit, per unit, the fp32 sum of
// the activations and the factor 2^24 / S.
template <>
struct XStage<WQ8> {
  static __host__ __device__ size_t bytes(int K) { return size_t(K) * 2 + size_t(K >> 4) * 8; }
  template <class F>
  static __device__ void stage_part(char* smem, int K, F& load, int t, int nt) {
    uint4* xh = reinterpret_cast<uint4*>(smem);
    const int nchunk = K >> 3, nu = K >> 4;
    float* xs = reinterpret_cast<float*>(smem + size_t(K) * 2);
    float* qm = xs + nu;
    for (int c0 = 0; c0 < nchunk; c0 += nt) {
      const int c = c0 + t;
      const bool valid = c < nchunk;               // nchunk is even: the two lanes of a unit are all-in or all-out
      float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (valid) load(c, f);
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      const int ex = (__float_as_int(amax) >> 23) & 0xff;
      const int e = max(-60, min(141 - ex, 40));
      const float S = __int_as_float((127 + e) << 23);
      const float inv = __int_as_float((127 - e) << 23);
      const __half2 p0 = __floats2half2_rn(f[0] * S, f[2] * S), p1 = __floats2half2_rn(f[1] * S, f[3] * S);
      const __half2 p2 = __floats2half2_rn(f[4] * S, f[6] * S), p3 = __floats2half2_rn(f[5] * S, f[7] * S);
      const float2 a = __half22float2(p0), b = __half22float2(p1), cc = __half22float2(p2), d = __half22float2(p3);
      float sum = ((a.x + a.y) + (b.x + b.y) + (cc.x + cc.y) + (d.x + d.y)) * inv;
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      if (valid) {
        uint4 o;
        o.x = *reinterpret_cast<const uint32_t*>(&p0); o.y = *reinterpret_cast<const uint32_t*>(&p1);
        o.z = *reinterpret_cast<const uint32_t*>(&p2); o.w = *reinterpret_cast<const uint32_t*>(&p3);
        xh[(c & 1) * nu + (c >> 1)] = o;
        if ((c & 1) == 0) { xs[c >> 1] = sum; qm[c >> 1] = inv * 16777216.f; }
      }
    }
  }
};

// One packed word (4 bytes) times the matching half of a 16-byte activation piece.
__device__ __forceinline__ void q8_word_fma(uint32_t w, const __half2& x02, const __half2& x13,
                                            __half2& a0, __half2& a1) {
  const uint32_t t0 = w & 0x00ff00ffu, t1 = (w >> 8) & 0x00ff00ffu;
  a0 = __hfma2(*reinterpret_cast<const __half2*>(&t0), x02, a0);
  a1 = __hfma2(*reinterpret_cast<const __half2*>(&t1), x13, a1);
}

// ------------------------------------------------------------------------------------------------
// Warp dot products. A "tile" is the slice of R weight rows that one warp pulls per iteration:
// two 16-byte loads per lane and row (64 chunks of 8 bf16, or 64 half-groups of 32 nibbles).
// Loading and multiplying are separate so a kernel can issue the first tile's loads before it
// stages the activations (and before it waits on the previous kernel): weights do not depend on
// either. acc[r][b] += dot(row r, activation b), partial per lane; the caller finishes with a warp
// reduction. smem_b_stride is the byte distance between the staged activations of consecutive b.
// ------------------------------------------------------------------------------------------------
template <class Row, int R>
struct Tile;
template <int R>
struct Tile<RowBf16, R> { uint4 w[2][R]; };
template <int R>
struct Tile<RowQ4, R> { uint4 w[2][R]; float sc[2][R], bi[2][R]; };

template <int R>
__device__ __forceinline__ void load_tile(const RowBf16 (&rows)[R], int K, int c0,
                                          Tile<RowBf16, R>& t) {
  const int lane = threadIdx.x & 31, nchunk = K >> 3;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int c = c0 + u * 32 + lane;
#pragma unroll
    for (int r = 0; r < R; ++r)
      t.w[u][r] = (c < nchunk) ? ldg_stream(rows[r].w + (size_t(c) << 3)) : make_uint4(0, 0, 0, 0);
  }
  // pull the next tile of every row (8 lines of 128 bytes each) towards L2 while this one is used
  if (lane < 8) {
    const int c = c0 + 64 + lane * 8;
    if (c < nchunk) {
#pragma unroll
      for (int r = 0; r < R; ++r) prefetch_l2(rows[r].w + (size_t(c) << 3));
    }
  }
}

template <int R, int B>
__device__ __forceinline__ void fma_tile(const Tile<RowBf16, R>& t, int c0, const char* smem,
                                         size_t smem_b_stride, int K, float (&acc)[R][B]) {
  const int lane = threadIdx.x & 31, nchunk = K >> 3;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int c = c0 + u * 32 + lane;
    if (c < nchunk) {
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const float4* xs = reinterpret_cast<const float4*>(smem + b * smem_b_stride);
        const float4 x0 = xs[c], x1 = xs[nchunk + c];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const uint4 w = t.w[u][r];
          float a = acc[r][b];
          a = fmaf(bf16lo(w.x), x0.x, a); a = fmaf(bf16hi(w.x), x0.y, a);
          a = fmaf(bf16lo(w.y), x0.z, a); a = fmaf(bf16hi(w.y), x0.w, a);
          a = fmaf(bf16lo(w.z), x1.x, a); a = fmaf(bf16hi(w.z), x1.y, a);
          a = fmaf(bf16lo(w.w), x1.z, a); a = fmaf(bf16hi(w.w), x1.w, a);
          acc[r][b] = a;
        }
      }
    }
  }
}

// One packed word (8 nibbles) times one 16-byte unit of staged fp16 activations. The masked
// nibbles are fp16 subnormals (q or 16q times 2^-24); the activations carry the matching scales.
__device__ __forceinline__ void q4_word_fma(uint32_t w, const uint4& xu, __half2& a0, __half2& a1) {
  const __half2* x = reinterpret_cast<const __half2*>(&xu);
  const uint32_t w8 = w >> 8;
  const uint32_t t0 = w & 0x000f000fu, t1 = w & 0x00f000f0u;       // (k0,k4), 16 x (k1,k5)
  const uint32_t t2 = w8 & 0x000f000fu, t3 = w8 & 0x00f000f0u;     // (k2,k6), 16 x (k3,k7)
  a0 = __hfma2(*reinterpret_cast<const __half2*>(&t0), x[0], a0);
  a1 = __hfma2(*reinterpret_cast<const __half2*>(&t1), x[1], a1);
  a0 = __hfma2(*reinterpret_cast<const __half2*>(&t2), x[2], a0);
  a1 = __hfma2(*reinterpret_cast<const __half2*>(&t3), x[3], a1);
}

template <int R>
__device__ __forceinline__ void load_tile(const RowQ4 (&rows)[R], int K, int h0, Tile<RowQ4, R>& t) {
  const int lane = threadIdx.x & 31, nhg = K >> 5;  // half-groups of 32 k = one uint4
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int hg = h0 + u * 32 + lane;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (hg < nhg) {
        t.w[u][r] = ldg_stream(rows[r].w + (size_t(hg) << 2));
        t.sc[u][r] = __bfloat162float(rows[r].scales[hg >> 1]);
        t.bi[u][r] = __bfloat162float(rows[r].biases[hg >> 1]);
      } else {
        t.w[u][r] = make_uint4(0, 0, 0, 0); t.sc[u][r] = 0.f; t.bi[u][r] = 0.f;
      }
    }
  }
  // pull the next tile of every row (8 lines of 128 bytes each) towards L2 while this one is used
  if (lane < 8) {
    const int hg = h0 + 64 + lane * 8;
    if (hg < nhg) {
#pragma unroll
      for (int r = 0; r < R; ++r) prefetch_l2(rows[r].w + (size_t(hg) << 2));
    }
  }
}

template <int R, int B>
__device__ __forceinline__ void fma_tile(const Tile<RowQ4, R>& t, int h0, const char* smem,
                                         size_t smem_b_stride, int K, float (&acc)[R][B]) {
  const int lane = threadIdx.x & 31, nhg = K >> 5;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int hg = h0 + u * 32 + lane;
    if (hg < nhg) {
#pragma unroll
      for (int b = 0; b < B; ++b) {
        const uint4* xh = reinterpret_cast<const uint4*>(smem + b * smem_b_stride);
        const float* aux = reinterpret_cast<const float*>(smem + b * smem_b_stride + size_t(K) * 2);
        const float xsum = aux[hg], qmul = aux[nhg + hg];
        const uint4 x0 = xh[hg], x1 = xh[nhg + hg], x2 = xh[2 * nhg + hg], x3 = xh[3 * nhg + hg];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          __half2 a0 = __float2half2_rn(0.f), a1 = a0;
          q4_word_fma(t.w[u][r].x, x0, a0, a1);
          q4_word_fma(t.w[u][r].y, x1, a0, a1);
          q4_word_fma(t.w[u][r].z, x2, a0, a1);
          q4_word_fma(t.w[u][r].w, x3, a0, a1);
          const float2 f0 = __half22float2(a0), f1 = __half22float2(a1);
          const float qx = ((f0.x + f0.y) + (f1.x + f1.y)) * qmul;
          acc[r][b] = fmaf(t.sc[u][r], qx, fmaf(t.bi[u][r], xsum, acc[r][b]));
        }
      }
    }
  }
}

// Number of loop positions a row spans: chunks (bf16) or half-groups (Q4); a tile covers 64.
__device__ __forceinline__ int row_units(const RowBf16&, int K) { return K >> 3; }
__device__ __forceinline__ int row_units(const RowQ4&, int K) { return K >> 5; }

// Whole-row dot product; `first` holds the already-loaded tile at position 0.
template <int R, int B, class Row>
__device__ __forceinline__ void warp_dot(const Row (&rows)[R], const char* smem,
                                         size_t smem_b_stride, int K, float (&acc)[R][B],
                                         const Tile<Row, R>& first) {
  const int n = row_units(rows[0], K);
  fma_tile<R, B>(first, 0, smem, smem_b_stride, K, acc);
  for (int p = 64; p < n; p += 64) {
    Tile<Row, R> t;
    load_tile<R>(rows, K, p, t);
    fma_tile<R, B>(t, p, smem, smem_b_stride, K, acc);
  }
}
template <int R, int B, class Row>
__device__ __forceinline__ void warp_dot(const Row (&rows)[R], const char* smem,
                                         size_t smem_b_stride, int K, float (&acc)[R][B]) {
  Tile<Row, R> t;
  load_tile<R>(rows, K, 0, t);
  warp_dot<R, B, Row>(rows, smem, smem_b_stride, K, acc, t);
}

// Row accessors for plain [N, K] matrices.
template <class WT>
struct Matrix;
template <>
struct Matrix<WBf16> {
  using Row = RowBf16;
  const __nv_bfloat16* w;
  int K;
  __device__ Row row(size_t n) const { return Row{w + n * size_t(K)}; }
};
template <>
struct Matrix<WQ4> {
  using Row = RowQ4;
  const uint32_t* w;
  const __nv_bfloat16* scales;
  const __nv_bfloat16* biases;
  int K;
  __device__ Row row(size_t n) const {
    return Row{w + n * size_t(K >> 3), scales + n * size_t(K >> 6), biases + n * size_t(K >> 6)};
  }
};

}  // namespace rb
