// Building blocks for the bandwidth-bound decode kernels (matrix-vector products with a handful of
// activation vectors): activation staging into shared memory, and per-warp dot products against
// bf16 rows or MLX-affine 4-bit rows (packed uint32, group 64, bf16 scale and bias: w = s*q + b).
//
// Weights are streamed with 16-byte no-allocate loads, one contiguous 512-byte span per warp
// instruction; activations sit in shared memory in a layout that makes every 16-byte shared load
// conflict-free. Accumulation is fp32 (the 4-bit path accumulates 16 products in fp16 pairs before
// flushing to fp32).
#pragma once
#include "ptx.cuh"

namespace rb {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = kGemvThreads / 32;

struct WBf16 {};  // weights: bf16 [N, K] row-major
struct WQ4 {};    // weights: uint32 [N, K/8], scales/biases bf16 [N, K/64]

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
// The sum of each half-group (fp32) is kept beside it for the affine bias term.
// ------------------------------------------------------------------------------------------------
template <class WT>
struct XStage;

template <>
struct XStage<WBf16> {
  static __host__ __device__ size_t bytes(int K) { return size_t(K) * 4; }
  // x: K bf16 (global), scale_w: K bf16 or nullptr. Returns sum of squares of x (block-wide).
  static __device__ float stage(char* smem, const __nv_bfloat16* x, const __nv_bfloat16* scale_w,
                                int K, float* red, bool want_ssq) {
    float4* xs = reinterpret_cast<float4*>(smem);
    const int nchunk = K >> 3;
    float ssq = 0.f;
    for (int c = threadIdx.x; c < nchunk; c += kGemvThreads) {
      uint4 v = *reinterpret_cast<const uint4*>(x + (c << 3));
      float f[8] = {bf16lo(v.x), bf16hi(v.x), bf16lo(v.y), bf16hi(v.y),
                    bf16lo(v.z), bf16hi(v.z), bf16lo(v.w), bf16hi(v.w)};
#pragma unroll
      for (int i = 0; i < 8; ++i) ssq += f[i] * f[i];
      if (scale_w) {
        uint4 s = *reinterpret_cast<const uint4*>(scale_w + (c << 3));
        f[0] *= bf16lo(s.x); f[1] *= bf16hi(s.x); f[2] *= bf16lo(s.y); f[3] *= bf16hi(s.y);
        f[4] *= bf16lo(s.z); f[5] *= bf16hi(s.z); f[6] *= bf16lo(s.w); f[7] *= bf16hi(s.w);
      }
      xs[c] = make_float4(f[0], f[1], f[2], f[3]);
      xs[nchunk + c] = make_float4(f[4], f[5], f[6], f[7]);
    }
    if (want_ssq) return block_sum_256(ssq, red);
    __syncthreads();
    return 0.f;
  }
  // Same, from fp32 values already in registers/global (used by kernels whose prologue computes
  // the activation, e.g. SwiGLU). Caller synchronises.
  static __device__ void put(char* smem, int k, int K, float v) {
    float* xs = reinterpret_cast<float*>(smem);
    const int c = k >> 3, j = k & 7;
    xs[((((j >> 2) * (K >> 3)) + c) << 2) + (j & 3)] = v;
  }
  static __device__ void finish(char*, int) {}
};

template <>
struct XStage<WQ4> {
  // fp16 units + one fp32 sum per half-group.
  static __host__ __device__ size_t bytes(int K) { return size_t(K) * 2 + size_t(K >> 5) * 4; }
  static __device__ float* xsum(char* smem, int K) {
    return reinterpret_cast<float*>(smem + size_t(K) * 2);
  }
  static __device__ float stage(char* smem, const __nv_bfloat16* x, const __nv_bfloat16* scale_w,
                                int K, float* red, bool want_ssq) {
    uint4* xh = reinterpret_cast<uint4*>(smem);
    const int nchunk = K >> 3, nhg = K >> 5;
    float ssq = 0.f;
    for (int c = threadIdx.x; c < nchunk; c += kGemvThreads) {
      uint4 v = *reinterpret_cast<const uint4*>(x + (c << 3));
      float f[8] = {bf16lo(v.x), bf16hi(v.x), bf16lo(v.y), bf16hi(v.y),
                    bf16lo(v.z), bf16hi(v.z), bf16lo(v.w), bf16hi(v.w)};
#pragma unroll
      for (int i = 0; i < 8; ++i) ssq += f[i] * f[i];
      if (scale_w) {
        uint4 s = *reinterpret_cast<const uint4*>(scale_w + (c << 3));
        f[0] *= bf16lo(s.x); f[1] *= bf16hi(s.x); f[2] *= bf16lo(s.y); f[3] *= bf16hi(s.y);
        f[4] *= bf16lo(s.z); f[5] *= bf16hi(s.z); f[6] *= bf16lo(s.w); f[7] *= bf16hi(s.w);
      }
      __half2 p0 = __floats2half2_rn(f[0], f[4]), p1 = __floats2half2_rn(f[1], f[5]);
      __half2 p2 = __floats2half2_rn(f[2], f[6]), p3 = __floats2half2_rn(f[3], f[7]);
      uint4 o;
      o.x = *reinterpret_cast<uint32_t*>(&p0); o.y = *reinterpret_cast<uint32_t*>(&p1);
      o.z = *reinterpret_cast<uint32_t*>(&p2); o.w = *reinterpret_cast<uint32_t*>(&p3);
      xh[(c & 3) * nhg + (c >> 2)] = o;
    }
    float r = 0.f;
    if (want_ssq) r = block_sum_256(ssq, red); else __syncthreads();
    finish(smem, K);
    return r;
  }
  static __device__ void put(char* smem, int k, int K, float v) {
    __half* xh = reinterpret_cast<__half*>(smem);
    const int hg = k >> 5, j = (k & 31) >> 3, n = k & 7;
    xh[((j * (K >> 5) + hg) << 3) + ((n & 3) << 1) + (n >> 2)] = __float2half_rn(v);
  }
  // Half-group sums from the stored (rounded) values. Ends with a barrier.
  static __device__ void finish(char* smem, int K) {
    const uint4* xh = reinterpret_cast<const uint4*>(smem);
    float* xs = xsum(smem, K);
    const int nhg = K >> 5;
    for (int hg = threadIdx.x; hg < nhg; hg += kGemvThreads) {
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 u = xh[j * nhg + hg];
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int p = 0; p < 4; ++p) { float2 t = __half22float2(h[p]); s += t.x + t.y; }
      }
      xs[hg] = s;
    }
    __syncthreads();
  }
};

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

// One packed word (8 nibbles) times one 16-byte unit of staged fp16 activations.
// (1024 + q) is built exactly in fp16 by OR-ing the nibble into the mantissa of 1024.0.
__device__ __forceinline__ void q4_word_fma(uint32_t w, const uint4& xu, __half2& a0, __half2& a1) {
  const __half2 k1024 = __float2half2_rn(1024.f);
  const __half2* x = reinterpret_cast<const __half2*>(&xu);
  uint32_t t0 = (w & 0x000f000fu) | 0x64006400u;
  uint32_t t1 = ((w >> 4) & 0x000f000fu) | 0x64006400u;
  uint32_t t2 = ((w >> 8) & 0x000f000fu) | 0x64006400u;
  uint32_t t3 = ((w >> 12) & 0x000f000fu) | 0x64006400u;
  a0 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&t0), k1024), x[0], a0);
  a1 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&t1), k1024), x[1], a1);
  a0 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&t2), k1024), x[2], a0);
  a1 = __hfma2(__hsub2(*reinterpret_cast<__half2*>(&t3), k1024), x[3], a1);
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
        const float xsum = reinterpret_cast<const float*>(smem + b * smem_b_stride +
                                                          size_t(K) * 2)[hg];
        const uint4 x0 = xh[hg], x1 = xh[nhg + hg], x2 = xh[2 * nhg + hg], x3 = xh[3 * nhg + hg];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          __half2 a0 = __float2half2_rn(0.f), a1 = a0;
          q4_word_fma(t.w[u][r].x, x0, a0, a1);
          q4_word_fma(t.w[u][r].y, x1, a0, a1);
          q4_word_fma(t.w[u][r].z, x2, a0, a1);
          q4_word_fma(t.w[u][r].w, x3, a0, a1);
          const float2 f0 = __half22float2(a0), f1 = __half22float2(a1);
          const float qx = (f0.x + f0.y) + (f1.x + f1.y);
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
